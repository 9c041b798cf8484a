"""moonep_b200: a Blackwell-native (sm_100a) expert-parallel communication framework."""
from .plan import CommPlan  # noqa: F401

__version__ = "0.1.0"
