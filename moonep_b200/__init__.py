"""moonep_b200: a Blackwell-native (sm_100a) expert-parallel communication framework."""
from .plan import CommPlan  # noqa: F401

MoonEPCommPlan = CommPlan      # the reference's name for the same object (moonep/planning.py:31)

__version__ = "0.1.0"
__all__ = ["Buffer", "CommPlan", "MoonEPCommPlan", "CommTimeoutError"]


def __getattr__(name):
    # Buffer pulls in torch.distributed and the native library; import it lazily so that
    # `import moonep_b200` stays cheap for users of the CPU oracle only.
    if name in ("Buffer", "CommTimeoutError", "destroy_live_buffers"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)
