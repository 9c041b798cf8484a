"""Reference arm of bench.py: the UNMODIFIED reference (installed under baseline/_ref) driving the
same MoE-layer training step through its own public API, with plain PyTorch for the expert math
the reference leaves to the host framework."""
import json


def run_reference(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired up yet"}), flush=True)
