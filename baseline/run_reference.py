"""Reference arm of bench.py: runs the UNMODIFIED reference (installed under baseline/_ref) through
its own modules on the same metric and config.  Filled in by `run_reference`."""
import json


def run_reference(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference harness not wired yet"}))
