"""Reference arm of the benchmark: the unmodified reference GridNeRF trainer from ``baseline/_ref``."""
import json


def run_reference(args, *unused):
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}), flush=True)
