"""Reference arm of the benchmark (filled in by `baseline/run_reference.py`)."""


def run_reference(args):
    return {"impl": "reference", "unavailable": "reference harness not installed yet"}
