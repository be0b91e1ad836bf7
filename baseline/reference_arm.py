"""The reference arm of bench.py: the unmodified reference, installed under baseline/_ref."""
import json


def main(args) -> int:
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired up yet"}))
    return 0
