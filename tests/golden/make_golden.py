#!/usr/bin/env python3
"""Writes tests/golden/cases.json: for every shared edge case and mode, the SHA-256 of the oracle's canonical dump.
The oracle itself is pinned by tests/test_oracle_reference_vectors.py against the reference's own test vectors; these
hashes freeze its output so that later edits to the oracle or to the dump format are noticed.
Run from the repository root:  python tests/golden/make_golden.py"""
import hashlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import cases  # noqa: E402
import oracle_lib  # noqa: E402


def main():
    o = oracle_lib.load()
    out = []
    for i, text in enumerate(cases.all_cases()):
        row = {"index": i, "sha256": []}
        for mode in (0, 1, 2):
            row["sha256"].append(hashlib.sha256(o.parse(text, mode)[1].encode()).hexdigest())
        out.append(row)
    with open(os.path.join(HERE, "cases.json"), "w") as f:
        json.dump({"n": len(out), "cases": out}, f, indent=0)
    print("wrote", len(out), "cases")


if __name__ == "__main__":
    main()
