#!/usr/bin/env python3
"""Writes tests/golden/pattern_pins.json: for every statement of tests/pattern_statements.py the Instruction line of the
canonical dump in unchecked mode (None when the statement raises an error: the reference drops a directive that raised
one, lib.rs:581-611) and the errors it raises.  The lines are produced by the oracle and frozen here; tests/test_pattern_pins.py says which of them were then
read against the reference's code blocks and which detail constructors are re-derived independently.
Run from the repository root:  python tests/golden/make_pattern_pins.py"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib  # noqa: E402
import pattern_statements as ps  # noqa: E402


def pin(o, stmt):
    d1 = o.parse(ps.module([stmt]), 1)[1].split("\n")
    lines = [l.strip() for l in d1 if l.strip().startswith("Instruction(")]
    k = max(i for i, l in enumerate(d1) if l.startswith("errors: "))
    return {"stmt": stmt, "line": lines[0] if len(lines) > 1 else None, "errors": [l for l in d1[k + 1:] if l]}


def main():
    o = oracle_lib.load()
    rows = [pin(o, s) for s in ps.STATEMENTS]
    with open(os.path.join(HERE, "pattern_pins.json"), "w") as f:
        json.dump(rows, f, indent=0)
    print("wrote", len(rows), "pins")


if __name__ == "__main__":
    main()
