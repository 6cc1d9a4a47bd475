#!/usr/bin/env python3
"""Packs the .ptx inputs of the reference's own parser tests into tests/golden/reference_fixtures.bin, so that the GPU
tests can feed them to the CUDA path on a machine without the reference checkout.

Every `ptx` test of the reference enters through parse_module_checked(text).unwrap() (ptx/src/test/mod.rs:32-75); the
files are test vectors (inputs), not source code.  The pass tests hold input and expected output in one file, split at
"// %%% output %%%": only the input part is a parser input.  Packed form: zlib(JSON list of {name, text (latin-1),
sha256 of the oracle's dump per mode}).  Run from the repository root with the reference mounted:
    python tests/golden/pack_reference_fixtures.py <path of the reference checkout>
"""
import glob
import hashlib
import json
import os
import sys
import zlib

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib  # noqa: E402


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref = sys.argv[1]
    o = oracle_lib.load()
    rows = []
    for f in sorted(glob.glob(os.path.join(ref, "**", "*.ptx"), recursive=True)):
        t = open(f, "rb").read()
        if "/pass/test/" in f:
            t = t.split(b"// %%% output %%%")[0].strip()
        rows.append({"name": os.path.relpath(f, ref), "text": t.decode("latin-1"),
                     "sha256": [hashlib.sha256(o.parse(t, mode)[1].encode()).hexdigest() for mode in (0, 1, 2)],
                     "accepted": o.parse(t, 0)[0] == 0})
    blob = zlib.compress(json.dumps(rows).encode(), 9)
    with open(os.path.join(HERE, "reference_fixtures.bin"), "wb") as out:
        out.write(blob)
    print("packed %d fixtures, %d bytes" % (len(rows), len(blob)))


if __name__ == "__main__":
    main()
