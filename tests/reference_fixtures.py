"""The .ptx inputs of the reference's own parser tests, as packed by tests/golden/pack_reference_fixtures.py (name, text,
sha256 of the oracle's dump per mode when the pack was made, accepted by the checked mode)."""
import json
import os
import zlib

HERE = os.path.dirname(os.path.abspath(__file__))


def rows():
    return json.loads(zlib.decompress(open(os.path.join(HERE, "golden", "reference_fixtures.bin"), "rb").read()))


def texts():
    return {r["name"]: r["text"].encode("latin-1") for r in rows()}
