"""GPU parity at the stated sizes of the five benchmark configurations, against the CPU oracle, through the C ABI.

Small instances of the same shapes are compared dump for dump in test_gpu_parity.py; here every size-dependent piece of
machinery is in play: 32-bit offsets near their limits, slicing with the class store carried across slices, millions of
initialisers on the element-parallel path, nesting to depth 32 over hundreds of megabytes.  The comparison is the 64-bit
hash of the canonical dump per module (the dumps themselves run to gigabytes); the oracle runs one module per task on
all host cores, single modules on one core beside the others.  The texts are generated (seeded), never stored.

Also here: the reference's own .ptx test inputs through the CUDA path (packed under tests/golden/), and decimal floating
point literals converted on the device against Python's correctly rounded float().
"""
import json
import os
import random
import struct
import threading
import time
import zlib

import numpy as np
import pytest

import zluda_b200
from zluda_b200 import corpus

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ctx():
    c = zluda_b200.Context(0)
    yield c
    c.close()


def _spans(blob, spans):
    base = blob.ctypes.data
    return [(base + o, l) for o, l in spans]


def _gpu_hashes(ctx, texts, which=None, mode=0):
    from concurrent.futures import ThreadPoolExecutor
    b = ctx.parse_batch(texts, mode)
    idx = range(len(b)) if which is None else which
    with ThreadPoolExecutor(min(32, os.cpu_count() or 1)) as ex:
        hashes = list(ex.map(b.dump_hash, idx))
    errors = sum(b.error_count(i) for i in idx)
    stats = ctx.stats()
    b.free()
    return hashes, errors, stats


def test_config0_single_module(oracle, ctx):
    """64 entry kernels x 2,000 instructions, one module; the whole dump is compared."""
    mods = corpus.config0()
    assert 4_000_000 < len(mods[0]) < 9_000_000
    b = ctx.parse_batch(mods, 0)
    st, expect = oracle.parse(mods[0], 0)
    assert st == 0 and b.status(0) == 0
    assert b.dump(0) == expect
    b.free()


def test_config1_all_modules(oracle, ctx):
    """4,096 modules, ~1 GiB, one ptxfe_parse_batch call (sliced internally): every module's dump hash."""
    blob = np.empty(corpus.config1_total_bound(), dtype=np.uint8)
    mods = _spans(blob, corpus.config1_into(blob))
    total = sum(l for _, l in mods)
    assert len(mods) == 4096 and 1.0e9 < total < 1.15e9
    got, errors, stats = _gpu_hashes(ctx, mods)
    expect = oracle.dump_hashes(mods)
    bad = [i for i in range(len(mods)) if got[i] != expect[i]]
    assert not bad, bad[:10]
    assert errors == 0 and stats["n_sequential"] == 0
    # every statement is drawn afresh, yet the batch has few classes and nearly every unit is templated
    assert stats["n_classes"] < 2000, stats
    assert stats["n_untemplated"] < 0.01 * stats["n_units"], stats
    # the resident path (stage / run / fetch, unsliced) gives the same records
    ctx.stage(mods)
    ctx.run(0)
    b = ctx.fetch()
    sample = list(range(0, len(mods), 64))
    assert [b.dump_hash(i) for i in sample] == [expect[i] for i in sample]
    b.free()


def test_config2_literal_heavy(oracle, ctx):
    """16 arrays x 4 Mi initialisers (hex and decimal) + 1 Mi scalar constants (0d / 0f hex, 9- and 17-digit decimals):
    ~400 MB in one module."""
    mods = corpus.config2()
    assert 3.5e8 < len(mods[0]) < 7.0e8      # the stated counts give ~620 MB; the configuration text says "~400 MB"
    expect = {}
    t = threading.Thread(target=lambda: expect.setdefault("h", oracle.dump_hash(mods[0])))
    t.start()
    got, errors, stats = _gpu_hashes(ctx, mods)
    t.join()
    assert got[0] == expect["h"]
    assert errors == 0 and stats["n_sequential"] == 0


def test_config3_structure_heavy(oracle, ctx):
    """~256 MB in one module: .loc before every instruction, 40 % comments, scopes to depth 32, call sequences, 20,000
    labels."""
    mods = corpus.config3()
    text = mods[0]
    assert 2.5e8 < len(text) < 2.9e8
    comment_bytes = sum(len(c) for c in __import__("re").findall(rb"//[^\n]*|/\*.*?\*/", text[:4 << 20]))
    assert 0.25 < comment_bytes / (4 << 20) < 0.55
    expect = {}
    t = threading.Thread(target=lambda: expect.setdefault("h", oracle.dump_hash(text)))
    t.start()
    got, errors, stats = _gpu_hashes(ctx, mods)
    t.join()
    assert got[0] == expect["h"]
    assert errors == 0 and stats["n_sequential"] == 0


def test_config4_sweep_sample(oracle, ctx):
    """65,536 modules (~16 GiB) as 16 batches of 4,096 drawn with seeds 1004 + shard; parity on every 16th module."""
    blob = np.empty(corpus.config1_total_bound(), dtype=np.uint8)
    total, checked = 0, 0
    for shard in range(16):
        mods = _spans(blob, corpus.config1_into(blob, seed=1004 + shard))
        total += sum(l for _, l in mods)
        sample = list(range(shard % 16, len(mods), 16))
        got, errors, stats = _gpu_hashes(ctx, mods, sample)
        expect = oracle.dump_hashes([mods[i] for i in sample])
        assert got == expect, shard
        assert errors == 0 and stats["n_sequential"] == 0
        checked += len(sample)
    assert checked == 4096 and total > 16e9


def test_reference_fixtures_on_the_device(oracle, ctx):
    """The .ptx inputs of the reference's own tests (ptx/src/test/mod.rs:32-75 feeds them to parse_module_checked),
    packed by tests/golden/pack_reference_fixtures.py: GPU dump against the oracle's, in all three modes, and against the
    hashes recorded when the pack was made."""
    import hashlib
    rows = json.loads(zlib.decompress(open(os.path.join(HERE, "golden", "reference_fixtures.bin"), "rb").read()))
    assert len(rows) >= 240
    texts = [r["text"].encode("latin-1") for r in rows]
    for mode in (0, 1, 2):
        b = ctx.parse_batch(texts, mode)
        for i, r in enumerate(rows):
            d = b.dump(i)
            assert d == oracle.parse(texts[i], mode)[1], (r["name"], mode)
            assert hashlib.sha256(d.encode()).hexdigest() == r["sha256"][mode], (r["name"], mode)
            if mode == 0:
                assert (b.status(i) == 0) == r["accepted"], r["name"]
        b.free()


def _f64_bits(s):
    return struct.unpack("<Q", struct.pack("<d", float(s)))[0]


def decimal_literals():
    """Fixed hard cases, random 9- and 17-digit decimals, long digit strings with large exponents, and exact halfway
    points between adjacent doubles with their neighbours."""
    rng = random.Random(3)
    out = ["1.5", ".5", "0.1", "1.7976931348623157e308", "1.7976931348623159e308", "4.9e-324", "2.4703282292062327e-324",
           "2.4703282292062328e-324", "1.0e400", "1.0e-400", "9007199254740993.0", "9007199254740992.9999999999999999999999",
           "2.2250738585072011e-308", "2.2250738585072014e-308", "8.98846567431158e307", "0.0", "000.000e5",
           "123456789012345678901234567890.5e-10"]
    for _ in range(20000):
        k = rng.random()
        if k < 0.3:
            out.append("%.8e" % abs(rng.gauss(0, 1)))
        elif k < 0.6:
            out.append("%.16e" % abs(rng.gauss(0, 1)))
        elif k < 0.8:
            out.append("%d.%de%d" % (rng.randrange(10 ** rng.randrange(1, 25)), rng.randrange(10 ** rng.randrange(1, 30)), rng.randrange(-340, 300)))
        else:
            x = struct.unpack("<d", struct.pack("<Q", rng.getrandbits(63)))[0]
            if x == x and x != float("inf"):
                out.append("%.17e" % x)
    from decimal import Decimal, getcontext
    getcontext().prec = 1200
    for _ in range(300):
        bits = rng.getrandbits(62) | (rng.randrange(1, 2046) << 52) if rng.random() < 0.8 else rng.getrandbits(52)
        bits &= (1 << 63) - 1
        if (bits >> 52) >= 2046:
            continue
        x = struct.unpack("<d", struct.pack("<Q", bits))[0]
        y = struct.unpack("<d", struct.pack("<Q", bits + 1))[0]
        mid = (Decimal(x) + Decimal(y)) / 2
        ulp = Decimal(y) - Decimal(x)
        for v in (mid, mid + ulp / 1000000, mid - ulp / 1000000):
            s = format(v, "f")
            if "." not in s:
                s += ".0"
            if len(s) < 60000:
                out.append(s)
    return out


def test_decimal_literals_on_the_device(ctx):
    """`.global .f64 c = <literal>;` for every case: the bits in the GPU's dump against Python's correctly rounded
    float() (the device conversion runs Eisel-Lemire with an exact big-integer fallback, in its device arithmetic)."""
    lits = decimal_literals()
    text = ".version 7.8\n.target sm_80\n.address_size 64\n" + "".join(".global .f64 c%d = %s;\n" % (i, s) for i, s in enumerate(lits))
    b = ctx.parse_batch([text], 0)
    assert b.status(0) == 0
    lines = [l for l in b.dump(0).split("\n") if l.startswith("Variable(")]
    b.free()
    assert len(lines) == len(lits)
    for s, line in zip(lits, lines):
        assert "array_init: [Imm(F64(bits=0x%016X))]" % _f64_bits(s) in line, (s[:80], line[-80:])
    # the same literals as immediates of instructions: converted when a record template is instantiated
    stmts = "\n".join("mov.f64 %%fd1, %s;" % s for s in lits[:4000])
    text = ".version 7.8\n.target sm_80\n.address_size 64\n.visible .entry k()\n{\n.reg .f64 %fd<4>;\n" + stmts + "\nret;\n}\n"
    b = ctx.parse_batch([text], 0)
    assert b.status(0) == 0
    lines = [l for l in b.dump(0).split("\n") if "Instruction(" in l and "Mov" in l]
    stats = ctx.stats()
    b.free()
    assert len(lines) == 4000
    for s, line in zip(lits, lines):
        assert "Imm(F64(bits=0x%016X))" % _f64_bits(s) in line, (s[:80], line[-120:])
    assert stats["n_untemplated"] < 100, stats
