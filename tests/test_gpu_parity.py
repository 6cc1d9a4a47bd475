"""GPU parity: the CUDA path, called through the C ABI (include/ptxfe.h), against the CPU oracle on the same inputs.
Bit-exact: the canonical dumps (tree + ordered error list) must be byte-equal."""
import hashlib
import json
import os
import random

import pytest

import cases
import zluda_b200
from zluda_b200 import corpus

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ctx():
    c = zluda_b200.Context(0)
    yield c
    c.close()


def first_difference(a, b):
    al, bl = a.split("\n"), b.split("\n")
    for i, (x, y) in enumerate(zip(al, bl)):
        if x != y:
            return "line %d\n oracle: %s\n gpu:    %s" % (i, x[:300], y[:300])
    return "length %d vs %d" % (len(al), len(bl))


def assert_parity(oracle, ctx, texts, modes=(0, 1, 2)):
    for mode in modes:
        b = ctx.parse_batch(texts, mode)
        assert len(b) == len(texts)
        for i, t in enumerate(texts):
            st, o = oracle.parse(t, mode)
            d = b.dump(i)
            assert o == d, (mode, i, first_difference(o, d))
            assert (b.status(i) == 0) == (st == 0)
            # the verdict and the error count are read off the module's result row, not off the dump
            n_err = [int(l.split()[1]) for l in d.split("\n") if l.startswith("errors: ")][-1]
            assert b.error_count(i) == n_err, (mode, i, b.error_count(i), n_err)
            verdict = d.split("\n")[1]
            assert (b.status(i) == 3) == (verdict == "status: ReferenceDiverges")
            assert (b.status(i) == 2) == (verdict == "status: ReferencePanics")
        b.free()
    return ctx.stats()


def test_edge_cases_and_golden_hashes(oracle, ctx):
    texts = cases.all_cases()
    stats = assert_parity(oracle, ctx, texts)
    assert stats["n_kernel_launches"] > 20
    golden = json.load(open(os.path.join(HERE, "golden", "cases.json")))
    for mode in (0, 1, 2):
        b = ctx.parse_batch(texts, mode)
        for row in golden["cases"]:
            assert hashlib.sha256(b.dump(row["index"]).encode()).hexdigest() == row["sha256"][mode], (row["index"], mode)
        b.free()


def test_statement_classes(oracle, ctx):
    """Record templates: statements of one shape share the grammar work; what must stay different does.  Parsed twice
    in one batch and as several batches through one context (the class store is emptied per batch)."""
    texts = cases.class_cases()
    assert_parity(oracle, ctx, texts)
    assert_parity(oracle, ctx, texts + texts[::-1], modes=(0,))


def test_nested_damage_and_divergence(oracle, ctx):
    """Damage below nested blocks: identical while the reference's doubling recovery stays within its work budget,
    the verdict ReferenceDiverges (PTXFE_MODULE_REF_DIVERGES) beyond it; the kernel that parses such a module returns."""
    texts = cases.nested_damage_cases()
    assert_parity(oracle, ctx, texts)
    b = ctx.parse_batch(texts, 0)
    assert b.status(len(texts) - 1) == 3 and b.status(0) == 1
    b.free()


def test_negative_decimal_side_file(oracle, ctx):
    assert_parity(oracle, ctx, [cases.negative_decimal_side_file()])


def test_bulk_initialisers(oracle, ctx):
    """Initialiser lists long enough for the element-parallel path, regular and irregular."""
    assert_parity(oracle, ctx, cases.bulk_cases(), modes=(0, 2))


def test_class_store_capacity_and_long_names(oracle, ctx, monkeypatch):
    """More classes than the store holds (the rest is decoded the ordinary way), in one slice and across slices."""
    texts = cases.capacity_cases()
    assert_parity(oracle, ctx, texts, modes=(0,))
    monkeypatch.setenv("PTXFE_SLICE_BYTES", "2000000")
    assert_parity(oracle, ctx, [texts[0][:3000000] + "\nret;\n}\n"] * 3 + texts, modes=(0,))


def test_lexer_tokens(oracle, ctx):
    rng = random.Random(7)
    pieces = ["add", ".f32", "%r1", ",", ";", " ", "\n", "// c\n", "/* x */", "/*", "*/", "\"s\"", "\"", "0f3F800000", "0x1F", "1.5e-3",
              "1.5e", ".5", "12U", ".L2::cache_hint", ".shared::cta", ".shared::", "::", ":", "+", "-", "{", "}", "[", "]", "#", "$L_1",
              "%", ".", ".1d", "WARP_SZ", "0d3FF0000000000000", "abc" * 60, "/", "*", "é", "a.b", "1e5", "0xU",
              "0x1F_a", "0f3F800000U", "0f3F80000_", "12Ua", "00x1F", "0x" + "A" * 20, "0x" + "b" * 16, "5U", "0F3f800000", "0d3FF000000000000", "0x1$"]
    for trial in range(60):
        text = "".join(rng.choice(pieces) for _ in range(rng.randrange(1, 120)))
        ot, oe = oracle.lex(text)
        gt, ge = ctx.lex(text)
        assert ot == gt, text
        assert oe == ge, text
    for pad in range(0, 140, 3):
        text = " " * pad + "ld.global.L2::cache_hint.v4.f32 {%f1,%f2,%f3,%f4}, [%rd1+16]; /* c */ 0f3F800000 1.25e-3 // e\n\"str\""
        assert oracle.lex(text) == ctx.lex(text), pad


def test_dense_tiles_lex_like_the_oracle(oracle, ctx):
    """Tiles that the emit step takes in several passes, and tiles that overflow its lists of numbers and keyword candidates."""
    for text in cases.dense_token_texts():
        assert oracle.lex(text) == ctx.lex(text), text[:40]


def test_numbers_across_tile_ends(oracle, ctx):
    """Every kind of numeric literal at every position around the end of an 8 KiB lexer tile."""
    for t in cases.numbers_across_tile_ends():          # one module per batch: the module begins where a tile begins
        b = ctx.parse_batch([t], 1)
        dump = b.dump(0)
        b.free()
        assert dump == oracle.parse(t, 1)[1], t[-80:]


def test_corpora(oracle, ctx):
    sets = {
        "config0": corpus.config0(n_kernels=8, n_instr=2000),
        "config1": corpus.config1(n_modules=256, total_bytes=16 << 20, pool_lines=40000),
        "config2": corpus.config2(n_arrays=4, n_init=50000, n_consts=20000),
        "config3": corpus.config3(total_bytes=4 << 20, n_funcs=16, n_labels=1000),
    }
    for name, mods in sets.items():
        stats = assert_parity(oracle, ctx, mods, modes=(0,))
        assert stats["n_sequential"] == 0, name


def test_sliced_batches(oracle, ctx, monkeypatch):
    """The one-call entry point cuts a batch into slices and overlaps their copies with the kernels: with slices of a
    few KB every edge case, error list and lexer error lands in a different slice and both working arenas are reused
    many times.  The unsliced stage / run / fetch path must give the same dumps."""
    texts = cases.all_cases() + corpus.config1(n_modules=16, total_bytes=1 << 20, pool_lines=5000)
    for slice_bytes in ("1", "3000", "70000"):
        monkeypatch.setenv("PTXFE_SLICE_BYTES", slice_bytes)
        assert_parity(oracle, ctx, texts, modes=(0, 2))
    monkeypatch.delenv("PTXFE_SLICE_BYTES")
    b = ctx.parse_batch(texts, 0)
    sliced = [b.dump_hash(i) for i in range(len(texts))]
    b.free()
    ctx.stage(texts)
    ctx.run(0)
    b = ctx.fetch()
    assert sliced == [b.dump_hash(i) for i in range(len(texts))]
    b.free()
    # modules that lie back to back in host memory travel as one copy and are re-aligned on the device
    import numpy as np
    raw = [t.encode() if isinstance(t, str) else bytes(t) for t in texts]
    blob = np.frombuffer(b"".join(raw), dtype=np.uint8).copy()
    spans, off = [], 0
    for t in raw:
        spans.append((blob.ctypes.data + off, len(t)))
        off += len(t)
    for slice_bytes in ("5000", "1000000000"):
        monkeypatch.setenv("PTXFE_SLICE_BYTES", slice_bytes)
        b = ctx.parse_batch(spans, 0)
        assert sliced == [b.dump_hash(i) for i in range(len(texts))], slice_bytes
        b.free()


def test_mutated_modules(oracle, ctx):
    rng = random.Random(11)
    base = corpus.config1(n_modules=4, total_bytes=24 << 10, pool_lines=2000) + corpus.config3(total_bytes=24 << 10, n_funcs=4, n_labels=20)
    junk = [";", "{", "}", ":", ",", "(", ")", "foo", ".bar", "[", "]", "@", "\"", "/*", "#", ".global", ".entry", ".func", "<", "0x", "-", "ret", ""]
    texts = []
    for t in base:
        s = t.decode()
        for _ in range(12):
            m = s
            for _ in range(rng.randrange(1, 4)):
                pos = rng.randrange(len(m))
                m = m[:pos] + rng.choice(junk) + m[pos:] if rng.random() < 0.5 else m[:pos] + m[pos + rng.randrange(1, 12):]
            texts.append(m)
    assert_parity(oracle, ctx, texts)


def test_full_size_properties(ctx):
    """At benchmark scale the oracle is too slow to run on everything: check size-independent properties instead.
    (1) parsing a batch twice gives identical records; (2) a module's result does not depend on its neighbours:
    the dump hash of every module in a shuffled batch equals its hash in the original order; (3) clean input
    produces no errors and never takes the recovery path."""
    mods = corpus.config1(n_modules=512, total_bytes=128 << 20)
    b = ctx.parse_batch(mods)
    h1 = [b.dump_hash(i) for i in range(0, len(mods), 7)]
    assert all(b.error_count(i) == 0 for i in range(len(mods)))
    assert ctx.stats()["n_sequential"] == 0
    b.free()
    order = list(range(len(mods)))
    random.Random(1).shuffle(order)
    b = ctx.parse_batch([mods[i] for i in order])
    pos = {m: k for k, m in enumerate(order)}
    h2 = [b.dump_hash(pos[i]) for i in range(0, len(mods), 7)]
    b.free()
    assert h1 == h2


def test_damage_is_confined_to_the_tail(oracle, ctx):
    """Damage in one top-level directive: the directives in front of it keep their speculated units, the sequential
    parser (one thread) takes over from that directive to the end of the module."""
    n_sequential = 0
    for text, front in cases.confined_damage_cases():
        for mode in (0, 1, 2):
            b = ctx.parse_batch([text], mode)
            assert b.dump(0) == oracle.parse(text, mode)[1], (text[-300:], mode)
            b.free()
            st = ctx.stats()
            assert st["n_sequential_tokens"] <= (1.0 - front) * st["n_tokens"] + 64, (front, st)
            n_sequential += st["n_sequential"]
    assert n_sequential >= 30


def test_stray_tokens_in_a_large_module(oracle, ctx):
    """One stray token in the middle of a function body of a 4 MB module: recovered by the speculated units, no
    sequential parse, milliseconds."""
    text = corpus.config1(n_modules=1, total_bytes=4 << 20)[0]
    mods = cases.stray_token_modules(text)
    b = ctx.parse_batch(mods, 1)
    st = ctx.stats()
    expect = oracle.dump_hashes(mods, 1)
    assert [b.dump_hash(i) for i in range(len(mods))] == expect
    assert all(b.error_count(i) >= 1 for i in range(len(mods)))
    b.free()
    assert st["n_sequential"] == 0, st
    assert st["kernel_ms"] < 10.0 * len(mods), st


def test_long_sequential_tail_is_refused(oracle, ctx, monkeypatch):
    text, front = cases.confined_damage_cases()[1]
    fine = cases.HEADER + ".global .u32 fine;\n"
    monkeypatch.setenv("PTXFE_SEQ_MAX_TOKENS", "1000")
    b = ctx.parse_batch([text, fine], 1)
    assert b.dump(0) == "mode: unchecked\nstatus: SequentialPathRefused\nerrors: 0\n"
    assert b.status(0) == 4 and b.error_count(0) == 0
    assert b.dump(1) == oracle.parse(fine, 1)[1] and b.status(1) == 0
    b.free()
    monkeypatch.delenv("PTXFE_SEQ_MAX_TOKENS")
    b = ctx.parse_batch([text], 1)
    assert b.dump(0) == oracle.parse(text, 1)[1]
    b.free()


def test_large_truncated_module(oracle, ctx):
    """A 4 MB module cut off in the middle of its last function (what a dump of a crashed process looks like): only
    that function goes through the one-thread parser, and the module costs milliseconds, not seconds."""
    text = corpus.config1(n_modules=1, total_bytes=4 << 20)[0]
    last = text.rfind(b".visible .entry")
    assert last > 0.8 * len(text)
    cut = text[:last + (len(text) - last) // 2]
    ctx.parse_batch([text], 1).free()          # first use of a context pays for its tables, arenas and the kernels' loading
    b = ctx.parse_batch([cut], 1)
    st = ctx.stats()
    assert b.dump_hash(0) == oracle.dump_hash(cut, 1)
    assert b.error_count(0) >= 1
    b.free()
    assert st["n_sequential"] == 1
    assert st["n_sequential_tokens"] < 0.2 * st["n_tokens"], st
    assert st["kernel_ms"] < 100, st          # the whole module through the one-thread parser: 4.4 s
    # a stray '{' in the last tenth of the module: the sequential tail is that tenth
    at = text.find(b"\n", int(0.9 * len(text))) + 1
    damaged = text[:at] + b"{\n" + text[at:]
    b = ctx.parse_batch([damaged], 1)
    st = ctx.stats()
    assert b.dump_hash(0) == oracle.dump_hash(damaged, 1)
    b.free()
    assert st["n_sequential"] == 1 and st["n_sequential_tokens"] < 0.3 * st["n_tokens"], st


def test_long_runs_of_soft_bytes(oracle, ctx):
    """A quarter of a MiB of sigils and dots in one run, lexer errors all along it: the oracle's errors, and a kernel time
    that one thread's single walk over the module explains (the per-chunk error pass used to be quadratic here)."""
    n = 256 << 10
    for run in ("%." * (n // 2), "a" * n, "a.b::" * (n // 5)):
        text = cases.HEADER + ".visible .entry k()\n{\nmov.u32 %r1, " + run + ";\nret;\n}\n"
        for mode in (1, 2):
            b = ctx.parse_batch([text], mode)
            st = ctx.stats()
            assert b.dump(0) == oracle.parse(text, mode)[1], (run[:8], mode)
            b.free()
            assert st["kernel_ms"] < 2000, (run[:8], st)


def test_small_modules_behind_a_large_batch_repeatedly(oracle, ctx):
    """Three thousand one-statement modules of a thousand shapes (most units are decoded one by one, through the staging
    table), parsed forty times, each time behind a 4 MB module that leaves the arenas full of other data: every parse
    must give the oracle's dumps.  (A cooperative copy of the staged records used to lose words in about one such parse
    in ten.)"""
    import test_pattern_pins as pins
    import pattern_statements as ps
    texts = zluda_b200.Texts([ps.module([c[0]]) for c in pins.sweep_cases()])
    expect = oracle.dump_hashes([ps.module([c[0]]) for c in pins.sweep_cases()], 1)
    big = corpus.config1(n_modules=1, total_bytes=4 << 20)
    for rep in range(40):
        ctx.parse_batch(big, 1).free()
        b = ctx.parse_batch(texts, 1)
        got = [b.dump_hash(i) for i in range(len(expect))]
        b.free()
        bad = [i for i in range(len(expect)) if got[i] != expect[i]]
        assert not bad, (rep, bad[:8])


def test_pattern_pins_on_the_device(ctx):
    """Every instruction pattern through the CUDA path: the frozen line per statement (tests/golden/pattern_pins.json) and
    the sweeps of cvt / setp / atom / ldmatrix against their re-derivations from the reference (test_pattern_pins.py)."""
    import test_pattern_pins as pins

    def parse(texts, mode):
        b = ctx.parse_batch(texts, mode)
        dumps = [b.dump(i) for i in range(len(texts))]
        b.free()
        return dumps
    pins.check_pins(parse)
    assert pins.check_sweep(parse) > 2500


def test_multi_device_entry_point(oracle):
    """ptxfe_parse_batch_multi: the batch split over a device list inside the library, one host thread and context per
    entry, results in the caller's module order.  With one GPU visible the list names it twice (two contexts, two
    threads); with more, the first two or four devices."""
    import torch
    n_dev = torch.cuda.device_count()
    devices = [0, 0] if n_dev < 2 else list(range(min(n_dev, 4)))
    texts = cases.all_cases()[:80] + corpus.config1(n_modules=64, total_bytes=8 << 20) + cases.nested_damage_cases()[:4]
    mc = zluda_b200.MultiContext(devices)
    for mode in (0, 2):
        b = mc.parse_batch(texts, mode)
        assert len(b) == len(texts)
        for i, t in enumerate(texts):
            st, o = oracle.parse(t, mode)
            assert b.dump(i) == o, (mode, i)
            assert (b.status(i) == 0) == (st == 0)
        parts = [b.part_of(i) for i in range(len(texts))]
        assert set(parts) == set(range(len(devices)))
        stats = mc.part_stats()
        assert sum(s["n_modules"] for s in stats) == len(texts)
        loads = [s["text_bytes"] for s in stats]
        assert max(loads) - min(loads) <= max(len(t) for t in texts)
        b.free()
    # a second batch through the same contexts, and an empty one
    b = mc.parse_batch(texts[:3], 0)
    assert [b.dump(i) for i in range(3)] == [oracle.parse(t, 0)[1] for t in texts[:3]]
    b.free()
    assert len(mc.parse_batch([], 0)) == 0
    mc.close()


def test_public_api(oracle):
    text = cases.body("add.s32 %r1, %r2, %r3;")
    r = zluda_b200.parse_module_checked(text)
    assert r.ok and r.dump == oracle.parse(text, 0)[1]
    bad = cases.body("bogus %r1;")
    assert not zluda_b200.parse_module_checked(bad).ok
    assert zluda_b200.parse_module_unchecked(bad).ok
    assert zluda_b200.parse_for_errors(bad) == oracle.errors(bad, 2)
