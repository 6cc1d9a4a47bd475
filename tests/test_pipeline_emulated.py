"""The product's pipeline steps (lexer chunks, unit speculation, decoders, record format, dump) run on the host through
the sequential test backend and compared with the oracle.  No GPU needed; the GPU runs of the same comparisons are in
test_gpu_parity.py."""
import glob
import hashlib
import json
import os
import random
import struct

import numpy as np
import pytest

import cases
import emu_lib
from zluda_b200 import corpus

import reference_fixtures
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def emu():
    return emu_lib.load()


def first_difference(a, b):
    al, bl = a.split("\n"), b.split("\n")
    for i, (x, y) in enumerate(zip(al, bl)):
        if x != y:
            return "line %d\n oracle: %s\n ours:   %s" % (i, x[:300], y[:300])
    return "length %d vs %d" % (len(al), len(bl))


def assert_parity(oracle, emu, texts, modes=(0, 1, 2)):
    for mode in modes:
        dumps, stats = emu.parse(texts, mode)
        for t, d in zip(texts, dumps):
            o = oracle.parse(t, mode)[1]
            assert o == d, (mode, t[-200:], first_difference(o, d))
    return stats


def test_golden_oracle_hashes(oracle):
    golden = json.load(open(os.path.join(HERE, "golden", "cases.json")))
    texts = cases.all_cases()
    assert golden["n"] == len(texts)
    for row, t in zip(golden["cases"], texts):
        for mode in (0, 1, 2):
            assert hashlib.sha256(oracle.parse(t, mode)[1].encode()).hexdigest() == row["sha256"][mode], (row["index"], mode)


def test_edge_cases(oracle, emu):
    stats = assert_parity(oracle, emu, cases.all_cases())
    assert stats["sequential"] > 0      # the recovery path is exercised
    assert stats["sequential"] < len(cases.all_cases()) // 2


def test_statement_classes(oracle, emu):
    """Record templates: statements of one shape share the grammar work; what must stay different does."""
    assert_parity(oracle, emu, cases.class_cases())
    # literal digits are not part of a class: 3,000 statements with fresh immediates, offsets and hex floats are a
    # handful of classes, and all but their representatives are instantiated from templates
    rng = random.Random(3)
    stmts = []
    for i in range(1000):
        stmts.append("mov.u32 %%r%d, %d;" % (i % 7, rng.randrange(-2**31, 2**31)))
        stmts.append("ld.global.f32 %%f%d, [%%rd%d+%d];" % (i % 5, i % 3, 4 * rng.randrange(1024)))
        stmts.append("fma.rn.f32 %%f1, %%f2, %%f3, 0f%08X;" % rng.randrange(2**32))
    text = cases.body("\n".join(stmts))
    stats = assert_parity(oracle, emu, [text], modes=(0,))
    assert stats["classes"] < 40, stats
    assert stats["untemplated"] < 60, stats


def test_bulk_initialisers(oracle, emu):
    """Initialiser lists long enough for the element-parallel path, regular and irregular."""
    texts = cases.bulk_cases()
    stats = assert_parity(oracle, emu, texts, modes=(0, 2))
    assert stats["bulk"] >= len(texts)      # every module has at least one statement that long


def test_nested_damage_and_divergence(oracle, emu):
    texts = cases.nested_damage_cases()
    assert_parity(oracle, emu, texts)
    verdicts = [oracle.parse(t, 0)[1].split("\n")[1] for t in texts]
    assert verdicts[0] == "status: Err" and verdicts[-1] == "status: ReferenceDiverges", verdicts


def test_materialised_tree_prints_the_same_text(oracle, emu, monkeypatch):
    """The materialiser (records -> tree) and its printer against the record reader and the oracle, on every edge case
    in all three modes, the class cases, nested damage and small corpora."""
    monkeypatch.setenv("PTXFE_EMU_TREE", "1")
    assert_parity(oracle, emu, cases.all_cases())
    assert_parity(oracle, emu, cases.class_cases() + cases.nested_damage_cases() + [cases.negative_decimal_side_file()], modes=(0, 1))
    mods = corpus.config3(total_bytes=200 << 10, n_funcs=8, n_labels=100) + corpus.config1(n_modules=8, total_bytes=256 << 10) + \
        corpus.config2(n_arrays=2, n_init=3000, n_consts=500)
    assert_parity(oracle, emu, mods, modes=(0,))


def test_sharded_over_two_host_threads(oracle, emu):
    """The library's multi-device entry point splits a batch with byte-balanced greedy partitioning, parses every shard
    on a host thread of its own and hands the modules back in the caller's order: the same partitioner and the same
    gather on two (and three) host threads here, every dump against the oracle's."""
    texts = cases.all_cases()[:60] + [t.decode() for t in corpus.config1(n_modules=24, total_bytes=1 << 20)] + cases.nested_damage_cases()[:6]
    for n_parts in (2, 3):
        dumps, part_of, part_bytes = emu.parse_multi(texts, n_parts)
        assert len(dumps) == len(texts)
        for t, d in zip(texts, dumps):
            assert oracle.parse(t, 0)[1] == d
        assert set(part_of) == set(range(n_parts))
        sizes = [len(t.encode()) for t in texts]
        assert sum(part_bytes) == sum(sizes)
        assert max(part_bytes) - min(part_bytes) <= max(sizes)      # greedy: no part is more than one module above another
    assert emu.parse_multi([], 2)[0] == []
    assert emu.parse_multi(texts[:1], 4)[1] == [0]


def test_negative_decimal_side_file(oracle, emu):
    assert_parity(oracle, emu, [cases.negative_decimal_side_file()])


def test_class_store_capacity_and_long_names(oracle, emu):
    assert_parity(oracle, emu, cases.capacity_cases(), modes=(0,))


def test_edge_cases_in_reverse_thread_order(oracle, emu, monkeypatch):
    """Every parallel-for of the pipeline run backwards: no step may depend on the order of its threads."""
    monkeypatch.setenv("PTXFE_EMU_ORDER", "reverse")
    stats = assert_parity(oracle, emu, cases.all_cases())
    assert stats["pass_mismatch"] == 0
    mods = corpus.config3(total_bytes=200 << 10, n_funcs=8, n_labels=100) + corpus.config1(n_modules=8, total_bytes=256 << 10, pool_lines=4000)
    assert_parity(oracle, emu, mods, modes=(0,))


def test_lexer_tokens_match_oracle(oracle, emu):
    rng = random.Random(7)
    pieces = ["add", ".f32", "%r1", ",", ";", " ", "\n", "\t", "// c\n", "/* x */", "/*", "*/", "\"s\"", "\"", "0f3F800000", "0x1F",
              "1.5e-3", "1.5e", ".5", "12U", ".L2::cache_hint", ".shared::cta", ".shared::", ".param::funcx", "::", ":", "+", "-", "{",
              "}", "[", "]", "(", ")", "<", ">", "=", "@", "!", "|", "#", "~", "$L_1", "_a", "%", "$", ".", "..", ".1d", ".2dx", "WARP_SZ",
              "0d3FF0000000000000", "0f123", "abc" * 60, "/", "*", "é", "\r\n", "a.b", "a:b", "1e5", "0X", "0xU", "09",
              "0x1F_a", "0f3F800000U", "0f3F80000_", "12Ua", "00x1F", "0x" + "A" * 20, "0x" + "b" * 16, "5U", "0F3f800000", "0D3FF0000000000000", "0d3FF000000000000", "0x1$"]
    for trial in range(300):
        n = rng.randrange(1, 80)
        text = "".join(rng.choice(pieces) for _ in range(n))
        ot, oe = oracle.lex(text)
        et, ee = emu.lex(text)
        assert ot == et, (text, ot[:5], et[:5])
        assert oe == ee, text
    # tokens and comments that straddle chunk boundaries at every offset
    for pad in range(0, 140):
        text = " " * pad + "ld.global.L2::cache_hint.v4.f32 {%f1,%f2,%f3,%f4}, [%rd1+16]; /* c */ 0f3F800000 1.25e-3 // e\n\"str\""
        assert oracle.lex(text) == emu.lex(text), pad
    for size in (0, 1, 127, 128, 129, 255, 256, 257):
        text = ("a" * size)
        assert oracle.lex(text) == emu.lex(text)
        text = "/*" + "x" * size + "*/b"
        assert oracle.lex(text) == emu.lex(text)


def test_dense_tiles_lex_like_the_oracle(oracle, emu):
    """Tiles that the emit step takes in several passes, and tiles that overflow its lists of numbers and keyword candidates."""
    for text in cases.dense_token_texts():
        ot, oe = oracle.lex(text)
        et, ee = emu.lex(text)
        assert ot == et, text[:40]
        assert oe == ee, text[:40]


def test_corpora_small(oracle, emu):
    sets = {
        "config0": corpus.config0(n_kernels=3, n_instr=400),
        "config1": corpus.config1(n_modules=24, total_bytes=1 << 20, pool_lines=8000),
        "config2": corpus.config2(n_arrays=4, n_init=3000, n_consts=3000),
        "config3": corpus.config3(total_bytes=400 << 10, n_funcs=8, n_labels=200),
    }
    for name, mods in sets.items():
        for m in mods:
            st, dump = oracle.parse(m)
            assert st == 0, (name, dump[-400:])     # every generated statement is one the reference accepts
        stats = assert_parity(oracle, emu, mods, modes=(0,))
        assert stats["sequential"] == 0, name       # clean input never takes the recovery path


def test_mutated_modules(oracle, emu):
    """Random token-level damage: the data-parallel path or the sequential recovery must still agree with the oracle."""
    rng = random.Random(11)
    base = corpus.config1(n_modules=4, total_bytes=24 << 10, pool_lines=2000) + corpus.config3(total_bytes=24 << 10, n_funcs=4, n_labels=20)
    junk = [";", "{", "}", ":", ",", "(", ")", "foo", ".bar", "[", "]", "@", "\"", "/*", "#", ".global", ".entry", ".func", "<", "0x", "-", "ret", ""]
    texts = []
    for t in base:
        s = t.decode()
        for _ in range(12):
            k = rng.randrange(1, 4)
            m = s
            for _ in range(k):
                pos = rng.randrange(len(m))
                if rng.random() < 0.5:
                    m = m[:pos] + rng.choice(junk) + m[pos:]
                else:
                    m = m[:pos] + m[pos + rng.randrange(1, 12):]
            texts.append(m)
    assert_parity(oracle, emu, texts)


def test_damage_is_confined_to_the_tail(oracle, emu):
    """The sequential parser takes over at the top-level directive with the first damage, not at the module's header."""
    n_sequential = 0
    for text, front in cases.confined_damage_cases():
        for mode in (0, 1, 2):
            dumps, st = emu.parse([text], mode)
            assert dumps[0] == oracle.parse(text, mode)[1], (text[-300:], mode)
            assert st["sequential_tokens"] <= (1.0 - front) * st["tokens"] + 64, (front, st)
            n_sequential += st["sequential"]
    assert n_sequential >= 30


def test_long_runs_of_soft_bytes_stay_linear(oracle, emu):
    """Runs of identifier characters, dots, colons, sigils and signs a few hundred KiB long, with and without lexer
    errors inside: the same tokens and errors as the oracle, in time that grows with the length (the chunk lexer's
    rewind to the start of such a run used to make the error pass quadratic: 4.6 s for the 256 KiB case below, 18 s
    for twice that)."""
    import time
    n = 256 << 10
    runs = ["a" * n, "%." * (n // 2), "::" * (n // 2), ".1" * (n // 2), "%" * n, "1." * (n // 2), "+-" * (n // 2), "a.b::" * (n // 5)]
    for run in runs:
        text = cases.HEADER + ".visible .entry k()\n{\nmov.u32 %r1, " + run + ";\nret;\n}\n"
        for mode in (1, 2):
            t0 = time.time()
            dumps, _ = emu.parse([text], mode)
            took = time.time() - t0
            assert dumps[0] == oracle.parse(text, mode)[1], (run[:8], mode)
            assert took < 3.0, (run[:8], mode, took)


def test_numbers_across_tile_ends(oracle, emu):
    """Every kind of numeric literal at every position around the end of an 8 KiB lexer tile: the number rules run on
    the tile's copy of the text only when the number and what the rules look at behind it lie inside the tile."""
    for t in cases.numbers_across_tile_ends():          # one module per batch: the module begins where a tile begins
        assert emu.parse([t], 1)[0][0] == oracle.parse(t, 1)[1], t[-80:]


def test_stray_tokens_need_no_sequential_parse(oracle, emu):
    text = corpus.config1(n_modules=1, total_bytes=300000)[0]
    for t in cases.stray_token_modules(text):
        for mode in (0, 1):
            dumps, st = emu.parse([t], mode)
            assert dumps[0] == oracle.parse(t, mode)[1]
            assert st["sequential"] == 0


def test_long_sequential_tail_is_refused(oracle, emu, monkeypatch):
    """The one-thread parser does not take on a tail above its token limit: the module's verdict says so."""
    text, front = cases.confined_damage_cases()[1]
    monkeypatch.setenv("PTXFE_SEQ_MAX_TOKENS", "1000")
    dumps, st = emu.parse([text, cases.HEADER + ".global .u32 fine;\n"], 1)
    assert dumps[0] == "mode: unchecked\nstatus: SequentialPathRefused\nerrors: 0\n"
    assert dumps[1] == oracle.parse(cases.HEADER + ".global .u32 fine;\n", 1)[1]
    monkeypatch.setenv("PTXFE_SEQ_MAX_TOKENS", "100000")
    assert emu.parse([text], 1)[0][0] == oracle.parse(text, 1)[1]


def test_reference_fixtures(oracle, emu):
    texts = list(reference_fixtures.texts().values())
    assert len(texts) >= 240
    assert_parity(oracle, emu, texts)


def _f64_bits(s):
    return struct.unpack("<Q", struct.pack("<d", float(s)))[0]


def test_decimal_to_f64_bit_exact(emu):
    rng = random.Random(3)
    fixed = ["1.5", ".5", "0.1", "1.7976931348623157e308", "1.7976931348623159e308", "4.9e-324", "2.4703282292062327e-324",
             "2.4703282292062328e-324", "1.0e400", "1.0e-400", "9007199254740993.0", "9007199254740992.9999999999999999999999",
             "2.2250738585072011e-308", "2.2250738585072014e-308", "8.98846567431158e307", "0.0", "000.000e5",
             "123456789012345678901234567890.5e-10"]
    for s in fixed:
        assert emu.parse_f64(s) == _f64_bits(s), s
    for _ in range(20000):
        k = rng.random()
        if k < 0.3:
            s = "%.8e" % abs(rng.gauss(0, 1))
        elif k < 0.6:
            s = "%.16e" % abs(rng.gauss(0, 1))
        elif k < 0.8:
            s = "%d.%de%d" % (rng.randrange(10 ** rng.randrange(1, 25)), rng.randrange(10 ** rng.randrange(1, 30)), rng.randrange(-340, 300))
        else:
            x = struct.unpack("<d", struct.pack("<Q", rng.getrandbits(63)))[0]
            if x != x or x == float("inf"):
                continue
            s = "%.17e" % x
        assert emu.parse_f64(s) == _f64_bits(s), s
    # exact halfway points between adjacent doubles and their neighbours (many more than 19 digits)
    from decimal import Decimal, getcontext
    getcontext().prec = 1200
    for _ in range(300):
        bits = rng.getrandbits(62) | (rng.randrange(1, 2046) << 52) if rng.random() < 0.8 else rng.getrandbits(52)
        bits &= (1 << 63) - 1
        if (bits >> 52) == 2047:
            continue
        x = struct.unpack("<d", struct.pack("<Q", bits))[0]
        y = struct.unpack("<d", struct.pack("<Q", bits + 1))[0]
        if y == float("inf"):
            continue
        mid = (Decimal(x) + Decimal(y)) / 2
        for delta in (Decimal(0), Decimal(1), Decimal(-1)):
            d = mid + delta * Decimal(10) ** (mid.adjusted() - 60)
            s = format(d, "e")
            if "." not in s:
                s = s.replace("e", ".0e")
            s = s.replace("e+", "e")
            assert emu.parse_f64(s) == _f64_bits(s), s


def test_greedy_partition_is_balanced():
    rng = np.random.default_rng(5)
    sizes = np.clip(rng.lognormal(np.log(128 * 1024), 1.0, 4096), 4096, 8 << 20).astype(np.int64)
    for n in (1, 2, 4, 8):
        parts = corpus.greedy_partition(sizes, n)
        assert sorted(i for p in parts for i in p) == list(range(len(sizes)))
        loads = [int(sizes[p].sum()) for p in parts]
        assert max(loads) - min(loads) <= sizes.max()
