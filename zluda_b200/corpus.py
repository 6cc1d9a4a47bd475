"""Seeded synthetic PTX corpora with the shapes of the five benchmark configurations.

They stand in for real fatbin PTX (none ships with the reference beyond its small test fixtures): the statement mix,
operand ranges, literal forms, module-size distribution, comment density and nesting follow the configuration text;
every statement form used here is one the reference parser accepts (tests check the generators against the oracle).
Every statement is drawn independently (fresh registers, fresh int32 immediates, fresh normal(0,1) hex floats): the
generator is plain C (csrc/ptx_corpus.c, built into libptxcorpus.so), so a gigabyte of i.i.d. text takes seconds.
"""
import ctypes
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libptxcorpus.so")
_lib = None


def _gen():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError("%s is missing: build it with `python -m zluda_b200.build`" % _LIB_PATH)
        L = ctypes.CDLL(_LIB_PATH)
        u64, u32, vp, sz = ctypes.c_uint64, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_size_t
        L.ptx_corpus_config0.restype = sz
        L.ptx_corpus_config0.argtypes = [u64, u32, u32, vp, sz]
        L.ptx_corpus_config1_module.restype = sz
        L.ptx_corpus_config1_module.argtypes = [u64, u32, u64, vp, sz]
        L.ptx_corpus_config2.restype = sz
        L.ptx_corpus_config2.argtypes = [u64, u32, u32, u32, vp, sz]
        L.ptx_corpus_config3.restype = sz
        L.ptx_corpus_config3.argtypes = [u64, u64, u32, u32, vp, sz]
        _lib = L
    return _lib


def _render(fn, *args):
    """Call a generator twice: for the size, then into a buffer of that size."""
    n = fn(*args, None, 0)
    buf = ctypes.create_string_buffer(n)
    got = fn(*args, ctypes.addressof(buf), n)
    assert got == n
    return buf.raw


def config0(seed=1000, n_kernels=64, n_instr=2000):
    """One module: 64 entry kernels x 2,000 i.i.d. instructions (~5 MB)."""
    return [_render(_gen().ptx_corpus_config0, seed, n_kernels, n_instr)]


def config1_sizes(seed=1001, n_modules=4096, total_bytes=1 << 30):
    """Target byte size of every module of a config-1 batch (cheap; used to partition before generating)."""
    rng = np.random.default_rng(seed)
    sizes = np.clip(rng.lognormal(np.log(128 * 1024), 1.0, n_modules), 4096, 8 << 20)
    return np.clip(sizes * (total_bytes / sizes.sum()), 1024, None)


def config1_into(blob, seed=1001, n_modules=4096, total_bytes=1 << 30, indices=None, threads=None):
    """Generate the selected modules of a config-1 batch back to back into `blob` (a writable uint8 numpy array, e.g.
    pinned host memory).  Returns [(offset, length)] per module.  A module is at most ~6 % longer than its target."""
    L = _gen()
    sizes = config1_sizes(seed, n_modules, total_bytes)
    idx = list(range(n_modules)) if indices is None else list(indices)
    base = blob.ctypes.data
    cap = blob.nbytes
    # exact sizes first (a dry run of the generator costs about as much as the real one; both are spread over threads)
    threads = threads or min(32, os.cpu_count() or 1)

    def size_of(m):
        return L.ptx_corpus_config1_module(seed, m, int(sizes[m]), None, 0)

    with ThreadPoolExecutor(threads) as ex:
        lens = list(ex.map(size_of, idx))
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    if offs[-1] > cap:
        raise ValueError("blob of %d bytes is too small for %d bytes of text" % (cap, offs[-1]))

    def fill(k):
        got = L.ptx_corpus_config1_module(seed, idx[k], int(sizes[idx[k]]), base + int(offs[k]), lens[k])
        assert got == lens[k]

    with ThreadPoolExecutor(threads) as ex:
        list(ex.map(fill, range(len(idx))))
    return [(int(offs[k]), int(lens[k])) for k in range(len(idx))]


def config1_total_bound(seed=1001, n_modules=4096, total_bytes=1 << 30, indices=None):
    """An upper bound of the bytes config1_into writes for this selection."""
    sizes = config1_sizes(seed, n_modules, total_bytes)
    idx = range(n_modules) if indices is None else indices
    return int(sum(sizes[m] for m in idx) * 1.10) + 4096 * len(list(idx)) + (1 << 20)


def config1(seed=1001, n_modules=4096, total_bytes=1 << 30, pool_lines=None, indices=None):
    """Fatbin-scale batch: log-normal module sizes (median 128 KiB, clamped to [4 KiB, 8 MiB]) rescaled to
    `total_bytes`, mixed targets, 10 % tensor-core tile statements.  `indices` selects a subset of the batch's
    modules (each module's content depends only on the seed, its index and its target size).  `pool_lines` is ignored
    (kept for callers of the earlier pool-based generator)."""
    L = _gen()
    sizes = config1_sizes(seed, n_modules, total_bytes)
    return [_render(L.ptx_corpus_config1_module, seed, m, int(sizes[m])) for m in (range(n_modules) if indices is None else indices)]


def config2(seed=1002, n_arrays=16, n_init=4 << 20, n_consts=1 << 20):
    """Literal-heavy data module: .global arrays with comma-separated initialisers (hex and decimal) and
    .f64/.f32 constants as 0d/0f hex and as decimals with 9 or 17 significant digits."""
    return [_render(_gen().ptx_corpus_config2, seed, n_arrays, n_init, n_consts)]


def config3(seed=1003, total_bytes=256 << 20, n_funcs=64, n_labels=20000):
    """Debug-info and structure-heavy module: .file table, .loc before every instruction, // and /* */ comments
    (~40 % of bytes), { } scopes nested 1-32 deep with scoped .reg declarations, call sequences to .func
    declarations made earlier in the file, forward and backward branches."""
    return [_render(_gen().ptx_corpus_config3, seed, total_bytes, n_funcs, n_labels)]


def greedy_partition(sizes, n_parts):
    """Byte-balanced greedy partitioning: largest module first onto the least-loaded part.
    Returns a list of index lists, one per part."""
    import heapq
    order = np.argsort(-np.asarray(sizes, dtype=np.int64), kind="stable")
    parts = [[] for _ in range(n_parts)]
    heap = [(0, i) for i in range(n_parts)]
    heapq.heapify(heap)
    for idx in order:
        load, p = heapq.heappop(heap)
        parts[p].append(int(idx))
        heapq.heappush(heap, (load + int(sizes[idx]), p))
    return parts
