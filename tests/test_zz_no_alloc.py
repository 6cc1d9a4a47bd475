"""ptxfe_lex_device_noalloc: the lexer for callers that must not allocate device memory.

Such callers exist around this library: a host that has handed the whole device heap to another component, code
running where the CUDA allocator may not be entered, or a process whose device memory is exhausted.  They pass the
text and the token table themselves; the library's only working memory is a fixed array inside its own image.  This
test calls the entry point through the C ABI on two inputs in a row (the second shorter, so that anything left behind
by the first call would show) and requires exactly the token table that the ordinary lexer entry point returns.
It is collected last so that a failure here cannot hide the result of any other test."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _lex_noalloc(lib, torch, text, capacity):
    raw = np.frombuffer(text, dtype=np.uint8)
    d_text = torch.from_numpy(raw.copy()).cuda()
    d_tokens = torch.zeros(capacity * 2, dtype=torch.int32, device="cuda")
    d_counts = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    st = lib.ptxfe_lex_device_noalloc(0, ctypes.c_void_p(d_text.data_ptr()), ctypes.c_uint64(len(text)),
                                      ctypes.c_void_p(d_tokens.data_ptr()), ctypes.c_uint64(capacity),
                                      ctypes.c_void_p(d_counts.data_ptr()), ctypes.c_void_p(0))
    assert st == 0
    torch.cuda.synchronize()
    n_tok, n_err = [int(x) for x in d_counts.cpu().numpy().astype(np.uint32)]
    words = d_tokens.cpu().numpy().view(np.uint32)[: 2 * min(n_tok, capacity)].reshape(-1, 2)
    toks = [(int(w[1] >> 16), int(w[0]), int(w[1] & 0xFFFF)) for w in words]
    return toks, n_tok, n_err


def test_allocation_free_lexer_matches_the_ordinary_one():
    import torch
    import zluda_b200
    from zluda_b200 import corpus
    lib = zluda_b200.lib()
    lib.ptxfe_lex_device_noalloc.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64,
                                             ctypes.c_void_p, ctypes.c_void_p]
    ctx = zluda_b200.Context(0)
    first = corpus.config3(total_bytes=3 << 20, n_funcs=8, n_labels=300)[0]          # comments, strings, nesting
    second = corpus.config1(n_modules=1, total_bytes=200 << 10, pool_lines=4000)[0] + b"\n# /* open"   # shorter, with lex errors
    for text in (first, second):
        want_toks, want_errs = ctx.lex(text)
        got, n_tok, n_err = _lex_noalloc(lib, torch, text, len(want_toks) + 16)
        assert n_tok == len(want_toks)
        assert n_err == len(want_errs)
        assert got == want_toks
    # a table that is too small is filled up to its capacity and the full count is still reported
    got, n_tok, _ = _lex_noalloc(lib, torch, second, 100)
    assert len(got) == 100 and n_tok == len(ctx.lex(second)[0]) and got == ctx.lex(second)[0][:100]
    # the claim in the name: device memory in use is the same before and after calls (the buffers are the test's own)
    edge = (b"add.s32 %r1, %r2, 0x1F; // c\n" * ((16 << 20) // 29 + 1))
    for n in ((16 << 20) - 1, 16 << 20):
        text = edge[:n]
        want_toks, want_errs = ctx.lex(text)
        raw = torch.from_numpy(np.frombuffer(text, dtype=np.uint8).copy()).cuda()
        d_tokens = torch.zeros((len(want_toks) + 16) * 2, dtype=torch.int32, device="cuda")
        d_counts = torch.full((2,), -1, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        st = lib.ptxfe_lex_device_noalloc(0, ctypes.c_void_p(raw.data_ptr()), ctypes.c_uint64(n), ctypes.c_void_p(d_tokens.data_ptr()),
                                          ctypes.c_uint64(len(want_toks) + 16), ctypes.c_void_p(d_counts.data_ptr()), ctypes.c_void_p(0))
        torch.cuda.synchronize()
        assert st == 0 and torch.cuda.mem_get_info()[0] == free_before
        assert [int(x) for x in d_counts.cpu().numpy().astype(np.uint32)] == [len(want_toks), len(want_errs)]
        words = d_tokens.cpu().numpy().view(np.uint32)[: 2 * len(want_toks)].reshape(-1, 2)
        step = max(1, len(want_toks) // 5000)
        assert [(int(w[1] >> 16), int(w[0]), int(w[1] & 0xFFFF)) for w in words[::step]] == want_toks[::step]
    # one run of word characters longer than the look-back bound: refused through the counts, quickly
    long_run = b"mov.u32 %r1, " + b"a" * (200 << 10) + b";"
    got, n_tok, n_err = _lex_noalloc(lib, torch, long_run, 64)
    assert n_tok == 0xFFFFFFFF and n_err == 0xFFFFFFFF
    # inputs beyond the fixed working memory are refused
    big = torch.zeros(8, dtype=torch.uint8, device="cuda")
    st = lib.ptxfe_lex_device_noalloc(0, ctypes.c_void_p(big.data_ptr()), ctypes.c_uint64((16 << 20) + 1),
                                      ctypes.c_void_p(big.data_ptr()), ctypes.c_uint64(0), ctypes.c_void_p(big.data_ptr()), ctypes.c_void_p(0))
    assert st == 3
    ctx.close()
