"""ctypes binding of the host emulation backend (tests/emu/libptxfe_emu.so): the product's pipeline step bodies run
sequentially on the CPU.  Test infrastructure only."""
import ctypes
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO = os.path.join(ROOT, "tests", "emu", "libptxfe_emu.so")
_cached = None


class Emu:
    def __init__(self, lib):
        self.lib = lib
        lib.emu_parse.restype = ctypes.c_void_p
        lib.emu_parse.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint32,
                                  ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
        lib.emu_parse_multi.restype = ctypes.c_void_p
        lib.emu_parse_multi.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint32, ctypes.c_uint32,
                                        ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint32),
                                        ctypes.POINTER(ctypes.c_uint64)]
        lib.emu_lex.restype = ctypes.c_void_p
        lib.emu_lex.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
        lib.emu_free.argtypes = [ctypes.c_void_p]
        lib.emu_parse_f64.restype = ctypes.c_uint64
        lib.emu_parse_f64.argtypes = [ctypes.c_char_p, ctypes.c_uint32]

    def parse(self, texts, mode=0):
        """-> (list of dumps, stats dict)"""
        texts = [t.encode() if isinstance(t, str) else t for t in texts]
        n = len(texts)
        arr = (ctypes.c_char_p * n)(*texts)
        lens = (ctypes.c_uint64 * n)(*[len(t) for t in texts])
        ol = ctypes.c_uint64()
        st = (ctypes.c_uint64 * 16)()
        p = self.lib.emu_parse(arr, lens, n, mode, ctypes.byref(ol), st)
        s = ctypes.string_at(p, ol.value)
        self.lib.emu_free(p)
        dumps = [x.decode("utf-8", "replace") for x in s.split(b"\0")[:-1]]
        return dumps, dict(tokens=st[0], units=st[1], words=st[2], errors=st[3], sequential=st[4], pass_mismatch=st[5], bulk=st[6], untemplated=st[7], classes=st[8], sequential_tokens=st[9])

    def parse_multi(self, texts, n_parts, mode=0):
        """Sharded over n_parts host threads with the product's partitioner -> (dumps in the caller's order, shard of
        every module, bytes per shard)."""
        texts = [t.encode() if isinstance(t, str) else t for t in texts]
        n = len(texts)
        arr = (ctypes.c_char_p * n)(*texts)
        lens = (ctypes.c_uint64 * n)(*[len(t) for t in texts])
        ol = ctypes.c_uint64()
        part_of = (ctypes.c_uint32 * max(1, n))()
        part_bytes = (ctypes.c_uint64 * n_parts)()
        p = self.lib.emu_parse_multi(arr, lens, n, n_parts, mode, ctypes.byref(ol), part_of, part_bytes)
        s = ctypes.string_at(p, ol.value)
        self.lib.emu_free(p)
        return [x.decode("utf-8", "replace") for x in s.split(b"\0")[:-1]], list(part_of)[:n], list(part_bytes)

    def lex(self, text):
        if isinstance(text, str):
            text = text.encode()
        nt, ne = ctypes.c_uint64(), ctypes.c_uint64()
        p = self.lib.emu_lex(text, len(text), ctypes.byref(nt), ctypes.byref(ne))
        arr = (ctypes.c_uint32 * max(1, nt.value * 3 + ne.value * 2)).from_address(p)
        toks = [(arr[3 * i], arr[3 * i + 1], arr[3 * i + 2]) for i in range(nt.value)]
        errs = [(arr[nt.value * 3 + 2 * i], arr[nt.value * 3 + 2 * i + 1]) for i in range(ne.value)]
        self.lib.emu_free(p)
        return toks, errs

    def parse_f64(self, s):
        b = s.encode()
        return self.lib.emu_parse_f64(b, len(b))


def load():
    global _cached
    if _cached is None:
        import build_helpers
        build_helpers.build()       # only what is out of date
        _cached = Emu(ctypes.CDLL(SO))
    return _cached
