"""ctypes binding of the CPU oracle (oracle/libptx_oracle.so).  Test infrastructure only."""
import ctypes
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO = os.path.join(ROOT, "oracle", "libptx_oracle.so")

CHECKED, UNCHECKED, ERRORS_ONLY = 0, 1, 2


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.oracle_parse.restype = ctypes.c_void_p
        lib.oracle_parse.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_int,
                                     ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_int)]
        lib.oracle_lex.restype = ctypes.c_void_p
        lib.oracle_lex.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64),
                                   ctypes.POINTER(ctypes.c_uint64)]
        # text as an address: bytes objects and raw buffers (pinned host memory) are both accepted
        lib.oracle_parse_only.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_uint64),
                                          ctypes.POINTER(ctypes.c_uint64)]
        lib.oracle_dump_hash.restype = ctypes.c_uint64
        lib.oracle_dump_hash.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        lib.oracle_free.argtypes = [ctypes.c_void_p]
        lib.oracle_token_text.restype = ctypes.c_char_p

    def parse(self, text, mode=CHECKED):
        """-> (status, dump).  status 0 = a module was returned."""
        if isinstance(text, str):
            text = text.encode()
        n = ctypes.c_uint64()
        st = ctypes.c_int()
        p = self.lib.oracle_parse(text, len(text), mode, ctypes.byref(n), ctypes.byref(st))
        s = ctypes.string_at(p, n.value).decode("utf-8", "replace")
        self.lib.oracle_free(p)
        return st.value, s

    def dump_hash(self, text, mode=CHECKED):
        """64-bit FNV-1a of the dump of `text` (bytes, or an (address, length) pair)."""
        if isinstance(text, tuple):
            return self.lib.oracle_dump_hash(text[0], text[1], mode, None)
        if isinstance(text, str):
            text = text.encode()
        return self.lib.oracle_dump_hash(ctypes.cast(ctypes.c_char_p(text), ctypes.c_void_p), len(text), mode, None)

    def dump_hashes(self, texts, mode=CHECKED, threads=None):
        """The same for many modules, one per task over a thread pool (the library call releases the GIL)."""
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(threads or min(32, os.cpu_count() or 1)) as ex:
            return list(ex.map(lambda t: self.dump_hash(t, mode), texts))

    def errors(self, text, mode=CHECKED):
        dump = self.parse(text, mode)[1]
        lines = dump.split("\n")
        i = max(k for k, l in enumerate(lines) if l.startswith("errors: "))
        return [l for l in lines[i + 1:] if l]

    def lex(self, text):
        """-> ([(kind, start, length)], [(start, length)])"""
        if isinstance(text, str):
            text = text.encode()
        nt = ctypes.c_uint64()
        ne = ctypes.c_uint64()
        p = self.lib.oracle_lex(text, len(text), ctypes.byref(nt), ctypes.byref(ne))
        arr = (ctypes.c_uint32 * (nt.value * 3 + ne.value * 2)).from_address(p)
        toks = [(arr[3 * i], arr[3 * i + 1], arr[3 * i + 2]) for i in range(nt.value)]
        base = nt.value * 3
        errs = [(arr[base + 2 * i], arr[base + 2 * i + 1]) for i in range(ne.value)]
        self.lib.oracle_free(p)
        return toks, errs

    def token_text(self, kind):
        return self.lib.oracle_token_text(kind).decode()

    def schema_ok(self):
        return bool(self.lib.oracle_schema_ok())


_cached = None


def load():
    global _cached
    if _cached is None:
        import build_helpers
        build_helpers.build()       # only what is out of date
        _cached = Oracle(ctypes.CDLL(SO))
    return _cached
