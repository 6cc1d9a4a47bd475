"""zluda_b200 - GPU-resident PTX front end for B200 (sm_100a).

Host-side mirror of the three public entry points of ZLUDA's ``ptx_parser`` crate (ptx_parser/src/lib.rs:392-501)
on top of the C ABI in ``include/ptxfe.h``:

    parse_module_checked(text)    -> ParseResult   (``ok`` is True only for an error-free module, lib.rs:428-468)
    parse_module_unchecked(text)  -> ParseResult   (a module even with recoverable errors, lib.rs:470-501)
    parse_for_errors(text)        -> list of error strings (lib.rs:392-411)

plus the batch form the GPU wants (``Context.parse_batch``): many independent modules per call, as
``zluda_precompile`` feeds the reference from a thread pool (zluda_precompile/src/main.rs:57-64).

Everything runs in hand-written CUDA kernels inside ``libptxfe.so``.  There is no CPU implementation behind this
module: importing it without the built library, or creating a Context without a CUDA device, raises.
"""
import ctypes
import os

import numpy as np

CHECKED, UNCHECKED, ERRORS_ONLY = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libptxfe.so")
_lib = None


class PtxfeError(RuntimeError):
    pass


class Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in (
        "text_bytes", "n_modules", "n_tokens", "n_units", "n_result_words", "n_errors", "n_lex_errors", "n_sequential",
        "n_kernel_launches", "h2d_bytes", "d2h_bytes")] + [(n, ctypes.c_float) for n in (
            "h2d_ms", "kernel_ms", "d2h_ms", "lex_ms", "structure_ms", "decode_ms")] + [(n, ctypes.c_uint64) for n in (
                "n_classes", "n_class_capacity", "n_untemplated", "n_signature_words", "n_signature_capacity", "n_sequential_tokens")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


def lib():
    """The loaded C-ABI library.  Raises if it has not been built (python -m zluda_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise PtxfeError("%s is missing: build it with `python -m zluda_b200.build` (needs nvcc); "
                             "there is no CPU fallback" % _LIB_PATH)
        L = ctypes.CDLL(_LIB_PATH)
        vp, u32, u64 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64
        L.ptxfe_create.argtypes = [ctypes.c_int, ctypes.POINTER(vp)]
        L.ptxfe_destroy.argtypes = [vp]
        L.ptxfe_last_error.argtypes = [vp]
        L.ptxfe_last_error.restype = ctypes.c_char_p
        L.ptxfe_status_str.argtypes = [ctypes.c_int]
        L.ptxfe_status_str.restype = ctypes.c_char_p
        L.ptxfe_parse_batch.argtypes = [vp, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(u64), u32, u32, ctypes.POINTER(vp)]
        L.ptxfe_stage.argtypes = [vp, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(u64), u32]
        L.ptxfe_run.argtypes = [vp, u32]
        L.ptxfe_fetch.argtypes = [vp, ctypes.POINTER(vp)]
        L.ptxfe_batch_free.argtypes = [vp]
        L.ptxfe_batch_size.argtypes = [vp]
        L.ptxfe_batch_size.restype = u32
        L.ptxfe_module_status.argtypes = [vp, u32]
        L.ptxfe_module_error_count.argtypes = [vp, u32]
        L.ptxfe_module_error_count.restype = u32
        L.ptxfe_get_stats.argtypes = [vp, ctypes.POINTER(Stats)]
        L.ptxfe_profile.argtypes = [vp]
        L.ptxfe_profile.restype = ctypes.c_char_p
        L.ptxfe_module_records.argtypes = [vp, u32, ctypes.POINTER(ctypes.POINTER(u32)), ctypes.POINTER(u64), ctypes.POINTER(u64)]
        L.ptxfe_module_dump.argtypes = [vp, u32, ctypes.POINTER(vp), ctypes.POINTER(u64)]
        L.ptxfe_module_dump_hash.argtypes = [vp, u32, ctypes.POINTER(u64)]
        L.ptxfe_free.argtypes = [vp]
        L.ptxfe_lex_module.argtypes = [vp, ctypes.c_char_p, u64, ctypes.POINTER(vp), ctypes.POINTER(u64), ctypes.POINTER(u64)]
        L.ptxfe_batch_materialize.argtypes = [vp, u32, ctypes.POINTER(u64)]
        L.ptxfe_multi_create.argtypes = [ctypes.POINTER(ctypes.c_int), u32, ctypes.POINTER(vp)]
        L.ptxfe_multi_destroy.argtypes = [vp]
        L.ptxfe_multi_last_error.argtypes = [vp]
        L.ptxfe_multi_last_error.restype = ctypes.c_char_p
        L.ptxfe_parse_batch_multi.argtypes = [vp, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(u64), u32, u32, ctypes.POINTER(vp)]
        L.ptxfe_multi_parts.argtypes = [vp]
        L.ptxfe_multi_parts.restype = u32
        L.ptxfe_multi_part_stats.argtypes = [vp, u32, ctypes.POINTER(Stats)]
        L.ptxfe_multi_part_of.argtypes = [vp, u32]
        _lib = L
    return _lib


class Texts:
    """Module texts already converted to the C ABI's (char**, uint64*) form: build once, parse many times."""

    def __init__(self, texts):
        self.buffers = _as_buffers(texts)

    def __len__(self):
        return len(self.buffers[1])


def _as_buffers(texts):
    """-> (keepalive list, char* array, length array).  Accepts bytes, str, or (address, length) pairs."""
    if isinstance(texts, Texts):
        return texts.buffers
    keep, ptrs, lens = [], [], []
    for t in texts:
        if isinstance(t, tuple):
            ptrs.append(ctypes.c_char_p(t[0]))
            lens.append(t[1])
            continue
        if isinstance(t, str):
            t = t.encode()
        keep.append(t)
        ptrs.append(ctypes.cast(ctypes.c_char_p(t), ctypes.c_char_p))
        lens.append(len(t))
    n = len(ptrs)
    return keep, (ctypes.c_char_p * n)(*ptrs), (ctypes.c_uint64 * n)(*lens)


class Batch:
    """Result of one parse call.  Valid until the next call on its Context."""

    def __init__(self, ctx, handle, keep):
        self._ctx, self._h, self._keep = ctx, handle, keep

    def __len__(self):
        return lib().ptxfe_batch_size(self._h)

    def free(self):
        if self._h:
            lib().ptxfe_batch_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def status(self, i):
        return lib().ptxfe_module_status(self._h, i)

    def materialize(self, threads=None):
        """Build (and drop) the tree of every module on `threads` host threads; returns the number of nodes built."""
        n = ctypes.c_uint64()
        st = lib().ptxfe_batch_materialize(self._h, threads or (os.cpu_count() or 1), ctypes.byref(n))
        if st != 0:
            raise PtxfeError("ptxfe_batch_materialize failed")
        return n.value

    def part_of(self, i):
        """The shard (index into the device list) that parsed module i; 0 for a single-device batch."""
        return lib().ptxfe_multi_part_of(self._h, i)

    def error_count(self, i):
        return lib().ptxfe_module_error_count(self._h, i)

    def dump(self, i):
        p = ctypes.c_void_p()
        n = ctypes.c_uint64()
        self._ctx._check(lib().ptxfe_module_dump(self._h, i, ctypes.byref(p), ctypes.byref(n)))
        s = ctypes.string_at(p, n.value).decode("utf-8", "replace")
        lib().ptxfe_free(p)
        return s

    def dump_hash(self, i):
        h = ctypes.c_uint64()
        self._ctx._check(lib().ptxfe_module_dump_hash(self._h, i, ctypes.byref(h)))
        return h.value

    def records(self, i):
        """(uint32 array of module i's records, byte offset of the module in the batch text buffer)"""
        p = ctypes.POINTER(ctypes.c_uint32)()
        n = ctypes.c_uint64()
        base = ctypes.c_uint64()
        self._ctx._check(lib().ptxfe_module_records(self._h, i, ctypes.byref(p), ctypes.byref(n), ctypes.byref(base)))
        if n.value == 0:
            return np.zeros(0, np.uint32), base.value
        return np.ctypeslib.as_array(p, shape=(n.value,)).copy(), base.value

    def errors(self, i):
        lines = self.dump(i).split("\n")
        k = max(j for j, l in enumerate(lines) if l.startswith("errors: "))
        return [l for l in lines[k + 1:] if l]


class Context:
    """One CUDA device, one stream, reusable device arenas (ptxfe_ctx)."""

    def __init__(self, device=0):
        self._h = ctypes.c_void_p()
        st = lib().ptxfe_create(device, ctypes.byref(self._h))
        if st != 0:
            self._h = None
            raise PtxfeError("ptxfe_create(device=%d) failed: %s (a CUDA device is required; there is no CPU path)"
                             % (device, lib().ptxfe_status_str(st).decode()))

    def close(self):
        if self._h:
            lib().ptxfe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st != 0:
            raise PtxfeError("%s: %s" % (lib().ptxfe_status_str(st).decode(), lib().ptxfe_last_error(self._h).decode()))

    def parse_batch(self, texts, mode=CHECKED):
        keep, ptrs, lens = _as_buffers(texts)
        h = ctypes.c_void_p()
        self._check(lib().ptxfe_parse_batch(self._h, ptrs, lens, len(ptrs), mode, ctypes.byref(h)))
        return Batch(self, h, (keep, ptrs, lens))

    # the same in three steps
    def stage(self, texts):
        self._staged = _as_buffers(texts)
        self._check(lib().ptxfe_stage(self._h, self._staged[1], self._staged[2], len(self._staged[1])))

    def run(self, mode=CHECKED):
        self._check(lib().ptxfe_run(self._h, mode))

    def fetch(self):
        h = ctypes.c_void_p()
        self._check(lib().ptxfe_fetch(self._h, ctypes.byref(h)))
        return Batch(self, h, self._staged)

    def stats(self):
        s = Stats()
        lib().ptxfe_get_stats(self._h, ctypes.byref(s))
        return s.as_dict()

    def profile(self):
        """{step name: milliseconds} of the last run (needs PTXFE_PROFILE=1 in the environment at creation)."""
        out = {}
        for line in lib().ptxfe_profile(self._h).decode().split("\n"):
            if line:
                name, ms = line.split()
                out[name] = out.get(name, 0.0) + float(ms)
        return out

    def profile_steps(self):
        """[(step name, milliseconds)] of the last run in launch order (needs PTXFE_PROFILE=1 at creation)."""
        out = []
        for line in lib().ptxfe_profile(self._h).decode().split("\n"):
            if line:
                name, ms = line.split()
                out.append((name, float(ms)))
        return out

    def lex(self, text):
        """Lexer only: ([(kind, start, length)], [(start, length) of lex errors])."""
        if isinstance(text, str):
            text = text.encode()
        p = ctypes.c_void_p()
        nt, ne = ctypes.c_uint64(), ctypes.c_uint64()
        self._check(lib().ptxfe_lex_module(self._h, text, len(text), ctypes.byref(p), ctypes.byref(nt), ctypes.byref(ne)))
        total = nt.value * 3 + ne.value * 2
        arr = (ctypes.c_uint32 * max(total, 1)).from_address(p.value)
        toks = [(arr[3 * i], arr[3 * i + 1], arr[3 * i + 2]) for i in range(nt.value)]
        errs = [(arr[nt.value * 3 + 2 * i], arr[nt.value * 3 + 2 * i + 1]) for i in range(ne.value)]
        lib().ptxfe_free(p)
        return toks, errs


class MultiContext:
    """Several CUDA devices of one machine (ptxfe_multi): a batch is sharded by module, byte-balanced, one host thread
    and one context per device; the returned Batch indexes modules as they were passed."""

    def __init__(self, devices):
        self._h = ctypes.c_void_p()
        arr = (ctypes.c_int * len(devices))(*devices)
        st = lib().ptxfe_multi_create(arr, len(devices), ctypes.byref(self._h))
        if st != 0:
            self._h = None
            raise PtxfeError("ptxfe_multi_create(%s) failed: %s" % (list(devices), lib().ptxfe_status_str(st).decode()))

    def close(self):
        if self._h:
            lib().ptxfe_multi_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st != 0:
            raise PtxfeError("%s: %s" % (lib().ptxfe_status_str(st).decode(), lib().ptxfe_multi_last_error(self._h).decode()))

    def parse_batch(self, texts, mode=CHECKED):
        keep, ptrs, lens = _as_buffers(texts)
        h = ctypes.c_void_p()
        self._check(lib().ptxfe_parse_batch_multi(self._h, ptrs, lens, len(ptrs), mode, ctypes.byref(h)))
        return Batch(self, h, (keep, ptrs, lens))

    def part_stats(self):
        out = []
        for k in range(lib().ptxfe_multi_parts(self._h)):
            s = Stats()
            lib().ptxfe_multi_part_stats(self._h, k, ctypes.byref(s))
            out.append(s.as_dict())
        return out


class ParseResult:
    def __init__(self, ok, dump, errors):
        self.ok, self.dump, self.errors = ok, dump, errors

    def __repr__(self):
        return "ParseResult(ok=%s, errors=%d)" % (self.ok, len(self.errors))


_default_ctx = None


def _ctx():
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context(int(os.environ.get("LOCAL_RANK", "0")))
    return _default_ctx


def _single(text, mode):
    b = _ctx().parse_batch([text], mode)
    r = ParseResult(b.status(0) == 0, b.dump(0), b.errors(0))
    b.free()
    return r


def parse_module_checked(text):
    """Ok only when lexing, parsing and every directive were error-free (ptx_parser/src/lib.rs:428-468)."""
    return _single(text, CHECKED)


def parse_module_unchecked(text):
    """A module even when recoverable errors occurred; the empty module on a lex or module-level failure (lib.rs:470-501)."""
    return _single(text, UNCHECKED)


def parse_for_errors(text):
    """Only the ordered error list; keeps parsing after lex errors (lib.rs:392-411)."""
    return _single(text, ERRORS_ONLY).errors
