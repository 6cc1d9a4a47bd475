"""Seeded synthetic PTX corpora with the shapes of the five benchmark configurations.

They stand in for real fatbin PTX (none ships with the reference beyond its small test fixtures): the statement mix,
operand ranges, literal forms, module-size distribution, comment density and nesting follow the configuration text;
every statement form used here is one the reference parser accepts (tests check the generators against the oracle).
Generation is pool based - a few hundred thousand i.i.d. statement lines are drawn once and modules are cut from
them - so that a gigabyte of text takes seconds, not minutes.
"""
import numpy as np

TARGETS = ("sm_80", "sm_86", "sm_90")


def _hexf(rng, n):
    v = rng.standard_normal(n).astype(np.float32).view(np.uint32)
    return ["0f%08X" % x for x in v]


class LinePool:
    """i.i.d. instruction lines with the config-0 mix (optionally +10 % mma / ld.shared.v4 tiles)."""

    def __init__(self, seed, n_lines=200_000, tiles=False, func_id=0):
        rng = np.random.default_rng(seed)
        r = lambda: "%%r%d" % rng.integers(0, 256)
        rd = lambda: "%%rd%d" % rng.integers(0, 128)
        f = lambda: "%%f%d" % rng.integers(0, 256)
        p = lambda: "%%p%d" % rng.integers(0, 32)
        imm = lambda: str(int(rng.integers(-2**31, 2**31)))
        hexf = _hexf(rng, 4096)
        fimm = lambda: hexf[rng.integers(0, 4096)]
        lines = []
        n_labels = max(1, n_lines // 50)
        for i in range(n_lines):
            if i % 50 == 0:
                lines.append("$L__BB%d_%d:\n" % (func_id, i // 50))
            u = rng.random()
            if tiles:
                if u < 0.05:
                    lines.append("\tmma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%s, %s, %s, %s}, {%s, %s, %s, %s}, {%s, %s}, {%s, %s, %s, %s};\n"
                                 % (f(), f(), f(), f(), r(), r(), r(), r(), r(), r(), f(), f(), f(), f()))
                    continue
                if u < 0.10:
                    lines.append("\tld.shared.v4.b32 {%s, %s, %s, %s}, [%s+%d];\n" % (r(), r(), r(), r(), rd(), 16 * rng.integers(0, 256)))
                    continue
                u = (u - 0.10) / 0.90
            if u < 0.30:
                k = rng.integers(0, 12)
                t = ("s32", "u32", "f32")[k % 3]
                op = ("add", "sub", "mul", "mad")[k // 3]
                reg = f if t == "f32" else r
                last = (fimm() if t == "f32" else imm()) if rng.random() < 0.25 else reg()
                if op in ("add", "sub"):
                    lines.append("\t%s.%s %s, %s, %s;\n" % (op, t, reg(), reg(), last))
                elif op == "mul":
                    lines.append("\tmul%s.%s %s, %s, %s;\n" % ("" if t == "f32" else ".lo", t, reg(), reg(), last))
                else:
                    lines.append("\tmad%s.%s %s, %s, %s, %s;\n" % ("" if t == "f32" else ".lo", t, reg(), reg(), reg(), last))
            elif u < 0.45:
                lines.append("\tfma.rn.f32 %s, %s, %s, %s;\n" % (f(), f(), f(), fimm() if rng.random() < 0.25 else f()))
            elif u < 0.60:
                k = rng.integers(0, 8)
                space = ("global", "shared")[k & 1]
                t = ("f32", "u32")[(k >> 1) & 1]
                reg = f if t == "f32" else r
                addr = "[%s+%d]" % (rd(), 4 * rng.integers(0, 1024))
                vec = rng.random() < 0.25
                n = (2, 4)[rng.integers(0, 2)]
                val = "{%s}" % ", ".join(reg() for _ in range(n)) if vec else reg()
                v = ".v%d" % n if vec else ""
                if k & 4:
                    lines.append("\tst.%s%s.%s %s, %s;\n" % (space, v, t, addr, val))
                else:
                    lines.append("\tld.%s%s.%s %s, %s;\n" % (space, v, t, val, addr))
            elif u < 0.70:
                k = rng.integers(0, 5)
                if k == 0:
                    lines.append("\tmov.u32 %s, %s;\n" % (r(), imm() if rng.random() < 0.5 else r()))
                elif k == 1:
                    lines.append("\tmov.f32 %s, %s;\n" % (f(), fimm() if rng.random() < 0.5 else f()))
                elif k == 2:
                    lines.append("\tcvt.rn.f32.s32 %s, %s;\n" % (f(), r()))
                elif k == 3:
                    lines.append("\tcvt.rzi.s32.f32 %s, %s;\n" % (r(), f()))
                else:
                    lines.append("\tmov.u64 %s, %s;\n" % (rd(), rd()))
            elif u < 0.78:
                cmp_ = ("lt", "ge", "eq")[rng.integers(0, 3)]
                t = ("s32", "u32", "f32")[rng.integers(0, 3)]
                reg = f if t == "f32" else r
                pr = p()
                lines.append("\tsetp.%s.%s %s, %s, %s;\n" % (cmp_, t, pr, reg(), reg()))
                lines.append("\t@%s bra $L__BB%d_%d;\n" % (pr, func_id, rng.integers(0, n_labels)))
            elif u < 0.83:
                if rng.random() < 0.5:
                    lines.append("\tshfl.sync.bfly.b32 %s|%s, %s, %d, 31, -1;\n" % (r(), p(), r(), 1 << rng.integers(0, 5)))
                else:
                    lines.append("\tbar.sync %d;\n" % rng.integers(0, 16))
            else:
                k = rng.integers(0, 4)
                if k == 0:
                    lines.append("\tand.b32 %s, %s, %s;\n" % (r(), r(), imm() if rng.random() < 0.3 else r()))
                elif k == 1:
                    lines.append("\tor.b32 %s, %s, %s;\n" % (r(), r(), r()))
                elif k == 2:
                    lines.append("\tshl.b32 %s, %s, %d;\n" % (r(), r(), rng.integers(0, 32)))
                else:
                    lines.append("\tselp.f32 %s, %s, %s, %s;\n" % (f(), f(), f(), p()))
        self.lines = [l.encode() for l in lines]
        self.sizes = np.fromiter((len(l) for l in self.lines), dtype=np.int64, count=len(self.lines))
        self.cum = np.concatenate([[0], np.cumsum(self.sizes)])
        self.mean = float(self.sizes.mean())

    def body(self, rng, n_lines):
        o = int(rng.integers(0, len(self.lines) - n_lines)) if n_lines < len(self.lines) else 0
        return b"".join(self.lines[o:o + n_lines])


def _header(target="sm_80"):
    return (".version 7.8\n.target %s\n.address_size 64\n\n" % target).encode()


def _kernel(name, body):
    params = ",\n".join("\t.param .%s %s_param_%d" % ("u64" if i < 4 else "u32", name, i) for i in range(8))
    return (".visible .entry %s(\n%s\n)\n{\n\t.reg .pred %%p<32>;\n\t.reg .b32 %%r<256>;\n\t.reg .f32 %%f<256>;\n\t.reg .b64 %%rd<128>;\n\n"
            % (name, params)).encode() + body + b"\tret;\n}\n\n"


def config0(seed=1000, n_kernels=64, n_instr=2000):
    """One module: 64 entry kernels x 2,000 instructions (~6 MB)."""
    rng = np.random.default_rng(seed)
    pool = LinePool(seed, n_lines=max(4000, n_kernels * n_instr // 8))
    parts = [_header()]
    for k in range(n_kernels):
        parts.append(_kernel("k%d" % k, pool.body(rng, n_instr)))
    return [b"".join(parts)]


def config1_sizes(seed=1001, n_modules=4096, total_bytes=1 << 30):
    """Target byte size of every module of a config-1 batch (cheap; used to partition before generating)."""
    rng = np.random.default_rng(seed)
    sizes = np.clip(rng.lognormal(np.log(128 * 1024), 1.0, n_modules), 4096, 8 << 20)
    return np.clip(sizes * (total_bytes / sizes.sum()), 1024, None)


def config1(seed=1001, n_modules=4096, total_bytes=1 << 30, pool_lines=200_000, indices=None):
    """Fatbin-scale batch: log-normal module sizes (median 128 KiB, clamped to [4 KiB, 8 MiB]) rescaled to
    `total_bytes`, mixed targets, 10 % tensor-core tile statements.  `indices` selects a subset of the batch's
    modules (each module's content depends only on the seed and its index)."""
    pool = LinePool(seed, n_lines=pool_lines, tiles=True)
    sizes = config1_sizes(seed, n_modules, total_bytes)
    mods = []
    per_kernel = 2000
    for m in (range(n_modules) if indices is None else indices):
        rng = np.random.default_rng([seed, m])
        n_lines = max(8, int(sizes[m] / pool.mean))
        parts = [_header(TARGETS[int(rng.integers(0, 3))])]
        k = 0
        while n_lines > 0:
            take = min(per_kernel, n_lines)
            parts.append(_kernel("m%d_k%d" % (m, k), pool.body(rng, take)))
            n_lines -= take
            k += 1
        mods.append(b"".join(parts))
    return mods


def config2(seed=1002, n_arrays=16, n_init=4 << 20, n_consts=1 << 20):
    """Literal-heavy data module: .global arrays with comma-separated initialisers (hex and decimal) and
    .f64/.f32 constants as 0d/0f hex and as decimals with 9 or 17 significant digits.  Decimal floats are written
    non-negative: the reference has no rule for '-' in front of a float literal (ptx_parser/src/lib.rs:366-377)."""
    rng = np.random.default_rng(seed)
    parts = [_header()]
    for a in range(n_arrays):
        if a % 2 == 0:
            vals = rng.integers(0, 256, n_init)
            ty = "b8"
        else:
            vals = rng.integers(0, 2**32, n_init)
            ty = "u32"
        hexm = rng.random(n_init) < 0.5
        strs = np.where(hexm, np.char.add("0x", np.char.upper(np.vectorize(lambda v: "%x" % v, otypes=[str])(vals))), vals.astype(str))
        # decimals must not start with '0' unless they are zero itself (a leading 0 means octal, lib.rs:235)
        parts.append((".global .align 16 .%s arr%d[%d] = {" % (ty, a, n_init)).encode())
        parts.append(", ".join(strs.tolist()).encode())
        parts.append(b"};\n")
    x = rng.standard_normal(n_consts)
    kind = rng.integers(0, 5, n_consts)
    out = []
    for i in range(n_consts):
        k = kind[i]
        if k == 0:
            out.append(".global .f64 c%d = 0d%016X;\n" % (i, np.float64(x[i]).view(np.uint64)))
        elif k == 1:
            out.append(".global .f32 c%d = 0f%08X;\n" % (i, np.float32(x[i]).view(np.uint32)))
        elif k == 2:
            out.append(".global .f64 c%d = %s;\n" % (i, _dec(abs(x[i]), 17)))
        elif k == 3:
            out.append(".global .f32 c%d = %s;\n" % (i, _dec(abs(x[i]), 9)))
        else:
            out.append(".const .f64 c%d = %s;\n" % (i, _dec(abs(x[i]) * 10.0 ** int(rng.integers(-30, 30)), 17)))
    parts.append("".join(out).encode())
    return [b"".join(parts)]


def _dec(v, digits):
    s = "%.*e" % (digits - 1, v)      # d.ddddde+XX : matches [0-9]*\.[0-9]+([eE][-+]?[0-9]+)?
    return s


def config3(seed=1003, total_bytes=256 << 20, n_funcs=64, n_labels=20000):
    """Debug-info and structure-heavy module: .file table, .loc before every instruction, // and /* */ comments
    (~40 % of bytes), { } scopes nested 1-32 deep with scoped .reg declarations, call sequences to .func
    declarations made earlier in the file, forward and backward branches."""
    rng = np.random.default_rng(seed)
    pool = LinePool(seed, n_lines=100_000)
    parts = [_header()]
    for i in range(256):
        parts.append(('.file %d "/build/src/dir%d/file%d.cu"\n' % (i + 1, i % 16, i)).encode())
    for j in range(n_funcs):
        parts.append((".func (.param .b32 func_retval0) f%d(.param .b32 f%d_param_0)\n;\n" % (j, j)).encode())
    comments = [("\t// %s\n" % ("inlined from helper_%d at line %d, column %d" % (i, i * 7 % 1000, i % 80))).encode() for i in range(512)]
    comments += [("\t/* %s */\n" % ("block comment %d: loop body, unrolled by %d * stride */ /* second part" % (i, i % 8))).encode() for i in range(512)]
    size = sum(len(p) for p in parts)
    kid = 0
    label_budget = n_labels
    per_kernel_target = max(64 << 10, total_bytes // 64)
    while size < total_bytes:
        body = []
        depth = 0
        bsize = 0
        line_no = 1
        lbl = 0
        while bsize < per_kernel_target:
            u = rng.random()
            pad = b"\t" * depth
            if u < 0.04 and depth < 32:
                want = int(rng.integers(1, 33))
                while depth < want:
                    s = pad + b"{\n" + pad + b"\t.reg .b32 %%t%d;\n" % depth
                    s = s.replace(b"%%", b"%")
                    body.append(s)
                    bsize += len(s)
                    depth += 1
                    pad = b"\t" * depth
                continue
            if u < 0.08 and depth > 0:
                k = int(rng.integers(1, depth + 1))
                for _ in range(k):
                    depth -= 1
                    s = b"\t" * depth + b"}\n"
                    body.append(s)
                    bsize += len(s)
                continue
            if u < 0.28:
                j = int(rng.integers(0, n_funcs))
                s = (".loc %d %d %d\n{\n.param .b32 p0;\nst.param.b32 [p0+0], %%r%d;\n.param .b32 rv;\ncall.uni (rv), f%d, (p0);\nld.param.b32 %%r%d, [rv+0];\n}\n"
                     % (1 + line_no % 256, line_no, 1 + line_no % 40, rng.integers(0, 256), j, rng.integers(0, 256))).encode()
            elif u < 0.30 and label_budget > 0:
                s = ("$L_dbg_%d_%d:\n" % (kid, lbl)).encode()
                lbl += 1
                label_budget -= 1
            elif u < 0.33 and lbl > 0:
                s = (".loc %d %d %d\nbra $L_dbg_%d_%d;\n" % (1 + line_no % 256, line_no, 3, kid, rng.integers(0, lbl + 4))).encode()
            else:
                s = (".loc %d %d %d\n" % (1 + line_no % 256, line_no, 1 + line_no % 40)).encode() + pool.lines[int(rng.integers(0, len(pool.lines)))]
                if s.endswith(b":\n"):     # the pool holds labels too; keep them unique per kernel
                    s = (".loc %d %d %d\n\tbar.sync 0;\n" % (1 + line_no % 256, line_no, 2)).encode()
            line_no += 1
            c = comments[int(rng.integers(0, len(comments)))] if rng.random() < 0.75 else b""
            body.append(s)
            body.append(c)
            bsize += len(s) + len(c)
        while depth > 0:
            depth -= 1
            body.append(b"\t" * depth + b"}\n")
        k = _kernel("dbg%d" % kid, b"".join(body))
        parts.append(k)
        size += len(k)
        kid += 1
    return [b"".join(parts)]


def greedy_partition(sizes, n_parts):
    """Byte-balanced greedy partitioning: largest module first onto the least-loaded part.
    Returns a list of index lists, one per part."""
    order = np.argsort(-np.asarray(sizes, dtype=np.int64), kind="stable")
    loads = [0] * n_parts
    parts = [[] for _ in range(n_parts)]
    import heapq
    heap = [(0, i) for i in range(n_parts)]
    heapq.heapify(heap)
    for idx in order:
        load, p = heapq.heappop(heap)
        parts[p].append(int(idx))
        load += int(sizes[idx])
        loads[p] = load
        heapq.heappush(heap, (load, p))
    return parts
