#!/usr/bin/env python3
"""Generate ptx_tables.h (token, pattern, selection and schema tables) from ptx.def.

The instruction-pattern algorithm follows the reference's proc macro so that the generated decoder picks
patterns and orders modifiers exactly as ptx_parser does:
  * rule resolution, Direct vs Indirect modifiers      ptx_parser_macros/src/lib.rs:233-304
  * ordered (postfix) vs free-order modifiers          ptx_parser_macros/src/lib.rs:18-28, 306-340
  * the per-opcode if/else-if selection chain          ptx_parser_macros/src/lib.rs:35-150, 505-538
  * variant naming (.param::func -> ParamFunc, .bf16 -> BF16)   ptx_parser_macros_impl/src/parser.rs:350-381

Usage:
  gen_tables.py --out DIR [--out DIR2 ...]              write ptx_tables.h into each DIR
  gen_tables.py --check-against path/to/ptx_parser/src/lib.rs
        parse the reference's derive_parser! body and require identical opcodes, patterns, rules, modifier
        slots and selection chains (exit 1 with a diff otherwise)
  gen_tables.py --dump-chains                           print the selection chains (for inspection)
"""
import argparse
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

POSTFIX_MODIFIERS = {
    ".v2", ".v4", ".v8", ".s8", ".s16", ".s16x2", ".s32", ".s64", ".u8", ".u16", ".u16x2", ".u32", ".u64",
    ".f16", ".f16x2", ".f32", ".f64", ".b8", ".b16", ".b32", ".b64", ".b128", ".pred", ".bf16", ".bf16x2",
    ".e4m3", ".e5m2", ".tf32",
}
POSTFIX_TYPES = {"ScalarType", "VectorPrefix"}

# Tokens of the base lexer enum (ptx_parser/src/lib.rs:1933-2030), in this project's own numbering.
BASE_TOKENS = [
    ("COMMA", ","), ("DOT", "."), ("COLON", ":"), ("SEMI", ";"), ("AT", "@"), ("IDENT", None), ("DOTIDENT", None),
    ("STRING", None), ("PIPE", "|"), ("EXCL", "!"), ("LPAREN", "("), ("RPAREN", ")"), ("LBRACKET", "["),
    ("RBRACKET", "]"), ("LBRACE", "{"), ("RBRACE", "}"), ("LT", "<"), ("GT", ">"), ("F32HEX", None),
    ("F64HEX", None), ("HEX", None), ("F64", None), ("DECIMAL", None), ("MINUS", "-"), ("PLUS", "+"), ("EQ", "="),
]
WORD_TOKENS = [
    ("WARP_SZ", "WARP_SZ"), ("DOT_VERSION", ".version"), ("DOT_LOC", ".loc"), ("DOT_REG", ".reg"),
    ("DOT_ALIGN", ".align"), ("DOT_PRAGMA", ".pragma"), ("DOT_MAXNREG", ".maxnreg"), ("DOT_MAXNTID", ".maxntid"),
    ("DOT_REQNTID", ".reqntid"), ("DOT_MINNCTAPERSM", ".minnctapersm"), ("DOT_ENTRY", ".entry"),
    ("DOT_FUNC", ".func"), ("DOT_EXTERN", ".extern"), ("DOT_VISIBLE", ".visible"), ("DOT_TARGET", ".target"),
    ("DOT_ADDRESS_SIZE", ".address_size"), ("DOT_SECTION", ".section"), ("DOT_FILE", ".file"), ("DOT_PTR", ".ptr"),
    ("DOT_NORETURN", ".noreturn"), ("DOT_TEXREF", ".texref"), ("DOT_SURFREF", ".surfref"),
]


def variant_capitalized(mod):
    """'.param::func' -> 'ParamFunc', '.bf16x2' -> 'BF16x2', '.L2::64B' -> 'L264B'."""
    s = mod[1:].replace("::", "_")
    out = ""
    cap = True
    for c in s:
        if c == "_":
            cap = True
            continue
        if cap or (c == "f" and out.endswith("B")):
            cap = False
            c = c.upper()
        out += c
    return out


def var_name(mod):
    """Name of the C++ local that carries a modifier's value inside a pattern body."""
    s = mod[1:]
    if "::" in s:
        s = s.replace("::", "_")
    elif s in ("match", "type", "const", "async"):
        s += "_"
    if s[0].isdigit():
        s = "x" + s
    return s.lower()


def c_ident(s):
    return re.sub(r"[^A-Za-z0-9_]", "_", s)


# --------------------------------------------------------------------------------------------- .def parser
class Pattern:
    def __init__(self, opcode, mods, args, variant=None, body="", line=0):
        self.opcode, self.mods, self.args, self.variant, self.body, self.line = opcode, mods, args, variant, body, line

    def head(self):
        s = self.opcode
        for opt, m in self.mods:
            s += "{%s}" % m if opt else m
        return s


def parse_head(text):
    """'st{.weak}.type' -> ('st', [(True,'.weak'), (False,'.type')])."""
    m = re.match(r"[A-Za-z_][A-Za-z0-9_]*", text)
    opcode = m.group(0)
    rest = text[m.end():]
    mods = []
    pos = 0
    mre = re.compile(r"\.[A-Za-z0-9_]+(?:::[A-Za-z0-9_]+)?")
    while pos < len(rest):
        if rest[pos] == "{":
            end = rest.index("}", pos)
            mm = mre.fullmatch(rest[pos + 1:end].strip())
            assert mm, text
            mods.append((True, mm.group(0)))
            pos = end + 1
        elif rest[pos] == ".":
            mm = mre.match(rest, pos)
            mods.append((False, mm.group(0)))
            pos = mm.end()
        elif rest[pos].isspace():
            pos += 1
        else:
            raise ValueError("bad pattern head: " + text)
    return opcode, mods


def parse_args(text):
    """Argument list notation of ptx_parser_macros_impl/src/parser.rs:524-602 -> list of dicts."""
    toks = re.findall(r"[A-Za-z_][A-Za-z0-9_]*(?:-[A-Za-z_][A-Za-z0-9_]*)*|\.[a-z]+|[\[\]{},|!]", text)
    pos = 0

    def new(name, **kw):
        d = dict(name=name.replace("-", "_"), optional=False, pre_bracket=False, post_bracket=False, pre_pipe=False,
                 can_be_negated=False, unified=False)
        d.update(kw)
        return d

    def parse_list(closer):
        nonlocal pos
        out = []
        while pos < len(toks) and toks[pos] != closer:
            t = toks[pos]
            if t == ",":
                pos += 1
            elif t == "{":
                if toks[pos + 1] == "!":
                    assert toks[pos + 2] == "}"
                    out.append(new(toks[pos + 3], can_be_negated=True))
                    pos += 4
                elif toks[pos + 1] == ",":
                    assert toks[pos + 3] == "}"
                    out.append(new(toks[pos + 2], optional=True))
                    pos += 4
                elif toks[pos + 1] == ".unified":
                    raise ValueError("{.unified} must follow a bracket group")
                else:
                    raise ValueError("bad brace group in args: " + text)
            elif t == "[":
                pos += 1
                if toks[pos] == "|":
                    out.append(new(toks[pos + 1], optional=True, pre_pipe=True))
                    assert toks[pos + 2] == "]"
                    pos += 3
                else:
                    sub = parse_list("]")
                    pos += 1
                    sub[0]["pre_bracket"] = True
                    sub[-1]["post_bracket"] = True
                    if pos + 2 < len(toks) and toks[pos] == "{" and toks[pos + 1] == ".unified":
                        for a in sub:
                            a["unified"] = True
                        pos += 3
                    out.extend(sub)
            elif t == "|":
                out.append(new(toks[pos + 1], pre_pipe=True))
                pos += 2
            else:
                out.append(new(t))
                pos += 1
        return out

    return parse_list(None)


class Spec:
    def __init__(self):
        self.plain_enums = {}   # name -> [variants] (hand-declared part)
        self.enum_order = []
        self.types = []         # ('struct', name, fields) | ('enum', name, variants)
        self.instrs = []        # (name, data_type or None, [(arg, optional)])
        self.sets = {}
        self.groups = []        # [(patterns, rules)] ; rules: (name, type|None, [alts])
        self.specials = []


def split_top(s, sep=","):
    out, depth, cur = [], 0, ""
    for c in s:
        if c in "({<":
            depth += 1
        elif c in ")}>":
            depth -= 1
        if c == sep and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += c
    if cur.strip():
        out.append(cur.strip())
    return out


def parse_def(path):
    spec = Spec()
    lines = open(path).read().split("\n")
    i = 0
    cur = None
    while i < len(lines):
        raw = lines[i]
        line = raw.strip()
        i += 1
        if not line or line.startswith("#"):
            continue
        if line.startswith("set "):
            name, rhs = line[4:].split("=", 1)
            spec.sets[name.strip()] = rhs.split()
        elif line.startswith("enum ") or line.startswith("struct "):
            kind, rest = line.split(" ", 1)
            name = rest[:rest.index("{")].strip()
            body = rest[rest.index("{") + 1:rest.rindex("}")].strip()
            items = split_top(body)
            if kind == "struct":
                fields = [tuple(x.strip() for x in it.split(":", 1)) for it in items]
                spec.types.append(("struct", name, fields))
            else:
                variants = []
                plain = True
                for it in items:
                    m = re.match(r"(\w+)\s*\((.*)\)$", it)
                    m2 = re.match(r"(\w+)\s*\{(.*)\}$", it)
                    if m:
                        plain = False
                        variants.append((m.group(1), [(None, t) for t in split_top(m.group(2))]))
                    elif m2:
                        plain = False
                        variants.append((m2.group(1), [tuple(x.strip() for x in f.split(":", 1)) for f in split_top(m2.group(2))]))
                    else:
                        variants.append((it, []))
                if plain:
                    spec.plain_enums[name] = [v[0] for v in variants]
                    spec.enum_order.append(name)
                else:
                    spec.types.append(("enum", name, variants))
        elif line.startswith("instr "):
            m = re.match(r"instr (\w+)\((\w*)\)\s*(.*)$", line)
            args = [(a.rstrip("?"), a.endswith("?")) for a in m.group(3).split()]
            spec.instrs.append((m.group(1), m.group(2) or None, args))
        elif line == "block":
            cur = ([], [])
        elif line == "end":
            spec.groups.append(cur)
            cur = None
        elif line.startswith("special "):
            spec.specials.append(line.split()[1])
        elif line.startswith("pat "):
            m = re.match(r"pat (\S+)\s*(.*?)\s*=>\s*(\w+)\s*\{$", line)
            assert m, line
            opcode, mods = parse_head(m.group(1))
            args = parse_args(m.group(2))
            body = []
            while lines[i].rstrip() != "}":
                body.append(lines[i])
                i += 1
            i += 1
            cur[0].append(Pattern(opcode, mods, args, m.group(3), "\n".join(body), i))
        elif line.startswith("rule "):
            lhs, rhs = line[5:].split(" = ", 1)
            name, typ = (lhs.split(": ", 1) + [None])[:2]
            alts = []
            for a in rhs.split():
                alts.extend(spec.sets[a[1:]] if a.startswith("@") else [a])
            cur[1].append((name.strip(), typ.strip() if typ else None, alts))
        else:
            raise ValueError("cannot parse line %d: %s" % (i, raw))
    return spec


# --------------------------------------------------------------------------------------------- reference DSL parser (check mode)
def parse_reference(path):
    """Read the derive_parser! body of the reference's lib.rs into the same (patterns, rules) groups."""
    text = open(path).read()
    start = text.index("derive_parser!(\n")
    end = text.index("#[cfg(test)]", start)
    body = text[start + len("derive_parser!(\n"):end]
    body = body[:body.rindex(");")]
    body = re.sub(r"/\*.*?\*/", " ", body, flags=re.S)
    body = re.sub(r"//[^\n]*", " ", body)
    pos = 0
    n = len(body)

    def skip_ws():
        nonlocal pos
        while pos < n and body[pos].isspace():
            pos += 1

    def match_brace(p):
        depth = 0
        while True:
            c = body[p]
            if c == "{":
                depth += 1
            elif c == "}":
                depth -= 1
                if depth == 0:
                    return p
            p += 1

    groups = []
    specials = []
    cur_p, cur_r = [], []
    seen_rule = False
    while True:
        skip_ws()
        if pos >= n:
            break
        if body[pos] == "#" or body.startswith("pub enum", pos) or body.startswith("enum", pos):
            b = body.index("{", pos)
            pos = match_brace(b) + 1
            continue
        # rule?  ".name[: Type] = {..};"  or  "Type = {..};"
        m = re.compile(r"(\.[A-Za-z0-9_]+(?:::[A-Za-z0-9_]+)?)\s*(?::\s*(\w+))?\s*=\s*\{").match(body, pos)
        m2 = re.compile(r"(\w+)\s*=\s*\{").match(body, pos)
        if m or m2:
            mm = m or m2
            b = mm.end() - 1
            e = match_brace(b)
            alts_text = body[b + 1:e]
            alts = []
            for part in split_top(alts_text):
                pm = re.match(r"(\.[A-Za-z0-9_]+)\s*\{(.*)\}$", part.strip(), flags=re.S)
                if pm:
                    alts.append(pm.group(1))
                    for suf in pm.group(2).split(","):
                        alts.append(pm.group(1) + suf.strip())
                else:
                    alts.append(re.sub(r"\s+", "", part))
            pos = e + 1
            skip_ws()
            assert body[pos] == ";", body[pos:pos + 40]
            pos += 1
            if m:
                cur_r.append((m.group(1), m.group(2), alts))
            # type-only rules only type literal modifiers for the code block; they still close a pattern group
            seen_rule = True
            continue
        # pattern: up to '=>' or '<='
        if seen_rule:
            groups.append((cur_p, cur_r))
            cur_p, cur_r = [], []
            seen_rule = False
        arrow = re.compile(r"=>|<=").search(body, pos)
        head = body[pos:arrow.start()].strip()
        b = body.index("{", arrow.end())
        e = match_brace(b)
        pos = e + 1
        if arrow.group(0) == "<=":
            specials.append(head)
            continue
        hm = re.match(r"(\S+)\s*(.*)$", head, flags=re.S)
        # the modifier part may contain no spaces; arguments follow the first whitespace
        opcode, mods = parse_head(hm.group(1))
        args = parse_args(hm.group(2))
        cur_p.append(Pattern(opcode, mods, args))
    if cur_p or cur_r:
        groups.append((cur_p, cur_r))
    return groups, specials


# --------------------------------------------------------------------------------------------- the reference generator's algorithm
class Slot:
    def __init__(self, name, optional, alts, typ, direct):
        self.name, self.optional, self.alts, self.typ, self.direct = name, optional, alts, typ, direct

    def key(self):
        return (self.name, self.optional, tuple(self.alts), self.typ, self.direct)


class Definition:
    def __init__(self, pat, unordered, ordered, possible):
        self.pat, self.unordered, self.ordered, self.possible = pat, unordered, ordered, possible


def build_definitions(groups):
    """-> {opcode: [Definition in definition-index order]}"""
    defs = {}
    order = []
    for patterns, rules in groups:
        named = {r[0]: r for r in rules}
        last_opcode = patterns[-1].opcode
        for pat in reversed(patterns):
            if pat.opcode != last_opcode:
                named = {}
            slots = []
            possible = set()
            for optional, mod in pat.mods:
                if mod in named:
                    _, typ, alts = named[mod]
                    possible.update(alts)
                    if len(alts) == 1 and typ is None:
                        slots.append(Slot(mod, optional, [alts[0]], None, True))
                    else:
                        assert typ is not None, "rule %s of %s needs a type" % (mod, pat.head())
                        slots.append(Slot(mod, optional, list(alts), typ, False))
                else:
                    possible.add(mod)
                    slots.append(Slot(mod, optional, [mod], None, True))
            ordered = []
            while slots:
                s = slots[-1]
                is_ordered = (s.alts[0] in POSTFIX_MODIFIERS) if s.direct else (s.typ in POSTFIX_TYPES)
                if not is_ordered:
                    break
                ordered.append(slots.pop())
            if len(ordered) == 1:
                slots.append(ordered.pop())
            if len(slots) == 1:
                ordered.append(slots.pop())
            ordered.reverse()
            if pat.opcode not in defs:
                defs[pat.opcode] = []
                order.append(pat.opcode)
            defs[pat.opcode].append(Definition(pat, slots, ordered, possible))
            last_opcode = pat.opcode
    return defs, order


def build_chain(opcode, definitions):
    """-> [(key alternatives or None for the default, definition index)] in if/else-if order."""
    n = len(definitions)
    sel = [None] * n
    gen = 0
    while True:
        unselected = [i for i in range(n) if sel[i] is None]
        if not unselected:
            break
        if len(unselected) == 1:
            sel[unselected[0]] = (None, gen)
            break
        selected_something = False
        for i in unselected:
            d = definitions[i]
            cands = [s for s in d.unordered + d.ordered if not s.optional]
            cands.sort(key=lambda s: 1 if s.direct else len(s.alts))
            for c in cands:
                clash = False
                for j in unselected:
                    if j == i:
                        continue
                    if any(v in definitions[j].possible for v in c.alts):
                        clash = True
                        break
                if clash:
                    continue
                sel[i] = (list(c.alts), gen)
                selected_something = True
                break
        if not selected_something:
            raise SystemExit("cannot build the selection chain for " + opcode)
        gen += 1
    # NOTE: `unselected` is computed once per generation in the reference, and selections made earlier in the same
    # generation do not remove a pattern from the clash check of later ones; the loop above matches that because
    # `unselected` is a snapshot.
    chain = []
    g = 0
    while True:
        layer = [(sel[i][0], i) for i in range(n) if sel[i][1] == g]
        if not layer:
            break
        chain.extend(layer)
        g += 1
    return chain


def structure(groups):
    defs, order = build_definitions(groups)
    out = {}
    for op in order:
        chain = build_chain(op, defs[op])
        out[op] = dict(
            defs=[(d.pat.head(), [s.key() for s in d.unordered], [s.key() for s in d.ordered],
                   [tuple(sorted(a.items())) for a in d.pat.args]) for d in defs[op]],
            chain=[(tuple(k) if k is not None else None, i) for k, i in chain])
    return out, defs, order


# --------------------------------------------------------------------------------------------- emission
def keyword_hash(word, mult=16777619):
    h = 2166136261
    for ch in word.encode():
        h = ((h ^ ch) * mult) & 0xFFFFFFFF
    return h ^ (h >> 15)


def perfect_hash(words):
    """Open-addressing table (linear probing, 512 slots, load < 0.5) over FNV-1a of the token bytes."""
    size = 512
    table = {}
    for w in words:
        h = keyword_hash(w) & (size - 1)
        while h in table:
            h = (h + 1) & (size - 1)
        table[h] = w
    return 16777619, size, table


def emit(spec, out_dirs):
    struct, defs, order = structure(spec.groups)
    opcodes = list(order)
    for s in spec.specials:
        if s not in opcodes:
            opcodes.append(s)
    # modifiers: every alternative of every pattern, plus .unified (ptx_parser_macros/src/lib.rs:913-959)
    modifiers = []
    seen = set()
    for op in order:
        for d in defs[op]:
            for s in d.unordered + d.ordered:
                for a in s.alts:
                    if a not in seen:
                        seen.add(a)
                        modifiers.append(a)
    modifiers.append(".unified")
    mod_id = {m: i for i, m in enumerate(modifiers)}
    assert len(modifiers) <= 192

    # typed enums from rules
    enums = {}
    for name in spec.enum_order:
        enums[name] = list(spec.plain_enums[name])
    rule_text = {}  # (enum, variant) -> modifier text (Display)
    for patterns, rules in spec.groups:
        for _, typ, alts in rules:
            if typ is None:
                continue
            vs = enums.setdefault(typ, [])
            for a in alts:
                v = variant_capitalized(a)
                if v not in vs:
                    vs.append(v)
                rule_text[(typ, v)] = a

    L = []
    w = L.append
    w("// GENERATED by zluda_b200/grammar/gen_tables.py from zluda_b200/grammar/ptx.def -- do not edit.")
    w("// Token ids, keyword table, instruction patterns, pattern-selection chains, result schema.")
    w("#pragma once")
    w("#include <stdint.h>")
    w("#ifndef PTX_HD")
    w("#ifdef __CUDACC__")
    w("#define PTX_HD __host__ __device__")
    w("#define PTX_TABLE static __device__ const")
    w("#else")
    w("#define PTX_HD")
    w("#define PTX_TABLE static const")
    w("#endif")
    w("#endif")
    w("#ifndef PTX_NOINLINE")
    w("#ifdef __CUDACC__")
    w("#define PTX_NOINLINE __noinline__")
    w("#else")
    w("#define PTX_NOINLINE __attribute__((noinline))")
    w("#endif")
    w("#endif")
    w("#ifndef PTX_HOST_TABLE")
    w("#define PTX_HOST_TABLE static const")
    w("#endif")
    w("")
    # ---- token kinds
    w("enum PtxTok : uint16_t {")
    k = 0
    tok_words = []
    for name, text in BASE_TOKENS:
        w("    T_%s = %d," % (name, k))
        k += 1
    for name, text in WORD_TOKENS:
        w("    T_%s = %d,   // %s" % (name, k, text))
        tok_words.append((text, k))
        k += 1
    w("    T_OP_FIRST = %d," % k)
    op_first = k
    for op in opcodes:
        w("    T_OP_%s = %d," % (op.upper(), k))
        tok_words.append((op, k))
        k += 1
    w("    T_MOD_FIRST = %d," % k)
    mod_first = k
    for m in modifiers:
        w("    T_MOD_%s = %d,   // %s" % (c_ident(m[1:]), k, m))
        tok_words.append((m, k))
        k += 1
    w("    T_COUNT = %d," % k)
    w("    T_ERROR = 0xFFFF")
    w("};")
    w("#define PTX_N_OPCODES %d" % len(opcodes))
    w("#define PTX_N_MODIFIERS %d" % len(modifiers))
    w("#define PTX_MOD_WORDS 3   // 64-bit words of a modifier-set bitmask")
    w("")
    # ---- keyword table (perfect hash)
    words = [t for t, _ in tok_words]
    assert len(set(words)) == len(words)
    mult, size, table = perfect_hash(words)
    kind_of = dict(tok_words)
    pool = ""
    offs = {}
    for t in words:
        offs[t] = len(pool)
        pool += t
    w("#define PTX_KW_MULT %du" % mult)
    w("#define PTX_KW_SIZE %d" % size)
    w("#define PTX_KW_MAXLEN %d" % max(len(t) for t in words))
    w("struct PtxKwEntry { uint16_t kind; uint8_t len; uint8_t pad; uint16_t off; uint16_t pad2; };")
    w("PTX_TABLE PtxKwEntry ptx_kw_table[PTX_KW_SIZE] = {")
    row = []
    for h in range(size):
        if h in table:
            t = table[h]
            row.append("{%d,%d,0,%d,0}" % (kind_of[t], len(t), offs[t]))
        else:
            row.append("{0xFFFF,0,0,0,0}")
        if len(row) == 8:
            w("    " + ",".join(row) + ",")
            row = []
    w("};")
    w('PTX_TABLE char ptx_kw_pool[] = "%s";' % pool)
    # ---- the same keywords keyed by their first eight bytes (little-endian, zero padded) and length: a lookup is one
    # probe and two word compares for keywords of up to eight bytes
    M32 = 0xFFFFFFFF

    def hash8(lo, hi, ln):
        h = ((lo ^ hi) * 0x9E3779B1) & M32
        h ^= (ln * 0x85EBCA6B) & M32
        h ^= h >> 15
        h = (h * 0x2C1B3C6D) & M32
        h ^= h >> 12
        return h

    size8 = 1024
    table8 = {}
    for t in words:
        b8 = t.encode()[:8].ljust(8, b"\0")
        lo, hi = int.from_bytes(b8[:4], "little"), int.from_bytes(b8[4:], "little")
        h = hash8(lo, hi, len(t)) & (size8 - 1)
        while h in table8:
            h = (h + 1) & (size8 - 1)
        table8[h] = (lo, hi, t)
    w("#define PTX_KW8_SIZE %d" % size8)
    w("struct PtxKw8Entry { uint32_t lo, hi; uint16_t kind; uint8_t len; uint8_t pad; uint16_t off; uint16_t pad2; };")
    w("PTX_TABLE PtxKw8Entry ptx_kw8_table[PTX_KW8_SIZE] = {")
    row = []
    for h in range(size8):
        if h in table8:
            lo, hi, t = table8[h]
            row.append("{%du,%du,%d,%d,0,%d,0}" % (lo, hi, kind_of[t], len(t), offs[t]))
        else:
            row.append("{0,0,0xFFFF,0,0,0,0}")
        if len(row) == 4:
            w("    " + ",".join(row) + ",")
            row = []
    w("};")
    w("// token text for every literal token kind (host side: dump, oracle lexer)")
    w("PTX_HOST_TABLE char* const ptx_tok_text[T_COUNT] = {")
    texts = [t if t is not None else "" for _, t in BASE_TOKENS] + [t for _, t in WORD_TOKENS] + opcodes + modifiers
    for i in range(0, len(texts), 8):
        w("    " + ",".join('"%s"' % t.replace('"', '\\"') for t in texts[i:i + 8]) + ",")
    w("};")
    w("")
    # ---- enums
    for name, vs in enums.items():
        w("enum { " + ", ".join("%s_%s = %d" % (name, v, i) for i, v in enumerate(vs)) + " };")
        w("PTX_HOST_TABLE char* const %s_names[] = { %s };" % (name, ", ".join('"%s"' % v for v in vs)))
        if any((name, v) in rule_text for v in vs):
            w("PTX_HOST_TABLE char* const %s_text[] = { %s };" % (
                name, ", ".join('"%s"' % rule_text.get((name, v), "") for v in vs)))
    for kind, name, items in spec.types:
        if kind == "enum":
            w("enum { " + ", ".join("%s_%s = %d" % (name, v[0], i) for i, v in enumerate(items)) + " };")
    w("")
    # ---- schema
    prim = {"bool": 0, "u8": 1, "u32": 2, "u64": 3, "f32": 4}
    type_ids = {}
    type_rows = []   # (kind, name, first_child, n_children)   kind: 0 prim,1 plain enum,2 struct,3 data enum,4 option
    child_rows = []  # (field name or "", type id, n_fields(for variants), first_field)
    field_rows = []

    def tid(t):
        t = t.strip()
        if t in type_ids:
            return type_ids[t]
        if t in prim:
            type_ids[t] = len(type_rows)
            type_rows.append([0, t, prim[t], 0])
            return type_ids[t]
        m = re.match(r"Option<(.*)>$", t)
        if m:
            inner = tid(m.group(1))
            type_ids[t] = len(type_rows)
            type_rows.append([4, t, inner, 0])
            return type_ids[t]
        if t in enums:
            type_ids[t] = len(type_rows)
            type_rows.append([1, t, 0, len(enums[t])])
            return type_ids[t]
        for kind, name, items in spec.types:
            if name != t:
                continue
            me = len(type_rows)
            type_ids[t] = me
            type_rows.append(None)
            if kind == "struct":
                fids = [(fn, tid(ft)) for fn, ft in items]
                first = len(field_rows)
                field_rows.extend(fids)
                type_rows[me] = [2, t, first, len(fids)]
            else:
                vrows = []
                for vname, fields in items:
                    fids = [(fn or "", tid(ft)) for fn, ft in fields]
                    first = len(field_rows)
                    field_rows.extend(fids)
                    named = 1 if (fields and fields[0][0] is not None) else 0
                    vrows.append((vname, first, len(fids), named))
                firstv = len(child_rows)
                child_rows.extend(vrows)
                type_rows[me] = [3, t, firstv, len(vrows)]
            return me
        raise SystemExit("unknown schema type " + t)

    instr_rows = []
    arg_rows = []
    for name, data, args in spec.instrs:
        d = tid(data) if data else -1
        first = len(arg_rows)
        arg_rows.extend(args)
        instr_rows.append((name, d, first, len(args)))
    w("struct PtxType { uint8_t kind; const char* name; int32_t a; int32_t b; };  // kind 0 prim(a=prim id) 1 enum 2 struct(a=first field,b=n) 3 data enum(a=first variant,b=n) 4 Option(a=inner)")
    w("struct PtxField { const char* name; int32_t type; };")
    w("struct PtxVariant { const char* name; int32_t first_field; int32_t n_fields; int32_t named; };")
    w("struct PtxInstr { const char* name; int32_t data_type; int32_t first_arg; int32_t n_args; };")
    w("struct PtxArg { const char* name; int32_t optional; };")
    w("PTX_HOST_TABLE PtxType ptx_types[] = {")
    for kind, name, a, b in type_rows:
        w('    {%d, "%s", %d, %d},' % (kind, name, a, b))
    w("};")
    w("PTX_HOST_TABLE PtxField ptx_fields[] = {")
    for fn, ft in field_rows:
        w('    {"%s", %d},' % (fn, ft))
    w('    {"", 0}};')
    w("PTX_HOST_TABLE PtxVariant ptx_variants[] = {")
    for vname, first, nf, named in child_rows:
        w('    {"%s", %d, %d, %d},' % (vname, first, nf, named))
    w("};")
    w("PTX_HOST_TABLE char* const* const ptx_enum_names[] = {")
    for kind, name, a, b in type_rows:
        w("    %s," % (name + "_names" if kind == 1 else "0"))
    w("};")
    w("enum { " + ", ".join("I_%s = %d" % (r[0], i) for i, r in enumerate(instr_rows)) + " };")
    w("PTX_HOST_TABLE PtxInstr ptx_instrs[] = {")
    for name, d, first, na in instr_rows:
        w('    {"%s", %d, %d, %d},' % (name, d, first, na))
    w("};")
    w("PTX_HOST_TABLE PtxArg ptx_args[] = {")
    for an, opt in arg_rows:
        w('    {"%s", %d},' % (an, 1 if opt else 0))
    w('    {"", 0}};')
    w("")
    # ---- patterns
    instr_id = {r[0]: i for i, r in enumerate(instr_rows)}
    pat_rows = []
    slot_rows = []
    alt_rows = []
    parg_rows = []
    pat_index = {}
    all_pats = []
    for op in order:
        for di, d in enumerate(defs[op]):
            pat_index[(op, di)] = len(pat_rows)
            sfirst = len(slot_rows)
            for s in d.unordered + d.ordered:
                afirst = len(alt_rows)
                enum_vals = enums[s.typ] if s.typ else None
                for a in s.alts:
                    val = enum_vals.index(variant_capitalized(a)) if enum_vals else 1
                    alt_rows.append((mod_id[a], val))
                slot_rows.append((1 if s.optional else 0, 1 if s.typ else 0, afirst, len(s.alts)))
            afirst = len(parg_rows)
            for a in d.pat.args:
                flags = (a["optional"] * 1 | a["pre_bracket"] * 2 | a["post_bracket"] * 4 | a["pre_pipe"] * 8 |
                         a["can_be_negated"] * 16 | a["unified"] * 32)
                parg_rows.append(flags)
            pat_rows.append((opcodes.index(op), len(d.unordered), len(d.ordered), sfirst, afirst, len(d.pat.args),
                             instr_id[d.pat.variant], d.pat.head()))
            all_pats.append(d)
    chain_rows = []
    op_rows = []
    for op in opcodes:
        if op in spec.specials:
            op_rows.append((0, 0, 1 + spec.specials.index(op)))
            continue
        first = len(chain_rows)
        for keys, di in struct[op]["chain"]:
            mask = [0, 0, 0]
            if keys is not None:
                for kmod in keys:
                    mask[mod_id[kmod] // 64] |= 1 << (mod_id[kmod] % 64)
            chain_rows.append((pat_index[(op, di)], 1 if keys is None else 0, mask))
        op_rows.append((first, len(chain_rows) - first, 0))
    w("#define PTX_ARG_OPTIONAL 1\n#define PTX_ARG_PRE_BRACKET 2\n#define PTX_ARG_POST_BRACKET 4\n#define PTX_ARG_PRE_PIPE 8\n#define PTX_ARG_NEGATED 16\n#define PTX_ARG_UNIFIED 32")
    w("#define PTX_MAX_SLOTS 12\n#define PTX_MAX_ARGS 8")
    assert max(r[1] + r[2] for r in pat_rows) <= 12 and max(r[5] for r in pat_rows) <= 8
    w("struct PtxPattern { uint8_t opcode, n_unordered, n_ordered, n_args; uint16_t first_slot, first_arg, instr; };")
    w("struct PtxSlot { uint8_t optional, typed; uint16_t first_alt; uint16_t n_alt; };")
    w("struct PtxAlt { uint8_t mod; int8_t value; };")
    w("struct PtxChain { uint16_t pattern; uint16_t is_default; uint64_t key[PTX_MOD_WORDS]; };")
    w("struct PtxOpcode { uint16_t first_chain, n_chain, special; };   // special: 1 bra, 2 call, 3 vshr")
    w("#define PTX_N_PATTERNS %d" % len(pat_rows))
    w("PTX_TABLE PtxPattern ptx_patterns[PTX_N_PATTERNS] = {")
    for opi, nu, no, sf, af, na, ins, head in pat_rows:
        w("    {%d,%d,%d,%d,%d,%d,%d},   // %s" % (opi, nu, no, na, sf, af, ins, head))
    w("};")
    w("PTX_TABLE PtxSlot ptx_slots[] = {")
    for o, t, af, na in slot_rows:
        w("    {%d,%d,%d,%d}," % (o, t, af, na))
    w("    {0,0,0,0}};")
    w("PTX_TABLE PtxAlt ptx_alts[] = {")
    for i in range(0, len(alt_rows), 10):
        w("    " + ",".join("{%d,%d}" % r for r in alt_rows[i:i + 10]) + ",")
    w("    {0,0}};")
    w("PTX_TABLE uint8_t ptx_pattern_args[] = {" + ",".join(str(f) for f in parg_rows) + ",0};")
    w("PTX_TABLE PtxChain ptx_chains[] = {")
    for p, isd, mask in chain_rows:
        w("    {%d,%d,{0x%xull,0x%xull,0x%xull}}," % (p, isd, mask[0], mask[1], mask[2]))
    w("    {0,0,{0,0,0}}};")
    w("PTX_TABLE PtxOpcode ptx_opcodes[PTX_N_OPCODES] = {")
    for f, nn, sp in op_rows:
        w("    {%d,%d,%d}," % (f, nn, sp))
    w("};")
    w("PTX_HOST_TABLE char* const ptx_pattern_heads[PTX_N_PATTERNS] = {")
    for r in pat_rows:
        w('    "%s",' % r[7])
    w("};")
    w("")
    # ---- messages + builders
    msgs = []

    def msg_id(m):
        s = m.group(1)
        if s not in msgs:
            msgs.append(s)
        return "b.err_todo(%d)" % msgs.index(s)

    bodies = []
    for pi, d in enumerate(all_pats):
        body = re.sub(r'b\.err_todo\("([^"]*)"\)', msg_id, d.pat.body)
        decl = []
        declared = set()
        for si, s in enumerate(d.unordered + d.ordered):
            vn = var_name(s.name)
            if not (s.optional or s.typ) or vn in declared or vn in ("volatile", "const", "auto", "register"):
                continue
            declared.add(vn)
            decl.append("const int %s = mv[%d]; (void)%s;" % (vn, si, vn))
        for ai, a in enumerate(d.pat.args):
            an = a["name"]
            if an == "b":
                an = "b_"
            decl.append("const int %s = av[%d]; (void)%s;" % (an, ai, an))
            if a["can_be_negated"]:
                decl.append("const int %s_neg = aneg[%d]; (void)%s_neg;" % (an, ai, an))
            if a["unified"]:
                decl.append("const int %s_unified = auni[%d]; (void)%s_unified;" % (an, ai, an))
        bodies.append("    case %d: {  // %s\n        %s\n%s\n        break; }" % (
            pi, d.pat.head(), " ".join(decl), "\n".join("    " + l for l in body.split("\n"))))
    w("PTX_HOST_TABLE char* const ptx_todo_msgs[] = {")
    for m in msgs:
        w('    "%s",' % m)
    w("    0};")
    w("")
    sem = open(os.path.join(HERE, "ptx_sem.inc")).read()
    w(sem)
    w("")
    w("// One case per pattern: append the variant's data words (schema order), then its operands.")
    w("template <class B>")
    w("PTX_HD PTX_NOINLINE inline void ptx_build(int pattern, B& b, const int* mv, const int* av, const int* aneg, const int* auni) {")
    w("    switch (pattern) {")
    for bd in bodies:
        w(bd)
    w("    default: break;")
    w("    }")
    w("}")
    text = "\n".join(L) + "\n"
    for d in out_dirs:
        os.makedirs(d, exist_ok=True)
        p = os.path.join(d, "ptx_tables.h")
        if not os.path.exists(p) or open(p).read() != text:
            open(p, "w").write(text)
    return dict(opcodes=opcodes, modifiers=modifiers, patterns=len(pat_rows))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--def", dest="deff", default=os.path.join(HERE, "ptx.def"))
    ap.add_argument("--out", action="append", default=[])
    ap.add_argument("--check-against")
    ap.add_argument("--dump-chains", action="store_true")
    a = ap.parse_args()
    spec = parse_def(a.deff)
    if a.dump_chains:
        st, defs, order = structure(spec.groups)
        for op in order:
            print(op)
            for keys, i in st[op]["chain"]:
                print("   ", "DEFAULT" if keys is None else " | ".join(keys), "<-", st[op]["defs"][i][0])
    if a.check_against:
        ref_groups, ref_specials = parse_reference(a.check_against)
        mine, _, order = structure(spec.groups)
        ref, _, rorder = structure(ref_groups)
        bad = 0
        if sorted(order) != sorted(rorder):
            print("opcode sets differ:", sorted(set(order) ^ set(rorder)))
            bad += 1
        if sorted(ref_specials) != sorted(spec.specials):
            print("special opcodes differ:", ref_specials, spec.specials)
            bad += 1
        for op in rorder:
            if op in mine and mine[op] != ref[op]:
                bad += 1
                print("MISMATCH for opcode", op)
                for x, y in zip(mine[op]["defs"], ref[op]["defs"]):
                    if x != y:
                        print("  mine:", x)
                        print("  ref :", y)
                if mine[op]["chain"] != ref[op]["chain"]:
                    print("  chain mine:", mine[op]["chain"])
                    print("  chain ref :", ref[op]["chain"])
        npat = sum(len(v["defs"]) for v in ref.values())
        print("reference: %d opcodes (+%d special), %d patterns; spec: %d opcodes, %d patterns; %d mismatches" % (
            len(rorder), len(ref_specials), npat, len(order), sum(len(v["defs"]) for v in mine.values()), bad))
        if bad:
            sys.exit(1)
    if a.out:
        info = emit(spec, a.out)
        print("wrote ptx_tables.h: %d opcodes, %d modifier literals, %d patterns" % (
            len(info["opcodes"]), len(info["modifiers"]), info["patterns"]))


if __name__ == "__main__":
    main()
