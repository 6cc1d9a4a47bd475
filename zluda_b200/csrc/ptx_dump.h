// Host side: rebuilds each module's tree from the flat result records and prints the canonical dump.
//
// The dump is what a caller compares against ptx_parser: one line per statement, every AST node printed as if it
// derived Debug (names from ptx_parser/src/ast.rs and from the variant naming of
// ptx_parser_macros_impl/src/parser.rs:350-381), floats as bit patterns.  The error policy is the reference's:
// a directive that raised any error is dropped and counted (ptx_parser/src/lib.rs:613-615), parse_module_checked is
// Ok only without errors (lib.rs:460-467), a lex error stops before parsing (lib.rs:447-449).
#pragma once
#include <stdarg.h>
#include <string.h>

#include <string>
#include <vector>

#include "ptxfe_pipeline.h"

namespace ptxdump {

struct Out {
    std::string s;
    // hash-only mode: the text is folded into a 64-bit FNV-1a hash as it grows and is not kept (a module with millions of
    // initialisers dumps to gigabytes)
    bool hashing = false;
    uint64_t h = 1469598103934665603ull;
    void fold() {
        for (unsigned char c : s) h = (h ^ c) * 1099511628211ull;
        s.clear();
    }
    void tick() { if (hashing && s.size() > (1u << 16)) fold(); }
    void put(const char* x) { s.append(x); tick(); }
    void putn(const char* x, size_t n) { s.append(x, n); tick(); }
    void putf(const char* fmt, ...) __attribute__((format(printf, 2, 3))) {
        char buf[160];
        va_list ap;
        va_start(ap, fmt);
        int n = vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        s.append(buf, (size_t)n);
    }
    void str(const char* x, size_t n) {
        s.push_back('"');
        for (size_t i = 0; i < n; i++) {
            unsigned char c = (unsigned char)x[i];
            if (c == '"') s += "\\\"";
            else if (c == '\\') s += "\\\\";
            else if (c == '\n') s += "\\n";
            else if (c == '\r') s += "\\r";
            else if (c == '\t') s += "\\t";
            else if (c < 0x20 || c == 0x7f) putf("\\u{%x}", c);
            else s.push_back((char)c);
        }
        s.push_back('"');
    }
    void indent(int d) { s.append((size_t)d * 2, ' '); }
};

struct Reader {
    const PtxBatchView& v;
    uint32_t m;
    const char* text;
    uint64_t text_off;
    Reader(const PtxBatchView& view, uint32_t mod) : v(view), m(mod), text(view.texts[mod]), text_off(view.layout[mod].text_off) {}
    const char* at(uint32_t off) const { return text + ((uint64_t)off - text_off); }
    void span(Out& o, uint32_t off, uint32_t len) const { o.str(at(off), len); }
    // a name written by PtxDecoder::w_name: head word (length in bits 8..31) and text offset
    void name(Out& o, uint32_t head, uint32_t off) const {
        uint32_t len = head >> 8;
        if (len == 0xFFFFFFu) {
            const char* s = at(off);
            len = 1;
            while (s[len] == '_' || s[len] == '$' || (s[len] >= '0' && s[len] <= '9') || ((s[len] | 32) >= 'a' && (s[len] | 32) <= 'z')) len++;
        }
        o.str(at(off), len);
    }
};

inline void imm(Out& o, uint32_t kind, uint32_t lo, uint32_t hi) {
    uint64_t bits = lo | ((uint64_t)hi << 32);
    switch (kind) {
    case 0: o.putf("U64(%llu)", (unsigned long long)bits); break;
    case 1: o.putf("S64(%lld)", (long long)bits); break;
    case 2: o.putf("F32(bits=0x%08X)", (unsigned)bits); break;
    default: o.putf("F64(bits=0x%016llX)", (unsigned long long)bits); break;
    }
}
inline const uint32_t* reg_or_imm(const Reader& r, Out& o, const uint32_t* w) {
    if ((w[0] & 0xFF) == 0) { o.put("Reg("); r.name(o, w[0], w[1]); o.put(")"); return w + 2; }
    o.put("Imm("); imm(o, w[0] - 1, w[1], w[2]); o.put(")");
    return w + 3;
}
inline const uint32_t* operand(const Reader& r, Out& o, const uint32_t* w) {
    uint32_t kind = w[0] & 0xF, aux = (w[0] >> 4) & 0xF;
    switch (kind) {
    case OPK_REG: o.put("Reg("); r.name(o, w[0], w[1]); o.put(")"); return w + 2;
    case OPK_REG_OFFSET: o.put("RegOffset("); r.name(o, w[0], w[1]); o.putf(", %d)", (int32_t)w[2]); return w + 3;
    case OPK_IMM: o.put("Imm("); imm(o, aux, w[1], w[2]); o.put(")"); return w + 3;
    case OPK_VEC_MEMBER: o.put("VecMember("); r.name(o, w[0], w[1]); o.putf(", %u)", aux); return w + 2;
    default:
        o.put("VecPack([");
        w++;
        for (uint32_t i = 0; i < aux; i++) {
            if (i) o.put(", ");
            w = reg_or_imm(r, o, w);
        }
        o.put("])");
        return w;
    }
}
inline void type_of(Out& o, uint32_t w0, const uint32_t* dims, uint32_t ndims) {
    uint32_t vec = (w0 >> 4) & 0xF, scalar = (w0 >> 8) & 0xFF, tkind = w0 >> 24;
    if (tkind == 3) { o.put("Texref"); return; }
    if (tkind == 2) {
        if (vec) o.putf("Array(Some(%u), %s, [", vec, ScalarType_names[scalar]);
        else o.putf("Array(None, %s, [", ScalarType_names[scalar]);
        for (uint32_t i = 0; i < ndims; i++) o.putf(i ? ", %u" : "%u", dims[i]);
        o.put("])");
        return;
    }
    if (vec) o.putf("Vector(%u, %s)", vec, ScalarType_names[scalar]);
    else o.putf("Scalar(%s)", ScalarType_names[scalar]);
}
inline void zero_of(Out& o, uint32_t scalar) {
    int k = scalar_kind((int)scalar);
    o.put(k == KIND_SIGNED ? "Imm(S64(0))" : k == KIND_FLOAT ? "Imm(F64(bits=0x0000000000000000))" : "Imm(U64(0))");
}
inline const uint32_t* skip_inits(const uint32_t* p, uint32_t n) {
    for (uint32_t i = 0; i < n; i++) p += (p[0] & 0xFF) == 0 ? 2 : 3;   // name: 2 words, immediate: 3
    return p;
}
// INFO record: [w0, align, ndims, dims..., n_init, RegOrImm...]
inline const uint32_t* info(const Reader& r, Out& o, const uint32_t* w, bool type_space_only = false) {
    uint32_t w0 = w[0], align = w[1], ndims = w[2];
    const uint32_t* dims = w + 3;
    const uint32_t* p = dims + ndims;
    uint32_t n_init = *p++;
    uint32_t space = (w0 >> 16) & 0xFF, scalar = (w0 >> 8) & 0xFF, tkind = w0 >> 24;
    if (type_space_only) {
        o.put("(");
        type_of(o, w0, dims, ndims);
        o.putf(", %s)", StateSpace_names[space]);
        return skip_inits(p, n_init);
    }
    if (w0 & 1) o.putf("VariableInfo { align: Some(%u), v_type: ", align);
    else o.put("VariableInfo { align: None, v_type: ");
    type_of(o, w0, dims, ndims);
    o.putf(", state_space: %s, array_init: [", StateSpace_names[space]);
    uint32_t printed = 0;
    for (uint32_t i = 0; i < n_init; i++) {
        if (printed++) o.put(", ");
        p = reg_or_imm(r, o, p);
    }
    bool initialised_space = space == StateSpace_Global || space == StateSpace_Const;
    if (initialised_space && tkind == 2) {
        for (uint32_t i = n_init; i < dims[0]; i++) {
            if (printed++) o.put(", ");
            zero_of(o, scalar);
        }
    } else if (initialised_space && tkind == 0 && n_init == 0) {
        zero_of(o, scalar);
    }
    o.put("] }");
    return p;
}
// VARIABLE record: INFO, name_off, name_len
inline const uint32_t* variable(const Reader& r, Out& o, const uint32_t* w) {
    o.put("Variable { info: ");
    w = info(r, o, w);
    o.put(", name: ");
    r.span(o, w[0], w[1]);
    o.put(" }");
    return w + 2;
}
inline const uint32_t* skip_variable(const uint32_t* w) {
    uint32_t ndims = w[2];
    const uint32_t* p = w + 3 + ndims;
    uint32_t n_init = *p++;
    return skip_inits(p, n_init) + 2;
}

// cursor over the byte-packed data fields of an instruction record (PtxDecoder::put_packed)
struct PackedCursor {
    const uint32_t* w;
    uint32_t acc = 0, left = 0;
    uint32_t byte() {
        if (!left) { acc = *w++; left = 4; }
        uint32_t b = acc & 0xFFu;
        acc >>= 8;
        left--;
        return b;
    }
    uint32_t next() {
        uint32_t b = byte();
        if (b != 0xFFu) return b;
        uint32_t x = byte();
        x |= byte() << 8;
        x |= byte() << 16;
        x |= byte() << 24;
        return x;
    }
};
inline void schema(Out& o, int type, PackedCursor& w) {
    const PtxType& ty = ptx_types[type];
    switch (ty.kind) {
    case 0:
        switch (ty.a) {
        case 0: o.put(w.next() ? "true" : "false"); break;
        case 3: { uint64_t x = w.next(); x |= (uint64_t)w.next() << 32; o.putf("%llu", (unsigned long long)x); break; }
        case 4: o.putf("bits=0x%08X", w.next()); break;
        default: o.putf("%u", w.next()); break;
        }
        break;
    case 1: o.put(ptx_enum_names[type][w.next()]); break;
    case 2:
        o.put(ty.name);
        if (ty.b) {
            o.put(" { ");
            for (int i = 0; i < ty.b; i++) {
                if (i) o.put(", ");
                o.put(ptx_fields[ty.a + i].name);
                o.put(": ");
                schema(o, ptx_fields[ty.a + i].type, w);
            }
            o.put(" }");
        }
        break;
    case 3: {
        const PtxVariant& vr = ptx_variants[ty.a + w.next()];
        o.put(vr.name);
        if (vr.n_fields) {
            o.put(vr.named ? " { " : "(");
            for (int i = 0; i < vr.n_fields; i++) {
                if (i) o.put(", ");
                if (vr.named) { o.put(ptx_fields[vr.first_field + i].name); o.put(": "); }
                schema(o, ptx_fields[vr.first_field + i].type, w);
            }
            o.put(vr.named ? " }" : ")");
        }
        break;
    }
    default:
        if (w.next()) { o.put("Some("); schema(o, ty.a, w); o.put(")"); }
        else o.put("None");
        break;
    }
}

// payload words of a record, given its header word
inline uint32_t rec_len(uint32_t w0) { return (w0 & 0xFF) == U_INSTR ? (w0 >> 8) & 0x3FFFu : w0 >> 8; }
// U_INSTR / U_INSTR_LONG: `w` = the record (header word first)
inline void instruction(const Reader& r, Out& o, const uint32_t* rec) {
    uint32_t w0 = rec[0];
    const uint32_t* w = rec + 1;
    // head = has_pred | pred_not << 1 | variant << 16
    uint32_t w1 = (w0 & 0xFF) == U_INSTR ? (((w0 >> 29) & 3u) | (((w0 >> 22) & 0x7Fu) << 16)) : rec[rec_len(w0)];
    int variant = (int)(w1 >> 16);
    o.put("Instruction(");
    if (w1 & 1) {
        o.putf("Some(PredAt { not: %s, label: ", (w1 & 2) ? "true" : "false");
        r.span(o, w[0], w[1]);
        o.put(" }), ");
        w += 2;
    } else {
        o.put("None, ");
    }
    const PtxInstr& in = ptx_instrs[variant];
    o.put(in.name);
    if (variant == I_Bra) {
        o.put(" { arguments: BraArgs { src: ");
        r.span(o, w[0], w[1]);
        o.put(" } })\n");
        return;
    }
    if (variant == I_Call) {
        uint32_t uniform = w[0], callee = w[1], foff = w[2], flen = w[3], n_rets = w[4];
        const uint32_t* rets = w + 5;
        const uint32_t* p = rets + 2 * n_rets;
        uint32_t n_inputs = *p++;
        const uint32_t* inputs = p;
        // find `resolved` after the operand records
        const uint32_t* q = inputs;
        {
            Out scratch;
            for (uint32_t i = 0; i < n_inputs; i++) q = operand(r, scratch, q);
        }
        bool resolved = *q != 0;
        o.putf(" { data: CallDetails { uniform: %s, return_arguments: [", uniform ? "true" : "false");
        if (resolved) {
            const uint32_t* f = r.v.words + callee;   // callee's U_FUNC record
            uint32_t cr = f[4], ci = f[5];
            const uint32_t* var = f + 8;
            for (uint32_t i = 0; i < cr; i++) {
                if (i) o.put(", ");
                info(r, o, var, true);
                var = skip_variable(var);
            }
            o.put("], input_arguments: [");
            for (uint32_t i = 0; i < ci; i++) {
                if (i) o.put(", ");
                info(r, o, var, true);
                var = skip_variable(var);
            }
        } else {
            o.put("], input_arguments: [");
        }
        o.put("] }, arguments: CallArgs { return_arguments: [");
        if (resolved)
            for (uint32_t i = 0; i < n_rets; i++) {
                if (i) o.put(", ");
                r.span(o, rets[2 * i], rets[2 * i + 1]);
            }
        o.put("], func: ");
        r.span(o, foff, flen);
        o.put(", input_arguments: [");
        if (resolved) {
            const uint32_t* x = inputs;
            for (uint32_t i = 0; i < n_inputs; i++) {
                if (i) o.put(", ");
                x = operand(r, o, x);
            }
        }
        o.put("], is_external: false } })\n");
        return;
    }
    if (in.data_type < 0 && in.n_args == 0) { o.put(")\n"); return; }
    o.put(" { ");
    if (in.data_type >= 0) {
        o.put("data: ");
        if (ptx_types[in.data_type].kind == 2 && ptx_types[in.data_type].b == 0) {
            o.put("()");
        } else {
            PackedCursor cur;
            cur.w = w;
            schema(o, in.data_type, cur);
            w = cur.w;      // the operand records start at the next word
        }
        if (in.n_args) o.put(", ");
    }
    if (in.n_args) {
        o.putf("arguments: %sArgs { ", in.name);
        for (int i = 0; i < in.n_args; i++) {
            if (i) o.put(", ");
            const PtxArg& a = ptx_args[in.first_arg + i];
            o.put(a.name);
            o.put(": ");
            if (*w == PTX_ABSENT) { o.put(a.optional ? "None" : "<missing>"); w++; }
            else if (a.optional) { o.put("Some("); w = operand(r, o, w); o.put(")"); }
            else w = operand(r, o, w);
        }
        o.put(" }");
    }
    o.put(" })\n");
}

inline void multi_variable_stmt(const Reader& r, Out& o, const uint32_t* w) {
    uint32_t parameterized = w[0], count = w[1], n_names = w[2];
    const uint32_t* names = w + 3;
    const uint32_t* inf = names + 2 * n_names;
    if (parameterized) {
        o.put("Variable(Parameterized { info: ");
        info(r, o, inf);
        o.put(", name: ");
        r.span(o, names[0], names[1]);
        o.putf(", count: %u })\n", count);
    } else {
        o.put("Variable(Names { info: ");
        info(r, o, inf);
        o.put(", names: [");
        for (uint32_t i = 0; i < n_names; i++) {
            if (i) o.put(", ");
            r.span(o, names[2 * i], names[2 * i + 1]);
        }
        o.put("] })\n");
    }
}

static const char* const kErrNames[] = {"ParseInt", "ParseFloat", "Lexer", "Parser", "Todo", "SyntaxError", "NonF32Ftz",
                                        "Unsupported32Bit", "WrongType", "UnknownFunction", "MalformedCall", "WrongArrayType",
                                        "WrongVectorElement", "MultiArrayVariable", "ZeroDimensionArray", "ArrayInitalizer",
                                        "NonExternPointer", "UnrecognizedStatement", "UnrecognizedDirective", "UnsupportedSreg"};
static const char* const kIntErr[] = {"Empty", "InvalidDigit", "PosOverflow", "NegOverflow"};

inline void error_line(const Reader& r, Out& o, uint32_t w0, uint32_t a, uint32_t b) {
    uint32_t kind = w0 & 0xFFFF, sub = w0 >> 16;
    o.put(kErrNames[kind]);
    switch (kind) {
    case E_PARSE_INT: o.putf("(%s)", kIntErr[sub]); break;
    case E_LEXER: o.putf("(start=%u)", a); break;
    case E_PARSER: o.put("(ContextError)"); break;
    case E_TODO: o.put("("); o.str(ptx_todo_msgs[sub], strlen(ptx_todo_msgs[sub])); o.put(")"); break;
    case E_SYNTAX:
        switch (sub) {
        case SYN_LD_NC_BOTH:
            o.putf("(\"cannot have both %s and %s in <text>\")", RawLdCacheOperator_text[a], EvictionPriority_text[b]);
            break;
        case SYN_CP_SIZE: o.put("(\"invalid cp.async cp-size "); o.putn(r.at(a), b); o.put(" in <text>\")"); break;
        case SYN_CVT_MISSING_RND: o.put("(\"missing rounding mode for cvt\")"); break;
        case SYN_CVT_RND_ON_EXTEND: o.put("(\"should not have rounding mode when dst is larger than src in cvt\")"); break;
        default: o.put("(\"unexpected pairing of dst and src types in cvt\")"); break;
        }
        break;
    case E_UNRECOGNIZED_STATEMENT:
    case E_UNRECOGNIZED_DIRECTIVE:
    case E_UNSUPPORTED_SREG: o.put("("); r.span(o, a, b); o.put(")"); break;
    default: break;
    }
    o.put("\n");
}

struct Directive {
    const uint32_t* rec;     // record header
    const uint32_t* end;     // one past the directive's last record (body included)
    uint32_t kind, start_off;
    uint32_t n_errors = 0;
};

// With `hash_out` the dump is not kept: its FNV-1a hash is returned there and the string comes back empty.
inline std::string dump_module(const PtxBatchView& v, uint32_t m, int* status_out, uint64_t* hash_out = nullptr) {
    Reader r(v, m);
    const PtxModuleResult& res = v.results[m];
    Out o;
    o.hashing = hash_out != nullptr;
    const char* mode_name = v.mode == 0 ? "checked" : v.mode == 1 ? "unchecked" : "errors";
    uint32_t n_lex = res.lexerr_end - res.lexerr_begin;
    uint64_t base = v.layout[m].text_off;
    std::vector<Directive> dirs;
    bool have_module = false, parsed_ok = false;
    const char* verdict;
    const uint32_t* w = v.words + res.word_begin;
    const uint32_t* wend = v.words + res.word_end;
    const uint32_t* header = nullptr;
    uint32_t n_parse_errs = 0;
    bool skip_parse = n_lex != 0 && v.mode != 2;
    if (!skip_parse) {
        // split the record stream into directives
        parsed_ok = true;
        if (w == wend) parsed_ok = false;   // no tokens at all: the header does not parse
        while (w < wend) {
            uint32_t kind = w[0] & 0xFF, len = rec_len(w[0]);
            const uint32_t* next = w + 1 + len;
            switch (kind) {
            case U_HEADER: header = w; break;
            case U_MODULE_FAIL: parsed_ok = false; break;
            case U_FUNC: {
                Directive d;
                d.rec = w;
                d.kind = kind;
                d.start_off = w[7];
                bool has_body = (w[1] & FUNC_HAS_BODY) != 0;
                if (has_body) {
                    // the body runs to the matching U_FUNC_END
                    const uint32_t* q = next;
                    while (q < wend && (q[0] & 0xFF) != U_FUNC_END) q += 1 + rec_len(q[0]);
                    if (q < wend) q += 1 + rec_len(q[0]);
                    next = q;
                }
                d.end = next;
                dirs.push_back(d);
                break;
            }
            case U_MODVAR:
            case U_DIR_NONE:
            case U_DIR_FAIL: {
                Directive d;
                d.rec = w;
                d.end = next;
                d.kind = kind;
                d.start_off = w[1];
                dirs.push_back(d);
                break;
            }
            default: break;
            }
            w = next;
        }
        if (!header) parsed_ok = false;
        // attribute errors to directives by position
        size_t di = 0;
        for (uint32_t e = res.err_begin; e < res.err_end; e++) {
            const PtxErrRec& er = v.errs[e];
            if ((er.w0 & 0xFFFF) == E_NONE) continue;
            n_parse_errs++;
            while (di + 1 < dirs.size() && dirs[di + 1].start_off <= er.pos) di++;
            if (!dirs.empty() && dirs[di].start_off <= er.pos) dirs[di].n_errors++;
        }
    }
    uint64_t invalid = 0, kept = 0;
    for (const Directive& d : dirs) {
        if (d.n_errors) invalid++;
        else if (d.kind == U_FUNC || d.kind == U_MODVAR) kept++;
    }
    bool panicked = res.sequential && (res.status & US_MASK) == US_PANIC;
    if (res.sequential && ((res.status & US_MASK) == US_DIVERGE || (res.status & US_MASK) == US_REFUSED) && !skip_parse) {
        o.putf("mode: %s\nstatus: %s\nerrors: 0\n", mode_name, (res.status & US_MASK) == US_DIVERGE ? "ReferenceDiverges" : "SequentialPathRefused");
        if (status_out) *status_out = 1;
        if (hash_out) { o.fold(); *hash_out = o.h; }
        return std::move(o.s);
    }
    if (skip_parse) verdict = v.mode == 0 ? "Err" : "Empty";
    else if (v.mode == 0) {
        have_module = parsed_ok && n_parse_errs == 0 && invalid == 0 && n_lex == 0;
        verdict = have_module ? "Ok" : "Err";
    } else if (v.mode == 1) {
        have_module = parsed_ok;
        verdict = parsed_ok ? "Module" : "Empty";
    } else {
        verdict = "Errors";
    }
    if (panicked) { verdict = "ReferencePanics"; have_module = false; }
    o.putf("mode: %s\nstatus: %s\n", mode_name, verdict);
    if (have_module) {
        uint32_t h = header[1];
        o.putf("Module { ptx_version: (%u, %u), sm_version: %u, address_size: %u, invalid_directives: %llu, directives: %llu }\n",
               h & 0xFF, (h >> 8) & 0xFF, header[2], (h >> 16) & 0xFF, (unsigned long long)invalid, (unsigned long long)kept);
        for (const Directive& d : dirs) {
            if (d.n_errors) continue;
            const uint32_t* p = d.rec;
            if (d.kind == U_MODVAR) {
                // [hdr, start_off, linking, MULTIVARIABLE(parameterized, count, n_names, name, INFO)]
                o.putf("Variable(LinkingDirective(%u), Variable { info: ", p[2]);
                const uint32_t* mv = p + 3;
                info(r, o, mv + 3 + 2 * mv[2]);
                o.put(", name: ");
                r.span(o, mv[3], mv[4]);
                o.put(" })\n");
                continue;
            }
            if (d.kind != U_FUNC) continue;
            uint32_t flags = p[1], n_rets = p[4], n_inputs = p[5];
            o.putf("Method(LinkingDirective(%u), Function { func_directive: MethodDeclaration { return_arguments: [", flags & FUNC_LINKING_MASK);
            const uint32_t* var = p + 8;
            for (uint32_t i = 0; i < n_rets; i++) {
                if (i) o.put(", ");
                var = variable(r, o, var);
            }
            o.put((flags & FUNC_IS_KERNEL) ? "], name: Kernel(" : "], name: Func(");
            r.span(o, p[2], p[3]);
            o.put("), input_arguments: [");
            for (uint32_t i = 0; i < n_inputs; i++) {
                if (i) o.put(", ");
                var = variable(r, o, var);
            }
            o.put("], shared_mem: None }, tuning: [");
            uint32_t n_tuning = flags >> FUNC_TUNING_SHIFT;
            for (uint32_t i = 0; i < n_tuning; i++, var += 4) {
                if (i) o.put(", ");
                switch (var[0]) {
                case 0: o.putf("MaxNReg(%u)", var[1]); break;
                case 1: o.putf("MaxNtid(%u, %u, %u)", var[1], var[2], var[3]); break;
                case 2: o.putf("ReqNtid(%u, %u, %u)", var[1], var[2], var[3]); break;
                case 3: o.putf("MinNCtaPerSm(%u)", var[1]); break;
                default: o.put("NoReturn"); break;
                }
            }
            if (!(flags & FUNC_HAS_BODY)) { o.put("], body: None })\n"); continue; }
            o.put("], body: Some([\n");
            int depth = 1;
            const uint32_t* q = p + 1 + rec_len(p[0]);
            while (q < d.end) {
                uint32_t kind = q[0] & 0xFF, len = rec_len(q[0]);
                const uint32_t* payload = q + 1;
                switch (kind) {
                case U_LABEL: o.indent(depth); o.put("Label("); r.span(o, payload[0], payload[1]); o.put(")\n"); break;
                case U_VAR: o.indent(depth); multi_variable_stmt(r, o, payload); break;
                case U_INSTR:
                case U_INSTR_LONG: o.indent(depth); instruction(r, o, q); break;
                case U_BLOCK_OPEN: o.indent(depth); o.put("Block([\n"); depth++; break;
                case U_BLOCK_CLOSE: depth--; o.indent(depth); o.put("])\n"); break;
                default: break;
                }
                q += 1 + len;
            }
            o.put("]) })\n");
        }
    } else if (v.mode == 1) {
        o.put("Module { ptx_version: (1, 0), sm_version: 0, address_size: 64, invalid_directives: 18446744073709551615, directives: 0 }\n");
    }
    // errors: lexer errors first, then the parser's in order
    uint32_t total = n_lex + (skip_parse ? 0 : n_parse_errs);
    if (!skip_parse && !parsed_ok && res.word_begin == res.word_end) total++;   // token-less module: Parser error
    o.putf("errors: %u\n", total);
    for (uint32_t i = res.lexerr_begin; i < res.lexerr_end; i++)
        o.putf("Lexer(start=%llu)\n", (unsigned long long)(v.lexerrs[2 * (size_t)i] - base));
    if (!skip_parse) {
        for (uint32_t e = res.err_begin; e < res.err_end; e++) {
            const PtxErrRec& er = v.errs[e];
            if ((er.w0 & 0xFFFF) == E_NONE) continue;
            error_line(r, o, er.w0, er.a, er.b);
        }
        if (!parsed_ok && res.word_begin == res.word_end) o.put("Parser(ContextError)\n");
    }
    if (status_out) *status_out = have_module ? 0 : 1;
    if (hash_out) { o.fold(); *hash_out = o.h; }
    return std::move(o.s);
}

}   // namespace ptxdump
