// Host side: materialises a module's flat result records into a tree, and prints the tree.
//
// The tree mirrors what parse_module_checked hands to its callers: ast::Module (ptx_parser/src/ast.rs:1999-2005) holding
// Directive::{Variable, Method} (ast.rs:1991-1997), Function / MethodDeclaration (ast.rs:1922-1989), Statement::{Label,
// Variable, Instruction(Option<PredAt>, Instruction), Block} (ast.rs:14-19), MultiVariable / Variable / VariableInfo
// (ast.rs:1216-1240, 1284-1293), ParsedOperand (ast.rs:1558-1565) and ImmediateValue (ast.rs:1626-1631).  Names are slices
// of the caller's text, as the reference's tree borrows from its input.  An instruction keeps its variant id, the values
// of its data fields in schema order (the schema of every variant is a generated table, gen/ptx_tables.h) and its
// operands; a binding in another language turns (variant, values, operands) into its own enum with a generated match.
// The policy is the reference's: a directive that raised an error is dropped and counted (lib.rs:613-615), arrays are
// padded with typed zeros to their first dimension and uninitialised .global/.const scalars get one (lib.rs:1170-1178,
// 1228-1232).  ptx_ast_print writes the same canonical text as the record reader in ptx_dump.h; the tests hold the two
// against each other and against the oracle.
#pragma once
#include "ptx_dump.h"

namespace ptxast {

struct Str {
    const char* p = nullptr;
    uint32_t n = 0;
};
struct Imm {
    uint8_t kind = 0;      // 0 U64, 1 S64, 2 F32, 3 F64
    uint64_t bits = 0;
};
struct RegOrImm {
    bool is_reg = false;
    Str reg;
    Imm imm;
};
struct Operand {
    uint8_t kind = OPK_REG;    // OPK_*
    uint8_t index = 0;         // VecMember: the element
    bool absent = false;       // an optional argument that is not there
    Str name;
    Imm imm;
    int32_t offset = 0;
    std::vector<RegOrImm> pack;
};
struct Type {
    uint8_t tkind = 0;         // 0 scalar or vector, 2 array, 3 texref
    uint8_t vec = 0, scalar = 0;
    std::vector<uint32_t> dims;
};
struct VariableInfo {
    bool has_align = false;
    uint32_t align = 0;
    Type type;
    uint8_t space = 0;
    std::vector<RegOrImm> array_init;
};
struct Variable {
    VariableInfo info;
    Str name;
};
struct MultiVariable {
    bool parameterized = false;
    VariableInfo info;
    Str name;                  // Parameterized
    uint32_t count = 0;
    std::vector<Str> names;    // Names
};
struct TypeSpace {
    Type type;
    uint8_t space = 0;
};
struct Instruction {
    uint16_t variant = 0;
    bool has_pred = false, pred_not = false;
    Str pred;
    std::vector<uint32_t> data;     // the values of the data fields, schema order
    std::vector<Operand> args;
    Str target;                     // Bra
    bool uniform = false, resolved = false;                 // Call
    std::vector<TypeSpace> callee_rets, callee_inputs;
    std::vector<Str> call_rets;
    Str func;
};
enum { ST_LABEL = 0, ST_VARIABLE = 1, ST_INSTRUCTION = 2, ST_BLOCK = 3 };
struct Statement {
    uint8_t kind = ST_LABEL;
    Str label;
    MultiVariable var;
    Instruction ins;
    std::vector<Statement> block;
};
struct Tuning {
    uint32_t kind = 0, v[3] = {0, 0, 0};
};
struct Function {
    bool is_kernel = false, has_body = false;
    Str name;
    std::vector<Variable> rets, inputs;
    std::vector<Tuning> tuning;
    std::vector<Statement> body;
};
struct Directive {
    bool is_method = false;
    uint8_t linking = 0;
    Variable var;
    Function func;
};
struct Error {
    uint32_t w0 = 0, a = 0, b = 0;
    bool lexer = false;
    uint64_t lex_start = 0;
};
enum { V_OK = 0, V_ERR, V_MODULE, V_EMPTY, V_ERRORS, V_PANICS, V_DIVERGES, V_REFUSED };
struct Module {
    int verdict = V_ERR;
    bool have_module = false;       // the reference returns a module (checked: Ok; unchecked: not Module::empty())
    uint8_t major = 0, minor = 0, address_size = 0;
    uint32_t sm = 0;
    uint64_t invalid_directives = 0;
    std::vector<Directive> directives;
    std::vector<Error> errors;
    bool implicit_parser_error = false;
    size_t nodes = 0;               // statements + directives + operands built (a size figure for callers)
};

struct Builder {
    const ptxdump::Reader& r;
    Module& m;
    Str str(uint32_t off, uint32_t len) const {
        Str s;
        s.p = r.at(off);
        s.n = len;
        return s;
    }
    Str name(uint32_t head, uint32_t off) const {
        uint32_t len = head >> 8;
        if (len == 0xFFFFFFu) {
            const char* s = r.at(off);
            len = 1;
            while (s[len] == '_' || s[len] == '$' || (s[len] >= '0' && s[len] <= '9') || ((s[len] | 32) >= 'a' && (s[len] | 32) <= 'z')) len++;
        }
        return str(off, len);
    }
    const uint32_t* reg_or_imm(const uint32_t* w, RegOrImm* o) const {
        if ((w[0] & 0xFF) == 0) {
            o->is_reg = true;
            o->reg = name(w[0], w[1]);
            return w + 2;
        }
        o->is_reg = false;
        o->imm.kind = (uint8_t)(w[0] - 1);
        o->imm.bits = w[1] | ((uint64_t)w[2] << 32);
        return w + 3;
    }
    const uint32_t* operand(const uint32_t* w, Operand* o) const {
        const uint32_t kind = w[0] & 0xF, aux = (w[0] >> 4) & 0xF;
        o->kind = (uint8_t)kind;
        m.nodes++;
        switch (kind) {
        case OPK_REG: o->name = name(w[0], w[1]); return w + 2;
        case OPK_REG_OFFSET: o->name = name(w[0], w[1]); o->offset = (int32_t)w[2]; return w + 3;
        case OPK_IMM: o->imm.kind = (uint8_t)aux; o->imm.bits = w[1] | ((uint64_t)w[2] << 32); return w + 3;
        case OPK_VEC_MEMBER: o->name = name(w[0], w[1]); o->index = (uint8_t)aux; return w + 2;
        default:
            w++;
            o->pack.resize(aux);
            for (uint32_t i = 0; i < aux; i++) w = reg_or_imm(w, &o->pack[i]);
            return w;
        }
    }
    static RegOrImm zero_of(uint32_t scalar) {
        RegOrImm z;
        int k = scalar_kind((int)scalar);
        z.imm.kind = k == KIND_SIGNED ? 1 : k == KIND_FLOAT ? 3 : 0;
        return z;
    }
    // INFO record: [w0, align, ndims, dims..., n_init, RegOrImm...]
    const uint32_t* info(const uint32_t* w, VariableInfo* o) const {
        const uint32_t w0 = w[0], ndims = w[2];
        const uint32_t* dims = w + 3;
        const uint32_t* p = dims + ndims;
        const uint32_t n_init = *p++;
        o->has_align = (w0 & 1) != 0;
        o->align = w[1];
        o->type.tkind = (uint8_t)(w0 >> 24);
        o->type.vec = (uint8_t)((w0 >> 4) & 0xF);
        o->type.scalar = (uint8_t)((w0 >> 8) & 0xFF);
        o->type.dims.assign(dims, dims + ndims);
        o->space = (uint8_t)((w0 >> 16) & 0xFF);
        const bool initialised_space = o->space == StateSpace_Global || o->space == StateSpace_Const;
        size_t total = n_init;
        if (initialised_space && o->type.tkind == 2 && ndims && dims[0] > n_init) total = dims[0];
        else if (initialised_space && o->type.tkind == 0 && n_init == 0) total = 1;
        o->array_init.resize(total);
        for (uint32_t i = 0; i < n_init; i++) p = reg_or_imm(p, &o->array_init[i]);
        for (size_t i = n_init; i < total; i++) o->array_init[i] = zero_of(o->type.scalar);
        return p;
    }
    const uint32_t* variable(const uint32_t* w, Variable* o) const {
        w = info(w, &o->info);
        o->name = str(w[0], w[1]);
        return w + 2;
    }
    void type_space(const uint32_t* w, TypeSpace* o) const {
        const uint32_t w0 = w[0], ndims = w[2];
        o->type.tkind = (uint8_t)(w0 >> 24);
        o->type.vec = (uint8_t)((w0 >> 4) & 0xF);
        o->type.scalar = (uint8_t)((w0 >> 8) & 0xFF);
        o->type.dims.assign(w + 3, w + 3 + ndims);
        o->space = (uint8_t)((w0 >> 16) & 0xFF);
    }
    // the values of a data type's fields, flattened in schema order
    void data_values(int type, ptxdump::PackedCursor& cur, std::vector<uint32_t>* out) const {
        const PtxType& ty = ptx_types[type];
        switch (ty.kind) {
        case 0:
            out->push_back(cur.next());
            if (ty.a == 3) out->push_back(cur.next());       // 64-bit value: two halves
            break;
        case 1: out->push_back(cur.next()); break;
        case 2:
            for (int i = 0; i < ty.b; i++) data_values(ptx_fields[ty.a + i].type, cur, out);
            break;
        case 3: {
            const uint32_t v = cur.next();
            out->push_back(v);
            const PtxVariant& vr = ptx_variants[ty.a + v];
            for (int i = 0; i < vr.n_fields; i++) data_values(ptx_fields[vr.first_field + i].type, cur, out);
            break;
        }
        default: {
            const uint32_t some = cur.next();
            out->push_back(some);
            if (some) data_values(ty.a, cur, out);
            break;
        }
        }
    }
    void instruction(const uint32_t* rec, Instruction* o) const {
        const uint32_t w0 = rec[0];
        const uint32_t* w = rec + 1;
        const uint32_t w1 = (w0 & 0xFF) == U_INSTR ? (((w0 >> 29) & 3u) | (((w0 >> 22) & 0x7Fu) << 16)) : rec[ptxdump::rec_len(w0)];
        o->variant = (uint16_t)(w1 >> 16);
        o->has_pred = (w1 & 1) != 0;
        o->pred_not = (w1 & 2) != 0;
        if (o->has_pred) { o->pred = str(w[0], w[1]); w += 2; }
        const PtxInstr& in = ptx_instrs[o->variant];
        if (o->variant == I_Bra) { o->target = str(w[0], w[1]); return; }
        if (o->variant == I_Call) {
            const uint32_t callee = w[1], n_rets = w[4];
            o->uniform = w[0] != 0;
            o->func = str(w[2], w[3]);
            const uint32_t* rets = w + 5;
            const uint32_t* p = rets + 2 * n_rets;
            const uint32_t n_inputs = *p++;
            std::vector<Operand> inputs(n_inputs);
            for (uint32_t i = 0; i < n_inputs; i++) p = operand(p, &inputs[i]);
            o->resolved = *p != 0;
            if (o->resolved) {
                const uint32_t* f = r.v.words + callee;      // the callee's U_FUNC record
                const uint32_t cr = f[4], ci = f[5];
                const uint32_t* var = f + 8;
                o->callee_rets.resize(cr);
                o->callee_inputs.resize(ci);
                for (uint32_t i = 0; i < cr; i++) { type_space(var, &o->callee_rets[i]); var = ptxdump::skip_variable(var); }
                for (uint32_t i = 0; i < ci; i++) { type_space(var, &o->callee_inputs[i]); var = ptxdump::skip_variable(var); }
                for (uint32_t i = 0; i < n_rets; i++) o->call_rets.push_back(str(rets[2 * i], rets[2 * i + 1]));
                o->args = std::move(inputs);
            }
            return;
        }
        if (in.data_type >= 0 && !(ptx_types[in.data_type].kind == 2 && ptx_types[in.data_type].b == 0)) {
            ptxdump::PackedCursor cur;
            cur.w = w;
            data_values(in.data_type, cur, &o->data);
            w = cur.w;
        }
        o->args.resize((size_t)in.n_args);
        for (int i = 0; i < in.n_args; i++) {
            if (*w == PTX_ABSENT) { o->args[i].absent = true; w++; }
            else w = operand(w, &o->args[i]);
        }
    }
    void multi_variable(const uint32_t* w, MultiVariable* o) const {
        const uint32_t n_names = w[2];
        const uint32_t* names = w + 3;
        o->parameterized = w[0] != 0;
        o->count = w[1];
        info(names + 2 * n_names, &o->info);
        if (o->parameterized) o->name = str(names[0], names[1]);
        else
            for (uint32_t i = 0; i < n_names; i++) o->names.push_back(str(names[2 * i], names[2 * i + 1]));
    }
    // the statements of a function body: records from q up to (not including) the U_FUNC_END at `end`
    void body(const uint32_t* q, const uint32_t* end, std::vector<Statement>* out) const {
        std::vector<std::vector<Statement>*> stack;
        stack.push_back(out);
        while (q < end) {
            const uint32_t kind = q[0] & 0xFF, len = ptxdump::rec_len(q[0]);
            std::vector<Statement>* cur = stack.back();
            switch (kind) {
            case U_LABEL: {
                cur->emplace_back();
                cur->back().kind = ST_LABEL;
                cur->back().label = str(q[1], q[2]);
                m.nodes++;
                break;
            }
            case U_VAR:
                cur->emplace_back();
                cur->back().kind = ST_VARIABLE;
                multi_variable(q + 1, &cur->back().var);
                m.nodes++;
                break;
            case U_INSTR:
            case U_INSTR_LONG:
                cur->emplace_back();
                cur->back().kind = ST_INSTRUCTION;
                instruction(q, &cur->back().ins);
                m.nodes++;
                break;
            case U_BLOCK_OPEN:
                cur->emplace_back();
                cur->back().kind = ST_BLOCK;
                m.nodes++;
                stack.push_back(&cur->back().block);
                break;
            case U_BLOCK_CLOSE:
                if (stack.size() > 1) stack.pop_back();
                break;
            default: break;
            }
            q += 1 + len;
        }
    }
};

// module `mi` of a fetched batch as a tree
inline void materialize(const PtxBatchView& v, uint32_t mi, Module* out) {
    ptxdump::Reader r(v, mi);
    Module& m = *out;
    Builder b{r, m};
    const PtxModuleResult& res = v.results[mi];
    const uint32_t n_lex = res.lexerr_end - res.lexerr_begin;
    const uint64_t base = v.layout[mi].text_off;
    const bool skip_parse = n_lex != 0 && v.mode != 2;
    for (uint32_t i = res.lexerr_begin; i < res.lexerr_end; i++) {
        Error e;
        e.lexer = true;
        e.lex_start = v.lexerrs[2 * (size_t)i] - base;
        m.errors.push_back(e);
    }
    if (res.sequential && ((res.status & US_MASK) == US_DIVERGE || (res.status & US_MASK) == US_REFUSED) && !skip_parse) {
        m.verdict = (res.status & US_MASK) == US_DIVERGE ? V_DIVERGES : V_REFUSED;
        m.errors.clear();
        return;
    }
    struct Dir {
        const uint32_t* rec;
        const uint32_t* end;
        uint32_t kind, start_off, n_errors;
    };
    std::vector<Dir> dirs;
    bool parsed_ok = false;
    const uint32_t* header = nullptr;
    uint32_t n_parse_errs = 0;
    if (!skip_parse) {
        const uint32_t* w = v.words + res.word_begin;
        const uint32_t* wend = v.words + res.word_end;
        parsed_ok = w != wend;
        while (w < wend) {
            const uint32_t kind = w[0] & 0xFF, len = ptxdump::rec_len(w[0]);
            const uint32_t* next = w + 1 + len;
            switch (kind) {
            case U_HEADER: header = w; break;
            case U_MODULE_FAIL: parsed_ok = false; break;
            case U_FUNC: {
                if (w[1] & FUNC_HAS_BODY) {
                    const uint32_t* q = next;
                    while (q < wend && (q[0] & 0xFF) != U_FUNC_END) q += 1 + ptxdump::rec_len(q[0]);
                    if (q < wend) q += 1 + ptxdump::rec_len(q[0]);
                    next = q;
                }
                dirs.push_back(Dir{w, next, kind, w[7], 0});
                break;
            }
            case U_MODVAR:
            case U_DIR_NONE:
            case U_DIR_FAIL: dirs.push_back(Dir{w, next, kind, w[1], 0}); break;
            default: break;
            }
            w = next;
        }
        if (!header) parsed_ok = false;
        size_t di = 0;
        for (uint32_t e = res.err_begin; e < res.err_end; e++) {
            const PtxErrRec& er = v.errs[e];
            if ((er.w0 & 0xFFFF) == E_NONE) continue;
            n_parse_errs++;
            Error x;
            x.w0 = er.w0;
            x.a = er.a;
            x.b = er.b;
            m.errors.push_back(x);
            while (di + 1 < dirs.size() && dirs[di + 1].start_off <= er.pos) di++;
            if (!dirs.empty() && dirs[di].start_off <= er.pos) dirs[di].n_errors++;
        }
        m.implicit_parser_error = !parsed_ok && res.word_begin == res.word_end;
    }
    uint64_t invalid = 0;
    for (const Dir& d : dirs) invalid += d.n_errors ? 1 : 0;
    if (skip_parse) m.verdict = v.mode == 0 ? V_ERR : V_EMPTY;
    else if (v.mode == 0) {
        m.have_module = parsed_ok && n_parse_errs == 0 && invalid == 0 && n_lex == 0;
        m.verdict = m.have_module ? V_OK : V_ERR;
    } else if (v.mode == 1) {
        m.have_module = parsed_ok;
        m.verdict = parsed_ok ? V_MODULE : V_EMPTY;
    } else {
        m.verdict = V_ERRORS;
    }
    if (res.sequential && (res.status & US_MASK) == US_PANIC) { m.verdict = V_PANICS; m.have_module = false; }
    if (!m.have_module) return;
    const uint32_t h = header[1];
    m.major = (uint8_t)(h & 0xFF);
    m.minor = (uint8_t)((h >> 8) & 0xFF);
    m.address_size = (uint8_t)((h >> 16) & 0xFF);
    m.sm = header[2];
    m.invalid_directives = invalid;
    for (const Dir& d : dirs) {
        if (d.n_errors || (d.kind != U_FUNC && d.kind != U_MODVAR)) continue;
        m.directives.emplace_back();
        Directive& out_d = m.directives.back();
        m.nodes++;
        const uint32_t* p = d.rec;
        if (d.kind == U_MODVAR) {
            // [hdr, start_off, linking, MULTIVARIABLE(parameterized, count, n_names, name, INFO)]
            out_d.linking = (uint8_t)p[2];
            const uint32_t* mv = p + 3;
            b.info(mv + 3 + 2 * mv[2], &out_d.var.info);
            out_d.var.name = b.str(mv[3], mv[4]);
            continue;
        }
        out_d.is_method = true;
        const uint32_t flags = p[1], n_rets = p[4], n_inputs = p[5];
        out_d.linking = (uint8_t)(flags & FUNC_LINKING_MASK);
        Function& f = out_d.func;
        f.is_kernel = (flags & FUNC_IS_KERNEL) != 0;
        f.has_body = (flags & FUNC_HAS_BODY) != 0;
        f.name = b.str(p[2], p[3]);
        const uint32_t* var = p + 8;
        f.rets.resize(n_rets);
        f.inputs.resize(n_inputs);
        for (uint32_t i = 0; i < n_rets; i++) var = b.variable(var, &f.rets[i]);
        for (uint32_t i = 0; i < n_inputs; i++) var = b.variable(var, &f.inputs[i]);
        const uint32_t n_tuning = flags >> FUNC_TUNING_SHIFT;
        for (uint32_t i = 0; i < n_tuning; i++, var += 4) {
            Tuning t;
            t.kind = var[0];
            t.v[0] = var[1];
            t.v[1] = var[2];
            t.v[2] = var[3];
            f.tuning.push_back(t);
        }
        if (f.has_body) {
            const uint32_t* q = p + 1 + ptxdump::rec_len(p[0]);
            const uint32_t* end = d.end;
            // d.end lies behind the U_FUNC_END record: the body's records stop in front of it
            b.body(q, end, &f.body);
        }
    }
}

// ---- the canonical text of a tree
struct Printer {
    ptxdump::Out& o;
    void str(const Str& s) { o.str(s.p, s.n); }
    void roi(const RegOrImm& x) {
        if (x.is_reg) { o.put("Reg("); str(x.reg); o.put(")"); }
        else { o.put("Imm("); ptxdump::imm(o, x.imm.kind, (uint32_t)x.imm.bits, (uint32_t)(x.imm.bits >> 32)); o.put(")"); }
    }
    void operand(const Operand& p) {
        switch (p.kind) {
        case OPK_REG: o.put("Reg("); str(p.name); o.put(")"); break;
        case OPK_REG_OFFSET: o.put("RegOffset("); str(p.name); o.putf(", %d)", p.offset); break;
        case OPK_IMM: o.put("Imm("); ptxdump::imm(o, p.imm.kind, (uint32_t)p.imm.bits, (uint32_t)(p.imm.bits >> 32)); o.put(")"); break;
        case OPK_VEC_MEMBER: o.put("VecMember("); str(p.name); o.putf(", %u)", p.index); break;
        default:
            o.put("VecPack([");
            for (size_t i = 0; i < p.pack.size(); i++) {
                if (i) o.put(", ");
                roi(p.pack[i]);
            }
            o.put("])");
            break;
        }
    }
    void type(const Type& t) {
        if (t.tkind == 3) { o.put("Texref"); return; }
        if (t.tkind == 2) {
            if (t.vec) o.putf("Array(Some(%u), %s, [", t.vec, ScalarType_names[t.scalar]);
            else o.putf("Array(None, %s, [", ScalarType_names[t.scalar]);
            for (size_t i = 0; i < t.dims.size(); i++) o.putf(i ? ", %u" : "%u", t.dims[i]);
            o.put("])");
            return;
        }
        if (t.vec) o.putf("Vector(%u, %s)", t.vec, ScalarType_names[t.scalar]);
        else o.putf("Scalar(%s)", ScalarType_names[t.scalar]);
    }
    void info(const VariableInfo& v) {
        if (v.has_align) o.putf("VariableInfo { align: Some(%u), v_type: ", v.align);
        else o.put("VariableInfo { align: None, v_type: ");
        type(v.type);
        o.putf(", state_space: %s, array_init: [", StateSpace_names[v.space]);
        for (size_t i = 0; i < v.array_init.size(); i++) {
            if (i) o.put(", ");
            roi(v.array_init[i]);
        }
        o.put("] }");
    }
    void variable(const Variable& v) {
        o.put("Variable { info: ");
        info(v.info);
        o.put(", name: ");
        str(v.name);
        o.put(" }");
    }
    void type_space(const TypeSpace& t) {
        o.put("(");
        type(t.type);
        o.putf(", %s)", StateSpace_names[t.space]);
    }
    void schema(int ty_id, const uint32_t*& w) {
        const PtxType& ty = ptx_types[ty_id];
        switch (ty.kind) {
        case 0:
            switch (ty.a) {
            case 0: o.put(*w++ ? "true" : "false"); break;
            case 3: { uint64_t x = w[0] | ((uint64_t)w[1] << 32); w += 2; o.putf("%llu", (unsigned long long)x); break; }
            case 4: o.putf("bits=0x%08X", *w++); break;
            default: o.putf("%u", *w++); break;
            }
            break;
        case 1: o.put(ptx_enum_names[ty_id][*w++]); break;
        case 2:
            o.put(ty.name);
            if (ty.b) {
                o.put(" { ");
                for (int i = 0; i < ty.b; i++) {
                    if (i) o.put(", ");
                    o.put(ptx_fields[ty.a + i].name);
                    o.put(": ");
                    schema(ptx_fields[ty.a + i].type, w);
                }
                o.put(" }");
            }
            break;
        case 3: {
            const PtxVariant& vr = ptx_variants[ty.a + *w++];
            o.put(vr.name);
            if (vr.n_fields) {
                o.put(vr.named ? " { " : "(");
                for (int i = 0; i < vr.n_fields; i++) {
                    if (i) o.put(", ");
                    if (vr.named) { o.put(ptx_fields[vr.first_field + i].name); o.put(": "); }
                    schema(ptx_fields[vr.first_field + i].type, w);
                }
                o.put(vr.named ? " }" : ")");
            }
            break;
        }
        default:
            if (*w++) { o.put("Some("); schema(ty.a, w); o.put(")"); }
            else o.put("None");
            break;
        }
    }
    void instruction(const Instruction& x) {
        o.put("Instruction(");
        if (x.has_pred) {
            o.putf("Some(PredAt { not: %s, label: ", x.pred_not ? "true" : "false");
            str(x.pred);
            o.put(" }), ");
        } else {
            o.put("None, ");
        }
        const PtxInstr& in = ptx_instrs[x.variant];
        o.put(in.name);
        if (x.variant == I_Bra) {
            o.put(" { arguments: BraArgs { src: ");
            str(x.target);
            o.put(" } })\n");
            return;
        }
        if (x.variant == I_Call) {
            o.putf(" { data: CallDetails { uniform: %s, return_arguments: [", x.uniform ? "true" : "false");
            for (size_t i = 0; i < x.callee_rets.size(); i++) { if (i) o.put(", "); type_space(x.callee_rets[i]); }
            o.put("], input_arguments: [");
            for (size_t i = 0; i < x.callee_inputs.size(); i++) { if (i) o.put(", "); type_space(x.callee_inputs[i]); }
            o.put("] }, arguments: CallArgs { return_arguments: [");
            for (size_t i = 0; i < x.call_rets.size(); i++) { if (i) o.put(", "); str(x.call_rets[i]); }
            o.put("], func: ");
            str(x.func);
            o.put(", input_arguments: [");
            for (size_t i = 0; i < x.args.size(); i++) { if (i) o.put(", "); operand(x.args[i]); }
            o.put("], is_external: false } })\n");
            return;
        }
        if (in.data_type < 0 && in.n_args == 0) { o.put(")\n"); return; }
        o.put(" { ");
        if (in.data_type >= 0) {
            o.put("data: ");
            if (ptx_types[in.data_type].kind == 2 && ptx_types[in.data_type].b == 0) o.put("()");
            else {
                const uint32_t* w = x.data.data();
                schema(in.data_type, w);
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
                if (x.args[i].absent) o.put(a.optional ? "None" : "<missing>");
                else if (a.optional) { o.put("Some("); operand(x.args[i]); o.put(")"); }
                else operand(x.args[i]);
            }
            o.put(" }");
        }
        o.put(" })\n");
    }
    void statements(const std::vector<Statement>& body, int depth) {
        for (const Statement& s : body) {
            o.indent(depth);
            switch (s.kind) {
            case ST_LABEL: o.put("Label("); str(s.label); o.put(")\n"); break;
            case ST_VARIABLE:
                if (s.var.parameterized) {
                    o.put("Variable(Parameterized { info: ");
                    info(s.var.info);
                    o.put(", name: ");
                    str(s.var.name);
                    o.putf(", count: %u })\n", s.var.count);
                } else {
                    o.put("Variable(Names { info: ");
                    info(s.var.info);
                    o.put(", names: [");
                    for (size_t i = 0; i < s.var.names.size(); i++) { if (i) o.put(", "); str(s.var.names[i]); }
                    o.put("] })\n");
                }
                break;
            case ST_INSTRUCTION: instruction(s.ins); break;
            default:
                o.put("Block([\n");
                statements(s.block, depth + 1);
                o.indent(depth);
                o.put("])\n");
                break;
            }
        }
    }
};

inline std::string print(const PtxBatchView& v, uint32_t mi, const Module& m) {
    ptxdump::Out o;
    Printer p{o};
    ptxdump::Reader r(v, mi);
    static const char* const verdicts[] = {"Ok", "Err", "Module", "Empty", "Errors", "ReferencePanics", "ReferenceDiverges", "SequentialPathRefused"};
    o.putf("mode: %s\nstatus: %s\n", v.mode == 0 ? "checked" : v.mode == 1 ? "unchecked" : "errors", verdicts[m.verdict]);
    if (m.verdict == V_DIVERGES || m.verdict == V_REFUSED) { o.put("errors: 0\n"); return std::move(o.s); }
    if (m.have_module) {
        uint64_t kept = m.directives.size();
        o.putf("Module { ptx_version: (%u, %u), sm_version: %u, address_size: %u, invalid_directives: %llu, directives: %llu }\n", m.major, m.minor,
               m.sm, m.address_size, (unsigned long long)m.invalid_directives, (unsigned long long)kept);
        for (const Directive& d : m.directives) {
            if (!d.is_method) {
                o.putf("Variable(LinkingDirective(%u), ", d.linking);
                p.variable(d.var);
                o.put(")\n");
                continue;
            }
            const Function& f = d.func;
            o.putf("Method(LinkingDirective(%u), Function { func_directive: MethodDeclaration { return_arguments: [", d.linking);
            for (size_t i = 0; i < f.rets.size(); i++) { if (i) o.put(", "); p.variable(f.rets[i]); }
            o.put(f.is_kernel ? "], name: Kernel(" : "], name: Func(");
            p.str(f.name);
            o.put("), input_arguments: [");
            for (size_t i = 0; i < f.inputs.size(); i++) { if (i) o.put(", "); p.variable(f.inputs[i]); }
            o.put("], shared_mem: None }, tuning: [");
            for (size_t i = 0; i < f.tuning.size(); i++) {
                if (i) o.put(", ");
                const Tuning& t = f.tuning[i];
                switch (t.kind) {
                case 0: o.putf("MaxNReg(%u)", t.v[0]); break;
                case 1: o.putf("MaxNtid(%u, %u, %u)", t.v[0], t.v[1], t.v[2]); break;
                case 2: o.putf("ReqNtid(%u, %u, %u)", t.v[0], t.v[1], t.v[2]); break;
                case 3: o.putf("MinNCtaPerSm(%u)", t.v[0]); break;
                default: o.put("NoReturn"); break;
                }
            }
            if (!f.has_body) { o.put("], body: None })\n"); continue; }
            o.put("], body: Some([\n");
            p.statements(f.body, 1);
            o.put("]) })\n");
        }
    } else if (v.mode == 1) {
        o.put("Module { ptx_version: (1, 0), sm_version: 0, address_size: 64, invalid_directives: 18446744073709551615, directives: 0 }\n");
    }
    const bool skip_parse = !m.errors.empty() && m.errors[0].lexer && v.mode != 2;
    size_t total = 0;
    for (const Error& e : m.errors) total += (e.lexer || !skip_parse) ? 1 : 0;
    if (m.implicit_parser_error) total++;
    o.putf("errors: %u\n", (unsigned)total);
    for (const Error& e : m.errors) {
        if (e.lexer) o.putf("Lexer(start=%llu)\n", (unsigned long long)e.lex_start);
        else if (!skip_parse) ptxdump::error_line(r, o, e.w0, e.a, e.b);
    }
    if (m.implicit_parser_error) o.put("Parser(ContextError)\n");
    return std::move(o.s);
}

}   // namespace ptxast
