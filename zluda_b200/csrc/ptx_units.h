// Unit drivers on top of PtxDecoder: the data-parallel one (one speculated unit per thread) and the sequential one that
// re-parses a whole module with the reference's recovery rules when the speculated units of a module do not meet.
#pragma once
#include "ptx_decode.h"

enum PtxUnitStatus { US_OK = 0, US_FAIL = 1, US_PANIC = 2, US_DIVERGE = 3, US_REFUSED = 4 };
// The sequential parser is one thread at about a microsecond per token and pass: a damaged tail longer than this is not
// parsed at all and its module gets the verdict SequentialPathRefused (a bound on the running time of one launch).
#define PTX_SEQ_MAX_TOKENS (2u << 20)
#define US_MASK 0xFu
#define US_MODULE_FAILED 0x10u     // sequential path: the module-level parse failed (a U_MODULE_FAIL record was written)

struct PtxUnitResult {
    uint32_t end;        // token index where the unit stopped
    uint32_t status;     // PtxUnitStatus
    uint32_t kind;       // PtxUnitKind of the (last) record, 0 if none
    // for U_FUNC:
    uint32_t name_tok, n_rets, n_inputs;
};

// One speculated unit.  `depth` is the scope depth in front of its first token (0 = top level).
PTX_HD PTX_NOINLINE inline PtxUnitResult ptx_decode_unit(PtxDecoder& d, uint32_t start, uint32_t depth, bool module_first) {
    PtxUnitResult r;
    r.status = US_OK;
    r.kind = 0;
    r.name_tok = r.n_rets = r.n_inputs = 0;
    d.pos = start;
    d.unit_tok0 = start;
    d.max_seen = start;
    d.pos_is_unit_mode = true;
    d.unit_off = start < d.te ? d.tk(start).start : 0;
    if (module_first) {
        if (d.header()) r.kind = U_HEADER;
        else r.status = US_FAIL;
    } else if (depth == 0) {
        bool has_body = false;
        int k = d.directive(PTX_ABSENT, &has_body, &r.name_tok, &r.n_rets, &r.n_inputs);
        if (k == 0) {
            if (d.recover_directive()) k = U_DIR_FAIL;
            else r.status = US_FAIL;
        }
        r.kind = (uint32_t)k;
    } else {
        uint16_t k = d.kind();
        uint32_t m;
        if (k == T_LBRACE) {
            d.begin_record(&m);
            d.end_record(m, U_BLOCK_OPEN);
            d.pos++;
            r.kind = U_BLOCK_OPEN;
        } else if (k == T_RBRACE) {
            d.begin_record(&m);
            d.end_record(m, depth == 1 ? U_FUNC_END : U_BLOCK_CLOSE);
            d.pos++;
            r.kind = depth == 1 ? U_FUNC_END : U_BLOCK_CLOSE;
        } else {
            int s = d.statement();
            if (s == -2) s = d.recover_statement();
            if (s == 0) r.status = US_FAIL;
            else if (s < 0) r.status = US_PANIC;
            r.kind = U_INSTR;
        }
    }
    r.end = d.pos;
    return r;
}

#define PTX_SEQ_MAX_DEPTH 64

// Whole module, sequentially, exactly as the reference's `module` parser would (lib.rs:503-526, 579-617, 847-880).
// `tb` = first token of the module.  `base` = global word offset of the sink's first word (write mode).
// Returns US_OK, US_PANIC where the reference would panic, or US_DIVERGE: a block that fails to parse is recovered from
// its '{' and its contents are parsed again as statements of the enclosing block, so damage below d levels of nesting
// costs the reference 2^d times the work (it does not memoise) and appends as many errors.  After 4 * tokens + 1024
// statement attempts the module is given up with the verdict ReferenceDiverges; this also bounds the running time of
// the one thread that parses it.
// With from_directive set, tb is the first token of a top-level directive instead: the module's header and the
// directives in front of tb were parsed by the speculated units, which met one another up to there, so the sequential
// parser would stand at tb in its directive loop with nothing but the errors so far behind it.
PTX_HD PTX_NOINLINE inline int ptx_decode_module_sequential(PtxDecoder& d, uint32_t tb, uint32_t base, bool from_directive = false) {
    d.stmt_attempts = 0;
    d.stmt_budget = 4ull * (uint64_t)(d.te - tb) + 1024ull;
    d.diverged = false;
    d.pos = tb;
    d.unit_off = tb < d.te ? d.tk(tb).start : 0;
    uint32_t m;
    if (!from_directive && !d.header()) {
        d.push(E_PARSER, 0, 0, 0);
        d.begin_record(&m);
        d.end_record(m, U_MODULE_FAIL);
        return US_OK | US_MODULE_FAILED;
    }
    for (;;) {
        uint32_t save = d.pos;
        uint32_t m0 = d.out.mark();
        if (d.pos < d.te) d.unit_off = d.tk(d.pos).start;
        bool has_body = false;
        uint32_t name_tok, n_rets, n_inputs;
        int k = d.directive(d.resolver.last_func, &has_body, &name_tok, &n_rets, &n_inputs);
        if (k == U_FUNC && has_body) {
            // function body: statements and nested blocks; a block whose statements stop before its '}' fails as a
            // whole and the statement recovery restarts from its '{' (lib.rs:858-880, 1422-1431)
            uint32_t blk_pos[PTX_SEQ_MAX_DEPTH], blk_mark[PTX_SEQ_MAX_DEPTH];
            int sp = 0;
            bool body_ok = false, failed = false;
            while (!failed) {
                uint16_t tk = d.kind();
                if ((tk == T_LBRACE || tk == T_RBRACE) && ++d.stmt_attempts > d.stmt_budget) return US_DIVERGE;
                if (tk == T_LBRACE) {
                    if (sp == PTX_SEQ_MAX_DEPTH) { d.push(E_PARSER, 1, 0, 0); failed = true; break; }
                    blk_pos[sp] = d.pos;
                    blk_mark[sp] = d.out.mark();
                    sp++;
                    d.begin_record(&m);
                    d.end_record(m, U_BLOCK_OPEN);
                    d.pos++;
                    continue;
                }
                if (tk == T_RBRACE) {
                    d.begin_record(&m);
                    d.end_record(m, sp == 0 ? U_FUNC_END : U_BLOCK_CLOSE);
                    d.pos++;
                    if (sp == 0) { body_ok = true; break; }
                    sp--;
                    continue;
                }
                int s = d.statement();
                if (d.diverged) return US_DIVERGE;
                if (s == -2) s = d.recover_statement();
                if (s == 1) continue;
                if (s < 0) return US_PANIC;
                // neither statement nor recovery: the innermost open construct fails
                for (;;) {
                    if (sp == 0) { failed = true; break; }
                    sp--;
                    d.pos = blk_pos[sp];
                    d.out.reset(blk_mark[sp]);
                    int s2 = d.recover_statement();
                    if (s2 == 1) break;
                    if (s2 < 0) return US_PANIC;
                }
            }
            if (!body_ok) {
                d.pos = save;
                d.out.reset(m0);
                k = 0;
            }
        }
        if (k == U_FUNC) d.resolver.last_func = base + m0;
        if (k == 0) {
            d.pos = save;
            if (!d.recover_directive()) break;
        }
    }
    if (d.pos != d.te) {
        d.push(E_PARSER, 0, 0, 0);
        d.begin_record(&m);
        d.end_record(m, U_MODULE_FAIL);
        return US_OK | US_MODULE_FAILED;
    }
    return US_OK;
}
