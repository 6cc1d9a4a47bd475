// Unit drivers on top of PtxDecoder: the data-parallel one (one speculated unit per thread) and the sequential one that
// re-parses a whole module with the reference's recovery rules when the speculated units of a module do not meet.
#pragma once
#include "ptx_decode.h"

enum PtxUnitStatus { US_OK = 0, US_FAIL = 1, US_PANIC = 2 };

struct PtxPair {
    uint32_t a, b;
};

// ---- call resolution
// Data-parallel path: an open-addressing table over all function directives of the batch.
struct PtxFnEntry {
    uint32_t unit;       // unit index of the function's header
    uint32_t dir_ord;    // ordinal of that directive among the batch's top-level units
    uint32_t name_off, name_len;
    uint32_t n_rets, n_inputs;
    uint32_t module;
    uint32_t pad;
};
PTX_HD inline uint32_t ptx_name_hash(const uint8_t* text, uint32_t off, uint32_t len, uint32_t module) {
    uint32_t h = 2166136261u ^ (module * 0x9E3779B9u);
    for (uint32_t i = 0; i < len; i++) h = (h ^ text[off + i]) * 16777619u;
    return h ^ (h >> 13);
}
struct PtxHashResolver {
    const PtxFnEntry* entries;
    const uint32_t* slots;      // entry index or PTX_ABSENT
    uint32_t mask;
    const PtxPair* unit_off;    // .a = word offset of every unit's records
    uint32_t module, my_dir_ord;
    PTX_HD PtxCallee find(const uint8_t* text, uint32_t off, uint32_t len) const {
        PtxCallee best;
        best.record = PTX_ABSENT;
        best.n_rets = best.n_inputs = 0;
        if (!slots) return best;
        uint32_t best_ord = 0;
        bool have = false;
        uint32_t h = ptx_name_hash(text, off, len, module) & mask;
        for (uint32_t probes = 0; probes <= mask; probes++) {
            uint32_t e = slots[h];
            if (e == PTX_ABSENT) break;
            const PtxFnEntry en = entries[e];
            if (en.module == module && en.name_len == len && en.dir_ord < my_dir_ord && (!have || en.dir_ord > best_ord)) {
                bool same = true;
                for (uint32_t i = 0; i < len; i++)
                    if (text[en.name_off + i] != text[off + i]) { same = false; break; }
                if (same) {
                    have = true;
                    best_ord = en.dir_ord;
                    best.record = unit_off[en.unit].a;
                    best.n_rets = en.n_rets;
                    best.n_inputs = en.n_inputs;
                }
            }
            h = (h + 1) & mask;
        }
        return best;
    }
};
// Sequential path: function records of one module are chained through their prev_func_record word.
struct PtxChainResolver {
    const uint32_t* words;   // the batch's output words (global offsets)
    uint32_t last_func;      // record offset of the last function recorded so far, PTX_ABSENT if none
    PTX_HD PtxCallee find(const uint8_t* text, uint32_t off, uint32_t len) const {
        PtxCallee r;
        r.record = PTX_ABSENT;
        r.n_rets = r.n_inputs = 0;
        uint32_t f = last_func;
        while (f != PTX_ABSENT && words) {
            uint32_t noff = words[f + 2], nlen = words[f + 3];
            bool same = nlen == len;
            for (uint32_t i = 0; same && i < len; i++) same = text[noff + i] == text[off + i];
            if (same) {
                r.record = f;
                r.n_rets = words[f + 4];
                r.n_inputs = words[f + 5];
                return r;
            }
            f = words[f + 6];
        }
        return r;
    }
};

struct PtxUnitResult {
    uint32_t end;        // token index where the unit stopped
    uint32_t status;     // PtxUnitStatus
    uint32_t kind;       // PtxUnitKind of the (last) record, 0 if none
    // for U_FUNC:
    uint32_t name_tok, n_rets, n_inputs;
};

// One speculated unit.  `depth` is the scope depth in front of its first token (0 = top level).
template <class Sink, class Resolver>
PTX_HD inline PtxUnitResult ptx_decode_unit(PtxDecoder<Sink, Resolver>& d, uint32_t start, uint32_t depth, bool module_first) {
    PtxUnitResult r;
    r.status = US_OK;
    r.kind = 0;
    r.name_tok = r.n_rets = r.n_inputs = 0;
    d.pos = start;
    d.unit_off = start < d.te ? d.tok[start].start : 0;
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
// Returns US_OK, or US_PANIC where the reference would panic.
template <class Sink>
PTX_HD inline int ptx_decode_module_sequential(PtxDecoder<Sink, PtxChainResolver>& d, uint32_t tb, uint32_t base) {
    d.pos = tb;
    d.unit_off = tb < d.te ? d.tok[tb].start : 0;
    uint32_t m;
    if (!d.header()) {
        d.push(E_PARSER, 0, 0, 0);
        d.begin_record(&m);
        d.end_record(m, U_MODULE_FAIL);
        return US_OK;
    }
    for (;;) {
        uint32_t save = d.pos;
        uint32_t m0 = d.out.mark();
        if (d.pos < d.te) d.unit_off = d.tok[d.pos].start;
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
    }
    return US_OK;
}
