// Sequential host backend for the front-end pipeline.  TEST INFRASTRUCTURE: it runs the product's own step bodies
// (zluda_b200/csrc/ptxfe_pipeline.h) one index at a time on the CPU so that the lexer, the unit speculation, the
// decoders and the record format can be checked against the oracle on a machine without a GPU.  It is not linked
// into the product library and is never a fallback for it.
#include <stdint.h>
#include <time.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <math.h>
#include <string>
#include <vector>

#define PTX_HD
#define PTX_TABLE static const
#include "../../zluda_b200/csrc/ptx_ast.h"
#include "../../zluda_b200/csrc/ptx_partition.h"
#include <thread>

struct HostBackend {
    std::vector<void*> blocks;
    ~HostBackend() { for (void* p : blocks) free(p); }
    void* alloc(size_t bytes) {
        void* p = calloc(bytes + 64, 1);
        blocks.push_back(p);
        return p;
    }
    void zero(void* p, size_t bytes) { memset(p, 0, bytes); }
    void download(void* host, const void* dev, size_t bytes) { memcpy(host, dev, bytes); }
    // PTXFE_EMU_ORDER=reverse runs every parallel-for backwards: a step whose result depends on the order in which its
    // indices run (a data race on the GPU) then shows up as a parity failure on the host.
    bool reverse = getenv("PTXFE_EMU_ORDER") && !strcmp(getenv("PTXFE_EMU_ORDER"), "reverse");
    // PTXFE_EMU_TIMES=1 prints the host time of every step that takes more than 50 ms (to find what is slow in a case)
    bool times = getenv("PTXFE_EMU_TIMES") != nullptr;
    template <class F> void pf(const char* name, size_t n, F f) {
        const clock_t t0 = times ? clock() : 0;
        if (reverse) {
            for (size_t i = n; i-- > 0;) f(i);
        } else {
            for (size_t i = 0; i < n; i++) f(i);
        }
        if (times && (double)(clock() - t0) / CLOCKS_PER_SEC > 0.05) fprintf(stderr, "emu step %s: %.2f s\n", name, (double)(clock() - t0) / CLOCKS_PER_SEC);
    }
    // per-chunk lexer steps: the reader is plain memory (n chunks of text are readable)
    template <class F> void pf_text(const char* name, size_t n, const uint8_t* text, F f) {
        PtxGlobalReader rd{text, (uint32_t)(n * PTX_CHUNK)};
        pf(name, n, [&](size_t c) { f(c, rd); });
    }
    std::vector<char> store_mem;
    PtxClassStore class_store(bool reset) {
        PtxClassStore cs;
        if (store_mem.empty()) { store_mem.assign(PtxClassStore::bytes(), 0); reset = false; }
        cs.carve(store_mem.data());
        if (reset) {
            memset(cs.keys, 0, sizeof(unsigned long long) * PTX_CLASS_SLOTS);
            memset(cs.state, 0, 16);
        }
        return cs;
    }
    // the block-cooperative lexer steps, phase by phase with one "thread" after the other (a small thread count, so
    // that the strided loops of every phase take several rounds)
    PtxLexTables tables;
    bool tables_filled = false;
    const PtxLexTables* lex_tables() {
        if (!tables_filled) { lt_fill_tables(&tables, 0, 1); tables_filled = true; }
        return &tables;
    }
    void lex_mark(const char*, size_t n_tiles, const PtxLexTileArgs& a) {
        const clock_t t0 = clock();
        struct Report { clock_t t0; bool on; ~Report() { if (on && (double)(clock() - t0) / CLOCKS_PER_SEC > 0.05) fprintf(stderr, "emu step lex_mark: %.2f s\n", (double)(clock() - t0) / CLOCKS_PER_SEC); } } report{t0, times};
        const uint32_t nt = 24;
        std::vector<PtxLexMarkShared> shv(1);
        PtxLexMarkShared& sh = shv[0];
        auto phase = [&](auto f) {
            if (reverse) { for (uint32_t t = nt; t-- > 0;) f(t); } else { for (uint32_t t = 0; t < nt; t++) f(t); }
        };
        phase([&](uint32_t t) { lt_mark_tables(sh, a, t, nt); });
        phase([&](uint32_t t) { lt_mark_reset(sh, t, nt); });
        for (size_t tile = 0; tile < n_tiles; tile++) {
            phase([&](uint32_t t) { lt_mark_simple(sh, a, (uint32_t)tile, t, nt); });
            phase([&](uint32_t t) { lt_mark_special(sh, a, (uint32_t)tile, t, nt); });
            phase([&](uint32_t t) { lt_mark_triggers(sh, a, (uint32_t)tile, t, nt); });
            phase([&](uint32_t t) { lt_mark_finish(sh, a, (uint32_t)tile, t, nt); });
        }
    }
    void lex_emit(const char*, size_t n_tiles, const PtxLexTileArgs& a) {
        const clock_t t0 = clock();
        struct Report { clock_t t0; bool on; ~Report() { if (on && (double)(clock() - t0) / CLOCKS_PER_SEC > 0.05) fprintf(stderr, "emu step lex_emit: %.2f s\n", (double)(clock() - t0) / CLOCKS_PER_SEC); } } report{t0, times};
        const uint32_t nt = 256;     // the device's block size: the init phase then holds its text words the same way
        std::vector<PtxLexEmitShared> shv(1);
        PtxLexEmitShared& sh = shv[0];
        auto phase = [&](auto f) {
            if (reverse) { for (uint32_t t = nt; t-- > 0;) f(t); } else { for (uint32_t t = 0; t < nt; t++) f(t); }
        };
        phase([&](uint32_t t) { lt_emit_tables(sh, a, t, nt); });
        for (size_t tile = 0; tile < n_tiles; tile++) {
            phase([&](uint32_t t) { lt_emit_init(sh, a, (uint32_t)tile, t, nt); });
            for (uint32_t pass = 0, passes = lt_emit_passes(sh); pass < passes; pass++) {
                phase([&](uint32_t t) { lt_emit_list(sh, pass, t, nt); });
                phase([&](uint32_t t) { lt_emit_first(sh, a, (uint32_t)tile, pass, t, nt); });
                phase([&](uint32_t t) { lt_emit_keywords(sh, a, (uint32_t)tile, pass, t, nt); });
                phase([&](uint32_t t) { lt_emit_second(sh, a, (uint32_t)tile, pass, t, nt); });
            }
        }
    }
    // stage B: the per-thread bodies of the device kernel, tile after tile; the prefix of the earlier tiles is a running
    // value here (the device finds it by looking back along the tiles)
    void fail(const char* why) {
        fprintf(stderr, "ptxfe_emu: %s\n", why);
        abort();
    }
    void structure(const char*, const PtxStructArgs& a) {
        const size_t n_tiles = ((size_t)a.n_tokens + SX_TILE - 1) / SX_TILE;
        std::vector<SxThread> th(SX_THREADS);
        std::vector<PtxSeg3> before(SX_THREADS);
        std::vector<uint32_t> ubefore(SX_THREADS), starts(SX_THREADS);
        uint8_t table[512];
        for (uint32_t k = 0; k < 512; k++) table[k] = (uint8_t)sx_flags(k);
        PtxSeg3 run{0, 0, 0};
        uint32_t units = 0;
        SegDepthOp op;
        auto phase = [&](auto f) {
            if (reverse) { for (uint32_t t = SX_THREADS; t-- > 0;) f(t); } else { for (uint32_t t = 0; t < SX_THREADS; t++) f(t); }
        };
        std::vector<uint32_t> marks(n_tiles + 1, 0);
        pf("structure_mark", a.n_modules, [&](size_t m) { sx_mark_tiles(a, (uint32_t)m, marks.data(), 1); });
        if (marks[n_tiles]) fail("structure: a mark behind the last tile");
        for (size_t tile = 0; tile < n_tiles; tile++) {
            std::vector<PtxSeg3> agg(SX_THREADS);
            const bool has_first = marks[tile] != 0;
            if (has_first != sx_tile_has_first(a, (uint32_t)(tile * SX_TILE))) fail("structure: tile marks and module table disagree");
            phase([&](uint32_t t) {
                sx_load(a, (uint32_t)(tile * SX_TILE + t * SX_ITEMS), th[t], table, has_first);
                agg[t] = sx_aggregate(a, th[t]);
            });
            for (uint32_t t = 0; t < SX_THREADS; t++) { before[t] = run; run = op(run, agg[t]); }
            phase([&](uint32_t t) { starts[t] = sx_decide(a, th[t], sx_depth(before[t])); });
            // the bitwise case against the token-by-token case, thread by thread
            for (uint32_t t = 0; t < SX_THREADS; t++) {
                if (!th[t].fast) continue;
                SxThread slow;
                sx_load(a, th[t].tb, slow, table, true, false);
                PtxSeg3 x = sx_aggregate(a, slow);
                if (x.scope != agg[t].scope || sx_depth(x) != sx_depth(agg[t]) || x.flag != agg[t].flag || sx_decide(a, slow, sx_depth(before[t])) != starts[t])
                    fail("structure: the bitwise case and the token-by-token case disagree");
            }
            for (uint32_t t = 0; t < SX_THREADS; t++) { ubefore[t] = units; units += sx_popc(starts[t]); }
            phase([&](uint32_t t) { sx_write(a, th[t], sx_depth(before[t]), starts[t], ubefore[t]); });
        }
    }
    template <class F> void pf_staged(const char* name, size_t n, uint32_t* table, uint32_t row_words, F f) {
        const uint32_t cap = 40, win_cap = 5;   // a small window, so that decoders cross its end
        std::vector<uint32_t> stage(cap);
        std::vector<PtxTokenWord> win(win_cap);
        PtxScratch sc{stage.data(), 1u, cap, win.data(), 1u, win_cap};
        pf(name, n, [&](size_t i) {
            PtxStaged r = f(i, sc);
            for (uint32_t k = 0; k < r.n; k++) table[(size_t)r.unit * row_words + k] = stage[k];
        });
    }
    template <class F> void pf_segments(const char* name, size_t n, const PtxPair* off, F f) {
        pf(name, n, [&](size_t s) {
            for (uint32_t i = 0, cnt = off[s + 1].a - off[s].a; i < cnt; i++) f(s, i, off[s].a + i);
        });
    }
    void emit_records(const char* name, size_t n, const PtxPair* off, const PtxEmitStep& e) {
        std::vector<std::pair<size_t, uint32_t>> later;
        pf(name, n, [&](size_t u) {
            const PtxEmitUnit info = e.unit(u);
            for (uint32_t i = 0, cnt = off[u + 1].a - off[u].a; i < cnt; i++) {
                uint32_t x = 0;
                const int what = e.word(info, u, i, x);
                if (what == PtxEmitStep::WRITE) e.words[off[u].a + i] = x;
                else if (what == PtxEmitStep::SECOND_ROUND) later.push_back({u, i});
            }
        });
        for (auto& it : later) e.literal(e.unit(it.first), it.second, off[it.first].a + it.second);
    }
    void sort_by_key(const char*, size_t n, const uint16_t* key, uint32_t* order) {
        std::vector<uint32_t> cursor(PTX_SORT_BUCKETS + 1, 0);
        for (size_t i = 0; i < n; i++) cursor[key[i] + 1]++;
        for (size_t b = 0; b < PTX_SORT_BUCKETS; b++) cursor[b + 1] += cursor[b];
        for (size_t i = 0; i < n; i++) order[cursor[key[i]]++] = (uint32_t)i;
    }
    template <class T, class Ld, class St, class Op> void scan(const char*, size_t n, Ld ld, St st, Op op, T identity) {
        T acc = identity;
        for (size_t i = 0; i < n; i++) {
            acc = op(acc, ld(i));
            st(i, acc);
        }
    }
};

extern "C" {

// Parse n modules; returns the dumps concatenated with '\0' separators (malloc'ed).  stats: tokens, units, words,
// errors, modules that took the sequential path.
char* emu_parse(const char* const* texts, const uint64_t* lens, uint32_t n, uint32_t mode, uint64_t* out_len, uint64_t* stats) {
    HostBackend bk;
    PtxWork w;
    if (const char* e = getenv("PTXFE_SEQ_MAX_TOKENS")) w.seq_max_tokens = (uint32_t)strtoul(e, nullptr, 10);
    std::vector<PtxModuleLayout> layout(n);
    std::vector<uint32_t> mcb(n + 1);
    uint64_t off = 0;
    uint32_t chunks = 0;
    for (uint32_t m = 0; m < n; m++) {
        layout[m].text_off = off;
        layout[m].text_len = lens[m];
        layout[m].chunk_begin = chunks;
        layout[m].pad = 0;
        mcb[m] = chunks;
        uint32_t c = (uint32_t)((lens[m] + PTX_CHUNK - 1) / PTX_CHUNK);
        chunks += c;
        off += (uint64_t)c * PTX_CHUNK;
    }
    mcb[n] = chunks;
    uint8_t* text = (uint8_t*)bk.alloc(off + 64);
    for (uint32_t m = 0; m < n; m++) memcpy(text + layout[m].text_off, texts[m], lens[m]);
    w.text = text;
    w.n_modules = n;
    w.n_chunks = chunks;
    w.layout = layout.data();
    w.mod_chunk_begin = mcb.data();
    w.results = (PtxModuleResult*)bk.alloc(sizeof(PtxModuleResult) * (n + 1));
    w.counters = (PtxCounters*)bk.alloc(sizeof(PtxCounters));
    PtxCounters hc;
    memset(&hc, 0, sizeof hc);
    ptx_stage_lex(bk, w, hc);
    ptx_stage_structure(bk, w, hc, mode);
    ptx_stage_decode(bk, w, hc);
    PtxBatchView v;
    v.n_modules = n;
    v.mode = mode;
    v.layout = w.layout;
    v.results = w.results;
    v.words = w.words;
    v.errs = w.errs;
    v.lexerrs = w.lexerrs;
    v.texts = texts;
    std::string all;
    uint64_t seq = 0, seq_tokens = 0;
    for (uint32_t m = 0; m < n; m++) {
        int st;
        std::string by_records = ptxdump::dump_module(v, m, &st);
        if (getenv("PTXFE_EMU_TREE")) {
            // the materialiser's way: records -> tree -> text; must be the same text
            ptxast::Module mod;
            ptxast::materialize(v, m, &mod);
            std::string by_tree = ptxast::print(v, m, mod);
            if (by_tree != by_records) by_records = "TREE DUMP DIFFERS\n" + by_tree;
        }
        all += by_records;
        all.push_back('\0');
        seq += w.results[m].sequential;
        seq_tokens += w.results[m].seq_tokens;
    }
    if (stats) {
        stats[0] = hc.n_tokens;
        stats[1] = hc.n_units;
        stats[2] = hc.n_words;
        stats[3] = hc.n_errs;
        stats[4] = seq;
        stats[5] = hc.pad;
        stats[6] = hc.n_bulk;
        stats[7] = hc.n_rest;
        stats[8] = hc.n_classes;
        stats[9] = seq_tokens;
    }
    char* r = (char*)malloc(all.size() + 1);
    memcpy(r, all.data(), all.size());
    *out_len = all.size();
    return r;
}

// The sharded form: the product's partitioner splits the batch into n_parts shards, every shard runs through the
// pipeline on a host thread of its own, and the dumps come back in the caller's module order.  part_of[i] = shard of
// module i.
char* emu_parse_multi(const char* const* texts, const uint64_t* lens, uint32_t n, uint32_t n_parts, uint32_t mode, uint64_t* out_len,
                      uint32_t* part_of, uint64_t* part_bytes) {
    PtxPartition part = ptx_partition_greedy(lens, n, n_parts);
    std::vector<std::vector<std::string>> dumps(part.members.size());
    std::vector<std::thread> threads;
    for (size_t k = 0; k < part.members.size(); k++)
        threads.emplace_back([&, k]() {
            std::vector<const char*> t;
            std::vector<uint64_t> l;
            for (uint32_t i : part.members[k]) { t.push_back(texts[i]); l.push_back(lens[i]); }
            uint64_t ol = 0;
            char* r = emu_parse(t.data(), l.data(), (uint32_t)t.size(), mode, &ol, nullptr);
            const char* p = r;
            for (size_t j = 0; j < t.size(); j++) {
                dumps[k].push_back(std::string(p));
                p += dumps[k].back().size() + 1;
            }
            free(r);
        });
    for (std::thread& th : threads) th.join();
    std::string all;
    for (uint32_t i = 0; i < n; i++) {
        all += dumps[part.where[i].first][part.where[i].second];
        all.push_back('\0');
        if (part_of) part_of[i] = part.where[i].first;
    }
    if (part_bytes)
        for (size_t k = 0; k < part.bytes.size(); k++) part_bytes[k] = part.bytes[k];
    char* r = (char*)malloc(all.size() + 1);
    memcpy(r, all.data(), all.size());
    *out_len = all.size();
    return r;
}

// Tokens of one module: triples (kind, start, len), then lex errors (start, len).
uint32_t* emu_lex(const char* text, uint64_t len, uint64_t* n_tokens, uint64_t* n_errors) {
    HostBackend bk;
    PtxWork w;
    PtxModuleLayout layout;
    layout.text_off = 0;
    layout.text_len = len;
    layout.chunk_begin = 0;
    layout.pad = 0;
    uint32_t mcb[2] = {0, (uint32_t)((len + PTX_CHUNK - 1) / PTX_CHUNK)};
    uint8_t* t = (uint8_t*)bk.alloc(len + 256);
    memcpy(t, text, len);
    w.text = t;
    w.n_modules = 1;
    w.n_chunks = mcb[1];
    w.layout = &layout;
    w.mod_chunk_begin = mcb;
    w.results = (PtxModuleResult*)bk.alloc(sizeof(PtxModuleResult) * 2);
    w.counters = (PtxCounters*)bk.alloc(sizeof(PtxCounters));
    PtxCounters hc;
    memset(&hc, 0, sizeof hc);
    ptx_stage_lex(bk, w, hc);
    uint32_t* r = (uint32_t*)malloc(((size_t)hc.n_tokens * 3 + (size_t)hc.n_lexerrs * 2 + 1) * 4);
    size_t k = 0;
    for (uint32_t i = 0; i < hc.n_tokens; i++) {
        r[k++] = w.tokens[i].kind;
        r[k++] = w.tokens[i].start;
        r[k++] = ptx_token_len(t, w.tokens[i], len);
    }
    for (uint32_t i = 0; i < hc.n_lexerrs; i++) { r[k++] = w.lexerrs[2 * i]; r[k++] = w.lexerrs[2 * i + 1]; }
    *n_tokens = hc.n_tokens;
    *n_errors = hc.n_lexerrs;
    return r;
}

uint64_t emu_parse_f64(const char* s, uint32_t len) { return ptx_parse_f64((const uint8_t*)s, len); }
void emu_free(void* p) { free(p); }
}
