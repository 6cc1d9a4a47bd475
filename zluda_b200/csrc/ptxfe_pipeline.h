// The front-end pipeline as a sequence of data-parallel steps (parallel-for over chunks, tokens or units) and prefix
// scans, written once against a small backend interface.  The CUDA backend (ptxfe.cu) runs every step as a kernel on
// the context's stream; the test suite has a sequential backend that runs the same step bodies on the host to check
// the logic where no GPU is present.  No step reads another thread's work of the same step.
//
//   text -> [context vectors | scan] -> [count tokens | scan | emit tokens]
//        -> [brace / paren classification | segmented scan] -> [unit starts | scan | compact]
//        -> [decode units: count] -> [chain check per module] -> [scan sizes] -> [function table] -> [decode units: emit]
#pragma once
#include "ptx_units.h"

struct PtxModuleLayout {
    uint64_t text_off;    // byte offset in the batch text buffer (multiple of PTX_CHUNK)
    uint64_t text_len;
    uint32_t chunk_begin; // first chunk index
    uint32_t pad;
};

// per-module results, copied to the host
struct PtxModuleResult {
    uint32_t tok_begin, tok_end;
    uint32_t lexerr_begin, lexerr_end;
    uint32_t unit_begin, unit_end;
    uint32_t word_begin, word_end;
    uint32_t err_begin, err_end;
    uint32_t sequential;   // 1 = parsed by the sequential path
    uint32_t status;       // sequential path: PtxUnitStatus | US_MODULE_FAILED
    uint32_t n_errors;     // parser errors raised (reserved slots that stayed unused not counted)
    uint32_t seq_tokens;   // tokens that went through the sequential path
};

// host view of one fetched batch (input of the dump)
struct PtxErrRec;
struct PtxBatchView {
    uint32_t n_modules = 0, mode = 0;
    const PtxModuleLayout* layout = nullptr;
    const PtxModuleResult* results = nullptr;
    const uint32_t* words = nullptr;
    const PtxErrRec* errs = nullptr;
    const uint32_t* lexerrs = nullptr;
    const char* const* texts = nullptr;
};

struct PtxDepth {
    int32_t scope, paren;
};
struct PtxSeg3 {
    int32_t scope, paren, flag;
};

#define PTX_SORT_BUCKETS 4096u
#define PTX_BULK_MIN_TOKENS 8192u   // statements at least this long get the bulk initialiser path
#define PTX_MAX_BULK 32u            // per batch slice; further ones are decoded by one thread each
#define PTX_TMP_STRIDE 48u     // words per unit in the staging table of the first decode pass (192 bytes: sector aligned)

// fast per-thread memory the backend lends to a staged decoder: room for `stage_cap` record words (word k at
// stage[k * stage_stride]) and for `win_cap` tokens (token k at win[k * win_stride])
struct PtxScratch {
    uint32_t* stage;
    uint32_t stage_stride, stage_cap;
    PtxTokenWord* win;
    uint32_t win_stride, win_cap;
};

// ---- unit classes and record templates
// Two units are in the same class when they have the same token kinds, the same literal codes (ptx_lex.h: what the
// decoder's control flow can learn from a number), the same text in every other token whose text the decoder reads
// (dot-identifiers that are no keyword, strings, `%envreg` names) and the same depth class.  The decoder then takes
// the same path for both, and their records differ only in words taken from tokens (offsets, lengths, converted
// literal values).  One
// representative per class is decoded with tagged output (PtxSink::tags); every other unit is compared with its
// representative token by token and its record is instantiated from the template.
#define PTX_TMPL_WORDS 40u            // longest record that gets a template
#define PTX_MAX_CLASSES (1u << 18)    // templates per batch slice; later classes are decoded the ordinary way
#define PTX_MAX_CLASS_TOKENS 250u
enum { PTX_UNIT_STAGED = 0, PTX_UNIT_FLAGGED = 1, PTX_UNIT_NOTHING = 2, PTX_UNIT_TEMPLATED = 3, PTX_UNIT_UNDECIDED = 0xFF };
struct PtxTemplateInfo {
    uint32_t n_words, n_tokens, ok, depth1;
};
// The per-token side array `kinds` holds kind | aux << 9 (ptx_kind_entry): aux is the literal code of a numeric literal
// and min(length, 127) of any other token.  Most passes want the kind alone; the class passes need the token itself
// only for dot-identifiers, strings and identifiers of 8 or 9 bytes.
#define PTX_KL_KIND(x) ((uint16_t)((x) & 0x1FFu))
#define PTX_KL_LEN(x) ((uint32_t)(x) >> 9)
#define PTX_KL_LONG 127u
static_assert(T_COUNT <= 512, "token kinds must fit 9 bits of the kinds array");
// four bytes of text at any offset (little-endian), bytes at and after `rem` zeroed: two aligned loads and a shift.
// Reads up to 7 bytes past off: the text buffers of the pipeline have that slack.
PTX_HD inline uint32_t ptx_text_word(const uint8_t* text, uint32_t off, uint32_t rem) {
    const uint8_t* a = text + off;
    const uint32_t mis = (uint32_t)((uintptr_t)a & 3u);
    const uint32_t* w = (const uint32_t*)(a - mis);
    uint32_t v = w[0];
    if (mis) v = (v >> (8u * mis)) | (w[1] << (32u - 8u * mis));
    if (rem < 4) v &= (1u << (8u * rem)) - 1u;
    return v;
}
PTX_HD inline bool ptx_text_matters(uint16_t k) { return k == T_DOTIDENT || k == T_STRING; }
// 64-bit class key of the tokens [start, end); 0 = this unit gets no template
PTX_HD inline uint64_t ptx_class_key(const uint8_t* text, const PtxToken* tokens, const uint16_t* kinds, uint32_t start, uint32_t end, uint32_t depth,
                                     bool module_first) {
    if (depth == 0 || module_first || end - start > PTX_MAX_CLASS_TOKENS || end <= start) return 0;
    uint32_t h1 = 2166136261u ^ (depth == 1 ? 1u : 0u), h2 = 0x811C9DC5u + (end - start);
    for (uint32_t i = start; i < end; i++) {
        const uint32_t kl = kinds[i];
        const uint16_t kind = PTX_KL_KIND(kl);
        h1 = (h1 ^ kind) * 16777619u;
        h2 = (h2 + kind) * 0x9E3779B1u;
        h2 ^= h2 >> 15;
        if (ptx_is_numeric_kind(kind)) {
            const uint32_t code = PTX_KL_LEN(kl);
            if (code & PTX_LC_LONG) return 0;
            h1 = (h1 ^ code) * 16777619u;
            h2 = (h2 + code) * 0x85EBCA6Bu;
        } else if (ptx_text_matters(kind)) {
            const PtxToken t = tokens[i];
            if (t.len == 0xFFFF) return 0;
            h2 = (h2 ^ t.len) * 0x85EBCA6Bu;
            for (uint32_t j = 0; j < t.len; j += 4) {
                uint32_t c = ptx_text_word(text, t.start + j, t.len - j);
                h1 = (h1 ^ c) * 16777619u;
                h1 ^= h1 >> 13;
                h2 = (h2 + c) * 0x9E3779B1u;
            }
        } else if (kind == T_IDENT) {
            const uint32_t l = PTX_KL_LEN(kl);
            if (l == PTX_KL_LONG) {
                if (tokens[i].len == 0xFFFF) return 0;
            } else if (l == 8 || l == 9) {
                if (ptx_envreg_number(text + tokens[i].start, l)) h1 = (h1 ^ 0x1234u) * 16777619u;
            }
        }
    }
    uint64_t k = ((uint64_t)h1 << 32) | h2;
    return k ? k : 1;
}
// The class store lives as long as a batch: the slices of one ptxfe_parse_batch call share it, so a class met in
// slice 3 is not decoded again in slice 4.  A class keeps a SIGNATURE (what ptx_class_key hashed, spelled out), so that
// membership can be checked exactly without the representative's tokens, which are gone when its slice is.
//   signature = [n_tokens | depth1 << 31, then per token: kind | x << 16 with x = the literal code of a numeric literal,
//                the envreg flag of an identifier, the length of a token whose text matters, which is followed by
//                ceil(len / 4) words of text]
#define PTX_CLASS_SLOTS (1u << 20)          // hash slots (power of two)
#define PTX_SIG_POOL_WORDS (16u << 20)      // 64 MiB of signatures
struct PtxClassStore {
    unsigned long long* keys;   // [PTX_CLASS_SLOTS] 0 = empty
    uint32_t* slot_tmpl;        // [PTX_CLASS_SLOTS] template id of the slot's class, PTX_ABSENT = none
    uint32_t* tmpl_words;       // [PTX_MAX_CLASSES][PTX_TMPL_WORDS]
    uint16_t* tmpl_tags;        // [PTX_MAX_CLASSES][PTX_TMPL_WORDS]
    PtxTemplateInfo* info;      // [PTX_MAX_CLASSES]
    uint32_t* sig_off;          // [PTX_MAX_CLASSES] word offset of the signature in sig_pool
    uint32_t* sig_pool;         // [PTX_SIG_POOL_WORDS]
    uint32_t* rep_unit;         // [PTX_MAX_CLASSES] representative unit (valid for the classes added by the current slice)
    uint32_t* state;            // [0] classes so far, [1] signature words used, [2] classes before the current slice
    static size_t bytes() {
        return sizeof(unsigned long long) * PTX_CLASS_SLOTS + 4ull * PTX_CLASS_SLOTS + 4ull * PTX_TMPL_WORDS * PTX_MAX_CLASSES +
               2ull * PTX_TMPL_WORDS * PTX_MAX_CLASSES + sizeof(PtxTemplateInfo) * PTX_MAX_CLASSES + 4ull * PTX_MAX_CLASSES +
               4ull * PTX_SIG_POOL_WORDS + 4ull * PTX_MAX_CLASSES + 256;
    }
    // carve the arrays out of one allocation of bytes() bytes (256-byte aligned)
    void carve(void* base) {
        char* p = (char*)base;
        keys = (unsigned long long*)p; p += sizeof(unsigned long long) * PTX_CLASS_SLOTS;
        slot_tmpl = (uint32_t*)p; p += 4ull * PTX_CLASS_SLOTS;
        tmpl_words = (uint32_t*)p; p += 4ull * PTX_TMPL_WORDS * PTX_MAX_CLASSES;
        tmpl_tags = (uint16_t*)p; p += 2ull * PTX_TMPL_WORDS * PTX_MAX_CLASSES;
        info = (PtxTemplateInfo*)p; p += sizeof(PtxTemplateInfo) * PTX_MAX_CLASSES;
        sig_off = (uint32_t*)p; p += 4ull * PTX_MAX_CLASSES;
        sig_pool = (uint32_t*)p; p += 4ull * PTX_SIG_POOL_WORDS;
        rep_unit = (uint32_t*)p; p += 4ull * PTX_MAX_CLASSES;
        state = (uint32_t*)p;
    }
};
PTX_HD inline uint32_t ptx_signature_words(const PtxToken* tokens, uint32_t start, uint32_t n) {
    uint32_t w = 1 + n;
    for (uint32_t i = 0; i < n; i++) {
        const PtxToken t = tokens[start + i];
        if (ptx_text_matters(t.kind)) w += (t.len + 3u) / 4u;
    }
    return w;
}
PTX_HD inline void ptx_signature_write(uint32_t* sig, const uint8_t* text, const PtxToken* tokens, const uint16_t* kinds, uint32_t start, uint32_t n,
                                       uint32_t depth1) {
    *sig++ = n | (depth1 << 31);
    for (uint32_t i = 0; i < n; i++) {
        const PtxToken t = tokens[start + i];
        if (ptx_is_numeric_kind(t.kind)) {
            *sig++ = t.kind | (PTX_KL_LEN(kinds[start + i]) << 16);
        } else if (ptx_text_matters(t.kind)) {
            *sig++ = t.kind | ((uint32_t)t.len << 16);
            for (uint32_t j = 0; j < t.len; j += 4) {
                uint32_t v = ptx_text_word(text, t.start + j, t.len - j);
                *sig++ = v;
            }
        } else if (t.kind == T_IDENT) {
            bool e = (t.len == 8 || t.len == 9) && ptx_envreg_number(text + t.start, t.len);
            *sig++ = t.kind | (e ? 1u << 16 : 0u);
        } else {
            *sig++ = t.kind;
        }
    }
}
// exact check that the unit with tokens [start, start + n) at depth class depth1 has this signature
PTX_HD inline bool ptx_signature_matches(const uint32_t* sig, const uint8_t* text, const PtxToken* tokens, const uint16_t* kinds, uint32_t start,
                                         uint32_t n, uint32_t depth1) {
    if (*sig++ != (n | (depth1 << 31))) return false;
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t kl = kinds[start + i];
        const uint16_t kind = PTX_KL_KIND(kl);
        uint32_t head = *sig++;
        if ((head & 0xFFFFu) != kind) return false;
        if (ptx_is_numeric_kind(kind)) {
            if ((head >> 16) != PTX_KL_LEN(kl)) return false;
        } else if (ptx_text_matters(kind)) {
            const PtxToken t = tokens[start + i];
            if ((head >> 16) != t.len || t.len == 0xFFFF) return false;
            for (uint32_t j = 0; j < t.len; j += 4) {
                uint32_t v = ptx_text_word(text, t.start + j, t.len - j);
                if (*sig++ != v) return false;
            }
        } else if (kind == T_IDENT) {
            const uint32_t l = PTX_KL_LEN(kl);
            bool e = false;
            if (l == PTX_KL_LONG) {
                if (tokens[start + i].len == 0xFFFF) return false;
            } else if (l == 8 || l == 9) {
                e = ptx_envreg_number(text + tokens[start + i].start, l) != 0;
            }
            if ((head >> 16) != (e ? 1u : 0u)) return false;
        }
    }
    return true;
}

// what a staged decoder hands back to the backend: copy n words of this thread's staging buffer to row `unit`
struct PtxStaged {
    uint32_t unit, n;
};

// token classification bits

struct PtxCounters {
    uint32_t n_tokens, n_lexerrs, n_units, n_words, n_errs, n_funcs, any_sequential, pad;
    uint32_t n_flagged;         // units whose records are written by the second decode pass
    uint32_t n_bulk;            // statements long enough for the bulk initialiser path
    uint32_t n_rest;            // units without a template
    uint32_t n_listed;
    uint32_t n_classes;         // statement classes met so far in this batch (all slices)
    uint32_t n_sig_words;       // words of the signature pool in use
    uint32_t struct_abort;      // the structure pass ran into its wait limit (its results are void)
    uint32_t n_skipped;         // modules with tokens that are not parsed (a lexer error, and not the errors-only mode)
};

PTX_HD inline uint32_t ptx_upper_bound_u32(const uint32_t* a, uint32_t n, uint32_t x) {
    // number of entries <= x
    uint32_t lo = 0, hi = n;
    while (lo < hi) {
        uint32_t mid = (lo + hi) >> 1;
        if (a[mid] <= x) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// Device-resident working set of one batch.  Pointers are owned by the backend's arena.
struct PtxWork {
    const uint8_t* text = nullptr;
    uint32_t n_modules = 0, n_chunks = 0;
    PtxModuleLayout* layout = nullptr;     // [n_modules]
    uint32_t* mod_chunk_begin = nullptr;   // [n_modules + 1]
    uint32_t* chunk_vec = nullptr;         // [n_chunks] transition vectors, then inclusive prefix
    PtxPair* chunk_cnt = nullptr;          // [n_chunks + 1] tokens/errors per chunk, then exclusive prefix
    PtxToken* tokens = nullptr;            // [n_tokens]
    uint32_t* lexerrs = nullptr;           // [2 * n_lexerrs]
    uint32_t* mod_tok_begin = nullptr;     // [n_modules + 1]
    bool first_slice = true;               // the class store is emptied before the first slice of a batch
    uint32_t seq_max_tokens = PTX_SEQ_MAX_TOKENS;   // longest tail the sequential parser takes on
    uint16_t* kinds = nullptr;             // [n_tokens] tokens[i].kind | min(tokens[i].len, 127) << 9
    int32_t* mod_final_scope = nullptr;    // [n_modules] scope depth behind the module's last token
    uint32_t* unit_start = nullptr;        // [n_units + 1]
    uint32_t* unit_depth = nullptr;        // [n_units]  scope depth in front of the unit | module-first << 31
    uint32_t* unit_end = nullptr;          // [n_units]
    uint32_t* unit_dir = nullptr;          // [n_units]  inclusive scan of top-level flags
    PtxPair* unit_size = nullptr;          // [n_units + 1] words/errors per unit, then exclusive prefix
    uint8_t* unit_status = nullptr;        // [n_units]
    uint32_t* mod_unit_begin = nullptr;    // [n_modules + 1]
    uint32_t* mod_bad = nullptr;           // [n_modules]
    uint32_t* mod_skip = nullptr;          // [n_modules] not parsed: lex errors (checked/unchecked mode) or no tokens
    PtxPair* mod_seq_size = nullptr;       // [n_modules]
    uint32_t* mod_seq_status = nullptr;    // [n_modules]
    PtxFnEntry* fn_entries = nullptr;      // [n_funcs]
    uint32_t* fn_slots = nullptr;          // [fn_mask + 1]
    uint32_t fn_mask = 0;
    uint32_t* words = nullptr;             // [n_words]
    PtxErrRec* errs = nullptr;             // [n_errs]
    PtxModuleResult* results = nullptr;    // [n_modules]
    PtxCounters* counters = nullptr;       // device copy
};

struct ComposeOp {
    PTX_HD uint32_t operator()(uint32_t a, uint32_t b) const { return cx_compose(a, b); }
};
struct PairAddOp {
    PTX_HD PtxPair operator()(PtxPair x, PtxPair y) const { PtxPair r; r.a = x.a + y.a; r.b = x.b + y.b; return r; }
};
struct AddOp {
    PTX_HD uint32_t operator()(uint32_t a, uint32_t b) const { return a + b; }
};
// Backend concept:
//   template <class F> void pf(const char* name, size_t n, F f);                f(i) for i in [0, n)
//   template <class T, class Op, class Ld, class St> void scan(const char* name, size_t n, Ld ld, St st, Op op, T identity);
//        inclusive scan: st(i, op(ld(0), ..., ld(i)))
//   void structure(const char* name, const PtxStructArgs& a);                    stage B in one pass (ptx_struct_tile.h)
//   void fail(const char* why);                                                  the batch cannot be finished
//   void sort_by_key(const char* name, size_t n, const uint16_t* key, uint32_t* order);
//        order = a permutation of 0..n-1 that puts equal keys next to each other, either over the whole range or
//        inside consecutive segments of the backend's choice (keys < PTX_SORT_BUCKETS; order inside a group is free)
//   template <class F> void pf_staged(const char* name, size_t n, uint32_t* table, uint32_t row_words, F f);
//        PtxStaged r = f(i, scratch) for i in [0, n), scratch a PtxScratch of the backend's;
//        afterwards the backend copies the first r.n staged words to table[r.unit * row_words ...]
//   template <class F> void pf_segments(const char* name, size_t n, const PtxPair* off, F f);
//        segment s owns the items [off[s].a, off[s + 1].a): f(s, i, off[s].a + i) for every s < n and every item i of s
//   void emit_records(const char* name, size_t n_units, const PtxPair* off, const PtxEmitStep& e);   C5, see PtxEmitStep
//        the same in two rounds: an item for which f returns true is handled by g(s, i, off[s].a + i) afterwards, the
//        items put off packed together (work that few scattered items need)
//   PtxClassStore class_store(bool reset);   the batch's class store (device memory that outlives the arena), emptied if asked
//   const PtxLexTables* lex_tables();   the constant tables of ptx_lex_tile.h where the steps can read them (filled by lt_fill_tables)
//   void lex_mark(const char* name, size_t n_tiles, const PtxLexTileArgs& a);   the phases of ptx_lex_tile.h's mark step, one block per tile
//   void lex_emit(const char* name, size_t n_tiles, const PtxLexTileArgs& a);   the phases of its emit step
//   void* alloc(size_t bytes); void zero(void* p, size_t bytes);
//   void download(void* host, const void* dev, size_t bytes);   (synchronises the stream)
// The pipeline allocates through the backend and never frees: the backend's arena is reset per batch.

// ------------------------------------------------------------------------------------------------ stage A: lexer
// The three per-chunk steps are functors (not lambdas) because the backend hands them a text reader of its own type:
// plain global memory on the host, a shared-memory tile on the GPU.  Chunk c covers text[c * PTX_CHUNK, ...).
struct PtxLexChunkInfo {
    const PtxModuleLayout* layout;
    const uint32_t* mcb;
    uint32_t n_modules;
    PTX_HD void locate(size_t c, uint32_t& ms, uint32_t& me, bool& first) const {
        uint32_t m = ptx_upper_bound_u32(mcb, n_modules, (uint32_t)c) - 1;
        ms = (uint32_t)layout[m].text_off;
        me = ms + (uint32_t)layout[m].text_len;
        first = c == mcb[m];
    }
};
#include "ptx_lex_tile.h"
struct PtxLexVectorsStep {
    PtxLexChunkInfo info;
    uint32_t* vec;
    template <class R> PTX_HD void operator()(size_t c, const R& rd) const {
        uint32_t ms, me, cs = (uint32_t)c * PTX_CHUNK;
        bool first;
        info.locate(c, ms, me, first);
        uint32_t ce = cs + PTX_CHUNK < me ? cs + PTX_CHUNK : me;
        uint32_t v = cx_chunk_vector(rd, cs, ce);
        vec[c] = first ? cx_restart(v) : v;
    }
};
struct PtxLexTokensStep {
    PtxLexChunkInfo info;
    const uint8_t* text;
    const uint32_t* vec;
    PtxPair* cnt;
    PtxToken* slots;
    template <class R> PTX_HD void operator()(size_t c, const R& rd) const {
        uint32_t ms, me, cs = (uint32_t)c * PTX_CHUNK;
        bool first;
        info.locate(c, ms, me, first);
        int state = first ? CX_CODE : (int)(vec[c - 1] & 7u);
        LexSlotSink sink;
        sink.slots = slots + c * PTX_CHUNK;
        lx_chunk(rd, text, ms, me, cs, cs + PTX_CHUNK, state, sink);
        PtxPair p;
        p.a = sink.n_tokens;
        p.b = sink.n_errors;
        cnt[c + 1] = p;
        if (c == 0) { PtxPair z; z.a = z.b = 0; cnt[0] = z; }
    }
};
struct PtxLexErrorsStep {
    PtxLexChunkInfo info;
    const uint8_t* text;
    const uint32_t* vec;
    const PtxPair* cnt;
    uint32_t* lexerrs;
    const uint32_t* mod_flag;     // 1 = the module was lexed by one thread (a long run of soft bytes): so are its errors
    template <class R> PTX_HD void operator()(size_t c, const R& rd) const {
        if (cnt[c + 1].b == cnt[c].b) return;     // no error starts in this chunk
        // (a chunk re-lexes the run of soft bytes that reaches into it from the run's start: bounded by the look-back
        // of the marking step for every module that step did not flag)
        if (mod_flag[ptx_upper_bound_u32(info.mcb, info.n_modules, (uint32_t)c) - 1]) return;
        uint32_t ms, me, cs = (uint32_t)c * PTX_CHUNK;
        bool first;
        info.locate(c, ms, me, first);
        int state = first ? CX_CODE : (int)(vec[c - 1] & 7u);
        LexErrorSink sink;
        sink.errors = lexerrs + 2 * (size_t)cnt[c].b;
        lx_chunk(rd, text, ms, me, cs, cs + PTX_CHUNK, state, sink);
    }
};

template <class BK>
inline void ptx_stage_lex(BK& bk, PtxWork& w, PtxCounters& host_counters) {
    const uint8_t* text = w.text;
    const PtxModuleLayout* layout = w.layout;
    const uint32_t* mcb = w.mod_chunk_begin;
    const uint32_t n_modules = w.n_modules, n_chunks = w.n_chunks;
    uint32_t* vec = w.chunk_vec = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_chunks + 1));
    PtxPair* cnt = w.chunk_cnt = (PtxPair*)bk.alloc(sizeof(PtxPair) * (n_chunks + 2));
    w.mod_tok_begin = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 2));
    uint32_t* mod_lexerr_begin = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 2));
    PtxCounters* counters = w.counters;
    const PtxLexChunkInfo info{layout, mcb, n_modules};

    // A1: transition vector of every chunk
    bk.pf_text("lex_context_vectors", n_chunks, text, PtxLexVectorsStep{info, vec});
    // A2: inclusive scan with composition; chunk c starts in state (prefix[c-1])[CODE]
    bk.template scan<uint32_t>("scan_context", n_chunks, [=] PTX_HD(size_t i) { return vec[i]; }, [=] PTX_HD(size_t i, uint32_t v) { vec[i] = v; },
                               ComposeOp(), CX_IDENTITY);
    // A3: token boundaries, byte-parallel: one bit per text byte and the token / error count of every chunk
    const size_t n_tiles = ((size_t)n_chunks + LT_CHUNKS - 1) / LT_CHUNKS;
    uint32_t* start_bits = (uint32_t*)bk.alloc(sizeof(uint32_t) * LT_WORDS * (n_tiles + 1));
    uint32_t* mod_flag = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 1));
    bk.zero(mod_flag, sizeof(uint32_t) * (n_modules + 1));
    uint32_t* word_bits = (uint32_t*)bk.alloc(sizeof(uint32_t) * LT_WORDS * (n_tiles + 1));
    uint32_t* tile_mod = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_tiles + 1));
    bk.pf("lex_tile_modules", n_tiles, [=] PTX_HD(size_t t) { tile_mod[t] = ptx_upper_bound_u32(mcb, n_modules, (uint32_t)t * LT_CHUNKS) - 1; });
    PtxLexTileArgs la{info, text, vec, n_chunks, bk.lex_tables(), tile_mod, start_bits, word_bits, cnt, mod_flag, nullptr, nullptr};
    bk.lex_mark("lex_mark", n_tiles, la);
    // modules with a run of soft bytes too long for the look-back of the parallel step: one thread each (rare)
    bk.pf("lex_serial_modules", n_modules, [=] PTX_HD(size_t m) { lt_lex_module_serial(la, (uint32_t)m); });
    // A4: exclusive offsets (cnt[c] = tokens before chunk c; cnt[n_chunks] = total)
    bk.template scan<PtxPair>("scan_token_counts", n_chunks + 1, [=] PTX_HD(size_t i) { return cnt[i]; }, [=] PTX_HD(size_t i, PtxPair v) { cnt[i] = v; },
                              PairAddOp(), PtxPair{0, 0});
    bk.pf("set_token_total", 1, [=] PTX_HD(size_t) {
        counters->n_tokens = n_chunks ? cnt[n_chunks].a : 0;
        counters->n_lexerrs = n_chunks ? cnt[n_chunks].b : 0;
    });
    bk.download(&host_counters, counters, sizeof(PtxCounters));
    const uint32_t n_tokens = host_counters.n_tokens, n_lexerrs = host_counters.n_lexerrs;
    PtxToken* tokens = w.tokens = (PtxToken*)bk.alloc(sizeof(PtxToken) * (size_t)(n_tokens + 1));
    uint16_t* kinds = w.kinds = (uint16_t*)bk.alloc(sizeof(uint16_t) * ((size_t)n_tokens + 32));   // the kinds alone, for the passes that read nothing else
    uint32_t* lexerrs = w.lexerrs = (uint32_t*)bk.alloc(sizeof(uint32_t) * 2 * (size_t)(n_lexerrs + 1));
    // A5: one thread per token: length, kind (identifiers that spell an opcode, modifier or directive word get that
    // kind), literal code; written to the token's final place
    la.tokens = tokens;
    la.kinds = kinds;
    bk.lex_emit("lex_emit", n_tiles, la);
    // A6: lexer errors are rare: a second walk, only when there are any, and only over the chunks that have one
    if (n_lexerrs) {
        bk.pf_text("lex_emit_errors", n_chunks, text, PtxLexErrorsStep{info, text, vec, cnt, lexerrs, mod_flag});
        // the flagged modules: one thread each, one walk over the module (linear in its length whatever its runs)
        bk.pf("lex_emit_errors_serial", n_modules, [=] PTX_HD(size_t m) {
            if (!mod_flag[m]) return;
            const uint32_t c0 = mcb[m], c1 = mcb[m + 1];
            if (c0 == c1 || cnt[c1].b == cnt[c0].b) return;
            const uint32_t ms = (uint32_t)layout[m].text_off, me = ms + (uint32_t)layout[m].text_len;
            LexErrorSink sink;
            sink.errors = lexerrs + 2 * (size_t)cnt[c0].b;
            lx_chunk(PtxGlobalReader{text, me}, text, ms, me, ms, me, CX_CODE, sink);
        });
    }
    uint32_t* mtb = w.mod_tok_begin;
    bk.pf("module_token_ranges", n_modules + 1, [=] PTX_HD(size_t m) {
        uint32_t c = mcb[m];   // mod_chunk_begin[n_modules] = n_chunks
        mtb[m] = n_chunks ? cnt[c].a : 0;
        mod_lexerr_begin[m] = n_chunks ? cnt[c].b : 0;
    });
    PtxModuleResult* results = w.results;
    bk.pf("module_results_init", n_modules, [=] PTX_HD(size_t m) {
        PtxModuleResult r;
        r.tok_begin = mtb[m];
        r.tok_end = mtb[m + 1];
        r.lexerr_begin = mod_lexerr_begin[m];
        r.lexerr_end = mod_lexerr_begin[m + 1];
        r.unit_begin = r.unit_end = r.word_begin = r.word_end = r.err_begin = r.err_end = 0;
        r.sequential = r.status = r.n_errors = r.seq_tokens = 0;
        results[m] = r;
    });
}

// ------------------------------------------------------------------------------------------------ stage B: structure
PTX_HD inline bool ptx_opens_operand(uint16_t prev) {
    // a '{' after one of these starts a vector operand or an initialiser, not a scope
    return prev == T_COMMA || prev == T_EQ || prev == T_LPAREN || (prev >= T_OP_FIRST && prev < T_COUNT);
}
PTX_HD inline bool ptx_is_directive_start(uint16_t k) {
    return k == T_DOT_EXTERN || k == T_DOT_VISIBLE || k == T_MOD_weak || k == T_DOT_FUNC || k == T_DOT_ENTRY ||
           k == T_MOD_global || k == T_MOD_const || k == T_MOD_shared || k == T_DOT_FILE || k == T_DOT_SECTION;
}

// Scope delta of a token: +1 for a '{' that opens a scope, -1 for a '}' that closes one, 0 otherwise (also for the
// braces of vector operands, initialisers and .section bodies, told apart by two tokens of left context): sx_brace.
#include "ptx_struct_tile.h"

template <class BK>
inline void ptx_stage_structure(BK& bk, PtxWork& w, PtxCounters& host_counters, uint32_t mode) {
    const uint32_t n_tokens = host_counters.n_tokens, n_modules = w.n_modules;
    const uint16_t* kinds = w.kinds;
    const uint32_t* mtb = w.mod_tok_begin;
    const PtxModuleResult* results = w.results;
    int32_t* mod_final_scope = w.mod_final_scope = (int32_t*)bk.alloc(sizeof(int32_t) * (n_modules + 1));
    w.mod_unit_begin = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 2));
    PtxCounters* counters = w.counters;
    uint32_t* mod_skip = w.mod_skip = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 1));
    bk.zero(mod_final_scope, sizeof(int32_t) * (n_modules + 1));
    bk.pf("reset_skipped", 1, [=] PTX_HD(size_t) { counters->n_skipped = 0; });
    // B0: a module with a lex error is not parsed unless only its errors
    // are wanted (lib.rs:392-411 vs 447-449, 487-489)
    bk.pf("mark_module_skip", n_modules, [=] PTX_HD(size_t m) {
        bool lexerr = results[m].lexerr_end > results[m].lexerr_begin;
        mod_skip[m] = (mtb[m] == mtb[m + 1] || (lexerr && mode != 2)) ? 1u : 0u;
        if (mtb[m] != mtb[m + 1] && lexerr && mode != 2) {
#ifdef __CUDA_ARCH__
            atomicAdd(&counters->n_skipped, 1u);
#else
            counters->n_skipped++;
#endif
        }
    });
    // B1: one pass over the token kinds: (scope, paren) depth restarting at every module, the unit starts, their
    // numbering and the unit table (at most one unit per token); nothing per token is kept of it
    uint32_t* ustart = w.unit_start = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_tokens + 2));
    uint32_t* udepth = w.unit_depth = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_tokens + 2));
    uint32_t* mub = w.mod_unit_begin;
    bk.pf("reset_unit_total", 1, [=] PTX_HD(size_t) { counters->n_units = 0; counters->struct_abort = 0; });
    bk.structure("structure", PtxStructArgs{kinds, n_tokens, mtb, n_modules, mod_final_scope, ustart, udepth, mub, counters});
    bk.download(&host_counters, counters, sizeof(PtxCounters));
    if (host_counters.struct_abort) {
        bk.fail("the structure pass gave up waiting for an earlier tile");
        host_counters.n_units = 0;
    }
    const uint32_t n_units = host_counters.n_units;
    // modules without tokens begin where the next module with tokens begins; mub[n_modules] = n_units
    bk.pf("module_unit_ranges", n_modules + 1, [=] PTX_HD(size_t m) {
        if (m < n_modules && mtb[m] < mtb[m + 1]) return;      // written by the scan
        size_t k = m;
        while (k < n_modules && mtb[k] == mtb[k + 1]) k++;
        mub[m] = k < n_modules ? (0x80000000u | (uint32_t)k) : n_units;   // a reference to module k is resolved below
    });
    bk.pf("module_unit_ranges_fill", n_modules + 1, [=] PTX_HD(size_t m) {
        uint32_t v = mub[m];
        if (v & 0x80000000u) mub[m] = mub[v & 0x7FFFFFFFu];
    });
}

// C5 as a step object: one output word at a time.  unit() is what a word needs of its unit (loaded once per unit by
// the backend); word() only reads and says what to do with the word, so that a backend can have several words in flight
// per thread; literal() is the second round (one literal per call, written in place).
struct PtxEmitUnit {
    uint32_t tmpl, start, flag;
};
struct PtxEmitStep {
    const uint8_t* uflag;
    const uint32_t* utmpl;
    const uint32_t* ustart;
    const uint32_t* table;
    PtxClassStore cs;
    const PtxToken* tokens;
    const uint8_t* text;
    uint32_t* words;
    enum { NOTHING = 0, WRITE = 1, SECOND_ROUND = 2 };
    PTX_HD PtxEmitUnit unit(size_t u) const {
        PtxEmitUnit e;
        e.flag = uflag[u];
        e.tmpl = e.flag == PTX_UNIT_TEMPLATED ? utmpl[u] : 0u;
        e.start = ustart[u];
        return e;
    }
    PTX_HD int word(const PtxEmitUnit& e, size_t u, uint32_t i, uint32_t& x) const {
        if (e.flag == PTX_UNIT_STAGED) {
            x = table[u * PTX_TMP_STRIDE + i];
            return WRITE;
        }
        if (e.flag != PTX_UNIT_TEMPLATED) return NOTHING;
        const size_t at = (size_t)e.tmpl * PTX_TMPL_WORDS + i;
        x = cs.tmpl_words[at];
        const uint32_t g = cs.tmpl_tags[at];
        if (g) {
            const uint32_t type = g >> 8;
            if (type >= PTX_TAG_VAL_LO) {
                if (!(type & 1u)) return SECOND_ROUND;      // low word
                // high word: written by the low-word thread in front of it, unless it stands alone
                if (i > 0 && cs.tmpl_tags[at - 1] == (uint16_t)(g - 0x100u)) return NOTHING;
                return SECOND_ROUND;
            }
            const PtxToken t = tokens[e.start + (g & 0xFFu)];
            x = type == PTX_TAG_START ? t.start : type == PTX_TAG_LEN ? (uint32_t)t.len : ((x & 0xFFu) | ((uint32_t)t.len << 8));
        }
        return WRITE;
    }
    // Literal values, one thread per literal with the warps full: the low-word thread also writes the high word when
    // the template has it next (the two value words of an immediate)
    PTX_HD void literal(const PtxEmitUnit& e, uint32_t i, uint32_t j) const {
        const size_t at = (size_t)e.tmpl * PTX_TMPL_WORDS + i;
        const uint32_t g = cs.tmpl_tags[at], type = g >> 8;
        const PtxToken t = tokens[e.start + (g & 0xFFu)];
        uint64_t v = ptx_literal_value(text, t.start, t.len, t.kind);
        if (type >= PTX_TAG_NEG_LO) v = 0 - v;
        if (type & 1u) { words[j] = (uint32_t)(v >> 32); return; }
        words[j] = (uint32_t)v;
        if (i + 1 < cs.info[e.tmpl].n_words && cs.tmpl_tags[at + 1] == (uint16_t)(g + 0x100u)) words[j + 1] = (uint32_t)(v >> 32);
    }
};

// ------------------------------------------------------------------------------------------------ stage C: decode
template <class BK>
inline void ptx_stage_decode(BK& bk, PtxWork& w, PtxCounters& host_counters) {
    const uint32_t n_tokens = host_counters.n_tokens, n_units = host_counters.n_units, n_modules = w.n_modules;
    const uint8_t* text = w.text;
    const PtxToken* tokens = w.tokens;
    const uint16_t* kinds = w.kinds;
    const PtxModuleLayout* layout = w.layout;
    const uint32_t* mtb = w.mod_tok_begin;
    const uint32_t* mub = w.mod_unit_begin;
    const uint32_t* ustart = w.unit_start;
    const uint32_t* udepth = w.unit_depth;
    const int32_t* mod_final_scope = w.mod_final_scope;
    const uint32_t* mod_skip = w.mod_skip;
    PtxModuleResult* results = w.results;
    PtxCounters* counters = w.counters;
    const uint32_t seq_max_tokens = w.seq_max_tokens;
    uint32_t* uend = w.unit_end = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_units + 1));
    uint32_t* udir = w.unit_dir = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_units + 1));
    PtxPair* usize = w.unit_size = (PtxPair*)bk.alloc(sizeof(PtxPair) * ((size_t)n_units + 2));
    uint8_t* ustatus = w.unit_status = (uint8_t*)bk.alloc((size_t)n_units + 16);
    uint32_t* mod_bad = w.mod_bad = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 1));
    PtxPair* mod_seq = w.mod_seq_size = (PtxPair*)bk.alloc(sizeof(PtxPair) * (n_modules + 1));
    uint32_t* mod_seq_status = w.mod_seq_status = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 1));
    // worst case one function per top-level unit; sized after the top-level scan below
    bk.zero(mod_bad, sizeof(uint32_t) * (n_modules + 1));
    bk.zero(mod_seq, sizeof(PtxPair) * (n_modules + 1));
    bk.zero(mod_seq_status, sizeof(uint32_t) * (n_modules + 1));

    // C0: ordinal of the enclosing top-level unit
    bk.template scan<uint32_t>("scan_toplevel_ordinal", n_units, [=] PTX_HD(size_t u) { return (udepth[u] & 0x7FFFFFFFu) == 0 ? 1u : 0u; },
                               [=] PTX_HD(size_t u, uint32_t v) { udir[u] = v; }, AddOp(), 0u);
    // ... and the unit that heads each top-level ordinal (a module's first unit, or a top-level directive's first)
    uint32_t* top_unit = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_units + 1));
    bk.pf("list_toplevel_units", n_units, [=] PTX_HD(size_t u) {
        if ((udepth[u] & 0x7FFFFFFFu) == 0) top_unit[udir[u] - 1] = (uint32_t)u;
    });
    // Very long top-level statements (arrays with huge initialisers) are listed for the bulk path
    PtxBulkInfo* bulk_info = (PtxBulkInfo*)bk.alloc(sizeof(PtxBulkInfo) * PTX_MAX_BULK);
    bk.pf("reset_bulk", 1, [=] PTX_HD(size_t) { counters->n_bulk = 0; });
    bk.pf("find_bulk_units", n_units, [=] PTX_HD(size_t u) {
        uint32_t dp = udepth[u];
        if (dp != 0) return;       // top level, not the module header
        uint32_t m = ptx_upper_bound_u32(mub, n_modules, (uint32_t)u) - 1;
        if (mod_skip[m]) return;
        uint32_t start = ustart[u];
        uint32_t end = (u + 1 < mub[m + 1]) ? ustart[u + 1] : mtb[m + 1];
        if (end - start < PTX_BULK_MIN_TOKENS) return;
#ifdef __CUDA_ARCH__
        uint32_t slot = atomicAdd(&counters->n_bulk, 1u);
#else
        uint32_t slot = counters->n_bulk++;
#endif
        if (slot >= PTX_MAX_BULK) return;
        PtxBulkInfo bi;
        bi.first_tok = start;      // for now: the statement's token range
        bi.close_tok = end;
        bi.n_elems = bi.n_words = 0;
        bi.bad = 1;
        bi.unit = (uint32_t)u;
        bi.elems = nullptr;
        bi.dst = nullptr;
        bulk_info[slot] = bi;
    });
    // T0: class key of every unit (see "unit classes and record templates" above)
    uint16_t* ukey = (uint16_t*)bk.alloc(sizeof(uint16_t) * ((size_t)n_units + 2));
    uint32_t* order = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_units + 1));
    uint64_t* ckey_of = (uint64_t*)bk.alloc(sizeof(uint64_t) * ((size_t)n_units + 1));
    bk.pf("unit_class_key", n_units, [=] PTX_HD(size_t u) {
        // units lie back to back over the whole batch: a unit ends where the next one starts.  The unit's module is looked
        // up only when some module of the slice is not parsed at all (a lexer error outside the errors-only mode)
        uint32_t start = ustart[u];
        uint32_t end = u + 1 < n_units ? ustart[u + 1] : n_tokens;
        uint32_t dp = udepth[u];
        const bool skipped = counters->n_skipped != 0 && mod_skip[ptx_upper_bound_u32(mub, n_modules, (uint32_t)u) - 1] != 0;
        ckey_of[u] = skipped ? 0 : ptx_class_key(text, tokens, kinds, start, end, dp & 0x7FFFFFFFu, (dp >> 31) != 0);
    });

    // T1: class table (open addressing on the 64-bit key), shared by the slices of a batch; the thread that inserts
    // a key makes its unit the representative of the class
    const PtxClassStore cs = bk.class_store(w.first_slice);
    uint32_t* uclass = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_units + 1));
    uint32_t* utmpl = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_units + 1));
    uint8_t* uflag = (uint8_t*)bk.alloc((size_t)n_units + 16);
    bk.pf("reset_flagged", 1, [=] PTX_HD(size_t) {
        counters->n_flagged = 0;
        cs.state[2] = cs.state[0] < PTX_MAX_CLASSES ? cs.state[0] : PTX_MAX_CLASSES;
    });
    bk.pf("class_insert", n_units, [=] PTX_HD(size_t u) {
        uclass[u] = PTX_ABSENT;
        unsigned long long key = ckey_of[u];
        if (!key) return;
        uint32_t h = (uint32_t)(key ^ (key >> 29)) & (PTX_CLASS_SLOTS - 1);
        for (int probe = 0; probe < 64; probe++) {
#ifdef __CUDA_ARCH__
            // most units find their class already there: look before competing for the slot, and look through the
            // SM's own cache first (a batch has few classes: every SM asking L2 for the same few lines is what this
            // step otherwise waits for; a stale empty slot only sends the thread on to the exact look)
            unsigned long long old = __ldca(&cs.keys[h]);
            if (old != key) old = *(volatile unsigned long long*)&cs.keys[h];
            if (old == 0) old = atomicCAS(&cs.keys[h], 0ull, key);
#else
            unsigned long long old = cs.keys[h];
            if (old == 0) cs.keys[h] = key;
#endif
            if (old == 0) {
#ifdef __CUDA_ARCH__
                uint32_t id = atomicAdd(&cs.state[0], 1u);
#else
                uint32_t id = cs.state[0]++;
#endif
                if (id < PTX_MAX_CLASSES) {
                    cs.rep_unit[id] = (uint32_t)u;
                    cs.slot_tmpl[h] = id;
                } else {
                    cs.slot_tmpl[h] = PTX_ABSENT;
                }
                uclass[u] = h;
                return;
            }
            if (old == key) { uclass[u] = h; return; }
            h = (h + 1) & (PTX_CLASS_SLOTS - 1);
        }
    });
    // T2: decode the representatives of the classes this slice added, with tagged output, and spell out their signature
    // (thread i takes new class (i / 32) + (i % 32) * (PTX_MAX_CLASSES / 32): the first 8,192 new classes go to lane 0 of
    // a warp each.  Representatives are statements of different shapes; 32 of them in one warp ran one after the other.)
    bk.pf("decode_representatives", PTX_MAX_CLASSES, [=] PTX_HD(size_t i) {
        const size_t k = (i >> 5) + (i & 31u) * (PTX_MAX_CLASSES / 32u);
        size_t id = (size_t)cs.state[2] + k;
        if (id >= cs.state[0] || id >= PTX_MAX_CLASSES) return;
        uint32_t u = cs.rep_unit[id];
        uint32_t m = ptx_upper_bound_u32(mub, n_modules, u) - 1;
        uint32_t start = ustart[u];
        uint32_t end = (u + 1 < mub[m + 1]) ? ustart[u + 1] : mtb[m + 1];
        PtxSink sink;
        sink.words = cs.tmpl_words + id * PTX_TMPL_WORDS;
        sink.tags = cs.tmpl_tags + id * PTX_TMPL_WORDS;
        sink.words_cap = PTX_TMPL_WORDS;
        PtxResolver res;
        res.module = m;
        PtxDecoder d(text, tokens, mtb[m + 1], layout[m].text_off + layout[m].text_len, sink, res);
        uint32_t dp = udepth[u];
        PtxUnitResult r = ptx_decode_unit(d, start, dp & 0x7FFFFFFFu, (dp >> 31) != 0);
        PtxTemplateInfo ti;
        ti.n_words = sink.nw;
        ti.n_tokens = end - start;
        ti.depth1 = (dp & 0x7FFFFFFFu) == 1 ? 1u : 0u;
        ti.ok = (r.status == US_OK && sink.ne == 0 && sink.peak <= PTX_TMPL_WORDS && !sink.poison && r.kind != U_FUNC && r.end == end &&
                 d.max_seen < end) ? 1u : 0u;
        if (ti.ok) {
            uint32_t need = ptx_signature_words(tokens, start, ti.n_tokens);
#ifdef __CUDA_ARCH__
            uint32_t at = atomicAdd(&cs.state[1], need);
#else
            uint32_t at = cs.state[1];
            cs.state[1] += need;
#endif
            if (at + need <= PTX_SIG_POOL_WORDS) {
                cs.sig_off[id] = at;
                ptx_signature_write(cs.sig_pool + at, text, tokens, kinds, start, ti.n_tokens, ti.depth1);
            } else {
                ti.ok = 0;
            }
        }
        cs.info[id] = ti;
    });
    // T3: every unit of a class with a usable template is checked against the class signature and takes its size
    uint32_t* rest_count = (uint32_t*)bk.alloc(sizeof(uint32_t) * 64);     // striped count of the units left without a template
    bk.zero(rest_count, sizeof(uint32_t) * 64);
    bk.pf("apply_templates", n_units, [=] PTX_HD(size_t u) {
        uflag[u] = PTX_UNIT_UNDECIDED;
        utmpl[u] = PTX_ABSENT;
        auto rest = [&]() {      // this unit stays without a template
#ifdef __CUDA_ARCH__
            atomicAdd(&rest_count[u & 63], 1u);
#else
            rest_count[u & 63]++;
#endif
        };
        uint32_t slot = uclass[u];
        if (slot == PTX_ABSENT) { rest(); return; }
        uint32_t id = cs.slot_tmpl[slot];
        if (id == PTX_ABSENT) { rest(); return; }
        const PtxTemplateInfo ti = cs.info[id];
        if (!ti.ok) { rest(); return; }
        uint32_t start = ustart[u];
        uint32_t end = u + 1 < n_units ? ustart[u + 1] : n_tokens;
        uint32_t dp = udepth[u];
        uint32_t depth1 = (dp & 0x7FFFFFFFu) == 1 ? 1u : 0u;
        if (end - start != ti.n_tokens || !ptx_signature_matches(cs.sig_pool + cs.sig_off[id], text, tokens, kinds, start, ti.n_tokens, depth1)) { rest(); return; }
        PtxPair sz;
        sz.a = ti.n_words;
        sz.b = 0;
        usize[u + 1] = sz;
        if (u == 0) { PtxPair z; z.a = z.b = 0; usize[0] = z; }
        uend[u] = end;
        ustatus[u] = US_OK;
        uflag[u] = PTX_UNIT_TEMPLATED;
        utmpl[u] = id;
    });

    bk.pf("reset_func_count", 1, [=] PTX_HD(size_t) {
        counters->n_funcs = 0;
        counters->any_sequential = 0;
        counters->pad = n_units ? udir[n_units - 1] : 0;   // number of top-level units: bound for the function table
        uint32_t rest = 0;
        for (int i = 0; i < 64; i++) rest += rest_count[i];
        counters->n_rest = rest;
        counters->n_classes = cs.state[0];
        counters->n_sig_words = cs.state[1];
    });
    bk.download(&host_counters, counters, sizeof(PtxCounters));
    const uint32_t max_funcs = host_counters.pad;
    bk.pf("reset_mismatch", 1, [=] PTX_HD(size_t) { counters->pad = 0; });
    // Bulk path: the elements of each listed statement's initialiser are decoded one thread per element into a dense
    // run; the statement's own decoder later takes the run in one step (PtxDecoder::multi_variable).  A list that is
    // not plainly "element, element, ... }" followed by ';' stays marked bad and is decoded the ordinary way.
    const uint32_t n_bulk = host_counters.n_bulk < PTX_MAX_BULK ? host_counters.n_bulk : PTX_MAX_BULK;
    PtxBulkTable bulk_table;
    bulk_table.info = bulk_info;
    bulk_table.n = n_bulk;
    uint32_t bulk_tokens[PTX_MAX_BULK];     // tokens of each listed statement
    if (n_bulk) {
        PtxBulkInfo host_bulk[PTX_MAX_BULK];
        bk.download(host_bulk, bulk_info, sizeof(PtxBulkInfo) * n_bulk);
        for (uint32_t j = 0; j < n_bulk; j++) {
            const uint32_t ts = host_bulk[j].first_tok, te = host_bulk[j].close_tok, nt = te - ts;
            bulk_tokens[j] = nt;
            PtxBulkInfo* bi = bulk_info + j;
            uint32_t* lo_dev = (uint32_t*)bk.alloc(sizeof(uint32_t) * 4);
            PtxPair* esz = (PtxPair*)bk.alloc(sizeof(PtxPair) * ((size_t)nt + 2));
            uint32_t* elems = (uint32_t*)bk.alloc(sizeof(uint32_t) * (2 * (size_t)nt + 8));
            bk.pf("bulk_reset", 1, [=] PTX_HD(size_t) { lo_dev[0] = PTX_ABSENT; lo_dev[1] = 0; });
            bk.pf("bulk_find_open", nt, [=] PTX_HD(size_t k) {
                uint32_t i = ts + (uint32_t)k;
                if (i > ts && PTX_KL_KIND(kinds[i]) == T_LBRACE && PTX_KL_KIND(kinds[i - 1]) == T_EQ) {
#ifdef __CUDA_ARCH__
                    atomicMin(&lo_dev[0], i);
#else
                    if (i < lo_dev[0]) lo_dev[0] = i;
#endif
                }
            });
            bk.pf("bulk_measure", nt, [=] PTX_HD(size_t k) {
                uint32_t i = ts + (uint32_t)k;
                PtxPair z;
                z.a = z.b = 0;
                esz[k] = z;
                const uint32_t lo = lo_dev[0], hi = te - 2;
                bool shape_ok = lo != PTX_ABSENT && nt >= 6 && lo + 1 < hi && PTX_KL_KIND(kinds[te - 2]) == T_RBRACE &&
                                PTX_KL_KIND(kinds[te - 1]) == T_SEMI && PTX_KL_KIND(kinds[hi - 1]) != T_COMMA;
                if (!shape_ok) { if (k == 0) lo_dev[1] = 1; return; }
                if (i <= lo || i >= hi) return;
                uint16_t kd = PTX_KL_KIND(kinds[i]);
                if (kd == T_LBRACE || kd == T_RBRACE) { lo_dev[1] = 1; return; }
                if (!(i == lo + 1 || PTX_KL_KIND(kinds[i - 1]) == T_COMMA)) return;
                // an element starts here: measure it
                uint32_t mm = ptx_upper_bound_u32(mtb, n_modules, i) - 1;
                PtxSink sink;
                PtxResolver res;
                PtxDecoder d(text, tokens, mtb[mm + 1], layout[mm].text_off + layout[mm].text_len, sink, res);
                d.pos = i;
                d.unit_tok0 = i;
                bool ok = d.reg_or_immediate(true) && sink.ne == 0 && d.pos <= hi;
                if (ok) {
                    uint16_t nk = PTX_KL_KIND(kinds[d.pos]);
                    ok = (d.pos == hi) || nk == T_COMMA;
                }
                if (!ok) { lo_dev[1] = 1; return; }
                z.a = sink.nw;
                z.b = 1;
                esz[k] = z;
            });
            bk.template scan<PtxPair>("bulk_scan", (size_t)nt, [=] PTX_HD(size_t k) { return esz[k]; }, [=] PTX_HD(size_t k, PtxPair v) {
                                          PtxPair own = esz[k];
                                          if (k + 1 == nt) {     // totals, before the entry turns exclusive
                                              bi->n_words = v.a;
                                              bi->n_elems = v.b;
                                          }
                                          PtxPair ex;
                                          ex.a = v.a - own.a;
                                          ex.b = own.b;      // keeps "an element starts here"
                                          esz[k] = ex;
                                      },
                                      PairAddOp(), PtxPair{0, 0});
            bk.pf("bulk_decode", nt, [=] PTX_HD(size_t k) {
                if (lo_dev[1] || !esz[k].b) return;
                uint32_t i = ts + (uint32_t)k;
                uint32_t mm = ptx_upper_bound_u32(mtb, n_modules, i) - 1;
                PtxSink sink;
                sink.words = elems + esz[k].a;
                PtxResolver res;
                PtxDecoder d(text, tokens, mtb[mm + 1], layout[mm].text_off + layout[mm].text_len, sink, res);
                d.pos = i;
                d.unit_tok0 = i;
                d.reg_or_immediate(true);
            });
            bk.pf("bulk_publish", 1, [=] PTX_HD(size_t) {
                bi->first_tok = lo_dev[0] + 1;
                bi->close_tok = te - 2;
                bi->bad = lo_dev[1];
                bi->elems = elems;
                bi->dst = nullptr;
            });
        }
    }
    PtxFnEntry* fn_entries = w.fn_entries = (PtxFnEntry*)bk.alloc(sizeof(PtxFnEntry) * ((size_t)max_funcs + 1));

    // The units without a template are decoded next.  When they are few (clean input: calls, function headers,
    // statements whose class was poisoned) they are simply listed; when they are many they are sorted by a "shape key"
    // (a hash of their token kinds) first: the decoder's control flow depends on token kinds only, so the threads of a
    // warp then follow the same path.  Results are written at offsets computed in unit order either way, so the order
    // of processing does not show in the output.  order[0 .. n_rest) = the units to decode.
    const uint32_t n_rest = host_counters.n_rest;
    if (n_rest <= 131072) {
        bk.pf("list_rest_units", n_units, [=] PTX_HD(size_t u) {
            if (uflag[u] == PTX_UNIT_TEMPLATED) return;
#ifdef __CUDA_ARCH__
            uint32_t slot = atomicAdd(&counters->n_listed, 1u);
#else
            uint32_t slot = counters->n_listed++;
#endif
            order[slot] = (uint32_t)u;
        });
    } else {
        // templated units share the last bucket, so they sort behind all the others
        bk.pf("unit_shape_key", n_units, [=] PTX_HD(size_t u) {
            if (uflag[u] == PTX_UNIT_TEMPLATED) { ukey[u] = (uint16_t)(PTX_SORT_BUCKETS - 1); return; }
            uint32_t m = ptx_upper_bound_u32(mub, n_modules, (uint32_t)u) - 1;
            uint32_t start = ustart[u];
            uint32_t end = (u + 1 < mub[m + 1]) ? ustart[u + 1] : mtb[m + 1];
            if (end > start + 20) end = start + 20;
            uint32_t h = 2166136261u ^ (udepth[u] >> 31) ^ ((udepth[u] & 0x7FFFFFFFu) ? 2u : 0u);
            for (uint32_t i = start; i < end; i++) h = (h ^ PTX_KL_KIND(kinds[i])) * 16777619u;
            h ^= h >> 15;
            h &= PTX_SORT_BUCKETS - 1;
            if (h == PTX_SORT_BUCKETS - 1) h = 0;
            ukey[u] = (uint16_t)h;
        });
        bk.sort_by_key("sort_units_by_shape", n_units, ukey, order);
    }

    // C1: decode every unit once.  The record is built in a small per-thread staging buffer (failed alternatives are
    // rolled back there) and lands in row u of a table; its final place is known only after the sizes are scanned.
    // Units that report errors (every `call` reserves one), or whose record outgrows the buffer, are only measured
    // here and written by the second pass (C6), which also has the function table.
    uint32_t* table = (uint32_t*)bk.alloc(sizeof(uint32_t) * PTX_TMP_STRIDE * ((size_t)n_units + 1));
    bk.pf_staged("decode_units", n_rest, table, PTX_TMP_STRIDE, [=] PTX_HD(size_t idx, const PtxScratch& sc) -> PtxStaged {
        PtxStaged ret;
        size_t u = order[idx];
        ret.unit = (uint32_t)u;
        ret.n = 0;
        if (uflag[u] == PTX_UNIT_TEMPLATED) return ret;
        uint32_t start = ustart[u];
        uint32_t m = ptx_upper_bound_u32(mub, n_modules, (uint32_t)u) - 1;
        // modules without units share their begin with the next one: take the last module that starts at or before u
        if (u == 0) { PtxPair z; z.a = z.b = 0; usize[0] = z; }
        if (mod_skip[m]) {
            PtxPair z;
            z.a = z.b = 0;
            usize[u + 1] = z;
            uend[u] = 0;
            ustatus[u] = US_OK;
            uflag[u] = 0;
            return ret;
        }
        PtxSink sink;
        sink.stage = sc.stage;
        sink.stage_stride = sc.stage_stride;
        sink.stage_cap = sc.stage_cap < PTX_TMP_STRIDE ? sc.stage_cap : PTX_TMP_STRIDE;
        PtxResolver res;
        res.module = m;
        PtxDecoder d(text, tokens, mtb[m + 1], layout[m].text_off + layout[m].text_len, sink, res);
        d.bulk = bulk_table;
        // the unit's first tokens go to the fast window: the decoder looks at every token many times
        {
            uint32_t avail = mtb[m + 1] - start;
            uint32_t nwin = avail < sc.win_cap ? avail : sc.win_cap;
            const PtxTokenWord* src = (const PtxTokenWord*)(tokens + start);
            for (uint32_t k = 0; k < sc.win_cap; k++)
                if (k < nwin) sc.win[k * sc.win_stride] = src[k];
            d.win = sc.win;
            d.win_base = start;
            d.win_n = nwin;
            d.win_stride = sc.win_stride;
        }
        uint32_t dp = udepth[u];
        PtxUnitResult r = ptx_decode_unit(d, start, dp & 0x7FFFFFFFu, (dp >> 31) != 0);
        uend[u] = r.end;
        ustatus[u] = (uint8_t)r.status;
        bool flagged = sink.peak > sink.stage_cap || sink.ne > 0;
        PtxPair sz;
        sz.a = flagged ? sink.peak : sink.nw;
        sz.b = sink.ne;
        usize[u + 1] = sz;
        uflag[u] = flagged ? 1 : 0;
        if (flagged) {
#ifdef __CUDA_ARCH__
            atomicAdd(&counters->n_flagged, 1u);
#else
            counters->n_flagged++;
#endif
        } else {
            ret.n = sink.nw;
        }
        if (r.status == US_OK && r.kind == U_FUNC) {
#ifdef __CUDA_ARCH__
            uint32_t slot = atomicAdd(&counters->n_funcs, 1u);
#else
            uint32_t slot = counters->n_funcs++;
#endif
            PtxFnEntry e;
            e.unit = (uint32_t)u;
            e.dir_ord = udir[u];
            e.name_off = tokens[r.name_tok].start;
            e.name_len = ptx_token_len(text, tokens[r.name_tok], layout[m].text_off + layout[m].text_len);
            e.n_rets = r.n_rets;
            e.n_inputs = r.n_inputs;
            e.module = m;
            e.pad = 0;
            fn_entries[slot] = e;
        }
        return ret;
    });
    // C2: do consecutive units meet, and does every module return to depth 0?  Where they do not, everything from
    // the top-level directive that holds the first such place to the end of the module is parsed again by one thread
    // with the reference's recovery rules; the directives in front of it keep their units.  (A module that does not
    // return to depth 0 went wrong in or behind its last top-level unit: nothing behind an unclosed scope is one.)
    // mod_bad[m] = 1 + the unit that heads the first bad directive, 0 = none
    bk.pf("chain_check", n_units, [=] PTX_HD(size_t u) {
        // units lie back to back over the whole batch, and a module's first unit says so in its depth word: the common
        // case (the unit meets the next one, which is in the same module) needs no module look-up
        const bool last_of_module = u + 1 == n_units || (udepth[u + 1] >> 31) != 0;
        const uint32_t next_start = u + 1 < n_units ? ustart[u + 1] : n_tokens;
        if (!last_of_module && ustatus[u] == US_OK && uend[u] == next_start) return;
        uint32_t m = ptx_upper_bound_u32(mub, n_modules, (uint32_t)u) - 1;
        if (mod_skip[m]) return;
        uint32_t next = (u + 1 < mub[m + 1]) ? ustart[u + 1] : mtb[m + 1];
        bool ok = ustatus[u] == US_OK && uend[u] == next;
        if (u + 1 == mub[m + 1]) ok = ok && mod_final_scope[m] == 0;
        if (ok) return;
        const uint32_t head = top_unit[udir[u] - 1];
#ifdef __CUDA_ARCH__
        atomicMax(&mod_bad[m], 0xFFFFFFFFu - head);       // the smallest head wins
#else
        if (0xFFFFFFFFu - head > mod_bad[m]) mod_bad[m] = 0xFFFFFFFFu - head;
#endif
    });
    bk.pf("first_bad_directive", n_modules, [=] PTX_HD(size_t m) {
        if (mod_bad[m]) mod_bad[m] = (0xFFFFFFFFu - mod_bad[m]) + 1u;
    });
    // C3: the sequential parse, one thread per such module (count)
    bk.pf("sequential_count", n_modules, [=] PTX_HD(size_t m) {
        if (!mod_bad[m]) return;
        counters->any_sequential = 1;
        const uint32_t head = mod_bad[m] - 1u;
        if (mtb[m + 1] - ustart[head] > seq_max_tokens) {
            mod_seq_status[m] = US_REFUSED;       // sizes stay 0: the module's verdict says so, nothing is parsed
            return;
        }
        PtxSink sink;
        PtxResolver res;
        PtxDecoder d(text, tokens, mtb[m + 1], layout[m].text_off + layout[m].text_len, sink, res);
        d.bulk = bulk_table;
        int st = ptx_decode_module_sequential(d, ustart[head], 0, head != mub[m]);
        PtxPair sz;
        sz.a = sink.peak;
        sz.b = sink.ne;
        mod_seq[m] = sz;
        mod_seq_status[m] = (uint32_t)st;
    });
    // C4: its sizes replace those of the units it covers
    bk.pf("merge_sequential_sizes", n_units, [=] PTX_HD(size_t u) {
        if (!counters->any_sequential) return;       // no module of this slice needs the sequential parser
        uint32_t m = ptx_upper_bound_u32(mub, n_modules, (uint32_t)u) - 1;
        if (!mod_bad[m] || u < mod_bad[m] - 1u) return;
        PtxPair z;
        z.a = z.b = 0;
        const bool head = u == mod_bad[m] - 1u;
        usize[u + 1] = head ? mod_seq[m] : z;
        uflag[u] = head ? 1 : 2;    // the head unit stands for the whole tail in C6; the others write nothing
    });
    bk.template scan<PtxPair>("scan_unit_sizes", (size_t)n_units + 1, [=] PTX_HD(size_t i) { return usize[i]; },
                              [=] PTX_HD(size_t i, PtxPair v) { usize[i] = v; }, PairAddOp(), PtxPair{0, 0});
    bk.pf("set_output_totals", 1, [=] PTX_HD(size_t) {
        counters->n_words = n_units ? usize[n_units].a : 0;
        counters->n_errs = n_units ? usize[n_units].b : 0;
        if (counters->any_sequential) counters->n_flagged += 1;
    });
    bk.download(&host_counters, counters, sizeof(PtxCounters));
    const uint32_t n_words = host_counters.n_words, n_errs = host_counters.n_errs, n_funcs = host_counters.n_funcs;
    uint32_t* words = w.words = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n_words + 4));
    PtxErrRec* errs = w.errs = (PtxErrRec*)bk.alloc(sizeof(PtxErrRec) * ((size_t)n_errs + 1));
    // C5: records of the units that were staged go to their final place
    // one thread per output word (the backend maps words to units): staged records come from their table row,
    // templated ones are instantiated from the class template and the unit's own tokens
    // Literal values are converted in a second round, one thread per literal with the warps full: the low-word thread
    // also writes the high word when the template has it next (the two value words of an immediate)
    bk.emit_records("emit_records", n_units, usize, PtxEmitStep{uflag, utmpl, ustart, table, cs, tokens, text, words});
    if (host_counters.n_flagged) {
        // function table for `call`
        uint32_t mask = 1;
        while (mask < 2 * n_funcs + 2) mask <<= 1;
        mask -= 1;
        uint32_t* slots = w.fn_slots = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)mask + 1));
        w.fn_mask = mask;
        bk.pf("fn_table_clear", (size_t)mask + 1, [=] PTX_HD(size_t i) { slots[i] = PTX_ABSENT; });
        bk.pf("fn_table_insert", n_funcs, [=] PTX_HD(size_t i) {
            const PtxFnEntry e = fn_entries[i];
            uint32_t h = ptx_name_hash(text, e.name_off, e.name_len, e.module) & mask;
            for (;;) {
#ifdef __CUDA_ARCH__
                uint32_t old = atomicCAS(&slots[h], PTX_ABSENT, (uint32_t)i);
#else
                uint32_t old = slots[h];
                if (old == PTX_ABSENT) slots[h] = (uint32_t)i;
#endif
                if (old == PTX_ABSENT) break;
                h = (h + 1) & mask;
            }
        });
        // C6: decode the flagged units again, writing in place
    bk.pf("decode_emit_flagged", n_rest, [=] PTX_HD(size_t idx) {
        size_t u = order[idx];
        if (uflag[u] != 1) return;
        uint32_t m = ptx_upper_bound_u32(mub, n_modules, (uint32_t)u) - 1;
        PtxSink sink;
        sink.words = words + usize[u].a;
        sink.errs = errs + usize[u].b;
        uint64_t text_end = layout[m].text_off + layout[m].text_len;
        if (mod_skip[m]) return;
        if (mod_bad[m] && u >= mod_bad[m] - 1u) {
            if (u != mod_bad[m] - 1u || (mod_seq_status[m] & US_MASK) == US_REFUSED) return;
            // functions declared in the tail are found through the records written so far, those in front of it
            // through the table of the speculated function headers
            PtxResolver res;
            res.words = words;
            res.entries = fn_entries;
            res.slots = slots;
            res.mask = mask;
            res.unit_off = usize;
            res.module = m;
            res.my_dir_ord = udir[u];
            PtxDecoder d(text, tokens, mtb[m + 1], text_end, sink, res);
            d.bulk = bulk_table;
            ptx_decode_module_sequential(d, ustart[u], usize[u].a, u != mub[m]);
            if (sink.peak != usize[u + 1].a - usize[u].a || sink.ne != usize[u + 1].b - usize[u].b) counters->pad = (uint32_t)u + 1;
            sink.pad_to(usize[u + 1].a - usize[u].a);
            return;
        }
        PtxResolver res;
        res.entries = fn_entries;
        res.slots = slots;
        res.mask = mask;
        res.unit_off = usize;
        res.module = m;
        res.my_dir_ord = udir[u];
        PtxDecoder d(text, tokens, mtb[m + 1], text_end, sink, res);
        d.bulk = bulk_table;
        uint32_t dp = udepth[u];
        ptx_decode_unit(d, ustart[u], dp & 0x7FFFFFFFu, (dp >> 31) != 0);
        // both passes must agree on the size of every record (a mismatch would overwrite a neighbour's record)
        if (sink.peak != usize[u + 1].a - usize[u].a || sink.ne != usize[u + 1].b - usize[u].b) counters->pad = (uint32_t)u + 1;
        sink.pad_to(usize[u + 1].a - usize[u].a);
    });
    }
    // the element runs of the bulk path go where the statements' decoders left room for them
    for (uint32_t j = 0; j < n_bulk; j++) {
        const PtxBulkInfo* bi = bulk_info + j;
        bk.pf("bulk_copy", 2 * (size_t)bulk_tokens[j], [=] PTX_HD(size_t k) {
            if (bi->bad || !bi->dst || k >= bi->n_words) return;
            bi->dst[k] = bi->elems[k];
        });
    }
    // parser errors per module, so that a module's verdict can be read off its result row
    uint32_t* mod_nerr = (uint32_t*)bk.alloc(sizeof(uint32_t) * (n_modules + 1));
    bk.zero(mod_nerr, sizeof(uint32_t) * (n_modules + 1));
    bk.pf("count_module_errors", n_errs, [=] PTX_HD(size_t e) {
        if ((errs[e].w0 & 0xFFFFu) == E_NONE) return;
        uint32_t lo = 0, hi = n_modules;       // last module whose errors begin at or before e
        while (hi - lo > 1) {
            uint32_t mid = (lo + hi) >> 1;
            if (usize[mub[mid]].b <= (uint32_t)e) lo = mid; else hi = mid;
        }
#ifdef __CUDA_ARCH__
        atomicAdd(&mod_nerr[lo], 1u);
#else
        mod_nerr[lo]++;
#endif
    });
    bk.pf("module_results_final", n_modules, [=] PTX_HD(size_t m) {
        PtxModuleResult r = results[m];
        r.n_errors = mod_nerr[m];
        r.unit_begin = mub[m];
        r.unit_end = mub[m + 1];
        r.word_begin = n_units ? usize[mub[m]].a : 0;
        r.word_end = n_units ? usize[mub[m + 1]].a : 0;
        r.err_begin = n_units ? usize[mub[m]].b : 0;
        r.err_end = n_units ? usize[mub[m + 1]].b : 0;
        r.sequential = mod_bad[m] ? 1u : 0u;
        r.status = mod_seq_status[m];
        r.seq_tokens = mod_bad[m] ? mtb[m + 1] - ustart[mod_bad[m] - 1u] : 0u;
        results[m] = r;
    });
    bk.download(&host_counters, counters, sizeof(PtxCounters));   // .pad != 0: unit (index + 1) whose two passes disagreed
    (void)n_tokens;
}
