// Byte-parallel token boundaries and token-parallel classification: the two block-cooperative steps of the lexer.
//
// Replaces the byte-serial walk for ordinary text.  Both steps are written as PHASES: functions of (tile, thread) that
// read what earlier phases wrote and never what another thread of the same phase writes (except through the atomic
// bit operations below, whose operands every writer agrees on).  The CUDA backend runs a phase with all threads of a
// block and a __syncthreads() behind it; the host test backend runs the same phases thread by thread.
//
// Step 1, lex_mark (one tile = 64 chunks = 8 KiB): one bit per text byte, "a token starts here".
//   In code, outside comments and strings, whether a token starts at byte c depends on c and the byte p in front of it
//   only (ptx_parser/src/lib.rs:1930-2030: single-character tokens, '.'-led and sigil-led words, maximal munch over
//   [A-Za-z0-9_$]) - except around numbers that are more than a run of digits, lone sigils and the few literals with
//   "::" inside.  So every thread takes 16 bytes through a 256-entry class table and a small transition table
//   (state = what the bytes in front amount to: nothing, a word, a run of digits that started a token, a dot, a
//   word-starting sigil, a colon), and the exceptions are collected as TRIGGERS and settled afterwards, one thread per
//   trigger, by lexing forward from a known token start with the exact per-token rules (lx_one):
//     T1  a word character behind a number (12U, 0x1F, 1e5, 0f3F800000) or a digit behind a dot (.5, 1.5e-3): the run
//         of "soft" bytes around it (word characters and % . : + -) is lexed from its first byte, a token start;
//     T3  "::": .shared::cta and its like are single tokens, and what follows them starts a new one; same treatment;
//     T2  a sigil (_ $ %) that starts a word and is followed by no word character: a lexer error, not a token.
//   Chunks that contain a comment or string character (/ * ") or start inside a comment or string take the proven
//   byte-serial walk (lx_chunk), one thread per chunk.  Every writer of the second round sets bits to the true lexing,
//   so where two of them meet they agree.
// Step 2, lex_emit: the set bits are first listed (one thread per 32-byte window writes the tile offsets of its tokens
//   to their ranks in shared memory); then one thread per TOKEN finds the token's length and kind - punctuation and
//   sigil-led words at once, words that may spell a keyword through the 8-byte keyword table, numbers through the
//   exact rules - and writes the 8-byte token and the kinds entry to their final place (tile base from the scanned
//   per-chunk counts + rank inside the tile): the threads of a warp hold consecutive tokens and write consecutive entries.
#pragma once
#include "ptx_lex.h"

#define LT_CHUNKS 64u
#define LT_BYTES (LT_CHUNKS * PTX_CHUNK)
#define LT_PIECES (LT_BYTES / 16u)
#define LT_WORDS (LT_BYTES / 32u)
#define LT_TRIG_CAP 1536u          // triggers per tile; a tile with more is lexed chunk by chunk by the serial walk
#define LT_BACK_CAP 2048u          // longest look-back over a run of soft bytes; beyond it the module is lexed by one thread
#define LT_TOK_CAP 3072u           // tokens the emit step lists at a time; a tile with more goes in passes of LT_TOK_CAP / PTX_CHUNK chunks
#define LT_EXACT_CAP 2048u         // tokens of a pass the emit step leaves to its second round (more are settled on the spot)
#define LT_KW_CAP 2048u            // keyword candidates of a pass listed for the keyword round (more are looked up on the spot)

enum { TC_WS = 0, TC_ALPHA = 1, TC_DIGIT = 2, TC_SIGIL = 3, TC_PCT = 4, TC_DOT = 5, TC_COLON = 6, TC_PM = 7, TC_PUNCT = 8, TC_SPECIAL = 9, TC_BAD = 10 };
enum { LP_START = 1, LP_ERR = 2, LP_WORD = 4, LP_T1 = 8, LP_T2 = 16, LP_T3 = 32, LP_SPECIAL = 64 };

PTX_HD inline uint32_t lt_class(unsigned c) {
    if (lx_alpha(c)) return TC_ALPHA;
    if (lx_digit(c)) return TC_DIGIT;
    if (lx_ws(c)) return TC_WS;
    switch (c) {
    case '_': case '$': return TC_SIGIL;
    case '%': return TC_PCT;
    case '.': return TC_DOT;
    case ':': return TC_COLON;
    case '+': case '-': return TC_PM;
    case ',': case ';': case '@': case '|': case '!': case '(': case ')': case '[': case ']': case '{': case '}': case '<': case '>': case '=':
        return TC_PUNCT;
    case '/': case '*': case '"': return TC_SPECIAL;
    default: return TC_BAD;
    }
}
PTX_HD inline bool lt_word(uint32_t cls) { return cls == TC_ALPHA || cls == TC_DIGIT || cls == TC_SIGIL; }
// what the bytes in front of a byte amount to
enum { TS_OTHER = 0, TS_WORD = 1, TS_NUM = 2, TS_DOT = 3, TS_SIGIL = 4, TS_COLON = 5, TS_COUNT = 8 };
// byte class cc in state st: flags in the low byte, next state << 8
PTX_HD inline uint32_t lt_step(uint32_t st, uint32_t cc) {
    uint32_t e = 0, nx = TS_OTHER;
    switch (cc) {
    case TC_ALPHA:
        nx = TS_WORD;
        if (st == TS_NUM) e |= LP_T1;
        else if (!(st == TS_WORD || st == TS_SIGIL || st == TS_DOT)) e |= LP_START;
        break;
    case TC_DIGIT:
        nx = TS_WORD;
        if (st == TS_DOT) e |= LP_T1;
        else if (st == TS_NUM) nx = TS_NUM;
        else if (!(st == TS_WORD || st == TS_SIGIL)) { e |= LP_START; nx = TS_NUM; }
        break;
    case TC_SIGIL:
        nx = TS_WORD;
        if (st == TS_NUM) e |= LP_T1;
        else if (st == TS_DOT) nx = TS_SIGIL;
        else if (!(st == TS_WORD || st == TS_SIGIL)) { e |= LP_START; nx = TS_SIGIL; }
        break;
    case TC_PCT:
        nx = TS_SIGIL;
        if (st != TS_DOT) e |= LP_START;
        break;
    case TC_DOT: e |= LP_START; nx = TS_DOT; break;
    case TC_PM: case TC_PUNCT: e |= LP_START; break;
    case TC_COLON:
        e |= LP_START;
        nx = TS_COLON;
        if (st == TS_COLON) e |= LP_T3;
        break;
    case TC_SPECIAL: e |= LP_SPECIAL; break;
    case TC_BAD: e |= LP_ERR; break;
    default: break;
    }
    if (!lt_word(cc) && st == TS_SIGIL) e |= LP_T2;      // the sigil in front of this byte stands alone
    if (lt_word(cc)) e |= LP_WORD;
    return e | (nx << 12);      // entry >> 8 = next state << 4: the next table index without its class
}
// state in front of text[pos] (pos > ms), from the bytes before it; false: the look-back outgrew its cap
PTX_HD inline bool lt_state_before(const uint8_t* cls, const uint8_t* text, uint32_t pos, uint32_t ms, uint32_t* st) {
    const unsigned p = text[pos - 1];
    const uint32_t pc = cls[p];
    *st = TS_OTHER;
    switch (pc) {
    case TC_ALPHA: *st = TS_WORD; break;
    case TC_DOT: *st = TS_DOT; break;
    case TC_COLON: *st = TS_COLON; break;
    case TC_PCT: *st = TS_SIGIL; break;
    case TC_SIGIL: {
        const unsigned q = pos - 1 > ms ? text[pos - 2] : ' ';
        *st = (lx_identc(q) || q == '%') ? TS_WORD : TS_SIGIL;
        break;
    }
    case TC_DIGIT: {
        // digits inside a word, behind a dot, or a number of their own?
        uint32_t j = pos - 1;
        while (j > ms && pos - j <= LT_BACK_CAP && lx_digit(text[j - 1])) j--;
        if (pos - j > LT_BACK_CAP) return false;
        const unsigned q = j > ms ? text[j - 1] : ' ';
        *st = (lx_identc(q) || q == '%' || q == '.') ? TS_WORD : TS_NUM;
        break;
    }
    default: break;
    }
    return true;
}
// the constant tables of both steps, filled once per context
struct PtxLexTables {
    uint8_t cls[256];
    uint16_t step[TS_COUNT * 16];
    uint16_t first[256];       // emit step: what a token's first byte says about it (FK_* flags)
    // class and transition in one look-up: row `state` (1 KiB), entry `byte`: the flags of step[] in the low byte, the
    // byte offset of the next state's row above it
    uint32_t step2[TS_COUNT * 256];
};

#ifdef __CUDA_ARCH__
#define LT_ATOMIC_OR(p, v) atomicOr((p), (v))
#define LT_ATOMIC_AND(p, v) atomicAnd((p), (v))
#define LT_ATOMIC_ADD(p, v) atomicAdd((p), (v))
#else
#define LT_ATOMIC_OR(p, v) (*(p) |= (v))
#define LT_ATOMIC_AND(p, v) (*(p) &= (v))
#define LT_ATOMIC_ADD(p, v) ((*(p) += (v)) - (v))
#endif

struct PtxLexTileArgs {
    PtxLexChunkInfo info;
    const uint8_t* text;
    const uint32_t* vec;        // scanned context vectors per chunk
    uint32_t n_chunks;
    const PtxLexTables* tables;
    const uint32_t* tile_mod;   // [n_tiles] module of the tile's first chunk
    uint32_t* start_bits;       // [n_chunks * 4]: bit b of word w = a token starts at text byte 32 w + b
    uint32_t* word_bits;        // the same shape: the byte is a word character [A-Za-z0-9_$]
    PtxPair* cnt;               // [n_chunks + 1]: mark step: tokens / errors of chunk c at [c + 1]; emit step: their exclusive prefix
    uint32_t* mod_flag;         // [n_modules] 1 = a run of soft bytes outgrew the look-back: the module is lexed by one thread
    PtxToken* tokens;           // emit step
    uint16_t* kinds;
};

// working memory of one tile (shared memory on the GPU)
struct PtxLexMarkShared {
    uint8_t cls[256];
    uint16_t step[TS_COUNT * 16];
    uint32_t step2[TS_COUNT * 256];
    uint32_t start[LT_WORDS], err[LT_WORDS], word[LT_WORDS];
    uint32_t chunk_ms[LT_CHUNKS], chunk_me[LT_CHUNKS];
    uint8_t chunk_cx[LT_CHUNKS], chunk_special[LT_CHUNKS];
    uint32_t chunk_errs[LT_CHUNKS];      // errors of a chunk lexed by the serial walk
    uint32_t n_trig;
    uint32_t trig[LT_TRIG_CAP];          // position in the tile (0 .. LT_BYTES: a trigger may sit on the first byte of the next tile) | kind << 16
};

// ---- mark step, phase 0: tables, chunk geometry
// module bounds of the chunks of a tile: the tile's first module is known, the others follow in order
PTX_HD inline void lt_locate(const PtxLexTileArgs& a, uint32_t tile, uint32_t c, uint32_t* ms, uint32_t* me, bool* first) {
    uint32_t m = a.tile_mod[tile];
    while (m + 1 < a.info.n_modules && a.info.mcb[m + 1] <= c) m++;
    *ms = (uint32_t)a.info.layout[m].text_off;
    *me = *ms + (uint32_t)a.info.layout[m].text_len;
    *first = c == a.info.mcb[m];
}
// once per block: the constant tables
PTX_HD inline void lt_mark_tables(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tid, uint32_t nt) {
    for (uint32_t i = tid; i < 256; i += nt) sh.cls[i] = a.tables->cls[i];
    for (uint32_t i = tid; i < TS_COUNT * 16; i += nt) sh.step[i] = a.tables->step[i];
    for (uint32_t i = tid; i < TS_COUNT * 256; i += nt) sh.step2[i] = a.tables->step2[i];
}
// per-tile state that the first phase adds to: cleared before the first tile and by the last phase of every tile
PTX_HD inline void lt_mark_reset(PtxLexMarkShared& sh, uint32_t tid, uint32_t nt) {
    for (uint32_t k = tid; k < LT_CHUNKS; k += nt) {
        sh.chunk_special[k] = 0;
        sh.chunk_errs[k] = 0;
    }
    if (tid == 0) sh.n_trig = 0;
}
// fills the constant tables (one block of 256 threads on the GPU)
PTX_HD inline void lt_fill_tables(PtxLexTables* t, uint32_t tid, uint32_t nt);

struct alignas(16) LtWord4 {
    uint32_t x, y, z, w;
};
// ---- phase 1: chunk geometry, and 32 bytes per thread through the tables; the thread owns one word of each bit map
PTX_HD inline void lt_mark_simple(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    for (uint32_t win = tid; win < LT_WORDS; win += nt) {
        const uint32_t k = win >> 2, c = tile * LT_CHUNKS + k;
        uint32_t sm = 0, em = 0, wm = 0, any = 0;
        const uint32_t pos0 = c * PTX_CHUNK + (win & 3u) * 32u;
        // the window's text is asked for first; the chunk's module bounds and entry context (dependent look-ups, the
        // same for the four windows of a chunk) arrive while it is on its way
        LtWord4 lo = {0, 0, 0, 0}, hi = {0, 0, 0, 0};
        uint32_t ms = 0, me = 0;
        int cx = CX_CODE;
        if (c < a.n_chunks) {
            const LtWord4* w = (const LtWord4*)(a.text + pos0);
            lo = w[0];
            hi = w[1];
            bool first;
            lt_locate(a, tile, c, &ms, &me, &first);
            if (!first) cx = (int)(a.vec[c - 1] & 7u);
        }
        if ((win & 3u) == 0) {
            sh.chunk_ms[k] = ms;
            sh.chunk_me[k] = me;
            sh.chunk_cx[k] = (uint8_t)cx;
        }
        if (cx != CX_CODE) sh.chunk_special[k] = 1;
        if (c < a.n_chunks && pos0 < me) {
            uint32_t st = TS_OTHER;
            if (pos0 > ms && !lt_state_before(sh.cls, a.text, pos0, ms, &st)) {
                // the module goes to the one-thread path, which rewrites its token starts; the word bits below stay valid
                a.mod_flag[ptx_upper_bound_u32(a.info.mcb, a.info.n_modules, c) - 1] = 1;
                st = TS_WORD;
            }
            const uint32_t n = me - pos0 < 32u ? me - pos0 : 32u;
            uint32_t st4 = st << 4;      // the table entries carry the next state shifted the same way
            if (n == 32u) {
                // one look-up per byte: the entry holds the flags and where the next state's row begins; the start and
                // word bits are shifted in from the top, errors and triggers are rare and handled aside
                const uint8_t* rows = (const uint8_t*)sh.step2;
                uint32_t row = st * 1024u;
#pragma unroll
                for (uint32_t i = 0; i < 32; i++) {
                    const uint32_t wd = i < 4 ? lo.x : i < 8 ? lo.y : i < 12 ? lo.z : i < 16 ? lo.w : i < 20 ? hi.x : i < 24 ? hi.y : i < 28 ? hi.z : hi.w;
                    const uint32_t ch = (wd >> (8u * (i & 3u))) & 0xFFu;
                    const uint32_t e = *(const uint32_t*)(rows + row + ch * 4u);
#ifdef __CUDA_ARCH__
                    sm = __funnelshift_r(sm, e, 1);
                    wm = __funnelshift_r(wm, e >> 2, 1);
#else
                    sm = (sm >> 1) | (e << 31);
                    wm = (wm >> 1) | ((e >> 2) << 31);
#endif
                    any |= e;
                    if (e & (LP_ERR | LP_T1 | LP_T2 | LP_T3)) {
                        em |= ((e >> 1) & 1u) << i;
                        if (e & (LP_T1 | LP_T2 | LP_T3)) {
                            uint32_t slot = LT_ATOMIC_ADD(&sh.n_trig, 1u);
                            if (slot < LT_TRIG_CAP) sh.trig[slot] = (win * 32u + i) | ((e & (LP_T1 | LP_T2 | LP_T3)) << 16);
                        }
                    }
                    row = e >> 8;
                }
                st4 = (row >> 10) << 4;
            } else {
                for (uint32_t i = 0; i < n; i++) {
                    const uint32_t e = sh.step[st4 | sh.cls[a.text[pos0 + i]]];
                    sm |= (e & 1u) << i;
                    em |= ((e >> 1) & 1u) << i;
                    wm |= ((e >> 2) & 1u) << i;
                    any |= e;
                    if (e & (LP_T1 | LP_T2 | LP_T3)) {
                        uint32_t slot = LT_ATOMIC_ADD(&sh.n_trig, 1u);
                        if (slot < LT_TRIG_CAP) sh.trig[slot] = (win * 32u + i) | ((e & (LP_T1 | LP_T2 | LP_T3)) << 16);
                    }
                    st4 = e >> 8;
                }
            }
            st = st4 >> 4;
            // the triggers that look one byte back also fire behind the last byte of the tile and behind the last byte of
            // the module (where nothing follows)
            if ((win == LT_WORDS - 1 && n == 32 && pos0 + 32 < me) || pos0 + n == me) {
                const uint32_t e = sh.step[(st << 4) | (pos0 + n == me ? (uint32_t)TC_WS : (uint32_t)sh.cls[a.text[pos0 + 32]])];
                if (e & (LP_T1 | LP_T2 | LP_T3)) {
                    uint32_t slot = LT_ATOMIC_ADD(&sh.n_trig, 1u);
                    if (slot < LT_TRIG_CAP) sh.trig[slot] = (win * 32u + n) | ((e & (LP_T1 | LP_T2 | LP_T3)) << 16);
                }
            }
        }
        sh.start[win] = sm;
        sh.err[win] = em;
        sh.word[win] = wm;
        if (any & LP_SPECIAL) sh.chunk_special[k] = 1;
    }
}

// set the true lexing of [start, start + len) inside the tile: a token (or an error) starts at `start`, nothing after it
PTX_HD inline void lt_truth(PtxLexMarkShared& sh, uint32_t tile_base, uint32_t start, uint32_t len, bool is_err) {
    const uint32_t lo = tile_base, hi = tile_base + LT_BYTES;
    uint32_t b = start < lo ? lo : start, e = start + len > hi ? hi : start + len;
    if (start + len < start) e = hi;     // wrapped: cannot happen below 4 GiB of text
    if (b >= e) return;
    for (uint32_t p = b; p < e;) {
        const uint32_t o = p - lo, w = o >> 5, bit = o & 31u;
        const uint32_t upto = (e - lo) - (w << 5) < 32u ? (e - lo) - (w << 5) : 32u;      // bits [bit, upto) of word w
        uint32_t mask = (upto == 32u ? 0xFFFFFFFFu : ((1u << upto) - 1u)) & ~((1u << bit) - 1u);
        uint32_t set_s = 0, set_e = 0;
        if (p == start) { if (is_err) set_e = 1u << bit; else set_s = 1u << bit; }
        const uint32_t clr_s = mask & ~set_s, clr_e = mask & ~set_e;
        if (sh.start[w] & clr_s) LT_ATOMIC_AND(&sh.start[w], ~clr_s);
        if (sh.err[w] & clr_e) LT_ATOMIC_AND(&sh.err[w], ~clr_e);
        if (set_s) LT_ATOMIC_OR(&sh.start[w], set_s);
        if (set_e) LT_ATOMIC_OR(&sh.err[w], set_e);
        p = lo + (w << 5) + upto;
    }
}
// lex forward from a token start through the rest of the run of soft bytes, setting the true lexing inside the tile
PTX_HD inline void lt_chain(PtxLexMarkShared& sh, const uint8_t* text, uint32_t tile_base, uint32_t pos, uint32_t me) {
    const uint32_t hi = tile_base + LT_BYTES;
    while (pos < me && pos < hi && lx_soft(text[pos])) {
        uint32_t len;
        uint16_t k = lx_one(text, pos, me, &len);
        lt_truth(sh, tile_base, pos, len, k == T_ERROR);
        pos += len;
    }
}
// The helpers of the trigger phase go through the class and transition tables in shared memory: a few threads of a
// tile run them while the others wait, so they are kept short (the arithmetic forms lt_class / lt_step cost more in
// instruction fetches than in execution there).
PTX_HD inline bool lt_soft_class(uint32_t cls) { return (0xFEu >> cls) & 1u; }       // TC_ALPHA .. TC_PM: what lx_soft accepts
// does the run of soft bytes [q, end), which begins at a token start, hold a T1 or T3 trigger?
PTX_HD inline bool lt_run_has_trigger(const PtxLexMarkShared& sh, const uint8_t* text, uint32_t q, uint32_t end) {
    uint32_t st4 = (uint32_t)TS_OTHER << 4;
    for (uint32_t j = q; j < end; j++) {
        const uint32_t e = sh.step[st4 | sh.cls[text[j]]];
        if (e & (LP_T1 | LP_T3)) return true;
        st4 = e >> 8;
    }
    return false;
}
// token sink of the serial walk over one chunk
struct LexMarkSink {
    PtxLexMarkShared* sh;
    uint32_t tile_base;
    uint32_t n_errors = 0, last_end = 0;
    PTX_HD void token(uint32_t start, uint32_t len, uint16_t) {
        lt_truth(*sh, tile_base, start, len, false);
        last_end = start + len;
    }
    PTX_HD void error(uint32_t start, uint32_t len) {
        n_errors++;
        if (start + len > last_end) last_end = start + len;
    }
};

// ---- phase 2a: chunks with comment or string characters, one thread per chunk
PTX_HD inline void lt_mark_special(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    const bool overflow = sh.n_trig > LT_TRIG_CAP;      // too many triggers to list: every chunk takes the serial walk
    for (uint32_t k = tid; k < LT_CHUNKS; k += nt) {
        const uint32_t c = tile * LT_CHUNKS + k;
        if (c >= a.n_chunks) continue;
        if (overflow) sh.chunk_special[k] = 1;
        if (!sh.chunk_special[k]) continue;
        const uint32_t ms = sh.chunk_ms[k], me = sh.chunk_me[k], cs = c * PTX_CHUNK, tile_base = tile * LT_BYTES;
        for (uint32_t w = 0; w < 4; w++) sh.start[k * 4 + w] = sh.err[k * 4 + w] = 0;
        if (cs >= me) continue;
        // the walk looks back over one run of soft bytes; a run longer than the cap goes to the one-thread path
        uint32_t run_start = cs;
        if (sh.chunk_cx[k] == CX_CODE && cs > ms && lx_soft(a.text[cs - 1]) && lx_soft(a.text[cs])) {
            uint32_t q = cs - 1;
            while (q > ms && cs - q <= LT_BACK_CAP && lx_soft(a.text[q - 1])) q--;
            if (cs - q > LT_BACK_CAP) { a.mod_flag[ptx_upper_bound_u32(a.info.mcb, a.info.n_modules, c) - 1] = 1; continue; }
            run_start = q;
        }
        LexMarkSink sink;
        sink.sh = &sh;
        sink.tile_base = tile_base;
        lx_chunk(PtxGlobalReader{a.text, me}, a.text, ms, me, cs, cs + PTX_CHUNK, (int)sh.chunk_cx[k], sink);
        sh.chunk_errs[k] = sink.n_errors;
        // the bytes behind the last token that belong to the same run of soft bytes, in the chunks that follow
        if (sink.last_end >= cs + PTX_CHUNK) lt_chain(sh, a.text, tile_base, sink.last_end, me);
        // a run of soft bytes that reaches into the chunk from the chunk in front is code: its triggers may lie in this
        // chunk, where nobody else answers them, and can change a token start in front of the chunk
        if (run_start < cs) lt_chain(sh, a.text, tile_base, run_start, me);
    }
}

// A word character behind a number (the trigger at `pos`) whose token, by the number rules (lx_number), ends where the
// run of word characters ends - 0x1F, 0f3F800000, 0d and sixteen, 12U, with no word character behind them: the first
// round took the whole run for one token that starts at the number's first digit, which is the true lexing, and what
// follows starts afresh.  Nothing to settle; other triggers of the same run of soft bytes look after themselves.
PTX_HD inline bool lt_trigger_benign(const PtxLexMarkShared& sh, const uint8_t* text, uint32_t pos, uint32_t ms, uint32_t me) {
    if (pos <= ms || pos >= me) return false;
    const unsigned c = text[pos];
    if (sh.cls[c] == TC_DIGIT) return false;     // the other kind of trigger: a digit behind a dot
    if (c == 'U') return pos + 1 >= me || !lt_word(sh.cls[text[pos + 1]]);
    const unsigned d = c | 32u;
    if (d != 'x' && d != 'f' && d != 'd') return false;
    if (text[pos - 1] != '0' || (pos - 1 > ms && sh.cls[text[pos - 2]] == TC_DIGIT)) return false;      // the number is a single 0
    const uint32_t stop = d == 'x' ? pos + 18u : d == 'f' ? pos + 9u : pos + 17u;
    uint32_t q = pos + 1;
    for (; q < me && q < stop; q++) {
        const uint32_t cc = sh.cls[text[q]];
        if (cc != TC_ALPHA && cc != TC_DIGIT) break;
    }
    if (d == 'x' ? (q == pos + 1 || q == stop) : q != stop) return false;      // hex: a digit, and no longer than looked at here
    return q >= me || !lt_word(sh.cls[text[q]]);
}
// ---- phase 2b: one thread per trigger, and one for the run of soft bytes that enters the tile
PTX_HD inline void lt_mark_triggers(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    const uint32_t tile_base = tile * LT_BYTES;
    const uint32_t n_trig = sh.n_trig > LT_TRIG_CAP ? 0u : sh.n_trig;
    // the block's last thread: a run of soft bytes that begins in front of the tile may hold a number or a "::" literal;
    // it is lexed from its start (the triggers go to the first threads: on the device another warp, at the same time)
    if (tid == nt - 1) {
        const uint32_t c = tile * LT_CHUNKS;
        const uint32_t ms = sh.chunk_ms[0], me = sh.chunk_me[0];
        if (c < a.n_chunks && !sh.chunk_special[0] && tile_base < me && tile_base > ms && lt_soft_class(sh.cls[a.text[tile_base]]) &&
            lt_soft_class(sh.cls[a.text[tile_base - 1]])) {
            uint32_t q = tile_base - 1;
            while (q > ms && tile_base - q <= LT_BACK_CAP && lt_soft_class(sh.cls[a.text[q - 1]])) q--;
            if (tile_base - q > LT_BACK_CAP) a.mod_flag[ptx_upper_bound_u32(a.info.mcb, a.info.n_modules, c) - 1] = 1;
            // one byte past the tile's first: a trigger there (a digit behind a dot, the second colon) looks back into the run
            else if (lt_run_has_trigger(sh, a.text, q, tile_base + 1 < me ? tile_base + 1 : me)) lt_chain(sh, a.text, tile_base, q, me);
        }
    }
    for (uint32_t t = tid; t < n_trig; t += nt) {
        const uint32_t off = sh.trig[t] & 0xFFFFu, kind = sh.trig[t] >> 16;
        const uint32_t pos = tile_base + off;
        // T1 sits on its digit; T2 and T3 sit one byte behind the sigil / the first colon they are about
        const uint32_t at = ((kind & LP_T1) && off < LT_BYTES) ? off : (off ? off - 1 : 0u);
        const uint32_t k = at >> 7;
        if (sh.chunk_special[k]) continue;        // lexed by the serial walk
        const uint32_t ms = sh.chunk_ms[k], me = sh.chunk_me[k];
        if (kind == LP_T1 && off < LT_BYTES && lt_trigger_benign(sh, a.text, pos, ms, me)) continue;
        if (kind & (LP_T1 | LP_T3)) {
            // the run of soft bytes around the trigger is lexed from its first byte, which is a token start (several
            // triggers in one run do the same work and write the same bits)
            uint32_t j = pos < me ? pos : me - 1;
            while (j > ms && pos - j <= LT_BACK_CAP && lt_soft_class(sh.cls[a.text[j - 1]])) j--;
            if (pos - j > LT_BACK_CAP) { a.mod_flag[ptx_upper_bound_u32(a.info.mcb, a.info.n_modules, tile * LT_CHUNKS + k) - 1] = 1; continue; }
            lt_chain(sh, a.text, tile_base, j, me);
        }
        if (kind & LP_T2) lt_truth(sh, tile_base, pos - 1, 1, true);      // the sigil at pos - 1 stands alone: an error, no token
    }
}

// ---- phase 3: counts and the bit map
PTX_HD inline void lt_mark_finish(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    for (uint32_t k = tid; k < LT_CHUNKS; k += nt) {
        const uint32_t c = tile * LT_CHUNKS + k;
        const bool special = sh.chunk_special[k];
        const uint32_t serial_errs = sh.chunk_errs[k];
        sh.chunk_special[k] = 0;         // for the next tile (lt_mark_reset)
        sh.chunk_errs[k] = 0;
        if (c >= a.n_chunks) continue;
        uint32_t ntok = 0, nerr = 0;
        for (uint32_t w = 0; w < 4; w++) {
#ifdef __CUDA_ARCH__
            ntok += __popc(sh.start[k * 4 + w]);
            nerr += __popc(sh.err[k * 4 + w]);
#else
            ntok += (uint32_t)__builtin_popcount(sh.start[k * 4 + w]);
            nerr += (uint32_t)__builtin_popcount(sh.err[k * 4 + w]);
#endif
        }
        PtxPair p;
        p.a = ntok;
        p.b = special ? serial_errs : nerr;
        a.cnt[c + 1] = p;
        if (c == 0) { PtxPair z; z.a = z.b = 0; a.cnt[0] = z; }
    }
    for (uint32_t w = tid; w < LT_WORDS; w += nt)
        if (tile * LT_CHUNKS + (w >> 2) < a.n_chunks) {
            a.start_bits[(size_t)tile * LT_WORDS + w] = sh.start[w];
            a.word_bits[(size_t)tile * LT_WORDS + w] = sh.word[w];
        }
    if (tid == 0) sh.n_trig = 0;
}

// ---- modules whose soft runs outgrew the look-back: one thread lexes the whole module and rewrites its bits and counts
struct LexModuleSink {
    uint32_t* start_bits;
    PtxPair* cnt;
    PTX_HD void token(uint32_t start, uint32_t, uint16_t) {
        start_bits[start >> 5] |= 1u << (start & 31u);
        cnt[(start >> 7) + 1].a++;
    }
    PTX_HD void error(uint32_t start, uint32_t) { cnt[(start >> 7) + 1].b++; }
};
PTX_HD inline void lt_lex_module_serial(const PtxLexTileArgs& a, uint32_t m) {
    if (!a.mod_flag[m]) return;
    const uint32_t c0 = a.info.mcb[m], c1 = a.info.mcb[m + 1];
    const uint32_t ms = (uint32_t)a.info.layout[m].text_off, me = ms + (uint32_t)a.info.layout[m].text_len;
    for (uint32_t c = c0; c < c1; c++) {
        for (uint32_t w = 0; w < 4; w++) a.start_bits[(size_t)c * 4 + w] = 0;
        PtxPair z;
        z.a = z.b = 0;
        a.cnt[c + 1] = z;
    }
    LexModuleSink sink{a.start_bits, a.cnt};
    // an error reported at the end of the module (unterminated comment) is counted with the module's last chunk
    struct Clamp {
        LexModuleSink& s;
        uint32_t last;
        PTX_HD void token(uint32_t st, uint32_t l, uint16_t k) { s.token(st, l, k); }
        PTX_HD void error(uint32_t st, uint32_t l) { s.error(st < last ? st : last, l); }
    } clamp{sink, me > ms ? me - 1 : ms};
    lx_chunk(PtxGlobalReader{a.text, me}, a.text, ms, me, ms, me, CX_CODE, clamp);
}

// =============================================================================================== emit step
// what a token's first byte says about it: provisional kind in the low 9 bits, then
enum { FK_WORD = 0x200,      // a word: length 1 + the run of word characters behind the first byte
       FK_KW = 0x400,        // may spell a keyword
       FK_EXACT = 0x800,     // numbers, strings, anything unusual: the exact per-token rules
       FK_DOT = 0x1000 };    // '.': depends on the next byte
struct PtxLexEmitShared {
    uint8_t cls[256];
    uint16_t first[256];
    PtxKw8Entry kw[PTX_KW8_SIZE];       // the keyword table
    uint32_t bits[LT_WORDS], word[LT_WORDS + 2];
    uint32_t chunk_me[LT_CHUNKS], chunk_rank[LT_CHUNKS + 1];     // rank of the chunk's first token inside the tile
    uint16_t tokoff[LT_TOK_CAP];        // tile offset of token r of the pass
    uint16_t exact[LT_EXACT_CAP];       // tokens left to the second round, by their rank in the pass
    uint16_t kwlist[LT_KW_CAP];         // first round -> keyword round: the tokens that may spell a keyword, likewise
    uint32_t n_listed;                  // entries of exact[] << 16 | entries of kwlist[]
    // The tile's text and twelve words of zeros behind it.  The threads of a warp work on consecutive tokens: their byte
    // reads fall into a stretch of a hundred bytes or so, different banks without further ado.
    uint32_t text[LT_BYTES / 4 + 12];
};
// byte `o` of the tile (o may run a few bytes past the tile: zeros), and text word `i`
PTX_HD inline unsigned lt_tb(const PtxLexEmitShared& sh, uint32_t o) { return ((const uint8_t*)sh.text)[o]; }
PTX_HD inline uint32_t lt_tw(const PtxLexEmitShared& sh, uint32_t i) { return sh.text[i]; }

// once per block: the constant tables
PTX_HD inline void lt_emit_tables(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tid, uint32_t nt) {
    for (uint32_t i = tid; i < 256; i += nt) {
        sh.cls[i] = a.tables->cls[i];
        sh.first[i] = a.tables->first[i];
    }
    for (uint32_t i = tid; i < PTX_KW8_SIZE; i += nt) sh.kw[i] = ptx_kw8_table[i];
}
#define LT_TEXT_LOADS 8u              // text words a thread of a 256-thread block holds in registers during the init phase
PTX_HD inline void lt_emit_init(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    const uint32_t c0 = tile * LT_CHUNKS;
    const uint32_t n_words = (c0 + LT_CHUNKS <= a.n_chunks ? LT_CHUNKS : a.n_chunks - c0) * (PTX_CHUNK / 4);
    const uint32_t* src = (const uint32_t*)(a.text + (size_t)tile * LT_BYTES);
    // The text loads go out first and land in registers: the look-ups below (three dependent loads per chunk) then
    // run under their latency instead of after it.
    const bool held = nt * LT_TEXT_LOADS >= LT_BYTES / 4;
    uint32_t tx[LT_TEXT_LOADS];
    if (held) {
#ifdef __CUDA_ARCH__
#pragma unroll
#endif
        for (uint32_t j = 0; j < LT_TEXT_LOADS; j++) {
            const uint32_t i = tid + j * nt;
            tx[j] = i < n_words ? src[i] : 0u;
        }
    }
    for (uint32_t w = tid; w < LT_WORDS + 2; w += nt) {
        const bool in = w < LT_WORDS && c0 + (w >> 2) < a.n_chunks;
        if (w < LT_WORDS) sh.bits[w] = in ? a.start_bits[(size_t)tile * LT_WORDS + w] : 0u;
        sh.word[w] = in ? a.word_bits[(size_t)tile * LT_WORDS + w] : 0u;
    }
    for (uint32_t k = tid; k <= LT_CHUNKS; k += nt) {
        uint32_t c = c0 + k < a.n_chunks ? c0 + k : a.n_chunks;
        sh.chunk_rank[k] = a.cnt[c].a - a.cnt[c0].a;
        if (k < LT_CHUNKS) {
            uint32_t ms = 0, me = 0;
            bool first;
            if (c0 + k < a.n_chunks) lt_locate(a, tile, c0 + k, &ms, &me, &first);
            sh.chunk_me[k] = me;
        }
    }
    if (held) {
#ifdef __CUDA_ARCH__
#pragma unroll
#endif
        for (uint32_t j = 0; j < LT_TEXT_LOADS; j++) {
            const uint32_t i = tid + j * nt;
            if (i < LT_BYTES / 4) sh.text[i] = tx[j];
        }
        for (uint32_t i = LT_BYTES / 4 + tid; i < LT_BYTES / 4 + 12; i += nt) sh.text[i] = 0u;
    } else {
        for (uint32_t i = tid; i < LT_BYTES / 4 + 12; i += nt) sh.text[i] = i < n_words ? src[i] : 0u;
    }
}
// length of the run of word characters that starts at tile offset o (at most 32; the bits behind the tile are zero)
PTX_HD inline uint32_t lt_word_run(const PtxLexEmitShared& sh, uint32_t o) {
    const uint32_t w = o >> 5, b = o & 31u;
#ifdef __CUDA_ARCH__
    const uint32_t win = __funnelshift_r(sh.word[w], sh.word[w + 1], b);
    const uint32_t inv = ~win;
    return inv ? (uint32_t)(__ffs(inv) - 1) : 32u;
#else
    const uint64_t both = ((uint64_t)sh.word[w + 1] << 32) | sh.word[w];
    const uint32_t inv = ~(uint32_t)(both >> b);
    return inv ? (uint32_t)__builtin_ctz(inv) : 32u;
#endif
}
PTX_HD inline void lt_put_token(const PtxLexTileArgs& a, uint32_t j, uint32_t start, uint32_t len, uint16_t kind) {
    PtxTokenWord t;
    t.x = start;
    t.y = (len >= 0xFFFFu ? 0xFFFFu : len) | ((uint32_t)kind << 16);
    ((PtxTokenWord*)a.tokens)[j] = t;
    a.kinds[j] = ptx_kind_entry(a.text, start, len, kind);
}
// a token that is no numeric literal: the kinds entry is kind and capped length
PTX_HD inline void lt_put_plain(const PtxLexTileArgs& a, uint32_t j, uint32_t start, uint32_t len, uint32_t kind) {
    PtxTokenWord t;
    t.x = start;
    t.y = len | (kind << 16);
    ((PtxTokenWord*)a.tokens)[j] = t;
    a.kinds[j] = (uint16_t)(kind | ((len < 127u ? len : 127u) << 9));
}
// the keyword table through the tile's text in shared memory: the token lies inside the tile
PTX_HD inline uint32_t lt_keyword8(const PtxLexEmitShared& sh, uint32_t off, uint32_t len) {
    if (len > PTX_KW_MAXLEN) return T_ERROR;
    const uint32_t shft = (off & 3u) * 8u;
    const uint32_t wi = off >> 2;
    const uint32_t w0 = lt_tw(sh, wi), w1 = lt_tw(sh, wi + 1), w2 = lt_tw(sh, wi + 2);
#ifdef __CUDA_ARCH__
    uint32_t lo = __funnelshift_r(w0, w1, shft), hi = __funnelshift_r(w1, w2, shft);
#else
    uint32_t lo = shft ? (w0 >> shft) | (w1 << (32u - shft)) : w0;
    uint32_t hi = shft ? (w1 >> shft) | (w2 << (32u - shft)) : w1;
#endif
    if (len < 4) { lo &= (1u << (8u * len)) - 1u; hi = 0; }
    else if (len < 8) hi &= (1u << (8u * (len - 4u))) - 1u;
    uint32_t h = (lo ^ hi) * 0x9E3779B1u;
    h ^= len * 0x85EBCA6Bu;
    h ^= h >> 15;
    h *= 0x2C1B3C6Du;
    h ^= h >> 12;
    h &= PTX_KW8_SIZE - 1;
    for (;;) {
        const PtxKw8Entry e = sh.kw[h];
        if (e.kind == 0xFFFF) return T_ERROR;
        if (e.lo == lo && e.hi == hi && e.len == len) {
            bool same = true;
            for (uint32_t i = 8; i < len; i++)
                if ((uint8_t)ptx_kw_pool[e.off + i] != lt_tb(sh, off + i)) { same = false; break; }
            if (same) return e.kind;
        }
        h = (h + 1) & (PTX_KW8_SIZE - 1);
    }
}
// the exact rules for one token
PTX_HD inline void lt_emit_exact(const PtxLexTileArgs& a, uint32_t j, uint32_t pos, uint32_t me) {
    uint32_t len;
    uint16_t k;
    if (a.text[pos] == '"') {
        uint32_t q = pos + 1;
        while (q < me && a.text[q] != '"') q++;
        len = q + 1 - pos;
        k = T_STRING;
    } else {
        k = lx_one(a.text, pos, me, &len);
    }
    lt_put_token(a, j, pos, len, k);
}
// The tile's text in shared memory as something to index by byte offset
struct LtTileBytes {
    const PtxLexEmitShared* sh;
    uint32_t base;                       // offset inside the tile that index 0 stands for
    PTX_HD unsigned operator[](uint64_t i) const { return lt_tb(*sh, base + (uint32_t)i); }
};
// Numbers are most of what the exact rules see: the number rules and the literal code straight from the tile in shared
// memory, unless the number, or what the rules look at behind it (three bytes: an exponent's 'e', sign and first digit;
// eighteen for the shortest reading of what may be a hexadecimal float), may lie behind the tile (then, as everything else, through lt_emit_exact)
PTX_HD inline void lt_emit_exact_tile(const PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile_base, uint32_t j, uint32_t off, uint32_t me) {
    const bool module_ends_here = me - tile_base <= LT_BYTES;
    const uint32_t end = module_ends_here ? me - tile_base : LT_BYTES;
    // Most numbers are a few decimal digits or a 0f float: short straight-line code for those (the threads of a warp hold
    // numbers of all sorts, and the general rules below are long).  Up to nine decimal digits with no '.', 'U' or tenth
    // digit behind them are a DECIMAL below 2^31 (literal code 0: lx_number, ptx_literal_scan); a lone 0 likewise; 0f and
    // eight hexadecimal digits are an F32HEX with code 0.  Everything else, and anything near the end of the tile or the
    // module, takes the general rules.
    if (off + 12u <= end) {
        const unsigned c0 = lt_tb(sh, off);
        uint32_t len = 0, kind = T_DECIMAL;
        if (c0 - '1' < 9u) {
            uint32_t q = off + 1;
            while (q < off + 9u && lt_tb(sh, q) - '0' < 10u) q++;
            const unsigned c = lt_tb(sh, q);
            if (c - '0' >= 10u && c != '.' && c != 'U') len = q - off;
        } else if (c0 == '0') {
            const unsigned c = lt_tb(sh, off + 1), d = c | 32u;
            if (d == 'f') {
                uint32_t hex = 1;
                for (uint32_t i = 2; i < 10; i++) {
                    const unsigned ch = lt_tb(sh, off + i);
                    hex &= (uint32_t)(ch - '0' < 10u) | (uint32_t)((ch | 32u) - 'a' < 6u);
                }
                if (hex) { len = 10; kind = T_F32HEX; }
            } else if (c - '0' >= 10u && c != '.' && c != 'U' && d != 'x' && d != 'd') {
                len = 1;
            }
        }
        if (len) {
            PtxTokenWord t;
            t.x = tile_base + off;
            t.y = len | (kind << 16);
            ((PtxTokenWord*)a.tokens)[j] = t;
            a.kinds[j] = (uint16_t)kind;
            return;
        }
    }
    if (off < end && lx_digit(lt_tb(sh, off))) {
        const LtTileBytes bytes{&sh, 0};
        uint32_t len;
        const uint16_t k = lx_number(bytes, off, end, &len);
        if (module_ends_here || off + (len > 18u ? len : 18u) + 3u <= end) {
            PtxTokenWord t;
            t.x = tile_base + off;
            t.y = len | ((uint32_t)k << 16);                  // a length inside a tile
            ((PtxTokenWord*)a.tokens)[j] = t;
            uint64_t mag;
            a.kinds[j] = (uint16_t)(k | (ptx_literal_scan(LtTileBytes{&sh, off}, len, k, &mag) << 9));
            return;
        }
    }
    lt_emit_exact(a, j, tile_base + off, me);
}
PTX_HD inline uint32_t lt_window_rank(const PtxLexEmitShared& sh, uint32_t w) {
    uint32_t rank = sh.chunk_rank[w >> 2];
    for (uint32_t v = w & ~3u; v < w; v++) {
#ifdef __CUDA_ARCH__
        rank += __popc(sh.bits[v]);
#else
        rank += (uint32_t)__builtin_popcount(sh.bits[v]);
#endif
    }
    return rank;
}
// A tile is emitted in passes: one, if its tokens fit the list; else chunk ranges that always fit (a chunk holds at
// most PTX_CHUNK tokens).  Every thread of the block computes the same ranges.
struct LtPass {
    uint32_t c_a, c_b;        // chunks [c_a, c_b) of the tile
    uint32_t base, n;         // rank in the tile of the pass's first token; tokens in the pass
};
PTX_HD inline uint32_t lt_emit_passes(const PtxLexEmitShared& sh) {
    const uint32_t per = LT_TOK_CAP / PTX_CHUNK;
    return sh.chunk_rank[LT_CHUNKS] <= LT_TOK_CAP ? 1u : (LT_CHUNKS + per - 1) / per;
}
PTX_HD inline LtPass lt_emit_pass(const PtxLexEmitShared& sh, uint32_t pass) {
    LtPass p;
    if (sh.chunk_rank[LT_CHUNKS] <= LT_TOK_CAP) {
        p.c_a = 0;
        p.c_b = LT_CHUNKS;
    } else {
        const uint32_t per = LT_TOK_CAP / PTX_CHUNK;
        p.c_a = pass * per;
        p.c_b = p.c_a + per < LT_CHUNKS ? p.c_a + per : LT_CHUNKS;
    }
    p.base = sh.chunk_rank[p.c_a];
    p.n = sh.chunk_rank[p.c_b] - p.base;
    return p;
}
// Slots in the two lists of the block (numbers and their like; keyword candidates) for every caller that wants one;
// the counter holds both lengths (the first list's in the high half).  On the device all 32 lanes of the warp call it
// together and the warp takes its slots with one atomic operation.
PTX_HD inline void lt_list_slots(uint32_t* counter, bool want_exact, bool want_kw, uint32_t* slot_exact, uint32_t* slot_kw) {
#ifdef __CUDA_ARCH__
    const uint32_t me = __ballot_sync(0xFFFFFFFFu, want_exact), mk = __ballot_sync(0xFFFFFFFFu, want_kw);
    if (!(me | mk)) return;
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t base = 0;
    if (lane == 0) base = atomicAdd(counter, ((uint32_t)__popc(me) << 16) | (uint32_t)__popc(mk));
    base = __shfl_sync(0xFFFFFFFFu, base, 0);
    const uint32_t below = (1u << lane) - 1u;
    *slot_exact = (base >> 16) + (uint32_t)__popc(me & below);
    *slot_kw = (base & 0xFFFFu) + (uint32_t)__popc(mk & below);
#else
    *slot_exact = *counter >> 16;
    *slot_kw = *counter & 0xFFFFu;
    *counter += ((uint32_t)want_exact << 16) | (uint32_t)want_kw;
#endif
}
// Listing: one thread per 32-byte window of the pass writes the tile offsets of its tokens to their ranks
PTX_HD inline void lt_emit_list(PtxLexEmitShared& sh, uint32_t pass, uint32_t tid, uint32_t nt) {
    const LtPass p = lt_emit_pass(sh, pass);
    for (uint32_t w = p.c_a * 4u + tid; w < p.c_b * 4u; w += nt) {
        uint32_t bits = sh.bits[w];
        if (!bits) continue;
        uint32_t r = lt_window_rank(sh, w) - p.base;
        while (bits) {
#ifdef __CUDA_ARCH__
            const uint32_t b = (uint32_t)(__ffs(bits) - 1);
#else
            const uint32_t b = (uint32_t)__builtin_ctz(bits);
#endif
            bits &= bits - 1;
            sh.tokoff[r++] = (uint16_t)(w * 32u + b);
        }
    }
    if (tid == 0) sh.n_listed = 0;
}
// First round: one thread per token, the same few steps for every token: first byte, length from the word-character
// bits, kind by the first byte.  Every token but the numbers, strings and the unusual (second round: exact rules) is
// written here; words that may spell a keyword are written as plain words and listed for the keyword round, so that
// no thread looks up a keyword while its neighbours wait.  Every thread of the block makes the same number of turns.
PTX_HD inline void lt_emit_first(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t pass, uint32_t tid, uint32_t nt) {
    const uint32_t tile_base = tile * LT_BYTES;
    const uint32_t j0 = a.cnt[tile * LT_CHUNKS].a;
    const LtPass p = lt_emit_pass(sh, pass);
    for (uint32_t r0 = 0; r0 < p.n; r0 += nt) {
        const uint32_t r = r0 + tid;
        const bool valid = r < p.n;
        // straight-line on purpose (bitwise logic, no short-circuit): the tokens of a warp are of all sorts, and every
        // branch taken by some of them would be paid by all
        const uint32_t off = valid ? sh.tokoff[r] : 0u;
        const uint32_t f = sh.first[lt_tb(sh, off)];
        const uint32_t dc = sh.cls[lt_tb(sh, off + 1)];        // the bytes behind the tile read as 0: no word characters
        const uint32_t run = lt_word_run(sh, off + 1);
        const uint32_t e = off + 1 + run;
        const uint32_t colons = (uint32_t)(lt_tb(sh, e) == ':') & (uint32_t)(lt_tb(sh, e + 1) == ':');
        const uint32_t isdot = (f >> 12) & 1u;                                                // FK_DOT
        const uint32_t dotword = isdot & ((uint32_t)(dc == TC_ALPHA) | (uint32_t)(dc == TC_SIGIL));
        const uint32_t word = ((f >> 9) & 1u) | dotword;                                        // FK_WORD
        const uint32_t len = 1u + (word ? run : 0u);
        const uint32_t kind = dotword ? (uint32_t)T_DOTIDENT : (f & 0x1FFu);
        const uint32_t kw = ((f >> 10) & 1u) | dotword;                                         // FK_KW
        // exact rules: numbers, strings, the unusual; a dot in front of a digit or '%'; a lone sigil behind a dot or "::"
        // behind a dot-word; a long word, or one that may go on behind the tile
        const uint32_t exact = ((f >> 11) & 1u) |
                               (isdot & ((uint32_t)(dc == TC_DIGIT) | (uint32_t)(dc == TC_PCT) | (uint32_t)(off + 1 >= LT_BYTES))) |
                               (dotword & (((uint32_t)(dc == TC_SIGIL) & (uint32_t)(run == 1u)) | colons | (uint32_t)(e + 1 >= LT_BYTES))) |
                               (word & ((uint32_t)(run >= 32u) | (uint32_t)(off + len >= LT_BYTES)));
        const bool want_exact = valid && exact;
        const bool want_kw = valid && !exact && kw && len <= PTX_KW_MAXLEN;
        uint32_t slot_e = 0, slot_k = 0;
        lt_list_slots(&sh.n_listed, want_exact, want_kw, &slot_e, &slot_k);
        if (!valid) continue;
        const uint32_t j = j0 + p.base + r;
        if (exact) {
            if (slot_e < LT_EXACT_CAP) sh.exact[slot_e] = (uint16_t)r;
            else lt_emit_exact_tile(sh, a, tile_base, j, off, sh.chunk_me[off >> 7]);       // no room in the list (a tile of numbers)
            continue;
        }
        lt_put_plain(a, j, tile_base + off, len, kind);
        if (want_kw) {
            if (slot_k < LT_KW_CAP) sh.kwlist[slot_k] = (uint16_t)r;
            else {
                const uint32_t k = lt_keyword8(sh, off, len);
                if (k != T_ERROR) {
                    a.tokens[j].kind = (uint16_t)k;
                    a.kinds[j] = (uint16_t)(k | (len << 9));
                }
            }
        }
    }
}
// keyword round: the listed words through the keyword table; a word that spells one gets that kind
PTX_HD inline void lt_emit_keywords(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t pass, uint32_t tid, uint32_t nt) {
    const uint32_t j0 = a.cnt[tile * LT_CHUNKS].a;
    const LtPass p = lt_emit_pass(sh, pass);
    const uint32_t listed = sh.n_listed & 0xFFFFu, n_kw = listed < LT_KW_CAP ? listed : LT_KW_CAP;
    for (uint32_t x = tid; x < n_kw; x += nt) {
        const uint32_t r = sh.kwlist[x], off = sh.tokoff[r];
        const uint32_t len = 1 + lt_word_run(sh, off + 1);
        const uint32_t k = lt_keyword8(sh, off, len);
        if (k != T_ERROR) {
            const uint32_t j = j0 + p.base + r;
            a.tokens[j].kind = (uint16_t)k;
            a.kinds[j] = (uint16_t)(k | (len << 9));      // a keyword is at most 20 bytes long
        }
    }
}
// second round: the exact rules, one thread per token left over
PTX_HD inline void lt_emit_second(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t pass, uint32_t tid, uint32_t nt) {
    const uint32_t tile_base = tile * LT_BYTES, j0 = a.cnt[tile * LT_CHUNKS].a;
    const LtPass p = lt_emit_pass(sh, pass);
    const uint32_t listed = sh.n_listed >> 16, n_exact = listed < LT_EXACT_CAP ? listed : LT_EXACT_CAP;
    // from the block's last thread down: the keyword round, which runs just before without a barrier, leaves its last,
    // partly filled turn to the first threads
    for (uint32_t x = nt - 1 - tid; x < n_exact; x += nt) {
        const uint32_t r = sh.exact[x], off = sh.tokoff[r];
        lt_emit_exact_tile(sh, a, tile_base, j0 + p.base + r, off, sh.chunk_me[off >> 7]);
    }
}

PTX_HD inline void lt_fill_tables(PtxLexTables* t, uint32_t tid, uint32_t nt) {
    for (uint32_t i = tid; i < 256; i += nt) {
        const uint32_t cc = lt_class(i);
        t->cls[i] = (uint8_t)cc;
        uint32_t f;
        switch (cc) {
        case TC_ALPHA: f = T_IDENT | FK_WORD | FK_KW; break;
        case TC_SIGIL: case TC_PCT: f = T_IDENT | FK_WORD; break;
        case TC_DOT: f = T_DOT | FK_DOT; break;
        case TC_COLON: case TC_PM: case TC_PUNCT: f = ptx_lex_single[i]; break;
        default: f = FK_EXACT; break;
        }
        t->first[i] = (uint16_t)f;
    }
    for (uint32_t i = tid; i < TS_COUNT * 16; i += nt) t->step[i] = (uint16_t)lt_step(i >> 4, i & 15u);
    for (uint32_t i = tid; i < TS_COUNT * 256; i += nt) {
        const uint32_t e = lt_step(i >> 8, lt_class(i & 255u));
        t->step2[i] = (e & 0xFFu) | (((e >> 12) * 1024u) << 8);
    }
}
