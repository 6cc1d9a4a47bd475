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
//   [A-Za-z0-9_$]) - except around numbers, lone sigils and the few literals with "::" inside.  So every thread
//   classifies 16 bytes through a 256-entry class table and a (class of p, class of c) table, and the exceptions are
//   collected as TRIGGERS and settled afterwards, one thread per trigger, by lexing forward from a known token start
//   with the exact per-token rules (lx_one):
//     T1  a digit that does not continue a word: the run of "soft" bytes around it (word characters and % . : + -)
//         can hold one number (1.5e-3) or several tokens (12Ux, 0f3F800000z);
//     T3  "::": .shared::cta and its like are single tokens, and what follows them starts a new one;
//         a run with a T1 or T3 in it is lexed from its first byte by the thread of its first trigger;
//     T2  a sigil (_ $ %) that starts a word and is followed by no word character: a lexer error, not a token.
//   Chunks that contain a comment or string character (/ * ") or start inside a comment or string take the proven
//   byte-serial walk (lx_chunk), one thread per chunk.  Every writer of the second round sets bits to the true lexing,
//   so where two of them meet they agree.
// Step 2, lex_emit: one thread per token (the set bits, enumerated per 32-byte window) finds the token's length and
//   kind - punctuation and sigil-led words at once, words that may spell a keyword through the 8-byte keyword table,
//   numbers through lx_one - and writes the 8-byte token and the kinds entry to their final place
//   (chunk base from the scanned per-chunk counts + rank inside the chunk).
#pragma once
#include "ptx_lex.h"

#define LT_CHUNKS 64u
#define LT_BYTES (LT_CHUNKS * PTX_CHUNK)
#define LT_PIECES (LT_BYTES / 16u)
#define LT_WORDS (LT_BYTES / 32u)
#define LT_TRIG_CAP 6144u          // triggers per tile; a tile with more is lexed chunk by chunk by the serial walk
#define LT_BACK_CAP 2048u          // longest look-back over a run of soft bytes; beyond it the module is lexed by one thread
#define LT_BATCH 2048u             // tokens classified per round of the emit step

enum { TC_WS = 0, TC_ALPHA = 1, TC_DIGIT = 2, TC_SIGIL = 3, TC_PCT = 4, TC_DOT = 5, TC_COLON = 6, TC_PM = 7, TC_PUNCT = 8, TC_SPECIAL = 9, TC_BAD = 10 };
enum { LP_START = 1, LP_ERR = 2, LP_T1 = 4, LP_T2 = 8, LP_T3 = 16, LP_SPECIAL = 32 };

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
// what byte class cc does behind byte class pc (TC_WS stands for "nothing in front": start of a module)
PTX_HD inline uint32_t lt_pair(uint32_t pc, uint32_t cc) {
    const bool continues = lt_word(pc) || pc == TC_PCT || pc == TC_DOT;     // a word character here continues a word
    uint32_t e = 0;
    switch (cc) {
    case TC_ALPHA: case TC_SIGIL: if (!continues) e |= LP_START; break;
    case TC_DIGIT:
        if (!continues) e |= LP_START;
        if (!(lt_word(pc) || pc == TC_PCT)) e |= LP_T1;
        break;
    case TC_PCT: if (pc != TC_DOT) e |= LP_START; break;
    case TC_DOT: case TC_PM: case TC_PUNCT: e |= LP_START; break;
    case TC_COLON:
        e |= LP_START;
        if (pc == TC_COLON) e |= LP_T3;
        break;
    case TC_SPECIAL: e |= LP_SPECIAL; break;
    case TC_BAD: e |= LP_ERR; break;
    default: break;
    }
    if (!lt_word(cc) && (pc == TC_SIGIL || pc == TC_PCT)) e |= LP_T2;      // the sigil in front of this byte may stand alone
    return e;
}

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
    uint32_t* start_bits;       // [n_chunks * 4]: bit b of word w = a token starts at text byte 32 w + b
    PtxPair* cnt;               // [n_chunks + 1]: mark step: tokens / errors of chunk c at [c + 1]; emit step: their exclusive prefix
    uint32_t* mod_flag;         // [n_modules] 1 = a run of soft bytes outgrew the look-back: the module is lexed by one thread
    PtxToken* tokens;           // emit step
    uint16_t* kinds;
};

// working memory of one tile (shared memory on the GPU)
struct PtxLexMarkShared {
    uint8_t cls[256];
    uint8_t pair[256];
    uint32_t start[LT_WORDS], err[LT_WORDS];
    uint32_t chunk_ms[LT_CHUNKS], chunk_me[LT_CHUNKS];
    uint8_t chunk_cx[LT_CHUNKS], chunk_special[LT_CHUNKS];
    uint32_t chunk_errs[LT_CHUNKS];      // errors of a chunk lexed by the serial walk
    uint32_t n_trig;
    uint32_t trig[LT_TRIG_CAP];          // position in the tile (0 .. LT_BYTES: a trigger may sit on the first byte of the next tile) | kind << 16
};

// ---- mark step, phase 0: tables, chunk geometry
PTX_HD inline void lt_mark_init(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    for (uint32_t i = tid; i < 256; i += nt) {
        sh.cls[i] = (uint8_t)lt_class(i);
        sh.pair[i] = (uint8_t)lt_pair(i >> 4, i & 15u);
    }
    for (uint32_t i = tid; i < LT_WORDS; i += nt) sh.start[i] = sh.err[i] = 0;
    for (uint32_t k = tid; k < LT_CHUNKS; k += nt) {
        uint32_t c = tile * LT_CHUNKS + k;
        sh.chunk_special[k] = 0;
        sh.chunk_errs[k] = 0;
        if (c >= a.n_chunks) { sh.chunk_ms[k] = sh.chunk_me[k] = 0; sh.chunk_cx[k] = CX_CODE; continue; }
        uint32_t ms, me;
        bool first;
        a.info.locate(c, ms, me, first);
        sh.chunk_ms[k] = ms;
        sh.chunk_me[k] = me;
        int cx = first ? CX_CODE : (int)(a.vec[c - 1] & 7u);
        sh.chunk_cx[k] = (uint8_t)cx;
        if (cx != CX_CODE) sh.chunk_special[k] = 1;
    }
    if (tid == 0) sh.n_trig = 0;
}

// ---- phase 1: 16 bytes per thread through the two tables
PTX_HD inline void lt_mark_simple(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    for (uint32_t piece = tid; piece < LT_PIECES; piece += nt) {
        const uint32_t k = piece >> 3, c = tile * LT_CHUNKS + k;
        if (c >= a.n_chunks) continue;
        const uint32_t ms = sh.chunk_ms[k], me = sh.chunk_me[k];
        const uint32_t pos0 = c * PTX_CHUNK + (piece & 7u) * 16u;
        if (pos0 >= me) continue;
        const uint32_t* w = (const uint32_t*)(a.text + pos0);
        uint32_t words[4] = {w[0], w[1], w[2], w[3]};
        uint32_t pc = pos0 > ms ? sh.cls[a.text[pos0 - 1]] : (uint32_t)TC_WS;
        uint32_t n = me - pos0 < 16u ? me - pos0 : 16u;
        uint32_t acc = 0, any = 0;
        for (uint32_t i = 0; i < n; i++) {
            const uint32_t ch = (words[i >> 2] >> (8u * (i & 3u))) & 0xFFu;
            const uint32_t cc = sh.cls[ch];
            const uint32_t e = sh.pair[(pc << 4) | cc];
            acc |= (e & 3u) << (2u * i);
            any |= e;
            if (e & (LP_T1 | LP_T2 | LP_T3)) {
                uint32_t slot = LT_ATOMIC_ADD(&sh.n_trig, 1u);
                if (slot < LT_TRIG_CAP) sh.trig[slot] = (piece * 16u + i) | ((e & (LP_T1 | LP_T2 | LP_T3)) << 16);
            }
            pc = cc;
        }
        // the triggers that look one byte back also fire behind the last byte of the tile and behind the last byte of
        // the module (where nothing follows)
        if ((piece == LT_PIECES - 1 && n == 16 && pos0 + 16 < me) || pos0 + n == me) {
            const uint32_t e = sh.pair[(pc << 4) | (pos0 + n == me ? (uint32_t)TC_WS : (uint32_t)sh.cls[a.text[pos0 + 16]])];
            if (e & (LP_T2 | LP_T3)) {
                uint32_t slot = LT_ATOMIC_ADD(&sh.n_trig, 1u);
                if (slot < LT_TRIG_CAP) sh.trig[slot] = (piece * 16u + n) | ((e & (LP_T2 | LP_T3)) << 16);
            }
        }
        // even bits of acc: starts, odd bits: errors
        uint32_t s = acc & 0x55555555u, r = (acc >> 1) & 0x55555555u;
        s = (s | (s >> 1)) & 0x33333333u; s = (s | (s >> 2)) & 0x0F0F0F0Fu; s = (s | (s >> 4)) & 0x00FF00FFu; s = (s | (s >> 8)) & 0xFFFFu;
        r = (r | (r >> 1)) & 0x33333333u; r = (r | (r >> 2)) & 0x0F0F0F0Fu; r = (r | (r >> 4)) & 0x00FF00FFu; r = (r | (r >> 8)) & 0xFFFFu;
        const uint32_t sft = 16u * (piece & 1u);
        if (s) LT_ATOMIC_OR(&sh.start[piece >> 1], s << sft);
        if (r) LT_ATOMIC_OR(&sh.err[piece >> 1], r << sft);
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
// a digit that does not continue a word, or the first colon of "::"
PTX_HD inline bool lt_is_trigger(const uint8_t* text, uint32_t j, uint32_t ms, uint32_t me) {
    const unsigned c = text[j];
    if (c == ':') return j + 1 < me && text[j + 1] == ':';
    if (!lx_digit(c)) return false;
    if (j == ms) return true;
    const unsigned p = text[j - 1];
    return !(lx_identc(p) || p == '%');
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
        if (sh.chunk_cx[k] == CX_CODE && cs > ms && lx_soft(a.text[cs - 1]) && lx_soft(a.text[cs])) {
            uint32_t q = cs - 1;
            while (q > ms && cs - q <= LT_BACK_CAP && lx_soft(a.text[q - 1])) q--;
            if (cs - q > LT_BACK_CAP) { a.mod_flag[ptx_upper_bound_u32(a.info.mcb, a.info.n_modules, c) - 1] = 1; continue; }
        }
        LexMarkSink sink;
        sink.sh = &sh;
        sink.tile_base = tile_base;
        lx_chunk(PtxGlobalReader{a.text, me}, a.text, ms, me, cs, cs + PTX_CHUNK, (int)sh.chunk_cx[k], sink);
        sh.chunk_errs[k] = sink.n_errors;
        // the bytes behind the last token that belong to the same run of soft bytes, in the chunks that follow
        if (sink.last_end >= cs + PTX_CHUNK) lt_chain(sh, a.text, tile_base, sink.last_end, me);
    }
}

// ---- phase 2b: one thread per trigger, and one for the run of soft bytes that enters the tile
PTX_HD inline void lt_mark_triggers(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    const uint32_t tile_base = tile * LT_BYTES;
    const uint32_t n_trig = sh.n_trig > LT_TRIG_CAP ? 0u : sh.n_trig;
    for (uint32_t t = tid; t < n_trig + 1; t += nt) {
        if (t == n_trig) {
            // a run of soft bytes that begins in front of the tile may hold a number or a "::" literal: lex it from its start
            const uint32_t c = tile * LT_CHUNKS;
            if (c >= a.n_chunks || sh.chunk_special[0]) continue;
            const uint32_t ms = sh.chunk_ms[0], me = sh.chunk_me[0];
            if (tile_base >= me || tile_base <= ms || !lx_soft(a.text[tile_base]) || !lx_soft(a.text[tile_base - 1])) continue;
            uint32_t q = tile_base - 1;
            bool any = false;
            while (q > ms && tile_base - q <= LT_BACK_CAP && lx_soft(a.text[q - 1])) q--;
            if (tile_base - q > LT_BACK_CAP) { a.mod_flag[ptx_upper_bound_u32(a.info.mcb, a.info.n_modules, c) - 1] = 1; continue; }
            for (uint32_t j = q; j < tile_base && !any; j++) any = lt_is_trigger(a.text, j, ms, me);
            if (any) lt_chain(sh, a.text, tile_base, q, me);
            continue;
        }
        const uint32_t off = sh.trig[t] & 0xFFFFu, kind = sh.trig[t] >> 16;
        const uint32_t pos = tile_base + off;
        // T1 sits on its digit; T2 and T3 sit one byte behind the sigil / the first colon they are about
        const uint32_t at = (kind & LP_T1) ? off : (off ? off - 1 : 0u);
        const uint32_t k = at >> 7;
        if (sh.chunk_special[k]) continue;        // lexed by the serial walk
        const uint32_t ms = sh.chunk_ms[k], me = sh.chunk_me[k];
        if (kind & (LP_T1 | LP_T3)) {
            // A run of soft bytes with a number or a "::" in it is lexed from its first byte, which is a token start, by
            // the thread of its first trigger (T3 sits one byte behind the first colon).
            const uint32_t own = (kind & LP_T1) ? pos : pos - 1;
            uint32_t j = own;
            bool earlier = false;
            while (j > ms && own - j <= LT_BACK_CAP && lx_soft(a.text[j - 1])) {
                j--;
                if (lt_is_trigger(a.text, j, ms, me)) { earlier = true; break; }
            }
            if (own - j > LT_BACK_CAP) { a.mod_flag[ptx_upper_bound_u32(a.info.mcb, a.info.n_modules, tile * LT_CHUNKS + k) - 1] = 1; continue; }
            if (!earlier) lt_chain(sh, a.text, tile_base, j, me);
        }
        if (kind & LP_T2) {
            // the sigil at pos - 1, followed by no word character: alone unless it continues a word
            const uint32_t s = pos - 1;
            const unsigned ch = a.text[s];
            bool alone = ch == '%' || s == ms;
            if (!alone) {
                unsigned p = a.text[s - 1];
                alone = !(lx_identc(p) || p == '%');
            }
            if (alone) lt_truth(sh, tile_base, s, 1, true);
        }
    }
}

// ---- phase 3: counts and the bit map
PTX_HD inline void lt_mark_finish(PtxLexMarkShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    for (uint32_t k = tid; k < LT_CHUNKS; k += nt) {
        const uint32_t c = tile * LT_CHUNKS + k;
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
        p.b = sh.chunk_special[k] ? sh.chunk_errs[k] : nerr;
        a.cnt[c + 1] = p;
        if (c == 0) { PtxPair z; z.a = z.b = 0; a.cnt[0] = z; }
    }
    for (uint32_t w = tid; w < LT_WORDS; w += nt)
        if (tile * LT_CHUNKS + (w >> 2) < a.n_chunks) a.start_bits[(size_t)tile * LT_WORDS + w] = sh.start[w];
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
struct PtxLexEmitShared {
    uint8_t cls[256];
    uint32_t bits[LT_WORDS];
    uint32_t chunk_me[LT_CHUNKS], chunk_rank[LT_CHUNKS + 1];     // rank of the chunk's first token inside the tile
    uint16_t list[LT_BYTES];            // tile offset of every token, in order
    uint16_t len[LT_BATCH];             // length found by the first round (capped), for the second
    uint16_t kw[LT_BATCH], num[LT_BATCH];
    uint32_t n_kw, n_num;
    uint32_t text[LT_BYTES / 4 + 4];
};

PTX_HD inline void lt_emit_init(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t tid, uint32_t nt) {
    for (uint32_t i = tid; i < 256; i += nt) sh.cls[i] = (uint8_t)lt_class(i);
    const uint32_t c0 = tile * LT_CHUNKS;
    for (uint32_t w = tid; w < LT_WORDS; w += nt) sh.bits[w] = c0 + (w >> 2) < a.n_chunks ? a.start_bits[(size_t)tile * LT_WORDS + w] : 0u;
    for (uint32_t k = tid; k <= LT_CHUNKS; k += nt) {
        uint32_t c = c0 + k < a.n_chunks ? c0 + k : a.n_chunks;
        sh.chunk_rank[k] = a.cnt[c].a - a.cnt[c0].a;
        if (k < LT_CHUNKS) {
            uint32_t ms = 0, me = 0;
            bool first;
            if (c0 + k < a.n_chunks) a.info.locate(c0 + k, ms, me, first);
            sh.chunk_me[k] = me;
        }
    }
    const uint32_t n_words = (c0 + LT_CHUNKS <= a.n_chunks ? LT_CHUNKS : a.n_chunks - c0) * (PTX_CHUNK / 4);
    const uint32_t* src = (const uint32_t*)(a.text + (size_t)tile * LT_BYTES);
    for (uint32_t i = tid; i < LT_BYTES / 4 + 4; i += nt) sh.text[i] = i < n_words ? src[i] : 0u;
    if (tid == 0) sh.n_kw = sh.n_num = 0;
}
// positions of the set bits, window by window
PTX_HD inline void lt_emit_list(PtxLexEmitShared& sh, uint32_t tid, uint32_t nt) {
    for (uint32_t w = tid; w < LT_WORDS; w += nt) {
        uint32_t r = sh.chunk_rank[w >> 2];
        for (uint32_t v = w & ~3u; v < w; v++) {
#ifdef __CUDA_ARCH__
            r += __popc(sh.bits[v]);
#else
            r += (uint32_t)__builtin_popcount(sh.bits[v]);
#endif
        }
        uint32_t b = sh.bits[w];
        while (b) {
#ifdef __CUDA_ARCH__
            uint32_t i = __ffs(b) - 1;
#else
            uint32_t i = (uint32_t)__builtin_ctz(b);
#endif
            b &= b - 1;
            sh.list[r++] = (uint16_t)(w * 32u + i);
        }
    }
}
struct PtxLexEmitReader {      // text of the tile from shared memory, everything else from global memory
    const PtxLexEmitShared& sh;
    const uint8_t* g;
    uint32_t base;
    PTX_HD unsigned operator[](uint32_t p) const {
        uint32_t o = p - base;
        if (o < LT_BYTES) return ((const uint8_t*)sh.text)[o];
        return g[p];
    }
};
PTX_HD inline void lt_put_token(const PtxLexTileArgs& a, uint32_t j, uint32_t start, uint32_t len, uint16_t kind) {
    PtxTokenWord t;
    t.x = start;
    t.y = (len >= 0xFFFFu ? 0xFFFFu : len) | ((uint32_t)kind << 16);
    ((PtxTokenWord*)a.tokens)[j] = t;
    a.kinds[j] = ptx_kind_entry(a.text, start, len, kind);
}
// first round over the tokens [t0, t0 + LT_BATCH) of the tile: lengths; punctuation and sigil-led words are finished
PTX_HD inline void lt_emit_first(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t t0, uint32_t tid, uint32_t nt) {
    const uint32_t n_tok = sh.chunk_rank[LT_CHUNKS], tile_base = tile * LT_BYTES;
    const uint32_t j0 = a.cnt[tile * LT_CHUNKS].a;
    const PtxLexEmitReader rd{sh, a.text, tile_base};
    for (uint32_t i = tid; i < LT_BATCH && t0 + i < n_tok; i += nt) {
        const uint32_t off = sh.list[t0 + i], pos = tile_base + off, me = sh.chunk_me[off >> 7];
        const unsigned c = rd[pos];
        const uint32_t cc = sh.cls[c];
        uint32_t q = pos + 1;
        if (cc == TC_PUNCT || cc == TC_PM || cc == TC_COLON) {
            lt_put_token(a, j0 + t0 + i, pos, 1, ptx_lex_single[c]);
            continue;
        }
        if (cc == TC_ALPHA || cc == TC_SIGIL || cc == TC_PCT) {
            while (q < me && lx_identc(rd[q])) q++;
            if (cc != TC_ALPHA) { lt_put_token(a, j0 + t0 + i, pos, q - pos, T_IDENT); continue; }
            sh.len[i] = (uint16_t)(q - pos < 0xFFFFu ? q - pos : 0xFFFFu);
            sh.kw[LT_ATOMIC_ADD(&sh.n_kw, 1u)] = (uint16_t)i;
            continue;
        }
        if (cc == TC_DOT) {
            const unsigned d = q < me ? rd[q] : 0;
            const uint32_t dc = sh.cls[d];
            if (dc == TC_ALPHA || dc == TC_SIGIL || dc == TC_PCT) {
                q++;
                while (q < me && lx_identc(rd[q])) q++;
                const bool colons = q + 1 < me && rd[q] == ':' && rd[q + 1] == ':';
                if ((dc != TC_ALPHA && q == pos + 2) || colons) {
                    sh.num[LT_ATOMIC_ADD(&sh.n_num, 1u)] = (uint16_t)i;      // a lone sigil behind the dot, or a "::" literal: exact rules
                } else {
                    sh.len[i] = (uint16_t)(q - pos < 0xFFFFu ? q - pos : 0xFFFFu);
                    sh.kw[LT_ATOMIC_ADD(&sh.n_kw, 1u)] = (uint16_t)i;
                }
                continue;
            }
            if (dc != TC_DIGIT) { lt_put_token(a, j0 + t0 + i, pos, 1, T_DOT); continue; }
        }
        if (c == '"') {
            while (q < me && rd[q] != '"') q++;
            lt_put_token(a, j0 + t0 + i, pos, q + 1 - pos, T_STRING);
            continue;
        }
        sh.num[LT_ATOMIC_ADD(&sh.n_num, 1u)] = (uint16_t)i;      // numbers and whatever else: the exact per-token rules
    }
}
// second round: keyword lookups and numbers, each with full warps
PTX_HD inline void lt_emit_second(PtxLexEmitShared& sh, const PtxLexTileArgs& a, uint32_t tile, uint32_t t0, uint32_t tid, uint32_t nt) {
    const uint32_t tile_base = tile * LT_BYTES, j0 = a.cnt[tile * LT_CHUNKS].a;
    const uint32_t n_kw = sh.n_kw, n_num = sh.n_num;
    for (uint32_t x = tid; x < n_kw + n_num; x += nt) {
        if (x < n_kw) {
            const uint32_t i = sh.kw[x], pos = tile_base + sh.list[t0 + i];
            uint32_t len = sh.len[i];
            const bool dot = ((const uint8_t*)sh.text)[pos - tile_base] == '.';
            if (len == 0xFFFFu) {       // re-measure a very long word
                uint32_t me = sh.chunk_me[(pos - tile_base) >> 7], q = pos + 1;
                while (q < me && lx_identc(a.text[q])) q++;
                len = q - pos;
            }
            uint16_t k = lx_keyword8(a.text, pos, len);
            if (k == T_ERROR) k = dot ? (uint16_t)T_DOTIDENT : (uint16_t)T_IDENT;
            lt_put_token(a, j0 + t0 + i, pos, len, k);
        } else {
            const uint32_t i = sh.num[x - n_kw], off = sh.list[t0 + i], pos = tile_base + off;
            uint32_t len;
            uint16_t k = lx_one(a.text, pos, sh.chunk_me[off >> 7], &len);
            lt_put_token(a, j0 + t0 + i, pos, len, k);
        }
    }
}
PTX_HD inline void lt_emit_reset(PtxLexEmitShared& sh, uint32_t tid) {
    if (tid == 0) sh.n_kw = sh.n_num = 0;
}
