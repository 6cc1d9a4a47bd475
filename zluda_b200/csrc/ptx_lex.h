// Byte-parallel PTX lexer: per-thread pieces (host/device), used by the kernels in ptxfe.cu.
//
// Replaces the logos-generated lexer that ptx_parser drives in parse_module_checked
// (ptx_parser/src/lib.rs:431-446; token set at lib.rs:1930-2030 plus one literal per opcode and modifier).
//
// The text of a batch is one device buffer; every module starts on a CHUNK boundary.  Lexing is split so that
// no thread depends on its left neighbour:
//   1. comment/string context is a 6-state automaton over raw bytes.  Each chunk computes its transition vector
//      (all 6 start states at once, 4 bits each, packed in one 32-bit word); an exclusive scan with function
//      composition gives every chunk its incoming state.
//   2. inside code, every byte outside [A-Za-z0-9_$%.:+-] ends a token unconditionally, so a thread finds the
//      first token boundary of its chunk by walking back over at most one run of those "soft" bytes and
//      re-lexing that run; it then owns every token that starts inside its chunk (a token may run past the end).
#pragma once
#include "gen/ptx_tables.h"
#include "gen/ptx_lex_tables.h"

#ifndef PTX_NOINLINE
#ifdef __CUDACC__
#define PTX_NOINLINE __noinline__
#else
#define PTX_NOINLINE __attribute__((noinline))
#endif
#endif

#define PTX_CHUNK 128u

enum { CX_CODE = 0, CX_SLASH = 1, CX_LINE = 2, CX_BLOCK = 3, CX_STAR = 4, CX_STR = 5, CX_STATES = 6 };
#define CX_IDENTITY 0x543210u

// one token: byte offset in the batch text, length (0xFFFF = longer; re-lex to get it), kind (PtxTok)
struct PtxToken {
    uint32_t start;
    uint16_t len;
    uint16_t kind;
};

// a token as two words (start, len | kind << 16): the form kept in the decoders' token window
struct alignas(8) PtxTokenWord {
    uint32_t x, y;
};

PTX_HD inline int cx_step(int s, unsigned c) {
    switch (s) {
    case CX_CODE: return c == '/' ? CX_SLASH : c == '"' ? CX_STR : CX_CODE;
    case CX_SLASH: return c == '/' ? CX_LINE : c == '*' ? CX_BLOCK : c == '"' ? CX_STR : CX_CODE;
    case CX_LINE: return (c == '\n' || c == '\r') ? CX_CODE : CX_LINE;
    case CX_BLOCK: return c == '*' ? CX_STAR : CX_BLOCK;
    case CX_STAR: return c == '/' ? CX_CODE : c == '*' ? CX_STAR : CX_BLOCK;
    default: return c == '"' ? CX_CODE : CX_STR;
    }
}

// transition vector of one byte: nibble i = state reached from state i
PTX_HD inline uint32_t cx_byte_vector(unsigned c) {
    switch (c) {
    case '/': return (CX_SLASH) | (CX_LINE << 4) | (CX_LINE << 8) | (CX_BLOCK << 12) | (CX_CODE << 16) | (CX_STR << 20);
    case '*': return (CX_CODE) | (CX_BLOCK << 4) | (CX_LINE << 8) | (CX_STAR << 12) | (CX_STAR << 16) | (CX_STR << 20);
    case '"': return (CX_STR) | (CX_STR << 4) | (CX_LINE << 8) | (CX_BLOCK << 12) | (CX_BLOCK << 16) | (CX_CODE << 20);
    case '\n': case '\r':
        return (CX_CODE) | (CX_CODE << 4) | (CX_CODE << 8) | (CX_BLOCK << 12) | (CX_BLOCK << 16) | (CX_STR << 20);
    default: return (CX_CODE) | (CX_CODE << 4) | (CX_LINE << 8) | (CX_BLOCK << 12) | (CX_BLOCK << 16) | (CX_STR << 20);
    }
}

// (f then g): result[i] = g[f[i]]
PTX_HD inline uint32_t cx_compose(uint32_t f, uint32_t g) {
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < CX_STATES; i++) {
        uint32_t mid = (f >> (4 * i)) & 7u;
        r |= ((g >> (4 * mid)) & 7u) << (4 * i);
    }
    return r;
}
// a vector that ignores its input and always yields the state reached from CX_CODE (first chunk of a module)
PTX_HD inline uint32_t cx_restart(uint32_t f) { return (f & 7u) * 0x111111u; }

PTX_HD inline bool cx_word_has(uint32_t w, uint32_t byte) {
    uint32_t x = w ^ (0x01010101u * byte);
    return ((x - 0x01010101u) & ~x & 0x80808080u) != 0;
}
// transition vector of text[begin, end); begin is a multiple of 4.  `rd` is a text reader (see PtxGlobalReader).
// Four bytes at a time: a word without '/', '*' and '"' acts as one map (the newline map if it holds a newline, else
// the map of an ordinary byte: both are idempotent and the newline map absorbs the other, in either order), so only
// words inside or next to comments and strings are walked byte by byte, and a run of the others costs one map.
template <class R>
PTX_HD inline uint32_t cx_chunk_vector(const R& rd, uint32_t begin, uint32_t end) {
    uint32_t s0 = 0, s1 = 1, s2 = 2, s3 = 3, s4 = 4, s5 = 5;
    // a run of words without '/', '*' and '"' is applied as ONE map when it ends: the newline map if any of its words
    // holds a newline, else the map of an ordinary byte
    bool run = false, run_newline = false;
    for (uint32_t p = begin; p < end; p += 4) {
        uint32_t wd = rd.word(p);
        uint32_t nb = end - p < 4u ? end - p : 4u;
        if (nb < 4) wd &= (1u << (8 * nb)) - 1u;          // bytes past the end read as NUL: ordinary bytes
        if (cx_word_has(wd, '/') || cx_word_has(wd, '*') || cx_word_has(wd, '"')) {
            if (run) {
                const uint32_t v = run_newline ? cx_byte_vector('\n') : cx_byte_vector('a');
                s0 = (v >> (4 * s0)) & 7u; s1 = (v >> (4 * s1)) & 7u; s2 = (v >> (4 * s2)) & 7u;
                s3 = (v >> (4 * s3)) & 7u; s4 = (v >> (4 * s4)) & 7u; s5 = (v >> (4 * s5)) & 7u;
                run = run_newline = false;
            }
            for (uint32_t k = 0; k < nb; k++) {
                uint32_t v = cx_byte_vector((wd >> (8 * k)) & 0xFFu);
                s0 = (v >> (4 * s0)) & 7u; s1 = (v >> (4 * s1)) & 7u; s2 = (v >> (4 * s2)) & 7u;
                s3 = (v >> (4 * s3)) & 7u; s4 = (v >> (4 * s4)) & 7u; s5 = (v >> (4 * s5)) & 7u;
            }
        } else {
            run = true;
            run_newline |= cx_word_has(wd, '\n') || cx_word_has(wd, '\r');
        }
    }
    if (run) {
        const uint32_t v = run_newline ? cx_byte_vector('\n') : cx_byte_vector('a');
        s0 = (v >> (4 * s0)) & 7u; s1 = (v >> (4 * s1)) & 7u; s2 = (v >> (4 * s2)) & 7u;
        s3 = (v >> (4 * s3)) & 7u; s4 = (v >> (4 * s4)) & 7u; s5 = (v >> (4 * s5)) & 7u;
    }
    return s0 | (s1 << 4) | (s2 << 8) | (s3 << 12) | (s4 << 16) | (s5 << 20);
}

// ------------------------------------------------------------------------------------------------ character classes
PTX_HD inline bool lx_alpha(unsigned c) { return ((c | 32u) - 'a') < 26u; }
PTX_HD inline bool lx_digit(unsigned c) { return (c - '0') < 10u; }
PTX_HD inline bool lx_alnum(unsigned c) { return lx_alpha(c) || lx_digit(c); }
PTX_HD inline bool lx_identc(unsigned c) { return lx_alnum(c) || c == '_' || c == '$'; }
PTX_HD inline bool lx_sigil(unsigned c) { return c == '_' || c == '$' || c == '%'; }
PTX_HD inline bool lx_ws(unsigned c) { return c == ' ' || (c - 9u) < 5u; }
// bytes that can continue or join tokens; every other byte is an unconditional token boundary in code
PTX_HD inline bool lx_soft(unsigned c) { return lx_identc(c) || c == '%' || c == '.' || c == ':' || c == '+' || c == '-'; }

// ------------------------------------------------------------------------------------------------ keyword lookup
PTX_HD PTX_NOINLINE inline uint16_t lx_keyword(const uint8_t* s, uint32_t len) {
    if (len > PTX_KW_MAXLEN) return T_ERROR;
    uint32_t h = 2166136261u;
    for (uint32_t i = 0; i < len; i++) h = (h ^ s[i]) * PTX_KW_MULT;
    h = (h ^ (h >> 15)) & (PTX_KW_SIZE - 1);
    for (;;) {
        PtxKwEntry e = ptx_kw_table[h];
        if (e.kind == 0xFFFF) return T_ERROR;
        if (e.len == len) {
            bool same = true;
            for (uint32_t i = 0; i < len; i++)
                if ((uint8_t)ptx_kw_pool[e.off + i] != s[i]) { same = false; break; }
            if (same) return e.kind;
        }
        h = (h + 1) & (PTX_KW_SIZE - 1);
    }
}

// ".L1::" ".L2::" ".param::" ".shared::" literals: `p` is at the '.', `q` at the first ':' ; returns the literal's
// length and kind when the text continues with one of the known suffixes (longest match beats the DotIdent prefix)
PTX_HD PTX_NOINLINE inline uint32_t lx_colon_literal(const uint8_t* s, uint64_t p, uint64_t q, uint64_t n, uint16_t* kind) {
    uint64_t r = q + 2;
    if (r >= n) return 0;
    uint64_t e = r;
    while (e < n && e < r + 16 && lx_identc(s[e])) e++;
    // try every prefix length of the suffix run, longest first: the literal is a prefix of the text
    for (uint64_t end = e; end > r; end--) {
        uint16_t k = lx_keyword(s + p, (uint32_t)(end - p));
        if (k != T_ERROR) { *kind = k; return (uint32_t)(end - p); }
    }
    return 0;
}

// The number rules: the token at p, whose first byte is a digit.  `s` is anything that can be indexed by byte offset (a
// pointer into the text, or a reader of a copy of it).
template <class S>
PTX_HD inline uint16_t lx_number(const S& s, uint64_t p, uint64_t n, uint32_t* len) {
    const unsigned c = s[p];
    {
        if (c == '0' && p + 1 < n) {
            unsigned d = s[p + 1] | 32u;
            if (d == 'x') {
                uint64_t q = p + 2;
                while (q < n && lx_alnum(s[q])) q++;
                if (q > p + 2) { *len = (uint32_t)(q - p); return T_HEX; }
            } else if (d == 'f' || d == 'd') {
                uint64_t need = d == 'f' ? 8 : 16;
                uint64_t q = p + 2;
                while (q < n && q < p + 2 + need && lx_alnum(s[q])) q++;
                if (q == p + 2 + need) { *len = (uint32_t)(q - p); return d == 'f' ? T_F32HEX : T_F64HEX; }
            }
        }
        uint64_t q = p + 1;
        while (q < n && lx_digit(s[q])) q++;
        if (q + 1 < n && s[q] == '.' && lx_digit(s[q + 1])) {
            uint64_t r = q + 1;
            while (r < n && lx_digit(s[r])) r++;
            if (r < n && (s[r] | 32u) == 'e') {
                uint64_t e = r + 1;
                if (e < n && (s[e] == '-' || s[e] == '+')) e++;
                if (e < n && lx_digit(s[e])) {
                    while (e < n && lx_digit(s[e])) e++;
                    r = e;
                }
            }
            *len = (uint32_t)(r - p);
            return T_F64;
        }
        if (q < n && s[q] == 'U') q++;
        *len = (uint32_t)(q - p);
        return T_DECIMAL;
    }
    *len = 1;
    return T_ERROR;
}

// Longest token at p (p < n; text[p] is not whitespace, '/', or '"').  Returns its kind; *len = its length.
// T_ERROR: no rule matches here (*len = 1).
PTX_HD PTX_NOINLINE inline uint16_t lx_one(const uint8_t* s, uint64_t p, uint64_t n, uint32_t* len) {
    unsigned c = s[p];
    switch (c) {
    case ',': *len = 1; return T_COMMA;
    case ':': *len = 1; return T_COLON;
    case ';': *len = 1; return T_SEMI;
    case '@': *len = 1; return T_AT;
    case '|': *len = 1; return T_PIPE;
    case '!': *len = 1; return T_EXCL;
    case '(': *len = 1; return T_LPAREN;
    case ')': *len = 1; return T_RPAREN;
    case '[': *len = 1; return T_LBRACKET;
    case ']': *len = 1; return T_RBRACKET;
    case '{': *len = 1; return T_LBRACE;
    case '}': *len = 1; return T_RBRACE;
    case '<': *len = 1; return T_LT;
    case '>': *len = 1; return T_GT;
    case '-': *len = 1; return T_MINUS;
    case '+': *len = 1; return T_PLUS;
    case '=': *len = 1; return T_EQ;
    default: break;
    }
    if (lx_alpha(c) || lx_sigil(c)) {
        uint64_t q = p + 1;
        while (q < n && lx_identc(s[q])) q++;
        if (lx_sigil(c) && q == p + 1) { *len = 1; return T_ERROR; }
        *len = (uint32_t)(q - p);
        if (lx_alpha(c)) {
            uint16_t k = lx_keyword(s + p, (uint32_t)(q - p));
            if (k != T_ERROR) return k;
        }
        return T_IDENT;
    }
    if (c == '.') {
        unsigned d = p + 1 < n ? s[p + 1] : 0;
        if (lx_alpha(d) || lx_sigil(d)) {
            uint64_t q = p + 2;
            while (q < n && lx_identc(s[q])) q++;
            if (lx_sigil(d) && q == p + 2) { *len = 1; return T_DOT; }
            if (q + 1 < n && s[q] == ':' && s[q + 1] == ':') {
                uint16_t k;
                uint32_t l = lx_colon_literal(s, p, q, n, &k);
                if (l) { *len = l; return k; }
            }
            *len = (uint32_t)(q - p);
            uint16_t k = lx_keyword(s + p, (uint32_t)(q - p));
            return k != T_ERROR ? k : (uint16_t)T_DOTIDENT;
        }
        if (lx_digit(d)) {
            if ((d == '1' || d == '2' || d == '3') && p + 2 < n && s[p + 2] == 'd') {
                *len = 3;
                return lx_keyword(s + p, 3);
            }
            uint64_t q = p + 1;
            while (q < n && lx_digit(s[q])) q++;
            if (q < n && (s[q] | 32u) == 'e') {
                uint64_t r = q + 1;
                if (r < n && (s[r] == '-' || s[r] == '+')) r++;
                if (r < n && lx_digit(s[r])) {
                    while (r < n && lx_digit(s[r])) r++;
                    q = r;
                }
            }
            *len = (uint32_t)(q - p);
            return T_F64;
        }
        *len = 1;
        return T_DOT;
    }
    if (lx_digit(c)) return lx_number(s, p, n, len);
    *len = 1;
    return T_ERROR;
}

// ------------------------------------------------------------------------------------------------ chunk lexing
// Sink concept: void token(uint64_t start, uint32_t len, uint16_t kind); void error(uint64_t start, uint32_t len);
struct LexCountSink {
    uint32_t n_tokens = 0, n_errors = 0;
    PTX_HD void token(uint32_t, uint32_t, uint16_t) { n_tokens++; }
    PTX_HD void error(uint32_t, uint32_t) { n_errors++; }
};
// writes lexer errors only (second pass, run only when the first found some)
struct LexErrorSink {
    uint32_t* errors;      // pairs (start, len), already offset to this chunk's first error
    uint32_t n_errors = 0;
    PTX_HD void token(uint32_t, uint32_t, uint16_t) {}
    PTX_HD void error(uint32_t start, uint32_t len) {
        errors[2 * n_errors] = start;
        errors[2 * n_errors + 1] = len;
        n_errors++;
    }
};
// Token slots: every chunk owns PTX_CHUNK slots (a token is at least one byte long), so one pass can write the
// tokens before their final positions are known.
struct LexSlotSink {
    PtxToken* slots;       // this chunk's row
    uint32_t n_tokens = 0, n_errors = 0;
    PTX_HD void token(uint32_t start, uint32_t len, uint16_t kind) {
        PtxTokenWord t;       // one 8-byte store
        t.x = start;
        t.y = (len >= 0xFFFFu ? 0xFFFFu : len) | ((uint32_t)kind << 16);
        ((PtxTokenWord*)slots)[n_tokens] = t;
        n_tokens++;
    }
    PTX_HD void error(uint32_t, uint32_t) { n_errors++; }
};

// Text readers: the lockstep lexer gets bytes and table entries through one of these.  This one reads global memory;
// the CUDA backend has another that serves a shared-memory tile of the text and a shared-memory copy of the table.
struct PtxGlobalReader {
    const uint8_t* s;
    uint32_t n;      // readable bytes
    PTX_HD unsigned operator[](uint32_t p) const { return s[p]; }
    PTX_HD uint32_t word(uint32_t p) const {
        if (p + 4 <= n) return (uint32_t)s[p] | ((uint32_t)s[p + 1] << 8) | ((uint32_t)s[p + 2] << 16) | ((uint32_t)s[p + 3] << 24);
        uint32_t w = 0;
        for (uint32_t k = 0; p + k < n; k++) w |= (uint32_t)s[p + k] << (8 * k);
        return w;
    }
    // table entry of (state, byte): see ptx_lex_fused in gen/ptx_lex_tables.h
    PTX_HD uint32_t lookup(int st, unsigned c) const { return ptx_lex_fused[st * 256 + c]; }
};

PTX_HD inline bool lx_state_open(int st) {
    // a token (or a '/' whose meaning depends on the next byte) is in progress
    const uint32_t closed = (1u << LS_S0) | (1u << LS_LINE) | (1u << LS_BLOCK) | (1u << LS_STAR) | (1u << LS_SLASH_IN);
    return ((closed >> st) & 1u) == 0;
}

// Lex the tokens that START in [cs, ce) of a module occupying [ms, me).  `cx` is the comment/string context at cs.
// One byte per loop iteration, driven by ptx_lex_fused; the common cases (advance, begin a token, emit a token) are
// flag bits handled without branching on an action code, so the threads of a warp stay together.
// `g` is the text in global memory (used by the rare helpers), `tx` the reader for the byte loop.
// Offsets are 32-bit: a batch holds less than 4 GiB of text.
template <class TX, class Sink>
PTX_HD inline void lx_chunk(const TX& tx, const uint8_t* g, uint32_t ms, uint32_t me, uint32_t cs, uint32_t ce, int cx, Sink& out) {
    if (ce > me) ce = me;
    if (cs >= me) return;
    uint32_t p = cs, tstart = cs ? cs - 1 : 0, acc_pos = 0;
    uint32_t acc_kind = T_ERROR, cnt = 0, need = 0;
    int st;
    switch (cx) {
    case CX_SLASH: st = LS_SLASH_IN; break;
    case CX_LINE: st = LS_LINE; break;
    case CX_BLOCK: st = LS_BLOCK; break;
    case CX_STAR: st = LS_STAR; break;
    case CX_STR: st = LS_STR; break;
    default:
        st = LS_S0;
        if (cs > ms && lx_soft(tx[cs - 1]) && lx_soft(tx[cs])) {
            // cs may be inside a token: start at the beginning of the run of soft bytes that reaches into this chunk
            uint32_t q = cs - 1;
            while (q > ms && lx_soft(tx[q - 1])) q--;
            p = q;
        }
        break;
    }
    // Past the end of the chunk the walk goes on while a token that started inside it is open - and, for a few bytes,
    // while any token is open: a token that fails late backs up by at most 18 bytes ("0d" + 16 digits), and where it
    // backs up to a byte of this chunk the tokens from there on are this chunk's.
    while (p <= me && (p < ce || (lx_state_open(st) && (tstart >= cs || p < ce + 32u)))) {
        const unsigned c = p < me ? tx[p] : ' ';
        const uint32_t e = tx.lookup(st, c);
        const int prev = st;
        const uint32_t flags = e >> LF_FLAG_SHIFT, aux = e >> LF_AUX_SHIFT;
        st = (int)(e & LF_STATE_MASK);
        if (flags & LF_BEGIN) tstart = p;
        if (flags & LF_EMIT) {
            const uint32_t s0 = (aux & LF_SELF) ? p : tstart;
            if (s0 >= cs) out.token(s0, p + (aux & LF_INCL) - s0, (aux & LF_SELF) ? ptx_lex_single[c] : ptx_lex_end_kind[prev]);
        }
        if (flags & LF_RARE) {
            switch (aux & 0xFu) {
            case LA_ACCEPT: acc_pos = p; acc_kind = ptx_lex_end_kind[prev]; p++; break;
            case LA_BACKUP:
                if (prev != LS_SLASH_IN) {
                    if (tstart >= cs) out.token(tstart, acc_pos - tstart, (uint16_t)acc_kind);
                    p = acc_pos;
                }
                break;
            case LA_ERR_HERE:
                if (p >= cs) out.error(p, 1);
                p++;
                break;
            case LA_ERR_TOKEN:
            case LA_ERR_SLASH:
                if (tstart >= cs) out.error(tstart, 1);
                break;
            case LA_COUNT:
                if (++cnt == need) {
                    if (tstart >= cs) out.token(tstart, p + 1 - tstart, need == 8 ? T_F32HEX : T_F64HEX);
                    st = LS_S0;
                }
                p++;
                break;
            case LA_BEGIN_HF32: acc_pos = p; acc_kind = T_DECIMAL; cnt = 0; need = 8; p++; break;
            case LA_BEGIN_HF64: acc_pos = p; acc_kind = T_DECIMAL; cnt = 0; need = 16; p++; break;
            case LA_COLON_CHECK: {
                uint16_t k = T_DOTIDENT;
                uint32_t l = 0;
                if (p + 1 < me && tx[p + 1] == ':') l = lx_colon_literal(g, tstart, p, me, &k);
                if (l) {
                    // a literal with "::" inside: its kind is final
                    if (tstart >= cs) out.token(tstart, l, k);
                    p = tstart + l;
                } else if (tstart >= cs) {
                    out.token(tstart, p - tstart, T_DOTIDENT);
                }
                break;
            }
            case LA_REWIND_DOT:
                if (tstart >= cs) out.token(tstart, 1, T_DOT);
                p = tstart + 1;
                break;
            default:   // LA_DIM: ".1d" ".2d" ".3d" are literals; an upper-case D ends the F64 in front of it
                if (c == 'd') {
                    unsigned digit = tx[tstart + 1];
                    if (tstart >= cs) out.token(tstart, 3, digit == '1' ? T_MOD_1d : digit == '2' ? T_MOD_2d : T_MOD_3d);
                    p++;
                } else if (tstart >= cs) {
                    out.token(tstart, p - tstart, T_F64);
                }
                break;
            }
        }
        p += flags & LF_ADV;
    }
    if (p > me || (p == me && ce == me)) {
        // this thread saw the end of the module
        if (st == LS_STR && tstart >= cs) out.error(tstart, me - tstart);
        if ((st == LS_BLOCK || st == LS_STAR) && ce == me) out.error(me, 0);
    }
}

// The same lookup through the table keyed by a word's first eight bytes.  Reads up to 11 bytes past `start`: the text
// buffer must have that much slack (the pipeline's buffers do; a caller's buffer may not: use lx_keyword there).
PTX_HD inline uint16_t lx_keyword8(const uint8_t* g, uint32_t start, uint32_t len) {
    if (len > PTX_KW_MAXLEN) return T_ERROR;
    const uint8_t* a = g + start;
    const uint32_t sh = (uint32_t)((uintptr_t)a & 3u) * 8u;
    const uint32_t* w = (const uint32_t*)(a - ((uintptr_t)a & 3u));
    uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    uint32_t lo = sh ? (w0 >> sh) | (w1 << (32u - sh)) : w0;
    uint32_t hi = sh ? (w1 >> sh) | (w2 << (32u - sh)) : w1;
    if (len < 4) { lo &= (1u << (8u * len)) - 1u; hi = 0; }
    else if (len < 8) hi &= (1u << (8u * (len - 4u))) - 1u;
    uint32_t h = (lo ^ hi) * 0x9E3779B1u;
    h ^= len * 0x85EBCA6Bu;
    h ^= h >> 15;
    h *= 0x2C1B3C6Du;
    h ^= h >> 12;
    h &= PTX_KW8_SIZE - 1;
    for (;;) {
        const PtxKw8Entry e = ptx_kw8_table[h];
        if (e.kind == 0xFFFF) return T_ERROR;
        if (e.lo == lo && e.hi == hi && e.len == len) {
            bool same = true;
            for (uint32_t i = 8; i < len; i++)
                if ((uint8_t)ptx_kw_pool[e.off + i] != a[i]) { same = false; break; }
            if (same) return e.kind;
        }
        h = (h + 1) & (PTX_KW8_SIZE - 1);
    }
}
PTX_HD inline uint16_t lx_classify8(const uint8_t* g, uint32_t start, uint32_t len, uint16_t kind) {
    if (kind == T_IDENT) {
        if (!lx_alpha(g[start])) return kind;
    } else if (kind != T_DOTIDENT) {
        return kind;
    }
    uint16_t k = lx_keyword8(g, start, len);
    return k == T_ERROR ? kind : k;
}
// identifiers and dot-identifiers that spell a keyword (opcode, modifier, directive word): one thread per token
PTX_HD inline uint16_t lx_classify(const uint8_t* g, uint32_t start, uint32_t len, uint16_t kind) {
    if (kind == T_IDENT) {
        if (!lx_alpha(g[start])) return kind;
    } else if (kind != T_DOTIDENT) {
        return kind;
    }
    uint16_t k = lx_keyword(g + start, len);
    return k == T_ERROR ? kind : k;
}

// ------------------------------------------------------------------------------------------------ numeric literals
// What the parser does with a numeric literal depends on its digits only through a few facts: whether it carries the
// 'U' suffix, whether it converts at all, and which of the limits the grammar applies it exceeds (i32 for address
// offsets, u32 for counts, i63 / 2^63 for the S64-or-U64 choice and for negated literals; ptx_parser/src/lib.rs:263-350).
// Those facts are the literal's CODE.  Two statements whose tokens have the same kinds and the same codes take the same
// path through the decoder and differ only in the converted values.
#define PTX_LC_UNS 1u        // 'U' suffix
#define PTX_LC_ERR 2u        // does not convert to 64 bits: invalid digit for its radix, overflow, or no digits
#define PTX_LC_GT_I32 4u     // magnitude > 0x7FFFFFFF
#define PTX_LC_GT_U32 8u     // magnitude > 0xFFFFFFFF
#define PTX_LC_GT_I63 16u    // magnitude > 2^63 - 1
#define PTX_LC_GT_2P63 32u   // magnitude > 2^63
#define PTX_LC_LONG 64u      // a token of 65535 bytes or more: not looked at
PTX_HD inline bool ptx_is_numeric_kind(uint16_t k) {
    static_assert(T_F32HEX == 18 && T_DECIMAL == 22, "the five numeric literal kinds are consecutive");
    return (uint32_t)(k - T_F32HEX) <= (uint32_t)(T_DECIMAL - T_F32HEX);
}
// does v * radix + d exceed 64 bits (no division: the radix is not known at compile time)
PTX_HD inline bool ptx_mul_add_overflows(uint64_t v, uint32_t radix, uint32_t d) {
#ifdef __CUDA_ARCH__
    const uint64_t lo = v * radix;
    return __umul64hi(v, (uint64_t)radix) != 0 || lo + d < lo;
#else
    uint64_t lo, sum;
    return __builtin_mul_overflow(v, (uint64_t)radix, &lo) || __builtin_add_overflow(lo, (uint64_t)d, &sum);
#endif
}
// Magnitude (DECIMAL, HEX: radix 8 / 10 / 16 by prefix, 'U' stripped) or bit pattern (F32HEX, F64HEX) of a literal of
// `len` < 65535 bytes, and its code.  T_F64 (decimal floating point) has code 0 and is converted elsewhere.
template <class S>
PTX_HD inline uint32_t ptx_literal_scan(const S& s, uint32_t len, uint16_t kind, uint64_t* mag) {
    *mag = 0;
    if (kind == T_F64) return 0;
    uint32_t code = 0, i = 0, radix = 16;
    if (kind == T_DECIMAL || kind == T_HEX) {
        if (s[len - 1] == 'U') { code |= PTX_LC_UNS; len--; }
        if (kind == T_HEX) i = 2;
        else radix = s[0] == '0' ? 8 : 10;
    } else {
        i = 2;
    }
    if (i >= len) return code | PTX_LC_ERR;
    uint64_t v = 0;
    // 16 hexadecimal, 19 decimal or 21 octal digits cannot overflow 64 bits; longer ones are checked digit by digit
    const bool checked = len - i > (radix == 16 ? 16u : radix == 10 ? 19u : 21u);
    for (; i < len; i++) {
        uint32_t ch = s[i], d;
        if (ch - '0' < 10u) d = ch - '0';
        else if ((ch | 32u) - 'a' < 26u) d = (ch | 32u) - 'a' + 10;
        else return code | PTX_LC_ERR;
        if (d >= radix) return code | PTX_LC_ERR;
        if (checked && ptx_mul_add_overflows(v, radix, d)) return code | PTX_LC_ERR;
        v = v * radix + d;
    }
    *mag = v;
    if (kind == T_DECIMAL || kind == T_HEX) {
        if (v > 0x7FFFFFFFull) code |= PTX_LC_GT_I32;
        if (v > 0xFFFFFFFFull) code |= PTX_LC_GT_U32;
        if (v > 0x7FFFFFFFFFFFFFFFull) code |= PTX_LC_GT_I63;
        if (v > 0x8000000000000000ull) code |= PTX_LC_GT_2P63;
    }
    return code;
}
// the entry of the per-token side array `kinds`: kind in the low 9 bits; above them the literal code of a numeric
// literal, min(length, 127) of every other token
PTX_HD inline uint16_t ptx_kind_entry(const uint8_t* text, uint32_t start, uint32_t len, uint16_t kind) {
    uint32_t aux;
    if (ptx_is_numeric_kind(kind)) {
        uint64_t mag;
        aux = len >= 0xFFFFu ? PTX_LC_LONG : ptx_literal_scan(text + start, len, kind, &mag);
    } else {
        aux = len < 127u ? len : 127u;
    }
    return (uint16_t)(kind | (aux << 9));
}

PTX_HD inline uint32_t ptx_token_len(const uint8_t* s, const PtxToken& t, uint64_t me) {
    if (t.len != 0xFFFF) return t.len;
    if (t.kind == T_STRING) {
        uint64_t q = (uint64_t)t.start + 1;
        while (q < me && s[q] != '"') q++;
        return (uint32_t)(q + 1 - t.start);
    }
    uint32_t l;
    lx_one(s, t.start, me, &l);
    return l;
}
