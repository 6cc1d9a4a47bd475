// Stage B in one pass over the token kinds: scope depth (a segmented scan that restarts at every module), the decision
// "a parse unit starts at this token", the numbering of the unit starts, and the unit table (start token, depth in
// front of it, first unit of every module, scope depth behind every module's last token).
//
// Depth.  '{' that opens a scope counts +1, '}' that closes one counts -1 but never below 0: at the top level the
// reference's directive recovery skips a '}' like any other token (lib.rs:590-607), so a stray '}' in a function body
// ends the function early and must not throw off everything behind it.  "Add, but not below a floor" composes:
// f(x) = max(x + a, b) with (a2, b2) after (a1, b1) = (a1 + a2, max(b1 + a2, b2)); that pair is what the scan carries
// (PtxSeg3: scope = a, paren = b, flag = a module begins inside, everything in front is forgotten), and the depth
// behind a prefix P of a module is max(P.scope, P.paren).
//
// Unit starts, for a token that does not begin a module:
//   at depth 0: a directive keyword that does not continue a run of linking keywords and is not the state space of a
//     `.ptr` parameter (lib.rs:973), and the token behind a scope-closing '}' (what follows a function; anything but a
//     directive keyword there is skipped up to the next one by the directive's recovery);
//   inside a scope: the token behind ';', ':' or a scope brace, and a scope brace itself.
//
// The work is cut into tiles of SX_TILE tokens; a tile is SX_THREADS threads with SX_ITEMS consecutive tokens each.
// Per tile: thread aggregates -> ordered scan over the tile's threads -> the prefix of the tiles before (the backend's
// business: a look-back chain on the device, a running value in the host emulation) -> the start decisions -> their
// count, scanned the same way -> the unit table rows.  The functions here are the per-thread bodies of those steps.
#pragma once
// (included by ptxfe_pipeline.h after the token kinds, PtxSeg3 and the brace rules are defined)

constexpr uint32_t SX_THREADS = 256, SX_ITEMS = 16, SX_TILE = SX_THREADS * SX_ITEMS;

struct PtxStructArgs {
    const uint16_t* kinds;        // [n_tokens + 32] readable
    uint32_t n_tokens;
    const uint32_t* mtb;          // [n_modules + 1] first token of every module (empty modules repeat the next begin)
    uint32_t n_modules;
    int32_t* mod_final_scope;     // [n_modules] out: scope depth behind the module's last token
    uint32_t* ustart;             // out: start token of unit u
    uint32_t* udepth;             // out: scope depth in front of unit u, bit 31 = first unit of a module
    uint32_t* mub;                // out: first unit of module m (modules with tokens only)
    PtxCounters* counters;        // out: n_units
};

// the scan's operator and what a prefix says about the depth
struct SegDepthOp {
    PTX_HD PtxSeg3 operator()(PtxSeg3 x, PtxSeg3 y) const {
        if (y.flag) return y;
        PtxSeg3 r;
        r.scope = x.scope + y.scope;
        r.paren = x.paren + y.scope > y.paren ? x.paren + y.scope : y.paren;
        r.flag = x.flag;
        return r;
    }
};
PTX_HD inline int32_t sx_depth(PtxSeg3 p) { return p.scope > p.paren ? p.scope : p.paren; }
// one token: delta d (+1, 0, -1) applied to the pair
PTX_HD inline void sx_step(PtxSeg3& v, int d) {
    v.scope += d;
    v.paren += d;
    if (v.paren < 0) v.paren = 0;
}

// ---- flags of a token kind, one byte: what the structure pass wants to know of a token
enum : uint32_t { SXF_L = 1, SXF_R = 2, SXF_OPENS = 4, SXF_S = 32, SXF_DIR = 64, SXF_SECTION = 128 };
PTX_HD inline uint32_t sx_flags(uint32_t k) {
    uint32_t f = 0;
    if (k == T_LBRACE) f |= SXF_L;
    if (k == T_RBRACE) f |= SXF_R;
    if (ptx_opens_operand((uint16_t)k)) f |= SXF_OPENS;
    if (k == T_SEMI || k == T_COLON) f |= SXF_S;
    if (ptx_is_directive_start((uint16_t)k)) f |= SXF_DIR;
    if (k == T_DOT_SECTION) f |= SXF_SECTION;
    return f;
}
PTX_HD inline uint32_t sx_popc(uint32_t x) {
#ifdef __CUDA_ARCH__
    return (uint32_t)__popc(x);
#else
    return (uint32_t)__builtin_popcount(x);
#endif
}
PTX_HD inline uint32_t sx_lowest(uint32_t x) {     // x != 0
#ifdef __CUDA_ARCH__
    return (uint32_t)(__ffs(x) - 1);
#else
    return (uint32_t)__builtin_ctz(x);
#endif
}

// A thread's 16 tokens.  The common case ("fast": no module begins among the tokens or the three in front, and the
// batch does not end here) never looks at a kind again after the table look-up: the flag bytes go into four words,
// token i in byte i / 4 of word i % 4, so that the token before the tokens of word r are the same bytes of word r - 1,
// and four tokens are judged by one bitwise operation.  One-bit-per-token results are kept as "spread" masks: token i
// at bit 8 * (i / 4) + i % 4, which keeps the tokens in order (so "the tokens before i" is a mask of lower bits) and
// leaves the upper half of every byte for a second mask:
//   braces: scope-opening '{' (low halves) and scope-closing '}' (high halves);
//   marks: previous token is ';' or ':' (low halves) and directive keywords (high halves).
// Threads of the other case go token by token and read the kinds again.
struct SxThread {
    uint32_t tb, n_valid;
    uint32_t first;               // bit i: token tb - 3 + i is the first token of a module
    bool fast;
    uint32_t braces, marks;
    uint32_t brace_before;        // the token in front of the thread's first: bit 0 = a scope brace, bit 1 = a closing one
};
// token-by-token case: the kinds of the thread's tokens and the three in front, w[3 + k] = token tb + k
struct SxWindow {
    uint16_t w[SX_ITEMS + 3];
};
PTX_HD inline void sx_window(const PtxStructArgs& a, const SxThread& t, SxWindow& win) {
    union { LtWord4 q[2]; uint16_t h[16]; } own;
    own.q[0] = ((const LtWord4*)(a.kinds + t.tb))[0];
    own.q[1] = ((const LtWord4*)(a.kinds + t.tb))[1];
    union { unsigned long long q; uint16_t h[4]; } halo;
    halo.q = t.tb ? *(const unsigned long long*)(a.kinds + t.tb - 4) : 0ull;
    for (uint32_t k = 0; k < SX_ITEMS; k++) win.w[3 + k] = PTX_KL_KIND(own.h[k]);
    for (uint32_t k = 0; k < 3; k++) win.w[k] = t.tb ? PTX_KL_KIND(halo.h[1 + k]) : (uint16_t)0;
}
constexpr uint32_t SX_LOW = 0x0F0F0F0Fu, SX_ONES = 0x01010101u;
// spread position of token i, and the tokens of a spread mask moved one place up (token i's bit to token i + 1)
PTX_HD inline uint32_t sx_pos(uint32_t i) { return 8u * (i >> 2) + (i & 3u); }
PTX_HD inline uint32_t sx_up(uint32_t m) { return ((m & 0x07070707u) << 1) | ((m & 0x08080808u) << 5); }

// The tiles in which a module begins, or whose three tokens in front hold a module begin: module m marks them in a
// word per tile (stride in words), ahead of the pass.
PTX_HD inline void sx_mark_tiles(const PtxStructArgs& a, uint32_t m, uint32_t* marks, uint32_t stride) {
    const uint32_t b = a.mtb[m];
    if (b >= a.n_tokens) return;
    marks[(size_t)(b / SX_TILE) * stride] = 1u;
    if (b % SX_TILE >= SX_TILE - 3u && (uint64_t)(b / SX_TILE + 1u) * SX_TILE < a.n_tokens) marks[(size_t)(b / SX_TILE + 1u) * stride] = 1u;
}
// the same by a search of the module table
PTX_HD inline bool sx_tile_has_first(const PtxStructArgs& a, uint32_t tile_base) {
    uint32_t lowest = tile_base >= 3 ? tile_base - 3 : 0;
    uint32_t lo = 0, hi = a.n_modules;
    while (lo < hi) {
        uint32_t mid = (lo + hi) >> 1;
        if (a.mtb[mid] < lowest) lo = mid + 1;
        else hi = mid;
    }
    return lo < a.n_modules && (uint64_t)a.mtb[lo] < (uint64_t)tile_base + SX_TILE;
}

// table: flags of every kind (512 entries; the caller's copy in fast memory); has_first: a module begins somewhere in
// the tile or in the three tokens in front of it
PTX_HD inline void sx_load(const PtxStructArgs& a, uint32_t tb, SxThread& t, const uint8_t* table, bool has_first, bool allow_fast = true) {
    t.tb = tb;
    t.n_valid = tb >= a.n_tokens ? 0u : (a.n_tokens - tb < SX_ITEMS ? a.n_tokens - tb : SX_ITEMS);
    t.first = 0;
    t.fast = false;
    t.braces = t.marks = t.brace_before = 0;
    if (!t.n_valid) return;
    if (has_first) {
        // module begins inside [tb - 3, tb + 16)
        uint32_t lowest = tb >= 3 ? tb - 3 : 0;
        uint32_t lo = 0, hi = a.n_modules;
        while (lo < hi) {
            uint32_t mid = (lo + hi) >> 1;
            if (a.mtb[mid] < lowest) lo = mid + 1;
            else hi = mid;
        }
        for (uint32_t m = lo; m < a.n_modules; m++) {
            uint32_t b = a.mtb[m];
            if (b >= tb + SX_ITEMS) break;
            t.first |= 1u << (b + 3 - tb);
        }
    }
    // tb is a multiple of 16: two aligned 16-byte loads, and one of 8 bytes for the tokens in front
    union { LtWord4 q[2]; uint16_t h[16]; uint32_t u[8]; } own;
    own.q[0] = ((const LtWord4*)(a.kinds + tb))[0];
    own.q[1] = ((const LtWord4*)(a.kinds + tb))[1];
    union { unsigned long long q; uint16_t h[4]; } halo;
    halo.q = tb ? *(const unsigned long long*)(a.kinds + tb - 4) : 0ull;
    t.fast = allow_fast && t.first == 0 && (uint64_t)tb + SX_ITEMS < a.n_tokens;
    if (!t.fast) return;      // the token-by-token case reads the kinds where it needs them
    uint32_t F[4] = {0, 0, 0, 0};
#pragma unroll
    for (uint32_t i = 0; i < 8; i++) {      // word i: tokens 2i and 2i + 1 -> byte i / 2 of words (i % 2) * 2 and + 1
        const uint32_t lo = table[own.u[i] & 0x1FFu], hi = table[(own.u[i] >> 16) & 0x1FFu];
        F[(i & 1u) * 2u] |= lo << (8u * (i >> 1));
        F[(i & 1u) * 2u + 1u] |= hi << (8u * (i >> 1));
    }
    // without tokens in front (tb == 0 cannot be fast: token 0 begins a module) the three flag bytes are read anyway
    const uint32_t h1 = table[PTX_KL_KIND(halo.h[1])], h2 = table[PTX_KL_KIND(halo.h[2])], h3 = table[PTX_KL_KIND(halo.h[3])];
    const uint32_t P1[4] = {(F[3] << 8) | h3, F[0], F[1], F[2]};          // the token before
    const uint32_t P2[4] = {(F[2] << 8) | h2, P1[0], F[0], F[1]};         // the token two before
    uint32_t braces = 0, marks = 0;
#pragma unroll
    for (uint32_t r = 0; r < 4; r++) {
        const uint32_t f = F[r], p1 = P1[r], p2 = P2[r];
        const uint32_t plus = f & ~(p1 >> 2) & ~(p2 >> 7) & SX_ONES;                   // '{' not after an operand opener or .section x
        const uint32_t minus = (f >> 1) & (p1 | (p1 >> 1) | (p1 >> 5)) & SX_ONES;      // '}' after ';' ':' '{' '}'
        braces |= (plus << r) | (minus << (4u + r));
        marks |= (((p1 >> 5) & SX_ONES) << r) | (((f >> 6) & SX_ONES) << (4u + r));
    }
    t.braces = braces; t.marks = marks;
    const uint32_t plus_h = h3 & ~(h2 >> 2) & ~(h1 >> 7) & 1u, minus_h = (h3 >> 1) & (h2 | (h2 >> 1) | (h2 >> 5)) & 1u;
    t.brace_before = plus_h | minus_h | (minus_h << 1);
}

// scope delta of the token at window index x (x >= 3): see ptx_brace_class
PTX_HD inline int sx_brace(const SxWindow& win, const SxThread& t, uint32_t x) {
    uint16_t k = win.w[x];
    if (k != T_LBRACE && k != T_RBRACE) return 0;
    bool first = (t.first >> x) & 1u;
    uint16_t prev = first ? (uint16_t)0xFFFE : win.w[x - 1];
    if (k == T_LBRACE) {
        bool section = false;
        if (!first && !((t.first >> (x - 1)) & 1u) && t.tb + x >= 5) section = win.w[x - 2] == T_DOT_SECTION;
        return (!ptx_opens_operand(prev) && !section) ? 1 : 0;
    }
    return (prev == T_SEMI || prev == T_COLON || prev == T_LBRACE || prev == T_RBRACE) ? -1 : 0;
}
// the same for the token just in front of the thread's first (window index 2), whose own left context is w[0..1]
PTX_HD inline int sx_brace_before(const SxWindow& win, const SxThread& t) {
    return t.tb ? sx_brace(win, t, 2) : 0;
}

// step 1: the thread's aggregate (flag = a module begins among its tokens)
PTX_HD inline PtxSeg3 sx_aggregate(const PtxStructArgs& a, const SxThread& t) {
    PtxSeg3 v{0, 0, 0};
    if (t.fast) {
        const uint32_t plus = t.braces & SX_LOW, minus = (t.braces >> 4) & SX_LOW;
        if (!minus) return PtxSeg3{(int32_t)sx_popc(plus), 0, 0};
#pragma unroll 1
        for (uint32_t k = 0; k < SX_ITEMS; k++) sx_step(v, (int)((plus >> sx_pos(k)) & 1u) - (int)((minus >> sx_pos(k)) & 1u));
        return v;
    }
    if (!t.n_valid) return v;
    SxWindow win;
    sx_window(a, t, win);
#pragma unroll 1
    for (uint32_t k = 0; k < t.n_valid; k++) {
        uint32_t x = 3 + k;
        if ((t.first >> x) & 1u) v = PtxSeg3{0, 0, 1};
        sx_step(v, sx_brace(win, t, x));
    }
    return v;
}

PTX_HD inline bool sx_continues(uint16_t prev) {      // a directive keyword behind one of these is no start
    return prev == T_DOT_EXTERN || prev == T_DOT_VISIBLE || prev == T_MOD_weak || prev == T_DOT_PTR;
}

// step 2: with the depth in front of the thread's first token: where units start, as a spread mask; the scope depth
// behind a module's last token goes to mod_final_scope.
// Token by token from the kinds; with write set, the rows of the unit table are written as well (step 3).
PTX_HD inline uint32_t sx_walk(const PtxStructArgs& a, const SxThread& t, int32_t depth, bool write, uint32_t units_before) {
    int32_t sd = depth;
    uint32_t starts = 0, u = units_before;
    if (!t.n_valid) return 0;
    SxWindow win;
    sx_window(a, t, win);
    int bc_prev = sx_brace_before(win, t);
#pragma unroll 1
    for (uint32_t k = 0; k < t.n_valid; k++) {
        const uint32_t x = 3 + k, j = t.tb + k;
        const int bc = sx_brace(win, t, x);
        const uint16_t kk = win.w[x];
        bool start, first = (t.first >> x) & 1u;
        if (first) {
            if (j) a.mod_final_scope[ptx_upper_bound_u32(a.mtb, a.n_modules, j - 1) - 1] = sd;
            start = true;
            sd = 0;
        } else if (sd == 0) {
            start = (ptx_is_directive_start(kk) && !sx_continues(win.w[x - 1])) || bc_prev < 0;
        } else {
            const uint16_t prev = win.w[x - 1];
            start = prev == T_SEMI || prev == T_COLON || bc != 0 || bc_prev != 0;
        }
        if (start) {
            starts |= 1u << sx_pos(k);
            if (write) {
                a.ustart[u] = j;
                a.udepth[u] = (sd > 0x7FF0 ? 0x7FF0u : (uint32_t)sd) | (first ? 0x80000000u : 0u);
                if (first) a.mub[ptx_upper_bound_u32(a.mtb, a.n_modules, j) - 1] = u;
                u++;
            }
        }
        sd += bc;
        if (sd < 0) sd = 0;
        bc_prev = bc;
        if (j + 1 == a.n_tokens) {
            a.mod_final_scope[ptx_upper_bound_u32(a.mtb, a.n_modules, j) - 1] = sd;
            if (write) a.counters->n_units = u;
        }
    }
    return starts;
}
PTX_HD inline uint32_t sx_decide(const PtxStructArgs& a, const SxThread& t, int32_t depth) {
    if (!t.fast) return sx_walk(a, t, depth, false, 0);
    const uint32_t plus = t.braces & SX_LOW, minus = (t.braces >> 4) & SX_LOW;
    const uint32_t in_scope = (t.marks & SX_LOW) | plus | minus | sx_up(plus | minus) | (t.brace_before & 1u);
    if (depth - (int32_t)sx_popc(minus) > 0) return in_scope;                              // inside a scope all the way
    uint32_t dirs = (t.marks >> 4) & SX_LOW;
    const uint32_t behind_close = sx_up(minus) | (t.brace_before >> 1);
    if (depth == 0 && !plus) {                                                             // top level all the way
        uint32_t starts = behind_close;
        while (dirs) {
            const uint32_t pos = sx_lowest(dirs);
            dirs &= dirs - 1u;
            const uint32_t k = (pos >> 3) * 4u + (pos & 3u);
            if (!sx_continues(PTX_KL_KIND(a.kinds[t.tb + k - 1]))) starts |= 1u << pos;     // fast threads have tb > 0
        }
        return starts;
    }
    // a bit of both: token by token
    int32_t sd = depth;
    uint32_t starts = 0;
#pragma unroll 1
    for (uint32_t k = 0; k < SX_ITEMS; k++) {
        const uint32_t pos = sx_pos(k), bit = 1u << pos;
        if (sd > 0) {
            starts |= in_scope & bit;
        } else {
            starts |= behind_close & bit;
            if ((dirs & bit) && !sx_continues(PTX_KL_KIND(a.kinds[t.tb + k - 1]))) starts |= bit;
        }
        sd += (int32_t)((plus >> pos) & 1u) - (int32_t)((minus >> pos) & 1u);
        if (sd < 0) sd = 0;
    }
    return starts;
}

// step 3: with the number of unit starts in front of the thread's first token: the rows of the unit table
PTX_HD inline void sx_write(const PtxStructArgs& a, const SxThread& t, int32_t depth, uint32_t starts, uint32_t units_before) {
    if (!t.fast) {
        if (t.n_valid) sx_walk(a, t, depth, true, units_before);
        return;
    }
    uint32_t u = units_before;
    const uint32_t plus = t.braces & SX_LOW, minus = (t.braces >> 4) & SX_LOW;
    if (depth - (int32_t)sx_popc(minus) >= 0) {
        // the depth never meets its floor: plain sums
        while (starts) {
            const uint32_t pos = sx_lowest(starts), below = (1u << pos) - 1u;
            starts &= starts - 1u;
            const int32_t sd = depth + (int32_t)sx_popc(plus & below) - (int32_t)sx_popc(minus & below);
            a.ustart[u] = t.tb + (pos >> 3) * 4u + (pos & 3u);
            a.udepth[u] = sd > 0x7FF0 ? 0x7FF0u : (uint32_t)sd;
            u++;
        }
        return;
    }
    int32_t sd = depth;
#pragma unroll 1
    for (uint32_t k = 0; k < SX_ITEMS; k++) {
        const uint32_t pos = sx_pos(k);
        if ((starts >> pos) & 1u) {
            a.ustart[u] = t.tb + k;
            a.udepth[u] = sd > 0x7FF0 ? 0x7FF0u : (uint32_t)sd;
            u++;
        }
        sd += (int32_t)((plus >> pos) & 1u) - (int32_t)((minus >> pos) & 1u);
        if (sd < 0) sd = 0;
    }
}
