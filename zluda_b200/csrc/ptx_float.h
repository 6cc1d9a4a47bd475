// Decimal text -> binary64, correctly rounded (round-half-even), for tokens matching [0-9]*\.[0-9]+([eE][-+]?[0-9]+)?
// Replaces Rust's str::parse::<f64> in ptx_parser's f64 literal rule (ptx_parser/src/lib.rs:307-310).
//
// Three tiers, all on the device:
//   1. exact: <= 15 significant digits and |exponent| <= 22 -> one IEEE multiply or divide (Clinger).
//   2. Eisel-Lemire: 64-bit significand x 128-bit truncated power of five (Lemire 2021; sufficiency of the 128-bit
//      product for 64-bit significands: Mushtak & Lemire 2023).
//   3. more than 19 significant digits where the truncated significand w and w+1 round differently: exact
//      comparison of the decimal value with the halfway point between the two candidates in fixed-width
//      multi-limb integers.
#pragma once
#include "gen/ptx_tables.h"
#include "gen/ptx_pow5.h"

#ifndef PTX_NOINLINE
#ifdef __CUDACC__
#define PTX_NOINLINE __noinline__
#else
#define PTX_NOINLINE __attribute__((noinline))
#endif
#endif

struct PtxAdjMant {
    uint64_t mantissa;
    int32_t power2;   // biased exponent; 0x7FF = infinity
};

PTX_HD inline void ptx_mul64(uint64_t a, uint64_t b, uint64_t* hi, uint64_t* lo) {
#ifdef __CUDA_ARCH__
    *lo = a * b;
    *hi = __umul64hi(a, b);
#else
    unsigned __int128 p = (unsigned __int128)a * b;
    *lo = (uint64_t)p;
    *hi = (uint64_t)(p >> 64);
#endif
}
PTX_HD inline int ptx_clz64(uint64_t x) {
#ifdef __CUDA_ARCH__
    return __clzll((long long)x);
#else
    return __builtin_clzll(x);
#endif
}

// value = w * 10^q, w != 0
PTX_HD PTX_NOINLINE inline PtxAdjMant ptx_eisel_lemire(int64_t q, uint64_t w) {
    PtxAdjMant ans;
    ans.mantissa = 0;
    ans.power2 = 0;
    if (w == 0 || q < PTX_POW5_MIN) return ans;
    if (q > PTX_POW5_MAX) { ans.power2 = 0x7FF; return ans; }
    int lz = ptx_clz64(w);
    w <<= lz;
    uint64_t t_hi = ptx_pow5[q - PTX_POW5_MIN][0], t_lo = ptx_pow5[q - PTX_POW5_MIN][1];
    uint64_t hi, lo;
    ptx_mul64(w, t_hi, &hi, &lo);
    const uint64_t precision_mask = 0xFFFFFFFFFFFFFFFFull >> 55;   // 52 + 3 bits
    if ((hi & precision_mask) == precision_mask) {
        uint64_t hi2, lo2;
        ptx_mul64(w, t_lo, &hi2, &lo2);
        lo += hi2;
        if (hi2 > lo) hi++;
    }
    int upperbit = (int)(hi >> 63);
    int shift = upperbit + 64 - 52 - 3;
    ans.mantissa = hi >> shift;
    int32_t pw = (int32_t)((((152170 + 65536) * q) >> 16) + 63);
    ans.power2 = pw + upperbit - lz + 1023;
    if (ans.power2 <= 0) {   // subnormal
        if (-ans.power2 + 1 >= 64) { ans.power2 = 0; ans.mantissa = 0; return ans; }
        ans.mantissa >>= -ans.power2 + 1;
        ans.mantissa += (ans.mantissa & 1);
        ans.mantissa >>= 1;
        ans.power2 = (ans.mantissa < (1ull << 52)) ? 0 : 1;
        return ans;
    }
    if (lo <= 1 && q >= -4 && q <= 23 && (ans.mantissa & 3) == 1) {
        if ((ans.mantissa << shift) == hi) ans.mantissa &= ~1ull;
    }
    ans.mantissa += (ans.mantissa & 1);
    ans.mantissa >>= 1;
    if (ans.mantissa >= (2ull << 52)) { ans.mantissa = 1ull << 52; ans.power2++; }
    ans.mantissa &= ~(1ull << 52);
    if (ans.power2 >= 0x7FF) { ans.power2 = 0x7FF; ans.mantissa = 0; }
    return ans;
}

PTX_HD inline uint64_t ptx_am_bits(PtxAdjMant a) { return a.mantissa | ((uint64_t)a.power2 << 52); }

// ---- fixed-width unsigned big integers (little-endian 32-bit limbs) for the tie-break
#define PTX_BIG_LIMBS 176
struct PtxBig {
    uint32_t v[PTX_BIG_LIMBS];
    int n;
};
PTX_HD inline void big_set(PtxBig& b, uint64_t x) {
    b.n = 0;
    while (x) { b.v[b.n++] = (uint32_t)x; x >>= 32; }
}
PTX_HD inline void big_mul_add(PtxBig& b, uint32_t m, uint32_t add) {
    uint64_t carry = add;
    for (int i = 0; i < b.n; i++) {
        uint64_t t = (uint64_t)b.v[i] * m + carry;
        b.v[i] = (uint32_t)t;
        carry = t >> 32;
    }
    if (carry && b.n < PTX_BIG_LIMBS) b.v[b.n++] = (uint32_t)carry;
}
PTX_HD inline void big_mul_pow5(PtxBig& b, uint32_t e) {
    while (e >= 13) { big_mul_add(b, 1220703125u, 0); e -= 13; }   // 5^13
    uint32_t m = 1;
    while (e--) m *= 5;
    if (m > 1) big_mul_add(b, m, 0);
}
PTX_HD inline void big_shl(PtxBig& b, uint32_t bits) {
    uint32_t limbs = bits / 32, r = bits % 32;
    if (b.n == 0) return;
    if (r) {
        uint32_t carry = 0;
        for (int i = 0; i < b.n; i++) {
            uint32_t t = b.v[i];
            b.v[i] = (t << r) | carry;
            carry = t >> (32 - r);
        }
        if (carry && b.n < PTX_BIG_LIMBS) b.v[b.n++] = carry;
    }
    if (limbs) {
        int nn = b.n + (int)limbs;
        if (nn > PTX_BIG_LIMBS) nn = PTX_BIG_LIMBS;
        for (int i = nn - 1; i >= (int)limbs; i--) b.v[i] = b.v[i - limbs];
        for (int i = 0; i < (int)limbs && i < nn; i++) b.v[i] = 0;
        b.n = nn;
    }
}
PTX_HD inline int big_cmp(const PtxBig& a, const PtxBig& b) {
    if (a.n != b.n) return a.n < b.n ? -1 : 1;
    for (int i = a.n - 1; i >= 0; i--)
        if (a.v[i] != b.v[i]) return a.v[i] < b.v[i] ? -1 : 1;
    return 0;
}

// digits: the token text; [d0, d1) covers the significand characters (digits and one '.'), leading zeros allowed.
// Returns sign of (decimal value - M * 2^P).  exp10 is the exponent applied after the last significand digit.
PTX_HD PTX_NOINLINE inline int ptx_cmp_decimal_to_binary(const uint8_t* s, uint32_t d0, uint32_t d1, int64_t exp10, uint64_t M, int32_t P) {
    PtxBig a, b;
    a.n = 0;
    const int max_digits = 800;   // more digits cannot change the comparison except through "sticky"
    int used = 0;
    bool sticky = false;
    for (uint32_t i = d0; i < d1; i++) {
        if (s[i] == '.') continue;
        uint32_t d = s[i] - '0';
        if (used == 0 && d == 0) continue;   // leading zeros
        if (used < max_digits) {
            if (a.n == 0) { if (d) { a.v[0] = d; a.n = 1; } }
            else big_mul_add(a, 10, d);
            used++;
        } else {
            if (d) sticky = true;
            exp10++;
        }
    }
    big_set(b, M);
    // a * 10^exp10  vs  b * 2^P
    int64_t two = exp10 - P;   // a * 5^exp10 * 2^(exp10 - P) vs b
    if (exp10 >= 0) big_mul_pow5(a, (uint32_t)exp10);
    else big_mul_pow5(b, (uint32_t)(-exp10));
    if (two >= 0) big_shl(a, (uint32_t)two);
    else big_shl(b, (uint32_t)(-two));
    int c = big_cmp(a, b);
    if (c == 0 && sticky) c = 1;
    return c;
}

// Convert a token matching [0-9]*\.[0-9]+([eE][-+]?[0-9]+)? to the bits of the nearest binary64.
PTX_HD PTX_NOINLINE inline uint64_t ptx_parse_f64(const uint8_t* s, uint32_t len) {
    uint64_t w = 0;
    int ndigits = 0;          // significant digits accumulated into w (max 19)
    int64_t exp10 = 0;
    bool truncated = false, seen_dot = false, nonzero = false;
    uint32_t i = 0;
    for (; i < len; i++) {
        unsigned c = s[i];
        if (c == '.') { seen_dot = true; continue; }
        if (c - '0' >= 10u) break;
        unsigned d = c - '0';
        if (d || nonzero) {
            nonzero = true;
            if (ndigits < 19) { w = w * 10 + d; ndigits++; }
            else { truncated = truncated || d != 0; exp10++; }
        }
        if (seen_dot) exp10--;
    }
    uint32_t sig_end = i;
    if (i < len && (s[i] | 32u) == 'e') {
        i++;
        bool neg = false;
        if (i < len && (s[i] == '-' || s[i] == '+')) { neg = s[i] == '-'; i++; }
        int64_t e = 0;
        for (; i < len; i++) {
            if (e < 100000) e = e * 10 + (s[i] - '0');
        }
        exp10 += neg ? -e : e;
    }
    if (w == 0) return 0;
    if (!truncated && w <= (1ull << 53) && exp10 >= -22 && exp10 <= 22) {
        const double p10[23] = {1e0, 1e1, 1e2, 1e3, 1e4, 1e5, 1e6, 1e7, 1e8, 1e9, 1e10, 1e11, 1e12, 1e13, 1e14, 1e15,
                                1e16, 1e17, 1e18, 1e19, 1e20, 1e21, 1e22};
        double v = (double)w;
        v = exp10 < 0 ? v / p10[-exp10] : v * p10[exp10];
        union { double d; uint64_t u; } cv;
        cv.d = v;
        return cv.u;
    }
    PtxAdjMant lo = ptx_eisel_lemire(exp10, w);
    if (!truncated) return ptx_am_bits(lo);
    PtxAdjMant hi = ptx_eisel_lemire(exp10, w + 1);
    uint64_t blo = ptx_am_bits(lo), bhi = ptx_am_bits(hi);
    if (blo == bhi) return blo;
    // the true value lies strictly between w*10^q and (w+1)*10^q whose roundings are adjacent doubles blo < bhi:
    // compare it with their midpoint (2*m+1) * 2^(e-1)
    uint64_t m = lo.mantissa | (lo.power2 ? (1ull << 52) : 0);
    int32_t e = (lo.power2 ? lo.power2 : 1) - 1075;   // value = m * 2^e
    // recompute exp10 as "exponent after the last significand digit of the full digit string"
    int64_t full_exp = 0;
    {
        bool dot = false;
        for (uint32_t k = 0; k < sig_end; k++) {
            if (s[k] == '.') dot = true;
            else if (dot) full_exp--;
        }
        uint32_t k = sig_end;
        if (k < len && (s[k] | 32u) == 'e') {
            k++;
            bool neg = false;
            if (k < len && (s[k] == '-' || s[k] == '+')) { neg = s[k] == '-'; k++; }
            int64_t ee = 0;
            for (; k < len; k++)
                if (ee < 100000) ee = ee * 10 + (s[k] - '0');
            full_exp += neg ? -ee : ee;
        }
    }
    int c = ptx_cmp_decimal_to_binary(s, 0, sig_end, full_exp, 2 * m + 1, e - 1);
    if (c < 0) return blo;
    if (c > 0) return bhi;
    return (blo & 1) ? bhi : blo;
}
