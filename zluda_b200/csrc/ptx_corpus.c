/* Seeded synthetic PTX corpora with the shapes of the five benchmark configurations (plain C, host only).
 *
 * They stand in for real fatbin PTX, of which the reference ships none beyond its small test fixtures.  Every statement
 * is drawn independently: opcode mix, operand registers uniform over the declared ranges, immediates uniform over int32
 * or the bit pattern of a float32 normal(0,1) sample written as 0fXXXXXXXX, address offsets, labels and branch targets.
 * Nothing is cut from a pool: a gigabyte of text holds a gigabyte of independently drawn statements.  Every statement
 * form used here is one the reference parser accepts (the tests check the generators against the CPU oracle).
 *
 * The content of a module depends only on (seed, module index, target size), so any subset of a batch can be generated
 * by itself and the ranks of a multi-GPU run generate only their own share.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

/* ---- random numbers: xoshiro256** seeded through splitmix64 */
typedef struct { uint64_t s[4]; } Rng;
static uint64_t splitmix(uint64_t* x) {
    uint64_t z = (*x += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static void rng_seed(Rng* r, uint64_t seed, uint64_t stream) {
    uint64_t x = seed * 0xD1342543DE82EF95ull + stream * 0x9E3779B97F4A7C15ull + 0x2545F4914F6CDD1Dull;
    for (int i = 0; i < 4; i++) r->s[i] = splitmix(&x);
}
static inline uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
static inline uint64_t rng_next(Rng* r) {
    uint64_t* s = r->s;
    uint64_t result = rotl(s[1] * 5, 7) * 9, t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl(s[3], 45);
    return result;
}
static inline uint32_t rng_below(Rng* r, uint32_t n) { return (uint32_t)(((rng_next(r) >> 32) * (uint64_t)n) >> 32); }
static inline double rng_unit(Rng* r) { return (double)(rng_next(r) >> 11) * (1.0 / 9007199254740992.0); }
static double rng_normal(Rng* r) {
    double u1 = rng_unit(r), u2 = rng_unit(r);
    if (u1 < 1e-300) u1 = 1e-300;
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
}

/* ---- output buffer */
typedef struct { char* p; size_t n, cap; } Out;
static inline void put_mem(Out* o, const char* s, size_t l) {
    if (o->n + l <= o->cap) memcpy(o->p + o->n, s, l);
    o->n += l;
}
static inline void put(Out* o, const char* s) { put_mem(o, s, strlen(s)); }
static inline void put_ch(Out* o, char c) { put_mem(o, &c, 1); }
static void put_u64(Out* o, uint64_t v) {
    char b[24];
    int i = 24;
    do { b[--i] = (char)('0' + v % 10); v /= 10; } while (v);
    put_mem(o, b + i, (size_t)(24 - i));
}
static void put_i64(Out* o, int64_t v) {
    if (v < 0) { put_ch(o, '-'); put_u64(o, (uint64_t)0 - (uint64_t)v); }
    else put_u64(o, (uint64_t)v);
}
static void put_hex(Out* o, uint64_t v, int digits, int upper) {   /* digits = 0: as many as needed */
    static const char lo[] = "0123456789abcdef", up[] = "0123456789ABCDEF";
    char b[16];
    int n = 0;
    do { b[n++] = (upper ? up : lo)[v & 15]; v >>= 4; } while (v || n < digits);
    while (n) put_ch(o, b[--n]);
}
static void put_reg(Out* o, const char* prefix, uint32_t n) { put(o, prefix); put_u64(o, n); }
static void put_hexf(Out* o, Rng* r) {
    union { float f; uint32_t u; } c;
    c.f = (float)rng_normal(r);
    put(o, "0f");
    put_hex(o, c.u, 8, 1);
}
#define R(o, r) put_reg(o, "%r", rng_below(r, 256))
#define RD(o, r) put_reg(o, "%rd", rng_below(r, 128))
#define F(o, r) put_reg(o, "%f", rng_below(r, 256))
#define P(o, r) put_reg(o, "%p", rng_below(r, 32))
static void put_imm32(Out* o, Rng* r) { put_i64(o, (int64_t)(int32_t)(uint32_t)(rng_next(r) >> 32)); }

static void put_label(Out* o, const char* kernel, uint32_t i) { put(o, "$L__"); put(o, kernel); put_ch(o, '_'); put_u64(o, i); }

/* one instruction line of the configuration-0 mix (tiles: + 10 % mma / ld.shared.v4 statements).  A setp is followed by
 * the branch it guards, as one draw. */
static void gen_statement(Out* o, Rng* r, const char* kernel, uint32_t n_labels, int tiles) {
    double u = rng_unit(r);
    if (tiles) {
        if (u < 0.05) {
            put(o, "\tmma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {");
            F(o, r); put(o, ", "); F(o, r); put(o, ", "); F(o, r); put(o, ", "); F(o, r); put(o, "}, {");
            R(o, r); put(o, ", "); R(o, r); put(o, ", "); R(o, r); put(o, ", "); R(o, r); put(o, "}, {");
            R(o, r); put(o, ", "); R(o, r); put(o, "}, {");
            F(o, r); put(o, ", "); F(o, r); put(o, ", "); F(o, r); put(o, ", "); F(o, r); put(o, "};\n");
            return;
        }
        if (u < 0.10) {
            put(o, "\tld.shared.v4.b32 {");
            R(o, r); put(o, ", "); R(o, r); put(o, ", "); R(o, r); put(o, ", "); R(o, r); put(o, "}, [");
            RD(o, r); put_ch(o, '+'); put_u64(o, 16u * rng_below(r, 256)); put(o, "];\n");
            return;
        }
        u = (u - 0.10) / 0.90;
    }
    if (u < 0.30) {
        uint32_t k = rng_below(r, 12), t = k % 3, op = k / 3;
        static const char* ty[] = {"s32", "u32", "f32"};
        int isf = t == 2;
        put_ch(o, '\t');
        put(o, op == 0 ? "add" : op == 1 ? "sub" : op == 2 ? "mul" : "mad");
        if (op >= 2 && !isf) put(o, ".lo");
        put_ch(o, '.'); put(o, ty[t]); put_ch(o, ' ');
        int n_src = op == 3 ? 3 : 2;
        if (isf) F(o, r); else R(o, r);
        for (int i = 0; i < n_src; i++) {
            put(o, ", ");
            if (i == n_src - 1 && rng_unit(r) < 0.25) { if (isf) put_hexf(o, r); else put_imm32(o, r); }
            else if (isf) F(o, r);
            else R(o, r);
        }
        put(o, ";\n");
    } else if (u < 0.45) {
        put(o, "\tfma.rn.f32 "); F(o, r); put(o, ", "); F(o, r); put(o, ", "); F(o, r); put(o, ", ");
        if (rng_unit(r) < 0.25) put_hexf(o, r); else F(o, r);
        put(o, ";\n");
    } else if (u < 0.60) {
        uint32_t k = rng_below(r, 8);
        int shared = k & 1, isu = (k >> 1) & 1, store = (k & 4) != 0;
        int vec = rng_unit(r) < 0.25, n = vec ? (rng_below(r, 2) ? 4 : 2) : 1;
        uint32_t base = rng_below(r, 128), off = 4u * rng_below(r, 1024);
        uint32_t regs[4];
        for (int i = 0; i < n; i++) regs[i] = rng_below(r, 256);
        put(o, store ? "\tst." : "\tld.");
        put(o, shared ? "shared" : "global");
        if (vec) put(o, n == 2 ? ".v2" : ".v4");
        put(o, isu ? ".u32 " : ".f32 ");
        for (int pass = 0; pass < 2; pass++) {
            if ((pass == 0) == (store != 0)) {
                put_ch(o, '['); put_reg(o, "%rd", base); put_ch(o, '+'); put_u64(o, off); put_ch(o, ']');
            } else {
                if (vec) put_ch(o, '{');
                for (int i = 0; i < n; i++) { if (i) put(o, ", "); put_reg(o, isu ? "%r" : "%f", regs[i]); }
                if (vec) put_ch(o, '}');
            }
            if (pass == 0) put(o, ", ");
        }
        put(o, ";\n");
    } else if (u < 0.70) {
        switch (rng_below(r, 5)) {
        case 0: put(o, "\tmov.u32 "); R(o, r); put(o, ", "); if (rng_unit(r) < 0.5) put_imm32(o, r); else R(o, r); break;
        case 1: put(o, "\tmov.f32 "); F(o, r); put(o, ", "); if (rng_unit(r) < 0.5) put_hexf(o, r); else F(o, r); break;
        case 2: put(o, "\tcvt.rn.f32.s32 "); F(o, r); put(o, ", "); R(o, r); break;
        case 3: put(o, "\tcvt.rzi.s32.f32 "); R(o, r); put(o, ", "); F(o, r); break;
        default: put(o, "\tmov.u64 "); RD(o, r); put(o, ", "); RD(o, r); break;
        }
        put(o, ";\n");
    } else if (u < 0.78) {
        static const char* cmp[] = {"lt", "ge", "eq"};
        static const char* ty[] = {"s32", "u32", "f32"};
        uint32_t c = rng_below(r, 3), t = rng_below(r, 3), p = rng_below(r, 32);
        put(o, "\tsetp."); put(o, cmp[c]); put_ch(o, '.'); put(o, ty[t]); put_ch(o, ' ');
        put_reg(o, "%p", p); put(o, ", ");
        if (t == 2) { F(o, r); put(o, ", "); F(o, r); } else { R(o, r); put(o, ", "); R(o, r); }
        put(o, ";\n\t@"); put_reg(o, "%p", p); put(o, " bra "); put_label(o, kernel, rng_below(r, n_labels)); put(o, ";\n");
    } else if (u < 0.83) {
        if (rng_unit(r) < 0.5) {
            put(o, "\tshfl.sync.bfly.b32 "); R(o, r); put_ch(o, '|'); P(o, r); put(o, ", "); R(o, r); put(o, ", ");
            put_u64(o, 1u << rng_below(r, 5)); put(o, ", 31, -1;\n");
        } else {
            put(o, "\tbar.sync "); put_u64(o, rng_below(r, 16)); put(o, ";\n");
        }
    } else {
        switch (rng_below(r, 4)) {
        case 0: put(o, "\tand.b32 "); R(o, r); put(o, ", "); R(o, r); put(o, ", "); if (rng_unit(r) < 0.3) put_imm32(o, r); else R(o, r); break;
        case 1: put(o, "\tor.b32 "); R(o, r); put(o, ", "); R(o, r); put(o, ", "); R(o, r); break;
        case 2: put(o, "\tshl.b32 "); R(o, r); put(o, ", "); R(o, r); put(o, ", "); put_u64(o, rng_below(r, 32)); break;
        default: put(o, "\tselp.f32 "); F(o, r); put(o, ", "); F(o, r); put(o, ", "); F(o, r); put(o, ", "); P(o, r); break;
        }
        put(o, ";\n");
    }
}

static void put_header(Out* o, const char* target) {
    put(o, ".version 7.8\n.target "); put(o, target); put(o, "\n.address_size 64\n\n");
}
static void put_kernel_open(Out* o, const char* name) {
    put(o, ".visible .entry "); put(o, name); put(o, "(\n");
    for (int i = 0; i < 8; i++) {
        put(o, i < 4 ? "\t.param .u64 " : "\t.param .u32 "); put(o, name); put(o, "_param_"); put_u64(o, (uint64_t)i);
        put(o, i < 7 ? ",\n" : "\n");
    }
    put(o, ")\n{\n\t.reg .pred %p<32>;\n\t.reg .b32 %r<256>;\n\t.reg .f32 %f<256>;\n\t.reg .b64 %rd<128>;\n\n");
}
/* a kernel of up to n_instr draws, one label in front of every 50th; it ends early once the text has `stop_at` bytes */
static void gen_kernel(Out* o, Rng* r, const char* name, uint32_t n_instr, int tiles, size_t stop_at) {
    put_kernel_open(o, name);
    uint32_t n_labels = (n_instr + 49) / 50;
    if (!n_labels) n_labels = 1;
    put_label(o, name, 0); put(o, ":\n");
    for (uint32_t i = 0; i < n_instr && o->n < stop_at; i++) {
        /* later labels appear as the kernel grows; a branch may name one that an early stop leaves out, which the
         * grammar does not mind (labels are resolved by a later pass) */
        if (i && i % 50 == 0) { put_label(o, name, i / 50); put(o, ":\n"); }
        gen_statement(o, r, name, n_labels, tiles);
    }
    put(o, "\tret;\n}\n\n");
}

/* Every entry point writes at most `cap` bytes and returns the size of the whole text: call once with cap = 0 for the
 * size, or with a buffer known to be large enough. */

/* configuration 0: one module, n_kernels entry kernels of n_instr instructions */
size_t ptx_corpus_config0(uint64_t seed, uint32_t n_kernels, uint32_t n_instr, char* out, size_t cap) {
    Out o = {out, 0, cap};
    Rng r;
    rng_seed(&r, seed, 0);
    put_header(&o, "sm_80");
    for (uint32_t k = 0; k < n_kernels; k++) {
        char name[32];
        snprintf(name, sizeof name, "k%u", k);
        gen_kernel(&o, &r, name, n_instr, 0, (size_t)-1);
    }
    return o.n;
}

/* configuration 1 / 4: module `index` of a batch, target_bytes long to within a line or two: kernels of 2,000 instructions
 * (the last one shorter) with 10 % tensor-core tile statements, target drawn from sm_80 / sm_86 / sm_90 */
size_t ptx_corpus_config1_module(uint64_t seed, uint32_t index, uint64_t target_bytes, char* out, size_t cap) {
    static const char* targets[] = {"sm_80", "sm_86", "sm_90"};
    Out o = {out, 0, cap};
    Rng r;
    rng_seed(&r, seed, (uint64_t)index + 1);
    put_header(&o, targets[rng_below(&r, 3)]);
    const size_t stop_at = target_bytes > 64 ? (size_t)target_bytes - 64 : 0;   /* room for the last line and the closing lines */
    uint32_t k = 0;
    do {
        char name[48];
        snprintf(name, sizeof name, "m%u_k%u", index, k++);
        gen_kernel(&o, &r, name, 2000, 1, stop_at);
    } while (o.n + 700 < stop_at);      /* a kernel's opening lines take about 600 bytes */
    return o.n;
}

/* configuration 2: literal-heavy data module.  n_arrays arrays (.b8 and .u32 alternating) of n_init initialisers,
 * values uniform over the type's range, half written as 0x hex and half as decimal; then n_consts scalar constants as
 * 0d / 0f hex and as decimals with 17 or 9 significant digits.  Decimal floats are written non-negative: the reference
 * grammar has no '-' in front of a float literal (ptx_parser/src/lib.rs:366-377). */
size_t ptx_corpus_config2(uint64_t seed, uint32_t n_arrays, uint32_t n_init, uint32_t n_consts, char* out, size_t cap) {
    Out o = {out, 0, cap};
    Rng r;
    rng_seed(&r, seed, 0);
    put_header(&o, "sm_80");
    for (uint32_t a = 0; a < n_arrays; a++) {
        int bytes8 = (a % 2) == 0;
        put(&o, bytes8 ? ".global .align 16 .b8 arr" : ".global .align 16 .u32 arr");
        put_u64(&o, a); put_ch(&o, '['); put_u64(&o, n_init); put(&o, "] = {");
        for (uint32_t i = 0; i < n_init; i++) {
            uint64_t bits = rng_next(&r);
            uint32_t v = bytes8 ? (uint32_t)(bits >> 56) : (uint32_t)(bits >> 32);
            if (i) put(&o, ", ");
            if (bits & 1) { put(&o, "0x"); put_hex(&o, v, 0, 1); }
            else put_u64(&o, v);     /* never a leading 0 unless the value is 0: a leading 0 means octal */
        }
        put(&o, "};\n");
    }
    for (uint32_t i = 0; i < n_consts; i++) {
        double x = rng_normal(&r);
        uint32_t kind = rng_below(&r, 5);
        char num[64];
        union { double d; uint64_t u; } c64;
        union { float f; uint32_t u; } c32;
        put(&o, kind == 4 ? ".const " : ".global ");
        put(&o, (kind == 1 || kind == 3) ? ".f32 c" : ".f64 c");
        put_u64(&o, i); put(&o, " = ");
        switch (kind) {
        case 0: c64.d = x; put(&o, "0d"); put_hex(&o, c64.u, 16, 1); break;
        case 1: c32.f = (float)x; put(&o, "0f"); put_hex(&o, c32.u, 8, 1); break;
        case 2: snprintf(num, sizeof num, "%.16e", fabs(x)); put(&o, num); break;
        case 3: snprintf(num, sizeof num, "%.8e", fabs(x)); put(&o, num); break;
        default: snprintf(num, sizeof num, "%.16e", fabs(x) * pow(10.0, (double)((int)rng_below(&r, 60) - 30))); put(&o, num); break;
        }
        put(&o, ";\n");
    }
    return o.n;
}

/* configuration 3: debug-info and structure-heavy module.  A 256-entry .file table, n_funcs .func declarations, then
 * entry kernels until total_bytes: a .loc line in front of every instruction, // and block comments (about 40 % of the
 * bytes), scopes nested to a uniformly drawn depth of 1-32 with a scoped .reg declaration each, call sequences to the
 * functions declared above (20 % of the statements), n_labels labels with forward and backward branches. */
size_t ptx_corpus_config3(uint64_t seed, uint64_t total_bytes, uint32_t n_funcs, uint32_t n_labels, char* out, size_t cap) {
    Out o = {out, 0, cap};
    Rng r;
    rng_seed(&r, seed, 0);
    put_header(&o, "sm_80");
    for (uint32_t i = 0; i < 256; i++) {
        put(&o, ".file "); put_u64(&o, i + 1); put(&o, " \"/build/src/dir"); put_u64(&o, i % 16); put(&o, "/file"); put_u64(&o, i);
        put(&o, ".cu\"\n");
    }
    for (uint32_t j = 0; j < n_funcs; j++) {
        put(&o, ".func (.param .b32 func_retval0) f"); put_u64(&o, j); put(&o, "(.param .b32 f"); put_u64(&o, j); put(&o, "_param_0)\n;\n");
    }
    if (!n_funcs) n_funcs = 1;
    uint64_t per_kernel = total_bytes / 64;
    if (per_kernel < (64u << 10)) per_kernel = 64u << 10;
    uint32_t kid = 0, label_budget = n_labels;
    while (o.n < total_bytes) {
        char name[32];
        snprintf(name, sizeof name, "dbg%u", kid);
        put_kernel_open(&o, name);
        put_label(&o, name, 0); put(&o, ":\n");     /* target of the branches drawn with ordinary statements */
        size_t body_start = o.n;
        uint32_t depth = 0, line_no = 1, lbl = 0;
        while (o.n - body_start < per_kernel) {
            double u = rng_unit(&r);
            if (u < 0.04 && depth < 32) {
                uint32_t want = 1 + rng_below(&r, 32);
                while (depth < want) {
                    for (uint32_t t = 0; t < depth; t++) put_ch(&o, '\t');
                    put(&o, "{\n");
                    for (uint32_t t = 0; t <= depth; t++) put_ch(&o, '\t');
                    put(&o, ".reg .b32 %t"); put_u64(&o, depth); put(&o, ";\n");
                    depth++;
                }
                continue;
            }
            if (u < 0.08 && depth > 0) {
                uint32_t k = 1 + rng_below(&r, depth);
                while (k--) {
                    depth--;
                    for (uint32_t t = 0; t < depth; t++) put_ch(&o, '\t');
                    put(&o, "}\n");
                }
                continue;
            }
            if (u < 0.28) {
                put(&o, ".loc "); put_u64(&o, 1 + line_no % 256); put_ch(&o, ' '); put_u64(&o, line_no); put_ch(&o, ' '); put_u64(&o, 1 + line_no % 40);
                put(&o, "\n{\n.param .b32 p0;\nst.param.b32 [p0+0], "); R(&o, &r);
                put(&o, ";\n.param .b32 rv;\ncall.uni (rv), f"); put_u64(&o, rng_below(&r, n_funcs)); put(&o, ", (p0);\nld.param.b32 "); R(&o, &r);
                put(&o, ", [rv+0];\n}\n");
            } else if (u < 0.30 && label_budget > 0) {
                put(&o, "$L_dbg_"); put_u64(&o, kid); put_ch(&o, '_'); put_u64(&o, lbl); put(&o, ":\n");
                lbl++;
                label_budget--;
            } else if (u < 0.33 && lbl > 0) {
                put(&o, ".loc "); put_u64(&o, 1 + line_no % 256); put_ch(&o, ' '); put_u64(&o, line_no); put(&o, " 3\nbra $L_dbg_");
                put_u64(&o, kid); put_ch(&o, '_'); put_u64(&o, rng_below(&r, lbl + 4)); put(&o, ";\n");
            } else {
                put(&o, ".loc "); put_u64(&o, 1 + line_no % 256); put_ch(&o, ' '); put_u64(&o, line_no); put_ch(&o, ' '); put_u64(&o, 1 + line_no % 40);
                put_ch(&o, '\n');
                gen_statement(&o, &r, name, 1, 0);    /* its rare branches go to the kernel's first generated label */
            }
            line_no++;
            if (rng_unit(&r) < 0.95) {
                uint32_t i = rng_below(&r, 512);
                if (rng_below(&r, 2)) {
                    put(&o, "\t// inlined from helper_"); put_u64(&o, i); put(&o, " at line "); put_u64(&o, i * 7 % 1000);
                    put(&o, ", column "); put_u64(&o, i % 80); put_ch(&o, '\n');
                } else {
                    put(&o, "\t/* block comment "); put_u64(&o, i); put(&o, ": loop body, unrolled by "); put_u64(&o, i % 8);
                    put(&o, " * stride */ /* second part */\n");
                }
            }
        }
        while (depth > 0) {
            depth--;
            for (uint32_t t = 0; t < depth; t++) put_ch(&o, '\t');
            put(&o, "}\n");
        }
        put(&o, "\tret;\n}\n\n");
        kid++;
    }
    return o.n;
}
