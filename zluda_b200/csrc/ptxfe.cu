// CUDA backend and C ABI of the PTX front end (include/ptxfe.h).  Built for sm_100a only.
//
// Every pipeline step of ptxfe_pipeline.h runs as a kernel on the context's stream: a grid-stride-free parallel-for
// (one thread per chunk, token or unit) or a three-phase block scan (reduce tiles, scan tile totals, rescan tiles).
// Device memory comes from a per-context arena of retained cudaMalloc blocks, so a steady stream of batches allocates
// nothing.  There is no host parsing path: without a device every entry point returns PTXFE_ERR_CUDA.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <string>
#include <type_traits>
#include <vector>

#define PTX_HD __device__
#define PTX_TABLE static __device__ const
#include "../../include/ptxfe.h"
#include "ptxfe_pipeline.h"
#include "ptx_partition.h"
#include <thread>

// host side (ptxfe_dump.cpp)
std::string ptxfe_dump_module_impl(const PtxBatchView& v, uint32_t m, int* status);
uint64_t ptxfe_dump_hash_impl(const PtxBatchView& v, uint32_t m, int* status);
std::string ptxfe_dump_module_tree_impl(const PtxBatchView& v, uint32_t m, int* status);
uint64_t ptxfe_materialize_impl(const PtxBatchView& v, uint32_t m);

#define CUDA_TRY(call)                                                                      \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess) {                                                            \
            snprintf(ctx->err, sizeof ctx->err, "%s: %s", #call, cudaGetErrorString(e_));   \
            return PTXFE_ERR_CUDA;                                                          \
        }                                                                                   \
    } while (0)

// ------------------------------------------------------------------------------------------------ kernels
template <class F>
__global__ void __launch_bounds__(256) pf_kernel(size_t n, F f) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) f(i);
}

// ---- per-chunk lexer steps over a shared-memory tile of the text
// One block = 256 chunks = 32 KiB of text, staged with coalesced 16-byte loads.  Thread t then walks chunk t byte by
// byte; rows are padded to 33 words so that 32 threads reading the same column of 32 rows hit 32 different banks.
// The token automaton's [state][byte] table (ptx_lex_fused) is copied to shared memory as well.
#define LEX_TILE_CHUNKS 256u
#define LEX_ROW_WORDS 33u
struct PtxTileReader {
    const uint32_t* tile;      // [LEX_TILE_CHUNKS][LEX_ROW_WORDS]
    const uint16_t* fused;     // [LS_COUNT][256], copy of ptx_lex_fused
    const uint8_t* g;          // the whole text, for bytes outside the tile
    uint32_t base;             // text offset of the tile
    __device__ unsigned operator[](uint32_t p) const {
        uint32_t o = p - base;
        if (o < LEX_TILE_CHUNKS * PTX_CHUNK) return ((const uint8_t*)tile)[(o >> 7) * (LEX_ROW_WORDS * 4) + (o & 127u)];
        return g[p];
    }
    __device__ uint32_t word(uint32_t p) const {   // p is a multiple of 4 inside the tile
        uint32_t o = p - base;
        return tile[(o >> 7) * LEX_ROW_WORDS + ((o & 127u) >> 2)];
    }
    __device__ uint32_t lookup(int st, unsigned c) const { return fused[st * 256 + c]; }
};

#define LEX_TILE_BYTES (LEX_TILE_CHUNKS * LEX_ROW_WORDS * 4u)
#define LEX_TABLE_BYTES (LS_COUNT * 256u * 2u)
template <bool TABLES, class F>
__global__ void __launch_bounds__(256) lex_tile_kernel(uint32_t n_chunks, const uint8_t* text, F f) {
    extern __shared__ __align__(16) uint32_t lex_smem[];
    uint32_t* tile = lex_smem;                                       // [LEX_TILE_CHUNKS][LEX_ROW_WORDS]
    uint16_t* fused = (uint16_t*)(lex_smem + LEX_TILE_CHUNKS * LEX_ROW_WORDS);    // [LS_COUNT][256] when TABLES
    const uint32_t c0 = blockIdx.x * LEX_TILE_CHUNKS;
    const uint4* src = (const uint4*)text + (size_t)c0 * (PTX_CHUNK / 16);
#pragma unroll
    for (uint32_t k = 0; k < 8; k++) {
        uint32_t idx = threadIdx.x + k * 256;      // 16-byte piece of the tile
        uint32_t row = idx >> 3;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (c0 + row < n_chunks) v = src[idx];
        uint32_t* d = tile + row * LEX_ROW_WORDS + (idx & 7u) * 4;
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
    if (TABLES) {
        for (uint32_t i = threadIdx.x; i < LS_COUNT * 256; i += 256) fused[i] = ptx_lex_fused[i];
    }
    __syncthreads();
    uint32_t c = c0 + threadIdx.x;
    if (c < n_chunks) f((size_t)c, PtxTileReader{tile, fused, text, c0 * PTX_CHUNK});
}

// ---- the two block-cooperative lexer steps (ptx_lex_tile.h): one block per tile, a barrier between the phases
__global__ void lex_fill_tables_kernel(PtxLexTables* t) { lt_fill_tables(t, threadIdx.x, blockDim.x); }
// Persistent blocks: the tables are loaded once, then the block takes every gridDim.x-th tile.
__global__ void __launch_bounds__(256, 8) lex_mark_kernel(PtxLexTileArgs a, uint32_t n_tiles) {
    __shared__ PtxLexMarkShared sh;
    const uint32_t tid = threadIdx.x;
    lt_mark_tables(sh, a, tid, 256);
    lt_mark_reset(sh, tid, 256);
    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        __syncthreads();
        lt_mark_simple(sh, a, tile, tid, 256);
        __syncthreads();
        // ask for the text of the block's next tile while the rest of this one is settled
        if (tid < LT_BYTES / 128u && (uint64_t)tile + gridDim.x + 1 < n_tiles)       // a whole tile
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a.text + ((size_t)tile + gridDim.x) * LT_BYTES + tid * 128u));
        lt_mark_special(sh, a, tile, tid, 256);
        __syncthreads();
        lt_mark_triggers(sh, a, tile, tid, 256);
        __syncthreads();
        lt_mark_finish(sh, a, tile, tid, 256);
    }
}
__global__ void __launch_bounds__(256, 5) lex_emit_kernel(PtxLexTileArgs a, uint32_t n_tiles) {
    extern __shared__ __align__(16) unsigned char lex_emit_smem[];
    PtxLexEmitShared& sh = *(PtxLexEmitShared*)lex_emit_smem;
    const uint32_t tid = threadIdx.x;
    lt_emit_tables(sh, a, tid, 256);
    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        __syncthreads();
        lt_emit_init(sh, a, tile, tid, 256);
        __syncthreads();
        // ask for the block's next tile (text, start bits, word bits) while this one is worked on
        if ((uint64_t)tile + gridDim.x + 1 < n_tiles) {     // a whole tile: every line asked for lies inside the arrays
            const size_t next = (size_t)tile + gridDim.x;
            if (tid < LT_BYTES / 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.text + next * LT_BYTES + tid * 128u));
            else if (tid < LT_BYTES / 128u + 8u) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.start_bits + next * LT_WORDS + (tid - LT_BYTES / 128u) * 32u));
            else if (tid < LT_BYTES / 128u + 16u) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.word_bits + next * LT_WORDS + (tid - LT_BYTES / 128u - 8u) * 32u));
        }
        const uint32_t passes = lt_emit_passes(sh);
        for (uint32_t pass = 0; pass < passes; pass++) {
            if (pass) __syncthreads();
            lt_emit_list(sh, pass, tid, 256);
            __syncthreads();
            lt_emit_first(sh, a, tile, pass, tid, 256);
            __syncthreads();
            lt_emit_keywords(sh, a, tile, pass, tid, 256);
            lt_emit_second(sh, a, tile, pass, tid, 256);
        }
    }
}

// ---- first decode pass: every thread builds its record in shared memory and copies it to its row of the staging
// table.  Word k of thread t lives at stage[k * STAGE_STRIDE + t]: threads of a warp decode units of the same shape in
// lockstep, so they write the same k at the same time (32 consecutive banks).
#define STAGE_STRIDE 257u
#define STAGE_CAP 40u
#define WIN_CAP 12u
#define STAGED_SMEM_BYTES (STAGE_CAP * STAGE_STRIDE * 4u + WIN_CAP * STAGE_STRIDE * 8u)
template <class F>
__global__ void __launch_bounds__(256) staged_kernel(size_t n, uint32_t* table, uint32_t row_words, F f) {
    extern __shared__ __align__(16) unsigned char staged_smem[];
    PtxTokenWord* win = (PtxTokenWord*)staged_smem;                                    // [WIN_CAP][STAGE_STRIDE]
    uint32_t* stage = (uint32_t*)(staged_smem + WIN_CAP * STAGE_STRIDE * 8u);          // [STAGE_CAP][STAGE_STRIDE]
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    PtxStaged r;
    r.unit = 0;
    r.n = 0;
    if (i < n) r = f(i, PtxScratch{stage + threadIdx.x, STAGE_STRIDE, STAGE_CAP, win + threadIdx.x, STAGE_STRIDE, WIN_CAP});
    // Every thread copies its own record.  (The copy used to be cooperative, 32 lanes per record behind a __syncwarp and
    // two __shfl_sync per record.  About one parse in ten of a batch of 3,000 small modules of many shapes, run behind
    // a large batch, then lost words of a few records: lanes that came late out of long decoders skipped the records of
    // lanes that were done.  With each thread writing what it staged, 300 such parses in a row come out identical.)
    uint32_t* row = table + (size_t)r.unit * row_words;
    for (uint32_t k = 0; k < r.n; k++) row[k] = stage[k * STAGE_STRIDE + threadIdx.x];
}

// ---- one thread per item of a segmented range: a block takes 256 consecutive segments, whose items are contiguous,
// and every thread finds the segment of its item by binary search over the block's offsets in shared memory
// Record emission (PtxEmitStep): a block takes 256 consecutive units, whose words are contiguous, loads what a word
// needs of its unit into shared memory once, and then goes over the words with EMIT_ILP words per thread at a time:
// all their reads are issued before the first of them is written, so that several chains of dependent loads (unit ->
// template -> token) are in flight per thread.  The literals are collected and converted in a second round with the
// warps full.
#define SEG_DEFER_CAP 2048u
#define EMIT_ILP 4
__global__ void __launch_bounds__(256, 6) emit_records_kernel(uint32_t n_units, const PtxPair* off, PtxEmitStep e) {
    __shared__ uint32_t so[257];
    __shared__ PtxEmitUnit su[256];
    __shared__ uint32_t later[SEG_DEFER_CAP];
    __shared__ uint32_t n_later;
    const uint32_t u0 = blockIdx.x * 256;
    const uint32_t nu = n_units - u0 < 256u ? n_units - u0 : 256u;
    for (uint32_t k = threadIdx.x; k <= nu; k += 256) so[k] = off[u0 + k].a;
    if (threadIdx.x < nu) su[threadIdx.x] = e.unit(u0 + threadIdx.x);
    if (threadIdx.x == 0) n_later = 0;
    __syncthreads();
    const uint32_t first = so[0], total = so[nu] - so[0];
    // Every warp takes a contiguous eighth of the block's words, 32 at a time.  The unit of a word: `ua` is the unit of
    // the window's first word; the lanes read the next 32 unit offsets, those inside the window mark their place in a
    // 32-bit mask, and a lane's unit is ua + the number of marks at or below it.  (Units without words put two marks on
    // one place: such a window searches, as does the first of a warp.)
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t per_warp = ((total + 255u) / 256u) * 32u;
    const uint32_t wbeg = warp * per_warp, wend = wbeg + per_warp < total ? wbeg + per_warp : total;
    uint32_t ua = 0;
    if (wbeg < wend) {
        const uint32_t o = first + wbeg;
        uint32_t lo = 0, hi = nu;              // last k with so[k] <= o
        while (hi - lo > 1) {
            uint32_t mid = (lo + hi) >> 1;
            if (so[mid] <= o) lo = mid; else hi = mid;
        }
        ua = lo;
    }
    for (uint32_t jb = wbeg; jb < wend; jb += 32 * EMIT_ILP) {
        uint32_t x[EMIT_ILP], unit[EMIT_ILP];
        int what[EMIT_ILP];
#pragma unroll
        for (int q = 0; q < EMIT_ILP; q++) {
            const uint32_t j0 = jb + q * 32, j = j0 + lane;       // j0 is the same for the whole warp
            what[q] = PtxEmitStep::NOTHING;
            unit[q] = 0;
            if (j0 >= wend) continue;
            const uint32_t o0 = first + j0, o = o0 + lane;
            while (ua + 1 < nu && so[ua + 1] <= o0) ua++;        // the unit of the window's first word (a step or none)
            const uint32_t k = ua + 1 + lane;
            const uint32_t rel = k <= nu ? so[k] - o0 : 0xFFFFFFFFu;
            const bool inside = rel < 32u;
            const uint32_t n_in = (uint32_t)__popc(__ballot_sync(0xFFFFFFFFu, inside));
            const uint32_t marks = __reduce_or_sync(0xFFFFFFFFu, inside ? 1u << rel : 0u);
            uint32_t lo;
            if ((uint32_t)__popc(marks) == n_in) {
                lo = ua + (uint32_t)__popc(marks & (0xFFFFFFFFu >> (31u - lane)));
            } else {
                uint32_t hi = nu;
                lo = ua;
                while (hi - lo > 1) {
                    uint32_t mid = (lo + hi) >> 1;
                    if (so[mid] <= o) lo = mid; else hi = mid;
                }
            }
            ua = ua + n_in < nu - 1u ? ua + n_in : nu - 1u;     // the marks are all in front of the next window
            if (j >= wend) continue;
            unit[q] = lo;
            what[q] = e.word(su[lo], (size_t)(u0 + lo), o - so[lo], x[q]);
        }
#pragma unroll
        for (int q = 0; q < EMIT_ILP; q++) {
            const uint32_t j = jb + q * 32 + lane;
            if (what[q] == PtxEmitStep::WRITE) {
                e.words[first + j] = x[q];
            } else if (what[q] == PtxEmitStep::SECOND_ROUND) {
                const uint32_t slot = atomicAdd(&n_later, 1u);
                if (slot < SEG_DEFER_CAP && j < (1u << 24)) later[slot] = j | (unit[q] << 24);
                else e.literal(su[unit[q]], first + j - so[unit[q]], first + j);
            }
        }
    }
    __syncthreads();
    const uint32_t nl = n_later < SEG_DEFER_CAP ? n_later : SEG_DEFER_CAP;
    for (uint32_t x = threadIdx.x; x < nl; x += 256) {
        const uint32_t j = later[x] & 0xFFFFFFu, lo = later[x] >> 24, o = first + j;
        e.literal(su[lo], o - so[lo], o);
    }
}
template <class F>
__global__ void __launch_bounds__(256) segments_kernel(uint32_t n_units, const PtxPair* off, F f) {
    __shared__ uint32_t so[257];
    const uint32_t u0 = blockIdx.x * 256;
    const uint32_t nu = n_units - u0 < 256u ? n_units - u0 : 256u;
    for (uint32_t k = threadIdx.x; k <= nu; k += 256) so[k] = off[u0 + k].a;
    __syncthreads();
    const uint32_t first = so[0], total = so[nu] - so[0];
    for (uint32_t j = threadIdx.x; j < total; j += 256) {
        uint32_t o = first + j;
        uint32_t lo = 0, hi = nu;          // last k with so[k] <= o
        while (hi - lo > 1) {
            uint32_t mid = (lo + hi) >> 1;
            if (so[mid] <= o) lo = mid; else hi = mid;
        }
        f((size_t)(u0 + lo), o - so[lo], o);
    }
}

__global__ void copy_words_kernel(uint32_t* dst, const uint32_t* src, uint32_t n) {
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
}

// ---- text that arrived as one host-contiguous run: move every module to its chunk-aligned slot
// One thread per 16 bytes of destination.  `raw_off` of a module is where its first byte lies in `raw`.
struct RepackModule {
    uint32_t chunk_begin, raw_off, len;
};
__global__ void __launch_bounds__(256) repack_text_kernel(uint32_t n_pieces, uint32_t n_modules, const RepackModule* mods, const uint32_t* mcb,
                                                          const uint8_t* raw, uint8_t* text) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pieces) return;
    uint32_t chunk = i >> 3;
    uint32_t m = ptx_upper_bound_u32(mcb, n_modules, chunk) - 1;
    uint32_t o = (chunk - mods[m].chunk_begin) * PTX_CHUNK + (i & 7u) * 16;   // offset inside the module
    uint4 v = make_uint4(0, 0, 0, 0);
    if (o < mods[m].len) {
        size_t a = (size_t)mods[m].raw_off + o;
        const uint32_t* w = (const uint32_t*)(raw + (a & ~(size_t)3));       // the raw buffer has 32 spare bytes at its end
        uint32_t sh = (uint32_t)(a & 3) * 8;
        uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = w[4];
        v.x = __funnelshift_r(w0, w1, sh);
        v.y = __funnelshift_r(w1, w2, sh);
        v.z = __funnelshift_r(w2, w3, sh);
        v.w = __funnelshift_r(w3, w4, sh);
    }
    ((uint4*)text)[i] = v;
}

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

// Ordered block-wide scan of one value per thread (associative, not necessarily commutative): warp shuffles, then
// the eight warp totals through shared memory.  incl = everything up to and including this thread, excl = before it.
template <class T>
__device__ inline T shfl_up_words(T v, int d) {
    static_assert(sizeof(T) % 4 == 0, "scan element must be made of 32-bit words");
    union { T t; uint32_t w[sizeof(T) / 4]; } a, b;
    a.t = v;
#pragma unroll
    for (size_t i = 0; i < sizeof(T) / 4; i++) b.w[i] = __shfl_up_sync(0xFFFFFFFFu, a.w[i], d);
    return b.t;
}
template <class T>
__device__ inline T shfl_down_words(T v, int d) {
    union { T t; uint32_t w[sizeof(T) / 4]; } a, b;
    a.t = v;
#pragma unroll
    for (size_t i = 0; i < sizeof(T) / 4; i++) b.w[i] = __shfl_down_sync(0xFFFFFFFFu, a.w[i], d);
    return b.t;
}
template <class T>
__device__ inline T shfl_words(T v, int src) {
    union { T t; uint32_t w[sizeof(T) / 4]; } a, b;
    a.t = v;
#pragma unroll
    for (size_t i = 0; i < sizeof(T) / 4; i++) b.w[i] = __shfl_sync(0xFFFFFFFFu, a.w[i], src);
    return b.t;
}
template <class T, class Op>
__device__ inline void block_scan(T v, Op op, T identity, T* warp_tot, T& incl, T& excl) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        T y = shfl_up_words(x, d);
        if (lane >= d) x = op(y, x);
    }
    T prev = shfl_up_words(x, 1);
    if (lane == 0) prev = identity;
    if (lane == 31) warp_tot[warp] = x;
    __syncthreads();
    T wp = identity;
    for (int w = 0; w < warp; w++) wp = op(wp, warp_tot[w]);
    incl = op(wp, x);
    excl = op(wp, prev);
}

template <class T, class Op, class Ld>
__global__ void __launch_bounds__(SCAN_THREADS) scan_reduce_kernel(size_t n, Ld ld, Op op, T identity, T* partial) {
    __shared__ T warp_tot[SCAN_THREADS / 32];
    size_t base = (size_t)blockIdx.x * SCAN_TILE + (size_t)threadIdx.x * SCAN_ITEMS;
    T acc = identity;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++)
        if (base + k < n) acc = op(acc, ld(base + k));
    T incl, excl;
    block_scan(acc, op, identity, warp_tot, incl, excl);
    if (threadIdx.x == SCAN_THREADS - 1) partial[blockIdx.x] = incl;
}

template <class T, class Op, class Ld, class St>
__global__ void __launch_bounds__(SCAN_THREADS) scan_apply_kernel(size_t n, Ld ld, St st, Op op, T identity, const T* partial_incl) {
    __shared__ T warp_tot[SCAN_THREADS / 32];
    size_t base = (size_t)blockIdx.x * SCAN_TILE + (size_t)threadIdx.x * SCAN_ITEMS;
    T vals[SCAN_ITEMS];
    T acc = identity;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        if (base + k < n) acc = op(acc, ld(base + k));
        vals[k] = acc;
    }
    T incl, excl;
    block_scan(acc, op, identity, warp_tot, incl, excl);
    // everything before this thread: the tiles before this block, then the threads before it in the block
    T prefix = blockIdx.x ? op(partial_incl[blockIdx.x - 1], excl) : excl;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++)
        if (base + k < n) st(base + k, op(prefix, vals[k]));
}

// ---- stage B in one pass (ptx_struct_tile.h).  Tiles are handed out in order by an atomic counter, so a tile only
// ever waits for tiles that are already running or done.  Every tile publishes the aggregate of its tokens, then looks
// back along the tiles before it until it meets one whose whole prefix is known (or, for the depths, one in which a
// module begins: nothing before that matters), and publishes its own prefix.  A published value is self-contained:
// 64-bit words with the state in the top two bits (0 nothing yet, 1 the tile's own aggregate, 2 the prefix up to
// and including the tile); the depths take two words, which a reader accepts only when both carry the same state.
// Waiting is bounded: a tile that waits too long sets the abort word, every other waiter sees it and leaves, and the
// host reads struct_abort with the counters.
struct StructDesc {
    unsigned long long depth0, depth1, count;
    uint32_t has_first, pad;      // has_first: set ahead of the pass (sx_mark_tiles)
};
__global__ void structure_mark_kernel(PtxStructArgs a, StructDesc* desc) {
    uint32_t m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m < a.n_modules) sx_mark_tiles(a, m, &desc[0].has_first, (uint32_t)(sizeof(StructDesc) / 4));
}
constexpr unsigned long long SXD_AGG = 1ull << 62, SXD_PREFIX = 2ull << 62, SXD_STATE = 3ull << 62;
constexpr uint32_t SX_WAIT_LIMIT = 1u << 22;
constexpr int SX_DEPTH_PER_LANE = 1, SX_COUNT_PER_LANE = 1;     // tiles a lane of the look-back reads per trip to memory

__device__ inline unsigned long long sx_ld(const unsigned long long* p) { return *(const volatile unsigned long long*)p; }
__device__ inline void sx_st(unsigned long long* p, unsigned long long v) { *(volatile unsigned long long*)p = v; }
__device__ inline void sx_publish_depth(StructDesc* d, unsigned long long state, PtxSeg3 v) {
    sx_st(&d->depth0, state | ((unsigned long long)(v.flag ? 1u : 0u) << 32) | (uint32_t)v.scope);
    sx_st(&d->depth1, state | (uint32_t)v.paren);
}
// false = gave up (abort set by this or another tile)
__device__ inline bool sx_read_depth(const StructDesc* d, uint32_t* ctl, unsigned long long& state, PtxSeg3& v) {
    for (uint32_t spin = 0;; spin++) {
        unsigned long long a = sx_ld(&d->depth0), b = sx_ld(&d->depth1);
        if ((a & SXD_STATE) && (a & SXD_STATE) == (b & SXD_STATE)) {
            state = a & SXD_STATE;
            v.scope = (int32_t)(uint32_t)a;
            v.flag = (int32_t)((a >> 32) & 1u);
            v.paren = (int32_t)(uint32_t)b;
            return true;
        }
        if ((spin & 63u) == 63u && *(volatile uint32_t*)&ctl[1]) return false;
        if (spin >= SX_WAIT_LIMIT) { atomicExch(&ctl[1], 1u); return false; }
        __nanosleep(20);
    }
}
__device__ inline bool sx_read_count(const StructDesc* d, uint32_t* ctl, unsigned long long& state, uint32_t& v) {
    for (uint32_t spin = 0;; spin++) {
        unsigned long long a = sx_ld(&d->count);
        if (a & SXD_STATE) { state = a & SXD_STATE; v = (uint32_t)a; return true; }
        if ((spin & 63u) == 63u && *(volatile uint32_t*)&ctl[1]) return false;
        if (spin >= SX_WAIT_LIMIT) { atomicExch(&ctl[1], 1u); return false; }
        __nanosleep(20);
    }
}

__global__ void __launch_bounds__(SX_THREADS) structure_kernel(PtxStructArgs a, uint32_t n_tiles, StructDesc* desc, uint32_t* ctl) {
    __shared__ PtxSeg3 warp_depth[SX_THREADS / 32];
    __shared__ uint32_t warp_count[SX_THREADS / 32];
    __shared__ uint32_t s_tile, s_has_first, s_units_before, s_ok;
    __shared__ PtxSeg3 s_before;
    __shared__ uint8_t s_table[512];
    const int lane = threadIdx.x & 31;
    const SegDepthOp op;
    for (uint32_t k = threadIdx.x; k < 512; k += SX_THREADS) s_table[k] = (uint8_t)sx_flags(k);
    for (;;) {
        __syncthreads();                                   // the shared words of the tile before are no longer read
        if (threadIdx.x == 0) {
            const uint32_t mine = atomicAdd(&ctl[0], 1u);
            s_tile = mine;
            s_ok = *(volatile uint32_t*)&ctl[1] ? 0u : 1u;  // aborted: later tiles do nothing
            s_has_first = mine < n_tiles ? desc[mine].has_first : 0u;
        }
        __syncthreads();
        const uint32_t tile = s_tile;
        const bool has_first = s_has_first != 0;
        if (tile >= n_tiles) return;
        // the blocks take tiles more or less in turn: ask for the kinds of the tile one round ahead (whoever gets it)
        if ((threadIdx.x & 3u) == 0 && (uint64_t)tile + gridDim.x < n_tiles) {
            const uint16_t* ahead = a.kinds + ((size_t)tile + gridDim.x) * SX_TILE + threadIdx.x * SX_ITEMS;     // a 128-byte line
            asm volatile("prefetch.global.L2 [%0];" ::"l"(ahead));
        }
        SxThread t;
        sx_load(a, tile * SX_TILE + threadIdx.x * SX_ITEMS, t, s_table, has_first);
        PtxSeg3 incl, excl;
        block_scan(sx_aggregate(a, t), op, PtxSeg3{0, 0, 0}, warp_depth, incl, excl);
        if (threadIdx.x == SX_THREADS - 1) s_before = incl;         // the tile's aggregate, for warp 0
        __syncthreads();
        if (threadIdx.x < 32) {
            const PtxSeg3 agg = s_before;
            __syncwarp();
            PtxSeg3 before{0, 0, 0};
            bool ok = true;
            if (tile == 0) {
                if (lane == 0) sx_publish_depth(&desc[0], SXD_PREFIX, agg);
            } else {
                if (lane == 0) sx_publish_depth(&desc[tile], SXD_AGG, agg);
                // windows of 32 * SX_DEPTH_PER_LANE earlier tiles, nearest first; every lane takes consecutive tiles (its
                // nearest first) and stops at one with a known prefix or a module begin (or in front of tile 0)
                for (int64_t back = (int64_t)tile - 1; ok;) {
                    const int64_t mine = back - (int64_t)lane * SX_DEPTH_PER_LANE;
                    unsigned long long w0[SX_DEPTH_PER_LANE], w1[SX_DEPTH_PER_LANE];
#pragma unroll
                    for (int r = 0; r < SX_DEPTH_PER_LANE; r++) {       // all loads first: one trip to memory for the lot
                        w0[r] = mine - r >= 0 ? sx_ld(&desc[mine - r].depth0) : 0ull;
                        w1[r] = mine - r >= 0 ? sx_ld(&desc[mine - r].depth1) : 0ull;
                    }
                    PtxSeg3 v{0, 0, 0};
                    bool done = false, got = true;
#pragma unroll
                    for (int r = 0; r < SX_DEPTH_PER_LANE; r++) {
                        if (done || !got) continue;
                        if (mine - r < 0) { done = true; continue; }
                        unsigned long long state = w0[r] & SXD_STATE;
                        PtxSeg3 x{(int32_t)(uint32_t)w0[r], (int32_t)(uint32_t)w1[r], (int32_t)((w0[r] >> 32) & 1u)};
                        if (!state || state != (w1[r] & SXD_STATE)) got = sx_read_depth(&desc[mine - r], ctl, state, x);
                        if (!got) continue;
                        v = op(x, v);
                        done = state == SXD_PREFIX || x.flag;
                    }
                    if (!__all_sync(0xFFFFFFFFu, got)) { ok = false; break; }
                    unsigned ends = __ballot_sync(0xFFFFFFFFu, done);
                    int last = ends ? __ffs(ends) - 1 : 31;
                    if (lane > last) v = PtxSeg3{0, 0, 0};
                    // ordered reduction: lane 0 ends up with op(v[last], ..., v[1], v[0])
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        PtxSeg3 y = shfl_down_words(v, d);
                        if (lane + d < 32) v = op(y, v);
                    }
                    v = shfl_words(v, 0);
                    before = op(v, before);
                    if (ends) break;
                    back -= 32 * SX_DEPTH_PER_LANE;
                }
                if (ok && lane == 0) sx_publish_depth(&desc[tile], SXD_PREFIX, op(before, agg));
            }
            if (lane == 0) { s_before = before; if (!ok) s_ok = 0; }
        }
        __syncthreads();
        if (!s_ok) {
            if (threadIdx.x == 0) a.counters->struct_abort = 1;
            return;
        }
        const int32_t before = sx_depth(op(s_before, excl));
        const uint32_t starts = sx_decide(a, t, before);
        uint32_t cincl, cexcl;
        block_scan((uint32_t)__popc(starts), AddOp(), 0u, warp_count, cincl, cexcl);
        if (threadIdx.x == SX_THREADS - 1) s_units_before = cincl;
        __syncthreads();
        if (threadIdx.x < 32) {
            const uint32_t agg = s_units_before;
            __syncwarp();
            uint32_t before = 0;
            bool ok = true;
            if (tile == 0) {
                if (lane == 0) sx_st(&desc[0].count, SXD_PREFIX | agg);
            } else {
                if (lane == 0) sx_st(&desc[tile].count, SXD_AGG | agg);
                for (int64_t back = (int64_t)tile - 1; ok;) {
                    const int64_t mine = back - (int64_t)lane * SX_COUNT_PER_LANE;
                    unsigned long long w[SX_COUNT_PER_LANE];
#pragma unroll
                    for (int r = 0; r < SX_COUNT_PER_LANE; r++) w[r] = mine - r >= 0 ? sx_ld(&desc[mine - r].count) : 0ull;
                    uint32_t v = 0;
                    bool done = false, got = true;
#pragma unroll
                    for (int r = 0; r < SX_COUNT_PER_LANE; r++) {
                        if (done || !got) continue;
                        if (mine - r < 0) { done = true; continue; }
                        unsigned long long state = w[r] & SXD_STATE;
                        uint32_t x = (uint32_t)w[r];
                        if (!state) got = sx_read_count(&desc[mine - r], ctl, state, x);
                        if (!got) continue;
                        v += x;
                        done = state == SXD_PREFIX;
                    }
                    if (!__all_sync(0xFFFFFFFFu, got)) { ok = false; break; }
                    unsigned ends = __ballot_sync(0xFFFFFFFFu, done);
                    int last = ends ? __ffs(ends) - 1 : 31;
                    if (lane > last) v = 0;
                    before += __reduce_add_sync(0xFFFFFFFFu, v);
                    if (ends) break;
                    back -= 32 * SX_COUNT_PER_LANE;
                }
                if (ok && lane == 0) sx_st(&desc[tile].count, SXD_PREFIX | (uint32_t)(before + agg));
            }
            if (lane == 0) { s_units_before = before; if (!ok) s_ok = 0; }
        }
        __syncthreads();
        if (!s_ok) {
            if (threadIdx.x == 0) a.counters->struct_abort = 1;
            return;
        }
        sx_write(a, t, before, starts, s_units_before + cexcl);
    }
}

// ---- counting sort of unit indices by a 12-bit key: block-local histograms / ranks in shared memory, one global
// atomic per (block, non-empty bucket)
constexpr int SORT_THREADS = 512;
constexpr int SORT_ITEMS = 8;
constexpr int SORT_TILE = SORT_THREADS * SORT_ITEMS;

__global__ void __launch_bounds__(SORT_THREADS) sort_hist_kernel(size_t n, const uint16_t* key, uint32_t* hist) {
    __shared__ uint32_t sh[PTX_SORT_BUCKETS];
    for (int i = threadIdx.x; i < (int)PTX_SORT_BUCKETS; i += SORT_THREADS) sh[i] = 0;
    __syncthreads();
    size_t base = (size_t)blockIdx.x * SORT_TILE;
    for (int k = 0; k < SORT_ITEMS; k++) {
        size_t i = base + (size_t)k * SORT_THREADS + threadIdx.x;
        if (i < n) atomicAdd(&sh[key[i]], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (int)PTX_SORT_BUCKETS; i += SORT_THREADS)
        if (sh[i]) atomicAdd(&hist[i], sh[i]);
}

__global__ void __launch_bounds__(SORT_THREADS) sort_scatter_kernel(size_t n, const uint16_t* key, const uint32_t* bucket_begin,
                                                                    uint32_t* cursor, uint32_t* order) {
    __shared__ uint32_t sh[PTX_SORT_BUCKETS];
    for (int i = threadIdx.x; i < (int)PTX_SORT_BUCKETS; i += SORT_THREADS) sh[i] = 0;
    __syncthreads();
    size_t base = (size_t)blockIdx.x * SORT_TILE;
    uint32_t rank[SORT_ITEMS];
    uint16_t kk[SORT_ITEMS];
    for (int k = 0; k < SORT_ITEMS; k++) {
        size_t i = base + (size_t)k * SORT_THREADS + threadIdx.x;
        kk[k] = 0;
        rank[k] = 0;
        if (i < n) {
            kk[k] = key[i];
            rank[k] = atomicAdd(&sh[kk[k]], 1u);
        }
    }
    __syncthreads();
    // reserve this block's range in every non-empty bucket; sh[b] becomes the block's base inside the bucket
    for (int i = threadIdx.x; i < (int)PTX_SORT_BUCKETS; i += SORT_THREADS) {
        uint32_t c = sh[i];
        sh[i] = c ? bucket_begin[i] + atomicAdd(&cursor[i], c) : 0;
    }
    __syncthreads();
    for (int k = 0; k < SORT_ITEMS; k++) {
        size_t i = base + (size_t)k * SORT_THREADS + threadIdx.x;
        if (i < n) order[sh[kk[k]] + rank[k]] = (uint32_t)i;
    }
}

// token sink of the allocation-free lexer: writes into a caller-provided table, dropping what does not fit
struct LexCapSink {
    PtxToken* tokens;
    const uint8_t* text;
    uint64_t next, capacity;
    __device__ void token(uint32_t start, uint32_t len, uint16_t kind) {
        if (next < capacity) {
            PtxToken t;
            t.start = (uint32_t)start;
            t.len = len >= 0xFFFFu ? (uint16_t)0xFFFF : (uint16_t)len;
            t.kind = lx_classify(text, t.start, len, kind);
            tokens[next] = t;
        }
        next++;
    }
    __device__ void error(uint32_t, uint32_t) {}
};

template <class T> struct ArrayLoad {
    const T* p;
    __device__ T operator()(size_t i) const { return p[i]; }
};
template <class T> struct ArrayStore {
    T* p;
    __device__ void operator()(size_t i, T v) const { p[i] = v; }
};

struct SubtractOwn {   // inclusive -> exclusive prefix
    uint32_t* incl;
    const uint32_t* own;
    __device__ void operator()(size_t i) const { incl[i] -= own[i]; }
};

// ------------------------------------------------------------------------------------------------ context
struct ArenaBlock {
    char* base;
    size_t size, used;
};

struct ptxfe_batch {
    // a batch parsed on several devices is a list of per-device batches and a map from the caller's module index
    std::vector<ptxfe_batch*> parts;
    std::vector<std::pair<uint32_t, uint32_t>> where;
    ptxfe_ctx* ctx;
    uint32_t n, mode;
    std::vector<const char*> texts;
    std::vector<PtxModuleLayout> layout;
    std::vector<PtxModuleResult> results;
    std::vector<int> status;        // lazily filled by dump
    const uint32_t* words;
    const PtxErrRec* errs;
    const uint32_t* lexerrs;
};

struct ptxfe_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;        // kernels (and everything of the stage / run / fetch calls)
    cudaStream_t s_in = nullptr;          // host -> device copies of the pipelined parse
    cudaStream_t s_out = nullptr;         // device -> host copies of the pipelined parse
    cudaEvent_t ev[8] = {nullptr};
    std::vector<cudaEvent_t> slice_ev;    // 5 per slice: text arrived, kernels begin / end, results begin / end
    std::vector<ArenaBlock> arenas[2];    // device working memory; the pipelined parse alternates between the two
    int cur = 0;
    char err[512] = {0};
    bool failed = false;
    uint64_t launches = 0;
    // staged batch
    std::vector<const char*> texts;
    std::vector<PtxModuleLayout> layout;
    std::vector<uint32_t> mcb;
    uint64_t text_bytes = 0, padded_bytes = 0;
    uint8_t* d_text = nullptr;
    size_t d_text_cap = 0;
    void* d_class_store = nullptr;        // PtxClassStore arrays (one allocation, made at the first parse)
    PtxLexTables* d_lex_tables = nullptr; // constant tables of the lexer steps (filled at the first parse)
    uint8_t* d_raw = nullptr;             // host-contiguous runs land here before they are repacked into d_text
    size_t d_raw_cap = 0;
    PtxWork work;
    PtxCounters counters;
    bool staged = false, ran = false;
    uint32_t mode = 0;
    // pinned result buffers
    void* h_words = nullptr; size_t h_words_cap = 0;
    void* h_errs = nullptr; size_t h_errs_cap = 0;
    void* h_lexerrs = nullptr; size_t h_lexerrs_cap = 0;
    void* h_results = nullptr; size_t h_results_cap = 0;
    PtxCounters* h_counters = nullptr;    // mapped pinned memory, written by the device
    void* d_counters_mapped = nullptr;    // its device address
    ptxfe_stats stats;
    ptxfe_batch* live = nullptr;
    // per-step profile
    bool profile = false;
    std::vector<cudaEvent_t> prof_events;
    std::vector<const char*> prof_names;
    size_t prof_used = 0;
    std::string prof_text;
};

struct CudaBackend {
    ptxfe_ctx* ctx;
    void* alloc(size_t bytes) {
        bytes = (bytes + 255) & ~(size_t)255;
        for (ArenaBlock& b : ctx->arenas[ctx->cur])
            if (b.size - b.used >= bytes) {
                void* p = b.base + b.used;
                b.used += bytes;
                return p;
            }
        size_t sz = bytes > ((size_t)256 << 20) ? bytes : ((size_t)256 << 20);
        ArenaBlock nb;
        nb.base = nullptr;
        if (cudaMalloc((void**)&nb.base, sz) != cudaSuccess) {
            if (!ctx->failed) snprintf(ctx->err, sizeof ctx->err, "cudaMalloc of %zu bytes failed", sz);
            ctx->failed = true;
            cudaGetLastError();
            // keep going with a small dummy block is not possible: callers check ctx->failed before launching
            return nullptr;
        }
        nb.size = sz;
        nb.used = bytes;
        ctx->arenas[ctx->cur].push_back(nb);
        return nb.base;
    }
    void reset() {
        for (ArenaBlock& b : ctx->arenas[ctx->cur]) b.used = 0;
    }
    void zero(void* p, size_t bytes) {
        if (ctx->failed || !p) return;
        cudaMemsetAsync(p, 0, bytes, ctx->stream);
    }
    void download(void* host, const void* dev, size_t bytes) {
        if (ctx->failed) { memset(host, 0, bytes); return; }
        // a kernel writes the few words into mapped host memory: a copy-engine transfer would queue behind the
        // result copies of the previous slice, which run on another stream at the same time
        copy_words_kernel<<<1, 32, 0, ctx->stream>>>((uint32_t*)ctx->d_counters_mapped, (const uint32_t*)dev, (uint32_t)(bytes / 4));
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) {
            snprintf(ctx->err, sizeof ctx->err, "kernel or copy failed: %s", cudaGetErrorString(e));
            ctx->failed = true;
            memset(host, 0, bytes);
            return;
        }
        memcpy(host, ctx->h_counters, bytes);
    }
    // optional per-step timing (PTXFE_PROFILE=1): one event pair per step, read back by ptxfe_profile
    void prof_begin(const char* name) {
        if (!ctx->profile) return;
        if (ctx->prof_used + 2 > ctx->prof_events.size()) {
            for (int i = 0; i < 2; i++) {
                cudaEvent_t e;
                cudaEventCreate(&e);
                ctx->prof_events.push_back(e);
            }
        }
        ctx->prof_names.push_back(name);
        cudaEventRecord(ctx->prof_events[ctx->prof_used++], ctx->stream);
    }
    void prof_end() {
        if (!ctx->profile) return;
        cudaEventRecord(ctx->prof_events[ctx->prof_used++], ctx->stream);
    }
    template <class F> void pf(const char* name, size_t n, F f) {
        if (ctx->failed || n == 0) return;
        size_t blocks = (n + 255) / 256;
        prof_begin(name);
        pf_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(n, f);
        prof_end();
        ctx->launches++;
    }
    PtxClassStore class_store(bool reset) {
        PtxClassStore cs;
        if (!ctx->d_class_store) {
            if (cudaMalloc(&ctx->d_class_store, PtxClassStore::bytes()) != cudaSuccess) {
                if (!ctx->failed) snprintf(ctx->err, sizeof ctx->err, "cudaMalloc of the class store (%zu bytes) failed", PtxClassStore::bytes());
                ctx->failed = true;
                cudaGetLastError();
                ctx->d_class_store = nullptr;
            }
            reset = true;
        }
        cs.carve(ctx->d_class_store);
        if (reset && ctx->d_class_store) {
            cudaMemsetAsync(cs.keys, 0, sizeof(unsigned long long) * PTX_CLASS_SLOTS, ctx->stream);
            cudaMemsetAsync(cs.state, 0, 16, ctx->stream);
        }
        return cs;
    }
    template <class F> void pf_staged(const char* name, size_t n, uint32_t* table, uint32_t row_words, F f) {
        if (ctx->failed || n == 0) return;
        prof_begin(name);
        // more shared memory than a kernel gets by default: opt in (cheap, so done at every launch)
        cudaFuncSetAttribute(staged_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)STAGED_SMEM_BYTES);
        staged_kernel<<<(unsigned)((n + 255) / 256), 256, STAGED_SMEM_BYTES, ctx->stream>>>(n, table, row_words, f);
        prof_end();
        ctx->launches++;
    }
    template <class F> void pf_segments(const char* name, size_t n, const PtxPair* off, F f) {
        if (ctx->failed || n == 0) return;
        prof_begin(name);
        segments_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>((uint32_t)n, off, f);
        prof_end();
        ctx->launches++;
    }
    void emit_records(const char* name, size_t n, const PtxPair* off, const PtxEmitStep& e) {
        if (ctx->failed || n == 0) return;
        prof_begin(name);
        emit_records_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>((uint32_t)n, off, e);
        prof_end();
        ctx->launches++;
    }
    // per-chunk lexer steps; text holds n whole chunks and is 16-byte aligned (it is an arena block)
    template <class F> void pf_text(const char* name, size_t n, const uint8_t* text, F f) {
        if (ctx->failed || n == 0) return;
        unsigned blocks = (unsigned)((n + LEX_TILE_CHUNKS - 1) / LEX_TILE_CHUNKS);
        prof_begin(name);
        if constexpr (std::is_same<F, PtxLexVectorsStep>::value) {
            lex_tile_kernel<false><<<blocks, 256, LEX_TILE_BYTES, ctx->stream>>>((uint32_t)n, text, f);
        } else {
            // tile + table need more shared memory than a kernel gets by default
            cudaFuncSetAttribute(lex_tile_kernel<true, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(LEX_TILE_BYTES + LEX_TABLE_BYTES));
            lex_tile_kernel<true><<<blocks, 256, LEX_TILE_BYTES + LEX_TABLE_BYTES, ctx->stream>>>((uint32_t)n, text, f);
        }
        prof_end();
        ctx->launches++;
    }
    const PtxLexTables* lex_tables() {
        if (!ctx->d_lex_tables && !ctx->failed) {
            if (cudaMalloc((void**)&ctx->d_lex_tables, sizeof(PtxLexTables)) != cudaSuccess) {
                snprintf(ctx->err, sizeof ctx->err, "cudaMalloc of the lexer tables failed");
                ctx->failed = true;
                cudaGetLastError();
                ctx->d_lex_tables = nullptr;
                return nullptr;
            }
            lex_fill_tables_kernel<<<1, 256, 0, ctx->stream>>>(ctx->d_lex_tables);
        }
        return ctx->d_lex_tables;
    }
    // persistent grids: as many blocks as the device holds at once
    unsigned resident_blocks(const void* kernel, size_t smem, size_t n_tiles) {
        int per_sm = 0, sms = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, smem);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctx->device);
        size_t g = (size_t)(per_sm > 0 ? per_sm : 1) * (size_t)(sms > 0 ? sms : 1);
        return (unsigned)(g < n_tiles ? g : n_tiles);
    }
    void lex_mark(const char* name, size_t n_tiles, const PtxLexTileArgs& a) {
        if (ctx->failed || n_tiles == 0) return;
        prof_begin(name);
        lex_mark_kernel<<<resident_blocks((const void*)lex_mark_kernel, 0, n_tiles), 256, 0, ctx->stream>>>(a, (uint32_t)n_tiles);
        prof_end();
        ctx->launches++;
    }
    void lex_emit(const char* name, size_t n_tiles, const PtxLexTileArgs& a) {
        if (ctx->failed || n_tiles == 0) return;
        prof_begin(name);
        cudaFuncSetAttribute(lex_emit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(PtxLexEmitShared));
        lex_emit_kernel<<<resident_blocks((const void*)lex_emit_kernel, sizeof(PtxLexEmitShared), n_tiles), 256, sizeof(PtxLexEmitShared), ctx->stream>>>(a, (uint32_t)n_tiles);
        prof_end();
        ctx->launches++;
    }
    void fail(const char* why) {
        if (!ctx->failed) snprintf(ctx->err, sizeof ctx->err, "%s", why);
        ctx->failed = true;
    }
    void structure(const char* name, const PtxStructArgs& a) {
        if (ctx->failed || a.n_tokens == 0) return;
        const size_t n_tiles = ((size_t)a.n_tokens + SX_TILE - 1) / SX_TILE;
        StructDesc* desc = (StructDesc*)alloc(sizeof(StructDesc) * n_tiles + 256);
        if (!desc) return;
        uint32_t* ctl = (uint32_t*)(desc + n_tiles);      // [0] next tile, [1] abort
        prof_begin(name);
        cudaMemsetAsync(desc, 0, sizeof(StructDesc) * n_tiles + 256, ctx->stream);
        structure_mark_kernel<<<(a.n_modules + 255) / 256, 256, 0, ctx->stream>>>(a, desc);
        const unsigned grid = resident_blocks((const void*)structure_kernel, 0, n_tiles);
        structure_kernel<<<grid, SX_THREADS, 0, ctx->stream>>>(a, (uint32_t)n_tiles, desc, ctl);
        prof_end();
        ctx->launches++;
    }
    void sort_by_key(const char* name, size_t n, const uint16_t* key, uint32_t* order) {
        if (ctx->failed || n == 0) return;
        uint32_t* hist = (uint32_t*)alloc(sizeof(uint32_t) * PTX_SORT_BUCKETS * 3);
        if (!hist) return;
        uint32_t* begin = hist + PTX_SORT_BUCKETS;
        uint32_t* cursor = begin + PTX_SORT_BUCKETS;
        prof_begin(name);
        cudaMemsetAsync(hist, 0, sizeof(uint32_t) * PTX_SORT_BUCKETS * 3, ctx->stream);
        size_t blocks = (n + SORT_TILE - 1) / SORT_TILE;
        sort_hist_kernel<<<(unsigned)blocks, SORT_THREADS, 0, ctx->stream>>>(n, key, hist);
        // exclusive scan of the 4096 counts: begin[b] = sum of hist[0..b)
        ArrayLoad<uint32_t> ld{hist};
        ArrayStore<uint32_t> st{begin};
        scan_impl<uint32_t>((size_t)PTX_SORT_BUCKETS, ld, st, AddOp(), 0u);   // inclusive into begin[]
        pf_kernel<<<(PTX_SORT_BUCKETS + 255) / 256, 256, 0, ctx->stream>>>((size_t)PTX_SORT_BUCKETS, SubtractOwn{begin, hist});
        sort_scatter_kernel<<<(unsigned)blocks, SORT_THREADS, 0, ctx->stream>>>(n, key, begin, cursor, order);
        prof_end();
        ctx->launches += 3;
    }
    template <class T, class Ld, class St, class Op> void scan(const char* name, size_t n, Ld ld, St st, Op op, T identity) {
        if (ctx->failed || n == 0) return;
        prof_begin(name);
        scan_impl<T>(n, ld, st, op, identity);
        prof_end();
    }
    template <class T, class Ld, class St, class Op> void scan_impl(size_t n, Ld ld, St st, Op op, T identity) {
        if (ctx->failed || n == 0) return;
        size_t tiles = (n + SCAN_TILE - 1) / SCAN_TILE;
        T* partial = (T*)alloc(sizeof(T) * (tiles + 1));
        if (!partial) return;
        scan_reduce_kernel<T><<<(unsigned)tiles, SCAN_THREADS, 0, ctx->stream>>>(n, ld, op, identity, partial);
        ctx->launches++;
        if (tiles > 1) {
            // scan the tile totals in place (recursively)
            scan_impl<T>(tiles, ArrayLoad<T>{partial}, ArrayStore<T>{partial}, op, identity);
        }
        scan_apply_kernel<T><<<(unsigned)tiles, SCAN_THREADS, 0, ctx->stream>>>(n, ld, st, op, identity, partial);
        ctx->launches++;
    }
};

// ------------------------------------------------------------------------------------------------ C ABI
extern "C" {

const char* ptxfe_status_str(int s) {
    switch (s) {
    case PTXFE_OK: return "ok";
    case PTXFE_ERR_BAD_ARG: return "bad argument";
    case PTXFE_ERR_CUDA: return "CUDA error";
    case PTXFE_ERR_TOO_LARGE: return "batch too large";
    case PTXFE_ERR_OOM: return "out of memory";
    default: return "unknown status";
    }
}

int ptxfe_create(int device, ptxfe_ctx** out) {
    if (!out) return PTXFE_ERR_BAD_ARG;
    *out = nullptr;
    ptxfe_ctx* ctx = new ptxfe_ctx();
    ctx->device = device;
    memset(&ctx->stats, 0, sizeof ctx->stats);
    ctx->profile = getenv("PTXFE_PROFILE") && atoi(getenv("PTXFE_PROFILE")) != 0;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        fprintf(stderr, "ptxfe: no usable CUDA device %d (this library has no CPU path)\n", device);
        delete ctx;
        return PTXFE_ERR_CUDA;
    }
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->s_in, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->s_out, cudaStreamNonBlocking);
    for (int i = 0; i < 8 && e == cudaSuccess; i++) e = cudaEventCreate(&ctx->ev[i]);
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&ctx->h_counters, 4096, cudaHostAllocMapped);   // counters and other small read-backs
    if (e == cudaSuccess) e = cudaHostGetDevicePointer(&ctx->d_counters_mapped, ctx->h_counters, 0);
    if (e != cudaSuccess) {
        fprintf(stderr, "ptxfe: context set-up failed: %s\n", cudaGetErrorString(e));
        delete ctx;
        return PTXFE_ERR_CUDA;
    }
    *out = ctx;
    return PTXFE_OK;
}

void ptxfe_destroy(ptxfe_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    for (int a = 0; a < 2; a++)
        for (ArenaBlock& b : ctx->arenas[a]) cudaFree(b.base);
    for (cudaEvent_t e : ctx->slice_ev) cudaEventDestroy(e);
    for (cudaEvent_t e : ctx->prof_events) cudaEventDestroy(e);
    if (ctx->s_in) cudaStreamDestroy(ctx->s_in);
    if (ctx->s_out) cudaStreamDestroy(ctx->s_out);
    if (ctx->d_text) cudaFree(ctx->d_text);
    if (ctx->d_raw) cudaFree(ctx->d_raw);
    if (ctx->d_class_store) cudaFree(ctx->d_class_store);
    if (ctx->d_lex_tables) cudaFree(ctx->d_lex_tables);
    if (ctx->h_words) cudaFreeHost(ctx->h_words);
    if (ctx->h_errs) cudaFreeHost(ctx->h_errs);
    if (ctx->h_lexerrs) cudaFreeHost(ctx->h_lexerrs);
    if (ctx->h_results) cudaFreeHost(ctx->h_results);
    if (ctx->h_counters) cudaFreeHost(ctx->h_counters);
    for (int i = 0; i < 8; i++)
        if (ctx->ev[i]) cudaEventDestroy(ctx->ev[i]);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    if (ctx->live) ctx->live->ctx = nullptr;
    delete ctx;
}

const char* ptxfe_last_error(const ptxfe_ctx* ctx) { return ctx ? ctx->err : "no context"; }

// Lay the modules [m0, m1) out as one slice: module i starts at a multiple of PTX_CHUNK inside the slice.
// Returns the padded size of the slice.
static uint64_t layout_slice(ptxfe_ctx* ctx, const uint64_t* lens, uint32_t m0, uint32_t m1) {
    uint64_t off = 0, chunks = 0;
    for (uint32_t m = m0; m < m1; m++) {
        PtxModuleLayout& l = ctx->layout[m];
        l.text_off = off;
        l.text_len = lens[m];
        l.chunk_begin = (uint32_t)chunks;
        l.pad = 0;
        uint64_t c = (lens[m] + PTX_CHUNK - 1) / PTX_CHUNK;
        chunks += c;
        off += c * PTX_CHUNK;
    }
    return off;
}

static int ensure_text(ptxfe_ctx* ctx, uint64_t bytes) {
    if (bytes + 256 > ctx->d_text_cap) {
        if (ctx->d_text) cudaFree(ctx->d_text);
        ctx->d_text = nullptr;
        ctx->d_text_cap = 0;
        size_t cap = bytes + bytes / 8 + 4096;
        CUDA_TRY(cudaMalloc((void**)&ctx->d_text, cap));
        ctx->d_text_cap = cap;
    }
    return PTXFE_OK;
}

int ptxfe_stage(ptxfe_ctx* ctx, const char* const* texts, const uint64_t* lens, uint32_t n) {
    if (!ctx || (n && (!texts || !lens))) return PTXFE_ERR_BAD_ARG;
    CUDA_TRY(cudaSetDevice(ctx->device));
    ctx->failed = false;
    ctx->staged = ctx->ran = false;
    ctx->texts.assign(texts, texts + n);
    ctx->layout.resize(n);
    uint64_t total = 0;
    for (uint32_t m = 0; m < n; m++) total += lens[m];
    uint64_t off = layout_slice(ctx, lens, 0, n);
    if (off >= 0xFFFFFF00ull) return PTXFE_ERR_TOO_LARGE;
    ctx->text_bytes = total;
    ctx->padded_bytes = off;
    int st = ensure_text(ctx, off);
    if (st != PTXFE_OK) return st;
    CUDA_TRY(cudaEventRecord(ctx->ev[0], ctx->stream));
    for (uint32_t m = 0; m < n; m++)
        if (lens[m])
            CUDA_TRY(cudaMemcpyAsync(ctx->d_text + ctx->layout[m].text_off, texts[m], lens[m], cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(cudaEventRecord(ctx->ev[1], ctx->stream));
    CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(cudaEventElapsedTime(&ctx->stats.h2d_ms, ctx->ev[0], ctx->ev[1]));
    ctx->stats.h2d_bytes = total;
    ctx->stats.text_bytes = total;
    ctx->stats.n_modules = n;
    ctx->staged = true;
    return PTXFE_OK;
}

// The three stages over one slice: `text` is the slice's text on the device, `layout` its n module layouts (host).
// Uses the current arena; leaves the device results in ctx->work and the totals in ctx->counters.  Returns after
// the kernels have finished.
static int run_pipeline(ptxfe_ctx* ctx, uint8_t* text, const PtxModuleLayout* layout, uint32_t n, uint32_t mode,
                        cudaEvent_t ev_begin, cudaEvent_t ev_lex, cudaEvent_t ev_structure, cudaEvent_t ev_end,
                        const RepackModule* repack = nullptr, const uint8_t* raw = nullptr, bool first_slice = true) {
    CudaBackend bk{ctx};
    bk.reset();
    ctx->mcb.resize((size_t)n + 1);
    uint32_t chunks = 0;
    for (uint32_t m = 0; m < n; m++) {
        ctx->mcb[m] = layout[m].chunk_begin;
        chunks = layout[m].chunk_begin + (uint32_t)((layout[m].text_len + PTX_CHUNK - 1) / PTX_CHUNK);
    }
    ctx->mcb[n] = chunks;
    PtxWork& w = ctx->work;
    w = PtxWork();
    w.first_slice = first_slice;
    if (const char* e = getenv("PTXFE_SEQ_MAX_TOKENS")) w.seq_max_tokens = (uint32_t)strtoul(e, nullptr, 10);
    w.text = text;
    w.n_modules = n;
    w.n_chunks = chunks;
    w.layout = (PtxModuleLayout*)bk.alloc(sizeof(PtxModuleLayout) * ((size_t)n + 1));
    w.mod_chunk_begin = (uint32_t*)bk.alloc(sizeof(uint32_t) * ((size_t)n + 2));
    w.results = (PtxModuleResult*)bk.alloc(sizeof(PtxModuleResult) * ((size_t)n + 1));
    w.counters = (PtxCounters*)bk.alloc(sizeof(PtxCounters));
    if (ctx->failed) return PTXFE_ERR_OOM;
    CUDA_TRY(cudaEventRecord(ev_begin, ctx->stream));
    if (n) CUDA_TRY(cudaMemcpyAsync(w.layout, layout, sizeof(PtxModuleLayout) * n, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(cudaMemcpyAsync(w.mod_chunk_begin, ctx->mcb.data(), sizeof(uint32_t) * ((size_t)n + 1), cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(cudaMemsetAsync(w.counters, 0, sizeof(PtxCounters), ctx->stream));
    // layout and mcb are pageable host memory: the copies above have consumed them when the calls return
    if (repack && chunks) {
        RepackModule* d_mods = (RepackModule*)bk.alloc(sizeof(RepackModule) * (size_t)n);
        if (ctx->failed) return PTXFE_ERR_OOM;
        CUDA_TRY(cudaMemcpyAsync(d_mods, repack, sizeof(RepackModule) * (size_t)n, cudaMemcpyHostToDevice, ctx->stream));
        uint32_t pieces = chunks * (PTX_CHUNK / 16);
        repack_text_kernel<<<(pieces + 255) / 256, 256, 0, ctx->stream>>>(pieces, n, d_mods, w.mod_chunk_begin, raw, text);
        ctx->launches++;
    }
    memset(&ctx->counters, 0, sizeof ctx->counters);
    ptx_stage_lex(bk, w, ctx->counters);
    if (ev_lex) CUDA_TRY(cudaEventRecord(ev_lex, ctx->stream));
    if (!ctx->failed) ptx_stage_structure(bk, w, ctx->counters, mode);
    if (ev_structure) CUDA_TRY(cudaEventRecord(ev_structure, ctx->stream));
    if (!ctx->failed) ptx_stage_decode(bk, w, ctx->counters);
    CUDA_TRY(cudaEventRecord(ev_end, ctx->stream));
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(ctx->err, sizeof ctx->err, "pipeline failed: %s", cudaGetErrorString(e));
        return PTXFE_ERR_CUDA;
    }
    if (ctx->failed) return strstr(ctx->err, "cudaMalloc") ? PTXFE_ERR_OOM : PTXFE_ERR_CUDA;
    return PTXFE_OK;
}

static void collect_profile(ptxfe_ctx* ctx) {
    if (!ctx->profile) return;
    ctx->prof_text.clear();
    for (size_t i = 0; i < ctx->prof_names.size(); i++) {
        float ms = 0;
        cudaEventElapsedTime(&ms, ctx->prof_events[2 * i], ctx->prof_events[2 * i + 1]);
        char line[160];
        snprintf(line, sizeof line, "%s %.6f\n", ctx->prof_names[i], ms);
        ctx->prof_text += line;
    }
}

int ptxfe_run(ptxfe_ctx* ctx, uint32_t mode) {
    if (!ctx || !ctx->staged || mode > 2) return PTXFE_ERR_BAD_ARG;
    CUDA_TRY(cudaSetDevice(ctx->device));
    if (ctx->live) { ctx->live->ctx = nullptr; ctx->live = nullptr; }
    ctx->failed = false;
    ctx->launches = 0;
    ctx->prof_used = 0;
    ctx->prof_names.clear();
    ctx->mode = mode;
    ctx->cur = 0;
    uint32_t n = (uint32_t)ctx->layout.size();
    int st = run_pipeline(ctx, ctx->d_text, ctx->layout.data(), n, mode, ctx->ev[2], ctx->ev[3], ctx->ev[4], ctx->ev[5]);
    if (st != PTXFE_OK) return st;
    ptxfe_stats& s = ctx->stats;
    cudaEventElapsedTime(&s.kernel_ms, ctx->ev[2], ctx->ev[5]);
    cudaEventElapsedTime(&s.lex_ms, ctx->ev[2], ctx->ev[3]);
    cudaEventElapsedTime(&s.structure_ms, ctx->ev[3], ctx->ev[4]);
    cudaEventElapsedTime(&s.decode_ms, ctx->ev[4], ctx->ev[5]);
    s.n_tokens = ctx->counters.n_tokens;
    s.n_units = ctx->counters.n_units;
    s.n_result_words = ctx->counters.n_words;
    s.n_errors = ctx->counters.n_errs;
    s.n_lex_errors = ctx->counters.n_lexerrs;
    s.n_kernel_launches = ctx->launches;
    s.n_sequential = 0;
    s.n_sequential_tokens = 0;
    s.n_classes = ctx->counters.n_classes;
    s.n_class_capacity = PTX_MAX_CLASSES;
    s.n_untemplated = ctx->counters.n_rest;
    s.n_signature_words = ctx->counters.n_sig_words;
    s.n_signature_capacity = PTX_SIG_POOL_WORDS;
    ctx->ran = true;
    collect_profile(ctx);
    return PTXFE_OK;
}

const char* ptxfe_profile(const ptxfe_ctx* ctx) { return ctx ? ctx->prof_text.c_str() : ""; }

// Grow a pinned host buffer, keeping its first `keep` bytes.  Copies that target the old buffer must have finished.
static int grow_pinned(ptxfe_ctx* ctx, void** p, size_t* cap, size_t need, size_t keep) {
    if (need <= *cap) return PTXFE_OK;
    void* np = nullptr;
    size_t sz = need + need / 4 + 4096;
    CUDA_TRY(cudaMallocHost(&np, sz));
    if (*p && keep) memcpy(np, *p, keep);
    if (*p) cudaFreeHost(*p);
    *p = np;
    *cap = sz;
    return PTXFE_OK;
}

static ptxfe_batch* make_batch(ptxfe_ctx* ctx, uint32_t n) {
    ptxfe_batch* b = new ptxfe_batch();
    b->ctx = ctx;
    b->n = n;
    b->mode = ctx->mode;
    b->texts = ctx->texts;
    b->layout = ctx->layout;
    b->results.assign((PtxModuleResult*)ctx->h_results, (PtxModuleResult*)ctx->h_results + n);
    b->status.assign(n, -1);
    b->words = (const uint32_t*)ctx->h_words;
    b->errs = (const PtxErrRec*)ctx->h_errs;
    b->lexerrs = (const uint32_t*)ctx->h_lexerrs;
    return b;
}

int ptxfe_fetch(ptxfe_ctx* ctx, ptxfe_batch** out) {
    if (!ctx || !out || !ctx->ran) return PTXFE_ERR_BAD_ARG;
    *out = nullptr;
    CUDA_TRY(cudaSetDevice(ctx->device));
    const PtxCounters& c = ctx->counters;
    uint32_t n = (uint32_t)ctx->layout.size();
    size_t wb = sizeof(uint32_t) * (size_t)c.n_words, eb = sizeof(PtxErrRec) * (size_t)c.n_errs;
    size_t lb = sizeof(uint32_t) * 2 * (size_t)c.n_lexerrs, rb = sizeof(PtxModuleResult) * (size_t)n;
    int st;
    if ((st = grow_pinned(ctx, &ctx->h_words, &ctx->h_words_cap, wb + 16, 0)) != PTXFE_OK) return st;
    if ((st = grow_pinned(ctx, &ctx->h_errs, &ctx->h_errs_cap, eb + 16, 0)) != PTXFE_OK) return st;
    if ((st = grow_pinned(ctx, &ctx->h_lexerrs, &ctx->h_lexerrs_cap, lb + 16, 0)) != PTXFE_OK) return st;
    if ((st = grow_pinned(ctx, &ctx->h_results, &ctx->h_results_cap, rb + 16, 0)) != PTXFE_OK) return st;
    CUDA_TRY(cudaEventRecord(ctx->ev[6], ctx->stream));
    if (wb) CUDA_TRY(cudaMemcpyAsync(ctx->h_words, ctx->work.words, wb, cudaMemcpyDeviceToHost, ctx->stream));
    if (eb) CUDA_TRY(cudaMemcpyAsync(ctx->h_errs, ctx->work.errs, eb, cudaMemcpyDeviceToHost, ctx->stream));
    if (lb) CUDA_TRY(cudaMemcpyAsync(ctx->h_lexerrs, ctx->work.lexerrs, lb, cudaMemcpyDeviceToHost, ctx->stream));
    if (rb) CUDA_TRY(cudaMemcpyAsync(ctx->h_results, ctx->work.results, rb, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(cudaEventRecord(ctx->ev[7], ctx->stream));
    CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(cudaEventElapsedTime(&ctx->stats.d2h_ms, ctx->ev[6], ctx->ev[7]));
    ctx->stats.d2h_bytes = wb + eb + lb + rb;
    ptxfe_batch* b = make_batch(ctx, n);
    uint64_t seq = 0, seq_tokens = 0;
    for (uint32_t m = 0; m < n; m++) { seq += b->results[m].sequential; seq_tokens += b->results[m].seq_tokens; }
    ctx->stats.n_sequential = seq;
    ctx->stats.n_sequential_tokens = seq_tokens;
    ctx->live = b;
    *out = b;
    return PTXFE_OK;
}

// One call, host text in, host records out.  The batch is cut into slices of whole modules; the text of slice k+1
// travels to the device and the records of slice k-1 travel back while the kernels of slice k run (three streams,
// two working arenas).  Text offsets inside the records are relative to the slice, as ptxfe_module_records reports.
int ptxfe_parse_batch(ptxfe_ctx* ctx, const char* const* texts, const uint64_t* lens, uint32_t n, uint32_t mode, ptxfe_batch** out) {
    if (!out) return PTXFE_ERR_BAD_ARG;
    *out = nullptr;
    if (!ctx || (n && (!texts || !lens)) || mode > 2) return PTXFE_ERR_BAD_ARG;
    CUDA_TRY(cudaSetDevice(ctx->device));
    if (ctx->live) { ctx->live->ctx = nullptr; ctx->live = nullptr; }
    ctx->failed = false;
    ctx->staged = ctx->ran = false;
    ctx->launches = 0;
    ctx->prof_used = 0;
    ctx->prof_names.clear();
    ctx->mode = mode;
    ctx->texts.assign(texts, texts + n);
    ctx->layout.resize(n);
    // ---- slices
    // Small slices at both ends (the first text copy and the last result copy overlap with nothing), large ones in
    // between (every slice costs a few host synchronisations and ~70 launches).  PTXFE_SLICE_BYTES forces one size.
    uint64_t grand_total = 0;
    for (uint32_t m = 0; m < n; m++) grand_total += lens[m];
    uint64_t edge = (uint64_t)32 << 20, div = 8;
    if (const char* e = getenv("PTXFE_SLICE_DIV")) { uint64_t v = strtoull(e, nullptr, 10); if (v) div = v; }
    uint64_t middle = grand_total / div;
    if (middle < ((uint64_t)64 << 20)) middle = (uint64_t)64 << 20;
    if (middle > ((uint64_t)512 << 20)) middle = (uint64_t)512 << 20;
    if (const char* e = getenv("PTXFE_SLICE_BYTES")) {
        uint64_t v = strtoull(e, nullptr, 10);
        if (v) edge = middle = v;
    }
    struct Slice { uint32_t m0, m1; uint64_t text_off, padded, bytes; };
    std::vector<Slice> slices;
    uint64_t total = 0, text_off = 0;
    for (uint32_t m = 0; m < n;) {
        uint64_t left = grand_total - total;
        uint64_t target = slices.empty() ? edge : middle;
        if (!slices.empty() && left > edge && left <= middle + edge) target = left - edge;   // leave a small last slice
        uint32_t m1 = m;
        uint64_t bytes = 0;
        while (m1 < n && (m1 == m || bytes + lens[m1] <= target)) bytes += lens[m1++];
        uint64_t padded = layout_slice(ctx, lens, m, m1);
        if (padded >= 0xFFFFFF00ull) return PTXFE_ERR_TOO_LARGE;
        slices.push_back(Slice{m, m1, text_off, padded, bytes});
        text_off += padded;
        total += bytes;
        m = m1;
    }
    if (slices.empty()) slices.push_back(Slice{0, 0, 0, 0, 0});
    const size_t ns = slices.size();
    int st = ensure_text(ctx, text_off);
    if (st != PTXFE_OK) return st;
    while (ctx->slice_ev.size() < ns * 5) {
        cudaEvent_t e;
        CUDA_TRY(cudaEventCreate(&e));
        ctx->slice_ev.push_back(e);
    }
    // ---- text copies, in slice order, on their own stream; submitted two slices ahead of the kernels.
    // Modules that follow one another in host memory travel as one copy into a raw buffer and are moved to their
    // chunk-aligned slots by a kernel; modules scattered over the host are copied straight into their slots.
    std::vector<RepackModule> repack(n);
    std::vector<uint64_t> raw_base(ns, 0);
    std::vector<char> use_raw(ns, 0);
    uint64_t raw_total = 0;
    for (size_t k = 0; k < ns; k++) {
        const Slice& sl = slices[k];
        uint32_t runs = 0;
        for (uint32_t m = sl.m0; m < sl.m1; m++)
            if (m == sl.m0 || texts[m] != texts[m - 1] + lens[m - 1]) runs++;
        if (runs * 2 <= sl.m1 - sl.m0) {
            use_raw[k] = 1;
            raw_base[k] = raw_total;
            raw_total += ((sl.bytes + 15) & ~(uint64_t)15) + 16 * (uint64_t)runs;
        }
    }
    if (raw_total + 64 > ctx->d_raw_cap) {
        if (ctx->d_raw) cudaFree(ctx->d_raw);
        ctx->d_raw = nullptr;
        ctx->d_raw_cap = 0;
        size_t cap = raw_total + raw_total / 8 + 4096;
        CUDA_TRY(cudaMalloc((void**)&ctx->d_raw, cap));
        ctx->d_raw_cap = cap;
    }
    auto submit_text = [&](size_t k) -> int {
        const Slice& sl = slices[k];
        if (k == 0) CUDA_TRY(cudaEventRecord(ctx->ev[0], ctx->s_in));
        if (use_raw[k]) {
            uint64_t at = 0;     // offset of the current run inside the slice's raw region (multiple of 16)
            for (uint32_t m = sl.m0; m < sl.m1;) {
                uint32_t e = m + 1;
                uint64_t bytes = lens[m];
                while (e < sl.m1 && texts[e] == texts[e - 1] + lens[e - 1]) bytes += lens[e++];
                if (bytes) CUDA_TRY(cudaMemcpyAsync(ctx->d_raw + raw_base[k] + at, texts[m], bytes, cudaMemcpyHostToDevice, ctx->s_in));
                for (uint32_t j = m; j < e; j++) {
                    repack[j].chunk_begin = ctx->layout[j].chunk_begin;
                    repack[j].raw_off = (uint32_t)(at + (uint64_t)(texts[j] - texts[m]));
                    repack[j].len = (uint32_t)lens[j];
                }
                at += (bytes + 15) & ~(uint64_t)15;
                m = e;
            }
        } else {
            for (uint32_t m = sl.m0; m < sl.m1; m++)
                if (lens[m])
                    CUDA_TRY(cudaMemcpyAsync(ctx->d_text + sl.text_off + ctx->layout[m].text_off, texts[m], lens[m], cudaMemcpyHostToDevice, ctx->s_in));
        }
        CUDA_TRY(cudaEventRecord(ctx->slice_ev[5 * k], ctx->s_in));
        if (k + 1 == ns) CUDA_TRY(cudaEventRecord(ctx->ev[1], ctx->s_in));
        return PTXFE_OK;
    };
    // From here on copies may be in flight that read the caller's text and write the pinned result buffers: every error
    // exit waits for all three streams first, so that the caller may free `texts` as soon as the call returns.
    auto drain = [&](int code) -> int {
        cudaStreamSynchronize(ctx->s_in);
        cudaStreamSynchronize(ctx->s_out);
        cudaStreamSynchronize(ctx->stream);
        return code;
    };
#define DRAIN_TRY(call)                                                                     \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess) {                                                            \
            snprintf(ctx->err, sizeof ctx->err, "%s: %s", #call, cudaGetErrorString(e_));   \
            return drain(PTXFE_ERR_CUDA);                                                   \
        }                                                                                   \
    } while (0)
    for (size_t k = 0; k < ns && k < 2; k++)
        if ((st = submit_text(k)) != PTXFE_OK) return drain(st);
    // ---- host result buffers: sized from the text; grown (after the copies in flight have landed) if a slice needs more
    int rc;
    if ((rc = grow_pinned(ctx, &ctx->h_results, &ctx->h_results_cap, sizeof(PtxModuleResult) * (size_t)n + 16, 0)) != PTXFE_OK) return drain(rc);
    if ((rc = grow_pinned(ctx, &ctx->h_words, &ctx->h_words_cap, (size_t)(total * 2) + 4096, 0)) != PTXFE_OK) return drain(rc);
    size_t words_done = 0, errs_done = 0, lexerrs_done = 0;
    std::vector<size_t> base_w(ns), base_e(ns), base_l(ns);
    ptxfe_stats& s = ctx->stats;
    s.n_tokens = s.n_units = s.n_result_words = s.n_errors = s.n_lex_errors = 0;
    s.n_classes = s.n_untemplated = s.n_signature_words = 0;
    s.n_class_capacity = PTX_MAX_CLASSES;
    s.n_signature_capacity = PTX_SIG_POOL_WORDS;
    for (size_t k = 0; k < ns; k++) {
        const Slice& sl = slices[k];
        ctx->cur = (int)(k & 1);
        // this arena held the results of slice k-2: wait until they have left the device
        if (k >= 2) DRAIN_TRY(cudaEventSynchronize(ctx->slice_ev[5 * (k - 2) + 4]));
        DRAIN_TRY(cudaStreamWaitEvent(ctx->stream, ctx->slice_ev[5 * k], 0));
        if (k + 2 < ns && (rc = submit_text(k + 2)) != PTXFE_OK) return drain(rc);
        rc = run_pipeline(ctx, ctx->d_text + sl.text_off, ctx->layout.data() + sl.m0, sl.m1 - sl.m0, mode,
                          ctx->slice_ev[5 * k + 1], nullptr, nullptr, ctx->slice_ev[5 * k + 2],
                          use_raw[k] ? repack.data() + sl.m0 : nullptr, ctx->d_raw + raw_base[k], k == 0);
        if (rc != PTXFE_OK) return drain(rc);
        const PtxCounters& c = ctx->counters;
        size_t nw = c.n_words, ne = c.n_errs, nl = c.n_lexerrs, nm = sl.m1 - sl.m0;
        if ((words_done + nw) * sizeof(uint32_t) + 16 > ctx->h_words_cap || (errs_done + ne) * sizeof(PtxErrRec) + 16 > ctx->h_errs_cap ||
            (lexerrs_done + nl) * 8 + 16 > ctx->h_lexerrs_cap) {
            DRAIN_TRY(cudaStreamSynchronize(ctx->s_out));
            // extrapolate from what the slices so far produced
            double done_bytes = 0;
            for (size_t j = 0; j <= k; j++) done_bytes += (double)slices[j].bytes;
            double scale = done_bytes > 0 ? (double)total / done_bytes * 1.1 : 1.0;
            if ((rc = grow_pinned(ctx, &ctx->h_words, &ctx->h_words_cap, (size_t)((words_done + nw) * scale) * 4 + 4096, words_done * 4)) != PTXFE_OK) return drain(rc);
            if ((rc = grow_pinned(ctx, &ctx->h_errs, &ctx->h_errs_cap, (size_t)((errs_done + ne) * scale) * sizeof(PtxErrRec) + 4096, errs_done * sizeof(PtxErrRec))) != PTXFE_OK) return drain(rc);
            if ((rc = grow_pinned(ctx, &ctx->h_lexerrs, &ctx->h_lexerrs_cap, (size_t)((lexerrs_done + nl) * scale) * 8 + 4096, lexerrs_done * 8)) != PTXFE_OK) return drain(rc);
        }
        // the kernels of this slice have finished (run_pipeline waits for them)
        DRAIN_TRY(cudaEventRecord(ctx->slice_ev[5 * k + 3], ctx->s_out));
        if (nw) DRAIN_TRY(cudaMemcpyAsync((uint32_t*)ctx->h_words + words_done, ctx->work.words, nw * 4, cudaMemcpyDeviceToHost, ctx->s_out));
        if (ne) DRAIN_TRY(cudaMemcpyAsync((PtxErrRec*)ctx->h_errs + errs_done, ctx->work.errs, ne * sizeof(PtxErrRec), cudaMemcpyDeviceToHost, ctx->s_out));
        if (nl) DRAIN_TRY(cudaMemcpyAsync((uint32_t*)ctx->h_lexerrs + 2 * lexerrs_done, ctx->work.lexerrs, nl * 8, cudaMemcpyDeviceToHost, ctx->s_out));
        if (nm) DRAIN_TRY(cudaMemcpyAsync((PtxModuleResult*)ctx->h_results + sl.m0, ctx->work.results, nm * sizeof(PtxModuleResult), cudaMemcpyDeviceToHost, ctx->s_out));
        DRAIN_TRY(cudaEventRecord(ctx->slice_ev[5 * k + 4], ctx->s_out));
        if (words_done + nw > 0xFFFFFFFFull) return drain(PTXFE_ERR_TOO_LARGE);   // module results index words with 32 bits
        base_w[k] = words_done; base_e[k] = errs_done; base_l[k] = lexerrs_done;
        words_done += nw; errs_done += ne; lexerrs_done += nl;
        s.n_tokens += c.n_tokens;
        s.n_units += c.n_units;
        s.n_result_words += nw;
        s.n_errors += ne;
        s.n_lex_errors += nl;
        s.n_untemplated += c.n_rest;
        s.n_classes = c.n_classes;
        s.n_signature_words = c.n_sig_words;
    }
    DRAIN_TRY(cudaStreamSynchronize(ctx->s_out));
    DRAIN_TRY(cudaStreamSynchronize(ctx->s_in));
#undef DRAIN_TRY
    // ---- module results index the batch-wide host arrays
    PtxModuleResult* res = (PtxModuleResult*)ctx->h_results;
    uint64_t seq = 0, seq_tokens = 0;
    for (size_t k = 0; k < ns; k++)
        for (uint32_t m = slices[k].m0; m < slices[k].m1; m++) {
            res[m].word_begin += (uint32_t)base_w[k]; res[m].word_end += (uint32_t)base_w[k];
            res[m].err_begin += (uint32_t)base_e[k]; res[m].err_end += (uint32_t)base_e[k];
            res[m].lexerr_begin += (uint32_t)base_l[k]; res[m].lexerr_end += (uint32_t)base_l[k];
            seq += res[m].sequential;
            seq_tokens += res[m].seq_tokens;
        }
    // ---- statistics: busy time of each of the three streams
    cudaEventElapsedTime(&s.h2d_ms, ctx->ev[0], ctx->ev[1]);
    s.kernel_ms = s.d2h_ms = 0;
    s.lex_ms = s.structure_ms = s.decode_ms = 0;
    for (size_t k = 0; k < ns; k++) {
        float ms = 0;
        cudaEventElapsedTime(&ms, ctx->slice_ev[5 * k + 1], ctx->slice_ev[5 * k + 2]);
        s.kernel_ms += ms;
        cudaEventElapsedTime(&ms, ctx->slice_ev[5 * k + 3], ctx->slice_ev[5 * k + 4]);
        s.d2h_ms += ms;
    }
    if (getenv("PTXFE_TRACE")) {
        // device-side timeline of the three streams, milliseconds since the first text copy was submitted
        for (size_t k = 0; k < ns; k++) {
            float t[5];
            for (int j = 0; j < 5; j++) cudaEventElapsedTime(&t[j], ctx->ev[0], ctx->slice_ev[5 * k + j]);
            fprintf(stderr, "ptxfe slice %zu: text arrived %.2f, kernels %.2f - %.2f, results %.2f - %.2f\n", k, t[0], t[1], t[2], t[3], t[4]);
        }
    }
    s.h2d_bytes = total;
    s.text_bytes = total;
    s.n_modules = n;
    s.d2h_bytes = words_done * 4 + errs_done * sizeof(PtxErrRec) + lexerrs_done * 8 + sizeof(PtxModuleResult) * (size_t)n;
    s.n_kernel_launches = ctx->launches;
    s.n_sequential = seq;
    s.n_sequential_tokens = seq_tokens;
    collect_profile(ctx);
    ptxfe_batch* b = make_batch(ctx, n);
    ctx->live = b;
    *out = b;
    return PTXFE_OK;
}

void ptxfe_batch_free(ptxfe_batch* b) {
    if (!b) return;
    for (ptxfe_batch* p : b->parts) ptxfe_batch_free(p);
    if (b->ctx && b->ctx->live == b) b->ctx->live = nullptr;
    delete b;
}
uint32_t ptxfe_batch_size(const ptxfe_batch* b) { return b ? b->n : 0; }
// module i of a batch that was parsed on several devices lives in one of its parts
#define PTXFE_ROUTE(b, i, fn, ...)                                                                   \
    if ((b) && !(b)->parts.empty()) {                                                                \
        if ((i) >= (b)->n) return PTXFE_ERR_BAD_ARG;                                                 \
        return fn((b)->parts[(b)->where[(i)].first], (b)->where[(i)].second, ##__VA_ARGS__);         \
    }
void ptxfe_get_stats(const ptxfe_ctx* ctx, ptxfe_stats* out) {
    if (ctx && out) *out = ctx->stats;
}

static PtxBatchView view_of(const ptxfe_batch* b) {
    PtxBatchView v;
    v.n_modules = b->n;
    v.mode = b->mode;
    v.layout = b->layout.data();
    v.results = b->results.data();
    v.words = b->words;
    v.errs = b->errs;
    v.lexerrs = b->lexerrs;
    v.texts = b->texts.data();
    return v;
}

int ptxfe_module_dump(const ptxfe_batch* b, uint32_t i, char** out, uint64_t* out_len) {
    PTXFE_ROUTE(b, i, ptxfe_module_dump, out, out_len)
    if (!b || !b->ctx || i >= b->n || !out) return PTXFE_ERR_BAD_ARG;
    int status = 0;
    // records -> tree -> text (the hash below walks the records directly: both readers must tell the same story)
    std::string s = ptxfe_dump_module_tree_impl(view_of(b), i, &status);
    char* r = (char*)malloc(s.size() + 1);
    if (!r) return PTXFE_ERR_OOM;
    memcpy(r, s.data(), s.size() + 1);
    *out = r;
    if (out_len) *out_len = s.size();
    return PTXFE_OK;
}

int ptxfe_module_dump_hash(const ptxfe_batch* b, uint32_t i, uint64_t* out_hash) {
    PTXFE_ROUTE(b, i, ptxfe_module_dump_hash, out_hash)
    if (!b || !b->ctx || i >= b->n || !out_hash) return PTXFE_ERR_BAD_ARG;
    int status = 0;
    *out_hash = ptxfe_dump_hash_impl(view_of(b), i, &status);
    return PTXFE_OK;
}

// The verdict and the error count come from the module's result row (filled on the device): no record is read.
int ptxfe_module_status(const ptxfe_batch* b, uint32_t i) {
    if (b && !b->parts.empty()) return i < b->n ? ptxfe_module_status(b->parts[b->where[i].first], b->where[i].second) : PTXFE_MODULE_ERR;
    if (!b || !b->ctx || i >= b->n) return PTXFE_MODULE_ERR;
    const PtxModuleResult& r = b->results[i];
    const uint32_t n_lex = r.lexerr_end - r.lexerr_begin;
    if (n_lex && b->mode != PTXFE_ERRORS_ONLY) return PTXFE_MODULE_ERR;      // not parsed (lib.rs:447-449, 487-489)
    if (r.sequential && (r.status & US_MASK) == US_DIVERGE) return PTXFE_MODULE_REF_DIVERGES;
    if (r.sequential && (r.status & US_MASK) == US_REFUSED) return PTXFE_MODULE_SEQ_REFUSED;
    if (r.sequential && (r.status & US_MASK) == US_PANIC) return PTXFE_MODULE_REF_PANICS;
    if (b->mode == PTXFE_ERRORS_ONLY) return PTXFE_MODULE_ERR;               // no module is returned in this mode
    const bool parsed_ok = r.word_end > r.word_begin && !(r.status & US_MODULE_FAILED);
    if (b->mode == PTXFE_UNCHECKED) return parsed_ok ? PTXFE_MODULE_OK : PTXFE_MODULE_ERR;
    return (parsed_ok && r.n_errors == 0 && n_lex == 0) ? PTXFE_MODULE_OK : PTXFE_MODULE_ERR;
}

uint32_t ptxfe_module_error_count(const ptxfe_batch* b, uint32_t i) {
    if (b && !b->parts.empty()) return i < b->n ? ptxfe_module_error_count(b->parts[b->where[i].first], b->where[i].second) : 0u;
    if (!b || !b->ctx || i >= b->n) return 0;
    const PtxModuleResult& r = b->results[i];
    const uint32_t n_lex = r.lexerr_end - r.lexerr_begin;
    if (n_lex && b->mode != PTXFE_ERRORS_ONLY) return n_lex;
    if (r.sequential && ((r.status & US_MASK) == US_DIVERGE || (r.status & US_MASK) == US_REFUSED)) return 0;
    // a module without tokens: the implicit Parser error of the reference (the header does not parse)
    return n_lex + r.n_errors + (r.word_end == r.word_begin ? 1u : 0u);
}

int ptxfe_module_records(const ptxfe_batch* b, uint32_t i, const uint32_t** words, uint64_t* n_words, uint64_t* text_base) {
    PTXFE_ROUTE(b, i, ptxfe_module_records, words, n_words, text_base)
    if (!b || !b->ctx || i >= b->n) return PTXFE_ERR_BAD_ARG;
    if (words) *words = b->words + b->results[i].word_begin;
    if (n_words) *n_words = b->results[i].word_end - b->results[i].word_begin;
    if (text_base) *text_base = b->layout[i].text_off;
    return PTXFE_OK;
}

// Builds the tree of every module of the batch (and drops it again), modules spread over n_threads host threads: the
// cost a caller pays after the parse call to hold ast-like structures instead of flat records.
int ptxfe_batch_materialize(const ptxfe_batch* b, uint32_t n_threads, uint64_t* n_nodes) {
    if (!b) return PTXFE_ERR_BAD_ARG;
    if (n_threads == 0) n_threads = 1;
    std::vector<uint64_t> nodes(n_threads, 0);
    std::vector<std::thread> threads;
    std::atomic<uint32_t> next{0};
    for (uint32_t t = 0; t < n_threads; t++)
        threads.emplace_back([&, t]() {
            for (;;) {
                const uint32_t i = next.fetch_add(1);
                if (i >= b->n) return;
                const ptxfe_batch* part = b->parts.empty() ? b : b->parts[b->where[i].first];
                const uint32_t j = b->parts.empty() ? i : b->where[i].second;
                nodes[t] += ptxfe_materialize_impl(view_of(part), j);
            }
        });
    for (std::thread& t : threads) t.join();
    uint64_t total = 0;
    for (uint64_t x : nodes) total += x;
    if (n_nodes) *n_nodes = total;
    return PTXFE_OK;
}

void ptxfe_free(void* p) { free(p); }

// ------------------------------------------------------------------------------------------------ several devices
struct ptxfe_multi {
    std::vector<ptxfe_ctx*> ctxs;
    std::vector<ptxfe_stats> stats;
    char err[512] = {0};
};

int ptxfe_multi_create(const int* devices, uint32_t n_devices, ptxfe_multi** out) {
    if (!out || !devices || n_devices == 0) return PTXFE_ERR_BAD_ARG;
    *out = nullptr;
    ptxfe_multi* m = new ptxfe_multi();
    for (uint32_t k = 0; k < n_devices; k++) {
        ptxfe_ctx* c = nullptr;
        int st = ptxfe_create(devices[k], &c);
        if (st != PTXFE_OK) {
            ptxfe_multi_destroy(m);
            return st;
        }
        m->ctxs.push_back(c);
    }
    m->stats.resize(n_devices);
    memset(m->stats.data(), 0, sizeof(ptxfe_stats) * n_devices);
    *out = m;
    return PTXFE_OK;
}
void ptxfe_multi_destroy(ptxfe_multi* m) {
    if (!m) return;
    for (ptxfe_ctx* c : m->ctxs) ptxfe_destroy(c);
    delete m;
}
const char* ptxfe_multi_last_error(const ptxfe_multi* m) { return m ? m->err : "no context"; }
uint32_t ptxfe_multi_parts(const ptxfe_multi* m) { return m ? (uint32_t)m->ctxs.size() : 0; }
void ptxfe_multi_part_stats(const ptxfe_multi* m, uint32_t part, ptxfe_stats* out) {
    if (m && out && part < m->stats.size()) *out = m->stats[part];
}
int ptxfe_multi_part_of(const ptxfe_batch* b, uint32_t i) {
    if (!b || i >= b->n) return -1;
    return b->parts.empty() ? 0 : (int)b->where[i].first;
}

int ptxfe_parse_batch_multi(ptxfe_multi* m, const char* const* texts, const uint64_t* lens, uint32_t n, uint32_t mode, ptxfe_batch** out) {
    if (!out) return PTXFE_ERR_BAD_ARG;
    *out = nullptr;
    if (!m || m->ctxs.empty() || (n && (!texts || !lens)) || mode > 2) return PTXFE_ERR_BAD_ARG;
    const uint32_t n_parts = (uint32_t)m->ctxs.size();
    PtxPartition part = ptx_partition_greedy(lens, n, n_parts);
    // every shard gets its own (char**, uint64*) arrays and its own host thread; a thread makes its context's device
    // current (ptxfe_parse_batch does) and touches nothing of the others
    std::vector<std::vector<const char*>> ptexts(n_parts);
    std::vector<std::vector<uint64_t>> plens(n_parts);
    for (uint32_t k = 0; k < n_parts; k++)
        for (uint32_t i : part.members[k]) {
            ptexts[k].push_back(texts[i]);
            plens[k].push_back(lens[i]);
        }
    std::vector<ptxfe_batch*> batches(n_parts, nullptr);
    std::vector<int> status(n_parts, PTXFE_OK);
    std::vector<std::thread> threads;
    for (uint32_t k = 0; k < n_parts; k++)
        threads.emplace_back([&, k]() {
            status[k] = ptxfe_parse_batch(m->ctxs[k], ptexts[k].data(), plens[k].data(), (uint32_t)ptexts[k].size(), mode, &batches[k]);
        });
    for (std::thread& t : threads) t.join();
    int rc = PTXFE_OK;
    for (uint32_t k = 0; k < n_parts; k++) {
        ptxfe_get_stats(m->ctxs[k], &m->stats[k]);
        if (status[k] != PTXFE_OK && rc == PTXFE_OK) {
            rc = status[k];
            snprintf(m->err, sizeof m->err, "device part %u: %s", k, ptxfe_last_error(m->ctxs[k]));
        }
    }
    if (rc != PTXFE_OK) {
        for (ptxfe_batch* b : batches) ptxfe_batch_free(b);
        return rc;
    }
    ptxfe_batch* b = new ptxfe_batch();
    b->ctx = nullptr;
    b->n = n;
    b->mode = mode;
    b->words = nullptr;
    b->errs = nullptr;
    b->lexerrs = nullptr;
    b->parts = batches;
    b->where = part.where;
    *out = b;
    return PTXFE_OK;
}

int ptxfe_lex_module(ptxfe_ctx* ctx, const char* text, uint64_t len, uint32_t** out, uint64_t* n_tokens, uint64_t* n_errors) {
    if (!ctx || !out || !n_tokens || !n_errors) return PTXFE_ERR_BAD_ARG;
    const char* texts[1] = {text};
    uint64_t lens[1] = {len};
    int st = ptxfe_stage(ctx, texts, lens, 1);
    if (st != PTXFE_OK) return st;
    CudaBackend bk{ctx};
    bk.reset();
    ctx->failed = false;
    PtxWork& w = ctx->work;
    w = PtxWork();
    w.text = ctx->d_text;
    w.n_modules = 1;
    ctx->mcb.assign({0u, (uint32_t)((len + PTX_CHUNK - 1) / PTX_CHUNK)});
    w.n_chunks = ctx->mcb[1];
    w.layout = (PtxModuleLayout*)bk.alloc(sizeof(PtxModuleLayout) * 2);
    w.mod_chunk_begin = (uint32_t*)bk.alloc(sizeof(uint32_t) * 3);
    w.results = (PtxModuleResult*)bk.alloc(sizeof(PtxModuleResult) * 2);
    w.counters = (PtxCounters*)bk.alloc(sizeof(PtxCounters));
    if (ctx->failed) return PTXFE_ERR_OOM;
    CUDA_TRY(cudaMemcpyAsync(w.layout, ctx->layout.data(), sizeof(PtxModuleLayout), cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(cudaMemcpyAsync(w.mod_chunk_begin, ctx->mcb.data(), sizeof(uint32_t) * 2, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(cudaMemsetAsync(w.counters, 0, sizeof(PtxCounters), ctx->stream));
    memset(&ctx->counters, 0, sizeof ctx->counters);
    ptx_stage_lex(bk, w, ctx->counters);
    CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (ctx->failed) return PTXFE_ERR_CUDA;
    uint32_t nt = ctx->counters.n_tokens, ne = ctx->counters.n_lexerrs;
    std::vector<PtxToken> toks(nt);
    std::vector<uint32_t> errs((size_t)ne * 2);
    if (nt) CUDA_TRY(cudaMemcpy(toks.data(), w.tokens, sizeof(PtxToken) * nt, cudaMemcpyDeviceToHost));
    if (ne) CUDA_TRY(cudaMemcpy(errs.data(), w.lexerrs, sizeof(uint32_t) * 2 * ne, cudaMemcpyDeviceToHost));
    uint32_t* r = (uint32_t*)malloc(((size_t)nt * 3 + (size_t)ne * 2 + 1) * 4);
    if (!r) return PTXFE_ERR_OOM;
    size_t k = 0;
    for (uint32_t i = 0; i < nt; i++) {
        r[k++] = toks[i].kind;
        r[k++] = toks[i].start;
        r[k++] = toks[i].len;   // 0xFFFF means "65535 or longer"
    }
    for (uint32_t i = 0; i < ne; i++) { r[k++] = errs[2 * i]; r[k++] = errs[2 * i + 1]; }
    *out = r;
    *n_tokens = nt;
    *n_errors = ne;
    return PTXFE_OK;
}
}   // extern "C"

// ------------------------------------------------------------------------------------------------ allocation-free lexer
// Working memory of ptxfe_lex_device_noalloc: it lives in the library image, one copy per GPU that loads the library,
// for the life of the process.  Layout (bytes): [0, 512K+4) chunk transition vectors, then the per-chunk
// token/error counts, then two levels of scan tile totals.
#define PTXFE_NOALLOC_MAX_TEXT (16u << 20)
#define PTXFE_NOALLOC_MAX_CHUNKS (PTXFE_NOALLOC_MAX_TEXT / PTX_CHUNK)
#define PTXFE_NOALLOC_SCRATCH_BYTES (2u << 20)
#define PTXFE_NOALLOC_MAX_BACK (64u << 10)
static __device__ __align__(256) unsigned char ptxfe_noalloc_scratch[PTXFE_NOALLOC_SCRATCH_BYTES];

// inclusive scan of at most SCAN_TILE * SCAN_TILE elements with caller-provided room for the tile totals
template <class T, class Ld, class St, class Op>
static void scan_in_scratch(cudaStream_t stream, size_t n, Ld ld, St st, Op op, T identity, T* partial) {
    if (n == 0) return;
    size_t tiles = (n + SCAN_TILE - 1) / SCAN_TILE;
    scan_reduce_kernel<T><<<(unsigned)tiles, SCAN_THREADS, 0, stream>>>(n, ld, op, identity, partial);
    if (tiles > 1) {
        T* partial2 = partial + tiles;   // one tile is enough for the second level
        scan_reduce_kernel<T><<<1, SCAN_THREADS, 0, stream>>>(tiles, ArrayLoad<T>{partial}, op, identity, partial2);
        scan_apply_kernel<T><<<1, SCAN_THREADS, 0, stream>>>(tiles, ArrayLoad<T>{partial}, ArrayStore<T>{partial}, op, identity, partial2);
    }
    scan_apply_kernel<T><<<(unsigned)tiles, SCAN_THREADS, 0, stream>>>(n, ld, st, op, identity, partial);
}

extern "C" int ptxfe_lex_device_noalloc(int device, const void* d_text_v, uint64_t len, void* d_tokens_v, uint64_t token_capacity,
                             uint32_t* d_counts, void* stream_v) {
    // Device addresses of the scratch array, looked up once per device.  The array's name is only a host-side handle:
    // kernels must be given the address that cudaGetSymbolAddress returns while that device is current.
    static std::atomic<unsigned char*> scratch_addr[64];
    if (!d_text_v || !d_tokens_v || !d_counts || device < 0 || device >= 64) return PTXFE_ERR_BAD_ARG;
    if (len > PTXFE_NOALLOC_MAX_TEXT) {
        fprintf(stderr, "ptxfe_lex_device_noalloc: %llu bytes of text exceed the fixed working memory (limit %u bytes)\n",
                (unsigned long long)len, PTXFE_NOALLOC_MAX_TEXT);
        return PTXFE_ERR_TOO_LARGE;
    }
    // the device is made current for the look-up and the launches and the caller's current device is put back on return
    int caller_device = -1;
    if (cudaGetDevice(&caller_device) != cudaSuccess) return PTXFE_ERR_CUDA;
    struct RestoreDevice {
        int dev;
        ~RestoreDevice() { if (dev >= 0) cudaSetDevice(dev); }
    } restore{caller_device != device ? caller_device : -1};
    if (caller_device != device && cudaSetDevice(device) != cudaSuccess) return PTXFE_ERR_CUDA;
    unsigned char* scratch = scratch_addr[device].load(std::memory_order_acquire);
    if (!scratch) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, ptxfe_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "ptxfe_lex_device_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            return PTXFE_ERR_CUDA;
        }
        scratch = (unsigned char*)p;
        scratch_addr[device].store(scratch, std::memory_order_release);      // every thread that looks it up stores the same address
    }
    cudaStream_t stream = (cudaStream_t)stream_v;
    const uint8_t* text = (const uint8_t*)d_text_v;
    PtxToken* tokens = (PtxToken*)d_tokens_v;
    const uint32_t n_chunks = (uint32_t)((len + PTX_CHUNK - 1) / PTX_CHUNK);
    unsigned char* base = scratch;
    uint32_t* vec = (uint32_t*)base;                                                    // n_chunks + 1
    PtxPair* cnt = (PtxPair*)(base + sizeof(uint32_t) * (PTXFE_NOALLOC_MAX_CHUNKS + 64));   // n_chunks + 2
    unsigned char* tail = (unsigned char*)(cnt + PTXFE_NOALLOC_MAX_CHUNKS + 64);
    uint32_t* partial_u32 = (uint32_t*)tail;                                            // <= 64 + 1 tile totals
    PtxPair* partial_pair = (PtxPair*)(tail + 4096);
    uint32_t* refused = (uint32_t*)(tail + 8192);                                       // 1 = a run of soft bytes outgrew the look-back
    if (n_chunks == 0) {
        if (cudaMemsetAsync(d_counts, 0, 2 * sizeof(uint32_t), stream) != cudaSuccess) return PTXFE_ERR_CUDA;
        return PTXFE_OK;
    }
    const uint64_t me = len;
    // every scratch word that is read below is written first by this call, so what an earlier call left behind
    // does not matter
    pf_kernel<<<(n_chunks + 255) / 256, 256, 0, stream>>>((size_t)n_chunks, [=] __device__(size_t c) {
        uint64_t cs = (uint64_t)c * PTX_CHUNK;
        uint64_t ce = cs + PTX_CHUNK < me ? cs + PTX_CHUNK : me;
        uint32_t v = cx_chunk_vector(PtxGlobalReader{text, (uint32_t)me}, (uint32_t)cs, (uint32_t)ce);
        vec[c] = c == 0 ? cx_restart(v) : v;
        if (c == 0) *refused = 0;
    });
    // The byte walk of a chunk that begins inside a run of soft bytes starts over at the head of that run: bounded
    // here, so that a module made of one enormous run cannot keep the kernels busy for hours
    auto run_too_long = [=] __device__(uint32_t cs) -> bool {
        if (cs == 0 || cs >= (uint32_t)me || !lx_soft(text[cs - 1]) || !lx_soft(text[cs])) return false;
        uint32_t q = cs - 1;
        while (q > 0 && cs - q <= PTXFE_NOALLOC_MAX_BACK && lx_soft(text[q - 1])) q--;
        return cs - q > PTXFE_NOALLOC_MAX_BACK;
    };
    scan_in_scratch<uint32_t>(stream, n_chunks, ArrayLoad<uint32_t>{vec}, ArrayStore<uint32_t>{vec}, ComposeOp(), CX_IDENTITY, partial_u32);
    pf_kernel<<<(n_chunks + 255) / 256, 256, 0, stream>>>((size_t)n_chunks, [=] __device__(size_t c) {
        uint64_t cs = (uint64_t)c * PTX_CHUNK;
        int state = c == 0 ? CX_CODE : (int)(vec[c - 1] & 7u);
        LexCountSink sink;
        if (state == CX_CODE && run_too_long((uint32_t)cs)) *refused = 1;
        else lx_chunk(PtxGlobalReader{text, (uint32_t)me}, text, 0u, (uint32_t)me, (uint32_t)cs, (uint32_t)cs + PTX_CHUNK, state, sink);
        PtxPair p;
        p.a = sink.n_tokens;
        p.b = sink.n_errors;
        cnt[c + 1] = p;
        if (c == 0) { PtxPair z; z.a = z.b = 0; cnt[0] = z; }
    });
    scan_in_scratch<PtxPair>(stream, (size_t)n_chunks + 1, ArrayLoad<PtxPair>{cnt}, ArrayStore<PtxPair>{cnt}, PairAddOp(), PtxPair{0, 0}, partial_pair);
    pf_kernel<<<(n_chunks + 255) / 256, 256, 0, stream>>>((size_t)n_chunks, [=] __device__(size_t c) {
        uint64_t cs = (uint64_t)c * PTX_CHUNK;
        int state = c == 0 ? CX_CODE : (int)(vec[c - 1] & 7u);
        LexCapSink sink;
        sink.tokens = tokens;
        sink.text = text;
        sink.next = cnt[c].a;
        sink.capacity = token_capacity;
        if (!*refused) lx_chunk(PtxGlobalReader{text, (uint32_t)me}, text, 0u, (uint32_t)me, (uint32_t)cs, (uint32_t)cs + PTX_CHUNK, state, sink);
        if (c == 0) {
            d_counts[0] = *refused ? 0xFFFFFFFFu : cnt[n_chunks].a;
            d_counts[1] = *refused ? 0xFFFFFFFFu : cnt[n_chunks].b;
        }
    });
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "ptxfe_lex_device_noalloc: launch failed: %s\n", cudaGetErrorString(e));
        return PTXFE_ERR_CUDA;
    }
    return PTXFE_OK;
}
