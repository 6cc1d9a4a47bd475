/* ptxfe - a GPU-resident PTX front end (text -> directive / instruction records).  C ABI.
 *
 * Drop-in boundary for the three public entry points of ZLUDA's ptx_parser crate.  Those are plain Rust functions
 * (no FFI layer exists in the reference); a binding crate would declare the functions below `extern "C"` and
 * rebuild `ast::Module` from the records (zluda_b200/csrc/ptx_dump.h is a complete reader of them).
 *
 *   reference (ptx_parser/src/lib.rs)                                  here
 *   parse_module_checked(text)   -> Result<Module, Vec<PtxError>>      ptxfe_parse_batch(.., PTXFE_CHECKED, ..)     lib.rs:428-468
 *   parse_module_unchecked(text) -> Module                             ptxfe_parse_batch(.., PTXFE_UNCHECKED, ..)   lib.rs:470-501
 *   parse_for_errors(text)       -> Vec<PtxError>                      ptxfe_parse_batch(.., PTXFE_ERRORS_ONLY, ..) lib.rs:392-411
 *
 * The reference parses one module per call on one CPU thread; its only batch caller (zluda_precompile/src/main.rs:57-64)
 * fans modules out over a thread pool.  Here a call takes a whole batch of independent modules and processes it on one
 * GPU.  All work happens on the device; there is no CPU parsing path, and every function fails with PTXFE_ERR_CUDA when
 * no device is usable.
 *
 * Ownership: the caller keeps `texts` alive until the batch is freed - identifiers in the records are (offset, length)
 * references into it, as the reference's AST borrows from its input (`&'input str`).  A batch stays valid until the
 * next ptxfe_parse_batch / ptxfe_run on the same context or until ptxfe_batch_free; a context serves one thread at a time.
 */
#ifndef PTXFE_H
#define PTXFE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ptxfe_ctx ptxfe_ctx;
typedef struct ptxfe_batch ptxfe_batch;

enum { PTXFE_CHECKED = 0, PTXFE_UNCHECKED = 1, PTXFE_ERRORS_ONLY = 2 };

enum {
    PTXFE_OK = 0,
    PTXFE_ERR_BAD_ARG = 1,
    PTXFE_ERR_CUDA = 2,      /* a CUDA call failed; ptxfe_last_error(ctx) has the text */
    PTXFE_ERR_TOO_LARGE = 3, /* batch text (with per-module padding) exceeds 4 GiB - 1, or a result table exceeds 2^32 entries */
    PTXFE_ERR_OOM = 4
};

/* per-module verdict, mirroring the three reference return shapes */
enum {
    PTXFE_MODULE_OK = 0,        /* checked: Ok(module); unchecked: a module was returned */
    PTXFE_MODULE_ERR = 1,       /* checked: Err(errors); unchecked: Module::empty() (ptx_parser/src/ast.rs:2008-2016) */
    PTXFE_MODULE_REF_PANICS = 2, /* input on which the reference unwraps an empty slice (lib.rs:939) */
    PTXFE_MODULE_REF_DIVERGES = 3, /* damage below deeply nested blocks: the reference's statement recovery re-parses the
                                     contents of every enclosing block and doubles its work per level (lib.rs:858-880,
                                     921-951); given up after 4 * tokens + 1024 statement attempts, no module, no errors */
    PTXFE_MODULE_SEQ_REFUSED = 4   /* no counterpart in the reference.  A module whose structure is damaged is parsed with
                                     the reference's recovery rules by ONE device thread from the top-level directive with
                                     the first damage to its end (about a microsecond per token, twice).  A tail of more
                                     than 2 Mi tokens (environment: PTXFE_SEQ_MAX_TOKENS) is refused instead of running
                                     for minutes: no module, no errors.  Parse such a module on the CPU. */
};

typedef struct ptxfe_stats {
    uint64_t text_bytes;      /* sum of module lengths */
    uint64_t n_modules, n_tokens, n_units, n_result_words, n_errors, n_lex_errors;
    uint64_t n_sequential;    /* modules re-parsed by the single-thread recovery path */
    uint64_t n_kernel_launches;
    uint64_t h2d_bytes, d2h_bytes;
    float h2d_ms, kernel_ms, d2h_ms;   /* CUDA-event times of the three phases of the last call */
    float lex_ms, structure_ms, decode_ms;   /* kernel_ms split by stage */
    /* statement classes: units of one class share the grammar work through a record template */
    uint64_t n_classes;          /* classes in the batch's class store after the last slice */
    uint64_t n_class_capacity;   /* templates the store holds; classes beyond it are decoded unit by unit */
    uint64_t n_untemplated;      /* units that were decoded one by one */
    uint64_t n_signature_words, n_signature_capacity;
    /* tokens that went through the single-thread recovery path: only the part of a damaged module from the top-level
     * directive with the first damage to the module's end does */
    uint64_t n_sequential_tokens;
} ptxfe_stats;

/* Create a context on CUDA device `device` (one stream, reusable device arenas, pinned result buffers). */
int ptxfe_create(int device, ptxfe_ctx** out);
void ptxfe_destroy(ptxfe_ctx* ctx);
const char* ptxfe_last_error(const ptxfe_ctx* ctx);
const char* ptxfe_status_str(int status);

/* Whole path: copy `n` module texts to the device, parse them, copy the records back.  `texts[i]` need not be
 * NUL-terminated.  Host buffers may be pageable or pinned (pinned text, and modules that lie back to back in memory,
 * give the fastest copies).  A large batch is cut into slices of whole modules whose copies overlap with the kernels of
 * their neighbours; text offsets in a module's records are relative to its slice: subtract the `text_base` that
 * ptxfe_module_records reports.  In ptxfe_stats, h2d_ms / kernel_ms / d2h_ms are then the busy times of the three
 * streams, which overlap.  Environment: PTXFE_SLICE_BYTES forces one slice size, PTXFE_SLICE_DIV the divisor that
 * sizes the middle slices (default 8), PTXFE_TRACE=1 prints the slices' device timeline to stderr. */
int ptxfe_parse_batch(ptxfe_ctx* ctx, const char* const* texts, const uint64_t* lens, uint32_t n, uint32_t mode,
                      ptxfe_batch** out);

/* The same in three steps, for callers that keep text resident in device memory across calls or overlap transfers:
 *   ptxfe_stage : host text -> device (module i starts at a 128-byte boundary of the batch buffer)
 *   ptxfe_run   : all kernels; results stay on the device
 *   ptxfe_fetch : device -> host records, returns the batch */
int ptxfe_stage(ptxfe_ctx* ctx, const char* const* texts, const uint64_t* lens, uint32_t n);
int ptxfe_run(ptxfe_ctx* ctx, uint32_t mode);
int ptxfe_fetch(ptxfe_ctx* ctx, ptxfe_batch** out);

/* Several GPUs of one machine.  Modules are independent, so a batch is sharded by module with byte-balanced greedy
 * partitioning (largest module first onto the device with the fewest bytes so far) and nothing is exchanged between
 * the devices.  The reference's counterpart is its one fan-out caller, which hands modules to a thread pool
 * (zluda_precompile/src/main.rs:57-64).  ptxfe_multi_create makes one context per entry of `devices` (a device may be
 * named more than once: each entry gets its own context, streams and arenas); ptxfe_parse_batch_multi splits the
 * batch, runs ptxfe_parse_batch on every shard from a host thread of its own, and returns ONE batch whose modules are
 * indexed as the caller passed them: every ptxfe_module_* function below works on it unchanged.
 * ptxfe_multi_part_stats reports the statistics of shard `part` of the last call, ptxfe_multi_part_of the shard a
 * module went to. */
typedef struct ptxfe_multi ptxfe_multi;
int ptxfe_multi_create(const int* devices, uint32_t n_devices, ptxfe_multi** out);
void ptxfe_multi_destroy(ptxfe_multi* m);
const char* ptxfe_multi_last_error(const ptxfe_multi* m);
int ptxfe_parse_batch_multi(ptxfe_multi* m, const char* const* texts, const uint64_t* lens, uint32_t n, uint32_t mode,
                            ptxfe_batch** out);
uint32_t ptxfe_multi_parts(const ptxfe_multi* m);
void ptxfe_multi_part_stats(const ptxfe_multi* m, uint32_t part, ptxfe_stats* out);
int ptxfe_multi_part_of(const ptxfe_batch* batch, uint32_t i);

void ptxfe_batch_free(ptxfe_batch* batch);
uint32_t ptxfe_batch_size(const ptxfe_batch* batch);
int ptxfe_module_status(const ptxfe_batch* batch, uint32_t i);
uint32_t ptxfe_module_error_count(const ptxfe_batch* batch, uint32_t i);
void ptxfe_get_stats(const ptxfe_ctx* ctx, ptxfe_stats* out);
/* When the environment variable PTXFE_PROFILE=1 was set at ptxfe_create: one line "step_name milliseconds" per pipeline
 * step of the last ptxfe_run (CUDA-event time on the context's stream).  Empty otherwise. */
const char* ptxfe_profile(const ptxfe_ctx* ctx);

/* Raw record views of module i (layout: zluda_b200/csrc/ptx_decode.h).  Offsets inside records index the batch text
 * buffer; subtract *text_base to index texts[i]. */
int ptxfe_module_records(const ptxfe_batch* batch, uint32_t i, const uint32_t** words, uint64_t* n_words,
                         uint64_t* text_base);

/* Canonical text dump of module i: the tree printed as if every ptx_parser AST type derived Debug (floats as bit
 * patterns), followed by the ordered error list.  malloc'ed; release with ptxfe_free. */
int ptxfe_module_dump(const ptxfe_batch* batch, uint32_t i, char** out, uint64_t* out_len);
/* Materialiser: builds, for every module of the batch, the tree a caller of the reference holds - module, directives,
 * functions, statements with nested blocks, variables with their padded initialisers, instructions with typed data and
 * operands, names as slices of the caller's text (zluda_b200/csrc/ptx_ast.h mirrors ptx_parser/src/ast.rs:14-19,
 * 1216-1240, 1922-2005) - on n_threads host threads, and drops it again; *n_nodes = nodes built.  ptxfe_module_dump
 * prints from the same tree.  This is what a binding pays on top of ptxfe_parse_batch to hand out ast-like values. */
int ptxfe_batch_materialize(const ptxfe_batch* batch, uint32_t n_threads, uint64_t* n_nodes);
/* 64-bit FNV-1a of the same dump, without materialising it beyond one module at a time. */
int ptxfe_module_dump_hash(const ptxfe_batch* batch, uint32_t i, uint64_t* out_hash);
void ptxfe_free(void* p);

/* Token table of module i of the staged batch (lexer only; for tests): triples (kind, start, length) relative to the
 * module text, then error spans (start, length).  malloc'ed. */
int ptxfe_lex_module(ptxfe_ctx* ctx, const char* text, uint64_t len, uint32_t** out, uint64_t* n_tokens, uint64_t* n_errors);

/* Lexer without any allocation.  It has no counterpart in the reference, which lexes on the CPU into a Vec.
 *
 * For callers that are not allowed to call cudaMalloc (or anything that might): code running while another component
 * owns the device's memory budget, inside a region where the allocator may not be entered (a stream callback, a
 * library's own hook), or in a process whose device heap is exhausted or fragmented.  The usual entry points grow a per-context arena and
 * pinned buffers on demand; this one touches only memory the caller passes in plus a fixed 2 MiB working array that is
 * part of the library image (each GPU that loads the library carries that array until the process exits).
 *
 *   d_text     device pointer to `len` bytes of one module's text; len <= 16 MiB, larger inputs are refused with
 *              PTXFE_ERR_TOO_LARGE and a message on stderr
 *   d_tokens   device pointer to room for `token_capacity` 8-byte token records {start:u32, len:u16, kind:u16}
 *              (same records as ptxfe_lex_module; len 0xFFFF = 65535 or longer); tokens beyond the capacity are
 *              dropped but still counted
 *   d_counts   device pointer to two uint32: number of tokens, number of lex errors; both 0xFFFFFFFF when the text was
 *              refused because one run of word characters and . : + - % is longer than 64 KiB (no real PTX has one;
 *              lexing it chunk by chunk would walk that run once per chunk)
 *   stream     cudaStream_t to launch on (0 = default stream).  The call only enqueues kernels.
 *
 * The call makes `device` current while it works and puts the caller's current device back before it returns.  The
 * first call on a device looks up the device address of the working array (cudaGetSymbolAddress; any thread may make
 * it, concurrent first calls look up the same address); make that first call outside any stream capture.  All calls on one GPU share the working array: two calls whose kernels can overlap
 * on the device (different streams, different threads) race - serialise them.  Nothing in the array has to survive
 * between calls and nothing needs clearing by the caller. */
int ptxfe_lex_device_noalloc(int device, const void* d_text, uint64_t len, void* d_tokens, uint64_t token_capacity,
                             uint32_t* d_counts, void* stream);

#ifdef __cplusplus
}
#endif
#endif
