/* unholy_pkv.h — C ABI of the B200 paged KV-cache library (libunholy_pkv.so).
 *
 * Plain pointers and sizes only. Every pointer named "device" is CUDA device memory owned by the caller; the
 * library never allocates or frees it (the reference's kernels never allocate either: src/rt/hip.hpp:39-83 is the
 * caller's RAII). Every data-path entry point enqueues work on `stream` and returns without synchronising; a NULL
 * stream is the default stream (src/rt/hip.hpp:11-19 convention). Return value: PKV_OK or an error code;
 * pkv_last_error() gives the message of the calling thread's last failure. The C++ wrappers in
 * unholy_b200/csrc/host/kernels.hpp keep the reference's signatures and turn a non-zero code into
 * std::runtime_error, as UH_CHECK_LAUNCH does in the reference.
 *
 * There is no CPU fallback: without a CUDA device every data-path call returns PKV_ERR_CUDA.
 *
 * Types: bf16 = uint16_t bit patterns, fp8 (e4m3fn) = uint8_t, scales = e8m0 exponent bytes (src/kernels/ref.hpp:6-7).
 */
#ifndef UNHOLY_PKV_H
#define UNHOLY_PKV_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PKV_API __attribute__((visibility("default")))
#else
#define PKV_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* pkv_stream_t; /* == cudaStream_t */

enum {
  PKV_OK = 0,
  PKV_ERR_ARG = 1,    /* bad shape / pointer / alignment: nothing was launched */
  PKV_ERR_CUDA = 2,   /* a CUDA runtime call failed (message has cudaGetErrorString) */
  PKV_ERR_DEVICE = 3, /* a kernel's own bounds check tripped (see pkv_device_status) */
  PKV_ERR_LIMIT = 4   /* a size exceeds a compiled-in maximum */
};

#define PKV_MAX_LAYERS 48     /* layers one pkv_step_run launch can take */
#define PKV_FP4_ROW_DIM 128   /* indexer key width the fp4 page layout is defined for */

PKV_API const char* pkv_last_error(void);
PKV_API int pkv_abi_version(void);
/* Performance knobs (no counterpart in the reference; results never depend on them). knob 0: bulk pipeline shape
 * STAGES*100+ROWS, one of 304, 308, 408, 316 (0 = chosen by launch size); 1: bulk CTAs per SM (0 = fill shared memory); 2: programmatic dependent
 * launch on/off; 3: CTAs per SM of the vector kernels; 4: appends as tiles of the bulk launch on/off; 5: tiles whose
 * addresses are resolved together (-1 = by launch size, 0 = a warp's worth); 6: resolve the next batch late (0/1);
 * 7: top-k path (0 = one thread-block-cluster launch where the shape allows it, 1 = always the four launches that use
 * the scratch); 8: which bulk pipeline runs a step (-1 = by launch shape, 0 = the single-warp kernel, 1 = the
 * warp-specialised kernel); 9: polls, of up to a microsecond each, before a device-side wait of the warp-specialised
 * kernel gives up and reports kind 3 (0 = the default, about two seconds). The defaults come from PKV_* environment
 * variables. Knob 10 is a test hook, not a performance knob: CTA 0 of the warp-specialised kernel expects 16 bytes more
 * than its tile number `value` brings (-1 = off), so that its wait runs out without anything being wrong on the GPU. */
PKV_API int pkv_tune(int knob, int value);

/* First failed device-side check since the last call (0 = none): bit 0..7 = kind (1 page id out of range,
 * 2 chunk row, chunk index or slot out of range, 3 bounded wait gave up), the rest = an index identifying the entry.
 * Synchronises the device. The kernels skip the offending access instead of faulting. Kernels that can report: the
 * step kernels (pkv_step_run, pkv_step_gather_fp8*) and pkv_copy_pages; the others take no ids from device memory
 * that the host has not already checked. */
PKV_API int pkv_device_status(int* status_out);
/* The same check as an error code, ordered after the work queued on `stream` so far: waits for that stream only,
 * returns PKV_OK, or PKV_ERR_DEVICE with the kind and index in pkv_last_error() (and clears the record). */
PKV_API int pkv_stream_check(pkv_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Reference-shaped single-sequence entry points. `table` is ONE slot's row of the block table (device).
 * ---------------------------------------------------------------------------------------------------------------- */

/* store_rows — src/kernels/ref.hpp:92-100, src/kernels/ref_attn.hip:88-93,377-381.
 * rows [n][width] bf16 -> logical rows [row0, row0+n): pool + (table[r/rpp]*rpp + r%rpp) * row_stride elements. */
PKV_API int pkv_store_rows(const uint16_t* rows, int n, int width, uint16_t* pool, const int32_t* table, int rows_per_page,
                   int row_stride, int row0, pkv_stream_t stream);

/* fake_quant_fp8 + store_rows in one pass — the pair compress_chunk issues for KV rows (src/model/forward_ref.hip:739-741:
 * fake_quant_fp8(rb, d, nrows, d - rope_dim, 64) then store_rows(rb, ...)): the first quant_cols columns of every row
 * are quantised to e4m3 with one power-of-two scale per `block` values and dequantised (src/kernels/ref_elem.hip:18-41),
 * the other columns are copied, and the row goes to its place in the pool; `rows` is read once and not modified.
 * width % block == 0, quant_cols % block == 0, block 32 / 64 / 128, rows and pool 16-byte aligned. */
PKV_API int pkv_store_rows_fake_fp8(const uint16_t* rows, int n, int width, int quant_cols, int block, uint16_t* pool,
                                    const int32_t* table, int rows_per_page, int row_stride, int row0, pkv_stream_t stream);

/* kv_chain + store_rows in one pass — kv_chain (src/kernels/elem_fast.hpp:29, src/kernels/elem_fast.hip:87-92,124-128;
 * device body kv_chain_row, src/kernels/elem_dev.hip.hpp:50-87) is the last thing that happens to a step's KV rows
 * before compress_chunk appends them: rmsnorm with weight w [dim] (bf16), rope on the last 2 * npair values with
 * freqs float2 [positions][npair] = (cos, sin) at the row's position pos[r], then fake_quant_fp8 (block 64) of the other
 * values (quant == 0 stops in front of the quantisation). The result goes to the rows' place in the pool (pool NULL:
 * not appended) and, when rows_out is not NULL, to rows_out [n][dim] (rows_out == rows gives the reference's in-place
 * kv_chain); `rows` is read once. NOT bit-exact against the reference's GPUs by construction: the reference sums the
 * squares over 256 threads and uses the hardware rsqrtf, neither of which the source pins down; this kernel uses an
 * fp32 sum and the correctly rounded 1 / sqrt. Tolerance: one bf16 step on a normalised value (a rotated value inherits
 * the steps of its two inputs); the quantisation is exact on equal inputs. dim <= 1024 and a multiple of 8, (2 * npair) % 8 == 0, (dim - 2 * npair) % 64 == 0. */
PKV_API int pkv_store_rows_kv_chain(const uint16_t* rows, uint16_t* rows_out, const uint16_t* w, int n, int dim, float eps,
                                    const int32_t* pos, const float* freqs, int npair, int quant, uint16_t* pool,
                                    const int32_t* table, int rows_per_page, int row_stride, int row0, pkv_stream_t stream);

/* store_rows_fp4 — src/kernels/indexer.hpp:20-32, src/kernels/indexer.hip:18-53,802-806.
 * rows [n][128] bf16 -> MXFP4: page p at pool + p*rows_per_page*68; rows_per_page code rows of 64 B (even column =
 * low nibble) followed by rows_per_page scale rows of 4 e8m0 bytes. The reference fixes rows_per_page = 64. */
PKV_API int pkv_store_rows_fp4(const uint16_t* rows, int n, uint8_t* pool, const int32_t* table, int rows_per_page, int row0,
                       pkv_stream_t stream);

/* load_rows_fp4 — src/kernels/indexer.hpp:34, src/kernels/indexer.hip:55-62. Decodes rows back to bf16 [n][128]. */
PKV_API int pkv_load_rows_fp4(const uint8_t* pool, const int32_t* table, int rows_per_page, int row0, int n, uint16_t* out,
                      pkv_stream_t stream);

/* act_quant_fp8 — src/kernels/ref.hpp:22, src/kernels/ref_elem.hip:18-41,282-286. x bf16 [rows][ldx] ->
 * q e4m3 [rows][cols], s e8m0 [rows][cols/block]; block in {32, 64, 128}. */
PKV_API int pkv_act_quant_fp8(const uint16_t* x, int ldx, uint8_t* q, uint8_t* s, int rows, int cols, int block,
                      pkv_stream_t stream);
/* fake_quant_fp8 / fake_quant_fp4 — src/kernels/ref.hpp:24-25, src/kernels/ref_elem.hip:18-59,287-296. In place. */
PKV_API int pkv_fake_quant_fp8(uint16_t* x, int ldx, int rows, int cols, int block, pkv_stream_t stream);
PKV_API int pkv_fake_quant_fp4(uint16_t* x, int ldx, int rows, int cols, int block, pkv_stream_t stream);

/* glm_store_latent — src/kernels/glm_fast.hpp:23-32, src/kernels/glm_fast.hip:29-51,752-756, with the row width,
 * quantisation block and page size as parameters (the reference fixes 512 / 64 / 256). rows bf16 [n][width] of
 * positions [s0, s0+n): codes[rid][width] and scales[rid][width/block] at rid = table[p/rpp]*rpp + p%rpp. */
PKV_API int pkv_store_rows_fp8(const uint16_t* rows, int n, int width, int block, uint8_t* codes, uint8_t* scales,
                       const int32_t* table, int rows_per_page, int s0, pkv_stream_t stream);

/* copy_kernel — src/kernels/ref.hpp:90, src/kernels/ref_elem.hip:269-278,358-366. A byte copy executed by SMs
 * (16-byte vectors when dst, src and bytes allow), ordered in `stream` like any kernel. */
PKV_API int pkv_copy(void* dst, const void* src, size_t bytes, pkv_stream_t stream);

/* The sparse gather as a standalone operation. Replaces the gather loop fused into the reference's attention kernels:
 * src/kernels/attn_wmma.hip:75-113 (row_of + staging), src/kernels/ref_attn.hip:285-301, src/kernels/glm_fast.hip:190-195.
 * idx device [T][k]; q_visible device [T]. Entry e of query t = logical row idx[t][e] of the slot; entries < 0 or
 * >= q_visible[t] are masked and produce a row of zeros (src/kernels/attn_wmma.hip:107,277-291).
 * out device bf16 [T][k][width], contiguous. */
PKV_API int pkv_gather_rows(const uint16_t* pool, const int32_t* table, int rows_per_page, int row_stride, int width,
                    const int32_t* idx, const int32_t* q_visible, int T, int k, uint16_t* out, pkv_stream_t stream);

/* The same gather over fp8 rows with dequantisation to bf16 — replaces the gather loop of the reference's GLM attention
 * (src/kernels/glm_fast.hip:29-31,190-227) for rows stored by pkv_store_rows_fp8 / glm_store_latent: entry -> physical
 * row -> e4m3 codes [width] and e8m0 scales [width/block] -> out bf16 [T][k][width] = code * 2^scale (exact in bf16);
 * masked entries (< 0 or >= q_visible[t]) give zero rows. width a multiple of 16, codes and out 16-byte aligned (a
 * 32-byte aligned out is written with 256-bit stores); launched with programmatic stream serialisation like the step
 * kernels. */
PKV_API int pkv_gather_rows_fp8(const uint8_t* codes, const uint8_t* scales, const int32_t* table, int rows_per_page, int width,
                        int block, const int32_t* idx, const int32_t* q_visible, int T, int k, uint16_t* out,
                        pkv_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Batched step: all chunks of a step (src/engine/step.hpp:20-26 Chunk, src/model/forward_ref.hpp:50-60 BatchDesc),
 * for 1..PKV_MAX_LAYERS layers in ONE launch. Replaces the reference's one launch per (chunk, layer, pool)
 * (src/model/forward_ref.hip:719-745,843-857) and the gather loops of its attention launches (:951-999).
 * ---------------------------------------------------------------------------------------------------------------- */

typedef struct pkv_chunk { /* src/engine/step.hpp:20-26 */
  int32_t slot;            /* block-table row */
  int32_t s0;              /* first logical row written */
  int32_t n;               /* rows */
  int32_t t0;              /* first batch row */
} pkv_chunk;

typedef struct pkv_layer { /* device pointers of one layer; any pair may be NULL to skip that part */
  const uint16_t* rows;    /* bf16 [T][width]: the step's new KV rows */
  uint16_t* row_pool;      /* bf16 [num_pages][rows_per_page][row_stride] */
  const uint16_t* keys;    /* bf16 [T][128]: the step's new indexer keys */
  uint8_t* key_pool_fp4;   /* MXFP4 pool, layout of pkv_store_rows_fp4 */
  uint8_t* key_fp8_codes;  /* e4m3 [num_pages*rows_per_page][128] */
  uint8_t* key_fp8_scales; /* e8m0 [num_pages*rows_per_page][128/fp8_block] */
  const int32_t* idx;      /* int32 [Q][k] index lists (src/kernels/indexer.hpp:74 format: -1 padded) */
  uint16_t* gathered;      /* bf16 [Q][k][width] */
} pkv_layer;

typedef struct pkv_step {
  int32_t width;             /* bf16 values per KV row */
  int32_t row_stride;        /* elements between pool rows (>= width) */
  int32_t rows_per_page;
  int32_t max_pages_per_seq; /* block-table width */
  int32_t num_pages;         /* physical pages per pool; ids outside [0, num_pages) are reported, not dereferenced */
  int32_t fp8_block;         /* 32, 64 or 128 (only read when fp8 key arrays are given) */
  int32_t nchunks;
  int32_t T;                 /* batch rows */
  int32_t Q;                 /* query rows */
  int32_t k;                 /* index-list width */
  int32_t max_slots;         /* block-table rows; a chunk's slot outside [0, max_slots) is reported, not dereferenced */
  int32_t reserved;          /* 0 */
  const int32_t* tables;     /* device [max_slots][max_pages_per_seq] (src/engine/step.hpp:100) */
  const pkv_chunk* chunks;   /* device [nchunks] */
  const int32_t* q_chunk;    /* device [Q]: index into chunks of the chunk the query row belongs to (outside
                                [0, nchunks): reported, the query's rows are zeros) */
  const int32_t* q_visible;  /* device [Q]: logical rows visible to the query (row >= visible is masked) */
} pkv_step;

enum {
  PKV_DO_ROWS = 1,     /* append layer.rows into layer.row_pool */
  PKV_DO_KEYS_FP4 = 2, /* quantise layer.keys into layer.key_pool_fp4 */
  PKV_DO_KEYS_FP8 = 4, /* quantise layer.keys into layer.key_fp8_codes / key_fp8_scales */
  PKV_DO_GATHER = 8,   /* gather layer.idx rows into layer.gathered */
  PKV_KEYS_HADAMARD = 32, /* rotate every 128-wide key row by hadamard128 (src/kernels/ref_elem.hip:111-135, bf16 result)
                             before it is quantised: the reference's hadamard128 + store_rows_fp4 pair of
                             compress_chunk (src/model/forward_ref.hip:736-738) in the append itself; layer.keys is
                             not modified */
  PKV_VARIANT_BULK = 256 /* gather through the bulk-copy (TMA) pipeline instead of vector loads */
};

/* `layers` is a HOST array of L structs holding device pointers (copied into the launch parameters).
 * When PKV_DO_ROWS and PKV_DO_GATHER are both set, an index that falls inside its own chunk's range
 * [s0, s0+n) is read from layer.rows (the value being appended in this launch), everything else from the pool; the
 * result equals "append, then gather" (the reference reads in-chunk window rows from the chunk the same way:
 * src/kernels/attn_wmma.hip:84). Rows of other chunks appended in the same launch must not be gathered. */
PKV_API int pkv_step_run(const pkv_step* step, const pkv_layer* layers, int L, int flags, pkv_stream_t stream);

/* The fp8 gather with dequantisation (pkv_gather_rows_fp8) for every sequence of a step in one launch: query row t of
 * the step gathers idx[t][0..k) from the sequence of its chunk (step->q_chunk, chunks, tables, q_visible, Q, k,
 * rows_per_page, max_pages_per_seq, num_pages as in pkv_step_run; width and row_stride of the step are not used) out of
 * the fp8 pool codes [rows][width] / scales [rows][width / block] into out bf16 [Q][k][width]. Replaces one
 * mla_attn launch per chunk's gather loop (src/kernels/glm_fast.hip:190-227, src/model/glm5_fast.hip:276-299). */
PKV_API int pkv_step_gather_fp8(const pkv_step* step, const uint8_t* codes, const uint8_t* scales, int width, int block,
                                const int32_t* idx, uint16_t* out, pkv_stream_t stream);

/* pkv_step_gather_fp8 with the list expansion folded in: instead of a token list the caller passes what the top-k over
 * pools wrote — pools [Q][kp] (valid pools first) and the queries' positions pos [Q] — and entry j of query row t is
 * what glm_idx_expand (src/kernels/glm_fast.hpp:115-122, src/kernels/glm_fast.hip:737-748) would have written at
 * idx[t][j]; out is bf16 [Q][kp * pool + pool - 1][width] (step->k is not used). Saves the expanded list's round trip
 * through memory and one launch. */
PKV_API int pkv_step_gather_fp8_pools(const pkv_step* step, const uint8_t* codes, const uint8_t* scales, int width, int block,
                                      const int32_t* pools, const int32_t* pos, int kp, int pool, uint16_t* out,
                                      pkv_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Index-list producer (the step before the gather).
 * ---------------------------------------------------------------------------------------------------------------- */

/* topk_bf16 / topk_bf16_batch — src/kernels/indexer.hpp:74-94, src/kernels/indexer.hip:408-560,878-902.
 * scores device bf16 [T][ld] (n <= ld keys per row); idx device int32 [T][k]: per row the min(k, #valid) largest
 * scores ordered (score descending, index ascending), ties at the threshold to the lowest indices, -1 padded; -inf is
 * never selected. k <= 4096. As in the reference, `scratch` is OPTIONAL (NULL / 0 words allowed): shapes with
 * k <= 2048 and n <= 655,360 run as one launch of thread-block clusters that needs none. Other shapes (and pkv_tune
 * knob 7 = 1) run as four launches through pkv_topk_scratch_words(T, n, k) uint32 words: the caller's `scratch` when it
 * is 8-byte aligned and large enough (its contents need not be initialised and are garbage afterwards; two calls that
 * overlap on the GPU must not share it), else the library's built-in 4 MiB array (pkv_topk_bf16_static's: calls that
 * land there must not overlap on the GPU, and the first such call per device should come before any stream capture),
 * else PKV_ERR_LIMIT with the word count in the message. */
PKV_API size_t pkv_topk_scratch_words(int T, int n, int k);
PKV_API int pkv_topk_bf16(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, uint32_t* scratch,
                          size_t scratch_words, pkv_stream_t stream);

/* topk_bf16_batch — src/kernels/indexer.hpp:76-94 (TopkRows / TopkBatch), src/kernels/indexer.hip:878-902: several
 * score blocks in one call (the decode chunks of a step): group g's rows [rows][n] start at scores + off (elements),
 * its index lists [rows][k] at idx + idx_off (elements); per row the same result as pkv_topk_bf16. All groups run in
 * one launch of thread-block clusters (32 groups per launch) when every group has k <= 2048 and n <= 655,360; else one
 * after the other on the stream, sharing `scratch` (pkv_topk_batch_scratch_words words; optional as for pkv_topk_bf16). */
typedef struct pkv_topk_group {
  size_t off;
  int32_t rows, n, k, idx_off;
} pkv_topk_group;
PKV_API size_t pkv_topk_batch_scratch_words(const pkv_topk_group* groups, int ngroups);
PKV_API int pkv_topk_bf16_batch(const uint16_t* scores, const pkv_topk_group* groups, int ngroups, int32_t* idx, uint32_t* scratch,
                        size_t scratch_words, pkv_stream_t stream);

/* topk_rows — src/kernels/ref.hpp:107, src/kernels/ref_attn.hip:143-254,390-393 — and glm_topk —
 * src/kernels/glm_fast.hpp:86-93, src/kernels/glm_fast.hip:557-681,852-874 (the same selection in one or two stages;
 * its cand scratch is not needed here). scores: device fp32 [T][ld] (ld >= n elements between rows; topk_rows has
 * ld = n); idx: device int32 [T][k]. Per row the min(k, #scores above -inf) largest scores ordered by (score
 * descending, index ascending), threshold ties to the lowest indices, -1 padded; -inf and negative NaN patterns are
 * never selected. k <= 1024 as in the reference (PKV_ERR_ARG beyond). No scratch: one CTA per row selects in shared
 * memory. T <= 0 or n <= 0 returns PKV_OK without a launch. */
PKV_API int pkv_topk_f32(const float* scores, int T, int n, long long ld, int k, int32_t* idx, pkv_stream_t stream);

/* hadamard128 — src/kernels/ref.hpp:63, src/kernels/ref_elem.hip:111-135,310-313: in place, every segment of 128 bf16
 * values of x [nseg][128] becomes its Hadamard transform (seven fp32 butterfly stages in the reference's order, times
 * 128^-0.5, rounded to bf16). x must be 16-byte aligned. */
PKV_API int pkv_hadamard128(uint16_t* x, size_t nseg, pkv_stream_t stream);

/* glm_idx_expand — src/kernels/glm_fast.hpp:115-122, src/kernels/glm_fast.hip:737-748,915-920. Selected pools
 * device int32 [n][k] (a top-k's output: valid pools first) and the queries' positions pos [n] -> the compact token
 * list idx [n][k*pool + pool-1]: the tokens of the min((p+1)/pool, k) valid pools, then the (p+1) % pool tokens of the
 * query's incomplete pool, then -1. The result is an index list in the format the gather takes. */
PKV_API int pkv_idx_expand(const int32_t* pools, const int32_t* pos, int32_t* idx, int n, int k, int pool, pkv_stream_t stream);

/* Slot-state snapshots — ResidentModel::state_copies, src/engine/resident.hip:545-557. pkv_state_seg is the
 * reference's SnapSeg (src/engine/resident.hpp:180-183): a per-slot state buffer (slot s at dev + s * bytes) and its
 * offset in a snapshot; pkv_state_op is StateOp (src/engine/step.hpp:32-34). For every op and every segment,
 * save != 0 copies the slot's slice into snapshot op.snapshot (at snap_base + snapshot * snap_bytes + off), save == 0
 * copies it back — the reference's loop of copy_kernel calls, here one launch per 256 segments x 32 ops. segs and ops
 * are HOST arrays; snap_base is any memory the device can address: mapped pinned host memory as in the reference
 * (resident.hip:538-541) or device memory. An op outside [0, num_snapshots) x [0, max_slots) fails with the
 * reference's message "step: bad state op" before anything is launched. Ops of one call must not overlap each other. */
typedef struct pkv_state_seg {
  void* dev;
  size_t bytes, off;
} pkv_state_seg;
typedef struct pkv_state_op {
  int32_t slot, snapshot;
} pkv_state_op;
PKV_API int pkv_state_copies(const pkv_state_seg* segs, int nsegs, const pkv_state_op* ops, int nops, void* snap_base,
                             size_t snap_bytes, int num_snapshots, int max_slots, int save, pkv_stream_t stream);

/* pkv_topk_bf16 for callers that cannot hand the library any device memory of their own and cannot let it allocate
 * either — an engine thread that is recording its step into a CUDA graph (cudaMalloc is illegal while a stream is
 * capturing), a latency-critical decode loop (cudaMalloc/cudaFree synchronise the whole device), or a plugin host that
 * owns every allocation and hands none to plugins. This entry point has no counterpart in the reference. It takes
 * only inputs and outputs; the scratch is a 4 MiB array compiled into the library (pkv_topk_static_scratch_words()
 * uint32 words = 1,048,576), which every GPU that loads the library keeps until the process exits. It calls no
 * cudaMalloc, cudaFree or other allocating routine. Shapes whose pkv_topk_scratch_words(T, n, k) exceeds the built-in
 * size are refused with PKV_ERR_LIMIT (64 rows x 131,072 keys x k = 2048 needs 788,992 words and fits). The first
 * call on each device looks the array's device address up (cudaGetSymbolAddress), so make that first call outside any
 * stream capture. Every call on a device shares the one array: it keeps the previous call's contents (harmless: each
 * call clears or overwrites what it reads), and two calls that overlap on the GPU (different streams) race — serialise them.
 * Results are identical to pkv_topk_bf16's. Nothing is stated here about recording this call itself into a graph. */
PKV_API size_t pkv_topk_static_scratch_words(void);
PKV_API int pkv_topk_bf16_static(const uint16_t* scores, int T, int n, long long ld, int k, int32_t* idx, pkv_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Page moves: copy-on-write duplication, hole-filling compaction, migration between shards. The reference has no
 * such operation (it never copies page payloads: src/engine/engine.cpp:284-336 shares full pages only); the copy
 * primitive they generalise is copy_kernel (src/kernels/ref_elem.hip:269-278).
 * ---------------------------------------------------------------------------------------------------------------- */

typedef struct pkv_pool_desc {
  const void* src_base; /* device (may be a peer device's mapped pool for migration) */
  void* dst_base;       /* device; == src_base for moves inside one pool */
  uint64_t page_bytes;  /* multiple of 16 */
} pkv_pool_desc;

/* For every pool p < npools and i < n: dst_base[p] + dst_ids[i]*page_bytes <- src_base[p] + src_ids[i]*page_bytes.
 * `pools` is a HOST array (npools <= 128); src_ids/dst_ids are device int32 [n]. Source and destination id sets
 * must be disjoint when src_base == dst_base. */
PKV_API int pkv_copy_pages(const pkv_pool_desc* pools, int npools, const int32_t* src_ids, const int32_t* dst_ids, int n,
                   int num_src_pages, int num_dst_pages, pkv_stream_t stream);

/* Device memory sharing between the one-process-per-GPU shards (migration over NVLink with ordinary loads).
 * pkv_ipc_export fills a 64-byte handle for a cudaMalloc'd base pointer; pkv_ipc_open maps a peer's handle into this
 * process; pkv_ipc_close unmaps. pkv_device_alloc / pkv_device_free are cudaMalloc / cudaFree for callers that need
 * an exportable allocation. */
PKV_API int pkv_device_alloc(void** ptr_out, size_t bytes);
PKV_API int pkv_device_free(void* ptr);
PKV_API int pkv_ipc_export(void* base, unsigned char handle_out[64]);
PKV_API int pkv_ipc_open(const unsigned char handle[64], void** ptr_out);
PKV_API int pkv_ipc_close(void* ptr);

/* ------------------------------------------------------------------------------------------------------------------
 * The pool sharded over the GPUs of one box by request ownership, with migration between shards: a C++ host object
 * (one process, one host thread and one stream per shard; no torch, no collective). The reference has no counterpart:
 * its pools are per card and pages never move (the design notes at the root of its repository, lines 119-123 and
 * 148-149); the ordering pattern — a pull kernel behind events — is that of src/engine/resident.hip:213-232,908-910. A shard owns `layers` bf16 row pools (and MXFP4
 * key pools when key_pools != 0), one page pool (the allocator above) and one block table. Calls on one pkv_shards
 * object must come from one thread at a time.
 * ---------------------------------------------------------------------------------------------------------------- */
typedef struct pkv_shards pkv_shards;
typedef struct pkv_shard_config {
  int32_t ngpus;             /* shards; devices[i] of pkv_shards_create is shard i's CUDA device (two shards may share one) */
  int32_t num_pages;         /* pages per shard */
  int32_t rows_per_page, width, row_stride;
  int32_t layers;
  int32_t max_slots, max_pages_per_seq;
  int32_t k;                 /* index-list width of the steps */
  int32_t key_pools;         /* != 0: every layer also has an MXFP4 key pool; its pages move with the row pages */
} pkv_shard_config;
typedef struct pkv_shard_io { /* one layer of one shard's step: device pointers on that shard's GPU */
  const uint16_t* rows;      /* bf16 [Q][width]: the row each local request appends, in pkv_shards_local order */
  const uint16_t* keys;      /* bf16 [Q][128] or NULL */
  const int32_t* idx;        /* int32 [Q][k] */
  uint16_t* gathered;        /* bf16 [Q][k][width] */
} pkv_shard_io;
/* Allocates every shard's pools, tables, streams and staging on its device and enables peer access between distinct
 * devices once. NULL (pkv_last_error) on failure. */
PKV_API pkv_shards* pkv_shards_create(const pkv_shard_config* cfg, const int* devices);
PKV_API void pkv_shards_destroy(pkv_shards* s);
/* A request of `length` rows owned by `shard` (round-robin ownership is request % ngpus, the caller's choice): takes a
 * slot and pages from that shard's allocator. */
PKV_API int pkv_shards_add(pkv_shards* s, int request, int shard, int length);
PKV_API int pkv_shards_remove(pkv_shards* s, int request);
PKV_API int pkv_shards_owner(const pkv_shards* s, int request);
PKV_API int pkv_shards_length(const pkv_shards* s, int request);
PKV_API int pkv_shards_slot(const pkv_shards* s, int request);
/* The shard's requests that take part in steps, ascending: the order of the rows of pkv_shard_io. Returns the count. */
PKV_API int pkv_shards_local(const pkv_shards* s, int shard, int32_t* requests_out, int cap);
PKV_API int pkv_shards_free_pages(const pkv_shards* s, int shard);
/* Device pointers of a shard (for filling pools and reading requests back with the single-sequence entry points) and
 * its step stream (a cudaStream_t). pkv_shards_tables uploads the block table first if it changed; the upload is
 * ordered on the step stream. */
PKV_API void* pkv_shards_row_pool(pkv_shards* s, int shard, int layer);
PKV_API void* pkv_shards_key_pool(pkv_shards* s, int shard, int layer);
PKV_API const int32_t* pkv_shards_tables(pkv_shards* s, int shard);
PKV_API void* pkv_shards_stream(pkv_shards* s, int shard);
/* One decode step on every shard at once: each local request appends one row per layer at its length and gathers its
 * k index entries (one pkv_step_run per layer on the shard's stream, issued by the shard's own host thread); lengths
 * advance by one. io is [ngpus][layers]. Returns when every shard's launches are queued. */
PKV_API int pkv_shards_step(pkv_shards* s, const pkv_shard_io* io);
/* Timing on the device: pkv_shards_mark records event 0 / 1 on every shard's step stream, pkv_shards_elapsed_ms waits
 * for events 1 and gives the milliseconds between the two per shard (ms_out [ngpus]). pkv_shards_sync waits for all
 * streams of all shards. */
PKV_API int pkv_shards_mark(pkv_shards* s, int which);
PKV_API int pkv_shards_elapsed_ms(pkv_shards* s, float* ms_out);
PKV_API int pkv_shards_sync(pkv_shards* s);
/* Migration. begin: each request leaves its shard's steps at once; the destination takes pages from its own
 * allocator (ids as alloc_pages gives them, logical order) and queues ONE pull of all layers' pages on its migration
 * stream, behind an event that orders it after the steps already queued on the source. Other requests keep stepping on
 * both shards meanwhile. end: for every pull whose event has completed (wait != 0: waits on the host for all of them)
 * the source's pages are released, the destination's later steps are ordered behind the pull and the request joins
 * the destination's steps; returns how many finished. stats: bytes moved and, per destination shard, the summed
 * device time of the pull kernels alone (CUDA events on the migration stream). */
PKV_API int pkv_shards_migrate_begin(pkv_shards* s, const int32_t* requests, const int32_t* dst_shards, int n);
PKV_API int pkv_shards_migrate_end(pkv_shards* s, int wait);
PKV_API int pkv_shards_migrate_pending(const pkv_shards* s); /* begun and not yet ended */
PKV_API int pkv_shards_migrate_landed(pkv_shards* s);        /* of those, pulls whose event has completed (a query: nothing changes) */
PKV_API int pkv_shards_migrate_stats(pkv_shards* s, double* bytes_out, float* kernel_ms_out);

/* ------------------------------------------------------------------------------------------------------------------
 * Page pool: the block allocator, prefix-cache bookkeeping and block tables of src/engine/engine.{hpp,cpp}
 * (free_pages_/evictable_/page_by_hash_/page_info_/tables_: engine.hpp:258-306) as a host-side object, plus the
 * copy-on-write, LRU-free and compaction rules. Host only; single-threaded like the engine thread.
 * ---------------------------------------------------------------------------------------------------------------- */

typedef struct pkv_pool pkv_pool;

PKV_API pkv_pool* pkv_pool_create(int num_pages, int page_tokens, int max_slots, int max_pages_per_seq, int prefix_cache);
PKV_API void pkv_pool_destroy(pkv_pool* p);

/* A sequence handle is a small integer owned by the pool. */
PKV_API int pkv_pool_seq_open(pkv_pool* p);                 /* new empty sequence (no slot yet); returns handle >= 0 */
/* match_prefix (engine.cpp:284-336) without the snapshot condition: shares every cached full page whose chained
 * hash matches tokens[0..ntokens), up to (ntokens-1)/page_tokens pages (or `limit_pages` if >= 0). Returns the
 * number of tokens covered. boundary_ok[i] (may be NULL = all) says whether the sequence may resume at the end of page
 * i (the reference resumes only where a state snapshot was saved). */
PKV_API int pkv_pool_match_prefix(pkv_pool* p, int seq, const int32_t* tokens, int ntokens, const uint8_t* boundary_ok);
/* The same two calls for sequences that hold image blocks: positions are named by 64-bit keys instead of token ids —
 * token_key of src/engine/engine.cpp:264-270: uint32(token) for text, mix64(image hash + offset in the block) for the
 * positions of an image block (every image's placeholder tokens are the same few ids, so the tokens alone would name
 * different images alike). pkv_token_keys fills keys_out [n] from the tokens and the blocks (starts, lens, hashes)
 * [nimages] in position order; pkv_page_hash_keys is pkv_page_hash over keys. The reference's second image rule,
 * "never resume inside a whole image block" (engine.cpp:292-296), is the caller's boundary_ok. */
PKV_API int pkv_token_keys(const int32_t* tokens, int n, const int32_t* starts, const int32_t* lens, const uint64_t* hashes,
                           int nimages, uint64_t* keys_out);
PKV_API int pkv_pool_match_prefix_keys(pkv_pool* p, int seq, const uint64_t* keys, int nkeys, const uint8_t* boundary_ok);
PKV_API int pkv_pool_register_keys(pkv_pool* p, int seq, const uint64_t* keys, int nkeys, int done_pos);
/* How many leading full pages (at most (nkeys - 1) / page_tokens) the prefix cache names right now — the walk
 * match_prefix makes (engine.cpp:289-291) before it looks for a boundary with a saved state; nothing changes. */
PKV_API int pkv_pool_cached_prefix_keys(const pkv_pool* p, const uint64_t* keys, int nkeys);
PKV_API uint64_t pkv_page_hash_keys(const uint64_t* keys, int page_tokens, int page_index);
PKV_API int pkv_pool_assign_slot(pkv_pool* p, int seq);     /* free_slots_.back(); writes the table row; -1 if none */
/* alloc_pages (engine.cpp:437-444): pages for positions [0, upto). Returns 1, or 0 (nothing changed) when the pool
 * cannot supply them. */
PKV_API int pkv_pool_alloc(pkv_pool* p, int seq, int upto);
/* register_pages (engine.cpp:340-353): names the sequence's full pages below done_pos by the chained hash of
 * tokens. */
PKV_API int pkv_pool_register(pkv_pool* p, int seq, const int32_t* tokens, int ntokens, int done_pos);
/* release (engine.cpp:208-232): unref pages tail first and give the slot back. The handle stays open and empty (a
 * preempted request is admitted again later, engine.cpp:428-435); pkv_pool_seq_close releases and retires it. */
PKV_API int pkv_pool_release(pkv_pool* p, int seq);
/* The page half of drop_prefix (engine.cpp:419-425): the pages of a matched prefix whose snapshot could not be read
 * back are unreferenced tail first; the sequence keeps its slot and is computed again from position 0. */
PKV_API int pkv_pool_drop_prefix(pkv_pool* p, int seq);
PKV_API int pkv_pool_seq_close(pkv_pool* p, int seq);

/* Copy-on-write fork: the new sequence shares ALL pages of positions [0, ntokens) of `from`, including a partial
 * last page (refs++ each). Returns the new handle. */
PKV_API int pkv_pool_fork(pkv_pool* p, int from, int ntokens);
/* Before writing rows [s0, s0+n) of seq: every touched page that is not privately writable — another sequence
 * references it (refs > 1), or the prefix cache names it (writing in place would leave modified rows under the old
 * name for a later pkv_pool_match_prefix) — is replaced by take_page() in the sequence's table (old refs--; a named
 * page whose last reference this was stays cached and becomes evictable). Emits the (src, dst) page pairs whose
 * payload must be duplicated with pkv_copy_pages before the write. A named page held by this sequence alone loses its
 * name and is written in place when the pool has no page to spare. Returns the pair count; -1 when the pool cannot
 * supply the pages or an argument is bad; -2 when cap (or a NULL output) cannot take the pairs. On -1 and -2 NOTHING
 * has changed: pkv_pool_cow_pairs gives the count to size the arrays with, and the call can be repeated. */
PKV_API int pkv_pool_cow(pkv_pool* p, int seq, int s0, int n, int32_t* src_out, int32_t* dst_out, int cap);
PKV_API int pkv_pool_cow_pairs(const pkv_pool* p, int seq, int s0, int n); /* pairs pkv_pool_cow would emit now; -1: no room */
/* Moves up to `count` pages from the LRU front of the evictable list to the free list (the evict branch of
 * take_page, engine.cpp:239-245, without handing the page out). Returns how many were freed. */
PKV_API int pkv_pool_free_lru(pkv_pool* p, int count, int32_t* freed_out, int cap);
/* Hole-filling compaction: with W live pages, live ids >= W (ascending) move into free ids < W (ascending);
 * tables, page info, hash map and LRU entries are rewritten and the free list rebuilt descending. Emits the moves for
 * pkv_copy_pages. Returns the move count; -2 (and nothing has changed) when cap or a NULL output cannot take the moves
 * that pkv_pool_compact_pairs counts. */
PKV_API int pkv_pool_compact(pkv_pool* p, int32_t* src_out, int32_t* dst_out, int cap);
PKV_API int pkv_pool_compact_pairs(const pkv_pool* p);

/* Migration between two pools (shards): the sequence's pages leave `src` (unref) and are taken from `dst` in
 * logical order; returns the pair count, the new handle in dst through seq_out, and emits the (src page, dst page)
 * pairs. -1: dst cannot hold the sequence or a bad argument; -2: cap (or a NULL output) is smaller than the sequence's
 * page count (pkv_pool_seq_pages). Nothing has changed on -1 and -2. */
PKV_API int pkv_pool_migrate(pkv_pool* src, int seq, pkv_pool* dst, int* seq_out, int32_t* src_out, int32_t* dst_out,
                     int cap);

/* Introspection (tests, metrics: src/engine/engine.hpp:134-152 free_pages / cached_pages). */
PKV_API int pkv_pool_available(const pkv_pool* p);       /* available_pages(): free + evictable (engine.hpp:181) */
PKV_API int pkv_pool_free_count(const pkv_pool* p);      /* free_pages_.size() */
PKV_API int pkv_pool_evictable_count(const pkv_pool* p); /* evictable_.size() */
PKV_API int pkv_pool_cached_count(const pkv_pool* p);    /* page_by_hash_.size() */
PKV_API int pkv_pool_seq_pages(const pkv_pool* p, int seq, int32_t* out, int cap);
PKV_API int pkv_pool_seq_slot(const pkv_pool* p, int seq);
PKV_API int pkv_pool_page_refs(const pkv_pool* p, int page);
PKV_API uint64_t pkv_pool_page_hash(const pkv_pool* p, int page); /* 0 when not cached */
PKV_API int pkv_pool_dirty(pkv_pool* p);                 /* tables_dirty_: 1 once since the last pkv_pool_tables call */
/* tables_ [max_slots][max_pages_per_seq] (host pointer, valid until the pool is destroyed); clears the dirty flag. */
PKV_API const int32_t* pkv_pool_tables(pkv_pool* p);
PKV_API int pkv_pool_free_list(const pkv_pool* p, int32_t* out, int cap);      /* in vector order (back is taken next) */
PKV_API int pkv_pool_evictable_list(const pkv_pool* p, int32_t* out, int cap); /* oldest first */
/* The chained page hash (engine.cpp:257-280) of page `page_index` of a token sequence. */
PKV_API uint64_t pkv_page_hash(const int32_t* tokens, int page_tokens, int page_index);

/* ------------------------------------------------------------------------------------------------------------------
 * Snapshot store: the bookkeeping around pkv_state_copies — which snapshot slot a save goes into, which one a prefix
 * hit restores, eviction, and the disk tier (a preallocated O_DIRECT file, one I/O thread, a 64-bit checksum checked on
 * read) — of src/engine/engine.cpp:87-92,284-336,361-397,949-970,1011-1261, as a host-side object (the C++ class is
 * unholy_b200/csrc/snapshot_store.hpp; this C form takes snapshots that are one contiguous host region each, snapshot
 * id at host_base + id * snap_bytes). Host only; one owner thread, like the engine thread. Entries do not outlive the
 * store: the file is removed when it is destroyed.
 * ---------------------------------------------------------------------------------------------------------------- */
typedef struct pkv_snap pkv_snap;
typedef struct pkv_snap_hit {
  int32_t pages;      /* the prefix covers this many full pages; 0: no hit */
  int32_t snap;       /* RAM snapshot to restore; the caller holds a reference until pkv_snap_put */
  int32_t disk_slot;  /* >= 0: snap is an empty RAM slot that pkv_snap_start_load must fill from this disk slot first */
  int32_t reserved;
  uint64_t hash;      /* name of the boundary */
} pkv_snap_hit;
typedef struct pkv_snap_done { /* a finished disk operation */
  int32_t write, ok, snap, reserved;
  uint64_t load_id;   /* reads: what pkv_snap_start_load returned */
} pkv_snap_done;
typedef struct pkv_snap_counters_t { /* src/engine/engine.hpp:147-149 (snapshots, free_snapshots, disk_snapshots, snapshot_io, ...) */
  int32_t cached, free_or_evictable, on_disk, io_pending;
  uint64_t spills, disk_hits, disk_read_bytes, disk_write_bytes;
} pkv_snap_counters_t;
/* dir NULL / empty or disk_slots <= 0: no disk tier. io_hook (may be NULL) runs on the I/O thread before every
 * operation (the reference's EngineConfig::io_hook, src/engine/engine.hpp:131: tests stall or corrupt through it). */
PKV_API pkv_snap* pkv_snap_create(int ram_slots, uint8_t* host_base, size_t snap_bytes, const char* dir, int disk_slots,
                                  void (*io_hook)(int write, void* user), void* hook_user);
PKV_API void pkv_snap_destroy(pkv_snap* s);
PKV_API int pkv_snap_disk_on(const pkv_snap* s);
/* match_prefix's snapshot half (engine.cpp:287-333): page_hashes[i] names the boundary at the end of page i (only
 * boundaries whose pages are all cached should be offered), allow[i] == 0 rules one out (NULL: all allowed). */
PKV_API int pkv_snap_match(pkv_snap* s, const uint64_t* page_hashes, int npages, const uint8_t* allow, pkv_snap_hit* hit_out);
PKV_API uint64_t pkv_snap_start_load(pkv_snap* s, const pkv_snap_hit* hit); /* start_load, engine.cpp:1128-1137; returns the load id */
PKV_API void pkv_snap_cancel_load(pkv_snap* s, const pkv_snap_hit* hit);    /* a disk hit given up before its load was started */
PKV_API int pkv_snap_take(pkv_snap* s);                                     /* take_snapshot; -1: none */
PKV_API void pkv_snap_put(pkv_snap* s, int id);                             /* put_snapshot */
/* commit_snapshot: the save into id completed and names `hash`; rolling_id / rolling_hash are the sequence's (in and out). */
PKV_API void pkv_snap_commit(pkv_snap* s, int id, uint64_t hash, int past_prompt, int* rolling_id, uint64_t* rolling_hash);
PKV_API int pkv_snap_spare(const pkv_snap* s);                              /* free + droppable slots (engine.cpp:577-580) */
PKV_API void pkv_snap_spill(pkv_snap* s);                                   /* spill, engine.cpp:1163-1187 */
PKV_API int pkv_snap_poll(pkv_snap* s, pkv_snap_done* done_out, int cap);   /* poll_io; returns the number of completions */
PKV_API void pkv_snap_clear(pkv_snap* s);                                   /* the snapshot half of clear_cache */
PKV_API void pkv_snap_wait_idle(pkv_snap* s);                               /* tests: the I/O thread has nothing queued or running */
PKV_API int pkv_snap_counters(const pkv_snap* s, pkv_snap_counters_t* out);

#ifdef __cplusplus
}
#endif
#endif /* UNHOLY_PKV_H */
