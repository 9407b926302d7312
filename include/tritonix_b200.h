/*
 * tritonix_b200 — C ABI of the dense-contraction path (GEMM, split-K GEMM, fused GLU/SwiGLU)
 * for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes.  The library never allocates or frees
 * device memory (outputs, the split-K workspace and the status word all belong to the caller)
 * and never synchronises the host with the device unless the function's comment says so.  Kernels are enqueued on the
 * stream handle that is passed in (a cudaStream_t cast to void*; NULL = default stream).
 *
 * Status codes (returned by every function that returns int):
 *   TNX_OK                0  success (kernel enqueued)
 *   TNX_ERR_INVALID       1  bad shape / stride / alignment / dtype / null pointer
 *   TNX_ERR_RESOURCES     2  configuration exceeds the shared-memory or TMEM budget of one SM
 *                            (the "out of resources" condition the tuner prunes on; decided on
 *                            the host before any launch)
 *   TNX_ERR_NOT_BUILT     3  configuration is valid in principle but has no compiled kernel
 *   TNX_ERR_CUDA          4  CUDA runtime / driver error; text in tnx_last_error()
 *   TNX_ERR_DEVICE        5  the device status word is non-zero (a bounded wait in a kernel
 *                            gave up); only returned by tnx_read_status()
 */
#ifndef TRITONIX_B200_H_
#define TRITONIX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TNX_OK 0
#define TNX_ERR_INVALID 1
#define TNX_ERR_RESOURCES 2
#define TNX_ERR_NOT_BUILT 3
#define TNX_ERR_CUDA 4
#define TNX_ERR_DEVICE 5

/* element types of A, B and C (C always has the type of A and B) */
#define TNX_F16 0
#define TNX_BF16 1
#define TNX_F32 2

/* epilogue applied to the fp32 accumulator before the cast to the output type */
#define TNX_EPI_NONE 0        /* C = A.B                                                    */
#define TNX_EPI_GLU_LINEAR 1  /* Z[:, j] = acc[:, 2j] * acc[:, 2j+1]        (activation="none") */
#define TNX_EPI_GLU_SILU 2    /* Z[:, j] = silu(acc[:, 2j]) * acc[:, 2j+1]  (activation="silu") */
#define TNX_EPI_GLU_SIGMOID 3 /* Z[:, j] = sigmoid(acc[:, 2j]) * acc[:, 2j+1]                   */

/* order in which the persistent CTAs walk the output tiles */
#define TNX_ORDER_GROUPED 0    /* bands of group_m tile rows, column-major inside a band       */
#define TNX_ORDER_SERPENTINE 1 /* same bands, boustrophedon: consecutive tiles share an operand */
#define TNX_ORDER_TABLE 2      /* caller-supplied table (e.g. a Hilbert curve), see tile_table  */

/* which kernel family executes the call */
#define TNX_KERNEL_AUTO 0    /* tcgen05 path when the operands qualify, else the strided path */
#define TNX_KERNEL_TCGEN05 1 /* TMA + tcgen05.mma + TMEM; fails with TNX_ERR_INVALID otherwise */
#define TNX_KERNEL_STRIDED 2 /* CUDA-core kernel for arbitrary strides, odd sizes and fp32     */

/*
 * One contraction problem.  Replaces the positional arguments of the reference's Triton
 * kernels: (a_ptr, b_ptr, c_ptr, m, n, k, stride_am, stride_ak, stride_bk, stride_bn,
 * stride_cm, stride_cn) of matmul_kernel (tritonix/ops/matmul.py:42-56), gemm_splitk_kernel
 * (tritonix/ops/matmul.py:147-161) and glu_kernel (tritonix/ops/swiglu.py:24-37).
 * Strides are in elements.  For the GLU epilogues n is the number of columns of the
 * interleaved weight matrix W12 (n = 2F) and the output has n/2 columns, exactly as the
 * reference passes it (tritonix/ops/swiglu.py:104-110).
 */
typedef struct tnx_problem {
  int32_t m, n, k;
  int32_t dtype;    /* TNX_F16 | TNX_BF16 | TNX_F32 */
  int32_t epilogue; /* TNX_EPI_* */
  int32_t reserved0;
  int64_t stride_am, stride_ak;
  int64_t stride_bk, stride_bn;
  int64_t stride_cm, stride_cn;
} tnx_problem;

/*
 * Kernel configuration = the tuner's search space (replaces the constexpr / launch keyword
 * arguments block_m, block_n, block_k, group_m, split_k, num_stages of the reference's kernels,
 * tritonix/ops/matmul.py:33-39,136-143).  Zero in any field selects the library default.
 */
typedef struct tnx_config {
  int32_t tile_m;     /* rows of C per CTA (128) or per CTA pair (256 when cta_group == 2)        */
  int32_t tile_n;     /* columns of B per tile: 64, 128 or 256; 512 = a CTA pair computes two
                         column-adjacent 256-column tiles from one stream of A (needs
                         cta_group 2, split_k 1, acc_stages 2, a computed tile order, row-major B) */
  int32_t tile_k;     /* K elements per pipeline stage: 64 or 128                                 */
  int32_t stages;     /* depth of the TMA -> shared-memory ring, >= 2                             */
  int32_t acc_stages; /* TMEM accumulator buffers: 1 or 2 (2 overlaps epilogue and main loop)     */
  int32_t cta_group;  /* 1 = one SM per tile, 2 = tcgen05 cta_group::2 (CTA pair shares one tile) */
  int32_t split_k;    /* K slices per tile, >= 1; > 1 needs the workspace                         */
  int32_t group_m;    /* band height of the grouped / serpentine order                            */
  int32_t tile_order; /* TNX_ORDER_*                                                              */
  int32_t kernel;     /* TNX_KERNEL_*                                                             */
  int32_t max_ctas;   /* cap on the persistent grid (0 = one CTA per SM)                          */
  int32_t reserved0;
} tnx_config;

/* What a (problem, config) pair needs.  Filled by tnx_gemm_query(). */
typedef struct tnx_resources {
  int32_t kernel;          /* TNX_KERNEL_TCGEN05 or TNX_KERNEL_STRIDED: the family that will run */
  int32_t smem_bytes;      /* dynamic shared memory per CTA                                      */
  int32_t tmem_columns;    /* TMEM columns allocated per CTA (power of two, <= 512)              */
  int32_t grid;            /* CTAs launched                                                      */
  int32_t tiles_m, tiles_n;
  int32_t split_k;         /* effective split (clamped so that no slice is empty)                */
  int32_t reserved0;
  int64_t workspace_bytes; /* bytes of caller-owned scratch needed at this split_k (0 if none)   */
} tnx_resources;

/* Library version, "major.minor.patch". */
const char* tnx_version(void);

/* Text of the most recent error on the calling thread ("" if none). */
const char* tnx_last_error(void);

/* Number of SMs of the current device (0 and TNX_ERR_CUDA text if there is none). */
int tnx_sm_count(void);

/*
 * Resource query: validates (problem, config), fills *out and returns TNX_OK,
 * TNX_ERR_INVALID, TNX_ERR_RESOURCES or TNX_ERR_NOT_BUILT without touching the device.
 * This is the host-side replacement for Triton raising OutOfResources at launch
 * (tritonix/autotune.py:134-138): the tuner calls it (through tnx_gemm) before timing.
 */
int tnx_gemm_query(const tnx_problem* problem, const tnx_config* config, tnx_resources* out);

/*
 * C = epilogue(A . B).  Replaces a launch of matmul_kernel / gemm_splitk_kernel / glu_kernel
 * (tritonix/ops/matmul.py:222-236, :249-263; tritonix/ops/swiglu.py:24-110).
 *
 *   a, b, c      device pointers (c: m x n, or m x n/2 for a GLU epilogue)
 *   workspace    device scratch of at least tnx_resources.workspace_bytes, 256-byte aligned;
 *                may be NULL when workspace_bytes == 0.  The first 64 KiB hold the split-K
 *                tile counters and MUST be zero before the first call that uses the buffer;
 *                the kernel leaves them zero again, so no clearing is needed between calls.
 *                Calls that share a workspace must be ordered on one stream.
 *   tile_table   device int32[tiles_m*tiles_n], entry t = (tile_row << 16) | tile_col of the
 *                t-th tile to process; only read when config->tile_order == TNX_ORDER_TABLE
 *   status_word  device int32 that a kernel sets to a non-zero code if one of its bounded
 *                waits expires (may be NULL).  Read it with tnx_read_status().
 *   stream       cudaStream_t
 */
int tnx_gemm(const tnx_problem* problem, const tnx_config* config, const void* a, const void* b,
             void* c, void* workspace, size_t workspace_bytes, const int32_t* tile_table,
             int32_t* status_word, void* stream);

/*
 * Convenience wrapper over tnx_gemm for the fused gate*up product: problem->epilogue is
 * overridden by `activation` (TNX_EPI_GLU_LINEAR / _SILU / _SIGMOID).  Replaces
 * glu_kernel[grid](x, w12, z, m, n, k, ..., activation=...) (tritonix/ops/swiglu.py:24-43).
 */
int tnx_glu(const tnx_problem* problem, const tnx_config* config, int activation, const void* x,
            const void* w12, void* z, const int32_t* tile_table, int32_t* status_word,
            void* stream);

/* Size of the split-K scratch built into the library (per GPU): 64 KiB of tile counters plus
 * 16 MiB of fp32 partial tiles. */
#define TNX_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u + 65536u)

/*
 * Split-K GEMM for callers that cannot provide a workspace.  No counterpart in the reference:
 * its split-K accumulates into C with atomics and needs no scratch
 * (tritonix/ops/matmul.py:195-202); the ordered reduction here does.
 *
 * Same computation and arguments as tnx_gemm with epilogue, split_k and the other config fields
 * honoured, but the scratch is a fixed array inside the library instead of a caller-owned
 * buffer, and the call performs no device-memory allocation of any kind (no cudaMalloc, no
 * cudaFree, no allocating library routine).  It is meant for hosts that must not allocate once
 * they are running — e.g. a serving runtime whose device memory is fully owned by its own
 * arena, or a latency-critical loop that cannot afford the device-wide synchronisation an
 * allocation may cause.
 *
 * Limits and rules:
 *   - the scratch the problem needs at the chosen split_k (tnx_resources.workspace_bytes from
 *     tnx_gemm_query) must not exceed TNX_STATIC_SCRATCH_BYTES, else TNX_ERR_INVALID with the
 *     required and available sizes in tnx_last_error(); the array costs that much memory on
 *     every GPU that loads the library, for the life of the process;
 *   - only the tcgen05 kernel family is served (operands that would need the strided kernel are
 *     rejected with TNX_ERR_INVALID); tile_order TNX_ORDER_TABLE is not available;
 *   - the first call on each device looks up the array's device address (a one-time set-up
 *     under that device); make that first call before any stream capture begins;
 *   - all calls on a device share the one array, which still holds the previous call's
 *     contents: the counters are cleared on `stream` at the start of every call, the rest is
 *     overwritten before it is read.  Two calls whose kernels can overlap on the GPU (different
 *     streams, no ordering between them) race on it — order them.
 */
int tnx_gemm_splitk_static(const tnx_problem* problem, const tnx_config* config, const void* a,
                           const void* b, void* c, int32_t* status_word, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The SwiGLU MLP block in one launch:  Y = ( act(X.W1) * (X.W2) ) . W3.
 * Replaces a launch of swiglu_kernel[grid](x, w12, w3, z, m, n, k, f, stride_xm, stride_xk,
 * stride_wk, stride_wn, stride_w3n, stride_w3l, stride_zm, stride_zl, ...) (tritonix/ops/
 * swiglu.py:113-230; the two-phase design with a workspace and per-row-block flags is sketched
 * in playground/fused_mlp.py:10-161).  Unlike the reference's kernel it is correct for any size,
 * takes fp16/bf16, and is deterministic (no atomics on data).
 * ------------------------------------------------------------------------------------------- */
typedef struct tnx_mlp_problem {
  int32_t m;          /* rows of X and Y (tokens)                                               */
  int32_t d_model;    /* columns of X = rows of W12           (the reference's k)               */
  int32_t d_ff;       /* hidden units F: W12 has 2F interleaved columns (the reference's n / 2) */
  int32_t n_out;      /* columns of W3 and Y                  (the reference's f)               */
  int32_t dtype;      /* TNX_F16 or TNX_BF16, shared by X, W12, W3, Y and the hidden activation */
  int32_t activation; /* TNX_EPI_GLU_LINEAR / _SILU / _SIGMOID                                  */
  int64_t stride_xm;  /* row pitches in elements; rows are contiguous (inner stride 1)          */
  int64_t stride_w12k;
  int64_t stride_w3k;
  int64_t stride_ym;
} tnx_mlp_problem;

typedef struct tnx_mlp_resources {
  int32_t smem_bytes, tmem_columns, grid;
  int32_t tiles_m;             /* 256-row tiles                                                 */
  int32_t band_rows;           /* rows of X per band = group_m * 256                            */
  int32_t num_bands;
  int64_t min_workspace_bytes; /* counters + two bands of the hidden activation (or all of it)  */
  int64_t workspace_bytes;     /* recommended size (currently the minimum: it measured best)    */
} tnx_mlp_resources;

/*
 * Tensor-parallel use: the hidden dimension is split over `world` GPUs (rank r holds columns
 * [2 r F/p, 2 (r+1) F/p) of W12 and rows [r F/p, (r+1) F/p) of W3, d_ff = F/p in the problem), so
 * every rank computes a partial Y; the kernel then sums the partials itself, row tile by row
 * tile while later tiles are still being computed, through an NVLink multicast mapping
 * (multimem.ld_reduce / multimem.st), and every rank ends up with the full Y.  The partial
 * outputs stay in fp32 until they have been summed, so Y carries one rounding, as on one GPU.
 * No counterpart in the reference (it has no multi-GPU code).  Requirements, all the caller's to
 * set up:
 *   - `y` (the pointer passed to tnx_swiglu_mlp) is this rank's mapping of a buffer that every
 *     rank allocated symmetrically and bound to ONE multicast object; y_multicast is the
 *     multicast address of the same bytes;
 *   - partial_local / partial_multicast: likewise for a buffer of m x n_out fp32 values (rows
 *     contiguous, pitch n_out) that receives this rank's partial outputs.  Both may be NULL:
 *     the partial outputs are then rounded to the output type, stored in Y and summed in place
 *     (fp32 accumulation in the switch, a second rounding) — half the NVLink traffic, for an
 *     error of about two roundings instead of one;
 *   - signal_local / signal_multicast: likewise for an array of 1 + signal_tiles uint32
 *     counters (signal_tiles >= (m + 255) / 256 for the largest m ever passed with these
 *     buffers), zero before the first call and never written by the caller afterwards;
 *   - epoch: 1 for the first call on these buffers, 2 for the second, ... identical on every
 *     rank (counters are never reset; call number e waits for e * world arrivals).  After a
 *     call that reported TNX_ERR_DEVICE the counters are undefined: zero them on every rank and
 *     restart at 1;
 *   - every rank makes the same sequence of calls with the same m, n_out, tile_split and
 *     signal_tiles (m may change from call to call).
 * A tensor-parallel launch has 256 threads per CTA: two warps of every CTA form a crew that
 * exchanges while the other six compute.  tile_split (1, 2, 4 ...; 0 = 16, halved until
 * world * tile_split divides 256) is the number of crews that share one row tile's exchange.
 */
typedef struct tnx_mlp_exchange {
  int32_t world, rank;
  int32_t tile_split;
  uint32_t epoch;
  int32_t signal_tiles;
  int32_t reserved0;
  void* y_multicast;
  float* partial_local;
  const float* partial_multicast;
  uint32_t* signal_multicast;
  const uint32_t* signal_local;
} tnx_mlp_exchange;

/* Validates (problem, config) and reports what the launch needs.  `config` may be NULL; used
 * fields: tile_k (64 or 128), stages, group_m (256-row tiles per band, default 8), max_ctas.
 * tile_m / tile_n / cta_group, if set, must be 256 / 256 / 2. */
int tnx_swiglu_mlp_query(const tnx_mlp_problem* problem, const tnx_config* config,
                         tnx_mlp_resources* out);

/*
 * The fixed global order in which the kernel's work units are walked (host-side, no device
 * needed; used to check the dependency rule: a unit only waits for units earlier in the order).
 * Writes up to `capacity` entries (down << 30) | (row_tile << 14) | column_tile — down = 0 for a
 * hidden-activation tile, 1 for an output tile — and returns the number of units, or minus a
 * TNX_ERR_* code.
 */
int tnx_swiglu_mlp_unit_order(const tnx_mlp_problem* problem, const tnx_config* config,
                              int32_t* units, int32_t capacity);

/*
 * Enqueues the fused MLP on `stream`.  `workspace` (256-byte aligned, at least
 * min_workspace_bytes) holds the dependency counters, which this call clears on `stream`, and
 * a ring of bands of the hidden activation: the larger it is (up to counters + the whole
 * m x d_ff activation) the further a band's readers are ahead of its slot's next writers.
 * Its content before and after the call is meaningless.  Calls sharing a workspace must be
 * ordered on one stream.  The kernel's CTAs wait for one another through the counters (bounded
 * waits that report through `status_word`), so the launch is sized to what the GPU can hold
 * at once.
 */
int tnx_swiglu_mlp(const tnx_mlp_problem* problem, const tnx_config* config, const void* x,
                   const void* w12, const void* w3, void* y, void* workspace,
                   size_t workspace_bytes, const tnx_mlp_exchange* exchange /* NULL: one GPU */,
                   int32_t* status_word, void* stream);

/*
 * Synchronises `stream`, copies *status_word to the host and returns TNX_OK if it is zero,
 * else TNX_ERR_DEVICE (code available in *code_out if not NULL) after resetting it to zero.
 */
int tnx_read_status(int32_t* status_word, int32_t* code_out, void* stream);

/*
 * Self-test of the failure path (no counterpart in the reference): enqueues a one-warp kernel
 * that waits, with the same bounded wait the GEMM kernels use, on a barrier nothing signals.
 * After `limit_ms` (1..5000) the wait gives up, the kernel writes code 0x1ff to *status_word and
 * returns normally; tnx_read_status() then reports TNX_ERR_DEVICE.  Nothing traps or faults.
 */
int tnx_selftest_bounded_wait(int32_t* status_word, uint32_t limit_ms, void* stream);

/* ---------------------------------------------------------------------------------------------
 * 2-D convolution forward as an implicit GEMM (GEMM_M = batch*h_out*w_out, GEMM_N = c_out,
 * GEMM_K = c_in*filter_h*filter_w).  Replaces a launch of conv2d_forward_kernel[grid](...) as
 * made by conv2d_forward (tritonix/ops/conv2d/forward.py:8-165 and :202-319): same operands
 * (input N x C x H x W, weight C_OUT x C x R x S, optional bias of C_OUT values, all of one
 * dtype), same geometry arguments, fp32 accumulation, output cast to the operand type.
 * ------------------------------------------------------------------------------------------- */
#define TNX_LAYOUT_NCHW 0 /* contiguous N x C x H x W (what the reference requires)             */
#define TNX_LAYOUT_NHWC 1 /* contiguous N x H x W x C (torch.channels_last): no repacking pass */

#define TNX_WEIGHT_KCRS 0   /* C_OUT x C x R x S, contiguous (what the reference passes)        */
#define TNX_WEIGHT_PACKED 1 /* the buffer tnx_conv2d_pack_weights() filled (fp16/bf16 only)     */

typedef struct tnx_conv2d_problem {
  int32_t batch, c_in, h_in, w_in; /* input                                                       */
  int32_t c_out, filter_h, filter_w;
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int32_t dtype;         /* TNX_F16 / TNX_BF16 / TNX_F32                                          */
  int32_t has_bias;      /* 0 or 1                                                                */
  int32_t input_layout;  /* TNX_LAYOUT_*                                                          */
  int32_t output_layout; /* TNX_LAYOUT_*                                                          */
  int32_t weight_layout; /* TNX_WEIGHT_*                                                          */
} tnx_conv2d_problem;

typedef struct tnx_conv2d_resources {
  int32_t kernel;          /* TNX_KERNEL_TCGEN05 (fp16/bf16) or TNX_KERNEL_STRIDED (fp32)        */
  int32_t h_out, w_out;
  int32_t tile_w, tile_h;  /* tcgen05 only: the rows of a tile are tile_w x tile_h output pixels;
                              128 x 1 = 128 consecutive pixels in (image, row, column) order    */
  int32_t smem_bytes, tmem_columns, grid;
  int64_t workspace_bytes; /* repacked input, weights and output; 0 for the fp32 kernel         */
} tnx_conv2d_resources;

/* Output geometry, kernel family, resources and the workspace the caller must provide.
 * `config` may be NULL; only tile_m (128 or 256 rows = one CTA or a CTA pair), tile_n, tile_k,
 * stages, cta_group, group_m and max_ctas are used. */
int tnx_conv2d_query(const tnx_conv2d_problem* problem, const tnx_config* config,
                     tnx_conv2d_resources* out);

/*
 * Weights that do not change between calls (inference) can be repacked once instead of on
 * every call: tnx_conv2d_packed_weight_bytes() gives the size of the packed buffer (0 for
 * fp32, which has no packed form), tnx_conv2d_pack_weights() fills it from C_OUT x C x R x S
 * weights on `stream`; pass it as `weight` with problem->weight_layout = TNX_WEIGHT_PACKED.
 * The packed form depends only on c_in, c_out, filter_h, filter_w and dtype (and on
 * TNX_CONV_NO_FOLD, which must not change between packing and use).
 */
int64_t tnx_conv2d_packed_weight_bytes(const tnx_conv2d_problem* problem);
int tnx_conv2d_pack_weights(const tnx_conv2d_problem* problem, const void* weight, void* packed,
                            void* stream);

/*
 * Enqueues output = conv2d(input, weight) + bias on `stream`.  Never allocates.
 *   fp16/bf16: the input is repacked to N x H x W x C (skipped for TNX_LAYOUT_NHWC with c_in a
 *   multiple of 8), the weights to C_OUT x (R*S) x C zero-padded to 64 channels, both into
 *   `workspace`; a tcgen05 kernel then multiplies tiles of 128 output pixels by the weights,
 *   one TMA box load per filter tap and 64-channel block (im2col-mode boxes of 128 consecutive
 *   pixels; rectangles of pixels fetched with tiled boxes when the padding or the dilated
 *   filter exceeds what an im2col box can express, or when TNX_CONV_TILED is set in the
 *   environment); padding comes from TMA's out-of-range zero fill; the result is written
 *   N x H x W x C and repacked if NCHW is wanted.  Inputs with c_in <= 16 and
 *   filter_w * c_in <= 64 are repacked so that the taps of a filter row become channels
 *   (N x H x W_OUT x filter_w*c_in), which shortens K filter_w-fold; TNX_CONV_NO_FOLD in the
 *   environment keeps one zero-padded 64-channel block per tap instead.
 *   Stride-1 layers with c_in <= 64 and c_out <= 64 whose output rows (plus the filter's halo
 *   columns) have at most 128 pixels keep the weights of all taps in shared memory and load each
 *   tile's input patch once, every tap multiplying a shifted window of it (TNX_CONV_NO_HALO in
 *   the environment disables this).
 *   A 1 x 1, stride-1, unpadded convolution with NCHW input and output, unpacked weights and
 *   h_in*w_in and c_in multiples of 8 runs as one GEMM per image on the tensors as they are (one
 *   launch for the batch, no workspace); TNX_CONV_NO_BATCHED_GEMM in the environment disables it.
 *   fp32: a CUDA-core kernel reads and writes the tensors in place (no workspace).
 * `bias` may be NULL when has_bias == 0.  `workspace` needs workspace_bytes from the query and
 * 256-byte alignment; its content before and after the call is meaningless.
 */
int tnx_conv2d_forward(const tnx_conv2d_problem* problem, const tnx_config* config,
                       const void* input, const void* weight, const void* bias, void* output,
                       void* workspace, size_t workspace_bytes, int32_t* status_word,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRITONIX_B200_H_ */
