// Persistent, warp-specialised GEMM for sm_100a:
//   TMA (cp.async.bulk.tensor) -> 128B-swizzled shared-memory ring -> tcgen05.mma with the fp32
//   accumulator in TMEM -> tcgen05.ld epilogue (plain cast, fused GLU gate*up, or deterministic
//   split-K fix-up) -> TMA store.
//
// It computes what the reference's Triton kernels compute, one 128 x TILE_N tile of C per work
// unit: matmul_kernel (tritonix/ops/matmul.py:42-108), gemm_splitk_kernel (:147-202, with the
// atomic_add of :202 replaced by an ordered fp32 reduction) and glu_kernel
// (tritonix/ops/swiglu.py:24-110).  A is row-major M x K (K-major operand), B is row-major K x N
// (an "MN-major" tcgen05 operand: no transpose pass is needed).
//
// Warp roles in a CTA of 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + tcgen05.mma issue (one elected lane; leader CTA only in pair mode)
//   warps 2..5  epilogue: warp w reads TMEM lanes [32*(w%4), 32*(w%4)+32)
//
// CTA_GROUP == 2 runs tcgen05 cta_group::2: a cluster of two CTAs owns a 256 x TILE_N tile, each
// CTA loads its own 128 rows of A and its own half of the B columns (plain per-CTA TMA loads),
// and the leader CTA issues M=256 MMAs that read both CTAs' shared memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>

#include "tnx_internal.h"
#include "tnx_ptx.cuh"

namespace tnx {

namespace {

constexpr int kRowsPerCta = 128;  // TMEM lanes = rows of C owned by one CTA
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kEpiBarrier = 1;               // named barrier id of the epilogue warps
constexpr int kAtomBytes = 128;              // swizzle span: 64 16-bit elements
constexpr int kAtomElems = 64;
constexpr int kStagingBytes = kRowsPerCta * kAtomBytes;  // 128 rows x 128 B of output
constexpr int kMaxStages = 14;
constexpr int kCtrlBytes = 512;
constexpr int kAlignSlack = 1024;

// Status-word codes written when a bounded wait expires.
constexpr int kAbortProducer = 0x101;
constexpr int kAbortMma = 0x102;
constexpr int kAbortEpilogue = 0x103;

struct UmmaParams {
  int m, n, k;          // n counts columns of B (2F for GLU)
  int n_out;            // columns of C
  int tiles_m, tiles_n; // tiles_m counts (128*CTA_GROUP)-row tiles
  int num_kb;           // K blocks of tile_k in total
  int kb_per_slice;     // K blocks per split-K slice
  int split_k;
  int cluster_split;    // > 0: the split_k slices of a tile form one cluster and exchange their
                        // partials through distributed shared memory (no workspace)
  int tile_k;
  int b_kmajor;         // 1: B is stored N x K (K contiguous, e.g. a transposed weight view)
  int a_mmajor;         // 1: A is stored K x M (M contiguous, e.g. a transposed activation view)
  int staging_bytes;    // epilogue staging region (two 16 KiB store buffers, or one split-K partial)
  int a_rows;           // rows of A that TMA brings in per stage (128, or fewer for a skinny M)
  int stages;
  int acc_stages;
  int wide;             // 1: a CTA pair works on two column-adjacent 256-column tiles at once (one
                        // A stage feeds both accumulators; tiles_n counts such double tiles)
  int group_m;
  int tile_order;
  int epilogue;
  const int32_t* tile_table;
  void* c_ptr;          // C base and row pitch (elements): the split-K fix-up stores C directly
  long long ldc;
  float* partials;      // split-K: fp32 partial tiles
  int* counters;        // split-K: one arrival counter per 128-row output tile
  int* status;
  unsigned long long timeout_ns;
  // Convolution (implicit GEMM): the rows of a CTA's tile are a cv_tw x cv_th rectangle of output
  // pixels of one image, A comes from an N x H x W x C tensor through a 4-D tensor map, and K
  // runs over (filter tap, 64-channel block).
  int conv;                    // 1: rectangles of pixels (tiled boxes); 2: 128 consecutive pixels (im2col boxes);
                               // 3: full-width rectangles, at most 64 input and 64 output channels: a stage =
                               //    the tile's input patch with its halo, the weights of all taps stay in
                               //    shared memory, each tap multiplies a row-shifted window of the patch
  int a_box_bytes;             // conv == 3: bytes one patch load delivers
  int cv_wout, cv_hout;        // output image size
  int cv_tw, cv_th;            // output pixels per CTA tile (cv_tw * cv_th = a_rows)
  int cv_tiles_w, cv_tiles_h;  // CTA tiles per image
  int cv_row_tiles;            // batch * cv_tiles_h * cv_tiles_w
  int cv_cblocks;              // 64-channel blocks per filter tap
  int cv_taps, cv_fw;          // filter_h * filter_w, filter_w
  int cv_sh, cv_sw, cv_ph, cv_pw, cv_dh, cv_dw;
  const void* bias;            // one value per output column, of the operand type, or nullptr
  // Batched GEMM: `batched` independent problems that share A.  B and C are 3-D tensor maps
  // (column, row, matrix); tile row index = matrix * bt_tiles_m + row tile inside the matrix.
  int batched;
  int bt_tiles_m;              // row tiles (CTA pairs count as one) per matrix
  int bias_per_row;            // the bias is indexed by the output row instead of the column
#ifdef TNX_DEV_TRACE
  unsigned long long* trace;  // development builds only: 256 timestamp slots per CTA
#endif
};

// Development aid, compiled only with -DTNX_DEV_TRACE: records %globaltimer into a per-CTA slot.
#ifdef TNX_DEV_TRACE
#define TNX_TRACE(slot)                                                                       \
  do {                                                                                        \
    if (p.trace != nullptr && (slot) < 256)                                                   \
      p.trace[blockIdx.x * 256 + (slot)] = ptx::globaltimer_ns();                             \
  } while (0)
#else
#define TNX_TRACE(slot) do { } while (0)
#endif

// Control block at the end of dynamic shared memory.
struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t xchg_full;   // cluster split-K: every slice's share of this CTA's rows has landed here
  uint64_t xchg_free;   // cluster split-K: every slice has summed what was pushed to it
  uint32_t tmem_base;
  int abort;
  int is_last;
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

__device__ __forceinline__ void tile_coords(const UmmaParams& p, int t, int& tm, int& tn) {
  if (p.tile_order == TNX_ORDER_TABLE) {
    const int v = __ldg(p.tile_table + t);
    tm = v >> 16;
    tn = v & 0xffff;
    return;
  }
  // Bands of group_m tile rows, walked column by column (tl.swizzle2d's mapping, used at
  // tritonix/ops/matmul.py:70).
  const int band_tiles = p.group_m * p.tiles_n;
  const int band = t / band_tiles;
  const int first_row = band * p.group_m;
  const int rows = min(p.tiles_m - first_row, p.group_m);
  const int r = t - band * band_tiles;
  const int col = r / rows;
  int row_in_band = r - col * rows;
  tn = col;
  if (p.tile_order == TNX_ORDER_SERPENTINE) {
    // Boustrophedon variant (the intent of swizzle2d_rows, tritonix/ops/matmul.py:9-27):
    // odd columns run bottom-up, odd bands run right-to-left.
    if (col & 1) row_in_band = rows - 1 - row_in_band;
    if (band & 1) tn = p.tiles_n - 1 - col;
  }
  tm = first_row + row_in_band;
}

__device__ __forceinline__ float gate_act(float g, int epilogue) {
  if (epilogue == TNX_EPI_GLU_LINEAR) return g;
  const float s = __fdividef(1.0f, 1.0f + __expf(-g));
  return epilogue == TNX_EPI_GLU_SILU ? g * s : s;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

template <bool BF16>
__device__ __forceinline__ float unpack1(uint16_t bits) {
  if (BF16) return __uint_as_float(static_cast<uint32_t>(bits) << 16);
  return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ float4 ld_shared_v4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

// Split-K fix-up output: four summed accumulator columns of one row -> epilogue -> C.
// `left` = valid accumulator columns from `acc_col` on (a ragged N leaves fewer than four).
template <bool GLU, bool BF16>
__device__ __forceinline__ void store_fixup(const UmmaParams& p, int row, int acc_col, int left,
                                            const float4& sum) {
  const size_t row_off = static_cast<size_t>(row) * p.ldc;
  uint16_t* c16 = reinterpret_cast<uint16_t*>(p.c_ptr);
  if (GLU) {
    const uint32_t z = pack2<BF16>(gate_act(sum.x, p.epilogue) * sum.y,
                                   gate_act(sum.z, p.epilogue) * sum.w);
    const size_t o = row_off + (acc_col >> 1);
    if (left >= 4) {
      *reinterpret_cast<uint32_t*>(c16 + o) = z;
    } else {  // n is even: exactly one (gate, up) pair is left
      c16[o] = static_cast<uint16_t>(z & 0xffffu);
    }
  } else {
    const uint32_t lo = pack2<BF16>(sum.x, sum.y);
    const uint32_t hi = pack2<BF16>(sum.z, sum.w);
    const size_t o = row_off + acc_col;
    if (left >= 4) {
      *reinterpret_cast<uint2*>(c16 + o) = make_uint2(lo, hi);
    } else {
      c16[o] = static_cast<uint16_t>(lo & 0xffffu);
      if (left > 1) c16[o + 1] = static_cast<uint16_t>(lo >> 16);
      if (left > 2) c16[o + 2] = static_cast<uint16_t>(hi & 0xffffu);
    }
  }
}

template <int TILE_N, int TILE_K, int CTA_GROUP, bool GLU, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const UmmaParams p) {
  constexpr int LOAD_N = TILE_N / CTA_GROUP;          // B columns this CTA loads per stage
  constexpr int ACC_PER_CHUNK = GLU ? 128 : 64;       // accumulator columns per 128-byte output row
  constexpr int OUT_PER_TILE = GLU ? TILE_N / 2 : TILE_N;
  static_assert(LOAD_N % kAtomElems == 0, "each CTA must load whole 64-column swizzle atoms of B");
  static_assert(TILE_N % ACC_PER_CHUNK == 0, "tile_n must cover whole output chunks");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base_addr = (raw_addr + 1023u) & ~1023u;  // 128B swizzle needs 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base_addr - raw_addr);

  // When M < 128 only a_rows rows of A are loaded and stored per stage.  The MMA still reads 128
  // rows: the extra ones come from whatever follows in shared memory and only feed accumulator
  // rows >= M, which are never written out.
  const int a_stage_bytes = p.a_rows * TILE_K * 2;
  const int a_atom_bytes = p.a_rows * kAtomBytes;  // one 64-element K slab of the A stage
  const bool halo = CTA_GROUP == 1 && p.conv == 3;
  constexpr int kBHalfBytes = LOAD_N * TILE_K * 2;  // this CTA's B columns of one tile, one stage
  const int b_stage_bytes = halo ? p.cv_taps * LOAD_N * kAtomBytes : (p.wide ? 2 : 1) * kBHalfBytes;
  const uint32_t smem_a = base_addr;
  const uint32_t smem_b = smem_a + p.stages * a_stage_bytes;
  // (halo convolution: the weights are loaded once per CTA and stay put: one B buffer, not a ring)
  const uint32_t smem_out = smem_b + (halo ? 1 : p.stages) * b_stage_bytes;  // 2 staging buffers
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(base_ptr + (smem_out - base_addr) + p.staging_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Cluster layouts: CTA pair (CTA_GROUP == 2), or the K slices of one tile (cluster_split).
  const bool xchg = CTA_GROUP == 1 && p.cluster_split > 0;
  const uint32_t cluster_size = xchg ? static_cast<uint32_t>(p.cluster_split) : CTA_GROUP;
  const uint32_t cluster_rank = (CTA_GROUP == 2 || xchg) ? ptx::cluster_ctarank() : 0u;
  const uint32_t cta_rank = CTA_GROUP == 2 ? cluster_rank : 0u;  // position inside a CTA pair
  const bool leader = cta_rank == 0;
  const int cluster_id = blockIdx.x / cluster_size;
  const int num_clusters = gridDim.x / cluster_size;
  // Work units: (tile, slice) pairs, or whole tiles when the cluster's CTAs are the slices.
  const int total_units = p.tiles_m * p.tiles_n * (xchg ? 1 : p.split_k);
  const uint32_t tmem_cols_needed = p.acc_stages * TILE_N;
  uint32_t tmem_alloc_cols = 32;
  while (tmem_alloc_cols < tmem_cols_needed) tmem_alloc_cols <<= 1;

  volatile int* abort_flag = &ctrl->abort;

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
    ptx::prefetch_tensormap(&tmap_c);
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->tmem_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->tmem_empty[a]), 4 * CTA_GROUP);  // one arrive per epilogue warp
    }
    ptx::mbar_init(ptx::smem_u32(&ctrl->xchg_full), 1);  // completes by the bytes pushed into this CTA
    ptx::mbar_init(ptx::smem_u32(&ctrl->xchg_free), xchg ? cluster_size : 1);
    ctrl->abort = 0;
    ctrl->is_last = 0;
    ptx::fence_mbar_init();
  }
  __syncwarp();
  if (CTA_GROUP == 2 || xchg) {  // the peers' barriers must exist before anything signals them
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    ptx::tmem_alloc<CTA_GROUP>(ptx::smem_u32(&ctrl->tmem_base), tmem_alloc_cols);
    ptx::tmem_relinquish<CTA_GROUP>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;
  if (threadIdx.x == 0) TNX_TRACE(0);
  // Launched with programmatic stream serialization, everything above (no global memory touched
  // yet: the tensor maps are kernel parameters) ran while the previous kernel of the stream was
  // still finishing.  Its writes are needed, and ours must not overtake its reads, from the
  // first access to global memory on: the producer waits for that kernel just before its first
  // load (its first unit's coordinates are computed by then), every epilogue thread on entry;
  // the MMA thread touches no global memory.  The kernel after this one may start its own
  // set-up as soon as SMs fall free.  Without the launch attribute the instructions do nothing.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ------------------------------------------------------------------ roles
  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t stage_tx =
          halo ? static_cast<uint32_t>(p.a_box_bytes)
               : static_cast<uint32_t>(a_stage_bytes + b_stage_bytes) * CTA_GROUP;
      bool weights_resident = false;  // halo convolution: this CTA's copy of the weights is in place
      bool ok = true;
      bool dependency_met = false;
      if (p.tile_order == TNX_ORDER_TABLE) {  // the tile table is read from global memory
        asm volatile("griddepcontrol.wait;" ::: "memory");
        dependency_met = true;
      }
      for (int u = cluster_id; u < total_units && ok; u += num_clusters) {
        const int t = xchg ? u : u / p.split_k;
        const int slice = xchg ? static_cast<int>(cluster_rank) : u - t * p.split_k;
        int tm, tn;
        tile_coords(p, t, tm, tn);
        const int bt_img = p.batched ? tm / p.bt_tiles_m : 0;  // which matrix of a batch
        const int row0 = ((tm - bt_img * p.bt_tiles_m) * CTA_GROUP + static_cast<int>(cta_rank)) * kRowsPerCta;
        const int col0 = tn * TILE_N * (p.wide ? 2 : 1) + static_cast<int>(cta_rank) * LOAD_N;
        const int kb0 = slice * p.kb_per_slice;
        const int kb1 = min(kb0 + p.kb_per_slice, p.num_kb);
        // Convolution: image and first input column / row (before the tap's offset) of this
        // CTA's pixel rectangle.  A pair's missing last tile gets image = batch: all zero fill.
        int cv_n = 0, cv_x = 0, cv_y = 0;
        // (tap row, tap column, channel block) of the next 64-element K slab; K starts at 0 for
        // every tile of a convolution (no split-K)
        int cv_fr = 0, cv_fs = 0, cv_cb = 0;
        const int cv_fh = p.cv_taps / max(p.cv_fw, 1);
        if (p.conv == 1) {
          const int row_tile = tm * CTA_GROUP + static_cast<int>(cta_rank);
          const int per_image = p.cv_tiles_h * p.cv_tiles_w;
          cv_n = row_tile / per_image;
          const int rem = row_tile - cv_n * per_image;
          const int hb = rem / p.cv_tiles_w;
          cv_y = hb * p.cv_th * p.cv_sh - p.cv_ph;
          cv_x = (rem - hb * p.cv_tiles_w) * p.cv_tw * p.cv_sw - p.cv_pw;
        } else if (p.conv == 2) {
          // first of the tile's 128 consecutive pixels (a pair's missing last tile re-reads
          // tile 0; its rows are never stored)
          int row_tile = tm * CTA_GROUP + static_cast<int>(cta_rank);
          if (row_tile >= p.cv_row_tiles) row_tile = 0;
          const int first = row_tile * kRowsPerCta;
          const int per_image = p.cv_hout * p.cv_wout;
          cv_n = first / per_image;
          const int rem = first - cv_n * per_image;
          const int ho = rem / p.cv_wout;
          cv_y = ho * p.cv_sh - p.cv_ph;
          cv_x = (rem - ho * p.cv_wout) * p.cv_sw - p.cv_pw;
        }
        if (!dependency_met) {
          asm volatile("griddepcontrol.wait;" ::: "memory");
          dependency_met = true;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          const uint32_t empty_bar = ptx::smem_u32(&ctrl->empty[stage]);
          if (!ptx::mbar_wait(empty_bar, phase ^ 1u, abort_flag, p.timeout_ns)) {
            ok = false;
            break;
          }
          const uint32_t full_bar = ptx::smem_u32(&ctrl->full[stage]);
          const uint32_t a_dst = smem_a + stage * a_stage_bytes;
          const uint32_t b_dst = smem_b + stage * b_stage_bytes;
          const int k0 = kb * TILE_K;
          if (CTA_GROUP == 1) {
            ptx::mbar_arrive_expect_tx(
                full_bar, stage_tx + (halo && !weights_resident ? static_cast<uint32_t>(b_stage_bytes) : 0u));
            if (halo) {
              // The stage is the tile's input patch (tile rows + halo rows, full width with halo
              // columns; one channel block).  The first stage of this CTA also brings the weights
              // of every tap, which then stay in shared memory for all its tiles.
              const int row_tile = tm;
              const int img = row_tile / p.cv_tiles_h;
              const int y0 = (row_tile - img * p.cv_tiles_h) * p.cv_th - p.cv_ph;
              ptx::tma_load_4d(a_dst, &tmap_a, 0, -p.cv_pw, y0, img, full_bar);
              if (!weights_resident) {
                for (int tap = 0; tap < p.cv_taps; ++tap)
                  ptx::tma_load_2d(smem_b + tap * (LOAD_N * kAtomBytes), &tmap_b, tap * kAtomElems,
                                   col0, full_bar);
                weights_resident = true;
              }
            } else if (p.conv) {  // one box of pixels x 64 channels per (tap, channel block)
#pragma unroll
              for (int ka = 0; ka < TILE_K / kAtomElems; ++ka) {
                // (past the last tap, in the second half of an odd last K block, a channel
                // coordinate beyond C reads zeros)
                const bool past = cv_fr >= cv_fh;
                const int ch = past ? p.cv_cblocks * kAtomElems : cv_cb * kAtomElems;
                const int off_w = past ? 0 : cv_fs * p.cv_dw, off_h = past ? 0 : cv_fr * p.cv_dh;
                if (p.conv == 1)
                  ptx::tma_load_4d(a_dst + ka * a_atom_bytes, &tmap_a, ch, cv_x + off_w, cv_y + off_h,
                                   cv_n, full_bar);
                else
                  ptx::tma_load_im2col_4d(a_dst + ka * a_atom_bytes, &tmap_a, ch, cv_x, cv_y, cv_n,
                                          static_cast<uint16_t>(off_w), static_cast<uint16_t>(off_h),
                                          full_bar);
                // next (tap, channel block) without dividing
                if (++cv_cb == p.cv_cblocks) {
                  cv_cb = 0;
                  if (++cv_fs == p.cv_fw) {
                    cv_fs = 0;
                    ++cv_fr;
                  }
                }
              }
            } else if (p.a_mmajor) {  // two 64-row atoms of tile_k x 128 B, like a row-major B
#pragma unroll
              for (int ma = 0; ma < kRowsPerCta / kAtomElems; ++ma)
                ptx::tma_load_2d(a_dst + ma * (TILE_K * kAtomBytes), &tmap_a, row0 + ma * kAtomElems,
                                 k0, full_bar);
            } else {
#pragma unroll
              for (int ka = 0; ka < TILE_K / kAtomElems; ++ka)
                ptx::tma_load_2d(a_dst + ka * a_atom_bytes, &tmap_a, k0 + ka * kAtomElems, row0,
                                 full_bar);
            }
            if (halo) {
              // (the weights of this channel block were issued with its patch)
            } else if (p.b_kmajor) {
#pragma unroll
              for (int ka = 0; ka < TILE_K / kAtomElems; ++ka)
                ptx::tma_load_2d(b_dst + ka * (LOAD_N * kAtomBytes), &tmap_b, k0 + ka * kAtomElems,
                                 col0, full_bar);
            } else if (p.batched) {
#pragma unroll
              for (int na = 0; na < LOAD_N / kAtomElems; ++na)
                ptx::tma_load_3d(b_dst + na * (TILE_K * kAtomBytes), &tmap_b, col0 + na * kAtomElems,
                                 k0, bt_img, full_bar);
            } else {
#pragma unroll
              for (int na = 0; na < LOAD_N / kAtomElems; ++na)
                ptx::tma_load_2d(b_dst + na * (TILE_K * kAtomBytes), &tmap_b,
                                 col0 + na * kAtomElems, k0, full_bar);
            }
          } else {
            // Both CTAs' loads complete on the leader's barrier; the leader announces the bytes.
            const uint32_t leader_bar = ptx::mapa(full_bar, 0);
            if (leader) ptx::mbar_arrive_expect_tx(full_bar, stage_tx);
            if (p.conv) {
#pragma unroll
              for (int ka = 0; ka < TILE_K / kAtomElems; ++ka) {
                const bool past = cv_fr >= cv_fh;
                const int ch = past ? p.cv_cblocks * kAtomElems : cv_cb * kAtomElems;
                const int off_w = past ? 0 : cv_fs * p.cv_dw, off_h = past ? 0 : cv_fr * p.cv_dh;
                if (p.conv == 1)
                  ptx::tma_load_4d_pair(a_dst + ka * a_atom_bytes, &tmap_a, ch, cv_x + off_w,
                                        cv_y + off_h, cv_n, leader_bar);
                else
                  ptx::tma_load_im2col_4d_pair(a_dst + ka * a_atom_bytes, &tmap_a, ch, cv_x, cv_y,
                                               cv_n, static_cast<uint16_t>(off_w),
                                               static_cast<uint16_t>(off_h), leader_bar);
                if (++cv_cb == p.cv_cblocks) {
                  cv_cb = 0;
                  if (++cv_fs == p.cv_fw) {
                    cv_fs = 0;
                    ++cv_fr;
                  }
                }
              }
            } else if (p.a_mmajor) {
#pragma unroll
              for (int ma = 0; ma < kRowsPerCta / kAtomElems; ++ma)
                ptx::tma_load_2d_pair(a_dst + ma * (TILE_K * kAtomBytes), &tmap_a,
                                      row0 + ma * kAtomElems, k0, leader_bar);
            } else {
#pragma unroll
              for (int ka = 0; ka < TILE_K / kAtomElems; ++ka)
                ptx::tma_load_2d_pair(a_dst + ka * a_atom_bytes, &tmap_a, k0 + ka * kAtomElems,
                                      row0, leader_bar);
            }
            if (p.b_kmajor) {
#pragma unroll
              for (int ka = 0; ka < TILE_K / kAtomElems; ++ka)
                ptx::tma_load_2d_pair(b_dst + ka * (LOAD_N * kAtomBytes), &tmap_b,
                                      k0 + ka * kAtomElems, col0, leader_bar);
            } else if (p.batched) {
#pragma unroll
              for (int na = 0; na < LOAD_N / kAtomElems; ++na)
                ptx::tma_load_3d_pair(b_dst + na * (TILE_K * kAtomBytes), &tmap_b,
                                      col0 + na * kAtomElems, k0, bt_img, leader_bar);
            } else {
#pragma unroll
              for (int na = 0; na < LOAD_N / kAtomElems; ++na)
                ptx::tma_load_2d_pair(b_dst + na * (TILE_K * kAtomBytes), &tmap_b,
                                      col0 + na * kAtomElems, k0, leader_bar);
              if (p.wide) {  // the same columns of the right-hand tile, behind the left-hand ones
#pragma unroll
                for (int na = 0; na < LOAD_N / kAtomElems; ++na)
                  ptx::tma_load_2d_pair(b_dst + kBHalfBytes + na * (TILE_K * kAtomBytes), &tmap_b,
                                        col0 + TILE_N + na * kAtomElems, k0, leader_bar);
              }
            }
          }
          if (u == cluster_id) TNX_TRACE(64 + (kb - kb0));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      TNX_TRACE(2);
      if (!ok && p.status != nullptr) atomicCAS(p.status, 0, kAbortProducer);
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    if (leader && lane == 0) {
      // Instruction descriptor: fp32 accumulate, A K-major, B MN-major, M x N = (128*CTA_GROUP) x TILE_N.
      const uint32_t fmt = BF16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((p.a_mmajor ? 1u : 0u) << 15) |
                             ((p.b_kmajor ? 0u : 1u) << 16) |
                             (static_cast<uint32_t>(TILE_N >> 3) << 17) |
                             (static_cast<uint32_t>((kRowsPerCta * CTA_GROUP) >> 4) << 24);
      // A: rows of 128 B, 8-row groups 1024 B apart.  B: 64-column atoms of tile_k rows x 128 B;
      // LBO = bytes between atoms along N, SBO = bytes between 8-row groups along K.
      // An A stored K x M is an MN-major operand: 64-row atoms of tile_k x 128 B, LBO to the next atom.
      const uint64_t a_desc_hi =
          p.a_mmajor ? ptx::make_smem_desc(0, TILE_K * kAtomBytes, 1024) : ptx::make_smem_desc(0, 0, 1024);
      // A K-major B (stored N x K) is laid out like A: rows of 128 B, one slab per 64 K elements.
      const uint64_t b_desc_hi =
          p.b_kmajor ? ptx::make_smem_desc(0, 0, 1024) : ptx::make_smem_desc(0, TILE_K * kAtomBytes, 1024);
      // Address steps along K in 16-byte units.  A K-major operand advances 32 B per 16 elements
      // inside a 64-element slab and one slab (rows x 128 B) per 64; an MN-major operand advances
      // 16 rows of 128 B per 16 elements, i.e. 2048 B, and 8192 B per 64.
      const uint32_t a_step16 = (p.a_mmajor ? 2048u : 32u) >> 4;
      const uint32_t a_slab16 = (p.a_mmajor ? 8192u : static_cast<uint32_t>(a_atom_bytes)) >> 4;
      const uint32_t b_step16 = (p.b_kmajor ? 32u : 2048u) >> 4;
      const uint32_t b_slab16 = (p.b_kmajor ? static_cast<uint32_t>(LOAD_N * kAtomBytes) : 8192u) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // The MMAs of one K block of one tile: A and B from ring slot `slot`, B `b_byte_off` bytes
      // into the slot's B area, accumulator at TMEM column `d`.
      auto mma_block = [&](int slot, uint32_t d, uint32_t b_byte_off, uint32_t& accumulate) {
        const uint32_t a16 = (smem_a + slot * a_stage_bytes) >> 4;
        const uint32_t b16 = (smem_b + slot * b_stage_bytes + b_byte_off) >> 4;
#pragma unroll
        for (int k16 = 0; k16 < TILE_K / 16; ++k16) {
          const uint32_t a_off = a16 + (k16 >> 2) * a_slab16 + (k16 & 3) * a_step16;
          const uint32_t b_off = b16 + (k16 >> 2) * b_slab16 + (k16 & 3) * b_step16;
          ptx::umma_f16<CTA_GROUP>(d, a_desc_hi | (a_off & 0x3fffu), b_desc_hi | (b_off & 0x3fffu), idesc,
                                   accumulate);
          accumulate = 1;
        }
      };
      auto commit_to = [&](uint64_t* bar) {
        if (CTA_GROUP == 1)
          ptx::umma_commit(ptx::smem_u32(bar));
        else
          ptx::umma_commit_pair(ptx::smem_u32(bar), 0x3);
      };
      for (int u = cluster_id; u < total_units && ok; u += num_clusters) {
        const int slice = xchg ? static_cast<int>(cluster_rank) : u % p.split_k;
        const int kb0 = slice * p.kb_per_slice;
        const int kb1 = min(kb0 + p.kb_per_slice, p.num_kb);
        if (CTA_GROUP == 2 && p.wide) {
          // ---- two column-adjacent tiles at once: left accumulator in TMEM buffer 0, right in
          // buffer 1, every ring slot's A feeds both.  The epilogue drains the left buffer first,
          // so the left tile's MMAs of the first K blocks (as many as the ring holds) are issued
          // before the right buffer is waited for: the tensor pipe has work while it drains.
          const int nkb = kb1 - kb0;
          const int ahead = min(nkb, p.stages);
          const uint32_t d_left = tmem_base, d_right = tmem_base + TILE_N;
          if (!ptx::mbar_wait<true>(ptx::smem_u32(&ctrl->tmem_empty[0]), acc_phase ^ 1u, abort_flag,
                                    p.timeout_ns)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          uint32_t acc_left = 0, acc_right = 0;
          {
            int st = stage;
            uint32_t ph = phase;
            for (int i = 0; i < ahead && ok; ++i) {
              if (!ptx::mbar_wait(ptx::smem_u32(&ctrl->full[st]), ph, abort_flag, p.timeout_ns)) {
                ok = false;
                break;
              }
              ptx::tc_fence_after_sync();
              mma_block(st, d_left, 0, acc_left);
              if (++st == p.stages) {
                st = 0;
                ph ^= 1u;
              }
            }
          }
          if (!ok) break;
          if (nkb == ahead) commit_to(&ctrl->tmem_full[0]);  // the left tile is complete
          if (!ptx::mbar_wait<true>(ptx::smem_u32(&ctrl->tmem_empty[1]), acc_phase ^ 1u, abort_flag,
                                    p.timeout_ns)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          for (int i = 0; i < nkb && ok; ++i) {
            if (i >= ahead) {
              if (!ptx::mbar_wait(ptx::smem_u32(&ctrl->full[stage]), phase, abort_flag, p.timeout_ns)) {
                ok = false;
                break;
              }
              ptx::tc_fence_after_sync();
              mma_block(stage, d_left, 0, acc_left);
              if (i == nkb - 1) commit_to(&ctrl->tmem_full[0]);
            }
            mma_block(stage, d_right, kBHalfBytes, acc_right);
            commit_to(&ctrl->empty[stage]);  // frees the slot in both CTAs once both tiles have read it
            if (++stage == p.stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (!ok) break;
          commit_to(&ctrl->tmem_full[1]);
          acc_phase ^= 1u;
          continue;
        }
        const uint32_t te_bar = ptx::smem_u32(&ctrl->tmem_empty[acc]);
        if (!ptx::mbar_wait<CTA_GROUP == 2>(te_bar, acc_phase ^ 1u, abort_flag, p.timeout_ns)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          const uint32_t full_bar = ptx::smem_u32(&ctrl->full[stage]);
          if (!ptx::mbar_wait(full_bar, phase, abort_flag, p.timeout_ns)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          if (u == cluster_id) TNX_TRACE(128 + (kb - kb0));
          const uint32_t a_src = smem_a + stage * a_stage_bytes;
          const uint32_t b_src = smem_b + (halo ? 0 : stage * b_stage_bytes);
          const uint32_t a16 = a_src >> 4, b16 = b_src >> 4;  // descriptor addresses count 16 B
          if (halo) {
            // Every tap multiplies the window of the patch that starts (tap row * patch width +
            // tap column) pixel rows further down: the 128B swizzle is a function of the
            // shared-memory address, so a row-shifted start needs no re-layout.
            const int fh = p.cv_taps / p.cv_fw;
            int tap = 0;
            for (int fr = 0; fr < fh; ++fr) {
              for (int fs = 0; fs < p.cv_fw; ++fs, ++tap) {
                // one pixel row of the patch = 128 B = 8 descriptor units
                const uint32_t win16 = a16 + static_cast<uint32_t>(fr * p.cv_dh * p.cv_tw + fs * p.cv_dw) * 8u;
                const uint32_t wgt16 = b16 + static_cast<uint32_t>(tap) * (LOAD_N * kAtomBytes / 16);
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16) {
                  ptx::umma_f16<CTA_GROUP>(d_tmem, a_desc_hi | ((win16 + k16 * 2u) & 0x3fffu),
                                           b_desc_hi | ((wgt16 + k16 * 2u) & 0x3fffu), idesc, accumulate);
                  accumulate = 1;
                }
              }
            }
          } else {
#pragma unroll
            for (int k16 = 0; k16 < TILE_K / 16; ++k16) {
              // K step = (k16 / 4) slabs of 64 elements + (k16 % 4) steps of 16 inside a slab
              const uint32_t a_off = a16 + (k16 >> 2) * a_slab16 + (k16 & 3) * a_step16;
              const uint32_t b_off = b16 + (k16 >> 2) * b_slab16 + (k16 & 3) * b_step16;
              // (in a cluster launch the shared-window address carries the CTA rank above bit 18)
              ptx::umma_f16<CTA_GROUP>(d_tmem, a_desc_hi | (a_off & 0x3fffu),
                                       b_desc_hi | (b_off & 0x3fffu), idesc, accumulate);
              accumulate = 1;
            }
          }
          // Frees this ring slot (in both CTAs of a pair) once the MMAs above have read it.
          if (CTA_GROUP == 1)
            ptx::umma_commit(ptx::smem_u32(&ctrl->empty[stage]));
          else
            ptx::umma_commit_pair(ptx::smem_u32(&ctrl->empty[stage]), 0x3);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (CTA_GROUP == 1)
          ptx::umma_commit(ptx::smem_u32(&ctrl->tmem_full[acc]));
        else
          ptx::umma_commit_pair(ptx::smem_u32(&ctrl->tmem_full[acc]), 0x3);
        if (++acc == p.acc_stages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      TNX_TRACE(3);
      if (!ok && p.status != nullptr) atomicCAS(p.status, 0, kAbortMma);
    }
  } else {
    // ===== epilogue =====
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int quarter = warp & 3;                 // TMEM lanes this warp may touch
    const int row_in_tile = quarter * 32 + lane;  // row of the CTA's 128-row tile held by this thread
    const int epi_tid = threadIdx.x - 64;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t stage_row = static_cast<uint32_t>(row_in_tile) * kAtomBytes;
    const uint32_t sw = static_cast<uint32_t>(row_in_tile & 7);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t stores = 0;  // staging buffers used so far (selects the buffer)
    uint32_t xchg_round = 0;  // tiles this cluster has exchanged so far (barrier parity)
    bool ok = true;
    // (a double tile is written out as its left tile, then its right tile: accumulator buffers 0, 1)
    int half = 0;
    for (int u = cluster_id; u < total_units && ok;
         (p.wide && half == 0) ? (half = 1) : (half = 0, u += num_clusters)) {
      const int t = xchg ? u : u / p.split_k;
      const int slice = xchg ? static_cast<int>(cluster_rank) : u - t * p.split_k;
      int tm, tn;
      tile_coords(p, t, tm, tn);
      if (p.wide) tn = tn * 2 + half;
      const int bt_img = p.batched ? tm / p.bt_tiles_m : 0;  // which matrix of a batch
      // 128-row tile index (inside its matrix for a batch)
      const int row_tile = (tm - bt_img * p.bt_tiles_m) * CTA_GROUP + static_cast<int>(cta_rank);
      const int row0 = row_tile * kRowsPerCta;
      const int acc_col0 = tn * TILE_N;        // first B column of the tile
      const int out_col0 = tn * OUT_PER_TILE;  // first C column of the tile
      const int kb0 = slice * p.kb_per_slice;
      const bool has_k = kb0 < p.num_kb;

      const uint32_t tf_bar = ptx::smem_u32(&ctrl->tmem_full[acc]);
      bool got = !has_k || ptx::mbar_wait(tf_bar, acc_phase, abort_flag, p.timeout_ns);
      // All 128 epilogue threads continue or give up together (they share named barriers below).
      if (!ptx::named_barrier_all(kEpiBarrier, kEpiThreads, got)) {
        ok = false;
        break;
      }
      ptx::tc_fence_after_sync();
      if (epi_tid == 0 && u == cluster_id) TNX_TRACE(4);
#ifdef TNX_DEV_TRACE
      const int trace_tile = (u - cluster_id) / num_clusters;  // n-th tile of this CTA
      if (epi_tid == 0 && trace_tile < 40) TNX_TRACE(160 + trace_tile);
#endif
      const uint32_t t_acc = tmem_base + lane_sel + acc * TILE_N;

      if (xchg) {
        // ---- split-K inside a cluster: the S slices of this tile are the S CTAs of the cluster.
        // Each parks its fp32 partial in its own shared memory (the staging area), all of them
        // meet on an mbarrier, and each then sums ITS share of the tile from all S shared
        // memories (slice order, so the result is bit-reproducible) and stores it to C.
        constexpr uint32_t kChunkMask = TILE_N / 4 - 1;  // 16-byte chunks per row, XOR-swizzled by row
        const uint32_t S = cluster_size;
        const uint32_t full_bar = ptx::smem_u32(&ctrl->xchg_full);
        const uint32_t free_bar = ptx::smem_u32(&ctrl->xchg_free);
        if (xchg_round > 0) {  // peers must be done reading the previous partial
          const bool got_free = ptx::mbar_wait<true>(free_bar, (xchg_round - 1) & 1u, abort_flag, p.timeout_ns);
          if (!ptx::named_barrier_all(kEpiBarrier, kEpiThreads, got_free)) {
            ok = false;
            break;
          }
        }
        // Rows of the tile are dealt out to the slices in blocks of R: slice d sums (and stores)
        // rows [d*R, (d+1)*R).  Every slice PUSHES its partial rows into their owner's shared
        // memory (slot [source slice][row in block][TILE_N floats], 16-byte chunks XOR-swizzled
        // by row) with st.async, whose bytes complete the owner's mbarrier: no round trip, and
        // the owner then sums from its own shared memory.
        const int R = (p.a_rows + static_cast<int>(S) - 1) / static_cast<int>(S);
        const int my_rows = max(0, min(R, p.a_rows - static_cast<int>(cluster_rank) * R));
        if (epi_tid == 0)
          ptx::mbar_arrive_expect_tx(full_bar, static_cast<uint32_t>(my_rows) * S * (TILE_N * 4));
        if (quarter * 32 < p.a_rows) {  // warp-uniform: this warp's lanes hold loaded rows
          const uint32_t owner = static_cast<uint32_t>(row_in_tile / R);
          const uint32_t row_local = static_cast<uint32_t>(row_in_tile) - owner * R;
          const uint32_t dst_row = ptx::mapa(
              smem_out + (cluster_rank * static_cast<uint32_t>(R) + row_local) * (TILE_N * 4), owner);
          const uint32_t dst_bar = ptx::mapa(full_bar, owner);
          // (32 columns at a time, one read ahead of the push: whole warp, converged)
          uint32_t ra[2][32];
          ptx::tmem_ld_32x32(t_acc, ra[0]);
#pragma unroll
          for (int c = 0; c < TILE_N / 32; ++c) {
            uint32_t (&r)[32] = ra[c & 1];
            ptx::tmem_ld_wait(r);
            if (c + 1 < TILE_N / 32) ptx::tmem_ld_32x32(t_acc + (c + 1) * 32, ra[(c + 1) & 1]);
            if (row_in_tile < p.a_rows) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t chunk = (static_cast<uint32_t>(c * 8 + j) ^ row_local) & kChunkMask;
                ptx::st_async_v4(dst_row + chunk * 16, r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3],
                                 dst_bar);
              }
            }
            __syncwarp();
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctrl->tmem_empty[acc]));
        if (++acc == p.acc_stages) {
          acc = 0;
          acc_phase ^= 1u;
        }
        const bool got_full = ptx::mbar_wait<true>(full_bar, xchg_round & 1u, abort_flag, p.timeout_ns);
        if (!ptx::named_barrier_all(kEpiBarrier, kEpiThreads, got_full)) {
          ok = false;
          break;
        }
        if (epi_tid == 0 && u == cluster_id) TNX_TRACE(5);
        const int first_row = static_cast<int>(cluster_rank) * R;
        const int rows_valid = max(0, min(my_rows, p.m - row0 - first_row));
        const int cols_valid = min(TILE_N, p.n - acc_col0);
        const int vec_per_row = (cols_valid + 3) >> 2;
        const int total_vec = rows_valid * vec_per_row;
        constexpr int kInFlight = 4;
        for (int base = epi_tid; base < total_vec; base += kEpiThreads * kInFlight) {
          float4 sum[kInFlight];
          int rr[kInFlight], cc[kInFlight];
          uint32_t off[kInFlight];
#pragma unroll
          for (int u2 = 0; u2 < kInFlight; ++u2) {
            const int idx = base + u2 * kEpiThreads;
            const int safe = idx < total_vec ? idx : base;
            rr[u2] = safe / vec_per_row;
            const int c4 = safe - rr[u2] * vec_per_row;
            cc[u2] = c4 << 2;
            off[u2] = smem_out + static_cast<uint32_t>(rr[u2]) * (TILE_N * 4) +
                      (((static_cast<uint32_t>(c4) ^ static_cast<uint32_t>(rr[u2])) & kChunkMask) << 4);
            sum[u2] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
          for (uint32_t src = 0; src < S; ++src) {  // slice order: bit-reproducible
#pragma unroll
            for (int u2 = 0; u2 < kInFlight; ++u2) {
              const float4 v = ld_shared_v4(off[u2] + src * static_cast<uint32_t>(R) * (TILE_N * 4));
              sum[u2].x += v.x;
              sum[u2].y += v.y;
              sum[u2].z += v.z;
              sum[u2].w += v.w;
            }
          }
#pragma unroll
          for (int u2 = 0; u2 < kInFlight; ++u2) {
            if (base + u2 * kEpiThreads >= total_vec) continue;
            store_fixup<GLU, BF16>(p, row0 + first_row + rr[u2], acc_col0 + cc[u2], cols_valid - cc[u2], sum[u2]);
          }
        }
        // Tell every slice that this one has read what they pushed: they may push the next tile.
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
        if (epi_tid == 0)
          for (uint32_t r = 0; r < S; ++r) ptx::mbar_arrive_cluster(ptx::mapa(free_bar, r));
        ++xchg_round;
        continue;
      }

      if (p.split_k > 1) {
        // ---- split-K: park the fp32 partial; the last slice to arrive sums all of them ----
        // Partials are row-major [128 rows][TILE_N] per (tile, slice).
        const size_t tile_slot = static_cast<size_t>(row_tile * p.tiles_n + tn) * p.split_k;
        constexpr size_t kPartFloats = static_cast<size_t>(TILE_N) * kRowsPerCta;
        float* part = p.partials + (tile_slot + slice) * kPartFloats;
        const bool row_ok = row0 + row_in_tile < p.m;
        for (int c = 0; c < TILE_N / 32; ++c) {
          if (acc_col0 + c * 32 >= p.n) break;
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_acc + c * 32, r);
          ptx::tmem_ld_wait();
          if (row_ok) {
            float4* dst = reinterpret_cast<float4*>(part + row_in_tile * TILE_N + c * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              __stcg(dst + j, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
          }
        }
        // TMEM buffer can be refilled now.
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          const uint32_t te = ptx::smem_u32(&ctrl->tmem_empty[acc]);
          if (CTA_GROUP == 1 || leader)
            ptx::mbar_arrive(te);
          else
            ptx::mbar_arrive_cluster(ptx::mapa(te, 0));
        }
        if (++acc == p.acc_stages) {
          acc = 0;
          acc_phase ^= 1u;
        }
        __threadfence();
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
        if (epi_tid == 0) {
          int* counter = p.counters + (row_tile * p.tiles_n + tn);
          const int seen = atomicAdd(counter, 1);
          const int last = seen == p.split_k - 1;
          if (last) *counter = 0;  // leaves the counters clean for the next launch
          ctrl->is_last = last;
          __threadfence();
        }
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
        const bool is_last = ctrl->is_last != 0;
        if (epi_tid == 0 && u == cluster_id) TNX_TRACE(5);
        if (!is_last) continue;
        __threadfence();

        // Fix-up by the last arriver: all 128 threads walk the valid part of the tile in float4
        // steps, several steps in flight, and add the slices in slice order (bit-reproducible).
        // The result goes straight to C with 8-byte (plain) or 4-byte (GLU) stores.
        const float* part0 = p.partials + tile_slot * kPartFloats;
        const int rows_valid = min(kRowsPerCta, p.m - row0);
        const int cols_valid = min(TILE_N, p.n - acc_col0);
        const int vec_per_row = (cols_valid + 3) >> 2;
        const int total_vec = rows_valid * vec_per_row;
        constexpr int kInFlight = 4;
        for (int base = epi_tid; base < total_vec; base += kEpiThreads * kInFlight) {
          float4 sum[kInFlight];
          int rr[kInFlight], cc[kInFlight];
#pragma unroll
          for (int u2 = 0; u2 < kInFlight; ++u2) {
            const int idx = base + u2 * kEpiThreads;
            const int safe = idx < total_vec ? idx : base;
            rr[u2] = safe / vec_per_row;
            cc[u2] = (safe - rr[u2] * vec_per_row) << 2;
            sum[u2] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
          for (int s0 = 0; s0 < p.split_k; s0 += 4) {
            float4 v[4][kInFlight];
#pragma unroll
            for (int ds = 0; ds < 4; ++ds)
#pragma unroll
              for (int u2 = 0; u2 < kInFlight; ++u2)
                v[ds][u2] = s0 + ds < p.split_k
                                ? __ldcg(reinterpret_cast<const float4*>(
                                      part0 + (s0 + ds) * kPartFloats + rr[u2] * TILE_N + cc[u2]))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int ds = 0; ds < 4; ++ds)
#pragma unroll
              for (int u2 = 0; u2 < kInFlight; ++u2) {
                sum[u2].x += v[ds][u2].x;
                sum[u2].y += v[ds][u2].y;
                sum[u2].z += v[ds][u2].z;
                sum[u2].w += v[ds][u2].w;
              }
          }
#pragma unroll
          for (int u2 = 0; u2 < kInFlight; ++u2) {
            if (base + u2 * kEpiThreads >= total_vec) continue;
            store_fixup<GLU, BF16>(p, row0 + rr[u2], acc_col0 + cc[u2], cols_valid - cc[u2], sum[u2]);
          }
        }
        continue;
      }

      // ---- write the tile: chunks of 128 bytes of output per row, through swizzled staging ----
      // The accumulator is read 32 columns at a time, one read ahead: while a piece is converted
      // and staged (and while a chunk's store is handed to TMA and the next buffer is waited
      // for) the next piece is already on its way out of TMEM.
      constexpr int kSubs = ACC_PER_CHUNK / 32;  // even: the read-ahead buffers alternate cleanly
      constexpr int kChunks = TILE_N / ACC_PER_CHUNK;
      static_assert(kSubs % 2 == 0, "read-ahead needs an even number of pieces per chunk");
      uint32_t racc[2][32];
      if (out_col0 < p.n_out) ptx::tmem_ld_32x32(t_acc, racc[0]);
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        const int out_col = out_col0 + chunk * kAtomElems;
        if (out_col >= p.n_out) break;
        const bool more_chunks = chunk + 1 < kChunks && out_col + kAtomElems < p.n_out;
        const uint32_t buf = smem_out + (stores & 1u) * kStagingBytes;
        // The TMA store issued two chunks ago must have finished reading this buffer.
        if (epi_tid == 0) ptx::tma_store_wait_read<1>();
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
#pragma unroll
        for (int sub = 0; sub < kSubs; ++sub) {
          const int col = chunk * ACC_PER_CHUNK + sub * 32;
          float v[32];
          {
            uint32_t (&r)[32] = racc[sub & 1];
            ptx::tmem_ld_wait(r);
            // (whole warp, converged: the conditions depend on the tile only)
            if (sub + 1 < kSubs || more_chunks) ptx::tmem_ld_32x32(t_acc + col + 32, racc[(sub + 1) & 1]);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          }
          if (GLU) {
            // Columns come interleaved (gate_j, up_j): adjacent registers form one output.
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float z0 = gate_act(v[4 * j], p.epilogue) * v[4 * j + 1];
              const float z1 = gate_act(v[4 * j + 2], p.epilogue) * v[4 * j + 3];
              o[j] = pack2<BF16>(z0, z1);
            }
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
              const uint32_t pos = static_cast<uint32_t>(sub * 2 + piece) ^ sw;
              st_shared_v4(buf + stage_row + pos * 16, o[piece * 4], o[piece * 4 + 1],
                           o[piece * 4 + 2], o[piece * 4 + 3]);
            }
          } else {
            if (p.bias != nullptr) {
              const uint16_t* bias16 = reinterpret_cast<const uint16_t*>(p.bias);
              if (p.bias_per_row) {
                const int br = row0 + row_in_tile;
                const float bv = br < p.m ? unpack1<BF16>(__ldg(bias16 + br)) : 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += bv;
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const int bc = acc_col0 + col + j;
                  if (bc < p.n) v[j] += unpack1<BF16>(__ldg(bias16 + bc));
                }
              }
            }
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = pack2<BF16>(v[2 * j], v[2 * j + 1]);
#pragma unroll
            for (int piece = 0; piece < 4; ++piece) {
              const uint32_t pos = static_cast<uint32_t>(sub * 4 + piece) ^ sw;
              st_shared_v4(buf + stage_row + pos * 16, o[piece * 4], o[piece * 4 + 1],
                           o[piece * 4 + 2], o[piece * 4 + 3]);
            }
          }
        }
        ptx::fence_proxy_async_smem();
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
        if (epi_tid == 0) {
          if (p.batched) {
            ptx::tma_store_3d(&tmap_c, out_col, row0, bt_img, buf);
          } else if (p.conv != 1 && p.conv != 3) {
            ptx::tma_store_2d(&tmap_c, out_col, row0, buf);
          } else if (row_tile < p.cv_row_tiles) {  // rows are a rectangle of pixels of one image
            const int per_image = p.cv_tiles_h * p.cv_tiles_w;
            const int img = row_tile / per_image;
            const int rem = row_tile - img * per_image;
            const int hb = rem / p.cv_tiles_w;
            ptx::tma_store_4d(&tmap_c, out_col, (rem - hb * p.cv_tiles_w) * p.cv_tw, hb * p.cv_th,
                              img, buf);
          }
          ptx::tma_store_commit();
        }
        ++stores;
      }

      // All tcgen05.ld of this accumulator are complete: hand the TMEM buffer back.
#ifdef TNX_DEV_TRACE
      if (epi_tid == 0 && trace_tile < 40) TNX_TRACE(200 + trace_tile);
#endif
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        const uint32_t te = ptx::smem_u32(&ctrl->tmem_empty[acc]);
        if (CTA_GROUP == 1 || leader)
          ptx::mbar_arrive(te);
        else
          ptx::mbar_arrive_cluster(ptx::mapa(te, 0));
      }
      if (++acc == p.acc_stages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (epi_tid == 0) ptx::tma_store_wait_all<0>();
    if (epi_tid == 0) TNX_TRACE(6);
    if (!ok && lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, kAbortEpilogue);
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (ctrl->abort != 0) {
    // A wait gave up: let copies and MMAs that are still in flight drain before the shared
    // memory and TMEM they target are released (bounded: about a millisecond).
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  __syncwarp();
  if (CTA_GROUP == 2 || xchg) {  // peers may still signal barriers in, or read, this CTA's shared memory
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<CTA_GROUP>(tmem_base, tmem_alloc_cols);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e =
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 2-D row-major tensor of 16-bit elements: `cols` contiguous elements per row, `rows` rows,
// `pitch_elems` elements between rows; box = box_cols x box_rows with the 128-byte swizzle.
// Small cache of encoded tensor maps: serving loops call with the same buffers over and over,
// and the driver call that encodes a map costs more than the lookup.
struct TmapKey {
  const void* ptr;
  int64_t cols, rows, pitch;
  int32_t dtype, box_cols, box_rows, is_operand;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && cols == o.cols && rows == o.rows && pitch == o.pitch &&
           dtype == o.dtype && box_cols == o.box_cols && box_rows == o.box_rows &&
           is_operand == o.is_operand;
  }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kTmapSlots = 256;
std::mutex g_tmap_mu;
TmapSlot g_tmap_cache[kTmapSlots];

inline unsigned tmap_hash(const TmapKey& k) {
  uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(k.cols) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(k.rows) * 0x165667B19E3779F9ull;
  h ^= static_cast<uint64_t>(k.pitch) << 17 ^ static_cast<uint64_t>(k.box_rows) << 7 ^ static_cast<uint64_t>(k.box_cols);
  h ^= h >> 29;
  return static_cast<unsigned>(h) % kTmapSlots;
}

int make_tmap(CUtensorMap* out, const void* ptr, int dtype, int64_t cols, int64_t rows,
              int64_t pitch_elems, int box_cols, int box_rows, bool is_operand) {
  const TmapKey key{ptr, cols, rows, pitch_elems, dtype, box_cols, box_rows, is_operand ? 1 : 0};
  const unsigned slot = tmap_hash(key);
  {
    std::lock_guard<std::mutex> lock(g_tmap_mu);
    if (g_tmap_cache[slot].valid && g_tmap_cache[slot].key == key) {
      *out = g_tmap_cache[slot].map;
      return TNX_OK;
    }
  }
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return TNX_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  // (16-bit operands and outputs everywhere, except fp32 partial outputs of the MLP exchange)
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_elems) * (dtype == TNX_F32 ? 4 : 2)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == TNX_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == TNX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = encode(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      is_operand ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (ptr %p, %lld x %lld, pitch %lld)",
              static_cast<int>(r), ptr, static_cast<long long>(rows), static_cast<long long>(cols),
              static_cast<long long>(pitch_elems));
    return TNX_ERR_CUDA;
  }
  {
    std::lock_guard<std::mutex> lock(g_tmap_mu);
    g_tmap_cache[slot].key = key;
    g_tmap_cache[slot].map = *out;
    g_tmap_cache[slot].valid = true;
  }
  return TNX_OK;
}

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const UmmaParams);

template <int TILE_N, int CTA_GROUP, bool GLU>
KernelFn pick_dtype(int tile_k, int dtype) {
  if (tile_k == 64)
    return dtype == TNX_BF16 ? umma_gemm_kernel<TILE_N, 64, CTA_GROUP, GLU, true>
                             : umma_gemm_kernel<TILE_N, 64, CTA_GROUP, GLU, false>;
  if (tile_k == 128)
    return dtype == TNX_BF16 ? umma_gemm_kernel<TILE_N, 128, CTA_GROUP, GLU, true>
                             : umma_gemm_kernel<TILE_N, 128, CTA_GROUP, GLU, false>;
  return nullptr;
}

// The set of compiled kernels.  nullptr = not built.
KernelFn pick_kernel(int tile_n, int tile_k, int cta_group, bool glu, int dtype) {
  if (cta_group == 1) {
    if (!glu) {
      if (tile_n == 64) return pick_dtype<64, 1, false>(tile_k, dtype);
      if (tile_n == 128) return pick_dtype<128, 1, false>(tile_k, dtype);
      if (tile_n == 256) return pick_dtype<256, 1, false>(tile_k, dtype);
    } else {
      if (tile_n == 128) return pick_dtype<128, 1, true>(tile_k, dtype);
      if (tile_n == 256) return pick_dtype<256, 1, true>(tile_k, dtype);
    }
  } else if (cta_group == 2) {
    if (!glu) {
      if (tile_n == 128) return pick_dtype<128, 2, false>(tile_k, dtype);
      if (tile_n == 256) return pick_dtype<256, 2, false>(tile_k, dtype);
    } else {
      if (tile_n == 128) return pick_dtype<128, 2, true>(tile_k, dtype);
      if (tile_n == 256) return pick_dtype<256, 2, true>(tile_k, dtype);
    }
  }
  return nullptr;
}

// Opts a kernel into the full 227 KiB of dynamic shared memory, once per (kernel, device).
cudaError_t allow_full_smem(KernelFn fn) {
  static std::mutex mu;
  static std::vector<std::pair<KernelFn, int>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  for (const auto& d : done)
    if (d.first == fn && d.second == dev) return cudaSuccess;
  e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn),
                           cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
  if (e == cudaSuccess) done.emplace_back(fn, dev);
  return e;
}

constexpr int kWideHalf = 256;  // tile_n = 512 is two 256-column tiles per CTA pair

// Whether launches ask for programmatic stream serialization (the kernel's set-up overlaps the
// tail of the kernel before it).  On unless TRITONIX_B200_OVERLAP_SETUP=0.
bool overlap_setup() {
  static const bool on = [] {
    const char* v = getenv("TRITONIX_B200_OVERLAP_SETUP");
    return !(v != nullptr && v[0] == '0');
  }();
  return on;
}

// cudaOccupancyMaxActiveClusters, remembered per (kernel, device, shared memory, cluster size).
cudaError_t max_active_clusters(KernelFn fn, const cudaLaunchConfig_t& lc, int* out) {
  struct Entry {
    KernelFn fn;
    int dev;
    size_t smem;
    unsigned cluster;
    int fit;
  };
  static std::mutex mu;
  static std::vector<Entry> seen;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned cluster = lc.attrs[0].val.clusterDim.x;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry& en : seen)
      if (en.fn == fn && en.dev == dev && en.smem == lc.dynamicSmemBytes && en.cluster == cluster) {
        *out = en.fit;
        return cudaSuccess;
      }
  }
  int fit = 0;
  e = cudaOccupancyMaxActiveClusters(&fit, reinterpret_cast<const void*>(fn), &lc);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  seen.push_back({fn, dev, lc.dynamicSmemBytes, cluster, fit});
  *out = fit;
  return cudaSuccess;
}

int device_sm_count() {
  static int sms = -1;
  if (sms < 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
      sms = v;
    else
      return 148;  // B200; used only for sizing when no device is visible (resource queries)
  }
  return sms;
}

unsigned long long wait_limit_ns() {
  static unsigned long long v = 0;
  if (v == 0) {
    const char* e = getenv("TNX_WAIT_LIMIT_MS");
    long ms = e ? atol(e) : 0;
    if (ms <= 0) ms = 2000;
    v = static_cast<unsigned long long>(ms) * 1000000ull;
  }
  return v;
}

inline int cdiv(int a, int b) { return (a + b - 1) / b; }

// Rows of A fetched per stage: a single-CTA tile over a problem with fewer than 128 rows only
// needs (and only pays shared memory for) M rounded up to the 8-row swizzle group.
inline int a_box_rows(const tnx_problem& p, const tnx_config& cfg) {
  if (cfg.cta_group == 1 && p.m < kRowsPerCta && p.stride_ak == 1) return ((p.m + 7) / 8) * 8;
  return kRowsPerCta;
}

}  // namespace

int make_tmap_2d(CUtensorMap* out, const void* ptr, int dtype, int64_t cols, int64_t rows,
                 int64_t pitch_elems, int box_cols, int box_rows, bool is_operand) {
  return make_tmap(out, ptr, dtype, cols, rows, pitch_elems, box_cols, box_rows, is_operand);
}
int sm_count() { return device_sm_count(); }
unsigned long long bounded_wait_limit_ns() { return wait_limit_ns(); }

// Split-K slices can exchange partials through distributed shared memory when they fit one
// portable cluster (2, 4 or 8 CTAs, one SM each) and a slice's fp32 partial fits the epilogue
// staging area.  Then no workspace is needed at all.
// Rows of staging a CTA needs for the exchange: a block of ceil(rows / split) rows from each slice.
static int exchange_rows(int rows, int split) { return (rows + split - 1) / split * split; }
static bool use_cluster_split(const tnx_problem& p, const tnx_config& cfg, int split) {
  if (cfg.cta_group != 1 || (split != 2 && split != 4 && split != 8)) return false;
  if (getenv("TNX_NO_CLUSTER_SPLITK") != nullptr) return false;  // read every time: tests flip it
  const int rows = a_box_rows(p, cfg);
  const long long partial = static_cast<long long>(exchange_rows(rows, split)) * cfg.tile_n * 4;
  // Fits the regular staging area, or (skinny M only) a staging area grown to 64 KiB.
  return partial <= 2 * kStagingBytes || (rows <= 64 && partial <= 4 * kStagingBytes);
}

// Bytes of shared memory set aside for the epilogue.
static int staging_bytes_for(const tnx_problem& p, const tnx_config& cfg, int split) {
  if (split > 1 && use_cluster_split(p, cfg, split)) {
    const int partial = exchange_rows(a_box_rows(p, cfg), split) * cfg.tile_n * 4;
    if (partial > 2 * kStagingBytes) return (partial + 1023) / 1024 * 1024;
  }
  return 2 * kStagingBytes;
}

bool umma_eligible(const tnx_problem& p, const char** why) {
  const char* w = nullptr;
  if (p.dtype != TNX_F16 && p.dtype != TNX_BF16)
    w = "tcgen05 path takes fp16 or bf16 operands";
  else if (p.stride_cn != 1 || (p.stride_ak != 1 && p.stride_am != 1) ||
           (p.stride_bn != 1 && p.stride_bk != 1))
    w = "tcgen05 path needs a unit stride in A, in B (either dimension) and along the rows of C";
  else if (((p.stride_ak == 1 ? p.stride_am : p.stride_ak) % 8) != 0 || (p.stride_cm % 8) != 0 ||
           ((p.stride_bn == 1 ? p.stride_bk : p.stride_bn) % 8) != 0)
    w = "tcgen05 path needs row pitches that are multiples of 16 bytes";
  else if (p.stride_ak != 1 && (p.m % 8) != 0)
    w = "tcgen05 path needs M to be a multiple of 8 when A is stored K x M";
  else if (p.k < 1 || p.m < 1 || p.n < 1)
    w = "empty problem";
  else if ((p.k % 8) != 0 || (p.n % 8) != 0 || (p.epilogue != TNX_EPI_NONE && (p.n % 16) != 0))
    // TMA clips and zero-fills in 16-byte units along the contiguous dimension
    w = "tcgen05 path needs K, N (and N/2 for a GLU epilogue) to be multiples of 8 elements";
  else if ((p.stride_ak == 1 ? p.stride_am < p.k : p.stride_ak < p.m) ||
           (p.stride_bn == 1 ? p.stride_bk < p.n : p.stride_bn < p.k))
    w = "row pitch smaller than the row length";
  if (why) *why = w;
  return w == nullptr;
}

int umma_query(const tnx_problem& p, tnx_config* cfg, tnx_resources* out) {
  const bool glu = p.epilogue != TNX_EPI_NONE;
  if (cfg->cta_group == 0) cfg->cta_group = cfg->tile_m == 2 * kRowsPerCta ? 2 : 1;  // 256 rows = a CTA pair
  if (cfg->tile_m == 0) cfg->tile_m = kRowsPerCta * cfg->cta_group;
  if (cfg->tile_n == 0) cfg->tile_n = (p.n >= 256) ? 256 : (p.n > 64 || glu ? 128 : 64);
  if (cfg->tile_k == 0) cfg->tile_k = 64;
  if (cfg->acc_stages == 0) cfg->acc_stages = 2;
  if (cfg->split_k == 0) cfg->split_k = 1;
  if (cfg->group_m == 0) cfg->group_m = 8;

  if (cfg->cta_group != 1 && cfg->cta_group != 2) {
    set_error("cta_group must be 1 or 2, got %d", cfg->cta_group);
    return TNX_ERR_INVALID;
  }
  if (cfg->tile_m != kRowsPerCta * cfg->cta_group) {
    set_error("tile_m=%d is not built: cta_group=%d tiles have %d rows", cfg->tile_m,
              cfg->cta_group, kRowsPerCta * cfg->cta_group);
    return TNX_ERR_NOT_BUILT;
  }
  if (cfg->tile_k != 64 && cfg->tile_k != 128) {
    set_error("tile_k=%d is not built (64 or 128)", cfg->tile_k);
    return TNX_ERR_NOT_BUILT;
  }
  if (cfg->acc_stages < 1 || cfg->acc_stages > 2 || cfg->split_k < 1 || cfg->group_m < 1 ||
      cfg->tile_order < 0 || cfg->tile_order > TNX_ORDER_TABLE) {
    set_error("invalid acc_stages/split_k/group_m/tile_order (%d/%d/%d/%d)", cfg->acc_stages,
              cfg->split_k, cfg->group_m, cfg->tile_order);
    return TNX_ERR_INVALID;
  }
  // tile_n = 512: a CTA pair works on two column-adjacent 256-column tiles at once (both TMEM
  // buffers are live accumulators, one A stage feeds both).
  const bool wide = cfg->tile_n == 2 * kWideHalf;
  if (wide && (cfg->cta_group != 2 || cfg->split_k != 1 || cfg->acc_stages != 2 ||
               cfg->tile_order == TNX_ORDER_TABLE || p.stride_bn != 1)) {
    set_error("tile_n=512 needs cta_group=2, split_k=1, acc_stages=2, a computed tile order and a row-major B");
    return TNX_ERR_NOT_BUILT;
  }
  const int kernel_tile_n = wide ? kWideHalf : cfg->tile_n;
  if (pick_kernel(kernel_tile_n, cfg->tile_k, cfg->cta_group, glu, p.dtype) == nullptr) {
    set_error("no kernel built for tile_n=%d cta_group=%d%s", cfg->tile_n, cfg->cta_group,
              glu ? " with a GLU epilogue" : "");
    return TNX_ERR_NOT_BUILT;
  }
  if (glu && (p.n % 2) != 0) {
    set_error("GLU epilogue needs an even number of interleaved columns, got n=%d", p.n);
    return TNX_ERR_INVALID;
  }

  const int tile_rows = kRowsPerCta * cfg->cta_group;
  const int tiles_m = cdiv(p.m, tile_rows);
  const int tiles_n = cdiv(p.n, cfg->tile_n);
  const int num_kb = cdiv(p.k, cfg->tile_k);
  int split = cfg->split_k > num_kb ? num_kb : cfg->split_k;
  const int kb_per = cdiv(num_kb, split);
  split = cdiv(num_kb, kb_per);  // no empty slice

  const int load_n = cfg->tile_n / cfg->cta_group;  // (a double tile: the B columns of both tiles)
  const int stage_bytes = (a_box_rows(p, *cfg) + load_n) * cfg->tile_k * 2;
  const int fixed = staging_bytes_for(p, *cfg, split) + kCtrlBytes + kAlignSlack;
  if (cfg->stages == 0) {
    int s = (kMaxDynamicSmem - fixed) / stage_bytes;
    cfg->stages = s > 8 ? 8 : s;
  }
  if (cfg->stages < 2 || cfg->stages > kMaxStages) {
    set_error("stages must be in [2, %d], got %d", kMaxStages, cfg->stages);
    return TNX_ERR_INVALID;
  }
  const long long smem = static_cast<long long>(cfg->stages) * stage_bytes + fixed;
  int tmem = 32;
  while (tmem < cfg->acc_stages * kernel_tile_n) tmem <<= 1;

  out->kernel = TNX_KERNEL_TCGEN05;
  out->smem_bytes = static_cast<int32_t>(smem > 0x7fffffff ? 0x7fffffff : smem);
  out->tmem_columns = tmem;
  out->tiles_m = tiles_m;
  out->tiles_n = tiles_n;
  out->split_k = split;
  const bool xchg = split > 1 && use_cluster_split(p, *cfg, split);
  out->workspace_bytes =
      split > 1 && !xchg ? kCounterBytes + static_cast<int64_t>(tiles_m) * cfg->cta_group * tiles_n *
                                               split * cfg->tile_n * kRowsPerCta * 4
                         : 0;
  // Persistent grid: one cluster per SM group; a cluster is a CTA pair, the slices of a tile, or 1 CTA.
  const int cluster_size = xchg ? split : cfg->cta_group;
  const long long units = static_cast<long long>(tiles_m) * tiles_n * (xchg ? 1 : split);
  int max_clusters = device_sm_count() / cluster_size;
  if (cfg->max_ctas > 0 && cfg->max_ctas / cluster_size < max_clusters)
    max_clusters = cfg->max_ctas / cluster_size;
  if (max_clusters < 1) max_clusters = 1;
  out->grid = static_cast<int32_t>((units < max_clusters ? units : max_clusters) * cluster_size);

  if (smem > kMaxDynamicSmem) {
    set_error("shared memory budget exceeded: %lld B needed (%d stages x %d B + %d B), %d B per SM",
              smem, cfg->stages, stage_bytes, fixed, kMaxDynamicSmem);
    return TNX_ERR_RESOURCES;
  }
  if (tmem > kTmemColumns) {
    set_error("TMEM budget exceeded: %d accumulator buffers x %d columns > %d", cfg->acc_stages,
              cfg->tile_n, kTmemColumns);
    return TNX_ERR_RESOURCES;
  }
  if (tiles_m > 0xffff || tiles_n > 0xffff) {
    set_error("problem has too many tiles (%d x %d)", tiles_m, tiles_n);
    return TNX_ERR_INVALID;
  }
  if (split > 1 && static_cast<long long>(tiles_m) * cfg->cta_group * tiles_n > kMaxCounterTiles) {
    set_error("split-K supports at most %d output tiles, problem has %lld", kMaxCounterTiles,
              static_cast<long long>(tiles_m) * cfg->cta_group * tiles_n);
    return TNX_ERR_INVALID;
  }
  return TNX_OK;
}

int umma_launch(const tnx_problem& p, const tnx_config& cfg, const tnx_resources& res,
                const void* a, const void* b, void* c, void* workspace, const int32_t* tile_table,
                int32_t* status_word, cudaStream_t stream) {
  const bool glu = p.epilogue != TNX_EPI_NONE;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
       reinterpret_cast<uintptr_t>(c)) & 15u) {
    set_error("tcgen05 path needs 16-byte aligned A, B and C base addresses");
    return TNX_ERR_INVALID;
  }
  const bool wide = cfg.tile_n == 2 * kWideHalf;
  KernelFn fn = pick_kernel(wide ? kWideHalf : cfg.tile_n, cfg.tile_k, cfg.cta_group, glu, p.dtype);
  if (fn == nullptr) return TNX_ERR_NOT_BUILT;

  const int n_out = glu ? p.n / 2 : p.n;
  CUtensorMap ta, tb, tc;
  const int a_rows = a_box_rows(p, cfg);
  const bool a_mmajor = p.stride_ak != 1;
  int rc = a_mmajor ? make_tmap(&ta, a, p.dtype, p.m, p.k, p.stride_ak, kAtomElems, cfg.tile_k, true)
                    : make_tmap(&ta, a, p.dtype, p.k, p.m, p.stride_am, kAtomElems, a_rows, true);
  if (rc != TNX_OK) return rc;
  // B row-major (K x N): boxes of 64 columns x tile_k rows.  B stored N x K (a transposed view):
  // boxes of 64 K elements x the CTA's B columns, like A.
  const bool b_kmajor = p.stride_bn != 1;
  if (b_kmajor)
    rc = make_tmap(&tb, b, p.dtype, p.k, p.n, p.stride_bn, kAtomElems, cfg.tile_n / cfg.cta_group, true);
  else
    rc = make_tmap(&tb, b, p.dtype, p.n, p.k, p.stride_bk, kAtomElems, cfg.tile_k, true);
  if (rc != TNX_OK) return rc;
  rc = make_tmap(&tc, c, p.dtype, n_out, p.m, p.stride_cm, kAtomElems, kRowsPerCta, false);
  if (rc != TNX_OK) return rc;

  UmmaParams kp = {};
  kp.m = p.m;
  kp.n = p.n;
  kp.k = p.k;
  kp.n_out = n_out;
  kp.tiles_m = res.tiles_m;
  kp.tiles_n = res.tiles_n;
  kp.num_kb = cdiv(p.k, cfg.tile_k);
  kp.split_k = res.split_k;
  const bool xchg = res.split_k > 1 && res.workspace_bytes == 0;
  kp.cluster_split = xchg ? res.split_k : 0;
  kp.kb_per_slice = cdiv(kp.num_kb, res.split_k);
  kp.tile_k = cfg.tile_k;
  kp.a_rows = a_rows;
  kp.staging_bytes = staging_bytes_for(p, cfg, res.split_k);
  kp.b_kmajor = b_kmajor ? 1 : 0;
  kp.a_mmajor = a_mmajor ? 1 : 0;
  kp.stages = cfg.stages;
  kp.acc_stages = cfg.acc_stages;
  kp.wide = wide ? 1 : 0;
  kp.group_m = cfg.group_m;
  kp.tile_order = cfg.tile_order;
  kp.epilogue = p.epilogue;
  kp.tile_table = tile_table;
  kp.c_ptr = c;
  kp.ldc = p.stride_cm;
  kp.counters = reinterpret_cast<int*>(workspace);
  kp.partials = workspace ? reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes)
                          : nullptr;
  kp.status = status_word;
  kp.timeout_ns = wait_limit_ns();
#ifdef TNX_DEV_TRACE
  {
    const char* t = getenv("TNX_TRACE_PTR");
    kp.trace = t ? reinterpret_cast<unsigned long long*>(strtoull(t, nullptr, 0)) : nullptr;
  }
#endif

  cudaError_t e = allow_full_smem(fn);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%d B dynamic smem): %s", kMaxDynamicSmem, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }

  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(res.grid, 1, 1);
  lc.blockDim = dim3(kThreads, 1, 1);
  lc.dynamicSmemBytes = res.smem_bytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = xchg ? res.split_k : cfg.cta_group;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // The kernel's set-up (barriers, TMEM, cluster rendezvous) may overlap the tail of the kernel
  // before it in the stream; it waits for that kernel to complete before touching global memory.
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = overlap_setup() ? 2 : 1;
  if (xchg) {
    // Clusters of split_k CTAs do not always tile the GPU evenly: ask how many fit at once.
    int fit = 0;
    e = max_active_clusters(fn, lc, &fit);
    if (e != cudaSuccess || fit < 1) {
      set_error("clusters of %d CTAs cannot be scheduled for the split-K exchange: %s", res.split_k,
                e != cudaSuccess ? cudaGetErrorString(e) : "none fit");
      (void)cudaGetLastError();
      return TNX_ERR_CUDA;
    }
    const int want = res.grid / res.split_k;
    lc.gridDim.x = static_cast<unsigned>((want < fit ? want : fit) * res.split_k);
  }
  e = cudaLaunchKernelEx(&lc, fn, ta, tb, tc, kp);
  if (e != cudaSuccess) {
    set_error("kernel launch failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}


// ---------------------------------------------------------------------------------------------
// Convolution forward on the same kernel
// ---------------------------------------------------------------------------------------------
namespace {

inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

// 4-D tensor map over an N x H x W x C tensor of 16-bit elements (dimension order C, W, H, N).
// A box is 64 channels x box_w x box_h pixels of one image, walked with the given pixel steps.
int make_tmap_nhwc(CUtensorMap* out, const void* ptr, int dtype, int64_t c, int64_t w, int64_t h,
                   int64_t n, int box_w, int box_h, int step_w, int step_h, bool is_operand) {
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return TNX_ERR_CUDA;
  }
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(c), static_cast<cuuint64_t>(w),
                              static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(n)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(c) * 2, static_cast<cuuint64_t>(w * c) * 2,
                                 static_cast<cuuint64_t>(h * w * c) * 2};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(kAtomElems), static_cast<cuuint32_t>(box_w),
                             static_cast<cuuint32_t>(box_h), 1};
  const cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(step_w), static_cast<cuuint32_t>(step_h), 1};
  const CUtensorMapDataType dt =
      dtype == TNX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = encode(out, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      is_operand ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (4-D) failed with CUresult %d (ptr %p, %lld x %lld x %lld x %lld, "
              "box %d x %d, steps %d x %d)",
              static_cast<int>(r), ptr, static_cast<long long>(n), static_cast<long long>(h),
              static_cast<long long>(w), static_cast<long long>(c), box_w, box_h, step_w, step_h);
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                    cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

EncodeIm2colFn get_encode_im2col_fn() {
  static EncodeIm2colFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e =
        cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &sym, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeIm2colFn>(sym);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// im2col-mode tensor map over an N x H x W x C tensor: a box is 128 consecutive filter-window
// origins (walking W, then H, then N in steps of the convolution's stride inside the window
// origins' bounding box) x 64 channels; the load adds the filter tap's offset.
int make_tmap_im2col(CUtensorMap* out, const void* ptr, const tnx_conv2d_problem& p, int c_pitch) {
  EncodeIm2colFn encode = get_encode_im2col_fn();
  if (encode == nullptr) {
    set_error("cuTensorMapEncodeIm2col is not available from the CUDA driver");
    return TNX_ERR_CUDA;
  }
  const cuuint64_t c = c_pitch, w = p.w_in, h = p.h_in, n = p.batch;
  const cuuint64_t dims[4] = {c, w, h, n};
  const cuuint64_t strides[3] = {c * 2, w * c * 2, h * w * c * 2};
  const int lower[2] = {-p.pad_w, -p.pad_h};
  const int upper[2] = {p.pad_w - (p.filter_w - 1) * p.dil_w, p.pad_h - (p.filter_h - 1) * p.dil_h};
  const cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(p.stride_w),
                              static_cast<cuuint32_t>(p.stride_h), 1};
  const CUtensorMapDataType dt =
      p.dtype == TNX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = encode(out, dt, 4, const_cast<void*>(ptr), dims, strides, lower, upper, kAtomElems,
                      kRowsPerCta, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeIm2col failed with CUresult %d (ptr %p, %d x %d x %d x %d, corners "
              "(%d, %d) (%d, %d))",
              static_cast<int>(r), ptr, p.batch, p.h_in, p.w_in, c_pitch, lower[0], lower[1], upper[0],
              upper[1]);
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

// im2col-mode boxes keep the window origins' bounding-box corners in 8 bits each.
bool im2col_usable(const tnx_conv2d_problem& p) {
  if (getenv("TNX_CONV_TILED") != nullptr) return false;  // read every time: tests flip it
  const int up_w = p.pad_w - (p.filter_w - 1) * p.dil_w, up_h = p.pad_h - (p.filter_h - 1) * p.dil_h;
  return p.pad_w <= 128 && p.pad_h <= 128 && up_w >= -128 && up_w <= 127 && up_h >= -128 &&
         up_h <= 127 && (p.filter_w - 1) * p.dil_w < 65536 && (p.filter_h - 1) * p.dil_h < 65536;
}

// Picks the rectangle of output pixels one CTA tile covers: at most 128 pixels, a multiple of 8
// (whole swizzle groups), fewest tiles per image first, then most pixels per tile, then widest.
void pick_pixel_tile(int h_out, int w_out, int step_h, int step_w, int* tile_w, int* tile_h) {
  long long best_tiles = -1;
  int best_w = 8, best_h = 1, best_px = 0;
  for (int tw = 1; tw <= kRowsPerCta; ++tw) {
    if ((tw - 1) * step_w + 1 > 256) break;
    if (tw > w_out && tw > 8) break;
    for (int th = 1; tw * th <= kRowsPerCta; ++th) {
      if ((th - 1) * step_h + 1 > 256) break;
      const int px = tw * th;
      if (px % 8 != 0) continue;
      const long long tiles = static_cast<long long>(cdiv(w_out, tw)) * cdiv(h_out, th);
      const bool better = best_tiles < 0 || tiles < best_tiles ||
                          (tiles == best_tiles && (px < best_px || (px == best_px && tw > best_w)));
      if (better) {
        best_tiles = tiles;
        best_w = tw;
        best_h = th;
        best_px = px;
      }
    }
  }
  *tile_w = best_w;
  *tile_h = best_h;
}

}  // namespace

int umma_conv_query(const tnx_conv2d_problem& p, tnx_config* cfg, tnx_conv2d_resources* out,
                    ConvPlan* plan) {
  const int h_out = (p.h_in + 2 * p.pad_h - p.dil_h * (p.filter_h - 1) - 1) / p.stride_h + 1;
  const int w_out = (p.w_in + 2 * p.pad_w - p.dil_w * (p.filter_w - 1) - 1) / p.stride_w + 1;
  plan->h_out = h_out;
  plan->w_out = w_out;
  if (p.stride_h > 8 || p.stride_w > 8) {  // a tensor map walks a box in steps of at most 8
    set_error("convolution strides above 8 are not supported for fp16/bf16 (got %d x %d)",
              p.stride_h, p.stride_w);
    return TNX_ERR_INVALID;
  }
  // Shallow layers (at most 64 input and 64 output channels) are bound by re-reading the input
  // once per filter tap and the weights once per tile; for them (stride 1, rows of at most 128
  // pixels with the halo) the weights of all taps stay in shared memory, a stage is one tile's
  // input patch, and every tap multiplies a shifted window of the patch.
  const int taps = p.filter_h * p.filter_w;
  const int halo_w = w_out + (p.filter_w - 1) * p.dil_w;
  const int halo_th = halo_w <= kRowsPerCta ? std::min(kRowsPerCta / halo_w, h_out) : 0;
  const int halo_ph = halo_th + (p.filter_h - 1) * p.dil_h;
  const long long halo_rows = (static_cast<long long>(halo_w) * halo_ph + 7) / 8 * 8;
  const long long halo_weights = static_cast<long long>(taps) * 64 * kAtomBytes;
  const long long halo_stage = halo_rows * kAtomBytes;
  plan->halo = getenv("TNX_CONV_NO_HALO") == nullptr && p.stride_h == 1 && p.stride_w == 1 &&
               taps > 1 && p.c_in <= kAtomElems && p.c_out <= 64 && p.input_layout >= 0 &&
               halo_w <= kRowsPerCta && halo_ph <= 256 &&
               (cfg->cta_group == 0 || cfg->cta_group == 1) &&
               (cfg->tile_m == 0 || cfg->tile_m == kRowsPerCta) &&
               (cfg->tile_n == 64 || (cfg->tile_n == 0 && p.c_out <= 64)) &&
               (cfg->tile_k == 0 || cfg->tile_k == kAtomElems) &&
               2 * halo_stage + halo_weights + 2 * kStagingBytes + kCtrlBytes + kAlignSlack <=
                   kMaxDynamicSmem;
  plan->patch_h = plan->halo ? halo_ph : 0;
  plan->patch_rows = plan->halo ? static_cast<int>(halo_rows) : 0;
  plan->im2col = !plan->halo && im2col_usable(p);
  long long row_tiles;
  if (plan->halo) {
    plan->tile_w = halo_w;
    plan->tile_h = halo_th;
    plan->tiles_w = 1;
    plan->tiles_h = cdiv(h_out, halo_th);
    row_tiles = static_cast<long long>(p.batch) * plan->tiles_h;
    cfg->cta_group = 1;
    cfg->tile_n = 64;
    cfg->tile_k = kAtomElems;
  } else if (plan->im2col) {  // a tile = 128 consecutive pixels in (image, row, column) order
    plan->tile_w = kRowsPerCta;
    plan->tile_h = 1;
    plan->tiles_w = plan->tiles_h = 0;
    row_tiles = (static_cast<long long>(p.batch) * h_out * w_out + kRowsPerCta - 1) / kRowsPerCta;
  } else {
    pick_pixel_tile(h_out, w_out, p.stride_h, p.stride_w, &plan->tile_w, &plan->tile_h);
    plan->tiles_w = cdiv(w_out, plan->tile_w);
    plan->tiles_h = cdiv(h_out, plan->tile_h);
    row_tiles = static_cast<long long>(p.batch) * plan->tiles_w * plan->tiles_h;
  }
  if (row_tiles > 0x7fffffLL) {
    set_error("convolution output has too many pixel tiles (%lld)", row_tiles);
    return TNX_ERR_INVALID;
  }
  plan->row_tiles = static_cast<int>(row_tiles);
  const int a_rows = plan->halo ? plan->patch_rows : plan->tile_w * plan->tile_h;

  // Workspace: the kernel reads N x H x W x C with C a multiple of 8 and writes the same way.
  plan->repack_input = !(p.input_layout == TNX_LAYOUT_NHWC && p.c_in % 8 == 0);
  plan->repack_output = !(p.output_layout == TNX_LAYOUT_NHWC && p.c_out % 8 == 0);
  plan->c_pitch = (p.c_in + 7) / 8 * 8;
  plan->c_out_pitch = (p.c_out + 7) / 8 * 8;
  plan->cblocks = cdiv(p.c_in, kAtomElems);
  plan->k_packed = p.filter_h * p.filter_w * plan->cblocks * kAtomElems;
  int64_t off = 0;
  plan->off_input = off;
  if (plan->repack_input)
    off += align256(static_cast<int64_t>(p.batch) * p.h_in * p.w_in * plan->c_pitch * 2);
  plan->off_weight = off;
  off += align256(static_cast<int64_t>(p.c_out) * plan->k_packed * 2);
  plan->off_output = off;
  if (plan->repack_output)
    off += align256(static_cast<int64_t>(p.batch) * h_out * w_out * plan->c_out_pitch * 2);
  plan->workspace_bytes = off;

  if (cfg->cta_group == 0) {
    if (cfg->tile_m != 0)
      cfg->cta_group = cfg->tile_m == 2 * kRowsPerCta ? 2 : 1;  // 256 rows = a CTA pair
    else
      cfg->cta_group = (row_tiles >= 2 && p.c_out > 64) ? 2 : 1;
  }
  if (cfg->tile_m != 0 && cfg->tile_m != kRowsPerCta * cfg->cta_group) {
    set_error("tile_m=%d is not built: cta_group=%d tiles have %d rows", cfg->tile_m,
              cfg->cta_group, kRowsPerCta * cfg->cta_group);
    return TNX_ERR_NOT_BUILT;
  }
  if (cfg->cta_group != 1 && cfg->cta_group != 2) {
    set_error("cta_group must be 1 or 2, got %d", cfg->cta_group);
    return TNX_ERR_INVALID;
  }
  if (cfg->tile_n == 0) cfg->tile_n = p.c_out > 128 ? 256 : (p.c_out > 64 || cfg->cta_group == 2 ? 128 : 64);
  if (cfg->tile_k == 0) cfg->tile_k = (plan->k_packed % 128 == 0) ? 128 : 64;
  if (cfg->group_m == 0) cfg->group_m = 8;
  cfg->acc_stages = 2;
  cfg->split_k = 1;
  cfg->tile_m = kRowsPerCta * cfg->cta_group;
  if (cfg->tile_k != 64 && cfg->tile_k != 128) {
    set_error("tile_k=%d is not built (64 or 128)", cfg->tile_k);
    return TNX_ERR_NOT_BUILT;
  }
  if (pick_kernel(cfg->tile_n, cfg->tile_k, cfg->cta_group, false, p.dtype) == nullptr) {
    set_error("no kernel built for tile_n=%d cta_group=%d", cfg->tile_n, cfg->cta_group);
    return TNX_ERR_NOT_BUILT;
  }
  const int load_n = cfg->tile_n / cfg->cta_group;
  // (halo: the ring holds patches only; the weights of all taps are one more, fixed, buffer)
  const int stage_bytes = plan->halo ? a_rows * kAtomBytes : (a_rows + load_n) * cfg->tile_k * 2;
  const int fixed = 2 * kStagingBytes + kCtrlBytes + kAlignSlack +
                    (plan->halo ? taps * load_n * kAtomBytes : 0);
  if (cfg->stages == 0) {
    int s = (kMaxDynamicSmem - fixed) / stage_bytes;
    cfg->stages = s > 8 ? 8 : s;
  }
  if (cfg->stages < 2 || cfg->stages > kMaxStages) {
    set_error("stages must be in [2, %d], got %d", kMaxStages, cfg->stages);
    return TNX_ERR_INVALID;
  }
  const long long smem = static_cast<long long>(cfg->stages) * stage_bytes + fixed;
  const int tiles_m = cdiv(plan->row_tiles, cfg->cta_group);
  const int tiles_n = cdiv(p.c_out, cfg->tile_n);
  int max_clusters = device_sm_count() / cfg->cta_group;
  if (cfg->max_ctas > 0 && cfg->max_ctas / cfg->cta_group < max_clusters)
    max_clusters = cfg->max_ctas / cfg->cta_group;
  if (max_clusters < 1) max_clusters = 1;
  const long long units = static_cast<long long>(tiles_m) * tiles_n;
  out->kernel = TNX_KERNEL_TCGEN05;
  out->h_out = h_out;
  out->w_out = w_out;
  out->tile_w = plan->tile_w;
  out->tile_h = plan->tile_h;
  out->smem_bytes = static_cast<int32_t>(smem > 0x7fffffff ? 0x7fffffff : smem);
  out->tmem_columns = 2 * cfg->tile_n < 32 ? 32 : 2 * cfg->tile_n;
  out->grid = static_cast<int32_t>((units < max_clusters ? units : max_clusters) * cfg->cta_group);
  out->workspace_bytes = plan->workspace_bytes;
  if (smem > kMaxDynamicSmem) {
    set_error("shared memory budget exceeded: %lld B needed (%d stages x %d B + %d B), %d B per SM",
              smem, cfg->stages, stage_bytes, fixed, kMaxDynamicSmem);
    return TNX_ERR_RESOURCES;
  }
  if (tiles_n > 0xffff) {
    set_error("too many output-channel tiles (%d)", tiles_n);
    return TNX_ERR_INVALID;
  }
  return TNX_OK;
}

int umma_conv_launch(const tnx_conv2d_problem& p, const tnx_config& cfg,
                     const tnx_conv2d_resources& res, const ConvPlan& plan, const void* x,
                     const void* w, const void* bias, void* y, int32_t* status_word,
                     cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
       reinterpret_cast<uintptr_t>(y)) & 15u) {
    set_error("tcgen05 convolution needs 16-byte aligned input, weight and output buffers");
    return TNX_ERR_INVALID;
  }
  KernelFn fn = pick_kernel(cfg.tile_n, cfg.tile_k, cfg.cta_group, false, p.dtype);
  if (fn == nullptr) return TNX_ERR_NOT_BUILT;
  const int a_rows = plan.halo ? plan.patch_rows : plan.tile_w * plan.tile_h;
  CUtensorMap ta, tb, tc;
  int rc = plan.halo
               ? make_tmap_nhwc(&ta, x, p.dtype, plan.c_pitch, p.w_in, p.h_in, p.batch, plan.tile_w,
                                plan.patch_h, 1, 1, true)
           : plan.im2col
               ? make_tmap_im2col(&ta, x, p, plan.c_pitch)
               : make_tmap_nhwc(&ta, x, p.dtype, plan.c_pitch, p.w_in, p.h_in, p.batch,
                                (plan.tile_w - 1) * p.stride_w + 1,
                                (plan.tile_h - 1) * p.stride_h + 1, p.stride_w, p.stride_h, true);
  if (rc != TNX_OK) return rc;
  rc = make_tmap(&tb, w, p.dtype, plan.k_packed, p.c_out, plan.k_packed, kAtomElems,
                 cfg.tile_n / cfg.cta_group, true);
  if (rc != TNX_OK) return rc;
  const long long pixels = static_cast<long long>(p.batch) * plan.h_out * plan.w_out;
  rc = plan.im2col ? make_tmap(&tc, y, p.dtype, plan.c_out_pitch, pixels, plan.c_out_pitch,
                               kAtomElems, kRowsPerCta, false)
                   : make_tmap_nhwc(&tc, y, p.dtype, plan.c_out_pitch, plan.w_out, plan.h_out,
                                    p.batch, plan.tile_w, plan.tile_h, 1, 1, false);
  if (rc != TNX_OK) return rc;

  UmmaParams kp = {};
  kp.m = plan.im2col ? static_cast<int>(pixels) : plan.row_tiles * kRowsPerCta;
  kp.n = p.c_out;
  kp.k = plan.k_packed;
  kp.n_out = plan.c_out_pitch;
  kp.tiles_m = cdiv(plan.row_tiles, cfg.cta_group);
  kp.tiles_n = cdiv(p.c_out, cfg.tile_n);
  kp.num_kb = cdiv(plan.k_packed, cfg.tile_k);
  kp.split_k = 1;
  kp.cluster_split = 0;
  kp.kb_per_slice = kp.num_kb;
  kp.tile_k = cfg.tile_k;
  kp.a_rows = a_rows;
  kp.staging_bytes = 2 * kStagingBytes;
  kp.b_kmajor = 1;
  kp.a_mmajor = 0;
  kp.stages = cfg.stages;
  kp.acc_stages = 2;
  kp.group_m = cfg.group_m;
  kp.tile_order = TNX_ORDER_GROUPED;
  kp.epilogue = TNX_EPI_NONE;
  kp.status = status_word;
  kp.timeout_ns = wait_limit_ns();
  kp.conv = plan.halo ? 3 : (plan.im2col ? 2 : 1);
  if (plan.halo) {  // K blocks are channel blocks; the taps are walked inside a stage
    kp.num_kb = plan.cblocks;
    kp.kb_per_slice = plan.cblocks;
    kp.a_box_bytes = plan.tile_w * plan.patch_h * kAtomBytes;
  }
  kp.cv_wout = plan.w_out;
  kp.cv_hout = plan.h_out;
  kp.cv_tw = plan.tile_w;
  kp.cv_th = plan.tile_h;
  kp.cv_tiles_w = plan.tiles_w;
  kp.cv_tiles_h = plan.tiles_h;
  kp.cv_row_tiles = plan.row_tiles;
  kp.cv_cblocks = plan.cblocks;
  kp.cv_taps = p.filter_h * p.filter_w;
  kp.cv_fw = p.filter_w;
  kp.cv_sh = p.stride_h;
  kp.cv_sw = p.stride_w;
  kp.cv_ph = p.pad_h;
  kp.cv_pw = p.pad_w;
  kp.cv_dh = p.dil_h;
  kp.cv_dw = p.dil_w;
  kp.bias = p.has_bias ? bias : nullptr;
#ifdef TNX_DEV_TRACE
  {
    const char* t = getenv("TNX_TRACE_PTR");
    kp.trace = t ? reinterpret_cast<unsigned long long*>(strtoull(t, nullptr, 0)) : nullptr;
  }
#endif

  cudaError_t e = allow_full_smem(fn);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%d B dynamic smem): %s", kMaxDynamicSmem, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(res.grid, 1, 1);
  lc.blockDim = dim3(kThreads, 1, 1);
  lc.dynamicSmemBytes = res.smem_bytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cfg.cta_group;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  e = cudaLaunchKernelEx(&lc, fn, ta, tb, tc, kp);
  if (e != cudaSuccess) {
    set_error("convolution kernel launch failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}


// ---------------------------------------------------------------------------------------------
// 1 x 1 convolution over NCHW tensors = a batch of GEMMs that share the weights
// ---------------------------------------------------------------------------------------------
namespace {

// 3-D tensor map (column, row, matrix) over `batch` row-major matrices of 16-bit elements.
int make_tmap_batched(CUtensorMap* out, const void* ptr, int dtype, int64_t cols, int64_t rows,
                      int64_t batch, int box_cols, int box_rows, bool is_operand) {
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return TNX_ERR_CUDA;
  }
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * 2,
                                 static_cast<cuuint64_t>(cols * rows) * 2};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt =
      dtype == TNX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = encode(out, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      is_operand ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (3-D) failed with CUresult %d (ptr %p, %lld x %lld x %lld)",
              static_cast<int>(r), ptr, static_cast<long long>(batch), static_cast<long long>(rows),
              static_cast<long long>(cols));
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

// The GEMM one image amounts to: M = c_out, N = h*w, K = c_in, all row-major and dense.
tnx_problem image_gemm(const tnx_conv2d_problem& p) {
  tnx_problem g = {};
  g.m = p.c_out;
  g.n = p.h_in * p.w_in;
  g.k = p.c_in;
  g.dtype = p.dtype;
  g.epilogue = TNX_EPI_NONE;
  g.stride_am = p.c_in;
  g.stride_ak = 1;
  g.stride_bk = g.n;
  g.stride_bn = 1;
  g.stride_cm = g.n;
  g.stride_cn = 1;
  return g;
}

}  // namespace

bool conv_is_batched_gemm(const tnx_conv2d_problem& p) {
  if (getenv("TNX_CONV_NO_BATCHED_GEMM") != nullptr) return false;  // read every time: tests flip it
  const long long hw = static_cast<long long>(p.h_in) * p.w_in;
  return p.dtype != TNX_F32 && p.filter_h == 1 && p.filter_w == 1 && p.stride_h == 1 &&
         p.stride_w == 1 && p.pad_h == 0 && p.pad_w == 0 && p.input_layout == TNX_LAYOUT_NCHW &&
         p.output_layout == TNX_LAYOUT_NCHW && p.weight_layout == TNX_WEIGHT_KCRS && hw % 8 == 0 &&
         hw <= 0x7fffffff && p.c_in % 8 == 0;
}

int umma_conv1x1_query(const tnx_conv2d_problem& p, tnx_config* cfg, tnx_conv2d_resources* out) {
  const tnx_problem g = image_gemm(p);
  if (cfg->cta_group == 0 && cfg->tile_m == 0) cfg->cta_group = p.c_out >= 256 ? 2 : 1;
  if (cfg->tile_n == 0 && cfg->cta_group == 2 && g.n <= 64) cfg->tile_n = 128;
  if (cfg->tile_k == 0) cfg->tile_k = p.c_in % 128 == 0 ? 128 : 64;
  cfg->split_k = 1;
  cfg->tile_order = TNX_ORDER_GROUPED;
  tnx_resources r;
  int rc = umma_query(g, cfg, &r);
  out->kernel = TNX_KERNEL_TCGEN05;
  out->h_out = p.h_in;
  out->w_out = p.w_in;
  out->tile_w = cfg->tile_n;  // here the pixels are the columns of a tile, the rows output channels
  out->tile_h = 1;
  out->smem_bytes = r.smem_bytes;
  out->tmem_columns = r.tmem_columns;
  out->workspace_bytes = 0;
  if (rc != TNX_OK) return rc;
  const long long units = static_cast<long long>(p.batch) * r.tiles_m * r.tiles_n;
  if (static_cast<long long>(p.batch) * r.tiles_m > 0xffff) {
    set_error("too many row tiles in the batch (%lld)", static_cast<long long>(p.batch) * r.tiles_m);
    return TNX_ERR_INVALID;
  }
  int max_clusters = device_sm_count() / cfg->cta_group;
  if (cfg->max_ctas > 0 && cfg->max_ctas / cfg->cta_group < max_clusters)
    max_clusters = cfg->max_ctas / cfg->cta_group;
  if (max_clusters < 1) max_clusters = 1;
  out->grid = static_cast<int32_t>((units < max_clusters ? units : max_clusters) * cfg->cta_group);
  return TNX_OK;
}

int umma_conv1x1_launch(const tnx_conv2d_problem& p, const tnx_config& cfg,
                        const tnx_conv2d_resources& res, const void* x, const void* w,
                        const void* bias, void* y, int32_t* status_word, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
       reinterpret_cast<uintptr_t>(y)) & 15u) {
    set_error("tcgen05 convolution needs 16-byte aligned input, weight and output buffers");
    return TNX_ERR_INVALID;
  }
  const tnx_problem g = image_gemm(p);
  KernelFn fn = pick_kernel(cfg.tile_n, cfg.tile_k, cfg.cta_group, false, p.dtype);
  if (fn == nullptr) return TNX_ERR_NOT_BUILT;
  const int a_rows = a_box_rows(g, cfg);
  CUtensorMap ta, tb, tc;
  int rc = make_tmap(&ta, w, p.dtype, g.k, g.m, g.k, kAtomElems, a_rows, true);
  if (rc != TNX_OK) return rc;
  rc = make_tmap_batched(&tb, x, p.dtype, g.n, g.k, p.batch, kAtomElems, cfg.tile_k, true);
  if (rc != TNX_OK) return rc;
  rc = make_tmap_batched(&tc, y, p.dtype, g.n, g.m, p.batch, kAtomElems, kRowsPerCta, false);
  if (rc != TNX_OK) return rc;

  const int tiles_m_img = cdiv(g.m, kRowsPerCta * cfg.cta_group);
  UmmaParams kp = {};
  kp.m = g.m;
  kp.n = g.n;
  kp.k = g.k;
  kp.n_out = g.n;
  kp.tiles_m = p.batch * tiles_m_img;
  kp.tiles_n = cdiv(g.n, cfg.tile_n);
  kp.num_kb = cdiv(g.k, cfg.tile_k);
  kp.split_k = 1;
  kp.kb_per_slice = kp.num_kb;
  kp.tile_k = cfg.tile_k;
  kp.a_rows = a_rows;
  kp.staging_bytes = 2 * kStagingBytes;
  kp.stages = cfg.stages;
  kp.acc_stages = cfg.acc_stages;
  kp.group_m = cfg.group_m;
  kp.tile_order = TNX_ORDER_GROUPED;
  kp.epilogue = TNX_EPI_NONE;
  kp.status = status_word;
  kp.timeout_ns = wait_limit_ns();
  kp.bias = p.has_bias ? bias : nullptr;
  kp.bias_per_row = 1;
  kp.batched = p.batch;
  kp.bt_tiles_m = tiles_m_img;

  cudaError_t e = allow_full_smem(fn);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%d B dynamic smem): %s", kMaxDynamicSmem, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(res.grid, 1, 1);
  lc.blockDim = dim3(kThreads, 1, 1);
  lc.dynamicSmemBytes = res.smem_bytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cfg.cta_group;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  e = cudaLaunchKernelEx(&lc, fn, ta, tb, tc, kp);
  if (e != cudaSuccess) {
    set_error("convolution kernel launch failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

}  // namespace tnx

// ---------------------------------------------------------------------------------------------
// Split-K GEMM on scratch that lives inside the library
// ---------------------------------------------------------------------------------------------
// Some hosts cannot hand this library a workspace: a serving runtime that gave its whole
// device-memory budget to its own arena at start-up and forbids further driver allocations, or
// a latency-critical loop where an allocation call is unacceptable because cudaMalloc may
// synchronise the whole device.  For them the split-K scratch is this fixed array, which every
// GPU that loads the library carries until the process exits.
static __device__ __align__(256) unsigned char tnx_builtin_scratch[TNX_STATIC_SCRATCH_BYTES];

namespace {

// `tnx_builtin_scratch` names a host-side handle here, not a device address.  The address the
// kernel needs is looked up once per device, with that device current.
int builtin_scratch_address(void** out) {
  static std::mutex mu;
  static void* address[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    tnx::set_error("cannot identify the current device: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (address[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, tnx_builtin_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      tnx::set_error("cudaGetSymbolAddress(built-in scratch) failed on device %d: %s", dev,
                     cudaGetErrorString(e));
      (void)cudaGetLastError();
      return TNX_ERR_CUDA;
    }
    address[dev] = ptr;
  }
  *out = address[dev];
  return TNX_OK;
}

}  // namespace

extern "C" int tnx_gemm_splitk_static(const tnx_problem* problem, const tnx_config* config,
                                      const void* a, const void* b, void* c,
                                      int32_t* status_word, void* stream) {
  tnx_resources res;
  int rc = tnx_gemm_query(problem, config, &res);  // full validation of problem and config
  if (rc != TNX_OK) return rc;
  if (res.kernel != TNX_KERNEL_TCGEN05) {
    tnx::set_error("tnx_gemm_splitk_static runs the tcgen05 kernel only and these operands do not "
                   "qualify for it (fp16/bf16, row-major, 16-byte pitches, K and N multiples of 8)");
    return TNX_ERR_INVALID;
  }
  tnx_config cfg;
  if (config != nullptr)
    cfg = *config;
  else
    memset(&cfg, 0, sizeof(cfg));
  rc = tnx::umma_query(*problem, &cfg, &res);  // same answer, plus the defaults filled into cfg
  if (rc != TNX_OK) return rc;
  if (cfg.tile_order == TNX_ORDER_TABLE) {
    tnx::set_error("tnx_gemm_splitk_static takes no tile table; use a grouped or serpentine order");
    return TNX_ERR_INVALID;
  }
  if (res.workspace_bytes > static_cast<int64_t>(TNX_STATIC_SCRATCH_BYTES)) {
    tnx::set_error("this problem needs %lld bytes of split-K scratch at split_k=%d but the built-in "
                   "scratch holds %lld; lower split_k or tile_n, or call tnx_gemm with a workspace "
                   "of your own",
                   static_cast<long long>(res.workspace_bytes), res.split_k,
                   static_cast<long long>(TNX_STATIC_SCRATCH_BYTES));
    return TNX_ERR_INVALID;
  }
  if (problem->m == 0 || problem->n == 0) return TNX_OK;
  if (a == nullptr || b == nullptr || c == nullptr) {
    tnx::set_error("NULL operand pointer");
    return TNX_ERR_INVALID;
  }
  void* scratch = nullptr;
  rc = builtin_scratch_address(&scratch);
  if (rc != TNX_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (res.split_k > 1) {
    // The array keeps whatever the previous call (or an interrupted one) left behind; the tile
    // counters are the only part that has to start at zero.
    const size_t counters = static_cast<size_t>(res.tiles_m) * cfg.cta_group * res.tiles_n * 4;
    cudaError_t e = cudaMemsetAsync(scratch, 0, (counters + 255) & ~static_cast<size_t>(255), s);
    if (e != cudaSuccess) {
      tnx::set_error("clearing the split-K counters failed: %s", cudaGetErrorString(e));
      (void)cudaGetLastError();
      return TNX_ERR_CUDA;
    }
  }
  return tnx::umma_launch(*problem, cfg, res, a, b, c, scratch, nullptr, status_word, s);
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded-wait machinery
// ---------------------------------------------------------------------------------------------
namespace {

// One warp waits on an mbarrier that nothing ever arrives on, through the same ptx::mbar_wait the
// GEMM kernels use.  The wait must give up after `limit_ns`, record a code and let the kernel
// return normally: no trap, no fault, the context stays usable.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tnx::ptx::mbar_init(tnx::ptx::smem_u32(&bar), 1);
    abort_flag = 0;
    tnx::ptx::fence_mbar_init();
  }
  __syncthreads();
  const bool ok = tnx::ptx::mbar_wait(tnx::ptx::smem_u32(&bar), 0, &abort_flag, limit_ns);
  if (!ok && threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, 0x1ff);
}

}  // namespace

extern "C" int tnx_selftest_bounded_wait(int32_t* status_word, uint32_t limit_ms, void* stream) {
  if (status_word == nullptr || limit_ms == 0 || limit_ms > 5000) {
    tnx::set_error("tnx_selftest_bounded_wait needs a status word and a limit of 1..5000 ms");
    return TNX_ERR_INVALID;
  }
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      status_word, static_cast<unsigned long long>(limit_ms) * 1000000ull);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tnx::set_error("self-test launch failed: %s", cudaGetErrorString(e));
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}
