// The whole SwiGLU MLP block in ONE persistent launch for sm_100a:
//     Y[M, n_out] = ( act(X.W1) * (X.W2) ) . W3        W12 = W1/W2 column-interleaved, K x 2F
// This is what the reference's three-matrix kernel attempts (swiglu_kernel,
// tritonix/ops/swiglu.py:113-230: one program per gate/up tile, its slice of the hidden
// activation multiplied by W3 at once and added to Z with atomics; wrong W3 indexing beyond one
// tile, fp32 only) and what its design sketch describes (playground/fused_mlp.py:10-161: two
// phases, a workspace for the hidden activation, spin-wait flags per row block).  Here:
//
//  * Two kinds of work unit share one TMA -> shared-memory ring -> tcgen05.mma -> TMEM pipeline
//    on CTA pairs (256 x 256 tiles, cta_group::2):
//      G(t, j)  hidden tile: rows of 256-row tile t, interleaved W12 columns [256 j, 256 j + 256),
//               K = d_model, GLU epilogue -> 128 columns of the hidden activation H (bf16/fp16)
//      D(t, j)  output tile: same rows, columns [256 j, 256 j + 256) of Y, K = d_ff, A operand = H
//  * Units are walked in ONE fixed global order, cluster c taking units c, c + G, c + 2G, ...:
//    row tiles are grouped in bands; the order is G(band 0), G(band 1), D(band 0), G(band 2),
//    D(band 1), ... so that the hidden rows a D unit needs were finished about one band earlier
//    and its wait is normally already satisfied.  Inside a band units run column by column, so
//    the clusters working side by side share a weight tile through L2.
//  * H lives in a ring of a few bands inside a caller-owned workspace: it is written by TMA
//    stores and read back by TMA loads while still in L2, and a band's slot is reused once the
//    D units of the band that held it are done.  Cross-CTA dependencies are plain counters in
//    global memory, one pair per row tile: g_done (G units finished: H rows complete) and d_done
//    (D units finished reading: slot reusable).  A unit only ever waits for units EARLIER in the
//    global order, every cluster walks its units in increasing order, and the grid never exceeds
//    what is resident at once, so the unit with the smallest index never waits: no deadlock.
//    Every wait is bounded all the same (wall clock), and gives up through the status word.
//  * Deterministic: no atomics on data, fixed summation order per tile.
//  * Tensor parallel (optional): when the hidden dimension is split over `world` GPUs, every rank
//    computes a partial Y and the partials must be summed.  The sum runs INSIDE this kernel, row
//    tile by row tile, while later tiles are still being computed.  A tensor-parallel launch has
//    256 threads per CTA: warps 0-5 work as above, warps 6-7 of EVERY CTA form its exchange
//    crew.  The crews share out the row tiles (each tile's share of rows is cut in `tile_split`
//    pieces so that a burst of finished tiles spreads over many SMs).  For its piece a crew
//    waits for a third counter (y_done: every output tile of the row tile stored), tells the
//    other ranks through a multicast counter (multimem.red), waits until every rank has the row
//    tile, then sums 256 / (world * tile_split) rows of it across all ranks with
//    multimem.ld_reduce (the NVSwitch adds) and writes the result to all ranks with multimem.st.
//    A multimem access occupies an SM's load/store path for a few cycles whatever the number of
//    threads behind it (about half a million 16-byte accesses per millisecond and SM were
//    measured), and a crew that saturates that path starves the barrier polls and shared-memory
//    stores of the computing warps next to it.  Hence small crews (two warps: their own latency
//    throttles them to a fraction of that rate) on ALL SMs, and small pieces, instead of a few
//    SMs that do nothing else.  The partial outputs are either kept in fp32 (a buffer of their
//    own) and rounded to the output type only after the cross-rank sum, so that the result
//    carries ONE rounding as on a single GPU, or (no such buffer given) rounded to the output
//    type, stored in Y and summed in place with fp32 accumulation in the switch: half the
//    NVLink traffic and half the multimem requests for a second rounding.  The partial buffer, Y and the
//    counters live in symmetric memory mapped into one multicast object; no TMA operation
//    touches another GPU's memory; the computing warps never wait for a crew.  Cross-rank
//    counters are never reset: call number `epoch` waits for epoch * world arrivals.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <utility>
#include <vector>

#include "tnx_internal.h"
#include "tnx_ptx.cuh"

namespace tnx {

namespace {

constexpr int kRows = 128;       // rows per CTA (TMEM lanes); a pair owns 256
constexpr int kTileN = 256;      // accumulator columns per unit
constexpr int kLoadN = 128;      // B columns each CTA of the pair loads
constexpr int kThreads = 192;         // producer warp, MMA warp, four epilogue warps
constexpr int kExchangeThreads = 256; // block size of a tensor-parallel launch: warps 6 and 7 are the exchange crew
constexpr int kCrewBarrier = 2;       // named barrier of the crew
constexpr int kEpiThreads = 128;
constexpr int kEpiBarrier = 1;
constexpr int kAtomBytes = 128;
constexpr int kAtomElems = 64;
constexpr int kStagingBytes = kRows * kAtomBytes;
constexpr int kMaxStages = 8;
constexpr int kCtrlBytes = 512;
constexpr int kAlignSlack = 1024;

constexpr int kAbortProducer = 0x201;
constexpr int kAbortMma = 0x202;
constexpr int kAbortEpilogue = 0x203;
constexpr int kAbortExchange = 0x204;

struct MlpParams {
  int m, d_model, d_ff, n_out;
  int tiles_m;             // 256-row tiles
  int n_g, n_d;            // column tiles per row tile: G units (2 d_ff / 256), D units (n_out / 256)
  int kb_g, kb_d;          // K blocks per G unit (over d_model) and per D unit (over d_ff)
  int band;                // row tiles per band
  int num_bands, last_rows;  // last_rows = row tiles of the last band
  int ring_bands;          // bands of H the workspace holds
  int stages;
  int epilogue;            // TNX_EPI_GLU_*
  int total_units;
  int* g_done;             // [tiles_m] CTAs (2 per unit) that finished a G unit of the row tile
  int* d_done;             // [tiles_m] CTAs that finished a D unit of the row tile
  int* status;
  unsigned long long timeout_ns;
  // tensor-parallel exchange (world == 1: none of this is used)
  int world, rank;
  int exchange;            // 1: tensor-parallel launch (fp32 partial outputs, crews sum them across ranks)
  int tile_split;          // pieces a row tile's share of rows is cut into (one crew each)
  int* y_done;             // [tiles_m] CTAs that finished STORING a D unit of the row tile
  int* crews_done;         // [1] exchange crews of this GPU that have written all their pieces
  void* y_mc;              // multicast address of Y (the same buffer on every rank)
  long long ldy;           // row pitch of Y in elements
  const float* part_mc;    // multicast address of the fp32 partial outputs ([rows, n_out], pitch n_out)
  float* part_local;       // this rank's mapping of the same buffer
  unsigned* sig_mc;        // [1 + sig_tiles] arrival counters: multicast address ...
  const unsigned* sig_local;  // ... and this rank's copy.  [0]: closing barrier; [1 + t]: row tile t
  int sig_tiles;           // row-tile counters in the array (>= tiles_m)
  unsigned epoch;          // ordinal of this call (1, 2, ...)
};

struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort;
  int flag;
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

struct Unit {
  int down;   // 0: G unit, 1: D unit
  int t, j;   // row tile, column tile
};

// Position u of the global order -> unit.  Segments: G(0), then for q = 0 .. num_bands-2 the pair
// [G(q+1), D(q)], then D(num_bands-1).  All bands have `band` row tiles except the last.
__host__ __device__ __forceinline__ Unit decode_unit(const MlpParams& p, int u) {
  Unit r;
  const int g_full = p.band * p.n_g, d_full = p.band * p.n_d;
  const int last = p.num_bands - 1;
  int b, rows, idx;
  const int g0 = (last == 0 ? p.last_rows : p.band) * p.n_g;  // size of G(0)
  if (u < g0) {
    r.down = 0; b = 0; rows = last == 0 ? p.last_rows : p.band; idx = u;
  } else {
    int v = u - g0;
    if (last == 0) {
      r.down = 1; b = 0; rows = p.last_rows; idx = v;
    } else {
      const int period = g_full + d_full;
      int q = v / period;
      if (q > last - 1) q = last - 1;
      v -= q * period;
      const int g_size = (q + 1 == last ? p.last_rows : p.band) * p.n_g;
      if (v < g_size) {
        r.down = 0; b = q + 1; rows = q + 1 == last ? p.last_rows : p.band; idx = v;
      } else if (v - g_size < d_full) {
        r.down = 1; b = q; rows = p.band; idx = v - g_size;
      } else {
        r.down = 1; b = last; rows = p.last_rows; idx = v - g_size - d_full;
      }
    }
  }
  r.j = idx / rows;
  r.t = b * p.band + (idx - r.j * rows);
  return r;
}

// Row tile of the H ring that holds row tile t.
__device__ __forceinline__ int ring_tile(const MlpParams& p, int t) {
  const int b = t / p.band;
  return (b % p.ring_bands) * p.band + (t - b * p.band);
}

__device__ __forceinline__ int ld_acquire_gpu(const int* ptr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// Orders accesses made through the async proxy (TMA) with generic-proxy accesses to global memory.
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// Bounded wait until *counter >= target.  Gives up after limit_ns, when this CTA has aborted, or
// when any CTA has already reported a failure through the status word.
__device__ __forceinline__ bool wait_counter(const int* counter, int target, volatile int* abort_flag,
                                             const int* status, uint64_t limit_ns) {
  if (ld_acquire_gpu(counter) >= target) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (ld_acquire_gpu(counter) >= target) return true;
    __nanosleep(100);
    if ((it & 0x3fu) == 0) {
      if (*abort_flag != 0) return false;
      if ((status != nullptr && ld_acquire_gpu(status) != 0) ||
          ptx::globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* ptr) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// Same bounded wait on a counter that other GPUs increment.
__device__ __forceinline__ bool wait_counter_sys(const unsigned* counter, unsigned target,
                                                 volatile int* abort_flag, const int* status,
                                                 uint64_t limit_ns) {
  if (ld_acquire_sys(counter) >= target) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (ld_acquire_sys(counter) >= target) return true;
    __nanosleep(200);
    if ((it & 0x3fu) == 0) {
      if (*abort_flag != 0) return false;
      if ((status != nullptr && ld_acquire_gpu(status) != 0) ||
          ptx::globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
// The multicast address and a GPU's own (unicast) address of the same bytes are virtual aliases:
// accesses made through one are ordered with accesses made through the other only across this
// fence (the partial outputs are written through the unicast alias and read through the
// multicast one; Y and the counters the other way round).
__device__ __forceinline__ void fence_proxy_alias() {
  asm volatile("fence.proxy.alias;" ::: "memory");
}
// Adds 1 to the counter's copy on every GPU of the multicast object; earlier writes of this
// thread (and those it has observed) are visible to whoever acquires the new value.
__device__ __forceinline__ void multimem_signal(unsigned* mc_counter) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], 1;" ::"l"(mc_counter) : "memory");
}
// Four fp32 values summed over all GPUs of the multicast object (the switch adds them).  The
// data accesses are relaxed at system scope, so that the fences and the counters'
// release/acquire pairs order them across the ranks: with .weak accesses (same speed) a rank was
// seen to leave the closing barrier before all of a peer's multimem.st had landed in its memory.
__device__ __forceinline__ float4 multimem_sum(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// Eight 16-bit values summed over all GPUs, accumulated in fp32 by the switch, rounded once.
template <bool BF16>
__device__ __forceinline__ uint4 multimem_sum16(const void* mc_addr) {
  uint4 v;
  if (BF16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
  return v;
}
__device__ __forceinline__ void multimem_store(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
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

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

template <int TILE_K, bool BF16>
__global__ void __launch_bounds__(kExchangeThreads, 1)
swiglu_mlp_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w12,
                  const __grid_constant__ CUtensorMap tmap_h_st, const __grid_constant__ CUtensorMap tmap_h_ld,
                  const __grid_constant__ CUtensorMap tmap_w3, const __grid_constant__ CUtensorMap tmap_y,
                  const MlpParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t base_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base_addr - raw_addr);

  constexpr int a_stage_bytes = kRows * TILE_K * 2;
  constexpr int a_atom_bytes = kRows * kAtomBytes;
  constexpr int b_stage_bytes = kLoadN * TILE_K * 2;
  const uint32_t smem_a = base_addr;
  const uint32_t smem_b = smem_a + p.stages * a_stage_bytes;
  const uint32_t smem_out = smem_b + p.stages * b_stage_bytes;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(base_ptr + (smem_out - base_addr) + 2 * kStagingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  volatile int* abort_flag = &ctrl->abort;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tmap_x);
    ptx::prefetch_tensormap(&tmap_w12);
    ptx::prefetch_tensormap(&tmap_h_st);
    ptx::prefetch_tensormap(&tmap_h_ld);
    ptx::prefetch_tensormap(&tmap_w3);
    ptx::prefetch_tensormap(&tmap_y);
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&ctrl->tmem_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctrl->tmem_empty[a]), 8);  // one arrive per epilogue warp of the pair
    }
    ctrl->abort = 0;
    ctrl->flag = 0;
    ptx::fence_mbar_init();
  }
  __syncwarp();
  ptx::cluster_arrive();  // the peer's barriers must exist before anything signals them
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tmem_alloc<2>(ptx::smem_u32(&ctrl->tmem_base), 512);
    ptx::tmem_relinquish<2>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = ctrl->tmem_base;

  if (warp >= 6) {
    // ===== exchange crew (tensor-parallel launches only): cross-rank sum of Y, piece by piece =====
    const int crew_tid = threadIdx.x - kThreads;
    const int crew_n = blockDim.x - kThreads;
    const int rows_per_piece = (2 * kRows) / (p.world * p.tile_split);
    const int vec_per_row = p.n_out >> 3;  // 16-byte vectors (eight values) per output row
    char* y_mc = static_cast<char*>(p.y_mc);
    const int pieces = p.tiles_m * p.tile_split;
    bool ok = true;
    for (int j = blockIdx.x; j < pieces && ok; j += gridDim.x) {
      const int t = j / p.tile_split, q = j - t * p.tile_split;
      if (crew_tid == 0) {
        bool got = true;
        if (q == 0) {
          // this rank's partial rows are complete (every output tile of the row tile is stored):
          // tell every rank
          got = wait_counter(p.y_done + t, 2 * p.n_d, abort_flag, p.status, p.timeout_ns);
          fence_proxy_alias();
          if (got) multimem_signal(p.sig_mc + 1 + t);
        }
        // every rank has said so in this call
        if (got)
          got = wait_counter_sys(p.sig_local + 1 + t, p.epoch * static_cast<unsigned>(p.world), abort_flag,
                                 p.status, p.timeout_ns);
        ctrl->flag = got ? 1 : 0;
      }
      ptx::named_barrier_sync(kCrewBarrier, crew_n);
      ok = ctrl->flag != 0;
      fence_proxy_alias();  // the sums below go through the multicast alias
      if (ok) {
        const int row_lo = t * 2 * kRows + (p.rank * p.tile_split + q) * rows_per_piece;
        const int rows = min(rows_per_piece, p.m - row_lo);
        const int total = rows > 0 ? rows * vec_per_row : 0;
        constexpr int kVec = 8;  // output vectors (eight values each) per thread and round
        if (p.part_mc == nullptr) {
          // partial outputs in the output type, summed in place in Y
          for (int base = crew_tid; base < total; base += crew_n * kVec) {
            uint4 v[kVec];
            size_t off[kVec];
#pragma unroll
            for (int i = 0; i < kVec; ++i) {
              const int idx = base + i * crew_n;
              const int safe = idx < total ? idx : base;
              const int r = safe / vec_per_row;
              off[i] = (static_cast<size_t>(row_lo + r) * p.ldy + static_cast<size_t>(safe - r * vec_per_row) * 8) * 2;
              v[i] = multimem_sum16<BF16>(y_mc + off[i]);
            }
#pragma unroll
            for (int i = 0; i < kVec; ++i)
              if (base + i * crew_n < total) multimem_store(y_mc + off[i], v[i]);
          }
        } else
        for (int base = crew_tid; base < total; base += crew_n * kVec) {
          float4 lo[kVec], hi[kVec];
#pragma unroll
          for (int i = 0; i < kVec; ++i) {
            const int idx = base + i * crew_n;
            const int safe = idx < total ? idx : base;
            const int r = safe / vec_per_row;
            const float* src = p.part_mc + static_cast<size_t>(row_lo + r) * p.n_out +
                               static_cast<size_t>(safe - r * vec_per_row) * 8;
            lo[i] = multimem_sum(src);
            hi[i] = multimem_sum(src + 4);
          }
#pragma unroll
          for (int i = 0; i < kVec; ++i) {
            const int idx = base + i * crew_n;
            if (idx < total) {
              const int r = idx / vec_per_row;
              const size_t off = (static_cast<size_t>(row_lo + r) * p.ldy +
                                  static_cast<size_t>(idx - r * vec_per_row) * 8) * 2;
              uint4 v;  // the one rounding of the cross-rank fp32 sum
              v.x = pack2<BF16>(lo[i].x, lo[i].y);
              v.y = pack2<BF16>(lo[i].z, lo[i].w);
              v.z = pack2<BF16>(hi[i].x, hi[i].y);
              v.w = pack2<BF16>(hi[i].z, hi[i].w);
              multimem_store(y_mc + off, v);
            }
          }
        }
      }
      ptx::named_barrier_sync(kCrewBarrier, crew_n);  // ctrl->flag is rewritten for the next piece
    }
    // Counters of row tiles this call does not have (it has fewer rows than the array was sized
    // for) advance all the same, so that "epoch * world" stays the target of every counter.
    if (crew_tid == 0 && ok)
      for (int t = p.tiles_m + blockIdx.x; t < p.sig_tiles; t += gridDim.x) multimem_signal(p.sig_mc + 1 + t);
    // Every rank leaves only when all crews of all ranks have written their pieces: Y is complete
    // everywhere, and nobody still reads this rank's partial rows.
    fence_proxy_alias();
    __threadfence_system();
    ptx::named_barrier_sync(kCrewBarrier, crew_n);
    if (crew_tid == 0) {
      if (ok) {
        // The last crew of this GPU to get here tells every rank once (so the target does not
        // depend on how many CTAs a call launched).
        if (atomicAdd(p.crews_done, 1) == static_cast<int>(gridDim.x) - 1) {
          __threadfence_system();
          multimem_signal(p.sig_mc);
        }
        ok = wait_counter_sys(p.sig_local, p.epoch * static_cast<unsigned>(p.world), abort_flag,
                              p.status, p.timeout_ns);
        fence_proxy_alias();  // Y was written through the multicast alias; it is read through the unicast one
      }
      if (!ok && p.status != nullptr) atomicCAS(p.status, 0, kAbortExchange);
    }
  } else if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      constexpr uint32_t stage_tx = static_cast<uint32_t>(a_stage_bytes + b_stage_bytes) * 2;
      bool ok = true;
      for (int u = cluster_id; u < p.total_units && ok; u += num_clusters) {
        const Unit un = decode_unit(p, u);
        const CUtensorMap* map_a = un.down ? &tmap_h_ld : &tmap_x;
        const CUtensorMap* map_b = un.down ? &tmap_w3 : &tmap_w12;
        const int num_kb = un.down ? p.kb_d : p.kb_g;
        const int row0 = ((un.down ? ring_tile(p, un.t) : un.t) * 2 + static_cast<int>(cta_rank)) * kRows;
        const int col0 = un.j * kTileN + static_cast<int>(cta_rank) * kLoadN;
        if (un.down) {
          // every G unit of this row tile (both CTAs of each) must have stored its part of H
          if (!wait_counter(p.g_done + un.t, 2 * p.n_g, abort_flag, p.status, p.timeout_ns)) {
            ok = false;
            break;
          }
          fence_proxy_async_global();  // the TMA loads below must observe those stores
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t empty_bar = ptx::smem_u32(&ctrl->empty[stage]);
          if (!ptx::mbar_wait(empty_bar, phase ^ 1u, abort_flag, p.timeout_ns)) {
            ok = false;
            break;
          }
          const uint32_t full_bar = ptx::smem_u32(&ctrl->full[stage]);
          const uint32_t a_dst = smem_a + stage * a_stage_bytes;
          const uint32_t b_dst = smem_b + stage * b_stage_bytes;
          const int k0 = kb * TILE_K;
          // Both CTAs' loads complete on the leader's barrier; the leader announces the bytes.
          const uint32_t leader_bar = ptx::mapa(full_bar, 0);
          if (leader) ptx::mbar_arrive_expect_tx(full_bar, stage_tx);
#pragma unroll
          for (int ka = 0; ka < TILE_K / kAtomElems; ++ka)
            ptx::tma_load_2d_pair(a_dst + ka * a_atom_bytes, map_a, k0 + ka * kAtomElems, row0,
                                  leader_bar);
#pragma unroll
          for (int na = 0; na < kLoadN / kAtomElems; ++na)
            ptx::tma_load_2d_pair(b_dst + na * (TILE_K * kAtomBytes), map_b, col0 + na * kAtomElems,
                                  k0, leader_bar);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok && p.status != nullptr) atomicCAS(p.status, 0, kAbortProducer);
    }
  } else if (warp == 1) {
    // ===== MMA issuer (leader CTA) =====
    if (leader && lane == 0) {
      const uint32_t fmt = BF16 ? 1u : 0u;
      // fp32 accumulate, A K-major, B MN-major, M x N = 256 x 256
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) |
                             (static_cast<uint32_t>(kTileN >> 3) << 17) |
                             (static_cast<uint32_t>((kRows * 2) >> 4) << 24);
      const uint64_t a_desc_hi = ptx::make_smem_desc(0, 0, 1024);
      const uint64_t b_desc_hi = ptx::make_smem_desc(0, TILE_K * kAtomBytes, 1024);
      constexpr uint32_t a_step16 = 32u >> 4, a_slab16 = static_cast<uint32_t>(a_atom_bytes) >> 4;
      constexpr uint32_t b_step16 = 2048u >> 4, b_slab16 = 8192u >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = cluster_id; u < p.total_units && ok; u += num_clusters) {
        const Unit un = decode_unit(p, u);
        const int num_kb = un.down ? p.kb_d : p.kb_g;
        const uint32_t te_bar = ptx::smem_u32(&ctrl->tmem_empty[acc]);
        if (!ptx::mbar_wait<true>(te_bar, acc_phase ^ 1u, abort_flag, p.timeout_ns)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t full_bar = ptx::smem_u32(&ctrl->full[stage]);
          if (!ptx::mbar_wait(full_bar, phase, abort_flag, p.timeout_ns)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a16 = (smem_a + stage * a_stage_bytes) >> 4;
          const uint32_t b16 = (smem_b + stage * b_stage_bytes) >> 4;
#pragma unroll
          for (int k16 = 0; k16 < TILE_K / 16; ++k16) {
            const uint32_t a_off = a16 + (k16 >> 2) * a_slab16 + (k16 & 3) * a_step16;
            const uint32_t b_off = b16 + (k16 >> 2) * b_slab16 + (k16 & 3) * b_step16;
            ptx::umma_f16<2>(d_tmem, a_desc_hi | (a_off & 0x3fffu), b_desc_hi | (b_off & 0x3fffu),
                             idesc, accumulate);
            accumulate = 1;
          }
          ptx::umma_commit_pair(ptx::smem_u32(&ctrl->empty[stage]), 0x3);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit_pair(ptx::smem_u32(&ctrl->tmem_full[acc]), 0x3);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok && p.status != nullptr) atomicCAS(p.status, 0, kAbortMma);
    }
  } else {
    // ===== epilogue =====
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t stage_row = static_cast<uint32_t>(row_in_tile) * kAtomBytes;
    const uint32_t sw = static_cast<uint32_t>(row_in_tile & 7);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t stores = 0;
    bool ok = true;
    for (int u = cluster_id; u < p.total_units && ok; u += num_clusters) {
      const Unit un = decode_unit(p, u);
      const int row0 = ((un.down ? un.t : ring_tile(p, un.t)) * 2 + static_cast<int>(cta_rank)) * kRows;
      // (when ranks exchange, a D unit stores its fp32 accumulator as it is, with plain stores)
      const bool raw = un.down && p.exchange != 0 && p.part_local != nullptr;
      const CUtensorMap* map_c = un.down ? &tmap_y : &tmap_h_st;
      const int acc_per_chunk = un.down ? 64 : 128;  // accumulator columns per 128-byte output row
      const int out_col0 = un.j * (un.down ? kTileN : kTileN / 2);
      const int out_cols = un.down ? p.n_out : p.d_ff;

      const uint32_t tf_bar = ptx::smem_u32(&ctrl->tmem_full[acc]);
      bool got = ptx::mbar_wait(tf_bar, acc_phase, abort_flag, p.timeout_ns);
      if (got && epi_tid == 0) {
        if (un.down) {
          // all MMAs of this unit are complete, so its loads of H are: one more reader done
          atomicAdd(p.d_done + un.t, 1);
        } else if (un.t >= p.ring_bands * p.band) {
          // this unit overwrites the ring slot of row tile t - ring_bands*band: its readers
          // (the D units of that row tile, both CTAs of each) must be done
          got = wait_counter(p.d_done + (un.t - p.ring_bands * p.band), 2 * p.n_d, abort_flag,
                             p.status, p.timeout_ns);
        }
      }
      if (!ptx::named_barrier_all(kEpiBarrier, kEpiThreads, got)) {
        ok = false;
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + lane_sel + acc * kTileN;
      if (raw) {
        // This rank's fp32 partial rows, straight from registers (each thread a row: 128 contiguous
        // bytes per step).  Plain stores, so that the fence below orders them for the other GPUs.
        const int row = row0 + row_in_tile;
        float* dst = p.part_local + static_cast<size_t>(row) * p.n_out + out_col0;
        for (int chunk = 0; chunk < kTileN / 32; ++chunk) {
          const int col = chunk * 32;
          if (out_col0 + col >= p.n_out) break;
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_acc + col, r);
          ptx::tmem_ld_wait();
          if (row < p.m) {
#pragma unroll
            for (int piece = 0; piece < 8; ++piece)
              if (out_col0 + col + piece * 4 < p.n_out)
                *reinterpret_cast<float4*>(dst + col + piece * 4) =
                    make_float4(__uint_as_float(r[piece * 4]), __uint_as_float(r[piece * 4 + 1]),
                                __uint_as_float(r[piece * 4 + 2]), __uint_as_float(r[piece * 4 + 3]));
          }
        }
      }
      const int chunks = raw ? 0 : kTileN / acc_per_chunk;
      for (int chunk = 0; chunk < chunks; ++chunk) {
        const int out_col = out_col0 + chunk * kAtomElems;
        if (out_col >= out_cols) break;
        const uint32_t buf = smem_out + (stores & 1u) * kStagingBytes;
        if (epi_tid == 0) ptx::tma_store_wait_read<1>();
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
        if (!un.down) {
#pragma unroll
          for (int sub = 0; sub < 4; ++sub) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(t_acc + chunk * 128 + sub * 32, r);
            ptx::tmem_ld_wait();
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float z0 = gate_act(__uint_as_float(r[4 * j]), p.epilogue) * __uint_as_float(r[4 * j + 1]);
              const float z1 = gate_act(__uint_as_float(r[4 * j + 2]), p.epilogue) * __uint_as_float(r[4 * j + 3]);
              o[j] = pack2<BF16>(z0, z1);
            }
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
              const uint32_t pos = static_cast<uint32_t>(sub * 2 + piece) ^ sw;
              st_shared_v4(buf + stage_row + pos * 16, o[piece * 4], o[piece * 4 + 1], o[piece * 4 + 2],
                           o[piece * 4 + 3]);
            }
          }
        } else {
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(t_acc + chunk * 64 + sub * 32, r);
            ptx::tmem_ld_wait();
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
              o[j] = pack2<BF16>(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
#pragma unroll
            for (int piece = 0; piece < 4; ++piece) {
              const uint32_t pos = static_cast<uint32_t>(sub * 4 + piece) ^ sw;
              st_shared_v4(buf + stage_row + pos * 16, o[piece * 4], o[piece * 4 + 1], o[piece * 4 + 2],
                           o[piece * 4 + 3]);
            }
          }
        }
        ptx::fence_proxy_async_smem();
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
        if (epi_tid == 0) {
          ptx::tma_store_2d(map_c, out_col, row0, buf);
          ptx::tma_store_commit();
        }
        ++stores;
      }
      // All tcgen05.ld of this accumulator are complete: hand the TMEM buffer back.
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        const uint32_t te = ptx::smem_u32(&ctrl->tmem_empty[acc]);
        if (leader)
          ptx::mbar_arrive(te);
        else
          ptx::mbar_arrive_cluster(ptx::mapa(te, 0));
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
      if (raw) {
        // Publish this CTA's partial rows of Y: every thread orders its stores for the whole
        // system (other GPUs read them through the multicast mapping), then one counts the CTA in.
        fence_proxy_alias();
        __threadfence_system();
        ptx::named_barrier_sync(kEpiBarrier, kEpiThreads);
        if (epi_tid == 0) atomicAdd(p.y_done + un.t, 1);
      } else if ((!un.down || p.exchange != 0) && epi_tid == 0) {
        // Publish this CTA's part of H (or, when ranks exchange 16-bit partial outputs in place,
        // of Y): the TMA stores must have landed (not merely have been read out of shared memory)
        // before the counter moves; Y is read by other GPUs, hence the system-wide fence.
        ptx::tma_store_wait_all<0>();
        fence_proxy_async_global();
        if (un.down) {
          fence_proxy_alias();
          __threadfence_system();
        } else {
          __threadfence();
        }
        atomicAdd((un.down ? p.y_done : p.g_done) + un.t, 1);
      }
    }
    if (epi_tid == 0) ptx::tma_store_wait_all<0>();
    if (!ok && lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, kAbortEpilogue);
  }

  // ------------------------------------------------------------------ teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (ctrl->abort != 0) {
    // A wait gave up: let copies and MMAs still in flight drain before shared memory and TMEM
    // are released (bounded: about a millisecond).
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  __syncwarp();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<2>(tmem_base, 512);
  }
}

using MlpKernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                             const CUtensorMap, const CUtensorMap, const MlpParams);

MlpKernelFn pick_mlp_kernel(int tile_k, int dtype) {
  if (tile_k == 64) return dtype == TNX_BF16 ? swiglu_mlp_kernel<64, true> : swiglu_mlp_kernel<64, false>;
  if (tile_k == 128) return dtype == TNX_BF16 ? swiglu_mlp_kernel<128, true> : swiglu_mlp_kernel<128, false>;
  return nullptr;
}

inline int cdiv(int a, int b) { return (a + b - 1) / b; }
inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

struct MlpPlan {
  tnx_config cfg;
  int tiles_m, n_g, n_d, band, num_bands, last_rows, ring_bands_min;
  int64_t counter_bytes, band_bytes;
};

int plan_mlp(const tnx_mlp_problem* p, const tnx_config* config, MlpPlan* plan, tnx_mlp_resources* out) {
  if (p == nullptr || out == nullptr) {
    set_error("problem or out is NULL");
    return TNX_ERR_INVALID;
  }
  if (p->dtype != TNX_F16 && p->dtype != TNX_BF16) {
    set_error("the fused MLP kernel takes fp16 or bf16 operands");
    return TNX_ERR_INVALID;
  }
  if (p->activation < TNX_EPI_GLU_LINEAR || p->activation > TNX_EPI_GLU_SIGMOID) {
    set_error("activation must be TNX_EPI_GLU_LINEAR, _SILU or _SIGMOID, got %d", p->activation);
    return TNX_ERR_INVALID;
  }
  if (p->m < 1 || p->d_model < 8 || p->d_ff < 8 || p->n_out < 8 || (p->d_model % 8) || (p->d_ff % 8) ||
      (p->n_out % 8)) {
    set_error("the fused MLP kernel needs m >= 1 and d_model, d_ff, n_out positive multiples of 8 "
              "(got m=%d d_model=%d d_ff=%d n_out=%d)", p->m, p->d_model, p->d_ff, p->n_out);
    return TNX_ERR_INVALID;
  }
  if (p->stride_xm < p->d_model || p->stride_w12k < 2LL * p->d_ff || p->stride_w3k < p->n_out ||
      p->stride_ym < p->n_out || (p->stride_xm % 8) || (p->stride_w12k % 8) || (p->stride_w3k % 8) ||
      (p->stride_ym % 8)) {
    set_error("row pitches must cover their rows and be multiples of 8 elements (16 bytes)");
    return TNX_ERR_INVALID;
  }
  tnx_config cfg = {};
  if (config != nullptr) cfg = *config;
  if (cfg.tile_k == 0) cfg.tile_k = 128;
  if (cfg.tile_m == 0) cfg.tile_m = 256;
  if (cfg.tile_n == 0) cfg.tile_n = 256;
  if (cfg.cta_group == 0) cfg.cta_group = 2;
  if (cfg.group_m == 0) cfg.group_m = 8;
  if (cfg.tile_m != 256 || cfg.tile_n != 256 || cfg.cta_group != 2 || (cfg.tile_k != 64 && cfg.tile_k != 128)) {
    set_error("the fused MLP kernel is built for 256 x 256 tiles on CTA pairs with tile_k 64 or 128 "
              "(got tile_m=%d tile_n=%d cta_group=%d tile_k=%d)", cfg.tile_m, cfg.tile_n, cfg.cta_group,
              cfg.tile_k);
    return TNX_ERR_NOT_BUILT;
  }
  if (cfg.group_m < 1) {
    set_error("group_m (row tiles per band) must be positive");
    return TNX_ERR_INVALID;
  }
  const int stage_bytes = (kRows + kLoadN) * cfg.tile_k * 2;
  const int fixed = 2 * kStagingBytes + kCtrlBytes + kAlignSlack;
  if (cfg.stages == 0) {
    const int s = (kMaxDynamicSmem - fixed) / stage_bytes;
    cfg.stages = s > kMaxStages ? kMaxStages : s;
  }
  if (cfg.stages < 2 || cfg.stages > kMaxStages) {
    set_error("stages must be in [2, %d], got %d", kMaxStages, cfg.stages);
    return TNX_ERR_INVALID;
  }
  const long long smem = static_cast<long long>(cfg.stages) * stage_bytes + fixed;
  plan->cfg = cfg;
  plan->tiles_m = cdiv(p->m, 2 * kRows);
  plan->n_g = cdiv(2 * p->d_ff, kTileN);
  plan->n_d = cdiv(p->n_out, kTileN);
  plan->band = cfg.group_m < plan->tiles_m ? cfg.group_m : plan->tiles_m;
  plan->num_bands = cdiv(plan->tiles_m, plan->band);
  plan->last_rows = plan->tiles_m - (plan->num_bands - 1) * plan->band;
  plan->ring_bands_min = plan->num_bands < 2 ? plan->num_bands : 2;
  plan->counter_bytes = align256((3LL * plan->tiles_m + 1) * 4);
  plan->band_bytes = static_cast<int64_t>(plan->band) * 2 * kRows * p->d_ff * 2;

  out->smem_bytes = static_cast<int32_t>(smem > 0x7fffffff ? 0x7fffffff : smem);
  out->tmem_columns = 512;
  out->tiles_m = plan->tiles_m;
  out->band_rows = plan->band * 2 * kRows;
  out->num_bands = plan->num_bands;
  const long long units = static_cast<long long>(plan->tiles_m) * (plan->n_g + plan->n_d);
  int clusters = sm_count() / 2;
  if (cfg.max_ctas > 0 && cfg.max_ctas / 2 < clusters) clusters = cfg.max_ctas / 2;
  if (clusters < 1) clusters = 1;
  out->grid = static_cast<int32_t>((units < clusters ? units : clusters) * 2);
  out->min_workspace_bytes = plan->counter_bytes + plan->ring_bands_min * plan->band_bytes;
  // Two bands measured best: a slot's previous readers are already a whole band of work ahead
  // of its next writers, and the smaller the ring the more of it stays in L2.
  out->workspace_bytes = out->min_workspace_bytes;
  if (smem > kMaxDynamicSmem) {
    set_error("shared memory budget exceeded: %lld B needed (%d stages x %d B + %d B), %d B per SM", smem,
              cfg.stages, stage_bytes, fixed, kMaxDynamicSmem);
    return TNX_ERR_RESOURCES;
  }
  if (units > 0x7fffffffLL || plan->tiles_m > 0xffff || plan->n_g > 0x3fff || plan->n_d > 0x3fff) {
    set_error("problem has too many tiles (%d row tiles, %d + %d column tiles)", plan->tiles_m, plan->n_g,
              plan->n_d);
    return TNX_ERR_INVALID;
  }
  return TNX_OK;
}

cudaError_t allow_full_smem_mlp(MlpKernelFn fn) {
  static std::mutex mu;
  static std::vector<std::pair<MlpKernelFn, int>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  for (const auto& d : done)
    if (d.first == fn && d.second == dev) return cudaSuccess;
  e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kMaxDynamicSmem);
  if (e == cudaSuccess) done.emplace_back(fn, dev);
  return e;
}

}  // namespace
}  // namespace tnx

extern "C" {

int tnx_swiglu_mlp_query(const tnx_mlp_problem* problem, const tnx_config* config, tnx_mlp_resources* out) {
  tnx::MlpPlan plan;
  return tnx::plan_mlp(problem, config, &plan, out);
}

int tnx_swiglu_mlp_unit_order(const tnx_mlp_problem* problem, const tnx_config* config, int32_t* units,
                              int32_t capacity) {
  using namespace tnx;
  MlpPlan plan;
  tnx_mlp_resources res;
  int rc = plan_mlp(problem, config, &plan, &res);
  if (rc != TNX_OK) return -rc;
  MlpParams kp = {};
  kp.n_g = plan.n_g;
  kp.n_d = plan.n_d;
  kp.band = plan.band;
  kp.num_bands = plan.num_bands;
  kp.last_rows = plan.last_rows;
  const int total = plan.tiles_m * (plan.n_g + plan.n_d);
  if (units != nullptr) {
    for (int u = 0; u < total && u < capacity; ++u) {
      const Unit un = decode_unit(kp, u);
      units[u] = (un.down << 30) | (un.t << 14) | un.j;
    }
  }
  return total;
}

int tnx_swiglu_mlp(const tnx_mlp_problem* problem, const tnx_config* config, const void* x, const void* w12,
                   const void* w3, void* y, void* workspace, size_t workspace_bytes,
                   const tnx_mlp_exchange* exchange, int32_t* status_word, void* stream) {
  using namespace tnx;
  MlpPlan plan;
  tnx_mlp_resources res;
  int tile_split = 0;  // > 0: tensor-parallel launch
  // (world == 1 is the degenerate exchange: same protocol, one participant)
  if (exchange != nullptr) {
    const tnx_mlp_exchange& ex = *exchange;
    tile_split = ex.tile_split > 0 ? ex.tile_split : 16;
    while (ex.world > 0 && tile_split > 1 && (2 * kRows) % (ex.world * tile_split) != 0) tile_split >>= 1;
    if (ex.world < 1 || ex.world > 2 * kRows || (2 * kRows) % ex.world != 0 || ex.rank < 0 || ex.rank >= ex.world ||
        (2 * kRows) % (ex.world * tile_split) != 0 || ex.epoch == 0 ||
        ex.signal_tiles < (problem != nullptr ? (problem->m + 2 * kRows - 1) / (2 * kRows) : 0)) {
      set_error("exchange: world * tile_split must divide 256, 0 <= rank < world, epoch >= 1, signal_tiles >= "
                "row tiles (got world=%d rank=%d tile_split=%d epoch=%u signal_tiles=%d)",
                ex.world, ex.rank, ex.tile_split, ex.epoch, ex.signal_tiles);
      return TNX_ERR_INVALID;
    }
    if (ex.y_multicast == nullptr || ex.signal_multicast == nullptr || ex.signal_local == nullptr ||
        (ex.partial_local == nullptr) != (ex.partial_multicast == nullptr) ||
        ((reinterpret_cast<uintptr_t>(ex.y_multicast) | reinterpret_cast<uintptr_t>(ex.partial_local) |
          reinterpret_cast<uintptr_t>(ex.partial_multicast)) & 15u) ||
        (reinterpret_cast<uintptr_t>(ex.signal_multicast) & 3u)) {
      set_error("exchange: y_multicast (16-byte aligned), signal_multicast and signal_local must be set; "
                "partial_local and partial_multicast (16-byte aligned) both or neither");
      return TNX_ERR_INVALID;
    }
  }
  int rc = plan_mlp(problem, config, &plan, &res);
  if (rc != TNX_OK) return rc;
  if (x == nullptr || w12 == nullptr || w3 == nullptr || y == nullptr || workspace == nullptr) {
    set_error("NULL operand or workspace pointer");
    return TNX_ERR_INVALID;
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w12) | reinterpret_cast<uintptr_t>(w3) |
       reinterpret_cast<uintptr_t>(y)) & 15u) {
    set_error("the fused MLP kernel needs 16-byte aligned x, w12, w3 and y base addresses");
    return TNX_ERR_INVALID;
  }
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) {
    set_error("workspace must be 256-byte aligned");
    return TNX_ERR_INVALID;
  }
  if (workspace_bytes < static_cast<size_t>(res.min_workspace_bytes)) {
    set_error("the fused MLP needs a workspace of at least %lld bytes (%lld recommended), got %zu",
              static_cast<long long>(res.min_workspace_bytes), static_cast<long long>(res.workspace_bytes),
              workspace_bytes);
    return TNX_ERR_INVALID;
  }
  const tnx_mlp_problem& p = *problem;
  int64_t ring = (static_cast<int64_t>(workspace_bytes) - plan.counter_bytes) / plan.band_bytes;
  if (ring > plan.num_bands) ring = plan.num_bands;
  MlpKernelFn fn = pick_mlp_kernel(plan.cfg.tile_k, p.dtype);
  if (fn == nullptr) return TNX_ERR_NOT_BUILT;

  int* counters = reinterpret_cast<int*>(workspace);
  void* h = static_cast<char*>(workspace) + plan.counter_bytes;
  const int64_t h_rows = ring * plan.band * 2 * kRows;
  const int tk = plan.cfg.tile_k;
  CUtensorMap tx, tw12, thst, thld, tw3, ty;
  rc = make_tmap_2d(&tx, x, p.dtype, p.d_model, p.m, p.stride_xm, kAtomElems, kRows, true);
  if (rc == TNX_OK) rc = make_tmap_2d(&tw12, w12, p.dtype, 2LL * p.d_ff, p.d_model, p.stride_w12k, kAtomElems, tk, true);
  if (rc == TNX_OK) rc = make_tmap_2d(&thst, h, p.dtype, p.d_ff, h_rows, p.d_ff, kAtomElems, kRows, false);
  if (rc == TNX_OK) rc = make_tmap_2d(&thld, h, p.dtype, p.d_ff, h_rows, p.d_ff, kAtomElems, kRows, true);
  if (rc == TNX_OK) rc = make_tmap_2d(&tw3, w3, p.dtype, p.n_out, p.d_ff, p.stride_w3k, kAtomElems, tk, true);
  if (rc == TNX_OK) rc = make_tmap_2d(&ty, y, p.dtype, p.n_out, p.m, p.stride_ym, kAtomElems, kRows, false);
  if (rc != TNX_OK) return rc;

  MlpParams kp = {};
  kp.m = p.m;
  kp.d_model = p.d_model;
  kp.d_ff = p.d_ff;
  kp.n_out = p.n_out;
  kp.tiles_m = plan.tiles_m;
  kp.n_g = plan.n_g;
  kp.n_d = plan.n_d;
  kp.kb_g = cdiv(p.d_model, tk);
  kp.kb_d = cdiv(p.d_ff, tk);
  kp.band = plan.band;
  kp.num_bands = plan.num_bands;
  kp.last_rows = plan.last_rows;
  kp.ring_bands = static_cast<int>(ring);
  kp.stages = plan.cfg.stages;
  kp.epilogue = p.activation;
  kp.total_units = plan.tiles_m * (plan.n_g + plan.n_d);
  kp.g_done = counters;
  kp.d_done = counters + plan.tiles_m;
  kp.status = status_word;
  kp.timeout_ns = bounded_wait_limit_ns();
  kp.world = 1;
  kp.y_done = counters + 2 * plan.tiles_m;
  kp.crews_done = counters + 3 * plan.tiles_m;
  if (tile_split > 0) {
    kp.exchange = 1;
    kp.tile_split = tile_split;
    kp.world = exchange->world;
    kp.rank = exchange->rank;
    kp.y_mc = exchange->y_multicast;
    kp.ldy = p.stride_ym;
    kp.part_mc = static_cast<const float*>(exchange->partial_multicast);
    kp.part_local = exchange->partial_local;
    kp.sig_mc = exchange->signal_multicast;
    kp.sig_local = exchange->signal_local;
    kp.sig_tiles = exchange->signal_tiles;
    kp.epoch = exchange->epoch;
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = allow_full_smem_mlp(fn);
  if (e == cudaSuccess) e = cudaMemsetAsync(counters, 0, static_cast<size_t>(plan.counter_bytes), s);
  if (e != cudaSuccess) {
    set_error("fused MLP set-up failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(res.grid, 1, 1);
  lc.blockDim = dim3(tile_split > 0 ? kExchangeThreads : kThreads, 1, 1);
  lc.dynamicSmemBytes = res.smem_bytes;
  lc.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  // Units wait for one another, so every cluster of the grid must be resident at once.
  int fit = 0;
  e = cudaOccupancyMaxActiveClusters(&fit, reinterpret_cast<const void*>(fn), &lc);
  if (e != cudaSuccess || fit < 1) {
    set_error("the fused MLP kernel cannot be scheduled: %s", e != cudaSuccess ? cudaGetErrorString(e) : "no cluster fits");
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  if (static_cast<int>(lc.gridDim.x) > fit * 2) lc.gridDim.x = static_cast<unsigned>(fit * 2);
  e = cudaLaunchKernelEx(&lc, fn, tx, tw12, thst, thld, tw3, ty, kp);
  if (e != cudaSuccess) {
    set_error("kernel launch failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

}  // extern "C"
