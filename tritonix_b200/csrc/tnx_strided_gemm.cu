// CUDA-core GEMM for operands the TMA/tcgen05 path cannot take: arbitrary (positive or zero)
// element strides, sizes that break TMA's 16-byte pitch rule, and fp32 inputs (full-precision
// FMA, i.e. the reference's input_precision="ieee" branch, tritonix/ops/swiglu.py:93).
// Same contract as the reference kernels it stands in for (tritonix/ops/matmul.py:42-108,
// tritonix/ops/swiglu.py:24-110): fp32 accumulation, one round-to-nearest cast at the end,
// optional fused gate*up epilogue over interleaved columns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "tnx_internal.h"

namespace tnx {
namespace {

constexpr int kBM = 64, kBN = 64, kBK = 16;
constexpr int kTX = 16, kTY = 16;  // 256 threads, each owns a 4 x 4 patch of the tile

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float gate_act(float g, int epilogue) {
  if (epilogue == TNX_EPI_GLU_LINEAR) return g;
  const float s = 1.0f / (1.0f + expf(-g));
  return epilogue == TNX_EPI_GLU_SILU ? g * s : s;
}

template <typename T>
__global__ void __launch_bounds__(kTX * kTY)
strided_gemm_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c, int m,
                    int n, int k, long long sam, long long sak, long long sbk, long long sbn,
                    long long scm, long long scn, int epilogue) {
  __shared__ float as[kBK][kBM + 1];
  __shared__ float bs[kBK][kBN + 1];
  const int tx = threadIdx.x % kTX, ty = threadIdx.x / kTX;
  const int row0 = blockIdx.y * kBM, col0 = blockIdx.x * kBN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += kBK) {
    for (int i = threadIdx.x; i < kBM * kBK; i += kTX * kTY) {
      const int r = i / kBK, kk = i % kBK;
      const int gr = row0 + r, gk = k0 + kk;
      as[kk][r] = (gr < m && gk < k) ? to_f32(a[gr * sam + gk * sak]) : 0.0f;
    }
    for (int i = threadIdx.x; i < kBK * kBN; i += kTX * kTY) {
      const int kk = i / kBN, cidx = i % kBN;
      const int gk = k0 + kk, gc = col0 + cidx;
      bs[kk][cidx] = (gk < k && gc < n) ? to_f32(b[gk * sbk + gc * sbn]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kBK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + ty * 4 + i;
    if (gr >= m) continue;
    if (epilogue == TNX_EPI_NONE) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gc = col0 + tx * 4 + j;
        if (gc < n) c[gr * scm + gc * scn] = from_f32<T>(acc[i][j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int gc = col0 + tx * 4 + 2 * j;  // gate column; its partner is gc + 1
        if (gc + 1 < n)
          c[gr * scm + (gc / 2) * scn] =
              from_f32<T>(gate_act(acc[i][2 * j], epilogue) * acc[i][2 * j + 1]);
      }
    }
  }
}

template <typename T>
int launch_typed(const tnx_problem& p, const void* a, const void* b, void* c, cudaStream_t stream) {
  dim3 grid((p.n + kBN - 1) / kBN, (p.m + kBM - 1) / kBM, 1);
  if (grid.y > 65535u) {
    set_error("strided kernel: m=%d needs more than 65535 tile rows", p.m);
    return TNX_ERR_INVALID;
  }
  strided_gemm_kernel<T><<<grid, kTX * kTY, 0, stream>>>(
      static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(c), p.m, p.n, p.k,
      p.stride_am, p.stride_ak, p.stride_bk, p.stride_bn, p.stride_cm, p.stride_cn, p.epilogue);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("strided kernel launch failed: %s", cudaGetErrorString(e));
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

}  // namespace

int strided_query(const tnx_problem& p, tnx_config* cfg, tnx_resources* out) {
  (void)cfg;
  out->kernel = TNX_KERNEL_STRIDED;
  out->smem_bytes = static_cast<int32_t>(sizeof(float) * kBK * (kBM + 1 + kBN + 1));
  out->tmem_columns = 0;
  out->tiles_m = (p.m + kBM - 1) / kBM;
  out->tiles_n = (p.n + kBN - 1) / kBN;
  out->grid = out->tiles_m * out->tiles_n;
  out->split_k = 1;
  out->workspace_bytes = 0;
  return TNX_OK;
}

int strided_launch(const tnx_problem& p, const void* a, const void* b, void* c,
                   cudaStream_t stream) {
  switch (p.dtype) {
    case TNX_F16: return launch_typed<__half>(p, a, b, c, stream);
    case TNX_BF16: return launch_typed<__nv_bfloat16>(p, a, b, c, stream);
    case TNX_F32: return launch_typed<float>(p, a, b, c, stream);
    default: set_error("unknown dtype %d", p.dtype); return TNX_ERR_INVALID;
  }
}

}  // namespace tnx
