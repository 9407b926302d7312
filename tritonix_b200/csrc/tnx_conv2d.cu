// 2-D convolution forward: the C entry points, the repacking kernels around the tcgen05
// implicit GEMM, and a CUDA-core kernel for fp32.
//
// What is computed is what conv2d_forward_kernel of the reference computes
// (tritonix/ops/conv2d/forward.py:8-165): out[n, co, ho, wo] = bias[co] +
// sum over (c, r, s) of in[n, c, ho*stride_h - pad_h + r*dil_h, wo*stride_w - pad_w + s*dil_w] *
// w[co, c, r, s], taps outside the image contributing zero, accumulated in fp32 and cast to the
// operand type.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "tnx_internal.h"

namespace tnx {

namespace {

// ---------------------------------------------------------------------------------------------
// Repacking (16-bit types).  A batched 2-D transpose through shared memory: src is
// [batch][rows][cols] with row pitch src_pitch, dst is [batch][cols][rows] with row pitch
// dst_pitch >= rows; dst columns in [rows, dst_pitch) are written as zero.
//   N x C x H x W -> N x H x W x Cpad : rows = C,  cols = H*W, dst_pitch = Cpad
//   N x H x W x Cpad -> N x C x H x W : rows = H*W, cols = C,  src_pitch = Cpad
// ---------------------------------------------------------------------------------------------
__global__ void transpose16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                   int rows, int cols, long long src_pitch, long long dst_pitch,
                                   long long src_batch, long long dst_batch) {
  __shared__ uint16_t tile[32][33];
  const uint16_t* s = src + static_cast<long long>(blockIdx.z) * src_batch;
  uint16_t* d = dst + static_cast<long long>(blockIdx.z) * dst_batch;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < rows && c < cols) ? s[r * src_pitch + c] : static_cast<uint16_t>(0);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;  // dst row = c, dst column = r
    if (c < cols && r < dst_pitch) d[c * dst_pitch + r] = tile[threadIdx.x][i];
  }
}

// The same transpose moving 32-bit words: a thread turns a 2 x 2 block of elements (two words
// of two adjacent rows) into the two words of the transposed block, a 64 x 64 tile goes through
// shared memory so that both the reads and the writes are whole 128-byte lines.  Needs an even
// cols, even pitches and batch strides, and 4-byte aligned bases.
__global__ void transpose16_pairs_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                         int rows, int cols, long long src_pitch,
                                         long long dst_pitch, long long src_batch,
                                         long long dst_batch) {
  __shared__ uint32_t tile[64][33];
  const uint16_t* s = src + static_cast<long long>(blockIdx.z) * src_batch;
  uint16_t* d = dst + static_cast<long long>(blockIdx.z) * dst_batch;
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int tx = threadIdx.x;
  for (int br = threadIdx.y; br < 32; br += blockDim.y) {
    const int r = r0 + 2 * br, c = c0 + 2 * tx;
    uint32_t w0 = 0, w1 = 0;
    if (c < cols) {
      if (r < rows) w0 = *reinterpret_cast<const uint32_t*>(s + r * src_pitch + c);
      if (r + 1 < rows) w1 = *reinterpret_cast<const uint32_t*>(s + (r + 1) * src_pitch + c);
    }
    tile[2 * tx][br] = (w0 & 0xffffu) | (w1 << 16);            // column c:     rows r, r+1
    tile[2 * tx + 1][br] = (w0 >> 16) | (w1 & 0xffff0000u);    // column c + 1: rows r, r+1
  }
  __syncthreads();
  for (int dr = threadIdx.y; dr < 64; dr += blockDim.y) {
    const int c = c0 + dr, r = r0 + 2 * tx;
    if (c < cols && r < dst_pitch)
      *reinterpret_cast<uint32_t*>(d + c * dst_pitch + r) = tile[dr][tx];
  }
}

// The same transpose with 16-byte accesses and no shared memory: a thread loads an 8 x 8 block
// (one uint4 from each of 8 rows), transposes it in registers with byte permutes and stores 8
// uint4.  The 8 threads that share a row of blocks read (and the 8 that share a column write)
// one whole 128-byte line.  Needs cols, both pitches and both batch strides to be multiples of
// 8 and 16-byte aligned bases.
__global__ void __launch_bounds__(64)
transpose16_vec8_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int rows,
                        int cols, long long src_pitch, long long dst_pitch, long long src_batch,
                        long long dst_batch) {
  const uint16_t* s = src + static_cast<long long>(blockIdx.z) * src_batch;
  uint16_t* d = dst + static_cast<long long>(blockIdx.z) * dst_batch;
  const int c = blockIdx.x * 64 + (threadIdx.x & 7) * 8;   // first source column of the block
  const int r = blockIdx.y * 64 + (threadIdx.x >> 3) * 8;  // first source row of the block
  if (c >= cols || r >= dst_pitch) return;
  uint4 in[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    in[i] = r + i < rows ? *reinterpret_cast<const uint4*>(s + (r + i) * src_pitch + c)
                         : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {  // word column j holds source columns 2j and 2j + 1
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      w[i] = j == 0 ? in[i].x : j == 1 ? in[i].y : j == 2 ? in[i].z : in[i].w;
    uint4 lo, hi;  // destination rows c + 2j and c + 2j + 1: source rows r .. r + 7
    lo.x = __byte_perm(w[0], w[1], 0x5410); hi.x = __byte_perm(w[0], w[1], 0x7632);
    lo.y = __byte_perm(w[2], w[3], 0x5410); hi.y = __byte_perm(w[2], w[3], 0x7632);
    lo.z = __byte_perm(w[4], w[5], 0x5410); hi.z = __byte_perm(w[4], w[5], 0x7632);
    lo.w = __byte_perm(w[6], w[7], 0x5410); hi.w = __byte_perm(w[6], w[7], 0x7632);
    *reinterpret_cast<uint4*>(d + (c + 2 * j) * dst_pitch + r) = lo;
    *reinterpret_cast<uint4*>(d + (c + 2 * j + 1) * dst_pitch + r) = hi;
  }
}

int launch_transpose16(const void* src, void* dst, int batch, int rows, int cols,
                       long long src_pitch, long long dst_pitch, long long src_batch,
                       long long dst_batch, cudaStream_t stream) {
  const long long all = cols | src_pitch | dst_pitch | src_batch | dst_batch;
  const uintptr_t bases = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst);
  const bool vec8 = (all & 7) == 0 && (bases & 15u) == 0;
  const bool pairs = (all & 1) == 0 && (bases & 3u) == 0;
  const int edge = (vec8 || pairs) ? 64 : 32;
  // grid.y covers dst_pitch so that the zero padding of the last block of columns is written
  const int row_blocks = static_cast<int>((dst_pitch + edge - 1) / edge);
  const int col_blocks = (cols + edge - 1) / edge;
  if (row_blocks > 65535 || batch > 65535) {
    set_error("tensor too large to repack (%d row blocks, batch %d)", row_blocks, batch);
    return TNX_ERR_INVALID;
  }
  dim3 grid(col_blocks, row_blocks, batch), block(32, 8, 1);
  if (vec8)
    transpose16_vec8_kernel<<<grid, 64, 0, stream>>>(static_cast<const uint16_t*>(src),
                                                     static_cast<uint16_t*>(dst), rows, cols,
                                                     src_pitch, dst_pitch, src_batch, dst_batch);
  else if (pairs)
    transpose16_pairs_kernel<<<grid, block, 0, stream>>>(static_cast<const uint16_t*>(src),
                                                       static_cast<uint16_t*>(dst), rows, cols,
                                                       src_pitch, dst_pitch, src_batch, dst_batch);
  else
    transpose16_kernel<<<grid, block, 0, stream>>>(static_cast<const uint16_t*>(src),
                                                   static_cast<uint16_t*>(dst), rows, cols, src_pitch,
                                                   dst_pitch, src_batch, dst_batch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("repacking kernel launch failed: %s", cudaGetErrorString(e));
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

// Pads the channels of an N x H x W x C tensor to c_pitch (C not a multiple of 8).
__global__ void pad_channels16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                      long long pixels, int c, int c_pitch) {
  const long long total = pixels * c_pitch;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long px = i / c_pitch;
    const int ch = static_cast<int>(i - px * c_pitch);
    dst[i] = ch < c ? src[px * c + ch] : static_cast<uint16_t>(0);
  }
}

// The reverse: drops the padding channels.
__global__ void unpad_channels16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                        long long pixels, int c, int c_pitch) {
  const long long total = pixels * c;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long px = i / c;
    const int ch = static_cast<int>(i - px * c);
    dst[i] = src[px * c_pitch + ch];
  }
}

// Weights C_OUT x C x R x S -> C_OUT x (R*S) x (cblocks*64), zero beyond C: the K order of the
// implicit GEMM (tap-major, channels contiguous) with every tap starting on a 128-byte boundary.
// One thread writes 8 channels (16 bytes) of one (output channel, tap).
__global__ void pack_weights16_kernel(const uint16_t* __restrict__ w, uint16_t* __restrict__ out,
                                      int c_out, int c, int taps, int c_padded) {
  const int groups = c_padded / 8;
  const long long total = static_cast<long long>(c_out) * taps * groups;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int grp = static_cast<int>(i % groups);
    const long long rest = i / groups;
    const int tap = static_cast<int>(rest % taps);
    const long long co = rest / taps;
    const uint16_t* src = w + (co * c + grp * 8) * taps + tap;
    uint16_t v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      v[j] = grp * 8 + j < c ? src[static_cast<long long>(j) * taps] : static_cast<uint16_t>(0);
    uint4 q;
    q.x = v[0] | (static_cast<uint32_t>(v[1]) << 16);
    q.y = v[2] | (static_cast<uint32_t>(v[3]) << 16);
    q.z = v[4] | (static_cast<uint32_t>(v[5]) << 16);
    q.w = v[6] | (static_cast<uint32_t>(v[7]) << 16);
    *reinterpret_cast<uint4*>(out + i * 8) = q;
  }
}

// ---------------------------------------------------------------------------------------------
// Width folding for thin inputs.  With C channels padded to 64 per filter tap, a 3-channel 7x7
// stem would spend 21 of every 22 multiply-adds on zeros.  Instead the S taps of a filter row
// become channels: X'[n][h][wo][s*C + c] = X[n][c][h][wo*stride_w - pad_w + s*dil_w] (zero outside
// the image), and the convolution becomes an R x 1 one over X' with S*C channels, stride_w = 1 and
// no horizontal padding.  Applies when C <= 16 and S*C <= 64.
// ---------------------------------------------------------------------------------------------
__global__ void fold_width16_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out,
                                    int batch, int c, int h, int w, int w_out, int fw, int cf,
                                    int stride_w, int pad_w, int dil_w, long long sn, long long sc,
                                    long long sh, long long sw) {
  const long long total = static_cast<long long>(batch) * h * w_out * fw;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int s = static_cast<int>(i % fw);
    long long rest = i / fw;
    const int wo = static_cast<int>(rest % w_out);
    rest /= w_out;
    const int hh = static_cast<int>(rest % h);
    const long long n = rest / h;
    const int wi = wo * stride_w - pad_w + s * dil_w;
    const bool inside = wi >= 0 && wi < w;
    uint16_t* dst = out + ((n * h + hh) * w_out + wo) * cf + s * c;
    const uint16_t* src = x + n * sn + hh * sh + wi * sw;
    for (int ch = 0; ch < c; ++ch) dst[ch] = inside ? src[ch * sc] : static_cast<uint16_t>(0);
    if (s == fw - 1)
      for (int ch = fw * c; ch < cf; ++ch) out[((n * h + hh) * w_out + wo) * cf + ch] = 0;
  }
}

// Weights for the folded problem: C_OUT x R x 64 with K index s*C + c inside a filter row.
__global__ void pack_weights_folded16_kernel(const uint16_t* __restrict__ w,
                                             uint16_t* __restrict__ out, int c_out, int c, int fh,
                                             int fw) {
  const long long total = static_cast<long long>(c_out) * fh * 64;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int k = static_cast<int>(i % 64);
    const long long rest = i / 64;
    const int r = static_cast<int>(rest % fh);
    const long long co = rest / fh;
    const int s = k / c, ch = k - s * c;
    out[i] = s < fw ? w[((co * c + ch) * fh + r) * fw + s] : static_cast<uint16_t>(0);
  }
}

bool folds_width(const tnx_conv2d_problem& p) {
  if (getenv("TNX_CONV_NO_FOLD") != nullptr) return false;  // read every time: tests flip it
  return p.dtype != TNX_F32 && p.filter_w > 1 && p.c_in <= 16 && p.c_in * p.filter_w <= 64;
}

inline int conv_w_out(const tnx_conv2d_problem& p) {
  return (p.w_in + 2 * p.pad_w - p.dil_w * (p.filter_w - 1) - 1) / p.stride_w + 1;
}

// The problem the tcgen05 kernel is given after folding: N x H x W_OUT x (S*C padded to 8)
// input in the workspace, R x 1 filter, packed weights.
tnx_conv2d_problem folded_problem(const tnx_conv2d_problem& p) {
  tnx_conv2d_problem q = p;
  q.c_in = (p.c_in * p.filter_w + 7) / 8 * 8;
  q.w_in = conv_w_out(p);
  q.filter_w = 1;
  q.stride_w = 1;
  q.pad_w = 0;
  q.dil_w = 1;
  q.input_layout = TNX_LAYOUT_NHWC;
  q.weight_layout = TNX_WEIGHT_PACKED;
  return q;
}

inline long long align256ll(long long v) { return (v + 255) / 256 * 256; }

inline long long folded_input_bytes(const tnx_conv2d_problem& p) {
  return align256ll(static_cast<long long>(p.batch) * p.h_in * conv_w_out(p) *
                    ((p.c_in * p.filter_w + 7) / 8 * 8) * 2);
}

inline int grid_for(long long total);

// N x H_OUT x W_OUT x c_out_pitch (what the kernel wrote) -> the caller's output tensor.
int repack_output16(const tnx_conv2d_problem& p, const void* y, void* output, long long out_pixels,
                    int c_out_pitch, cudaStream_t stream);

inline int grid_for(long long total) {
  long long blocks = (total + 255) / 256;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

// ---------------------------------------------------------------------------------------------
// fp32 (and any layout): implicit GEMM on CUDA cores, 64 pixels x 64 output channels per block,
// K in steps of 16, 4 x 4 outputs per thread, operands and result addressed in place.
// ---------------------------------------------------------------------------------------------
struct DirectGeom {
  int batch, c_in, h_in, w_in, c_out, fh, fw, h_out, w_out;
  int sh, sw, ph, pw, dh, dw;
  long long in_sn, in_sc, in_sh, in_sw;      // element strides of the input
  long long out_sn, out_sc, out_sh, out_sw;  // element strides of the output
};

__global__ void __launch_bounds__(256)
conv2d_direct_f32_kernel(const DirectGeom g, const float* __restrict__ x, const float* __restrict__ w,
                         const float* __restrict__ bias, float* __restrict__ y) {
  __shared__ float xs[16][64 + 4];
  __shared__ float ws[16][64 + 4];
  const long long gemm_m = static_cast<long long>(g.batch) * g.h_out * g.w_out;
  const int gemm_k = g.c_in * g.fh * g.fw;
  const long long m0 = static_cast<long long>(blockIdx.x) * 64;
  const int n0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  const int taps = g.fh * g.fw;
  for (int k0 = 0; k0 < gemm_k; k0 += 16) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      const int kk = i >> 6, mm = i & 63;
      const int k = k0 + kk;
      const long long m = m0 + mm;
      float v = 0.f;
      if (k < gemm_k && m < gemm_m) {
        const int c = k / taps, tap = k - c * taps;
        const int r = tap / g.fw, s = tap - r * g.fw;
        const long long img = m / (g.h_out * g.w_out);
        const int rem = static_cast<int>(m - img * (g.h_out * g.w_out));
        const int ho = rem / g.w_out, wo = rem - ho * g.w_out;
        const int hi = ho * g.sh - g.ph + r * g.dh, wi = wo * g.sw - g.pw + s * g.dw;
        if (hi >= 0 && hi < g.h_in && wi >= 0 && wi < g.w_in)
          v = x[img * g.in_sn + c * g.in_sc + hi * g.in_sh + wi * g.in_sw];
      }
      xs[kk][mm] = v;
      const int n = n0 + mm;
      ws[kk][mm] = (k < gemm_k && n < g.c_out) ? w[static_cast<long long>(n) * gemm_k + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = xs[kk][ty * 4 + i];
        b[i] = ws[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long m = m0 + ty * 4 + i;
    if (m >= gemm_m) continue;
    const long long img = m / (g.h_out * g.w_out);
    const int rem = static_cast<int>(m - img * (g.h_out * g.w_out));
    const int ho = rem / g.w_out, wo = rem - ho * g.w_out;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.c_out) continue;
      const float v = acc[i][j] + (bias != nullptr ? bias[n] : 0.f);
      y[img * g.out_sn + n * g.out_sc + ho * g.out_sh + wo * g.out_sw] = v;
    }
  }
}

int repack_output16(const tnx_conv2d_problem& p, const void* y, void* output, long long out_pixels,
                    int c_out_pitch, cudaStream_t stream) {
  if (p.output_layout == TNX_LAYOUT_NCHW)
    return launch_transpose16(y, output, p.batch, static_cast<int>(out_pixels), p.c_out, c_out_pitch,
                              out_pixels, out_pixels * c_out_pitch, out_pixels * p.c_out, stream);
  const long long px = out_pixels * p.batch;
  unpad_channels16_kernel<<<grid_for(px * p.c_out), 256, 0, stream>>>(
      static_cast<const uint16_t*>(y), static_cast<uint16_t*>(output), px, p.c_out, c_out_pitch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("repacking kernel launch failed: %s", cudaGetErrorString(e));
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

int validate_conv(const tnx_conv2d_problem* p) {
  if (p == nullptr) {
    set_error("problem is NULL");
    return TNX_ERR_INVALID;
  }
  if (p->batch < 1 || p->c_in < 1 || p->h_in < 1 || p->w_in < 1 || p->c_out < 1 ||
      p->filter_h < 1 || p->filter_w < 1 || p->stride_h < 1 || p->stride_w < 1 || p->pad_h < 0 ||
      p->pad_w < 0 || p->dil_h < 1 || p->dil_w < 1) {
    set_error("invalid convolution geometry");
    return TNX_ERR_INVALID;
  }
  if (p->dtype != TNX_F16 && p->dtype != TNX_BF16 && p->dtype != TNX_F32) {
    set_error("unknown dtype %d", p->dtype);
    return TNX_ERR_INVALID;
  }
  if ((p->input_layout != TNX_LAYOUT_NCHW && p->input_layout != TNX_LAYOUT_NHWC) ||
      (p->output_layout != TNX_LAYOUT_NCHW && p->output_layout != TNX_LAYOUT_NHWC)) {
    set_error("unknown tensor layout");
    return TNX_ERR_INVALID;
  }
  const long long h_eff = static_cast<long long>(p->h_in) + 2LL * p->pad_h -
                          static_cast<long long>(p->dil_h) * (p->filter_h - 1) - 1;
  const long long w_eff = static_cast<long long>(p->w_in) + 2LL * p->pad_w -
                          static_cast<long long>(p->dil_w) * (p->filter_w - 1) - 1;
  if (h_eff < 0 || w_eff < 0) {
    set_error("the dilated filter is larger than the padded input");
    return TNX_ERR_INVALID;
  }
  if (p->weight_layout != TNX_WEIGHT_KCRS &&
      !(p->weight_layout == TNX_WEIGHT_PACKED && p->dtype != TNX_F32)) {
    set_error("weight_layout must be TNX_WEIGHT_KCRS, or TNX_WEIGHT_PACKED for fp16/bf16");
    return TNX_ERR_INVALID;
  }
  if (p->has_bias != 0 && p->has_bias != 1) {
    set_error("has_bias must be 0 or 1");
    return TNX_ERR_INVALID;
  }
  return TNX_OK;
}

}  // namespace

}  // namespace tnx

extern "C" int tnx_conv2d_query(const tnx_conv2d_problem* problem, const tnx_config* config,
                                tnx_conv2d_resources* out) {
  int rc = tnx::validate_conv(problem);
  if (rc != TNX_OK) return rc;
  if (out == nullptr) {
    tnx::set_error("out is NULL");
    return TNX_ERR_INVALID;
  }
  *out = tnx_conv2d_resources{};
  if (problem->dtype == TNX_F32) {
    out->kernel = TNX_KERNEL_STRIDED;
    out->h_out = (problem->h_in + 2 * problem->pad_h - problem->dil_h * (problem->filter_h - 1) - 1) /
                     problem->stride_h + 1;
    out->w_out = (problem->w_in + 2 * problem->pad_w - problem->dil_w * (problem->filter_w - 1) - 1) /
                     problem->stride_w + 1;
    const long long gemm_m = static_cast<long long>(problem->batch) * out->h_out * out->w_out;
    const long long blocks = (gemm_m + 63) / 64;
    if (blocks > 0x7fffffffLL || (problem->c_out + 63) / 64 > 65535) {
      tnx::set_error("convolution too large for the fp32 kernel's grid");
      return TNX_ERR_INVALID;
    }
    out->grid = static_cast<int32_t>(blocks);
    out->smem_bytes = 2 * 16 * 68 * 4;
    return TNX_OK;
  }
  tnx_config cfg = config ? *config : tnx_config{};
  tnx::ConvPlan plan;
  if (tnx::conv_is_batched_gemm(*problem)) return tnx::umma_conv1x1_query(*problem, &cfg, out);
  if (tnx::folds_width(*problem)) {
    const tnx_conv2d_problem q = tnx::folded_problem(*problem);
    rc = tnx::umma_conv_query(q, &cfg, out, &plan);
    out->workspace_bytes += tnx::folded_input_bytes(*problem);  // the folded input follows the plan's areas
    return rc;
  }
  return tnx::umma_conv_query(*problem, &cfg, out, &plan);
}

extern "C" int64_t tnx_conv2d_packed_weight_bytes(const tnx_conv2d_problem* problem) {
  if (tnx::validate_conv(problem) != TNX_OK || problem->dtype == TNX_F32) return 0;
  if (tnx::folds_width(*problem))
    return static_cast<int64_t>(problem->c_out) * problem->filter_h * 64 * 2;
  const int64_t c_padded = (problem->c_in + 63) / 64 * 64;
  return static_cast<int64_t>(problem->c_out) * problem->filter_h * problem->filter_w * c_padded * 2;
}

extern "C" int tnx_conv2d_pack_weights(const tnx_conv2d_problem* problem, const void* weight,
                                       void* packed, void* stream_ptr) {
  int rc = tnx::validate_conv(problem);
  if (rc != TNX_OK) return rc;
  if (problem->dtype == TNX_F32) {
    tnx::set_error("fp32 weights have no packed form");
    return TNX_ERR_INVALID;
  }
  if (weight == nullptr || packed == nullptr || (reinterpret_cast<uintptr_t>(packed) & 15u)) {
    tnx::set_error("weight and packed must not be NULL and packed must be 16-byte aligned");
    return TNX_ERR_INVALID;
  }
  if (tnx::folds_width(*problem)) {
    tnx::pack_weights_folded16_kernel<<<tnx::grid_for(static_cast<long long>(problem->c_out) *
                                                      problem->filter_h * 64),
                                        256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
        static_cast<const uint16_t*>(weight), static_cast<uint16_t*>(packed), problem->c_out,
        problem->c_in, problem->filter_h, problem->filter_w);
  } else {
    const int taps = problem->filter_h * problem->filter_w;
    const int c_padded = (problem->c_in + 63) / 64 * 64;
    const long long groups = static_cast<long long>(problem->c_out) * taps * (c_padded / 8);
    tnx::pack_weights16_kernel<<<tnx::grid_for(groups), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
        static_cast<const uint16_t*>(weight), static_cast<uint16_t*>(packed), problem->c_out,
        problem->c_in, taps, c_padded);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tnx::set_error("weight packing kernel launch failed: %s", cudaGetErrorString(e));
    return TNX_ERR_CUDA;
  }
  return TNX_OK;
}

extern "C" int tnx_conv2d_forward(const tnx_conv2d_problem* problem, const tnx_config* config,
                                  const void* input, const void* weight, const void* bias,
                                  void* output, void* workspace, size_t workspace_bytes,
                                  int32_t* status_word, void* stream_ptr) {
  int rc = tnx::validate_conv(problem);
  if (rc != TNX_OK) return rc;
  if (input == nullptr || weight == nullptr || output == nullptr ||
      (problem->has_bias && bias == nullptr)) {
    tnx::set_error("input, weight, output (and bias when has_bias is set) must not be NULL");
    return TNX_ERR_INVALID;
  }
  const tnx_conv2d_problem& p = *problem;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  tnx_conv2d_resources res;
  rc = tnx_conv2d_query(problem, config, &res);
  if (rc != TNX_OK) return rc;

  if (p.dtype == TNX_F32) {
    tnx::DirectGeom g;
    g.batch = p.batch; g.c_in = p.c_in; g.h_in = p.h_in; g.w_in = p.w_in; g.c_out = p.c_out;
    g.fh = p.filter_h; g.fw = p.filter_w; g.h_out = res.h_out; g.w_out = res.w_out;
    g.sh = p.stride_h; g.sw = p.stride_w; g.ph = p.pad_h; g.pw = p.pad_w;
    g.dh = p.dil_h; g.dw = p.dil_w;
    if (p.input_layout == TNX_LAYOUT_NCHW) {
      g.in_sw = 1; g.in_sh = p.w_in; g.in_sc = static_cast<long long>(p.h_in) * p.w_in;
      g.in_sn = g.in_sc * p.c_in;
    } else {
      g.in_sc = 1; g.in_sw = p.c_in; g.in_sh = static_cast<long long>(p.w_in) * p.c_in;
      g.in_sn = g.in_sh * p.h_in;
    }
    if (p.output_layout == TNX_LAYOUT_NCHW) {
      g.out_sw = 1; g.out_sh = res.w_out; g.out_sc = static_cast<long long>(res.h_out) * res.w_out;
      g.out_sn = g.out_sc * p.c_out;
    } else {
      g.out_sc = 1; g.out_sw = p.c_out; g.out_sh = static_cast<long long>(res.w_out) * p.c_out;
      g.out_sn = g.out_sh * res.h_out;
    }
    dim3 grid(res.grid, (p.c_out + 63) / 64, 1);
    tnx::conv2d_direct_f32_kernel<<<grid, 256, 0, stream>>>(
        g, static_cast<const float*>(input), static_cast<const float*>(weight),
        p.has_bias ? static_cast<const float*>(bias) : nullptr, static_cast<float*>(output));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      tnx::set_error("fp32 convolution kernel launch failed: %s", cudaGetErrorString(e));
      return TNX_ERR_CUDA;
    }
    return TNX_OK;
  }

  tnx_config cfg = config ? *config : tnx_config{};
  tnx::ConvPlan plan;
  if (tnx::conv_is_batched_gemm(p)) {  // 1 x 1 on NCHW tensors: one GEMM per image, nothing to repack
    rc = tnx::umma_conv1x1_query(p, &cfg, &res);
    if (rc != TNX_OK) return rc;
    return tnx::umma_conv1x1_launch(p, cfg, res, input, weight, bias, output, status_word, stream);
  }
  const bool fold = tnx::folds_width(p);
  const tnx_conv2d_problem folded = fold ? tnx::folded_problem(p) : p;
  rc = tnx::umma_conv_query(folded, &cfg, &res, &plan);
  if (rc != TNX_OK) return rc;
  const long long need = plan.workspace_bytes + (fold ? tnx::folded_input_bytes(p) : 0);
  if (need > 0 && (workspace == nullptr || workspace_bytes < static_cast<size_t>(need))) {
    tnx::set_error("convolution needs a workspace of %lld bytes (tnx_conv2d_query), got %zu", need,
                   workspace_bytes);
    return TNX_ERR_INVALID;
  }
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) {
    tnx::set_error("workspace must be 256-byte aligned");
    return TNX_ERR_INVALID;
  }
  char* ws = static_cast<char*>(workspace);
  const long long in_pixels = static_cast<long long>(p.h_in) * p.w_in;
  const long long out_pixels = static_cast<long long>(res.h_out) * res.w_out;

  if (fold) {
    // Thin input: the taps of a filter row become channels (see fold_width16_kernel), then the
    // same kernel runs an R x 1 convolution over the folded copy.
    uint16_t* xf = reinterpret_cast<uint16_t*>(ws + plan.workspace_bytes);
    long long sn, sc, sh, sw;
    if (p.input_layout == TNX_LAYOUT_NCHW) {
      sw = 1; sh = p.w_in; sc = in_pixels; sn = in_pixels * p.c_in;
    } else {
      sc = 1; sw = p.c_in; sh = static_cast<long long>(p.w_in) * p.c_in; sn = sh * p.h_in;
    }
    const long long threads = static_cast<long long>(p.batch) * p.h_in * res.w_out * p.filter_w;
    tnx::fold_width16_kernel<<<tnx::grid_for(threads), 256, 0, stream>>>(
        static_cast<const uint16_t*>(input), xf, p.batch, p.c_in, p.h_in, p.w_in, res.w_out,
        p.filter_w, folded.c_in, p.stride_w, p.pad_w, p.dil_w, sn, sc, sh, sw);
    const void* w_packed = weight;
    if (p.weight_layout != TNX_WEIGHT_PACKED) {
      tnx::pack_weights_folded16_kernel<<<tnx::grid_for(static_cast<long long>(p.c_out) * p.filter_h * 64),
                                          256, 0, stream>>>(
          static_cast<const uint16_t*>(weight), reinterpret_cast<uint16_t*>(ws + plan.off_weight),
          p.c_out, p.c_in, p.filter_h, p.filter_w);
      w_packed = ws + plan.off_weight;
    }
    cudaError_t fe = cudaGetLastError();
    if (fe != cudaSuccess) {
      tnx::set_error("folding kernel launch failed: %s", cudaGetErrorString(fe));
      return TNX_ERR_CUDA;
    }
    void* yf = plan.repack_output ? static_cast<void*>(ws + plan.off_output) : output;
    rc = tnx::umma_conv_launch(folded, cfg, res, plan, xf, w_packed, bias, yf, status_word, stream);
    if (rc != TNX_OK) return rc;
    if (plan.repack_output)
      return tnx::repack_output16(p, yf, output, out_pixels, plan.c_out_pitch, stream);
    return TNX_OK;
  }

  // 1. input as N x H x W x c_pitch
  const void* x = input;
  if (plan.repack_input) {
    void* dst = ws + plan.off_input;
    if (p.input_layout == TNX_LAYOUT_NCHW) {
      rc = tnx::launch_transpose16(input, dst, p.batch, p.c_in, static_cast<int>(in_pixels),
                                   in_pixels, plan.c_pitch, in_pixels * p.c_in,
                                   in_pixels * plan.c_pitch, stream);
      if (rc != TNX_OK) return rc;
    } else {
      const long long px = in_pixels * p.batch;
      tnx::pad_channels16_kernel<<<tnx::grid_for(px * plan.c_pitch), 256, 0, stream>>>(
          static_cast<const uint16_t*>(input), static_cast<uint16_t*>(dst), px, p.c_in, plan.c_pitch);
    }
    x = dst;
  }
  // 2. weights as C_OUT x (R*S) x padded channels
  const void* w_packed = weight;
  if (p.weight_layout != TNX_WEIGHT_PACKED) {
    const int taps = p.filter_h * p.filter_w;
    const int c_padded = plan.k_packed / taps;
    tnx::pack_weights16_kernel<<<tnx::grid_for(static_cast<long long>(p.c_out) * plan.k_packed / 8),
                                 256, 0, stream>>>(static_cast<const uint16_t*>(weight),
                                                   reinterpret_cast<uint16_t*>(ws + plan.off_weight),
                                                   p.c_out, p.c_in, taps, c_padded);
    w_packed = ws + plan.off_weight;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    tnx::set_error("repacking kernel launch failed: %s", cudaGetErrorString(e));
    return TNX_ERR_CUDA;
  }
  // 3. the implicit GEMM
  void* y = plan.repack_output ? static_cast<void*>(ws + plan.off_output) : output;
  rc = tnx::umma_conv_launch(p, cfg, res, plan, x, w_packed, bias, y, status_word, stream);
  if (rc != TNX_OK) return rc;
  // 4. output in the layout the caller wants
  if (plan.repack_output)
    return tnx::repack_output16(p, y, output, out_pixels, plan.c_out_pitch, stream);
  return TNX_OK;
}
