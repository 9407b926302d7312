// Declarations shared by the translation units of libtritonix_b200.so (not part of the ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tritonix_b200.h"

namespace tnx {

// Budgets of one B200 SM.
constexpr int kMaxDynamicSmem = 232448;  // 227 KiB opt-in dynamic shared memory per CTA
constexpr int kTmemColumns = 512;        // TMEM columns per SM (x 128 lanes x 32 bit)

// Split-K scratch layout: [counters: kCounterBytes][fp32 partial tiles].
constexpr int64_t kCounterBytes = 65536;
constexpr int kMaxCounterTiles = static_cast<int>(kCounterBytes / 4);

void set_error(const char* fmt, ...);

// Fills defaults into *cfg, validates, computes resources.  Returns a TNX_* status.
int umma_query(const tnx_problem& p, tnx_config* cfg, tnx_resources* out);
int umma_launch(const tnx_problem& p, const tnx_config& cfg, const tnx_resources& res,
                const void* a, const void* b, void* c, void* workspace, const int32_t* tile_table,
                int32_t* status_word, cudaStream_t stream);

// Helpers of the tcgen05 GEMM translation unit that other kernels of the library share.
// 2-D row-major tensor of 16-bit elements (TNX_F16 / TNX_BF16; TNX_F32 = 32-bit elements) ->
// tensor map with 128-byte swizzle: `cols` contiguous elements per row, `rows` rows,
// `pitch_elems` between rows, boxes of box_cols x box_rows (a box row must be 128 bytes; encoded
// maps are cached).  is_operand selects the L2 promotion used for loads.
int make_tmap_2d(CUtensorMap* out, const void* ptr, int dtype, int64_t cols, int64_t rows,
                 int64_t pitch_elems, int box_cols, int box_rows, bool is_operand);
int sm_count();                             // SMs of the current device (148 when none is visible)
unsigned long long bounded_wait_limit_ns(); // wall-clock limit of every device-side wait

// True when the operands can use the TMA/tcgen05 path (16-bit type, unit inner strides,
// 16-byte aligned row pitches).  Pointer alignment is checked at launch.
bool umma_eligible(const tnx_problem& p, const char** why);

// Convolution on the tcgen05 kernel.  The plan fixes the pixel rectangle a CTA tile covers and
// the layout of the caller's workspace (offsets in bytes, each a multiple of 256).
struct ConvPlan {
  int h_out, w_out;
  int tile_w, tile_h;        // output pixels per CTA tile
  int tiles_w, tiles_h;      // CTA tiles per image
  int row_tiles;             // batch * tiles_h * tiles_w
  int c_pitch;               // channels per pixel of the N x H x W x C input the kernel reads
  int cblocks;               // 64-channel blocks per filter tap
  int k_packed;              // taps * cblocks * 64: row length of the packed weights
  int c_out_pitch;           // channels per pixel of the N x H x W x C output the kernel writes
  bool repack_input, repack_output;
  bool im2col;               // tiles are 128 consecutive pixels fetched with im2col-mode boxes
  bool halo;                 // tiles are full output rows (plus the filter's halo columns); a stage is
                             // one channel block's input patch + its weights for all taps
  int patch_h;               // halo: input rows per patch = tile_h + (filter_h - 1) * dil_h
  int patch_rows;            // halo: shared-memory rows per patch (multiple of 8)
  int64_t off_input, off_weight, off_output, workspace_bytes;
};
int umma_conv_query(const tnx_conv2d_problem& p, tnx_config* cfg, tnx_conv2d_resources* out,
                    ConvPlan* plan);
// x: N x H x W x c_pitch, w: c_out x k_packed, y: N x h_out x w_out x c_out_pitch.
int umma_conv_launch(const tnx_conv2d_problem& p, const tnx_config& cfg,
                     const tnx_conv2d_resources& res, const ConvPlan& plan, const void* x,
                     const void* w, const void* bias, void* y, int32_t* status_word,
                     cudaStream_t stream);

// A 1 x 1, stride-1, unpadded convolution over N x C x H x W tensors is one GEMM per image with
// no repacking at all: out_n (C_OUT x HW) = W (C_OUT x C) . x_n (C x HW).  The kernel runs the
// batch in one launch (3-D tensor maps over x and out).
bool conv_is_batched_gemm(const tnx_conv2d_problem& p);
int umma_conv1x1_query(const tnx_conv2d_problem& p, tnx_config* cfg, tnx_conv2d_resources* out);
int umma_conv1x1_launch(const tnx_conv2d_problem& p, const tnx_config& cfg,
                        const tnx_conv2d_resources& res, const void* x, const void* w,
                        const void* bias, void* y, int32_t* status_word, cudaStream_t stream);

int strided_query(const tnx_problem& p, tnx_config* cfg, tnx_resources* out);
int strided_launch(const tnx_problem& p, const void* a, const void* b, void* c,
                   cudaStream_t stream);

}  // namespace tnx
