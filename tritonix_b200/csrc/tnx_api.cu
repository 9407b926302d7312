// extern "C" surface of libtritonix_b200.so: argument validation, kernel-family selection,
// error text.  No device memory is allocated or freed anywhere in this library.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "tnx_internal.h"

namespace tnx {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

namespace {

int validate_problem(const tnx_problem* p) {
  if (p == nullptr) {
    set_error("problem is NULL");
    return TNX_ERR_INVALID;
  }
  if (p->m < 0 || p->n < 0 || p->k < 0) {
    set_error("negative dimension (m=%d n=%d k=%d)", p->m, p->n, p->k);
    return TNX_ERR_INVALID;
  }
  if (p->dtype != TNX_F16 && p->dtype != TNX_BF16 && p->dtype != TNX_F32) {
    set_error("unknown dtype %d", p->dtype);
    return TNX_ERR_INVALID;
  }
  if (p->epilogue < TNX_EPI_NONE || p->epilogue > TNX_EPI_GLU_SIGMOID) {
    set_error("unknown epilogue %d", p->epilogue);
    return TNX_ERR_INVALID;
  }
  if (p->stride_am < 0 || p->stride_ak < 0 || p->stride_bk < 0 || p->stride_bn < 0 ||
      p->stride_cm < 0 || p->stride_cn < 0) {
    set_error("negative strides are not supported");
    return TNX_ERR_INVALID;
  }
  if (p->epilogue != TNX_EPI_NONE && (p->n % 2) != 0) {
    set_error("GLU epilogue needs an even number of interleaved columns, got n=%d", p->n);
    return TNX_ERR_INVALID;
  }
  return TNX_OK;
}

// Resolves which kernel family runs and what it needs.  *cfg receives the defaults.
int resolve(const tnx_problem* p, const tnx_config* config, tnx_config* cfg, tnx_resources* res) {
  int rc = validate_problem(p);
  if (rc != TNX_OK) return rc;
  if (config != nullptr)
    *cfg = *config;
  else
    memset(cfg, 0, sizeof(*cfg));
  memset(res, 0, sizeof(*res));
  if (cfg->kernel < TNX_KERNEL_AUTO || cfg->kernel > TNX_KERNEL_STRIDED) {
    set_error("unknown kernel family %d", cfg->kernel);
    return TNX_ERR_INVALID;
  }
  const char* why = nullptr;
  const bool eligible = umma_eligible(*p, &why);
  if (cfg->kernel == TNX_KERNEL_TCGEN05 && !eligible) {
    set_error("%s", why);
    return TNX_ERR_INVALID;
  }
  if (cfg->kernel == TNX_KERNEL_STRIDED || !eligible) return strided_query(*p, cfg, res);
  return umma_query(*p, cfg, res);
}

}  // namespace
}  // namespace tnx

extern "C" {

const char* tnx_version(void) { return "0.1.0"; }

const char* tnx_last_error(void) { return tnx::g_error; }

int tnx_sm_count(void) {
  int dev = 0, v = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) {
    tnx::set_error("no CUDA device: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return 0;
  }
  return v;
}

int tnx_gemm_query(const tnx_problem* problem, const tnx_config* config, tnx_resources* out) {
  if (out == nullptr) {
    tnx::set_error("out is NULL");
    return TNX_ERR_INVALID;
  }
  tnx_config cfg;
  return tnx::resolve(problem, config, &cfg, out);
}

int tnx_gemm(const tnx_problem* problem, const tnx_config* config, const void* a, const void* b,
             void* c, void* workspace, size_t workspace_bytes, const int32_t* tile_table,
             int32_t* status_word, void* stream) {
  tnx_config cfg;
  tnx_resources res;
  int rc = tnx::resolve(problem, config, &cfg, &res);
  if (rc != TNX_OK) return rc;
  const int n_out = problem->epilogue != TNX_EPI_NONE ? problem->n / 2 : problem->n;
  if (problem->m == 0 || n_out == 0) return TNX_OK;  // nothing to write
  if (a == nullptr || b == nullptr || c == nullptr) {
    if (!(problem->k == 0 && c != nullptr)) {
      tnx::set_error("NULL operand pointer");
      return TNX_ERR_INVALID;
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // TMA needs 16-byte aligned base addresses.  When the caller left the choice of kernel open, a
  // view that starts at an odd offset (e.g. big[:, 4:4 + K]) runs on the strided kernel, which
  // honours the reference's "any strides, any pointer" contract (tritonix/ops/matmul.py:50-55).
  const bool misaligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                            reinterpret_cast<uintptr_t>(c)) & 15u) != 0;
  if (res.kernel == TNX_KERNEL_TCGEN05 && misaligned &&
      (config == nullptr || config->kernel == TNX_KERNEL_AUTO)) {
    rc = tnx::strided_query(*problem, &cfg, &res);
    if (rc != TNX_OK) return rc;
  }
  if (res.kernel == TNX_KERNEL_STRIDED) return tnx::strided_launch(*problem, a, b, c, s);
  if (res.workspace_bytes > 0) {
    if (workspace == nullptr || workspace_bytes < static_cast<size_t>(res.workspace_bytes)) {
      tnx::set_error("split_k=%d needs a workspace of %lld bytes, got %zu", res.split_k,
                     static_cast<long long>(res.workspace_bytes), workspace ? workspace_bytes : 0);
      return TNX_ERR_INVALID;
    }
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) {
      tnx::set_error("workspace must be 256-byte aligned");
      return TNX_ERR_INVALID;
    }
  }
  if (cfg.tile_order == TNX_ORDER_TABLE && tile_table == nullptr) {
    tnx::set_error("tile_order=TABLE needs a tile table");
    return TNX_ERR_INVALID;
  }
  return tnx::umma_launch(*problem, cfg, res, a, b, c, workspace, tile_table, status_word, s);
}

int tnx_glu(const tnx_problem* problem, const tnx_config* config, int activation, const void* x,
            const void* w12, void* z, const int32_t* tile_table, int32_t* status_word,
            void* stream) {
  if (problem == nullptr) {
    tnx::set_error("problem is NULL");
    return TNX_ERR_INVALID;
  }
  if (activation < TNX_EPI_GLU_LINEAR || activation > TNX_EPI_GLU_SIGMOID) {
    tnx::set_error("activation must be TNX_EPI_GLU_LINEAR, _SILU or _SIGMOID, got %d", activation);
    return TNX_ERR_INVALID;
  }
  tnx_problem p = *problem;
  p.epilogue = activation;
  tnx_config cfg;
  if (config != nullptr)
    cfg = *config;
  else
    memset(&cfg, 0, sizeof(cfg));
  cfg.split_k = 1;
  return tnx_gemm(&p, &cfg, x, w12, z, nullptr, 0, tile_table, status_word, stream);
}

int tnx_read_status(int32_t* status_word, int32_t* code_out, void* stream) {
  if (status_word == nullptr) {
    tnx::set_error("status_word is NULL");
    return TNX_ERR_INVALID;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int32_t code = 0;
  cudaError_t e = cudaMemcpyAsync(&code, status_word, sizeof(code), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    tnx::set_error("reading the status word failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return TNX_ERR_CUDA;
  }
  if (code_out != nullptr) *code_out = code;
  if (code == 0) return TNX_OK;
  e = cudaMemsetAsync(status_word, 0, sizeof(code), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  tnx::set_error("a kernel gave up a bounded wait (code 0x%x: 0x101 TMA producer, 0x102 MMA "
                 "issuer, 0x103 epilogue)", code);
  return TNX_ERR_DEVICE;
}

}  // extern "C"
