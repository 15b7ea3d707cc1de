// Attention backward for callers that cannot allocate device memory.
//
// The backward of an online-softmax style OnlineFunc needs one fp32 scratch word per query row
// (delta = rowsum(O * dO), written by the pre-pass, read by the dQ and dK/dV passes).  The regular
// entry points take that buffer from the caller.  Some callers have nowhere to get it from: a host
// program that binds this C ABI directly and only owns the input and output buffers it was handed
// (an inference-server plugin, a foreign-language binding with no tensor library behind it), or a
// runtime whose memory plan is frozen once it starts serving, where cudaMalloc is forbidden because
// it synchronises the whole device.  For them the scratch lives here, in a fixed array that is part
// of the library image.
//
// The array is file-scope device memory: every GPU that loads this library holds
// AE_STATIC_DELTA_MAX_ROWS * 4 bytes of it until the process exits.  On the host side the array's
// name is only a handle (a host-side shadow symbol), not a device address, so the device address is
// looked up once per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/ae_b200.h"
#include "ae_internal.h"

// AE_STATIC_SCRATCH_MAX_ROWS (include/ae_b200.h) = 8 Mi rows = 32 MiB per GPU: four times B * Hq * Sq of the
// Llama-3.1-8B benchmark shape (8 * 32 * 8192).
#define AE_STATIC_DELTA_MAX_ROWS ((long long)AE_STATIC_SCRATCH_MAX_ROWS)

static __device__ __align__(256) float g_ae_delta_scratch[AE_STATIC_DELTA_MAX_ROWS];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device; resolved on the first call per device.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    char msg[256];
    snprintf(msg, sizeof msg, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    ae_internal_set_error(msg);
    return AE_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_ae_delta_scratch);
    if (e != cudaSuccess || !p) {
      char msg[256];
      snprintf(msg, sizeof msg, "cudaGetSymbolAddress(g_ae_delta_scratch) failed on device %d: %s", dev,
               cudaGetErrorString(e));
      ae_internal_set_error(msg);
      return AE_ERR_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return AE_OK;
}
}  // namespace

extern "C" {

int ae_launch_attn_bwd_static_scratch(void* prep_module, void* dq_module, void* dkv_module, const AeAttnBwdParams* p,
                                      void* stream) {
  if (!prep_module || !dq_module || !dkv_module || !p) {
    ae_internal_set_error("null module or parameter block");
    return AE_ERR_INVALID;
  }
  if (p->B <= 0 || p->Hq <= 0 || p->Sq <= 0) {
    char msg[160];
    snprintf(msg, sizeof msg, "B, Hq and Sq must be positive (got %d, %d, %d)", p->B, p->Hq, p->Sq);
    ae_internal_set_error(msg);
    return AE_ERR_INVALID;
  }
  const long long rows = (long long)p->B * p->Hq * p->Sq;
  if (rows > AE_STATIC_DELTA_MAX_ROWS) {
    char msg[256];
    snprintf(msg, sizeof msg,
             "B * Hq * Sq = %lld rows exceeds the built-in scratch of %lld rows; use ae_launch_attn_bwd_prep/_dq/_dkv "
             "with a caller-provided delta buffer",
             rows, (long long)AE_STATIC_DELTA_MAX_ROWS);
    ae_internal_set_error(msg);
    return AE_ERR_INVALID;
  }
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  AeAttnBwdParams q = *p;
  q.delta = scratch;  // every row the passes read is rewritten by the pre-pass first: nothing to clear
  if ((rc = ae_launch_attn_bwd_prep(prep_module, &q, stream))) return rc;
  if ((rc = ae_launch_attn_bwd_dq(dq_module, &q, stream))) return rc;
  return ae_launch_attn_bwd_dkv(dkv_module, &q, stream);
}

}  // extern "C"
