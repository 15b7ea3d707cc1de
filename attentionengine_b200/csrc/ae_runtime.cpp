// Host side of libae_b200.so: NVRTC compile, cubin modules, TMA descriptors, launches.
// libcuda and libnvrtc are opened lazily with dlopen so that the library loads (and
// compiles kernels) on a machine without a GPU driver.
#include <cuda.h>
#include <dlfcn.h>
#include <nvrtc.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/ae_b200.h"
#include "kernels/ae_args.h"
#include "ae_internal.h"

namespace {

thread_local std::string g_last_error;

void set_error(const std::string& s) { g_last_error = s; }

// ------------------------------------------------------------------ driver symbols
struct Driver {
  void* lib = nullptr;
  CUresult (*cuInit)(unsigned) = nullptr;
  CUresult (*cuCtxGetCurrent)(CUcontext*) = nullptr;
  CUresult (*cuCtxSetCurrent)(CUcontext) = nullptr;
  CUresult (*cuCtxPushCurrent)(CUcontext) = nullptr;
  CUresult (*cuCtxPopCurrent)(CUcontext*) = nullptr;
  CUresult (*cuDeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*cuDevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
  CUresult (*cuModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*cuModuleUnload)(CUmodule) = nullptr;
  CUresult (*cuModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*cuFuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*cuFuncGetAttribute)(int*, CUfunction_attribute, CUfunction) = nullptr;
  CUresult (*cuLaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             CUstream, void**, void**) = nullptr;
  CUresult (*cuGetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*cuMemsetD32Async)(CUdeviceptr, unsigned, size_t, CUstream) = nullptr;
  CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
  bool ok = false;
};

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!d.lib) d.lib = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
    if (!d.lib) return;
#define AE_SYM(name, sym)                                 \
  d.name = (decltype(d.name))dlsym(d.lib, sym);           \
  if (!d.name) return;
    AE_SYM(cuInit, "cuInit")
    AE_SYM(cuCtxGetCurrent, "cuCtxGetCurrent")
    AE_SYM(cuCtxSetCurrent, "cuCtxSetCurrent")
    AE_SYM(cuCtxPushCurrent, "cuCtxPushCurrent_v2")
    AE_SYM(cuCtxPopCurrent, "cuCtxPopCurrent_v2")
    AE_SYM(cuDeviceGet, "cuDeviceGet")
    AE_SYM(cuDevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain")
    AE_SYM(cuModuleLoadData, "cuModuleLoadData")
    AE_SYM(cuModuleUnload, "cuModuleUnload")
    AE_SYM(cuModuleGetFunction, "cuModuleGetFunction")
    AE_SYM(cuFuncSetAttribute, "cuFuncSetAttribute")
    AE_SYM(cuFuncGetAttribute, "cuFuncGetAttribute")
    AE_SYM(cuLaunchKernel, "cuLaunchKernel")
    AE_SYM(cuGetErrorString, "cuGetErrorString")
    AE_SYM(cuMemsetD32Async, "cuMemsetD32Async")
    AE_SYM(cuTensorMapEncodeTiled, "cuTensorMapEncodeTiled")
#undef AE_SYM
    d.ok = (d.cuInit(0) == CUDA_SUCCESS);
  });
  return d;
}

int cu_fail(CUresult r, const char* what) {
  const char* s = nullptr;
  Driver& d = driver();
  if (d.cuGetErrorString) d.cuGetErrorString(r, &s);
  char buf[256];
  snprintf(buf, sizeof buf, "%s failed: %s (%d)", what, s ? s : "?", (int)r);
  set_error(buf);
  return AE_ERR_CUDA;
}
#define AE_CU(call)                                   \
  do {                                                \
    CUresult r_ = (call);                             \
    if (r_ != CUDA_SUCCESS) return cu_fail(r_, #call); \
  } while (0)

// ------------------------------------------------------------------ NVRTC symbols
struct Nvrtc {
  void* lib = nullptr;
  nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*,
                               const char* const*) = nullptr;
  nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
  nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
  nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
  nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
  const char* (*GetErrorString)(nvrtcResult) = nullptr;
  bool ok = false;
};

Nvrtc& nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12"};
    for (const char* nm : names) {
      n.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
      if (n.lib) break;
    }
    if (!n.lib) return;
#define AE_SYM(name, sym)                        \
  n.name = (decltype(n.name))dlsym(n.lib, sym);  \
  if (!n.name) return;
    AE_SYM(CreateProgram, "nvrtcCreateProgram")
    AE_SYM(CompileProgram, "nvrtcCompileProgram")
    AE_SYM(GetCUBINSize, "nvrtcGetCUBINSize")
    AE_SYM(GetCUBIN, "nvrtcGetCUBIN")
    AE_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
    AE_SYM(GetProgramLog, "nvrtcGetProgramLog")
    AE_SYM(DestroyProgram, "nvrtcDestroyProgram")
    AE_SYM(GetErrorString, "nvrtcGetErrorString")
#undef AE_SYM
    n.ok = true;
  });
  return n;
}

// ------------------------------------------------------------------ module
// A cubin is loaded once per CUDA context it is launched in (one context per device under the runtime API): an engine
// first used on one GPU and later given tensors of another gets that GPU's own function handle.
struct Loaded {
  CUcontext ctx = nullptr;
  CUmodule mod = nullptr;
  CUfunction fn = nullptr;
};
struct Module {
  std::vector<char> cubin;
  std::string kernel;
  AeKernelConfig cfg{};
  std::mutex mu;
  std::vector<Loaded> loaded;
};

// function handle of the last ensure_loaded() of this thread: launch() follows it directly
thread_local CUfunction g_fn = nullptr;

int ensure_context(CUcontext* out) {
  Driver& d = driver();
  if (!d.ok) {
    set_error("libcuda.so.1 not available or cuInit failed");
    return AE_ERR_NO_DRIVER;
  }
  CUcontext ctx = nullptr;
  AE_CU(d.cuCtxGetCurrent(&ctx));
  if (!ctx) {
    CUdevice dev;
    AE_CU(d.cuDeviceGet(&dev, 0));
    AE_CU(d.cuDevicePrimaryCtxRetain(&ctx, dev));
    AE_CU(d.cuCtxSetCurrent(ctx));
  }
  *out = ctx;
  return AE_OK;
}

int ensure_loaded(Module* m) {
  CUcontext ctx = nullptr;
  int rc = ensure_context(&ctx);
  if (rc) return rc;
  std::lock_guard<std::mutex> lk(m->mu);
  for (const Loaded& l : m->loaded)
    if (l.ctx == ctx) {
      g_fn = l.fn;
      return AE_OK;
    }
  Driver& d = driver();
  Loaded l;
  l.ctx = ctx;
  AE_CU(d.cuModuleLoadData(&l.mod, m->cubin.data()));
  AE_CU(d.cuModuleGetFunction(&l.fn, l.mod, m->kernel.c_str()));
  if (m->cfg.smem_bytes > 48 * 1024) {
    AE_CU(d.cuFuncSetAttribute(l.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, m->cfg.smem_bytes));
    // the largest shared-memory carve-out, so that kernels sized for two CTAs per SM (about 100 KB each) get both
    AE_CU(d.cuFuncSetAttribute(l.fn, CU_FUNC_ATTRIBUTE_PREFERRED_SHARED_MEMORY_CARVEOUT, CU_SHAREDMEM_CARVEOUT_MAX_SHARED));
  }
  m->loaded.push_back(l);
  g_fn = l.fn;
  return AE_OK;
}

int launch(Module* m, unsigned gx, unsigned gy, unsigned gz, void* args, void* stream) {
  Driver& d = driver();
  void* params[] = {args};
  AE_CU(d.cuLaunchKernel(g_fn, gx, gy, gz, (unsigned)m->cfg.threads, 1, 1, (unsigned)m->cfg.smem_bytes,
                         (CUstream)stream, params, nullptr));
  return AE_OK;
}

// Tensor map over a [B, S, H, D] tensor (element strides sb, ss, sh; d contiguous) seen as
// (d, h, s, b) with a box of {64, 1, rows, 1} and 128-byte swizzle: one box is a `rows` x 128 B
// tile in the K-major (for Q/K) or MN-major (for V) layout the UMMA descriptors expect.
int make_bshd_map(AeTmaDesc* out, const void* base, int dtype, int64_t B, int64_t S, int64_t H, int64_t D,
                  const int64_t st[3], int rows) {
  Driver& d = driver();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_error("tensor base address must be 16-byte aligned");
    return AE_ERR_INVALID;
  }
  for (int i = 0; i < 3; ++i)
    if ((st[i] * 2) % 16 != 0 && !((i == 0 && B == 1))) {
      set_error("tensor strides must be multiples of 8 elements");
      return AE_ERR_INVALID;
    }
  // dimension order (d, s, h, b): the rows of a box are the second dimension
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)st[1] * 2, (cuuint64_t)st[2] * 2, (cuuint64_t)(B == 1 ? S * st[1] : st[0]) * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = dtype == AE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  AE_CU(d.cuTensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(out), dt, 4, const_cast<void*>(base), dims, strides,
                                 box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return AE_OK;
}

int make_2d_map(AeTmaDesc* out, const void* base, int dtype, int64_t rows, int64_t cols, int box_rows) {
  Driver& d = driver();
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = dtype == AE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  AE_CU(d.cuTensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(out), dt, 2, const_cast<void*>(base), dims, strides,
                                 box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return AE_OK;
}

int check_attn_common(const Module* m, int kind, int B, int Hq, int Hkv, int Sq, int Skv) {
  if (m->cfg.kind != kind) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || Hq % Hkv != 0) {
    set_error("bad attention shape");
    return AE_ERR_INVALID;
  }
  if (m->cfg.head_dim % 64 || m->cfg.head_dim_v % 64) {
    set_error("head dims must be multiples of 64");
    return AE_ERR_INVALID;
  }
  return AE_OK;
}

}  // namespace

void ae_internal_set_error(const char* msg) { g_last_error = msg ? msg : ""; }

extern "C" {

const char* ae_strerror(int code) {
  switch (code) {
    case AE_OK: return "ok";
    case AE_ERR_INVALID: return "invalid argument";
    case AE_ERR_COMPILE: return "kernel compilation failed";
    case AE_ERR_NO_NVRTC: return "libnvrtc not available";
    case AE_ERR_NO_DRIVER: return "CUDA driver not available";
    case AE_ERR_CUDA: return "CUDA driver call failed";
    case AE_ERR_UNSUPPORTED: return "unsupported kernel kind for this entry point";
    default: return "unknown error";
  }
}

const char* ae_last_error(void) { return g_last_error.c_str(); }

int ae_compile(const char* cuda_src, const char* kernel_name, const char* arch, const char** opts, int nopts,
               const AeKernelConfig* cfg, void** out_module, char* log, size_t log_cap) {
  if (!cuda_src || !kernel_name || !cfg || !out_module) return AE_ERR_INVALID;
  if (log && log_cap) log[0] = 0;
  Nvrtc& n = nvrtc();
  if (!n.ok) {
    set_error("libnvrtc.so.12 not found");
    return AE_ERR_NO_NVRTC;
  }
  nvrtcProgram prog;
  nvrtcResult r = n.CreateProgram(&prog, cuda_src, "ae_kernel.cu", 0, nullptr, nullptr);
  if (r != NVRTC_SUCCESS) {
    set_error(n.GetErrorString(r));
    return AE_ERR_COMPILE;
  }
  std::vector<std::string> o;
  o.push_back(std::string("--gpu-architecture=") + (arch ? arch : "sm_100a"));
  o.push_back("--std=c++17");
  o.push_back("-lineinfo");
  o.push_back("-default-device");  // generic lambdas inside kernels are device code
  for (int i = 0; i < nopts; ++i) o.push_back(opts[i]);
  std::vector<const char*> oc;
  for (auto& s : o) oc.push_back(s.c_str());
  r = n.CompileProgram(prog, (int)oc.size(), oc.data());
  size_t ls = 0;
  n.GetProgramLogSize(prog, &ls);
  if (ls > 1) {
    std::vector<char> lb(ls + 1, 0);
    n.GetProgramLog(prog, lb.data());
    if (log && log_cap) {
      size_t c = ls < log_cap - 1 ? ls : log_cap - 1;
      memcpy(log, lb.data(), c);
      log[c] = 0;
    }
    if (r != NVRTC_SUCCESS) set_error(std::string(lb.data(), ls < 2000 ? ls : 2000));
  }
  if (r != NVRTC_SUCCESS) {
    n.DestroyProgram(&prog);
    return AE_ERR_COMPILE;
  }
  size_t cs = 0;
  n.GetCUBINSize(prog, &cs);
  Module* m = new Module();
  m->cubin.resize(cs);
  n.GetCUBIN(prog, m->cubin.data());
  n.DestroyProgram(&prog);
  m->kernel = kernel_name;
  m->cfg = *cfg;
  *out_module = m;
  return AE_OK;
}

int ae_module_from_cubin(const void* cubin, size_t size, const char* kernel_name, const AeKernelConfig* cfg,
                         void** out_module) {
  if (!cubin || !size || !kernel_name || !cfg || !out_module) return AE_ERR_INVALID;
  Module* m = new Module();
  m->cubin.assign((const char*)cubin, (const char*)cubin + size);
  m->kernel = kernel_name;
  m->cfg = *cfg;
  *out_module = m;
  return AE_OK;
}

int ae_module_cubin(void* module, const void** data, size_t* size) {
  if (!module || !data || !size) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  *data = m->cubin.data();
  *size = m->cubin.size();
  return AE_OK;
}

int ae_query(void* module, AeKernelInfo* info) {
  if (!module || !info) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  int rc = ensure_loaded(m);
  if (rc) return rc;
  Driver& d = driver();
  AE_CU(d.cuFuncGetAttribute(&info->num_regs, CU_FUNC_ATTRIBUTE_NUM_REGS, g_fn));
  AE_CU(d.cuFuncGetAttribute(&info->static_smem_bytes, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, g_fn));
  AE_CU(d.cuFuncGetAttribute(&info->max_dynamic_smem_bytes, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, g_fn));
  AE_CU(d.cuFuncGetAttribute(&info->local_bytes, CU_FUNC_ATTRIBUTE_LOCAL_SIZE_BYTES, g_fn));
  AE_CU(d.cuFuncGetAttribute(&info->max_threads, CU_FUNC_ATTRIBUTE_MAX_THREADS_PER_BLOCK, g_fn));
  return AE_OK;
}

void ae_release(void* module) {
  if (!module) return;
  Module* m = (Module*)module;
  Driver& d = driver();
  for (const Loaded& l : m->loaded) {  // a module is unloaded with its own context current
    if (d.cuCtxPushCurrent(l.ctx) != CUDA_SUCCESS) continue;
    d.cuModuleUnload(l.mod);
    CUcontext popped = nullptr;
    d.cuCtxPopCurrent(&popped);
  }
  delete m;
}

int ae_launch_probe(void* module, const void* a, const void* b, const void* p, float* d_out, int mode,
                    uint32_t* status, void* stream) {
  if (!module || !b || !d_out) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  if (m->cfg.kind != AE_KIND_PROBE) return AE_ERR_UNSUPPORTED;
  int rc = ensure_loaded(m);
  if (rc) return rc;
  AeProbeArgs args;
  memset(&args, 0, sizeof args);
  if (mode == 0) {
    if (!a) return AE_ERR_INVALID;
    rc = make_2d_map(&args.tm_a, a, m->cfg.dtype, 128, 128, 128);
    if (rc) return rc;
  } else if (!p) {
    return AE_ERR_INVALID;
  }
  rc = make_2d_map(&args.tm_b, b, m->cfg.dtype, 128, 128, 128);
  if (rc) return rc;
  args.p = p;
  args.d = d_out;
  if (mode != 0 && mode != 1) return AE_ERR_INVALID;
  args.mode = mode;
  args.status = status;
  return launch(m, 1, 1, 1, &args, stream);
}

int ae_launch_attn_fwd(void* module, const AeAttnParams* p, void* stream) {
  if (!module || !p || !p->q || !p->k || !p->v || !p->o) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  // the forward over CTA pairs takes the same parameter block; its K tiles are loaded as two 64-row halves
  const bool pair = m->cfg.kind == AE_KIND_ATTN_FWD_PAIR;
  int rc = check_attn_common(m, pair ? AE_KIND_ATTN_FWD_PAIR : AE_KIND_ATTN_FWD, p->B, p->Hq, p->Hkv, p->Sq, p->Skv);
  if (rc) return rc;
  if (pair && (m->cfg.mask_mode == 2 || m->cfg.head_dim_v != 128 || (m->cfg.head_dim != 64 && m->cfg.head_dim != 128))) {
    set_error("the pair forward takes mask modes 0, 1, 3, value head dim 128 and head dim 64 or 128");
    return AE_ERR_INVALID;
  }
  if (m->cfg.mask_mode == 2 && (!p->block_count || !p->block_index)) {
    set_error("block lists required for mask_mode 2");
    return AE_ERR_INVALID;
  }
  if (m->cfg.mask_mode == 2 && (p->Skv + 127) / 128 > 2048) {
    set_error("block lists cover at most 2048 kv tiles (262144 keys)");
    return AE_ERR_INVALID;
  }
  rc = ensure_loaded(m);
  if (rc) return rc;
  AeAttnFwdArgs args;
  memset(&args, 0, sizeof args);
  const int D = m->cfg.head_dim, DV = m->cfg.head_dim_v;
  rc = make_bshd_map(&args.tm_q, p->q, m->cfg.dtype, p->B, p->Sq, p->Hq, D, p->q_stride, 128);
  if (rc) return rc;
  rc = make_bshd_map(&args.tm_k, p->k, m->cfg.dtype, p->B, p->Skv, p->Hkv, D, p->k_stride, pair ? 64 : 128);
  if (rc) return rc;
  rc = make_bshd_map(&args.tm_v, p->v, m->cfg.dtype, p->B, p->Skv, p->Hkv, DV, p->v_stride, 128);
  if (rc) return rc;
  args.o = p->o;
  args.o_sb = p->o_stride[0];
  args.o_ss = p->o_stride[1];
  args.o_sh = p->o_stride[2];
  if ((reinterpret_cast<uintptr_t>(p->o) & 15) || (args.o_ss % 8) || (args.o_sh % 8) || (args.o_sb % 8)) {
    set_error("output must be 16-byte aligned with strides that are multiples of 8 elements");
    return AE_ERR_INVALID;
  }
  for (int i = 0; i < AE_MAX_FINAL; ++i) args.final_rs[i] = p->final_rowscales[i];
  for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
    args.custom[i] = p->custom[i];
    for (int k = 0; k < 4; ++k) args.custom_st[i][k] = p->custom_stride[i][k];
  }
  args.blk_cnt = p->block_count;
  args.blk_idx = p->block_index;
  args.B = p->B;
  args.Hq = p->Hq;
  args.Hkv = p->Hkv;
  args.Sq = p->Sq;
  args.Skv = p->Skv;
  args.n_qt = (p->Sq + 127) / 128;
  args.n_kt = (p->Skv + 127) / 128;
  args.status = p->status;
  // single-CTA kernel: two q tiles per CTA; pair kernel: one per CTA, two per cluster (of two CTAs along x)
  const unsigned gx = pair ? 2u * (unsigned)((args.n_qt + 1) / 2) : (unsigned)((args.n_qt + 1) / 2);
  return launch(m, gx, (unsigned)p->Hq, (unsigned)p->B, &args, stream);
}

static int fill_bwd_args(Module* m, const AeAttnBwdParams* p, AeAttnBwdArgs* a, int q_rows, int kv_rows) {
  memset(a, 0, sizeof *a);
  const int D = m->cfg.head_dim, DV = m->cfg.head_dim_v;
  int rc;
  if ((rc = make_bshd_map(&a->tm_q, p->q, m->cfg.dtype, p->B, p->Sq, p->Hq, D, p->q_stride, q_rows))) return rc;
  if ((rc = make_bshd_map(&a->tm_do, p->d_o, m->cfg.dtype, p->B, p->Sq, p->Hq, DV, p->do_stride, q_rows))) return rc;
  if ((rc = make_bshd_map(&a->tm_k, p->k, m->cfg.dtype, p->B, p->Skv, p->Hkv, D, p->k_stride, kv_rows))) return rc;
  if ((rc = make_bshd_map(&a->tm_v, p->v, m->cfg.dtype, p->B, p->Skv, p->Hkv, DV, p->v_stride, kv_rows))) return rc;
  a->dq = p->dq;
  a->dk = p->dk;
  a->dv = p->dv;
  a->dq_sb = p->dq_stride[0]; a->dq_ss = p->dq_stride[1]; a->dq_sh = p->dq_stride[2];
  a->dk_sb = p->dk_stride[0]; a->dk_ss = p->dk_stride[1]; a->dk_sh = p->dk_stride[2];
  a->dv_sb = p->dv_stride[0]; a->dv_ss = p->dv_stride[1]; a->dv_sh = p->dv_stride[2];
  const void* outs[3] = {p->dq, p->dk, p->dv};
  const int64_t* sts[3] = {p->dq_stride, p->dk_stride, p->dv_stride};
  for (int i = 0; i < 3; ++i) {
    if (!outs[i]) continue;
    if ((reinterpret_cast<uintptr_t>(outs[i]) & 15) || sts[i][0] % 8 || sts[i][1] % 8 || sts[i][2] % 8) {
      set_error("gradient outputs must be 16-byte aligned with strides that are multiples of 8 elements");
      return AE_ERR_INVALID;
    }
  }
  for (int i = 0; i < AE_MAX_FINAL; ++i) a->final_rs[i] = p->final_rowscales[i];
  a->delta = p->delta;
  for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
    a->custom[i] = p->custom[i];
    for (int k = 0; k < 4; ++k) a->custom_st[i][k] = p->custom_stride[i][k];
  }
  a->blk_cnt = p->block_count;
  a->blk_idx = p->block_index;
  a->blkT_cnt = p->block_count_t;
  a->blkT_idx = p->block_index_t;
  a->B = p->B; a->Hq = p->Hq; a->Hkv = p->Hkv; a->Sq = p->Sq; a->Skv = p->Skv;
  a->n_qt = (p->Sq + 127) / 128;
  a->n_kt = (p->Skv + 127) / 128;
  a->status = p->status;
  return AE_OK;
}

int ae_launch_attn_bwd_prep(void* module, const AeAttnBwdParams* p, void* stream) {
  if (!module || !p || !p->o || !p->d_o || !p->delta) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  int rc = check_attn_common(m, AE_KIND_ATTN_BWD_PREP, p->B, p->Hq, p->Hkv, p->Sq, p->Skv);
  if (rc) return rc;
  rc = ensure_loaded(m);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(p->o) & 15) || (reinterpret_cast<uintptr_t>(p->d_o) & 15)) {
    set_error("o / dO must be 16-byte aligned");
    return AE_ERR_INVALID;
  }
  AeAttnBwdPrepArgs a;
  memset(&a, 0, sizeof a);
  a.o = p->o;
  a.d_o = p->d_o;
  a.delta = p->delta;
  a.o_sb = p->o_stride[0]; a.o_ss = p->o_stride[1]; a.o_sh = p->o_stride[2];
  a.do_sb = p->do_stride[0]; a.do_ss = p->do_stride[1]; a.do_sh = p->do_stride[2];
  if (a.o_sb % 8 || a.o_ss % 8 || a.o_sh % 8 || a.do_sb % 8 || a.do_ss % 8 || a.do_sh % 8) {
    set_error("o / dO strides must be multiples of 8 elements");
    return AE_ERR_INVALID;
  }
  a.B = p->B; a.Hq = p->Hq; a.Sq = p->Sq; a.DV = m->cfg.head_dim_v;
  // 16 bytes per lane, four rows per lane group and iteration; the CTAs stride over the rest
  const int64_t rows = (int64_t)p->B * p->Sq * p->Hq;
  const int64_t rows_per_cta = 8 * (32 / (m->cfg.head_dim_v / 8)) * 4;
  int64_t blocks = (rows + rows_per_cta - 1) / rows_per_cta;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch(m, (unsigned)blocks, 1, 1, &a, stream);
}

int ae_launch_attn_bwd_dq(void* module, const AeAttnBwdParams* p, void* stream) {
  if (!module || !p || !p->q || !p->k || !p->v || !p->d_o || !p->dq) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  int rc = check_attn_common(m, AE_KIND_ATTN_BWD_DQ, p->B, p->Hq, p->Hkv, p->Sq, p->Skv);
  if (rc) return rc;
  if (m->cfg.mask_mode == 2 && (!p->block_count || !p->block_index)) {
    set_error("block lists required for mask_mode 2");
    return AE_ERR_INVALID;
  }
  const int bn = m->cfg.reserved[0];
  if (bn != 64 && bn != 128) {
    set_error("backward tile (reserved[0]) must be 64 or 128");
    return AE_ERR_INVALID;
  }
  rc = ensure_loaded(m);
  if (rc) return rc;
  AeAttnBwdArgs a;
  rc = fill_bwd_args(m, p, &a, 128, bn);
  if (rc) return rc;
  return launch(m, (unsigned)a.n_qt, (unsigned)p->Hq, (unsigned)p->B, &a, stream);
}

int ae_launch_attn_bwd_dkv(void* module, const AeAttnBwdParams* p, void* stream) {
  if (!module || !p || !p->q || !p->k || !p->v || !p->d_o || !p->dk || !p->dv) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  int rc = check_attn_common(m, AE_KIND_ATTN_BWD_DKV, p->B, p->Hq, p->Hkv, p->Sq, p->Skv);
  if (rc) return rc;
  if (m->cfg.mask_mode == 2 && (!p->block_count_t || !p->block_index_t)) {
    set_error("transposed block lists required for mask_mode 2");
    return AE_ERR_INVALID;
  }
  const int bn = m->cfg.reserved[0];
  if (bn != 64 && bn != 128) {
    set_error("backward tile (reserved[0]) must be 64 or 128");
    return AE_ERR_INVALID;
  }
  rc = ensure_loaded(m);
  if (rc) return rc;
  AeAttnBwdArgs a;
  rc = fill_bwd_args(m, p, &a, bn, 128);
  if (rc) return rc;
  return launch(m, (unsigned)a.n_kt, (unsigned)p->Hkv, (unsigned)p->B, &a, stream);
}

int ae_launch_attn_bwd_fused(void* module, const AeAttnBwdParams* p, void* stream) {
  if (!module || !p || !p->q || !p->k || !p->v || !p->d_o || !p->dk || !p->dv || !p->dq_accum) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  int rc = check_attn_common(m, AE_KIND_ATTN_BWD_FUSED, p->B, p->Hq, p->Hkv, p->Sq, p->Skv);
  if (rc) return rc;
  if (m->cfg.mask_mode == 2 && (!p->block_count_t || !p->block_index_t)) {
    set_error("transposed block lists required for mask_mode 2");
    return AE_ERR_INVALID;
  }
  if (reinterpret_cast<uintptr_t>(p->dq_accum) & 15) {
    set_error("dq_accum must be 16-byte aligned");
    return AE_ERR_INVALID;
  }
  rc = ensure_loaded(m);
  if (rc) return rc;
  AeAttnBwdArgs a;
  rc = fill_bwd_args(m, p, &a, 128, 128);
  if (rc) return rc;
  a.dq_acc = p->dq_accum;
  {
    // fp32 [B, Sq, Hq, D] seen as (d, s, h, b): boxes of 32 floats x 32 q rows, 128-byte swizzle
    const cuuint64_t D = (cuuint64_t)m->cfg.head_dim;
    cuuint64_t dims[4] = {D, (cuuint64_t)p->Sq, (cuuint64_t)p->Hq, (cuuint64_t)p->B};
    cuuint64_t strides[3] = {(cuuint64_t)p->Hq * D * 4, D * 4, (cuuint64_t)p->Sq * p->Hq * D * 4};
    cuuint32_t box[4] = {32, 32, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    AE_CU(driver().cuTensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(&a.tm_dqacc), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                                          p->dq_accum, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  }
  const size_t words = (size_t)p->B * p->Sq * p->Hq * m->cfg.head_dim;
  AE_CU(driver().cuMemsetD32Async((CUdeviceptr)(uintptr_t)p->dq_accum, 0u, words, (CUstream)stream));
  return launch(m, (unsigned)a.n_kt, (unsigned)p->Hkv, (unsigned)p->B, &a, stream);
}

int ae_launch_attn_bwd_dq_cast(void* module, const AeAttnBwdParams* p, void* stream) {
  if (!module || !p || !p->dq || !p->dq_accum) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  int rc = check_attn_common(m, AE_KIND_ATTN_BWD_CAST, p->B, p->Hq, p->Hkv > 0 ? p->Hkv : 1, p->Sq, p->Skv > 0 ? p->Skv : 1);
  if (rc) return rc;
  if ((reinterpret_cast<uintptr_t>(p->dq_accum) & 15) || (reinterpret_cast<uintptr_t>(p->dq) & 15) ||
      p->dq_stride[0] % 8 || p->dq_stride[1] % 8 || p->dq_stride[2] % 8) {
    set_error("dq / dq_accum must be 16-byte aligned, dq strides multiples of 8 elements");
    return AE_ERR_INVALID;
  }
  rc = ensure_loaded(m);
  if (rc) return rc;
  AeAttnBwdArgs a;
  memset(&a, 0, sizeof a);
  a.dq = p->dq;
  a.dq_sb = p->dq_stride[0]; a.dq_ss = p->dq_stride[1]; a.dq_sh = p->dq_stride[2];
  a.dq_acc = p->dq_accum;
  a.B = p->B; a.Hq = p->Hq; a.Sq = p->Sq;
  const int64_t vecs = (int64_t)p->B * p->Sq * p->Hq * (m->cfg.head_dim / 8);
  int64_t blocks = (vecs + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch(m, (unsigned)blocks, 1, 1, &a, stream);
}

static int make_3d_map(AeTmaDesc* out, const void* base, int dtype, int64_t cols, int64_t rows, int64_t batch,
                       int box_rows, int64_t row_stride = 0) {
  Driver& d = driver();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_error("tensor base address must be 16-byte aligned");
    return AE_ERR_INVALID;
  }
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  if (row_stride == 0) row_stride = cols;  // elements between rows; larger when the rows are slices of wider ones
  cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)rows * row_stride * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = dtype == AE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  AE_CU(d.cuTensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(out), dt, 3, const_cast<void*>(base), dims, strides,
                                 box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return AE_OK;
}

int ae_launch_mla_decode(void* module, const AeMlaParams* p, void* stream) {
  if (!module || !p || !p->q || !p->q_pe || !p->kv || !p->k_pe || !p->o) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  if (m->cfg.kind != AE_KIND_MLA_DECODE) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  const int bn = m->cfg.reserved[0];
  if (p->B <= 0 || p->S <= 0 || p->H <= 0 || p->H > 128 || p->n_split < 1 || p->n_split > 32 || (bn != 64 && bn != 128)) {
    set_error("MLA decode: need 1 <= H <= 128, S > 0, 1 <= n_split <= 32");
    return AE_ERR_INVALID;
  }
  const int n_tiles = (p->S + bn - 1) / bn;
  const int tps = (n_tiles + p->n_split - 1) / p->n_split;
  if ((int64_t)(p->n_split - 1) * tps >= n_tiles) {
    set_error("MLA decode: n_split leaves an empty split");
    return AE_ERR_INVALID;
  }
  if (p->n_split > 1 && !p->o_partial) {
    set_error("MLA decode: o_partial scratch required when n_split > 1");
    return AE_ERR_INVALID;
  }
  int rc = ensure_loaded(m);
  if (rc) return rc;
  AeMlaArgs a;
  memset(&a, 0, sizeof a);
  if ((rc = make_3d_map(&a.tm_q, p->q, m->cfg.dtype, 512, p->H, p->B, 128))) return rc;
  if ((rc = make_3d_map(&a.tm_qpe, p->q_pe, m->cfg.dtype, 64, p->H, p->B, 128))) return rc;
  if ((rc = make_3d_map(&a.tm_kv, p->kv, m->cfg.dtype, 512, p->S, p->B, bn))) return rc;
  if ((rc = make_3d_map(&a.tm_kpe, p->k_pe, m->cfg.dtype, 64, p->S, p->B, bn))) return rc;
  a.o = p->o;
  a.o_part = p->o_partial;
  for (int i = 0; i < AE_MAX_FINAL; ++i) a.fr_part[i] = p->rowscale_partial[i];
  a.B = p->B; a.H = p->H; a.S = p->S; a.n_split = p->n_split; a.tiles_per_split = tps;
  a.status = p->status;
  return launch(m, 2, (unsigned)p->n_split, (unsigned)p->B, &a, stream);
}

int ae_launch_mla_decode_paged(void* module, const AeMlaPagedParams* p, void* stream) {
  if (!module || !p || !p->q || !p->q_pe || !p->kcache || !p->block_table || !p->cache_seqlens || !p->o)
    return AE_ERR_INVALID;
  Module* m = (Module*)module;
  if (m->cfg.kind != AE_KIND_MLA_DECODE) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  if (m->cfg.reserved[0] != 64) {
    set_error("paged MLA decode: pages hold 64 keys, the kernel must stream 64-row tiles");
    return AE_ERR_UNSUPPORTED;
  }
  if (p->B <= 0 || p->H <= 0 || p->H > 128 || p->num_pages <= 0 || p->max_pages <= 0 || p->max_seqlen <= 0 ||
      p->max_seqlen > (int64_t)p->max_pages * 64 || p->n_split < 1 || p->n_split > 32) {
    set_error("paged MLA decode: need 1 <= H <= 128, 1 <= max_seqlen <= max_pages * 64, 1 <= n_split <= 32");
    return AE_ERR_INVALID;
  }
  const int n_tiles = (p->max_seqlen + 63) / 64;
  const int tps = (n_tiles + p->n_split - 1) / p->n_split;
  if ((int64_t)(p->n_split - 1) * tps >= n_tiles) {
    set_error("MLA decode: n_split leaves an empty split");
    return AE_ERR_INVALID;
  }
  if (p->n_split > 1 && !p->o_partial) {
    set_error("MLA decode: o_partial scratch required when n_split > 1");
    return AE_ERR_INVALID;
  }
  int rc = ensure_loaded(m);
  if (rc) return rc;
  AeMlaArgs a;
  memset(&a, 0, sizeof a);
  const int64_t pool_rows = (int64_t)p->num_pages * 64;
  if ((rc = make_3d_map(&a.tm_q, p->q, m->cfg.dtype, 512, p->H, p->B, 128))) return rc;
  if ((rc = make_3d_map(&a.tm_qpe, p->q_pe, m->cfg.dtype, 64, p->H, p->B, 128))) return rc;
  // the pool as one batch of num_pages * 64 rows of 576 elements: latent part and rope part are column slices
  if ((rc = make_3d_map(&a.tm_kv, p->kcache, m->cfg.dtype, 512, pool_rows, 1, 64, 576))) return rc;
  if ((rc = make_3d_map(&a.tm_kpe, (const char*)p->kcache + 512 * 2, m->cfg.dtype, 64, pool_rows, 1, 64, 576))) return rc;
  a.o = p->o;
  a.o_part = p->o_partial;
  for (int i = 0; i < AE_MAX_FINAL; ++i) a.fr_part[i] = p->rowscale_partial[i];
  a.B = p->B; a.H = p->H; a.S = p->max_seqlen; a.n_split = p->n_split; a.tiles_per_split = tps;
  a.status = p->status;
  a.block_table = p->block_table;
  a.seqlens = p->cache_seqlens;
  a.max_pages = p->max_pages;
  return launch(m, 2, (unsigned)p->n_split, (unsigned)p->B, &a, stream);
}

int ae_launch_mla_combine(void* module, const AeMlaParams* p, void* stream) {
  if (!module || !p || !p->o || !p->o_partial) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  if (m->cfg.kind != AE_KIND_MLA_COMBINE) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  if (p->n_split < 1 || p->n_split > 32) return AE_ERR_INVALID;
  int rc = ensure_loaded(m);
  if (rc) return rc;
  AeMlaCombineArgs a;
  memset(&a, 0, sizeof a);
  a.o = p->o;
  a.o_part = p->o_partial;
  for (int i = 0; i < AE_MAX_FINAL; ++i) a.fr_part[i] = p->rowscale_partial[i];
  a.B = p->B; a.H = p->H; a.DV = 512; a.n_split = p->n_split;
  return launch(m, (unsigned)((p->H + 3) / 4), (unsigned)p->B, 1, &a, stream);
}

int ae_launch_attn_decode(void* module, const AeDecodeParams* p, void* stream) {
  if (!module || !p || !p->q || !p->k || !p->v || !p->o) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  int rc = check_attn_common(m, AE_KIND_ATTN_DECODE, p->B, p->Hq, p->Hkv, p->Sq, p->Skv);
  if (rc) return rc;
  const int gq = p->Hq / p->Hkv;
  const int rows = gq > 1 ? gq : p->Sq;
  const int n_kt = (p->Skv + 127) / 128;
  if (gq > 1 && p->Sq != 1) {
    set_error("decode with grouped query heads takes one query position");
    return AE_ERR_UNSUPPORTED;
  }
  if (rows > 256) {
    set_error("decode packs at most 256 query rows per head unit");
    return AE_ERR_UNSUPPORTED;
  }
  if (m->cfg.mask_mode != 0 && m->cfg.mask_mode != 3) return AE_ERR_UNSUPPORTED;
  const bool varlen = p->work != nullptr;
  int tps = 0;
  if (varlen) {
    if (!p->seqlens || !p->part_off || p->n_items <= 0 || !p->o_partial) {
      set_error("a work list needs seqlens, part_off, n_items > 0 and the partial buffers");
      return AE_ERR_INVALID;
    }
  } else {
    if (p->n_split < 1 || p->n_split > 32 || p->n_split > n_kt) return AE_ERR_INVALID;
    tps = (n_kt + p->n_split - 1) / p->n_split;
    if ((p->n_split - 1) * tps >= n_kt) {
      set_error("n_split leaves a split without kv tiles");
      return AE_ERR_INVALID;
    }
    if (p->n_split > 1 && !p->o_partial) return AE_ERR_INVALID;
  }
  if (varlen || p->n_split > 1)
    for (int i = 0; i < m->cfg.reserved[1] && i < AE_MAX_FINAL; ++i)
      if (!p->rowscale_partial[i]) return AE_ERR_INVALID;
  if (p->block_table && (p->max_pages <= 0 || p->num_pages <= 0)) {
    set_error("paged K / V need max_pages and num_pages");
    return AE_ERR_INVALID;
  }
  rc = ensure_loaded(m);
  if (rc) return rc;
  AeAttnFwdArgs args;
  memset(&args, 0, sizeof args);
  const int D = m->cfg.head_dim, DV = m->cfg.head_dim_v;
  if (gq > 1) {
    // rows of the q tile = the query heads of one kv head: (d, head in group, kv head, b)
    const int64_t qs[3] = {p->q_stride[0], p->q_stride[2], (int64_t)gq * p->q_stride[2]};
    rc = make_bshd_map(&args.tm_q, p->q, m->cfg.dtype, p->B, gq, p->Hkv, D, qs, 128);
  } else {
    rc = make_bshd_map(&args.tm_q, p->q, m->cfg.dtype, p->B, p->Sq, p->Hq, D, p->q_stride, 128);
  }
  if (rc) return rc;
  if (p->block_table) {
    // pools [num_pages, 128, Hkv, D] seen as one batch of num_pages * 128 rows (a page's keys are contiguous rows)
    if (p->k_stride[0] != 128 * p->k_stride[1] || p->v_stride[0] != 128 * p->v_stride[1]) {
      set_error("paged K / V: a page must hold 128 keys at a constant stride");
      return AE_ERR_INVALID;
    }
    const int64_t ks[3] = {0, p->k_stride[1], p->k_stride[2]}, vs[3] = {0, p->v_stride[1], p->v_stride[2]};
    rc = make_bshd_map(&args.tm_k, p->k, m->cfg.dtype, 1, (int64_t)p->num_pages * 128, p->Hkv, D, ks, 128);
    if (rc) return rc;
    rc = make_bshd_map(&args.tm_v, p->v, m->cfg.dtype, 1, (int64_t)p->num_pages * 128, p->Hkv, DV, vs, 128);
    if (rc) return rc;
  } else {
    rc = make_bshd_map(&args.tm_k, p->k, m->cfg.dtype, p->B, p->Skv, p->Hkv, D, p->k_stride, 128);
    if (rc) return rc;
    rc = make_bshd_map(&args.tm_v, p->v, m->cfg.dtype, p->B, p->Skv, p->Hkv, DV, p->v_stride, 128);
    if (rc) return rc;
  }
  if (reinterpret_cast<uintptr_t>(p->o) & 15) {
    set_error("output must be 16-byte aligned");
    return AE_ERR_INVALID;
  }
  args.o = p->o;  // contiguous [B, Sq, Hq, DV]
  args.o_sh = DV;
  args.o_ss = (int64_t)p->Hq * DV;
  args.o_sb = (int64_t)p->Sq * p->Hq * DV;
  args.o_part = p->o_partial;
  for (int i = 0; i < AE_MAX_FINAL; ++i) args.fr_part[i] = p->rowscale_partial[i];
  for (int i = 0; i < AE_MAX_CUSTOM; ++i) {
    args.custom[i] = p->custom[i];
    for (int k = 0; k < 4; ++k) args.custom_st[i][k] = p->custom_stride[i][k];
  }
  args.B = p->B;
  args.Hq = p->Hq;
  args.Hkv = p->Hkv;
  args.Sq = p->Sq;
  args.Skv = p->Skv;
  args.n_qt = (rows + 127) / 128;
  args.n_kt = n_kt;
  args.status = p->status;
  args.n_split = p->n_split;
  args.tiles_per_split = tps;
  args.gq = gq;
  args.rows = rows;
  args.work = reinterpret_cast<const AeWorkItem*>(p->work);
  args.seqlens = p->seqlens;
  args.part_off = p->part_off;
  args.block_table = p->block_table;
  args.max_pages = p->max_pages;
  const unsigned units = (unsigned)(gq > 1 ? p->Hkv : p->Hq);
  if (varlen) return launch(m, (unsigned)p->n_items, units, 1, &args, stream);
  return launch(m, (unsigned)p->n_split, units, (unsigned)p->B, &args, stream);
}

int ae_launch_decode_combine(void* module, const AeDecodeParams* p, void* stream) {
  if (!module || !p || !p->o || !p->o_partial) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  if (m->cfg.kind != AE_KIND_MLA_COMBINE) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  if ((!p->part_off && (p->n_split < 2 || p->n_split > 32)) || m->cfg.head_dim_v % 4) return AE_ERR_INVALID;
  int rc = ensure_loaded(m);
  if (rc) return rc;
  AeMlaCombineArgs a;
  memset(&a, 0, sizeof a);
  a.o = p->o;
  a.o_part = p->o_partial;
  for (int i = 0; i < AE_MAX_FINAL; ++i) a.fr_part[i] = p->rowscale_partial[i];
  a.B = p->B;
  a.H = p->Sq * p->Hq;  // one output row per (query position, head)
  a.DV = m->cfg.head_dim_v;
  a.n_split = p->n_split;
  a.part_off = p->part_off;  // rows of different lengths: each row's own number of partial slots
  return launch(m, (unsigned)((a.H + 3) / 4), (unsigned)p->B, 1, &a, stream);
}

int ae_launch_rowscale(void* module, const AeRowScaleParams* p, void* stream) {
  if (!module || !p || !p->x || p->n_rows < 0) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  if (!p->s && m->kernel != "ae_head_sum") return AE_ERR_INVALID;
  if (m->cfg.kind != AE_KIND_ROWSCALE) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  if (m->kernel == "ae_head_sum") {
    // x [groups, G, T, D] -> y [groups, T, D]: n_rows output rows, rows_per_head = T, n_heads = G; s is not used
    if (!p->y || p->rows_per_head <= 0 || p->n_heads <= 0 || p->n_rows % p->rows_per_head) {
      set_error("ae_head_sum needs y, rows_per_head = T > 0, n_heads = G > 0 and n_rows a multiple of T");
      return AE_ERR_INVALID;
    }
    if ((reinterpret_cast<uintptr_t>(p->x) & 15) || (reinterpret_cast<uintptr_t>(p->y) & 15)) {
      set_error("row-scale tensors must be 16-byte aligned");
      return AE_ERR_INVALID;
    }
    if (p->n_rows == 0) return AE_OK;
    int rc = ensure_loaded(m);
    if (rc) return rc;
    AeRowScaleArgs a;
    memset(&a, 0, sizeof a);
    a.x = p->x; a.y = p->y; a.n_rows = p->n_rows; a.rows_per_head = p->rows_per_head; a.n_heads = p->n_heads;
    const int64_t lanes = p->n_rows * (m->cfg.head_dim / 8);
    int64_t blocks = (lanes + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return launch(m, (unsigned)blocks, 1, 1, &a, stream);
  }
  const bool both = m->kernel == "ae_vskip_bwd";
  const bool skip = m->kernel == "ae_skip_fwd" || m->kernel == "ae_skip_bwd" || both;
  const bool bwd = m->kernel == "ae_rowscale_bwd" || m->kernel == "ae_skip_bwd" || both;
  if (bwd ? (!p->g || !p->gx || !p->gs) : !p->y) return AE_ERR_INVALID;
  if (skip && (!p->g || p->rows_per_head <= 0 || p->n_heads <= 0)) {
    set_error("skip kernels need g, rows_per_head > 0 and n_heads > 0");
    return AE_ERR_INVALID;
  }
  if (both && (!p->g2 || !p->d || !p->gs2)) {
    set_error("ae_vskip_bwd needs g2, d and gs2");
    return AE_ERR_INVALID;
  }
  const void* ptrs[5] = {p->x, p->y, p->g, p->gx, both ? p->g2 : nullptr};
  for (const void* q : ptrs)
    if (q && (reinterpret_cast<uintptr_t>(q) & 15)) {
      set_error("row-scale tensors must be 16-byte aligned");
      return AE_ERR_INVALID;
    }
  if (p->n_rows == 0) return AE_OK;
  int rc = ensure_loaded(m);
  if (rc) return rc;
  AeRowScaleArgs a;
  memset(&a, 0, sizeof a);
  a.x = p->x; a.s = p->s; a.y = p->y; a.g = p->g; a.gx = p->gx; a.gs = p->gs;
  a.n_rows = p->n_rows;
  a.rows_per_head = skip ? p->rows_per_head : 1;
  a.n_heads = skip ? p->n_heads : 1;
  if (both) {
    a.g2 = p->g2;
    a.d = p->d;
    a.gs2 = p->gs2;
  }
  // 16 bytes per lane, 256 threads per CTA, up to 16 CTAs per SM's worth of blocks; the kernels stride over the rest
  const int64_t lanes = p->n_rows * (m->cfg.head_dim / 8);
  int64_t blocks = (lanes + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch(m, (unsigned)blocks, 1, 1, &a, stream);
}

// Tensor map over a contiguous [B, H, T, D] tensor seen as (d, t, h, b), box {64, rows, 1, 1}.
static int make_bhtd_map(AeTmaDesc* out, const void* base, int dtype, int64_t B, int64_t H, int64_t T, int64_t D,
                         int rows) {
  Driver& d = driver();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || D % 8) {
    set_error("tensor base address must be 16-byte aligned and the head dim a multiple of 8");
    return AE_ERR_INVALID;
  }
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)T * D * 2, (cuuint64_t)H * T * D * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = dtype == AE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  AE_CU(d.cuTensorMapEncodeTiled(reinterpret_cast<CUtensorMap*>(out), dt, 4, const_cast<void*>(base), dims, strides,
                                 box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return AE_OK;
}

int ae_launch_linear_fwd(void* module, const AeLinearParams* p, void* stream) {
  if (!module || !p || !p->q || !p->k || !p->v || !p->a || !p->o) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  if (m->cfg.kind != AE_KIND_LINEAR_FWD) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  if (p->B <= 0 || p->H <= 0 || p->HQ <= 0 || p->HK <= 0 || p->T <= 0 || p->H % p->HQ || p->H % p->HK ||
      m->cfg.head_dim != 128 || (m->cfg.head_dim_v != 64 && m->cfg.head_dim_v != 128)) {
    set_error("linear attention: need H % HQ == 0, H % HK == 0, DK = 128, DV in {64, 128}");
    return AE_ERR_INVALID;
  }
  if ((reinterpret_cast<uintptr_t>(p->o) & 15) || (reinterpret_cast<uintptr_t>(p->a) & 3)) {
    set_error("linear attention: output must be 16-byte aligned");
    return AE_ERR_INVALID;
  }
  int rc = ensure_loaded(m);
  if (rc) return rc;
  AeLinearArgs a;
  memset(&a, 0, sizeof a);
  if ((rc = make_bhtd_map(&a.tm_q, p->q, m->cfg.dtype, p->B, p->HQ, p->T, 128, 128))) return rc;
  if ((rc = make_bhtd_map(&a.tm_k, p->k, m->cfg.dtype, p->B, p->HK, p->T, 128, 128))) return rc;
  if ((rc = make_bhtd_map(&a.tm_v, p->v, m->cfg.dtype, p->B, p->H, p->T, m->cfg.head_dim_v, 128))) return rc;
  a.a = p->a;
  a.o = p->o;
  if ((rc = make_bhtd_map(&a.tm_o, p->o, m->cfg.dtype, p->B, p->H, p->T, m->cfg.head_dim_v, 128))) return rc;
  a.B = p->B; a.H = p->H; a.HQ = p->HQ; a.HK = p->HK; a.T = p->T;
  a.status = p->status;
  if (p->h_states_out && (reinterpret_cast<uintptr_t>(p->h_states_out) & 15)) {
    set_error("linear attention: h_states_out must be 16-byte aligned");
    return AE_ERR_INVALID;
  }
  a.h_out = p->h_states_out;
  a.ascale = p->ascale;
  if (p->h_states_out) {
    const int64_t nc = (p->T + 127) / 128;
    if ((rc = make_3d_map(&a.tm_hout, p->h_states_out, m->cfg.dtype, m->cfg.head_dim_v, 128, (int64_t)p->B * p->H * nc, 128)))
      return rc;
  }
  // modules built with the block's mods inside (config reserved[0] = 1) take the three optional operands
  if (m->cfg.reserved[0] == 1) {
    if ((p->v_out && (reinterpret_cast<uintptr_t>(p->v_out) & 15)) ||
        (p->vscale && (reinterpret_cast<uintptr_t>(p->vscale) & (p->vscale_16bit ? 1 : 3)))) {
      set_error("linear attention: v_out must be 16-byte aligned, vscale aligned to its element size");
      return AE_ERR_INVALID;
    }
    a.vscale = p->vscale;
    a.vscale_16 = p->vscale_16bit;
    a.dskip = p->dskip;
    a.v_out = p->v_out;
    if (p->v_out && (rc = make_bhtd_map(&a.tm_vout, p->v_out, m->cfg.dtype, p->B, p->H, p->T, m->cfg.head_dim_v, 128)))
      return rc;
  } else if (p->vscale || p->dskip || p->v_out) {
    set_error("linear attention: vscale / dskip / v_out need a module built with the mods inside (reserved[0] = 1)");
    return AE_ERR_INVALID;
  }
  return launch(m, (unsigned)p->H, (unsigned)p->B, 1, &a, stream);
}

static int fill_linear_bwd(Module* m, const AeLinearBwdParams* p, AeLinearBwdArgs* a, int kind) {
  if (m->cfg.kind != kind) {
    set_error("module kind does not match the entry point");
    return AE_ERR_UNSUPPORTED;
  }
  const int DV = m->cfg.head_dim_v;
  if (p->B <= 0 || p->H <= 0 || p->HQ <= 0 || p->HK <= 0 || p->T <= 0 || p->H % p->HQ || p->H % p->HK ||
      m->cfg.head_dim != 128 || (DV != 64 && DV != 128)) {
    set_error("linear attention: need H % HQ == 0, H % HK == 0, DK = 128, DV in {64, 128}");
    return AE_ERR_INVALID;
  }
  int rc = ensure_loaded(m);
  if (rc) return rc;
  memset(a, 0, sizeof *a);
  const int64_t nc = (p->T + 127) / 128;
  if ((rc = make_bhtd_map(&a->tm_k, p->k, m->cfg.dtype, p->B, p->HK, p->T, 128, 128))) return rc;
  if ((rc = make_bhtd_map(&a->tm_v, p->v, m->cfg.dtype, p->B, p->H, p->T, DV, 128))) return rc;
  if (kind == AE_KIND_LINEAR_BWD) {
    if ((rc = make_bhtd_map(&a->tm_q, p->q, m->cfg.dtype, p->B, p->HQ, p->T, 128, 128))) return rc;
    if ((rc = make_bhtd_map(&a->tm_do, p->d_o, m->cfg.dtype, p->B, p->H, p->T, DV, 128))) return rc;
    if ((rc = make_3d_map(&a->tm_h, p->h_states, m->cfg.dtype, DV, 128, (int64_t)p->B * p->H * nc, 128))) return rc;
    if ((rc = make_bhtd_map(&a->tm_dq, p->dq, m->cfg.dtype, p->B, p->H, p->T, 128, 128))) return rc;
    if ((rc = make_bhtd_map(&a->tm_dk, p->dk, m->cfg.dtype, p->B, p->H, p->T, 128, 128))) return rc;
    if ((rc = make_bhtd_map(&a->tm_dv, p->dv, m->cfg.dtype, p->B, p->H, p->T, DV, 128))) return rc;
    if (m->cfg.reserved[0] == 1) {  // built with the block's mods inside: dv receives the gradient of x
      if (!p->x || !p->vscale || !p->dskip || !p->gs || !p->gd || (reinterpret_cast<uintptr_t>(p->x) & 15)) {
        set_error("linear attention backward with mods: x (16-byte aligned), vscale, dskip, gs and gd are required");
        return AE_ERR_INVALID;
      }
      if ((rc = make_bhtd_map(&a->tm_x, p->x, m->cfg.dtype, p->B, p->H, p->T, DV, 128))) return rc;
      a->vscale = p->vscale; a->dskip = p->dskip; a->gs = p->gs; a->gd = p->gd;
      a->vscale_16 = p->vscale_16bit;
    }
  }
  if (p->ascale && kind == AE_KIND_LINEAR_BWD && !p->gasc) {
    set_error("linear attention backward: ascale needs gasc");
    return AE_ERR_INVALID;
  }
  a->ascale = p->ascale;
  a->gasc = p->gasc;
  a->a = p->a;
  a->h_states = p->h_states;
  a->dq = p->dq; a->dk = p->dk; a->dv = p->dv; a->da = p->da;
  a->B = p->B; a->H = p->H; a->HQ = p->HQ; a->HK = p->HK; a->T = p->T;
  a->status = p->status;
  return AE_OK;
}

int ae_launch_linear_states(void* module, const AeLinearBwdParams* p, void* stream) {
  if (!module || !p || !p->k || !p->v || !p->a || !p->h_states) return AE_ERR_INVALID;
  if (reinterpret_cast<uintptr_t>(p->h_states) & 15) return AE_ERR_INVALID;
  Module* m = (Module*)module;
  AeLinearBwdArgs a;
  int rc = fill_linear_bwd(m, p, &a, AE_KIND_LINEAR_STATES);
  if (rc) return rc;
  return launch(m, (unsigned)p->H, (unsigned)p->B, 1, &a, stream);
}

int ae_launch_linear_bwd(void* module, const AeLinearBwdParams* p, void* stream) {
  if (!module || !p || !p->q || !p->k || !p->v || !p->a || !p->d_o || !p->h_states || !p->dq || !p->dk || !p->dv ||
      !p->da)
    return AE_ERR_INVALID;
  const void* al[4] = {p->dq, p->dk, p->dv, p->h_states};
  for (const void* x : al)
    if (reinterpret_cast<uintptr_t>(x) & 15) {
      set_error("linear attention backward: buffers must be 16-byte aligned");
      return AE_ERR_INVALID;
    }
  Module* m = (Module*)module;
  if (m->cfg.head_dim_v != 64) {
    set_error("linear attention backward is built for DV = 64");
    return AE_ERR_INVALID;
  }
  AeLinearBwdArgs a;
  int rc = fill_linear_bwd(m, p, &a, AE_KIND_LINEAR_BWD);
  if (rc) return rc;
  return launch(m, (unsigned)p->H, (unsigned)p->B, 1, &a, stream);
}

}  // extern "C"
