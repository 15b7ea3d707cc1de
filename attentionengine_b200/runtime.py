"""ctypes binding of libae_b200.so (declared in include/ae_b200.h) plus the cubin cache.

This is the only place Python touches the native library.  There is no fallback: if the shared
library is missing, importing a kernel raises, and a launch without a CUDA device raises.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libae_b200.so"
KERNEL_DIR = _PKG / "csrc" / "kernels"
CACHE_DIR = Path(os.environ.get("AE_B200_CACHE", _PKG / "_cubin_cache"))

AE_MAX_CUSTOM = 4
AE_MAX_FINAL = 4
STATIC_SCRATCH_MAX_ROWS = 8 * 1024 * 1024  # AE_STATIC_SCRATCH_MAX_ROWS in include/ae_b200.h

KIND_PROBE, KIND_ATTN_FWD, KIND_ATTN_BWD_PREP, KIND_ATTN_BWD_DQ, KIND_ATTN_BWD_DKV = 0, 1, 2, 3, 4
KIND_MLA_DECODE, KIND_MLA_COMBINE, KIND_LINEAR_FWD, KIND_LINEAR_BWD, KIND_LINEAR_STATES = 5, 6, 7, 8, 9
KIND_ATTN_DECODE = 10
KIND_ROWSCALE = 11
KIND_ATTN_BWD_FUSED, KIND_ATTN_BWD_CAST = 12, 13
KIND_ATTN_FWD_PAIR = 14
DTYPE_F16, DTYPE_BF16 = 0, 1


class AeError(RuntimeError):
    pass


class KernelConfig(C.Structure):
    _fields_ = [("kind", C.c_int), ("dtype", C.c_int), ("head_dim", C.c_int), ("head_dim_v", C.c_int),
                ("threads", C.c_int), ("smem_bytes", C.c_int), ("stages", C.c_int), ("mask_mode", C.c_int),
                ("reserved", C.c_int * 8)]


class KernelInfo(C.Structure):
    _fields_ = [("num_regs", C.c_int), ("static_smem_bytes", C.c_int), ("max_dynamic_smem_bytes", C.c_int),
                ("local_bytes", C.c_int), ("max_threads", C.c_int)]


_S3 = C.c_int64 * 3


class AttnParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("q_stride", _S3), ("k_stride", _S3), ("v_stride", _S3), ("o_stride", _S3),
                ("final_rowscales", C.c_void_p * AE_MAX_FINAL),
                ("custom", C.c_void_p * AE_MAX_CUSTOM),
                ("custom_stride", (C.c_int64 * 4) * AE_MAX_CUSTOM),
                ("block_count", C.c_void_p), ("block_index", C.c_void_p),
                ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32),
                ("status", C.c_void_p)]


class AttnBwdParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("d_o", C.c_void_p),
                ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
                ("q_stride", _S3), ("k_stride", _S3), ("v_stride", _S3), ("o_stride", _S3), ("do_stride", _S3),
                ("dq_stride", _S3), ("dk_stride", _S3), ("dv_stride", _S3),
                ("final_rowscales", C.c_void_p * AE_MAX_FINAL),
                ("delta", C.c_void_p),
                ("custom", C.c_void_p * AE_MAX_CUSTOM),
                ("custom_stride", (C.c_int64 * 4) * AE_MAX_CUSTOM),
                ("block_count", C.c_void_p), ("block_index", C.c_void_p),
                ("block_count_t", C.c_void_p), ("block_index_t", C.c_void_p),
                ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32),
                ("status", C.c_void_p), ("dq_accum", C.c_void_p)]


class MlaParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_pe", C.c_void_p), ("kv", C.c_void_p), ("k_pe", C.c_void_p), ("o", C.c_void_p),
                ("o_partial", C.c_void_p), ("rowscale_partial", C.c_void_p * AE_MAX_FINAL),
                ("B", C.c_int32), ("H", C.c_int32), ("S", C.c_int32), ("n_split", C.c_int32), ("status", C.c_void_p)]


class DecodeParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
                ("o_partial", C.c_void_p), ("rowscale_partial", C.c_void_p * AE_MAX_FINAL),
                ("custom", C.c_void_p * AE_MAX_CUSTOM), ("custom_stride", (C.c_int64 * 4) * AE_MAX_CUSTOM),
                ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("Sq", C.c_int32), ("Skv", C.c_int32),
                ("n_split", C.c_int32), ("status", C.c_void_p),
                ("work", C.c_void_p), ("n_items", C.c_int32), ("seqlens", C.c_void_p), ("part_off", C.c_void_p),
                ("block_table", C.c_void_p), ("max_pages", C.c_int32), ("num_pages", C.c_int32)]


class RowScaleParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("s", C.c_void_p), ("y", C.c_void_p), ("g", C.c_void_p), ("gx", C.c_void_p),
                ("gs", C.c_void_p), ("n_rows", C.c_int64), ("rows_per_head", C.c_int64), ("n_heads", C.c_int32),
                ("g2", C.c_void_p), ("d", C.c_void_p), ("gs2", C.c_void_p)]


class MlaPagedParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_pe", C.c_void_p), ("kcache", C.c_void_p), ("block_table", C.c_void_p),
                ("cache_seqlens", C.c_void_p), ("o", C.c_void_p), ("o_partial", C.c_void_p),
                ("rowscale_partial", C.c_void_p * AE_MAX_FINAL),
                ("B", C.c_int32), ("H", C.c_int32), ("num_pages", C.c_int32), ("max_pages", C.c_int32),
                ("max_seqlen", C.c_int32), ("n_split", C.c_int32), ("status", C.c_void_p)]


class LinearParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("a", C.c_void_p), ("o", C.c_void_p),
                ("B", C.c_int32), ("H", C.c_int32), ("HQ", C.c_int32), ("HK", C.c_int32), ("T", C.c_int32),
                ("status", C.c_void_p), ("vscale", C.c_void_p), ("dskip", C.c_void_p), ("v_out", C.c_void_p),
                ("vscale_16bit", C.c_int32), ("h_states_out", C.c_void_p), ("ascale", C.c_void_p)]


class LinearBwdParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("a", C.c_void_p), ("d_o", C.c_void_p),
                ("h_states", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("da", C.c_void_p),
                ("B", C.c_int32), ("H", C.c_int32), ("HQ", C.c_int32), ("HK", C.c_int32), ("T", C.c_int32),
                ("status", C.c_void_p), ("x", C.c_void_p), ("vscale", C.c_void_p), ("dskip", C.c_void_p),
                ("gs", C.c_void_p), ("gd", C.c_void_p), ("vscale_16bit", C.c_int32), ("ascale", C.c_void_p),
                ("gasc", C.c_void_p)]


_lib = None
_lib_lock = threading.Lock()

EXPORTS = ["ae_compile", "ae_module_from_cubin", "ae_module_cubin", "ae_query", "ae_release", "ae_strerror",
           "ae_last_error", "ae_launch_attn_fwd", "ae_launch_attn_bwd_prep", "ae_launch_attn_bwd_dq",
           "ae_launch_attn_bwd_dkv", "ae_launch_attn_bwd_fused", "ae_launch_attn_bwd_dq_cast", "ae_launch_probe", "ae_launch_attn_bwd_static_scratch", "ae_launch_mla_decode", "ae_launch_mla_combine", "ae_launch_mla_decode_paged", "ae_launch_attn_decode", "ae_launch_decode_combine", "ae_launch_rowscale", "ae_launch_linear_fwd", "ae_launch_linear_states", "ae_launch_linear_bwd"]


def lib() -> C.CDLL:
    global _lib
    with _lib_lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise AeError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                              "(there is no fallback path)")
            L = C.CDLL(str(LIB_PATH))
            L.ae_strerror.restype = C.c_char_p
            L.ae_last_error.restype = C.c_char_p
            L.ae_compile.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_char_p), C.c_int,
                                     C.POINTER(KernelConfig), C.POINTER(C.c_void_p), C.c_char_p, C.c_size_t]
            L.ae_module_from_cubin.argtypes = [C.c_void_p, C.c_size_t, C.c_char_p, C.POINTER(KernelConfig),
                                               C.POINTER(C.c_void_p)]
            L.ae_module_cubin.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
            L.ae_query.argtypes = [C.c_void_p, C.POINTER(KernelInfo)]
            L.ae_release.argtypes = [C.c_void_p]
            L.ae_release.restype = None
            L.ae_launch_attn_fwd.argtypes = [C.c_void_p, C.POINTER(AttnParams), C.c_void_p]
            for n in ("ae_launch_attn_bwd_prep", "ae_launch_attn_bwd_dq", "ae_launch_attn_bwd_dkv",
                      "ae_launch_attn_bwd_fused", "ae_launch_attn_bwd_dq_cast"):
                getattr(L, n).argtypes = [C.c_void_p, C.POINTER(AttnBwdParams), C.c_void_p]
            L.ae_launch_attn_bwd_static_scratch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(AttnBwdParams),
                                                            C.c_void_p]
            L.ae_launch_mla_decode.argtypes = [C.c_void_p, C.POINTER(MlaParams), C.c_void_p]
            L.ae_launch_mla_combine.argtypes = [C.c_void_p, C.POINTER(MlaParams), C.c_void_p]
            L.ae_launch_mla_decode_paged.argtypes = [C.c_void_p, C.POINTER(MlaPagedParams), C.c_void_p]
            L.ae_launch_attn_decode.argtypes = [C.c_void_p, C.POINTER(DecodeParams), C.c_void_p]
            L.ae_launch_decode_combine.argtypes = [C.c_void_p, C.POINTER(DecodeParams), C.c_void_p]
            L.ae_launch_rowscale.argtypes = [C.c_void_p, C.POINTER(RowScaleParams), C.c_void_p]
            L.ae_launch_linear_fwd.argtypes = [C.c_void_p, C.POINTER(LinearParams), C.c_void_p]
            L.ae_launch_linear_states.argtypes = [C.c_void_p, C.POINTER(LinearBwdParams), C.c_void_p]
            L.ae_launch_linear_bwd.argtypes = [C.c_void_p, C.POINTER(LinearBwdParams), C.c_void_p]
            L.ae_launch_probe.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                          C.c_void_p, C.c_void_p]
            _lib = L
    return _lib


def check(rc: int, what: str = ""):
    if rc != 0:
        L = lib()
        raise AeError(f"{what}: {L.ae_strerror(rc).decode()} - {L.ae_last_error().decode()}")


def exp_poly_period() -> int:
    """Every n-th exponential of a score tile is evaluated with the FMA-pipe polynomial instead of ex2.approx
    (0 = none).  Tunable through AE_B200_EXP_POLY; see ae_exp2_mix in csrc/kernels/ae_sm100.cuh."""
    return int(os.environ.get("AE_B200_EXP_POLY", "0"))


def kernel_source(*files: str, prelude: str = "", exp_poly: int | None = None, defines: dict | None = None) -> str:
    """Common header + argument blocks + generated prelude + kernel template(s), as one translation unit.
    `exp_poly` is the kernel's own default for AE_EXP_POLY_PERIOD (the environment variable still wins); `defines`
    are build switches of the kernel file, placed before everything else."""
    poly = exp_poly_period() if (exp_poly is None or "AE_B200_EXP_POLY" in os.environ) else exp_poly
    parts = [f"#define AE_EXP_POLY_PERIOD {poly}\n#define AE_WAIT_MODE {int(os.environ.get('AE_B200_WAIT_MODE', '0'))}\n"
             + ("#define AE_TRACE 1\n" if os.environ.get("AE_B200_TRACE") else "")
             + "".join(f"#define {k} {v}\n" for k, v in (defines or {}).items())
             + ("#define AE_SELFCHECK 1\n" if os.environ.get("AE_B200_SELFCHECK") else ""),
             (KERNEL_DIR / "ae_sm100.cuh").read_text().replace("#pragma once\n", ""),
             (KERNEL_DIR / "ae_args.h").read_text(), prelude]
    parts += [(KERNEL_DIR / f).read_text() for f in files]
    return "\n".join(parts)


class Module:
    """One compiled kernel (cubin + entry name + launch configuration)."""

    def __init__(self, handle: int, cfg: KernelConfig, name: str):
        self.handle = C.c_void_p(handle)
        self.cfg = cfg
        self.name = name

    def __del__(self):
        try:
            if self.handle:
                lib().ae_release(self.handle)
                self.handle = None
        except Exception:
            pass

    def info(self) -> KernelInfo:
        ki = KernelInfo()
        check(lib().ae_query(self.handle, C.byref(ki)), f"ae_query({self.name})")
        return ki


def compile_module(src: str, kernel_name: str, cfg: KernelConfig, opts: tuple = ()) -> Module:
    """NVRTC-compile ``src`` for sm_100a (or fetch the cubin from the content-addressed cache)."""
    L = lib()
    cfg_bytes = bytes(cfg)
    key = hashlib.sha256(src.encode() + b"\0" + kernel_name.encode() + b"\0" + cfg_bytes + repr(opts).encode()).hexdigest()
    path = CACHE_DIR / f"{kernel_name}_{key[:24]}.cubin"
    out = C.c_void_p()
    if path.exists():
        data = path.read_bytes()
        check(L.ae_module_from_cubin(data, len(data), kernel_name.encode(), C.byref(cfg), C.byref(out)),
              "ae_module_from_cubin")
        return Module(out.value, cfg, kernel_name)
    log = C.create_string_buffer(1 << 16)
    arr = (C.c_char_p * max(1, len(opts)))(*[o.encode() for o in opts])
    rc = L.ae_compile(src.encode(), kernel_name.encode(), b"sm_100a", arr, len(opts), C.byref(cfg), C.byref(out), log,
                      len(log))
    if rc != 0:
        raise AeError(f"ae_compile({kernel_name}) failed: {L.ae_strerror(rc).decode()}\n{log.value.decode(errors='replace')}")
    m = Module(out.value, cfg, kernel_name)
    data, size = C.c_void_p(), C.c_size_t()
    check(L.ae_module_cubin(m.handle, C.byref(data), C.byref(size)), "ae_module_cubin")
    CACHE_DIR.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(f".tmp{os.getpid()}")
    tmp.write_bytes(C.string_at(data, size.value))
    os.replace(tmp, path)
    return m
