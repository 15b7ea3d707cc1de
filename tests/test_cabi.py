"""The C-ABI library: loads without a GPU, exports what include/ae_b200.h declares, reports errors by
return code.  No compute calls here."""
import ctypes as C
import os
import re

import pytest

from attentionengine_b200 import runtime as rt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ae_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ae_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    L = rt.lib()
    names = _declared()
    assert "ae_compile" in names and "ae_launch_attn_fwd" in names and len(names) >= 12
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/ae_b200.h but not exported"
    assert sorted(rt.EXPORTS) == names


def test_struct_sizes_match_header():
    """ctypes mirrors of the parameter blocks have the size the C compiler gives them."""
    import subprocess
    import tempfile
    names = ["AeKernelConfig", "AeKernelInfo", "AeAttnParams", "AeAttnBwdParams", "AeDecodeParams", "AeRowScaleParams",
             "AeMlaParams", "AeMlaPagedParams", "AeLinearParams", "AeLinearBwdParams", "AeDecodeWorkItem"]
    mirrors = [rt.KernelConfig, rt.KernelInfo, rt.AttnParams, rt.AttnBwdParams, rt.DecodeParams, rt.RowScaleParams,
               rt.MlaParams, rt.MlaPagedParams, rt.LinearParams, rt.LinearBwdParams, C.c_int32 * 4]
    src = '#include <stdio.h>\n#include "ae_b200.h"\nint main(){' + \
          "".join(f'printf("%zu\\n", sizeof({n}));' for n in names) + "return 0;}\n"
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        subprocess.run(["gcc", f"-I{ROOT}/include", c, "-o", os.path.join(d, "s")], check=True)
        out = subprocess.run([os.path.join(d, "s")], capture_output=True, text=True, check=True).stdout.split()
    for n, got, m in zip(names, out, mirrors):
        assert int(got) == C.sizeof(m), f"{n}: header {got} bytes, ctypes mirror {C.sizeof(m)}"


def test_strerror_and_invalid_arguments():
    L = rt.lib()
    assert L.ae_strerror(0) == b"ok"
    assert b"invalid" in L.ae_strerror(1)
    out = C.c_void_p()
    assert L.ae_compile(None, b"k", b"sm_100a", None, 0, None, C.byref(out), None, 0) == 1
    assert L.ae_launch_attn_fwd(None, None, None) == 1


def test_compile_error_is_reported_not_fatal():
    cfg = rt.KernelConfig(kind=rt.KIND_PROBE, threads=32)
    with pytest.raises(rt.AeError) as e:
        rt.compile_module("extern \"C\" __global__ void k() { this is not C++; }", "k", cfg)
    assert "error" in str(e.value).lower()


def test_compile_without_gpu_and_cubin_roundtrip(tmp_path, monkeypatch):
    monkeypatch.setattr(rt, "CACHE_DIR", tmp_path)
    cfg = rt.KernelConfig(kind=rt.KIND_PROBE, threads=32)
    src = 'extern "C" __global__ void k(float* p) { p[threadIdx.x] = 1.f; }'
    m1 = rt.compile_module(src, "k", cfg)
    files = list(tmp_path.glob("k_*.cubin"))
    assert len(files) == 1 and files[0].stat().st_size > 0
    m2 = rt.compile_module(src, "k", cfg)  # served from the cache
    data, size = C.c_void_p(), C.c_size_t()
    rt.check(rt.lib().ae_module_cubin(m2.handle, C.byref(data), C.byref(size)))
    assert size.value == files[0].stat().st_size


def test_wrong_kind_is_refused():
    cfg = rt.KernelConfig(kind=rt.KIND_PROBE, threads=32)
    m = rt.compile_module('extern "C" __global__ void k(float* p) { p[0] = 1.f; }', "k", cfg)
    p = rt.AttnParams()
    p.q = p.k = p.v = p.o = 16
    p.B = p.Hq = p.Hkv = 1
    p.Sq = p.Skv = 128
    rc = rt.lib().ae_launch_attn_fwd(m.handle, C.byref(p), None)
    assert rc == 6 and b"kind" in rt.lib().ae_last_error()
