"""CPU-side checks of the C-ABI boundary: the libraries build, load without a GPU, export
every symbol the public headers declare, and refuse to compute without a device."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mgpu[A-Za-z0-9_]+)\s*\(", text)))


def _exported(path):
    out = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


@pytest.fixture(scope="module")
def built(mdc):
    if not (os.path.exists(mdc.RUNTIME_LIB) and os.path.exists(mdc.OPS_LIB)):
        mdc.build()
    return mdc


def test_runtime_exports_every_declared_symbol(built):
    names = _declared("mdc_gpu_runtime.h")
    assert len(names) >= 35
    missing = [n for n in names if n not in _exported(built.RUNTIME_LIB)]
    assert not missing, missing
    assert set(names) == set(built.RUNTIME_SIGNATURES), set(names) ^ set(built.RUNTIME_SIGNATURES)


def test_ops_exports_every_declared_symbol(built):
    names = _declared("mdc_gpu_ops.h")
    exported = _exported(built.OPS_LIB)
    missing = [n for n in names if n not in exported]
    assert not missing, missing
    assert set(names) == set(built.OPS_SIGNATURES), set(names) ^ set(built.OPS_SIGNATURES)
    # the C++ symbols the reference's runner links against (Kernels/GPU/Ops.h:15-20)
    for mangled in ("_Z10gpuOpsInitv", "_Z12gpuOpsDeinitv", "_Z13gpuLLMOpsInitv", "_Z15gpuLLMOpsDeinitv"):
        assert mangled in exported


def test_libraries_load_and_bind(built):
    rt, ops = built.runtime(), built.ops()
    for name in built.RUNTIME_SIGNATURES:
        assert getattr(rt, name)
    for name in built.OPS_SIGNATURES:
        assert getattr(ops, name)


def test_no_cpu_fallback_without_a_gpu(built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    rt = built.runtime()
    rt.mgpuClearLastError()
    with pytest.raises(built.MdcError):
        built.add(np.ones(8, np.float32), np.ones(8, np.float32))
    rt.mgpuClearLastError()
    with pytest.raises(built.MdcError):
        built.init()
    rt.mgpuClearLastError()


def test_cnn_ops_reject_bad_geometry_before_touching_a_device(built):
    rt, ops = built.runtime(), built.ops()
    rt.mgpuClearLastError()
    # N, C, H, W, OH, OW, KH, KW, PHL, PWL, PHR, PWR, SH, SW, method: stride 0
    ops.mgpuPool2d(None, None, 1, 1, 4, 4, 2, 2, 2, 2, 0, 0, 0, 0, 0, 2, 0, None)
    assert rt.mgpuGetLastError() != 0
    assert b"mgpuPool2d" in rt.mgpuGetLastErrorString()
    rt.mgpuClearLastError()
    # output extent larger than the padded input allows
    ops.mgpuConv2d(None, None, None, None, None, 1, 3, 8, 8, 4, 3, 3, 9, 9, 0, 0, 0, 0, 1, 1, 1, 1,
                   False, False, None)
    assert rt.mgpuGetLastError() != 0
    assert b"mgpuConv2d" in rt.mgpuGetLastErrorString()
    rt.mgpuClearLastError()
    assert rt.mgpuGetLastError() == 0


def test_pool_size_classes(built):
    # size classes are a property of the allocator's host logic (no device needed)
    src = open(os.path.join(ROOT, "multi-device-model-compiler_b200", "csrc", "runtime", "device_pool.cpp")).read()
    assert "round_size" in src


def test_bf16_helpers_round_to_nearest_even(built):
    import torch
    x = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    bits = built.f32_to_bf16_bits(x)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, ref)
    assert np.array_equal(built.bf16_bits_to_f32(bits), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


_CXX_CALLER = r"""
// what a sibling translation unit of the reference does (lib/Kernels/GPU/LLM.cu:50-158):
// include the template declarations and call the instantiations the library exports
#include "mdc_gpu_ops_cxx.h"
void use(half *h, float *f, cudaStream_t s) {
  invokeCudaCast<half, float>(h, f, 16, s);
  invokeCudaCast<float, half>(f, h, 16, s);
  mgpuMatmulEx<half>(h, h, h, h, h, 8, 8, 8, true, false, true, s);
  mgpuMatmulEx<float>(f, f, f, f, f, 8, 8, 8, true, true, false, s);
  mgpuLayerNorm<half>(h, h, h, h, 1e-5f, 4, 64, nullptr, s);
  mgpuAddResidualPreLayerNorm<half>(h, h, h, h, h, h, 1e-5f, 4, 64, nullptr, s);
  mgpuAddFusedQKVBiasTranspose<half>(h, h, h, h, h, 1, 4, 4, 2, 8, s);
  gpuOpsInit(); gpuLLMOpsInit(); checkCudaStatus(cudaSuccess); gpuLLMOpsDeinit(); gpuOpsDeinit();
}
int main() { return 0; }
"""


def test_reference_style_cxx_caller_links_against_the_template_instantiations(built, tmp_path):
    """A C++ caller that sees only the template DECLARATIONS (as the reference's other
    translation units do, Kernels/GPU/Ops.h:51-74) must link: the library has to export the
    explicit instantiations under their C++ names."""
    src = tmp_path / "caller.cpp"
    src.write_text(_CXX_CALLER)
    exe = tmp_path / "caller"
    lib_dir = os.path.dirname(built.OPS_LIB)
    cmd = ["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include", str(src),
           "-o", str(exe), "-L", lib_dir, "-lMultiDeviceGPUOps", "-lMultiDeviceCUDARuntime",
           f"-Wl,-rpath,{lib_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0
