"""include/warp_kernels.hpp, the C++ host mirror of the reference's `warp_kernels::quantize` TW-Marlin
functions (crates/kernels/src/quantize.rs:1018-1360, 1731-1782; quantize_indirect.rs:228-253): it
compiles with plain g++ against the C ABI, rejects what the reference's asserts reject, and on a GPU
gives the results the oracle gives."""
import os
import subprocess

import numpy as np
import pytest

import oracle
from helpers import rel_err_floored

TOL_F16 = 1e-2          # max relative error per output element, FP16 output (denominator floored)
TOL_F32 = 1e-3          # FP32 output: summation order only

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "tensorwarp_b200")


def _build(tmp_path):
    exe = str(tmp_path / "mirror_check")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           os.path.join(ROOT, "tests", "cpp", "mirror_check.cpp"), "-o", exe, "-L", LIBDIR, "-ltwmarlin",
           "-L", os.path.join(cuda, "lib64"), "-lcudart", f"-Wl,-rpath,{LIBDIR}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_compiles_and_rejects_bad_shapes(twm_lib, tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and "host checks: ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_calls_match_oracle(tmp_path):
    exe = _build(tmp_path)
    out = tmp_path / "out"
    out.mkdir()
    r = subprocess.run([exe, "gpu", str(out)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    k, n1, n2, group = 1024, 384, 256, 128
    n = n1 + n2
    rd = lambda name, dt: np.fromfile(out / name, dtype=dt)
    w1, w2 = rd("w1.f32", np.float32).reshape(k, n1), rd("w2.f32", np.float32).reshape(k, n2)
    a32, a16 = rd("a.f32", np.float32), rd("a.f16", np.uint16)
    packed, scales = rd("packed.u8", np.uint8).reshape(k // 32, n, 16), rd("scales.u16", np.uint16).reshape(k // group, n)
    # quantise + fuse through the C++ calls == the oracle's quantiser on the concatenated matrix, bit for bit
    p_ref, s_ref = oracle.quantize_pack(np.concatenate([w1, w2], axis=1), k, n, group)
    assert np.array_equal(packed, p_ref) and np.array_equal(scales, s_ref)
    a16f = oracle.f16_bits_to_f32(a16)
    ref32 = oracle.w4a16_f64(a32[None], packed, scales, 1, n, k, group)
    ref16 = oracle.w4a16_f64(a16f[None], packed, scales, 1, n, k, group)
    assert rel_err_floored(rd("c.f32", np.float32)[None], ref32) < TOL_F32
    c16 = oracle.f16_bits_to_f32(rd("c.f16", np.uint16))
    assert rel_err_floored(c16[None], ref16) < TOL_F16
    # the sub-buffer and the expert-indexed forms give the same bits as the fused call's columns
    assert np.array_equal(rd("c_indirect.f16", np.uint16), rd("c.f16", np.uint16)[:n1])
    assert np.array_equal(rd("c_from_buffer.f16", np.uint16), rd("c.f16", np.uint16)[n1:])
