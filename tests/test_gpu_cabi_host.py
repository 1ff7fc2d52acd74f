"""A C++ host without Python or torch calls the layer through the C ABI (tests/cabi_host/host_moe.cpp:
dlopen + dlsym, CUDA-runtime allocations, raw pointers); its output must have the bits of the Python API's."""
import os
import shutil
import struct
import subprocess

import pytest
import torch

from lightop_b200 import synthetic

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _cuda_home():
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.isdir(os.path.join(cand, "include")):
            return cand
    return None


@pytest.mark.skipif(shutil.which("g++") is None or _cuda_home() is None, reason="needs g++ and the CUDA runtime headers")
def test_cpp_host_matches_python_api(tmp_path):
    import lightop_b200
    from lightop_b200 import _lib
    cuda = _cuda_home()
    exe = str(tmp_path / "host_moe")
    build = subprocess.run(["g++", "-O2", "-std=c++17", f"-I{cuda}/include", os.path.join(HERE, "cabi_host", "host_moe.cpp"),
                            "-o", exe, f"-L{cuda}/lib64", "-lcudart", "-ldl", f"-Wl,-rpath,{cuda}/lib64"],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr

    E, k, M, H, I = 16, 4, 70, 512, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=31)
    x, logits = synthetic.make_activations(M, H, E, seed=32)
    inp = str(tmp_path / "in.bin")
    with open(inp, "wb") as f:
        f.write(struct.pack("<5q", M, E, k, H, I))
        for t in (logits.float(), x.view(torch.int16), w1, w2, w1_s.float(), w2_s.float()):
            f.write(t.contiguous().numpy().tobytes())
    out = str(tmp_path / "out.bin")
    lib_path = os.environ.get("LIGHTOP_B200_LIB") or os.path.join(ROOT, "lightop_b200", "liblightop_b200.so")
    run = subprocess.run([exe, lib_path, inp, out], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stderr + run.stdout
    raw = open(out, "rb").read()
    n_ids = M * k
    ids = torch.frombuffer(bytearray(raw[: 4 * n_ids]), dtype=torch.int32).view(M, k)
    wts = torch.frombuffer(bytearray(raw[4 * n_ids: 8 * n_ids]), dtype=torch.float32).view(M, k)
    y = torch.frombuffer(bytearray(raw[8 * n_ids:]), dtype=torch.bfloat16).view(M, H)

    dev = "cuda"
    tw = torch.empty(M, k, dtype=torch.float32, device=dev)
    ti = torch.empty(M, k, dtype=torch.int32, device=dev)
    lightop_b200.moe.topk_softmax(tw, ti, None, logits.to(dev), True)
    y_py = lightop_b200.moe.fused_experts_impl_int8(x.to(dev), w1.to(dev), w2.to(dev), tw, ti, None, use_int8_w8a8=True,
                                                   block_shape=[128, 128], w1_scale=w1_s.to(dev), w2_scale=w2_s.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(ids, ti.cpu()) and torch.equal(wts, tw.cpu())
    assert torch.equal(y, y_py.cpu())
    assert _lib is not None
