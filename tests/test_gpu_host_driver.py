"""The C++ host mirror of the tract op interface (tract_b200/host/ops.hpp), driven by a small plan loop
(tests/host/plan_driver.cpp) and checked against the oracle: prefill 3 + 12 decode steps with GQA 4/2 as in
inplace_kv_cache.rs:595-658, resume from a frozen state bit-identical (:898-942), save_to == concat of the
inputs, a lone DynKeyValueCache returning the whole cache, a lone Sdpa over the saved tensors."""
import os
import struct
import subprocess

import numpy as np
import pytest

import oracle
from util import TOL, normal, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_driver(tmp):
    exe = os.path.join(tmp, "plan_driver")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call(["g++", "-O2", "-std=c++17", os.path.join(ROOT, "tests", "host", "plan_driver.cpp"), "-o", exe,
                           f"-I{cuda}/include", f"-L{cuda}/lib64", "-lcudart", f"-L{ROOT}/tract_b200", "-lb200kv",
                           f"-Wl,-rpath,{ROOT}/tract_b200", f"-Wl,-rpath,{cuda}/lib64"])
    return exe


@pytest.mark.parametrize("fmt,fmt_code,dt_name", [("f16", 1, "f16"), ("f32", 0, "f32")])
def test_plan_driver_matches_oracle(tmp_path, fmt, fmt_code, dt_name):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    import tract_b200

    tract_b200.lib()
    exe = build_driver(str(tmp_path))
    Hq, Hkv, D = 4, 2, 128
    steps = [3] + [1] * 12
    freeze_at = 8
    dt = np.float16 if dt_name == "f16" else np.float32
    qs = [normal(10 + i, (Hq, s, D)).astype(dt) for i, s in enumerate(steps)]
    ks = [normal(40 + i, (Hkv, s, D)).astype(dt) for i, s in enumerate(steps)]
    vs = [normal(70 + i, (Hkv, s, D)).astype(dt) for i, s in enumerate(steps)]
    blob = struct.pack("7i", fmt_code, 0 if dt_name == "f32" else 1, Hq, Hkv, D, len(steps), freeze_at)
    blob += struct.pack(f"{len(steps)}i", *steps)
    for q, k, v in zip(qs, ks, vs):
        blob += q.tobytes() + k.tobytes() + v.tobytes()
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    fin.write_bytes(blob)
    r = subprocess.run([exe, str(fin), str(fout)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    raw = fout.read_bytes()
    es, off = np.dtype(dt).itemsize, 0

    def take(shape):
        nonlocal off
        n = int(np.prod(shape)) * es
        a = np.frombuffer(raw[off:off + n], dtype=dt).reshape(shape)
        off += n
        return a

    K = V = None
    first_pass = []
    for i, s in enumerate(steps):
        K = oracle.dyn_kv_concat(K, ks[i][None], axis=2)
        V = oracle.dyn_kv_concat(V, vs[i][None], axis=2)
        got = take((Hq, s, D))
        want = oracle.flash_sdpa(qs[i][None], K, V, causal=True)[0]
        assert rel_err(got.astype(np.float32), want.astype(np.float32)) <= TOL[dt_name], i
        first_pass.append(got)
    for i in range(freeze_at, len(steps)):  # resumed from the frozen state: the same bytes
        assert take((Hq, steps[i], D)).tobytes() == first_pass[i].tobytes()
    (length,) = struct.unpack("q", raw[off:off + 8])
    off += 8
    T = sum(steps)
    assert length == T
    assert take((Hkv, T, D)).tobytes() == K[0].tobytes()       # save_to K
    assert take((Hkv, T, D)).tobytes() == V[0].tobytes()       # save_to V
    assert take((Hkv, T, D)).tobytes() == K[0].tobytes()       # lone DynKeyValueCache output == concat
    lone = take((Hq, steps[-1], D))
    want = oracle.flash_sdpa(qs[-1][None], K, V, causal=True)[0]
    assert rel_err(lone.astype(np.float32), want.astype(np.float32)) <= TOL[dt_name]
    assert off == len(raw)
