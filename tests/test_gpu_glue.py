"""RmsNorm, SiLU * up, residual add, argmax and row gather on the GPU against the CPU restatement of tract's generic kernels."""
import numpy as np
import pytest

import oracle
from util import normal, rel_err

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def kv():
    import tract_b200

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    tract_b200.lib()
    return tract_b200


@pytest.mark.parametrize("rows,d,dt", [(1, 4, "f32"), (8, 4096, "f32"), (3, 100, "f32"), (8, 4096, "f16"), (5, 14336, "f16")])
def test_rms_norm(kv, rows, d, dt):
    npdt = np.float32 if dt == "f32" else np.float16
    x = (normal(41, (rows, d)) * 3).astype(npdt)
    got = kv.rms_norm(torch.from_numpy(x).cuda(), 1e-5).cpu().numpy()
    want = oracle.rms_norm(x, 1e-5)
    # the reference's own tests hold this kernel to 1e-5; the sum of squares is a tree here, a left-to-right fold there
    if dt == "f32":
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    else:
        assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 2.0 ** -10 * np.abs(want.astype(np.float32)).max()
    w = normal(42, (d,)).astype(npdt)
    got_w = kv.rms_norm(torch.from_numpy(x).cuda(), 1e-5, weight=torch.from_numpy(w).cuda()).cpu().numpy()
    assert np.array_equal(got_w, (got.astype(np.float32) * w.astype(np.float32)).astype(npdt))  # the fused Mul, on the kernel's own norm


def test_rms_norm_known_answers(kv):
    got = kv.rms_norm(torch.tensor([[1.0, 2.0, 3.0, 4.0]], device="cuda"), 0.0).cpu().numpy()
    assert np.allclose(got, np.arange(1, 5, dtype=np.float32) / np.sqrt(np.float32(7.5)), atol=1e-6)
    z = kv.rms_norm(torch.zeros((2, 8), device="cuda"), 1e-5).cpu().numpy()
    assert not z.any()


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_silu_mul_bit_exact(kv, dt):
    npdt = np.float32 if dt == "f32" else np.float16
    g = np.concatenate([np.linspace(-25, 25, 5001), normal(51, (3000,)) * 4, [0.0, -0.0, np.inf, -np.inf, 1e-30]]).astype(npdt)
    u = normal(52, g.shape).astype(npdt)
    silu, silu_want = kv.silu_mul(torch.from_numpy(g).cuda()).cpu().numpy(), oracle.silu(g)
    finite = ~np.isnan(silu_want)  # -inf * 0 gives a NaN whose bits differ between CPU and GPU
    assert silu[finite].tobytes() == silu_want[finite].tobytes() and np.isnan(silu[~finite]).all()
    got = kv.silu_mul(torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda()).cpu().numpy()
    want = (oracle.silu(g).astype(np.float32) * u.astype(np.float32)).astype(npdt)
    keep = ~np.isnan(want)  # inf * 0 gives a NaN whose bits differ between CPU and GPU
    assert np.array_equal(got[keep], want[keep]) and np.isnan(got[~keep]).all()


def test_add_argmax_gather(kv):
    a, b = normal(61, (7, 4096)).astype(np.float16), normal(62, (7, 4096)).astype(np.float16)
    got = kv.add(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    assert np.array_equal(got, (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16))
    logits = normal(63, (9, 128256)).astype(np.float32)
    logits[2, 500] = logits[2, 90000] = 99.0  # a tie: the first index wins
    logits[3, 7] = np.nan
    want = np.array([np.nanargmax(r) for r in logits], np.int32)
    want[2] = 500
    assert np.array_equal(kv.argmax(torch.from_numpy(logits).cuda()).cpu().numpy(), want)
    table = normal(64, (1000, 256)).astype(np.float16)
    ids = np.array([5, 999, 0, 5, 123], np.int32)
    assert np.array_equal(kv.gather_rows(torch.from_numpy(table).cuda(), torch.from_numpy(ids).cuda()).cpu().numpy(), table[ids])


@pytest.mark.parametrize("n,offset", [(1, 0), (3, 0), (1027, 0), (1027, 1), (4096, 2), (4099, 3), (128256, 0), (20001, 1)])
def test_argmax_rows_of_any_length_and_alignment(kv, n, offset):
    # rows that start off a 16-byte boundary take the scalar walk, aligned ones the 16-byte loads plus a scalar tail;
    # the maximum sits in the tail, at the front and on a tie in turn
    rows = 5
    wide = torch.from_numpy(normal(71 + n, (rows, n + 8)).astype(np.float32)).cuda()
    x = wide[:, offset:offset + n]
    host = x.cpu().numpy().copy()
    host[0, n - 1] = 50.0
    host[1, 0] = 50.0
    host[2, n // 2] = host[2, n - 1] = 50.0
    host[3, :] = -np.inf
    x.copy_(torch.from_numpy(host))
    want = np.array([n - 1, 0, n // 2, 0, int(np.argmax(host[4]))], np.int32)
    assert np.array_equal(kv.argmax(x).cpu().numpy(), want)
