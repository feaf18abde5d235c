"""Q4_0 weights x int8-quantised activations on the GPU: bit-exact against the CPU restatement of Q4_0::w4a8_gemm."""
import numpy as np
import pytest

import oracle
from util import normal, normal_with_outliers

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def kv():
    import tract_b200

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    tract_b200.lib()
    return tract_b200


def ggml_blocks(sc, pk):
    """The reference's storage: [N, K/32] blocks of 18 bytes, f16 scale (little endian) then 16 nibble bytes."""
    n, nb = sc.shape
    blob = np.empty((n, nb, 18), np.uint8)
    blob[:, :, :2] = sc.reshape(n, nb, 1).view(np.uint8)
    blob[:, :, 2:] = pk.reshape(n, nb, 16)
    return blob


@pytest.mark.parametrize("m,n,k,adt", [
    (1, 64, 64, "f32"),
    (5, 7, 64, "f32"),        # the shape of the reference's own GEMM test: a ragged tile of rows, 5 activation rows
    (4, 6, 96, "f32"),
    (8, 100, 4096, "f32"),    # 128 blocks: 16 stages of the ring
    (3, 48, 14336, "f16"),    # the FFN inner dimension of the Llama-3-8B shape: 448 blocks
    (1, 1024, 4096, "bf16"),  # a K/V projection
    (13, 40, 352, "f32"),     # two groups of activation rows, a last stage of 3 blocks
    (40, 64, 4096, "f32"),    # five groups of 8 rows: a CTA row with four groups sharing the weight stages, one with a single group
    (33, 32, 14336, "f16"),   # 8 warps per tile, a last group with one live row
    (257, 48, 4096, "f32"),   # many rows: 33 groups over 5 blocks of 8 warps, the last block with one warp, the last group with one row
    (64, 40, 14336, "f16"),   # exactly one block of 8 full groups, 56 stages through a 4-deep weight ring
    (100, 24, 352, "bf16"),   # a last stage of 3 blocks, fewer stages than the activation ring is deep... and a ragged tile
    (32, 16, 64, "f32"),      # one stage only
    # 128 rows and more: the tcgen05 kernel over the tiled activation layout
    (128, 130, 64, "f32"),    # one partly filled stage of two blocks; two column tiles, the second with two live columns
    (130, 48, 4096, "f32"),   # two row tiles, the second with two live rows; fewer weight rows than a column tile
    (512, 200, 352, "bf16"),  # 11 blocks: a last stage of 3; a ragged last column tile
    (300, 16, 14336, "f16"),  # 448 blocks: 112 stages through the rings, 16 weight rows in a 128-column tile
    (384, 256, 1024, "f32"),  # full tiles only
])
def test_q40_gemm_bit_exact(kv, m, n, k, adt):
    w = normal_with_outliers(11, (n, k)).astype(np.float32)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[adt]
    a_t = torch.from_numpy(normal(12, (m, k)).astype(np.float32)).to(tdt)
    sc, pk = oracle.q4_0_quant(w)
    lin = kv.Q40Linear(torch.from_numpy(ggml_blocks(sc, pk)).cuda(), max_m=max(64, m))
    got = lin.gemm(a_t.cuda()).cpu().numpy()
    lin.check()
    want = oracle.w4a8_gemm(sc, pk, a_t.float().numpy())
    assert got.tobytes() == want.tobytes()


def test_q40_gemm_special_activations(kv):
    # zero blocks (scale 1), a NaN inside a block (code 0, ignored by the maximum), a block of equal magnitudes
    n, k = 32, 128
    w = normal(21, (n, k)).astype(np.float32)
    a = normal(22, (2, k)).astype(np.float32)
    a[0, :32] = 0.0
    a[0, 40] = np.nan
    a[1, 96:] = -2.5
    sc, pk = oracle.q4_0_quant(w)
    lin = kv.Q40Linear(torch.from_numpy(ggml_blocks(sc, pk)).cuda())
    got = lin.gemm(torch.from_numpy(a).cuda()).cpu().numpy()
    want = oracle.w4a8_gemm(sc, pk, a)
    assert got.tobytes() == want.tobytes()


@pytest.mark.parametrize("m", [8, 40, 130])
def test_q40_gemm_with_weight_scales_that_are_not_finite(kv, m):
    # a weight block whose largest value overflows the f16 scale (inf), and one made of NaNs: the products with them are inf
    # or NaN exactly where the reference's are -- in particular inf * 0 = NaN for a zero dot product
    n, k = 48, 256
    w = normal(41, (n, k)).astype(np.float32)
    w[3, 32:64] = 9.0e5          # scale = max / -8 overflows f16
    w[17, 0:32] = np.nan
    a = normal(42, (m, k)).astype(np.float32)
    a[1, 32:64] = 0.0            # a zero activation block against the infinite scale
    sc, pk = oracle.q4_0_quant(w)
    assert not np.isfinite(sc.view(np.float16).astype(np.float32)).all()
    lin = kv.Q40Linear(torch.from_numpy(ggml_blocks(sc, pk)).cuda(), max_m=max(64, m))
    got = lin.gemm(torch.from_numpy(a).cuda()).cpu().numpy()
    lin.check()
    want = oracle.w4a8_gemm(sc, pk, a)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert got[ok].tobytes() == want[ok].tobytes()
    assert np.isnan(want).any() or np.isinf(want).any()


def test_q40_errors(kv):
    blocks = torch.zeros((4, 2, 18), dtype=torch.uint8, device="cuda")
    lin = kv.Q40Linear(blocks)
    with pytest.raises(kv.B200KvError):
        kv._ck(kv.lib().b200kv_q40_gemm(None, 4, 64, None, 64, 1, 0, None, None, 4, None))
    assert kv.lib().b200kv_q40_packed_bytes(4, 33) == -1
    assert lin.gemm(torch.zeros((1, 64), device="cuda")).abs().sum().item() == 0.0


@pytest.mark.parametrize("m,n,k", [(1, 48, 64), (8, 64, 4096), (5, 32, 14336), (19, 48, 512), (40, 32, 2048), (130, 48, 512), (200, 160, 2048)])
def test_fused_producers_give_the_bits_of_the_separate_calls(kv, m, n, k):
    # add -> RmsNorm * weight -> quantise -> GEMM and Silu(gate) * up -> quantise -> GEMM, fused into the quantiser, against
    # the same ops launched one by one, and the first of them against the CPU restatements composed the same way
    w = normal_with_outliers(31, (n, k)).astype(np.float32)
    sc, pk = oracle.q4_0_quant(w)
    lin = kv.Q40Linear(torch.from_numpy(ggml_blocks(sc, pk)).cuda(), max_m=max(64, m))
    scratch = torch.empty(kv.Q40Linear.scratch_bytes(k, m), dtype=torch.uint8, device="cuda")
    x = torch.from_numpy(normal_with_outliers(32, (m, k)).astype(np.float32)).cuda()
    res = torch.from_numpy(normal(33, (m, k)).astype(np.float32)).cuda()
    gain = torch.from_numpy((normal(34, (k,)) * 0.1 + 1.0).astype(np.float32)).cuda()
    eps = 1e-5
    # separate launches
    s = kv.add(x, res)
    want_norm = lin.gemm(kv.rms_norm(s, eps, weight=gain))
    # fused, the sum written in place of x
    x_io = x.clone()
    kv.q40_add_rms_norm_quantize(x_io, scratch, eps, weight=gain, residual=res, x_out=x_io)
    got = lin.gemm_quantized(m, scratch=scratch)
    lin.check(scratch)
    assert torch.equal(x_io, s)
    assert got.cpu().numpy().tobytes() == want_norm.cpu().numpy().tobytes()
    # fused, nothing written back; and without residual or weight
    kv.q40_add_rms_norm_quantize(x, scratch, eps, weight=gain, residual=res)
    assert torch.equal(lin.gemm_quantized(m, scratch=scratch), want_norm)
    kv.q40_add_rms_norm_quantize(s, scratch, eps)
    assert torch.equal(lin.gemm_quantized(m, scratch=scratch), lin.gemm(kv.rms_norm(s, eps)))
    # the oracle: its RmsNorm folds the squares left to right (1e-5 apart from the tree here), so compare as values
    ref = oracle.w4a8_gemm(sc, pk, (oracle.rms_norm(s.cpu().numpy(), eps) * gain.cpu().numpy()).astype(np.float32))
    err = np.abs(got.cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err < 2e-2, err  # quantiser flips of single codes; the bit-exact check is the one against the separate launches

    # gated activation: windows of one wide buffer, as the stacked gate / up GEMM leaves them
    gu = torch.from_numpy(normal(35, (m, 2 * k)).astype(np.float32) * 3).cuda()
    want_act = lin.gemm(kv.silu_mul(gu[:, :k].contiguous(), gu[:, k:].contiguous()))
    kv.q40_silu_mul_quantize(gu[:, :k], gu[:, k:], scratch)
    got_act = lin.gemm_quantized(m, scratch=scratch)
    assert torch.equal(got_act, want_act)
    ref_act = oracle.w4a8_gemm(sc, pk, (oracle.silu(gu[:, :k].cpu().numpy()) * gu[:, k:].cpu().numpy()).astype(np.float32))
    assert got_act.cpu().numpy().tobytes() == ref_act.tobytes()  # Silu and the product are bit-exact restatements
    # one quantisation feeding two matrices
    kv.q40_quantize(x, scratch)
    assert torch.equal(lin.gemm_quantized(m, scratch=scratch), lin.gemm(x))
    assert torch.equal(lin.gemm_quantized(m, scratch=scratch), lin.gemm(x))
    lin.check(scratch)


@pytest.mark.parametrize("odt", ["f16", "bf16"])
def test_gemm_result_stored_in_a_16_bit_type(kv, odt):
    # the Cast after the MatMul folded into the store: the f32 result rounded once
    m, n, k = 11, 80, 1024
    sc, pk = oracle.q4_0_quant(normal_with_outliers(41, (n, k)).astype(np.float32))
    lin = kv.Q40Linear(torch.from_numpy(ggml_blocks(sc, pk)).cuda(), max_m=16)
    a = torch.from_numpy(normal(42, (m, k)).astype(np.float32)).cuda()
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16}[odt]
    wide = torch.zeros((m, n + 48), dtype=tdt, device="cuda")  # a window of a wider buffer
    kv.q40_quantize(a, lin.scratch)
    lin.gemm_quantized(m, out=wide[:, 16:16 + n])
    lin.check()
    want = torch.from_numpy(oracle.w4a8_gemm(sc, pk, a.cpu().numpy())).to(tdt)
    assert torch.equal(wide[:, 16:16 + n].cpu(), want)
    assert not wide[:, :16].any() and not wide[:, 16 + n:].any()
