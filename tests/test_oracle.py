"""Pins the CPU oracle: golden bundles of the reference, its unit-test known answers, and an
independent numpy restatement of every quantiser (the quantised formats have no golden vector
in the reference, so two independently written restatements must agree bit for bit)."""
import numpy as np
import pytest

import oracle
from util import lcg_tensor, normal, normal_with_outliers, ramp, rel_err


# ---- golden bundles: harness/nnef-test-cases/sdpa/*/io.npz --------------------------------------

ATTN_CASES = ["simple-causal-f32", "simple-non-causal-f32", "simple-scale-f32", "simple-f16", "simple-mask-f32"]


def bundle_inputs(golden, case):
    z, meta = golden
    a = meta[case]
    q, k, v = (z[f"{case}/{n}"] for n in a["qkv"])
    mask = z[f"{case}/mask"] if f"{case}/mask" in z.files else None
    if a["dtype"] == "f16":
        q, k, v = (x.astype(np.float16) for x in (q, k, v))
    return q, k, v, mask, a, z[f"{case}/output_0"]


@pytest.mark.parametrize("case", ATTN_CASES)
def test_flash_oracle_matches_reference_bundle(golden, case):
    q, k, v, mask, a, want = bundle_inputs(golden, case)
    got = oracle.flash_sdpa(q, k, v, mask=mask, scale=a["scale"], causal=a["causal"]).astype(np.float32)
    # the reference's CI checks these bundles with Approximation::Close (f32) / Approximate (f16)
    atol, rtol = (1e-3, 5e-3) if a["dtype"] == "f16" else (1e-7, 1e-7)
    assert np.all(np.abs(got - want) <= atol + rtol * np.abs(want) + 1.2e-7), np.abs(got - want).max()


@pytest.mark.parametrize("case", ATTN_CASES)
def test_naive_f64_matches_reference_bundle(golden, case):
    q, k, v, mask, a, want = bundle_inputs(golden, case)
    got = oracle.naive_sdpa_f64(q, k, v, mask=mask, scale=a["scale"], causal=a["causal"])
    tol = 3e-4 if a["dtype"] == "f16" else 2e-7  # f32 bundles: half an ulp of the stored f32 answer
    assert np.all(np.abs(got - want) <= tol + 1.2e-7 * np.abs(want))


def test_gqa_bundle_pins_cache_append(golden):
    z, _ = golden
    c = "simple-grouped-query-att-f32"
    for i_in, i_out in ((1, 1), (2, 2)):
        past, after = z[f"{c}/input_{i_in}"], z[f"{c}/output_{i_out}"]
        assert after.shape == (1, 2, 11, 2)
        got = oracle.dyn_kv_concat(past, after[:, :, 10:], axis=2)
        assert got.tobytes() == after.tobytes()


# ---- reference unit tests restated ------------------------------------------------------------

def test_flash_vs_naive_like_reference_unit_test():
    # flash_sdpa.rs:360-405: B=2, Hq=4, Hkv=2 shapes, LCG inputs, max_abs < 1e-5 vs naive
    for (b, hq, hkv, s, t, d, causal) in [(2, 4, 2, 7, 40, 16, False), (1, 4, 2, 33, 33, 64, True),
                                          (1, 8, 2, 1, 100, 32, True), (2, 2, 1, 40, 75, 8, False)]:
        q, k, v = lcg_tensor(1, (b, hq, s, d)), lcg_tensor(2, (b, hkv, t, d)), lcg_tensor(3, (b, hkv, t, d))
        got = oracle.flash_sdpa(q, k, v, causal=causal)
        want = oracle.naive_sdpa_f64(q, k, v, causal=causal)
        assert np.abs(got - want).max() < 1e-5


def test_flash_f16_vs_f32_like_reference_unit_test():
    # flash_sdpa.rs:407-435: GQA 4/2, causal, S=1, T=33; f16 eval within 5e-3 of the f32 eval
    q, k, v = lcg_tensor(11, (1, 4, 1, 64)), lcg_tensor(12, (1, 2, 33, 64)), lcg_tensor(13, (1, 2, 33, 64))
    o32 = oracle.flash_sdpa(q, k, v, causal=True)
    o16 = oracle.flash_sdpa(q.astype(np.float16), k.astype(np.float16), v.astype(np.float16), causal=True)
    assert o16.dtype == np.float16
    assert np.abs(o16.astype(np.float32) - o32).max() < 5e-3


HAND_CASES = {
    # test-rt/suite-unit/src/sdpa.rs:346-549 (inputs are literals; expected = the suite's naive attention)
    "trivial_f32_0": dict(q=np.zeros((1, 1, 1)), k=np.zeros((1, 1, 1)), v=np.zeros((1, 1, 1)), causal=True),
    "causal_f32_1": dict(q=np.zeros((1, 2, 1)), k=np.zeros((1, 2, 1)), v=np.zeros((1, 2, 1)), causal=True),
    "causal_with_s_and_p_0": dict(q=np.zeros((1, 2, 1)), k=np.zeros((1, 3, 1)),
                                  v=np.array([[[0.0], [0.0], [1.0]]]), causal=True),
    "gqa_f32_0": dict(q=np.zeros((1, 2, 1, 1)), k=np.zeros((1, 2, 1, 1)), v=np.array([[[[0.0]], [[1.0]]]]),
                      causal=False),
    "gqa_f32_1": dict(q=np.zeros((1, 2, 1, 1)), k=np.zeros((1, 1, 1, 1)), v=np.zeros((1, 1, 1, 1)), causal=False),
}


@pytest.mark.parametrize("name", sorted(HAND_CASES))
def test_hand_written_regressions(name):
    c = HAND_CASES[name]
    q, k, v = (c[n].astype(np.float32) for n in "qkv")
    got = oracle.flash_sdpa(q, k, v, causal=c["causal"])
    want = oracle.naive_sdpa_f64(q, k, v, causal=c["causal"])
    assert np.abs(got - want).max() <= 1e-6
    if name == "causal_with_s_and_p_0":  # row 0 sees keys 0..1 -> 0 ; row 1 sees 0..2 -> 1/3
        assert np.allclose(got.reshape(-1), [0.0, 1.0 / 3.0], atol=1e-7)
    if name == "gqa_f32_0":
        assert got.reshape(-1).tolist() == [0.0, 1.0]


def test_property_sweep_flash_vs_naive():
    # the proptest strategy of test-rt/suite-unit/src/sdpa.rs:94-142: values k/8, k in [-3, 3]
    g = np.random.default_rng(7)
    for _ in range(60):
        b, rep, hkv = g.integers(1, 3), g.integers(1, 5), g.integers(1, 5)
        p, s, d = g.integers(0, 5), g.integers(2, 5), int(g.choice([1, 2, 3, 64, 128]))
        hq = rep * hkv
        mk = lambda shape: (g.integers(-3, 4, size=shape) / 8.0).astype(np.float32)
        q, k, v = mk((b, hq, s, d)), mk((b, hkv, p + s, d)), mk((b, hkv, p + s, d))
        causal = bool(g.integers(0, 2))
        mask = None
        if not causal and g.integers(0, 2):
            mask = mk((b if g.integers(0, 2) else 1, hq if g.integers(0, 2) else 1, s, p + s))
        scale = float(g.uniform(0.1, 1.0)) if g.integers(0, 2) else None
        got = oracle.flash_sdpa(q, k, v, mask=mask, scale=scale, causal=causal)
        want = oracle.naive_sdpa_f64(q, k, v, mask=mask, scale=scale, causal=causal)
        assert np.abs(got - want).max() < 1e-5


def test_threads_do_not_change_result():
    q, k, v = normal(1, (2, 8, 5, 64)), normal(2, (2, 2, 70, 64)), normal(3, (2, 2, 70, 64))
    a = oracle.flash_sdpa(q, k, v, causal=True, threads=1)
    b = oracle.flash_sdpa(q, k, v, causal=True, threads=4)
    assert a.tobytes() == b.tobytes()


# ---- DynKeyValueCache: cache == concat of all pushes (dyn_kv_cache.rs:422-505, inplace_kv_cache.rs:366-386) ----

@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_dyn_kv_concat_is_concat(dtype):
    chunks = [ramp((1, 2, s, 4), start=i * 100.0, dtype=dtype) for i, s in enumerate([5] + [1] * 20)]
    cache = None
    for c in chunks:
        cache = oracle.dyn_kv_concat(cache, c, axis=2)
    assert cache.tobytes() == np.concatenate(chunks, axis=2).tobytes()


# ---- f16 conversion ----------------------------------------------------------------------------

def test_f16_conversion_matches_numpy_everywhere():
    L = oracle.lib()
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    f = allh.view(np.float16).astype(np.float32)
    for h in allh[::17]:
        x = L.orc_f16_to_f32(int(h))
        assert np.float32(x).tobytes() == f[h].tobytes() or (np.isnan(x) and np.isnan(f[h]))
    g = np.random.default_rng(0)
    xs = np.concatenate([g.standard_normal(20000).astype(np.float32) * 10.0 ** g.integers(-9, 6, 20000),
                         np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                                   np.inf, -np.inf, 6.1035156e-5, 6.0975552e-5], np.float32)]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([L.orc_f32_to_f16(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, want)


# ---- block quantisers: known answers + independent numpy restatement ---------------------------------

def np_round_half_away(x):
    return np.where(x >= 0, np.floor(x + np.float32(0.5)), np.ceil(x - np.float32(0.5))).astype(np.float32)


def np_signed_max(x):
    """First element of largest |v| per block of 32 (strictly greater replaces)."""
    a = np.where(np.isnan(x), np.float32(-1), np.abs(x))  # `amax < |v|` is false for NaN: NaN never wins
    idx = np.argmax(a, axis=-1)  # argmax returns the first maximum
    return np.take_along_axis(x, idx[..., None], -1)[..., 0]


def np_q8_1(x):
    x = x.reshape(-1, 32).astype(np.float32)
    mx = np_signed_max(x)
    scale = (mx / np.float32(127)).astype(np.float32)
    with np.errstate(divide="ignore"):
        r = np.where(scale == 0, np.float32(0), np.float32(1) / scale).astype(np.float32)
    t = (x * r[:, None]).astype(np.float32)
    rounded = np.where(np.abs(t) < 2 ** 23, np.sign(t) * np.floor(np.abs(t) + np.float32(0.5)), t)
    codes = np.clip(np.nan_to_num(rounded, nan=0.0), -128, 127).astype(np.int8)
    return scale.astype(np.float16).view(np.uint16), codes


def np_q4_0(x):
    x = x.reshape(-1, 32).astype(np.float32)
    mx = np_signed_max(x)
    scale = (mx / np.float32(-8)).astype(np.float32)
    with np.errstate(divide="ignore"):
        r = np.where(scale == 0, np.float32(0), np.float32(1) / scale).astype(np.float32)
    t = ((x * r[:, None]).astype(np.float32) + np.float32(8.5)).astype(np.float32)
    c = np.minimum(np.clip(np.trunc(np.nan_to_num(t, nan=0.0)), -128, 127), 15).astype(np.int8).astype(np.uint8)
    # helpers.rs:57-68 writes `first as u8 | (second as u8) << 4` without masking the first code: a
    # negative code (only reachable through an infinite reciprocal of a subnormal scale) leaks into
    # the high nibble, and that is what the reference stores.
    packed = (c[:, :16].astype(np.uint16) | (c[:, 16:].astype(np.uint16) << 4)) & 0xFF
    return scale.astype(np.float16).view(np.uint16), packed.astype(np.uint8)


def pad32(v):
    v = list(v)
    return np.array(v + [0.0] * (-len(v) % 32), np.float32)


@pytest.mark.parametrize("data", [[1, 2, 3, 4], [-1, -2, -3, -4], [1234.0], [-1234.0]])
def test_q4_0_round_trip_known_answers(data):
    # q4_0.rs:505-535: quant -> dequant returns the input exactly
    x = pad32(data)
    s, p = oracle.q4_0_quant(x)
    assert np.array_equal(oracle.q4_0_dequant(s, p)[: len(data)], np.array(data, np.float32))


@pytest.mark.parametrize("data", [[1, 2, 3, 4], [-1, -2, -3, -4], [1234.0], [-1234.0]])
def test_q8_1_round_trip_known_answers(data):
    # q8_1.rs:348-383: quant -> dequant within VeryApproximate (atol 5e-2, rtol 1e-2)
    x = pad32(data)
    s, _, c = oracle.q8_1_quant(x)
    back = oracle.q8_1_dequant(s, c)
    assert np.all(np.abs(back - x) <= 5e-2 + 1e-2 * np.abs(x))


@pytest.mark.parametrize("fmt", ["q4_0", "q8_1"])
def test_extract_known_answers(fmt):
    # q4_0.rs:589-593 / q8_1.rs:397-401: ((i % 14) - 6) for i in 1.., 5 blocks; round(dequant) == value
    data = np.array([((i % 14) - 6) for i in range(1, 1 + 5 * 32)], np.float32)
    if fmt == "q4_0":
        back = oracle.q4_0_dequant(*oracle.q4_0_quant(data))
    else:
        s, _, c = oracle.q8_1_quant(data)
        back = oracle.q8_1_dequant(s, c)
    assert np.array_equal(np_round_half_away(back), data)


def test_q4_0_nibble_order_and_prequantized_answer():
    # q4_0.rs:722-739 layout: byte j = element j (low nibble) | element j+16 (high nibble); dequant (n-8)*scale
    nib = (np.arange(64) % 16).astype(np.uint8).reshape(2, 32)
    packed = (nib[:, :16] | (nib[:, 16:] << 4)).astype(np.uint8)
    scales = np.array([0.5, 2.0], np.float16).view(np.uint16)
    got = oracle.q4_0_dequant(scales, packed.reshape(1, 32)).reshape(2, 32)
    want = (nib.astype(np.float32) - 8.0) * np.array([[0.5], [2.0]], np.float32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_block_quantisers_match_independent_numpy(seed):
    x = normal_with_outliers(seed, (257, 128))
    x[3, :32] = 0.0          # all-zero block -> scale 0, r 0
    x[4, 5] = -x[4, 9]       # tie in |v|: the first occurrence wins
    x[5, :32] = 1e-42        # subnormal scale
    x[6, 0] = np.inf
    x[7, 1] = np.nan
    s, _, c = oracle.q8_1_quant(x)
    with np.errstate(invalid="ignore", over="ignore"):
        s2, c2 = np_q8_1(x)
    assert np.array_equal(s.reshape(-1), s2) and np.array_equal(c.reshape(-1, 32), c2)
    s, p = oracle.q4_0_quant(x)
    with np.errstate(invalid="ignore", over="ignore"):
        s2, p2 = np_q4_0(x)
    assert np.array_equal(s.reshape(-1), s2) and np.array_equal(p.reshape(-1, 16), p2)


# ---- QuantizedDynKeyValueCache (KIVI) -------------------------------------------------------------

def np_kivi_codes(x, lo, scale, lv):
    t = ((x - lo).astype(np.float32) / scale).astype(np.float32)
    r = np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))
    return np.clip(r, 0, lv).astype(np.uint8)


@pytest.mark.parametrize("bits", [8, 4])
def test_kivi_value_store_matches_numpy(bits):
    d, lv = 64, np.float32(2 ** bits - 1)
    x = normal_with_outliers(5, (40, d))
    x[10] = 3.0  # hi == lo -> scale 1
    st = oracle.KiviStore(False, d, bits)
    st.push(x)
    raw = st.raw()
    assert len(st) == 40 and np.array_equal(raw["sink"], x[:4])
    lo, hi = x[4:].min(1), x[4:].max(1)
    scale = np.where(hi > lo, ((hi - lo) / lv).astype(np.float32), np.float32(1))
    codes = np_kivi_codes(x[4:], lo[:, None], scale[:, None], lv)
    if bits == 4:
        codes = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    assert np.array_equal(raw["lo"], lo) and np.array_equal(raw["scale"], scale)
    assert np.array_equal(raw["codes"], codes)


@pytest.mark.parametrize("bits", [8, 4])
def test_kivi_key_store_blocks_freeze(bits):
    d, lv = 32, np.float32(2 ** bits - 1)
    x = normal(9, (4 + 32 * 2 + 5, d))
    st = oracle.KiviStore(True, d, bits)
    st.push(x[:50])
    before = st.raw()
    st.push(x[50:])
    raw = st.raw()
    # the first block was finalised at token 36 and must not change afterwards (:760-783)
    rb = st.row_bytes
    assert np.array_equal(raw["codes"][:32], before["codes"][:32]) and rb == d * bits // 8
    assert np.array_equal(raw["residual"], x[68:]) and raw["lo"].size == 2 * d
    blk = x[4:36]
    lo, hi = blk.min(0), blk.max(0)
    scale = np.where(hi > lo, ((hi - lo) / lv).astype(np.float32), np.float32(1))
    codes = np_kivi_codes(blk, lo[None], scale[None], lv)
    if bits == 4:
        codes = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    assert np.array_equal(raw["codes"][:32], codes) and np.array_equal(raw["lo"][:d], lo)
    deq = st.dequant()
    assert np.array_equal(deq[:4], x[:4]) and np.array_equal(deq[68:], x[68:])
    assert np.abs(deq - x).max() <= 0.51 * raw["scale"].max() + 1e-6


@pytest.mark.parametrize("per_channel", [False, True])
def test_quantized_cache_close_to_concat_over_40_steps(per_channel):
    # quant_dyn_kv_cache.rs:728-756: 40 single-token steps, int8 cache ~ concat (SuperApproximate: 0.1 / 0.05)
    cache, chunks = oracle.QuantizedDynKeyValueCache(8, per_channel), []
    for i in range(40):
        c = normal(100 + i, (1, 2, 1, 16))
        chunks.append(c)
        out = cache.eval(c)
    want = np.concatenate(chunks, 2)
    assert out.shape == want.shape and np.all(np.abs(out - want) <= 0.1 + 0.05 * np.abs(want))


# ---- Q4_0 weights x int8 activations (q4_0.rs:199-310): the reference's own tests for the path, restated ----

def _w4a8_case(m, n, k, fw, fa):
    wf = np.array([fw(i) for i in range(n * k)], np.float32).reshape(n, k)
    a = np.array([fa(i) for i in range(m * k)], np.float32).reshape(m, k)
    sc, pk = oracle.q4_0_quant(wf)
    return a, sc, pk, oracle.w4a8_gemm(sc, pk, a, threads=2)


def test_w4a8_gemm_matches_gemv():
    # q4_0.rs:538-550: the GEMM is bit-identical to the GEMV run per activation row
    a, sc, pk, out = _w4a8_case(5, 7, 64, lambda i: ((i * 37 % 53) - 26.0) / 9.0, lambda i: ((i * 19 % 41) - 20.0) / 7.0)
    for mi in range(5):
        assert np.array_equal(oracle.w4a8_gemm(sc, pk, a[mi:mi + 1], threads=1)[0], out[mi])


def test_w4a8_gemm_approx_dequant_matmul():
    # q4_0.rs:553-575: within 0.15 |acc| + 1 of the sequential f32 product over the dequantised weights
    a, sc, pk, out = _w4a8_case(4, 6, 96, lambda i: ((i * 31 % 47) - 23.0) / 11.0, lambda i: ((i * 23 % 43) - 21.0) / 8.0)
    wd = oracle.q4_0_dequant(sc, pk)
    for mi in range(4):
        for ni in range(6):
            acc = np.float32(0)
            for ki in range(96):
                acc = np.float32(acc + np.float32(wd[ni, ki] * a[mi, ki]))
            assert abs(out[mi, ni] - acc) <= 0.15 * abs(acc) + 1.0


def test_w4a8_gemv_near_f32_dequant():
    # q4_0.rs:697-720: the reference's LCG inputs; relative L2 deviation from the f32-dequant GEMV below 2 %
    n, k = 8, 64
    state = 1
    vals = []
    for _ in range(n * k + k):
        state = (state * 6364136223846793005 + 1) % (1 << 64)
        vals.append(np.float32(np.float32(state >> 40) / np.float32(1 << 24)) - np.float32(0.5))
    w = np.array(vals[:n * k], np.float32).reshape(n, k)
    a = np.array(vals[n * k:], np.float32).reshape(1, k)
    sc, pk = oracle.q4_0_quant(w)
    deq = oracle.q4_0_dequant(sc, pk)
    y_ref = np.zeros(n, np.float32)
    for ni in range(n):
        for kk in range(k):
            y_ref[ni] = np.float32(y_ref[ni] + np.float32(deq[ni, kk] * a[0, kk]))
    y = oracle.w4a8_gemm(sc, pk, a)[0]
    assert np.sqrt(((y - y_ref) ** 2).sum()) / max(np.sqrt((y_ref ** 2).sum()), 1e-9) < 0.02


def test_w4a8_activation_quantiser_edges():
    # q4_0.rs:199-214: an all-zero block takes scale 1; the largest magnitude maps to +-127; a NaN becomes code 0
    a = np.zeros((1, 96), np.float32)
    a[0, 32:64] = np.linspace(-3, 5, 32, dtype=np.float32)
    a[0, 64] = np.nan
    a[0, 65] = 2.0
    q, sc = oracle.w4a8_quantize_row(a)
    assert sc[0, 0] == 1.0 and not q[0, :32].any()
    assert sc[0, 1] == np.float32(5.0) / np.float32(127.0) and q[0, 63] == 127 and q[0, 32] == round(-3 / (5 / 127))
    assert q[0, 64] == 0 and q[0, 65] == 127 and sc[0, 2] == np.float32(2.0) / np.float32(127.0)


# ---- decoder glue: the reference's own known answers -----------------------------------------------------

def test_rms_norm_known_answers():
    # linalg/src/generic/rms_norm.rs:28-61
    assert np.allclose(oracle.rms_norm(np.ones((1, 16), np.float32), 0.0), 1.0, atol=1e-5)
    got = oracle.rms_norm(np.array([[1.0, 2.0, 3.0, 4.0]], np.float32), 0.0)
    assert np.allclose(got, np.arange(1, 5, dtype=np.float32) / np.sqrt(np.float32(7.5)), atol=1e-5)
    z = oracle.rms_norm(np.zeros((1, 4), np.float32), 1e-5)
    assert np.isfinite(z).all() and not z.any()


def test_ssigmoid_and_silu_properties():
    # the rational fit stays within 2e-7 of the exact sigmoid, saturates to exactly 0 / 1, keeps NaN, and SiLU is x * sigmoid(x)
    x = np.linspace(-30, 30, 4001, dtype=np.float32)
    s = oracle.ssigmoid(x)
    exact = 1.0 / (1.0 + np.exp(-x.astype(np.float64)))
    assert np.abs(s - exact).max() < 2e-7
    assert s.min() >= 0.0 and s.max() <= 1.0 and s[0] < 1e-7 and s[-1] > 1 - 1e-7
    assert np.isnan(oracle.ssigmoid(np.array([np.nan], np.float32))[0])
    assert np.array_equal(oracle.silu(x), x * s)
    h = x.astype(np.float16)
    assert np.array_equal(oracle.silu(h), (h.astype(np.float32) * oracle.ssigmoid(h.astype(np.float32))).astype(np.float16))
