"""Parity of the CUDA path (through the C ABI) with the CPU oracle, on a B200.

Bar: cache contents, codes and scales bit-exact; attention within 2e-3 (f16 / bf16) and 1e-5 (f32)
of the oracle under util.rel_err.
"""
import numpy as np
import pytest

import oracle
from util import TOL, lcg_tensor, normal, normal_with_outliers, ramp, rel_err, rel_err_bf16

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def kv():
    import tract_b200

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    tract_b200.lib()  # fails loudly if the extension is missing
    return tract_b200


TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def np_dtype(name):
    return {"f32": np.float32, "f16": np.float16, "bf16": oracle.bfloat16}[name]


def to_dev(a, name=None):
    """numpy (incl. ml_dtypes bf16) -> CUDA tensor."""
    if a.dtype == np.float32 or a.dtype == np.float16:
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint16).copy()).view(torch.bfloat16).cuda()


def attn_err(out, io, q, k, v, **kw):
    """Error of a GPU attention output against the oracle run on the same inputs (see util.rel_err_bf16)."""
    if io == "bf16":
        want = oracle.flash_sdpa(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), **kw)
        return rel_err_bf16(to_np(out, io).astype(np.float32), want)
    want = oracle.flash_sdpa(q, k, v, **kw)
    return rel_err(to_np(out, io).astype(np.float32), want.astype(np.float32))


LAYOUTS = ["plain", "window", "offset"]


def as_layout(t, layout):
    """The values of t ([B, H, S, D]) in a tensor laid out three ways, as the reference's test runtime runs every case
    (test-rt/test-cuda/src/lib.rs:218-220): as they are; as a window of a wider buffer (every stride but the innermost
    differs from the dense one); or dense but starting one element past a 16-byte boundary (a 2- or 4-byte aligned base)."""
    if layout == "plain":
        return t
    B, H, S, D = t.shape
    if layout == "window":
        buf = torch.full((B + 1, H + 2, S + 1, D), 7.0, dtype=t.dtype, device=t.device)
        w = buf[1:, 1:H + 1, 1:]
    else:
        flat = torch.full((t.numel() + 8,), 7.0, dtype=t.dtype, device=t.device)
        w = flat[1:1 + t.numel()].view(B, H, S, D)
    w.copy_(t)
    return w


def to_np(t, name):
    t = t.detach().cpu().contiguous()
    if name == "bf16":
        return t.view(torch.uint16).numpy().view(oracle.bfloat16)
    return t.numpy()


# ---- append: DynKeyValueCache semantics, bit-exact ----------------------------------------------

@pytest.mark.parametrize("name", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("D", [128, 64])
def test_append_equals_concat_bit_exact(kv, name, D):
    # inplace_kv_cache.rs:388-399 drive: a prompt of 5 then 20 single-token steps; here for 3 sequences at once,
    # crossing a page boundary (64 tokens) on the way
    H, B = 2, 3
    cache = kv.KvCache(name, H, D, max_seqs=4, max_seq_tokens=256)
    seqs = [cache.new_seq() for _ in range(B)]
    ref_k = ref_v = None
    for i, s in enumerate([5] + [1] * 20 + [50, 3]):
        k = normal(10 + i, (B, H, s, D)).astype(np_dtype(name))
        v = ramp((B, H, s, D), start=i * 100.0).astype(np_dtype(name))
        cache.append(seqs, to_dev(k), to_dev(v))
        ref_k, ref_v = oracle.dyn_kv_concat(ref_k, k), oracle.dyn_kv_concat(ref_v, v)
    cache.check()
    for b, sq in enumerate(seqs):
        assert cache.seq_len(sq) == ref_k.shape[2]
        gk, gv = cache.export(sq, TDT[name])
        assert to_np(gk, name).tobytes() == ref_k[b].tobytes()
        assert to_np(gv, name).tobytes() == ref_v[b].tobytes()
    cache.close()


def test_append_strided_and_k_only(kv):
    # the reference runs every case with transposed (strided) inputs too (test-rt/test-cuda/src/lib.rs:218-220);
    # a lone DynKeyValueCache node holds a single tensor
    H, D = 2, 128
    cache = kv.KvCache("f16", H, D, max_seqs=1, max_seq_tokens=128, has_values=False)
    sq = cache.new_seq()
    x = normal(3, (1, 7, H, D)).astype(np.float16)         # [B, S, H, D] in memory
    xt = to_dev(x).permute(0, 2, 1, 3)                      # logical [B, H, S, D], strided
    cache.append([sq], xt)
    off = torch.zeros(1 * H * 3 * D + 1, dtype=torch.float16, device="cuda")[1:].view(1, H, 3, D)  # 2-byte aligned only
    y = normal(4, (1, H, 3, D)).astype(np.float16)
    off.copy_(to_dev(y))
    cache.append([sq], off)
    gk, gv = cache.export(sq, torch.float16)
    assert gv is None
    want = np.concatenate([x.transpose(0, 2, 1, 3), y], axis=2)[0]
    assert to_np(gk, "f16").tobytes() == want.tobytes()
    cache.close()


# ---- quantise-on-append: codes and scales bit-exact ----------------------------------------------

def nasty(seed, shape):
    x = normal_with_outliers(seed, shape)
    f = x.reshape(-1, 32)
    f[3] = 0.0                      # all-zero block: scale 0, reciprocal 0
    f[4, 5] = -f[4, 9]              # tie in magnitude: first occurrence wins
    f[5, 17] = -f[5, 2]             # tie across the two 16-element halves of a block
    f[6] = 1e-42                    # subnormal scale, infinite reciprocal
    f[7, 0] = np.inf
    f[8, 1] = np.nan
    f[9] = np.float32(65504.0) * 130.0  # f16 scale overflows to inf
    f[10, :] = np.arange(32) - 15.5     # exact .5 products: round half away from zero
    return x


@pytest.mark.parametrize("fmt", ["q8_1", "q4_0"])
@pytest.mark.parametrize("in_name", ["f32", "f16"])
@pytest.mark.parametrize("D", [128, 64])
def test_quantise_on_append_bit_exact(kv, fmt, in_name, D):
    H, B = 4, 2
    cache = kv.KvCache(fmt, H, D, max_seqs=B, max_seq_tokens=512)
    seqs = [cache.new_seq() for _ in range(B)]
    chunks_k, chunks_v = [], []
    for i, s in enumerate([70, 1, 1, 1, 130, 1]):
        with np.errstate(over="ignore", invalid="ignore"):
            k = nasty(20 + i, (B, H, s, D)).astype(np_dtype(in_name))
            v = normal_with_outliers(40 + i, (B, H, s, D)).astype(np_dtype(in_name))
        cache.append(seqs, to_dev(k), to_dev(v))
        chunks_k.append(k), chunks_v.append(v)
    cache.check()
    K, V = np.concatenate(chunks_k, 2), np.concatenate(chunks_v, 2)
    for b, sq in enumerate(seqs):
        for which, X in ((0, K), (1, V)):
            codes, scales = cache.export_codes(sq, which)
            codes, scales = codes.cpu().numpy(), scales.cpu().view(torch.uint16).numpy()
            if fmt == "q8_1":
                s_ref, _, c_ref = oracle.q8_1_quant(X[b])
            else:
                s_ref, c_ref = oracle.q4_0_quant(X[b])
            assert np.array_equal(scales, s_ref), (fmt, which)
            assert np.array_equal(codes, c_ref), (fmt, which)
        # dequantised export == oracle dequant, bit for bit in f32
        gk, gv = cache.export(sq, torch.float32)
        if fmt == "q8_1":
            s_ref, _, c_ref = oracle.q8_1_quant(V[b])
            want = oracle.q8_1_dequant(s_ref, c_ref)
        else:
            want = oracle.q4_0_dequant(*oracle.q4_0_quant(V[b]))
        assert gv.cpu().numpy().tobytes() == want.tobytes()
    cache.close()


# ---- decode attention ------------------------------------------------------------------------------

def oracle_cache_view(fmt, X, io_name):
    """What the fused cache + attention op attends over: the concatenated tensor itself, or, for a
    quantised cache, the dequantised f32 values (the reference's fused ops work in f32 internally:
    inplace_kv_cache.rs:201-206, kv_quant.rs:246-349; only the op OUTPUT is cast back to the model
    dtype).  The unfused chain, whose cache output is cast to the model dtype first
    (quant_dyn_kv_cache.rs:493), is what b200kv_export reproduces."""
    if fmt == "q8_1":
        s, _, c = oracle.q8_1_quant(X)
        return oracle.q8_1_dequant(s, c)
    if fmt == "q4_0":
        return oracle.q4_0_dequant(*oracle.q4_0_quant(X))
    return X


DECODE_CASES = [
    # fmt,   io,    B, Hq, Hkv, D,   lens
    ("f32", "f32", 1, 32, 8, 128, [2049]),            # BASELINE config 1
    ("f32", "f32", 2, 4, 2, 64, [33, 200]),
    ("f16", "f16", 3, 32, 8, 128, [1, 64, 777]),
    ("bf16", "bf16", 4, 32, 8, 128, [512, 65, 1300, 129]),  # ragged, like config 3
    ("f16", "f16", 2, 4, 4, 128, [100, 300]),          # no grouping (G = 1)
    ("f16", "f16", 2, 6, 2, 64, [100, 300]),           # G = 3
    ("f16", "f16", 1, 16, 2, 128, [260]),              # G = 8: two group tiles
    ("q8_1", "f16", 2, 32, 8, 128, [2000, 333]),
    ("q8_1", "f32", 1, 8, 2, 64, [500]),
    ("q4_0", "f16", 2, 32, 8, 128, [2000, 333]),
    ("q4_0", "bf16", 1, 8, 2, 64, [500]),
    ("q8_1", "f32", 1, 8, 2, 128, [300]),               # f32 queries: CUDA-core kernel on the permuted V rows
    ("q4_0", "f32", 2, 8, 2, 128, [300, 77]),
    ("q8_1", "bf16", 2, 32, 8, 128, [700, 90]),
    ("q8_1", "f16", 1, 24, 2, 128, [1000]),             # G = 12: two tensor-core group tiles (8 + 4)
    ("q4_0", "f16", 1, 2, 2, 128, [130]),               # G = 1 on the tensor-core kernel
    ("bf16", "bf16", 1, 8, 8, 128, [4097]),
]


@pytest.mark.parametrize("layout", LAYOUTS)
@pytest.mark.parametrize("fmt,io,B,Hq,Hkv,D,lens", DECODE_CASES)
def test_decode_matches_oracle(kv, fmt, io, B, Hq, Hkv, D, lens, layout):
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=max(lens) + 64)
    seqs = [cache.new_seq() for _ in range(B)]
    Ks, Vs = [], []
    for b, n in enumerate(lens):  # pre-fill the past (n - 1 tokens), one sequence at a time
        mk = normal_with_outliers if fmt.startswith("q") else normal
        k, v = mk(100 + b, (1, Hkv, n, D)).astype(np_dtype(io)), mk(200 + b, (1, Hkv, n, D)).astype(np_dtype(io))
        Ks.append(k), Vs.append(v)
        if n > 1:
            cache.append([seqs[b]], to_dev(k[:, :, : n - 1]), to_dev(v[:, :, : n - 1]))
    # the decode step: append one token per sequence, then attend
    k_new = np.concatenate([k[:, :, -1:] for k in Ks], 0)
    v_new = np.concatenate([v[:, :, -1:] for v in Vs], 0)
    q = normal(7, (B, Hq, 1, D)).astype(np_dtype(io))
    cache.append(seqs, as_layout(to_dev(k_new), layout), as_layout(to_dev(v_new), layout))
    dq = as_layout(to_dev(q), layout)
    out = cache.attend(seqs, dq, causal=True, out=as_layout(torch.zeros_like(to_dev(q)), layout))
    cache.check()
    for b in range(B):
        kc, vc = oracle_cache_view(fmt, Ks[b], io), oracle_cache_view(fmt, Vs[b], io)
        err = attn_err(out[b:b + 1], io, q[b:b + 1], kc, vc, causal=True, threads=8)
        assert err <= TOL[io], (b, err)
    cache.close()


@pytest.mark.parametrize("fmt", ["f16", "bf16", "q8_1", "q4_0"])
def test_tensor_core_and_cuda_core_decode_agree(kv, fmt):
    # the two formulations of the decode kernel read the same pages; they must agree far inside the tolerance
    io = "bf16" if fmt == "bf16" else "f16"
    Hq, Hkv, D, lens = 32, 8, 128, [1500, 64, 129, 63]
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=4, max_seq_tokens=2048)
    seqs = [cache.new_seq() for _ in lens]
    for b, n in enumerate(lens):
        k = normal_with_outliers(300 + b, (1, Hkv, n, D)).astype(np_dtype(io))
        v = normal_with_outliers(400 + b, (1, Hkv, n, D)).astype(np_dtype(io))
        cache.append([seqs[b]], to_dev(k), to_dev(v))
    q = to_dev(normal(9, (4, Hq, 1, D)).astype(np_dtype(io)))
    out_tc = cache.attend(seqs, q, causal=True).float().cpu().numpy()
    cache.profile(False, force_simt=True)
    out_cc = cache.attend(seqs, q, causal=True).float().cpu().numpy()
    cache.profile(False)
    cache.check()
    assert rel_err(out_tc, out_cc) <= 1e-3, rel_err(out_tc, out_cc)
    cache.close()


def test_decode_explicit_scale_and_reuse_after_truncate(kv):
    Hq, Hkv, D = 8, 2, 128
    cache = kv.KvCache("f16", Hkv, D, max_seqs=2, max_seq_tokens=512)
    sq = cache.new_seq()
    k, v = normal(1, (1, Hkv, 300, D)).astype(np.float16), normal(2, (1, Hkv, 300, D)).astype(np.float16)
    q = normal(3, (1, Hq, 1, D)).astype(np.float16)
    cache.append([sq], to_dev(k), to_dev(v))
    free_before = cache.free_pages()
    # speculative rollback: drop to 130 tokens, then re-append different tokens
    cache.truncate(sq, 130)
    assert cache.seq_len(sq) == 130 and cache.free_pages() == free_before + 2
    k2, v2 = normal(4, (1, Hkv, 10, D)).astype(np.float16), normal(5, (1, Hkv, 10, D)).astype(np.float16)
    cache.append([sq], to_dev(k2), to_dev(v2))
    kc, vc = np.concatenate([k[:, :, :130], k2], 2), np.concatenate([v[:, :, :130], v2], 2)
    gk, gv = cache.export(sq, torch.float16)
    assert to_np(gk, "f16").tobytes() == kc[0].tobytes() and to_np(gv, "f16").tobytes() == vc[0].tobytes()
    out = cache.attend([sq], to_dev(q), scale=0.3, causal=True)
    want = oracle.flash_sdpa(q, kc, vc, scale=0.3, causal=True)
    assert rel_err(to_np(out, "f16").astype(np.float32), want.astype(np.float32)) <= TOL["f16"]
    # fork = freeze / unfreeze on device: the copy decodes identically and then diverges independently
    f = cache.fork(sq)
    out_f = cache.attend([f], to_dev(q), scale=0.3, causal=True)
    assert torch.equal(out, out_f)
    cache.append([f], to_dev(k2[:, :, :1]), to_dev(v2[:, :, :1]))
    assert cache.seq_len(f) == 141 and cache.seq_len(sq) == 140
    gk2, _ = cache.export(sq, torch.float16)
    assert torch.equal(gk, gk2)
    cache.check()
    cache.close()


# ---- prefill over the cache --------------------------------------------------------------------------

@pytest.mark.parametrize("fmt,io,Hq,Hkv,D,P,S", [
    ("f16", "f16", 32, 8, 128, 0, 512),     # BASELINE config 2
    ("f16", "f16", 4, 2, 64, 3, 12),        # inplace_kv_cache.rs:595-658: prefill 3 then more, GQA 4/2
    ("f32", "f32", 4, 2, 64, 70, 33),
    ("bf16", "bf16", 8, 2, 128, 100, 64),
    ("q8_1", "f16", 8, 2, 128, 64, 64),
    # the tcgen05 prefill kernel (f16 / bf16 pages, head_dim 128)
    ("f16", "f16", 4, 1, 128, 0, 32),       # one partly filled page
    ("f16", "f16", 8, 2, 128, 100, 33),     # S not a multiple of the queries per tile, past not page aligned
    ("f16", "f16", 8, 8, 128, 70, 200),     # no grouping: 128 queries per tile
    ("f16", "f16", 6, 2, 128, 5, 100),      # G = 3: 42 queries per tile, two dead rows
    ("bf16", "bf16", 16, 2, 128, 300, 50),  # G = 8
    ("f16", "f16", 32, 8, 128, 4000, 512),  # chunked prefill: a 512-token chunk after 4000 cached tokens
    # enough query tiles for the double-tile CTAs (two 128-row tiles share each staged K/V chunk)
    ("f16", "f16", 32, 8, 128, 100, 1200),  # 1200 = 18 double tiles + 48 queries: the last CTA's second tile is half dead
    ("bf16", "bf16", 32, 8, 128, 37, 1250),
    # quantised and head_dim 64 pages on the tensor-core kernel (operand tiles rebuilt in shared memory)
    ("q8_1", "f16", 32, 8, 128, 1000, 300),
    ("q4_0", "f16", 8, 2, 128, 130, 70),
    ("q8_1", "bf16", 8, 2, 128, 64, 200),
    ("q4_0", "bf16", 32, 8, 128, 37, 600),
    ("f16", "f16", 32, 8, 64, 100, 300),
    ("bf16", "bf16", 8, 2, 64, 5, 130),
    ("q8_1", "f16", 8, 2, 64, 70, 100),
    ("q8_1", "f32", 4, 2, 128, 70, 33),     # f32 queries: the generic kernel reading the pages in place
])
@pytest.mark.parametrize("layout", LAYOUTS)
def test_prefill_matches_oracle(kv, fmt, io, Hq, Hkv, D, P, S, layout):
    scale = 0.5 if io != "f32" else 1.0
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=1, max_seq_tokens=P + S + 64)
    sq = cache.new_seq()
    k = normal(1, (1, Hkv, P + S, D), scale=scale).astype(np_dtype(io))
    v = normal(2, (1, Hkv, P + S, D), scale=scale).astype(np_dtype(io))
    q = normal(3, (1, Hq, S, D), scale=scale).astype(np_dtype(io))
    if P:
        cache.append([sq], to_dev(k[:, :, :P]), to_dev(v[:, :, :P]))
    cache.append([sq], as_layout(to_dev(k[:, :, P:]), layout), as_layout(to_dev(v[:, :, P:]), layout))
    out = cache.attend([sq], as_layout(to_dev(q), layout), causal=True, out=as_layout(torch.zeros_like(to_dev(q)), layout))
    cache.check()
    err = attn_err(out, io, q, oracle_cache_view(fmt, k, io), oracle_cache_view(fmt, v, io), causal=True, threads=8)
    assert err <= TOL[io], err
    cache.close()


@pytest.mark.parametrize("fmt,io,causal,Hq,Hkv,S,D", [
    ("f16", "f16", True, 16, 4, 96, 128), ("f16", "f16", False, 16, 4, 96, 128), ("bf16", "bf16", True, 16, 4, 96, 128),
    # double-tile CTAs; 600 = 9 x 64 + 24: the last CTA of each (sequence, head) has a second tile with no live row
    ("f16", "f16", True, 32, 8, 600, 128), ("bf16", "bf16", False, 32, 8, 600, 128),
    # converted sources and head_dim 64, with and without the causal mask, single and double tiles
    ("q8_1", "f16", False, 16, 4, 96, 128), ("q4_0", "bf16", False, 32, 8, 600, 128), ("q8_1", "f16", True, 32, 8, 600, 64),
    ("f16", "f16", False, 8, 8, 300, 64), ("kivi8", "f16", True, 16, 4, 150, 128),
])
def test_prefill_tensor_core_and_generic_paths_agree(kv, fmt, io, causal, Hq, Hkv, S, D):
    # two sequences of different length in one call; the tcgen05 kernels against the generic kernel reading the same pages
    pasts = [200, 31]
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=2, max_seq_tokens=1024)
    seqs = [cache.new_seq() for _ in pasts]
    for b, P in enumerate(pasts):
        k, v = normal(500 + b, (1, Hkv, P, D)).astype(np_dtype(io)), normal(600 + b, (1, Hkv, P, D)).astype(np_dtype(io))
        cache.append([seqs[b]], to_dev(k), to_dev(v))
    kn, vn = normal(7, (2, Hkv, S, D)).astype(np_dtype(io)), normal(8, (2, Hkv, S, D)).astype(np_dtype(io))
    cache.append(seqs, to_dev(kn), to_dev(vn))
    q = to_dev(normal(9, (2, Hq, S, D)).astype(np_dtype(io)))
    out_tc = cache.attend(seqs, q, causal=causal).float().cpu().numpy()
    cache.profile(False, force_simt=True)
    out_gen = cache.attend(seqs, q, causal=causal).float().cpu().numpy()
    cache.profile(False)
    cache.check()
    # both round an f32 result to 16 bits: about one unit in the last place apart, measured against the tensor's scale
    # (a converted source also rounds the dequantised V to f16 on its way to the tensor cores: 2^-11 per weight)
    assert rel_err(out_tc, out_gen) <= (8e-3 if io == "bf16" else (1e-3 if fmt == io else 2e-3))  # one ulp: 2^-7 (bf16), 2^-10 (f16) at most
    cache.close()


@pytest.mark.parametrize("io", ["f16", "bf16"])
def test_prefill_raises_its_reference_maximum_on_every_page(kv, io):
    # scores that grow along the key axis by ~30 (in log2 units) per page: every page past the first lifts the running
    # maximum by more than the 2^8 the kernel tolerates, so the rescale of O -- and its wait for the product before -- runs
    # on every page, for every tile
    Hq, Hkv, D, P, S = 8, 2, 128, 0, 700
    rng = np.random.default_rng(77)
    d = rng.standard_normal(D).astype(np.float32)
    d /= np.linalg.norm(d)
    ramp_t = (np.arange(P + S, dtype=np.float32) / 64.0)[None, None, :, None]
    k = (normal(71, (1, Hkv, P + S, D)) * 0.05 + ramp_t * 2.0 * d).astype(np_dtype(io))
    v = normal(72, (1, Hkv, P + S, D)).astype(np_dtype(io))
    q = (normal(73, (1, Hq, S, D)) * 0.05 + 120.0 * d).astype(np_dtype(io))  # q . k * scale ~ 120 * 2 * (t / 64) / 11.3 = 21 t / 64
    cache = kv.KvCache(io, Hkv, D, max_seqs=1, max_seq_tokens=P + S + 64)
    sq = cache.new_seq()
    cache.append([sq], to_dev(k), to_dev(v))
    out = cache.attend([sq], to_dev(q), causal=True)
    cache.check()
    err = attn_err(out, io, q, k, v, causal=True, threads=8)
    assert err <= TOL[io], err
    cache.close()


def test_prefill_repeats_bit_identically(kv):
    # 25 launches of one chunk whose last page is visible to the last eight queries of each tile only: a wait that
    # lets the epilogue read O before the last product has landed shows up as a changing result in exactly those rows
    Hq, Hkv, D, S, P = 32, 8, 128, 600, 200
    cache = kv.KvCache("f16", Hkv, D, max_seqs=1, max_seq_tokens=1024)
    sq = cache.new_seq()
    k, v = normal(31, (1, Hkv, P + S, D)).astype(np.float16), normal(32, (1, Hkv, P + S, D)).astype(np.float16)
    cache.append([sq], to_dev(k), to_dev(v))
    q = to_dev(normal(33, (1, Hq, S, D)).astype(np.float16))
    first = cache.attend([sq], q, causal=True).cpu().numpy()
    for _ in range(24):
        again = cache.attend([sq], q, causal=True).cpu().numpy()
        assert again.tobytes() == first.tobytes()
    cache.check()
    cache.close()


@pytest.mark.parametrize("fmt,io,D,G,window", [("f16", "f16", 128, 4, 100), ("q8_1", "f16", 128, 4, 257), ("bf16", "bf16", 128, 1, 64),
                                               ("f32", "f32", 64, 2, 33), ("q4_0", "bf16", 128, 8, 1000)])
def test_sliding_window_decode(kv, fmt, io, D, G, window):
    # WindowKvSdpa (window_kv_cache.rs:160-228): each step pushes one token and attends, unmasked, over the last `window`
    # cached tokens.  Sequences shorter than, equal to and longer than the window; pages given back as the window moves on.
    Hkv, lens = 2, [window - 7 if window > 7 else 1, window, 3 * window + 5, 700]
    B = len(lens)
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=max(lens) + 80)
    seqs = [cache.new_seq() for _ in range(B)]
    ks = [normal(5100 + b, (1, Hkv, lens[b] + 3, D)).astype(np_dtype(io)) for b in range(B)]
    vs = [normal_with_outliers(5200 + b, (1, Hkv, lens[b] + 3, D)).astype(np_dtype(io)) for b in range(B)]
    for b in range(B):
        cache.append([seqs[b]], to_dev(ks[b][:, :, :lens[b]]), to_dev(vs[b][:, :, :lens[b]]))
    free0 = cache.free_pages()
    for step in range(3):
        n = [l + step for l in lens]
        if step:
            k_new = np.concatenate([ks[b][:, :, n[b] - 1:n[b]] for b in range(B)]).astype(np_dtype(io))
            v_new = np.concatenate([vs[b][:, :, n[b] - 1:n[b]] for b in range(B)]).astype(np_dtype(io))
            cache.append(seqs, to_dev(k_new), to_dev(v_new))
        q = normal(5300 + step, (B, Hkv * G, 1, D)).astype(np_dtype(io))
        out = cache.attend_window(seqs, to_dev(q), window)
        cache.check()
        for b in range(B):
            lo = max(0, n[b] - window)
            kw, vw = ks[b][:, :, lo:n[b]], vs[b][:, :, lo:n[b]]
            err = attn_err(out[b:b + 1], io, q[b:b + 1], oracle_cache_view(fmt, kw, io), oracle_cache_view(fmt, vw, io), causal=False, threads=4)
            assert err <= TOL[io], (step, b, err)
        for s in seqs:  # bound the memory like the ring buffer does: nothing before the window is kept
            cache.trim(s, window)
    assert cache.free_pages() > free0  # the long sequences gave pages back
    # a trimmed sequence still answers plain decode attention (over what it holds) but no longer exports
    q = normal(5400, (B, Hkv * G, 1, D)).astype(np_dtype(io))
    out = cache.attend(seqs, to_dev(q), causal=True)
    b = 3
    lo = max(0, lens[b] + 2 - window)
    err = attn_err(out[b:b + 1], io, q[b:b + 1], oracle_cache_view(fmt, ks[b][:, :, lo:lens[b] + 2], io),
                   oracle_cache_view(fmt, vs[b][:, :, lo:lens[b] + 2], io), causal=False, threads=4)
    assert err <= TOL[io], err
    with pytest.raises(kv.B200KvError):
        cache.export(seqs[2], torch.float32)  # 3 * window + 7 tokens: always trimmed
    cache.close()


@pytest.mark.parametrize("fmt,io,D,G", [("f16", "f16", 128, 4), ("q8_1", "f16", 128, 4), ("q8_1", "bf16", 128, 8), ("q4_0", "f16", 128, 3),
                                        ("bf16", "bf16", 64, 1), ("f32", "f32", 64, 2), ("f16", "f16", 64, 4), ("f32", "f32", 128, 1)])
def test_decode_with_rope_on_the_query_load(kv, fmt, io, D, G):
    # ApplyRope (apply_rope.rs:143-176) folded into the decode kernels' query load: the same bits as rope, then attend,
    # on both decode kernels (tensor-core and CUDA-core), and the oracle's ApplyRope + Sdpa within the attention bound.
    Hkv, lens = 2, [1, 63, 64, 65, 700, 2049]
    B = len(lens)
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=max(lens))
    seqs = [cache.new_seq() for _ in range(B)]
    ks = [normal(6100 + b, (1, Hkv, lens[b], D)).astype(np_dtype(io)) for b in range(B)]
    vs = [normal_with_outliers(6200 + b, (1, Hkv, lens[b], D)).astype(np_dtype(io)) for b in range(B)]
    for b in range(B):
        cache.append([seqs[b]], to_dev(ks[b]), to_dev(vs[b]))
    q = normal(6300, (B, Hkv * G, 1, D)).astype(np_dtype(io))
    ang = np.random.default_rng(6400).uniform(-np.pi, np.pi, size=(B, 1, D // 2)).astype(np.float32)
    cos = np.concatenate([np.cos(ang), np.cos(ang)], -1).astype(np_dtype(io))
    sin = np.concatenate([np.sin(ang), np.sin(ang)], -1).astype(np_dtype(io))
    # cos / sin rows as windows of a wider table (a row stride that is not D)
    wide_c, wide_s = torch.zeros((B, 3 * D), dtype=to_dev(cos).dtype, device="cuda"), torch.zeros((B, 3 * D), dtype=to_dev(cos).dtype, device="cuda")
    wide_c[:, D:2 * D], wide_s[:, D:2 * D] = to_dev(cos)[:, 0], to_dev(sin)[:, 0]
    for force_simt in (False, True):
        cache.profile(False, force_simt=force_simt)
        two = cache.attend(seqs, kv.rope(to_dev(q), to_dev(cos), to_dev(sin)), causal=True)
        one = cache.attend_rope(seqs, to_dev(q), wide_c[:, D:2 * D], wide_s[:, D:2 * D])
        cache.check()
        assert torch.equal(one.view(torch.uint8), two.view(torch.uint8)), (force_simt, fmt)
    q_rot = oracle.apply_rope(q, cos[:, None], sin[:, None])
    for b in range(B):
        err = attn_err(one[b:b + 1], io, q_rot[b:b + 1], oracle_cache_view(fmt, ks[b], io), oracle_cache_view(fmt, vs[b], io), causal=False, threads=4)
        assert err <= TOL[io], (b, err)
    cache.profile(False)
    cache.close()


@pytest.mark.parametrize("fmt,io,D,G,B", [("f16", "f16", 128, 4, 8), ("q8_1", "f16", 128, 4, 5), ("bf16", "bf16", 64, 2, 11), ("f32", "f32", 128, 1, 3),
                                          ("q4_0", "bf16", 128, 8, 16), ("q8_1", "f16", 128, 4, 130)])  # 130 rows: the tiled activation layout
def test_decode_result_as_quantised_activation(kv, fmt, io, D, G, B):
    # the decode result left as the quantised activation of a W4A8 GEMM: the bits of attend (+ rope) -> quantise, on both
    # decode kernels, with row counts on and off the groups of 8 and the result tensor present or not
    import oracle as orc

    Hkv = 2
    Hq = Hkv * G
    lens = [1 + (37 if B < 64 else 3) * b for b in range(B)]
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=max(lens))
    seqs = [cache.new_seq() for _ in range(B)]
    for b in range(B):
        cache.append([seqs[b]], to_dev(normal(6600 + b, (1, Hkv, lens[b], D)).astype(np_dtype(io))),
                     to_dev(normal_with_outliers(6700 + b, (1, Hkv, lens[b], D)).astype(np_dtype(io))))
    q = to_dev(normal(6800, (B, Hq, 1, D)).astype(np_dtype(io)))
    ang = np.random.default_rng(6801).uniform(-np.pi, np.pi, size=(B, D // 2)).astype(np.float32)
    cos = to_dev(np.concatenate([np.cos(ang), np.cos(ang)], -1).astype(np_dtype(io)))
    sin = to_dev(np.concatenate([np.sin(ang), np.sin(ang)], -1).astype(np_dtype(io)))
    n, k = 48, Hq * D
    sc, pk = orc.q4_0_quant(normal(6802, (n, k)).astype(np.float32))
    blob = np.empty((n, k // 32, 18), np.uint8)
    blob[:, :, :2] = sc.reshape(n, k // 32, 1).view(np.uint8)
    blob[:, :, 2:] = pk.reshape(n, k // 32, 16)
    lin = kv.Q40Linear(torch.from_numpy(blob).cuda(), max_m=max(16, B))
    scratch = torch.empty(kv.Q40Linear.scratch_bytes(k, B), dtype=torch.uint8, device="cuda")
    for force_simt in (False, True):
        cache.profile(False, force_simt=force_simt)
        for rope in (False, True):
            plain = cache.attend_rope(seqs, q, cos, sin) if rope else cache.attend(seqs, q, causal=True)
            want = lin.gemm(plain.view(B, k))
            out = torch.zeros_like(plain)
            cache.attend_q40(seqs, q, scratch, cos=cos if rope else None, sin=sin if rope else None, out=out)
            got = lin.gemm_quantized(B, scratch=scratch)
            assert torch.equal(out.view(torch.uint8), plain.view(torch.uint8)) and torch.equal(got, want), (force_simt, rope)
            scratch.fill_(0xA5)  # no result tensor: the padding rows of the last group must still come out as zeros
            cache.attend_q40(seqs, q, scratch, cos=cos if rope else None, sin=sin if rope else None)
            assert torch.equal(lin.gemm_quantized(B, scratch=scratch), want), (force_simt, rope)
    lin.check(scratch)
    cache.check()
    cache.profile(False)
    cache.close()


@pytest.mark.parametrize("fmt,io,S", [("f16", "f16", 1), ("q8_1", "f16", 1), ("f32", "f32", 1), ("f16", "f16", 70), ("kivi8", "f16", 1)])
def test_fused_cache_and_attention_call(kv, fmt, io, S):
    # InPlaceKvSdpa as one call: the bits of append followed by attend, step after step
    Hkv, G, D, B = 2, 4, 128, 3
    a = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=512)
    b = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=512)
    sa, sb = [a.new_seq() for _ in range(B)], [b.new_seq() for _ in range(B)]
    for step in range(4):
        k = to_dev(normal(7000 + step, (B, Hkv, S, D)).astype(np_dtype(io)))
        v = to_dev(normal_with_outliers(7100 + step, (B, Hkv, S, D)).astype(np_dtype(io)))
        q = to_dev(normal(7200 + step, (B, Hkv * G, S, D)).astype(np_dtype(io)))
        a.append(sa, k, v)
        two = a.attend(sa, q, causal=True)
        one = b.append_attend(sb, k, v, q, causal=True)
        assert torch.equal(one.view(torch.uint8), two.view(torch.uint8)), step
    assert [a.seq_len(s) for s in sa] == [b.seq_len(s) for s in sb] == [4 * S] * B
    a.check(), b.check()
    a.close(), b.close()


def test_rope_on_the_query_load_refuses_what_it_cannot_do(kv):
    D, Hkv = 128, 2
    q = to_dev(normal(6500, (1, 4, 1, D)).astype(np.float16))
    cs = to_dev(np.ones((1, D), np.float16))
    kivi = kv.KvCache("kivi8", Hkv, D, max_seqs=1, max_seq_tokens=128)
    s = kivi.new_seq()
    kivi.append([s], to_dev(normal(6501, (1, Hkv, 40, D)).astype(np.float16)), to_dev(normal(6502, (1, Hkv, 40, D)).astype(np.float16)))
    with pytest.raises(kv.B200KvError):  # a KIVI cache takes its query already rotated
        kivi.attend_rope([s], q, cs, cs)
    kivi.close()
    cache = kv.KvCache("f16", Hkv, D, max_seqs=1, max_seq_tokens=128)
    s = cache.new_seq()
    with pytest.raises(kv.B200KvError):  # an empty sequence: nothing to attend to
        cache.attend_rope([s], q, cs, cs)
    cache.append([s], to_dev(normal(6503, (1, Hkv, 3, D)).astype(np.float16)), to_dev(normal(6504, (1, Hkv, 3, D)).astype(np.float16)))
    with pytest.raises(kv.B200KvError):  # 3 query heads over 2 kv heads
        cache.attend_rope([s], q[:, :3], cs, cs)
    cache.attend_rope([s], q, cs, cs)
    cache.check()
    cache.close()


def _sweep_cases():
    rng = np.random.default_rng(20260)
    cases = []
    for i in range(28):
        fmt = ["f16", "bf16", "q8_1", "q4_0", "f32"][i % 5]
        io = {"f16": "f16", "bf16": "bf16", "f32": "f32"}.get(fmt, ["f16", "bf16"][i % 2])
        D = 64 if i % 7 == 3 else 128
        Hkv = int(rng.choice([1, 2, 4]))
        G = int(rng.choice([1, 2, 4, 8]))
        P = int(rng.integers(0, 700))
        S = int(rng.choice([1, 1, 1, 7, 33, 130, 257]))
        B = int(rng.choice([1, 2, 3]))
        mag = float(rng.choice([0.3, 1.0, 3.0]))  # scale of q and k: from nearly uniform to sharply peaked attention
        cases.append((i, fmt, io, B, Hkv * G, Hkv, D, P, S, mag))
    return cases


@pytest.mark.parametrize("i,fmt,io,B,Hq,Hkv,D,P,S,mag", _sweep_cases())
def test_attend_property_sweep(kv, i, fmt, io, B, Hq, Hkv, D, P, S, mag):
    # seeded random geometry: every format, both head dims, group sizes 1..8, decode and prefill, batches whose sequences
    # differ in length, inputs from flat to sharply peaked score distributions; causal and (for S = 1) trivially so
    lens = [P + S + 13 * b for b in range(B)]
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=max(lens) + 64)
    seqs = [cache.new_seq() for _ in range(B)]
    ks, vs = [], []
    for b in range(B):
        k = (normal(9000 + 10 * i + b, (1, Hkv, lens[b], D)) * mag).astype(np_dtype(io))
        v = normal_with_outliers(9500 + 10 * i + b, (1, Hkv, lens[b], D)).astype(np_dtype(io))
        if lens[b] > S:
            cache.append([seqs[b]], to_dev(k[:, :, :-S]), to_dev(v[:, :, :-S]))
        ks.append(k), vs.append(v)
    k_new = np.concatenate([k[:, :, -S:] for k in ks]).astype(np_dtype(io))
    v_new = np.concatenate([v[:, :, -S:] for v in vs]).astype(np_dtype(io))
    cache.append(seqs, to_dev(k_new), to_dev(v_new))
    q = (normal(9900 + i, (B, Hq, S, D)) * mag).astype(np_dtype(io))
    out = cache.attend(seqs, to_dev(q), causal=True)
    cache.check()
    for b in range(B):
        err = attn_err(out[b:b + 1], io, q[b:b + 1], oracle_cache_view(fmt, ks[b], io), oracle_cache_view(fmt, vs[b], io), causal=True, threads=8)
        assert err <= TOL[io], (b, err)
    cache.close()


# ---- lone Sdpa: golden bundles, the reference's kernel-test shapes, property sweep ------------------------

ATTN_CASES = ["simple-causal-f32", "simple-non-causal-f32", "simple-scale-f32", "simple-f16", "simple-mask-f32"]


@pytest.mark.parametrize("case", ATTN_CASES)
def test_sdpa_golden_bundles_on_gpu(kv, golden, case):
    z, meta = golden
    a = meta[case]
    q, k, v = (z[f"{case}/{n}"] for n in a["qkv"])
    mask = z[f"{case}/mask"] if f"{case}/mask" in z.files else None
    if a["dtype"] == "f16":
        q, k, v = (x.astype(np.float16) for x in (q, k, v))
    out = kv.sdpa(to_dev(q), to_dev(k), to_dev(v), mask=to_dev(mask) if mask is not None else None,
                  scale=a["scale"], causal=a["causal"])
    got = out.float().cpu().numpy()
    want = z[f"{case}/output_0"]
    atol, rtol = (1e-3, 5e-3) if a["dtype"] == "f16" else (2e-7, 2e-7)
    assert np.all(np.abs(got - want) <= atol + rtol * np.abs(want)), np.abs(got - want).max()


@pytest.mark.parametrize("b,hq,hkv,p,s,d,causal,with_mask", [
    # cuda/src/kernels/flash_attn.rs:276-287, inputs are i/len ramps in f16, scale 1.0
    (1, 1, 1, 64, 1, 128, False, False), (1, 2, 1, 64, 1, 128, False, True), (1, 2, 2, 0, 1, 64, False, False),
    (2, 4, 2, 123, 1, 64, False, False), (1, 2, 2, 0, 1, 64, True, False), (1, 1, 1, 64, 64, 128, False, False),
    (2, 32, 4, 64, 64, 128, False, False), (1, 1, 1, 64, 64, 128, False, True), (1, 1, 1, 64, 64, 128, True, False),
])
def test_sdpa_reference_kernel_test_shapes(kv, b, hq, hkv, p, s, d, causal, with_mask):
    def rampf16(shape):
        n = int(np.prod(shape))
        return (np.arange(n, dtype=np.float32) / np.float32(n)).astype(np.float16).reshape(shape)

    q, k, v = rampf16((b, hq, s, d)), rampf16((b, hkv, p + s, d)), rampf16((b, hkv, p + s, d))
    mask = np.ones((1, 1, s, p + s), np.float16) if with_mask else None
    out = kv.sdpa(to_dev(q), to_dev(k), to_dev(v), mask=to_dev(mask) if with_mask else None, scale=1.0, causal=causal)
    want = oracle.flash_sdpa(q, k, v, mask=mask, scale=1.0, causal=causal, threads=8)
    assert rel_err(out.float().cpu().numpy(), want.astype(np.float32)) <= TOL["f16"]


@pytest.mark.parametrize("io,B,Hq,Hkv,P,S,D,mode", [
    ("f16", 2, 8, 2, 400, 300, 128, "causal"),       # keys not a multiple of 64, past + chunk
    ("f16", 1, 32, 8, 0, 1100, 128, "causal"),       # enough query tiles for the double-tile CTAs
    ("bf16", 2, 8, 8, 100, 200, 128, "none"),        # no grouping, no mask at all
    ("f16", 2, 6, 2, 37, 150, 64, "causal"),         # head_dim 64, G = 3
    ("bf16", 1, 16, 4, 0, 513, 64, "mask"),
    ("f16", 2, 8, 2, 130, 90, 128, "mask"),          # additive mask broadcast over the batch, with -inf stripes
    ("f16", 1, 4, 1, 64, 64, 128, "mask_bh"),        # a mask of its own for every batch entry and head
    ("f16", 3, 8, 2, 2000, 1, 128, "causal"),        # one query per sequence through the same kernel
])
def test_sdpa_on_the_tensor_cores(kv, io, B, Hq, Hkv, P, S, D, mode):
    # the lone Sdpa at the sizes of the reference's kernel bench (cuda/benches/cuda_flash.rs:84-110) and smaller ragged
    # ones: dense K / V given as strided windows ([B, T, Hkv, D] storage seen as [B, Hkv, T, D]), masks with -inf
    T = P + S
    q = normal(21, (B, Hq, S, D), scale=0.5).astype(np_dtype(io))
    k = normal(22, (B, Hkv, T, D), scale=0.5).astype(np_dtype(io))
    v = normal(23, (B, Hkv, T, D), scale=0.5).astype(np_dtype(io))
    mask = None
    if mode.startswith("mask"):
        shape = (B, Hq, S, T) if mode == "mask_bh" else (1, 1, S, T)
        mask = normal(24, shape).astype(np.float32)
        mask[..., :, 5:T:7] = -np.inf         # whole key columns masked out
        # a query that sees key 0 and the second half (a row whose first 32-key tile is masked out entirely comes out as
        # NaN from the reference's tile recurrence, exp(-inf - -inf): not a case to hold a kernel to)
        mask[..., 3, 1: T // 2] = -np.inf
        mask = mask.astype(np.float16) if io == "f16" else mask
    dk = to_dev(np.ascontiguousarray(np.swapaxes(k, 1, 2))).transpose(1, 2)  # [B, Hkv, T, D] view of [B, T, Hkv, D]
    dv = to_dev(np.ascontiguousarray(np.swapaxes(v, 1, 2))).transpose(1, 2)
    out = kv.sdpa(to_dev(q), dk, dv, mask=to_dev(mask) if mask is not None else None, causal=mode == "causal")
    kv.sdpa_check()
    if io == "bf16":
        want = oracle.flash_sdpa(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32),
                                 mask=mask.astype(np.float32) if mask is not None else None, causal=mode == "causal", threads=8)
        err = rel_err_bf16(to_np(out, io).astype(np.float32), want)
    else:
        want = oracle.flash_sdpa(q, k, v, mask=mask, causal=mode == "causal", threads=8)
        err = rel_err(to_np(out, io).astype(np.float32), want.astype(np.float32))
    assert err <= TOL[io], err


def test_sdpa_property_sweep(kv):
    # strategy of test-rt/suite-unit/src/sdpa.rs:94-142 (values k/8, B 1-2, GQA repeat 1-4, kv heads 1-4,
    # P 0-4, S 2-4, optional scale, causal or additive mask broadcast over b / h), embed dims of the CPU
    # and CUDA runners together, f32 and f16, rank 3 and rank 4
    g = np.random.default_rng(11)
    for it in range(80):
        b, rep, hkv = int(g.integers(1, 3)), int(g.integers(1, 5)), int(g.integers(1, 5))
        p, s, d = int(g.integers(0, 5)), int(g.integers(2, 5)), int(g.choice([1, 2, 3, 64, 128]))
        rank3 = bool(g.integers(0, 2))
        if rank3:
            rep = hkv = 1
        hq = rep * hkv
        dt = np.float16 if it % 2 else np.float32
        mk = lambda shape: (g.integers(-3, 4, size=shape) / 8.0).astype(dt)
        q, k, v = mk((b, hq, s, d)), mk((b, hkv, p + s, d)), mk((b, hkv, p + s, d))
        causal = bool(g.integers(0, 2))
        mask = None
        if not causal and g.integers(0, 2):
            mask = mk((b if g.integers(0, 2) else 1, hq if g.integers(0, 2) else 1, s, p + s))
        scale = float(g.uniform(0.1, 1.0)) if g.integers(0, 2) else None
        if rank3:
            q, k, v = q[:, 0], k[:, 0], v[:, 0]
            mask = mask[:, 0] if mask is not None else None
        out = kv.sdpa(to_dev(q), to_dev(k), to_dev(v), mask=to_dev(mask) if mask is not None else None, scale=scale,
                      causal=causal)
        want = oracle.flash_sdpa(q, k, v, mask=mask, scale=scale, causal=causal)
        err = rel_err(out.float().cpu().numpy(), want.astype(np.float32))
        assert err <= (TOL["f16"] if dt == np.float16 else TOL["f32"]), (it, err)


# ---- error behaviour: validation happens on the host, nothing is enqueued ------------------------------

def test_errors_are_reported_not_swallowed(kv):
    cache = kv.KvCache("f16", 2, 128, max_seqs=1, max_seq_tokens=128, pool_tokens=128)
    sq = cache.new_seq()
    with pytest.raises(kv.B200KvError, match="sequence slots"):
        cache.new_seq()
    x = torch.zeros(1, 2, 4, 128, dtype=torch.float32, device="cuda")
    with pytest.raises(kv.B200KvError, match="same type"):
        cache.append([sq], x, x)
    h = x.half()
    with pytest.raises(kv.B200KvError, match="v_new is required"):
        cache.append([sq], h)
    with pytest.raises(kv.B200KvError, match="empty|fewer"):
        cache.attend([sq], torch.zeros(1, 4, 1, 128, dtype=torch.float16, device="cuda"))
    big = torch.zeros(1, 2, 200, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(kv.B200KvError, match="max_seq_tokens"):
        cache.append([sq], big, big)
    assert cache.seq_len(sq) == 0  # a failed call changed nothing
    cache.append([sq], h, h)
    with pytest.raises(kv.B200KvError, match="truncate"):
        cache.truncate(sq, 10)
    with pytest.raises(kv.B200KvError, match="multiple"):
        cache.attend([sq], torch.zeros(1, 3, 1, 128, dtype=torch.float16, device="cuda"))
    with pytest.raises(kv.B200KvError, match="not live"):
        cache.seq_len(5)
    cache.check()
    cache.close()
    with pytest.raises(kv.B200KvError, match="head_dim"):
        kv.KvCache("f16", 2, 96, max_seqs=1, max_seq_tokens=128)
