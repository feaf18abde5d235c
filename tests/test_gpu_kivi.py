"""KIVI storage quantisation (QuantizedDynKeyValueCache) on the GPU against the oracle's stores:
codes, lo, scale, sinks and residual bit-exact; dequantised export bit-exact; attention within tolerance."""
import numpy as np
import pytest

import oracle
from util import TOL, normal, normal_with_outliers, rel_err, rel_err_bf16

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def kv():
    import tract_b200

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    tract_b200.lib()
    return tract_b200


STEPS = [3, 2, 40, 1, 1, 1, 70, 1, 33]  # sinks filled over two calls, blocks completing inside and across calls


def drive(cache, seqs, H, D, dt, seed, with_v=True):
    """Appends STEPS chunks to every sequence; returns the concatenated K (and V) inputs [B, H, T, D]."""
    ks, vs = [], []
    for i, s in enumerate(STEPS):
        k = normal_with_outliers(seed + i, (len(seqs), H, s, D)).astype(dt)
        v = normal_with_outliers(seed + 100 + i, (len(seqs), H, s, D)).astype(dt)
        if i == 4:
            k[0, 0, 0, :] = 2.5          # hi == lo over a row / a channel run: scale 1
            v[0, 0, 0, :] = -1.25
        cache.append(seqs, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda() if with_v else None)
        ks.append(k), vs.append(v)
    return np.concatenate(ks, 2), np.concatenate(vs, 2)


def check_stream(cache, sq, which, per_channel, X, bits):
    """X: [H, T, D] inputs of one sequence; compares the raw stores of every head with the oracle's."""
    raw = {k: v.cpu().numpy() for k, v in cache.export_kivi(sq, which, per_channel).items()}
    H, T, D = X.shape
    for h in range(H):
        st = oracle.KiviStore(per_channel, D, bits)
        st.push(X[h])
        want = st.raw()
        assert np.array_equal(raw["sink"][h], want["sink"])
        assert np.array_equal(raw["codes"][h], want["codes"]), (which, h)
        assert np.array_equal(raw["lo"][h].reshape(-1), want["lo"]) and np.array_equal(raw["scale"][h].reshape(-1), want["scale"])
        if per_channel:
            assert np.array_equal(raw["residual"][h], want["residual"])


@pytest.mark.parametrize("fmt,bits", [("kivi8", 8), ("kivi4", 4)])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_kivi_stores_bit_exact(kv, fmt, bits, D, dt):
    H, B = 2, 2
    T = sum(STEPS)
    cache = kv.KvCache(fmt, H, D, max_seqs=B, max_seq_tokens=T + 64)
    seqs = [cache.new_seq() for _ in range(B)]
    K, V = drive(cache, seqs, H, D, dt, seed=10)
    cache.check()
    tdt = torch.float32 if dt == np.float32 else torch.float16
    for b, sq in enumerate(seqs):
        assert cache.seq_len(sq) == T
        check_stream(cache, sq, 0, True, K[b], bits)
        check_stream(cache, sq, 1, False, V[b], bits)
        # the op's output: dequantised f32 cache cast to the input dtype (quant_dyn_kv_cache.rs:493)
        gk, gv = cache.export(sq, tdt)
        for got, X, pc in ((gk, K[b], True), (gv, V[b], False)):
            for h in range(H):
                st = oracle.KiviStore(pc, D, bits)
                st.push(X[h])
                assert got[h].cpu().numpy().tobytes() == st.dequant().astype(dt).tobytes()
    with pytest.raises(kv.B200KvError, match="cannot be truncated"):
        cache.truncate(seqs[0], 10)
    cache.close()


@pytest.mark.parametrize("per_token", [False, True])
def test_lone_kivi_cache_and_fork(kv, per_token):
    # a single QuantizedDynKeyValueCache node: one tensor, per channel (Keys) or per token (Values)
    H, D = 2, 64
    cache = kv.KvCache("kivi8", H, D, max_seqs=2, max_seq_tokens=256, has_values=False, per_token=per_token)
    sq = cache.new_seq()
    X, _ = drive(cache, [sq], H, D, np.float32, seed=50, with_v=False)
    check_stream(cache, sq, 0, not per_token, X[0], 8)
    f = cache.fork(sq)  # freeze / unfreeze on device
    extra = normal(77, (1, H, 9, D))
    cache.append([f], torch.from_numpy(extra).cuda())
    check_stream(cache, f, 0, not per_token, np.concatenate([X[0], extra[0]], 1), 8)
    check_stream(cache, sq, 0, not per_token, X[0], 8)
    cache.check()
    cache.close()


@pytest.mark.parametrize("fmt,bits,io", [("kivi8", 8, "f16"), ("kivi4", 4, "f32")])
def test_kivi_attention_matches_oracle(kv, fmt, bits, io):
    # prefill 3 + decode steps like the fused-op test of the reference (inplace_kv_cache.rs:595-658), GQA 4/2
    Hq, Hkv, D = 8, 2, 128
    dt = np.float16 if io == "f16" else np.float32
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=1, max_seq_tokens=256)
    sq = cache.new_seq()
    kstore = [oracle.KiviStore(True, D, bits) for _ in range(Hkv)]
    vstore = [oracle.KiviStore(False, D, bits) for _ in range(Hkv)]
    for step, s in enumerate([3, 1, 1, 45, 1, 1]):
        k, v = normal(200 + step, (1, Hkv, s, D)).astype(dt), normal(300 + step, (1, Hkv, s, D)).astype(dt)
        q = normal(400 + step, (1, Hq, s, D)).astype(dt)
        cache.append([sq], torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
        out = cache.attend([sq], torch.from_numpy(q).cuda(), causal=True)
        for h in range(Hkv):
            kstore[h].push(k[0, h]), vstore[h].push(v[0, h])
        kd = np.stack([st.dequant() for st in kstore])[None]
        vd = np.stack([st.dequant() for st in vstore])[None]
        want = oracle.flash_sdpa(q, kd, vd, causal=True)
        assert rel_err(out.float().cpu().numpy(), want.astype(np.float32)) <= TOL[io], step
    cache.check()
    cache.close()


@pytest.mark.parametrize("fmt,bits,D,Hq,Hkv", [("kivi8", 8, 128, 32, 8), ("kivi4", 4, 64, 6, 2), ("kivi4", 4, 128, 32, 8)])
def test_kivi_decode_kernel_ragged_batch(kv, fmt, bits, D, Hq, Hkv):
    # batched decode over sequences that are sinks only, shorter than one key block, and long
    lens = [700, 37, 5, 3, 1300]
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=len(lens), max_seq_tokens=2048)
    seqs = [cache.new_seq() for _ in lens]
    Ks, Vs = [], []
    for b, n in enumerate(lens):
        k, v = normal_with_outliers(700 + b, (1, Hkv, n, D)).astype(np.float16), normal(800 + b, (1, Hkv, n, D)).astype(np.float16)
        cache.append([seqs[b]], torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
        Ks.append(k), Vs.append(v)
    q = normal(9, (len(lens), Hq, 1, D)).astype(np.float16)
    out = cache.attend(seqs, torch.from_numpy(q).cuda(), causal=True)
    cache.profile(False, force_simt=True)  # the same through the generic kernel, which dequantises element by element
    out_gen = cache.attend(seqs, torch.from_numpy(q).cuda(), causal=True)
    cache.profile(False)
    cache.check()
    assert rel_err(out.float().cpu().numpy(), out_gen.float().cpu().numpy()) <= 1e-3
    cache.profile(False, kivi_cuda_core=True)  # and through the CUDA-core decode kernel alone
    out_cc = cache.attend(seqs, torch.from_numpy(q).cuda(), causal=True)
    cache.profile(False)
    assert rel_err(out_cc.float().cpu().numpy(), out_gen.float().cpu().numpy()) <= 1e-3
    for b in range(len(lens)):
        kd = np.stack([_deq(True, D, bits, Ks[b][0, h]) for h in range(Hkv)])[None]
        vd = np.stack([_deq(False, D, bits, Vs[b][0, h]) for h in range(Hkv)])[None]
        want = oracle.flash_sdpa(q[b:b + 1], kd, vd, causal=True)
        assert rel_err(out[b:b + 1].float().cpu().numpy(), want.astype(np.float32)) <= TOL["f16"], b
    cache.close()


@pytest.mark.parametrize("fmt,bits", [("kivi8", 8), ("kivi4", 4)])
def test_kivi_one_long_sequence_uses_every_split_the_combine_pass_has(kv, fmt, bits):
    # one sequence, 4 kv heads, more than 16.4k tokens: the split picker of the tensor-core kernel wants the most splits
    # it may take, and the partial of the sinks / residual block comes on top; together they must fit the 64 slots of
    # the combine pass
    Hq, Hkv, D, n = 16, 4, 128, 17500
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=1, max_seq_tokens=n + 64)
    sq = cache.new_seq()
    k, v = normal_with_outliers(31, (1, Hkv, n, D)).astype(np.float16), normal_with_outliers(32, (1, Hkv, n, D)).astype(np.float16)
    for t0 in range(0, n, 4096):
        cache.append([sq], torch.from_numpy(k[:, :, t0:t0 + 4096]).cuda(), torch.from_numpy(v[:, :, t0:t0 + 4096]).cuda())
    q = normal(33, (1, Hq, 1, D)).astype(np.float16)
    out = cache.attend([sq], torch.from_numpy(q).cuda(), causal=True)
    cache.check()
    kd = np.stack([_deq(True, D, bits, k[0, h]) for h in range(Hkv)])[None]
    vd = np.stack([_deq(False, D, bits, v[0, h]) for h in range(Hkv)])[None]
    want = oracle.flash_sdpa(q, kd, vd, causal=True, threads=8)
    assert rel_err(out.float().cpu().numpy(), want.astype(np.float32)) <= TOL["f16"]
    cache.close()


@pytest.mark.parametrize("fmt,bits,io,Hq,Hkv,P,S", [("kivi8", 8, "f16", 8, 2, 300, 200), ("kivi4", 4, "bf16", 32, 8, 37, 700),
                                                    ("kivi8", 8, "f16", 4, 4, 0, 3), ("kivi4", 4, "f16", 8, 2, 2, 130)])
def test_kivi_chunk_of_queries_on_the_tensor_cores(kv, fmt, bits, io, Hq, Hkv, P, S):
    # several queries per sequence over the KIVI stores (head_dim 128, 16-bit queries): sinks, finalised blocks and the
    # f32 residual block are widened to 16 bits in shared memory on their way to tcgen05; against flash attention over
    # the oracle's dequantised cache
    D = 128
    tdt = torch.float16 if io == "f16" else torch.bfloat16
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=1, max_seq_tokens=P + S + 64)
    sq = cache.new_seq()
    k = torch.from_numpy(normal_with_outliers(41, (1, Hkv, P + S, D))).to(tdt)
    v = torch.from_numpy(normal_with_outliers(42, (1, Hkv, P + S, D))).to(tdt)
    q = torch.from_numpy(normal(43, (1, Hq, S, D), scale=0.5)).to(tdt)
    if P:
        cache.append([sq], k[:, :, :P].cuda(), v[:, :, :P].cuda())
    cache.append([sq], k[:, :, P:].cuda(), v[:, :, P:].cuda())
    out = cache.attend([sq], q.cuda(), causal=True)
    cache.profile(False, force_simt=True)  # the generic kernel, element by element
    out_gen = cache.attend([sq], q.cuda(), causal=True)
    cache.profile(False)
    cache.check()
    kd = np.stack([_deq(True, D, bits, k[0, h].float().numpy()) for h in range(Hkv)])[None]
    vd = np.stack([_deq(False, D, bits, v[0, h].float().numpy()) for h in range(Hkv)])[None]
    want = oracle.flash_sdpa(q.float().numpy(), kd, vd, causal=True, threads=8).astype(np.float32)
    got = out.float().cpu().numpy()
    err = rel_err(got, want) if io == "f16" else rel_err_bf16(got, want)
    assert err <= TOL[io], err
    assert rel_err(got, out_gen.float().cpu().numpy()) <= (8e-3 if io == "bf16" else 2e-3)
    cache.close()


def _deq(per_channel, D, bits, rows):
    st = oracle.KiviStore(per_channel, D, bits)
    st.push(rows)
    return st.dequant()


@pytest.mark.parametrize("fmt,bits,io", [("kivi8", 8, "f16"), ("kivi8", 8, "bf16"), ("kivi4", 4, "f16"), ("kivi4", 4, "bf16")])
def test_kivi_tensor_core_decode_step_by_step(kv, fmt, bits, io):
    # decode steps across the points where a key block is finalised (length 4 + 32k) and a page fills; the tensor-core
    # kernel takes the finalised blocks, the CUDA-core kernel the sinks and the residual block
    Hq, Hkv, D = 8, 2, 128
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=1, max_seq_tokens=512)
    sq = cache.new_seq()
    kstore = [oracle.KiviStore(True, D, bits) for _ in range(Hkv)]
    vstore = [oracle.KiviStore(False, D, bits) for _ in range(Hkv)]
    tdt = torch.float16 if io == "f16" else torch.bfloat16
    for step, s in enumerate([30] + [1] * 12 + [55] + [1] * 12 + [60] + [1] * 6):
        k = normal_with_outliers(1200 + step, (1, Hkv, s, D)).astype(np.float32)
        v = normal_with_outliers(1300 + step, (1, Hkv, s, D)).astype(np.float32)
        kt, vt = torch.from_numpy(k).to(tdt), torch.from_numpy(v).to(tdt)
        cache.append([sq], kt.cuda(), vt.cuda())
        kf, vf = kt.float().numpy(), vt.float().numpy()
        for h in range(Hkv):
            kstore[h].push(kf[0, h]), vstore[h].push(vf[0, h])
        qt = torch.from_numpy(normal(1400 + step, (1, Hq, 1, D)).astype(np.float32)).to(tdt)
        out = cache.attend([sq], qt.cuda(), causal=True)
        kd = np.stack([st.dequant() for st in kstore])[None]
        vd = np.stack([st.dequant() for st in vstore])[None]
        want = oracle.flash_sdpa(qt.float().numpy(), kd, vd, causal=True).astype(np.float32)
        got = out.float().cpu().numpy()
        err = rel_err(got, want) if io == "f16" else rel_err_bf16(got, want)
        assert err <= TOL[io], (step, err)
    cache.check()
    cache.close()
