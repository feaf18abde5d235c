"""BASELINE configurations at their full sizes.

The oracle cannot attend over 16 x 32 x 32769 rows in test time, so parity is checked where it is affordable —
whole (sequence, kv head) slices against the oracle — and through properties that do not depend on size:
re-quantising the dequantised cache reproduces it bit for bit, scaling V by two scales the output by exactly
two, and a sequence attended alone (a different split of the work) agrees with the batched call."""
import numpy as np
import pytest

import oracle
from util import TOL, rel_err, rel_err_bf16

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

HQ, HKV, D = 32, 8, 128


@pytest.fixture(scope="module")
def kv():
    import tract_b200

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    tract_b200.lib()
    return tract_b200


def outlier_normal(gen, shape, dtype):
    """N(0,1) with 1% of the elements multiplied by 20 (config 4's value distribution)."""
    x = torch.randn(shape, generator=gen, device="cuda")
    x = torch.where(torch.rand(shape, generator=gen, device="cuda") < 0.01, x * 20, x)
    return x.to(dtype)


@pytest.mark.parametrize("fmt", ["q8_1", "q4_0"])
def test_config4_quantised_long_context_decode(kv, fmt):
    B, P = 16, 32768
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4)
    cache = kv.KvCache(fmt, HKV, D, max_seqs=B + 1, max_seq_tokens=P + 128)
    twice = kv.KvCache(fmt, HKV, D, max_seqs=2, max_seq_tokens=P + 128)  # sequences 0, 1 with V doubled
    seqs = [cache.new_seq() for _ in range(B)]
    tw = [twice.new_seq() for _ in range(2)]
    checked = [(0, 0), (7, 3), (15, 7)]  # (sequence, kv head) slices compared with the oracle in full
    kept = {c: ([], []) for c in checked}
    for t0 in range(0, P, 4096):  # quantise-on-append, 4096 tokens per call
        k, v = outlier_normal(gen, (B, HKV, 4096, D), torch.float16), outlier_normal(gen, (B, HKV, 4096, D), torch.float16)
        cache.append(seqs, k, v)
        twice.append(tw, k[:2], v[:2] * 2)
        for (b, h) in checked:
            kept[(b, h)][0].append(k[b, h].cpu().numpy()), kept[(b, h)][1].append(v[b, h].cpu().numpy())
    k1, v1 = outlier_normal(gen, (B, HKV, 1, D), torch.float16), outlier_normal(gen, (B, HKV, 1, D), torch.float16)
    q = torch.randn((B, HQ, 1, D), generator=gen, device="cuda").half()
    cache.append(seqs, k1, v1)  # the decode step: one token per sequence, then attention over 32769 positions
    twice.append(tw, k1[:2], v1[:2] * 2)
    out = cache.attend(seqs, q, causal=True)
    cache.check()
    assert all(cache.seq_len(s) == P + 1 for s in seqs)

    # (1) slices against the oracle: codes and scales bit-exact, attention within tolerance
    quant = oracle.q8_1_quant if fmt == "q8_1" else oracle.q4_0_quant
    dequant = oracle.q8_1_dequant if fmt == "q8_1" else oracle.q4_0_dequant
    for (b, h) in checked:
        K = np.concatenate(kept[(b, h)][0] + [k1[b, h].cpu().numpy()])
        V = np.concatenate(kept[(b, h)][1] + [v1[b, h].cpu().numpy()])
        deq = []
        for which, X in ((0, K), (1, V)):
            codes, scales = cache.export_codes(seqs[b], which)
            r = quant(X)
            s_ref, c_ref = r[0], r[-1]
            assert np.array_equal(scales[h].cpu().view(torch.uint16).numpy(), s_ref)
            assert np.array_equal(codes[h].cpu().numpy(), c_ref)
            deq.append(dequant(s_ref, c_ref))
        G = HQ // HKV
        want = oracle.flash_sdpa(q[b:b + 1, h * G:(h + 1) * G].cpu().numpy(), deq[0][None, None], deq[1][None, None],
                                 causal=True, threads=8)
        got = out[b:b + 1, h * G:(h + 1) * G].float().cpu().numpy()
        assert rel_err(got, want.astype(np.float32)) <= TOL["f16"], (b, h)

    # (2) re-quantising the dequantised cache reproduces its VALUES bit for bit (the resume path: save_to +
    # load_from).  Codes and scales may flip sign together: after quantisation a second element can tie the
    # block maximum in magnitude, and the first occurrence decides the sign of the scale.
    kd, vd = cache.export(seqs[3], torch.float32)
    again = cache.new_seq()
    cache.append([again], kd[None], vd[None])
    kd2, vd2 = cache.export(again, torch.float32)
    assert torch.equal(kd, kd2) and torch.equal(vd, vd2)
    redo = cache.attend([again], q[3:4], causal=True)
    assert rel_err(redo.float().cpu().numpy(), out[3:4].float().cpu().numpy()) <= 1e-3

    # (3) linearity in V: V -> 2V keeps the codes and doubles the scales, so the output doubles (up to the
    # different split of a 2-sequence batch and the rounding of the f16 result)
    out2 = twice.attend(tw, q[:2], causal=True)
    assert rel_err(out2.float().cpu().numpy(), out[:2].float().cpu().numpy() * 2) <= 1e-3

    # (4) a sequence alone is split differently from the same sequence inside the batch of 16
    alone = cache.attend([seqs[5]], q[5:6], causal=True)
    assert rel_err(alone.float().cpu().numpy(), out[5:6].float().cpu().numpy()) <= 1e-3
    cache.check()
    cache.close(), twice.close()


@pytest.mark.parametrize("fmt,bits", [("kivi8", 8), ("kivi4", 4)])
def test_config4_kivi_long_context_decode(kv, fmt, bits):
    # config 4 with tract's own storage quantisation (QuantizedDynKeyValueCache, quant_dyn_kv_cache.rs:98-250): 16
    # sequences of 32768 tokens, then the decode step.  Whole (sequence, kv head) slices against the oracle's stores
    # (codes, lo, scale, sinks, residual bit for bit) and against flash attention over the oracle's dequantised cache.
    B, P = 16, 32768
    gen = torch.Generator(device="cuda")
    gen.manual_seed(44)
    cache = kv.KvCache(fmt, HKV, D, max_seqs=B, max_seq_tokens=P + 128)
    seqs = [cache.new_seq() for _ in range(B)]
    checked = [(0, 0), (9, 5), (15, 7)]
    kept = {c: ([], []) for c in checked}
    for t0 in range(0, P, 4096):
        k, v = outlier_normal(gen, (B, HKV, 4096, D), torch.float16), outlier_normal(gen, (B, HKV, 4096, D), torch.float16)
        cache.append(seqs, k, v)
        for (b, h) in checked:
            kept[(b, h)][0].append(k[b, h].cpu().numpy()), kept[(b, h)][1].append(v[b, h].cpu().numpy())
    k1, v1 = outlier_normal(gen, (B, HKV, 1, D), torch.float16), outlier_normal(gen, (B, HKV, 1, D), torch.float16)
    q = torch.randn((B, HQ, 1, D), generator=gen, device="cuda").half()
    cache.append(seqs, k1, v1)
    out = cache.attend(seqs, q, causal=True)
    cache.check()
    assert all(cache.seq_len(s) == P + 1 for s in seqs)
    G = HQ // HKV
    raws = {}
    for (b, h) in checked:
        deq = []
        for which, per_channel in ((0, True), (1, False)):
            X = np.concatenate(kept[(b, h)][which] + [(k1 if which == 0 else v1)[b, h].cpu().numpy()])
            st = oracle.KiviStore(per_channel, D, bits)
            st.push(X)
            want = st.raw()
            if (b, which) not in raws:
                raws[(b, which)] = {key: val.cpu().numpy() for key, val in cache.export_kivi(seqs[b], which, per_channel).items()}
            raw = raws[(b, which)]
            assert np.array_equal(raw["sink"][h], want["sink"])
            assert np.array_equal(raw["codes"][h], want["codes"]), (b, h, which)
            assert np.array_equal(raw["lo"][h].reshape(-1), want["lo"]) and np.array_equal(raw["scale"][h].reshape(-1), want["scale"])
            if per_channel:
                assert np.array_equal(raw["residual"][h], want["residual"])
            deq.append(st.dequant())
        want = oracle.flash_sdpa(q[b:b + 1, h * G:(h + 1) * G].cpu().numpy(), deq[0][None, None], deq[1][None, None], causal=True, threads=8)
        got = out[b:b + 1, h * G:(h + 1) * G].float().cpu().numpy()
        assert rel_err(got, want.astype(np.float32)) <= TOL["f16"], (b, h)
    # a sequence alone is split differently from the same sequence inside the batch of 16
    alone = cache.attend([seqs[5]], q[5:6], causal=True)
    assert rel_err(alone.float().cpu().numpy(), out[5:6].float().cpu().numpy()) <= 1e-3
    cache.check()
    cache.close()


def test_config3_ragged_batched_decode_bf16(kv):
    B = 256
    lens = [int(x) for x in np.random.Generator(np.random.Philox(key=3)).integers(512, 16385, size=B)]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    cache = kv.KvCache("bf16", HKV, D, max_seqs=B, max_seq_tokens=max(lens) + 128, pool_tokens=sum(lens) + 64 * B)
    seqs = [cache.new_seq() for _ in range(B)]
    checked = [0, 100, int(np.argmax(lens)), int(np.argmin(lens))]
    kept = {}
    for b in range(B):
        n = lens[b] + 1  # the past plus the token of the decode step
        k = torch.randn((1, HKV, n, D), generator=gen, device="cuda").bfloat16()
        v = torch.randn((1, HKV, n, D), generator=gen, device="cuda").bfloat16()
        cache.append([seqs[b]], k[:, :, :-1], v[:, :, :-1])
        kept[b] = (k, v)
    k_new = torch.cat([kept[b][0][:, :, -1:] for b in range(B)])
    v_new = torch.cat([kept[b][1][:, :, -1:] for b in range(B)])
    q = torch.randn((B, HQ, 1, D), generator=gen, device="cuda").bfloat16()
    cache.append(seqs, k_new, v_new)
    out = cache.attend(seqs, q, causal=True)
    cache.check()
    for b in checked:
        k, v = kept[b]
        gk, gv = cache.export(seqs[b], torch.bfloat16)
        assert torch.equal(gk, k[0]) and torch.equal(gv, v[0])  # cache == concat of everything appended
        want = oracle.flash_sdpa(q[b:b + 1].float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                                 causal=True, threads=8)
        assert rel_err_bf16(out[b:b + 1].float().cpu().numpy(), want) <= TOL["bf16"], b
    # every sequence alone (its own split) against the batched call
    for b in checked[:2]:
        alone = cache.attend([seqs[b]], q[b:b + 1], causal=True)
        assert rel_err(alone.float().cpu().numpy(), out[b:b + 1].float().cpu().numpy()) <= 8e-3
    cache.close()
