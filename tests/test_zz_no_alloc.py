"""The allocation-free decode entry point against the regular one, through the C ABI.

b200kv_attend_static_scratch keeps its split-KV partials in a fixed array inside the library, for
callers that must not allocate device memory while a step runs (all HBM already given to page pools,
an arena sized once, a loop that cannot tolerate the device-wide synchronisation of cudaMalloc).  It
must return what b200kv_attend returns.  Two calls in a row check that what the first call leaves in
the shared array does not leak into the second.  This file sorts last so that a run stopping at the
first failure has already been through every other test.
"""
import numpy as np
import pytest

from util import TOL, normal, normal_with_outliers, rel_err

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_static_scratch_decode_matches_regular_decode_twice():
    import tract_b200 as kv

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    kv.lib()
    Hq, Hkv, D, lens = 32, 8, 128, [3000, 65, 700]
    cache = kv.KvCache("q8_1", Hkv, D, max_seqs=len(lens), max_seq_tokens=4096)
    seqs = [cache.new_seq() for _ in lens]
    for b, n in enumerate(lens):
        k = torch.from_numpy(normal_with_outliers(50 + b, (1, Hkv, n, D)).astype(np.float16)).cuda()
        v = torch.from_numpy(normal_with_outliers(60 + b, (1, Hkv, n, D)).astype(np.float16)).cuda()
        cache.append([seqs[b]], k, v)
    for call in range(2):  # the second call meets the first call's partials in the shared array
        q = torch.from_numpy(normal(70 + call, (len(lens), Hq, 1, D)).astype(np.float16)).cuda()
        want = cache.attend(seqs, q, causal=True)
        got = torch.full_like(want, float("nan"))
        cache.attend_static_scratch(seqs, q, out=got)
        cache.check()
        err = rel_err(got.float().cpu().numpy(), want.float().cpu().numpy())
        assert err <= TOL["f16"], (call, err)
        if call == 0:  # between the calls the batch changes, so the partial slots are laid out differently
            cache.truncate(seqs[0], 1000)
    # a call that would overflow the fixed array is refused with both numbers in the message, and enqueues nothing
    big = kv.KvCache("f16", 8, D, max_seqs=64, max_seq_tokens=64 * 70)
    ids = [big.new_seq() for _ in range(64)]
    x = torch.zeros((64, 8, 64 * 66, D), dtype=torch.float16, device="cuda")
    big.append(ids, x, x)
    qb = torch.zeros((64, 64, 1, D), dtype=torch.float16, device="cuda")
    ob = torch.empty_like(qb)
    with pytest.raises(kv.B200KvError, match="fixed scratch array holds"):
        big.attend_static_scratch(ids, qb, out=ob)
    big.attend(ids, qb, causal=True, out=ob)  # the regular entry point still serves it
    big.check()
    big.close()
    cache.close()


@pytest.mark.parametrize("fmt,io,D,Hq,Hkv", [("q8_1", "f32", 128, 8, 2), ("f16", "f16", 64, 6, 2), ("f32", "f32", 128, 4, 4)])
def test_static_scratch_decode_on_the_cuda_core_kernel(fmt, io, D, Hq, Hkv):
    # f32 queries and head_dim 64 are served by the CUDA-core decode kernel; through this entry point its partials go to
    # the fixed array as well.  Two calls in a row, against the regular entry point.
    import tract_b200 as kv

    dt = np.float32 if io == "f32" else np.float16
    lens = [900, 70, 300]
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=len(lens), max_seq_tokens=1024)
    seqs = [cache.new_seq() for _ in lens]
    for b, n in enumerate(lens):
        cache.append([seqs[b]], torch.from_numpy(normal(150 + b, (1, Hkv, n, D)).astype(dt)).cuda(),
                     torch.from_numpy(normal(160 + b, (1, Hkv, n, D)).astype(dt)).cuda())
    for call in range(2):
        q = torch.from_numpy(normal(170 + call, (len(lens), Hq, 1, D)).astype(dt)).cuda()
        want = cache.attend(seqs, q, causal=True)
        got = torch.full_like(want, float("nan"))
        cache.attend_static_scratch(seqs, q, out=got)
        cache.check()
        assert rel_err(got.float().cpu().numpy(), want.float().cpu().numpy()) <= TOL[io], call
        if call == 0:
            cache.truncate(seqs[0], 200)
    cache.close()


def test_static_scratch_refusals_enqueue_nothing():
    # What this entry point does not serve is refused during validation, before a descriptor slot is taken or anything is
    # enqueued: the output buffer still holds what it held, and the next regular call works.
    import tract_b200 as kv

    Hq, Hkv, D = 8, 2, 128
    sentinel = 3.25

    def refused(cache, seqs, pattern):
        q = torch.zeros((len(seqs), Hq, 1, D), dtype=torch.float16, device="cuda")
        out = torch.full_like(q, sentinel)
        with pytest.raises(kv.B200KvError, match=pattern):
            cache.attend_static_scratch(seqs, q, out=out)
        torch.cuda.synchronize()
        assert bool((out == sentinel).all())
        cache.attend(seqs, q, causal=True, out=out)  # the regular entry point serves the same call
        cache.check()
        assert torch.isfinite(out.float()).all() and not bool((out == sentinel).any())

    # a KIVI cache has decode kernels of its own
    kivi = kv.KvCache("kivi8", Hkv, D, max_seqs=1, max_seq_tokens=256)
    s = kivi.new_seq()
    x = torch.randn((1, Hkv, 100, D), device="cuda").half()
    kivi.append([s], x, x)
    refused(kivi, [s], "KIVI")
    kivi.close()
    # a sequence whose front pages were given back (sliding window)
    cache = kv.KvCache("f16", Hkv, D, max_seqs=1, max_seq_tokens=512)
    s = cache.new_seq()
    x = torch.randn((1, Hkv, 300, D), device="cuda").half()
    cache.append([s], x, x)
    cache.trim(s, 100)
    refused(cache, [s], "trimmed")
    cache.close()
