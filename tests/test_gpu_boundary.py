"""What the header promises about the boundary itself: no device allocation after b200kv_create, a failed call
changes nothing, and a bounded wait that runs out is reported while the cache stays usable.  No test here faults,
traps or hangs the GPU: the wait that runs out is a wait on a copy that was never issued, with a 1 ms limit."""
import numpy as np
import pytest

import oracle
from util import TOL, normal, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def kv():
    import tract_b200

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    tract_b200.lib()
    return tract_b200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def fill(cache, seqs, lens, Hkv, D, seed, dt=np.float16):
    for b, n in enumerate(lens):
        cache.append([seqs[b]], dev(normal(seed + b, (1, Hkv, n, D)).astype(dt)), dev(normal(seed + 50 + b, (1, Hkv, n, D)).astype(dt)))


@pytest.mark.parametrize("fmt", ["q8_1", "f16", "kivi8", "f32"])
def test_no_device_allocation_after_create(kv, fmt):
    # The split-KV workspace is sized at create (b200kv_workspace_bytes).  Calls that need ever more partials --
    # one short sequence, then many long ones, then several queries per sequence -- must leave the free device
    # memory where it was (torch's own tensors are made before the first reading).
    Hq, Hkv, D, B = 32, 8, 128, 24
    io = np.float32 if fmt == "f32" else np.float16
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=B, max_seq_tokens=6000, max_q_heads=Hq)
    assert cache.workspace_bytes > 0
    seqs = [cache.new_seq() for _ in range(B)]
    lens = [70] + [5000 + 7 * b for b in range(1, B)]
    fill(cache, seqs, lens, Hkv, D, 1, io)
    q1, qB = dev(normal(3, (1, Hq, 1, D)).astype(io)), dev(normal(4, (B, Hq, 1, D)).astype(io))
    qS = dev(normal(5, (2, Hq, 40, D)).astype(io))
    o1, oB, oS = torch.empty_like(q1), torch.empty_like(qB), torch.empty_like(qS)
    # the first launch of a kernel may make the CUDA runtime load its code (device memory of the runtime's own): every
    # kernel the calls below use is launched once, on the smallest case, before the first reading
    cache.attend(seqs[:1], q1, out=o1)
    cache.attend(seqs[:1], qS[:1], out=oS[:1])
    cache.check()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    cache.attend(seqs[:1], q1, out=o1)
    cache.attend(seqs, qB, out=oB)
    cache.attend(seqs[1:3], qS, out=oS)
    cache.attend(seqs[3:4], q1, out=o1)
    cache.check()
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.isfinite(oB.float()).all() and torch.isfinite(oS.float()).all()
    cache.close()


def test_workspace_too_small_for_the_natural_split_takes_longer_runs(kv):
    # a cache that announced one query head is asked for 64: the partials of the natural split (8 runs for each of the 40
    # sequences: 20480 records) do not fit the workspace sized at create (19584), so the call cuts its sequences into
    # fewer runs -- and gives the same answer
    Hkv, D, B, n = 1, 128, 40, 9000
    small = kv.KvCache("f16", Hkv, D, max_seqs=B, max_seq_tokens=n + 64, max_q_heads=1)
    big = kv.KvCache("f16", Hkv, D, max_seqs=B, max_seq_tokens=n + 64, max_q_heads=64)
    assert small.workspace_bytes == 19584 * (D + 2) * 4
    assert small.workspace_bytes < big.workspace_bytes
    ss, sb = [small.new_seq() for _ in range(B)], [big.new_seq() for _ in range(B)]
    fill(small, ss, [n] * B, Hkv, D, 9)
    fill(big, sb, [n] * B, Hkv, D, 9)
    q = dev(normal(2, (B, 64, 1, D)).astype(np.float16))
    a, b = small.attend(ss, q), big.attend(sb, q)
    small.check(), big.check()
    assert rel_err(a.float().cpu().numpy(), b.float().cpu().numpy()) <= 1e-3
    # so many sequences x heads that even one run per sequence does not fit: refused, with the remedy in the message
    tiny = kv.KvCache("f16", 1, D, max_seqs=200, max_seq_tokens=64, max_q_heads=1)
    ts = [tiny.new_seq() for _ in range(200)]
    x = torch.zeros((200, 1, 3, D), dtype=torch.float16, device="cuda")
    tiny.append(ts, x, x)
    with pytest.raises(kv.B200KvError, match="max_q_heads"):
        tiny.attend(ts, torch.zeros((200, 256, 1, D), dtype=torch.float16, device="cuda"))
    small.close(), big.close(), tiny.close()


@pytest.mark.parametrize("fmt,io", [("q8_1", "f16"), ("f32", "f32")])
def test_bounded_wait_runs_out_and_the_cache_stays_usable(kv, fmt, io):
    # The give-up path of the kernels' bounded waits: one CTA of one launch is told not to issue its copies (a test hook
    # of b200kv_profile), so its first barrier wait can never complete; with the limit at 1 ms it gives up, sets the
    # status word, publishes an empty partial and returns.  Nothing faults or spins on; the next call is served.
    Hq, Hkv, D, lens = 8, 2, 128, [700, 90]
    dt = np.float16 if io == "f16" else np.float32
    cache = kv.KvCache(fmt, Hkv, D, max_seqs=2, max_seq_tokens=1024)
    seqs = [cache.new_seq() for _ in lens]
    Ks = [normal(10 + b, (1, Hkv, n, D)).astype(dt) for b, n in enumerate(lens)]
    Vs = [normal(20 + b, (1, Hkv, n, D)).astype(dt) for b, n in enumerate(lens)]
    for b in range(2):
        cache.append([seqs[b]], dev(Ks[b]), dev(Vs[b]))
    q = normal(5, (2, Hq, 1, D)).astype(dt)
    good = cache.attend(seqs, dev(q))
    cache.check()
    cache.profile(False, stall_next_decode=True)
    cache.attend(seqs, dev(q))  # completes (about 1 ms later than usual); its output is not meaningful
    with pytest.raises(kv.B200KvError, match="bounded wait expired"):
        cache.check()
    cache.check()  # the status word was reported once and cleared
    again = cache.attend(seqs, dev(q))
    cache.check()
    assert torch.equal(good, again)
    if fmt == "q8_1":
        for b in range(2):
            s, _, c = oracle.q8_1_quant(Ks[b])
            sv, _, cv = oracle.q8_1_quant(Vs[b])
            want = oracle.flash_sdpa(q[b:b + 1], oracle.q8_1_dequant(s, c), oracle.q8_1_dequant(sv, cv), causal=True)
            assert rel_err(again[b:b + 1].float().cpu().numpy(), want.astype(np.float32)) <= TOL[io]
    cache.close()


def test_failed_calls_in_the_middle_of_a_batch_change_nothing(kv):
    Hkv, D = 2, 64
    # (1) page pool exhausted by the fourth sequence of a batch: the pages taken for the first three go back
    cache = kv.KvCache("f16", Hkv, D, max_seqs=5, max_seq_tokens=4096, pool_tokens=64 * 6)  # 6 + 5 pages
    seqs = [cache.new_seq() for _ in range(4)]
    free0 = cache.free_pages()
    x = torch.randn((4, Hkv, 64 * 3, D), device="cuda").half()  # 3 pages per sequence: 12 needed, 11 there
    with pytest.raises(kv.B200KvError, match="page pool exhausted"):
        cache.append(seqs, x, x)
    assert cache.free_pages() == free0 and all(cache.seq_len(s) == 0 for s in seqs)
    cache.append(seqs[:3], x[:3], x[:3])  # 9 pages: served
    assert cache.free_pages() == free0 - 9
    # (2) a fork that cannot get its pages leaves no half-made sequence behind
    with pytest.raises(kv.B200KvError, match="page pool exhausted"):
        cache.fork(seqs[0])
    assert cache.free_pages() == free0 - 9
    s4 = cache.new_seq()  # the slot the failed fork had taken is free again: this is the fifth and last one
    with pytest.raises(kv.B200KvError, match="sequence slots"):
        cache.new_seq()
    cache.free_seq(s4)
    # (3) a sequence longer than max_seq_tokens
    with pytest.raises(kv.B200KvError, match="max_seq_tokens"):
        cache.append([seqs[3]], torch.zeros((1, Hkv, 5000, D), dtype=torch.float16, device="cuda"),
                     torch.zeros((1, Hkv, 5000, D), dtype=torch.float16, device="cuda"))
    assert cache.seq_len(seqs[3]) == 0
    # the survivors still hold what was appended
    gk, _ = cache.export(seqs[1], torch.float16)
    assert torch.equal(gk, x[1])
    cache.check()
    cache.close()
    # (4) the ring of descriptor slots is reused over many more calls than it has slots
    many = kv.KvCache("f16", 1, D, max_seqs=300, max_seq_tokens=128)
    ids = [many.new_seq() for _ in range(300)]
    y = torch.randn((300, 1, 2, D), device="cuda").half()
    for _ in range(40):  # 300 sequences per call: beyond the inline batch, every call takes a ring slot
        many.append(ids, y, y)
    assert all(many.seq_len(i) == 80 for i in ids)
    o = many.attend(ids, torch.randn((300, 4, 1, D), device="cuda").half())
    many.check()
    assert torch.isfinite(o.float()).all()
    many.close()


def test_fork_of_a_sequence_longer_than_one_ring_slot(kv):
    # the page-table update of a fork travels in slot-sized pieces: 64 KiB / 8 bytes = 8192 pages per piece
    Hkv, D, n = 1, 64, 64 * 8300
    cache = kv.KvCache("q4_0", Hkv, D, max_seqs=2, max_seq_tokens=n + 64)
    s = cache.new_seq()
    x = torch.randn((1, Hkv, n // 2, D), device="cuda").half()
    cache.append([s], x, x)  # (one append call may take up to a slot's worth of new pages: two calls)
    cache.append([s], x, x)
    f = cache.fork(s)
    q = torch.randn((2, 2, 1, D), device="cuda").half()
    out = cache.attend([s, f], torch.cat([q[:1], q[:1]]))
    cache.check()
    assert torch.equal(out[0], out[1]) and cache.seq_len(f) == n
    cache.close()
