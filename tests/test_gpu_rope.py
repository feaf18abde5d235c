"""Rotary embedding: the stand-alone ApplyRope kernel and the key-side fusion into the cache append, bit-exact
against the oracle's restatement of ApplyRope::eval (transformers/src/ops/apply_rope.rs:155-163)."""
import numpy as np
import pytest

import oracle
from util import normal

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def kv():
    import tract_b200

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    tract_b200.lib()
    return tract_b200


def tables(S, D, dt, start=0, theta=500000.0):
    """cos / sin of Llama-3-style rotary angles for positions start .. start + S (theta as in BASELINE config 5)."""
    inv = 1.0 / theta ** (np.arange(0, D, 2, dtype=np.float64) / D)
    ang = np.outer(np.arange(start, start + S, dtype=np.float64), inv)
    emb = np.concatenate([ang, ang], axis=-1)
    return np.cos(emb)[None].astype(dt), np.sin(emb)[None].astype(dt)


def dev(a):
    if a.dtype in (np.float32, np.float16):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint16).copy()).view(torch.bfloat16).cuda()


def host(t, dt):
    t = t.cpu().contiguous()
    return t.view(torch.uint16).numpy().view(dt) if t.dtype == torch.bfloat16 else t.numpy()


@pytest.mark.parametrize("name", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("D", [128, 64, 6])
def test_apply_rope_kernel_bit_exact(kv, name, D):
    dt = {"f32": np.float32, "f16": np.float16, "bf16": oracle.bfloat16}[name]
    x = normal(1, (2, 3, 17, D)).astype(dt)
    cos, sin = tables(17, D, dt, start=5)
    got = host(kv.rope(dev(x), dev(cos), dev(sin)), dt)
    want = oracle.apply_rope(x, cos[:, None], sin[:, None])
    assert got.tobytes() == want.tobytes()
    # strided input (transposed [B, S, H, D] memory), per-batch tables
    xt = dev(np.ascontiguousarray(x.transpose(0, 2, 1, 3))).permute(0, 2, 1, 3)
    cos2, sin2 = np.concatenate([cos, cos[:, ::-1]]), np.concatenate([sin, sin[:, ::-1]])
    got = host(kv.rope(xt, dev(cos2), dev(sin2)), dt)
    assert got.tobytes() == oracle.apply_rope(x, cos2[:, None], sin2[:, None]).tobytes()


@pytest.mark.parametrize("fmt,name", [("f16", "f16"), ("f32", "f32"), ("bf16", "bf16"), ("q8_1", "f16"), ("q4_0", "f32")])
def test_append_with_fused_rope_equals_rope_then_append(kv, fmt, name):
    dt = {"f32": np.float32, "f16": np.float16, "bf16": oracle.bfloat16}[name]
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[name]
    H, D, B = 2, 128, 2
    fused = kv.KvCache(fmt, H, D, max_seqs=B, max_seq_tokens=256)
    plain = kv.KvCache(fmt, H, D, max_seqs=B, max_seq_tokens=256)
    sf, sp = [fused.new_seq() for _ in range(B)], [plain.new_seq() for _ in range(B)]
    pos, ks = 0, []
    for i, s in enumerate([70, 1, 1, 30]):
        k, v = normal(10 + i, (B, H, s, D)).astype(dt), normal(20 + i, (B, H, s, D)).astype(dt)
        cos, sin = tables(s, D, dt, start=pos)
        fused.append_rope(sf, dev(k), dev(v), dev(cos), dev(sin))
        kr = oracle.apply_rope(k, cos[:, None], sin[:, None])  # the unfused graph: ApplyRope, then the cache
        plain.append(sp, dev(kr), dev(v))
        ks.append(kr)
        pos += s
    fused.check()
    K = np.concatenate(ks, 2)
    for b in range(B):
        if fmt in ("q8_1", "q4_0"):
            for which in (0, 1):
                cf, scf = fused.export_codes(sf[b], which)
                cp, scp = plain.export_codes(sp[b], which)
                assert torch.equal(cf, cp) and torch.equal(scf.view(torch.uint16), scp.view(torch.uint16))
            quant = oracle.q8_1_quant if fmt == "q8_1" else oracle.q4_0_quant
            r = quant(K[b])
            cf, scf = fused.export_codes(sf[b], 0)
            assert np.array_equal(cf.cpu().numpy(), r[-1]) and np.array_equal(scf.cpu().view(torch.uint16).numpy(), r[0])
        else:
            gk, _ = fused.export(sf[b], tdt)
            assert host(gk, dt).tobytes() == K[b].tobytes()
    fused.close(), plain.close()
