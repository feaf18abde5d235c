"""Shared helpers for the parity tests: seeded inputs and the error metric."""
import numpy as np

# Tolerances of the parity bar: attention outputs within 2e-3 (f16 / bf16) and 1e-5 (f32)
# of the oracle; cache contents, codes and scales bit-exact.
TOL = {"f32": 1e-5, "f16": 2e-3, "bf16": 2e-3}


class Err(float):
    """A float that prints with the plain measures beside it: when `assert rel_err(...) <= tol` fails, pytest shows
    the largest absolute difference, the largest plain relative difference among the elements whose reference is above
    the rms, the rms itself and where the worst element is."""

    def __new__(cls, value, **details):
        self = super().__new__(cls, value)
        self.details = details
        return self

    def __repr__(self):
        extra = ", ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in self.details.items())
        return f"{float(self):.4g} ({extra})" if extra else f"{float(self):.4g}"

    __str__ = __repr__


def _plain_measures(got, ref, score):
    diff = np.abs(got - ref)
    rms = float(np.sqrt(np.mean(ref * ref)))
    big = np.abs(ref) > rms
    worst = np.unravel_index(int(np.argmax(score)), score.shape) if score.ndim else ()
    return dict(max_abs=float(diff.max()), max_rel_above_rms=float((diff[big] / np.abs(ref[big])).max()) if big.any() else 0.0,
                ref_rms=rms, worst_at=tuple(int(i) for i in worst), got=float(got[worst]), ref=float(ref[worst]))


def rel_err(got, ref) -> float:
    """Max relative error with an RMS floor: max_i |got_i - ref_i| / (|ref_i| + rms(ref)).

    A purely element-wise ratio is undefined where the reference output crosses zero; dividing
    by the tensor maximum alone would hide errors on small entries.  Adding the RMS of the
    reference to each denominator keeps the measure element-wise and finite.  The value returned
    prints with the plain max-abs and max-relative measures beside it (see Err).
    """
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if ref.size == 0:
        return Err(0.0)
    rms = float(np.sqrt(np.mean(ref * ref)))
    den = np.abs(ref) + (rms if rms > 0 else 1.0)
    score = np.abs(got - ref) / den
    with np.errstate(invalid="ignore"):
        value = float(np.max(score))
    if not np.isfinite(value):
        return Err(value)
    return Err(value, **_plain_measures(got, ref, score))


def rel_err_bf16(got_bf16, ref_f32) -> float:
    """rel_err for a bf16 result against the oracle's UNROUNDED f32 result.

    bf16 keeps 8 significant bits: one unit in the last place is 2^-8 relative, twice the 2e-3 bar, so
    two correct implementations whose f32 results straddle a rounding boundary differ by more than the
    bar after rounding.  The bar therefore applies to the computation: the distance to the f32 oracle
    result beyond the half-ulp that rounding to bf16 (round-to-nearest-even, exact) may add.
    """
    got = np.asarray(got_bf16, dtype=np.float64)
    ref = np.asarray(ref_f32, dtype=np.float64)
    assert got.shape == ref.shape
    rms = float(np.sqrt(np.mean(ref * ref)))
    half_ulp = np.where(ref != 0, 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 1e-300))) - 8), 0.0)
    excess = np.maximum(np.abs(got - ref) - half_ulp, 0.0)
    score = excess / (np.abs(ref) + (rms if rms > 0 else 1.0))
    value = float(np.max(score))
    if not np.isfinite(value) or ref.size == 0:
        return Err(value)
    return Err(value, **_plain_measures(got, ref, score))


def rng(seed: int) -> np.random.Generator:
    """Counter-based generator (Philox4x32-10) so every case is reproducible from its seed."""
    return np.random.Generator(np.random.Philox(key=seed))


def normal(seed, shape, dtype=np.float32, scale=1.0):
    return (rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(dtype)


def normal_with_outliers(seed, shape, dtype=np.float32, frac=0.01, mag=20.0):
    """N(0,1) with `frac` of the elements (i.i.d. Bernoulli) multiplied by `mag`."""
    g = rng(seed)
    x = g.standard_normal(shape, dtype=np.float32)
    x = np.where(g.random(shape, dtype=np.float32) < frac, x * np.float32(mag), x)
    return x.astype(dtype)


def lcg_tensor(seed: int, shape):
    """The generator of the reference's flash-attention unit tests (flash_sdpa.rs:349-357):
    s = s*6364136223846793005 + 1442695040888963407; value = (s >> 40) / 2^24 - 0.5."""
    n = int(np.prod(shape))
    out = np.empty(n, np.float32)
    s = seed & 0xFFFFFFFFFFFFFFFF
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(np.float32(s >> 40) / np.float32(1 << 24)) - np.float32(0.5)
    return out.reshape(shape)


def ramp(shape, start=0.0, step=0.5, dtype=np.float32):
    """`seq_tensor` of the reference's in-place cache tests (inplace_kv_cache.rs:359-363)."""
    n = int(np.prod(shape))
    return (start + np.arange(n, dtype=np.float32) * np.float32(step)).reshape(shape).astype(dtype)
