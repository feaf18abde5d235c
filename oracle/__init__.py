"""TEST INFRASTRUCTURE — ctypes front end of the CPU oracle (``tract_oracle.cpp``).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module.  It restates what tract's default CPU runtime computes for the KV-cache
+ attention path; every function names the reference lines it follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

try:  # bf16 is not a tract dtype; the oracle treats it as "f16 path with bf16 rounding"
    from ml_dtypes import bfloat16  # type: ignore
except Exception:  # pragma: no cover
    bfloat16 = None

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile liboracle.so with the committed Makefile (g++, no other dependency)."""
    src = os.path.join(_HERE, "tract_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        fp, dp, ip = C.POINTER(C.c_float), C.POINTER(C.c_double), C.c_int
        u8p, i8p, u16p = C.POINTER(C.c_uint8), C.POINTER(C.c_int8), C.POINTER(C.c_uint16)
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_dyn_kv_concat.argtypes = [u8p, C.c_int64, u8p, C.c_int64, C.c_int64, C.c_int64, u8p]
        L.orc_q8_1_quant.argtypes = [fp, C.c_int64, u16p, u16p, i8p]
        L.orc_q8_1_dequant.argtypes = [u16p, i8p, C.c_int64, fp]
        L.orc_q4_0_quant.argtypes = [fp, C.c_int64, u16p, u8p]
        L.orc_q4_0_dequant.argtypes = [u16p, u8p, C.c_int64, fp]
        L.orc_w4a8_quantize_row.argtypes = [fp, C.c_int64, i8p, fp]
        L.orc_w4a8_gemm.argtypes = [u16p, u8p, C.c_int64, C.c_int64, fp, C.c_int64, fp, ip]
        L.orc_rms_norm_f32.argtypes = [fp, C.c_int64, C.c_int64, C.c_float]
        L.orc_ssigmoid.argtypes = [fp, C.c_int64, fp]
        L.orc_silu_f32.argtypes = [fp, C.c_int64, fp]
        L.orc_kivi_new.restype = C.c_void_p
        L.orc_kivi_new.argtypes = [ip, ip, ip]
        L.orc_kivi_free.argtypes = [C.c_void_p]
        L.orc_kivi_push.argtypes = [C.c_void_p, fp]
        L.orc_kivi_push_rows.argtypes = [C.c_void_p, fp, C.c_int64, ip]
        L.orc_kivi_len.restype = C.c_int64
        L.orc_kivi_len.argtypes = [C.c_void_p]
        L.orc_kivi_counts.argtypes = [C.c_void_p] + [C.POINTER(C.c_int64)] * 3
        L.orc_kivi_raw.argtypes = [C.c_void_p, u8p, fp, fp, fp, fp]
        L.orc_kivi_dequant.argtypes = [C.c_void_p, fp]
        sd = [fp, fp, fp, fp, ip, ip, ip, ip, ip, ip, ip, ip, C.c_float, ip, ip]
        L.orc_flash_sdpa.argtypes = sd + [fp, ip]
        L.orc_naive_sdpa_f64.argtypes = sd + [dp, ip]
        L.orc_hardware_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a, ty):
    return a.ctypes.data_as(C.POINTER(ty))


# ---- dtype plumbing (tract: `cast_to::<f32>()` on the way in, `cast_to_dt` on the way out) ----

def to_f32(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).astype(np.float32)


def from_f32(a: np.ndarray, dtype) -> np.ndarray:
    """f32 -> dtype with round-to-nearest-even (numpy / ml_dtypes both do RNE)."""
    return a.astype(dtype)


# ---- a1 -------------------------------------------------------------------------------------------

def dyn_kv_concat(past: np.ndarray | None, new: np.ndarray, axis: int = 2) -> np.ndarray:
    """DynKeyValueCacheState::eval (transformers/src/ops/dyn_kv_cache.rs:158-174)."""
    new = np.ascontiguousarray(new)
    if past is None:
        return new.copy()
    past = np.ascontiguousarray(past)
    assert past.dtype == new.dtype and past.ndim == new.ndim
    lead = int(np.prod(new.shape[:axis], dtype=np.int64))
    row_bytes = int(np.prod(new.shape[axis + 1:], dtype=np.int64)) * new.dtype.itemsize
    P, S = past.shape[axis], new.shape[axis]
    shape = list(new.shape)
    shape[axis] = P + S
    out = np.empty(shape, dtype=new.dtype)
    lib().orc_dyn_kv_concat(_p(past.view(np.uint8).reshape(-1), C.c_uint8), P,
                            _p(new.view(np.uint8).reshape(-1), C.c_uint8), S, lead, row_bytes,
                            _p(out.view(np.uint8).reshape(-1), C.c_uint8))
    return out


# ---- a4 / a5 --------------------------------------------------------------------------------------

def q8_1_quant(x: np.ndarray):
    """Q8_1 blocks of 32 along the last axis (q8_1.rs:20-48).
    Returns (scales f16-bits uint16 [..., D/32], sums uint16 [..., D/32], codes int8 [..., D])."""
    x = to_f32(x)
    assert x.shape[-1] % 32 == 0
    nb = x.size // 32
    scales = np.empty(nb, np.uint16)
    sums = np.empty(nb, np.uint16)
    codes = np.empty(x.size, np.int8)
    lib().orc_q8_1_quant(_p(x, C.c_float), nb, _p(scales, C.c_uint16), _p(sums, C.c_uint16), _p(codes, C.c_int8))
    bs = x.shape[:-1] + (x.shape[-1] // 32,)
    return scales.reshape(bs), sums.reshape(bs), codes.reshape(x.shape)


def q8_1_dequant(scales: np.ndarray, codes: np.ndarray) -> np.ndarray:
    """q8_1.rs:50-63."""
    scales = np.ascontiguousarray(scales, np.uint16)
    codes = np.ascontiguousarray(codes, np.int8)
    out = np.empty(codes.shape, np.float32)
    lib().orc_q8_1_dequant(_p(scales, C.c_uint16), _p(codes, C.c_int8), scales.size, _p(out, C.c_float))
    return out


def q4_0_quant(x: np.ndarray):
    """Q4_0 blocks of 32 along the last axis (q4_0.rs:19-45).
    Returns (scales uint16 [..., D/32], packed uint8 [..., D/2]) in GGML nibble order."""
    x = to_f32(x)
    assert x.shape[-1] % 32 == 0
    nb = x.size // 32
    scales = np.empty(nb, np.uint16)
    packed = np.empty(nb * 16, np.uint8)
    lib().orc_q4_0_quant(_p(x, C.c_float), nb, _p(scales, C.c_uint16), _p(packed, C.c_uint8))
    return scales.reshape(x.shape[:-1] + (x.shape[-1] // 32,)), packed.reshape(x.shape[:-1] + (x.shape[-1] // 2,))


def q4_0_dequant(scales: np.ndarray, packed: np.ndarray) -> np.ndarray:
    """q4_0.rs:82-95."""
    scales = np.ascontiguousarray(scales, np.uint16)
    packed = np.ascontiguousarray(packed, np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.float32)
    lib().orc_q4_0_dequant(_p(scales, C.c_uint16), _p(packed, C.c_uint8), scales.size, _p(out, C.c_float))
    return out


def w4a8_quantize_row(a: np.ndarray):
    """Q4_0::quantize_row_q8 (q4_0.rs:199-214): (int8 codes [..., K], f32 scales [..., K/32])."""
    a = to_f32(a)
    assert a.shape[-1] % 32 == 0
    rows = a.reshape(-1, a.shape[-1])
    q = np.empty(rows.shape, np.int8)
    sc = np.empty((rows.shape[0], rows.shape[1] // 32), np.float32)
    for i in range(rows.shape[0]):
        lib().orc_w4a8_quantize_row(_p(rows[i], C.c_float), rows.shape[1], _p(q[i], C.c_int8), _p(sc[i], C.c_float))
    return q.reshape(a.shape), sc.reshape(a.shape[:-1] + (a.shape[-1] // 32,))


def w4a8_gemm(scales: np.ndarray, packed: np.ndarray, a: np.ndarray, threads: int = 0) -> np.ndarray:
    """Q4_0::w4a8_gemm (q4_0.rs:260-310): weights [N, K] as Q4_0 (scales uint16 [N, K/32], packed uint8 [N, K/2]),
    activations f32 [M, K]; returns f32 [M, N]."""
    scales = np.ascontiguousarray(scales, np.uint16)
    packed = np.ascontiguousarray(packed, np.uint8)
    a = to_f32(a)
    n, k = packed.shape[0], packed.shape[1] * 2
    m = a.shape[0]
    assert a.shape[1] == k and scales.shape == (n, k // 32)
    out = np.empty((m, n), np.float32)
    lib().orc_w4a8_gemm(_p(scales, C.c_uint16), _p(packed, C.c_uint8), n, k, _p(a, C.c_float), m, _p(out, C.c_float),
                        threads or hardware_threads())
    return out


def rms_norm(x: np.ndarray, eps: float) -> np.ndarray:
    """RmsNorm over the last axis (core/src/ops/nn/rms_norm.rs:28-66 with the generic rms_norm_f32 kernel): the
    input is cast to f32, normalised, and cast back to its own type."""
    dt = np.asarray(x).dtype
    buf = np.ascontiguousarray(to_f32(x)).copy()
    lib().orc_rms_norm_f32(_p(buf, C.c_float), buf.size // buf.shape[-1], buf.shape[-1], C.c_float(eps))
    return buf if dt == np.float32 else buf.astype(dt)


def ssigmoid(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(to_f32(x))
    out = np.empty_like(x)
    lib().orc_ssigmoid(_p(x, C.c_float), x.size, _p(out, C.c_float))
    return out


def silu(x: np.ndarray) -> np.ndarray:
    """Silu with the generic kernels (linalg/src/generic/silu.rs:26-30, :48-56): f32 in f32; f16 through f32 and back."""
    dt = np.asarray(x).dtype
    xf = np.ascontiguousarray(to_f32(x))
    out = np.empty_like(xf)
    lib().orc_silu_f32(_p(xf, C.c_float), xf.size, _p(out, C.c_float))
    return out if dt == np.float32 else out.astype(dt)


# ---- a3 -------------------------------------------------------------------------------------------

class KiviStore:
    """One per-(batch, head) store of QuantizedDynKeyValueCache
    (quant_dyn_kv_cache.rs:98-149 Value / :159-250 Key)."""

    def __init__(self, per_channel: bool, d: int, bits: int):
        assert bits in (4, 8)
        self.per_channel, self.d, self.bits = bool(per_channel), d, bits
        self.row_bytes = (d * bits + 7) // 8
        self._h = C.c_void_p(lib().orc_kivi_new(int(per_channel), d, bits))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_kivi_free(self._h)
            self._h = None

    def push(self, rows: np.ndarray):
        rows = np.ascontiguousarray(to_f32(rows).reshape(-1, self.d))
        lib().orc_kivi_push_rows(self._h, _p(rows, C.c_float), rows.shape[0], self.d)

    def __len__(self):
        return int(lib().orc_kivi_len(self._h))

    def raw(self):
        n_rows, n_par, n_res = C.c_int64(), C.c_int64(), C.c_int64()
        lib().orc_kivi_counts(self._h, C.byref(n_rows), C.byref(n_par), C.byref(n_res))
        n_sink = min(len(self), 4)
        codes = np.empty((n_rows.value, self.row_bytes), np.uint8)
        lo = np.empty(n_par.value, np.float32)
        scale = np.empty(n_par.value, np.float32)
        sink = np.empty((n_sink, self.d), np.float32)
        res = np.empty((n_res.value, self.d), np.float32)
        lib().orc_kivi_raw(self._h, _p(codes, C.c_uint8), _p(lo, C.c_float), _p(scale, C.c_float),
                           _p(sink, C.c_float), _p(res, C.c_float))
        return dict(codes=codes, lo=lo, scale=scale, sink=sink, residual=res)

    def dequant(self) -> np.ndarray:
        out = np.empty((len(self), self.d), np.float32)
        lib().orc_kivi_dequant(self._h, _p(out, C.c_float))
        return out


class QuantizedDynKeyValueCache:
    """QuantizedDynKvCacheState (quant_dyn_kv_cache.rs:366-495): one store per (b, h),
    ingest token by token, output the whole dequantised cache cast to the input dtype."""

    def __init__(self, bits: int, per_channel: bool):
        self.bits, self.per_channel, self.stores, self.lead = bits, per_channel, None, None

    def eval(self, x: np.ndarray) -> np.ndarray:
        assert x.ndim == 4
        b, h, s, d = x.shape
        if self.stores is None:
            self.lead = (b, h)
            self.stores = [KiviStore(self.per_channel, d, self.bits) for _ in range(b * h)]
        assert self.lead == (b, h)
        xf = to_f32(x)
        for bi in range(b):
            for hi in range(h):
                self.stores[bi * h + hi].push(xf[bi, hi])
        return from_f32(self.dequantized(), x.dtype)

    def dequantized(self) -> np.ndarray:
        b, h = self.lead
        t = len(self.stores[0])
        d = self.stores[0].d
        return np.stack([s.dequant() for s in self.stores]).reshape(b, h, t, d)


# ---- rotary embedding (the step right before the cache) ---------------------------------------------------

def rotate_half(x: np.ndarray) -> np.ndarray:
    """RotateHalf (transformers/src/ops/apply_rope.rs:58-74): concat(-x[.., D/2:], x[.., :D/2])."""
    half = x.shape[-1] // 2
    return np.concatenate([-x[..., half:], x[..., :half]], axis=-1)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """ApplyRope::eval (apply_rope.rs:155-163): Mul, Mul, Add as three ops of the input's dtype; numpy rounds
    every f16 / bf16 operation to the type, as the reference's element-wise ops do."""
    dt = x.dtype
    return ((x * cos.astype(dt)).astype(dt) + (rotate_half(x) * sin.astype(dt)).astype(dt)).astype(dt)


# ---- a7 -------------------------------------------------------------------------------------------

def _prep_sdpa(q, k, v, mask):
    in_dt = q.dtype
    q, k, v = to_f32(q), to_f32(k), to_f32(v)
    rank3 = q.ndim == 3
    if rank3:
        q, k, v = q[:, None], k[:, None], v[:, None]
    B, Hq, S, D = q.shape
    _, Hkv, T, _ = k.shape
    assert k.shape == v.shape and k.shape[0] == B and k.shape[3] == D and Hq % Hkv == 0
    Mb = Mh = 1
    m = None
    if mask is not None:
        m = to_f32(mask)
        if m.ndim == 3:
            m = m[:, None]
        Mb, Mh = m.shape[0], m.shape[1]
        m = np.ascontiguousarray(np.broadcast_to(m, (Mb, Mh, S, T)))
    return in_dt, rank3, q, k, v, m, (B, Hq, Hkv, S, T, D, Mb, Mh)


def flash_sdpa(q, k, v, mask=None, scale=None, causal=False, threads=1) -> np.ndarray:
    """FlashSdpaOp::eval (flash_sdpa.rs:103-163): cast to f32, attend per (b, q-head), cast back."""
    in_dt, rank3, q, k, v, m, dims = _prep_sdpa(q, k, v, mask)
    out = np.empty(q.shape, np.float32)
    lib().orc_flash_sdpa(_p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float),
                         _p(m, C.c_float) if m is not None else None, *dims,
                         float(scale) if scale is not None else 0.0, int(scale is not None), int(causal),
                         _p(out, C.c_float), int(threads))
    if rank3:
        out = out[:, 0]
    return from_f32(out, in_dt)


def naive_sdpa_f64(q, k, v, mask=None, scale=None, causal=False, threads=1) -> np.ndarray:
    """float64 softmax attention, the independent cross-check (test-rt/suite-unit/src/sdpa.rs:187-236)."""
    _, rank3, q, k, v, m, dims = _prep_sdpa(q, k, v, mask)
    out = np.empty(q.shape, np.float64)
    lib().orc_naive_sdpa_f64(_p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float),
                             _p(m, C.c_float) if m is not None else None, *dims,
                             float(scale) if scale is not None else 0.0, int(scale is not None), int(causal),
                             _p(out, C.c_double), int(threads))
    return out[:, 0] if rank3 else out


def hardware_threads() -> int:
    return int(lib().orc_hardware_threads())
