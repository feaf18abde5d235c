"""tract_b200 — B200 (sm_100a) KV-cache + attention path for tract, behind a C ABI.

The product is ``libb200kv.so`` (``include/b200kv.h``).  This package loads it with ctypes and
offers thin wrappers that take torch CUDA tensors (torch is used for device memory and streams
only).  There is no CPU fallback: if the library is missing or no CUDA device is present, calls
raise instead of computing something else.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200kv.so")

F32, F16, BF16 = 0, 1, 2
FMT_F32, FMT_F16, FMT_BF16, FMT_Q8_1, FMT_Q4_0, FMT_KIVI8, FMT_KIVI4 = 0, 1, 2, 3, 4, 5, 6
FORMATS = {"f32": FMT_F32, "f16": FMT_F16, "bf16": FMT_BF16, "q8_1": FMT_Q8_1, "q4_0": FMT_Q4_0,
           "kivi8": FMT_KIVI8, "kivi4": FMT_KIVI4}

# every symbol include/b200kv.h declares
EXPORTS = [
    "b200kv_last_error", "b200kv_version", "b200kv_create", "b200kv_destroy", "b200kv_seq_new", "b200kv_seq_free",
    "b200kv_seq_len", "b200kv_free_pages", "b200kv_page_bytes", "b200kv_append", "b200kv_attend", "b200kv_export",
    "b200kv_export_codes", "b200kv_truncate", "b200kv_fork", "b200kv_check", "b200kv_sdpa", "b200kv_profile",
    "b200kv_profile_read", "b200kv_attend_static_scratch", "b200kv_export_kivi", "b200kv_append_rope", "b200kv_rope",
    "b200kv_q40_packed_bytes", "b200kv_q40_pack", "b200kv_q40_scratch_bytes", "b200kv_q40_gemm", "b200kv_q40_check",
    "b200kv_rms_norm", "b200kv_silu_mul", "b200kv_add", "b200kv_argmax", "b200kv_gather_rows", "b200kv_cast",
    "b200kv_attend_window", "b200kv_trim", "b200kv_attend_rope", "b200kv_attend_q40", "b200kv_append_attend", "b200kv_q40_quantize", "b200kv_q40_gemm_quantized", "b200kv_q40_gemm_quantized_as",
    "b200kv_q40_silu_mul_quantize", "b200kv_q40_add_rms_norm_quantize", "b200kv_workspace_bytes", "b200kv_truncate_many", "b200kv_sdpa_check",
]
KERNEL_NAMES = {0: "table_scatter", 1: "append", 2: "decode", 3: "combine", 4: "export", 5: "sdpa_dense", 6: "prefill"}


class B200KvError(RuntimeError):
    pass


class Config(C.Structure):
    _fields_ = [("device", C.c_int32), ("format", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("has_values", C.c_int32), ("max_seqs", C.c_int32), ("max_seq_tokens", C.c_int64),
                ("pool_tokens", C.c_int64), ("flags", C.c_int32), ("max_q_heads", C.c_int32)]


_lib = None


def lib():
    """Loads the CUDA library; raises if it has not been built (no fallback path exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200KvError(f"{LIB_PATH} is missing: build it with `python -m tract_b200.build`")
        L = C.CDLL(LIB_PATH)
        vp, i32, i64, i64p, i32p = C.c_void_p, C.c_int32, C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int32)
        L.b200kv_last_error.restype = C.c_char_p
        L.b200kv_version.restype = C.c_char_p
        L.b200kv_create.argtypes = [C.POINTER(Config), C.POINTER(vp)]
        L.b200kv_destroy.argtypes = [vp]
        L.b200kv_workspace_bytes.argtypes = [C.POINTER(Config)]
        L.b200kv_workspace_bytes.restype = i64
        L.b200kv_seq_new.argtypes = [vp, i32p]
        L.b200kv_seq_free.argtypes = [vp, i32]
        L.b200kv_seq_len.argtypes = [vp, i32]
        L.b200kv_seq_len.restype = i64
        L.b200kv_free_pages.argtypes = [vp]
        L.b200kv_free_pages.restype = i64
        L.b200kv_page_bytes.argtypes = [vp]
        L.b200kv_page_bytes.restype = i64
        L.b200kv_append.argtypes = [vp, i32, i32p, i32, vp, i64p, vp, i64p, i32, vp]
        L.b200kv_append_rope.argtypes = [vp, i32, i32p, i32, vp, i64p, vp, i64p, vp, vp, i64p, i32, vp]
        L.b200kv_rope.argtypes = [vp, i64p, vp, vp, i64p, vp, i64p, i32, i32, i32, i32, i32, vp]
        L.b200kv_append_attend.argtypes = [vp, i32, i32p, i32, vp, i64p, vp, i64p, i32, vp, i64p, vp, i64p, i32, C.c_float, i32, vp]
        L.b200kv_attend.argtypes = [vp, i32, i32p, i32, i32, vp, i64p, vp, i64p, i32, C.c_float, i32, vp]
        L.b200kv_export.argtypes = [vp, i32, vp, i64p, vp, i64p, i32, vp]
        L.b200kv_export_codes.argtypes = [vp, i32, i32, vp, vp, vp]
        L.b200kv_truncate.argtypes = [vp, i32, i64]
        L.b200kv_truncate_many.argtypes = [vp, i32, i32p, i64p]
        L.b200kv_fork.argtypes = [vp, i32, i32p, vp]
        L.b200kv_attend_static_scratch.argtypes = [vp, i32, i32p, i32, vp, i64p, vp, i64p, i32, C.c_float, vp]
        L.b200kv_export_kivi.argtypes = [vp, i32, i32, vp, vp, vp, vp, vp, vp]
        L.b200kv_check.argtypes = [vp, vp]
        L.b200kv_profile.argtypes = [vp, i32]
        L.b200kv_profile_read.argtypes = [vp, i32, i32p, C.POINTER(C.c_float), i32p]
        L.b200kv_sdpa.argtypes = [vp, i64p, vp, i64p, vp, i64p, vp, i64p, i32, vp, i64p, i32, i32, i32, i32, i32, i32,
                                  i32, C.c_float, i32, vp]
        L.b200kv_attend_rope.argtypes = [vp, i32, i32p, i32, vp, i64p, vp, vp, i64, vp, i64p, i32, C.c_float, vp]
        L.b200kv_attend_q40.argtypes = [vp, i32, i32p, i32, vp, i64p, vp, vp, i64, vp, i64p, vp, i32, C.c_float, vp]
        L.b200kv_attend_window.argtypes = [vp, i32, i32p, i32, vp, i64p, vp, i64p, i32, C.c_float, i64, vp]
        L.b200kv_trim.argtypes = [vp, i32, i64]
        _lib = L
    return _lib


def _ck(rc):
    if rc != 0:
        raise B200KvError(lib().b200kv_last_error().decode())


def _dtype_code(t):
    import torch

    try:
        return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[t.dtype]
    except KeyError:
        raise B200KvError(f"unsupported dtype {t.dtype}") from None


def _strides(t, n):
    """Leading n strides of a tensor whose last axis must be contiguous."""
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        raise B200KvError("the innermost (head_dim) axis must be contiguous")
    return (C.c_int64 * n)(*[int(s) for s in t.stride()[:n]])


def _stream():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ids(seqs):
    return (C.c_int32 * len(seqs))(*[int(s) for s in seqs])


class KvCache:
    """One layer's paged K (and V) store for up to ``max_seqs`` independent sequences."""

    def __init__(self, fmt, n_kv_heads, head_dim, max_seqs, max_seq_tokens, pool_tokens=None, has_values=True,
                 device=None, per_token=False, max_q_heads=0):
        import torch

        if not torch.cuda.is_available():
            raise B200KvError("no CUDA device: tract_b200 has no CPU fallback")
        self.device = torch.cuda.current_device() if device is None else int(device)
        self.fmt = FORMATS[fmt] if isinstance(fmt, str) else int(fmt)
        self.n_kv_heads, self.head_dim, self.has_values = n_kv_heads, head_dim, bool(has_values)
        cfg = Config(self.device, self.fmt, n_kv_heads, head_dim, int(has_values), max_seqs, max_seq_tokens,
                     pool_tokens if pool_tokens is not None else max_seqs * max_seq_tokens, int(bool(per_token)), int(max_q_heads))
        self.workspace_bytes = int(lib().b200kv_workspace_bytes(C.byref(cfg)))  # what create allocates beside the pages, once
        h = C.c_void_p()
        _ck(lib().b200kv_create(C.byref(cfg), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib().b200kv_destroy(self._h)
            self._h = None

    __del__ = close

    # -- sequences --
    def new_seq(self) -> int:
        s = C.c_int32()
        _ck(lib().b200kv_seq_new(self._h, C.byref(s)))
        return s.value

    def free_seq(self, seq):
        _ck(lib().b200kv_seq_free(self._h, seq))

    def seq_len(self, seq) -> int:
        n = lib().b200kv_seq_len(self._h, seq)
        if n < 0:
            raise B200KvError(lib().b200kv_last_error().decode())
        return int(n)

    def free_pages(self) -> int:
        return int(lib().b200kv_free_pages(self._h))

    def page_bytes(self) -> int:
        return int(lib().b200kv_page_bytes(self._h))

    # -- hot path --
    def append(self, seqs, k_new, v_new=None):
        """k_new / v_new: [n_seqs, Hkv, S, D] CUDA tensors."""
        assert k_new.dim() == 4 and k_new.shape[0] == len(seqs)
        _ck(lib().b200kv_append(self._h, len(seqs), _ids(seqs), k_new.shape[2], k_new.data_ptr(), _strides(k_new, 3),
                                v_new.data_ptr() if v_new is not None else None,
                                _strides(v_new, 3) if v_new is not None else None, _dtype_code(k_new), _stream()))

    def append_rope(self, seqs, k_new, v_new, cos, sin):
        """append() with ApplyRope fused on the key side; cos / sin: [n_seqs or 1, S, D] of k_new's dtype."""
        assert k_new.dim() == 4 and cos.dim() == 3 and cos.shape == sin.shape and cos.stride() == sin.stride()
        rs = (C.c_int64 * 2)(0 if cos.shape[0] == 1 else cos.stride(0), cos.stride(1))
        _ck(lib().b200kv_append_rope(self._h, len(seqs), _ids(seqs), k_new.shape[2], k_new.data_ptr(), _strides(k_new, 3),
                                     v_new.data_ptr() if v_new is not None else None,
                                     _strides(v_new, 3) if v_new is not None else None, cos.data_ptr(), sin.data_ptr(), rs,
                                     _dtype_code(k_new), _stream()))

    def attend(self, seqs, q, scale=None, causal=True, out=None):
        """q: [n_seqs, Hq, S, D]; returns attention of the last S cached positions over the whole cache."""
        import torch

        assert q.dim() == 4 and q.shape[0] == len(seqs)
        if out is None:
            out = torch.empty_like(q, memory_format=torch.contiguous_format)
        _ck(lib().b200kv_attend(self._h, len(seqs), _ids(seqs), q.shape[1], q.shape[2], q.data_ptr(), _strides(q, 3),
                                out.data_ptr(), _strides(out, 3), _dtype_code(q), float(scale or 0.0), int(causal),
                                _stream()))
        return out

    def append_attend(self, seqs, k_new, v_new, q, scale=None, causal=True, out=None):
        """append(seqs, k_new, v_new) then attend(seqs, q): the fused cache + attention op as one call into the library."""
        import torch

        assert k_new.dim() == 4 and q.dim() == 4 and q.shape[0] == len(seqs) == k_new.shape[0] and q.shape[2] == k_new.shape[2]
        assert q.dtype == k_new.dtype
        if out is None:
            out = torch.empty_like(q, memory_format=torch.contiguous_format)
        _ck(lib().b200kv_append_attend(self._h, len(seqs), _ids(seqs), k_new.shape[2], k_new.data_ptr(), _strides(k_new, 3),
                                       v_new.data_ptr(), _strides(v_new, 3), q.shape[1], q.data_ptr(), _strides(q, 3), out.data_ptr(),
                                       _strides(out, 3), _dtype_code(q), float(scale or 0.0), int(causal), _stream()))
        return out

    def attend_static_scratch(self, seqs, q, scale=None, out=None):
        """Decode attention (q: [n_seqs, Hq, 1, D]) that allocates nothing on the device: the split partials go
        to a fixed array inside the library.  Raises if the call needs more partials than the array holds."""
        import torch

        assert q.dim() == 4 and q.shape[0] == len(seqs) and q.shape[2] == 1
        if out is None:
            raise B200KvError("pass `out`: this call path must not allocate")
        _ck(lib().b200kv_attend_static_scratch(self._h, len(seqs), _ids(seqs), q.shape[1], q.data_ptr(), _strides(q, 3),
                                               out.data_ptr(), _strides(out, 3), _dtype_code(q), float(scale or 0.0),
                                               _stream()))
        return out

    # -- state --
    def export(self, seq, dtype):
        """Contiguous [Hkv, len, D] K (and V) of one sequence, dequantised for quantised formats."""
        import torch

        n = self.seq_len(seq)
        k = torch.empty((self.n_kv_heads, n, self.head_dim), dtype=dtype, device=f"cuda:{self.device}")
        v = torch.empty_like(k) if self.has_values else None
        _ck(lib().b200kv_export(self._h, seq, k.data_ptr(), _strides(k, 2), v.data_ptr() if v is not None else None,
                                _strides(v, 2) if v is not None else None, _dtype_code(k), _stream()))
        return k, v

    def export_codes(self, seq, which):
        """(codes, scales-as-uint16-bits) of K (which=0) or V (which=1) for the block-quantised formats."""
        import torch

        n = self.seq_len(seq)
        row = self.head_dim if self.fmt == FMT_Q8_1 else self.head_dim // 2
        codes = torch.empty((self.n_kv_heads, n, row), dtype=torch.int8 if self.fmt == FMT_Q8_1 else torch.uint8,
                            device=f"cuda:{self.device}")
        scales = torch.empty((self.n_kv_heads, n, self.head_dim // 32), dtype=torch.float16, device=f"cuda:{self.device}")
        _ck(lib().b200kv_export_codes(self._h, seq, which, codes.data_ptr(), scales.data_ptr(), _stream()))
        return codes, scales

    def export_kivi(self, seq, which, per_channel):
        """Raw stores of a KIVI cache: dict(codes, lo, scale, sink, residual) in the reference's order."""
        import torch

        n, H, D = self.seq_len(seq), self.n_kv_heads, self.head_dim
        bits = 8 if self.fmt == FMT_KIVI8 else 4
        n_sink, n_after = min(n, 4), max(n - 4, 0)
        n_q = (n_after // 32) * 32 if per_channel else n_after
        n_res = n_after - n_q if per_channel else 0
        dev = f"cuda:{self.device}"
        codes = torch.zeros((H, n_q, D * bits // 8), dtype=torch.uint8, device=dev)
        npar = (H, n_q // 32, D) if per_channel else (H, n_q)
        lo, scale = torch.zeros(npar, device=dev), torch.zeros(npar, device=dev)
        sink, res = torch.zeros((H, n_sink, D), device=dev), torch.zeros((H, n_res, D), device=dev)
        _ck(lib().b200kv_export_kivi(self._h, seq, which, codes.data_ptr(), lo.data_ptr(), scale.data_ptr(), sink.data_ptr(),
                                     res.data_ptr(), _stream()))
        return dict(codes=codes, lo=lo, scale=scale, sink=sink, residual=res)

    def truncate(self, seq, length):
        _ck(lib().b200kv_truncate(self._h, seq, length))

    def truncate_many(self, seqs, lengths):
        """truncate() for a batch in one call: every sequence is checked before any changes."""
        _ck(lib().b200kv_truncate_many(self._h, len(seqs), _ids(seqs), (C.c_int64 * len(seqs))(*[int(n) for n in lengths])))

    def prepared_step(self, seqs, k_new, v_new, q, out, rollback_to=None, scale=None, causal=True):
        """A zero-argument callable that runs append_attend(seqs, k_new, v_new, q, out=out) -- and, when `rollback_to`
        (one length per sequence) is given, truncate_many(seqs, rollback_to) after it -- with every argument marshalled
        once, here: what a serving loop that calls the C ABI directly pays per step, without Python's per-call packing.
        The tensors must stay alive and in place; the current CUDA stream is looked up at every call."""
        import torch

        L, h, n = lib(), self._h, len(seqs)
        ids = _ids(seqs)
        ks, vs, qs, os_ = _strides(k_new, 3), _strides(v_new, 3), _strides(q, 3), _strides(out, 3)
        kp, vp_, qp, op = (C.c_void_p(t.data_ptr()) for t in (k_new, v_new, q, out))
        n_new, hq, dt, sc, ca = int(k_new.shape[2]), int(q.shape[1]), _dtype_code(q), C.c_float(scale or 0.0), int(causal)
        lens = (C.c_int64 * n)(*[int(x) for x in rollback_to]) if rollback_to is not None else None
        keep = (k_new, v_new, q, out)

        def call(_keep=keep):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            if L.b200kv_append_attend(h, n, ids, n_new, kp, ks, vp_, vs, hq, qp, qs, op, os_, dt, sc, ca, st) != 0:
                raise B200KvError(L.b200kv_last_error().decode())
            if lens is not None and L.b200kv_truncate_many(h, n, ids, lens) != 0:
                raise B200KvError(L.b200kv_last_error().decode())

        return call

    def trim(self, seq, keep_last):
        """Gives the pages before the last keep_last tokens back to the pool (sliding-window memory bound)."""
        _ck(lib().b200kv_trim(self._h, seq, C.c_int64(keep_last)))

    def attend_window(self, seqs, q, window, scale=None, out=None):
        """Decode attention (q: [n_seqs, Hq, 1, D]) over the last `window` cached tokens of every sequence."""
        import torch

        assert q.dim() == 4 and q.shape[0] == len(seqs) and q.shape[2] == 1
        if out is None:
            out = torch.empty_like(q, memory_format=torch.contiguous_format)
        _ck(lib().b200kv_attend_window(self._h, len(seqs), _ids(seqs), q.shape[1], q.data_ptr(), _strides(q, 3), out.data_ptr(),
                                       _strides(out, 3), _dtype_code(q), C.c_float(scale or 0.0), C.c_int64(window), _stream()))
        return out

    def attend_rope(self, seqs, q, cos, sin, scale=None, out=None):
        """Decode attention of ApplyRope(q, cos, sin) (q: [n_seqs, Hq, 1, D]; cos, sin: [n_seqs, 1, D] or [n_seqs, D])."""
        import torch

        assert q.dim() == 4 and q.shape[0] == len(seqs) and q.shape[2] == 1
        cos, sin = cos.reshape(len(seqs), -1), sin.reshape(len(seqs), -1)
        assert cos.dtype == q.dtype and sin.dtype == q.dtype and cos.stride(1) == 1 and sin.stride(1) == 1
        assert cos.stride(0) == sin.stride(0) and cos.shape[1] == q.shape[3]
        if out is None:
            out = torch.empty_like(q, memory_format=torch.contiguous_format)
        _ck(lib().b200kv_attend_rope(self._h, len(seqs), _ids(seqs), q.shape[1], q.data_ptr(), _strides(q, 3), cos.data_ptr(),
                                     sin.data_ptr(), C.c_int64(cos.stride(0)), out.data_ptr(), _strides(out, 3), _dtype_code(q),
                                     C.c_float(scale or 0.0), _stream()))
        return out

    def attend_q40(self, seqs, q, scratch, cos=None, sin=None, scale=None, out=None):
        """Decode attention (of ApplyRope(q) when cos / sin are given) left in `scratch` as the quantised activation of a
        Q40Linear over [n_seqs, Hq * D]; also written to `out` when given.  Follow with Q40Linear.gemm_quantized(n_seqs, ..)."""
        assert q.dim() == 4 and q.shape[0] == len(seqs) and q.shape[2] == 1
        assert scratch.numel() >= Q40Linear.scratch_bytes(q.shape[1] * q.shape[3], len(seqs))
        stride = 0
        if cos is not None:
            cos, sin = cos.reshape(len(seqs), -1), sin.reshape(len(seqs), -1)
            assert cos.dtype == q.dtype and sin.dtype == q.dtype and cos.stride(1) == 1 and sin.stride(1) == 1
            assert cos.stride(0) == sin.stride(0) and cos.shape[1] == q.shape[3]
            stride = cos.stride(0)
        _ck(lib().b200kv_attend_q40(self._h, len(seqs), _ids(seqs), q.shape[1], q.data_ptr(), _strides(q, 3),
                                    cos.data_ptr() if cos is not None else None, sin.data_ptr() if sin is not None else None,
                                    C.c_int64(stride), out.data_ptr() if out is not None else None,
                                    _strides(out, 3) if out is not None else None, scratch.data_ptr(), _dtype_code(q),
                                    C.c_float(scale or 0.0), _stream()))
        return out

    def fork(self, seq) -> int:
        s = C.c_int32()
        _ck(lib().b200kv_fork(self._h, seq, C.byref(s), _stream()))
        return s.value

    def check(self):
        _ck(lib().b200kv_check(self._h, _stream()))

    def profile(self, enable=True, force_simt=False, kivi_cuda_core=False, stall_next_decode=False):
        """Timing records on / off and the test hooks of b200kv_profile (stall_next_decode: one CTA of the next decode
        launch gives up on a copy nobody issued, after 1 ms)."""
        _ck(lib().b200kv_profile(self._h, int(bool(enable)) | (2 if force_simt else 0) | (4 if kivi_cuda_core else 0) |
                                 (8 if stall_next_decode else 0)))

    def profile_read(self, max_records=65536):
        """[(kernel name, milliseconds)] of the launches recorded since the last read."""
        ids = (C.c_int32 * max_records)()
        ms = (C.c_float * max_records)()
        n = C.c_int32()
        _ck(lib().b200kv_profile_read(self._h, max_records, ids, ms, C.byref(n)))
        return [(KERNEL_NAMES.get(ids[i], str(ids[i])), ms[i]) for i in range(n.value)]


class Q40Linear:
    """A Q4_0 weight matrix [N, K] on the device, applied with the arithmetic of Q4_0::w4a8_gemm
    (linalg/src/frame/block_quant/q4_0.rs:260-310).  `blocks`: uint8 CUDA tensor [N, K/32, 18], the reference's storage."""

    def __init__(self, blocks, max_m=8):
        import torch

        assert blocks.dtype == torch.uint8 and blocks.dim() == 3 and blocks.shape[2] == 18 and blocks.is_contiguous()
        self.n, self.k = int(blocks.shape[0]), int(blocks.shape[1]) * 32
        L = lib()
        L.b200kv_q40_packed_bytes.restype = C.c_int64
        L.b200kv_q40_scratch_bytes.restype = C.c_int64
        nbytes = L.b200kv_q40_packed_bytes(C.c_int64(self.n), C.c_int64(self.k))
        if nbytes < 0:
            raise B200KvError("Q4_0 weights need K a multiple of 32")
        self.packed = torch.empty(nbytes, dtype=torch.uint8, device=blocks.device)
        self.max_m = max_m
        self.scratch = torch.empty(L.b200kv_q40_scratch_bytes(C.c_int64(self.k), max_m), dtype=torch.uint8, device=blocks.device)
        with torch.cuda.device(blocks.device):
            _ck(L.b200kv_q40_pack(C.c_void_p(blocks.data_ptr()), C.c_int64(self.n), C.c_int64(self.k), C.c_void_p(self.packed.data_ptr()),
                                  _stream()))

    @staticmethod
    def scratch_bytes(k, m):
        L = lib()
        L.b200kv_q40_scratch_bytes.restype = C.c_int64
        return L.b200kv_q40_scratch_bytes(C.c_int64(k), int(m))

    def gemm(self, a, out=None, scratch=None):
        """a: [M, K] f32 / f16 / bf16 CUDA tensor (rows contiguous); returns f32 [M, N].  `scratch`: a uint8 CUDA tensor of at
        least scratch_bytes(K, M), for callers that share one scratch between layers (M above this layer's max_m needs it)."""
        import torch

        assert a.dim() == 2 and a.shape[1] == self.k and a.stride(1) == 1
        if scratch is None:
            assert a.shape[0] <= self.max_m
            scratch = self.scratch
        else:
            assert scratch.numel() >= self.scratch_bytes(self.k, a.shape[0])
        if out is None:
            out = torch.empty((a.shape[0], self.n), dtype=torch.float32, device=a.device)
        with torch.cuda.device(a.device):
            _ck(lib().b200kv_q40_gemm(C.c_void_p(self.packed.data_ptr()), C.c_int64(self.n), C.c_int64(self.k), C.c_void_p(a.data_ptr()),
                                      C.c_int64(a.stride(0)), int(a.shape[0]), _dtype_code(a), C.c_void_p(scratch.data_ptr()),
                                      C.c_void_p(out.data_ptr()), C.c_int64(out.stride(0)), _stream()))
        return out

    def gemm_quantized(self, m, out=None, scratch=None):
        """The product with the m activation rows that `scratch` already holds in quantised form (q40_quantize,
        q40_silu_mul_quantize or q40_add_rms_norm_quantize on the same stream)."""
        import torch

        scratch = self.scratch if scratch is None else scratch
        assert scratch.numel() >= self.scratch_bytes(self.k, m)
        if out is None:
            out = torch.empty((m, self.n), dtype=torch.float32, device=self.packed.device)
        assert out.shape == (m, self.n) and out.stride(1) == 1  # f32, or f16 / bf16: the result rounded once on the way out
        with torch.cuda.device(self.packed.device):
            _ck(lib().b200kv_q40_gemm_quantized_as(C.c_void_p(self.packed.data_ptr()), C.c_int64(self.n), C.c_int64(self.k), int(m),
                                                   C.c_void_p(scratch.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int64(out.stride(0)),
                                                   _dtype_code(out), _stream()))
        return out

    def check(self, scratch=None):
        _ck(lib().b200kv_q40_check(C.c_void_p((self.scratch if scratch is None else scratch).data_ptr()), _stream()))


def q40_quantize(a, scratch):
    """Q4_0::quantize_row_q8 of the rows of `a` ([M, K], rows contiguous) into `scratch` (Q40Linear.scratch_bytes(K, M))."""
    import torch

    assert a.dim() == 2 and a.stride(1) == 1 and scratch.numel() >= Q40Linear.scratch_bytes(a.shape[1], a.shape[0])
    with torch.cuda.device(a.device):
        _ck(lib().b200kv_q40_quantize(C.c_void_p(a.data_ptr()), C.c_int64(a.stride(0)), int(a.shape[0]), _dtype_code(a), C.c_int64(a.shape[1]),
                                      C.c_void_p(scratch.data_ptr()), _stream()))


def q40_silu_mul_quantize(gate, up, scratch):
    """scratch <- quantised Silu(gate) * up; gate, up: [M, K] windows with contiguous rows."""
    import torch

    assert gate.dim() == 2 and gate.shape == up.shape and gate.dtype == up.dtype and gate.stride(1) == 1 and up.stride(1) == 1
    assert scratch.numel() >= Q40Linear.scratch_bytes(gate.shape[1], gate.shape[0])
    with torch.cuda.device(gate.device):
        _ck(lib().b200kv_q40_silu_mul_quantize(C.c_void_p(gate.data_ptr()), C.c_int64(gate.stride(0)), C.c_void_p(up.data_ptr()),
                                               C.c_int64(up.stride(0)), int(gate.shape[0]), _dtype_code(gate), C.c_int64(gate.shape[1]),
                                               C.c_void_p(scratch.data_ptr()), _stream()))


def q40_add_rms_norm_quantize(x, scratch, eps, weight=None, residual=None, x_out=None):
    """v = x + residual (stored to x_out when given; x_out may be x); scratch <- quantised RmsNorm(v, eps) * weight.  f32."""
    import torch

    f32 = torch.float32
    assert x.dim() == 2 and x.dtype == f32 and x.stride(1) == 1 and scratch.numel() >= Q40Linear.scratch_bytes(x.shape[1], x.shape[0])
    for t in (residual, x_out):
        assert t is None or (t.dtype == f32 and t.shape == x.shape and t.stride(1) == 1)
    assert weight is None or (weight.dtype == f32 and weight.numel() == x.shape[1] and weight.is_contiguous())
    ptr = lambda t: C.c_void_p(t.data_ptr() if t is not None else 0)
    st = lambda t: C.c_int64(t.stride(0) if t is not None else 0)
    with torch.cuda.device(x.device):
        _ck(lib().b200kv_q40_add_rms_norm_quantize(ptr(x), st(x), ptr(residual), st(residual), ptr(weight), C.c_float(eps), ptr(x_out), st(x_out),
                                                   int(x.shape[0]), C.c_int64(x.shape[1]), C.c_void_p(scratch.data_ptr()), _stream()))


def rms_norm(x, eps, weight=None, out=None):
    """RmsNorm over the last axis of a 2-D CUDA tensor (rows contiguous), optionally times a weight vector."""
    import torch

    assert x.dim() == 2 and x.stride(1) == 1
    if out is None:
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
    with torch.cuda.device(x.device):
        _ck(lib().b200kv_rms_norm(C.c_void_p(x.data_ptr()), C.c_int64(x.stride(0)), C.c_void_p(weight.data_ptr() if weight is not None else 0),
                                  C.c_void_p(out.data_ptr()), C.c_int64(out.stride(0)), C.c_int64(x.shape[0]), int(x.shape[1]),
                                  C.c_float(eps), _dtype_code(x), _stream()))
    return out


def silu_mul(gate, up=None, out=None):
    import torch

    assert gate.is_contiguous() and (up is None or up.is_contiguous())
    if out is None:
        out = torch.empty_like(gate)
    with torch.cuda.device(gate.device):
        _ck(lib().b200kv_silu_mul(C.c_void_p(gate.data_ptr()), C.c_void_p(up.data_ptr() if up is not None else 0), C.c_void_p(out.data_ptr()),
                                  C.c_int64(gate.numel()), _dtype_code(gate), _stream()))
    return out


def add(a, b, out=None):
    import torch

    assert a.is_contiguous() and b.is_contiguous() and a.shape == b.shape
    if out is None:
        out = torch.empty_like(a)
    with torch.cuda.device(a.device):
        _ck(lib().b200kv_add(C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int64(a.numel()),
                             _dtype_code(a), _stream()))
    return out


def argmax(x, out=None):
    import torch

    assert x.dim() == 2 and x.dtype == torch.float32 and x.stride(1) == 1
    if out is None:
        out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        _ck(lib().b200kv_argmax(C.c_void_p(x.data_ptr()), C.c_int64(x.stride(0)), C.c_int64(x.shape[0]), int(x.shape[1]),
                                C.c_void_p(out.data_ptr()), _stream()))
    return out


def gather_rows(table, ids, out=None):
    import torch

    assert table.dim() == 2 and table.is_contiguous() and ids.dtype == torch.int32
    if out is None:
        out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    with torch.cuda.device(table.device):
        _ck(lib().b200kv_gather_rows(C.c_void_p(table.data_ptr()), C.c_int64(table.shape[0]), C.c_int64(table.shape[1] * table.element_size()),
                                     C.c_void_p(ids.data_ptr()), C.c_int64(ids.numel()), C.c_void_p(out.data_ptr()), _stream()))
    return out


def cast(src, dst):
    """dst[...] = src[...] converted through f32; 2-D windows (last axis contiguous) of CUDA tensors of equal shape."""
    import torch

    assert src.dim() == 2 and dst.shape == src.shape and src.stride(1) == 1 and dst.stride(1) == 1
    with torch.cuda.device(src.device):
        _ck(lib().b200kv_cast(C.c_void_p(src.data_ptr()), C.c_int64(src.stride(0)), _dtype_code(src), C.c_void_p(dst.data_ptr()),
                              C.c_int64(dst.stride(0)), _dtype_code(dst), C.c_int64(src.shape[0]), C.c_int64(src.shape[1]), _stream()))
    return dst


def rope(x, cos, sin, out=None):
    """ApplyRope on a [B, H, S, D] tensor; cos / sin: [B or 1, S, D]."""
    import torch

    if out is None:
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
    rs = (C.c_int64 * 2)(0 if cos.shape[0] == 1 else cos.stride(0), cos.stride(1))
    with torch.cuda.device(x.device):
        _ck(lib().b200kv_rope(x.data_ptr(), _strides(x, 3), cos.data_ptr(), sin.data_ptr(), rs, out.data_ptr(), _strides(out, 3),
                              x.shape[0], x.shape[1], x.shape[2], x.shape[3], _dtype_code(x), _stream()))
    return out


def sdpa_check():
    """Synchronises the current stream and raises if a bounded wait of an sdpa() call on this device expired."""
    lib().b200kv_sdpa_check.argtypes = [C.c_void_p]
    _ck(lib().b200kv_sdpa_check(_stream()))


def sdpa(q, k, v, mask=None, scale=None, causal=False):
    """Lone Sdpa on dense tensors (rank 3 [B,S,D] or rank 4 [B,H,S,D]); mask is additive, broadcast over b / h."""
    import torch

    rank3 = q.dim() == 3
    if rank3:
        q, k, v = q.unsqueeze(1), k.unsqueeze(1), v.unsqueeze(1)
        if mask is not None:
            mask = mask.unsqueeze(1)
    B, Hq, S, D = q.shape
    _, Hkv, T, _ = k.shape
    out = torch.empty((B, Hq, S, D), dtype=q.dtype, device=q.device)
    ms, mptr, mdt = None, None, 0
    if mask is not None:
        mask = mask.expand(mask.shape[0], mask.shape[1], S, T)  # stride 0 where broadcast
        st = list(mask.stride())
        if mask.shape[0] == 1:
            st[0] = 0
        if mask.shape[1] == 1:
            st[1] = 0
        ms, mptr, mdt = (C.c_int64 * 4)(*st), mask.data_ptr(), _dtype_code(mask)
    with torch.cuda.device(q.device):
        _ck(lib().b200kv_sdpa(q.data_ptr(), _strides(q, 3), k.data_ptr(), _strides(k, 3), v.data_ptr(), _strides(v, 3),
                              mptr, ms, mdt, out.data_ptr(), _strides(out, 3), B, Hq, Hkv, S, T, D, _dtype_code(q),
                              float(scale or 0.0), int(causal), _stream()))
    return out[:, 0] if rank3 else out
