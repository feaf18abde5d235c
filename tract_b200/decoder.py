"""Decode-loop driver for a Llama-shaped decoder built from the library's ops: per-layer paged KV caches, Q4_0 linear
layers, RmsNorm, RoPE, SiLU gating, greedy argmax.

The caller of the hot path in the reference is examples/causal_llm/src/lib.rs:290-408 (prompt processing, then one
token per step with the KV caches as model state) and cli/src/llm.rs:47-139 (the pp / tg benchmark loop).  Here the
decoder block is spelled out op by op, each op being the library's replacement for the node tract would run:

    x -> RmsNorm * w -> [Wq | Wk | Wv] (Q4_0, int8 activations) -> RoPE(q), RoPE(k) fused into the cache append
      -> attention over the cache -> Wo -> + x -> RmsNorm * w -> SiLU(Wg .) * (Wu .) -> Wd -> + x

Activations are f32 between ops (the W4A8 GEMM of tract-linalg returns f32); q, k, v and the attention output are
cast to the cache's 16-bit type, as tract-cuda casts them for its flash-attention kernel.  The stretches between two
cache calls are replayed as CUDA graphs (their launches have no per-step host state); the cache calls themselves
carry the sequence lengths and stay ordinary launches.
"""
from __future__ import annotations

import dataclasses
import math

import tract_b200 as kv


@dataclasses.dataclass
class Shape:
    hidden: int = 4096
    n_layers: int = 32
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5


def random_q40_blocks(torch, n, k, gen, device, scale=None):
    """[n, k/32, 18] uint8: random nibbles, f16 scales that keep the layer's output near unit variance."""
    blocks = torch.randint(0, 256, (n, k // 32, 18), dtype=torch.uint8, generator=gen, device=device)
    s = scale if scale is not None else 1.0 / (4.6 * math.sqrt(k))  # nibble - 8 has a standard deviation of ~4.6
    scales = (torch.rand((n, k // 32), generator=gen, device=device) * 0.5 + 0.75) * s
    blocks[:, :, :2] = scales.to(torch.float16).view(torch.uint8).reshape(n, k // 32, 2)
    return blocks


class Decoder:
    def __init__(self, shape: Shape, n_seqs: int, max_tokens: int, kv_format="f16", seed=0, device="cuda", use_graphs=True,
                 weights=None):
        import torch

        self.torch, self.shape, self.B = torch, shape, n_seqs
        sh, dev = shape, torch.device(device)
        self.dev = dev
        self.kv_dtype = torch.bfloat16 if kv_format == "bf16" else torch.float16
        gen = torch.Generator(device=dev).manual_seed(seed)
        qkv_rows = (sh.n_q_heads + 2 * sh.n_kv_heads) * sh.head_dim
        self.host_blocks = {}

        def linear(name, n, k):
            blocks = weights[name] if weights is not None else random_q40_blocks(torch, n, k, gen, dev)
            if weights is None and n * k <= 1 << 22:
                self.host_blocks[name] = blocks.cpu().numpy()  # small models: kept for the parity tests
            return kv.Q40Linear(blocks.to(dev), max_m=n_seqs)

        def linear_rows(names, n, k):
            """Matrices that read the same activation (gate and up), stacked row-wise into one: one quantisation, one launch."""
            parts = []
            for name in names:
                parts.append(weights[name].to(dev) if weights is not None else random_q40_blocks(torch, n, k, gen, dev))
                if weights is None and n * k <= 1 << 22:
                    self.host_blocks[name] = parts[-1].cpu().numpy()
            return kv.Q40Linear(torch.cat(parts, 0).contiguous(), max_m=n_seqs)

        def norm_weight(name):
            w = weights[name] if weights is not None else (torch.rand(sh.hidden, generator=gen, device=dev) * 0.2 + 0.9)
            return w.to(dev, torch.float32)

        self.layers = []
        for i in range(sh.n_layers):
            self.layers.append(dict(
                attn_norm=norm_weight(f"l{i}.attn_norm"), ffn_norm=norm_weight(f"l{i}.ffn_norm"),
                wqkv=linear(f"l{i}.wqkv", qkv_rows, sh.hidden), wo=linear(f"l{i}.wo", sh.hidden, sh.n_q_heads * sh.head_dim),
                wgu=linear_rows([f"l{i}.wg", f"l{i}.wu"], sh.ffn, sh.hidden), wd=linear(f"l{i}.wd", sh.hidden, sh.ffn),
                cache=kv.KvCache(kv_format, sh.n_kv_heads, sh.head_dim, max_seqs=n_seqs, max_seq_tokens=max_tokens)))
        self.final_norm = norm_weight("final_norm")
        self.lm_head = linear("lm_head", sh.vocab, sh.hidden)
        self.embed = (weights["embed"] if weights is not None else torch.randn((sh.vocab, sh.hidden), generator=gen, device=dev)).to(dev, torch.float32)
        self.seqs = [[layer["cache"].new_seq() for _ in range(n_seqs)] for layer in self.layers]
        # rotary tables for every position the caches can hold: cos / sin of [position, head_dim], halves repeated
        inv = 1.0 / (sh.rope_theta ** (torch.arange(0, sh.head_dim, 2, device=dev, dtype=torch.float64) / sh.head_dim))
        ang = torch.arange(max_tokens, device=dev, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = torch.cat([ang.cos(), ang.cos()], 1).to(self.kv_dtype).contiguous()
        self.sin = torch.cat([ang.sin(), ang.sin()], 1).to(self.kv_dtype).contiguous()
        B, f32 = n_seqs, torch.float32
        z = lambda *s, dt=f32: torch.zeros(s, dtype=dt, device=dev)
        self.x = z(B, sh.hidden)  # the residual stream
        # q, k and v of one step in the cache's tensor type: one buffer (one cast launch), three strided views of it
        nq, nk = sh.n_q_heads * sh.head_dim, sh.n_kv_heads * sh.head_dim
        self.qkv16 = z(B, nq + 2 * nk, dt=self.kv_dtype)
        heads = lambda lo, n: self.qkv16[:, lo:lo + n * sh.head_dim].unflatten(1, (n, 1, sh.head_dim))
        self.q16, self.k16, self.v16 = heads(0, sh.n_q_heads), heads(nq, sh.n_kv_heads), heads(nq + nk, sh.n_kv_heads)
        self.proj, self.gate_up = z(B, sh.hidden), z(B, 2 * sh.ffn)
        # the quantised activation of the GEMM in flight; every producer and GEMM of a step runs on one stream, in order
        self.scratch = torch.empty(kv.Q40Linear.scratch_bytes(max(sh.hidden, sh.ffn, nq), B), dtype=torch.uint8, device=dev)
        self.logits = z(B, sh.vocab)
        self.tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.cos_t, self.sin_t = z(B, sh.head_dim, dt=self.kv_dtype), z(B, sh.head_dim, dt=self.kv_dtype)
        self.lengths = [0] * n_seqs
        self.graphs = None
        if use_graphs:
            self._capture()

    # ---- the launches between two cache calls ----------------------------------------------------------
    # The residual add of a block's output is folded into the RmsNorm that follows it, and every RmsNorm and the gated
    # activation into the quantiser of the GEMM they feed: `proj` holds the output that is still to be added to `x`.
    def _pre_attention(self, L, first):
        sh = self.shape
        kv.q40_add_rms_norm_quantize(self.x, self.scratch, sh.eps, weight=L["attn_norm"], residual=None if first else self.proj,
                                     x_out=None if first else self.x)
        # q | k | v leave the GEMM in the cache's tensor type; the query is rotated where the decode kernel loads it (attend_rope)
        L["wqkv"].gemm_quantized(self.B, self.qkv16, scratch=self.scratch)

    def _post_attention(self, L):
        sh = self.shape
        L["wo"].gemm_quantized(self.B, self.proj, scratch=self.scratch)  # the attention left its result quantised (attend_q40)
        kv.q40_add_rms_norm_quantize(self.x, self.scratch, sh.eps, weight=L["ffn_norm"], residual=self.proj, x_out=self.x)
        L["wgu"].gemm_quantized(self.B, self.gate_up, scratch=self.scratch)
        kv.q40_silu_mul_quantize(self.gate_up[:, :sh.ffn], self.gate_up[:, sh.ffn:], self.scratch)
        L["wd"].gemm_quantized(self.B, self.proj, scratch=self.scratch)

    def _head(self):
        kv.gather_rows(self.cos, self.pos, out=self.cos_t)
        kv.gather_rows(self.sin, self.pos, out=self.sin_t)
        kv.gather_rows(self.embed, self.tokens, out=self.x)

    def _tail(self, residual=True):
        kv.q40_add_rms_norm_quantize(self.x, self.scratch, self.shape.eps, weight=self.final_norm, residual=self.proj if residual else None,
                                     x_out=self.x if residual else None)
        self.lm_head.gemm_quantized(self.B, self.logits, scratch=self.scratch)
        kv.argmax(self.logits, out=self.tokens)

    def _segments(self):
        """The launch sequences of one step that touch no cache: [head + pre(0)], [post(i) + pre(i+1)] ..., [post(last) + tail]."""
        n = len(self.layers)
        segs = [lambda: (self._head(), self._pre_attention(self.layers[0], True))]
        for i in range(n - 1):
            segs.append(lambda i=i: (self._post_attention(self.layers[i]), self._pre_attention(self.layers[i + 1], False)))
        segs.append(lambda: (self._post_attention(self.layers[n - 1]), self._tail()))
        return segs

    def _capture(self):
        torch = self.torch
        side = torch.cuda.Stream(device=self.dev)
        self.graphs = []
        with torch.cuda.stream(side):
            for seg in self._segments():  # one eager pass first: lazy initialisation happens outside the capture
                seg()
            side.synchronize()
            for seg in self._segments():
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    seg()
                self.graphs.append(g)
        torch.cuda.synchronize(self.dev)
        self.x.zero_(), self.tokens.zero_()

    # ---- one decode step: `tokens` in, greedy next tokens out (both in self.tokens) --------------------
    def step(self):
        run = (lambda i: self.graphs[i].replay()) if self.graphs else (lambda i, s=self._segments(): s[i]())
        run(0)
        for i, L in enumerate(self.layers):
            ids = self.seqs[i]
            L["cache"].append_rope(ids, self.k16, self.v16, self.cos_t.view(self.B, 1, -1), self.sin_t.view(self.B, 1, -1))
            L["cache"].attend_q40(ids, self.q16, self.scratch, cos=self.cos_t, sin=self.sin_t)
            run(i + 1)
        self.pos += 1
        self.lengths = [n + 1 for n in self.lengths]

    def set_tokens(self, tokens):
        self.tokens.copy_(self.torch.as_tensor(tokens, dtype=self.torch.int32))

    def prefill(self, prompt):
        """Prompt pass: `prompt` is an int32 [B, S] tensor of token ids, all sequences S tokens long, appended after whatever
        the caches hold.  Runs every layer over all B * S rows (the GEMMs share each weight stage between 4 groups of 8
        rows), fills the caches, and leaves the greedy next token of every sequence in self.tokens."""
        torch, sh, B = self.torch, self.shape, self.B
        S = int(prompt.shape[1])
        R = B * S
        dev, f32, kdt = self.dev, torch.float32, self.kv_dtype
        nq, nk = sh.n_q_heads * sh.head_dim, sh.n_kv_heads * sh.head_dim
        pos0 = self.lengths[0]
        assert all(n == pos0 for n in self.lengths) and prompt.shape[0] == B
        ids = prompt.to(dev, torch.int32).reshape(R).contiguous()
        x = kv.gather_rows(self.embed, ids)
        scratch = torch.empty(kv.Q40Linear.scratch_bytes(max(sh.hidden, sh.ffn, nq), R), dtype=torch.uint8, device=dev)
        # 16-bit q | k | v rows, seen by the cache ops as [B, H, S, D] tensors through their strides
        qkv16 = torch.empty((R, nq + 2 * nk), dtype=kdt, device=dev)
        bhsd = lambda lo, n: qkv16[:, lo:lo + n * sh.head_dim].unflatten(1, (n, sh.head_dim)).unflatten(0, (B, S)).permute(0, 2, 1, 3)
        q16, k16, v16 = bhsd(0, sh.n_q_heads), bhsd(nq, sh.n_kv_heads), bhsd(nq + nk, sh.n_kv_heads)
        q16r = torch.empty((B, S, sh.n_q_heads, sh.head_dim), dtype=kdt, device=dev).permute(0, 2, 1, 3)
        attn16 = torch.empty((B, S, sh.n_q_heads, sh.head_dim), dtype=kdt, device=dev)
        proj = torch.empty((R, sh.hidden), dtype=f32, device=dev)
        gate_up = torch.empty((R, 2 * sh.ffn), dtype=f32, device=dev)
        cos, sin = self.cos[pos0:pos0 + S].unsqueeze(0), self.sin[pos0:pos0 + S].unsqueeze(0)  # [1, S, D]: the same for every sequence
        for i, L in enumerate(self.layers):
            kv.q40_add_rms_norm_quantize(x, scratch, sh.eps, weight=L["attn_norm"], residual=proj if i else None, x_out=x if i else None)
            L["wqkv"].gemm_quantized(R, qkv16, scratch=scratch)
            kv.rope(q16, cos, sin, out=q16r)
            L["cache"].append_rope(self.seqs[i], k16, v16, cos, sin)
            L["cache"].attend(self.seqs[i], q16r, causal=True, out=attn16.permute(0, 2, 1, 3))
            L["wo"].gemm(attn16.view(R, nq), proj, scratch=scratch)
            kv.q40_add_rms_norm_quantize(x, scratch, sh.eps, weight=L["ffn_norm"], residual=proj, x_out=x)
            L["wgu"].gemm_quantized(R, gate_up, scratch=scratch)
            kv.q40_silu_mul_quantize(gate_up[:, :sh.ffn], gate_up[:, sh.ffn:], scratch)
            L["wd"].gemm_quantized(R, proj, scratch=scratch)
        kv.add(x, proj, out=x)
        kv.cast(x[S - 1::S], self.x)  # the last row of every sequence
        self._tail(residual=False)
        self.pos += S
        self.lengths = [n + S for n in self.lengths]

    def reset(self):
        """Empties every cache (the sequences stay allocated) and moves the positions back to 0."""
        for i, L in enumerate(self.layers):
            for s in self.seqs[i]:
                L["cache"].truncate(s, 0)
        self.pos.zero_()
        self.lengths = [0] * self.B

    def truncate(self, n_tokens):
        """Rolls every sequence of every layer back to its first n_tokens cached tokens (the reference's `truncate`, used to
        drop rejected draft tokens in speculative decoding: examples/causal_llm/src/lib.rs:383-408).  The next step or
        prompt pass continues from position n_tokens."""
        assert all(n_tokens <= n for n in self.lengths)
        for i, L in enumerate(self.layers):
            for s in self.seqs[i]:
                L["cache"].truncate(s, n_tokens)
        self.pos.fill_(n_tokens)
        self.lengths = [n_tokens] * self.B

    def prefill_synthetic(self, n_tokens, seed=1):
        """Fills every layer's cache with n_tokens of random K / V per sequence and moves the positions there: a stand-in for
        a long prompt where only the decode steps are of interest."""
        torch = self.torch
        gen = torch.Generator(device=self.dev).manual_seed(seed)
        sh = self.shape
        for i, L in enumerate(self.layers):
            done = 0
            while done < n_tokens:
                s = min(512, n_tokens - done)
                k = torch.randn((self.B, sh.n_kv_heads, s, sh.head_dim), generator=gen, device=self.dev).to(self.kv_dtype)
                v = torch.randn((self.B, sh.n_kv_heads, s, sh.head_dim), generator=gen, device=self.dev).to(self.kv_dtype)
                L["cache"].append(self.seqs[i], k, v)
                done += s
        self.pos += n_tokens
        self.lengths = [n + n_tokens for n in self.lengths]

    def check(self):
        for L in self.layers:
            L["cache"].check()
        self.lm_head.check(self.scratch)

    def close(self):
        for L in self.layers:
            L["cache"].close()
