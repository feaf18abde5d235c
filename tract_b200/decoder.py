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

        def norm_weight(name):
            w = weights[name] if weights is not None else (torch.rand(sh.hidden, generator=gen, device=dev) * 0.2 + 0.9)
            return w.to(dev, torch.float32)

        self.layers = []
        for i in range(sh.n_layers):
            self.layers.append(dict(
                attn_norm=norm_weight(f"l{i}.attn_norm"), ffn_norm=norm_weight(f"l{i}.ffn_norm"),
                wqkv=linear(f"l{i}.wqkv", qkv_rows, sh.hidden), wo=linear(f"l{i}.wo", sh.hidden, sh.n_q_heads * sh.head_dim),
                wg=linear(f"l{i}.wg", sh.ffn, sh.hidden), wu=linear(f"l{i}.wu", sh.ffn, sh.hidden), wd=linear(f"l{i}.wd", sh.hidden, sh.ffn),
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
        self.x, self.xn = z(B, sh.hidden), z(B, sh.hidden)
        self.qkv = z(B, qkv_rows)
        self.q16, self.q16r = z(B, sh.n_q_heads, 1, sh.head_dim, dt=self.kv_dtype), z(B, sh.n_q_heads, 1, sh.head_dim, dt=self.kv_dtype)
        self.k16, self.v16 = z(B, sh.n_kv_heads, 1, sh.head_dim, dt=self.kv_dtype), z(B, sh.n_kv_heads, 1, sh.head_dim, dt=self.kv_dtype)
        self.attn16, self.attn = z(B, sh.n_q_heads, 1, sh.head_dim, dt=self.kv_dtype), z(B, sh.n_q_heads * sh.head_dim)
        self.proj, self.gate, self.up, self.act = z(B, sh.hidden), z(B, sh.ffn), z(B, sh.ffn), z(B, sh.ffn)
        self.logits = z(B, sh.vocab)
        self.tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.cos_t, self.sin_t = z(B, sh.head_dim, dt=self.kv_dtype), z(B, sh.head_dim, dt=self.kv_dtype)
        self.lengths = [0] * n_seqs
        self.graphs = None
        if use_graphs:
            self._capture()

    # ---- the launches between two cache calls ----------------------------------------------------------
    def _pre_attention(self, L):
        sh = self.shape
        kv.rms_norm(self.x, sh.eps, weight=L["attn_norm"], out=self.xn)
        L["wqkv"].gemm(self.xn, self.qkv)
        nq, nk = sh.n_q_heads * sh.head_dim, sh.n_kv_heads * sh.head_dim
        kv.cast(self.qkv[:, :nq], self.q16.view(self.B, nq))
        kv.cast(self.qkv[:, nq:nq + nk], self.k16.view(self.B, nk))
        kv.cast(self.qkv[:, nq + nk:], self.v16.view(self.B, nk))
        kv.rope(self.q16, self.cos_t.view(self.B, 1, sh.head_dim), self.sin_t.view(self.B, 1, sh.head_dim), out=self.q16r)

    def _post_attention(self, L):
        sh = self.shape
        kv.cast(self.attn16.view(self.B, -1), self.attn)
        L["wo"].gemm(self.attn, self.proj)
        kv.add(self.x, self.proj, out=self.x)
        kv.rms_norm(self.x, sh.eps, weight=L["ffn_norm"], out=self.xn)
        L["wg"].gemm(self.xn, self.gate)
        L["wu"].gemm(self.xn, self.up)
        kv.silu_mul(self.gate, self.up, out=self.act)
        L["wd"].gemm(self.act, self.proj)
        kv.add(self.x, self.proj, out=self.x)

    def _head(self):
        kv.gather_rows(self.cos, self.pos, out=self.cos_t)
        kv.gather_rows(self.sin, self.pos, out=self.sin_t)
        kv.gather_rows(self.embed, self.tokens, out=self.x)

    def _tail(self):
        kv.rms_norm(self.x, self.shape.eps, weight=self.final_norm, out=self.xn)
        self.lm_head.gemm(self.xn, self.logits)
        kv.argmax(self.logits, out=self.tokens)

    def _segments(self):
        """The launch sequences of one step that touch no cache: [head + pre(0)], [post(i) + pre(i+1)] ..., [post(last) + tail]."""
        n = len(self.layers)
        segs = [lambda: (self._head(), self._pre_attention(self.layers[0]))]
        for i in range(n - 1):
            segs.append(lambda i=i: (self._post_attention(self.layers[i]), self._pre_attention(self.layers[i + 1])))
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
            L["cache"].attend(ids, self.q16r, causal=True, out=self.attn16)
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
        xn = torch.empty_like(x)
        scratch = torch.empty(kv.Q40Linear.scratch_bytes(max(sh.hidden, sh.ffn, nq), R), dtype=torch.uint8, device=dev)
        qkv = torch.empty((R, nq + 2 * nk), dtype=f32, device=dev)
        # 16-bit q / k / v as [B, S, H, D] in memory, seen by the cache ops as [B, H, S, D] through their strides
        q16, q16r = torch.empty((B, S, sh.n_q_heads, sh.head_dim), dtype=kdt, device=dev), torch.empty((B, S, sh.n_q_heads, sh.head_dim), dtype=kdt, device=dev)
        k16, v16 = torch.empty((B, S, sh.n_kv_heads, sh.head_dim), dtype=kdt, device=dev), torch.empty((B, S, sh.n_kv_heads, sh.head_dim), dtype=kdt, device=dev)
        attn16, attn = torch.empty_like(q16), torch.empty((R, nq), dtype=f32, device=dev)
        proj = torch.empty((R, sh.hidden), dtype=f32, device=dev)
        gate, up = torch.empty((R, sh.ffn), dtype=f32, device=dev), torch.empty((R, sh.ffn), dtype=f32, device=dev)
        cos, sin = self.cos[pos0:pos0 + S].unsqueeze(0), self.sin[pos0:pos0 + S].unsqueeze(0)  # [1, S, D]: the same for every sequence
        bhsd = lambda t: t.permute(0, 2, 1, 3)
        for i, L in enumerate(self.layers):
            kv.rms_norm(x, sh.eps, weight=L["attn_norm"], out=xn)
            L["wqkv"].gemm(xn, qkv, scratch=scratch)
            kv.cast(qkv[:, :nq], q16.view(R, nq))
            kv.cast(qkv[:, nq:nq + nk], k16.view(R, nk))
            kv.cast(qkv[:, nq + nk:], v16.view(R, nk))
            kv.rope(bhsd(q16), cos, sin, out=bhsd(q16r))
            L["cache"].append_rope(self.seqs[i], bhsd(k16), bhsd(v16), cos, sin)
            L["cache"].attend(self.seqs[i], bhsd(q16r), causal=True, out=bhsd(attn16))
            kv.cast(attn16.view(R, nq), attn)
            L["wo"].gemm(attn, proj, scratch=scratch)
            kv.add(x, proj, out=x)
            kv.rms_norm(x, sh.eps, weight=L["ffn_norm"], out=xn)
            L["wg"].gemm(xn, gate, scratch=scratch)
            L["wu"].gemm(xn, up, scratch=scratch)
            kv.silu_mul(gate, up, out=gate)
            L["wd"].gemm(gate, proj, scratch=scratch)
            kv.add(x, proj, out=x)
        kv.cast(x[S - 1::S], self.x)  # the last row of every sequence
        self._tail()
        self.pos += S
        self.lengths = [n + S for n in self.lengths]

    def reset(self):
        """Empties every cache (the sequences stay allocated) and moves the positions back to 0."""
        for i, L in enumerate(self.layers):
            for s in self.seqs[i]:
                L["cache"].truncate(s, 0)
        self.pos.zero_()
        self.lengths = [0] * self.B

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
        self.lm_head.check()

    def close(self):
        for L in self.layers:
            L["cache"].close()
