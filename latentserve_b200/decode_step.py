"""One decode step of a Qwen2-architecture model over the paged caches of this
package, eager or replayed from a CUDA graph.

This is the caller's side of the hot path, kept as small as it can be: the
reference builds it from Hugging Face modules (`LatentServeQwen._run_layers`,
model/latentserve_qwen.py:397-451; `GQAAttention.forward`,
model/attention/gqa.py:227-344; `GraphedDecoder`, runtime/cuda_graph.py:213-398)
and none of that is rebuilt here. It exists so that the decode-step time the
reference quotes (whole step, graph replay) can be measured with this library's
append and attention kernels inside a step of the same shape: dense
projections and the MLP are plain cuBLAS GEMMs through torch, weights are
random (N(0, 0.02), fp16).

Per layer, in stream order, with `projections="cublas"` (nine launches):
[residual add +] RMSNorm -> fused QKV GEMM (+ bias) -> RoPE(q, k) + KV append
(one launch) -> paged decode attention (one launch; dense, INT8 or
page-sparse) -> o_proj GEMM -> residual add + RMSNorm -> gate/up GEMM ->
SiLU * up -> down GEMM, the GEMMs being torch's. With `projections="ls"` the
projections are this library's weight-streaming kernel (`projections.linear`)
with the norms, residual adds and SiLU * up folded into them, and for the fp16
cache RoPE and the KV append folded into the QKV projection (five launches; six
with an INT8 cache): about 10 % faster per step than the cuBLAS route at batch
16, slower between 17 and 32 rows, not available beyond. `projections="auto"` (the default) takes the
streaming kernel up to 16 rows and cuBLAS above. With
`fused=False` the norms, RoPE and SwiGLU are plain torch element-wise ops and
the append is `cache.write` (the form the fused ones are tested against).
`cache.advance(1)` runs on the host before the step and is not part of a
captured graph, as in the reference (runtime/cuda_graph.py:337).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from latentserve_b200 import fused_elementwise as fe
from latentserve_b200 import paged_decode as pd
from latentserve_b200 import paged_sparse as ps
from latentserve_b200 import projections as pj


@dataclass
class QwenShape:
    """Defaults are Qwen2.5-1.5B (model/qwen.py:45 `ModelShape` in the reference)."""
    num_layers: int = 28
    hidden: int = 1536
    q_heads: int = 12
    kv_heads: int = 2
    head_dim: int = 128
    intermediate: int = 8960
    vocab: int = 151936
    rms_eps: float = 1e-6
    rope_theta: float = 1e6


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def rope_tables(shape: QwenShape, max_pos: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [max_pos, head_dim], halves duplicated (rotate-half convention)."""
    half = shape.head_dim // 2
    inv = shape.rope_theta ** (-torch.arange(half, dtype=torch.float32, device=device) / half)
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, heads, head_dim]; cos / sin [B, head_dim] (fp32)."""
    half = x.shape[-1] // 2
    xf = x.float()
    rot = torch.cat([-xf[..., half:], xf[..., :half]], dim=-1)
    return (xf * cos[:, None, :] + rot * sin[:, None, :]).to(x.dtype)


class DecodeModel:
    """Random-init weights of the given shape and the decode step over a cache."""

    def __init__(self, shape: QwenShape, device, max_pos: int, seed: int = 0,
                 dtype: torch.dtype = torch.float16, fused: bool = True, projections: str = "auto"):
        self.shape, self.device, self.dtype = shape, torch.device(device), dtype
        self.fused = fused
        if projections not in ("auto", "ls", "cublas"):
            raise ValueError(f"unknown projections {projections!r}")
        self.projections = projections
        g = torch.Generator(device=self.device).manual_seed(seed)
        s = shape

        def w(*dims):
            return (torch.randn(*dims, device=self.device, generator=g, dtype=torch.float32) * 0.02).to(dtype)

        qkv_out = (s.q_heads + 2 * s.kv_heads) * s.head_dim
        self.embed = w(s.vocab, s.hidden)                      # tied with the output head
        self.layers = []
        for _ in range(s.num_layers):
            self.layers.append(dict(
                ln1=torch.ones(s.hidden, device=self.device, dtype=dtype),
                wqkv=w(qkv_out, s.hidden), bqkv=w(qkv_out),
                wo=w(s.hidden, s.q_heads * s.head_dim),
                ln2=torch.ones(s.hidden, device=self.device, dtype=dtype),
                wgu=w(2 * s.intermediate, s.hidden), wd=w(s.hidden, s.intermediate)))
        self.ln_f = torch.ones(s.hidden, device=self.device, dtype=dtype)
        self.cos, self.sin = rope_tables(s, max_pos, self.device)
        self.cos16, self.sin16 = self.cos.to(dtype), self.sin.to(dtype)   # model-dtype tables, as HF's
        self.sparse_ratio: Optional[float] = None

    def weight_bytes(self) -> int:
        """Bytes of weights one decode step reads (embedding rows excluded, output head included)."""
        per_layer = sum(v.numel() * v.element_size() for v in self.layers[0].values())
        return per_layer * len(self.layers) + self.embed.numel() * self.embed.element_size()

    def set_sparse(self, ratio: Optional[float]) -> None:
        """Page-sparse attention at `ratio` (fp16 cache with page bounds), or dense for None."""
        self.sparse_ratio = ratio

    def attend(self, cache, layer: int, q: torch.Tensor, batch: int, context_hint: int) -> torch.Tensor:
        tables, lens = cache.block_tables_tensor(batch), cache.seq_lens_tensor(batch)
        extra = {}
        if hasattr(cache, "k_scale_pool"):
            extra = dict(k_scale=cache.k_scale_pool[layer], v_scale=cache.v_scale_pool[layer],
                         k_residual=cache.residual(layer), res_rows=cache.residual_rows_tensor(batch))
        bounds = cache.page_bounds(layer) if (self.sparse_ratio is not None
                                              and hasattr(cache, "page_bounds")) else None
        if bounds is not None:
            return ps.sparse_attention(q, cache.k_pool[layer], cache.v_pool[layer], tables, lens,
                                       bounds[0], bounds[1], ratio=self.sparse_ratio,
                                       max_seq_len=context_hint, **extra)
        if extra and cache.asymmetric:
            extra.update(k_zero=cache.k_zero_pool[layer], v_zero=cache.v_zero_pool[layer])
        return pd.paged_decode_attention(q, cache.k_pool[layer], cache.v_pool[layer], tables, lens,
                                         max_seq_len=context_hint, **extra)

    def streams_projections(self, rows: int) -> bool:
        """Whether a step of `rows` sequences uses `projections.linear` (else torch GEMMs)."""
        if self.projections == "ls":
            return rows <= pj.MAX_ROWS
        return self.projections == "auto" and rows <= 16

    def forward(self, cache, tokens: torch.Tensor, positions: torch.Tensor,
                context_hint: int, return_logits: bool = False) -> torch.Tensor:
        """tokens, positions [B] (device) -> next token ids [B] (greedy), or the
        logits [B, vocab]. The cache must have been advanced by one token for
        these B sequences."""
        if self.fused and self.streams_projections(tokens.shape[0]):
            return self._forward_streamed(cache, tokens, positions, context_hint, return_logits)
        if self.fused:
            return self._forward_fused(cache, tokens, positions, context_hint, return_logits)
        s = self.shape
        b = tokens.shape[0]
        x = self.embed[tokens]                                              # [B, hidden]
        cos, sin = self.cos16[positions].float(), self.sin16[positions].float()
        for i, L in enumerate(self.layers):
            h = rms_norm(x, L["ln1"], s.rms_eps)
            qkv = torch.addmm(L["bqkv"], h, L["wqkv"].t())                  # [B, (12+2+2)*128]
            q = qkv[:, : s.q_heads * s.head_dim].view(b, s.q_heads, s.head_dim)
            k = qkv[:, s.q_heads * s.head_dim:(s.q_heads + s.kv_heads) * s.head_dim].view(
                b, s.kv_heads, s.head_dim)
            v = qkv[:, (s.q_heads + s.kv_heads) * s.head_dim:].view(b, s.kv_heads, 1, s.head_dim)
            q = apply_rope(q, cos, sin).view(b, s.kv_heads, s.q_heads // s.kv_heads, s.head_dim)
            k = apply_rope(k, cos, sin).view(b, s.kv_heads, 1, s.head_dim)
            cache.write(i, k, v)
            a = self.attend(cache, i, q, b, context_hint)                   # [B, H, R, D]
            x = x + a.reshape(b, s.q_heads * s.head_dim) @ L["wo"].t()
            h = rms_norm(x, L["ln2"], s.rms_eps)
            gu = h @ L["wgu"].t()
            x = x + (torch.nn.functional.silu(gu[:, : s.intermediate]) * gu[:, s.intermediate:]) @ L["wd"].t()
        logits = rms_norm(x, self.ln_f, s.rms_eps) @ self.embed.t()
        return logits if return_logits else logits.argmax(dim=-1)


    def _forward_fused(self, cache, tokens, positions, context_hint, return_logits):
        s = self.shape
        b = tokens.shape[0]
        x = self.embed[tokens]
        residual = None
        for i, L in enumerate(self.layers):
            if residual is None:
                h, residual = fe.rms_norm(x, L["ln1"], s.rms_eps), x
            else:
                h, residual = fe.fused_add_rms_norm(x, residual, L["ln1"], s.rms_eps)
            qkv = torch.addmm(L["bqkv"], h, L["wqkv"].t())
            q = torch.empty(b, s.q_heads * s.head_dim, dtype=self.dtype, device=self.device)
            cache.rope_write(i, qkv, self.cos16, self.sin16, positions, q, s.q_heads)
            a = self.attend(cache, i, q.view(b, s.kv_heads, s.q_heads // s.kv_heads, s.head_dim), b,
                            context_hint)
            x = a.reshape(b, s.q_heads * s.head_dim) @ L["wo"].t()
            h, residual = fe.fused_add_rms_norm(x, residual, L["ln2"], s.rms_eps)
            x = fe.silu_and_mul(h @ L["wgu"].t()) @ L["wd"].t()
        h, _ = fe.fused_add_rms_norm(x, residual, self.ln_f, s.rms_eps)
        logits = h @ self.embed.t()
        return logits if return_logits else logits.argmax(dim=-1)


    def _forward_streamed(self, cache, tokens, positions, context_hint, return_logits):
        """Five launches per layer (six with an INT8 cache): the norms, residual adds, SiLU * up and --
        for the fp16 cache -- RoPE with the KV append ride on the projections."""
        # Rounding differs from `_forward_fused` in one place: the residual stream is
        # fp16(fp16(o) + r) in both, but here it is formed in o_proj's epilogue.
        s = self.shape
        b = tokens.shape[0]
        stream = self.embed[tokens]                 # the residual stream, fp16 [B, hidden]
        ss = None                                   # its row sums of squares, once a projection wrote it
        for i, L in enumerate(self.layers):
            q = torch.empty(b, s.q_heads * s.head_dim, dtype=self.dtype, device=self.device)
            if hasattr(cache, "qkv_rope_write"):    # fp16 cache: RoPE and the append ride on the projection
                cache.qkv_rope_write(i, stream, L["wqkv"], L["bqkv"], self.cos16, self.sin16, positions, q,
                                     s.q_heads, norm_weight=L["ln1"], row_sumsq=ss, eps=s.rms_eps)
            else:
                qkv = pj.linear(stream, L["wqkv"], L["bqkv"], norm_weight=L["ln1"], row_sumsq=ss,
                                eps=s.rms_eps)
                cache.rope_write(i, qkv, self.cos16, self.sin16, positions, q, s.q_heads)
            a = self.attend(cache, i, q.view(b, s.kv_heads, s.q_heads // s.kv_heads, s.head_dim), b,
                            context_hint)
            stream, ss = pj.linear(a.reshape(b, s.q_heads * s.head_dim), L["wo"], add_residual=stream,
                                   want_sumsq=True)
            act = pj.linear(stream, L["wgu"], norm_weight=L["ln2"], row_sumsq=ss, eps=s.rms_eps,
                            swiglu=True)
            stream, ss = pj.linear(act, L["wd"], add_residual=stream, want_sumsq=True)
        if s.vocab % 32 == 0:
            logits = pj.linear(stream, self.embed, norm_weight=self.ln_f, row_sumsq=ss, eps=s.rms_eps)
        else:
            logits = fe.rms_norm(stream, self.ln_f, s.rms_eps) @ self.embed.t()
        return logits if return_logits else logits.argmax(dim=-1)


class GraphedStep:
    """The step captured once per batch size and replayed: static token /
    position inputs, `cache.advance(1)` outside the graph, attention kernels
    reading lengths and block tables from the cache's persistent buffers."""

    def __init__(self, model: DecodeModel, cache, batch: int, context_hint: int):
        self.model, self.cache, self.batch, self.hint = model, cache, batch, context_hint
        dev = model.device
        self.tokens = torch.zeros(batch, dtype=torch.long, device=dev)
        self.positions = torch.zeros(batch, dtype=torch.long, device=dev)
        self.next_tokens = torch.zeros(batch, dtype=torch.long, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        # INT8 cache: completed K pages are quantised by the step's first launch, not by
        # advance() between replays.
        if hasattr(cache, "enable_finalize_in_step"):
            cache.enable_finalize_in_step()

    def _run(self):
        # Positions are the cache's lengths minus one: taken on the device, inside the
        # graph, from the buffer advance() ships, so a step needs no copy of its own.
        torch.sub(self.cache.seq_lens_tensor(self.batch), 1, out=self.positions)
        self.next_tokens.copy_(self.model.forward(self.cache, self.tokens, self.positions, self.hint))

    def capture(self) -> None:
        """Needs the cache advanced for the step being captured (it really runs)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._run()

    def step(self, feed_back: bool = True) -> torch.Tensor:
        """advance(1) must have been called; positions are taken from the cache."""
        if self.graph is None:
            self._run()
        else:
            self.graph.replay()
        if feed_back:
            self.tokens.copy_(self.next_tokens)
        return self.next_tokens
