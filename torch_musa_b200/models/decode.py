"""Batched autoregressive decoding for the Llama model with a static KV cache, one decode step captured in a device
graph.

Everything a step needs lives in fixed buffers (token ids, the position counter, the KV cache, the attention
mask), every index is a device tensor, and nothing synchronises with the host, so the whole step -- 32 layers of
norm / GEMM / RoPE / cache update / attention / SwiGLU plus the LM head and the greedy argmax -- is recorded
once and replayed per token with a single launch.  Parity: the reference's graph runtime and its
``musagraphs`` compile backend exist for exactly this loop (reference torch_musa/musa_graph/graphs.py:44-132,
torch_musa/_dynamo/backend/musagraphs.py:171-322).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import functional as BF
from .llama import Llama


class LlamaDecoder:
    def __init__(self, model: Llama, batch: int, max_len: int, device=None, dtype: Optional[torch.dtype] = None):
        cfg = model.cfg
        self.model, self.cfg, self.B, self.max_len = model, cfg, batch, max_len
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        dt = dtype or next(model.parameters()).dtype
        L, kv, hd = cfg.n_layers, cfg.kv_heads, cfg.head_dim
        self.k_cache = torch.zeros(L, batch, kv, max_len, hd, device=self.device, dtype=dt)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.tokens = torch.zeros(batch, 1, dtype=torch.long, device=self.device)      # input of the next step
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)                # position being written
        self.next_tokens = torch.zeros(batch, 1, dtype=torch.long, device=self.device)
        self._arange = torch.arange(max_len, device=self.device)
        cos, sin = BF.precompute_rope_cache(max_len, hd, cfg.rope_theta)
        self.cos, self.sin = cos.to(self.device), sin.to(self.device)
        self._graph = None
        self._fused_decode = (self.device.type == "blackwell" and hd == 128 and dt in (torch.bfloat16, torch.float16))

    # ------------------------------------------------------------------ prefill (eager, whole prompt at once)
    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor) -> None:
        """Runs the prompt [B, S0] through the model, filling the cache; afterwards ``tokens`` holds the greedy next
        token and ``pos`` equals S0."""
        B, S0 = prompt.shape
        assert B == self.B and S0 < self.max_len
        m, cfg = self.model, self.cfg
        hd, h, kv = cfg.head_dim, cfg.n_heads, cfg.kv_heads
        x = m.tok_emb(prompt)
        for li, layer in enumerate(m.layers):
            hn = layer.attn_norm(x)
            a = layer.attn
            if cfg.fused_qkv:
                q, k, v = a.wqkv(hn).view(B, S0, h + 2 * kv, hd).split([h, kv, kv], dim=2)
            else:
                q, k, v = a.wq(hn).view(B, S0, h, hd), a.wk(hn).view(B, S0, kv, hd), a.wv(hn).view(B, S0, kv, hd)
            q, k = BF.rope(q, self.cos, self.sin), BF.rope(k, self.cos, self.sin)
            self.k_cache[li, :, :, :S0] = k.transpose(1, 2)
            self.v_cache[li, :, :, :S0] = v.transpose(1, 2)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=(kv != h))
            x = x + a.wo(o.transpose(1, 2).reshape(B, S0, h * hd))
            x = x + layer.ffn(layer.ffn_norm(x))
        logits = m.lm_head(m.norm(x[:, -1:]))
        self.tokens.copy_(logits.argmax(-1))
        self.pos.fill_(S0)

    # ------------------------------------------------------------------ one decode step on fixed buffers
    @torch.no_grad()
    def _step(self) -> None:
        m, cfg, B = self.model, self.cfg, self.B
        hd, h, kv = cfg.head_dim, cfg.n_heads, cfg.kv_heads
        positions = self.pos.expand(B, 1)
        # keys at index <= pos are visible (additive mask, broadcast over batch and heads)
        mask = torch.where(self._arange <= self.pos, 0.0, float("-inf")).to(self.k_cache.dtype).view(1, 1, 1, self.max_len)
        x = m.tok_emb(self.tokens)
        for li, layer in enumerate(m.layers):
            hn = layer.attn_norm(x)
            a = layer.attn
            if cfg.fused_qkv:
                q, k, v = a.wqkv(hn).view(B, 1, h + 2 * kv, hd).split([h, kv, kv], dim=2)
            else:
                q, k, v = a.wq(hn).view(B, 1, h, hd), a.wk(hn).view(B, 1, kv, hd), a.wv(hn).view(B, 1, kv, hd)
            q = BF.rope(q, self.cos, self.sin, positions)
            k = BF.rope(k, self.cos, self.sin, positions)
            self.k_cache[li].index_copy_(2, self.pos, k.transpose(1, 2))
            self.v_cache[li].index_copy_(2, self.pos, v.transpose(1, 2))
            if self._fused_decode:
                # one memory-bound kernel over the cache; the visible length comes from the device counter
                o = torch.ops.blackwell.decode_attention(q.reshape(B, h, hd), self.k_cache[li], self.v_cache[li], self.pos)
                o = o.view(B, 1, h * hd)
            else:
                o = F.scaled_dot_product_attention(q.transpose(1, 2), self.k_cache[li], self.v_cache[li], attn_mask=mask,
                                                   enable_gqa=(kv != h)).transpose(1, 2).reshape(B, 1, h * hd)
            x = x + a.wo(o)
            x = x + layer.ffn(layer.ffn_norm(x))
        logits = m.lm_head(m.norm(x))
        self.next_tokens.copy_(logits.argmax(-1))
        self.tokens.copy_(self.next_tokens)
        self.pos.add_(1)

    def capture(self, warmup: int = 2) -> None:
        """Records one decode step into a device graph (after a few eager warm-up steps on a side stream; the
        warm-up steps advance the cache like real steps do)."""
        import torch_musa_b200 as bw

        saved = (self.tokens.clone(), self.pos.clone())
        side = bw.Stream()
        side.wait_stream(bw.current_stream())
        with bw.stream(side):
            for _ in range(warmup):
                self._step()
        bw.current_stream().wait_stream(side)
        self.tokens.copy_(saved[0])
        self.pos.copy_(saved[1])
        g = bw.BlackwellGraph() if hasattr(bw, "BlackwellGraph") else bw.graphs.BlackwellGraph()
        with bw.graph(g):
            self._step()
        # the capture itself does not execute: state is unchanged
        self._graph = g

    @torch.no_grad()
    def decode(self, n_tokens: int) -> torch.Tensor:
        """Generates ``n_tokens`` greedy tokens per sequence; returns [B, n_tokens]."""
        out = torch.empty(self.B, n_tokens, dtype=torch.long, device=self.device)
        for i in range(n_tokens):
            out[:, i:i + 1].copy_(self.tokens)
            if self._graph is not None:
                self._graph.replay()
            else:
                self._step()
        return out
