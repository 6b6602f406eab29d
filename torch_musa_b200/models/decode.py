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


def shard_for_tensor_parallel(model: Llama, rank: int, world: int) -> Llama:
    """Keeps this rank's slice of every projection, in place: q/k/v and gate/up by output rows (whole heads), output
    and down projections by input columns.  Norms, embedding and LM head stay replicated.  The model must use
    separate q/k/v and gate/up projections."""
    cfg = model.cfg
    assert not cfg.fused_qkv and not cfg.fused_gate_up, "tensor-parallel decode needs fused_qkv=False, fused_gate_up=False"
    assert cfg.n_heads % world == 0 and cfg.kv_heads % world == 0 and cfg.ffn_dim % world == 0

    def rows(lin, n):
        per = n // world
        lin.weight = torch.nn.Parameter(lin.weight.detach()[rank * per:(rank + 1) * per].clone(), requires_grad=False)
        lin.out_features = per

    def cols(lin, n):
        per = n // world
        lin.weight = torch.nn.Parameter(lin.weight.detach()[:, rank * per:(rank + 1) * per].clone(), requires_grad=False)
        lin.in_features = per

    hd = cfg.head_dim
    for layer in model.layers:
        a, f = layer.attn, layer.ffn
        rows(a.wq, cfg.n_heads * hd)
        rows(a.wk, cfg.kv_heads * hd)
        rows(a.wv, cfg.kv_heads * hd)
        cols(a.wo, cfg.n_heads * hd)
        rows(f.w1, cfg.ffn_dim)
        rows(f.w3, cfg.ffn_dim)
        cols(f.w2, cfg.ffn_dim)
    return model


class LlamaDecoder:
    """``tp_group``: the model was sharded with ``shard_for_tensor_parallel`` over this process group; every rank then
    holds 1/W of the heads and of the KV cache, and the two row-parallel projections of a layer end in an all-reduce
    (recorded into the graph like every other operation of the step)."""

    def __init__(self, model: Llama, batch: int, max_len: int, device=None, dtype: Optional[torch.dtype] = None,
                 tp_group=None):
        cfg = model.cfg
        self.model, self.cfg, self.B, self.max_len = model, cfg, batch, max_len
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        dt = dtype or next(model.parameters()).dtype
        self.tp_group = tp_group
        self.tp = 1
        if tp_group is not None:
            import torch.distributed as dist

            self.tp = dist.get_world_size(tp_group)
        L, kv, hd = cfg.n_layers, cfg.kv_heads // self.tp, cfg.head_dim
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

    def _reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp > 1:
            import torch.distributed as dist

            dist.all_reduce(t, group=self.tp_group)
        return t

    # ------------------------------------------------------------------ prefill (eager, whole prompt at once)
    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor) -> None:
        """Runs the prompt [B, S0] through the model, filling the cache; afterwards ``tokens`` holds the greedy next
        token and ``pos`` equals S0."""
        B, S0 = prompt.shape
        assert B == self.B and S0 < self.max_len
        m, cfg = self.model, self.cfg
        hd, h, kv = cfg.head_dim, cfg.n_heads // self.tp, cfg.kv_heads // self.tp
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
            x = x + self._reduce(a.wo(o.transpose(1, 2).reshape(B, S0, h * hd)))
            x = x + self._reduce(layer.ffn(layer.ffn_norm(x)))
        logits = m.lm_head(m.norm(x[:, -1:]))
        self.tokens.copy_(logits.argmax(-1))
        self.pos.fill_(S0)

    def _add_norm(self, norm, x, delta):
        """(norm(x + delta), x + delta); residual add and RMS norm are one kernel on the device."""
        if delta is None:
            return norm(x), x
        if self._fused_decode and isinstance(norm, torch.nn.RMSNorm) and norm.weight is not None:
            eps = norm.eps if norm.eps is not None else torch.finfo(x.dtype).eps
            y, res, _ = torch.ops.blackwell.rms_norm_residual(delta, x, norm.weight, eps)
            return y, res
        x = x + delta
        return norm(x), x

    # ------------------------------------------------------------------ one decode step on fixed buffers
    @torch.no_grad()
    def _step(self) -> None:
        m, cfg, B = self.model, self.cfg, self.B
        hd, h, kv = cfg.head_dim, cfg.n_heads // self.tp, cfg.kv_heads // self.tp
        positions = self.pos.expand(B, 1)
        # keys at index <= pos are visible (additive mask, broadcast over batch and heads)
        mask = torch.where(self._arange <= self.pos, 0.0, float("-inf")).to(self.k_cache.dtype).view(1, 1, 1, self.max_len)
        x = m.tok_emb(self.tokens)
        delta = None          # the previous block's output, added to the residual stream inside the next norm kernel
        for li, layer in enumerate(m.layers):
            hn, x = self._add_norm(layer.attn_norm, x, delta)
            a = layer.attn
            if cfg.fused_qkv:
                q, k, v = a.wqkv(hn).view(B, 1, h + 2 * kv, hd).split([h, kv, kv], dim=2)
            else:
                q, k, v = a.wq(hn).view(B, 1, h, hd), a.wk(hn).view(B, 1, kv, hd), a.wv(hn).view(B, 1, kv, hd)
            if self._fused_decode:
                # one launch rotates q and k, writes the new key / value rows into the caches at the device-side position;
                # one memory-bound kernel then reads the cache, its visible length from the same counter
                qr = torch.ops.blackwell.decode_rope_cache(q, k, v, self.cos, self.sin, self.pos, self.k_cache[li],
                                                           self.v_cache[li])
                o = torch.ops.blackwell.decode_attention(qr, self.k_cache[li], self.v_cache[li], self.pos)
                o = o.view(B, 1, h * hd)
            else:
                q = BF.rope(q, self.cos, self.sin, positions)
                k = BF.rope(k, self.cos, self.sin, positions)
                self.k_cache[li].index_copy_(2, self.pos, k.transpose(1, 2))
                self.v_cache[li].index_copy_(2, self.pos, v.transpose(1, 2))
                o = F.scaled_dot_product_attention(q.transpose(1, 2), self.k_cache[li], self.v_cache[li], attn_mask=mask,
                                                   enable_gqa=(kv != h)).transpose(1, 2).reshape(B, 1, h * hd)
            hn, x = self._add_norm(layer.ffn_norm, x, self._reduce(a.wo(o)))
            delta = self._reduce(layer.ffn(hn))
        hn, x = self._add_norm(m.norm, x, delta)
        logits = m.lm_head(hn)
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
