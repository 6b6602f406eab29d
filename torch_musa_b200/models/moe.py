"""Mixtral-style mixture-of-experts decoder with expert parallelism.

Every block is Llama attention followed by a routed FFN: a top-k softmax router picks k of E SwiGLU experts
per token; experts are split evenly over the ranks of the expert-parallel group (rank r owns experts
[r*E/W, (r+1)*E/W)) and tokens travel to their experts and back through
``torch_musa_b200.parallel.moe`` (fused peer-memory kernels on the blackwell device, the sort +
all_to_all reference elsewhere).  Attention, router, norms and embeddings are replicated.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import functional as BF
from .llama import Attention, LlamaConfig, RopeTables


@dataclass
class MoEConfig:
    vocab_size: int = 32000
    dim: int = 4096
    n_layers: int = 8
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    n_experts: int = 8
    top_k: int = 2
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq_len: int = 4096
    capacity_factor: float = 2.0
    # benchmark mode: router logits are drawn N(0,1) per token instead of computed, so that expert loads are
    # balanced in expectation whatever the weights are (the router projection stays in the graph with zero weight)
    synthetic_router_logits: bool = False

    def attention_config(self) -> LlamaConfig:
        return LlamaConfig(vocab_size=self.vocab_size, dim=self.dim, n_layers=self.n_layers, n_heads=self.n_heads,
                           n_kv_heads=self.n_kv_heads, ffn_dim=self.ffn_dim, norm_eps=self.norm_eps,
                           rope_theta=self.rope_theta, max_seq_len=self.max_seq_len)


def moe_tiny_config(**kw) -> MoEConfig:
    base = dict(vocab_size=512, dim=128, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=256, n_experts=4, top_k=2,
                max_seq_len=64)
    base.update(kw)
    return MoEConfig(**base)


class Experts(nn.Module):
    """This rank's experts: packed gate/up weights [E_local, 2*ffn, dim] and down weights [E_local, dim, ffn]."""

    def __init__(self, n_local: int, dim: int, ffn: int):
        super().__init__()
        self.w13 = nn.Parameter(torch.empty(n_local, 2 * ffn, dim))
        self.w2 = nn.Parameter(torch.empty(n_local, dim, ffn))
        for w in (self.w13, self.w2):
            nn.init.normal_(w, std=0.02)

    def forward(self, rows: torch.Tensor, rows_per_expert, y_out=None, dx_out=None) -> torch.Tensor:
        if isinstance(rows_per_expert, torch.Tensor):
            # counts on the device: one grouped GEMM per projection over the packed rows, nothing read on the host
            h = BF.grouped_linear(rows, self.w13, rows_per_expert, None, dx_out)
            return BF.grouped_linear(BF.swiglu(h, rows_per_expert), self.w2, rows_per_expert, y_out)
        outs, start = [], 0
        for e, n in enumerate(rows_per_expert):
            n = min(n, rows.shape[0] - start)
            if n <= 0:
                continue
            x = rows[start:start + n]
            outs.append(F.linear(BF.swiglu(F.linear(x, self.w13[e])), self.w2[e]))
            start += n
        if not outs:
            return rows.new_zeros((0, rows.shape[1]))
        return outs[0] if len(outs) == 1 else torch.cat(outs, 0)


class MoEFeedForward(nn.Module):
    def __init__(self, cfg: MoEConfig, n_local: int, layer_index: int):
        super().__init__()
        self.cfg, self.slot = cfg, layer_index
        self.router = nn.Linear(cfg.dim, cfg.n_experts, bias=False)
        self.experts = Experts(n_local, cfg.dim, cfg.ffn_dim)
        self._exchange = [None]   # set by MoETransformer.set_exchange (kept out of the module tree)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, D = x.shape
        flat = x.reshape(B * S, D)
        logits = self.router(flat).float()
        if self.cfg.synthetic_router_logits:
            logits = logits * 0.0 + torch.randn(logits.shape, device=logits.device, dtype=torch.float32)
        top, idx = torch.topk(logits, self.cfg.top_k, dim=-1)
        gates = torch.softmax(top, dim=-1)                 # softmax over the selected logits (Mixtral)
        ex = self._exchange[0]
        recv, rows_per_expert, ctx = ex.dispatch(flat, idx, self.slot)
        y = self.experts(recv, rows_per_expert, *ex.expert_buffers(self.slot))
        out = ex.combine(y, gates, ctx, self.slot)
        return out.view(B, S, D)


class MoEBlock(nn.Module):
    def __init__(self, cfg: MoEConfig, rope: RopeTables, n_local: int, layer_index: int):
        super().__init__()
        self.attn_norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.attn = Attention(cfg.attention_config(), rope)
        self.ffn_norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.moe = MoEFeedForward(cfg, n_local, layer_index)

    def forward(self, x):
        x = x + self.attn(self.attn_norm(x))
        return x + self.moe(self.ffn_norm(x))


class MoETransformer(nn.Module):
    def __init__(self, cfg: MoEConfig, ep_world: int = 1):
        super().__init__()
        assert cfg.n_experts % ep_world == 0
        self.cfg, self.ep_world = cfg, ep_world
        n_local = cfg.n_experts // ep_world
        self.tok_emb = nn.Embedding(cfg.vocab_size, cfg.dim)
        self._rope = RopeTables()
        self.layers = nn.ModuleList(MoEBlock(cfg, self._rope, n_local, i) for i in range(cfg.n_layers))
        self.norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)
        cos, sin = BF.precompute_rope_cache(cfg.max_seq_len, cfg.dim // cfg.n_heads, cfg.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def set_exchange(self, exchange) -> None:
        for layer in self.layers:
            layer.moe._exchange[0] = exchange

    def expert_parameters(self):
        return [p for layer in self.layers for p in layer.moe.experts.parameters()]

    def replicated_parameters(self):
        skip = {id(p) for p in self.expert_parameters()}
        return [p for p in self.parameters() if id(p) not in skip]

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None):
        B, S = tokens.shape
        if self.rope_cos.device != tokens.device:   # buffers created on the host follow the tokens
            self.rope_cos, self.rope_sin = self.rope_cos.to(tokens.device), self.rope_sin.to(tokens.device)
        self._rope.cos, self._rope.sin = self.rope_cos.float(), self.rope_sin.float()
        x = self.tok_emb(tokens)
        for layer in self.layers:
            x = layer(x)
        logits = self.lm_head(self.norm(x))
        if targets is None:
            return logits
        return BF.fused_cross_entropy(logits.view(B * S, -1), targets.reshape(-1), inplace_backward=True)
