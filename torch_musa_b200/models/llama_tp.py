"""Tensor-parallel Llama: column-parallel q/k/v/gate/up, row-parallel o/down, sequence-parallel norms and
residual stream, vocabulary-parallel LM head and loss.  Activations between layers are [T/W, dim] shards of
the flattened [batch * seq] token dimension.  The model is plain PyTorch plus the two primitives of
``torch_musa_b200.parallel.tensor_parallel``; with world size 1 it is an ordinary Llama."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ..ops import functional as BF
from ..parallel import tensor_parallel as TP
from ..parallel.loss import parallel_fused_cross_entropy
from .llama import LlamaConfig


class TPAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig, world: int, group=None):
        super().__init__()
        self.cfg, self.world = cfg, world
        hd, h, kv = cfg.head_dim, cfg.n_heads, cfg.kv_heads
        assert h % world == 0 and kv % world == 0
        self.h_l, self.kv_l = h // world, kv // world
        # local rows: [q heads | k heads | v heads] of this rank
        self.wqkv = TP.ColumnParallelLinear(cfg.dim, (h + 2 * kv) * hd, world, group)
        self.wo = TP.RowParallelLinear(h * hd, cfg.dim, world, group)

    def forward(self, x_shard, B, S, cos, sin):
        hd = self.cfg.head_dim
        qkv = self.wqkv(x_shard).view(B, S, self.h_l + 2 * self.kv_l, hd)
        q, k, v = qkv.split([self.h_l, self.kv_l, self.kv_l], dim=2)
        q, k = BF.rope(q, cos, sin), BF.rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=(self.kv_l != self.h_l))
        return self.wo(o.transpose(1, 2).reshape(B * S, self.h_l * hd))


class TPFeedForward(nn.Module):
    def __init__(self, cfg: LlamaConfig, world: int, group=None):
        super().__init__()
        # local rows: [gate_local ; up_local] so that the packed SwiGLU kernel sees matching halves
        self.w13 = TP.ColumnParallelLinear(cfg.dim, 2 * cfg.ffn_dim, world, group)
        self.w2 = TP.RowParallelLinear(cfg.ffn_dim, cfg.dim, world, group)

    def forward(self, x_shard):
        return self.w2(BF.swiglu(self.w13(x_shard)))


class TPBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, world: int, group=None):
        super().__init__()
        self.attn_norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.attn = TPAttention(cfg, world, group)
        self.ffn_norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.ffn = TPFeedForward(cfg, world, group)

    def forward(self, x, B, S, cos, sin):
        x = x + self.attn(self.attn_norm(x), B, S, cos, sin)
        return x + self.ffn(self.ffn_norm(x))


class TPLlama(nn.Module):
    def __init__(self, cfg: LlamaConfig, world: int = 1, group=None):
        super().__init__()
        assert cfg.vocab_size % world == 0
        self.cfg, self.world, self.group = cfg, world, (TP.SOLO if world == 1 else group)
        self.tok_emb = nn.Embedding(cfg.vocab_size, cfg.dim)                 # replicated
        self.layers = nn.ModuleList(TPBlock(cfg, world, group) for _ in range(cfg.n_layers))
        self.norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.lm_head = TP.ColumnParallelLinear(cfg.dim, cfg.vocab_size, world, group)   # vocabulary-parallel
        cos, sin = BF.precompute_rope_cache(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def replicated_parameters(self):
        """Replicated parameters whose gradients are partial sums over the token shards (the norm weights): they
        must be all-reduced (SUM) before the optimizer step.  The embedding is replicated too but its gradient is
        already complete on every rank (the backward of the row shard all-gathers the gradient blocks)."""
        out = [self.norm.weight]
        for l in self.layers:
            out += [l.attn_norm.weight, l.ffn_norm.weight]
        return out

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None):
        B, S = tokens.shape
        if self.rope_cos.device != tokens.device:
            self.rope_cos, self.rope_sin = self.rope_cos.to(tokens.device), self.rope_sin.to(tokens.device)
        cos, sin = self.rope_cos.float(), self.rope_sin.float()
        assert (B * S) % self.world == 0
        x = TP.shard_rows(self.tok_emb(tokens).view(B * S, -1), self.group)       # [T/W, dim]
        for layer in self.layers:
            x = layer(x, B, S, cos, sin)
        logits = self.lm_head(self.norm(x))                                         # [T, V/W]
        if targets is None:
            return logits
        if self.world == 1:
            return BF.fused_cross_entropy(logits, targets.reshape(-1), inplace_backward=True)
        return parallel_fused_cross_entropy(logits, targets.reshape(-1), self.group)
