"""Llama-style decoder (RMSNorm, RoPE, SwiGLU, causal attention, untied LM head).

The module uses only public torch APIs plus ``torch_musa_b200.ops``; on the blackwell device every
hot operator resolves to a hand-written sm_100a kernel (tcgen05 GEMMs with the bias/activation
epilogue, tcgen05 flash attention forward and backward, fused RMSNorm / RoPE / SwiGLU /
cross-entropy), on any other device to plain PyTorch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import functional as BF


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: Optional[int] = None
    ffn_dim: int = 11008
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq_len: int = 4096
    fused_gate_up: bool = True     # one [2*ffn, dim] GEMM + packed SwiGLU kernel
    fused_qkv: bool = True         # one [(h + 2*kv) * hd, dim] GEMM
    fused_loss: bool = True        # fused cross entropy (no probability tensor)

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def kv_heads(self) -> int:
        return self.n_kv_heads or self.n_heads


def llama_7b_config(**kw) -> LlamaConfig:
    return LlamaConfig(**kw)


def llama_tiny_config(**kw) -> LlamaConfig:
    base = dict(vocab_size=512, dim=256, n_layers=2, n_heads=4, ffn_dim=512, max_seq_len=128)
    base.update(kw)
    return LlamaConfig(**base)


class RopeTables:
    """Plain holder of the fp32 cos/sin tables shared by all layers.  It is deliberately not a tensor
    argument of the layers' ``forward``: FSDP's mixed-precision policy casts floating-point forward
    inputs to the compute dtype, and rotary tables must stay fp32."""

    def __init__(self):
        self.cos = None
        self.sin = None


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig, rope: RopeTables):
        super().__init__()
        self.cfg = cfg
        self._rope = [rope]  # in a list so nn.Module does not try to register it
        hd, h, kv = cfg.head_dim, cfg.n_heads, cfg.kv_heads
        if cfg.fused_qkv:
            self.wqkv = nn.Linear(cfg.dim, (h + 2 * kv) * hd, bias=False)
        else:
            self.wq = nn.Linear(cfg.dim, h * hd, bias=False)
            self.wk = nn.Linear(cfg.dim, kv * hd, bias=False)
            self.wv = nn.Linear(cfg.dim, kv * hd, bias=False)
        self.wo = nn.Linear(h * hd, cfg.dim, bias=False)

    def forward(self, x, positions=None):
        B, S, _ = x.shape
        cfg = self.cfg
        cos, sin = self._rope[0].cos, self._rope[0].sin
        hd, h, kv = cfg.head_dim, cfg.n_heads, cfg.kv_heads
        if cfg.fused_qkv:
            # split (not slicing): its backward is one concatenation instead of three zero-fill + add passes
            q, k, v = self.wqkv(x).view(B, S, h + 2 * kv, hd).split([h, kv, kv], dim=2)
        else:
            # -1: under tensor parallelism each rank holds a slice of the heads
            q = self.wq(x).view(B, S, -1, hd)
            k = self.wk(x).view(B, S, -1, hd)
            v = self.wv(x).view(B, S, -1, hd)
        q = BF.rope(q, cos, sin, positions)
        k = BF.rope(k, cos, sin, positions)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=(kv != h))
        return self.wo(o.transpose(1, 2).reshape(B, S, -1))


class FeedForward(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.fused = cfg.fused_gate_up
        if self.fused:
            self.w13 = nn.Linear(cfg.dim, 2 * cfg.ffn_dim, bias=False)
        else:
            self.w1 = nn.Linear(cfg.dim, cfg.ffn_dim, bias=False)
            self.w3 = nn.Linear(cfg.dim, cfg.ffn_dim, bias=False)
        self.w2 = nn.Linear(cfg.ffn_dim, cfg.dim, bias=False)

    def forward(self, x):
        if self.fused:
            return self.w2(BF.swiglu(self.w13(x)))
        return self.w2(BF.silu_mul(self.w1(x), self.w3(x)))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig, rope: RopeTables):
        super().__init__()
        self.attn_norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.attn = Attention(cfg, rope)
        self.ffn_norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.ffn = FeedForward(cfg)

    def forward(self, x, positions=None):
        x = x + self.attn(self.attn_norm(x), positions)
        return x + self.ffn(self.ffn_norm(x))


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.tok_emb = nn.Embedding(cfg.vocab_size, cfg.dim)
        self._rope = RopeTables()
        self.layers = nn.ModuleList(Block(cfg, self._rope) for _ in range(cfg.n_layers))
        self.norm = nn.RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)
        if torch.empty(0).device.type == "meta":
            # deferred initialisation: the tables are filled in after materialisation (see init_rope_cache)
            cos = torch.empty(cfg.max_seq_len, cfg.head_dim // 2, dtype=torch.float32)
            sin = torch.empty_like(cos)
        else:
            cos, sin = BF.precompute_rope_cache(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def init_rope_cache(self, device=None):
        """(Re)compute the fp32 cos/sin tables, e.g. after ``to_empty`` of a meta-initialised model."""
        cfg = self.cfg
        cos, sin = BF.precompute_rope_cache(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta)
        device = device if device is not None else self.rope_cos.device
        self.rope_cos = cos.to(device)
        self.rope_sin = sin.to(device)

    def reset_parameters(self, std: float = 0.02, seed: Optional[int] = None):
        g = None
        if seed is not None:
            g = torch.Generator(device="cpu").manual_seed(seed)
        for p in self.parameters():
            if p.dim() >= 2:
                if g is not None and p.device.type == "cpu":
                    nn.init.normal_(p, mean=0.0, std=std, generator=g)
                else:
                    nn.init.normal_(p, mean=0.0, std=std)
            else:
                nn.init.ones_(p)

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None, positions=None):
        B, S = tokens.shape
        if self.rope_cos.device != tokens.device and self.rope_cos.device.type != "meta":
            self.rope_cos, self.rope_sin = self.rope_cos.to(tokens.device), self.rope_sin.to(tokens.device)
        cos, sin = self.rope_cos, self.rope_sin
        if cos.dtype != torch.float32:  # a module-wide .to(bf16) must not degrade the tables
            cos, sin = cos.float(), sin.float()
        self._rope.cos, self._rope.sin = cos, sin
        x = self.tok_emb(tokens)
        for layer in self.layers:
            x = layer(x, positions)
        x = self.norm(x)
        logits = self.lm_head(x)
        if targets is None:
            return logits
        if getattr(self, "loss_fn", None) is not None:  # e.g. the vocabulary-parallel loss of a tensor-parallel plan
            return self.loss_fn(logits.view(B * S, -1), targets.reshape(-1))
        if self.cfg.fused_loss:
            return BF.fused_cross_entropy(logits.view(B * S, -1), targets.reshape(-1), inplace_backward=True)
        return F.cross_entropy(logits.view(B * S, -1).float(), targets.reshape(-1))

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (fwd + bwd = 3x fwd), attention counted causally."""
        c = self.cfg
        n = self.num_params() - c.vocab_size * c.dim  # embedding lookup is not a matmul
        attn = 2 * 2 * c.n_layers * c.dim * seq_len / 2  # QK^T and PV, causal half
        return 3.0 * (2 * n + attn)
