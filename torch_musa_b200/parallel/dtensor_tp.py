"""Tensor parallelism of the Llama model expressed with DTensor styles.

The plan is the standard one: embedding row-wise with sequence-sharded output, norms
``SequenceParallel`` (activations ``Shard(1)`` between blocks), q/k/v and gate/up projections
``ColwiseParallel``, output and down projections ``RowwiseParallel`` back to ``Shard(1)``, the LM
head column-wise with vocabulary-sharded logits that feed the vocabulary-parallel fused cross
entropy (``parallel.loss``).  Collectives issued by the styles run on whatever backend the mesh's
process group uses (``bccl`` on the device, gloo in the CPU tests).

This is the DTensor counterpart of ``parallel.tensor_parallel`` (hand-written column/row layers over
the fused all-gather->GEMM / GEMM->reduce-scatter kernels): same math, stock parallel styles.
Parity: the reference's TP configuration relies on stock Colwise/RowwiseParallel plus its own
sharding rules (reference torch_musa/distributed/tensor/_ops.py:27-189).
"""
from __future__ import annotations

import torch
from torch import nn


def parallelize_llama(model: nn.Module, tp_mesh, loss_parallel: bool = True) -> nn.Module:
    """Applies the plan in place.  The model must use separate q/k/v and gate/up projections
    (``fused_qkv=False``, ``fused_gate_up=False``): a column shard of a fused projection would mix them."""
    from torch.distributed.tensor import Replicate, Shard
    from torch.distributed.tensor.parallel import (ColwiseParallel, PrepareModuleInput, RowwiseParallel,
                                                   SequenceParallel, parallelize_module)

    from ..distributed import tensor_ops

    tensor_ops.register()
    cfg = model.cfg
    if cfg.fused_qkv or cfg.fused_gate_up:
        raise ValueError("the DTensor plan needs fused_qkv=False and fused_gate_up=False")
    tp = tp_mesh.size()
    if cfg.n_heads % tp or cfg.kv_heads % tp or cfg.vocab_size % tp:
        raise ValueError(f"heads ({cfg.n_heads}/{cfg.kv_heads}) and vocabulary ({cfg.vocab_size}) must divide by TP={tp}")
    parallelize_module(model, tp_mesh, {
        "tok_emb": RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1)),
        "norm": SequenceParallel(),
        "lm_head": ColwiseParallel(input_layouts=Shard(1),
                                   output_layouts=Shard(-1) if loss_parallel else Replicate(),
                                   use_local_output=True),
    })
    for block in model.layers:
        parallelize_module(block, tp_mesh, {
            "attn_norm": SequenceParallel(),
            "attn": PrepareModuleInput(input_layouts=(Shard(1), None), desired_input_layouts=(Replicate(), None)),
            "attn.wq": ColwiseParallel(),
            "attn.wk": ColwiseParallel(),
            "attn.wv": ColwiseParallel(),
            "attn.wo": RowwiseParallel(output_layouts=Shard(1)),
            "ffn_norm": SequenceParallel(),
            "ffn": PrepareModuleInput(input_layouts=(Shard(1),), desired_input_layouts=(Replicate(),)),
            "ffn.w1": ColwiseParallel(),
            "ffn.w3": ColwiseParallel(),
            "ffn.w2": RowwiseParallel(output_layouts=Shard(1)),
        })
    if loss_parallel:
        from .loss import parallel_fused_cross_entropy

        group = tp_mesh.get_group()

        def loss_fn(logits_shard: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
            return parallel_fused_cross_entropy(logits_shard, targets, group)

        model.loss_fn = loss_fn
    return model
