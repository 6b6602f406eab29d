#!/usr/bin/env python
"""Operator benchmark harness: times one hand-written operator on the blackwell device with CUDA
events (warm-up, L2 flush between iterations) and reports achieved FLOP/s or bytes/s as a fraction of
the measured peaks of this machine (MEASURED_PEAKS.json if present).

  python benchmark/op_bench.py gemm --m 4096 --n 4096 --k 4096
  python benchmark/op_bench.py rmsnorm --rows 4096 --cols 4096 [--backward]
  python benchmark/op_bench.py softmax|cross_entropy --rows 4096 --cols 32000
  python benchmark/op_bench.py swiglu --rows 4096 --cols 11008
  python benchmark/op_bench.py adamw --numel 268435456
  python benchmark/op_bench.py conv [--rows BATCH]   (ResNet-50 filter shapes, ours vs library, fwd and bwd)
  python benchmark/op_bench.py all            (a Llama-7B shaped sweep; one JSON line per case)

Every case prints one JSON line: {"op", "shape", "dtype", "us", "tflops" | "gbs", "frac_of_measured", ...}.
Parity: reference benchmark/operator_benchmark (harness + per-op FLOPs/bytes, README.md:35-227).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

import torch_musa_b200 as bw  # noqa: E402


def env_info():
    """Software stack and device of this run, as one JSON line (first line of a log that should stay interpretable).
    Parity: reference benchmark/operator_benchmark/README.md:86-165 (records its SDK versions beside the numbers)."""
    info = {"env": True, "torch": torch.__version__, "cuda": torch.version.cuda, "backend": bw.__version__,
            "nccl": ".".join(map(str, bw.bccl.version())), "python": sys.version.split()[0]}
    if bw.is_available():
        p = bw.get_device_properties(0)
        info.update({"device": bw.get_device_name(0), "sms": getattr(p, "multi_processor_count", None),
                     "memory_gb": round(getattr(p, "total_memory", 0) / 2**30, 1), "arch": bw.get_arch_list()})
    pk = peaks()
    info["roofline"] = {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["tflops"], "source": pk["src"]}
    print(json.dumps(info), flush=True)
    return info


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "src": "fallback"}


_FLUSH = None


def flush_l2(dev):
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # 2x the 126 MB L2
    _FLUSH.zero_()


def timeit(fn, dev, iters=20, warmup=5, flush=True):
    for _ in range(warmup):
        fn()
    bw.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush_l2(dev)
        s, e = bw.Event(enable_timing=True), bw.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        total += s.elapsed_time(e)
    return total / iters * 1e3  # us


def report(op, shape, dt, us, flops=None, nbytes=None, **extra):
    pk = peaks()
    out = {"op": op, "shape": shape, "dtype": str(dt).replace("torch.", ""), "us": round(us, 2)}
    if flops is not None:
        tf = flops / us / 1e6
        out["tflops"] = round(tf, 1)
        out["frac_of_" + pk["src"]] = round(tf / pk["tflops"], 3)
    if nbytes is not None:
        gbs = nbytes / us / 1e3
        out["gbs"] = round(gbs, 1)
        out["frac_of_" + pk["src"]] = round(gbs / pk["hbm_gbs"], 3)
    quiet = extra.pop("quiet", False)
    out.update(extra)
    if not quiet:
        print(json.dumps(out), flush=True)
    return out


def bench_gemm(dev, m, n, k, dt=torch.bfloat16, layout="nt", iters=20, quiet=False):
    a = torch.randn(m, k, device=dev, dtype=dt)
    w = torch.randn(n, k, device=dev, dtype=dt)
    if layout == "nt":      # y = x @ W^T (forward)
        fn = lambda: a @ w.t()
    elif layout == "nn":    # dx = dy @ W   (dgrad): [m,n] x [n,k]
        g = torch.randn(m, n, device=dev, dtype=dt)
        fn = lambda: g @ w
    else:                   # dW = dy^T @ x (wgrad): [n,m] x [m,k]
        g = torch.randn(m, n, device=dev, dtype=dt)
        fn = lambda: g.t() @ a
    us = timeit(fn, dev, iters)
    return report("gemm_" + layout, [m, n, k], dt, us, flops=2.0 * m * n * k, launches=1, quiet=quiet)


def bench_gemm_sweep(dev, iters=10, rounds=3):
    """Every tile configuration on the Llama-7B GEMM shapes (forward / dgrad / wgrad).  Configurations are
    interleaved per shape and the best of several rounds is kept, so clock drift does not favour one of them."""
    out = []
    shapes = [(4096, 4096, 4096), (4096, 12288, 4096), (4096, 22016, 4096), (4096, 4096, 11008), (4096, 32000, 4096),
              (8192, 8192, 8192), (2048, 4096, 4096), (4096, 4096, 12288), (4096, 4096, 22016)]
    prev = bw._C._gemm_force_config(0)
    try:
        for (m, n, k) in shapes:
            for layout in ("nt", "nn", "tn"):
                best = {}
                for _ in range(rounds):
                    for cfg in (1, 2, 3, 0):
                        bw._C._gemm_force_config(cfg)
                        r = bench_gemm(dev, m, n, k, layout=layout, iters=iters, quiet=True)
                        if cfg not in best or r["us"] < best[cfg]["us"]:
                            best[cfg] = r
                line = {"op": "gemm_" + layout, "shape": [m, n, k]}
                for cfg, name in ((1, "single_128x256"), (2, "pair_static"), (3, "pair_dynamic"), (0, "auto")):
                    line[name] = best[cfg]["tflops"]
                print(json.dumps(line), flush=True)
                out.append(line)
    finally:
        bw._C._gemm_force_config(prev)
    return out


def bench_gemm_fp8(dev, m, n, k, iters=20):
    """Block-scaled fp8 GEMM (1x128 activation scales, 128x128 weight scales); fraction is of the bf16 peak, so a
    value above 1 means fp8 beats the best bf16 GEMM of this machine."""
    a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    qa, sa = torch.ops.blackwell.quantize_fp8_1x128(a)
    qb = (torch.randn(n, k, device=dev) * 0.5).to(torch.float8_e4m3fn)
    sb = torch.rand((n + 127) // 128, k // 128, device=dev) + 0.5
    us = timeit(lambda: torch.ops.blackwell.scaled_mm(qa, qb, sa, sb, None, None, None, torch.bfloat16), dev, iters)
    r = report("gemm_fp8_blockwise", [m, n, k], "float8_e4m3fn", us, flops=2.0 * m * n * k, launches=1)
    usq = timeit(lambda: torch.ops.blackwell.quantize_fp8_1x128(a), dev, iters)
    report("quantize_fp8_1x128", [m, k], torch.bfloat16, usq, nbytes=m * k * 3 + m * k // 32)
    return r


def bench_attention(dev, batch, heads, seq, dt=torch.bfloat16, iters=10):
    """Causal attention forward and backward, head_dim 128: the hand-written tcgen05 kernels (impl 2) and the library
    cuDNN kernels (impl 1).  Backward FLOPs: five GEMMs against the forward's two."""
    q, k, v = (torch.randn(batch, seq, heads, 128, device=dev, dtype=dt).transpose(1, 2).requires_grad_() for _ in range(3))
    g = torch.randn(batch, seq, heads, 128, device=dev, dtype=dt).transpose(1, 2)
    flops = 4.0 * batch * heads * seq * seq * 128 / 2          # causal: half of QK^T and PV
    prev = bw._C._sdp_impl()
    out = {}
    try:
        for impl, name in ((2, "tcgen05"), (1, "library_cudnn")):
            bw._C._set_sdp_impl(impl)
            with torch.no_grad():
                us = timeit(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True), dev, iters)
            out["fwd_" + name] = report("attention_fwd_" + name, [batch, heads, seq, 128], dt, us, flops=flops)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            us = timeit(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True), dev, iters)
            out["bwd_" + name] = report("attention_bwd_" + name, [batch, heads, seq, 128], dt, us, flops=2.5 * flops)
    finally:
        bw._C._set_sdp_impl(prev)
    return out


RESNET_CONVS = [   # (Cin, H, Cout, R, stride, pad): the distinct non-pointwise filters of ResNet-50 + strided 1x1
    (3, 224, 64, 7, 2, 3), (64, 56, 64, 3, 1, 1), (128, 56, 128, 3, 2, 1), (128, 28, 128, 3, 1, 1),
    (256, 28, 256, 3, 2, 1), (256, 14, 256, 3, 1, 1), (512, 14, 512, 3, 2, 1), (512, 7, 512, 3, 1, 1),
    (256, 56, 512, 1, 2, 0), (1024, 14, 2048, 1, 2, 0),
]


def bench_conv(dev, batch, dt=torch.bfloat16, iters=10, cases=None):
    """Implicit-GEMM convolution (forward, and data + weight gradients) against the library convolution on the same
    tensors; channels-last.  FLOPs = 2 * N * Ho * Wo * K * C * R * S per pass."""
    out = []
    for (C, H, K, R, stride, pad) in (cases or RESNET_CONVS):
        x = torch.randn(batch, C, H, H, device=dev, dtype=dt).contiguous(memory_format=torch.channels_last)
        w = (torch.randn(K, C, R, R, device=dev, dtype=dt) * 0.05).contiguous(memory_format=torch.channels_last)
        Ho = (H + 2 * pad - R) // stride + 1
        flops = 2.0 * batch * Ho * Ho * K * C * R * R
        g = torch.randn(batch, K, Ho, Ho, device=dev, dtype=dt).contiguous(memory_format=torch.channels_last)
        shape = [batch, C, H, H, K, R, stride]
        for impl, name in ((True, "tcgen05"), (False, "library")):
            bw._C._set_implicit_conv_gemm(impl)
            try:
                with torch.no_grad():
                    us = timeit(lambda: F.conv2d(x, w, None, stride, pad), dev, iters)
                out.append(report("conv_fwd_" + name, shape, dt, us, flops=flops))
                xg, wg = x.detach().requires_grad_(C > 3), w.detach().requires_grad_()
                y = F.conv2d(xg, wg, None, stride, pad)
                ins = (xg, wg) if C > 3 else (wg,)
                us = timeit(lambda: torch.autograd.grad(y, ins, g, retain_graph=True), dev, iters)
                out.append(report("conv_bwd_" + name, shape, dt, us, flops=flops * len(ins)))
            finally:
                bw._C._set_implicit_conv_gemm(True)
    return out


def bench_rmsnorm(dev, rows, cols, dt=torch.bfloat16, backward=False):
    x = torch.randn(rows, cols, device=dev, dtype=dt, requires_grad=backward)
    w = torch.ones(cols, device=dev, dtype=dt, requires_grad=backward)
    es = x.element_size()
    if not backward:
        us = timeit(lambda: F.rms_norm(x, (cols,), w, 1e-5), dev)
        return report("rmsnorm_fwd", [rows, cols], dt, us, nbytes=2 * rows * cols * es)
    y = F.rms_norm(x, (cols,), w, 1e-5)
    g = torch.randn_like(y)
    us = timeit(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True), dev)
    return report("rmsnorm_bwd", [rows, cols], dt, us, nbytes=3 * rows * cols * es)


def bench_softmax(dev, rows, cols, dt=torch.bfloat16):
    x = torch.randn(rows, cols, device=dev, dtype=dt)
    us = timeit(lambda: torch.softmax(x, -1), dev)
    return report("softmax_fwd", [rows, cols], dt, us, nbytes=2 * rows * cols * x.element_size())


def bench_ce(dev, rows, cols, dt=torch.bfloat16):
    from torch_musa_b200.ops import fused_cross_entropy

    x = torch.randn(rows, cols, device=dev, dtype=dt, requires_grad=True)
    t = torch.randint(0, cols, (rows,), device="cpu").to(dev)

    def fn():
        loss = fused_cross_entropy(x, t)
        loss.backward()
        x.grad = None

    us = timeit(fn, dev)
    return report("fused_cross_entropy_fwd_bwd", [rows, cols], dt, us, nbytes=3 * rows * cols * x.element_size())


def bench_swiglu(dev, rows, cols, dt=torch.bfloat16):
    from torch_musa_b200.ops import swiglu

    x = torch.randn(rows, 2 * cols, device=dev, dtype=dt)
    us = timeit(lambda: swiglu(x), dev)
    return report("swiglu_fwd", [rows, cols], dt, us, nbytes=3 * rows * cols * x.element_size())


def bench_adamw(dev, numel):
    p = torch.randn(numel, device=dev, requires_grad=True)
    p.grad = torch.randn(numel, device=dev)
    opt = torch.optim.AdamW([p], lr=1e-3, fused=True)
    opt.step()
    us = timeit(opt.step, dev, flush=False)
    # read p, g, m, v; write p, m, v (fp32)
    return report("fused_adamw", [numel], torch.float32, us, nbytes=28 * numel)


def bench_grouped_gemm(dev, rows_per_group=(4300, 3900, 4200, 3984), n=28672, k=4096, dt=torch.bfloat16, iters=10):
    """MoE expert projection (Mixtral dims: 4096 -> 2 x 14336, four local experts, uneven rows): the grouped kernel
    with device-side counts (forward, input gradient, weight gradient) against one dense GEMM per expert after a
    host read of the counts."""
    G, R = len(rows_per_group), sum(rows_per_group)
    cap = 2 * R                                      # capacity-sized buffers, as the exchange hands them over
    x = torch.randn(cap, k, device=dev, dtype=dt)
    w = torch.randn(G, n, k, device=dev, dtype=dt) * 0.02
    dy = torch.randn(cap, n, device=dev, dtype=dt)
    counts = torch.tensor(rows_per_group, dtype=torch.int32, device=dev)
    flops = 2.0 * R * n * k
    out = []
    for mode, a, b, name in ((0, x, w, "fwd"), (1, dy, w, "dgrad"), (2, dy, x, "wgrad")):
        us = timeit(lambda: torch.ops.blackwell.grouped_mm(a, b, counts, mode), dev, iters)
        out.append(report("grouped_gemm_" + name, [list(rows_per_group), n, k], dt, us, flops=flops, launches=1))

    def loop_fwd():
        rows, s = counts.tolist(), 0                  # the host read the grouped kernel does without
        for g, r in enumerate(rows):
            x[s:s + r] @ w[g].t()
            s += r
    us = timeit(loop_fwd, dev, iters)
    out.append(report("expert_loop_fwd", [list(rows_per_group), n, k], dt, us, flops=flops, launches=G))
    return out


def bench_varlen_attention(dev, lens=(4096, 1024, 3000, 72), heads=32, dt=torch.bfloat16, iters=10):
    """Packed variable-length causal attention (one launch per pass) against the same sequences padded to the longest
    one and run as a dense batch."""
    from torch_musa_b200.ops import flash_attn_varlen_func

    total, mx = sum(lens), max(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    q, k, v = (torch.randn(total, heads, 128, device=dev, dtype=dt, requires_grad=True) for _ in range(3))
    flops_f = sum(4.0 * heads * L * L * 128 / 2 for L in lens)
    us = timeit(lambda: flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, causal=True), dev, iters)
    report("varlen_attention_fwd", [list(lens), heads, 128], dt, us, flops=flops_f, launches=1)
    g = torch.randn(total, heads, 128, device=dev, dtype=dt)

    def fb():
        o = flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, causal=True)
        o.backward(g)
        q.grad = k.grad = v.grad = None
    us_fb = timeit(fb, dev, iters)
    report("varlen_attention_fwd_bwd", [list(lens), heads, 128], dt, us_fb, flops=3.5 * flops_f, launches=2)
    qp, kp, vp = (torch.randn(len(lens), mx, heads, 128, device=dev, dtype=dt).transpose(1, 2) for _ in range(3))
    us_pad = timeit(lambda: F.scaled_dot_product_attention(qp, kp, vp, is_causal=True), dev, iters)
    report("padded_dense_attention_fwd", [len(lens), heads, mx, 128], dt, us_pad, flops=flops_f, launches=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--env", action="store_true", help="print the software stack and device as a first JSON line")
    ap.add_argument("--gemm-config", type=int, default=None, help="pin the GEMM tile configuration (1 single CTA, 2 SM pair)")
    a = ap.parse_args()
    if a.env:
        env_info()
        if a.op == "env":
            return
    if a.gemm_config is not None:
        bw._C._gemm_force_config(a.gemm_config)
    dev = torch.device("blackwell:0")
    dt = getattr(torch, a.dtype)
    if a.op == "gemm":
        bench_gemm(dev, a.m, a.n, a.k, dt, a.layout, a.iters)
    elif a.op == "gemm_fp8":
        bench_gemm_fp8(dev, a.m, a.n, a.k, a.iters)
    elif a.op == "attention":
        bench_attention(dev, 1, 32, a.rows, dt, a.iters)
    elif a.op == "conv":
        bench_conv(dev, a.rows if a.rows != 4096 else 64, dt, a.iters)
    elif a.op == "conv_small":      # one 3x3 layer (103 MB activations, larger than L2): the case used for profiler captures
        bench_conv(dev, 256, dt, 3, cases=[(64, 56, 64, 3, 1, 1)])
    elif a.op == "grouped_gemm":
        bench_grouped_gemm(dev, dt=dt, iters=a.iters)
    elif a.op == "varlen_attention":
        bench_varlen_attention(dev, dt=dt, iters=a.iters)
    elif a.op == "gemm_sweep":
        bench_gemm_sweep(dev, a.iters)
    elif a.op == "rmsnorm":
        bench_rmsnorm(dev, a.rows, a.cols, dt, a.backward)
    elif a.op == "softmax":
        bench_softmax(dev, a.rows, a.cols, dt)
    elif a.op == "cross_entropy":
        bench_ce(dev, a.rows, a.cols, dt)
    elif a.op == "swiglu":
        bench_swiglu(dev, a.rows, a.cols, dt)
    elif a.op == "adamw":
        bench_adamw(dev, a.numel)
    elif a.op == "all":
        for (m, n, k) in [(4096, 12288, 4096), (4096, 4096, 4096), (4096, 22016, 4096), (4096, 4096, 11008),
                          (4096, 32000, 4096)]:
            for lay in ("nt", "nn", "tn"):
                bench_gemm(dev, m, n, k, dt, lay)
        bench_rmsnorm(dev, 4096, 4096, dt)
        bench_rmsnorm(dev, 4096, 4096, dt, backward=True)
        bench_rmsnorm(dev, 256, 1024, torch.float16)
        bench_softmax(dev, 4096, 32000, dt)
        bench_ce(dev, 4096, 32000, dt)
        bench_swiglu(dev, 4096, 11008, dt)
        bench_adamw(dev, 1 << 28)
    else:
        raise SystemExit(f"unknown op {a.op}")
    st = bw._C._gemm_status()
    if st:
        raise SystemExit("a GEMM launch gave up on a bounded wait")


if __name__ == "__main__":
    main()
