"""CUDA C++ generation for fused pointwise groups.

A group is an FX sub-graph of element-wise aten operators whose outputs all have one shape; its
inputs broadcast against that shape.  The generated kernel loads every input once, evaluates the
whole expression tree in fp32 registers and stores the outputs, so a chain of N operators costs
one pass over memory instead of N.  Two code paths share the expression: 16-byte packets when all
operands are dense (or one-element), and per-element strided indexing otherwise.  Sources include
no headers (16-bit conversions are spelled out) and are compiled at run time for sm_100a.

Parity: reference torch_musa/_inductor/__init__.py:17-39 registers a Triton code generator for
its device; this module is the code generator of this backend (CUDA C++, no Triton).
"""
from __future__ import annotations

import hashlib
import math
from typing import Callable, Dict, List, Tuple

import torch

aten = torch.ops.aten

_CTYPE = {torch.float32: "float", torch.bfloat16: "bf16", torch.float16: "half", torch.bool: "bool8"}
_BYTES = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.bool: 1}

PRELUDE = r"""
typedef unsigned short u16;
typedef unsigned char u8;
struct bf16 { u16 v; };
struct half { u16 v; };
struct bool8 { u8 v; };
struct Args { void* ptr[12]; long long numel; int ndim; int sizes[6]; long long strides[12][6]; };

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __uint_as_float(((unsigned)x.v) << 16); }
__device__ __forceinline__ float to_f(half x) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(x.v)); return f; }
__device__ __forceinline__ float to_f(bool8 x) { return x.v ? 1.0f : 0.0f; }
__device__ __forceinline__ void from_f(float& o, float f) { o = f; }
__device__ __forceinline__ void from_f(bf16& o, float f) {
  unsigned u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) { o.v = 0x7fc0; return; }
  u += 0x7fffu + ((u >> 16) & 1u);
  o.v = (u16)(u >> 16);
}
__device__ __forceinline__ void from_f(half& o, float f) { asm("cvt.rn.f16.f32 %0, %1;" : "=h"(o.v) : "f"(f)); }
__device__ __forceinline__ void from_f(bool8& o, float f) { o.v = f != 0.0f; }
__device__ __forceinline__ float round_bf16(float f) { bf16 t; from_f(t, f); return to_f(t); }
__device__ __forceinline__ float round_half(float f) { half t; from_f(t, f); return to_f(t); }

template <class T, int V>
__device__ __forceinline__ void load_vec(const void* p, long long i, float (&out)[V]) {
  constexpr int B = V * (int)sizeof(T);
  union { T e[V]; uint4 q[B >= 16 ? B / 16 : 1]; uint2 d; unsigned w; } u;
  const char* src = (const char*)p + i * (long long)sizeof(T);
  if constexpr (B >= 16) {
#pragma unroll
    for (int k = 0; k < B / 16; ++k) u.q[k] = ((const uint4*)src)[k];
  } else if constexpr (B == 8) {
    u.d = *(const uint2*)src;
  } else {
    u.w = *(const unsigned*)src;
  }
#pragma unroll
  for (int k = 0; k < V; ++k) out[k] = to_f(u.e[k]);
}
template <class T, int V>
__device__ __forceinline__ void store_vec(void* p, long long i, const float (&in)[V]) {
  constexpr int B = V * (int)sizeof(T);
  union { T e[V]; uint4 q[B >= 16 ? B / 16 : 1]; uint2 d; unsigned w; } u;
#pragma unroll
  for (int k = 0; k < V; ++k) from_f(u.e[k], in[k]);
  char* dst = (char*)p + i * (long long)sizeof(T);
  if constexpr (B >= 16) {
#pragma unroll
    for (int k = 0; k < B / 16; ++k) ((uint4*)dst)[k] = u.q[k];
  } else if constexpr (B == 8) {
    *(uint2*)dst = u.d;
  } else {
    *(unsigned*)dst = u.w;
  }
}
template <class T> __device__ __forceinline__ float load1(const void* p, long long i) { return to_f(((const T*)p)[i]); }
template <class T> __device__ __forceinline__ void store1(void* p, long long i, float f) { from_f(((T*)p)[i], f); }
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float gelu_tanh(float x) {
  float inner = 0.79788456080286535588f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float gelu_erf_bwd(float g, float x) {
  float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
  float pdf = 0.39894228040143267794f * expf(-0.5f * x * x);
  return g * (cdf + x * pdf);
}
__device__ __forceinline__ float gelu_tanh_bwd(float g, float x) {
  float x2 = x * x;
  float inner = 0.79788456080286535588f * (x + 0.044715f * x * x2);
  float t = tanhf(inner);
  float dinner = 0.79788456080286535588f * (1.0f + 3.0f * 0.044715f * x2);
  return g * (0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * dinner);
}
__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }
"""


def _lit(x) -> str:
    if isinstance(x, bool):
        return "1.0f" if x else "0.0f"
    x = float(x)
    if math.isnan(x):
        return "__int_as_float(0x7fc00000)"
    if math.isinf(x):
        return "__int_as_float(0x7f800000)" if x > 0 else "__int_as_float(0xff800000)"
    return repr(x) + "f" if ("." in repr(x) or "e" in repr(x) or "inf" in repr(x)) else repr(x) + ".0f"


def _b(expr: str) -> str:
    """Boolean results are carried as 0/1 floats."""
    return f"(({expr}) ? 1.0f : 0.0f)"


# target -> function(list of C operand expressions, node) -> C expression (fp32)
OPS: Dict[object, Callable] = {}


def _reg(*targets):
    def deco(fn):
        for t in targets:
            OPS[t] = fn
        return fn
    return deco


def _alpha(node, default=1):
    return node.kwargs.get("alpha", default)


@_reg(aten.add.Tensor, aten.add.Scalar)
def _add(a, n):
    al = _alpha(n)
    return f"({a[0]} + {a[1]})" if al == 1 else f"({a[0]} + {_lit(al)} * {a[1]})"


@_reg(aten.sub.Tensor, aten.sub.Scalar)
def _sub(a, n):
    al = _alpha(n)
    return f"({a[0]} - {a[1]})" if al == 1 else f"({a[0]} - {_lit(al)} * {a[1]})"


@_reg(aten.rsub.Scalar, aten.rsub.Tensor)
def _rsub(a, n):
    return f"({a[1]} - {a[0]})"


_reg(aten.mul.Tensor, aten.mul.Scalar)(lambda a, n: f"({a[0]} * {a[1]})")
_reg(aten.div.Tensor, aten.div.Scalar)(lambda a, n: f"({a[0]} / {a[1]})")
_reg(aten.neg.default)(lambda a, n: f"(-{a[0]})")
_reg(aten.abs.default)(lambda a, n: f"fabsf({a[0]})")
_reg(aten.exp.default)(lambda a, n: f"expf({a[0]})")
_reg(aten.exp2.default)(lambda a, n: f"exp2f({a[0]})")
_reg(aten.expm1.default)(lambda a, n: f"expm1f({a[0]})")
_reg(aten.log.default)(lambda a, n: f"logf({a[0]})")
_reg(aten.log2.default)(lambda a, n: f"log2f({a[0]})")
_reg(aten.log1p.default)(lambda a, n: f"log1pf({a[0]})")
_reg(aten.sqrt.default)(lambda a, n: f"sqrtf({a[0]})")
_reg(aten.rsqrt.default)(lambda a, n: f"(1.0f / sqrtf({a[0]}))")
_reg(aten.reciprocal.default)(lambda a, n: f"(1.0f / {a[0]})")
_reg(aten.tanh.default)(lambda a, n: f"tanhf({a[0]})")
_reg(aten.sigmoid.default)(lambda a, n: f"sigmoidf({a[0]})")
_reg(aten.relu.default)(lambda a, n: f"fmaxf({a[0]}, 0.0f)")
_reg(aten.silu.default)(lambda a, n: f"({a[0]} * sigmoidf({a[0]}))")
_reg(aten.erf.default)(lambda a, n: f"erff({a[0]})")
_reg(aten.sin.default)(lambda a, n: f"sinf({a[0]})")
_reg(aten.cos.default)(lambda a, n: f"cosf({a[0]})")
_reg(aten.tan.default)(lambda a, n: f"tanf({a[0]})")
_reg(aten.asin.default)(lambda a, n: f"asinf({a[0]})")
_reg(aten.acos.default)(lambda a, n: f"acosf({a[0]})")
_reg(aten.atan.default)(lambda a, n: f"atanf({a[0]})")
_reg(aten.sinh.default)(lambda a, n: f"sinhf({a[0]})")
_reg(aten.cosh.default)(lambda a, n: f"coshf({a[0]})")
_reg(aten.asinh.default)(lambda a, n: f"asinhf({a[0]})")
_reg(aten.acosh.default)(lambda a, n: f"acoshf({a[0]})")
_reg(aten.atanh.default)(lambda a, n: f"atanhf({a[0]})")
_reg(aten.erfc.default)(lambda a, n: f"erfcf({a[0]})")
_reg(aten.log10.default)(lambda a, n: f"log10f({a[0]})")
_reg(aten.floor.default)(lambda a, n: f"floorf({a[0]})")
_reg(aten.ceil.default)(lambda a, n: f"ceilf({a[0]})")
_reg(aten.trunc.default)(lambda a, n: f"truncf({a[0]})")
_reg(aten.round.default)(lambda a, n: f"nearbyintf({a[0]})")
_reg(aten.sign.default)(lambda a, n: f"(float)(({a[0]} > 0.0f) - ({a[0]} < 0.0f))")
_reg(aten.atan2.default)(lambda a, n: f"atan2f({a[0]}, {a[1]})")
_reg(aten.fmod.Tensor, aten.fmod.Scalar)(lambda a, n: f"fmodf({a[0]}, {a[1]})")
_reg(aten.isnan.default)(lambda a, n: _b(f"{a[0]} != {a[0]}"))
_reg(aten.maximum.default)(lambda a, n: f"fmaxf({a[0]}, {a[1]})")
_reg(aten.minimum.default)(lambda a, n: f"fminf({a[0]}, {a[1]})")
_reg(aten.pow.Tensor_Tensor, aten.pow.Tensor_Scalar)(
    lambda a, n: f"({a[0]} * {a[0]})" if n.args[1] == 2 else f"powf({a[0]}, {a[1]})")
_reg(aten.where.self)(lambda a, n: f"(({a[0]}) != 0.0f ? {a[1]} : {a[2]})")
_reg(aten.gt.Tensor, aten.gt.Scalar)(lambda a, n: _b(f"{a[0]} > {a[1]}"))
_reg(aten.lt.Tensor, aten.lt.Scalar)(lambda a, n: _b(f"{a[0]} < {a[1]}"))
_reg(aten.ge.Tensor, aten.ge.Scalar)(lambda a, n: _b(f"{a[0]} >= {a[1]}"))
_reg(aten.le.Tensor, aten.le.Scalar)(lambda a, n: _b(f"{a[0]} <= {a[1]}"))
_reg(aten.eq.Tensor, aten.eq.Scalar)(lambda a, n: _b(f"{a[0]} == {a[1]}"))
_reg(aten.ne.Tensor, aten.ne.Scalar)(lambda a, n: _b(f"{a[0]} != {a[1]}"))
_reg(aten.logical_not.default)(lambda a, n: _b(f"{a[0]} == 0.0f"))
_reg(aten.logical_and.default)(lambda a, n: _b(f"{a[0]} != 0.0f && {a[1]} != 0.0f"))
_reg(aten.logical_or.default)(lambda a, n: _b(f"{a[0]} != 0.0f || {a[1]} != 0.0f"))
_reg(aten.sigmoid_backward.default)(lambda a, n: f"({a[0]} * (1.0f - {a[1]}) * {a[1]})")
_reg(aten.tanh_backward.default)(lambda a, n: f"({a[0]} * (1.0f - {a[1]} * {a[1]}))")
_reg(aten.threshold_backward.default)(lambda a, n: f"({a[1]} <= {a[2]} ? 0.0f : {a[0]})")
_reg(aten.leaky_relu.default)(
    lambda a, n: f"({a[0]} > 0.0f ? {a[0]} : {a[0]} * {a[1] if len(a) > 1 else '0.01f'})")


@_reg(aten.silu_backward.default)
def _silu_bwd(a, n):
    return f"({a[0]} * sigmoidf({a[1]}) * (1.0f + {a[1]} * (1.0f - sigmoidf({a[1]}))))"


@_reg(aten.gelu.default)
def _gelu(a, n):
    return f"gelu_tanh({a[0]})" if n.kwargs.get("approximate", "none") == "tanh" else f"gelu_erf({a[0]})"


@_reg(aten.gelu_backward.default)
def _gelu_bwd(a, n):
    fn = "gelu_tanh_bwd" if n.kwargs.get("approximate", "none") == "tanh" else "gelu_erf_bwd"
    return f"{fn}({a[0]}, {a[1]})"


@_reg(aten.clamp.default)
def _clamp(a, n):
    e = a[0]
    lo = n.args[1] if len(n.args) > 1 else n.kwargs.get("min")
    hi = n.args[2] if len(n.args) > 2 else n.kwargs.get("max")
    if lo is not None:
        e = f"fmaxf({e}, {_lit(lo)})"
    if hi is not None:
        e = f"fminf({e}, {_lit(hi)})"
    return e


_reg(aten.clamp_min.default)(lambda a, n: f"fmaxf({a[0]}, {a[1]})")
_reg(aten.clamp_max.default)(lambda a, n: f"fminf({a[0]}, {a[1]})")


@_reg(aten._to_copy.default, torch.ops.prims.convert_element_type.default)
def _cast(a, n):
    dt = n.kwargs.get("dtype", n.args[1] if len(n.args) > 1 else None)
    if dt == torch.bfloat16:
        return f"round_bf16({a[0]})"
    if dt == torch.float16:
        return f"round_half({a[0]})"
    if dt == torch.bool:
        return _b(f"{a[0]} != 0.0f")
    return a[0]


def supported_dtype(dt) -> bool:
    return dt in _CTYPE


def node_supported(node) -> bool:
    """Element-wise operator on supported dtypes with no layout-changing keyword."""
    if node.op != "call_function" or node.target not in OPS:
        return False
    val = node.meta.get("val")
    if not isinstance(val, torch.Tensor) or not supported_dtype(val.dtype) or val.device.type != "blackwell":
        return False
    if val.dim() > 6 or any(not isinstance(s, int) for s in val.shape):
        return False
    if node.target in (aten._to_copy.default,):
        extra = {k for k, v in node.kwargs.items() if v is not None} - {"dtype"}
        if extra or "dtype" not in node.kwargs:
            return False
    if node.target in (aten.div.Tensor, aten.div.Scalar) and node.kwargs.get("rounding_mode") is not None:
        return False
    for a in node.args:
        if isinstance(a, torch.fx.Node):
            v = a.meta.get("val")
            if not isinstance(v, torch.Tensor) or not supported_dtype(v.dtype) or v.device.type != "blackwell":
                return False
        elif isinstance(a, (list, tuple)):
            return False
        elif a is not None and not isinstance(a, (int, float, bool, torch.dtype)):
            return False
    return True


def generate(sub: torch.fx.GraphModule, name: str) -> Tuple[str, dict]:
    """CUDA source for a fused group plus its description (operand dtypes, output shape, vector width)."""
    placeholders = [n for n in sub.graph.nodes if n.op == "placeholder"]
    out_node = next(n for n in sub.graph.nodes if n.op == "output")
    outs = out_node.args[0]
    outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
    shape = tuple(outs[0].meta["val"].shape)
    for o in outs:
        if tuple(o.meta["val"].shape) != shape:
            raise ValueError("outputs of a fused group must share one shape")
    in_dt = [p.meta["val"].dtype for p in placeholders]
    out_dt = [o.meta["val"].dtype for o in outs]
    if len(in_dt) + len(out_dt) > 12:
        raise ValueError("too many operands for one fused kernel")
    if not in_dt:
        raise ValueError("a fused group needs at least one tensor input")
    for p in placeholders:
        ps = tuple(p.meta["val"].shape)
        if len(ps) > len(shape) or any(a != b and a != 1 for a, b in zip(reversed(ps), reversed(shape))):
            raise ValueError("input does not broadcast to the output shape")
    vec = 8 if any(_BYTES[d] == 2 for d in in_dt + out_dt) else 4
    if any(_BYTES[d] == 1 for d in in_dt + out_dt) and vec < 4:
        vec = 4

    names: Dict[torch.fx.Node, str] = {p: f"x{i}" for i, p in enumerate(placeholders)}
    body: List[str] = []
    k = 0
    for n in sub.graph.nodes:
        if n.op != "call_function":
            continue
        ops = []
        for a in n.args:
            if isinstance(a, torch.fx.Node):
                ops.append(names[a])
            elif isinstance(a, (int, float, bool)):
                ops.append(_lit(a))
            else:
                ops.append(None)
        expr = OPS[n.target](ops, n)
        # a 16-bit result rounds like the unfused operator would when something outside the group reads it;
        # inside the group the value stays in fp32
        names[n] = f"v{k}"
        body.append(f"float v{k} = {expr};")
        k += 1
    ni, no = len(in_dt), len(out_dt)
    lines = [PRELUDE, f'extern "C" __global__ void __launch_bounds__(256) {name}(Args a, int fast) {{',
             "  long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;",
             "  long long nthreads = (long long)gridDim.x * blockDim.x;",
             "  if (fast) {",
             f"    constexpr int V = {vec};"]
    for i in range(ni):
        lines.append(f"    const long long per{i} = a.strides[{i}][0], div{i} = a.strides[{i}][1];")
    lines.append("    for (long long base = tid * V; base < a.numel; base += nthreads * V) {")
    for i, dt in enumerate(in_dt):
        lines.append(f"      float in{i}[V];")
        lines.append(f"      if (div{i} || !per{i}) {{ float s = load1<{_CTYPE[dt]}>(a.ptr[{i}], div{i} ? base / div{i} : 0); "
                     f"for (int j = 0; j < V; ++j) in{i}[j] = s; }}")
        lines.append(f"      else load_vec<{_CTYPE[dt]}, V>(a.ptr[{i}], per{i} == a.numel ? base : base % per{i}, in{i});")
    for o in range(no):
        lines.append(f"      float out{o}[V];")
    lines.append("#pragma unroll")
    lines.append("      for (int j = 0; j < V; ++j) {")
    for i in range(ni):
        lines.append(f"        float x{i} = in{i}[j];")
    lines += ["        " + b for b in body]
    for o, on in enumerate(outs):
        lines.append(f"        out{o}[j] = {names[on]};")
    lines.append("      }")
    for o, dt in enumerate(out_dt):
        lines.append(f"      store_vec<{_CTYPE[dt]}, V>(a.ptr[{ni + o}], base, out{o});")
    lines += ["    }", "  } else {", "    for (long long i = tid; i < a.numel; i += nthreads) {",
              "      long long r = i;"]
    for i in range(ni):
        lines.append(f"      long long o{i} = 0;")
    lines.append("      for (int d = a.ndim - 1; d >= 0; --d) {")
    lines.append("        long long c = r % a.sizes[d]; r /= a.sizes[d];")
    for i in range(ni):
        lines.append(f"        o{i} += c * a.strides[{i}][d];")
    lines.append("      }")
    for i, dt in enumerate(in_dt):
        lines.append(f"      float x{i} = load1<{_CTYPE[dt]}>(a.ptr[{i}], o{i});")
    lines += ["      " + b for b in body]
    for o, (on, dt) in enumerate(zip(outs, out_dt)):
        lines.append(f"      store1<{_CTYPE[dt]}>(a.ptr[{ni + o}], i, {names[on]});")
    lines += ["    }", "  }", "}"]
    src = "\n".join(lines)
    info = {"in_dtypes": in_dt, "out_dtypes": out_dt, "shape": shape, "vec": vec, "n_ops": k}
    return src, info


def kernel_name(sub: torch.fx.GraphModule) -> str:
    h = hashlib.sha1(str(sub.graph).encode()).hexdigest()[:12]
    return f"b200_fused_{h}"
