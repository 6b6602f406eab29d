// General pointwise loops: up to three inputs, any broadcast / strided layout, any mix of the ten element types,
// scalar operands folded into the launch.  The host coalesces the iteration space to at most eight dimensions
// (usually one); a thread walks four consecutive output elements, decomposing the linear index with precomputed
// magic-number division, converts each operand to the operator's compute type (fp32 for the 16/32-bit floating
// types, fp64 for doubles, int64 for integers and bool), applies the operator and converts to the output type.
// The same-layout, same-dtype fast paths of elementwise.cu stay in front of this for the hot training operators;
// this file is what makes every other case run on our own code instead of the fallback.
// Parity: reference torch_musa/csrc/aten/ops/musa/elemwise/BinaryLoops.muh:8-268 and
// torch_musa/csrc/aten/utils/TensorIterator.h:14-171 (offset calculator, dynamic casting loops).
#include "common.cuh"

namespace b200k {
namespace {

constexpr int kEwThreads = 256;
constexpr int kPerThread = 4;

struct FastDiv {          // n / d for 0 <= n < 2^31 through one mulhi and a shift
  uint32_t d, m, s;
};
inline FastDiv make_fastdiv(uint32_t d) {
  FastDiv f;
  f.d = d;
  uint32_t s = 0;
  while ((1ull << s) < d) ++s;
  f.s = s;
  f.m = (uint32_t)(((1ull << 32) * ((1ull << s) - d)) / d + 1);
  return f;
}
__device__ __forceinline__ uint32_t fd_div(uint32_t n, const FastDiv& f) {
  return (__umulhi(n, f.m) + n) >> f.s;
}

struct EwArgs {
  int ndim, n_in, op;
  int dtype[4];
  char* ptr[4];
  int64_t strides[4][8];   // bytes
  FastDiv div[8];          // sizes, innermost first
  int64_t sizes[8];
  int64_t numel;
  double s[3];             // values of the scalar inputs
  double p0, p1;           // operator parameters (alpha, bounds, slopes)
  int scalar_mask;         // bit k: input k is the scalar s[k]
  int small_index;         // numel < 2^31: 32-bit index arithmetic
};

template <typename C>
__device__ __forceinline__ C load_as(const char* p, int dt) {
  switch (dt) {
    case B200_F32: return (C)(*reinterpret_cast<const float*>(p));
    case B200_BF16: return (C)__bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
    case B200_F16: return (C)__half2float(*reinterpret_cast<const __half*>(p));
    case B200_F64: return (C)(*reinterpret_cast<const double*>(p));
    case B200_I32: return (C)(*reinterpret_cast<const int32_t*>(p));
    case B200_I64: return (C)(*reinterpret_cast<const int64_t*>(p));
    case B200_U8: return (C)(*reinterpret_cast<const uint8_t*>(p));
    case B200_BOOL: return (C)(*reinterpret_cast<const uint8_t*>(p) != 0);
    case B200_I8: return (C)(*reinterpret_cast<const int8_t*>(p));
    case B200_I16: return (C)(*reinterpret_cast<const int16_t*>(p));
    default: return (C)0;
  }
}
template <typename C>
__device__ __forceinline__ void store_from(char* p, int dt, C v) {
  switch (dt) {
    case B200_F32: *reinterpret_cast<float*>(p) = (float)v; break;
    case B200_BF16: *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn((float)v); break;
    case B200_F16: *reinterpret_cast<__half*>(p) = __float2half_rn((float)v); break;
    case B200_F64: *reinterpret_cast<double*>(p) = (double)v; break;
    case B200_I32: *reinterpret_cast<int32_t*>(p) = (int32_t)v; break;
    case B200_I64: *reinterpret_cast<int64_t*>(p) = (int64_t)v; break;
    case B200_U8: *reinterpret_cast<uint8_t*>(p) = (uint8_t)v; break;
    case B200_BOOL: *reinterpret_cast<uint8_t*>(p) = (v != (C)0) ? 1 : 0; break;
    case B200_I8: *reinterpret_cast<int8_t*>(p) = (int8_t)v; break;
    case B200_I16: *reinterpret_cast<int16_t*>(p) = (int16_t)v; break;
    default: break;
  }
}

template <typename C> struct Math;
template <> struct Math<float> {
  static __device__ __forceinline__ float pw(float a, float b) { return powf(a, b); }
  static __device__ __forceinline__ float fl(float a) { return floorf(a); }
  static __device__ __forceinline__ float ce(float a) { return ceilf(a); }
  static __device__ __forceinline__ float rn(float a) { return nearbyintf(a); }
  static __device__ __forceinline__ float tr(float a) { return truncf(a); }
  static __device__ __forceinline__ float ex(float a) { return expf(a); }
  static __device__ __forceinline__ float lg(float a) { return logf(a); }
  static __device__ __forceinline__ float sq(float a) { return sqrtf(a); }
  static __device__ __forceinline__ float sn(float a) { return sinf(a); }
  static __device__ __forceinline__ float cs(float a) { return cosf(a); }
  static __device__ __forceinline__ float th(float a) { return tanhf(a); }
  static __device__ __forceinline__ float er(float a) { return erff(a); }
  static __device__ __forceinline__ float l1p(float a) { return log1pf(a); }
  static __device__ __forceinline__ float em1(float a) { return expm1f(a); }
  static __device__ __forceinline__ float fm(float a, float b) { return fmodf(a, b); }
  static __device__ __forceinline__ float ab(float a) { return fabsf(a); }
  static __device__ __forceinline__ float at2(float a, float b) { return atan2f(a, b); }
  static __device__ __forceinline__ float asn(float a) { return asinf(a); }
  static __device__ __forceinline__ float acs(float a) { return acosf(a); }
  static __device__ __forceinline__ float atn(float a) { return atanf(a); }
  static __device__ __forceinline__ float snh(float a) { return sinhf(a); }
  static __device__ __forceinline__ float csh(float a) { return coshf(a); }
  static __device__ __forceinline__ float asnh(float a) { return asinhf(a); }
  static __device__ __forceinline__ float acsh(float a) { return acoshf(a); }
  static __device__ __forceinline__ float atnh(float a) { return atanhf(a); }
  static __device__ __forceinline__ float erc(float a) { return erfcf(a); }
};
template <> struct Math<double> {
  static __device__ __forceinline__ double pw(double a, double b) { return pow(a, b); }
  static __device__ __forceinline__ double fl(double a) { return floor(a); }
  static __device__ __forceinline__ double ce(double a) { return ceil(a); }
  static __device__ __forceinline__ double rn(double a) { return nearbyint(a); }
  static __device__ __forceinline__ double tr(double a) { return trunc(a); }
  static __device__ __forceinline__ double ex(double a) { return exp(a); }
  static __device__ __forceinline__ double lg(double a) { return log(a); }
  static __device__ __forceinline__ double sq(double a) { return sqrt(a); }
  static __device__ __forceinline__ double sn(double a) { return sin(a); }
  static __device__ __forceinline__ double cs(double a) { return cos(a); }
  static __device__ __forceinline__ double th(double a) { return tanh(a); }
  static __device__ __forceinline__ double er(double a) { return erf(a); }
  static __device__ __forceinline__ double l1p(double a) { return log1p(a); }
  static __device__ __forceinline__ double em1(double a) { return expm1(a); }
  static __device__ __forceinline__ double fm(double a, double b) { return fmod(a, b); }
  static __device__ __forceinline__ double ab(double a) { return fabs(a); }
  static __device__ __forceinline__ double at2(double a, double b) { return atan2(a, b); }
  static __device__ __forceinline__ double asn(double a) { return asin(a); }
  static __device__ __forceinline__ double acs(double a) { return acos(a); }
  static __device__ __forceinline__ double atn(double a) { return atan(a); }
  static __device__ __forceinline__ double snh(double a) { return sinh(a); }
  static __device__ __forceinline__ double csh(double a) { return cosh(a); }
  static __device__ __forceinline__ double asnh(double a) { return asinh(a); }
  static __device__ __forceinline__ double acsh(double a) { return acosh(a); }
  static __device__ __forceinline__ double atnh(double a) { return atanh(a); }
  static __device__ __forceinline__ double erc(double a) { return erfc(a); }
};

// floating compute types
template <typename C>
__device__ __forceinline__ C apply_float(int op, C a, C b, C c, double s0, double s1) {
  using M = Math<C>;
  switch (op) {
    case B200_EW_ADD: return a + (C)s0 * b;
    case B200_EW_SUB: return a - (C)s0 * b;
    case B200_EW_RSUB: return b - (C)s0 * a;
    case B200_EW_MUL: return a * b;
    case B200_EW_DIV: return a / b;
    case B200_EW_DIV_FLOOR: return M::fl(a / b);
    case B200_EW_DIV_TRUNC: return M::tr(a / b);
    case B200_EW_REMAINDER: { C r = M::fm(a, b); return (r != (C)0 && ((r < (C)0) != (b < (C)0))) ? r + b : r; }
    case B200_EW_FMOD: return M::fm(a, b);
    case B200_EW_POW: return M::pw(a, b);
    case B200_EW_ATAN2: return M::at2(a, b);
    case B200_EW_MAXIMUM: return (a != a || b != b) ? (C)NAN : (a > b ? a : b);
    case B200_EW_MINIMUM: return (a != a || b != b) ? (C)NAN : (a < b ? a : b);
    case B200_EW_EQ: return (C)(a == b);
    case B200_EW_NE: return (C)(a != b);
    case B200_EW_LT: return (C)(a < b);
    case B200_EW_LE: return (C)(a <= b);
    case B200_EW_GT: return (C)(a > b);
    case B200_EW_GE: return (C)(a >= b);
    case B200_EW_LOGICAL_AND: return (C)((a != (C)0) && (b != (C)0));
    case B200_EW_LOGICAL_OR: return (C)((a != (C)0) || (b != (C)0));
    case B200_EW_LOGICAL_XOR: return (C)((a != (C)0) != (b != (C)0));
    case B200_EW_WHERE: return a != (C)0 ? b : c;
    case B200_EW_MASKED_FILL: return b != (C)0 ? (C)s0 : a;          // a = self, b = mask
    case B200_EW_CLAMP: { C v = a; if (v < (C)s0) v = (C)s0; if (v > (C)s1) v = (C)s1; return a != a ? a : v; }
    case B200_EW_CLAMP_TENSOR: { C v = a; if (v < b) v = b; if (v > c) v = c; return a != a ? a : v; }
    case B200_EW_ADDCMUL: return a + (C)s0 * b * c;
    case B200_EW_ADDCDIV: return a + (C)s0 * b / c;
    case B200_EW_LERP: return a + (C)s0 * (b - a);
    case B200_EW_LERP_TENSOR: return a + c * (b - a);
    case B200_EW_THRESHOLD_BWD: return b <= (C)s0 ? (C)0 : a;        // a = grad, b = input
    case B200_EW_LEAKY_RELU: return a > (C)0 ? a : a * (C)s0;
    case B200_EW_LEAKY_RELU_BWD: return b > (C)0 ? a : a * (C)s0;    // a = grad, b = input
    case B200_EW_ELU: return a > (C)0 ? a * (C)s1 : (C)s0 * (C)s1 * M::em1(a);   // s0 alpha, s1 scale
    case B200_EW_HARDTANH_BWD: return (b <= (C)s0 || b >= (C)s1) ? (C)0 : a;
    case B200_EW_XLOGY: return (b != b) ? b : (a == (C)0 ? (C)0 : a * M::lg(b));
    case B200_EW_LOG_SIGMOID_BWD: { C z = M::ex(-M::ab(b)); C s = b < (C)0 ? (C)1 / ((C)1 + z) : z / ((C)1 + z); return a * s; }   // a = grad, b = x: grad * sigmoid(-x)
    case B200_EW_SOFTPLUS: { C z = a * (C)s0; return z > (C)s1 ? a : M::l1p(M::ex(z)) / (C)s0; }
    // unary
    case B200_EW_NEG: return -a;
    case B200_EW_ABS: return M::ab(a);
    case B200_EW_SIGN: return (C)((a > (C)0) - (a < (C)0));
    case B200_EW_FLOOR: return M::fl(a);
    case B200_EW_CEIL: return M::ce(a);
    case B200_EW_ROUND: return M::rn(a);
    case B200_EW_TRUNC: return M::tr(a);
    case B200_EW_FRAC: return a - M::tr(a);
    case B200_EW_EXP: return M::ex(a);
    case B200_EW_EXP2: return M::pw((C)2, a);
    case B200_EW_EXPM1: return M::em1(a);
    case B200_EW_LOG: return M::lg(a);
    case B200_EW_LOG2: return M::lg(a) * (C)1.4426950408889634;
    case B200_EW_LOG10: return M::lg(a) * (C)0.4342944819032518;
    case B200_EW_LOG1P: return M::l1p(a);
    case B200_EW_SQRT: return M::sq(a);
    case B200_EW_RSQRT: return (C)1 / M::sq(a);
    case B200_EW_RECIPROCAL: return (C)1 / a;
    case B200_EW_SQUARE: return a * a;
    case B200_EW_SIN: return M::sn(a);
    case B200_EW_COS: return M::cs(a);
    case B200_EW_TAN: return M::sn(a) / M::cs(a);
    case B200_EW_TANH: return M::th(a);
    case B200_EW_SIGMOID: return (C)1 / ((C)1 + M::ex(-a));
    case B200_EW_ERF: return M::er(a);
    case B200_EW_RELU: return a > (C)0 ? a : (a != a ? a : (C)0);
    case B200_EW_SILU: return a / ((C)1 + M::ex(-a));
    case B200_EW_GELU_ERF: return (C)0.5 * a * ((C)1 + M::er(a * (C)0.70710678118654752));
    case B200_EW_GELU_TANH: { C in = (C)0.7978845608028654 * (a + (C)0.044715 * a * a * a); return (C)0.5 * a * ((C)1 + M::th(in)); }
    case B200_EW_LOG_SIGMOID: return (a < (C)0 ? a : (C)0) - M::l1p(M::ex(-M::ab(a)));
    case B200_EW_ASIN: return M::asn(a);
    case B200_EW_ACOS: return M::acs(a);
    case B200_EW_ATAN: return M::atn(a);
    case B200_EW_SINH: return M::snh(a);
    case B200_EW_COSH: return M::csh(a);
    case B200_EW_ASINH: return M::asnh(a);
    case B200_EW_ACOSH: return M::acsh(a);
    case B200_EW_ATANH: return M::atnh(a);
    case B200_EW_ERFC: return M::erc(a);
    case B200_EW_ISNAN: return (C)(a != a);
    case B200_EW_ISINF: return (C)(a == (C)INFINITY || a == -(C)INFINITY);
    case B200_EW_ISFINITE: return (C)(a == a && a != (C)INFINITY && a != -(C)INFINITY);
    case B200_EW_LOGICAL_NOT: return (C)(a == (C)0);
    case B200_EW_COPY: return a;
    case B200_EW_FILL: return (C)s0;
    default: return a;
  }
}

__device__ __forceinline__ int64_t ipow(int64_t a, int64_t b) {
  if (b < 0) return (a == 1) ? 1 : ((a == -1) ? ((b & 1) ? -1 : 1) : 0);
  int64_t r = 1;
  while (b) { if (b & 1) r *= a; a *= a; b >>= 1; }
  return r;
}

// integer / bool compute
__device__ __forceinline__ int64_t apply_int(int op, int64_t a, int64_t b, int64_t c, double s0, double s1) {
  switch (op) {
    case B200_EW_ADD: return a + (int64_t)s0 * b;
    case B200_EW_SUB: return a - (int64_t)s0 * b;
    case B200_EW_RSUB: return b - (int64_t)s0 * a;
    case B200_EW_MUL: return a * b;
    case B200_EW_DIV_TRUNC: return b ? a / b : 0;
    case B200_EW_DIV_FLOOR: { if (!b) return 0; int64_t q = a / b; return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q; }
    case B200_EW_REMAINDER: { if (!b) return 0; int64_t r = a % b; return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r; }
    case B200_EW_FMOD: return b ? a % b : 0;
    case B200_EW_POW: return ipow(a, b);
    case B200_EW_MAXIMUM: return a > b ? a : b;
    case B200_EW_MINIMUM: return a < b ? a : b;
    case B200_EW_EQ: return a == b;
    case B200_EW_NE: return a != b;
    case B200_EW_LT: return a < b;
    case B200_EW_LE: return a <= b;
    case B200_EW_GT: return a > b;
    case B200_EW_GE: return a >= b;
    case B200_EW_LOGICAL_AND: return (a != 0) && (b != 0);
    case B200_EW_LOGICAL_OR: return (a != 0) || (b != 0);
    case B200_EW_LOGICAL_XOR: return (a != 0) != (b != 0);
    case B200_EW_BITWISE_AND: return a & b;
    case B200_EW_BITWISE_OR: return a | b;
    case B200_EW_BITWISE_XOR: return a ^ b;
    case B200_EW_LSHIFT: return (b < 0 || b > 63) ? 0 : (int64_t)((uint64_t)a << b);
    case B200_EW_RSHIFT: return (b < 0 || b > 63) ? (a < 0 ? -1 : 0) : (a >> b);
    case B200_EW_WHERE: return a != 0 ? b : c;
    case B200_EW_MASKED_FILL: return b != 0 ? (int64_t)s0 : a;
    case B200_EW_CLAMP: { int64_t v = a; if ((double)v < s0) v = (int64_t)s0; if ((double)v > s1) v = (int64_t)s1; return v; }
    case B200_EW_CLAMP_TENSOR: { int64_t v = a; if (v < b) v = b; if (v > c) v = c; return v; }
    case B200_EW_ADDCMUL: return a + (int64_t)s0 * b * c;
    case B200_EW_NEG: return -a;
    case B200_EW_ABS: return a < 0 ? -a : a;
    case B200_EW_SIGN: return (a > 0) - (a < 0);
    case B200_EW_SQUARE: return a * a;
    case B200_EW_RELU: return a > 0 ? a : 0;
    case B200_EW_BITWISE_NOT: return ~a;
    case B200_EW_LOGICAL_NOT: return a == 0;
    case B200_EW_ISNAN: case B200_EW_ISINF: return 0;
    case B200_EW_ISFINITE: return 1;
    case B200_EW_FLOOR: case B200_EW_CEIL: case B200_EW_ROUND: case B200_EW_TRUNC: case B200_EW_COPY: return a;
    case B200_EW_FILL: return (int64_t)s0;
    default: return a;
  }
}

template <typename C, bool INT>
__device__ __forceinline__ C apply(int op, C a, C b, C c, double s0, double s1) {
  if constexpr (INT) return apply_int(op, a, b, c, s0, s1);
  else return apply_float<C>(op, a, b, c, s0, s1);
}

template <typename C, bool INT>
__global__ void __launch_bounds__(kEwThreads) ew_kernel(const EwArgs A) {
  const int64_t base = ((int64_t)blockIdx.x * kEwThreads + threadIdx.x) * kPerThread;
#pragma unroll
  for (int u = 0; u < kPerThread; ++u) {
    const int64_t i = base + u;
    if (i >= A.numel) return;
    int64_t off[4] = {0, 0, 0, 0};
    if (A.ndim == 1) {
#pragma unroll
      for (int t = 0; t < 4; ++t) off[t] = i * A.strides[t][0];
    } else if (A.small_index) {
      uint32_t rem = (uint32_t)i;
      for (int d = 0; d < A.ndim; ++d) {
        const uint32_t q = fd_div(rem, A.div[d]);
        const uint32_t idx = rem - q * A.div[d].d;
        rem = q;
#pragma unroll
        for (int t = 0; t < 4; ++t) off[t] += (int64_t)idx * A.strides[t][d];
      }
    } else {
      int64_t rem = i;
      for (int d = 0; d < A.ndim; ++d) {
        const int64_t q = rem / A.sizes[d];
        const int64_t idx = rem - q * A.sizes[d];
        rem = q;
#pragma unroll
        for (int t = 0; t < 4; ++t) off[t] += idx * A.strides[t][d];
      }
    }
    C in[3] = {(C)0, (C)0, (C)0};
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      if (k < A.n_in) {
        if ((A.scalar_mask >> k) & 1) in[k] = (C)A.s[k];
        else in[k] = load_as<C>(A.ptr[k + 1] + off[k + 1], A.dtype[k + 1]);
      }
    }
    const C r = apply<C, INT>(A.op, in[0], in[1], in[2], A.p0, A.p1);
    store_from<C>(A.ptr[0] + off[0], A.dtype[0], r);
  }
}

int elem_bytes(int dt) {
  switch (dt) {
    case B200_F32: case B200_I32: return 4;
    case B200_BF16: case B200_F16: case B200_I16: return 2;
    case B200_F64: case B200_I64: return 8;
    case B200_U8: case B200_BOOL: case B200_I8: return 1;
    default: return 0;
  }
}
bool is_float_dt(int dt) { return dt == B200_F32 || dt == B200_BF16 || dt == B200_F16 || dt == B200_F64; }

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200_ew(int op, const b200_ew_t* d, cudaStream_t stream) {
  if (!d || d->ndim < 1 || d->ndim > 8 || d->n_in < 0 || d->n_in > 3) return (int)cudaErrorInvalidValue;
  EwArgs A{};
  A.ndim = d->ndim;
  A.n_in = d->n_in;
  A.op = op;
  int64_t numel = 1;
  for (int i = 0; i < d->ndim; ++i) {
    if (d->sizes[i] < 0) return (int)cudaErrorInvalidValue;
    numel *= d->sizes[i];
  }
  if (numel == 0) return 0;
  bool any_f64 = false, any_float = false;
  for (int t = 0; t <= d->n_in; ++t) {
    const bool scalar = t > 0 && ((d->scalar_mask >> (t - 1)) & 1);
    if (scalar) {
      A.dtype[t] = B200_F64;
      A.ptr[t] = nullptr;
      continue;
    }
    const int eb = elem_bytes(d->dtype[t]);
    if (!eb || !d->ptr[t]) return (int)cudaErrorNotSupported;
    A.dtype[t] = d->dtype[t];
    A.ptr[t] = static_cast<char*>(d->ptr[t]);
    for (int i = 0; i < d->ndim; ++i) A.strides[t][i] = d->strides[t][i] * eb;
    if (t > 0) {   // the compute type follows the inputs (comparisons write bool from floats)
      any_f64 |= d->dtype[t] == B200_F64;
      any_float |= is_float_dt(d->dtype[t]);
    }
  }
  if (d->n_in == 0 || d->float_compute) {
    any_float |= is_float_dt(d->dtype[0]) || d->float_compute;
    any_f64 |= d->dtype[0] == B200_F64;
  }
  for (int i = 0; i < d->ndim; ++i) {
    A.sizes[i] = d->sizes[i];
    A.div[i] = make_fastdiv((uint32_t)std::min<int64_t>(d->sizes[i], 0x7fffffff));
  }
  A.numel = numel;
  A.small_index = numel < (int64_t)0x7fffffff ? 1 : 0;
  for (int k = 0; k < 3; ++k) A.s[k] = d->scalar[k];
  A.p0 = d->p0;
  A.p1 = d->p1;
  A.scalar_mask = d->scalar_mask;
  const int64_t per_block = (int64_t)kEwThreads * kPerThread;
  const int64_t blocks = cdiv(numel, per_block);
  if (blocks > 2147483647ll) return (int)cudaErrorNotSupported;
  if (any_f64) ew_kernel<double, false><<<(unsigned)blocks, kEwThreads, 0, stream>>>(A);
  else if (any_float) ew_kernel<float, false><<<(unsigned)blocks, kEwThreads, 0, stream>>>(A);
  else ew_kernel<int64_t, true><<<(unsigned)blocks, kEwThreads, 0, stream>>>(A);
  B200K_LAUNCH_RET();
}
