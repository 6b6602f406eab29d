// General reductions over a contiguous input viewed as [outer, reduce, inner]:
//   inner == 1   rows: one warp per short row, one CTA per long row (16-byte loads), and for few very long rows a
//                split of every row over many CTAs with a second pass over the partial states;
//   inner  > 1   columns: threads run along `inner` (coalesced), each loops over `reduce`; when outer * inner is too
//                small to fill the 148 SMs the reduce range is split over blockIdx.y, again with a second pass.
// An operator is a small functor over a state: plain accumulators (sum, product, max, min, any, all, sum of squares,
// sum of |x|, max |x|), value + index pairs (argmax / argmin, max / min with indices, NaN wins as in torch) and the
// (sum, sum of squares) pair in fp64 that gives variance and standard deviation in one pass.
// Accumulation: fp32 for the 16/32-bit floating types, fp64 for doubles and variance, int64 for integers.
// Parity: reference torch_musa/csrc/aten/ops/musa/Reduce.muh:92-227 (a port of ATen's reduce_kernel).
#include "common.cuh"

#include <cfloat>

namespace b200k {
namespace {

constexpr int kRedThreads = 256;

template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };
template <> struct AccOf<int32_t> { using type = int64_t; };
template <> struct AccOf<int64_t> { using type = int64_t; };
template <> struct AccOf<uint8_t> { using type = int64_t; };
template <> struct AccOf<int8_t> { using type = int64_t; };
template <> struct AccOf<int16_t> { using type = int64_t; };
template <> struct AccOf<bool> { using type = int64_t; };

template <typename T, typename A> __device__ __forceinline__ A to_acc(T v) { return (A)v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half, float>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ double to_acc<__nv_bfloat16, double>(__nv_bfloat16 v) { return (double)__bfloat162float(v); }
template <> __device__ __forceinline__ double to_acc<__half, double>(__half v) { return (double)__half2float(v); }

template <typename A> __device__ __forceinline__ bool is_nan(A v) { return v != v; }

// ---- operator functors: State, init(), step(state, value, index), merge(a, b)
template <typename A> struct OpSum {
  using State = A;
  static __device__ __forceinline__ State init() { return (A)0; }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s += v; }
  static __device__ __forceinline__ State merge(State a, State b) { return a + b; }
};
template <typename A> struct OpProd {
  using State = A;
  static __device__ __forceinline__ State init() { return (A)1; }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s *= v; }
  static __device__ __forceinline__ State merge(State a, State b) { return a * b; }
};
template <typename A> struct OpSumSq {
  using State = A;
  static __device__ __forceinline__ State init() { return (A)0; }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s += v * v; }
  static __device__ __forceinline__ State merge(State a, State b) { return a + b; }
};
template <typename A> struct OpSumAbs {
  using State = A;
  static __device__ __forceinline__ State init() { return (A)0; }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s += v < (A)0 ? -v : v; }
  static __device__ __forceinline__ State merge(State a, State b) { return a + b; }
};
template <typename A> struct Limits;
template <> struct Limits<float> { static __device__ __forceinline__ float lowest() { return -INFINITY; } static __device__ __forceinline__ float highest() { return INFINITY; } };
template <> struct Limits<double> { static __device__ __forceinline__ double lowest() { return -INFINITY; } static __device__ __forceinline__ double highest() { return INFINITY; } };
template <> struct Limits<int64_t> { static __device__ __forceinline__ int64_t lowest() { return INT64_MIN; } static __device__ __forceinline__ int64_t highest() { return INT64_MAX; } };
template <typename A> struct OpMax {
  using State = A;
  static __device__ __forceinline__ State init() { return Limits<A>::lowest(); }
  static __device__ __forceinline__ State merge(State a, State b) { return (is_nan(a) || a > b) ? a : (is_nan(b) ? b : (a > b ? a : b)); }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s = merge(s, v); }
};
template <typename A> struct OpMin {
  using State = A;
  static __device__ __forceinline__ State init() { return Limits<A>::highest(); }
  static __device__ __forceinline__ State merge(State a, State b) { return (is_nan(a) || a < b) ? a : (is_nan(b) ? b : (a < b ? a : b)); }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s = merge(s, v); }
};
template <typename A> struct OpAbsMax {
  using State = A;
  static __device__ __forceinline__ State init() { return (A)0; }
  static __device__ __forceinline__ State merge(State a, State b) { return OpMax<A>::merge(a, b); }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s = merge(s, v < (A)0 ? -v : v); }
};
template <typename A> struct OpAny {
  using State = A;
  static __device__ __forceinline__ State init() { return (A)0; }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s = (s != (A)0 || v != (A)0) ? (A)1 : (A)0; }
  static __device__ __forceinline__ State merge(State a, State b) { return (a != (A)0 || b != (A)0) ? (A)1 : (A)0; }
};
template <typename A> struct OpAll {
  using State = A;
  static __device__ __forceinline__ State init() { return (A)1; }
  static __device__ __forceinline__ void step(State& s, A v, int64_t) { s = (s != (A)0 && v != (A)0) ? (A)1 : (A)0; }
  static __device__ __forceinline__ State merge(State a, State b) { return (a != (A)0 && b != (A)0) ? (A)1 : (A)0; }
};
template <typename A> struct ValIdx { A v; int64_t i; };
template <typename A, bool MAX> struct OpArg {
  using State = ValIdx<A>;
  static __device__ __forceinline__ State init() { return State{MAX ? Limits<A>::lowest() : Limits<A>::highest(), INT64_MAX}; }
  // NaN beats everything; between equal values (or two NaNs) the smaller index wins
  static __device__ __forceinline__ State merge(State a, State b) {
    const bool an = is_nan(a.v), bn = is_nan(b.v);
    if (an || bn) {
      if (an && bn) return a.i <= b.i ? a : b;
      return an ? a : b;
    }
    if (a.v == b.v) return a.i <= b.i ? a : b;
    return (MAX ? a.v > b.v : a.v < b.v) ? a : b;
  }
  static __device__ __forceinline__ void step(State& s, A v, int64_t i) { s = merge(s, State{v, i}); }
};
struct SumSq2 { double s, q; };
struct OpVar {   // sum and sum of squares in fp64
  using State = SumSq2;
  static __device__ __forceinline__ State init() { return State{0.0, 0.0}; }
  static __device__ __forceinline__ void step(State& s, double v, int64_t) { s.s += v; s.q += v * v; }
  static __device__ __forceinline__ State merge(State a, State b) { return State{a.s + b.s, a.q + b.q}; }
};

template <typename S> __device__ __forceinline__ S shfl_down_state(S s, int off) {
  constexpr int N = (sizeof(S) + 3) / 4;
  union { S s; uint32_t w[N]; } u;
  u.s = s;
#pragma unroll
  for (int i = 0; i < N; ++i) u.w[i] = __shfl_down_sync(0xffffffffu, u.w[i], off);
  return u.s;
}
template <typename Op> __device__ __forceinline__ typename Op::State warp_reduce(typename Op::State s) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s = Op::merge(s, shfl_down_state(s, off));
  return s;
}
template <typename Op> __device__ __forceinline__ typename Op::State block_reduce(typename Op::State s, typename Op::State* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  s = warp_reduce<Op>(s);
  __syncthreads();
  if (lane == 0) sh[w] = s;
  __syncthreads();
  if (w == 0) {
    s = lane < nw ? sh[lane] : Op::init();
    s = warp_reduce<Op>(s);
  }
  return s;   // valid in thread 0
}

struct Finish {
  int mode;        // 0 plain, 1 scale by p0, 2 sqrt, 3 variance (p0 = correction, p1 = count), 4 std
  double p0, p1;
};
template <typename A> __device__ __forceinline__ A finish_scalar(A v, const Finish& f) {
  if (f.mode == 1) return (A)((double)v * f.p0);
  if (f.mode == 2) return (A)sqrt((double)v);
  return v;
}

// result writers ------------------------------------------------------------------------------------------------
template <typename TO, typename A> __device__ __forceinline__ void write_val(TO* out, int64_t i, A v) { out[i] = (TO)v; }
template <> __device__ __forceinline__ void write_val<__nv_bfloat16, float>(__nv_bfloat16* out, int64_t i, float v) { out[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void write_val<__half, float>(__half* out, int64_t i, float v) { out[i] = __float2half_rn(v); }
template <> __device__ __forceinline__ void write_val<__nv_bfloat16, double>(__nv_bfloat16* out, int64_t i, double v) { out[i] = __float2bfloat16_rn((float)v); }
template <> __device__ __forceinline__ void write_val<__half, double>(__half* out, int64_t i, double v) { out[i] = __float2half_rn((float)v); }
template <> __device__ __forceinline__ void write_val<bool, int64_t>(bool* out, int64_t i, int64_t v) { out[i] = v != 0; }

template <typename Op, typename TO, typename A>
struct Writer {
  static __device__ __forceinline__ void put(typename Op::State s, TO* out, int64_t* out_idx, int64_t i, const Finish& f) {
    write_val<TO, A>(out, i, finish_scalar<A>(s, f));
  }
};
template <typename TO, typename A, bool MAX>
struct Writer<OpArg<A, MAX>, TO, A> {
  static __device__ __forceinline__ void put(ValIdx<A> s, TO* out, int64_t* out_idx, int64_t i, const Finish&) {
    if (out) write_val<TO, A>(out, i, s.v);
    if (out_idx) out_idx[i] = s.i == INT64_MAX ? 0 : s.i;
  }
};
template <typename TO>
struct Writer<OpVar, TO, double> {
  static __device__ __forceinline__ void put(SumSq2 s, TO* out, int64_t*, int64_t i, const Finish& f) {
    const double n = f.p1;
    double var = (s.q - s.s * s.s / n) / fmax(n - f.p0, 0.0);
    if (var < 0.0) var = 0.0;
    if (!(n - f.p0 > 0.0)) var = NAN;
    write_val<TO, double>(out, i, f.mode == 4 ? sqrt(var) : var);
  }
};

// ---- kernels: `in` is either the typed input (FIRST pass) or an array of states (second pass over partials)
template <typename Op, typename T, typename A, bool FROM_STATE>
__device__ __forceinline__ void accumulate(typename Op::State& s, const void* in, int64_t off, int64_t index) {
  if constexpr (FROM_STATE) s = Op::merge(s, static_cast<const typename Op::State*>(in)[off]);
  else Op::step(s, to_acc<T, A>(static_cast<const T*>(in)[off]), index);
}

// rows (inner == 1): grid.x = rows (or rows * splits), one CTA per (row, split); splits > 1 writes states
template <typename Op, typename T, typename TO, typename A, bool FROM_STATE, bool TO_STATE>
__global__ void __launch_bounds__(kRedThreads) reduce_rows_kernel(const void* __restrict__ in, TO* __restrict__ out,
                                                                  int64_t* __restrict__ out_idx,
                                                                  typename Op::State* __restrict__ partial, int64_t R,
                                                                  int splits, Finish f) {
  __shared__ typename Op::State sh[kRedThreads / 32];
  const int64_t row = blockIdx.x / splits;
  const int split = (int)(blockIdx.x % splits);
  const int64_t chunk = (R + splits - 1) / splits;
  const int64_t r0 = split * chunk, r1 = min(R, r0 + chunk);
  typename Op::State s = Op::init();
  for (int64_t r = r0 + threadIdx.x; r < r1; r += kRedThreads) accumulate<Op, T, A, FROM_STATE>(s, in, row * R + r, r);
  s = block_reduce<Op>(s, sh);
  if (threadIdx.x == 0) {
    if constexpr (TO_STATE) partial[row * splits + split] = s;
    else Writer<Op, TO, A>::put(s, out, out_idx, row, f);
  }
}

// rows, one warp per row (short rows, many of them)
template <typename Op, typename T, typename TO, typename A>
__global__ void __launch_bounds__(kRedThreads) reduce_rows_warp_kernel(const void* __restrict__ in, TO* __restrict__ out,
                                                                       int64_t* __restrict__ out_idx, int64_t rows,
                                                                       int64_t R, Finish f) {
  const int64_t row = (int64_t)blockIdx.x * (kRedThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  typename Op::State s = Op::init();
  for (int64_t r = lane; r < R; r += 32) accumulate<Op, T, A, false>(s, in, row * R + r, r);
  s = warp_reduce<Op>(s);
  if (lane == 0) Writer<Op, TO, A>::put(s, out, out_idx, row, f);
}

// columns (inner > 1): thread = one (outer, inner) output; blockIdx.y splits the reduce range
template <typename Op, typename T, typename TO, typename A, bool FROM_STATE, bool TO_STATE>
__global__ void __launch_bounds__(kRedThreads) reduce_cols_kernel(const void* __restrict__ in, TO* __restrict__ out,
                                                                  int64_t* __restrict__ out_idx,
                                                                  typename Op::State* __restrict__ partial, int64_t outer,
                                                                  int64_t R, int64_t inner, int splits, Finish f) {
  const int64_t o = (int64_t)blockIdx.x * kRedThreads + threadIdx.x;
  if (o >= outer * inner) return;
  const int64_t oo = o / inner, ii = o - oo * inner;
  const int split = blockIdx.y;
  const int64_t chunk = (R + splits - 1) / splits;
  const int64_t r0 = split * chunk, r1 = min(R, r0 + chunk);
  typename Op::State s = Op::init();
  const int64_t base = oo * R * inner + ii;
  for (int64_t r = r0; r < r1; ++r) accumulate<Op, T, A, FROM_STATE>(s, in, base + r * inner, r);
  if constexpr (TO_STATE) partial[(oo * splits + split) * inner + ii] = s;
  else Writer<Op, TO, A>::put(s, out, out_idx, o, f);
}

template <typename Op, typename T, typename TO, typename A>
int launch_reduce(const b200_reduce_t* d, Finish f, cudaStream_t stream) {
  using State = typename Op::State;
  const int64_t outer = d->outer, R = d->reduce, inner = d->inner;
  TO* out = static_cast<TO*>(d->out);
  int64_t* oi = d->out_index;
  State* partial = static_cast<State*>(d->scratch);
  const int64_t n_out = outer * inner;
  if (n_out == 0) return 0;
  if (inner == 1) {
    if (R <= 1024 && outer >= 8 * kSMs) {
      const int64_t blocks = cdiv(outer, kRedThreads / 32);
      if (blocks > 2147483647ll) return (int)cudaErrorNotSupported;
      reduce_rows_warp_kernel<Op, T, TO, A><<<(unsigned)blocks, kRedThreads, 0, stream>>>(d->in, out, oi, outer, R, f);
      return 0;
    }
    int splits = 1;
    if (outer < 2 * kSMs && R > 16384) {
      splits = (int)std::min<int64_t>(cdiv(4 * kSMs, std::max<int64_t>(outer, 1)), cdiv(R, 4096));
      const int64_t cap = (int64_t)(d->scratch_bytes / sizeof(State)) / std::max<int64_t>(outer, 1);
      splits = (int)std::max<int64_t>(1, std::min<int64_t>(splits, cap));
    }
    if (outer * splits > 2147483647ll) return (int)cudaErrorNotSupported;
    if (splits == 1) {
      reduce_rows_kernel<Op, T, TO, A, false, false><<<(unsigned)outer, kRedThreads, 0, stream>>>(d->in, out, oi, nullptr, R, 1, f);
    } else {
      reduce_rows_kernel<Op, T, TO, A, false, true><<<(unsigned)(outer * splits), kRedThreads, 0, stream>>>(d->in, out, oi, partial, R, splits, f);
      note_launch();
      reduce_rows_kernel<Op, T, TO, A, true, false><<<(unsigned)outer, kRedThreads, 0, stream>>>(partial, out, oi, nullptr, splits, 1, f);
    }
    return 0;
  }
  const int64_t blocks_x = cdiv(n_out, kRedThreads);
  if (blocks_x > 2147483647ll) return (int)cudaErrorNotSupported;
  int splits = 1;
  if (blocks_x < 2 * kSMs && R >= 64) {
    splits = (int)std::min<int64_t>(cdiv(4 * kSMs, blocks_x), R / 16);
    const int64_t cap = (int64_t)(d->scratch_bytes / sizeof(State)) / std::max<int64_t>(n_out, 1);
    splits = (int)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(splits, cap), 65535));
  }
  if (splits == 1) {
    reduce_cols_kernel<Op, T, TO, A, false, false><<<dim3((unsigned)blocks_x, 1), kRedThreads, 0, stream>>>(d->in, out, oi, nullptr, outer, R, inner, 1, f);
  } else {
    reduce_cols_kernel<Op, T, TO, A, false, true><<<dim3((unsigned)blocks_x, (unsigned)splits), kRedThreads, 0, stream>>>(d->in, out, oi, partial, outer, R, inner, splits, f);
    note_launch();
    reduce_cols_kernel<Op, T, TO, A, true, false><<<dim3((unsigned)blocks_x, 1), kRedThreads, 0, stream>>>(partial, out, oi, nullptr, outer, splits, inner, 1, f);
  }
  return 0;
}

// which operators exist for which (input, output) pairs is decided here, to keep the number of kernels bounded:
//   floating inputs   every arithmetic operator, output = input type (or fp32 for the 16-bit types)
//   integer inputs    sum / prod into int64; amax / amin / argmax / argmin in the input type
//   any / all         every input type into bool (uint8 for uint8 inputs)
//   var / std         floating inputs, output = input type
template <typename T, typename TO>
int dispatch_float(const b200_reduce_t* d, cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  Finish f{0, d->p0, d->p1};
  switch (d->op) {
    case B200_RD_SUM: return launch_reduce<OpSum<A>, T, TO, A>(d, f, stream);
    case B200_RD_MEAN: f.mode = 1; return launch_reduce<OpSum<A>, T, TO, A>(d, f, stream);
    case B200_RD_PROD: return launch_reduce<OpProd<A>, T, TO, A>(d, f, stream);
    case B200_RD_AMAX: return launch_reduce<OpMax<A>, T, TO, A>(d, f, stream);
    case B200_RD_AMIN: return launch_reduce<OpMin<A>, T, TO, A>(d, f, stream);
    case B200_RD_SUMSQ: return launch_reduce<OpSumSq<A>, T, TO, A>(d, f, stream);
    case B200_RD_NORM2: f.mode = 2; return launch_reduce<OpSumSq<A>, T, TO, A>(d, f, stream);
    case B200_RD_SUMABS: return launch_reduce<OpSumAbs<A>, T, TO, A>(d, f, stream);
    case B200_RD_ABSMAX: return launch_reduce<OpAbsMax<A>, T, TO, A>(d, f, stream);
    default: return (int)cudaErrorNotSupported;
  }
}
template <typename T>
int dispatch_arg(const b200_reduce_t* d, cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  Finish f{0, 0.0, 0.0};
  if (d->op == B200_RD_ARGMAX) return launch_reduce<OpArg<A, true>, T, T, A>(d, f, stream);
  return launch_reduce<OpArg<A, false>, T, T, A>(d, f, stream);
}
template <typename T>
int dispatch_int(const b200_reduce_t* d, cudaStream_t stream) {
  Finish f{0, 0.0, 0.0};
  switch (d->op) {
    case B200_RD_SUM: return d->out_dtype == B200_I64 ? launch_reduce<OpSum<int64_t>, T, int64_t, int64_t>(d, f, stream) : (int)cudaErrorNotSupported;
    case B200_RD_PROD: return d->out_dtype == B200_I64 ? launch_reduce<OpProd<int64_t>, T, int64_t, int64_t>(d, f, stream) : (int)cudaErrorNotSupported;
    case B200_RD_AMAX: return d->out_dtype == d->in_dtype ? launch_reduce<OpMax<int64_t>, T, T, int64_t>(d, f, stream) : (int)cudaErrorNotSupported;
    case B200_RD_AMIN: return d->out_dtype == d->in_dtype ? launch_reduce<OpMin<int64_t>, T, T, int64_t>(d, f, stream) : (int)cudaErrorNotSupported;
    default: return (int)cudaErrorNotSupported;
  }
}
template <typename T, typename TO>
int dispatch_bool(const b200_reduce_t* d, cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  Finish f{0, 0.0, 0.0};
  if (d->op == B200_RD_ANY) return launch_reduce<OpAny<A>, T, TO, A>(d, f, stream);
  return launch_reduce<OpAll<A>, T, TO, A>(d, f, stream);
}
template <typename T>
int dispatch_var(const b200_reduce_t* d, cudaStream_t stream) {
  Finish f{d->op == B200_RD_STD ? 4 : 3, d->p0, (double)d->reduce};
  return launch_reduce<OpVar, T, T, double>(d, f, stream);
}

template <typename T, bool FLOATING>
int dispatch_type(const b200_reduce_t* d, int code, cudaStream_t stream) {
  const bool var = d->op == B200_RD_VAR || d->op == B200_RD_STD;
  const bool boolean = d->op == B200_RD_ANY || d->op == B200_RD_ALL;
  const bool arg = d->op == B200_RD_ARGMAX || d->op == B200_RD_ARGMIN;
  if (boolean) {
    if (d->out_dtype == B200_BOOL) return dispatch_bool<T, bool>(d, stream);
    if constexpr (std::is_same<T, uint8_t>::value)
      if (d->out_dtype == B200_U8) return dispatch_bool<T, uint8_t>(d, stream);
    return (int)cudaErrorNotSupported;
  }
  if (arg) return (!d->out || d->out_dtype == code) ? dispatch_arg<T>(d, stream) : (int)cudaErrorNotSupported;
  if constexpr (FLOATING) {
    if (var) return d->out_dtype == code ? dispatch_var<T>(d, stream) : (int)cudaErrorNotSupported;
    if (d->out_dtype == code) return dispatch_float<T, T>(d, stream);
    if constexpr (sizeof(T) == 2)
      if (d->out_dtype == B200_F32) return dispatch_float<T, float>(d, stream);
    return (int)cudaErrorNotSupported;
  } else {
    if (var) return (int)cudaErrorNotSupported;
    return dispatch_int<T>(d, stream);
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" size_t b200_reduce_state_bytes(void) { return sizeof(ValIdx<double>); }

extern "C" int b200_reduce(const b200_reduce_t* d, cudaStream_t stream) {
  if (!d || d->outer < 0 || d->reduce < 0 || d->inner < 0) return (int)cudaErrorInvalidValue;
  int e;
  switch (d->in_dtype) {
    case B200_F32: e = dispatch_type<float, true>(d, B200_F32, stream); break;
    case B200_BF16: e = dispatch_type<__nv_bfloat16, true>(d, B200_BF16, stream); break;
    case B200_F16: e = dispatch_type<__half, true>(d, B200_F16, stream); break;
    case B200_F64: e = dispatch_type<double, true>(d, B200_F64, stream); break;
    case B200_I64: e = dispatch_type<int64_t, false>(d, B200_I64, stream); break;
    case B200_I32: e = dispatch_type<int32_t, false>(d, B200_I32, stream); break;
    case B200_U8: e = dispatch_type<uint8_t, false>(d, B200_U8, stream); break;
    case B200_BOOL: e = dispatch_type<bool, false>(d, B200_BOOL, stream); break;
    case B200_I8: e = dispatch_type<int8_t, false>(d, B200_I8, stream); break;
    case B200_I16: e = dispatch_type<int16_t, false>(d, B200_I16, stream); break;
    default: e = (int)cudaErrorNotSupported;
  }
  if (e != 0) return e;
  B200K_LAUNCH_RET();
}
