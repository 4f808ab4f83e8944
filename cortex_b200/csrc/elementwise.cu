// assign! / unary-op! / binary-op! families: the B200 replacement of the
// reference's generic one-element-per-thread kernels
// (resources/tensor_assign.cu, tensor_unary_op.cu, tensor_binary_op*.cu,
//  tensor_binary_accum.cu, tensor_accum_constant.cu, memset.cu).
//
// Three kernels, chosen on the host from the operand descriptors:
//   ew_flat    every operand is dense and either full-size, a repeating
//              suffix (bias row over a matrix) or a single broadcast axis
//              (channel bias over NCHW); 128-bit accesses, 4 chunks in flight
//              per thread.
//   ew_rowvec  the fastest-changing dimension is contiguous for every operand;
//              the outer dimensions go through the general index system
//              (pitched sub-matrix views, row gathers through index arrays).
//   ew_generic the reference's general index system, one element at a time.
// HBM-bound: algorithmic bytes = sum over operands of bytes touched once.
#include "common.cuh"
#include <math.h>

namespace {

// ------------------------------ op semantics -------------------------------
// Restates perform-operation-impl / perform-unary-op-impl
// (src/cortex/compute/cpu/tensor_math.clj:211-223, 278-308).

__device__ __forceinline__ double bin_apply(int op, double a, double b) {
  switch (op) {
    case CB200_ADD: return a + b;
    case CB200_SUB: return a - b;
    case CB200_MUL: return a * b;
    case CB200_DIV: return a / b;
    case CB200_MAX: return a > b ? a : b;
    case CB200_MIN: return a > b ? b : a;
    case CB200_BIT_AND: return (double)(jvm_d2i(a) & jvm_d2i(b));
    case CB200_BIT_XOR: return (double)(jvm_d2i(a) ^ jvm_d2i(b));
    case CB200_EQ: return a == b ? 1.0 : 0.0;
    case CB200_GT: return a > b ? 1.0 : 0.0;
    case CB200_GE: return a >= b ? 1.0 : 0.0;
    case CB200_LT: return a < b ? 1.0 : 0.0;
    case CB200_LE: return a <= b ? 1.0 : 0.0;
  }
  return 0.0;
}

__device__ __forceinline__ long long bin_apply(int op, long long a, long long b) {
  typedef unsigned long long u64;
  switch (op) {
    case CB200_ADD: return (long long)((u64)a + (u64)b);
    case CB200_SUB: return (long long)((u64)a - (u64)b);
    case CB200_MUL: return (long long)((u64)a * (u64)b);
    case CB200_DIV:
      if (b == 0) return 0;  // the reference throws ArithmeticException here
      if (b == -1) return (long long)(0ull - (u64)a);
      return a / b;
    case CB200_MAX: return a > b ? a : b;
    case CB200_MIN: return a > b ? b : a;
    case CB200_BIT_AND: return (long long)((int)a & (int)b);
    case CB200_BIT_XOR: return (long long)((int)a ^ (int)b);
    case CB200_EQ: return a == b;
    case CB200_GT: return a > b;
    case CB200_GE: return a >= b;
    case CB200_LT: return a < b;
    case CB200_LE: return a <= b;
  }
  return 0;
}

__device__ __forceinline__ long long jvm_round(double a) {
  if (a != a) return 0;
  double r = floor(a);
  if (a - r >= 0.5) r += 1.0;
  return jvm_d2l(r);
}

// Unary result is a double except :round (long) and :- on integer views (long).
template <typename T>
__device__ __forceinline__ T unary_apply(int op, typename acc_of<T>::type v) {
  double d = (double)v;
  switch (op) {
    case CB200_FLOOR: return store_as<T>::from(floor(d));
    case CB200_CEIL: return store_as<T>::from(ceil(d));
    case CB200_ROUND: return store_as<T>::from(jvm_round(d));
    case CB200_NEG: return store_as<T>::from((typename acc_of<T>::type)(-v));
    case CB200_TANH: return store_as<T>::from(tanh(d));
    case CB200_LOGISTIC: return store_as<T>::from(1.0 / (1.0 + exp(-d)));
    case CB200_EXP: return store_as<T>::from(exp(d));
    case CB200_SQRT: return store_as<T>::from(sqrt(d));
    case CB200_NOOP: return store_as<T>::from(d);
  }
  return (T)0;
}

// fp32 views evaluate the transcendental ops in single precision (<= 2 ulp of
// the double-evaluated value, far inside the 1e-4 parity bound) so that these
// kernels stay HBM-bound.
template <>
__device__ __forceinline__ float unary_apply<float>(int op, double v) {
  switch (op) {
    case CB200_FLOOR: return (float)floor(v);
    case CB200_CEIL: return (float)ceil(v);
    case CB200_ROUND: return (float)jvm_round(v);
    case CB200_NEG: return (float)(-v);
    case CB200_TANH: return tanhf((float)v);
    case CB200_LOGISTIC: return 1.0f / (1.0f + expf(-(float)v));
    case CB200_EXP: return expf((float)v);
    case CB200_SQRT: return (float)sqrt(v);
    case CB200_NOOP: return (float)v;
  }
  return 0.f;
}

// Functors.  x is the first input (or the old dest value for accum forms),
// y the second.  NIN = number of tensor inputs read.
template <typename TD, typename TS>
struct AssignF {
  static const int NIN = 1;
  typedef TS TX;
  __device__ __forceinline__ TD operator()(TS x, TS) const {
    return store_as<TD>::from((typename acc_of<TS>::type)x);
  }
};

template <typename T>
struct FillF {
  static const int NIN = 0;
  typedef T TX;
  T value;
  __device__ __forceinline__ T operator()(T, T) const { return value; }
};

template <typename T>
struct UnaryF {
  static const int NIN = 1;
  typedef T TX;
  typedef typename acc_of<T>::type A;
  int op;
  A alpha;
  __device__ __forceinline__ T operator()(T x, T) const { return unary_apply<T>(op, (A)((A)x * alpha)); }
};

// float views: a float*float product is exact in double and every basic operation on two
// floats gives the same result whether it is rounded once from double or done in single
// precision (53 >= 2*24 + 2), so with alpha == 1 the whole op runs in fp32, bit-identically,
// and stays clear of the slow f32<->f64 conversion pipe.
__device__ __forceinline__ float bin_apply_f32(int op, float a, float b) {
  switch (op) {
    case CB200_ADD: return a + b;
    case CB200_SUB: return a - b;
    case CB200_MUL: return a * b;
    case CB200_DIV: return __fdiv_rn(a, b);
    case CB200_MAX: return a > b ? a : b;
    case CB200_MIN: return a > b ? b : a;
    case CB200_EQ: return a == b ? 1.f : 0.f;
    case CB200_GT: return a > b ? 1.f : 0.f;
    case CB200_GE: return a >= b ? 1.f : 0.f;
    case CB200_LT: return a < b ? 1.f : 0.f;
    case CB200_LE: return a <= b ? 1.f : 0.f;
  }
  return (float)bin_apply(op, (double)a, (double)b);
}

template <>
struct UnaryF<float> {
  static const int NIN = 1;
  typedef float TX;
  int op;
  double alpha;
  __device__ __forceinline__ float operator()(float x, float) const {
    if (alpha == 1.0) {
      switch (op) {
        case CB200_FLOOR: return floorf(x);
        case CB200_CEIL: return ceilf(x);
        case CB200_NEG: return -x;
        case CB200_TANH: return tanhf(x);
        case CB200_LOGISTIC: return 1.0f / (1.0f + expf(-x));
        case CB200_EXP: return expf(x);
        case CB200_SQRT: return __fsqrt_rn(x);
        case CB200_NOOP: return x;
      }
    }
    return unary_apply<float>(op, (double)x * alpha);
  }
};

template <typename T>
struct BinaryConstF {
  static const int NIN = 1;
  typedef T TX;
  typedef typename acc_of<T>::type A;
  int op;
  int rev;
  A alpha, scalar;
  __device__ __forceinline__ T operator()(T x, T) const {
    A a = (A)x * alpha;
    A r = rev ? bin_apply(op, scalar, a) : bin_apply(op, a, scalar);
    return store_as<T>::from(r);
  }
};

template <>
struct BinaryConstF<float> {
  static const int NIN = 1;
  typedef float TX;
  int op;
  int rev;
  double alpha, scalar;   // scalar was cast to float first, so (float)scalar is exact
  __device__ __forceinline__ float operator()(float x, float) const {
    if (alpha == 1.0) {
      const float sc = (float)scalar;
      return rev ? bin_apply_f32(op, sc, x) : bin_apply_f32(op, x, sc);
    }
    double a = (double)x * alpha;
    return (float)(rev ? bin_apply(op, scalar, a) : bin_apply(op, a, scalar));
  }
};

template <typename T>
struct BinaryF {
  static const int NIN = 2;
  typedef T TX;
  typedef typename acc_of<T>::type A;
  int op;
  int rev;
  A xa, ya;
  __device__ __forceinline__ T operator()(T x, T y) const {
    A a = (A)x * xa, b = (A)y * ya;
    A r = rev ? bin_apply(op, b, a) : bin_apply(op, a, b);
    return store_as<T>::from(r);
  }
};

template <>
struct BinaryF<float> {
  static const int NIN = 2;
  typedef float TX;
  int op;
  int rev;
  double xa, ya;
  __device__ __forceinline__ float operator()(float x, float y) const {
    if (xa == 1.0 && ya == 1.0) return rev ? bin_apply_f32(op, y, x) : bin_apply_f32(op, x, y);
    if (xa == 1.0 && ya == -1.0 && op == CB200_ADD) return rev ? (-y) + x : x - y;   // binary-op! :- arrives as :+ with -beta
    double a = (double)x * xa, b = (double)y * ya;
    return (float)(rev ? bin_apply(op, b, a) : bin_apply(op, a, b));
  }
};

// fp32, unit scale factors, operation fixed at compile time: what the dense layers issue
// (bias add, ReLU as max with 0, softmax's subtract / divide).  Same values as the generic
// functors above; the kernels they instantiate are a handful of instructions per element.
template <int OP> __device__ __forceinline__ float f32_op(float a, float b);
template <> __device__ __forceinline__ float f32_op<CB200_ADD>(float a, float b) { return a + b; }
template <> __device__ __forceinline__ float f32_op<CB200_SUB>(float a, float b) { return a - b; }
template <> __device__ __forceinline__ float f32_op<CB200_MUL>(float a, float b) { return a * b; }
template <> __device__ __forceinline__ float f32_op<CB200_DIV>(float a, float b) { return __fdiv_rn(a, b); }
template <> __device__ __forceinline__ float f32_op<CB200_MAX>(float a, float b) { return a > b ? a : b; }
template <> __device__ __forceinline__ float f32_op<CB200_MIN>(float a, float b) { return a > b ? b : a; }

template <int OP>
struct FastBinaryF {
  static const int NIN = 2;
  typedef float TX;
  __device__ __forceinline__ float operator()(float x, float y) const { return f32_op<OP>(x, y); }
};
template <int OP, int REV>
struct FastBinaryConstF {
  static const int NIN = 1;
  typedef float TX;
  float scalar;
  __device__ __forceinline__ float operator()(float x, float) const {
    return REV ? f32_op<OP>(scalar, x) : f32_op<OP>(x, scalar);
  }
};

// ------------------------------ kernels -------------------------------------

template <typename T, int N>
struct alignas(sizeof(T) * N) Vec { T v[N]; };

// Element counts are 32-bit, as in the reference (int n_elems in every kernel), so the
// index arithmetic below stays in 32-bit registers.
struct FlatMode {   // address of element i:  kind 0: i   1: i % ec   2: ((i / amt) % ec) * stride
  int kind;
  int stride;
  unsigned ec;
  unsigned amt;
};

template <typename T, int VEC>
__device__ __forceinline__ void flat_load(const T* p, const FlatMode& m, unsigned i0, bool vec_ok, T (&out)[VEC]) {
  if (m.kind == 0 || m.kind == 1) {
    unsigned a = m.kind == 0 ? i0 : (i0 % m.ec);
    if (vec_ok) {
      Vec<T, VEC> v = *reinterpret_cast<const Vec<T, VEC>*>(p + a);
#pragma unroll
      for (int k = 0; k < VEC; ++k) out[k] = v.v[k];
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) out[k] = p[m.kind == 0 ? (i0 + k) : ((i0 + k) % m.ec)];
    }
  } else {
    if (vec_ok) {
      T v = p[(size_t)((i0 / m.amt) % m.ec) * m.stride];
#pragma unroll
      for (int k = 0; k < VEC; ++k) out[k] = v;
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) out[k] = p[(size_t)(((i0 + k) / m.amt) % m.ec) * m.stride];
    }
  }
}

// dest is dense and full-size.  n_vec = n / VEC full chunks; the tail is done scalar by the
// first threads.  xv / yv say whether the input admits one vector (or one broadcast scalar)
// access per chunk.  Grid-stride: the grid is sized to fill every SM once, each thread keeps
// UNROLL independent 16-byte loads in flight per operand.
template <typename TD, typename F, int VEC, int UNROLL>
__global__ void __launch_bounds__(256)
ew_flat(TD* dest, const typename F::TX* x, const typename F::TX* y,
        FlatMode mx, FlatMode my, int xv, int yv, unsigned n, F f) {
  typedef typename F::TX TX;
  const unsigned n_vec = n / VEC;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned base = blockIdx.x * blockDim.x + threadIdx.x; base < n_vec; base += stride * UNROLL) {
    TX xs[UNROLL][VEC], ys[UNROLL][VEC];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      unsigned c = base + u * stride;
      if (c < n_vec) {
        if (F::NIN >= 1) flat_load<TX, VEC>(x, mx, c * VEC, xv != 0, xs[u]);
        if (F::NIN >= 2) flat_load<TX, VEC>(y, my, c * VEC, yv != 0, ys[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      unsigned c = base + u * stride;
      if (c < n_vec) {
        Vec<TD, VEC> o;
#pragma unroll
        for (int k = 0; k < VEC; ++k)
          o.v[k] = f(F::NIN >= 1 ? xs[u][k] : TX(), F::NIN >= 2 ? ys[u][k] : TX());
        *reinterpret_cast<Vec<TD, VEC>*>(dest + (size_t)c * VEC) = o;
      }
    }
  }
  // scalar tail
  unsigned t = n_vec * VEC + threadIdx.x;
  if (blockIdx.x == 0 && t < n) {
    TX xe = TX(), ye = TX();
    if (F::NIN >= 1) { TX tmp[1]; flat_load<TX, 1>(x, mx, t, false, tmp); xe = tmp[0]; }
    if (F::NIN >= 2) { TX tmp[1]; flat_load<TX, 1>(y, my, t, false, tmp); ye = tmp[0]; }
    dest[t] = f(xe, ye);
  }
}

// Fastest-changing dimension contiguous (or broadcast) for every operand.
// One thread = one VEC-wide chunk of a row; outer coordinates go through the
// general index system (dims 1..4).  row_mode: 1 = contiguous, 0 = broadcast.
template <typename TD, typename F, int VEC>
__global__ void __launch_bounds__(256)
ew_rowvec(TD* dest, const typename F::TX* x, const typename F::TX* y,
          Operand od, Operand ox, Operand oy, Geometry g, int x_row, int y_row, unsigned n_chunks, F f) {
  typedef typename F::TX TX;
  constexpr int UNROLL = 4;
  const unsigned chunks_per_row = (unsigned)g.max_shape[0] / VEC;
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned base = blockIdx.x * blockDim.x + threadIdx.x; base < n_chunks; base += stride * UNROLL) {
    TX xs[UNROLL][VEC], ys[UNROLL][VEC];
    long long doff[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const unsigned c = base + u * stride;
      if (c < n_chunks) {
        const unsigned row = c / chunks_per_row;
        const unsigned col = (c - row * chunks_per_row) * VEC;
        const unsigned i = row * (unsigned)g.max_shape[0];
        doff[u] = operand_offset(od, g, i) + col;
        if (F::NIN >= 1) {
          const TX* p = x + operand_offset(ox, g, i);
          if (x_row) {
            Vec<TX, VEC> v = *reinterpret_cast<const Vec<TX, VEC>*>(p + col);
#pragma unroll
            for (int k = 0; k < VEC; ++k) xs[u][k] = v.v[k];
          } else {
            TX v = *p;
#pragma unroll
            for (int k = 0; k < VEC; ++k) xs[u][k] = v;
          }
        }
        if (F::NIN >= 2) {
          const TX* p = y + operand_offset(oy, g, i);
          if (y_row) {
            Vec<TX, VEC> v = *reinterpret_cast<const Vec<TX, VEC>*>(p + col);
#pragma unroll
            for (int k = 0; k < VEC; ++k) ys[u][k] = v.v[k];
          } else {
            TX v = *p;
#pragma unroll
            for (int k = 0; k < VEC; ++k) ys[u][k] = v;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const unsigned c = base + u * stride;
      if (c < n_chunks) {
        Vec<TD, VEC> o;
#pragma unroll
        for (int k = 0; k < VEC; ++k)
          o.v[k] = f(F::NIN >= 1 ? xs[u][k] : TX(), F::NIN >= 2 ? ys[u][k] : TX());
        *reinterpret_cast<Vec<TD, VEC>*>(dest + doff[u]) = o;
      }
    }
  }
}

// Same contract as ew_rowvec for long rows (>= 32 chunks): one warp per row.  The outer
// addressing (index-array lookups included) is resolved once per row instead of once per
// chunk, and each lane keeps 8 independent 16-byte loads in flight.
template <typename TD, typename F, int VEC>
__global__ void __launch_bounds__(256)
ew_rowwarp(TD* dest, const typename F::TX* x, const typename F::TX* y,
           Operand od, Operand ox, Operand oy, Geometry g, int x_row, int y_row, unsigned n_rows, F f) {
  typedef typename F::TX TX;
  constexpr int U = 8;
  const unsigned lane = threadIdx.x & 31;
  const unsigned chunks = (unsigned)g.max_shape[0] / VEC;
  const unsigned warps = gridDim.x * (blockDim.x >> 5);
  for (unsigned row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows; row += warps) {
    const unsigned i = row * (unsigned)g.max_shape[0];
    Vec<TD, VEC>* d = reinterpret_cast<Vec<TD, VEC>*>(dest + operand_offset(od, g, i));
    const TX* xp = F::NIN >= 1 ? x + operand_offset(ox, g, i) : nullptr;
    const TX* yp = F::NIN >= 2 ? y + operand_offset(oy, g, i) : nullptr;
    const TX xb = (F::NIN >= 1 && !x_row) ? *xp : TX();
    const TX yb = (F::NIN >= 2 && !y_row) ? *yp : TX();
    for (unsigned c0 = lane; c0 < chunks; c0 += 32 * U) {
      Vec<TX, VEC> xv[U], yv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned c = c0 + 32 * u;
        if (c < chunks) {
          if (F::NIN >= 1 && x_row) xv[u] = reinterpret_cast<const Vec<TX, VEC>*>(xp)[c];
          if (F::NIN >= 2 && y_row) yv[u] = reinterpret_cast<const Vec<TX, VEC>*>(yp)[c];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const unsigned c = c0 + 32 * u;
        if (c < chunks) {
          Vec<TD, VEC> o;
#pragma unroll
          for (int k = 0; k < VEC; ++k)
            o.v[k] = f(F::NIN >= 1 ? (x_row ? xv[u].v[k] : xb) : TX(), F::NIN >= 2 ? (y_row ? yv[u].v[k] : yb) : TX());
          d[c] = o;
        }
      }
    }
  }
}

template <typename TD, typename F>
__global__ void __launch_bounds__(256)
ew_generic(TD* dest, const typename F::TX* x, const typename F::TX* y,
           Operand od, Operand ox, Operand oy, Geometry g, long long n, F f) {
  typedef typename F::TX TX;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    TX xe = TX(), ye = TX();
    if (F::NIN >= 1) xe = x[operand_offset(ox, g, i)];
    if (F::NIN >= 2) ye = y[operand_offset(oy, g, i)];
    dest[operand_offset(od, g, i)] = f(xe, ye);
  }
}

// dest = (alpha*dest) op (beta*y) when several element indexes may land on one
// dest address: compare-and-swap loop (resources/cas.h:5-19 plays this role in
// the reference).  int / long / float / double only.
template <typename T> struct cas_word;
template <> struct cas_word<int> { typedef int type; };
template <> struct cas_word<float> { typedef int type; };
template <> struct cas_word<long long> { typedef unsigned long long type; };
template <> struct cas_word<double> { typedef unsigned long long type; };

template <typename T>
__global__ void __launch_bounds__(256)
ew_accum_cas(T* dest, const T* y, Operand od, Operand oy, Geometry g, long long n, BinaryF<T> f, int has_y,
             BinaryConstF<T> fc) {
  typedef typename cas_word<T>::type W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    T ye = has_y ? y[operand_offset(oy, g, i)] : T();
    W* addr = reinterpret_cast<W*>(dest + operand_offset(od, g, i));
    W old = *addr, assumed;
    int guard = 0;
    do {
      assumed = old;
      T cur;
      memcpy(&cur, &assumed, sizeof(T));
      T nv = has_y ? f(cur, ye) : fc(cur, T());
      W nw;
      memcpy(&nw, &nv, sizeof(T));
      old = atomicCAS(addr, assumed, nw);
    } while (assumed != old && ++guard < (1 << 20));
  }
}

// Broadcast-sum accumulation  dest[c] += ya * sum over n, e of y[n, c, e]  (dest [C] dense, y [N, C, E] dense):
// what the bias gradients are (binary-op! with a destination smaller than the operation, y_alpha * y + dest).
// The compare-and-swap kernel above serialises every element that maps to one destination address (N * E of
// them); here each block sums a slab privately and issues ONE atomic add per destination it touches.  The sum
// order is as unspecified as with compare-and-swap; partial sums are kept in double.
template <typename T>
__global__ void __launch_bounds__(128)
bcast_sum_cols_kernel(T* dest, const T* y, int N, int C, double ya, int rows_per_slab, int vec) {
  // E == 1: columns are contiguous; a thread owns `vec` adjacent columns and walks the rows of its slab
  const long long col = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * vec;
  if (col >= C) return;
  const int r0 = blockIdx.y * rows_per_slab, r1 = min(N, r0 + rows_per_slab);
  double acc[4] = {0.0, 0.0, 0.0, 0.0};
  if (vec == 4) {
    struct alignas(16) V { T v[4]; };
    T p0[4] = {T(), T(), T(), T()}, p1[4] = {T(), T(), T(), T()};
    int r = r0;
    for (; r + 1 < r1; r += 2) {          // two rows in flight, accumulated in the element type over a short run
      const V a = *reinterpret_cast<const V*>(y + (long long)r * C + col);
      const V b = *reinterpret_cast<const V*>(y + (long long)(r + 1) * C + col);
#pragma unroll
      for (int e = 0; e < 4; ++e) { p0[e] += a.v[e]; p1[e] += b.v[e]; }
      if (((r - r0) & 62) == 62) {
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[e] += (double)p0[e] + (double)p1[e]; p0[e] = T(); p1[e] = T(); }
      }
    }
    if (r < r1) {
      const V a = *reinterpret_cast<const V*>(y + (long long)r * C + col);
#pragma unroll
      for (int e = 0; e < 4; ++e) p0[e] += a.v[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] += (double)p0[e] + (double)p1[e];
#pragma unroll
    for (int e = 0; e < 4; ++e) atomicAdd(dest + col + e, (T)(acc[e] * ya));
  } else {
    for (int r = r0; r < r1; ++r) acc[0] += (double)y[(long long)r * C + col];
    atomicAdd(dest + col, (T)(acc[0] * ya));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
bcast_sum_runs_kernel(T* dest, const T* y, int N, int C, long long E, double ya, int n_per_chunk, int vec) {
  // E > 1: for a fixed (n, c) the E elements are contiguous; block = (c, chunk of n)
  const int c = blockIdx.x;
  const int n0 = blockIdx.y * n_per_chunk, n1 = min(N, n0 + n_per_chunk);
  double acc = 0.0;
  for (int n = n0; n < n1; ++n) {
    const T* base = y + ((long long)n * C + c) * E;
    if (vec == 4) {
      struct alignas(16) V { T v[4]; };
      T p = T();
      for (long long e = threadIdx.x; e < E / 4; e += blockDim.x) {
        const V a = reinterpret_cast<const V*>(base)[e];
        p += (a.v[0] + a.v[1]) + (a.v[2] + a.v[3]);
      }
      acc += (double)p;
    } else {
      for (long long e = threadIdx.x; e < E; e += blockDim.x) acc += (double)base[e];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ double part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += part[w];
    atomicAdd(dest + c, (T)(t * ya));
  }
}

// Recognises dest [C] (+ unit dims) accumulated over a dense y [N, C, E]; returns false if the shapes are not of
// that form (the caller then uses compare-and-swap).
template <typename T>
bool try_bcast_sum(cb200_stream* s, T* dest, const cb200_dims* dd, const T* y, const cb200_dims* yd, long long n,
                   double ya, int* rc_out) {
  long long expect_y = 1, expect_d = 1, E = 1, Cn = 1, N = 1;
  int phase = 0;      // 0: inner dims absent from dest, 1: dims shared with dest, 2: outer dims absent from dest
  for (int d = 0; d < 5; ++d) {
    const long long ys = yd->rev_shape[d], ds = dd->rev_shape[d];
    if (yd->index[d] || dd->index[d]) return false;
    if (ys > 1 && yd->rev_strides[d] != expect_y) return false;
    if (ds > 1 && dd->rev_strides[d] != expect_d) return false;
    expect_y *= ys;
    expect_d *= ds;
    if (ys == 1 && ds == 1) continue;
    if (ds == ys) {                      // shared dimension
      if (phase == 2) return false;
      phase = 1;
      Cn *= ys;
    } else if (ds == 1) {                // summed dimension
      if (phase == 0) E *= ys; else { phase = 2; N *= ys; }
    } else {
      return false;
    }
  }
  if (phase == 0 || N * E == 1 || N * Cn * E != n) return false;
  if (N > 2147483647LL || Cn > 2147483647LL) return false;
  DeviceGuard guard(s->device);
  const int target_blocks = s->sm_count * 8;
  if (E == 1) {
    const int vec = (Cn % 4 == 0 && (((uintptr_t)y) & 15) == 0) ? 4 : 1;
    const long long col_threads = Cn / vec;
    const unsigned gx = (unsigned)((col_threads + 127) / 128);
    long long slabs = (target_blocks + gx - 1) / gx;
    if (slabs > N) slabs = N;
    if (slabs > 65535) slabs = 65535;
    if (slabs < 1) slabs = 1;
    const int rows_per_slab = (int)((N + slabs - 1) / slabs);
    dim3 grid(gx, (unsigned)((N + rows_per_slab - 1) / rows_per_slab), 1);
    bcast_sum_cols_kernel<T><<<grid, 128, 0, s->stream>>>(dest, y, (int)N, (int)Cn, ya, rows_per_slab, vec);
  } else {
    const int vec = (E % 4 == 0 && (((uintptr_t)y) & 15) == 0) ? 4 : 1;
    long long chunks = (target_blocks + Cn - 1) / Cn;
    if (chunks > N) chunks = N;
    if (chunks > 65535) chunks = 65535;
    if (chunks < 1) chunks = 1;
    const int n_per_chunk = (int)((N + chunks - 1) / chunks);
    dim3 grid((unsigned)Cn, (unsigned)((N + n_per_chunk - 1) / n_per_chunk), 1);
    bcast_sum_runs_kernel<T><<<grid, 256, 0, s->stream>>>(dest, y, (int)N, (int)Cn, E, ya, n_per_chunk, vec);
  }
  *rc_out = CB200_OK;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) *rc_out = cb200_cuda_fail(e, "bcast_sum launch", __FILE__, __LINE__);
  return true;
}

// ------------------------------ host-side planning --------------------------

struct Plan {
  Geometry g;
  long long n;
};

void make_geometry(Geometry& g, const Operand* ops, int n_ops) {
  g.ndims = 1;
  for (int d = 0; d < 5; ++d) {
    int m = 1;
    for (int k = 0; k < n_ops; ++k) m = ops[k].shape[d] > m ? ops[k].shape[d] : m;
    g.max_shape[d] = m;
    if (m > 1) g.ndims = d + 1;
  }
}

bool has_index(const Operand& o) {
  for (int d = 0; d < 5; ++d) if (o.index[d]) return true;
  return false;
}

// SIMPLE / REPEAT / BCAST classification, after the reference CPU backend's own
// fast paths (src/cortex/compute/cpu/tensor_math.clj:84-116).
bool flat_mode(const Operand& o, const Geometry& g, FlatMode& m) {
  if (has_index(o)) return false;
  int nontrivial = 0, last = -1;
  for (int d = 0; d < 5; ++d) if (o.shape[d] > 1) { ++nontrivial; last = d; }
  if (nontrivial == 0) { m.kind = 2; m.ec = 1; m.amt = 1; m.stride = 0; return true; }
  // repeating suffix: shape == max for the k fastest dims, 1 beyond, densely packed
  bool suffix = true;
  long long ec = 1;
  for (int d = 0; d <= last; ++d) {
    if (o.shape[d] != g.max_shape[d]) { suffix = false; break; }
    if (o.shape[d] > 1 && o.stride[d] != ec) { suffix = false; break; }
    ec *= o.shape[d];
  }
  if (suffix) {
    bool full = true;
    for (int d = last + 1; d < 5; ++d) if (g.max_shape[d] != 1) full = false;
    m.kind = full ? 0 : 1; m.ec = (unsigned)ec; m.amt = 1; m.stride = 1;
    return true;
  }
  if (nontrivial == 1 && o.shape[last] == g.max_shape[last]) {
    long long amt = 1;
    for (int d = 0; d < last; ++d) amt *= g.max_shape[d];
    m.kind = 2; m.ec = (unsigned)o.shape[last]; m.amt = (unsigned)amt; m.stride = o.stride[last];
    return true;
  }
  return false;
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

bool rowvec_ok(const Operand& o, const Geometry& g, const void* base, size_t esize, int vec, int& row_mode) {
  if (o.index[0]) return false;
  if (o.shape[0] == g.max_shape[0] && (o.stride[0] == 1 || g.max_shape[0] == 1)) row_mode = 1;
  else if (o.shape[0] == 1) { row_mode = 0; return true; }
  else return false;
  if (((uintptr_t)base % (esize * vec)) != 0) return false;
  for (int d = 1; d < g.ndims; ++d)
    if (o.shape[d] > 1 && (o.stride[d] % vec) != 0) return false;
  return true;
}

int grid_for(cb200_stream* s, long long work_items, int per_block) {
  long long blocks = (work_items + per_block - 1) / per_block;
  long long cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <int A, int B> struct max_of { static const int value = A > B ? A : B; };
template <typename A, typename B> struct acc_same { static const bool value = false; };
template <typename A> struct acc_same<A, A> { static const bool value = true; };

// Launch one elementwise map.  x / y may be null when F::NIN says so.
// PATHS: 0 = general index-system kernel only (dtype-marshalling copies), 1 = + flat and
// row-vector kernels, 2 = + warp-per-row kernel (what the dense layers and gathers hit).
template <typename TD, typename F, int PATHS = 1>
int launch_map(cb200_stream* s, TD* dest, const cb200_dims* dd, const typename F::TX* x, const cb200_dims* xd,
               const typename F::TX* y, const cb200_dims* yd, long long n, const F& f) {
  typedef typename F::TX TX;
  if (n <= 0) return CB200_OK;
  CB_REQUIRE(n <= 2147483647LL, "element count %lld exceeds the 32-bit index range of the tensor protocol", n);
  Operand ops[3];
  operand_from_dims(ops[0], dd);
  int n_ops = 1;
  if (F::NIN >= 1) operand_from_dims(ops[n_ops++], xd);
  if (F::NIN >= 2) operand_from_dims(ops[n_ops++], yd);
  for (int k = n_ops; k < 3; ++k) ops[k] = ops[0];
  Geometry g;
  make_geometry(g, ops, n_ops);
  DeviceGuard guard(s->device);

  if constexpr (PATHS >= 1) {
    constexpr int ES = max_of<sizeof(TD), sizeof(TX)>::value;
    constexpr int VEC = (16 / ES) > 4 ? 4 : (16 / ES);   // 16-byte accesses for 4- and 8-byte types
    constexpr int UNROLL = 4;

    FlatMode md, mx = {0, 1, 1, 1}, my = {0, 1, 1, 1};
    bool flat = flat_mode(ops[0], g, md) && md.kind == 0 && aligned16(dest);
    if (flat && F::NIN >= 1) flat = flat_mode(ops[1], g, mx);
    if (flat && F::NIN >= 2) flat = flat_mode(ops[2], g, my);
    if (flat) {
      auto vec_ok = [&](const FlatMode& m, const void* p) -> int {
        if (m.kind == 0) return ((uintptr_t)p % (sizeof(TX) * VEC)) == 0;
        if (m.kind == 1) return (m.ec % VEC) == 0 && ((uintptr_t)p % (sizeof(TX) * VEC)) == 0;
        return (m.amt % VEC) == 0;
      };
      int xv = F::NIN >= 1 ? vec_ok(mx, x) : 1, yv = F::NIN >= 2 ? vec_ok(my, y) : 1;
      long long n_vec = n / VEC;
      long long blocks = (n_vec + 256 * UNROLL - 1) / (256 * UNROLL);
      // twice the resident block count: measured best of 4x / 8x / 16x the SM count for a streaming
      // read + write on [8192, 4096] fp32 (5.4 / 5.9 / 6.2 TB/s; the driver's own device-to-device copy
      // of the same size: 6.1 TB/s)
      long long full = (long long)s->sm_count * 16;
      if (blocks > full) blocks = full;
      if (blocks < 1) blocks = 1;
      ew_flat<TD, F, VEC, UNROLL><<<(unsigned)blocks, 256, 0, s->stream>>>(dest, x, y, mx, my, xv, yv, (unsigned)n, f);
      CB_LAUNCH_CHECK(s);
      return CB200_OK;
    }

    if constexpr (VEC > 1) {
      int dr = 0, xr = 1, yr = 1;
      bool rv = (g.max_shape[0] % VEC) == 0 && rowvec_ok(ops[0], g, dest, sizeof(TD), VEC, dr) && dr == 1;
      if (rv && F::NIN >= 1) rv = rowvec_ok(ops[1], g, x, sizeof(TX), VEC, xr);
      if (rv && F::NIN >= 2) rv = rowvec_ok(ops[2], g, y, sizeof(TX), VEC, yr);
      long long total = 1;
      for (int d = 0; d < 5; ++d) total *= g.max_shape[d];
      if (rv && n == total) {
        const long long n_chunks = n / VEC;
        const long long chunks_per_row = g.max_shape[0] / VEC, n_rows = n / g.max_shape[0];
        if constexpr (PATHS >= 2) {
          if (chunks_per_row >= 32 && n_rows >= (long long)s->sm_count * 8) {
            long long wblocks = (n_rows + 7) / 8, wfull = (long long)s->sm_count * 8;
            if (wblocks > wfull) wblocks = wfull;
            ew_rowwarp<TD, F, VEC><<<(unsigned)wblocks, 256, 0, s->stream>>>(dest, x, y, ops[0], ops[1], ops[2], g, xr,
                                                                           yr, (unsigned)n_rows, f);
            CB_LAUNCH_CHECK(s);
            return CB200_OK;
          }
        }
        long long rblocks = (n_chunks + 1023) / 1024, rfull = (long long)s->sm_count * 8;
        if (rblocks > rfull) rblocks = rfull;
        ew_rowvec<TD, F, VEC><<<(unsigned)rblocks, 256, 0, s->stream>>>(dest, x, y, ops[0], ops[1], ops[2], g, xr, yr,
                                                                        (unsigned)n_chunks, f);
        CB_LAUNCH_CHECK(s);
        return CB200_OK;
      }
    }
  }

  ew_generic<TD, F><<<grid_for(s, n, 256), 256, 0, s->stream>>>(dest, x, y, ops[0], ops[1], ops[2], g, n, f);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

template <typename T>
int launch_accum_cas(cb200_stream* s, T* dest, const cb200_dims* dd, const T* y, const cb200_dims* yd, long long n,
                     const BinaryF<T>& f, int has_y, const BinaryConstF<T>& fc) {
  if (n <= 0) return CB200_OK;
  Operand ops[2];
  operand_from_dims(ops[0], dd);
  if (has_y) operand_from_dims(ops[1], yd); else ops[1] = ops[0];
  Geometry g;
  make_geometry(g, ops, has_y ? 2 : 1);
  DeviceGuard guard(s->device);
  ew_accum_cas<T><<<grid_for(s, n, 256), 256, 0, s->stream>>>(dest, y, ops[0], ops[1], g, n, f, has_y, fc);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

// fp32 + unit scale factors + one of the six arithmetic ops -> compile-time-op kernels
#define CB_FAST_OPS(X) X(CB200_ADD) X(CB200_SUB) X(CB200_MUL) X(CB200_DIV) X(CB200_MAX) X(CB200_MIN)

int fast_binary_f32(cb200_stream* s, float* dest, const cb200_dims* dd, const float* x, const cb200_dims* xd,
                    const float* y, const cb200_dims* yd, long long n, int op, int rev, bool* handled) {
  *handled = true;
  if (rev) { const float* t = x; x = y; y = t; const cb200_dims* td = xd; xd = yd; yd = td; }
  switch (op) {
#define X(OPC) \
    case OPC: return launch_map<float, FastBinaryF<OPC>, 2>(s, dest, dd, x, xd, y, yd, n, FastBinaryF<OPC>());
    CB_FAST_OPS(X)
#undef X
  }
  *handled = false;
  return CB200_OK;
}

int fast_binary_const_f32(cb200_stream* s, float* dest, const cb200_dims* dd, const float* x, const cb200_dims* xd,
                          float scalar, long long n, int op, int rev, bool* handled) {
  *handled = true;
  if (rev && (op == CB200_SUB || op == CB200_DIV)) {
    if (op == CB200_SUB) { FastBinaryConstF<CB200_SUB, 1> f; f.scalar = scalar;
      return launch_map<float, FastBinaryConstF<CB200_SUB, 1>, 2>(s, dest, dd, x, xd, nullptr, nullptr, n, f); }
    FastBinaryConstF<CB200_DIV, 1> f; f.scalar = scalar;
    return launch_map<float, FastBinaryConstF<CB200_DIV, 1>, 2>(s, dest, dd, x, xd, nullptr, nullptr, n, f);
  }
  switch (op) {   // + * max min are symmetric: operand order does not matter
#define X(OPC) \
    case OPC: { FastBinaryConstF<OPC, 0> f; f.scalar = scalar; \
      return launch_map<float, FastBinaryConstF<OPC, 0>, 2>(s, dest, dd, x, xd, nullptr, nullptr, n, f); }
    CB_FAST_OPS(X)
#undef X
  }
  *handled = false;
  return CB200_OK;
}

#define CB_ARGCHECK(s, ...)                                                     \
  do {                                                                          \
    CB_REQUIRE((s) != nullptr, "null stream");                                  \
    const void* ptrs__[] = {__VA_ARGS__};                                       \
    for (size_t i__ = 0; i__ < sizeof(ptrs__) / sizeof(ptrs__[0]); ++i__)       \
      CB_REQUIRE(ptrs__[i__] != nullptr, "null buffer or descriptor (argument %d)", (int)i__); \
  } while (0)

}  // namespace

extern "C" {

int cb200_memset(cb200_stream* s, int dtype, void* buf, int64_t elem_offset, double value, int64_t n_elems) {
  CB_ARGCHECK(s, buf);
  CB_REQUIRE(elem_offset >= 0 && n_elems >= 0, "memset: negative offset or count");
  if (n_elems == 0) return CB200_OK;
  size_t es = cb200_dtype_size(dtype);
  CB_REQUIRE(es != 0, "memset: unknown dtype %d", dtype);
  char* p = (char*)buf + (size_t)elem_offset * es;
  if (value == 0.0) {   // zero fill is a plain memset (src/cortex/compute/cuda/driver.clj:1020-1032)
    DeviceGuard guard(s->device);
    CB_CUDA(cudaMemsetAsync(p, 0, (size_t)n_elems * es, s->stream));
    return CB200_OK;
  }
  cb200_dims d;
  for (int i = 0; i < 5; ++i) { d.rev_shape[i] = 1; d.rev_strides[i] = 1; d.index[i] = nullptr; }
  CB_REQUIRE(n_elems <= 2147483647LL, "memset: more than 2^31-1 elements");
  d.rev_shape[0] = (int32_t)n_elems;
  CB_DISPATCH_DTYPE(dtype, T, {
    FillF<T> f; f.value = store_as<T>::from(value);
    return launch_map<T, FillF<T> >(s, (T*)p, &d, nullptr, nullptr, nullptr, nullptr, n_elems, f);
  });
  return CB200_OK;
}

int cb200_assign_constant(cb200_stream* s, int dtype, void* buf, const cb200_dims* dims, double value,
                          int64_t n_elems) {
  CB_ARGCHECK(s, buf, dims);
  int rc = cb200_check_dims(dims, "assign_constant");
  if (rc) return rc;
  CB_DISPATCH_DTYPE(dtype, T, {
    FillF<T> f; f.value = store_as<T>::from(value);
    return launch_map<T, FillF<T> >(s, (T*)buf, dims, nullptr, nullptr, nullptr, nullptr, n_elems, f);
  });
  return CB200_OK;
}

int cb200_assign(cb200_stream* s, int dest_dtype, void* dest, const cb200_dims* dest_dims, int src_dtype,
                 const void* src, const cb200_dims* src_dims, int64_t n_elems) {
  CB_ARGCHECK(s, dest, dest_dims, src, src_dims);
  int rc = cb200_check_dims(dest_dims, "assign dest");
  if (rc) return rc;
  rc = cb200_check_dims(src_dims, "assign src");
  if (rc) return rc;
  CB_DISPATCH_DTYPE(dest_dtype, TD, {
    CB_DISPATCH_DTYPE(src_dtype, TS, {
      AssignF<TD, TS> f;
      // same-dtype copies (bias broadcast, row gathers, transposes) get every fast path;
      // marshalling copies go through the general kernel
      constexpr int paths = (sizeof(TD) == sizeof(TS) && acc_same<TD, TS>::value) ? 2 : 0;
      return launch_map<TD, AssignF<TD, TS>, paths>(s, (TD*)dest, dest_dims, (const TS*)src, src_dims, nullptr,
                                                    nullptr, n_elems, f);
    });
  });
  return CB200_OK;
}

int cb200_unary_op(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims, const void* x,
                   const cb200_dims* x_dims, double alpha, int op, int64_t n_elems) {
  CB_ARGCHECK(s, dest, dest_dims, x, x_dims);
  CB_REQUIRE(op >= CB200_FLOOR && op <= CB200_NOOP, "unary_op: unknown op %d", op);
  int rc = cb200_check_dims(dest_dims, "unary_op dest");
  if (rc) return rc;
  rc = cb200_check_dims(x_dims, "unary_op x");
  if (rc) return rc;
  CB_DISPATCH_DTYPE(dtype, T, {
    UnaryF<T> f; f.op = op; f.alpha = scalar_as<T>(alpha);
    return launch_map<T, UnaryF<T> >(s, (T*)dest, dest_dims, (const T*)x, x_dims, nullptr, nullptr, n_elems, f);
  });
  return CB200_OK;
}

int cb200_unary_accum(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims, double alpha, int op,
                      int64_t n_elems) {
  return cb200_unary_op(s, dtype, dest, dest_dims, dest, dest_dims, alpha, op, n_elems);
}

int cb200_binary_op_constant(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims, const void* x,
                             const cb200_dims* x_dims, double x_alpha, double scalar, int64_t n_elems, int op,
                             int rev_ops) {
  CB_ARGCHECK(s, dest, dest_dims, x, x_dims);
  CB_REQUIRE(op >= CB200_ADD && op <= CB200_LE, "binary_op_constant: unknown op %d", op);
  int rc = cb200_check_dims(dest_dims, "binary_op_constant dest");
  if (rc) return rc;
  rc = cb200_check_dims(x_dims, "binary_op_constant x");
  if (rc) return rc;
  if (dtype == CB200_FLOAT && (float)x_alpha == 1.0f) {
    bool handled = false;
    rc = fast_binary_const_f32(s, (float*)dest, dest_dims, (const float*)x, x_dims, (float)scalar, n_elems, op,
                               rev_ops, &handled);
    if (handled) return rc;
  }
  CB_DISPATCH_DTYPE(dtype, T, {
    BinaryConstF<T> f; f.op = op; f.rev = rev_ops; f.alpha = scalar_as<T>(x_alpha); f.scalar = scalar_as<T>(scalar);
    return launch_map<T, BinaryConstF<T> >(s, (T*)dest, dest_dims, (const T*)x, x_dims, nullptr, nullptr, n_elems, f);
  });
  return CB200_OK;
}

int cb200_binary_accum_constant(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims,
                                double dest_alpha, double scalar, int64_t n_elems, int op, int rev_ops) {
  bool indexed_dest = false;
  if (dest_dims) for (int d = 0; d < 5; ++d) if (dest_dims->index[d]) indexed_dest = true;
  if (indexed_dest) {
    CB_ARGCHECK(s, dest, dest_dims);
    CB_REQUIRE(op >= CB200_ADD && op <= CB200_LE, "binary_accum_constant: unknown op %d", op);
    switch (dtype) {
#define CB_CASC_CASE(DT, T)                                                                       \
      case DT: {                                                                                  \
        BinaryF<T> f; f.op = op; f.rev = 0; f.xa = 0; f.ya = 0;                                   \
        BinaryConstF<T> fc; fc.op = op; fc.rev = rev_ops; fc.alpha = scalar_as<T>(dest_alpha);    \
        fc.scalar = scalar_as<T>(scalar);                                                         \
        return launch_accum_cas<T>(s, (T*)dest, dest_dims, nullptr, nullptr, n_elems, f, 0, fc);  \
      }
      CB_CASC_CASE(CB200_INT, int)
      CB_CASC_CASE(CB200_LONG, long long)
      CB_CASC_CASE(CB200_FLOAT, float)
      CB_CASC_CASE(CB200_DOUBLE, double)
#undef CB_CASC_CASE
      default:
        cb200_set_error("binary_accum_constant: indexed destinations need int, long, float or double");
        return CB200_ERR_INVALID;
    }
  }
  return cb200_binary_op_constant(s, dtype, dest, dest_dims, dest, dest_dims, dest_alpha, scalar, n_elems, op,
                                  rev_ops);
}

int cb200_binary_op(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims, const void* x,
                    const cb200_dims* x_dims, double x_alpha, const void* y, const cb200_dims* y_dims,
                    double y_alpha, int64_t n_elems, int op) {
  CB_ARGCHECK(s, dest, dest_dims, x, x_dims, y, y_dims);
  CB_REQUIRE(op >= CB200_ADD && op <= CB200_LE, "binary_op: unknown op %d", op);
  int rc = cb200_check_dims(dest_dims, "binary_op dest");
  if (rc) return rc;
  rc = cb200_check_dims(x_dims, "binary_op x");
  if (rc) return rc;
  rc = cb200_check_dims(y_dims, "binary_op y");
  if (rc) return rc;
  if (dtype == CB200_FLOAT && (float)x_alpha == 1.0f && ((float)y_alpha == 1.0f || ((float)y_alpha == -1.0f && op == CB200_ADD))) {
    // binary-op! :- reaches the backend as :+ with a negated beta (src/cortex/tensor.clj:774-778)
    bool handled = false;
    rc = fast_binary_f32(s, (float*)dest, dest_dims, (const float*)x, x_dims, (const float*)y, y_dims, n_elems,
                         (float)y_alpha == -1.0f ? CB200_SUB : op, 0, &handled);
    if (handled) return rc;
  }
  CB_DISPATCH_DTYPE(dtype, T, {
    BinaryF<T> f; f.op = op; f.rev = 0; f.xa = scalar_as<T>(x_alpha); f.ya = scalar_as<T>(y_alpha);
    return launch_map<T, BinaryF<T> >(s, (T*)dest, dest_dims, (const T*)x, x_dims, (const T*)y, y_dims, n_elems, f);
  });
  return CB200_OK;
}

int cb200_binary_accum(cb200_stream* s, int dtype, void* dest, const cb200_dims* dest_dims, double dest_alpha,
                       const void* y, const cb200_dims* y_dims, double y_alpha, int64_t n_elems, int op, int rev_ops,
                       int requires_cas) {
  CB_ARGCHECK(s, dest, dest_dims, y, y_dims);
  CB_REQUIRE(op >= CB200_ADD && op <= CB200_LE, "binary_accum: unknown op %d", op);
  int rc = cb200_check_dims(dest_dims, "binary_accum dest");
  if (rc) return rc;
  rc = cb200_check_dims(y_dims, "binary_accum y");
  if (rc) return rc;
  bool indexed_dest = false;
  for (int d = 0; d < 5; ++d) if (dest_dims->index[d]) indexed_dest = true;
  if (requires_cas && !indexed_dest && op == CB200_ADD && (dtype == CB200_FLOAT || dtype == CB200_DOUBLE) &&
      dest != y) {
    // bias-gradient shape: dest + y_alpha * y summed over the dimensions dest does not have
    int rc2 = CB200_OK;
    const bool unit = dtype == CB200_FLOAT ? (float)dest_alpha == 1.0f : dest_alpha == 1.0;
    if (unit) {
      bool done = dtype == CB200_FLOAT
                      ? try_bcast_sum<float>(s, (float*)dest, dest_dims, (const float*)y, y_dims, n_elems,
                                             (double)(float)y_alpha, &rc2)
                      : try_bcast_sum<double>(s, (double*)dest, dest_dims, (const double*)y, y_dims, n_elems, y_alpha, &rc2);
      if (done) { if (rc2 == CB200_OK) { CB_LAUNCH_CHECK(s); } return rc2; }
    }
  }
  if (requires_cas || indexed_dest) {
    switch (dtype) {
#define CB_CAS_CASE(DT, T)                                                                        \
      case DT: {                                                                                  \
        BinaryF<T> f; f.op = op; f.rev = rev_ops; f.xa = scalar_as<T>(dest_alpha); f.ya = scalar_as<T>(y_alpha); \
        BinaryConstF<T> fc; fc.op = op; fc.rev = 0; fc.alpha = 0; fc.scalar = 0;                 \
        return launch_accum_cas<T>(s, (T*)dest, dest_dims, (const T*)y, y_dims, n_elems, f, 1, fc); \
      }
      CB_CAS_CASE(CB200_INT, int)
      CB_CAS_CASE(CB200_LONG, long long)
      CB_CAS_CASE(CB200_FLOAT, float)
      CB_CAS_CASE(CB200_DOUBLE, double)
#undef CB_CAS_CASE
      default:
        cb200_set_error("binary_accum: compare-and-swap accumulation exists for int, long, float, double only");
        return CB200_ERR_INVALID;
    }
  }
  if (dtype == CB200_FLOAT && (float)dest_alpha == 1.0f && ((float)y_alpha == 1.0f || ((float)y_alpha == -1.0f && op == CB200_ADD && !rev_ops))) {
    bool handled = false;
    rc = fast_binary_f32(s, (float*)dest, dest_dims, (const float*)dest, dest_dims, (const float*)y, y_dims, n_elems,
                         (float)y_alpha == -1.0f ? CB200_SUB : op, rev_ops, &handled);
    if (handled) return rc;
  }
  CB_DISPATCH_DTYPE(dtype, T, {
    BinaryF<T> f; f.op = op; f.rev = rev_ops; f.xa = scalar_as<T>(dest_alpha); f.ya = scalar_as<T>(y_alpha);
    return launch_map<T, BinaryF<T> >(s, (T*)dest, dest_dims, (const T*)dest, dest_dims, (const T*)y, y_dims,
                                      n_elems, f);
  });
  return CB200_OK;
}

}  // extern "C"
