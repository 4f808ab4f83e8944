// unary-reduce!, softmax! and the fused bias+ReLU+row-statistics pass.
//
// The reference runs one thread per output row with a serial loop over the row
// (resources/tensor_unary_reduce.cu:38-88): adjacent threads are a whole row
// apart.  Here a row whose fastest dimension is contiguous is read by one warp
// (short rows) or one CTA (long rows) with coalesced loads, several loads in
// flight per thread, and combined with warp shuffles.  HBM-bound: algorithmic
// bytes = input read once + output written once.
//
// Arithmetic follows the reference CPU backend
// (src/cortex/compute/cpu/tensor_math.clj:588-629, 1037-1103): fp32 rows are
// accumulated in double and rounded once; integer rows in 64-bit.
#include "common.cuh"
#include <math.h>

namespace {

template <typename A> __device__ __forceinline__ A shfl_down_any(A v, int delta);
template <> __device__ __forceinline__ double shfl_down_any<double>(double v, int delta) {
  return __shfl_down_sync(0xffffffffu, v, delta);
}
template <> __device__ __forceinline__ long long shfl_down_any<long long>(long long v, int delta) {
  return __shfl_down_sync(0xffffffffu, v, delta);
}
template <> __device__ __forceinline__ float shfl_down_any<float>(float v, int delta) {
  return __shfl_down_sync(0xffffffffu, v, delta);
}

// clojure.core/max and min on primitives: NaN-propagating for doubles
__device__ __forceinline__ double clj_max(double a, double b) { return (a != a) ? a : ((b != b) ? b : (a > b ? a : b)); }
__device__ __forceinline__ double clj_min(double a, double b) { return (a != a) ? a : ((b != b) ? b : (a < b ? a : b)); }
__device__ __forceinline__ float clj_max(float a, float b) { return (a != a) ? a : ((b != b) ? b : (a > b ? a : b)); }
__device__ __forceinline__ long long clj_max(long long a, long long b) { return a > b ? a : b; }
__device__ __forceinline__ long long clj_min(long long a, long long b) { return a < b ? a : b; }

template <typename A> __device__ __forceinline__ A red_identity(int op);
template <> __device__ __forceinline__ double red_identity<double>(int op) {
  return op == CB200_RMAX ? -INFINITY : (op == CB200_RMIN ? INFINITY : 0.0);
}
template <> __device__ __forceinline__ long long red_identity<long long>(int op) {
  return op == CB200_RMAX ? (-9223372036854775807LL - 1) : (op == CB200_RMIN ? 9223372036854775807LL : 0);
}

template <typename A>
__device__ __forceinline__ A red_elem(int op, A v) {
  return (op == CB200_RMAGNITUDE || op == CB200_RMAGNITUDE_SQ) ? (A)(v * v) : v;
}
template <typename A>
__device__ __forceinline__ A red_combine(int op, A a, A b) {
  if (op == CB200_RMAX) return clj_max(a, b);
  if (op == CB200_RMIN) return clj_min(a, b);
  return (A)(a + b);
}

template <typename T>
__device__ __forceinline__ T red_finish(int op, typename acc_of<T>::type acc, long long len) {
  typedef typename acc_of<T>::type A;
  if (op == CB200_RMEAN) {
    // (/ sum n): double division for floating views, truncating for integer views
    return store_as<T>::from((A)(acc / (A)len));
  }
  if (op == CB200_RMAGNITUDE) return store_as<T>::from(sqrt((double)acc));
  return store_as<T>::from(acc);
}

template <typename A, int NWARPS>
__device__ __forceinline__ A block_combine(int op, A v, A* smem) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = red_combine(op, v, shfl_down_any<A>(v, d));
  if (NWARPS == 1) return v;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < NWARPS ? smem[lane] : red_identity<A>(op);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = red_combine(op, v, shfl_down_any<A>(v, d));
  }
  return v;  // valid in thread 0
}

// One CTA (NWARPS = 8) or one warp (NWARPS = 1, 8 rows per CTA) per row.
template <typename T, int NWARPS>
__global__ void __launch_bounds__(256)
reduce_rows(T* out, const T* in, Operand oo, Operand oi, Geometry go, Geometry gi, long long n_rows, int len, int op,
            typename acc_of<T>::type alpha) {
  typedef typename acc_of<T>::type A;
  __shared__ A smem[8];
  const int rows_per_block = NWARPS == 1 ? 8 : 1;
  const int tid = NWARPS == 1 ? (threadIdx.x & 31) : threadIdx.x;
  const int nthreads = NWARPS == 1 ? 32 : 256;
  for (long long r0 = (long long)blockIdx.x * rows_per_block; r0 < n_rows; r0 += (long long)gridDim.x * rows_per_block) {
    long long r = NWARPS == 1 ? r0 + (threadIdx.x >> 5) : r0;
    A acc = red_identity<A>(op);
    if (r < n_rows) {
      const T* row = in + operand_offset(oi, gi, r * len);
      int j = tid;
      // 4 independent loads in flight per thread
      for (; j + 3 * nthreads < len; j += 4 * nthreads) {
        T v0 = row[j], v1 = row[j + nthreads], v2 = row[j + 2 * nthreads], v3 = row[j + 3 * nthreads];
        acc = red_combine(op, acc, red_elem(op, (A)(alpha * (A)v0)));
        acc = red_combine(op, acc, red_elem(op, (A)(alpha * (A)v1)));
        acc = red_combine(op, acc, red_elem(op, (A)(alpha * (A)v2)));
        acc = red_combine(op, acc, red_elem(op, (A)(alpha * (A)v3)));
      }
      for (; j < len; j += nthreads) acc = red_combine(op, acc, red_elem(op, (A)(alpha * (A)row[j])));
    }
    acc = block_combine<A, NWARPS>(op, acc, smem);
    if (tid == 0 && r < n_rows) out[operand_offset(oo, go, r)] = red_finish<T>(op, acc, len);
  }
}

// 16-byte vector variant for aligned contiguous rows (len % VEC == 0): 8 independent
// 16-byte loads in flight per thread.  FAST (float rows, max / min, alpha == 1) compares
// in fp32 -- exact, and it avoids one f32->f64 conversion per element.
template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) RVec { T v[VEC]; };

// FAST keeps a plain fmaxf / fminf (which drop NaNs) plus a running sum whose only job is to turn NaN when
// the row holds one: a NaN sum sends the row through an exact second pass (clojure's max / min propagate
// NaN), so the common case costs two instructions per element.  Everything else keeps FOUR independent
// accumulators per thread (element k of a vector goes to accumulator k & 3): the dependent chain of fp64
// adds per load batch is a quarter as long.
template <typename T, typename A, bool FAST>
__device__ __forceinline__ void red_vec_accum(int op, A (&acc)[4], float& facc, float& fsum,
                                              const RVec<T, 16 / sizeof(T)>& v, A alpha, bool unit) {
  constexpr int VEC = 16 / sizeof(T);
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    if (FAST) {
      const float f = (float)v.v[k];
      facc = op == CB200_RMAX ? fmaxf(facc, f) : fminf(facc, f);
      fsum += f;
    } else {
      A e = unit ? (A)v.v[k] : (A)(alpha * (A)v.v[k]);
      acc[k & 3] = red_combine(op, acc[k & 3], red_elem(op, e));
    }
  }
}

template <typename T, int NWARPS, bool FAST>
__global__ void __launch_bounds__(256)
reduce_rows_vec(T* out, const T* in, Operand oo, Operand oi, Geometry go, Geometry gi, long long n_rows, int len,
                int op, typename acc_of<T>::type alpha) {
  typedef typename acc_of<T>::type A;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int U = 8;
  __shared__ A smem[8];
  __shared__ float fsmem[8];
  const int rows_per_block = NWARPS == 1 ? 8 : 1;
  const int tid = NWARPS == 1 ? (threadIdx.x & 31) : threadIdx.x;
  const int nthreads = NWARPS == 1 ? 32 : 256;
  const int nvec = len / VEC;
  const bool unit = alpha == (A)1;
  for (long long r0 = (long long)blockIdx.x * rows_per_block; r0 < n_rows; r0 += (long long)gridDim.x * rows_per_block) {
    long long r = NWARPS == 1 ? r0 + (threadIdx.x >> 5) : r0;
    A acc[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[k] = red_identity<A>(op);
    float facc = op == CB200_RMAX ? -INFINITY : INFINITY, fsum = 0.f;
    const RVec<T, VEC>* row = nullptr;
    if (r < n_rows) {
      row = reinterpret_cast<const RVec<T, VEC>*>(in + operand_offset(oi, gi, r * len));
      int j = tid;
      for (; j + (U - 1) * nthreads < nvec; j += U * nthreads) {
        RVec<T, VEC> v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          // read-once stream: evict-first loads (16 bytes whatever the element type)
          const float4 raw = __ldcs(reinterpret_cast<const float4*>(row + j + u * nthreads));
          v[u] = *reinterpret_cast<const RVec<T, VEC>*>(&raw);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) red_vec_accum<T, A, FAST>(op, acc, facc, fsum, v[u], alpha, unit);
      }
      for (; j < nvec; j += nthreads) {
        RVec<T, VEC> v0 = row[j];
        red_vec_accum<T, A, FAST>(op, acc, facc, fsum, v0, alpha, unit);
      }
    }
    A total;
    if (FAST) {
      // did any thread of the row see a NaN (or +inf and -inf together)?  then redo the row exactly
      float bad = fsum;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, d);
      if (NWARPS > 1) {
        __syncthreads();
        if ((threadIdx.x & 31) == 0) fsmem[threadIdx.x >> 5] = bad;
        __syncthreads();
        bad = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) bad += fsmem[w];
      }
      if (bad != bad && r < n_rows) {
        facc = op == CB200_RMAX ? -INFINITY : INFINITY;
        for (int j = tid; j < nvec; j += nthreads) {
          const RVec<T, VEC> v0 = row[j];
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            const float f = (float)v0.v[k];
            facc = op == CB200_RMAX ? clj_max(facc, f) : ((facc != facc) ? facc : ((f != f) ? f : (facc < f ? facc : f)));
          }
        }
      }
      total = (A)facc;
    } else {
      total = red_combine(op, red_combine(op, acc[0], acc[1]), red_combine(op, acc[2], acc[3]));
    }
    total = block_combine<A, NWARPS>(op, total, smem);
    if (tid == 0 && r < n_rows) out[operand_offset(oo, go, r)] = red_finish<T>(op, total, len);
  }
}

// Any layout: the reference's own shape, one thread per output element.
template <typename T>
__global__ void __launch_bounds__(256)
reduce_generic(T* out, const T* in, Operand oo, Operand oi, Geometry go, Geometry gi, long long n_rows, int len, int op,
               typename acc_of<T>::type alpha) {
  typedef typename acc_of<T>::type A;
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < n_rows;
       r += (long long)gridDim.x * blockDim.x) {
    A acc = red_elem(op, (A)(alpha * (A)in[operand_offset(oi, gi, r * len)]));
    for (int j = 1; j < len; ++j)
      acc = red_combine(op, acc, red_elem(op, (A)(alpha * (A)in[operand_offset(oi, gi, r * len + j)])));
    out[operand_offset(oo, go, r)] = red_finish<T>(op, acc, len);
  }
}

void geometry_of(Geometry& g, const Operand& o) {
  g.ndims = 1;
  for (int d = 0; d < 5; ++d) { g.max_shape[d] = o.shape[d]; if (o.shape[d] > 1) g.ndims = d + 1; }
}

// ------------------------------ softmax -------------------------------------
// Row r of a [rows, C] view with element stride cs inside the row and the row
// base given by (r / inner) * outer_stride + (r % inner) * inner_stride:
//   eltwise: inner = 1, outer_stride = row pitch, cs = 1
//   spatial [N, C, E] over C: inner = E, outer_stride = N-stride, inner_stride = E-stride, cs = C-stride
// Steps as softmax-impl (cpu/tensor_math.clj:1037-1088): m = max; e = exp(x - m)
// rounded to the element type; s = sum of the rounded e in double, rounded;
// y = e / s in the element type.
// fp32 rows: x - m in fp32 equals the double difference rounded once; the exponential is the
// hardware ex2 path (|rel err| ~ 1e-6 on the terms that matter), the row sum is a per-thread
// fp32 partial combined in double, and the divide is a multiply by the reciprocal: all within
// the 1e-4 parity bound, and the kernel stays on the HBM roofline.  fp64 rows follow the
// reference arithmetic exactly up to summation order.
template <typename T> __device__ __forceinline__ T sm_exp(T x, T m);
template <> __device__ __forceinline__ float sm_exp<float>(float x, float m) { return __expf(x - m); }
template <> __device__ __forceinline__ double sm_exp<double>(double x, double m) { return exp(x - m); }
template <typename T> __device__ __forceinline__ T sm_norm(T e, T s, T inv);
template <> __device__ __forceinline__ float sm_norm<float>(float e, float, float inv) { return e * inv; }
template <> __device__ __forceinline__ double sm_norm<double>(double e, double s, double) { return e / s; }

struct SoftmaxGeom {
  long long rows;
  int C;
  long long inner;
  long long in_outer, in_inner, in_cs;
  long long out_outer, out_inner, out_cs;
};

// One warp (NWARPS = 1) or CTA (NWARPS = 8) per row; the row lives in registers
// (PER values per thread), so x is read once and y written once.  VEC = 4 moves the row
// with 16-byte accesses (contiguous, aligned rows whose length is a multiple of 4).
template <int NWARPS>
__device__ __forceinline__ double block_all_reduce(int op, double v, double* slots) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = red_combine(op, v, __shfl_xor_sync(0xffffffffu, v, d));
  if (NWARPS == 1) return v;
  if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = v;
  __syncthreads();
  double r = slots[0];
#pragma unroll
  for (int w = 1; w < NWARPS; ++w) r = red_combine(op, r, slots[w]);
  return r;
}

template <typename T, int NWARPS, int PER, int VEC>
__global__ void __launch_bounds__(256)
softmax_rows(T* out, const T* in, SoftmaxGeom g) {
  __shared__ double slots_a[8], slots_b[8];
  const int rows_per_block = NWARPS == 1 ? 8 : 1;
  const int tid = NWARPS == 1 ? (threadIdx.x & 31) : threadIdx.x;
  const int nthreads = NWARPS == 1 ? 32 : 256;
  constexpr int NV = PER / VEC;
  for (long long r0 = (long long)blockIdx.x * rows_per_block; r0 < g.rows; r0 += (long long)gridDim.x * rows_per_block) {
    long long r = NWARPS == 1 ? r0 + (threadIdx.x >> 5) : r0;
    bool live = r < g.rows;
    long long rr = live ? r : 0;
    const T* x = in + (rr / g.inner) * g.in_outer + (rr % g.inner) * g.in_inner;
    T* y = out + (rr / g.inner) * g.out_outer + (rr % g.inner) * g.out_inner;
    T v[PER];
    // element k of chunk c sits at column (tid + c * nthreads) * VEC + k
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int j = (tid + c * nthreads) * VEC;
      if (VEC == 1) {
        if (live && j < g.C) v[c] = x[(long long)j * g.in_cs];
      } else if (live && j < g.C) {
        RVec<T, VEC> t = *reinterpret_cast<const RVec<T, VEC>*>(x + j);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[c * VEC + k] = t.v[k];
      }
    }
    T mloc = -INFINITY;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int j = (tid + c * nthreads) * VEC;
      if (live && j < g.C) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const T e = v[c * VEC + k];
          mloc = (mloc != mloc) ? mloc : ((e != e) ? e : (mloc > e ? mloc : e));
        }
      }
    }
    const T mt = (T)block_all_reduce<NWARPS>(CB200_RMAX, (double)mloc, slots_a);
    T sloc = (T)0;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int j = (tid + c * nthreads) * VEC;
      if (live && j < g.C) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) { v[c * VEC + k] = sm_exp<T>(v[c * VEC + k], mt); sloc += v[c * VEC + k]; }
      }
    }
    const double s = block_all_reduce<NWARPS>(CB200_RSUM, (double)sloc, slots_b);
    const T st = (T)s;
    const T inv = (T)1 / st;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int j = (tid + c * nthreads) * VEC;
      if (VEC == 1) {
        if (live && j < g.C) y[(long long)j * g.out_cs] = sm_norm<T>(v[c], st, inv);
      } else if (live && j < g.C) {
        RVec<T, VEC> t;
#pragma unroll
        for (int k = 0; k < VEC; ++k) t.v[k] = sm_norm<T>(v[c * VEC + k], st, inv);
        *reinterpret_cast<RVec<T, VEC>*>(y + j) = t;
      }
    }
    if (NWARPS != 1) __syncthreads();   // slots are reused by the next row
  }
}

// Rows too long for registers, or strided inner axis (spatial): one thread per
// row, three passes.  Adjacent threads take adjacent `inner` positions, which
// is the contiguous axis of a [N, C, E] tensor.
template <typename T>
__global__ void __launch_bounds__(256)
softmax_generic(T* out, const T* in, SoftmaxGeom g) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < g.rows;
       r += (long long)gridDim.x * blockDim.x) {
    const T* x = in + (r / g.inner) * g.in_outer + (r % g.inner) * g.in_inner;
    T* y = out + (r / g.inner) * g.out_outer + (r % g.inner) * g.out_inner;
    double m = (double)x[0];
    for (int j = 1; j < g.C; ++j) m = clj_max(m, (double)x[(long long)j * g.in_cs]);
    T mt = (T)m;
    double s = 0.0;
    for (int j = 0; j < g.C; ++j) {
      T e = sm_exp<T>(x[(long long)j * g.in_cs], mt);
      y[(long long)j * g.out_cs] = e;
      s = j == 0 ? (double)e : s + (double)e;
    }
    T st = (T)s;
    for (int j = 0; j < g.C; ++j) y[(long long)j * g.out_cs] = y[(long long)j * g.out_cs] / st;
  }
}

template <typename T>
int launch_softmax(cb200_stream* s, T* out, const T* in, const SoftmaxGeom& g) {
  if (g.rows <= 0 || g.C <= 0) return CB200_OK;
  DeviceGuard guard(s->device);
  long long cap = (long long)s->sm_count * 16;
  constexpr int V = 16 / sizeof(T);
  // 16-byte accesses need aligned rows: base, row pitch and length all multiples of V elements
  const bool vec = g.in_cs == 1 && g.out_cs == 1 && (g.C % V) == 0 && ((uintptr_t)in % 16) == 0 &&
                   ((uintptr_t)out % 16) == 0 && (g.in_outer % V) == 0 && (g.out_outer % V) == 0 &&
                   (g.in_inner % V) == 0 && (g.out_inner % V) == 0;
  if (g.in_cs == 1 && g.out_cs == 1 && g.C <= 32 * 32) {
    long long blocks = (g.rows + 7) / 8;
    if (blocks > cap) blocks = cap;
    if (g.C <= 32 * 4) softmax_rows<T, 1, 4, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
    else if (g.C <= 32 * 16) {
      if (vec) softmax_rows<T, 1, 16, V><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
      else softmax_rows<T, 1, 16, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
    } else {
      if (vec) softmax_rows<T, 1, 32, V><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
      else softmax_rows<T, 1, 32, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
    }
  } else if (g.in_cs == 1 && g.out_cs == 1 && g.C <= 256 * 32) {
    long long blocks = g.rows < cap ? g.rows : cap;
    if (g.C <= 256 * 8) {
      if (vec) softmax_rows<T, 8, 8, V><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
      else softmax_rows<T, 8, 8, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
    } else if (g.C <= 256 * 16) {
      if (vec) softmax_rows<T, 8, 16, V><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
      else softmax_rows<T, 8, 16, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
    } else {
      if (vec) softmax_rows<T, 8, 32, V><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
      else softmax_rows<T, 8, 32, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
    }
  } else {
    long long blocks = (g.rows + 255) / 256;
    if (blocks > cap) blocks = cap;
    softmax_generic<T><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g);
  }
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

// ---------------------- fused bias + ReLU + row max / sum --------------------
// One CTA per row, row in registers: X read once, Y written once.  VEC = 16 / sizeof(T) moves the
// row with 16-byte accesses when base pointers, pitches and the row length allow.
template <typename T, int PER, int VEC>
__global__ void __launch_bounds__(256)
bias_relu_rowstats_k(T* Y, long long ldy, const T* X, long long ldx, const T* bias, long long rows, int cols,
                     T* rowmax, T* rowsum) {
  __shared__ double slots_a[8], slots_b[8];
  constexpr int NV = PER / VEC;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* x = X + r * ldx;
    T* y = Y + r * ldy;
    T mx = -INFINITY, sum = (T)0;
    T v[PER], bv[PER];
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int j = (threadIdx.x + c * 256) * VEC;
      if (j < cols) {
        if (VEC == 1) { v[c] = x[j]; bv[c] = bias[j]; }
        else {
          RVec<T, VEC> t = *reinterpret_cast<const RVec<T, VEC>*>(x + j);
          RVec<T, VEC> tb = *reinterpret_cast<const RVec<T, VEC>*>(bias + j);
#pragma unroll
          for (int k = 0; k < VEC; ++k) { v[c * VEC + k] = t.v[k]; bv[c * VEC + k] = tb.v[k]; }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int j = (threadIdx.x + c * 256) * VEC;
      if (j < cols) {
        RVec<T, VEC> o;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const T t = v[c * VEC + k] + bv[c * VEC + k];   // binary-op! :+ (same value as the double sum rounded once)
          const T e = t > (T)0 ? t : (T)0;                // binary-op! :max with scalar 0
          o.v[k] = e;
          mx = (mx != mx) ? mx : ((e != e) ? e : (mx > e ? mx : e));
          sum += e;                                       // per-thread partial in the element type, combined in double
        }
        if (VEC == 1) y[j] = o.v[0];
        else *reinterpret_cast<RVec<T, VEC>*>(y + j) = o;
      }
    }
    const double mxd = block_all_reduce<8>(CB200_RMAX, (double)mx, slots_a);
    const double sumd = block_all_reduce<8>(CB200_RSUM, (double)sum, slots_b);
    if (threadIdx.x == 0 && rowmax) rowmax[r] = (T)mxd;
    if (threadIdx.x == 0 && rowsum) rowsum[r] = (T)sumd;
    __syncthreads();   // slots are reused by the next row
  }
}

}  // namespace

extern "C" {

int cb200_unary_reduce(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, double alpha,
                       const void* in, const cb200_dims* in_dims, int op) {
  CB_REQUIRE(s && out && out_dims && in && in_dims, "unary_reduce: null argument");
  CB_REQUIRE(op >= CB200_RMAX && op <= CB200_RMAGNITUDE_SQ, "unary_reduce: unknown op %d", op);
  int rc = cb200_check_dims(out_dims, "unary_reduce out");
  if (rc) return rc;
  rc = cb200_check_dims(in_dims, "unary_reduce in");
  if (rc) return rc;
  Operand oo, oi;
  operand_from_dims(oo, out_dims);
  operand_from_dims(oi, in_dims);
  Geometry go, gi;
  geometry_of(go, oo);
  geometry_of(gi, oi);
  long long n_out = 1, n_in = 1;
  for (int d = 0; d < 5; ++d) { n_out *= oo.shape[d]; n_in *= oi.shape[d]; }
  CB_REQUIRE(n_out > 0 && n_in % n_out == 0, "unary_reduce: output element count %lld does not divide input count %lld",
             n_out, n_in);
  long long len_ll = n_in / n_out;   // iter-amount, cpu/tensor_math.clj:641-643
  CB_REQUIRE(len_ll >= 1 && len_ll <= 2147483647LL, "unary_reduce: bad row length");
  int len = (int)len_ll;
  DeviceGuard guard(s->device);
  bool contiguous = !oi.index[0] && oi.shape[0] == len && (oi.stride[0] == 1 || len == 1);
  long long cap = (long long)s->sm_count * 16;
  CB_DISPATCH_DTYPE(dtype, T, {
    typedef typename acc_of<T>::type A;
    A a = scalar_as<T>(alpha);
    constexpr int VEC = 16 / sizeof(T);
    if (contiguous) {
      bool vec = (len % VEC) == 0 && ((uintptr_t)in % 16) == 0;
      for (int d = 1; d < gi.ndims && vec; ++d) if (oi.shape[d] > 1 && (oi.stride[d] % VEC) != 0) vec = false;
      // one warp per row while there are enough rows to occupy every SM, one CTA per row otherwise
      const bool cta_per_row = (size_t)len * sizeof(T) >= 2048 && n_out < (long long)s->sm_count * 32;
      const bool fast = sizeof(T) == 4 && dtype == CB200_FLOAT && (op == CB200_RMAX || op == CB200_RMIN) && a == (A)1;
      if (cta_per_row) {
        long long blocks = n_out < cap ? n_out : cap;
        if (vec && fast) reduce_rows_vec<T, 8, true><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)out, (const T*)in, oo, oi, go, gi, n_out, len, op, a);
        else if (vec) reduce_rows_vec<T, 8, false><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)out, (const T*)in, oo, oi, go, gi, n_out, len, op, a);
        else reduce_rows<T, 8><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)out, (const T*)in, oo, oi, go, gi, n_out, len, op, a);
      } else {
        long long blocks = (n_out + 7) / 8;
        if (blocks > cap) blocks = cap;
        if (vec && fast) reduce_rows_vec<T, 1, true><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)out, (const T*)in, oo, oi, go, gi, n_out, len, op, a);
        else if (vec) reduce_rows_vec<T, 1, false><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)out, (const T*)in, oo, oi, go, gi, n_out, len, op, a);
        else reduce_rows<T, 1><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)out, (const T*)in, oo, oi, go, gi, n_out, len, op, a);
      }
    } else {
      long long blocks = (n_out + 255) / 256;
      if (blocks > cap) blocks = cap;
      reduce_generic<T><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)out, (const T*)in, oo, oi, go, gi, n_out, len, op, a);
    }
    CB_LAUNCH_CHECK(s);
  });
  return CB200_OK;
}

static int softmax_entry(cb200_stream* s, int dtype, void* out, const cb200_dims* od, const void* in,
                         const cb200_dims* id, int spatial) {
  CB_REQUIRE(s && out && od && in && id, "softmax: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "softmax is only defined for float and double tensors");
  int rc = cb200_check_dims(od, "softmax out");
  if (rc) return rc;
  rc = cb200_check_dims(id, "softmax in");
  if (rc) return rc;
  for (int d = 0; d < 5; ++d) {
    CB_REQUIRE(!od->index[d] && !id->index[d], "softmax: index arrays are not supported");
    CB_REQUIRE(od->rev_shape[d] == id->rev_shape[d], "softmax: input and output shapes differ");
  }
  SoftmaxGeom g;
  if (!spatial) {
    // [rows, C]; anything above dim 1 must be trivial (softmax! passes as-batch-matrix views)
    for (int d = 2; d < 5; ++d) CB_REQUIRE(id->rev_shape[d] == 1, "softmax_eltwise expects a 2-d view");
    g.rows = id->rev_shape[1]; g.C = id->rev_shape[0]; g.inner = 1;
    g.in_outer = id->rev_strides[1]; g.in_inner = 0; g.in_cs = id->rev_strides[0];
    g.out_outer = od->rev_strides[1]; g.out_inner = 0; g.out_cs = od->rev_strides[0];
  } else {
    // [N, C, E]: softmax over C for every (n, e)
    for (int d = 3; d < 5; ++d) CB_REQUIRE(id->rev_shape[d] == 1, "softmax_spatial expects a 3-d view");
    long long N = id->rev_shape[2], E = id->rev_shape[0];
    g.rows = N * E; g.C = id->rev_shape[1]; g.inner = E;
    g.in_outer = id->rev_strides[2]; g.in_inner = id->rev_strides[0]; g.in_cs = id->rev_strides[1];
    g.out_outer = od->rev_strides[2]; g.out_inner = od->rev_strides[0]; g.out_cs = od->rev_strides[1];
  }
  if (g.C == 1) { g.in_cs = 1; g.out_cs = 1; }
  if (dtype == CB200_FLOAT) return launch_softmax<float>(s, (float*)out, (const float*)in, g);
  return launch_softmax<double>(s, (double*)out, (const double*)in, g);
}

int cb200_softmax_eltwise(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, const void* in,
                          const cb200_dims* in_dims) {
  return softmax_entry(s, dtype, out, out_dims, in, in_dims, 0);
}

int cb200_softmax_spatial(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, const void* in,
                          const cb200_dims* in_dims) {
  return softmax_entry(s, dtype, out, out_dims, in, in_dims, 1);
}

int cb200_bias_relu_rowstats(cb200_stream* s, int dtype, void* Y, int64_t ldy, const void* X, int64_t ldx,
                             const void* bias, int64_t rows, int64_t cols, void* rowmax, void* rowsum) {
  CB_REQUIRE(s && Y && X && bias, "bias_relu_rowstats: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "bias_relu_rowstats: float and double only");
  CB_REQUIRE(rows >= 0 && cols >= 1 && cols <= 256 * 32, "bias_relu_rowstats: cols must be in [1, 8192]");
  CB_REQUIRE(ldx >= cols && ldy >= cols, "bias_relu_rowstats: row pitch smaller than the row");
  if (rows == 0) return CB200_OK;
  DeviceGuard guard(s->device);
  long long cap = (long long)s->sm_count * 16;
  unsigned blocks = (unsigned)(rows < cap ? rows : cap);
#define CB_BRS_ARGS(T) (T*)Y, ldy, (const T*)X, ldx, (const T*)bias, rows, (int)cols, (T*)rowmax, (T*)rowsum
#define CB_BRS(T)                                                                                          \
  do {                                                                                                     \
    constexpr int V = 16 / sizeof(T);                                                                      \
    const bool vec = (cols % V) == 0 && (ldx % V) == 0 && (ldy % V) == 0 && ((uintptr_t)X % 16) == 0 &&    \
                     ((uintptr_t)Y % 16) == 0 && ((uintptr_t)bias % 16) == 0;                              \
    if (cols <= 256 * 8) { if (vec) bias_relu_rowstats_k<T, 8, V><<<blocks, 256, 0, s->stream>>>(CB_BRS_ARGS(T)); \
                           else bias_relu_rowstats_k<T, 8, 1><<<blocks, 256, 0, s->stream>>>(CB_BRS_ARGS(T)); }  \
    else if (cols <= 256 * 16) { if (vec) bias_relu_rowstats_k<T, 16, V><<<blocks, 256, 0, s->stream>>>(CB_BRS_ARGS(T)); \
                                 else bias_relu_rowstats_k<T, 16, 1><<<blocks, 256, 0, s->stream>>>(CB_BRS_ARGS(T)); } \
    else { if (vec) bias_relu_rowstats_k<T, 32, V><<<blocks, 256, 0, s->stream>>>(CB_BRS_ARGS(T));          \
           else bias_relu_rowstats_k<T, 32, 1><<<blocks, 256, 0, s->stream>>>(CB_BRS_ARGS(T)); }            \
  } while (0)
  if (dtype == CB200_FLOAT) CB_BRS(float); else CB_BRS(double);
#undef CB_BRS
#undef CB_BRS_ARGS
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // extern "C"
