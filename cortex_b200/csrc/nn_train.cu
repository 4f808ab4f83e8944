// The layer-gradient methods of the tensor-math protocol that the training path of a convolutional
// network calls next to the convolution gradients:
//   pooling-backward!                          src/cortex/tensor/math.clj:223-236
//   batch-normalize-update-and-apply-*!        src/cortex/tensor/math.clj:137-158
//   batch-normalize-gradients-*!               src/cortex/tensor/math.clj:159-174
// Arithmetic after the reference CPU backend (src/cortex/compute/cpu/tensor_math.clj:820-1032 and
// :1175-1284): every expression is evaluated in double and rounded to the element type where the
// reference stores or casts.
//
// Pooling backward is written in gather form: one thread per INPUT element walks the output positions whose
// window covers it, in (out-y, out-x) order, which is the order in which the reference's scatter loop
// (src/cortex/nn/impl.clj:8-107) reaches that element; so the running sum sees the same partial sums and
// the result is bit-identical, with no atomics.
//
// The batch-normalisation statistics are sums over (batch x element) per channel.  Elementwise form: one
// thread per column, rows visited in order (coalesced across threads, and the same summation order as the
// reference).  Spatial form: (channel x batch-slab) CTAs write double partial sums, a small kernel combines them
// in slab order (the summation order differs from the reference's sequential loop: results agree to rounding
// of the double sums).
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------------------
// pooling backward
// ------------------------------------------------------------------------------------------------------
struct PoolBwdGeom {
  int in_h, in_w, out_h, out_w, kw, kh, pad_x, pad_y, stride_x, stride_y;
};

__device__ __forceinline__ int floor_div(int a, int b) {   // b > 0
  int q = a / b;
  return (a % b != 0 && a < 0) ? q - 1 : q;
}

// VEC consecutive input columns per thread (VEC = 4 floats / 2 doubles with 16-byte accesses when the rows allow,
// else 1): the index decomposition and the output-row range are shared, the output / output-gradient values the
// neighbouring columns read come from the same cache lines.
// KS / ST: square window size and common stride as compile-time constants (0 = read from the geometry): the
// divisions by the stride become shifts and the window loops unroll.
template <typename T, int OP, int VEC, int KS, int ST>
__global__ void __launch_bounds__(256)
pooling_backward_kernel(T* in_grad, const T* in, const T* out, const T* out_grad, PoolBwdGeom gg, long long n_groups,
                        double in_grad_alpha) {
  PoolBwdGeom g = gg;
  if (KS) { g.kw = KS; g.kh = KS; }
  if (ST) { g.stride_x = ST; g.stride_y = ST; }
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  const int groups_per_row = g.in_w / VEC;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups; i += (long long)gridDim.x * blockDim.x) {
    const unsigned iu = (unsigned)i;
    const unsigned tq = iu / (unsigned)groups_per_row;
    const int ix0 = (int)(iu - tq * (unsigned)groups_per_row) * VEC;
    const unsigned plane = tq / (unsigned)g.in_h;
    const int iy = (int)(tq - plane * (unsigned)g.in_h);
    const long long e0 = ((long long)plane * g.in_h + iy) * g.in_w + ix0;
    const long long out_base = (long long)plane * g.out_h * g.out_w;
    // output rows whose window [o*stride - pad, o*stride - pad + k) holds iy
    const int oy0 = max(0, floor_div(iy + g.pad_y - g.kh + g.stride_y, g.stride_y));   // ceil((iy+pad-kh+1)/stride)
    const int oy1 = min(g.out_h - 1, (iy + g.pad_y) / g.stride_y);
    Pack x, acc;
    if (OP == CB200_POOL_MAX) x = *reinterpret_cast<const Pack*>(in + e0);
    if (in_grad_alpha == 0.0) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc.v[e] = (T)0;
    } else {
      acc = *reinterpret_cast<const Pack*>(in_grad + e0);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc.v[e] = (T)(in_grad_alpha * (double)acc.v[e]);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const int ix = ix0 + e;
      const int ox0 = max(0, floor_div(ix + g.pad_x - g.kw + g.stride_x, g.stride_x));
      const int ox1 = min(g.out_w - 1, (ix + g.pad_x) / g.stride_x);
      T a = acc.v[e];
      for (int oy = oy0; oy <= oy1; ++oy) {
        int exc_h = 0;
        if (OP == CB200_POOL_AVG_EXC_PAD) {
          const int rel_y = oy * g.stride_y - g.pad_y;
          exc_h = min(rel_y + g.kh, g.in_h) - max(rel_y, 0);
        }
        for (int ox = ox0; ox <= ox1; ++ox) {
          const long long o = out_base + (long long)oy * g.out_w + ox;
          if (OP == CB200_POOL_MAX) {
            // a + b in the element type IS the rounded exact sum: the reference's double add followed by its cast
            if (x.v[e] == out[o]) a = a + out_grad[o];
          } else if (OP == CB200_POOL_AVG) {
            a = (T)((double)a + (double)out_grad[o] / (double)(g.kw * g.kh));
          } else {
            const int rel_x = ox * g.stride_x - g.pad_x;
            const int exc_w = min(rel_x + g.kw, g.in_w) - max(rel_x, 0);
            a = (T)((double)a + (double)out_grad[o] / (double)(exc_w * exc_h));
          }
        }
      }
      acc.v[e] = a;
    }
    *reinterpret_cast<Pack*>(in_grad + e0) = acc;
  }
}

// Square window KS with stride ST known at compile time, and the horizontal padding's remainder PADP = pad_x % ST
// (the same for every thread: a thread's first column is a multiple of VEC, itself a multiple of ST).  An input
// position lies in at most NW = ceil(KS / ST) windows per dimension.  With PADP fixed, WHICH windows element e of
// a thread's VEC columns belongs to is known at compile time -- column (e + PADP) % ST of window q - dx,
// q = (e + PADP) / ST, for every dx with (e + PADP) % ST + dx * ST < KS -- so a thread loads each of the NJ
// distinct (output, output gradient) pairs of a window row once (3 instead of 8 per row for 3 x 3 / 2) and the
// inner loop is compares and adds only.  Windows are visited in ascending (out-y, out-x) order per element: the
// reference's summation order.  32-bit index arithmetic.
template <typename T, int OP, int VEC, int KS, int ST, int PADP>
__global__ void __launch_bounds__(256)
pooling_backward_fixed_kernel(T* in_grad, const T* in, const T* out, const T* out_grad, PoolBwdGeom g, long long n_groups,
                              double in_grad_alpha) {
  static_assert(VEC % ST == 0 && PADP < ST, "a thread's first column must be a multiple of the stride");
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  constexpr int NW = (KS + ST - 1) / ST;
  constexpr int JMIN = PADP / ST - (NW - 1);          // window offsets (relative to `wbase`) a thread can touch
  constexpr int JMAX = (VEC - 1 + PADP) / ST;
  constexpr int NJ = JMAX - JMIN + 1;
  const unsigned groups_per_row = (unsigned)(g.in_w / VEC);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups; i += (long long)gridDim.x * blockDim.x) {
    const unsigned iu = (unsigned)i;
    const unsigned tq = iu / groups_per_row;
    const int ix0 = (int)(iu - tq * groups_per_row) * VEC;
    const unsigned plane = tq / (unsigned)g.in_h;
    const int iy = (int)(tq - plane * (unsigned)g.in_h);
    const unsigned e0 = (plane * (unsigned)g.in_h + (unsigned)iy) * (unsigned)g.in_w + (unsigned)ix0;
    const unsigned out_base = plane * (unsigned)(g.out_h * g.out_w);
    const int oyh = (iy + g.pad_y) / ST;
    const int wbase = (ix0 + g.pad_x - PADP) / ST;    // exact: (ix0 + pad_x) % ST == PADP
    Pack x, acc;
    if (OP == CB200_POOL_MAX) x = *reinterpret_cast<const Pack*>(in + e0);
    if (in_grad_alpha == 0.0) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc.v[e] = (T)0;
    } else {
      acc = *reinterpret_cast<const Pack*>(in_grad + e0);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc.v[e] = (T)(in_grad_alpha * (double)acc.v[e]);
    }
#pragma unroll
    for (int dy = NW - 1; dy >= 0; --dy) {
      const int oy = oyh - dy;
      const int rel_y = oy * ST - g.pad_y;
      const bool ok_y = oy >= 0 && oy < g.out_h && iy - rel_y < KS;
      if (!ok_y) continue;
      const int exc_h = min(rel_y + KS, g.in_h) - max(rel_y, 0);
      const unsigned row_base = out_base + (unsigned)(oy * g.out_w);
      T ov[NJ], gv[NJ];
      int cnt[NJ];                                     // AVG_EXC_PAD: input positions the window really covers
      bool ok[NJ];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int ox = wbase + JMIN + j;
        ok[j] = ox >= 0 && ox < g.out_w;
        ov[j] = (T)0; gv[j] = (T)0; cnt[j] = 1;
        if (ok[j]) {
          if (OP == CB200_POOL_MAX) ov[j] = out[row_base + (unsigned)ox];
          gv[j] = out_grad[row_base + (unsigned)ox];
          if (OP == CB200_POOL_AVG_EXC_PAD) {
            const int rel_x = ox * ST - g.pad_x;
            cnt[j] = (min(rel_x + KS, g.in_w) - max(rel_x, 0)) * exc_h;
          }
        }
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const int r = (e + PADP) % ST, q = (e + PADP) / ST;             // constants once unrolled
#pragma unroll
        for (int dx = NW - 1; dx >= 0; --dx) {
          if (r + dx * ST < KS) {
            const int j = q - dx - JMIN;
            if (ok[j]) {
              if (OP == CB200_POOL_MAX) {
                // a + b in the element type IS the rounded exact sum: the reference's double add and its cast
                if (x.v[e] == ov[j]) acc.v[e] = acc.v[e] + gv[j];
              } else if (OP == CB200_POOL_AVG) {
                acc.v[e] = (T)((double)acc.v[e] + (double)gv[j] / (double)(KS * KS));
              } else {
                acc.v[e] = (T)((double)acc.v[e] + (double)gv[j] / (double)cnt[j]);
              }
            }
          }
        }
      }
    }
    *reinterpret_cast<Pack*>(in_grad + e0) = acc;
  }
}

template <typename T, int OP, int VEC, int KS, int ST>
void pooling_backward_fixed_launch(cb200_stream* s, unsigned blocks, T* in_grad, const T* in, const T* out, const T* out_grad,
                                   const PoolBwdGeom& g, long long n_groups, double alpha) {
  // the padding's remainder modulo the stride is a template constant of the kernel (0 or 1: strides 1 and 2)
  if (ST == 1 || (g.pad_x % ST) == 0)
    pooling_backward_fixed_kernel<T, OP, VEC, KS, ST, 0><<<blocks, 256, 0, s->stream>>>(in_grad, in, out, out_grad, g, n_groups, alpha);
  else
    pooling_backward_fixed_kernel<T, OP, VEC, KS, ST, (ST > 1 ? 1 : 0)><<<blocks, 256, 0, s->stream>>>(in_grad, in, out, out_grad, g, n_groups, alpha);
}

template <typename T, int VEC, int KS, int ST>
void pooling_backward_launch_v(cb200_stream* s, int op, T* in_grad, const T* in, const T* out, const T* out_grad,
                               const PoolBwdGeom& g, long long n_in, double alpha) {
  const long long n_groups = n_in / VEC;
  long long blocks = (n_groups + 255) / 256;
  const long long cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  const unsigned b = (unsigned)blocks;
  if constexpr (KS > 0) {
    static_assert(ST == 1 || ST == 2, "fixed-window kernels exist for strides 1 and 2");
    if (op == CB200_POOL_MAX)
      pooling_backward_fixed_launch<T, CB200_POOL_MAX, VEC, KS, ST>(s, b, in_grad, in, out, out_grad, g, n_groups, alpha);
    else if (op == CB200_POOL_AVG)
      pooling_backward_fixed_launch<T, CB200_POOL_AVG, VEC, KS, ST>(s, b, in_grad, in, out, out_grad, g, n_groups, alpha);
    else
      pooling_backward_fixed_launch<T, CB200_POOL_AVG_EXC_PAD, VEC, KS, ST>(s, b, in_grad, in, out, out_grad, g, n_groups, alpha);
    return;
  } else {
    if (op == CB200_POOL_MAX)
      pooling_backward_kernel<T, CB200_POOL_MAX, VEC, KS, ST><<<b, 256, 0, s->stream>>>(in_grad, in, out, out_grad, g, n_groups, alpha);
    else if (op == CB200_POOL_AVG)
      pooling_backward_kernel<T, CB200_POOL_AVG, VEC, KS, ST><<<b, 256, 0, s->stream>>>(in_grad, in, out, out_grad, g, n_groups, alpha);
    else
      pooling_backward_kernel<T, CB200_POOL_AVG_EXC_PAD, VEC, KS, ST><<<b, 256, 0, s->stream>>>(in_grad, in, out, out_grad, g, n_groups, alpha);
  }
}

template <typename T>
void pooling_backward_launch(cb200_stream* s, int op, T* in_grad, const T* in, const T* out, const T* out_grad,
                             const PoolBwdGeom& g, long long n_in, double alpha) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const bool vec = (g.in_w % VEC) == 0 && ((((uintptr_t)in_grad) | ((uintptr_t)in)) & 15) == 0;
  const bool square = g.kw == g.kh && g.stride_x == g.stride_y;
  if (vec && square && g.kw == 3 && g.stride_x == 2) pooling_backward_launch_v<T, VEC, 3, 2>(s, op, in_grad, in, out, out_grad, g, n_in, alpha);
  else if (vec && square && g.kw == 2 && g.stride_x == 2) pooling_backward_launch_v<T, VEC, 2, 2>(s, op, in_grad, in, out, out_grad, g, n_in, alpha);
  else if (vec && square && g.kw == 3 && g.stride_x == 1) pooling_backward_launch_v<T, VEC, 3, 1>(s, op, in_grad, in, out, out_grad, g, n_in, alpha);
  else if (vec) pooling_backward_launch_v<T, VEC, 0, 0>(s, op, in_grad, in, out, out_grad, g, n_in, alpha);
  else pooling_backward_launch_v<T, 1, 0, 0>(s, op, in_grad, in, out, out_grad, g, n_in, alpha);
}

// ------------------------------------------------------------------------------------------------------
// batch normalisation: statistics update and gradients
// ------------------------------------------------------------------------------------------------------
// (parallel index, running index) -> element offset; the reference's BNEltwiseOffsetter / BNSpatialOffsetter
// (src/cortex/compute/cpu/tensor_math.clj:716-756)
struct BnShape {
  long long batch;      // rows before the channel dimension
  int channels;         // parallel count
  int inner;            // elements per (row, channel): 1 in the elementwise form
  __device__ __forceinline__ long long count() const { return batch * inner; }
  __device__ __forceinline__ long long offset(int c, long long idx) const {
    const long long b = idx / inner;
    const int e = (int)(idx - b * inner);
    return (b * channels + c) * (long long)inner + e;
  }
};

constexpr int BN_TEAM = 512;

// Sum of one value per thread over the team that owns a parallel index: the thread itself (TEAM == 1) or
// the whole CTA (every thread receives the total).
template <int TEAM>
__device__ __forceinline__ double team_sum(double v, double* sh) {
  if (TEAM == 1) return v;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                      // sh may still be read by the previous call
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  double t = 0.0;
#pragma unroll
  for (int w = 0; w < TEAM / 32; ++w) t += sh[w];   // the same order in every thread
  return t;
}

template <typename T, int TEAM>
__global__ void __launch_bounds__(TEAM == 1 ? 128 : TEAM)
bn_update_kernel(const T* __restrict__ in, T* batch_means, T* batch_variances, T* running_means, T* running_variances,
                 double average_factor, BnShape sh) {
  __shared__ double red[32];
  const int c = TEAM == 1 ? (int)(blockIdx.x * blockDim.x + threadIdx.x) : (int)blockIdx.x;
  if (TEAM == 1 && c >= sh.channels) return;
  const long long count = sh.count();
  const int t0 = TEAM == 1 ? 0 : (int)threadIdx.x;
  const double factor = (double)(T)average_factor;
  const double lerp = (double)(T)1.0 - factor;
  const double n = count > 1 ? (double)count : 1.0;
  const double n_running = n - 1.0 > 1.0 ? n - 1.0 : 1.0;
  double sum = 0.0;
  for (long long idx = t0; idx < count; idx += TEAM) sum += (double)in[sh.offset(c, idx)];
  sum = team_sum<TEAM>(sum, red);
  const T new_mean = (T)(sum / n);
  double var = 0.0;
  for (long long idx = t0; idx < count; idx += TEAM) {
    const double d = (double)new_mean - (double)in[sh.offset(c, idx)];
    var = __dadd_rn(var, __dmul_rn(d, d));
  }
  var = team_sum<TEAM>(var, red);
  if (TEAM == 1 || threadIdx.x == 0) {
    const double mean_old = (double)running_means[c], var_old = (double)running_variances[c];
    batch_means[c] = new_mean;
    batch_variances[c] = (T)(var / n);
    running_means[c] = (T)(__dmul_rn(mean_old, lerp) + __dmul_rn((double)new_mean, factor));
    running_variances[c] = (T)(__dmul_rn(var_old, lerp) + __dmul_rn((double)(T)(var / n_running), factor));
  }
}

template <typename T, int TEAM>
__global__ void __launch_bounds__(TEAM == 1 ? 128 : TEAM)
bn_gradients_kernel(T* in_grad, T* scale_grad, T* bias_grad, const T* out_grad, const T* in,
                    const T* __restrict__ batch_means, const T* __restrict__ batch_variances,
                    const T* __restrict__ scale, double epsilon, BnShape sh) {
  __shared__ double red[32];
  const int c = TEAM == 1 ? (int)(blockIdx.x * blockDim.x + threadIdx.x) : (int)blockIdx.x;
  if (TEAM == 1 && c >= sh.channels) return;
  const long long count = sh.count();
  const int t0 = TEAM == 1 ? 0 : (int)threadIdx.x;
  const double g = (double)scale[c];
  const double variance = (double)(T)epsilon + (double)batch_variances[c];
  const double inv_std = 1.0 / sqrt(variance);
  const double mean = (double)batch_means[c];
  const double d_var = (double)(T)(-0.5 * pow(variance, -1.5));
  // pass 1: bias gradient, scale gradient, and the three sums of the input gradient
  double s_og = 0.0, s_og_xhat = 0.0, s_dvar = 0.0, s_dmean = 0.0, s_centered = 0.0;
  for (long long idx = t0; idx < count; idx += TEAM) {
    const long long o = sh.offset(c, idx);
    const double og = (double)out_grad[o];
    const double centered = (double)in[o] - mean;
    const double dxhat = (double)(T)__dmul_rn(g, og);          // the reference stores it in the input gradient
    s_og += og;
    s_og_xhat += __dmul_rn(og, __dmul_rn(centered, inv_std));
    s_dvar += __dmul_rn(__dmul_rn(dxhat, centered), d_var);
    s_dmean += __dmul_rn(-dxhat, inv_std);
    s_centered += __dmul_rn(-2.0, centered);
  }
  s_og = team_sum<TEAM>(s_og, red);
  s_og_xhat = team_sum<TEAM>(s_og_xhat, red);
  s_dvar = team_sum<TEAM>(s_dvar, red);
  s_dmean = team_sum<TEAM>(s_dmean, red);
  s_centered = team_sum<TEAM>(s_centered, red);
  if (TEAM == 1 || threadIdx.x == 0) {
    bias_grad[c] = (T)s_og;
    scale_grad[c] = (T)s_og_xhat;
  }
  const double d_var_d_out = (double)(T)s_dvar;
  const double d_mean_d_out = (double)(T)(s_dmean + __dmul_rn(d_var_d_out, s_centered / (double)count));
  const double one_over_count = 1.0 / (double)count;
  // pass 2: the input gradient
  const double part3 = __dmul_rn(d_mean_d_out, one_over_count);
  for (long long idx = t0; idx < count; idx += TEAM) {
    const long long o = sh.offset(c, idx);
    const double dxhat = (double)(T)__dmul_rn(g, (double)out_grad[o]);
    const double centered = (double)in[o] - mean;
    const double part1 = __dmul_rn(dxhat, inv_std);
    const double part2 = __dmul_rn(__dmul_rn(__dmul_rn(d_var_d_out, 2.0), centered), one_over_count);
    in_grad[o] = (T)__dadd_rn(__dadd_rn(part1, part2), part3);
  }
}

// ---- spatial form at scale: (channel x batch-slab) CTAs write partial sums, a small kernel combines them ----
// A row = the `inner` contiguous elements of one (batch entry, channel).  CTA (c, s) walks the rows of channel c
// whose batch entry lies in slab s with 16-byte loads; partial sums are doubles in the stream's scratch,
// combined per channel in slab order (deterministic).
constexpr int BN_SLAB_THREADS = 256;

template <typename T>
struct BnVec { T v[16 / sizeof(T)]; };

// one value per thread -> CTA total in thread 0 (others: undefined)
__device__ __forceinline__ double slab_reduce(double v, double* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
  if (threadIdx.x == 0)
    for (int w = 0; w < BN_SLAB_THREADS / 32; ++w) t += sh[w];
  return t;
}

// What the CTA that completes a channel's sums writes (the other slabs' CTAs have parked theirs): the statistics of
// the update pass, or the gradients of scale / bias and the five coefficients of the input-gradient pass.
template <typename T>
struct BnFinish {
  T* batch_means; T* batch_variances; T* running_means; T* running_variances;   // MODE 0 / 1
  double average_factor;
  double* coef; T* scale_grad; T* bias_grad;                                    // MODE 2
  long long count;
  int* counters;            // one per channel, zero between launches
};

// MODE 0: batch mean;  1: batch variance + running statistics;  2: per channel bias / scale gradient and the
// coefficients {g, inv_std, mean, d_var_d_out, part3} of the input-gradient pass
template <typename T, int MODE>
__device__ __forceinline__ void bn_finish_channel(const double* sums, int c, const BnFinish<T>& f, const T* means,
                                                  const T* variances, const T* scale, double epsilon) {
  const double n = f.count > 1 ? (double)f.count : 1.0;
  if (MODE == 0) {
    f.batch_means[c] = (T)(sums[0] / n);
  } else if (MODE == 1) {
    const double factor = (double)(T)f.average_factor, lerp = (double)(T)1.0 - factor;
    const double n_running = n - 1.0 > 1.0 ? n - 1.0 : 1.0;
    const double mean_old = (double)f.running_means[c], var_old = (double)f.running_variances[c];
    const double new_mean = (double)f.batch_means[c];
    f.batch_variances[c] = (T)(sums[0] / n);
    f.running_means[c] = (T)(__dmul_rn(mean_old, lerp) + __dmul_rn(new_mean, factor));
    f.running_variances[c] = (T)(__dmul_rn(var_old, lerp) + __dmul_rn((double)(T)(sums[0] / n_running), factor));
  } else {
    const double variance = (double)(T)epsilon + (double)variances[c];
    const double inv_std = 1.0 / sqrt(variance);
    f.bias_grad[c] = (T)sums[0];
    f.scale_grad[c] = (T)sums[1];
    const double d_var_d_out = (double)(T)sums[2];
    const double d_mean_d_out = (double)(T)(sums[3] + __dmul_rn(d_var_d_out, sums[4] / (double)f.count));
    const double one_over_count = 1.0 / (double)f.count;
    double* k = f.coef + (long long)c * 5;
    k[0] = (double)scale[c]; k[1] = inv_std; k[2] = (double)means[c]; k[3] = d_var_d_out;
    k[4] = __dmul_rn(d_mean_d_out, one_over_count);
  }
}

// NQ sums per (channel, slab).  MODE 0: {x};  1: {(mean - x)^2};  2: the five sums of the gradient pass.
// Every CTA parks its sums and takes a ticket of its channel's counter; the CTA that takes the last one adds the
// parked sums in slab order (a warp loads them side by side, lane 0 adds them in order: the same value whichever
// CTA that is) and writes the channel's results -- no separate finishing launch, and nobody waits.
template <typename T, int MODE, bool VECTOR>
__global__ void __launch_bounds__(BN_SLAB_THREADS)
bn_slab_sums_kernel(double* partial, const T* __restrict__ in, const T* out_grad, const T* __restrict__ means,
                    const T* __restrict__ variances, const T* __restrict__ scale, double epsilon, long long batch,
                    int channels, int inner, int slabs, BnFinish<T> fin) {
  constexpr int NQ = MODE == 2 ? 5 : 1;
  constexpr int VEC = VECTOR ? 16 / (int)sizeof(T) : 1;
  __shared__ double red[BN_SLAB_THREADS / 32];
  __shared__ int is_last;
  const int c = blockIdx.y, slab = blockIdx.x;
  const long long b0 = batch * slab / slabs, b1 = batch * (slab + 1) / slabs;
  const double mean = MODE >= 1 ? (double)means[c] : 0.0;
  double g = 0.0, inv_std = 0.0, d_var = 0.0;
  if (MODE == 2) {
    g = (double)scale[c];
    const double variance = (double)(T)epsilon + (double)variances[c];
    inv_std = 1.0 / sqrt(variance);
    d_var = (double)(T)(-0.5 * pow(variance, -1.5));
  }
  double acc[NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) acc[q] = 0.0;
  const int nvec = inner / VEC;
  for (long long b = b0; b < b1; ++b) {
    const long long base = (b * channels + c) * (long long)inner;
    for (int j = threadIdx.x; j < nvec; j += BN_SLAB_THREADS) {
      T x[VEC], og[VEC];
      if (VECTOR) {
        *reinterpret_cast<BnVec<T>*>(x) = *reinterpret_cast<const BnVec<T>*>(in + base + (long long)j * VEC);
        if (MODE == 2) *reinterpret_cast<BnVec<T>*>(og) = *reinterpret_cast<const BnVec<T>*>(out_grad + base + (long long)j * VEC);
      } else {
        x[0] = in[base + j];
        if (MODE == 2) og[0] = out_grad[base + j];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        if (MODE == 0) acc[0] += (double)x[e];
        else if (MODE == 1) { const double d = mean - (double)x[e]; acc[0] = __dadd_rn(acc[0], __dmul_rn(d, d)); }
        else {
          const double o = (double)og[e], centered = (double)x[e] - mean;
          const double dxhat = (double)(T)__dmul_rn(g, o);
          acc[0] += o;
          acc[1] += __dmul_rn(o, __dmul_rn(centered, inv_std));
          acc[2] += __dmul_rn(__dmul_rn(dxhat, centered), d_var);
          acc[3] += __dmul_rn(-dxhat, inv_std);
          acc[4] += __dmul_rn(-2.0, centered);
        }
      }
    }
  }
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const double t = slab_reduce(acc[q], red);
    if (threadIdx.x == 0) partial[((long long)q * channels + c) * slabs + slab] = t;
  }
  if (threadIdx.x == 0) {
    __threadfence();                                   // this CTA's sums, before its ticket
    is_last = atomicAdd(fin.counters + c, 1) == slabs - 1;
  }
  __syncthreads();
  if (!is_last || threadIdx.x >= 32) return;
  __threadfence();
  const int lane = threadIdx.x;
  double tot[NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) tot[q] = 0.0;
  for (int s0 = 0; s0 < slabs; s0 += 32) {
    double v[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q)
      v[q] = s0 + lane < slabs ? __ldcg(partial + ((long long)q * channels + c) * slabs + s0 + lane) : 0.0;
    const int nn = min(32, slabs - s0);
    for (int l = 0; l < nn; ++l)
#pragma unroll
      for (int q = 0; q < NQ; ++q) tot[q] += __shfl_sync(0xffffffffu, v[q], l);
  }
  if (lane == 0) {
    bn_finish_channel<T, MODE>(tot, c, fin, means, variances, scale, epsilon);
    fin.counters[c] = 0;                               // left zero for the next launch
  }
}

// input gradient: one CTA walks rows (batch entry, channel); the channel's coefficients are uniform per row
template <typename T, bool VECTOR>
__global__ void __launch_bounds__(BN_SLAB_THREADS)
bn_input_gradient_kernel(T* in_grad, const T* out_grad, const T* in, const double* __restrict__ coef, long long n_rows,
                         int channels, int inner, double one_over_count) {
  constexpr int VEC = VECTOR ? 16 / (int)sizeof(T) : 1;
  const int nvec = inner / VEC;
  for (long long r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const double* k = coef + (r % channels) * 5;
    const double g = k[0], inv_std = k[1], mean = k[2], dv2 = __dmul_rn(k[3], 2.0), part3 = k[4];
    const long long base = r * (long long)inner;
    for (int j = threadIdx.x; j < nvec; j += BN_SLAB_THREADS) {
      T x[VEC], og[VEC], res[VEC];
      if (VECTOR) {
        *reinterpret_cast<BnVec<T>*>(x) = *reinterpret_cast<const BnVec<T>*>(in + base + (long long)j * VEC);
        *reinterpret_cast<BnVec<T>*>(og) = *reinterpret_cast<const BnVec<T>*>(out_grad + base + (long long)j * VEC);
      } else {
        x[0] = in[base + j];
        og[0] = out_grad[base + j];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const double dxhat = (double)(T)__dmul_rn(g, (double)og[e]);
        const double centered = (double)x[e] - mean;
        const double part1 = __dmul_rn(dxhat, inv_std);
        const double part2 = __dmul_rn(__dmul_rn(dv2, centered), one_over_count);
        res[e] = (T)__dadd_rn(__dadd_rn(part1, part2), part3);
      }
      if (VECTOR) *reinterpret_cast<BnVec<T>*>(in_grad + base + (long long)j * VEC) = *reinterpret_cast<BnVec<T>*>(res);
      else in_grad[base + j] = res[0];
    }
  }
}

static int bn_slab_count(const cb200_stream* s, long long batch, long long channels) {
  long long slabs = ((long long)s->sm_count * 6 + channels - 1) / channels;
  if (slabs > batch) slabs = batch;
  if (slabs < 1) slabs = 1;
  if (slabs > 1024) slabs = 1024;
  return (int)slabs;
}

int bn_train_check(cb200_stream* s, int dtype, int64_t batch, int64_t channels, int64_t inner, const char* what) {
  CB_REQUIRE(s, "%s: null stream", what);
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "batch-normalization is only defined for float and double tensors");
  CB_REQUIRE(batch >= 0 && channels >= 1 && inner >= 1 && channels <= 2147483647LL && inner <= 2147483647LL,
             "%s: bad extents", what);
  CB_REQUIRE(batch * channels * inner < 4294967296LL, "%s: more than 2^32 - 1 elements", what);
  return CB200_OK;
}

template <typename T>
int bn_update_launch(cb200_stream* s, const void* in, void* bm, void* bv, void* rm, void* rv, double factor,
                     int64_t batch, int64_t channels, int64_t inner) {
  DeviceGuard guard(s->device);
  BnShape sh{batch, (int)channels, (int)inner};
  if (inner == 1) {
    bn_update_kernel<T, 1><<<(unsigned)((channels + 127) / 128), 128, 0, s->stream>>>(
        (const T*)in, (T*)bm, (T*)bv, (T*)rm, (T*)rv, factor, sh);
    CB_LAUNCH_CHECK(s);
    return CB200_OK;
  }
  if (channels > 65535) {      // grid.y limit: the one-CTA-per-channel kernel
    bn_update_kernel<T, BN_TEAM><<<(unsigned)channels, BN_TEAM, 0, s->stream>>>(
        (const T*)in, (T*)bm, (T*)bv, (T*)rm, (T*)rv, factor, sh);
    CB_LAUNCH_CHECK(s);
    return CB200_OK;
  }
  const int slabs = bn_slab_count(s, batch, channels);
  void* scratch = nullptr;
  int rc = cb200_scratch(s, (size_t)channels * slabs * sizeof(double), &scratch);
  if (rc) return rc;
  double* partial = (double*)scratch;
  BnFinish<T> fin;
  fin.batch_means = (T*)bm; fin.batch_variances = (T*)bv; fin.running_means = (T*)rm; fin.running_variances = (T*)rv;
  fin.average_factor = factor; fin.coef = nullptr; fin.scale_grad = nullptr; fin.bias_grad = nullptr;
  fin.count = batch * inner;
  if ((rc = cb200_tile_flags(s, (size_t)channels, &fin.counters))) return rc;
  constexpr int VEC = 16 / (int)sizeof(T);
  const bool vec = (inner % VEC) == 0 && (((uintptr_t)in) & 15) == 0;
  const dim3 grid((unsigned)slabs, (unsigned)channels, 1);
  // mean pass, then the variance pass (which reads the mean the first one's last CTAs wrote): two launches
  if (vec) bn_slab_sums_kernel<T, 0, true><<<grid, BN_SLAB_THREADS, 0, s->stream>>>(partial, (const T*)in, nullptr, nullptr, nullptr, nullptr, 0.0, batch, (int)channels, (int)inner, slabs, fin);
  else bn_slab_sums_kernel<T, 0, false><<<grid, BN_SLAB_THREADS, 0, s->stream>>>(partial, (const T*)in, nullptr, nullptr, nullptr, nullptr, 0.0, batch, (int)channels, (int)inner, slabs, fin);
  CB_LAUNCH_CHECK(s);
  if (vec) bn_slab_sums_kernel<T, 1, true><<<grid, BN_SLAB_THREADS, 0, s->stream>>>(partial, (const T*)in, nullptr, (const T*)bm, nullptr, nullptr, 0.0, batch, (int)channels, (int)inner, slabs, fin);
  else bn_slab_sums_kernel<T, 1, false><<<grid, BN_SLAB_THREADS, 0, s->stream>>>(partial, (const T*)in, nullptr, (const T*)bm, nullptr, nullptr, 0.0, batch, (int)channels, (int)inner, slabs, fin);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

int bn_update_entry(cb200_stream* s, int dtype, void* output, const void* input, void* batch_means, void* batch_variances,
                    void* running_means, void* running_variances, double average_factor, const void* scale,
                    const void* bias, double epsilon, int64_t batch, int64_t channels, int64_t inner) {
  int rc = bn_train_check(s, dtype, batch, channels, inner, "batch_normalize_update_and_apply");
  if (rc) return rc;
  CB_REQUIRE(output && input && batch_means && batch_variances && running_means && running_variances && scale && bias,
             "batch_normalize_update_and_apply: null argument");
  if (batch == 0) return CB200_OK;
  rc = dtype == CB200_FLOAT
           ? bn_update_launch<float>(s, input, batch_means, batch_variances, running_means, running_variances,
                                     average_factor, batch, channels, inner)
           : bn_update_launch<double>(s, input, batch_means, batch_variances, running_means, running_variances,
                                      average_factor, batch, channels, inner);
  if (rc) return rc;
  // the apply half is the inference kernel fed with this batch's statistics (cpu/tensor_math.clj:1574-1608)
  return inner == 1 ? cb200_batch_normalize_eltwise(s, dtype, output, input, batch_means, batch_variances, scale, bias,
                                                    epsilon, batch, channels)
                    : cb200_batch_normalize_spatial(s, dtype, output, input, batch_means, batch_variances, scale, bias,
                                                    epsilon, batch, channels, inner);
}

template <typename T>
int bn_gradients_launch(cb200_stream* s, void* ig, void* sg, void* bg, const void* og, const void* in, const void* bm,
                        const void* bv, const void* scale, double epsilon, int64_t batch, int64_t channels, int64_t inner) {
  DeviceGuard guard(s->device);
  BnShape sh{batch, (int)channels, (int)inner};
  if (inner == 1 || channels > 65535) {
    if (inner == 1)
      bn_gradients_kernel<T, 1><<<(unsigned)((channels + 127) / 128), 128, 0, s->stream>>>(
          (T*)ig, (T*)sg, (T*)bg, (const T*)og, (const T*)in, (const T*)bm, (const T*)bv, (const T*)scale, epsilon, sh);
    else
      bn_gradients_kernel<T, BN_TEAM><<<(unsigned)channels, BN_TEAM, 0, s->stream>>>(
          (T*)ig, (T*)sg, (T*)bg, (const T*)og, (const T*)in, (const T*)bm, (const T*)bv, (const T*)scale, epsilon, sh);
    CB_LAUNCH_CHECK(s);
    return CB200_OK;
  }
  const int slabs = bn_slab_count(s, batch, channels);
  void* scratch = nullptr;
  int rc = cb200_scratch(s, ((size_t)5 * channels * slabs + (size_t)5 * channels) * sizeof(double), &scratch);
  if (rc) return rc;
  double* partial = (double*)scratch;
  double* coef = partial + (size_t)5 * channels * slabs;
  constexpr int VEC = 16 / (int)sizeof(T);
  const bool vec = (inner % VEC) == 0 && ((((uintptr_t)in) | ((uintptr_t)og) | ((uintptr_t)ig)) & 15) == 0;
  const dim3 grid((unsigned)slabs, (unsigned)channels, 1);
  const long long count = batch * inner;
  BnFinish<T> fin;
  fin.batch_means = nullptr; fin.batch_variances = nullptr; fin.running_means = nullptr; fin.running_variances = nullptr;
  fin.average_factor = 0.0; fin.coef = coef; fin.scale_grad = (T*)sg; fin.bias_grad = (T*)bg; fin.count = count;
  if ((rc = cb200_tile_flags(s, (size_t)channels, &fin.counters))) return rc;
  if (vec) bn_slab_sums_kernel<T, 2, true><<<grid, BN_SLAB_THREADS, 0, s->stream>>>(partial, (const T*)in, (const T*)og, (const T*)bm, (const T*)bv, (const T*)scale, epsilon, batch, (int)channels, (int)inner, slabs, fin);
  else bn_slab_sums_kernel<T, 2, false><<<grid, BN_SLAB_THREADS, 0, s->stream>>>(partial, (const T*)in, (const T*)og, (const T*)bm, (const T*)bv, (const T*)scale, epsilon, batch, (int)channels, (int)inner, slabs, fin);
  CB_LAUNCH_CHECK(s);
  const long long n_rows = batch * channels;
  long long blocks = n_rows < (long long)s->sm_count * 8 ? n_rows : (long long)s->sm_count * 8;
  if (vec) bn_input_gradient_kernel<T, true><<<(unsigned)blocks, BN_SLAB_THREADS, 0, s->stream>>>((T*)ig, (const T*)og, (const T*)in, coef, n_rows, (int)channels, (int)inner, 1.0 / (double)count);
  else bn_input_gradient_kernel<T, false><<<(unsigned)blocks, BN_SLAB_THREADS, 0, s->stream>>>((T*)ig, (const T*)og, (const T*)in, coef, n_rows, (int)channels, (int)inner, 1.0 / (double)count);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

int bn_gradients_entry(cb200_stream* s, int dtype, void* input_gradient, void* scale_gradient, void* bias_gradient,
                       const void* output_gradient, const void* input, const void* batch_means,
                       const void* batch_variances, const void* scale, double epsilon, int64_t batch, int64_t channels,
                       int64_t inner) {
  int rc = bn_train_check(s, dtype, batch, channels, inner, "batch_normalize_gradients");
  if (rc) return rc;
  CB_REQUIRE(input_gradient && scale_gradient && bias_gradient && output_gradient && input && batch_means &&
                 batch_variances && scale, "batch_normalize_gradients: null argument");
  if (batch == 0) return CB200_OK;
  return dtype == CB200_FLOAT
             ? bn_gradients_launch<float>(s, input_gradient, scale_gradient, bias_gradient, output_gradient, input,
                                          batch_means, batch_variances, scale, epsilon, batch, channels, inner)
             : bn_gradients_launch<double>(s, input_gradient, scale_gradient, bias_gradient, output_gradient, input,
                                           batch_means, batch_variances, scale, epsilon, batch, channels, inner);
}

int dense_nchw(const cb200_dims* d, const char* what) {
  CB_REQUIRE(d->rev_shape[4] == 1, "%s: tensors must be 4-d [batch, channels, height, width]", what);
  long long expect = 1;
  for (int k = 0; k < 4; ++k) {
    CB_REQUIRE(!d->index[k], "%s: index arrays are not supported", what);
    CB_REQUIRE(d->rev_shape[k] == 1 || d->rev_strides[k] == expect, "%s: tensors must be dense", what);
    expect *= d->rev_shape[k];
  }
  return CB200_OK;
}

}  // namespace

extern "C" {

int cb200_pooling_backward(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims, double in_grad_alpha,
                           const void* in, const cb200_dims* in_dims, const void* out, const cb200_dims* out_dims,
                           const void* out_grad, const cb200_dims* out_grad_dims, const cb200_pool_desc* desc) {
  CB_REQUIRE(s && in_grad && in_grad_dims && in && in_dims && out && out_dims && out_grad && out_grad_dims && desc,
             "pooling_backward: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "pooling-backward! is only defined for float and double tensors");
  CB_REQUIRE(desc->pool_op >= CB200_POOL_MAX && desc->pool_op <= CB200_POOL_AVG_EXC_PAD, "pooling_backward: unknown pool op %d",
             desc->pool_op);
  CB_REQUIRE(desc->kernel_width >= 1 && desc->kernel_height >= 1 && desc->stride_x >= 1 && desc->stride_y >= 1 &&
                 desc->pad_x >= 0 && desc->pad_y >= 0, "pooling_backward: bad descriptor");
  for (const cb200_dims* d : {in_grad_dims, in_dims, out_dims, out_grad_dims}) {
    int rc = cb200_check_dims(d, "pooling_backward");
    if (rc) return rc;
    rc = dense_nchw(d, "pooling_backward");
    if (rc) return rc;
  }
  for (int k = 0; k < 4; ++k) {
    CB_REQUIRE(in_grad_dims->rev_shape[k] == in_dims->rev_shape[k], "pooling_backward: input and input-gradient shapes differ");
    CB_REQUIRE(out_grad_dims->rev_shape[k] == out_dims->rev_shape[k], "pooling_backward: output and output-gradient shapes differ");
  }
  CB_REQUIRE(out_dims->rev_shape[3] == in_dims->rev_shape[3] && out_dims->rev_shape[2] == in_dims->rev_shape[2],
             "pooling_backward: batch / channel counts of input and output differ");
  PoolBwdGeom g;
  g.in_h = in_dims->rev_shape[1]; g.in_w = in_dims->rev_shape[0];
  g.out_h = out_dims->rev_shape[1]; g.out_w = out_dims->rev_shape[0];
  g.kw = desc->kernel_width; g.kh = desc->kernel_height; g.pad_x = desc->pad_x; g.pad_y = desc->pad_y;
  g.stride_x = desc->stride_x; g.stride_y = desc->stride_y;
  const long long planes = (long long)in_dims->rev_shape[3] * in_dims->rev_shape[2];
  const long long n_in = planes * g.in_h * g.in_w;
  const long long n_out = planes * g.out_h * g.out_w;
  if (n_in == 0) return CB200_OK;
  CB_REQUIRE(n_in <= 2147483647LL && n_out <= 2147483647LL, "pooling_backward: a tensor has more than 2^31 - 1 elements");
  DeviceGuard guard(s->device);
  if (dtype == CB200_FLOAT)
    pooling_backward_launch<float>(s, desc->pool_op, (float*)in_grad, (const float*)in, (const float*)out,
                                   (const float*)out_grad, g, n_in, in_grad_alpha);
  else
    pooling_backward_launch<double>(s, desc->pool_op, (double*)in_grad, (const double*)in, (const double*)out,
                                    (const double*)out_grad, g, n_in, in_grad_alpha);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

int cb200_batch_normalize_update_and_apply_eltwise(cb200_stream* s, int dtype, void* output, const void* input,
                                                   void* batch_means, void* batch_variances, void* running_means,
                                                   void* running_variances, double average_factor, const void* scale,
                                                   const void* bias, double epsilon, int64_t batch_count,
                                                   int64_t element_count) {
  return bn_update_entry(s, dtype, output, input, batch_means, batch_variances, running_means, running_variances,
                         average_factor, scale, bias, epsilon, batch_count, element_count, 1);
}

int cb200_batch_normalize_update_and_apply_spatial(cb200_stream* s, int dtype, void* output, const void* input,
                                                   void* batch_means, void* batch_variances, void* running_means,
                                                   void* running_variances, double average_factor, const void* scale,
                                                   const void* bias, double epsilon, int64_t batch_count,
                                                   int64_t channel_count, int64_t element_count) {
  return bn_update_entry(s, dtype, output, input, batch_means, batch_variances, running_means, running_variances,
                         average_factor, scale, bias, epsilon, batch_count, channel_count, element_count);
}

int cb200_batch_normalize_gradients_eltwise(cb200_stream* s, int dtype, void* input_gradient, void* scale_gradient,
                                            void* bias_gradient, const void* output_gradient, const void* output,
                                            const void* input, const void* batch_means, const void* batch_variances,
                                            const void* scale, const void* bias, double epsilon, int64_t batch_count,
                                            int64_t element_count) {
  (void)output; (void)bias;      // carried by the protocol, not read by the arithmetic
  return bn_gradients_entry(s, dtype, input_gradient, scale_gradient, bias_gradient, output_gradient, input, batch_means,
                            batch_variances, scale, epsilon, batch_count, element_count, 1);
}

int cb200_batch_normalize_gradients_spatial(cb200_stream* s, int dtype, void* input_gradient, void* scale_gradient,
                                            void* bias_gradient, const void* output_gradient, const void* output,
                                            const void* input, const void* batch_means, const void* batch_variances,
                                            const void* scale, const void* bias, double epsilon, int64_t batch_count,
                                            int64_t channel_count, int64_t element_count) {
  (void)output; (void)bias;
  return bn_gradients_entry(s, dtype, input_gradient, scale_gradient, bias_gradient, output_gradient, input, batch_means,
                            batch_variances, scale, epsilon, batch_count, channel_count, element_count);
}

}  // extern "C"
