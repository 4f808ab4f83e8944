// lrn-forward! / lrn-backward! (local response normalisation across channels):
// src/cortex/tensor/math.clj:240-252; cudnnLRNCrossChannelForward / Backward with CUDNN_LRN_CROSS_CHANNEL_DIM1
// in the reference CUDA backend (src/cortex/compute/cuda/tensor_math.clj:1277-1335; its CPU backend has no
// implementation).  With the window W(c) = [c - floor((n-1)/2), c + n - 1 - floor((n-1)/2)] clipped to the
// channel range and s(c) = k + (alpha / n) * sum_{j in W(c)} x_j^2:
//   forward:   y_c  = x_c * s(c)^-beta
//   backward:  dx_c = dy_c * s(c)^-beta - (2 * alpha * beta / n) * x_c * sum_{j in W(c)} dy_j * y_j / s(j)
// (the backward sum runs over the same window as the forward one, as the library the reference calls does;
// the reference's literals for n = 2 pin this).  Dense [.., channels, height, width] tensors of rank 3 to 5;
// evaluated in the element type (float tensors in single precision, as the library call the reference makes).
#include "common.cuh"

namespace {

struct LrnGeom {
  long long batch;
  int channels;
  long long plane;       // height * width
  int look_behind, look_ahead;
  double k, alpha_over_n, beta;
};

// s > 0 (k + a sum of squares): 2^(e * log2 s) with the hardware log2 / exp2 (relative error ~1e-6 for |e| <= 1)
__device__ __forceinline__ float lrn_pow(float s, float e) { return exp2f(e * __log2f(s)); }
__device__ __forceinline__ double lrn_pow(double s, double e) { return pow(s, e); }

// `col` points at channel 0 of the element's (batch entry, pixel) column; channels are `plane` elements apart
template <typename T>
__device__ __forceinline__ T lrn_scale(const T* col, const LrnGeom& g, unsigned plane, int c) {
  const int c0 = max(0, c - g.look_behind), c1 = min(g.channels - 1, c + g.look_ahead);
  T sum = (T)0;
  for (int j = c0; j <= c1; ++j) {
    const T v = col[(unsigned)j * plane];
    sum += v * v;
  }
  return (T)g.k + (T)g.alpha_over_n * sum;
}

// WRITE_SCALE: store s(c) (backward pre-pass) instead of y
template <typename T, bool WRITE_SCALE>
__global__ void __launch_bounds__(256)
lrn_forward_kernel(T* out, T* scale_out, const T* in, LrnGeom g, long long n_elems) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_elems; i += (long long)gridDim.x * blockDim.x) {
    // 32-bit index arithmetic (the entry points limit a tensor to 2^32 - 1 elements)
    const unsigned iu = (unsigned)i, plane_u = (unsigned)g.plane;
    const unsigned bc = iu / plane_u;
    const unsigned p = iu - bc * plane_u;
    const unsigned b = bc / (unsigned)g.channels;
    const int c = (int)(bc - b * (unsigned)g.channels);
    const unsigned col0 = b * (unsigned)g.channels * plane_u + p;      // channel 0 of this element's column
    const T s = lrn_scale(in + col0, g, plane_u, c);
    if (WRITE_SCALE) scale_out[i] = s;
    else out[i] = in[i] * lrn_pow(s, (T)-g.beta);
  }
}

// Forward with the window width known at compile time (N <= 8, the common case): one thread owns a (batch entry,
// pixel) column and walks its channels with the window's N values in registers, so every input element is loaded
// once (adjacent threads = adjacent pixels: coalesced) and the sum of squares is N multiply-adds in channel order
// (the same order, hence the same value, as the per-element kernel above).
// The channel walk is a chain: the value loaded in one step joins the sum of squares of the next, so AHEAD more
// values are requested before they are needed and wait in registers behind the window.  A thread owns VEC
// adjacent pixels (16-byte accesses when the plane size and the base addresses allow): a CTA then moves 4 KB of
// one channel plane per step instead of 1 KB, which is what the DRAM pages want -- the walk jumps a whole plane
// between steps (one element per thread measured 1.7 TB/s, with or without the requests ahead; 2.9 TB/s with
// 16-byte accesses and a shifting window at 120 registers; 4.25 TB/s as a ring at 59).
template <typename T, int N, int AHEAD, int VEC>
__global__ void __launch_bounds__(256)
lrn_forward_columns_kernel(T* out, const T* in, LrnGeom g, long long n_groups) {
  struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
  const unsigned plane = (unsigned)g.plane;
  const unsigned groups_per_plane = plane / VEC;
  const int C = g.channels;
  constexpr int lb = (N - 1) / 2;                // = g.look_behind (lrn_geom)
  constexpr int W = N + AHEAD;
  const T k_t = (T)g.k, aon_t = (T)g.alpha_over_n, neg_beta_t = (T)-g.beta;
  for (long long grp = (long long)blockIdx.x * blockDim.x + threadIdx.x; grp < n_groups; grp += (long long)gridDim.x * blockDim.x) {
    const unsigned gu = (unsigned)grp;
    const unsigned b = gu / groups_per_plane, p = (gu - b * groups_per_plane) * VEC;
    const size_t base = (size_t)b * (unsigned)C * plane + p;
    const T* x = in + base;
    T* y = out + base;
    // ring of W channel values: channel ch sits in slot (ch + lb) % W, slots are compile-time constants because
    // the channel loop is unrolled W-fold (no register moves when the window slides)
    Pack win[W];
#pragma unroll
    for (int i = 0; i < W; ++i) {
      const int ch = i - lb;
      if (ch >= 0 && ch < C) {
        win[i] = *reinterpret_cast<const Pack*>(x + (size_t)ch * plane);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) win[i].v[e] = (T)0;
      }
    }
    for (int c0 = 0; c0 < C; c0 += W) {
#pragma unroll
      for (int r = 0; r < W; ++r) {
        const int c = c0 + r;
        if (c < C) {
          Pack o;
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            T sum = (T)0;
#pragma unroll
            for (int i = 0; i < N; ++i) sum += win[(r + i) % W].v[e] * win[(r + i) % W].v[e];
            const T s = k_t + aon_t * sum;
            // look_behind is (N - 1) / 2 for every descriptor: a constant here
            o.v[e] = win[(r + (N - 1) / 2) % W].v[e] * lrn_pow(s, neg_beta_t);
          }
          *reinterpret_cast<Pack*>(y + (size_t)c * plane) = o;
          const int next = c + W - lb;
          if (next < C) {
            win[r] = *reinterpret_cast<const Pack*>(x + (size_t)next * plane);
          } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) win[r].v[e] = (T)0;
          }
        }
      }
    }
  }
}

template <typename T, int N>
void lrn_forward_columns_launch(cb200_stream* s, T* out, const T* in, const LrnGeom& g) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const long long n_cols = g.batch * g.plane;
  const bool vec = (g.plane % VEC) == 0 && ((((uintptr_t)out) | ((uintptr_t)in)) & 15) == 0;
  const long long n_groups = vec ? n_cols / VEC : n_cols;
  // 128-thread blocks: at 64 registers eight fit an SM, and a shape with a few blocks per SM spreads evenly
  long long blocks = (n_groups + 127) / 128;
  const long long cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (vec) lrn_forward_columns_kernel<T, N, 6, VEC><<<(unsigned)blocks, 128, 0, s->stream>>>(out, in, g, n_groups);
  else lrn_forward_columns_kernel<T, N, 6, 1><<<(unsigned)blocks, 128, 0, s->stream>>>(out, in, g, n_groups);
}

template <typename T>
bool lrn_forward_columns(cb200_stream* s, T* out, const T* in, const LrnGeom& g, int n) {
  const long long n_cols = g.batch * g.plane;
  if (n < 1 || n > 8 || n_cols < 4096) return false;      // few columns: the per-element kernel has more threads
  switch (n) {
    case 1: lrn_forward_columns_launch<T, 1>(s, out, in, g); break;
    case 2: lrn_forward_columns_launch<T, 2>(s, out, in, g); break;
    case 3: lrn_forward_columns_launch<T, 3>(s, out, in, g); break;
    case 4: lrn_forward_columns_launch<T, 4>(s, out, in, g); break;
    case 5: lrn_forward_columns_launch<T, 5>(s, out, in, g); break;
    case 6: lrn_forward_columns_launch<T, 6>(s, out, in, g); break;
    case 7: lrn_forward_columns_launch<T, 7>(s, out, in, g); break;
    default: lrn_forward_columns_launch<T, 8>(s, out, in, g); break;
  }
  return true;
}

template <typename T>
__global__ void __launch_bounds__(256)
lrn_backward_kernel(T* in_grad, const T* out, const T* in, const T* out_grad, const T* scale, LrnGeom g,
                    long long n_elems) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_elems; i += (long long)gridDim.x * blockDim.x) {
    // 32-bit index arithmetic (the entry points limit a tensor to 2^32 - 1 elements)
    const unsigned iu = (unsigned)i, plane_u = (unsigned)g.plane;
    const unsigned bc = iu / plane_u;
    const unsigned p = iu - bc * plane_u;
    const unsigned b = bc / (unsigned)g.channels;
    const int c = (int)(bc - b * (unsigned)g.channels);
    const unsigned col0 = b * (unsigned)g.channels * plane_u + p;      // channel 0 of this element's column
    const int c0 = max(0, c - g.look_behind), c1 = min(g.channels - 1, c + g.look_ahead);
    T sum = (T)0;
    for (int j = c0; j <= c1; ++j) {
      const unsigned o = col0 + (unsigned)j * plane_u;
      sum += out_grad[o] * out[o] / scale[o];
    }
    const T direct = out_grad[i] * lrn_pow(scale[i], (T)-g.beta);
    in_grad[i] = direct - (T)(2.0 * g.alpha_over_n * g.beta) * in[i] * sum;
  }
}

int lrn_geom(const cb200_dims* const* all, int count, const cb200_lrn_desc* desc, LrnGeom* g, long long* n_elems,
             const char* what) {
  CB_REQUIRE(desc->n >= 1, "%s: window width n must be at least 1", what);
  for (int t = 0; t < count; ++t) {
    const cb200_dims* d = all[t];
    int rc = cb200_check_dims(d, what);
    if (rc) return rc;
    long long expect = 1;
    for (int k = 0; k < 5; ++k) {
      CB_REQUIRE(!d->index[k], "%s: index arrays are not supported", what);
      CB_REQUIRE(d->rev_shape[k] == 1 || d->rev_strides[k] == expect, "%s: tensors must be dense", what);
      CB_REQUIRE(d->rev_shape[k] == all[0]->rev_shape[k], "Input and output shapes must match");
      expect *= d->rev_shape[k];
    }
  }
  const cb200_dims* d = all[0];
  g->plane = (long long)d->rev_shape[0] * d->rev_shape[1];
  g->channels = d->rev_shape[2];
  g->batch = (long long)d->rev_shape[3] * d->rev_shape[4];
  g->look_behind = (desc->n - 1) / 2;
  g->look_ahead = desc->n - g->look_behind - 1;
  g->k = desc->k; g->alpha_over_n = desc->alpha / (double)desc->n; g->beta = desc->beta;
  *n_elems = g->plane * g->channels * g->batch;
  CB_REQUIRE(*n_elems < 4294967296LL, "%s: more than 2^32 - 1 elements", what);
  return CB200_OK;
}

unsigned lrn_blocks(cb200_stream* s, long long n) {
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)s->sm_count * 32;
  return (unsigned)(blocks < cap ? blocks : cap);
}

}  // namespace

extern "C" {

int cb200_lrn_forward(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, const void* in,
                      const cb200_dims* in_dims, const cb200_lrn_desc* desc) {
  CB_REQUIRE(s && out && out_dims && in && in_dims && desc, "lrn_forward: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "lrn-forward is only defined for float and double tensors");
  const cb200_dims* all[2] = {in_dims, out_dims};
  LrnGeom g;
  long long n = 0;
  int rc = lrn_geom(all, 2, desc, &g, &n, "lrn_forward");
  if (rc) return rc;
  if (n == 0) return CB200_OK;
  DeviceGuard guard(s->device);
  if (dtype == CB200_FLOAT) {
    if (!lrn_forward_columns<float>(s, (float*)out, (const float*)in, g, desc->n))
      lrn_forward_kernel<float, false><<<lrn_blocks(s, n), 256, 0, s->stream>>>((float*)out, nullptr, (const float*)in, g, n);
  } else {
    if (!lrn_forward_columns<double>(s, (double*)out, (const double*)in, g, desc->n))
      lrn_forward_kernel<double, false><<<lrn_blocks(s, n), 256, 0, s->stream>>>((double*)out, nullptr, (const double*)in, g, n);
  }
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

int cb200_lrn_backward(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims, const void* out,
                       const cb200_dims* out_dims, const void* in, const cb200_dims* in_dims, const void* out_grad,
                       const cb200_dims* out_grad_dims, const cb200_lrn_desc* desc) {
  CB_REQUIRE(s && in_grad && in_grad_dims && out && out_dims && in && in_dims && out_grad && out_grad_dims && desc,
             "lrn_backward: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "lrn-backward is only defined for float and double tensors");
  const cb200_dims* all[4] = {in_dims, out_dims, in_grad_dims, out_grad_dims};
  LrnGeom g;
  long long n = 0;
  int rc = lrn_geom(all, 4, desc, &g, &n, "lrn_backward");
  if (rc) return rc;
  if (n == 0) return CB200_OK;
  DeviceGuard guard(s->device);
  void* scratch = nullptr;
  rc = cb200_scratch(s, (size_t)n * cb200_dtype_size(dtype), &scratch);
  if (rc) return rc;
  if (dtype == CB200_FLOAT) {
    float* scale = (float*)scratch;
    lrn_forward_kernel<float, true><<<lrn_blocks(s, n), 256, 0, s->stream>>>(nullptr, scale, (const float*)in, g, n);
    CB_LAUNCH_CHECK(s);
    lrn_backward_kernel<float><<<lrn_blocks(s, n), 256, 0, s->stream>>>((float*)in_grad, (const float*)out, (const float*)in,
                                                                         (const float*)out_grad, scale, g, n);
  } else {
    double* scale = (double*)scratch;
    lrn_forward_kernel<double, true><<<lrn_blocks(s, n), 256, 0, s->stream>>>(nullptr, scale, (const double*)in, g, n);
    CB_LAUNCH_CHECK(s);
    lrn_backward_kernel<double><<<lrn_blocks(s, n), 256, 0, s->stream>>>((double*)in_grad, (const double*)out, (const double*)in,
                                                                          (const double*)out_grad, scale, g, n);
  }
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // extern "C"
