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
template <typename T, int N>
__global__ void __launch_bounds__(256)
lrn_forward_columns_kernel(T* out, const T* in, LrnGeom g, long long n_cols) {
  const unsigned plane = (unsigned)g.plane;
  const int C = g.channels, lb = g.look_behind, la = N - 1 - lb;
  for (long long col = (long long)blockIdx.x * blockDim.x + threadIdx.x; col < n_cols; col += (long long)gridDim.x * blockDim.x) {
    const unsigned cu = (unsigned)col;
    const unsigned b = cu / plane, p = cu - b * plane;
    const size_t base = (size_t)b * (unsigned)C * plane + p;
    const T* x = in + base;
    T* y = out + base;
    T win[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int ch = i - lb;
      win[i] = (ch >= 0 && ch < C) ? x[(unsigned)ch * plane] : (T)0;
    }
    for (int c = 0; c < C; ++c) {
      T sum = (T)0;
#pragma unroll
      for (int i = 0; i < N; ++i) sum += win[i] * win[i];
      const T s = (T)g.k + (T)g.alpha_over_n * sum;
      y[(unsigned)c * plane] = win[lb] * lrn_pow(s, (T)-g.beta);
      const int next = c + 1 + la;
#pragma unroll
      for (int i = 0; i + 1 < N; ++i) win[i] = win[i + 1];
      win[N - 1] = next < C ? x[(unsigned)next * plane] : (T)0;
    }
  }
}

template <typename T>
bool lrn_forward_columns(cb200_stream* s, T* out, const T* in, const LrnGeom& g, int n) {
  const long long n_cols = g.batch * g.plane;
  if (n < 1 || n > 8 || n_cols < 4096) return false;      // few columns: the per-element kernel has more threads
  long long blocks = (n_cols + 255) / 256;
  const long long cap = (long long)s->sm_count * 16;
  if (blocks > cap) blocks = cap;
  const unsigned bl = (unsigned)blocks;
  switch (n) {
    case 1: lrn_forward_columns_kernel<T, 1><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
    case 2: lrn_forward_columns_kernel<T, 2><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
    case 3: lrn_forward_columns_kernel<T, 3><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
    case 4: lrn_forward_columns_kernel<T, 4><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
    case 5: lrn_forward_columns_kernel<T, 5><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
    case 6: lrn_forward_columns_kernel<T, 6><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
    case 7: lrn_forward_columns_kernel<T, 7><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
    default: lrn_forward_columns_kernel<T, 8><<<bl, 256, 0, s->stream>>>(out, in, g, n_cols); break;
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
