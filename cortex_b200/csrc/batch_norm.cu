// batch-normalize! (inference form): batch-normalize-eltwise! / batch-normalize-spatial!
// (src/cortex/tensor/math.clj:125-148; cudnnBatchNormalizationForwardInference in the reference CUDA backend,
// src/cortex/compute/cuda/tensor_math.clj:662-730; arithmetic after the CPU backend,
// src/cortex/compute/cpu/tensor_math.clj:731-801):
//   inv_std[c] = (T) sqrt(1 / (variance[c] + (T)epsilon))           computed in double, rounded to T
//   out = ((x - mean[c]) * inv_std[c]) * scale[c] + bias[c]
// double tensors: every step in double, rounded (no fma), as the CPU backend: bit-identical to it.
// float tensors: the CPU backend widens every operand to double and rounds once at the end; here the three
// operations run in single precision (subtract, multiply, fused multiply-add: three roundings instead of
// one, |error| <= ~2 ulp, bound 1e-4): two f32<->f64 conversions per element go through a quarter-rate pipe
// and held the pass at 0.7 of the HBM copy rate.
// eltwise: input [batch, elements], c = column.  spatial: input [batch, channels, elements], c = channel.
// One pass over the data with 16-byte accesses; inv_std comes from a tiny pre-pass into the stream's scratch.
// Spatial inputs with long channel slabs are walked slab by slab (the channel's four parameters are read once
// per slab, no division per element); everything else takes the flat kernel with 32-bit index arithmetic.
#include "common.cuh"

namespace {

template <typename T>
__global__ void bn_inv_std_kernel(T* inv_std, const T* variances, double eps_t, int channels) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < channels) inv_std[c] = (T)sqrt(1.0 / ((double)variances[c] + eps_t));
}

__device__ __forceinline__ double bn_one(double x, double mean, double inv_std, double scale, double bias) {
  const double x_hat = __dmul_rn(__dsub_rn(x, mean), inv_std);
  return __dadd_rn(__dmul_rn(x_hat, scale), bias);
}
__device__ __forceinline__ float bn_one(float x, float mean, float inv_std, float scale, float bias) {
  return __fmaf_rn(__fmul_rn(__fsub_rn(x, mean), inv_std), scale, bias);
}

// spatial, long slabs: block b walks slabs b, b + grid, ...; slab = (image, channel), `inner` contiguous elements
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
bn_slab_kernel(T* out, const T* in, const T* means, const T* inv_std, const T* scale, const T* bias, long long slabs,
               int inner, int channels) {
  struct alignas(sizeof(T) * VEC) V { T v[VEC]; };
  const int nvec = inner / VEC;
  for (long long slab = blockIdx.x; slab < slabs; slab += gridDim.x) {
    const int c = (int)(slab % channels);
    const T m = means[c], sd = inv_std[c], g = scale[c], b = bias[c];
    const V* src = reinterpret_cast<const V*>(in + slab * inner);
    V* dst = reinterpret_cast<V*>(out + slab * inner);
    int j = threadIdx.x;
    for (; j + 3 * 256 < nvec; j += 4 * 256) {
      V x0 = src[j], x1 = src[j + 256], x2 = src[j + 512], x3 = src[j + 768];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        x0.v[e] = bn_one(x0.v[e], m, sd, g, b); x1.v[e] = bn_one(x1.v[e], m, sd, g, b);
        x2.v[e] = bn_one(x2.v[e], m, sd, g, b); x3.v[e] = bn_one(x3.v[e], m, sd, g, b);
      }
      dst[j] = x0; dst[j + 256] = x1; dst[j + 512] = x2; dst[j + 768] = x3;
    }
    for (; j < nvec; j += 256) {
      V x0 = src[j];
#pragma unroll
      for (int e = 0; e < VEC; ++e) x0.v[e] = bn_one(x0.v[e], m, sd, g, b);
      dst[j] = x0;
    }
  }
}

// channel of flat element i: (i / inner) % channels   (eltwise: inner = 1, channels = elements)
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
bn_apply_kernel(T* out, const T* in, const T* means, const T* inv_std, const T* scale, const T* bias, long long n,
                int inner, int channels) {
  struct alignas(sizeof(T) * VEC) V { T v[VEC]; };
  // n < 2^32 (checked by the caller): element indexes and their divisions stay 32-bit
  const unsigned nvec = (unsigned)(n / VEC);
  const unsigned uinner = (unsigned)inner, uch = (unsigned)channels;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += gridDim.x * blockDim.x) {
    const V x = reinterpret_cast<const V*>(in)[i];
    V o;
    const unsigned e0 = i * VEC;
    if (inner % VEC == 0) {
      // the whole vector lies in one channel
      const unsigned c = (e0 / uinner) % uch;
      const T m = means[c], s = inv_std[c], g = scale[c], b = bias[c];
#pragma unroll
      for (int e = 0; e < VEC; ++e) o.v[e] = bn_one(x.v[e], m, s, g, b);
    } else if (inner == 1) {
      unsigned c = e0 % uch;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        o.v[e] = bn_one(x.v[e], means[c], inv_std[c], scale[c], bias[c]);
        if (++c == uch) c = 0;
      }
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const unsigned c = ((e0 + e) / uinner) % uch;
        o.v[e] = bn_one(x.v[e], means[c], inv_std[c], scale[c], bias[c]);
      }
    }
    reinterpret_cast<V*>(out)[i] = o;
  }
  // tail
  for (unsigned i = nvec * VEC + blockIdx.x * blockDim.x + threadIdx.x; i < (unsigned)n; i += gridDim.x * blockDim.x) {
    const unsigned c = (i / uinner) % uch;
    out[i] = bn_one(in[i], means[c], inv_std[c], scale[c], bias[c]);
  }
}

template <typename T>
int bn_launch(cb200_stream* s, T* out, const T* in, const T* means, const T* variances, const T* scale, const T* bias,
              double epsilon, long long batch, int channels, int inner) {
  DeviceGuard guard(s->device);
  void* scratch = nullptr;
  int rc = cb200_scratch(s, (size_t)channels * sizeof(T), &scratch);
  if (rc) return rc;
  T* inv_std = (T*)scratch;
  bn_inv_std_kernel<T><<<(channels + 255) / 256, 256, 0, s->stream>>>(inv_std, variances, (double)(T)epsilon, channels);
  CB_LAUNCH_CHECK(s);
  const long long n = batch * channels * inner;
  constexpr int VEC = 16 / sizeof(T);
  const bool aligned = (((uintptr_t)out | (uintptr_t)in) & 15) == 0;
  long long blocks = (n / VEC + 255) / 256 + 1;
  const long long cap = (long long)s->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (aligned && inner >= 256 * VEC && (inner % VEC) == 0) {
    const long long slabs = batch * channels;
    long long sb = slabs < cap ? slabs : cap;
    bn_slab_kernel<T, VEC><<<(unsigned)sb, 256, 0, s->stream>>>(out, in, means, inv_std, scale, bias, slabs, inner, channels);
  } else if (aligned)
    bn_apply_kernel<T, VEC><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, means, inv_std, scale, bias, n, inner, channels);
  else
    bn_apply_kernel<T, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, means, inv_std, scale, bias, n, inner, channels);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

int bn_entry(cb200_stream* s, int dtype, void* out, const void* in, const void* means, const void* variances,
             const void* scale, const void* bias, double epsilon, int64_t batch, int64_t channels, int64_t inner) {
  CB_REQUIRE(s && out && in && means && variances && scale && bias, "batch_normalize: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "batch-normalization is only defined for float and double tensors");
  CB_REQUIRE(batch >= 0 && channels >= 1 && inner >= 1 && channels <= 2147483647LL && inner <= 2147483647LL,
             "batch_normalize: bad extents");
  CB_REQUIRE(batch * channels * inner < 4294967296LL, "batch_normalize: more than 2^32 - 1 elements");
  if (batch == 0) return CB200_OK;
  if (dtype == CB200_FLOAT)
    return bn_launch<float>(s, (float*)out, (const float*)in, (const float*)means, (const float*)variances,
                            (const float*)scale, (const float*)bias, epsilon, batch, (int)channels, (int)inner);
  return bn_launch<double>(s, (double*)out, (const double*)in, (const double*)means, (const double*)variances,
                           (const double*)scale, (const double*)bias, epsilon, batch, (int)channels, (int)inner);
}

}  // namespace

extern "C" {

int cb200_batch_normalize_eltwise(cb200_stream* s, int dtype, void* output, const void* input, const void* means,
                                  const void* variances, const void* scale, const void* bias, double epsilon,
                                  int64_t batch_count, int64_t element_count) {
  return bn_entry(s, dtype, output, input, means, variances, scale, bias, epsilon, batch_count, element_count, 1);
}

int cb200_batch_normalize_spatial(cb200_stream* s, int dtype, void* output, const void* input, const void* means,
                                  const void* variances, const void* scale, const void* bias, double epsilon,
                                  int64_t batch_count, int64_t channel_count, int64_t element_count) {
  return bn_entry(s, dtype, output, input, means, variances, scale, bias, epsilon, batch_count, channel_count,
                  element_count);
}

}  // extern "C"
