// Optimiser steps and rand!: the ring of the training path that touches the flat parameter buffer.
//
//   adam      resources/adam.cu:1-36 (CUDA), src/cortex/optimize/adam.clj:68-102 (CPU semantics restated here)
//   adadelta  resources/adadelta.cu:1-68 (CUDA), java/cortex/compute/optimize/AdadeltaOptimizer.java (CPU)
//   rand!     src/cortex/tensor/math.clj:237; CPU src/cortex/compute/cpu/tensor_math.clj:1867-1890,
//             CUDA (cuRAND) src/cortex/compute/cuda/tensor_math.clj:1246-1272
//
// Each step is ONE pass over the buffers (adam: gradient, parameters, m, v read; parameters, m, v written =
// 28 bytes per fp32 parameter), HBM-bound, 16-byte accesses, two vectors per array in flight per thread, grid
// sized to the SM count.  Arithmetic: double buffers follow the reference CPU backend operation for operation
// (explicit round-to-nearest intrinsics, no contraction into fused multiply-adds, as the JVM) and are
// bit-identical to it.  Float buffers are computed in single precision with IEEE-rounded divide and square
// root, as the reference's own CUDA kernels do (the CPU backend evaluates them in double and rounds on
// store: the two differ by a few units in the last place, far inside the 1e-4 bound; evaluating float
// buffers in double costs ~70 fp64 instructions per parameter, which makes the pass ALU-bound -- measured
// 0.76 / 0.38 of the HBM copy rate for adam / adadelta -- instead of memory-bound).  (SGD with momentum
// needs no kernel: the reference issues it as four tensor calls, src/cortex/optimize/sgd.clj:16-40.)
//
// rand! has no reproducible counterpart in the reference (SecureRandom on the CPU, cuRAND's default
// generator on CUDA; its test is statistical, src/cortex/verify/tensor.clj:1036-1066).  Here it is a
// counter-based generator (Philox-4x32 with 10 rounds, Salmon et al., SC'11): element 4i..4i+3 comes
// from counter (i, sequence) under key (seed), so a call is reproducible from (seed, sequence), any
// element can be computed independently, and no generator state lives in device memory.
#include "common.cuh"

namespace {

// ---- adam ------------------------------------------------------------------------------------
// CPU formula (adam.clj:83-95): g = ga * grad; m' = b1*m + (1-b1)*g; v' = b2*v + (1-b2)*g*g;
//   dx = alpha * (m' / ((1 - p1) * (sqrt(v' / (1 - p2)) + eps)));  param -= dx
// m' and v' enter dx unrounded (they are locals; the stores round copies of them).
struct AdamScalars {
  double alpha, beta1, beta2, eps, p1, p2, ga, omb1, omb2, omp1, omp2;
  float f_alpha, f_beta1, f_beta2, f_eps, f_ga, f_omb1, f_omb2, f_omp1, f_omp2;
};

template <typename T>
__device__ __forceinline__ void adam_one(const AdamScalars& c, T grad, T& param, T& m, T& v);

template <>
__device__ __forceinline__ void adam_one<double>(const AdamScalars& c, double grad, double& param, double& m, double& v) {
  const double g = __dmul_rn(c.ga, grad);
  const double lm = __dadd_rn(__dmul_rn(c.beta1, m), __dmul_rn(c.omb1, g));
  const double lv = __dadd_rn(__dmul_rn(c.beta2, v), __dmul_rn(__dmul_rn(c.omb2, g), g));
  const double denom = __dmul_rn(c.omp1, __dadd_rn(__dsqrt_rn(__ddiv_rn(lv, c.omp2)), c.eps));
  const double dx = __dmul_rn(c.alpha, __ddiv_rn(lm, denom));
  m = lm;
  v = lv;
  param = __dsub_rn(param, dx);
}

template <>
__device__ __forceinline__ void adam_one<float>(const AdamScalars& c, float grad, float& param, float& m, float& v) {
  const float g = c.f_ga * grad;
  const float lm = fmaf(c.f_beta1, m, c.f_omb1 * g);
  const float lv = fmaf(c.f_beta2, v, (c.f_omb2 * g) * g);
  const float denom = c.f_omp1 * (__fsqrt_rn(__fdiv_rn(lv, c.f_omp2)) + c.f_eps);
  const float dx = c.f_alpha * __fdiv_rn(lm, denom);
  m = lm;
  v = lv;
  param = param - dx;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
adam_kernel(AdamScalars c, const T* __restrict__ grad, T* __restrict__ param, T* __restrict__ m, T* __restrict__ v,
            long long n) {
  struct alignas(16) V { T e[VEC]; };
  const long long nvec = n / VEC;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < nvec; i += 2 * stride) {
    const V g0 = reinterpret_cast<const V*>(grad)[i], g1 = reinterpret_cast<const V*>(grad)[i + stride];
    V p0 = reinterpret_cast<V*>(param)[i], p1 = reinterpret_cast<V*>(param)[i + stride];
    V m0 = reinterpret_cast<V*>(m)[i], m1 = reinterpret_cast<V*>(m)[i + stride];
    V v0 = reinterpret_cast<V*>(v)[i], v1 = reinterpret_cast<V*>(v)[i + stride];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      adam_one<T>(c, g0.e[e], p0.e[e], m0.e[e], v0.e[e]);
      adam_one<T>(c, g1.e[e], p1.e[e], m1.e[e], v1.e[e]);
    }
    reinterpret_cast<V*>(param)[i] = p0; reinterpret_cast<V*>(param)[i + stride] = p1;
    reinterpret_cast<V*>(m)[i] = m0; reinterpret_cast<V*>(m)[i + stride] = m1;
    reinterpret_cast<V*>(v)[i] = v0; reinterpret_cast<V*>(v)[i + stride] = v1;
  }
  for (; i < nvec; i += stride) {
    const V g0 = reinterpret_cast<const V*>(grad)[i];
    V p0 = reinterpret_cast<V*>(param)[i], m0 = reinterpret_cast<V*>(m)[i], v0 = reinterpret_cast<V*>(v)[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) adam_one<T>(c, g0.e[e], p0.e[e], m0.e[e], v0.e[e]);
    reinterpret_cast<V*>(param)[i] = p0;
    reinterpret_cast<V*>(m)[i] = m0;
    reinterpret_cast<V*>(v)[i] = v0;
  }
  // ragged tail (n not a multiple of VEC)
  for (long long j = nvec * VEC + (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride)
    adam_one<T>(c, grad[j], param[j], m[j], v[j]);
}

// element-at-a-time form for buffers that are not 16-byte aligned (sub-buffers at odd parameter offsets)
template <typename T>
__global__ void __launch_bounds__(256)
adam_scalar_kernel(AdamScalars c, const T* grad, T* param, T* m, T* v, long long n) {
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x)
    adam_one<T>(c, grad[j], param[j], m[j], v[j]);
}

// ---- adadelta --------------------------------------------------------------------------------
// CPU (AdadeltaOptimizer.java): g = ga * grad (a FLOAT product in step_f, double in step_d);
//   ga' = g*g*decay + ga_acc*(1 - decay);  dx = (-1 * sqrt(dx_acc + eps) * g) / sqrt(ga' + eps);
//   dxa' = dx*dx*decay + dx_acc*(1 - decay);  param += (T)dx  (a float add in step_f)
struct AdadeltaScalars { double decay, eps, ga, omd; float ga_f, f_decay, f_eps, f_omd; };

template <typename T>
__device__ __forceinline__ void adadelta_one(const AdadeltaScalars& c, T grad, T& param, T& gacc, T& dxacc);

template <>
__device__ __forceinline__ void adadelta_one<double>(const AdadeltaScalars& c, double grad, double& param, double& gacc,
                                                     double& dxacc) {
  const double g = __dmul_rn(c.ga, grad);
  const double ga = __dadd_rn(__dmul_rn(__dmul_rn(g, g), c.decay), __dmul_rn(gacc, c.omd));
  const double rms_g = __dsqrt_rn(__dadd_rn(ga, c.eps));
  const double rms_dx = __dsqrt_rn(__dadd_rn(dxacc, c.eps));
  const double dx = __ddiv_rn(__dmul_rn(__dmul_rn(-1.0, rms_dx), g), rms_g);
  const double dxa = __dadd_rn(__dmul_rn(__dmul_rn(dx, dx), c.decay), __dmul_rn(dxacc, c.omd));
  gacc = ga;
  dxacc = dxa;
  param = __dadd_rn(param, dx);
}

template <>
__device__ __forceinline__ void adadelta_one<float>(const AdadeltaScalars& c, float grad, float& param, float& gacc,
                                                    float& dxacc) {
  const float g = c.ga_f * grad;
  const float ga = fmaf(g * g, c.f_decay, gacc * c.f_omd);
  const float rms_g = __fsqrt_rn(ga + c.f_eps);
  const float rms_dx = __fsqrt_rn(dxacc + c.f_eps);
  const float dx = __fdiv_rn(-rms_dx * g, rms_g);
  const float dxa = fmaf(dx * dx, c.f_decay, dxacc * c.f_omd);
  gacc = ga;
  dxacc = dxa;
  param = param + dx;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
adadelta_kernel(AdadeltaScalars c, const T* __restrict__ grad, T* __restrict__ param, T* __restrict__ gacc,
                T* __restrict__ dxacc, long long n) {
  struct alignas(16) V { T e[VEC]; };
  const long long nvec = n / VEC;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < nvec; i += 2 * stride) {
    const V g0 = reinterpret_cast<const V*>(grad)[i], g1 = reinterpret_cast<const V*>(grad)[i + stride];
    V p0 = reinterpret_cast<V*>(param)[i], p1 = reinterpret_cast<V*>(param)[i + stride];
    V a0 = reinterpret_cast<V*>(gacc)[i], a1 = reinterpret_cast<V*>(gacc)[i + stride];
    V d0 = reinterpret_cast<V*>(dxacc)[i], d1 = reinterpret_cast<V*>(dxacc)[i + stride];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      adadelta_one<T>(c, g0.e[e], p0.e[e], a0.e[e], d0.e[e]);
      adadelta_one<T>(c, g1.e[e], p1.e[e], a1.e[e], d1.e[e]);
    }
    reinterpret_cast<V*>(param)[i] = p0; reinterpret_cast<V*>(param)[i + stride] = p1;
    reinterpret_cast<V*>(gacc)[i] = a0; reinterpret_cast<V*>(gacc)[i + stride] = a1;
    reinterpret_cast<V*>(dxacc)[i] = d0; reinterpret_cast<V*>(dxacc)[i + stride] = d1;
  }
  for (; i < nvec; i += stride) {
    const V g0 = reinterpret_cast<const V*>(grad)[i];
    V p0 = reinterpret_cast<V*>(param)[i], a0 = reinterpret_cast<V*>(gacc)[i], d0 = reinterpret_cast<V*>(dxacc)[i];
#pragma unroll
    for (int e = 0; e < VEC; ++e) adadelta_one<T>(c, g0.e[e], p0.e[e], a0.e[e], d0.e[e]);
    reinterpret_cast<V*>(param)[i] = p0;
    reinterpret_cast<V*>(gacc)[i] = a0;
    reinterpret_cast<V*>(dxacc)[i] = d0;
  }
  for (long long j = nvec * VEC + (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride)
    adadelta_one<T>(c, grad[j], param[j], gacc[j], dxacc[j]);
}

template <typename T>
__global__ void __launch_bounds__(256)
adadelta_scalar_kernel(AdadeltaScalars c, const T* grad, T* param, T* gacc, T* dxacc, long long n) {
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (long long)gridDim.x * blockDim.x)
    adadelta_one<T>(c, grad[j], param[j], gacc[j], dxacc[j]);
}

// ---- rand! -----------------------------------------------------------------------------------
__host__ __device__ inline void philox_round(uint32_t (&ctr)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * ctr[0];
  const uint64_t p1 = (uint64_t)0xCD9E8D57u * ctr[2];
  const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
  const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
  const uint32_t c0 = hi1 ^ ctr[1] ^ k0, c1 = lo1, c2 = hi0 ^ ctr[3] ^ k1, c3 = lo0;
  ctr[0] = c0; ctr[1] = c1; ctr[2] = c2; ctr[3] = c3;
}

__host__ __device__ inline void philox4x32_10(uint64_t index, uint64_t sequence, uint64_t seed, uint32_t (&out)[4]) {
  uint32_t ctr[4] = {(uint32_t)index, (uint32_t)(index >> 32), (uint32_t)sequence, (uint32_t)(sequence >> 32)};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(ctr, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  for (int j = 0; j < 4; ++j) out[j] = ctr[j];
}

// 24 random bits -> [0, 1): includes 0, excludes 1, every value exactly representable
__device__ __forceinline__ float u01(uint32_t x) { return (float)(x >> 8) * 5.9604644775390625e-8f; }

// flat:      dest = min + u * (max - min): one fused multiply-add.  u has 24 bits and the range 24, so
//            the product is exact and the result is the correctly rounded sum -- what the CPU backend's
//            double evaluation followed by the float store gives too, short of a double-rounding tie
// gaussian:  dest = sqrt(variance) * z + mean, z from Box-Muller on two uniforms, the first in (0, 1]
__global__ void __launch_bounds__(256)
rand_kernel(float* dest, long long n, int gaussian, float a, float b, uint64_t seed, uint64_t sequence) {
  const long long groups = (n + 3) / 4;
  const bool vec_ok = (((uintptr_t)dest) & 15) == 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (long long)gridDim.x * blockDim.x) {
    uint32_t r[4];
    philox4x32_10((uint64_t)i, sequence, seed, r);
    float o[4];
    if (!gaussian) {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = fmaf(u01(r[j]), b, a);
    } else {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const float u1 = 1.0f - u01(r[j]);                // (0, 1]: the logarithm is finite
        const float rad = sqrtf(-2.0f * logf(u1));
        float sn, cs;
        sincospif(2.0f * u01(r[j + 1]), &sn, &cs);
        o[j] = fmaf(b, rad * cs, a);
        o[j + 1] = fmaf(b, rad * sn, a);
      }
    }
    if (vec_ok && 4 * i + 4 <= n) {
      *reinterpret_cast<float4*>(dest + 4 * i) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      for (int j = 0; j < 4 && 4 * i + j < n; ++j) dest[4 * i + j] = o[j];
    }
  }
}

template <typename T> inline bool aligned16(const void* a, const void* b, const void* c, const void* d) {
  return ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c) | ((uintptr_t)d)) & 15) == 0;
}

inline unsigned grid_for(const cb200_stream* s, long long work_items) {
  long long blocks = (work_items + 511) / 512;         // two items per thread in flight
  const long long cap = (long long)s->sm_count * 8;
  if (blocks > cap) blocks = cap;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

extern "C" {

int cb200_adam_step(cb200_stream* s, int dtype, double alpha, double beta1, double beta2, double epsilon,
                    double pow_beta1_t, double pow_beta2_t, double gradient_alpha, const void* gradients,
                    void* parameters, void* m, void* v, int64_t n) {
  CB_REQUIRE(s && gradients && parameters && m && v, "adam_step: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "adam_step: only float and double buffers");
  CB_REQUIRE(n >= 0, "adam_step: negative element count");
  if (n == 0) return CB200_OK;
  AdamScalars c;
  // scalars are cast to the buffers' element type first (drv/dtype-cast, adam.clj:128-136); 1 - x is then
  // evaluated in double from the cast values, as the JVM does
  auto cast = [&](double x) { return dtype == CB200_FLOAT ? (double)(float)x : x; };
  c.alpha = cast(alpha); c.beta1 = cast(beta1); c.beta2 = cast(beta2); c.eps = cast(epsilon);
  c.p1 = cast(pow_beta1_t); c.p2 = cast(pow_beta2_t); c.ga = cast(gradient_alpha);
  c.omb1 = 1.0 - c.beta1; c.omb2 = 1.0 - c.beta2; c.omp1 = 1.0 - c.p1; c.omp2 = 1.0 - c.p2;
  c.f_alpha = (float)c.alpha; c.f_beta1 = (float)c.beta1; c.f_beta2 = (float)c.beta2; c.f_eps = (float)c.eps;
  c.f_ga = (float)c.ga; c.f_omb1 = (float)c.omb1; c.f_omb2 = (float)c.omb2; c.f_omp1 = (float)c.omp1;
  c.f_omp2 = (float)c.omp2;
  DeviceGuard guard(s->device);
  if (dtype == CB200_FLOAT) {
    if (aligned16<float>(gradients, parameters, m, v))
      adam_kernel<float, 4><<<grid_for(s, n / 4 + 1), 256, 0, s->stream>>>(c, (const float*)gradients, (float*)parameters,
                                                                           (float*)m, (float*)v, n);
    else
      adam_scalar_kernel<float><<<grid_for(s, n), 256, 0, s->stream>>>(c, (const float*)gradients, (float*)parameters,
                                                                       (float*)m, (float*)v, n);
  } else {
    if (aligned16<double>(gradients, parameters, m, v))
      adam_kernel<double, 2><<<grid_for(s, n / 2 + 1), 256, 0, s->stream>>>(c, (const double*)gradients,
                                                                            (double*)parameters, (double*)m, (double*)v, n);
    else
      adam_scalar_kernel<double><<<grid_for(s, n), 256, 0, s->stream>>>(c, (const double*)gradients, (double*)parameters,
                                                                        (double*)m, (double*)v, n);
  }
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

int cb200_adadelta_step(cb200_stream* s, int dtype, double decay, double epsilon, void* grad_accum, void* dx_accum,
                        double gradient_beta, const void* gradient, void* parameters, int64_t n) {
  CB_REQUIRE(s && grad_accum && dx_accum && gradient && parameters, "adadelta_step: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "adadelta_step: only float and double buffers");
  CB_REQUIRE(n >= 0, "adadelta_step: negative element count");
  if (n == 0) return CB200_OK;
  AdadeltaScalars c;
  auto cast = [&](double x) { return dtype == CB200_FLOAT ? (double)(float)x : x; };
  c.decay = cast(decay); c.eps = cast(epsilon); c.ga = cast(gradient_beta); c.ga_f = (float)gradient_beta;
  c.omd = 1.0 - c.decay;
  c.f_decay = (float)c.decay; c.f_eps = (float)c.eps; c.f_omd = (float)c.omd;
  DeviceGuard guard(s->device);
  if (dtype == CB200_FLOAT) {
    if (aligned16<float>(gradient, parameters, grad_accum, dx_accum))
      adadelta_kernel<float, 4><<<grid_for(s, n / 4 + 1), 256, 0, s->stream>>>(
          c, (const float*)gradient, (float*)parameters, (float*)grad_accum, (float*)dx_accum, n);
    else
      adadelta_scalar_kernel<float><<<grid_for(s, n), 256, 0, s->stream>>>(
          c, (const float*)gradient, (float*)parameters, (float*)grad_accum, (float*)dx_accum, n);
  } else {
    if (aligned16<double>(gradient, parameters, grad_accum, dx_accum))
      adadelta_kernel<double, 2><<<grid_for(s, n / 2 + 1), 256, 0, s->stream>>>(
          c, (const double*)gradient, (double*)parameters, (double*)grad_accum, (double*)dx_accum, n);
    else
      adadelta_scalar_kernel<double><<<grid_for(s, n), 256, 0, s->stream>>>(
          c, (const double*)gradient, (double*)parameters, (double*)grad_accum, (double*)dx_accum, n);
  }
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

int cb200_rand(cb200_stream* s, void* dest, const cb200_dims* dest_dims, int distribution, double p0, double p1,
               uint64_t seed, uint64_t sequence) {
  CB_REQUIRE(s && dest && dest_dims, "rand: null argument");
  int rc = cb200_check_dims(dest_dims, "rand dest");
  if (rc) return rc;
  long long n = 1, expect = 1;
  for (int i = 0; i < 5; ++i) {
    CB_REQUIRE(!dest_dims->index[i] && (dest_dims->rev_shape[i] == 1 || dest_dims->rev_strides[i] == expect),
               "Rand generation must have simple dense buffers");
    expect *= dest_dims->rev_shape[i];
    n *= dest_dims->rev_shape[i];
  }
  double a, b;
  if (distribution == CB200_RAND_FLAT) {
    CB_REQUIRE(p0 < p1, "Minimum must be less than maximum");
    const float mn = (float)p0, mx = (float)p1;       // the CPU backend casts both to float, then subtracts in double
    a = (double)mn;
    b = (double)mx - (double)mn;
  } else if (distribution == CB200_RAND_GAUSSIAN) {
    CB_REQUIRE(p1 >= 0.0, "rand: negative variance");
    a = (double)(float)p0;                              // mean
    b = sqrt((double)(float)p1);                        // Math/sqrt of the float-cast variance
  } else {
    cb200_set_error("Unrecognized distribution: %d", distribution);
    return CB200_ERR_INVALID;
  }
  DeviceGuard guard(s->device);
  rand_kernel<<<grid_for(s, (n + 3) / 4 * 2), 256, 0, s->stream>>>((float*)dest, n, distribution == CB200_RAND_GAUSSIAN,
                                                                  (float)a, (float)b, seed, sequence);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // extern "C"
