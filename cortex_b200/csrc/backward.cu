// Backward-pass methods next to the dense-layer path: activation-gradient!
// (src/cortex/tensor.clj:1256-1283 -> tm/activation-gradient!, src/cortex/tensor/math.clj; CPU semantics
// src/cortex/compute/cpu/tensor_math.clj:1318-1363; CUDA reference: cudnnActivationBackward,
// src/cortex/compute/cuda/tensor_math.clj:843-...).
//
//   logistic: in_grad = out * (1 - out) * out_grad
//   tanh:     in_grad = (1 - out * out) * out_grad
//   relu:     in_grad = (out > 0 ? 1 : 0) * out_grad          (a zero factor keeps the sign / NaN of out_grad)
//
// Arithmetic as on the JVM: float views are computed in double, left to right, and rounded once by the final
// cast, so the result is bit-identical to the reference CPU backend.  HBM-bound: two reads and one write per
// element; dense operands take 16-byte accesses, everything else the index system.
//
// The other pieces of biased-multiply-backward! (src/cortex/compute/nn/backend.clj:115-139) need no kernels of
// their own: the bias gradient is binary-op! with a destination smaller than the operation (compare-and-swap
// accumulation), the input and weight gradients are gemm! NN and TN.
#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ T act_grad(T out, T grad, int op) {
  const double o = (double)out, g = (double)grad;
  switch (op) {
    // explicit round-to-nearest operations: no fused multiply-add (the JVM rounds after every operation)
    case CB200_ACT_LOGISTIC: return (T)__dmul_rn(__dmul_rn(o, __dsub_rn(1.0, o)), g);
    case CB200_ACT_TANH: return (T)__dmul_rn(__dsub_rn(1.0, __dmul_rn(o, o)), g);
    default: return (out > (T)0 ? (T)1 : (T)0) * grad;      // relu; exact in the element type
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
activation_gradient_kernel(T* in_grad, Operand oi, const T* out_grad, Operand og, const T* out, Operand oo, Geometry g,
                           long long n, int op) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    in_grad[operand_offset(oi, g, i)] = act_grad<T>(out[operand_offset(oo, g, i)], out_grad[operand_offset(og, g, i)], op);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(256)
activation_gradient_flat_kernel(T* in_grad, const T* out_grad, const T* out, long long nvec, int op) {
  struct alignas(16) V { T v[VEC]; };
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // two vectors per operand in flight
  for (; i + stride < nvec; i += 2 * stride) {
    const V g0 = reinterpret_cast<const V*>(out_grad)[i], g1 = reinterpret_cast<const V*>(out_grad)[i + stride];
    const V o0 = reinterpret_cast<const V*>(out)[i], o1 = reinterpret_cast<const V*>(out)[i + stride];
    V r0, r1;
#pragma unroll
    for (int e = 0; e < VEC; ++e) { r0.v[e] = act_grad<T>(o0.v[e], g0.v[e], op); r1.v[e] = act_grad<T>(o1.v[e], g1.v[e], op); }
    reinterpret_cast<V*>(in_grad)[i] = r0;
    reinterpret_cast<V*>(in_grad)[i + stride] = r1;
  }
  for (; i < nvec; i += stride) {
    const V g0 = reinterpret_cast<const V*>(out_grad)[i], o0 = reinterpret_cast<const V*>(out)[i];
    V r0;
#pragma unroll
    for (int e = 0; e < VEC; ++e) r0.v[e] = act_grad<T>(o0.v[e], g0.v[e], op);
    reinterpret_cast<V*>(in_grad)[i] = r0;
  }
}

bool dense_same(const cb200_dims* d, const cb200_dims* ref) {
  long long expect = 1;
  for (int i = 0; i < 5; ++i) {
    if (d->index[i] || d->rev_shape[i] != ref->rev_shape[i]) return false;
    if (d->rev_shape[i] > 1 && d->rev_strides[i] != expect) return false;
    expect *= d->rev_shape[i];
  }
  return true;
}

template <typename T>
int launch_generic(cb200_stream* s, void* in_grad, const cb200_dims* ig_dims, const void* out_grad,
                   const cb200_dims* og_dims, const void* out, const cb200_dims* o_dims, int op, long long n,
                   long long blocks) {
  Operand oi, og, oo;
  operand_from_dims(oi, ig_dims);
  operand_from_dims(og, og_dims);
  operand_from_dims(oo, o_dims);
  Geometry g;
  const cb200_dims* all[3] = {ig_dims, og_dims, o_dims};
  for (int d = 0; d < 5; ++d) {
    g.max_shape[d] = 1;
    for (int k = 0; k < 3; ++k) if (all[k]->rev_shape[d] > g.max_shape[d]) g.max_shape[d] = all[k]->rev_shape[d];
  }
  g.ndims = 1;
  for (int d = 0; d < 5; ++d) if (g.max_shape[d] > 1) g.ndims = d + 1;
  activation_gradient_kernel<T><<<(unsigned)blocks, 256, 0, s->stream>>>((T*)in_grad, oi, (const T*)out_grad, og,
                                                                        (const T*)out, oo, g, n, op);
  return CB200_OK;
}

}  // namespace

extern "C" int cb200_activation_gradient(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims,
                                         const void* out_grad, const cb200_dims* out_grad_dims, const void* out,
                                         const cb200_dims* out_dims, int act, int64_t n_elems) {
  CB_REQUIRE(s && in_grad && out_grad && out && in_grad_dims && out_grad_dims && out_dims,
             "activation_gradient: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE,
             "activation-gradient! is only defined for float and double tensors");
  CB_REQUIRE(act == CB200_ACT_RELU || act == CB200_ACT_TANH || act == CB200_ACT_LOGISTIC,
             "Only :logistic :tanh and :relu are supported (got %d)", act);
  CB_REQUIRE(n_elems >= 0 && n_elems <= 2147483647LL, "activation_gradient: element count out of range");
  int rc;
  if ((rc = cb200_check_dims(in_grad_dims, "activation_gradient input-gradient"))) return rc;
  if ((rc = cb200_check_dims(out_grad_dims, "activation_gradient output-gradient"))) return rc;
  if ((rc = cb200_check_dims(out_dims, "activation_gradient output"))) return rc;
  if (n_elems == 0) return CB200_OK;
  DeviceGuard guard(s->device);
  const long long cap = (long long)s->sm_count * 16;
  if (dense_same(in_grad_dims, in_grad_dims) && dense_same(out_grad_dims, in_grad_dims) && dense_same(out_dims, in_grad_dims)) {
    long long total = 1;
    for (int i = 0; i < 5; ++i) total *= in_grad_dims->rev_shape[i];
    const int vecn = dtype == CB200_FLOAT ? 4 : 2;
    const bool aligned = (((uintptr_t)in_grad | (uintptr_t)out_grad | (uintptr_t)out) & 15) == 0;
    if (total == n_elems && (total % vecn) == 0 && aligned) {
      const long long nvec = total / vecn;
      long long vb = (nvec + 511) / 512;
      if (vb > cap) vb = cap;
      if (vb < 1) vb = 1;
      if (dtype == CB200_FLOAT)
        activation_gradient_flat_kernel<float, 4><<<(unsigned)vb, 256, 0, s->stream>>>(
            (float*)in_grad, (const float*)out_grad, (const float*)out, nvec, act);
      else
        activation_gradient_flat_kernel<double, 2><<<(unsigned)vb, 256, 0, s->stream>>>(
            (double*)in_grad, (const double*)out_grad, (const double*)out, nvec, act);
      CB_LAUNCH_CHECK(s);
      return CB200_OK;
    }
  }
  long long blocks = (n_elems + 255) / 256;
  if (blocks > cap) blocks = cap;
  if (dtype == CB200_FLOAT)
    launch_generic<float>(s, in_grad, in_grad_dims, out_grad, out_grad_dims, out, out_dims, act, n_elems, blocks);
  else
    launch_generic<double>(s, in_grad, in_grad_dims, out_grad, out_grad_dims, out, out_dims, act, n_elems, blocks);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}
