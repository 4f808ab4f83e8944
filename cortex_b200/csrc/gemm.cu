// gemm! entry points (src/cortex/tensor/math.clj:106-115) and the plain SIMT
// kernel that takes the shapes the tensor-core kernels do not (pointers or
// pitches that TMA cannot address, K = 0).
#include "common.cuh"
#include <math.h>

int cb200_gemm_tf32x3_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                             const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                             float beta, const float* bias, int act, int store_mode, int hw, int flags);
int cb200_gemm_tf32x3_launch_peers(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                                   const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                                   float beta, const float* bias, int act, int store_mode, int hw, int flags,
                                   int n_peers, float* const* peers);
int cb200_gemm_tf32x3_max_slices(const cb200_stream* s, int M, int N);
bool cb200_gemm_tf32x3_eligible(const float* A, long long lda, const float* B, long long ldb, int M, int N, int K);
int cb200_gemm_f64_launch(cb200_stream* s, double* C, long long ldc, int trans_a, int trans_b, double alpha,
                          const double* A, int M, int K, long long lda, const double* B, int N, long long ldb,
                          double beta, const double* bias, int act, const PeerList* peers);

bool cb200_gemm_presplit_auto_ok(cb200_stream* s, int M, int N, int K, int trans_a, int trans_b);
int cb200_gemm_presplit_auto_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                                    const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                                    float beta, const float* bias, int act);

namespace {

// tanh / logistic (evaluated in double like the CPU backend) behind a call: next to the cheap cases the compiler
// evaluated them branch-free for every element
static __device__ __noinline__ double act_transcendental(double v, int act) {
  return act == CB200_ACT_TANH ? tanh(v) : 1.0 / (1.0 + exp(-v));
}
template <typename T> __device__ __forceinline__ T act_apply(T v, int act) {
  if (act == CB200_ACT_NONE) return v;
  if (act == CB200_ACT_RELU) return v > (T)0 ? v : (T)0;
  return (T)act_transcendental((double)v, act);
}

// 64x64 tile, 16x16 threads, 4x4 per thread.  Element (m,k) of op(A) is
// A[m*sam + k*sak]; element (k,n) of op(B) is B[k*sbk + n*sbn].
template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt(T* C, long long ldc, const T* A, long long sam, long long sak, const T* B, long long sbk, long long sbn,
          int M, int N, int K, T alpha, T beta, const T* bias, int act, PeerList peers) {
  __shared__ T As[16][64 + 1];
  __shared__ T Bs[16][64 + 1];
  const int t = threadIdx.x, tx = t % 16, ty = t / 16;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (T)0;
  for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int k, m;
      if (sak == 1) { k = t % 16; m = t / 16 + 16 * i; } else { m = t % 64; k = t / 64 + 4 * i; }
      T v = (T)0;
      if (m0 + m < M && k0 + k < K) v = A[(long long)(m0 + m) * sam + (long long)(k0 + k) * sak];
      As[k][m] = v;
      int kb, n;
      if (sbn == 1) { n = t % 64; kb = t / 64 + 4 * i; } else { kb = t % 16; n = t / 16 + 16 * i; }
      T w = (T)0;
      if (n0 + n < N && k0 + kb < K) w = B[(long long)(k0 + kb) * sbk + (long long)(n0 + n) * sbn];
      Bs[kb][n] = w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int m = m0 + ty + 16 * i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int n = n0 + tx + 16 * j;
      if (n >= N) continue;
      T* c = C + (long long)m * ldc + n;
      T o = alpha * acc[i][j];
      if (beta != (T)0) o += beta * (*c);
      if (bias) o += bias[n];
      o = act_apply<T>(o, act);
      *c = o;
      for (int d = 0; d < peers.n; ++d) ((T*)peers.p[d])[(long long)m * ldc + n] = o;
    }
  }
}

template <typename T>
int launch_simt(cb200_stream* s, T* C, long long ldc, int ta, int tb, T alpha, const T* A, int M, int K, long long lda,
                const T* B, int N, long long ldb, T beta, const T* bias, int act, const PeerList* peer_list = nullptr) {
  DeviceGuard guard(s->device);
  PeerList peers;
  if (peer_list) peers = *peer_list; else peers.n = 0;
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  long long sam = ta ? 1 : lda, sak = ta ? lda : 1;
  long long sbk = tb ? 1 : ldb, sbn = tb ? ldb : 1;
  gemm_simt<T><<<grid, 256, 0, s->stream>>>(C, ldc, A, sam, sak, B, sbk, sbn, M, N, K, alpha, beta, bias, act, peers);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

// ---- skinny outputs (N <= 16, op(A) row-major, op(B) = B^T row-major: a dense layer's small head) ----
// A [M, 16]-or-narrower output is one 64-column tensor-core tile per 128 rows with three quarters of it padding,
// plus the K-slice hand-over: 14.6 us for 128 x 10 x 500.  Here one CTA owns one output row: 128 threads stride
// over K with up to 16 accumulators each (A read once, coalesced; B's N rows stay in L1 / L2), partial sums are
// combined by shuffles inside a warp and in warp order across the four warps (fixed order), and lane n of
// warp 0 finishes column n: alpha, beta, bias, activation -- or the row's softmax, which those lanes hold whole.
constexpr int SKINNY_MAX_N = 16;
constexpr int SKINNY_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(SKINNY_THREADS)
gemm_skinny_nt_kernel(T* C, long long ldc, const T* A, long long lda, const T* B, long long ldb, int M, int N, int K,
                      T alpha, T beta, const T* bias, int act) {
  __shared__ T part[SKINNY_THREADS / 32][SKINNY_MAX_N];
  const int m = (int)blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* a = A + (long long)m * lda;
  // requested now, used after the reduction: the epilogue lanes' bias and C values would otherwise cost a memory
  // round trip each at the very end of a kernel that is nothing but latency
  const bool epi_lane = warp == 0 && lane < N;
  const T bias_v = (epi_lane && bias) ? bias[lane] : (T)0;
  const T c_old = (epi_lane && beta != (T)0) ? C[(long long)m * ldc + lane] : (T)0;
  T acc[SKINNY_MAX_N];
#pragma unroll
  for (int n = 0; n < SKINNY_MAX_N; ++n) acc[n] = (T)0;
#pragma unroll 4
  for (int k = (int)threadIdx.x; k < K; k += SKINNY_THREADS) {
    const T av = a[k];
#pragma unroll
    for (int n = 0; n < SKINNY_MAX_N; ++n)
      if (n < N) acc[n] += av * B[(long long)n * ldb + k];
  }
#pragma unroll
  for (int n = 0; n < SKINNY_MAX_N; ++n) {
    if (n < N) {
      T v = acc[n];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
      if (lane == 0) part[warp][n] = v;
    }
  }
  __syncthreads();
  if (warp != 0) return;
  const bool live = lane < N;
  T o = (T)0;
  if (live) {
    T sum = part[0][lane];
#pragma unroll
    for (int w = 1; w < SKINNY_THREADS / 32; ++w) sum += part[w][lane];
    o = alpha * sum;
    if (beta != (T)0) o += beta * c_old;
    if (bias) o += bias_v;
    if (act != CB200_ACT_SOFTMAX) o = act_apply<T>(o, act);
  }
  if (act == CB200_ACT_SOFTMAX) {
    // softmax of the row with the CPU backend's roundings (cpu/tensor_math.clj:1037-1088): exp(x - max) evaluated
    // in double and stored in the element type, the stored values summed in double, the sum rounded, one divide
    T mt = live ? o : (T)-INFINITY;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const T other = __shfl_xor_sync(0xffffffffu, mt, d);
      mt = other > mt ? other : mt;
    }
    const T et = live ? (T)exp((double)o - (double)mt) : (T)0;
    double tot = (double)et;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, d);
    o = et / (T)tot;
  }
  if (live) C[(long long)m * ldc + lane] = o;
}

// Shapes the skinny kernel takes: small heads in the latency-bound regime (the tensor-core path wins back
// once there are enough rows to fill the SMs with tiles).
bool skinny_ok(int M, int N, int K, int trans_a, int trans_b, const PeerList* peers) {
  // every row's CTA re-reads the N rows of B from L2 (M x N x K x 4 bytes in all): beyond about a million elements
  // of A that traffic costs more than the tensor-core path (4096 x 10 x 4096: 70 us here, 38 us there)
  return !trans_a && trans_b && N >= 1 && N <= SKINNY_MAX_N && M >= 1 && M <= 4096 && K >= 1 && K <= 16384 &&
         (long long)M * K <= (1ll << 20) && (!peers || peers->n == 0);
}

template <typename T>
int launch_skinny(cb200_stream* s, T* C, long long ldc, T alpha, const T* A, int M, int K, long long lda, const T* B, int N,
                  long long ldb, T beta, const T* bias, int act) {
  DeviceGuard guard(s->device);
  gemm_skinny_nt_kernel<T><<<(unsigned)M, SKINNY_THREADS, 0, s->stream>>>(C, ldc, A, lda, B, ldb, M, N, K, alpha, beta, bias, act);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

// tensor-core fp32 path.  (A CTA-pair variant with tcgen05.mma.cta_group::2 and 256 x 256 tiles was
// built and measured: correct, but 142 vs 210 TFLOP/s at 4096^3 -- the lo pass over shared memory
// slows to 1000-2000 cycles per k-block while the pair's MMAs stream operands -- so single CTAs stay.)
int tc_f32(cb200_stream* s, float* C, long long ldc, int ta, int tb, float alpha, const float* A, int M, int K,
           long long lda, const float* B, int N, long long ldb, float beta, const float* bias, int act,
           const PeerList* peers, int flags) {
  return cb200_gemm_tf32x3_launch_peers(s, C, ldc, ta, tb, alpha, A, M, K, lda, B, N, ldb, beta, bias, act, 0, 1, flags,
                                        peers ? peers->n : 0, peers ? (float* const*)peers->p : nullptr);
}

int gemm_impl(cb200_stream* s, int dtype, void* C, int64_t ldc, int trans_a, int trans_b, double alpha, const void* A,
              int64_t a_rows, int64_t a_cols, int64_t lda, const void* B, int64_t b_cols, int64_t ldb, double beta,
              const void* bias, int act, const PeerList* peers = nullptr, bool layer_stack = false,
              bool allow_workspace = true) {
  CB_REQUIRE(s && C && A && B, "gemm: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "gemm! is only defined for float and double tensors");
  CB_REQUIRE(a_rows >= 0 && a_cols >= 0 && b_cols >= 0, "gemm: negative extent");
  CB_REQUIRE(a_rows <= 2147483647LL && a_cols <= 2147483647LL && b_cols <= 2147483647LL, "gemm: extent over 2^31-1");
  const int M = (int)a_rows, K = (int)a_cols, N = (int)b_cols;
  CB_REQUIRE(ldc >= N, "gemm: ldc %lld smaller than N %d", (long long)ldc, N);
  CB_REQUIRE(lda >= (trans_a ? M : K), "gemm: lda %lld smaller than the stored row of A", (long long)lda);
  CB_REQUIRE(ldb >= (trans_b ? K : N), "gemm: ldb %lld smaller than the stored row of B", (long long)ldb);
  CB_REQUIRE(act >= CB200_ACT_NONE && act <= CB200_ACT_SOFTMAX, "gemm: unknown activation %d", act);
  CB_REQUIRE(act != CB200_ACT_SOFTMAX || !peers || peers->n == 0, "gemm: the softmax epilogue has no peer-store form");
  if (M == 0 || N == 0) return CB200_OK;
  if (skinny_ok(M, N, K, trans_a, trans_b, peers)) {
    if (dtype == CB200_FLOAT)
      return launch_skinny<float>(s, (float*)C, ldc, (float)alpha, (const float*)A, M, K, lda, (const float*)B, N, ldb,
                                  (float)beta, (const float*)bias, act);
    return launch_skinny<double>(s, (double*)C, ldc, alpha, (const double*)A, M, K, lda, (const double*)B, N, ldb, beta,
                                 (const double*)bias, act);
  }
  if (act == CB200_ACT_SOFTMAX) {
    // wider heads: the layer's kernel, then softmax! over the rows of C in place
    int rc = gemm_impl(s, dtype, C, ldc, trans_a, trans_b, alpha, A, a_rows, a_cols, lda, B, b_cols, ldb, beta, bias,
                       CB200_ACT_NONE, peers, layer_stack, allow_workspace);
    if (rc) return rc;
    CB_REQUIRE(ldc <= 2147483647LL, "gemm: row pitch of the softmax output over 2^31-1");
    cb200_dims d;                                    // [M, N] rows of pitch ldc in the wire form (innermost first)
    for (int i = 0; i < 5; ++i) { d.rev_shape[i] = 1; d.rev_strides[i] = (int32_t)ldc; d.index[i] = nullptr; }
    d.rev_shape[0] = N; d.rev_strides[0] = 1;
    d.rev_shape[1] = M;
    return cb200_softmax_eltwise(s, dtype, C, &d, C, &d);
  }
  if (dtype == CB200_FLOAT) {
    const float* a = (const float*)A;
    const float* b = (const float*)B;
    if (cb200_gemm_tf32x3_eligible(a, lda, b, ldb, M, N, K)) {
      // problems that fill the GPU with 256 x 256 tiles: split (and, for MN-major operands, transpose) the
      // operands into the stream's workspace once, then the CTA-pair kernel, whose main loop has no
      // shared-memory pass; its in-kernel accumulator read-outs replace the K chunking below
      if (allow_workspace && (!peers || peers->n == 0) && cb200_gemm_presplit_auto_ok(s, M, N, K, trans_a, trans_b))
        return cb200_gemm_presplit_auto_launch(s, (float*)C, ldc, trans_a, trans_b, (float)alpha, a, M, K, lda, b, N, ldb,
                                               (float)beta, (const float*)bias, act);
      // tcgen05 accumulates with truncation, so the result drifts toward zero by about 7e-9 * K
      // (relative, worst case all-positive data).  Long reductions are therefore cut into K chunks
      // chained through C (beta = 1), each chunk boundary being a round-to-nearest fp32 add in the
      // epilogue; bias and activation join on the last chunk.
      // layer_stack (the fused layer entry points): each launch also splits its K in two inside the kernel
      const int K_CHUNK = 4096;
      const int tc_flags = layer_stack ? 2 /* FLAG_SPLIT_K */ : 0;
      if (K <= K_CHUNK)
        return tc_f32(s, (float*)C, ldc, trans_a, trans_b, (float)alpha, a, M, K, lda, b, N, ldb, (float)beta,
                      (const float*)bias, act, peers, tc_flags);
      // A problem with few output tiles gets its K slices inside ONE launch (up to max_sl CTAs per tile, each
      // over at most K_CHUNK of the reduction, combined in slice order by round-to-nearest adds): a launch then
      // covers K_CHUNK * max_sl of K instead of K_CHUNK (576 x 64 x 200704: 49 launches, 0.95 ms -> 2 launches).
      const int max_sl = (layer_stack || (peers && peers->n > 0)) ? 1 : cb200_gemm_tf32x3_max_slices(s, M, N);
      const long long span = (long long)K_CHUNK * max_sl;
      const int n_chunks = (int)((K + span - 1) / span);
      const int chunk = ((K + n_chunks - 1) / n_chunks + 15) / 16 * 16;     // even chunks, whole k-blocks
      for (int k0 = 0; k0 < K; k0 += chunk) {
        const int kc = (K - k0 < chunk) ? (K - k0) : chunk;
        const bool last = k0 + kc >= K;
        const float* ak = trans_a ? a + (long long)k0 * lda : a + k0;
        const float* bk = trans_b ? b + k0 : b + (long long)k0 * ldb;
        const int need = (kc + K_CHUNK - 1) / K_CHUNK;
        int rc = tc_f32(s, (float*)C, ldc, trans_a, trans_b, (float)alpha, ak, M, kc, lda, bk, N, ldb,
                        k0 == 0 ? (float)beta : 1.0f, last ? (const float*)bias : nullptr, last ? act : 0,
                        last ? peers : nullptr, tc_flags | (need > 1 ? need << 8 : 0));
        if (rc) return rc;
      }
      return CB200_OK;
    }
    return launch_simt<float>(s, (float*)C, ldc, trans_a, trans_b, (float)alpha, a, M, K, lda, b, N, ldb, (float)beta,
                              (const float*)bias, act, peers);
  }
  if (K >= 1)
    return cb200_gemm_f64_launch(s, (double*)C, ldc, trans_a, trans_b, alpha, (const double*)A, M, K, lda,
                                 (const double*)B, N, ldb, beta, (const double*)bias, act, peers);
  return launch_simt<double>(s, (double*)C, ldc, trans_a, trans_b, alpha, (const double*)A, M, K, lda, (const double*)B,
                             N, ldb, beta, (const double*)bias, act, peers);
}

}  // namespace

// gemm! for callers that keep their own data in the stream's workspace (the convolution backward passes):
// same dispatch, but never the path that splits the operands into that workspace
int cb200_gemm_no_workspace(cb200_stream* s, int dtype, void* C, long long ldc, int trans_a, int trans_b, double alpha,
                            const void* A, long long a_rows, long long a_cols, long long lda, const void* B,
                            long long b_cols, long long ldb, double beta) {
  return gemm_impl(s, dtype, C, ldc, trans_a, trans_b, alpha, A, a_rows, a_cols, lda, B, b_cols, ldb, beta, nullptr,
                   CB200_ACT_NONE, nullptr, false, false);
}

// used by conv.cu when the weight pitch is not addressable by TMA
int cb200_gemm_simt_f32_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                               const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                               float beta) {
  return launch_simt<float>(s, C, ldc, trans_a, trans_b, alpha, A, M, K, lda, B, N, ldb, beta, nullptr, 0);
}

extern "C" {

int cb200_gemm(cb200_stream* s, int dtype, void* C, int64_t ldc, int trans_a, int trans_b, double alpha, const void* A,
               int64_t a_rows, int64_t a_cols, int64_t lda, const void* B, int64_t b_cols, int64_t ldb, double beta) {
  return gemm_impl(s, dtype, C, ldc, trans_a, trans_b, alpha, A, a_rows, a_cols, lda, B, b_cols, ldb, beta, nullptr,
                   CB200_ACT_NONE);
}

int cb200_gemm_bias_act(cb200_stream* s, int dtype, void* C, int64_t ldc, int trans_a, int trans_b, double alpha,
                        const void* A, int64_t a_rows, int64_t a_cols, int64_t lda, const void* B, int64_t b_cols,
                        int64_t ldb, double beta, const void* bias, int act) {
  return gemm_impl(s, dtype, C, ldc, trans_a, trans_b, alpha, A, a_rows, a_cols, lda, B, b_cols, ldb, beta, bias, act,
                   nullptr, true);
}

int cb200_gemm_bias_act_peers(cb200_stream* s, int dtype, void* C, int64_t ldc, int trans_a, int trans_b, double alpha,
                              const void* A, int64_t a_rows, int64_t a_cols, int64_t lda, const void* B,
                              int64_t b_cols, int64_t ldb, double beta, const void* bias, int act, int n_peers,
                              void* const* peer_C) {
  CB_REQUIRE(n_peers >= 0 && n_peers <= CB_MAX_PEERS, "gemm_bias_act_peers: n_peers %d outside [0, %d]", n_peers,
             (int)CB_MAX_PEERS);
  CB_REQUIRE(n_peers == 0 || peer_C, "gemm_bias_act_peers: null peer list");
  PeerList peers;
  peers.n = n_peers;
  for (int d = 0; d < CB_MAX_PEERS; ++d) {
    peers.p[d] = d < n_peers ? peer_C[d] : nullptr;
    CB_REQUIRE(d >= n_peers || peers.p[d], "gemm_bias_act_peers: peer destination %d is null", d);
  }
  return gemm_impl(s, dtype, C, ldc, trans_a, trans_b, alpha, A, a_rows, a_cols, lda, B, b_cols, ldb, beta, bias, act,
                   &peers, true);
}

// Test hooks (not part of the public header): force a specific fp32 kernel.
//   which = 0: SIMT kernel; 1: tensor-core kernel with `flags` (1 = single tf32 term, no split)
int cb200_gemm_f32_variant(cb200_stream* s, int which, int flags, void* C, int64_t ldc, int trans_a, int trans_b,
                           double alpha, const void* A, int64_t a_rows, int64_t a_cols, int64_t lda, const void* B,
                           int64_t b_cols, int64_t ldb, double beta) {
  CB_REQUIRE(s && C && A && B, "gemm_f32_variant: null argument");
  const int M = (int)a_rows, K = (int)a_cols, N = (int)b_cols;
  if (which == 0)
    return launch_simt<float>(s, (float*)C, ldc, trans_a, trans_b, (float)alpha, (const float*)A, M, K, lda,
                              (const float*)B, N, ldb, (float)beta, nullptr, 0);
  CB_REQUIRE(cb200_gemm_tf32x3_eligible((const float*)A, lda, (const float*)B, ldb, M, N, K),
             "gemm_f32_variant: operands are not addressable by TMA");
  return cb200_gemm_tf32x3_launch(s, (float*)C, ldc, trans_a, trans_b, (float)alpha, (const float*)A, M, K, lda,
                                  (const float*)B, N, ldb, (float)beta, nullptr, 0, 0, 1, flags);
}

}  // extern "C"
