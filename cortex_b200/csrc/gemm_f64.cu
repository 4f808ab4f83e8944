// fp64 gemm! on the double-precision tensor-core path (DMMA,
// mma.sync.aligned.m8n8k4.f64); tcgen05 has no f64 kind.  Replaces
// cublasDgemm_v2 of the reference backend
// (src/cortex/compute/cuda/tensor_math.clj:127-154).
//
// CTA tile 128 x 128 x 16, 8 warps as 2 (M) x 4 (N), warp tile 64 x 32 =
// 8 x 4 m8n8k4 tiles.  Operands are staged k-major in shared memory
// (As[k][m], Bs[k][n]; row pitch 132 doubles keeps the fragment loads
// conflict-free), with the next k-tile prefetched into registers while the
// current one is multiplied.  All four transpose combinations share the kernel:
// only the global->shared thread mapping depends on which axis is contiguous.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int DBM = 128, DBN = 128, DBK = 16, DLD = 128 + 4;

__device__ __forceinline__ void dmma(double& d0, double& d1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(d0), "+d"(d1)
               : "d"(a), "d"(b));
}

__device__ __forceinline__ double act_f64(double v, int act) {
  switch (act) {
    case CB200_ACT_RELU: return v > 0.0 ? v : 0.0;
    case CB200_ACT_TANH: return tanh(v);
    case CB200_ACT_LOGISTIC: return 1.0 / (1.0 + exp(-v));
  }
  return v;
}

template <bool A_K_CONTIG, bool B_N_CONTIG>
__global__ void __launch_bounds__(256)
gemm_f64_kernel(double* C, long long ldc, const double* A, long long sam, long long sak, const double* B,
                long long sbk, long long sbn, int M, int N, int K, double alpha, double beta, const double* bias,
                int act, PeerList peers) {
  __shared__ double As[DBK][DLD];
  __shared__ double Bs[DBK][DLD];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  const int m0 = blockIdx.y * DBM, n0 = blockIdx.x * DBN;
  const int fr = lane >> 2, fk = lane & 3;

  double acc[8][4][2];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  double ra[8], rb[8];
  auto load_tile = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int k, m;
      if (A_K_CONTIG) { k = t % 16; m = t / 16 + 16 * i; } else { m = t % 128; k = t / 128 + 2 * i; }
      ra[i] = (m0 + m < M && k0 + k < K) ? A[(long long)(m0 + m) * sam + (long long)(k0 + k) * sak] : 0.0;
      int kb, n;
      if (B_N_CONTIG) { n = t % 128; kb = t / 128 + 2 * i; } else { kb = t % 16; n = t / 16 + 16 * i; }
      rb[i] = (n0 + n < N && k0 + kb < K) ? B[(long long)(k0 + kb) * sbk + (long long)(n0 + n) * sbn] : 0.0;
    }
  };
  auto store_tile = [&]() {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int k, m;
      if (A_K_CONTIG) { k = t % 16; m = t / 16 + 16 * i; } else { m = t % 128; k = t / 128 + 2 * i; }
      As[k][m] = ra[i];
      int kb, n;
      if (B_N_CONTIG) { n = t % 128; kb = t / 128 + 2 * i; } else { kb = t % 16; n = t / 16 + 16 * i; }
      Bs[kb][n] = rb[i];
    }
  };

  load_tile(0);
  for (int k0 = 0; k0 < K; k0 += DBK) {
    store_tile();
    __syncthreads();
    if (k0 + DBK < K) load_tile(k0 + DBK);
#pragma unroll
    for (int kk = 0; kk < DBK / 4; ++kk) {
      double a[8], b[4];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = As[kk * 4 + fk][wm + i * 8 + fr];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk * 4 + fk][wn + j * 8 + fr];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma(acc[i][j][0], acc[i][j][1], a[i], b[j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + wm + i * 8 + fr;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int n = n0 + wn + j * 8 + fk * 2 + e;
        if (n >= N) continue;
        double* c = C + (long long)m * ldc + n;
        double o = alpha * acc[i][j][e];
        if (beta != 0.0) o += beta * (*c);
        if (bias) o += bias[n];
        o = act_f64(o, act);
        *c = o;
        for (int d = 0; d < peers.n; ++d) ((double*)peers.p[d])[(long long)m * ldc + n] = o;
      }
    }
  }
}

}  // namespace

int cb200_gemm_f64_launch(cb200_stream* s, double* C, long long ldc, int trans_a, int trans_b, double alpha,
                          const double* A, int M, int K, long long lda, const double* B, int N, long long ldb,
                          double beta, const double* bias, int act, const PeerList* peer_list) {
  DeviceGuard guard(s->device);
  PeerList peers;
  if (peer_list) peers = *peer_list; else peers.n = 0;
  dim3 grid((N + DBN - 1) / DBN, (M + DBM - 1) / DBM);
  const long long sam = trans_a ? 1 : lda, sak = trans_a ? lda : 1;
  const long long sbk = trans_b ? 1 : ldb, sbn = trans_b ? ldb : 1;
#define CB_F64(AK, BNC) \
  gemm_f64_kernel<AK, BNC><<<grid, 256, 0, s->stream>>>(C, ldc, A, sam, sak, B, sbk, sbn, M, N, K, alpha, beta, bias, act, peers)
  if (!trans_a && !trans_b) CB_F64(true, true);
  else if (!trans_a && trans_b) CB_F64(true, false);
  else if (trans_a && !trans_b) CB_F64(false, true);
  else CB_F64(false, false);
#undef CB_F64
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}
