// fp64 gemm! on the double-precision tensor-core path (DMMA, mma.sync .f64);
// tcgen05 has no f64 kind.  Replaces cublasDgemm_v2 of the reference backend
// (src/cortex/compute/cuda/tensor_math.clj:127-154).
//
// Two kernels:
//  * gemm_f64_pipe_kernel: operands whose base is 16-byte aligned and whose pitch is even.
//    CTA tile 128 x 128 x 32, 8 warps as 2 (M) x 4 (N), warp tile 64 x 32 = 4 x 4 m16n8k8 tiles.
//    Operand tiles travel global -> shared by 16-byte cp.async in a 3-stage ring (one barrier per
//    k-tile, no register staging).  An operand whose K axis is contiguous in memory is kept
//    [row][k] with a pitch of 36 doubles, the other kind [k][row] with a pitch of 132: both make
//    the fragment loads of a half-warp hit 16 different 8-byte banks.
//  * gemm_f64_kernel (below): any alignment, m8n8k4 tiles, register-staged single buffer.
//
// The second kernel:
// CTA tile 128 x 128 x 16, 8 warps as 2 (M) x 4 (N), warp tile 64 x 32 =
// 8 x 4 m8n8k4 tiles.  Operands are staged k-major in shared memory
// (As[k][m], Bs[k][n]; row pitch 132 doubles keeps the fragment loads
// conflict-free), with the next k-tile prefetched into registers while the
// current one is multiplied.  All four transpose combinations share the kernel:
// only the global->shared thread mapping depends on which axis is contiguous.
#include "common.cuh"
#include <math.h>
#include <mutex>

namespace {

constexpr int DBM = 128, DBN = 128, DBK = 16, DLD = 128 + 4;

__device__ __forceinline__ void dmma(double& d0, double& d1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(d0), "+d"(d1)
               : "d"(a), "d"(b));
}

// tanh / logistic behind a call, so that the epilogue of a layer without them does not evaluate them branch-free
__device__ __noinline__ double act_f64_transcendental(double v, int act) {
  return act == CB200_ACT_TANH ? tanh(v) : 1.0 / (1.0 + exp(-v));
}
__device__ __forceinline__ double act_f64(double v, int act) {
  if (act == CB200_ACT_NONE) return v;
  if (act == CB200_ACT_RELU) return v > 0.0 ? v : 0.0;
  return act_f64_transcendental(v, act);
}

__device__ __forceinline__ void dmma_16x8x8(double (&d)[4], const double (&a)[4], const double (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+d"(d[0]), "+d"(d[1]), "+d"(d[2]), "+d"(d[3])
               : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int PSTAGES = 3;
constexpr int PBK = 32;                          // k-tile of the pipelined kernel (one barrier per 32 k: 16 measured 29.3 TF)
constexpr int KPITCH = PBK + 4;                  // [row][k] layout: doubles per row (conflict-free per half-warp)
constexpr int OPERAND_DOUBLES = 128 * KPITCH;    // >= PBK * DLD
static_assert(OPERAND_DOUBLES >= PBK * DLD, "operand slot too small for the [k][row] layout");
constexpr int PIPE_SMEM = PSTAGES * 2 * OPERAND_DOUBLES * 8;

// Element (row r, k) of an operand tile in shared memory.
template <bool K_CONTIG> __device__ __forceinline__ int tile_at(int r, int k) {
  return K_CONTIG ? r * KPITCH + k : k * DLD + r;
}

// Copy one 128 x PBK operand tile.  K_CONTIG: element (r, k) at g[r*ld + k]; else at g[k*ld + r].
template <bool K_CONTIG>
__device__ __forceinline__ void load_operand_tile(double* sm, const double* g, long long ld, int r0, int k0, int R,
                                                  int K, int t) {
#pragma unroll
  for (int i = 0; i < 128 * PBK / 2 / 256; ++i) {
    const int c = t + 256 * i;
    int r, k, left;
    const double* src;
    if (K_CONTIG) {
      r = c / (PBK / 2); k = (c % (PBK / 2)) * 2;
      left = (r0 + r < R) ? (K - (k0 + k)) : 0;
      src = g + (long long)(r0 + r) * ld + k0 + k;
    } else {
      k = c >> 6; r = (c & 63) * 2;
      left = (k0 + k < K) ? (R - (r0 + r)) : 0;
      src = g + (long long)(k0 + k) * ld + r0 + r;
    }
    const int bytes = left >= 2 ? 16 : (left == 1 ? 8 : 0);
    cp_async_16(sm + tile_at<K_CONTIG>(r, k), bytes ? (const void*)src : (const void*)g, bytes);
  }
}

template <bool A_K_CONTIG, bool B_K_CONTIG>
__global__ void __launch_bounds__(256, 1)
gemm_f64_pipe_kernel(double* C, long long ldc, const double* A, long long lda, const double* B, long long ldb, int M,
                     int N, int K, double alpha, double beta, const double* bias, int act, PeerList peers) {
  extern __shared__ __align__(16) double psm[];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  const int m0 = blockIdx.y * DBM, n0 = blockIdx.x * DBN;
  const int g = lane >> 2, tig = lane & 3;
  const int nk = (K + PBK - 1) / PBK;

  double acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0;

  auto issue = [&](int kt) {
    if (kt < nk) {
      double* as = psm + (kt % PSTAGES) * 2 * OPERAND_DOUBLES;
      load_operand_tile<A_K_CONTIG>(as, A, lda, m0, kt * PBK, M, K, t);
      load_operand_tile<B_K_CONTIG>(as + OPERAND_DOUBLES, B, ldb, n0, kt * PBK, N, K, t);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < PSTAGES - 1; ++s) issue(s);

  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<PSTAGES - 2>();
    __syncthreads();
    issue(kt + PSTAGES - 1);
    const double* as = psm + (kt % PSTAGES) * 2 * OPERAND_DOUBLES;
    const double* bs = as + OPERAND_DOUBLES;
#pragma unroll
    for (int kk = 0; kk < PBK / 8; ++kk) {
      double a[4][4], b[4][2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = wm + i * 16 + g, k = kk * 8 + tig;
        a[i][0] = as[tile_at<A_K_CONTIG>(r, k)];
        a[i][1] = as[tile_at<A_K_CONTIG>(r + 8, k)];
        a[i][2] = as[tile_at<A_K_CONTIG>(r, k + 4)];
        a[i][3] = as[tile_at<A_K_CONTIG>(r + 8, k + 4)];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn + j * 8 + g, k = kk * 8 + tig;
        b[j][0] = bs[tile_at<B_K_CONTIG>(n, k)];
        b[j][1] = bs[tile_at<B_K_CONTIG>(n, k + 4)];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma_16x8x8(acc[i][j], a[i], b[j]);
    }
  }
  cp_async_wait<0>();

  const bool vec = (ldc % 2) == 0 && (((uintptr_t)C) & 15) == 0 && peers.n == 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = m0 + wm + i * 16 + g + h * 8;
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + wn + j * 8 + tig * 2;
        if (n >= N) continue;
        double* c = C + (long long)m * ldc + n;
        double o0 = alpha * acc[i][j][h * 2], o1 = alpha * acc[i][j][h * 2 + 1];
        const bool two = n + 1 < N;
        if (vec && two) {
          if (beta != 0.0) { const double2 cv = *reinterpret_cast<const double2*>(c); o0 += beta * cv.x; o1 += beta * cv.y; }
          if (bias) { o0 += bias[n]; o1 += bias[n + 1]; }
          *reinterpret_cast<double2*>(c) = make_double2(act_f64(o0, act), act_f64(o1, act));
        } else {
          if (beta != 0.0) { o0 += beta * c[0]; if (two) o1 += beta * c[1]; }
          if (bias) { o0 += bias[n]; if (two) o1 += bias[n + 1]; }
          o0 = act_f64(o0, act); o1 = act_f64(o1, act);
          c[0] = o0;
          if (two) c[1] = o1;
          for (int d = 0; d < peers.n; ++d) {
            double* pc = (double*)peers.p[d] + (long long)m * ldc + n;
            pc[0] = o0;
            if (two) pc[1] = o1;
          }
        }
      }
    }
  }
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
  const bool aligned = (((uintptr_t)A | (uintptr_t)B) & 15) == 0 && (lda % 2) == 0 && (ldb % 2) == 0;
  if (aligned && !s->opt_f64_simple) {
    static std::once_flag once[64];
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[s->device & 63], [&] {
      attr_err = cudaFuncSetAttribute(gemm_f64_pipe_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM);
      if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_f64_pipe_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM);
      if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_f64_pipe_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM);
      if (attr_err == cudaSuccess) attr_err = cudaFuncSetAttribute(gemm_f64_pipe_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM);
    });
    if (attr_err != cudaSuccess) return cb200_cuda_fail(attr_err, "cudaFuncSetAttribute", __FILE__, __LINE__);
    // A is K-contiguous when not transposed; B (as N x K) when transposed
#define CB_F64P(AK, BK) \
  gemm_f64_pipe_kernel<AK, BK><<<grid, 256, PIPE_SMEM, s->stream>>>(C, ldc, A, lda, B, ldb, M, N, K, alpha, beta, bias, act, peers)
    if (!trans_a && trans_b) CB_F64P(true, true);
    else if (!trans_a && !trans_b) CB_F64P(true, false);
    else if (trans_a && trans_b) CB_F64P(false, true);
    else CB_F64P(false, false);
#undef CB_F64P
    CB_LAUNCH_CHECK(s);
    return CB200_OK;
  }
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
