// Pieces shared by the fp32 tensor-core GEMM kernels: launch parameters, the
// hi/lo split, and the epilogue (TMEM -> registers -> alpha*acc + beta*C + bias -> activation -> global).
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace gemm3x {

using namespace sm100;

enum { STORE_ROW_MAJOR = 0, STORE_NCHW = 1 };
enum { FLAG_ONE_TERM = 1 };
enum { MAX_PEERS = 7 };

struct GemmParams {
  float* C;
  long long ldc;
  int M, N, K;
  float alpha, beta;
  const float* bias;   // [N] or null
  int act;
  int a_mn_major, b_mn_major;
  int store_mode;
  int hw;              // STORE_NCHW: pixels per image; C[(m / hw) * N * hw + n * hw + m % hw]
  int flags;
  int group_n;         // column tiles per rasterisation group (>= 1)
  int* status;
  // Row-major store only: every finished tile is also written to the same (row, column) position of
  // these buffers, which may live in other GPUs' memory (plain peer stores over NVLink).
  int n_peers;
  float* peers[MAX_PEERS];
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case CB200_ACT_RELU: return v > 0.f ? v : 0.f;
    case CB200_ACT_TANH: return tanhf(v);
    case CB200_ACT_LOGISTIC: return 1.f / (1.f + expf(-v));
  }
  return v;
}

// lo = x - trunc_tf32(x): exact in fp32; 0 for Inf / NaN so that they propagate through hi alone
__device__ __forceinline__ float lo_part(float x) {
  const uint32_t xb = __float_as_uint(x);
  const float lo = x - __uint_as_float(xb & 0xffffe000u);
  return ((xb & 0x7f800000u) == 0x7f800000u) ? 0.f : lo;
}

// Epilogue of one 128 x BN accumulator tile held in this CTA's TMEM (main accumulator at column 0,
// cross-term accumulator at column BN).  Called by warps 0-7 (all lanes): warp w reads TMEM lanes
// 32*(w%4).., warps 0-3 take the left half of the columns, warps 4-7 the right half.
template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t tmem_base, int m0, int n0, int warp,
                                              int lane) {
      const int q = warp & 3, half = warp >> 2;
      const int m = m0 + q * 32 + lane;
      constexpr int COLS_PER_HALF = BN / 2;
      constexpr int CHUNK = COLS_PER_HALF < 32 ? COLS_PER_HALF : 32;
      static_assert(CHUNK == 32, "BN must be >= 64");
      bool vec_ok = p.store_mode == STORE_ROW_MAJOR && (p.ldc % 4) == 0 && (((uintptr_t)p.C) & 15) == 0;
      for (int d = 0; d < p.n_peers; ++d) vec_ok = vec_ok && (((uintptr_t)p.peers[d]) & 15) == 0;
#pragma unroll 1
      for (int cc = 0; cc < COLS_PER_HALF / 32; ++cc) {
        const int col0 = half * COLS_PER_HALF + cc * 32;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col0, r);
        if (!(p.flags & FLAG_ONE_TERM)) {
          uint32_t rc[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(BN + col0), rc);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(rc[j]));
        } else {
          tmem_ld_wait();
        }
        const int nb = n0 + col0;
        if (m < p.M && nb < p.N) {
          if (p.store_mode == STORE_ROW_MAJOR) {
            float* crow = p.C + (long long)m * p.ldc + nb;
            if (vec_ok && nb + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o;
                o.x = p.alpha * __uint_as_float(r[j]);
                o.y = p.alpha * __uint_as_float(r[j + 1]);
                o.z = p.alpha * __uint_as_float(r[j + 2]);
                o.w = p.alpha * __uint_as_float(r[j + 3]);
                if (p.beta != 0.f) {
                  float4 c = *reinterpret_cast<const float4*>(crow + j);
                  o.x += p.beta * c.x; o.y += p.beta * c.y; o.z += p.beta * c.z; o.w += p.beta * c.w;
                }
                if (p.bias) {
                  float4 b = *reinterpret_cast<const float4*>(p.bias + nb + j);
                  o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                }
                if (p.act) { o.x = apply_act(o.x, p.act); o.y = apply_act(o.y, p.act); o.z = apply_act(o.z, p.act); o.w = apply_act(o.w, p.act); }
                *reinterpret_cast<float4*>(crow + j) = o;
                for (int d = 0; d < p.n_peers; ++d)
                  *reinterpret_cast<float4*>(p.peers[d] + (long long)m * p.ldc + nb + j) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (nb + j < p.N) {
                  float o = p.alpha * __uint_as_float(r[j]);
                  if (p.beta != 0.f) o += p.beta * crow[j];
                  if (p.bias) o += p.bias[nb + j];
                  o = apply_act(o, p.act);
                  crow[j] = o;
                  for (int d = 0; d < p.n_peers; ++d) p.peers[d][(long long)m * p.ldc + nb + j] = o;
                }
              }
            }
          } else {
            const long long img = m / p.hw, pix = m % p.hw;
            float* cbase = p.C + img * (long long)p.N * p.hw + pix;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (nb + j < p.N) {
                float* cp = cbase + (long long)(nb + j) * p.hw;
                float o = p.alpha * __uint_as_float(r[j]);
                if (p.beta != 0.f) o += p.beta * (*cp);
                if (p.bias) o += p.bias[nb + j];
                *cp = apply_act(o, p.act);
              }
            }
          }
        }
      }
}

}  // namespace gemm3x
