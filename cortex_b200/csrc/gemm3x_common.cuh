// Pieces shared by the fp32 tensor-core GEMM kernels: launch parameters, the
// hi/lo split, and the epilogue (TMEM -> registers -> alpha*acc + beta*C + bias -> activation -> global).
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace gemm3x {

using namespace sm100;

enum { STORE_ROW_MAJOR = 0, STORE_NCHW = 1 };
enum { FLAG_ONE_TERM = 1, FLAG_SPLIT_K = 2, FLAG_MIN_SLICES_SHIFT = 8 };   // bits 8..15: at least that many K slices
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
  // K split: with k_split == 2 the grid holds every output tile twice; CTA (tile, 0) reduces the first
  // half of K and stores alpha * acc + beta * C, CTA (tile, 1) the second half and stores
  // act(alpha * acc + C + bias) once tile_flags[tile] says the first part is in C.
  int drain_every;     // pre-split kernel only: k-blocks between drains of the main accumulator (0 = never)
  float* C_lo;         // pre-split kernel only: where lo_part(C) goes (same layout as C), or null
  int k_split;
  int split_from;      // pair kernel only: tiles from this index on are computed as two K halves by two clusters
  float* partials;     // pair kernel only: [tail tile][K half][rank][128][BN] partial accumulators
  int split_block;     // tiles per block of (first halves, second halves) in the grid order
  // Problems whose tiles leave SMs free: every tile is reduced by ksplit_n CTAs, each over a slice of K.
  // A CTA parks its raw tile in ksplit_ws[(tile * ksplit_n + slice)][BN / 4][BM] float4; the one that arrives last (per-tile
  // counter in tile_flags) sums the slices in slice order and runs the epilogue.  Nobody waits.
  int ksplit_n;
  int ksplit_cluster;  // 1: the slices of a tile are the CTAs of one thread-block cluster and meet in shared memory
  float* ksplit_ws;
  int* tile_flags;
  int* status;
  // Row-major store only: every finished tile is also written to the same (row, column) position of
  // these buffers, which may live in other GPUs' memory (plain peer stores over NVLink).
  int n_peers;
  float* peers[MAX_PEERS];
};

// tanh / logistic sit behind a call: inlined next to the cheap cases the compiler evaluated all of them
// branch-free for every element (about 150 instructions each, measured 4.5 us per 32 x 32 slab of a
// linear output in the per-element store paths).
static __device__ __noinline__ float apply_act_transcendental(float v, int act) {
  return act == CB200_ACT_TANH ? tanhf(v) : 1.f / (1.f + expf(-v));
}
__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == CB200_ACT_NONE) return v;
  if (act == CB200_ACT_RELU) return v > 0.f ? v : 0.f;
  return apply_act_transcendental(v, act);
}

// lo = x - trunc_tf32(x): exact in fp32; 0 for Inf / NaN so that they propagate through hi alone
__device__ __forceinline__ float lo_part(float x) {
  const uint32_t xb = __float_as_uint(x);
  const float lo = x - __uint_as_float(xb & 0xffffe000u);
  return ((xb & 0x7f800000u) == 0x7f800000u) ? 0.f : lo;
}

// tcgen05 accumulates in fp32 with truncation, so a long reduction shrinks toward zero (about 7e-9 * K
// relative, the same for every output, so it compounds through a stack of layers).  A kernel whose epilogue
// warps are idle during the main loop can move the main accumulator into per-thread partial sums every few
// thousand k values (round-to-nearest adds) and restart it from zero: thread (warp, lane) keeps the BN/2
// values of its own row and column half -- exactly the elements it stores in the epilogue -- in thread-local
// memory (touched once per drain and once in the epilogue).
template <int BN>
__device__ __noinline__ void drain_main(uint32_t tmem_base, int warp, float* part, bool first) {
  const int q = warp & 3, half = warp >> 2;
#pragma unroll 1
  for (int cc = 0; cc < BN / 2 / 32; ++cc) {
    uint32_t r[32];
    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * (BN / 2) + cc * 32), r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      part[cc * 32 + j] = first ? __uint_as_float(r[j]) : part[cc * 32 + j] + __uint_as_float(r[j]);
  }
}

// Epilogue of one 128 x BN accumulator tile held in this CTA's TMEM (main accumulator at column 0,
// cross-term accumulator at column BN).  Called by warps 0-7 (all lanes): warp w reads TMEM lanes
// 32*(w%4).., warps 0-3 take the left half of the columns, warps 4-7 the right half.
// Loads of C in the epilogue.  When C holds the partial tile another CTA stored moments ago the load must
// not be served from a stale L1 line (this SM may have read the original C earlier): L2 only.  Otherwise
// the default path, where the 16-byte pieces of one 128-byte line hit in L1.
__device__ __forceinline__ float ld_c(const float* p, bool partial) { return partial ? __ldcg(p) : *p; }
__device__ __forceinline__ float4 ld_c4(const float* p, bool partial) {
  return partial ? __ldcg(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
}

// Park this CTA's raw accumulators (main + cross terms) for the CTA that combines the K slices of the tile.
// A parked tile is BN / 4 column groups of [128 rows] float4: the 32 lanes of a warp (32 consecutive rows)
// write and read 512 contiguous bytes per instruction.
template <int BN>
__device__ __forceinline__ void dump_tile(const GemmParams& p, uint32_t tmem_base, float* dst, int warp, int lane) {
  const int q = warp & 3, half = warp >> 2;
  constexpr int COLS_PER_HALF = BN / 2;
  float4* slot = reinterpret_cast<float4*>(dst) + (q * 32 + lane);
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
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      __stcg(slot + ((col0 + j) >> 2) * 128, make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                         __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])));
  }
}

// The same parked tile ([BN / 4][128 rows] float4) in this CTA's own shared memory: the cluster form of the hand-over.
template <int BN>
__device__ __forceinline__ void dump_tile_smem(const GemmParams& p, uint32_t tmem_base, float* dst, int warp, int lane) {
  const int q = warp & 3, half = warp >> 2;
  constexpr int COLS_PER_HALF = BN / 2;
  float4* slot = reinterpret_cast<float4*>(dst) + (q * 32 + lane);
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
#pragma unroll
    for (int j = 0; j < 32; j += 4)       // plain stores: the cache-hinted form of dump_tile is for global memory only
      slot[((col0 + j) >> 2) * 128] = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                  __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
  }
}

// `beta_now`: factor applied to what C holds (the caller's beta, or 1 once C holds a partial result).
// `last_pass`: bias, activation and peer stores join only on the pass that completes the tile.
// `staging`: shared memory that is free by now (the pipeline stages), 32 x 36 floats per warp: slabs are
// transposed through it so that global loads / stores cover whole 128-byte row segments.
// WITH_LO: also store lo_part(result) at the same position of p.C_lo (last pass only): the next layer's
// pre-split operand.
// `part` (may be null): BN/2 partial sums per thread drained from the main accumulator earlier (drain_main),
// added to the accumulators before alpha / beta.
template <int BN, bool WITH_LO = false>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t tmem_base, int m0, int n0, int warp,
                                              int lane, float* staging, float beta_now, bool last_pass, bool c_is_partial,
                                              const float* part = nullptr, const float* gather = nullptr,
                                              int gather_n = 0, uint32_t cluster_src = 0, int item = -1) {
      float* c_lo = (WITH_LO && last_pass) ? p.C_lo : nullptr;
      const float* e_bias = last_pass ? p.bias : nullptr;
      const int e_act = last_pass ? p.act : 0;
      const int e_peers = last_pass ? p.n_peers : 0;
      // `item` >= 0 (cluster hand-over): this warp finishes the 32 x 32 slab (q, half, cc) = (item & 3,
      // (item >> 2) & 1, item >> 3) whatever its own index is -- the values come from shared memory, not from
      // the warp's TMEM lanes; `warp` still names its staging slot.
      const int sel = item >= 0 ? item : warp;
      const int q = sel & 3, half = (sel >> 2) & 1;
      const int m = m0 + q * 32 + lane;
      constexpr int COLS_PER_HALF = BN / 2;
      const int cc_lo = item >= 0 ? item >> 3 : 0, cc_hi = item >= 0 ? (item >> 3) + 1 : COLS_PER_HALF / 32;
      constexpr int CHUNK = COLS_PER_HALF < 32 ? COLS_PER_HALF : 32;
      static_assert(CHUNK == 32, "BN must be >= 64");
      bool vec_ok = p.store_mode == STORE_ROW_MAJOR && (p.ldc % 4) == 0 && (((uintptr_t)p.C) & 15) == 0;
      for (int d = 0; d < e_peers; ++d) vec_ok = vec_ok && (((uintptr_t)p.peers[d]) & 15) == 0;
      const bool vec8_ok = vec_ok && e_peers == 0 && (p.ldc % 8) == 0 && (((uintptr_t)p.C) & 31) == 0;
#pragma unroll 1
      for (int cc = cc_lo; cc < cc_hi; ++cc) {
        const int col0 = half * COLS_PER_HALF + cc * 32;
        uint32_t r[32];
        if (cluster_src) {
          // K slices parked in the shared memory of the gather_n CTAs of this cluster (rank = slice): summed in
          // slice order through distributed shared memory, two slices requested per round trip
          const uint32_t off = cluster_src + (uint32_t)(((col0 >> 2) * 128 + (q * 32 + lane)) * 16);
          float4 a[8];
          {
            const uint32_t b0 = mapa(off, 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = ld_dsmem_v4(b0 + j * 2048);
          }
          int sl = 1;
          for (; sl + 1 < gather_n; sl += 2) {
            const uint32_t b0 = mapa(off, (uint32_t)sl), b1 = mapa(off, (uint32_t)sl + 1);
            float4 v0[8], v1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { v0[j] = ld_dsmem_v4(b0 + j * 2048); v1[j] = ld_dsmem_v4(b1 + j * 2048); }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              a[j].x += v0[j].x; a[j].y += v0[j].y; a[j].z += v0[j].z; a[j].w += v0[j].w;
              a[j].x += v1[j].x; a[j].y += v1[j].y; a[j].z += v1[j].z; a[j].w += v1[j].w;
            }
          }
          if (sl < gather_n) {
            const uint32_t b0 = mapa(off, (uint32_t)sl);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 b = ld_dsmem_v4(b0 + j * 2048);
              a[j].x += b.x; a[j].y += b.y; a[j].z += b.z; a[j].w += b.w;
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            r[4 * j] = __float_as_uint(a[j].x); r[4 * j + 1] = __float_as_uint(a[j].y);
            r[4 * j + 2] = __float_as_uint(a[j].z); r[4 * j + 3] = __float_as_uint(a[j].w);
          }
        } else if (gather) {
          // K slices parked by gather_n CTAs (this one included): summed in slice order, whoever runs this.
          // Two slices (sixteen 16-byte loads) are requested before the first is added: the combine costs
          // about gather_n / 2 round trips to L2 per 32 columns instead of one per load.
          constexpr int SLICE4 = 128 * BN / 4;                         // float4 per parked tile
          const float4* g0 = reinterpret_cast<const float4*>(gather) + (col0 >> 2) * 128 + (q * 32 + lane);
          float4 a[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = __ldcg(g0 + j * 128);
          int sl = 1;
          for (; sl + 1 < gather_n; sl += 2) {
            float4 b0[8], b1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              b0[j] = __ldcg(g0 + (long long)sl * SLICE4 + j * 128);
              b1[j] = __ldcg(g0 + (long long)(sl + 1) * SLICE4 + j * 128);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              a[j].x += b0[j].x; a[j].y += b0[j].y; a[j].z += b0[j].z; a[j].w += b0[j].w;
              a[j].x += b1[j].x; a[j].y += b1[j].y; a[j].z += b1[j].z; a[j].w += b1[j].w;
            }
          }
          if (sl < gather_n) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 b = __ldcg(g0 + (long long)sl * SLICE4 + j * 128);
              a[j].x += b.x; a[j].y += b.y; a[j].z += b.z; a[j].w += b.w;
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            r[4 * j] = __float_as_uint(a[j].x); r[4 * j + 1] = __float_as_uint(a[j].y);
            r[4 * j + 2] = __float_as_uint(a[j].z); r[4 * j + 3] = __float_as_uint(a[j].w);
          }
        } else {
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
        }
        if (part) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + part[cc * 32 + j]);
        }
        const int nb = n0 + col0;
        if (e_peers > 0 && vec_ok && staging != nullptr && nb + 32 <= p.N) {
          // Tiles that also go to peer GPUs, whole 32 x 32 slab, 16-byte aligned rows: go through a
          // [32][36]-float shared tile per warp so that every store covers 128 contiguous bytes of a row
          // (8 lanes x 16 B: whole NVLink packets) instead of 16 bytes of 32 different rows.  (For local
          // stores alone this measured 2 % slower than the direct per-lane-row stores below.)  TMEM gives a lane one ROW; the tile
          // is written / read row-wise by (lane = row) and 4-rows-at-a-time by (lane / 8 = row, lane % 8
          // = 16-byte column group); with the 36-float pitch both patterns are bank-conflict free.
          float* t = staging + warp * (32 * 36);
          const int row_base = m0 + q * 32;
          const int sub_row = lane >> 3, col4 = (lane & 7) * 4;
          if (beta_now != 0.f) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int mr = row_base + it * 4 + sub_row;
              float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
              if (mr < p.M) c = ld_c4(p.C + (long long)mr * p.ldc + nb + col4, c_is_partial);
              *reinterpret_cast<float4*>(t + (it * 4 + sub_row) * 36 + col4) = c;
            }
            __syncwarp();
#pragma unroll
            for (int k4 = 0; k4 < 8; ++k4) {
              const float4 c = *reinterpret_cast<const float4*>(t + lane * 36 + k4 * 4);
              r[k4 * 4 + 0] = __float_as_uint(p.alpha * __uint_as_float(r[k4 * 4 + 0]) + beta_now * c.x);
              r[k4 * 4 + 1] = __float_as_uint(p.alpha * __uint_as_float(r[k4 * 4 + 1]) + beta_now * c.y);
              r[k4 * 4 + 2] = __float_as_uint(p.alpha * __uint_as_float(r[k4 * 4 + 2]) + beta_now * c.z);
              r[k4 * 4 + 3] = __float_as_uint(p.alpha * __uint_as_float(r[k4 * 4 + 3]) + beta_now * c.w);
            }
            __syncwarp();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(p.alpha * __uint_as_float(r[j]));
          }
#pragma unroll
          for (int k4 = 0; k4 < 8; ++k4) {
            float4 o;
            o.x = __uint_as_float(r[k4 * 4 + 0]); o.y = __uint_as_float(r[k4 * 4 + 1]);
            o.z = __uint_as_float(r[k4 * 4 + 2]); o.w = __uint_as_float(r[k4 * 4 + 3]);
            if (e_bias) {
              const float4 b = *reinterpret_cast<const float4*>(e_bias + nb + k4 * 4);
              o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
            }
            if (e_act) { o.x = apply_act(o.x, e_act); o.y = apply_act(o.y, e_act); o.z = apply_act(o.z, e_act); o.w = apply_act(o.w, e_act); }
            *reinterpret_cast<float4*>(t + lane * 36 + k4 * 4) = o;
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int mr = row_base + it * 4 + sub_row;
            if (mr < p.M) {
              const float4 v = *reinterpret_cast<const float4*>(t + (it * 4 + sub_row) * 36 + col4);
              const long long off = (long long)mr * p.ldc + nb + col4;
              *reinterpret_cast<float4*>(p.C + off) = v;
              for (int d = 0; d < e_peers; ++d) *reinterpret_cast<float4*>(p.peers[d] + off) = v;
            }
          }
          __syncwarp();
          continue;
        }
        // 16-byte stores also serve a last slab that ends on a multiple of 4 columns (N = 500): the same code as
        // every other slab with a predicate per store, instead of the transposed path below -- that path costs
        // ~2.7 us whatever it stores (it runs once, in one warp, from a cold instruction cache)
        const bool vec4_slab = vec_ok && (nb + 32 <= p.N || (p.N & 3) == 0);
        if (staging != nullptr && p.store_mode == STORE_ROW_MAJOR && !vec4_slab) {
          // Ragged or unaligned slab (the last columns of N, a row pitch that is not a multiple of 16 bytes):
          // transposed through a [32][33]-float shared tile per warp, so that a lane owns a COLUMN and every
          // load of C, store of C and peer store covers consecutive floats of one row.  (One 4-byte store per
          // lane per row with lane = row measured 5-8 us per 32 x 32 slab: 32 partly written sectors per
          // instruction.)  Arithmetic and its order per element are those of the direct paths below.
          float* t = staging + warp * (32 * 36);
#pragma unroll
          for (int j = 0; j < 32; ++j) t[lane * 33 + j] = p.alpha * __uint_as_float(r[j]);
          __syncwarp();
          const int n = nb + lane;
          if (n < p.N) {
            const int row_base = m0 + q * 32;
            const float bias_n = e_bias ? e_bias[n] : 0.f;
            // a compact loop on purpose: this path runs once per launch for one or two warps, straight from a cold
            // instruction cache -- fully unrolled (32 rows) it measured 4 us slower than as a loop
#pragma unroll 1
            for (int rr = 0; rr < 32; ++rr) {
              const int mr = row_base + rr;
              if (mr >= p.M) break;
              const long long off = (long long)mr * p.ldc + n;
              float v = t[rr * 33 + lane];
              if (beta_now != 0.f) v += beta_now * ld_c(p.C + off, c_is_partial);
              if (e_bias) v += bias_n;
              v = apply_act(v, e_act);
              p.C[off] = v;
              if (WITH_LO && c_lo) c_lo[off] = lo_part(v);
              for (int d = 0; d < e_peers; ++d) p.peers[d][off] = v;
            }
          }
          __syncwarp();
          continue;
        }
        if (m < p.M && nb < p.N) {
          if (p.store_mode == STORE_ROW_MAJOR) {
            float* crow = p.C + (long long)m * p.ldc + nb;
            if (vec8_ok && nb + 32 <= p.N) {
              // 32-byte aligned rows: one 256-bit access per sector
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = p.alpha * __uint_as_float(r[j + e]);
                if (beta_now != 0.f) {
                  float c[8];
                  ld_global_v8(crow + j, c, c_is_partial);
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[e] += beta_now * c[e];
                }
                if (e_bias) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[e] += e_bias[nb + j + e];
                }
                if (e_act) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[e] = apply_act(o[e], e_act);
                }
                st_global_v8(crow + j, o);
                if (WITH_LO && c_lo) {
                  float l[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) l[e] = lo_part(o[e]);
                  st_global_v8(c_lo + (long long)m * p.ldc + nb + j, l);
                }
              }
            } else if (vec4_slab) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                if (nb + j >= p.N) break;            // N is a multiple of 4 here whenever the slab is cut short
                float4 o;
                o.x = p.alpha * __uint_as_float(r[j]);
                o.y = p.alpha * __uint_as_float(r[j + 1]);
                o.z = p.alpha * __uint_as_float(r[j + 2]);
                o.w = p.alpha * __uint_as_float(r[j + 3]);
                if (beta_now != 0.f) {
                  float4 c = ld_c4(crow + j, c_is_partial);
                  o.x += beta_now * c.x; o.y += beta_now * c.y; o.z += beta_now * c.z; o.w += beta_now * c.w;
                }
                if (e_bias) {
                  float4 b = *reinterpret_cast<const float4*>(e_bias + nb + j);
                  o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                }
                if (e_act) { o.x = apply_act(o.x, e_act); o.y = apply_act(o.y, e_act); o.z = apply_act(o.z, e_act); o.w = apply_act(o.w, e_act); }
                *reinterpret_cast<float4*>(crow + j) = o;
                if (WITH_LO && c_lo)
                  *reinterpret_cast<float4*>(c_lo + (long long)m * p.ldc + nb + j) =
                      make_float4(lo_part(o.x), lo_part(o.y), lo_part(o.z), lo_part(o.w));
                for (int d = 0; d < e_peers; ++d)
                  *reinterpret_cast<float4*>(p.peers[d] + (long long)m * p.ldc + nb + j) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (nb + j < p.N) {
                  float o = p.alpha * __uint_as_float(r[j]);
                  if (beta_now != 0.f) o += beta_now * ld_c(crow + j, c_is_partial);
                  if (e_bias) o += e_bias[nb + j];
                  o = apply_act(o, e_act);
                  crow[j] = o;
                  if (WITH_LO && c_lo) c_lo[(long long)m * p.ldc + nb + j] = lo_part(o);
                  for (int d = 0; d < e_peers; ++d) p.peers[d][(long long)m * p.ldc + nb + j] = o;
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
                if (beta_now != 0.f) o += beta_now * ld_c(cp, c_is_partial);
                if (e_bias) o += e_bias[nb + j];
                *cp = apply_act(o, e_act);
              }
            }
          }
        }
      }
}

}  // namespace gemm3x
