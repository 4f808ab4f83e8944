// fp32 convolution-forward! (stride 1) as an implicit GEMM whose A operand -- the rows of the im2col
// matrix of the reference CPU backend (src/cortex/compute/cpu/tensor_math.clj:1118-1131, loop nest of
// src/cortex/nn/impl.clj:8-90) -- is fetched by TMA: no thread touches an input element.
//
//   M = batch*outH*outW output pixels, N = C_out, K = C_in*kH*kW
//   out[pixel, co] = sum_k im2col[pixel, k] * W[co, k]   (+ out_alpha * out)
//
// K runs channel-block-major / tap-inner: k' = ((c / 16)*kH*kW + ky*kW + kx)*16 + c % 16, so one 16-wide
// k-block is ONE filter tap (ky, kx) of 16 consecutive channels.  For such a k-block the A tile of a
// rectangular patch of output pixels is a rectangular patch of the input, shifted by (kx - pad, ky - pad):
// one tiled TMA load, whose out-of-bounds zero fill supplies the padding.  Two things stand between the
// NCHW input and that load, and one pre-pass removes both:
//   * a TMA copy must start on a 16-byte boundary of the innermost dimension, and in NCHW the innermost
//     dimension is x, where the tap shift kx - pad lands on arbitrary elements;
//   * the tensor core wants either 32 pixels contiguous per k value (MN-major) or the k values of a pixel
//     contiguous (K-major); a shifted NCHW patch is neither.
// `nchw_to_nhwc_split_kernel` writes the input once as NHWC, already split for the 3xTF32 product into
// hi = x and lo = x - trunc_tf32(x) (one HBM-bound pass: input read once, two copies written).  In NHWC the
// innermost dimension is the channel (always a multiple of 16 here), x and y are free coordinates, and a box
// {16 channels, bx, by} lands in shared memory as bx*by pixel rows of 64 bytes: exactly the K-major,
// 64-byte-swizzled operand tile of the GEMM kernels.  A 128-row CTA tile is 1, 2 or 4 such boxes (picked per
// geometry so that the boxes tile the output with the least overhang: 56x56 is covered exactly by 8x8 boxes).
// The weights are permuted to the same k order and split into hi / lo by `conv_prep_weights` (scratch), so
// every operand tile -- A_hi, A_lo, W_hi, W_lo -- arrives by TMA and the main loop contains no generic-proxy
// pass, no proxy fence and no thread-issued load.  Warp roles: 8 = A_hi boxes, 10 = A_lo boxes, 11 = W tiles,
// 9 = TMEM owner + MMA issuer, 0-7 = epilogue (TMEM -> registers -> NCHW stores).  W_lo is staged right behind
// W_hi, so hi x [hi | lo] is ONE instruction of width 2*C_out-tile (main product and the hi x lo cross term side by
// side in TMEM) and lo x hi a second one onto the cross columns: two MMAs per k-step instead of three.
// Persistent CTAs (two per SM for 64-channel tiles, one otherwise), two accumulator buffers in TMEM each.  What bounds it at C_out = 64: shared-memory
// bandwidth (per 16-wide k-block the tensor core reads 28 KB of operands and TMA writes 24 KB: ~52 KB per
// ~440 cycles against 128 B/clk), not the tensor pipe (224 cycles) and not HBM.  Only the order of the fp32
// summation over k differs from the reference.  Every wait is bounded (sm100.cuh).
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>

using namespace sm100;

namespace {

constexpr int TBM = 128;            // pixel rows per CTA tile
constexpr int TBK = 16;             // k values per stage
constexpr int T_EPI_WARPS = 8;
constexpr int T_THREADS = (T_EPI_WARPS + 4) * 32;

struct TmaConvParams {
  float* out;
  float out_alpha;
  const float* bias;   // [C_out] added after out_alpha * out, or null
  int act;             // enum cb200_act applied last
  int batch, cout, out_h, out_w, kh, kw, pad_x, pad_y;
  int stride_x, stride_y;   // 1 or 2: the boxes walk the input with the TMA's traversal stride
  int bx, by, nbox;         // one box = bx x by output pixels; nbox * bx * by = 128
  int tiles_x, tiles_y;     // boxes per image along x / y
  int n_boxes;              // batch * tiles_x * tiles_y
  int nkb;                  // (C_in / 16) * kH * kW
  int* status;
};

template <int BN> struct TmaConvCfg {
  static constexpr int A_TILE = TBM * TBK * 4;          // 8 KiB
  static constexpr int B_TILE = BN * TBK * 4;
  static constexpr int RAW = A_TILE + B_TILE;
  static constexpr int STAGE = 2 * RAW;                 // A_hi | W_hi | W_lo | A_lo
  static constexpr int A_LO_OFF = A_TILE + 2 * B_TILE;  // W_lo sits right behind W_hi: together one 2*BN-row operand
  // 64-channel tiles: TWO persistent CTAs per SM.  One issuing thread sustains one of these narrow MMAs per
  // ~135 cycles (measured: a k-block of four took ~540 cycles per CTA whether one or two CTAs shared the SM),
  // the tensor pipe needs only 48-64 cycles for each, so two issuers are needed to keep it busy.
  static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1;
  static constexpr int BUDGET = 196608 / CTAS_PER_SM;
  static constexpr int STAGES = (BUDGET / STAGE) > 8 ? 8 : (BUDGET / STAGE);
  // two accumulator buffers (main | cross each) so that a tile's read-out overlaps the next tile's MMAs
  static constexpr int TMEM_COLS = 4 * BN;
  static constexpr int SMEM = STAGES * STAGE + 1024 + 256;
};

__device__ __forceinline__ float tconv_lo_part(float x) {
  const uint32_t xb = __float_as_uint(x);
  const float lo = x - __uint_as_float(xb & 0xffffe000u);
  return ((xb & 0x7f800000u) == 0x7f800000u) ? 0.f : lo;
}

// 4-d tiled load {c, x, y, n} into this CTA's shared memory; c * 4 bytes must be a multiple of 16, the other
// coordinates are free and may lie outside the tensor (the box is zero-filled there)
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"((uint64_t)tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// in [N][C][HW]  ->  hi / lo [N][HW][C]   (hi = x, lo = x - trunc_tf32(x)); 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256)
nchw_to_nhwc_split_kernel(const float* __restrict__ in, float* __restrict__ hi, float* __restrict__ lo, int C, int HW) {
  __shared__ float t[32][33];
  const long long img = (long long)blockIdx.z * C * HW;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = c0 + threadIdx.y + 8 * j, p = p0 + threadIdx.x;
    if (c < C && p < HW) t[threadIdx.y + 8 * j][threadIdx.x] = in[img + (long long)c * HW + p];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = p0 + threadIdx.y + 8 * j, c = c0 + threadIdx.x;
    if (p < HW && c < C) {
      const float v = t[threadIdx.x][threadIdx.y + 8 * j];
      hi[img + (long long)p * C + c] = v;
      lo[img + (long long)p * C + c] = tconv_lo_part(v);
    }
  }
}

// W[cout][c*khkw + t]  ->  hi / lo [cout][((c/16)*khkw + t)*16 + c%16]
__global__ void __launch_bounds__(256)
tconv_prep_weights_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int cout, int cin,
                          int khkw) {
  const int K = cin * khkw;
  const int total = cout * K;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int co = i / K, kp = i - co * K;
    const int blk = kp >> 4, c16 = kp & 15;
    const int cb = blk / khkw, t = blk - cb * khkw;
    const float x = w[(long long)co * K + (cb * 16 + c16) * khkw + t];
    hi[i] = x;
    lo[i] = tconv_lo_part(x);
  }
}

// Persistent: CTA c computes tiles c, c + grid, ...  The three producers run ahead across tile boundaries; the
// MMA warp alternates between two accumulator buffers in TMEM; the eight epilogue warps read a finished buffer
// out into registers, hand it back (bar_acc_empty) and only then store to NCHW -- so the tensor cores never wait
// for a tile's stores, its launch or its set-up.  (Measured before: one CTA per tile, two per SM: 45 us of the
// 130 us kernel were per-tile launch / set-up / epilogue, only partly hidden behind the other CTA.)
template <int BN>
__global__ void __launch_bounds__(T_THREADS, TmaConvCfg<BN>::CTAS_PER_SM)
conv_tma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAlo,
                const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmWlo, TmaConvParams p) {
  typedef TmaConvCfg<BN> Cfg;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int A_TILE = Cfg::A_TILE, B_TILE = Cfg::B_TILE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::STAGE);
  // bars[0..S) full (three producers), [S..2S) empty, [2S..2S+2) accumulator buffer ready, [2S+2..2S+4)
  // accumulator buffer read out, [2S+4] used only when unwinding: every MMA issued has retired
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 5);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.cout + BN - 1) / BN;
  const int tiles_m = (p.n_boxes + p.nbox - 1) / p.nbox;
  const int n_tiles = tiles_m * tiles_n;
  const int per_img = p.tiles_x * p.tiles_y;
  const int box_rows = p.bx * p.by;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES), bar_acc_full = smem_u32(bars + 2 * STAGES),
                 bar_acc_empty = bar_acc_full + 16, bar_retired = bar_acc_full + 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 3);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, T_EPI_WARPS);
    }
    mbar_init(bar_retired, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == T_EPI_WARPS + 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (lane == 0) {
    if (warp == T_EPI_WARPS) tma_prefetch_desc(&tmA);
    if (warp == T_EPI_WARPS + 2) tma_prefetch_desc(&tmAlo);
    if (warp == T_EPI_WARPS + 3) { tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmWlo); }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == T_EPI_WARPS || warp == T_EPI_WARPS + 2) {
    // ---------------- A producers: warp 8 the hi boxes, warp 10 the lo boxes ----------------
    // the whole warp runs the loop (warp-uniform control flow); one elected lane issues
    const bool is_hi = warp == T_EPI_WARPS;
    const CUtensorMap* map = is_hi ? &tmA : &tmAlo;
    const uint32_t tile_off = is_hi ? 0u : (uint32_t)Cfg::A_LO_OFF;
    const uint32_t box_bytes = (uint32_t)box_rows * TBK * 4;
    long long issued = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      const int box0 = (tile / tiles_n) * p.nbox;
      const int boxes_here = min(p.nbox, p.n_boxes - box0);
      // coordinates of this tile's boxes (image, first input column / row at tap (0, 0))
      int bn[4], bx0[4], by0[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int id = box0 + b;
        const int img = id / per_img, rem = id - img * per_img;
        bn[b] = img;
        by0[b] = (rem / p.tiles_x) * p.by * p.stride_y - p.pad_y;
        bx0[b] = (rem % p.tiles_x) * p.bx * p.stride_x - p.pad_x;
      }
      int cb = 0, ky = 0, kx = 0;
      for (int i = 0; i < p.nkb; ++i) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1000 + s)) { ok = false; break; }
        const uint32_t full = bar_full + 8 * s;
        const uint32_t dst = smem_base + s * Cfg::STAGE + tile_off;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, box_bytes * boxes_here);
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if (b < boxes_here) tma_load_4d(dst + b * box_bytes, map, cb * 16, bx0[b] + kx, by0[b] + ky, bn[b], full);
        }
        __syncwarp();
        ++issued;
        if (++kx == p.kw) { kx = 0; if (++ky == p.kh) { ky = 0; ++cb; } }
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
    if (*abort_flag) {
      // let copies already issued land before this CTA gives its shared memory back
      for (long long i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_full + 8 * (int)(i % STAGES), (uint32_t)((i / STAGES) & 1))) break;
    }
  } else if (warp == T_EPI_WARPS + 3) {
    // ---------------- W producer: hi and lo tiles of the tile's output channels ----------------
    long long issued = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      const int n0 = (tile % tiles_n) * BN;
      for (int i = 0; i < p.nkb; ++i) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 1100 + s)) { ok = false; break; }
        const uint32_t full = bar_full + 8 * s;
        const uint32_t dst = smem_base + s * Cfg::STAGE + A_TILE;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, 2 * B_TILE);
          tma_load_2d(dst, &tmW, i * TBK, n0, full);
          tma_load_2d(dst + B_TILE, &tmWlo, i * TBK, n0, full);
        }
        __syncwarp();
        ++issued;
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
    if (*abort_flag) {
      for (long long i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_full + 8 * (int)(i % STAGES), (uint32_t)((i / STAGES) & 1))) break;
    }
  } else if (warp == T_EPI_WARPS + 1) {
    // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
    const uint32_t idesc = make_idesc_tf32(TBM, BN, 0, 0);
    const uint32_t idesc_wide = make_idesc_tf32(TBM, 2 * BN, 0, 0);
    // both operands K-major: 64-byte rows (16 k values), 8-row groups 512 B apart, 32 B per k-step
    const uint64_t d_a = make_smem_desc(smem_base, 16, 8 * TBK * 4, SWZ_64B);
    const uint64_t d_b = make_smem_desc(smem_base + A_TILE, 16, 8 * TBK * 4, SWZ_64B);
    const uint32_t a_hiw = (uint32_t)(d_a >> 32), b_hiw = (uint32_t)(d_b >> 32);
    const uint32_t a_low0 = (uint32_t)d_a, b_low0 = (uint32_t)d_b;
    constexpr uint32_t A_LO = Cfg::A_LO_OFF >> 4, STAGE_STEP = Cfg::STAGE >> 4;
    int s = 0;
    uint32_t ph = 0, stage_off = 0;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      // the buffer's previous tile (two tiles ago) must have been read out of TMEM
      if (!mbar_wait(bar_acc_empty + 8 * buf, ((local >> 1) & 1) ^ 1, abort_flag, p.status, 1250)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_main = tmem_base + buf * 2 * BN, tmem_cross = tmem_main + BN;
      uint32_t accumulate = 0;
      for (int i = 0; i < p.nkb; ++i) {
        if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 1200 + s)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < TBK / 8; ++kk) {
            const uint32_t al = a_low0 + stage_off + kk * 2, bl = b_low0 + stage_off + kk * 2;
            // A_hi x [W_hi ; W_lo]: columns [0, BN) of the result are the main product, [BN, 2BN) the hi x lo
            // cross term; A_lo x W_hi then adds the other cross term onto columns [BN, 2BN)
            mma_tf32_ss_words(tmem_main, al, a_hiw, bl, b_hiw, idesc_wide, kk ? 1u : accumulate);
            mma_tf32_ss_words(tmem_cross, al + A_LO, a_hiw, bl, b_hiw, idesc, 1);
          }
          mma_commit(bar_empty + 8 * s);
        }
        accumulate = 1;
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; stage_off = 0; } else { stage_off += STAGE_STEP; }
      }
      if (!ok) break;
      if (elect_one()) mma_commit(bar_acc_full + 8 * buf);
      __syncwarp();
    }
    if (*abort_flag) {
      // TMEM is freed below: every MMA issued must have retired by then
      if (elect_one()) mma_commit(bar_retired);
      __syncwarp();
      for (int it = 0; it < (1 << 20); ++it)
        if (mbar_try_wait(bar_retired, 0)) break;
    }
  } else {
    // ---------------- epilogue (warps 0-7): accumulators -> registers -> NCHW ----------------
    const int q = warp & 3, half = warp >> 2;
    const int row = q * 32 + lane;                      // tile row = TMEM lane
    const int b = row / box_rows, within = row - b * box_rows;
    const int ly = within / p.bx, lx = within % p.bx;
    const long long hw = (long long)p.out_h * p.out_w;
    constexpr int COLS_PER_HALF = BN / 2;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      ok = mbar_wait(bar_acc_full + 8 * buf, (local >> 1) & 1, abort_flag, p.status, 1300);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tbase = tmem_base + (uint32_t)(buf * 2 * BN) + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * COLS_PER_HALF);
      float acc[COLS_PER_HALF];
#pragma unroll
      for (int cc = 0; cc < COLS_PER_HALF / 32; ++cc) {
        uint32_t r[32];
        tmem_ld_32x32(tbase + cc * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[cc * 32 + j] = __uint_as_float(r[j]);
        tmem_ld_32x32(tbase + BN + cc * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[cc * 32 + j] += __uint_as_float(r[j]);
      }
      // the buffer may be overwritten by the tile after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      const int box0 = (tile / tiles_n) * p.nbox, n0 = (tile % tiles_n) * BN;
      const int id = box0 + b;
      const int img = id / per_img, rem = id - img * per_img;
      const int oy = (rem / p.tiles_x) * p.by + ly;
      const int ox = (rem % p.tiles_x) * p.bx + lx;
      if (id < p.n_boxes && b < p.nbox && oy < p.out_h && ox < p.out_w) {
        float* obase = p.out + (long long)img * p.cout * hw + (long long)oy * p.out_w + ox;
        const int nb = n0 + half * COLS_PER_HALF;
#pragma unroll
        for (int j = 0; j < COLS_PER_HALF; ++j) {
          if (nb + j < p.cout) {
            float* cp = obase + (long long)(nb + j) * hw;       // lanes of a box row = adjacent pixels
            float o = acc[j];
            if (p.out_alpha != 0.f) o += p.out_alpha * (*cp);
            *cp = conv_bias_act(o, p.bias, p.act, nb + j);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == T_EPI_WARPS + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn tconv_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)f;
  });
  return fn;
}

// NHWC activations [N][H][W][C] as the 4-d tensor {C, W, H, N}; box {16, bx, by, 1} output pixels.  A strided layer
// reads every sx-th column and sy-th row: the map's traversal strides do that (to deliver n elements along a
// dimension with traversal stride s the box extent is n * s), so the tile in shared memory is the same bx x by x 16.
int encode_nhwc(CUtensorMap* tm, const float* base, int C, int W, int H, int N, int bx, int by, int sx, int sy) {
  EncodeTiledFn fn = tconv_encode_fn();
  if (!fn) { cb200_set_error("cuTensorMapEncodeTiled is not available from this driver"); return CB200_ERR_CUDA; }
  cuuint64_t gdim[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t gstride[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
  cuuint32_t box[4] = {(cuuint32_t)TBK, (cuuint32_t)(bx * sx), (cuuint32_t)(by * sy), 1};
  cuuint32_t estr[4] = {1, (cuuint32_t)sx, (cuuint32_t)sy, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)base, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    cb200_set_error("cuTensorMapEncodeTiled failed with %d for the NHWC input (C %d W %d H %d N %d box %dx%d)", (int)r, C,
                    W, H, N, bx, by);
    return CB200_ERR_CUDA;
  }
  return CB200_OK;
}

int encode_w(CUtensorMap* tm, const float* w, int K, int cout, int BN) {
  EncodeTiledFn fn = tconv_encode_fn();
  if (!fn) { cb200_set_error("cuTensorMapEncodeTiled is not available from this driver"); return CB200_ERR_CUDA; }
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)cout};
  cuuint64_t gstride[1] = {(cuuint64_t)K * 4};
  cuuint32_t box[2] = {(cuuint32_t)TBK, (cuuint32_t)BN};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)w, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { cb200_set_error("cuTensorMapEncodeTiled failed with %d for the weights", (int)r); return CB200_ERR_CUDA; }
  return CB200_OK;
}

template <int BN>
int launch_tconv(cb200_stream* s, const CUtensorMap& tmA, const CUtensorMap& tmAlo, const CUtensorMap& tmW,
                 const CUtensorMap& tmWlo, const TmaConvParams& p) {
  typedef TmaConvCfg<BN> Cfg;
  static std::once_flag once[64];
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[s->device & 63], [&] {
    attr_err = cudaFuncSetAttribute(conv_tma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
  });
  if (attr_err != cudaSuccess) return cb200_cuda_fail(attr_err, "cudaFuncSetAttribute", __FILE__, __LINE__);
  const long long tiles_m = (p.n_boxes + p.nbox - 1) / p.nbox;
  const long long tiles = tiles_m * ((p.cout + BN - 1) / BN);
  const long long slots = (long long)s->sm_count * Cfg::CTAS_PER_SM;     // persistent: every resident CTA slot
  const long long grid = tiles < slots ? tiles : slots;
  conv_tma_kernel<BN><<<(unsigned)grid, T_THREADS, Cfg::SMEM, s->stream>>>(tmA, tmAlo, tmW, tmWlo, p);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // namespace

// Which box tiles the output with the least overhang: bx * by in {128, 64, 32}, both powers of two.
// Returns the padded / real pixel ratio (>= 1), or 0 when no geometry qualifies.
double cb200_conv_tma_plan(int out_w, int out_h, int* bx_out, int* by_out, int* nbox_out) {
  double best = 0.0;
  // candidates in order of preference (fewer boxes per tile, then wider rows for the stores): only a strictly
  // smaller overhang replaces an earlier one
  for (int rows = 128; rows >= 32; rows /= 2) {
    for (int bx = rows; bx >= 1; bx /= 2) {
      const int by = rows / bx;
      if (bx > 256 || by > 256) continue;
      const long long padded = (long long)((out_w + bx - 1) / bx) * bx * ((out_h + by - 1) / by) * by;
      const double ratio = (double)padded / ((double)out_w * out_h);
      if (best == 0.0 || ratio < best - 1e-9) {
        best = ratio; *bx_out = bx; *by_out = by; *nbox_out = 128 / rows;
      }
    }
  }
  return best;
}

// Eligible: stride 1 or 2, C_in a multiple of 16, the output tiles with <= 35 % overhang (and a box whose extent
// times the stride stays within the 256 elements a tensor-map box may span).
// Strided layers pay the same layout pre-pass over the whole input for a fraction of the products: they come here
// only when every input element feeds at least ~400 multiply-adds (measured: 64 x 64 x 56 x 56 -> 128, 3 x 3 / 2:
// 93 us here, 85 us on the gather kernel; 1 x 1 / 2: 62 against 31; 32 x 128 x 28 x 28 -> 256, 3 x 3 / 2: 40 against 58).
bool cb200_conv_tma_eligible(int cin, int cout, int kh, int kw, int out_w, int out_h, int stride_x, int stride_y,
                             long long in_elems) {
  if (stride_x < 1 || stride_x > 2 || stride_y < 1 || stride_y > 2 || (cin % 16) != 0 || in_elems >= 2147483647LL) return false;
  if (stride_x * stride_y > 1 && (long long)cout * kh * kw < 400ll * stride_x * stride_y) return false;
  int bx, by, nbox;
  const double ratio = cb200_conv_tma_plan(out_w, out_h, &bx, &by, &nbox);
  return ratio > 0.0 && ratio <= 1.35 && bx * stride_x <= 256 && by * stride_y <= 256;
}

int cb200_conv_tma_launch(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                          int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y,
                          int stride_x, int stride_y, float out_alpha, const float* bias, int act) {
  DeviceGuard guard(s->device);
  TmaConvParams p;
  p.stride_x = stride_x; p.stride_y = stride_y;
  p.out = out; p.out_alpha = out_alpha; p.batch = batch; p.bias = bias; p.act = act; p.cout = cout; p.out_h = out_h; p.out_w = out_w;
  p.kh = kh; p.kw = kw; p.pad_x = pad_x; p.pad_y = pad_y; p.status = s->status_dev;
  cb200_conv_tma_plan(out_w, out_h, &p.bx, &p.by, &p.nbox);
  p.tiles_x = (out_w + p.bx - 1) / p.bx;
  p.tiles_y = (out_h + p.by - 1) / p.by;
  p.n_boxes = batch * p.tiles_x * p.tiles_y;
  p.nkb = (cin / 16) * kh * kw;

  const int K = cin * kh * kw;
  const size_t in_elems = (size_t)batch * cin * in_h * in_w, w_elems = (size_t)cout * K;
  void* scratch = nullptr;
  int rc = cb200_scratch(s, (2 * in_elems + 2 * w_elems) * sizeof(float), &scratch);
  if (rc) return rc;
  float* a_hi = (float*)scratch;
  float* a_lo = a_hi + in_elems;
  float* w_hi = a_lo + in_elems;
  float* w_lo = w_hi + w_elems;
  const int hw = in_h * in_w;
  dim3 tgrid((unsigned)((hw + 31) / 32), (unsigned)((cin + 31) / 32), (unsigned)batch);
  nchw_to_nhwc_split_kernel<<<tgrid, dim3(32, 8, 1), 0, s->stream>>>(in, a_hi, a_lo, cin, hw);
  CB_LAUNCH_CHECK(s);
  int blocks = (int)((w_elems + 255) / 256);
  if (blocks > s->sm_count * 8) blocks = s->sm_count * 8;
  tconv_prep_weights_kernel<<<blocks, 256, 0, s->stream>>>(w, w_hi, w_lo, cout, cin, kh * kw);
  CB_LAUNCH_CHECK(s);
  const int BN = cout > 64 ? 128 : 64;       // wider layers take several 128-channel tiles
  CUtensorMap tmA, tmAlo, tmW, tmWlo;
  if ((rc = encode_nhwc(&tmA, a_hi, cin, in_w, in_h, batch, p.bx, p.by, stride_x, stride_y))) return rc;
  if ((rc = encode_nhwc(&tmAlo, a_lo, cin, in_w, in_h, batch, p.bx, p.by, stride_x, stride_y))) return rc;
  if ((rc = encode_w(&tmW, w_hi, K, cout, BN))) return rc;
  if ((rc = encode_w(&tmWlo, w_lo, K, cout, BN))) return rc;
  if (BN == 128) return launch_tconv<128>(s, tmA, tmAlo, tmW, tmWlo, p);
  return launch_tconv<64>(s, tmA, tmAlo, tmW, tmWlo, p);
}
