// fp32 convolution-forward! (stride 1, filters wider than 1x1) with the input patch kept in shared memory
// across the filter taps.
//
// Same implicit GEMM as conv_tma.cu (M = output pixels, N = C_out, K = C_in*kH*kW, the im2col matrix of
// src/cortex/compute/cpu/tensor_math.clj:1118-1131 / src/cortex/nn/impl.clj:8-90 never materialised), same
// k order (16 channels of ONE filter tap per k-block), same 3xTF32 split with [W_hi ; W_lo] stacked along N.
// What differs is how the A operand reaches the tensor core.  conv_tma.cu loads one shifted 8 KiB tile per tap:
// 9 loads of (almost) the same pixels for a 3x3 filter, and at C_out = 64 that traffic -- L2 to shared memory,
// ~12 TB/s sustained on this part -- is what bounds it.  Here the patch of input pixels a tile touches, halo
// included, is loaded ONCE per 16-channel block, and every tap's A operand is a VIEW of that patch:
//
//   * tile = 8 x 16 output pixels (x by y) of one image; patch = (8 + kW - 1) x (16 + kH - 1) input pixels;
//   * the patch sits in shared memory as [c/4][y][x][4 channels]: one pixel's 4 channels are 16 bytes, the 8
//     pixels of an output row segment are 128 contiguous bytes = one 8-row x 16-byte core matrix of the
//     tensor core's un-swizzled K-major operand layout; the next 8 rows (the next y line) are one patch line
//     further (the descriptor's stride-dimension offset), the next 4 channels one patch plane further (its
//     leading-dimension offset);
//   * tap (ky, kx) only moves the descriptor's start address by (ky * patch_width + kx) * 16 bytes.
//     (Checked on the B200 with a one-instruction probe: arbitrary strides and 16-byte-granular start
//     addresses are honoured by the un-swizzled layout.)
//
// A pre-pass writes the NCHW input as [N][C/4][H][W][4] hi / lo copies (hi = x, lo = x - trunc_tf32(x); one
// HBM-bound pass), which a 5-d TMA box {4, patch_w, patch_h, 4 channel quads, 1} fetches with out-of-bounds
// zero fill as the padding.  The weights are permuted / split as for conv_tma.cu.  Per 3x3 tile the A traffic
// drops from 9 x 16 KiB to 23 KiB per channel block.  Persistent CTAs, two accumulator buffers in TMEM, warp
// roles and bounded waits as in conv_tma.cu.
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>

using namespace sm100;

namespace {

constexpr int HBX = 8, HBY = 16;    // output pixels per tile: 8 wide, 16 high = 128 rows
constexpr int HBK = 16;             // k values per k-block (one tap x 16 channels)
constexpr int H_EPI_WARPS = 8;
constexpr int H_THREADS = (H_EPI_WARPS + 4) * 32;

struct HaloParams {
  float* out;
  float out_alpha;
  const float* bias;          // [C_out] added after out_alpha * out, or null
  int act;                    // enum cb200_act applied last
  int batch, cout, out_h, out_w, kh, kw, pad_x, pad_y;
  int tiles_x, tiles_y;       // tiles per image
  int ncb;                    // C_in / 16
  int patch_w, patch_h;       // HBX + kw - 1, HBY + kh - 1
  int patch_bytes;            // 4 planes x patch_h x patch_w x 16, rounded up to 128
  int n_patches, w_stages;    // ring depths
  int* status;
};

__device__ __forceinline__ float hconv_lo_part(float x) {
  const uint32_t xb = __float_as_uint(x);
  const float lo = x - __uint_as_float(xb & 0xffffe000u);
  return ((xb & 0x7f800000u) == 0x7f800000u) ? 0.f : lo;
}

// 5-d tiled load {c4, x, y, cq, n}; the innermost coordinate is always 0
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"((uint64_t)tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}

// 4-d tiled load {x, y, c, n} of an NCHW tensor; x must be a multiple of 4 elements
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"((uint64_t)tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// in [N][C][HW]  ->  hi / lo [N][C/4][HW][4]: thread = (image, channel quad, pixel); reads of a warp are 128
// contiguous bytes per channel, its writes 512 contiguous bytes
__global__ void __launch_bounds__(256)
nchw_to_c4_split_kernel(const float* __restrict__ in, float4* __restrict__ hi, float4* __restrict__ lo, int CQ, int HW,
                        long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long plane = i / HW;                    // image * CQ + channel quad
    const int p = (int)(i - plane * HW);
    const float* src = in + plane * 4 * HW + p;
    const float a = src[0], b = src[HW], c = src[2 * (long long)HW], d = src[3 * (long long)HW];
    hi[i] = make_float4(a, b, c, d);
    lo[i] = make_float4(hconv_lo_part(a), hconv_lo_part(b), hconv_lo_part(c), hconv_lo_part(d));
  }
}

// W[cout][c*khkw + t]  ->  hi / lo [cout][((c/16)*khkw + t)*16 + c%16]
__global__ void __launch_bounds__(256)
hconv_prep_weights_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int cout, int cin,
                          int khkw) {
  const int K = cin * khkw;
  const int total = cout * K;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int co = i / K, kp = i - co * K;
    const int blk = kp >> 4, c16 = kp & 15;
    const int cb = blk / khkw, t = blk - cb * khkw;
    const float x = w[(long long)co * K + (cb * 16 + c16) * khkw + t];
    hi[i] = x;
    lo[i] = hconv_lo_part(x);
  }
}

// Shared memory: [n_patches x (hi patch | lo patch)] [w_stages x (W_hi | W_lo)] [barriers]
template <int BN>
__global__ void __launch_bounds__(H_THREADS, (BN <= 64 ? 2 : 1))
conv_halo_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAlo,
                 const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmWlo, HaloParams p) {
  constexpr int B_TILE = BN * HBK * 4;
  constexpr int W_STAGE = 2 * B_TILE;
  constexpr int MAX_RING = 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t patch_pair = 2u * (uint32_t)p.patch_bytes;
  const uint32_t w_base_off = ((uint32_t)p.n_patches * patch_pair + 1023u) & ~1023u;
  uint64_t* bars = (uint64_t*)(smem + w_base_off + (uint32_t)p.w_stages * W_STAGE);
  // bars: [0..8) patch full, [8..16) patch empty, [16..24) W full, [24..32) W empty, [32..34) accumulator buffer
  // ready, [34..36) accumulator buffer read out, [36] unwinding only: every MMA issued has retired
  uint32_t* tmem_slot = (uint32_t*)(bars + 37);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.cout + BN - 1) / BN;
  const int per_img = p.tiles_x * p.tiles_y;
  const int n_tiles = p.batch * per_img * tiles_n;
  const int khkw = p.kh * p.kw;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_pfull = bar0, bar_pempty = bar0 + 8 * MAX_RING, bar_wfull = bar0 + 16 * MAX_RING,
                 bar_wempty = bar0 + 24 * MAX_RING, bar_acc_full = bar0 + 32 * MAX_RING, bar_acc_empty = bar_acc_full + 16,
                 bar_retired = bar_acc_full + 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_RING; ++s) {
      mbar_init(bar_pfull + 8 * s, 2);
      mbar_init(bar_pempty + 8 * s, 1);
      mbar_init(bar_wfull + 8 * s, 1);
      mbar_init(bar_wempty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, H_EPI_WARPS);
    }
    mbar_init(bar_retired, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == H_EPI_WARPS + 1) {
    tmem_alloc(smem_u32(tmem_slot), 4 * BN);
    tmem_relinquish();
  }
  if (lane == 0) {
    if (warp == H_EPI_WARPS) tma_prefetch_desc(&tmA);
    if (warp == H_EPI_WARPS + 2) tma_prefetch_desc(&tmAlo);
    if (warp == H_EPI_WARPS + 3) { tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmWlo); }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == H_EPI_WARPS || warp == H_EPI_WARPS + 2) {
    // ---------------- patch producers: warp 8 the hi patches, warp 10 the lo patches ----------------
    const bool is_hi = warp == H_EPI_WARPS;
    const CUtensorMap* map = is_hi ? &tmA : &tmAlo;
    const uint32_t half_off = is_hi ? 0u : (uint32_t)p.patch_bytes;
    const uint32_t bytes = (uint32_t)(4 * p.patch_h * p.patch_w * 16);
    long long issued = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      const int tm = tile / tiles_n;
      const int img = tm / per_img, rem = tm - img * per_img;
      const int y0 = (rem / p.tiles_x) * HBY - p.pad_y, x0 = (rem % p.tiles_x) * HBX - p.pad_x;
      for (int cb = 0; cb < p.ncb; ++cb) {
        if (!mbar_wait(bar_pempty + 8 * s, ph ^ 1, abort_flag, p.status, 1400 + s)) { ok = false; break; }
        const uint32_t full = bar_pfull + 8 * s;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, bytes);
          tma_load_5d(smem_base + s * patch_pair + half_off, map, 0, x0, y0, cb * 4, img, full);
        }
        __syncwarp();
        ++issued;
        if (++s == p.n_patches) { s = 0; ph ^= 1; }
      }
    }
    if (*abort_flag) {
      for (long long i = issued > p.n_patches ? issued - p.n_patches : 0; i < issued; ++i)
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_pfull + 8 * (int)(i % p.n_patches), (uint32_t)((i / p.n_patches) & 1))) break;
    }
  } else if (warp == H_EPI_WARPS + 3) {
    // ---------------- W producer: hi and lo tiles, one pair per (channel block, tap) ----------------
    long long issued = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    const int nkb = p.ncb * khkw;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      const int n0 = (tile % tiles_n) * BN;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(bar_wempty + 8 * s, ph ^ 1, abort_flag, p.status, 1500 + s)) { ok = false; break; }
        const uint32_t full = bar_wfull + 8 * s;
        const uint32_t dst = smem_base + w_base_off + s * W_STAGE;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, W_STAGE);
          tma_load_2d(dst, &tmW, i * HBK, n0, full);
          tma_load_2d(dst + B_TILE, &tmWlo, i * HBK, n0, full);
        }
        __syncwarp();
        ++issued;
        if (++s == p.w_stages) { s = 0; ph ^= 1; }
      }
    }
    if (*abort_flag) {
      for (long long i = issued > p.w_stages ? issued - p.w_stages : 0; i < issued; ++i)
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_wfull + 8 * (int)(i % p.w_stages), (uint32_t)((i / p.w_stages) & 1))) break;
    }
  } else if (warp == H_EPI_WARPS + 1) {
    // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
    const uint32_t idesc = make_idesc_tf32(128, BN, 0, 0);
    const uint32_t idesc_wide = make_idesc_tf32(128, 2 * BN, 0, 0);
    const uint32_t line = (uint32_t)p.patch_w * 16u, plane = (uint32_t)p.patch_h * line;
    // A: un-swizzled K-major view of the patch: 8 pixels of a row = one core matrix (128 B), y lines `line`
    // apart (stride dimension), channel quads `plane` apart (leading dimension); a k-step = 2 quads
    const uint64_t d_a = make_smem_desc(smem_base, plane, line, 0);
    // W: K-major, 64-byte rows, 64-byte swizzle, 8-row groups 512 B apart
    const uint64_t d_b = make_smem_desc(smem_base + w_base_off, 16, 8 * HBK * 4, SWZ_64B);
    const uint32_t a_hiw = (uint32_t)(d_a >> 32), b_hiw = (uint32_t)(d_b >> 32);
    const uint32_t a_low0 = (uint32_t)d_a, b_low0 = (uint32_t)d_b;
    const uint32_t a_lo_off = (uint32_t)p.patch_bytes >> 4, a_kstep = (2u * plane) >> 4, pair_step = patch_pair >> 4;
    int ps = 0, ws = 0;
    uint32_t pph = 0, wph = 0;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      if (!mbar_wait(bar_acc_empty + 8 * buf, ((local >> 1) & 1) ^ 1, abort_flag, p.status, 1650)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_main = tmem_base + buf * 2 * BN, tmem_cross = tmem_main + BN;
      uint32_t accumulate = 0;
      for (int cb = 0; ok && cb < p.ncb; ++cb) {
        if (!mbar_wait(bar_pfull + 8 * ps, pph, abort_flag, p.status, 1600 + ps)) { ok = false; break; }
        const uint32_t a_patch = a_low0 + (uint32_t)ps * pair_step;
        int ky = 0, kx = 0;
        for (int t = 0; t < khkw; ++t) {
          if (!mbar_wait(bar_wfull + 8 * ws, wph, abort_flag, p.status, 1700 + ws)) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) {
            const uint32_t a_tap = a_patch + (uint32_t)(ky * p.patch_w + kx);     // 16 bytes per pixel = 1 unit
            const uint32_t b_st = b_low0 + (uint32_t)ws * (W_STAGE >> 4);
#pragma unroll
            for (int kk = 0; kk < HBK / 8; ++kk) {
              const uint32_t al = a_tap + kk * a_kstep, bl = b_st + kk * 2;
              // A_hi x [W_hi ; W_lo] -> main | hi x lo;   A_lo x W_hi -> onto the cross columns
              mma_tf32_ss_words(tmem_main, al, a_hiw, bl, b_hiw, idesc_wide, kk ? 1u : accumulate);
              mma_tf32_ss_words(tmem_cross, al + a_lo_off, a_hiw, bl, b_hiw, idesc, 1);
            }
            mma_commit(bar_wempty + 8 * ws);
            if (t == khkw - 1) mma_commit(bar_pempty + 8 * ps);       // the patch is free once its last tap retires
          }
          accumulate = 1;
          __syncwarp();
          if (++kx == p.kw) { kx = 0; ++ky; }
          if (++ws == p.w_stages) { ws = 0; wph ^= 1; }
        }
        if (++ps == p.n_patches) { ps = 0; pph ^= 1; }
      }
      if (!ok) break;
      if (elect_one()) mma_commit(bar_acc_full + 8 * buf);
      __syncwarp();
    }
    if (*abort_flag) {
      if (elect_one()) mma_commit(bar_retired);
      __syncwarp();
      for (int it = 0; it < (1 << 20); ++it)
        if (mbar_try_wait(bar_retired, 0)) break;
    }
  } else {
    // ---------------- epilogue (warps 0-7): accumulators -> registers -> NCHW ----------------
    const int q = warp & 3, half = warp >> 2;
    const int row = q * 32 + lane;                      // tile row = TMEM lane: y line row / 8, column row % 8
    const int ly = row >> 3, lx = row & 7;
    const long long hw = (long long)p.out_h * p.out_w;
    constexpr int COLS_PER_HALF = BN / 2;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      ok = mbar_wait(bar_acc_full + 8 * buf, (local >> 1) & 1, abort_flag, p.status, 1800);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      const int tm = tile / tiles_n, n0 = (tile % tiles_n) * BN;
      const int img = tm / per_img, rem = tm - img * per_img;
      const int oy = (rem / p.tiles_x) * HBY + ly, ox = (rem % p.tiles_x) * HBX + lx;
      if (oy < p.out_h && ox < p.out_w) {
        float* obase = p.out + (long long)img * p.cout * hw + (long long)oy * p.out_w + ox;
        const int nb = n0 + half * COLS_PER_HALF;
#pragma unroll
        for (int j = 0; j < COLS_PER_HALF; ++j) {
          if (nb + j < p.cout) {
            float* cp = obase + (long long)(nb + j) * hw;
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
  if (warp == H_EPI_WARPS + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 4 * BN);
  }
}

// ------------------------------------------------------------------------------------------------------
// The same kernel fed from the NCHW input directly: no pre-pass over the activations.
//
// One TMA box {raw_w, patch_h, 16 channels, 1 image} of the caller's tensor (out-of-image coordinates zero-filled:
// the padding) lands in a raw staging buffer as [channel][y][x]; four CONVERT warps re-lay it as the
// [channel quad][y][x][4] hi patch and its lo patch (x - trunc_tf32(x)) in shared memory -- 12 loads and 6 16-byte
// stores per thread and channel block -- issue a generic->async proxy fence and signal the patch as full.  The box
// starts at an x that is a multiple of 4 elements (a TMA box must start on a 16-byte boundary): x_lead = pad_x
// rounded up to 4 columns left of the tile, and the convert step skips x_lead - pad_x columns.
// Warps: 0-3 epilogue (32 rows x BN columns each), 4-7 convert, 8 raw-patch producer, 9 MMA issuer / TMEM owner,
// 11 W producer.  Everything downstream of the patch (descriptors, MMAs, accumulators, epilogue) is as above.
struct DirectExtra {
  int raw_w, raw_bytes, raw_stages, x_lead;
};

template <int BN>
__global__ void __launch_bounds__(H_THREADS, (BN <= 64 ? 2 : 1))
conv_halo_direct_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                        const __grid_constant__ CUtensorMap tmWlo, HaloParams p, DirectExtra x) {
  constexpr int B_TILE = BN * HBK * 4;
  constexpr int W_STAGE = 2 * B_TILE;
  constexpr int MAX_RING = 8;
  constexpr int D_EPI_WARPS = 4, D_CONV_WARPS = 4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t patch_pair = 2u * (uint32_t)p.patch_bytes;
  const uint32_t raw_base_off = ((uint32_t)p.n_patches * patch_pair + 127u) & ~127u;
  const uint32_t w_base_off = (raw_base_off + (uint32_t)x.raw_stages * (uint32_t)x.raw_bytes + 1023u) & ~1023u;
  uint64_t* bars = (uint64_t*)(smem + w_base_off + (uint32_t)p.w_stages * W_STAGE);
  // bars: [0..8) patch full, [8..16) patch empty, [16..24) W full, [24..32) W empty, [32..34) accumulators ready,
  // [34..36) accumulators read out, [36] unwinding only, [37..39) raw full, [39..41) raw empty
  uint32_t* tmem_slot = (uint32_t*)(bars + 41);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.cout + BN - 1) / BN;
  const int per_img = p.tiles_x * p.tiles_y;
  const int n_tiles = p.batch * per_img * tiles_n;
  const int khkw = p.kh * p.kw;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_pfull = bar0, bar_pempty = bar0 + 8 * MAX_RING, bar_wfull = bar0 + 16 * MAX_RING,
                 bar_wempty = bar0 + 24 * MAX_RING, bar_acc_full = bar0 + 32 * MAX_RING, bar_acc_empty = bar_acc_full + 16,
                 bar_retired = bar_acc_full + 32, bar_rfull = bar_retired + 8, bar_rempty = bar_rfull + 16;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_RING; ++s) {
      mbar_init(bar_pfull + 8 * s, D_CONV_WARPS);
      mbar_init(bar_pempty + 8 * s, 1);
      mbar_init(bar_wfull + 8 * s, 1);
      mbar_init(bar_wempty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, D_EPI_WARPS);
      mbar_init(bar_rfull + 8 * b, 1);
      mbar_init(bar_rempty + 8 * b, D_CONV_WARPS);
    }
    mbar_init(bar_retired, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), 4 * BN);
    tmem_relinquish();
  }
  if (lane == 0) {
    if (warp == 8) tma_prefetch_desc(&tmIn);
    if (warp == 11) { tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmWlo); }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---------------- raw-patch producer: one box per (tile, channel block) ----------------
    long long issued = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      const int tm = tile / tiles_n;
      const int img = tm / per_img, rem = tm - img * per_img;
      const int y0 = (rem / p.tiles_x) * HBY - p.pad_y, x0 = (rem % p.tiles_x) * HBX - x.x_lead;
      for (int cb = 0; cb < p.ncb; ++cb) {
        if (!mbar_wait(bar_rempty + 8 * s, ph ^ 1, abort_flag, p.status, 3400 + s)) { ok = false; break; }
        const uint32_t full = bar_rfull + 8 * s;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, (uint32_t)(16 * p.patch_h * x.raw_w * 4));
          tma_load_4d(smem_base + raw_base_off + s * x.raw_bytes, &tmIn, x0, y0, cb * 16, img, full);
        }
        __syncwarp();
        ++issued;
        if (++s == x.raw_stages) { s = 0; ph ^= 1; }
      }
    }
    if (*abort_flag) {
      for (long long i = issued > x.raw_stages ? issued - x.raw_stages : 0; i < issued; ++i)
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_rfull + 8 * (int)(i % x.raw_stages), (uint32_t)((i / x.raw_stages) & 1))) break;
    }
  } else if (warp >= D_EPI_WARPS && warp < D_EPI_WARPS + D_CONV_WARPS) {
    // ---------------- convert warps: raw [c][y][x] -> hi / lo [c/4][y][x][4] ----------------
    const int ct = (warp - D_EPI_WARPS) * 32 + lane;              // 0 .. 127
    const int plane_px = p.patch_h * p.patch_w;                    // pixels per channel quad
    const int n_px = 4 * plane_px;
    const int raw_plane = p.patch_h * x.raw_w;                     // floats per channel in the raw buffer
    const int x_skip = x.x_lead - p.pad_x;
    int rs = 0, ps = 0;
    uint32_t rph = 0, pph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      for (int cb = 0; cb < p.ncb; ++cb) {
        ok = mbar_wait(bar_rfull + 8 * rs, rph, abort_flag, p.status, 3500 + rs) &&
             mbar_wait(bar_pempty + 8 * ps, pph ^ 1, abort_flag, p.status, 3550 + ps);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float* raw = reinterpret_cast<const float*>(smem + raw_base_off + rs * x.raw_bytes);
        float4* hi = reinterpret_cast<float4*>(smem + ps * patch_pair);
        float4* lo = reinterpret_cast<float4*>(smem + ps * patch_pair + p.patch_bytes);
        for (int i = ct; i < n_px; i += D_CONV_WARPS * 32) {
          const int q = i / plane_px, r = i - q * plane_px;
          const int y = r / p.patch_w, px = r - y * p.patch_w;
          const float* src = raw + (4 * q) * raw_plane + y * x.raw_w + px + x_skip;
          const float a = src[0], b = src[raw_plane], c = src[2 * raw_plane], d = src[3 * raw_plane];
          hi[i] = make_float4(a, b, c, d);
          lo[i] = make_float4(hconv_lo_part(a), hconv_lo_part(b), hconv_lo_part(c), hconv_lo_part(d));
        }
        fence_proxy_async_smem();         // these generic-proxy stores -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar_pfull + 8 * ps);
          mbar_arrive(bar_rempty + 8 * rs);
        }
        if (++rs == x.raw_stages) { rs = 0; rph ^= 1; }
        if (++ps == p.n_patches) { ps = 0; pph ^= 1; }
      }
    }
  } else if (warp == 11) {
    // ---------------- W producer: hi and lo tiles, one pair per (channel block, tap) ----------------
    long long issued = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    const int nkb = p.ncb * khkw;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
      const int n0 = (tile % tiles_n) * BN;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(bar_wempty + 8 * s, ph ^ 1, abort_flag, p.status, 3600 + s)) { ok = false; break; }
        const uint32_t full = bar_wfull + 8 * s;
        const uint32_t dst = smem_base + w_base_off + s * W_STAGE;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, W_STAGE);
          tma_load_2d(dst, &tmW, i * HBK, n0, full);
          tma_load_2d(dst + B_TILE, &tmWlo, i * HBK, n0, full);
        }
        __syncwarp();
        ++issued;
        if (++s == p.w_stages) { s = 0; ph ^= 1; }
      }
    }
    if (*abort_flag) {
      for (long long i = issued > p.w_stages ? issued - p.w_stages : 0; i < issued; ++i)
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_wfull + 8 * (int)(i % p.w_stages), (uint32_t)((i / p.w_stages) & 1))) break;
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
    const uint32_t idesc = make_idesc_tf32(128, BN, 0, 0);
    const uint32_t idesc_wide = make_idesc_tf32(128, 2 * BN, 0, 0);
    const uint32_t line = (uint32_t)p.patch_w * 16u, plane = (uint32_t)p.patch_h * line;
    const uint64_t d_a = make_smem_desc(smem_base, plane, line, 0);
    const uint64_t d_b = make_smem_desc(smem_base + w_base_off, 16, 8 * HBK * 4, SWZ_64B);
    const uint32_t a_hiw = (uint32_t)(d_a >> 32), b_hiw = (uint32_t)(d_b >> 32);
    const uint32_t a_low0 = (uint32_t)d_a, b_low0 = (uint32_t)d_b;
    const uint32_t a_lo_off = (uint32_t)p.patch_bytes >> 4, a_kstep = (2u * plane) >> 4, pair_step = patch_pair >> 4;
    int ps = 0, ws = 0;
    uint32_t pph = 0, wph = 0;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      if (!mbar_wait(bar_acc_empty + 8 * buf, ((local >> 1) & 1) ^ 1, abort_flag, p.status, 3650)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_main = tmem_base + buf * 2 * BN, tmem_cross = tmem_main + BN;
      uint32_t accumulate = 0;
      for (int cb = 0; ok && cb < p.ncb; ++cb) {
        if (!mbar_wait(bar_pfull + 8 * ps, pph, abort_flag, p.status, 3700 + ps)) { ok = false; break; }
        const uint32_t a_patch = a_low0 + (uint32_t)ps * pair_step;
        int ky = 0, kx = 0;
        for (int t = 0; t < khkw; ++t) {
          if (!mbar_wait(bar_wfull + 8 * ws, wph, abort_flag, p.status, 3750 + ws)) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) {
            const uint32_t a_tap = a_patch + (uint32_t)(ky * p.patch_w + kx);     // 16 bytes per pixel = 1 unit
            const uint32_t b_st = b_low0 + (uint32_t)ws * (W_STAGE >> 4);
#pragma unroll
            for (int kk = 0; kk < HBK / 8; ++kk) {
              const uint32_t al = a_tap + kk * a_kstep, bl = b_st + kk * 2;
              mma_tf32_ss_words(tmem_main, al, a_hiw, bl, b_hiw, idesc_wide, kk ? 1u : accumulate);
              mma_tf32_ss_words(tmem_cross, al + a_lo_off, a_hiw, bl, b_hiw, idesc, 1);
            }
            mma_commit(bar_wempty + 8 * ws);
            if (t == khkw - 1) mma_commit(bar_pempty + 8 * ps);       // the patch is free once its last tap retires
          }
          accumulate = 1;
          __syncwarp();
          if (++kx == p.kw) { kx = 0; ++ky; }
          if (++ws == p.w_stages) { ws = 0; wph ^= 1; }
        }
        if (++ps == p.n_patches) { ps = 0; pph ^= 1; }
      }
      if (!ok) break;
      if (elect_one()) mma_commit(bar_acc_full + 8 * buf);
      __syncwarp();
    }
    if (*abort_flag) {
      if (elect_one()) mma_commit(bar_retired);
      __syncwarp();
      for (int it = 0; it < (1 << 20); ++it)
        if (mbar_try_wait(bar_retired, 0)) break;
    }
  } else if (warp < D_EPI_WARPS) {
    // ---------------- epilogue (warps 0-3): accumulators -> registers -> NCHW ----------------
    const int row = warp * 32 + lane;                   // tile row = TMEM lane: y line row / 8, column row % 8
    const int ly = row >> 3, lx = row & 7;
    const long long hw = (long long)p.out_h * p.out_w;
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      ok = mbar_wait(bar_acc_full + 8 * buf, (local >> 1) & 1, abort_flag, p.status, 3800);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t tbase = tmem_base + (uint32_t)(buf * 2 * BN) + ((uint32_t)(warp * 32) << 16);
      const int tm = tile / tiles_n, n0 = (tile % tiles_n) * BN;
      const int img = tm / per_img, rem = tm - img * per_img;
      const int oy = (rem / p.tiles_x) * HBY + ly, ox = (rem % p.tiles_x) * HBX + lx;
      const bool inside = oy < p.out_h && ox < p.out_w;
      float* obase = p.out + (long long)img * p.cout * hw + (long long)oy * p.out_w + ox;
      // 32 columns at a time (the buffer is released after the last chunk: the tile after next needs it only a
      // whole tile of MMAs later)
#pragma unroll 1
      for (int cc = 0; cc < BN / 32; ++cc) {
        uint32_t r[32], rc[32];
        tmem_ld_32x32(tbase + cc * 32, r);
        tmem_ld_32x32(tbase + BN + cc * 32, rc);
        tmem_ld_wait();
        if (inside) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = n0 + cc * 32 + j;
            if (n < p.cout) {
              float* cp = obase + (long long)n * hw;
              float o = __uint_as_float(r[j]) + __uint_as_float(rc[j]);
              if (p.out_alpha != 0.f) o += p.out_alpha * (*cp);
              *cp = conv_bias_act(o, p.bias, p.act, n);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 4 * BN);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn hconv_encode_fn() {
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

// activations [N][C/4][H][W][4] as the 5-d tensor {4, W, H, C/4, N}; box {4, patch_w, patch_h, 4, 1}, no swizzle
int encode_c4(CUtensorMap* tm, const float* base, int CQ, int W, int H, int N, int patch_w, int patch_h) {
  EncodeTiledFn fn = hconv_encode_fn();
  if (!fn) { cb200_set_error("cuTensorMapEncodeTiled is not available from this driver"); return CB200_ERR_CUDA; }
  cuuint64_t gdim[5] = {4, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)CQ, (cuuint64_t)N};
  cuuint64_t gstride[4] = {16, (cuuint64_t)W * 16, (cuuint64_t)H * W * 16, (cuuint64_t)CQ * H * W * 16};
  cuuint32_t box[5] = {4, (cuuint32_t)patch_w, (cuuint32_t)patch_h, 4, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, (void*)base, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    cb200_set_error("cuTensorMapEncodeTiled failed with %d for the channel-quad input (CQ %d W %d H %d N %d patch %dx%d)",
                    (int)r, CQ, W, H, N, patch_w, patch_h);
    return CB200_ERR_CUDA;
  }
  return CB200_OK;
}

int encode_hw(CUtensorMap* tm, const float* w, int K, int cout, int BN) {
  EncodeTiledFn fn = hconv_encode_fn();
  if (!fn) { cb200_set_error("cuTensorMapEncodeTiled is not available from this driver"); return CB200_ERR_CUDA; }
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)cout};
  cuuint64_t gstride[1] = {(cuuint64_t)K * 4};
  cuuint32_t box[2] = {(cuuint32_t)HBK, (cuuint32_t)BN};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)w, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { cb200_set_error("cuTensorMapEncodeTiled failed with %d for the weights", (int)r); return CB200_ERR_CUDA; }
  return CB200_OK;
}

// ring depths that fit the per-CTA shared-memory budget; false if not even the minimum does
bool halo_plan(int BN, int kh, int kw, int* patch_bytes, int* n_patches, int* w_stages, int* smem_bytes) {
  const int pw = HBX + kw - 1, ph = HBY + kh - 1;
  if (pw > 256 || ph > 256) return false;
  const int pb = (4 * ph * pw * 16 + 127) & ~127;
  const int w_stage = 2 * BN * HBK * 4;
  const int budget = (BN <= 64 ? 112 : 224) * 1024 - 2048;      // two CTAs per SM for 64-channel tiles
  // two patch pairs are enough (a patch lasts kH*kW k-blocks); the W ring, one stage per k-block, is what
  // covers the load latency: as deep as fits (<= 8), and a third patch pair only if room is left
  int np = 2, ws = 8;
  auto total = [&](int a, int b) { return ((a * 2 * pb + 1023) & ~1023) + b * w_stage + 1024 + 512; };
  while (total(np, ws) > budget && ws > 3) --ws;
  if (total(np, ws) > budget) return false;
  if (total(3, ws) <= budget) np = 3;
  *patch_bytes = pb; *n_patches = np; *w_stages = ws; *smem_bytes = total(np, ws);
  return true;
}

template <int BN>
int launch_halo(cb200_stream* s, const CUtensorMap& tmA, const CUtensorMap& tmAlo, const CUtensorMap& tmW,
                const CUtensorMap& tmWlo, const HaloParams& p, int smem_bytes, long long tiles) {
  static std::mutex mu;
  static int configured[64] = {0};
  {
    std::lock_guard<std::mutex> lock(mu);
    if (configured[s->device & 63] < smem_bytes) {
      cudaError_t e = cudaFuncSetAttribute(conv_halo_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (BN <= 64 ? 112 : 224) * 1024);
      if (e != cudaSuccess) return cb200_cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__);
      configured[s->device & 63] = (BN <= 64 ? 112 : 224) * 1024;
    }
  }
  const long long slots = (long long)s->sm_count * (BN <= 64 ? 2 : 1);
  const long long grid = tiles < slots ? tiles : slots;
  conv_halo_kernel<BN><<<(unsigned)grid, H_THREADS, smem_bytes, s->stream>>>(tmA, tmAlo, tmW, tmWlo, p);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

// NCHW input as the 4-d tensor {W, H, C, N}; box {raw_w, patch_h, 16, 1}, no swizzle, zero fill outside
int encode_nchw(CUtensorMap* tm, const float* base, int W, int H, int C, int N, int raw_w, int patch_h) {
  EncodeTiledFn fn = hconv_encode_fn();
  if (!fn) { cb200_set_error("cuTensorMapEncodeTiled is not available from this driver"); return CB200_ERR_CUDA; }
  cuuint64_t gdim[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C, (cuuint64_t)N};
  cuuint64_t gstride[3] = {(cuuint64_t)W * 4, (cuuint64_t)H * W * 4, (cuuint64_t)C * H * W * 4};
  cuuint32_t box[4] = {(cuuint32_t)raw_w, (cuuint32_t)patch_h, 16, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)base, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    cb200_set_error("cuTensorMapEncodeTiled failed with %d for the NCHW input (W %d H %d C %d N %d box %dx%d)", (int)r, W,
                    H, C, N, raw_w, patch_h);
    return CB200_ERR_CUDA;
  }
  return CB200_OK;
}

// Shared-memory plan of the direct kernel (two CTAs per SM for 64-channel tiles, one for 128-channel tiles): two
// patch pairs, one or two raw staging buffers, the W ring as deep as fits (>= 3 stages).
bool direct_plan(int BN, int kh, int kw, int pad_x, HaloParams* p, DirectExtra* x, int* smem_bytes) {
  const int pw = HBX + kw - 1, ph = HBY + kh - 1;
  if (pw > 256 || ph > 256) return false;
  const int pb = (4 * ph * pw * 16 + 127) & ~127;
  const int x_lead = (pad_x + 3) & ~3;
  const int raw_w = (x_lead + HBX + kw - 1 - pad_x + 3) & ~3;
  if (raw_w > 256 || kw - 1 - pad_x < 0) return false;
  const int raw_bytes = (16 * ph * raw_w * 4 + 127) & ~127;
  const int w_stage = 2 * BN * HBK * 4;
  const int budget = (BN <= 64 ? 112 : 224) * 1024 - 2048;
  auto total = [&](int rs, int ws) {
    const int patches = (2 * 2 * pb + 127) & ~127;
    return ((patches + rs * raw_bytes + 1023) & ~1023) + ws * w_stage + 1024 + 512;
  };
  int rs = 2, ws = 8;
  while (total(rs, ws) > budget && ws > 6) --ws;
  if (total(rs, ws) > budget) { rs = 1; ws = 8; while (total(rs, ws) > budget && ws > 3) --ws; }
  if (total(rs, ws) > budget) return false;
  p->patch_bytes = pb; p->n_patches = 2; p->w_stages = ws;
  x->raw_w = raw_w; x->raw_bytes = raw_bytes; x->raw_stages = rs; x->x_lead = x_lead;
  *smem_bytes = total(rs, ws);
  return true;
}

template <int BN>
int launch_direct(cb200_stream* s, const CUtensorMap& tmIn, const CUtensorMap& tmW, const CUtensorMap& tmWlo,
                  const HaloParams& p, const DirectExtra& x, int smem_bytes, long long tiles) {
  static std::mutex mu;
  static int configured[64] = {0};
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[s->device & 63]) {
      cudaError_t e = cudaFuncSetAttribute(conv_halo_direct_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (BN <= 64 ? 112 : 224) * 1024);
      if (e != cudaSuccess) return cb200_cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__);
      configured[s->device & 63] = 1;
    }
  }
  const long long slots = (long long)s->sm_count * (BN <= 64 ? 2 : 1);
  const long long grid = tiles < slots ? tiles : slots;
  conv_halo_direct_kernel<BN><<<(unsigned)grid, H_THREADS, smem_bytes, s->stream>>>(tmIn, tmW, tmWlo, p, x);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // namespace

// Eligible: stride 1, a filter wider than one tap, C_in a multiple of 16, the 8 x 16 tiles cover the output with
// <= 35 % overhang, and the patch ring fits shared memory.
bool cb200_conv_halo_eligible(int cin, int cout, int out_w, int out_h, int kh, int kw, int stride_x, int stride_y,
                              long long in_elems) {
  if (stride_x != 1 || stride_y != 1 || (cin % 16) != 0 || kh * kw < 2 || in_elems >= 2147483647LL) return false;
  const double padded = (double)((out_w + HBX - 1) / HBX) * HBX * ((out_h + HBY - 1) / HBY) * HBY;
  if (padded > 1.35 * (double)out_w * out_h) return false;
  int pb, np, ws, sm;
  return halo_plan(cout > 64 ? 128 : 64, kh, kw, &pb, &np, &ws, &sm);
}

int cb200_conv_halo_launch(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                           int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y,
                           float out_alpha, const float* bias, int act) {
  DeviceGuard guard(s->device);
  const int BN = cout > 64 ? 128 : 64;
  HaloParams p;
  p.out = out; p.out_alpha = out_alpha; p.batch = batch; p.bias = bias; p.act = act; p.cout = cout; p.out_h = out_h; p.out_w = out_w;
  p.kh = kh; p.kw = kw; p.pad_x = pad_x; p.pad_y = pad_y; p.status = s->status_dev;
  p.tiles_x = (out_w + HBX - 1) / HBX;
  p.tiles_y = (out_h + HBY - 1) / HBY;
  p.ncb = cin / 16;
  p.patch_w = HBX + kw - 1;
  p.patch_h = HBY + kh - 1;
  int smem_bytes = 0;
  const int K = cin * kh * kw;
  // Rows of the input 16-byte aligned: the kernel that reads the caller's NCHW tensor itself (no pre-pass over the
  // activations; only the weights are re-laid, 2 x C_out x K floats of the stream's workspace)
  DirectExtra dx;
  if ((in_w % 4) == 0 && (((uintptr_t)in) & 15) == 0 && s->opt_conv_route != 3 &&
      direct_plan(BN, kh, kw, pad_x, &p, &dx, &smem_bytes)) {
    const size_t w_elems = (size_t)cout * K;
    void* scratch = nullptr;
    int rc = cb200_scratch(s, 2 * w_elems * sizeof(float), &scratch);
    if (rc) return rc;
    float* w_hi = (float*)scratch;
    float* w_lo = w_hi + w_elems;
    int blocks = (int)((w_elems + 255) / 256);
    if (blocks > s->sm_count * 8) blocks = s->sm_count * 8;
    hconv_prep_weights_kernel<<<blocks, 256, 0, s->stream>>>(w, w_hi, w_lo, cout, cin, kh * kw);
    CB_LAUNCH_CHECK(s);
    CUtensorMap tmIn, tmW, tmWlo;
    if ((rc = encode_nchw(&tmIn, in, in_w, in_h, cin, batch, dx.raw_w, p.patch_h))) return rc;
    if ((rc = encode_hw(&tmW, w_hi, K, cout, BN))) return rc;
    if ((rc = encode_hw(&tmWlo, w_lo, K, cout, BN))) return rc;
    const long long tiles = (long long)batch * p.tiles_x * p.tiles_y * ((cout + BN - 1) / BN);
    if (BN == 128) return launch_direct<128>(s, tmIn, tmW, tmWlo, p, dx, smem_bytes, tiles);
    return launch_direct<64>(s, tmIn, tmW, tmWlo, p, dx, smem_bytes, tiles);
  }
  if (!halo_plan(BN, kh, kw, &p.patch_bytes, &p.n_patches, &p.w_stages, &smem_bytes)) {
    cb200_set_error("convolution: the %dx%d filter's input patch does not fit shared memory", kw, kh);
    return CB200_ERR_INVALID;
  }
  const size_t in_elems = (size_t)batch * cin * in_h * in_w, w_elems = (size_t)cout * K;
  void* scratch = nullptr;
  int rc = cb200_scratch(s, (2 * in_elems + 2 * w_elems) * sizeof(float), &scratch);
  if (rc) return rc;
  float* a_hi = (float*)scratch;
  float* a_lo = a_hi + in_elems;
  float* w_hi = a_lo + in_elems;
  float* w_lo = w_hi + w_elems;
  const int hw = in_h * in_w;
  const long long quads = (long long)batch * (cin / 4) * hw;
  long long tb = (quads + 255) / 256;
  if (tb > (long long)s->sm_count * 16) tb = (long long)s->sm_count * 16;
  nchw_to_c4_split_kernel<<<(unsigned)tb, 256, 0, s->stream>>>(in, (float4*)a_hi, (float4*)a_lo, cin / 4, hw, quads);
  CB_LAUNCH_CHECK(s);
  int blocks = (int)((w_elems + 255) / 256);
  if (blocks > s->sm_count * 8) blocks = s->sm_count * 8;
  hconv_prep_weights_kernel<<<blocks, 256, 0, s->stream>>>(w, w_hi, w_lo, cout, cin, kh * kw);
  CB_LAUNCH_CHECK(s);
  CUtensorMap tmA, tmAlo, tmW, tmWlo;
  if ((rc = encode_c4(&tmA, a_hi, cin / 4, in_w, in_h, batch, p.patch_w, p.patch_h))) return rc;
  if ((rc = encode_c4(&tmAlo, a_lo, cin / 4, in_w, in_h, batch, p.patch_w, p.patch_h))) return rc;
  if ((rc = encode_hw(&tmW, w_hi, K, cout, BN))) return rc;
  if ((rc = encode_hw(&tmWlo, w_lo, K, cout, BN))) return rc;
  const long long tiles = (long long)batch * p.tiles_x * p.tiles_y * ((cout + BN - 1) / BN);
  if (BN == 128) return launch_halo<128>(s, tmA, tmAlo, tmW, tmWlo, p, smem_bytes, tiles);
  return launch_halo<64>(s, tmA, tmAlo, tmW, tmWlo, p, smem_bytes, tiles);
}
