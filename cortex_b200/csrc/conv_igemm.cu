// fp32 convolution-forward! as an implicit GEMM on the tensor cores: the im2col
// matrix of the reference CPU backend (src/cortex/compute/cpu/tensor_math.clj:1118-1131,
// loop nest of src/cortex/nn/impl.clj:8-90; column k = c*kH*kW + ky*kW + kx, zeros in
// the padding) is never materialised.  GEMM view:
//   M = batch*outH*outW output pixels, N = C_out, K = C_in*kH*kW
//   out[pixel, co] = sum_k im2col[pixel, k] * W[co, k]   (+ out_alpha * out)
// The A operand (im2col rows) is gathered from the NCHW input straight into the
// shared-memory tile the tensor core reads: for a fixed k, 32 consecutive pixels are
// (mostly) consecutive floats in global memory, so A is staged MN-major (128-byte rows
// of 32 pixels, 128-byte swizzle with 32-byte atoms) by 8 gather warps, one pixel per
// lane: coalesced global loads, conflict-free shared stores.  The same warps write the
// hi operand (the raw value) and the lo operand (x - trunc_tf32(x)) of the 3xTF32
// split, and run the lo pass over the W tile that TMA delivers (K-major, 64-byte
// swizzle).  MMA issue, TMEM accumulators (main + cross terms), bounded waits and the
// NCHW-scatter epilogue are as in gemm_tf32x3.cu.
//
// Two gather schemes share the kernel (template flag TAP):
//  * TAP = false, any geometry: K runs in the reference's order (c, ky, kx); every gathered
//    element decodes its own (c, ky, kx).
//  * TAP = true, C_in a multiple of 16: K runs as k' = ((c / 16)*kH*kW + ky*kW + kx)*16 + c % 16, so
//    a 16-wide k-block is ONE filter tap and 16 consecutive channels: the bounds test and the input
//    offset are computed once per k-block and the 8 elements of a thread are loads at a constant
//    stride (one input plane apart).  Consecutive k-blocks walk the taps of the same 16 channels,
//    so they re-read the same few input rows and hit in L1.  The weights are permuted to that order, and split into hi / lo,
//    by a small kernel into the stream's scratch ([2][C_out][K] floats) before the launch, so the
//    main kernel has no W pass at all: TMA delivers both W tiles.  Only the order of the fp32
//    summation over k differs from the reference order.
#include "common.cuh"
#include "sm100.cuh"
#include <mutex>

using namespace sm100;

namespace {

constexpr int CBM = 128;            // pixels per CTA tile
constexpr int CBK = 16;             // k values per stage
constexpr int GATHER_WARPS = 8;
constexpr int CONV_THREADS = (GATHER_WARPS + 2) * 32;

struct ConvParams {
  const float* in;
  float* out;
  int batch, cin, in_h, in_w, out_h, out_w, kh, kw, pad_x, pad_y, stride_x, stride_y;
  int cout, K, M;      // K = cin*kh*kw, M = batch*out_h*out_w
  float out_alpha;
  const float* bias;   // [C_out] added after out_alpha * out, or null
  int act;             // enum cb200_act applied last
  int* status;
};

template <int BN> struct ConvCfg {
  static constexpr int A_TILE = CBM * CBK * 4;          // 8 KiB: 4 boxes of [16 k-rows][32 pixels]
  static constexpr int B_TILE = BN * CBK * 4;
  static constexpr int STAGE = 2 * (A_TILE + B_TILE);   // A_hi | B_hi | A_lo | B_lo
  // BN = 64: 4 stages (~97 KB) so that two CTAs share an SM and one CTA's gather latency hides
  // behind the other's; wider tiles take the whole SM.
  static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1;
  static constexpr int BUDGET = 196608 / CTAS_PER_SM;
  static constexpr int STAGES = (BUDGET / STAGE) > 8 ? 8 : (BUDGET / STAGE);
  // BN = 64: two (main, cross) accumulator pairs, one per k-step of a k-block, so that back-to-back
  // MMAs do not form one dependency chain on a single accumulator; the epilogue adds them.
  static constexpr int ACC_SETS = BN <= 64 ? 2 : 1;
  static constexpr int TMEM_COLS = 2 * BN * ACC_SETS;
  static constexpr int SMEM = STAGES * STAGE + 1024 + 512;   // alignment slack + barriers and the tap table
};

__device__ __forceinline__ float conv_lo_part(float x) {
  const uint32_t xb = __float_as_uint(x);
  const float lo = x - __uint_as_float(xb & 0xffffe000u);
  return ((xb & 0x7f800000u) == 0x7f800000u) ? 0.f : lo;
}

// W[cout][c*khkw + t]  ->  hi / lo [cout][((c/16)*khkw + t)*16 + c%16]   (hi = raw value, lo = x - trunc_tf32(x))
__global__ void __launch_bounds__(256)
conv_prep_weights_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, int cout, int cin,
                         int khkw) {
  const int K = cin * khkw;
  const int total = cout * K;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int co = i / K, kp = i - co * K;
    const int blk = kp >> 4, c16 = kp & 15;
    const int cb = blk / khkw, t = blk - cb * khkw;
    const int c = cb * 16 + c16;
    const float x = w[(long long)co * K + c * khkw + t];
    hi[i] = x;
    lo[i] = conv_lo_part(x);
  }
}

template <int BN, bool TAP>
__global__ void __launch_bounds__(CONV_THREADS, ConvCfg<BN>::CTAS_PER_SM)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmWlo, ConvParams p) {
  typedef ConvCfg<BN> Cfg;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int A_TILE = Cfg::A_TILE, B_TILE = Cfg::B_TILE, RAW = A_TILE + B_TILE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::STAGE);
  uint32_t* tmem_slot = (uint32_t*)(bars + 3 * STAGES + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* tap_off = (int*)(bars + 32);      // [kh*kw <= 32] input offset ky*W + kx of each filter tap

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.cout + BN - 1) / BN;
  const int tile_m = blockIdx.x / tiles_n, tile_n = blockIdx.x % tiles_n;
  const int m0 = tile_m * CBM, n0 = tile_n * BN;
  const int nkb = (p.K + CBK - 1) / CBK;
  const int hw = p.out_h * p.out_w;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_conv = smem_u32(bars + STAGES), bar_empty = smem_u32(bars + 2 * STAGES),
                 bar_acc = smem_u32(bars + 3 * STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      // TAP: the W tiles (TMA) complete on the same barrier as the gather warps, so the MMA warp has
      // one wait per k-block
      mbar_init(bar_conv + 8 * s, TAP ? GATHER_WARPS + 1 : GATHER_WARPS);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 32 && (int)threadIdx.x < p.kh * p.kw)
    tap_off[threadIdx.x] = ((int)threadIdx.x / p.kw) * p.in_w + ((int)threadIdx.x % p.kw);
  if (warp == GATHER_WARPS + 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == GATHER_WARPS && lane == 0) {
    tma_prefetch_desc(&tmW);
    if (TAP) tma_prefetch_desc(&tmWlo);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == GATHER_WARPS) {
    // ---------------------------- TMA producer: W tiles ----------------------------
    // the whole warp runs the loop (warp-uniform control flow); one elected lane issues
    {
      int issued = 0;
      int s = 0;
      uint32_t ph = 0;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 500 + s)) break;
        const uint32_t full = (TAP ? bar_conv : bar_full) + 8 * s;
        if (elect_one()) {
          mbar_arrive_expect_tx(full, TAP ? 2 * B_TILE : B_TILE);
          tma_load_2d(smem_base + s * Cfg::STAGE + A_TILE, &tmW, i * CBK, n0, full);
          if (TAP) tma_load_2d(smem_base + s * Cfg::STAGE + RAW + A_TILE, &tmWlo, i * CBK, n0, full);
        }
        issued = i + 1;
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      if (*abort_flag) {
        for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait((TAP ? bar_conv : bar_full) + 8 * (i % STAGES), (i / STAGES) & 1)) break;
      }
    }
  } else if (warp == GATHER_WARPS + 1) {
    // ---------------------------- MMA issuer ---------------------------------------
    // the whole warp runs the loop; one elected lane issues the MMAs and commits
    {
      const uint32_t idesc = make_idesc_tf32(CBM, BN, 1 /*A: pixels contiguous*/, 0 /*W: K contiguous*/);
      uint32_t accumulate[2] = {0, 0};
      // descriptors of stage 0, k-step 0 as (low, high) words; stages and k-steps only move the
      // start-address field of the low word.
      // A: 32-pixel boxes 2048 B apart, 4-k-row atoms 512 B apart, 1024 B per k-step
      // W: 64-byte rows, 8-row groups 512 B apart, 32 B per k-step
      const uint64_t d_a = make_smem_desc(smem_base, 2048, 512, SWZ_128B_BASE32B);
      const uint64_t d_b = make_smem_desc(smem_base + A_TILE, 16, 512, SWZ_64B);
      const uint32_t a_hiw = (uint32_t)(d_a >> 32), b_hiw = (uint32_t)(d_b >> 32);
      const uint32_t a_low0 = (uint32_t)d_a, b_low0 = (uint32_t)d_b;
      constexpr uint32_t LO_TILE = RAW >> 4, STAGE_STEP = Cfg::STAGE >> 4;
      int s = 0;
      uint32_t ph = 0, stage_off = 0;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(bar_conv + 8 * s, ph, abort_flag, p.status, 600 + s)) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < CBK / 8; ++kk) {
            const uint32_t al = a_low0 + stage_off + kk * (1024 >> 4), bl = b_low0 + stage_off + kk * (32 >> 4);
            const int set = Cfg::ACC_SETS == 2 ? kk : 0;
            const uint32_t tmem_main = tmem_base + set * 2 * BN, tmem_cross = tmem_main + BN;
            const uint32_t acc = (Cfg::ACC_SETS == 1 && kk) ? 1u : accumulate[set];
            mma_tf32_ss_words(tmem_cross, al + LO_TILE, a_hiw, bl, b_hiw, idesc, acc);
            mma_tf32_ss_words(tmem_main, al, a_hiw, bl, b_hiw, idesc, acc);
            mma_tf32_ss_words(tmem_cross, al, a_hiw, bl + LO_TILE, b_hiw, idesc, 1);
          }
          mma_commit(bar_empty + 8 * s);
        }
        accumulate[0] = accumulate[1] = 1;
        __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; stage_off = 0; } else { stage_off += STAGE_STEP; }
      }
      if (elect_one()) mma_commit(bar_acc);
      __syncwarp();
      if (*abort_flag) {
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_acc, 0)) break;
      }
    }
  } else {
    // -------------- im2col gather (hi + lo) and W lo pass, then epilogue (warps 0-7) --------------
    const int tid = threadIdx.x;
    const int pb = warp & 3, khalf = warp >> 2;      // 32-pixel block, which 8 of the 16 k-rows
    const int m = m0 + pb * 32 + lane;
    const bool m_ok = m < p.M;
    const int img = m_ok ? m / hw : 0, pix = m_ok ? m % hw : 0;
    const int oy = pix / p.out_w, ox = pix % p.out_w;
    const int iy0 = oy * p.stride_y - p.pad_y, ix0 = ox * p.stride_x - p.pad_x;
    const float* img_base = p.in + (long long)img * p.cin * p.in_h * p.in_w;
    const int khkw = p.kh * p.kw;
    // byte offset of this lane's element inside a k-row of its box, before the per-row swizzle
    const uint32_t box_off = pb * 2048 + (lane & 7) * 4;
    const uint32_t chunk = lane >> 3;
    // im2col rows of k-block i for this lane's pixel, fetched one k-block ahead so that the
    // global-load latency overlaps the shared-memory work of the current k-block
    // Filters with at most 32 taps (3x3, 5x5): which taps fall inside the image is a per-pixel bit
    // mask computed once, and a tap's input offset comes from a small shared table, so that one
    // gathered element costs a handful of instructions.
    const bool tap_table = khkw <= 32;
    uint32_t tap_valid = 0;
    if (tap_table && m_ok) {
      for (int t = 0; t < khkw; ++t) {
        const int iy = iy0 + t / p.kw, ix = ix0 + t % p.kw;
        if (iy >= 0 && iy < p.in_h && ix >= 0 && ix < p.in_w) tap_valid |= 1u << t;
      }
    }
    const int in_hw = p.in_h * p.in_w;
    const int pix_off = iy0 * p.in_w + ix0;
    auto fetch = [&](int i, float (&v)[8]) {
      const int k0 = i * CBK + khalf * 8;
      int c = k0 / khkw, t = k0 - c * khkw;
      if (tap_table) {
        const float* cb = img_base + (long long)c * in_hw + pix_off;
        const int kleft = p.K - k0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bool valid = ((tap_valid >> t) & 1u) && j < kleft;
          v[j] = valid ? __ldg(cb + tap_off[t]) : 0.f;
          if (++t == khkw) { t = 0; cb += in_hw; }
        }
        return;
      }
      int ky = t / p.kw, kx = t - ky * p.kw;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int iy = iy0 + ky, ix = ix0 + kx;
        const bool valid = m_ok && (k0 + j) < p.K && iy >= 0 && iy < p.in_h && ix >= 0 && ix < p.in_w;
        v[j] = valid ? __ldg(img_base + ((long long)c * p.in_h + iy) * p.in_w + ix) : 0.f;
        if (++kx == p.kw) { kx = 0; if (++ky == p.kh) { ky = 0; ++c; } }
      }
    };
    bool ok = true;
    float vn[8];
    if (TAP) {
      // ---- k-block i = channels 16*(i / taps) + khalf*8 .. +7 at tap (i % taps) ----
      // shared-memory offsets of this thread's 8 k-rows (row = khalf*8 + j): 128 B per row, the
      // 32-byte chunk XOR-ed with (row & 3) = (j & 3)
      const uint32_t row0 = box_off + (uint32_t)khalf * 1024;
      const uint32_t sw0 = row0 + ((chunk ^ 0u) << 5), sw1 = row0 + ((chunk ^ 1u) << 5),
                     sw2 = row0 + ((chunk ^ 2u) << 5), sw3 = row0 + ((chunk ^ 3u) << 5);
      const long long img_off = (long long)img * p.cin * in_hw + (long long)khalf * 8 * in_hw + pix_off;
      int cb = 0, ky = 0, kx = 0;
      auto fetch_tap = [&](float (&v)[8]) {
        const int iy = iy0 + ky, ix = ix0 + kx;
        const bool valid = m_ok && iy >= 0 && iy < p.in_h && ix >= 0 && ix < p.in_w;
        const float* src = p.in + (img_off + (long long)cb * 16 * in_hw + ky * p.in_w + kx);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = valid ? __ldg(src + (long long)j * in_hw) : 0.f;
        if (++kx == p.kw) { kx = 0; if (++ky == p.kh) { ky = 0; ++cb; } }
      };
      if (nkb > 0) fetch_tap(vn);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES, ph = (i / STAGES) & 1;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = vn[j];
        if (i + 1 < nkb) fetch_tap(vn);
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 700 + s)) { ok = false; break; }
        uint8_t* a_hi = smem + s * Cfg::STAGE;
        uint8_t* a_lo = a_hi + RAW;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t off = ((j & 3) == 0 ? sw0 : (j & 3) == 1 ? sw1 : (j & 3) == 2 ? sw2 : sw3) + j * 128;
          *reinterpret_cast<float*>(a_hi + off) = v[j];
          *reinterpret_cast<float*>(a_lo + off) = conv_lo_part(v[j]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_conv + 8 * s);
      }
    } else {
    if (nkb > 0) fetch(0, vn);
    for (int i = 0; i < nkb; ++i) {
      const int s = i % STAGES, ph = (i / STAGES) & 1;
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = vn[j];
      if (i + 1 < nkb) fetch(i + 1, vn);
      // the stage is free once the MMAs that read it have retired
      if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 700 + s)) { ok = false; break; }
      uint8_t* a_hi = smem + s * Cfg::STAGE;
      uint8_t* a_lo = a_hi + RAW;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t row = khalf * 8 + j;
        const uint32_t off = box_off + row * 128 + ((chunk ^ (row & 3)) << 5);
        *reinterpret_cast<float*>(a_hi + off) = v[j];
        *reinterpret_cast<float*>(a_lo + off) = conv_lo_part(v[j]);
      }
      // W tile: lo pass once TMA has landed it
      if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 800 + s)) { ok = false; break; }
      uint8_t* b_hi = a_hi + A_TILE;
      uint8_t* b_lo = b_hi + RAW;
      for (int cidx = tid; cidx < B_TILE / 16; cidx += GATHER_WARPS * 32) {
        const float4 w4 = *reinterpret_cast<const float4*>(b_hi + cidx * 16);
        float4 l;
        l.x = conv_lo_part(w4.x); l.y = conv_lo_part(w4.y); l.z = conv_lo_part(w4.z); l.w = conv_lo_part(w4.w);
        *reinterpret_cast<float4*>(b_lo + cidx * 16) = l;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_conv + 8 * s);
    }
    }
    if (ok) ok = mbar_wait(bar_acc, 0, abort_flag, p.status, 900);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok) {
      const int q = warp & 3, half = warp >> 2;
      const int em = m0 + q * 32 + lane;
      constexpr int COLS_PER_HALF = BN / 2;
      const long long eimg = em / hw, epix = em % hw;
      float* obase = p.out + eimg * (long long)p.cout * hw + epix;
#pragma unroll 1
      for (int cc = 0; cc < COLS_PER_HALF / 32; ++cc) {
        const int col0 = half * COLS_PER_HALF + cc * 32;
        // sum of the (main, cross) accumulators of every set, one 32-column slab at a time
        uint32_t r[32], t[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)col0, r);
        tmem_ld_wait();
#pragma unroll 1
        for (int a = 1; a < 2 * Cfg::ACC_SETS; ++a) {
          tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + col0), t);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(t[j]));
        }
        const int nb = n0 + col0;
        if (em < p.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (nb + j < p.cout) {
              float* cp = obase + (long long)(nb + j) * hw;   // adjacent lanes = adjacent pixels: coalesced
              float o = __uint_as_float(r[j]);
              if (p.out_alpha != 0.f) o += p.out_alpha * (*cp);
              *cp = conv_bias_act(o, p.bias, p.act, nb + j);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == GATHER_WARPS + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn conv_encode_fn() {
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

template <int BN, bool TAP>
int launch_conv(cb200_stream* s, const CUtensorMap& tmW, const CUtensorMap& tmWlo, const ConvParams& p) {
  typedef ConvCfg<BN> Cfg;
  static std::once_flag once[64];
  cudaError_t attr_err = cudaSuccess;
  std::call_once(once[s->device & 63], [&] {
    attr_err = cudaFuncSetAttribute(conv_igemm_kernel<BN, TAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
  });
  if (attr_err != cudaSuccess) return cb200_cuda_fail(attr_err, "cudaFuncSetAttribute", __FILE__, __LINE__);
  long long tiles = (long long)((p.M + CBM - 1) / CBM) * ((p.cout + BN - 1) / BN);
  conv_igemm_kernel<BN, TAP><<<(unsigned)tiles, CONV_THREADS, Cfg::SMEM, s->stream>>>(tmW, tmWlo, p);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

// W[cout][K] -> padded[cout][K4], zero-filled (the generic gather zero-fills k >= K on the A side as well)
__global__ void conv_pad_weights_kernel(const float* __restrict__ w, float* __restrict__ padded, int cout, int K, int K4) {
  const int total = cout * K4;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int co = i / K4, k = i - co * K4;
    padded[i] = k < K ? w[(long long)co * K + k] : 0.f;
  }
}

int encode_weights(CUtensorMap* tm, const float* w, int K, int cout, int BN) {
  EncodeTiledFn fn = conv_encode_fn();
  if (!fn) { cb200_set_error("cuTensorMapEncodeTiled is not available from this driver"); return CB200_ERR_CUDA; }
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)cout};
  cuuint64_t gstride[1] = {(cuuint64_t)K * 4};
  cuuint32_t box[2] = {(cuuint32_t)CBK, (cuuint32_t)BN};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)w, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { cb200_set_error("cuTensorMapEncodeTiled failed with %d for the weights", (int)r); return CB200_ERR_CUDA; }
  return CB200_OK;
}

}  // namespace

// Dense NCHW fp32 input/output, weights [cout][cin*kh*kw] (rows that TMA cannot address -- length not a
// multiple of 4, or an unaligned base -- are copied, zero-padded, into the stream's scratch first).
int cb200_conv_igemm_launch(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                            int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y,
                            int stride_x, int stride_y, float out_alpha, const float* bias, int act) {
  DeviceGuard guard(s->device);
  ConvParams p;
  p.in = in; p.out = out; p.batch = batch; p.cin = cin; p.in_h = in_h; p.in_w = in_w; p.out_h = out_h; p.out_w = out_w;
  p.kh = kh; p.kw = kw; p.pad_x = pad_x; p.pad_y = pad_y; p.stride_x = stride_x; p.stride_y = stride_y;
  p.cout = cout; p.K = cin * kh * kw; p.M = batch * out_h * out_w; p.out_alpha = out_alpha; p.status = s->status_dev; p.bias = bias; p.act = act;
  const int BN = cout > 128 ? 256 : (cout > 64 ? 128 : 64);
  CUtensorMap tmW, tmWlo;
  int rc;
  const long long in_elems = (long long)batch * cin * in_h * in_w;
  if ((cin % 16) == 0 && in_elems < 2147483647LL) {
    // tap-major scheme: permuted hi / lo copies of the weights in the stream's scratch
    void* scratch = nullptr;
    const size_t wbytes = (size_t)cout * p.K * sizeof(float);
    rc = cb200_scratch(s, 2 * wbytes, &scratch);
    if (rc) return rc;
    float* w_hi = (float*)scratch;
    float* w_lo = w_hi + (size_t)cout * p.K;
    const int total = cout * p.K;
    int blocks = (total + 255) / 256;
    if (blocks > s->sm_count * 8) blocks = s->sm_count * 8;
    conv_prep_weights_kernel<<<blocks, 256, 0, s->stream>>>(w, w_hi, w_lo, cout, cin, kh * kw);
    CB_LAUNCH_CHECK(s);
    rc = encode_weights(&tmW, w_hi, p.K, cout, BN);
    if (rc) return rc;
    rc = encode_weights(&tmWlo, w_lo, p.K, cout, BN);
    if (rc) return rc;
    if (BN == 256) return launch_conv<256, true>(s, tmW, tmWlo, p);
    if (BN == 128) return launch_conv<128, true>(s, tmW, tmWlo, p);
    return launch_conv<64, true>(s, tmW, tmWlo, p);
  }
  const float* w_use = w;
  int k_pitch = p.K;
  if ((p.K % 4) != 0 || (((uintptr_t)w) & 15) != 0) {
    // TMA wants 16-byte aligned rows: copy the weights into the stream's scratch with the row length rounded up to 4
    k_pitch = (p.K + 3) & ~3;
    void* scratch = nullptr;
    rc = cb200_scratch(s, (size_t)cout * k_pitch * sizeof(float), &scratch);
    if (rc) return rc;
    const int total = cout * k_pitch;
    int blocks = (total + 255) / 256;
    if (blocks > s->sm_count * 8) blocks = s->sm_count * 8;
    conv_pad_weights_kernel<<<blocks, 256, 0, s->stream>>>(w, (float*)scratch, cout, p.K, k_pitch);
    CB_LAUNCH_CHECK(s);
    w_use = (const float*)scratch;
  }
  rc = encode_weights(&tmW, w_use, k_pitch, cout, BN);
  if (rc) return rc;
  tmWlo = tmW;
  if (BN == 256) return launch_conv<256, false>(s, tmW, tmWlo, p);
  if (BN == 128) return launch_conv<128, false>(s, tmW, tmWlo, p);
  return launch_conv<64, false>(s, tmW, tmWlo, p);
}

