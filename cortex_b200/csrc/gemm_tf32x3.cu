// fp32 gemm! on the 5th-generation tensor cores: C = alpha*op(A)*op(B) + beta*C
// (+ bias row, + activation), fp32 in / fp32 out, computed as a 3xTF32 split:
//   x = hi + lo,  hi = x with the low 13 mantissa bits cleared, lo = x - hi (exact)
//   A*B ~= A_hi*B_hi + (A_lo*B_hi + A_hi*B_lo)     (fp32 accumulation in TMEM)
// The tensor core itself ignores the low 13 bits of an fp32 word fed as tf32, so
// the raw tile TMA delivered IS the hi operand; only lo is computed and stored.
// tcgen05 accumulates with truncation, one truncation per MMA instruction, so the
// bias grows with the number of instructions chained on one accumulator: the two
// small cross terms therefore go to a second TMEM accumulator (their truncation
// error is 2^-11 of the main one's) and the epilogue adds the two in fp32.
// Replaces cublasSgemm_v2 of the reference backend
// (src/cortex/compute/cuda/tensor_math.clj:127-154, 633-649).
//
// One CTA computes a 128 x BN tile of C.  Warp roles:
//   warps 0-7  compute the lo tiles (second buffer) from the raw fp32 tiles that
//              TMA delivered into shared memory, then run the epilogue
//   warp  8    TMA producer (one lane)
//   warp  9    allocates TMEM, issues tcgen05.mma (one lane), frees TMEM
// Per k-block (16 or 32 fp32 = one 64- or 128-byte swizzle row) and pipeline stage:
//   empty[s] -> TMA -> full[s] -> split -> conv[s] -> 12 x tcgen05.mma -> commit -> empty[s]
// All four transpose combinations run on the tensor cores: a non-transposed A /
// transposed B is K-major in memory (128-byte swizzle); the other two are
// MN-major, for which tf32 only has the 128-byte swizzle with 32-byte atoms:
// 32x32 TMA boxes with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B and the matching
// shared-memory descriptor (4 k-rows per atom, atoms 512 B apart along K).
// Operand tiles outside the matrix are zero-filled by TMA, so any M, N, K works;
// pointers must be 16-byte aligned and row pitches a multiple of 4 elements
// (the host falls back to gemm_simt otherwise).
#include "gemm3x_common.cuh"
#include <type_traits>
#include <mutex>

using namespace sm100;
using namespace gemm3x;

namespace {

constexpr int BM = 128;
constexpr int NUM_CONV_WARPS = 8;
constexpr int NUM_THREADS = (NUM_CONV_WARPS + 2) * 32;

// BK = fp32 elements per k-block: 16 (64-byte swizzle rows).  Measured against 32 (128-byte rows,
// 2 stages of 96 KB): the smaller block doubles the number of stages that fit, so the TMA latency
// + lo-tile pass of one stage hides behind more MMA work (173 -> 207 TFLOP/s at 4096^3).
template <int BN, int BK> struct TileCfg {
  static constexpr int A_TILE = BM * BK * 4;
  static constexpr int B_TILE = BN * BK * 4;
  static constexpr int RAW = A_TILE + B_TILE;
  static constexpr int STAGE = 2 * RAW;                 // raw (= hi) tiles + lo tiles
  static constexpr int STAGES = (196608 / STAGE) > 8 ? 8 : (196608 / STAGE);
  static constexpr int TMEM_COLS = 2 * BN;              // main accumulator + cross-term accumulator
  static constexpr int SMEM = STAGES * STAGE + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN, int BK>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  typedef TileCfg<BN, BK> Cfg;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int A_TILE = Cfg::A_TILE;
  // Role loops run either by the whole warp with one elected lane issuing (warp-uniform control
  // flow: cheaper per issued instruction, which narrow tiles and multi-box MN-major loads need) or by
  // lane 0 alone (measured 1-2 % faster for 256-wide tiles fed by two K-major boxes per k-block).
  constexpr bool MMA_WHOLE = BN < 256;
  constexpr int BOX = BK * 128;          // bytes of one 32 x BK MN-major TMA box
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + STAGES * Cfg::STAGE);
  // bars[0..S) full, [S..2S) conv, [2S..3S) empty, [3S] accumulator ready
  uint32_t* tmem_slot = (uint32_t*)(bars + 3 * STAGES + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Tile order: column tiles are taken in groups of p.group_n; inside a group the CTAs sweep all row
  // tiles, so the group's B panel (group_n * BN * K floats) stays in L2 while A streams past it once
  // per group.
  // With a K split the grid holds the tiles twice, in blocks of p.split_block tiles: a block's first K
  // halves, then its second halves (which add onto what the first ones stored while that is still in L2).
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int n_tiles = tiles_m * tiles_n;
  int k_half = 0, tile_id = (int)blockIdx.x, k_slice = 0;
  if (p.ksplit_n > 1) {
    tile_id = (int)blockIdx.x / p.ksplit_n;
    k_slice = (int)blockIdx.x - tile_id * p.ksplit_n;
  }
  if (p.k_split == 2) {
    const int blk = (int)blockIdx.x / (2 * p.split_block);
    const int r = (int)blockIdx.x - blk * 2 * p.split_block;
    const int in_blk = min(p.split_block, n_tiles - blk * p.split_block);
    k_half = r >= in_blk ? 1 : 0;
    tile_id = blk * p.split_block + r - k_half * in_blk;
  }
  const int grp = tile_id / (tiles_m * p.group_n);
  const int rem = tile_id - grp * tiles_m * p.group_n;
  const int in_grp = min(p.group_n, tiles_n - grp * p.group_n);
  const int tile_m = rem / in_grp, tile_n = grp * p.group_n + rem % in_grp;
  const int m0 = tile_m * BM, n0 = tile_n * BN;
  const int nkb_all = (p.K + BK - 1) / BK;
  const int kb_first = p.k_split == 2 ? nkb_all / 2 : nkb_all;       // k-blocks of the first half
  int kb_begin = k_half ? kb_first : 0;
  int nkb = k_half ? nkb_all - kb_first : kb_first;
  if (p.ksplit_n > 1) {
    kb_begin = (int)((long long)nkb_all * k_slice / p.ksplit_n);
    nkb = (int)((long long)nkb_all * (k_slice + 1) / p.ksplit_n) - kb_begin;
  }

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_conv = smem_u32(bars + STAGES), bar_empty = smem_u32(bars + 2 * STAGES),
                 bar_acc = smem_u32(bars + 3 * STAGES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_conv + 8 * s, NUM_CONV_WARPS);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == NUM_CONV_WARPS + 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  int inject = 0;                 // host-injected fault word: requested here so that its latency hides under the set-up
  if (warp == NUM_CONV_WARPS) inject = p.status[3];
  if (warp == NUM_CONV_WARPS && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == NUM_CONV_WARPS) {
    // ------------------------------ TMA producer ------------------------------
    auto producer = [&](auto whole_tag) {
      constexpr bool PROD_WHOLE = decltype(whole_tag)::value;
      if (!PROD_WHOLE && lane != 0) return;
      int issued = 0;
      int s = 0;
      uint32_t ph = 0;
      const bool withhold = (inject & 1) != 0;          // host-injected fault: arm nothing, load nothing
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, p.status, 100 + s)) break;
        const uint32_t full = bar_full + 8 * s;
        const uint32_t a_dst = smem_base + s * Cfg::STAGE, b_dst = a_dst + A_TILE;
        const int k0 = (kb_begin + i) * BK;
        if (withhold) {
          if (++s == STAGES) { s = 0; ph ^= 1; }
          continue;
        }
        if (!PROD_WHOLE || elect_one()) {
          mbar_arrive_expect_tx(full, Cfg::RAW);
          if (!p.a_mn_major) {
            tma_load_2d(a_dst, &tmA, k0, m0, full);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 32; ++j) tma_load_2d(a_dst + j * BOX, &tmA, m0 + 32 * j, k0, full);
          }
          if (!p.b_mn_major) {
            tma_load_2d(b_dst, &tmB, k0, n0, full);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j) tma_load_2d(b_dst + j * BOX, &tmB, n0 + 32 * j, k0, full);
          }
        }
        issued = i + 1;
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
      if (*abort_flag) {
        // let copies already issued land before this CTA gives its shared memory back
        for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(bar_full + 8 * (i % STAGES), (i / STAGES) & 1)) break;
      }
    };
    if (BN < 256 || p.b_mn_major) producer(std::true_type{});
    else producer(std::false_type{});
  } else if (warp == NUM_CONV_WARPS + 1) {
    // ------------------------------ MMA issuer --------------------------------
    // the whole warp runs the loop; one elected lane issues the MMAs and commits
    if (MMA_WHOLE || lane == 0) {
      const uint32_t idesc = make_idesc_tf32(BM, BN, p.a_mn_major, p.b_mn_major);
      // K-major: rows of BK*4 bytes (128- or 64-byte swizzle), 8-row groups 8*BK*4 B apart, 32 B per
      // k-step inside the row.  MN-major: 32-element blocks along M/N one TMA box apart, 4-k-row
      // atoms 512 B apart, 1024 B per k-step.
      constexpr uint32_t K_SWZ = BK == 32 ? SWZ_128B : SWZ_64B;
      constexpr uint32_t K_SBO = 8 * BK * 4;
      const uint32_t a_lbo = p.a_mn_major ? (uint32_t)BOX : 16u, b_lbo = p.b_mn_major ? (uint32_t)BOX : 16u;
      const uint32_t a_sbo = p.a_mn_major ? 512u : K_SBO, b_sbo = p.b_mn_major ? 512u : K_SBO;
      const uint32_t a_sw = p.a_mn_major ? SWZ_128B_BASE32B : K_SWZ, b_sw = p.b_mn_major ? SWZ_128B_BASE32B : K_SWZ;
      const uint32_t a_kstep = p.a_mn_major ? 1024u : 32u, b_kstep = p.b_mn_major ? 1024u : 32u;
      const uint32_t tmem_main = tmem_base, tmem_cross = tmem_base + BN;
      // descriptors of stage 0, k-step 0 as (low, high) words; stages and k-steps only move the
      // start-address field of the low word
      const uint64_t d_a = make_smem_desc(smem_base, a_lbo, a_sbo, a_sw);
      const uint64_t d_b = make_smem_desc(smem_base + A_TILE, b_lbo, b_sbo, b_sw);
      const uint32_t a_hiw = (uint32_t)(d_a >> 32), b_hiw = (uint32_t)(d_b >> 32);
      const uint32_t a_low0 = (uint32_t)d_a, b_low0 = (uint32_t)d_b;
      constexpr uint32_t LO_TILE = Cfg::RAW >> 4, STAGE_STEP = Cfg::STAGE >> 4;
      const uint32_t a_step = a_kstep >> 4, b_step = b_kstep >> 4;
      const bool one_term = (p.flags & FLAG_ONE_TERM) != 0;
      uint32_t acc_cross = 0;
      uint32_t accumulate = 0;
      int s = 0;
      uint32_t ph = 0, stage_off = 0;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(bar_conv + 8 * s, ph, abort_flag, p.status, 200 + s)) break;
        tc_fence_after();
        if (!MMA_WHOLE || elect_one()) {
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint32_t al = a_low0 + stage_off + kk * a_step, bl = b_low0 + stage_off + kk * b_step;
            if (!one_term) {
              mma_tf32_ss_words(tmem_cross, al + LO_TILE, a_hiw, bl, b_hiw, idesc, kk ? 1u : acc_cross);
              mma_tf32_ss_words(tmem_cross, al, a_hiw, bl + LO_TILE, b_hiw, idesc, 1);
            }
            mma_tf32_ss_words(tmem_main, al, a_hiw, bl, b_hiw, idesc, kk ? 1u : accumulate);
          }
          mma_commit(bar_empty + 8 * s);
        }
        acc_cross = 1;
        accumulate = 1;
        if (MMA_WHOLE) __syncwarp();
        if (++s == STAGES) { s = 0; ph ^= 1; stage_off = 0; } else { stage_off += STAGE_STEP; }
      }
      if (!MMA_WHOLE || elect_one()) mma_commit(bar_acc);
      if (MMA_WHOLE) __syncwarp();
      if (*abort_flag) {
        // every MMA issued must have retired before TMEM is freed
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(bar_acc, 0)) break;
      }
    }
  } else {
    // ------------------- hi/lo split, then epilogue (warps 0-7) ---------------
    const int tid = threadIdx.x;
    bool ok = true;
    for (int i = 0; i < nkb; ++i) {
      const int s = i % STAGES, ph = (i / STAGES) & 1;
      if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 300 + s)) { ok = false; break; }
      uint8_t* hi = smem + s * Cfg::STAGE;
      uint8_t* lo = hi + Cfg::RAW;
      if (!(p.flags & FLAG_ONE_TERM)) {
#pragma unroll
        for (int c = 0; c < Cfg::RAW / 16 / (NUM_CONV_WARPS * 32); ++c) {
          const int off = (tid + c * NUM_CONV_WARPS * 32) * 16;
          const float4 v = *reinterpret_cast<const float4*>(hi + off);
          float4 l;
          l.x = lo_part(v.x); l.y = lo_part(v.y); l.z = lo_part(v.z); l.w = lo_part(v.w);
          *reinterpret_cast<float4*>(lo + off) = l;
        }
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_conv + 8 * s);   // one arrive per warp
    }
    if (ok) ok = mbar_wait(bar_acc, 0, abort_flag, p.status, 400);
    ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld below is warp-collective
    tc_fence_after();
    if (ok && k_half) {
      // the first half of this tile must be in C; by now it has been for a long time (its CTA started
      // a whole grid-half earlier), the bounded poll is there for correctness only
      if (lane == 0) {
        const int* flag = p.tile_flags + tile_id;
        int seen = 0;
        const long long t0 = clock64();
        for (;;) {
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
          if (seen != 0 || *abort_flag) break;
          if (clock64() - t0 > wait_limit(p.status)) {
            *abort_flag = 1;
            if (atomicCAS(p.status, 0, 4 /* CB200_ERR_TIMEOUT */) == 0) p.status[1] = 450;
            break;
          }
          __nanosleep(200);
        }
        ok = seen != 0;
      }
      ok = __all_sync(0xffffffffu, __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0);
    }
    if (p.ksplit_n > 1 && p.ksplit_cluster) {
      // K slices as the CTAs of one cluster: park the raw tile in this CTA's own shared memory (the pipeline
      // stages are free by now); the slices meet after the cluster barrier below
      if (ok) dump_tile_smem<BN>(p, tmem_base, reinterpret_cast<float*>(smem), warp, lane);
    } else if (p.ksplit_n > 1) {
      // K-sliced small problem: park the raw tile; the CTA that arrives last combines the slices and stores.
      // All eight warps take both barriers whatever their own wait returned (a warp that gave up has raised
      // the abort flag, which cancels the hand-over for the whole CTA).
      float* ws_tile = p.ksplit_ws + (long long)tile_id * p.ksplit_n * (BM * BN);
      if (ok) {
        dump_tile<BN>(p, tmem_base, ws_tile + (long long)k_slice * (BM * BN), warp, lane);
        __threadfence();
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NUM_CONV_WARPS * 32) : "memory");
      int* arrived = reinterpret_cast<int*>(const_cast<int*>(abort_flag)) + 1;      // a spare shared word
      if (threadIdx.x == 0) *arrived = *abort_flag ? -1 : atomicAdd(p.tile_flags + tile_id, 1);
      asm volatile("bar.sync 1, %0;" ::"n"(NUM_CONV_WARPS * 32) : "memory");
      if (*arrived == p.ksplit_n - 1) {
        __threadfence();
        epilogue_tile<BN>(p, tmem_base, m0, n0, warp, lane, reinterpret_cast<float*>(smem), p.beta, true, false, nullptr,
                          ws_tile, p.ksplit_n);
        if (threadIdx.x == 0) p.tile_flags[tile_id] = 0;      // left zero for the next launch
      }
    } else if (ok) {
      const bool last = p.k_split != 2 || k_half == 1;
      epilogue_tile<BN>(p, tmem_base, m0, n0, warp, lane, reinterpret_cast<float*>(smem), k_half ? 1.f : p.beta, last, k_half == 1);
      if (p.k_split == 2 && k_half == 0) __threadfence();     // this thread's part of C, before the flag below
    }
  }

  tc_fence_before();
  __syncthreads();
  if (p.ksplit_n > 1 && p.ksplit_cluster) {
    // Every thread of every CTA of the cluster takes both barriers, whatever happened before (a CTA whose waits
    // ran out has raised its abort flag and reported the status; its parked tile is then undefined, like the
    // output of a failed launch).  Between them each CTA finishes its share of the tile's 32 x 32 slabs: slab i
    // belongs to CTA i % n, the CTA's slabs go round its eight warps; the values are summed in slice order from
    // the n CTAs' shared memory, so the result does not depend on which CTA or warp does it.
    cluster_sync_all();
    if (warp < NUM_CONV_WARPS && !*abort_flag) {
      const int n = p.ksplit_n, rank = (int)cluster_ctarank();
      constexpr int ITEMS = 8 * (BN / 64);
      float* staging = reinterpret_cast<float*>(smem + 128 * BN * 4);       // behind the parked tile
      for (int i = rank + n * warp; i < ITEMS; i += n * NUM_CONV_WARPS)
        epilogue_tile<BN>(p, tmem_base, m0, n0, warp, lane, staging, p.beta, true, false, nullptr, nullptr, n,
                          smem_u32(smem), i);
    }
    cluster_sync_all();
  }
  if (p.k_split == 2 && threadIdx.x == 0 && !*abort_flag) {
    // first half: publish "C holds the partial tile"; second half: leave the flag zero for the next launch
    int* flag = p.tile_flags + tile_id;
    if (k_half == 0) {
      __threadfence();
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
    } else {
      *flag = 0;
    }
  }
  if (warp == NUM_CONV_WARPS + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------ host side -------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

// fp32 matrix [rows][cols] with row pitch ld (elements); box = {box_cols, box_rows}
int make_tmap(CUtensorMap* tm, const float* base, long long rows, long long cols, long long ld, int box_cols,
              int box_rows, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { cb200_set_error("cuTensorMapEncodeTiled is not available from this driver"); return CB200_ERR_CUDA; }
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    cb200_set_error("cuTensorMapEncodeTiled failed with %d (rows %lld cols %lld ld %lld box %dx%d)", (int)r, rows, cols,
                    ld, box_cols, box_rows);
    return CB200_ERR_CUDA;
  }
  return CB200_OK;
}

template <int BN, int BK>
cudaError_t tile_kernel_attributes(int dev) {
  typedef TileCfg<BN, BK> Cfg;
  static std::once_flag once[64];
  static cudaError_t result[64];
  std::call_once(once[dev & 63], [&] {
    result[dev & 63] = cudaFuncSetAttribute(gemm_tf32x3_kernel<BN, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
  });
  return result[dev & 63];
}

// How many clusters of `cluster` CTAs of this kernel the device holds at once (the CTAs of a cluster must sit in one
// GPC, so this is less than SMs / cluster); 0 when the query fails.  Cached per device and cluster size.
template <int BN, int BK>
int max_active_clusters(cb200_stream* s, int cluster) {
  typedef TileCfg<BN, BK> Cfg;
  static std::mutex mu;
  static int cache[64][9];
  static bool have[64][9];
  const int dev = s->device & 63;
  if (cluster < 1 || cluster > 8) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (!have[dev][cluster]) {
    int n = 0;
    if (tile_kernel_attributes<BN, BK>(s->device) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)cluster, 1, 1);
      cfg.blockDim = dim3(NUM_THREADS, 1, 1);
      cfg.dynamicSmemBytes = Cfg::SMEM;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = (unsigned)cluster;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tf32x3_kernel<BN, BK>, &cfg) != cudaSuccess) { n = 0; (void)cudaGetLastError(); }
    }
    cache[dev][cluster] = n;
    have[dev][cluster] = true;
  }
  return cache[dev][cluster];
}

template <int BN, int BK>
int launch_tile(cb200_stream* s, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p) {
  typedef TileCfg<BN, BK> Cfg;
  cudaError_t attr_err = tile_kernel_attributes<BN, BK>(s->device);
  if (attr_err != cudaSuccess) return cb200_cuda_fail(attr_err, "cudaFuncSetAttribute", __FILE__, __LINE__);
  long long tiles = (long long)((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.k_split * p.ksplit_n;
  if (p.ksplit_n > 1 && p.ksplit_cluster) {
    // the slices of a tile (consecutive block indices) as one thread-block cluster
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles, 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = s->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.ksplit_n;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tf32x3_kernel<BN, BK>, tmA, tmB, p);
    if (e != cudaSuccess) return cb200_cuda_fail(e, "cudaLaunchKernelEx(gemm_tf32x3_kernel)", __FILE__, __LINE__);
  } else {
    gemm_tf32x3_kernel<BN, BK><<<(unsigned)tiles, NUM_THREADS, Cfg::SMEM, s->stream>>>(tmA, tmB, p);
  }
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // namespace

// Shared with conv.cu.  A: op(A) is M x K; B: op(B) is K x N.
int cb200_gemm_tf32x3_launch_peers(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                                   const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                                   float beta, const float* bias, int act, int store_mode, int hw, int flags,
                                   int n_peers, float* const* peers);

int cb200_gemm_tf32x3_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                             const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                             float beta, const float* bias, int act, int store_mode, int hw, int flags) {
  return cb200_gemm_tf32x3_launch_peers(s, C, ldc, trans_a, trans_b, alpha, A, M, K, lda, B, N, ldb, beta, bias, act,
                                        store_mode, hw, flags, 0, nullptr);
}

// Most K slices one launch can give a problem (every tile's slices run side by side in one wave); 1 = none.
int cb200_gemm_tf32x3_max_slices(const cb200_stream* s, int M, int N) {
  const int bn_max = N > 128 ? 256 : (N > 64 ? 128 : 64);
  const long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn_max - 1) / bn_max);
  long long sl = tiles > 0 ? s->sm_count / tiles : 1;
  return (int)(sl < 1 ? 1 : (sl > 32 ? 32 : sl));
}

// The same launch with up to MAX_PEERS extra destinations: every output tile is also stored to
// peers[d] + (the same row-major position), d < n_peers.
int cb200_gemm_tf32x3_launch_peers(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                                   const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                                   float beta, const float* bias, int act, int store_mode, int hw, int flags,
                                   int n_peers, float* const* peers) {
  DeviceGuard guard(s->device);
  GemmParams p;
  p.n_peers = n_peers;
  for (int d = 0; d < MAX_PEERS; ++d) p.peers[d] = d < n_peers ? peers[d] : nullptr;
  p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.beta = beta; p.bias = bias; p.act = act;
  p.a_mn_major = trans_a ? 1 : 0;   // op(A)[m][k] = A[k][m]: M is the contiguous axis
  p.b_mn_major = trans_b ? 0 : 1;   // op(B)[k][n] = B[k][n]: N is the contiguous axis
  p.store_mode = store_mode; p.hw = hw > 0 ? hw : 1; p.flags = flags; p.status = s->status_dev;
  // ---- tile width and K slices --------------------------------------------------------------------
  // Problems whose tiles (at the widest useful width) do not fill the SMs are latency-bound, and two knobs
  // trade against each other: narrower tiles and more K slices both put more CTAs to work, but a narrow tile
  // re-reads more operand bytes per flop from shared memory (a k-block of 16 costs 0.39 / 0.455 / 0.56 us at
  // 64 / 128 / 256 columns: 1.4x the time for 4x the work) and every slice adds to the hand-over through L2
  // ((BN / 64) x (1.3 + 0.45 x slices) us).  The pair is chosen by that model, fitted to a sweep of twelve
  // shapes x three widths x seven slice counts (it predicts each of them within ~10 %):
  //     t = waves x (5 us + ceil(k-blocks / slices) x c[BN]) + hand-over,    slices > 1 only within one wave.
  // Against the earlier rule (narrow while one wave holds the tiles, then slice), us per call:
  //     1024^3 30.9 -> 25.2, 768 x 768 x 3072 46.1 -> 33.2, 1536^3 51.8 -> 43.1, 1024 x 512 x 2048 33.5 -> 25.9,
  //     256 x 1024 x 4096 34.1 -> 27.2, 640 x 1280 x 1280 36.6 -> 28.4; unchanged where that rule was already best.
  // Every column tile re-reads its rows of A from DRAM once A no longer stays in L2 (>= 24 MB, and A the larger
  // operand): the widest tile is kept there whatever the model says (measured: 4096 x 512 x 4096 232 -> 108 us,
  // 2048 x 1024 x 4096 220 -> 107, 8192 x 125 x 4096 159 -> 132 when that was introduced).
  const int bn_max = N > 128 ? 256 : (N > 64 ? 128 : 64);
  const long long tiles_m = (M + BM - 1) / BM;
  const int nkb_model = (K + 15) / 16;
  const bool big_a = (long long)M * K * 4 >= (24ll << 20) && (long long)M >= (long long)N;
  // FLAG_SPLIT_K (the fused layer entry points, K >= 4096): the reduction must be cut at least in two.  Where the
  // tiles leave room, two or more K slices do that (and fill the SMs); otherwise the two-halves form below.
  const bool want_halves = (flags & FLAG_SPLIT_K) && K >= 4096 && store_mode == STORE_ROW_MAJOR;
  const bool may_slice = !(flags & FLAG_ONE_TERM);
  int min_slices = (flags >> FLAG_MIN_SLICES_SHIFT) & 0xff;            // a long reduction the caller wants cut up
  if (want_halves && may_slice && min_slices < 2 && s->opt_gemm_k_slices != 1) min_slices = 2;
  int BN = bn_max, model_slices = min_slices > 1 ? min_slices : 1;
  bool sliced_instead_of_halves = false;
  for (int attempt = 0; attempt < 2; ++attempt) {
    double best = 1e30;
    if (attempt == 1) {                  // no room for the slices: one CTA per tile (and K halves where wanted)
      min_slices = (flags >> FLAG_MIN_SLICES_SHIFT) & 0xff;
      model_slices = min_slices > 1 ? min_slices : 1;
    }
    const bool slices_allowed = may_slice && !(attempt == 1 && want_halves);
    for (int bn = 256; bn >= 64; bn >>= 1) {
      if (bn > bn_max) continue;
      if (s->opt_gemm_tile_n > 0 ? bn != s->opt_gemm_tile_n : (big_a && bn != bn_max)) continue;
      const double c_kb = bn == 256 ? 0.56 : (bn == 128 ? 0.455 : 0.39);
      const long long tiles = tiles_m * ((N + bn - 1) / bn);
      for (int sl = min_slices > 1 ? min_slices : 1; sl <= 32; ++sl) {
        if (sl > 1 && (!slices_allowed || tiles * sl > s->sm_count || nkb_model / sl < 4)) break;
        const long long waves = (tiles * sl + s->sm_count - 1) / s->sm_count;
        // (up to 8 slices meet in distributed shared memory, measured at about three quarters of the L2 cost)
        const double t = (double)waves * (5.0 + (double)((nkb_model + sl - 1) / sl) * c_kb) +
                         (sl > 1 ? (sl <= 8 ? 0.75 : 1.0) * (bn / 64) * (1.3 + 0.45 * sl) : 0.0);
        if (t < best - 1e-9) { best = t; BN = bn; model_slices = sl; }      // ties: the wider tile, fewer slices
      }
    }
    if (s->opt_gemm_tile_n > 0 && s->opt_gemm_tile_n > bn_max) BN = s->opt_gemm_tile_n;   // forced wider than N needs
    if (best < 1e29) { sliced_instead_of_halves = want_halves && attempt == 0; break; }
    if (!(want_halves && attempt == 0)) break;      // nothing to retry (a forced minimum that does not fit runs as asked)
  }
  const int tiles_n = (N + BN - 1) / BN;
  const long long panel_bytes = (long long)BN * K * 4;          // one column tile's share of B
  // FLAG_SPLIT_K (the fused layer entry points): reductions of 4096 and more are cut in two K halves per
  // tile (see GemmParams::k_split).  tcgen05 accumulates with truncation, a result shrinks by about
  // 7e-9 * K (relative: 2.9e-5 at K = 4096, inside the 1e-4 bound of one gemm!), the same for every
  // output, so it compounds through a stack of layers (five 4096-wide layers: 1.4e-4 on the softmax
  // output); two 2048-long halves joined by a round-to-nearest add halve that, at 8-12 % of the speed.
  p.k_split = (want_halves && !sliced_instead_of_halves) ? 2 : 1;
  p.C_lo = nullptr;
  p.drain_every = 0;
  p.tile_flags = nullptr;
  p.split_block = 2 * s->sm_count;
  if (p.k_split == 2) {
    int rcf = cb200_tile_flags(s, (size_t)tiles_m * tiles_n, &p.tile_flags);
    if (rcf) return rcf;
  }
  // K slices: model_slices CTAs per tile, each over a slice of K, combined by the last one to finish.  The stream
  // option forces a count (old caps: at least 8 k-blocks per slice, slices x BN <= 1024, at most 16).
  p.ksplit_n = 1;
  p.ksplit_cluster = 0;
  p.ksplit_ws = nullptr;
  {
    const long long tiles = tiles_m * tiles_n;
    const int nkb_all = (K + 15) / 16;
    long long sl = model_slices;
    if (s->opt_gemm_k_slices > 0 && min_slices <= 1) {
      sl = s->opt_gemm_k_slices;
      if (sl > nkb_all / 8) sl = nkb_all / 8;
      if (sl > 1024 / BN) sl = 1024 / BN;
      if (sl > 16) sl = 16;
    }
    if (p.k_split == 1 && sl >= 2 && !(flags & FLAG_ONE_TERM)) {
      p.ksplit_n = (int)sl;
      // up to 8 slices (the portable cluster size): the slices of a tile are launched as one cluster and hand
      // their partial tiles over through distributed shared memory; more slices go through L2
      int fit = 0;
      if (sl <= 8 && s->opt_gemm_slice_handover != 1) {
        DeviceGuard guard_q(s->device);
        fit = BN == 256 ? max_active_clusters<256, 16>(s, (int)sl)
                        : (BN == 128 ? max_active_clusters<128, 16>(s, (int)sl) : max_active_clusters<64, 16>(s, (int)sl));
      }
      if (fit >= tiles) {          // every tile's cluster resident at once; otherwise a second wave would cost more than L2
        p.ksplit_cluster = 1;
      } else {
        void* ws = nullptr;
        int rcs = cb200_partials(s, (size_t)tiles * sl * BM * BN * sizeof(float), &ws);
        if (rcs) return rcs;
        if ((rcs = cb200_tile_flags(s, (size_t)tiles, &p.tile_flags))) return rcs;
        p.ksplit_ws = (float*)ws;
      }
    }
  }
  p.group_n = tiles_n;
  if (tiles_n * panel_bytes > (40ll << 20)) {
    long long g = (32ll << 20) / panel_bytes;
    p.group_n = (int)(g < 1 ? 1 : (g > tiles_n ? tiles_n : g));
  }
  constexpr int BK = 16;
  const CUtensorMapSwizzle kswz = CU_TENSOR_MAP_SWIZZLE_64B;
  CUtensorMap tmA, tmB;
  int rc;
  if (!p.a_mn_major) rc = make_tmap(&tmA, A, M, K, lda, BK, BM, kswz);
  else rc = make_tmap(&tmA, A, K, M, lda, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (rc) return rc;
  if (!p.b_mn_major) rc = make_tmap(&tmB, B, N, K, ldb, BK, BN, kswz);
  else rc = make_tmap(&tmB, B, K, N, ldb, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (rc) return rc;
  if (BN == 256) return launch_tile<256, 16>(s, tmA, tmB, p);
  if (BN == 128) return launch_tile<128, 16>(s, tmA, tmB, p);
  return launch_tile<64, 16>(s, tmA, tmB, p);
}

bool cb200_gemm_tf32x3_eligible(const float* A, long long lda, const float* B, long long ldb, int M, int N, int K) {
  if (M < 1 || N < 1 || K < 1) return false;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return false;
  if ((lda % 4) || (ldb % 4)) return false;
  return true;
}
