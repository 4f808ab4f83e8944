// pooling-forward! (max / avg / avg-exc-pad): src/cortex/tensor/math.clj:205-222; cudnnPoolingForward in the
// reference CUDA backend (src/cortex/compute/cuda/tensor_math.clj:1096-1160); arithmetic after the CPU backend
// (src/cortex/compute/cpu/tensor_math.clj:1153-1261 over the loop nest of src/cortex/nn/impl.clj:8-107):
//   window positions outside [-pad, extent + pad) are skipped; positions in the padding read 0;
//   max:         running maximum, initialised by the first window position (so padding counts as 0);
//   avg:         acc = (T)(acc + x / (kW*kH)) position by position (every partial sum rounded to T);
//   avg-exc-pad: the same with the number of window positions inside the image as divisor.
// NCHW dense input / output; one thread per output element, adjacent threads = adjacent output columns.
// output = result + output_alpha * output (the reference CPU backend ignores output-alpha; 0 is what its
// callers pass).
#include "common.cuh"

namespace {

struct PoolGeom {
  int channels, in_h, in_w, out_h, out_w, kw, kh, pad_x, pad_y, stride_x, stride_y, op;
};

// Window positions are visited in (k-y, k-x) order as in the reference, but the bounds tests are hoisted:
// only positions inside the image are loaded.  Skipping the padding positions changes nothing for the
// averages (they add 0 / divisor to the running sum: the identity) and for the maximum they only add the
// candidate 0, folded in once.
template <typename T, int OP>
__global__ void __launch_bounds__(256)
pooling_forward_kernel(T* out, const T* in, PoolGeom g, long long n_out, double out_alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_out; i += (long long)gridDim.x * blockDim.x) {
    // 32-bit index arithmetic (the entry point limits the output to 2^31 - 1 elements)
    const unsigned iu = (unsigned)i;
    const unsigned tq = iu / (unsigned)g.out_w;
    const int ox = (int)(iu - tq * (unsigned)g.out_w);
    const unsigned plane_u = tq / (unsigned)g.out_h;
    const int oy = (int)(tq - plane_u * (unsigned)g.out_h);
    const long long plane = plane_u;
    const T* src = in + plane * (long long)g.in_h * g.in_w;
    const int rel_x = ox * g.stride_x - g.pad_x, rel_y = oy * g.stride_y - g.pad_y;
    // rows / columns of the window inside the image, and inside the padded extent
    const int y0 = max(rel_y, 0), y1 = min(rel_y + g.kh, g.in_h);
    const int x0 = max(rel_x, 0), x1 = min(rel_x + g.kw, g.in_w);
    const int py1 = min(rel_y + g.kh, g.in_h + g.pad_y), px1 = min(rel_x + g.kw, g.in_w + g.pad_x);
    const int inside = max(0, y1 - y0) * max(0, x1 - x0);
    const int visited = max(0, py1 - rel_y) * max(0, px1 - rel_x);     // rel >= -pad always
    T acc = (T)0;
    if (OP == CB200_POOL_MAX) {
      bool first = true;
      for (int iy = y0; iy < y1; ++iy)
        for (int ix = x0; ix < x1; ++ix) {
          const T v = src[(long long)iy * g.in_w + ix];
          if (first || v > acc) acc = v;
          first = false;
        }
      if (visited > inside && (first || (T)0 > acc)) acc = (T)0;       // padding positions read 0
    } else {
      const double divisor = OP == CB200_POOL_AVG ? (double)(g.kw * g.kh) : (double)inside;
      for (int iy = y0; iy < y1; ++iy)
        for (int ix = x0; ix < x1; ++ix)
          acc = (T)((double)acc + (double)src[(long long)iy * g.in_w + ix] / divisor);
      if (OP == CB200_POOL_AVG_EXC_PAD && inside == 0 && visited > 0) acc = (T)((double)acc + 0.0 / divisor);   // 0/0 as the reference
    }
    out[i] = out_alpha == 0.0 ? acc : (T)((double)acc + out_alpha * (double)out[i]);
  }
}

// 2x2 and 3x3 windows (the common ones): the window is loaded with independent, predicated loads first
// (all in flight together) and folded afterwards in the same (k-y, k-x) order.
template <typename T, int OP, int KH, int KW>
__global__ void __launch_bounds__(256)
pooling_forward_small_kernel(T* out, const T* in, PoolGeom g, long long n_out, double out_alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_out; i += (long long)gridDim.x * blockDim.x) {
    // 32-bit index arithmetic (the entry point limits the output to 2^31 - 1 elements)
    const unsigned iu = (unsigned)i;
    const unsigned tq = iu / (unsigned)g.out_w;
    const int ox = (int)(iu - tq * (unsigned)g.out_w);
    const unsigned plane_u = tq / (unsigned)g.out_h;
    const int oy = (int)(tq - plane_u * (unsigned)g.out_h);
    const long long plane = plane_u;
    const T* src = in + plane * (long long)g.in_h * g.in_w;
    const int rel_x = ox * g.stride_x - g.pad_x, rel_y = oy * g.stride_y - g.pad_y;
    T v[KH * KW];
    bool ok[KH * KW];
    // row / column validity once per k-y / k-x, 32-bit offsets inside the plane
    bool row_ok[KH], col_ok[KW];
    int n_rows = 0, n_cols = 0;
#pragma unroll
    for (int ky = 0; ky < KH; ++ky) { row_ok[ky] = (unsigned)(rel_y + ky) < (unsigned)g.in_h; n_rows += row_ok[ky] ? 1 : 0; }
#pragma unroll
    for (int kx = 0; kx < KW; ++kx) { col_ok[kx] = (unsigned)(rel_x + kx) < (unsigned)g.in_w; n_cols += col_ok[kx] ? 1 : 0; }
    const int inside = n_rows * n_cols;
    const int base = rel_y * g.in_w + rel_x;
#pragma unroll
    for (int ky = 0; ky < KH; ++ky)
#pragma unroll
      for (int kx = 0; kx < KW; ++kx) {
        const bool in_img = row_ok[ky] && col_ok[kx];
        ok[ky * KW + kx] = in_img;
        v[ky * KW + kx] = in_img ? src[base + ky * g.in_w + kx] : (T)0;
      }
    const int py1 = min(rel_y + KH, g.in_h + g.pad_y), px1 = min(rel_x + KW, g.in_w + g.pad_x);
    const int visited = max(0, py1 - rel_y) * max(0, px1 - rel_x);
    T acc = (T)0;
    if (OP == CB200_POOL_MAX) {
      bool first = true;
#pragma unroll
      for (int k = 0; k < KH * KW; ++k)
        if (ok[k]) { if (first || v[k] > acc) acc = v[k]; first = false; }
      if (visited > inside && (first || (T)0 > acc)) acc = (T)0;
    } else {
      const double divisor = OP == CB200_POOL_AVG ? (double)(KW * KH) : (double)inside;
#pragma unroll
      for (int k = 0; k < KH * KW; ++k)
        if (ok[k]) acc = (T)((double)acc + (double)v[k] / divisor);
      if (OP == CB200_POOL_AVG_EXC_PAD && inside == 0 && visited > 0) acc = (T)((double)acc + 0.0 / divisor);
    }
    out[i] = out_alpha == 0.0 ? acc : (T)((double)acc + out_alpha * (double)out[i]);
  }
}

// The same for strides 1 and 2 with FOUR adjacent outputs of a row per thread: index arithmetic and row
// tests are paid once per four outputs, and neighbouring windows share their loaded columns
// (3x3 stride 2: 27 loads for four outputs instead of 36).
template <typename T, int OP, int KH, int KW, int SX>
__global__ void __launch_bounds__(256)
pooling_forward_quad_kernel(T* out, const T* in, PoolGeom g, long long n_groups, int groups_per_row, double out_alpha) {
  constexpr int NX = 4, W_IN = (NX - 1) * SX + KW;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups; i += (long long)gridDim.x * blockDim.x) {
    const unsigned iu = (unsigned)i;
    const unsigned tq = iu / (unsigned)groups_per_row;
    const int ox0 = (int)(iu - tq * (unsigned)groups_per_row) * NX;
    const unsigned plane_u = tq / (unsigned)g.out_h;
    const int oy = (int)(tq - plane_u * (unsigned)g.out_h);
    const T* src = in + (long long)plane_u * g.in_h * g.in_w;
    const int rel_x = ox0 * SX - g.pad_x, rel_y = oy * g.stride_y - g.pad_y;
    bool row_ok[KH], col_ok[W_IN];
    int n_rows = 0;
#pragma unroll
    for (int ky = 0; ky < KH; ++ky) { row_ok[ky] = (unsigned)(rel_y + ky) < (unsigned)g.in_h; n_rows += row_ok[ky] ? 1 : 0; }
#pragma unroll
    for (int c = 0; c < W_IN; ++c) col_ok[c] = (unsigned)(rel_x + c) < (unsigned)g.in_w;
    const int base = rel_y * g.in_w + rel_x;
    T v[KH][W_IN];
#pragma unroll
    for (int ky = 0; ky < KH; ++ky)
#pragma unroll
      for (int c = 0; c < W_IN; ++c) v[ky][c] = (row_ok[ky] && col_ok[c]) ? src[base + ky * g.in_w + c] : (T)0;
    const int py1 = min(rel_y + KH, g.in_h + g.pad_y);
    const int rows_visited = max(0, py1 - rel_y);
    T* dst = out + ((long long)plane_u * g.out_h + oy) * g.out_w + ox0;
    T res[NX];
#pragma unroll
    for (int o = 0; o < NX; ++o) {                       // fully unrolled: v and col_ok stay in registers
      int n_cols = 0;
#pragma unroll
      for (int kx = 0; kx < KW; ++kx) n_cols += col_ok[o * SX + kx] ? 1 : 0;
      const int inside = n_rows * n_cols;
      const int rx = rel_x + o * SX;
      const int visited = rows_visited * max(0, min(rx + KW, g.in_w + g.pad_x) - rx);
      T acc = (T)0;
      if (OP == CB200_POOL_MAX) {
        bool first = true;
#pragma unroll
        for (int ky = 0; ky < KH; ++ky)
#pragma unroll
          for (int kx = 0; kx < KW; ++kx)
            if (row_ok[ky] && col_ok[o * SX + kx]) { const T x = v[ky][o * SX + kx]; if (first || x > acc) acc = x; first = false; }
        if (visited > inside && (first || (T)0 > acc)) acc = (T)0;
      } else {
        const double divisor = OP == CB200_POOL_AVG ? (double)(KW * KH) : (double)inside;
#pragma unroll
        for (int ky = 0; ky < KH; ++ky)
#pragma unroll
          for (int kx = 0; kx < KW; ++kx)
            if (row_ok[ky] && col_ok[o * SX + kx]) acc = (T)((double)acc + (double)v[ky][o * SX + kx] / divisor);
        if (OP == CB200_POOL_AVG_EXC_PAD && inside == 0 && visited > 0) acc = (T)((double)acc + 0.0 / divisor);
      }
      res[o] = acc;
    }
#pragma unroll
    for (int o = 0; o < NX; ++o)
      if (ox0 + o < g.out_w) dst[o] = out_alpha == 0.0 ? res[o] : (T)((double)res[o] + out_alpha * (double)dst[o]);
  }
}

// float tensors whose rows are 16-byte aligned: the same four outputs per thread, but the input columns they
// share arrive as aligned 16-byte vectors (adjacent threads read adjacent vectors: fully coalesced), only the
// halo column(s) left / right of the aligned segment as scalars (L1 hits: the neighbouring thread fetches
// them as part of its vector).  3x3 stride 2 pad 1: 9 load instructions per thread instead of 27, and the
// kernel moves from issue-bound to HBM-bound.  PX = pad_x (0 or 1).  Same fold order as above.
template <int OP, int KH, int KW, int SX, int PX>
__global__ void __launch_bounds__(256)
pooling_forward_vec_kernel(float* out, const float* in, PoolGeom g, int planes, int groups_per_row, double out_alpha) {
  constexpr int NX = 4, W_IN = (NX - 1) * SX + KW, SEG = NX * SX;
  const bool out_vec = (g.out_w % 4) == 0 && ((((uintptr_t)out) & 15) == 0);
  const unsigned per_plane = (unsigned)(g.out_h * groups_per_row);
  const unsigned blocks_per_plane = (per_plane + 255) / 256;
  // block -> (plane, chunk of the plane's (row, group) pairs): one division per thread
  for (unsigned b = blockIdx.x; b < (unsigned)planes * blocks_per_plane; b += gridDim.x) {
    const unsigned plane_u = b / blocks_per_plane;
    const unsigned within = (b - plane_u * blocks_per_plane) * 256 + threadIdx.x;
    if (within >= per_plane) continue;
    const int oy = (int)(within / (unsigned)groups_per_row);
    const int ox0 = (int)(within - (unsigned)oy * (unsigned)groups_per_row) * NX;
    const float* src = in + (long long)plane_u * g.in_h * g.in_w;
    const int rel_x = ox0 * SX - PX, rel_y = oy * g.stride_y - g.pad_y;
    const int seg_x = ox0 * SX;                         // first column of the aligned segment (multiple of 4)
    float* dst = out + ((long long)plane_u * g.out_h + oy) * g.out_w + ox0;
    float res[NX];
    if (rel_y + KH <= g.in_h + g.pad_y && rel_x + W_IN <= g.in_w + g.pad_x && seg_x + SEG <= g.in_w) {
      // Every window position of this thread is inside the image or in the padding band (which reads 0 and takes
      // part like any other value): no per-position tests.  Only the halo columns left / right of the aligned
      // segment and whole rows can be padding.  This is the path of every thread unless a ceil-mode window
      // reaches past the band, so warps do not diverge into the general code below.
      float v[KH][W_IN];
      int n_rows = 0;
#pragma unroll
      for (int ky = 0; ky < KH; ++ky) {
        const int iy = rel_y + ky;
        const bool row_in = (unsigned)iy < (unsigned)g.in_h;
        n_rows += row_in ? 1 : 0;
        const float* row = src + iy * g.in_w;
        float seg[SEG];
#pragma unroll
        for (int q = 0; q < SEG / 4; ++q) {
          float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
          if (row_in) t = *reinterpret_cast<const float4*>(row + seg_x + 4 * q);
          seg[4 * q] = t.x; seg[4 * q + 1] = t.y; seg[4 * q + 2] = t.z; seg[4 * q + 3] = t.w;
        }
#pragma unroll
        for (int c = 0; c < W_IN; ++c) {
          if (c >= PX && c < PX + SEG) v[ky][c] = seg[c - PX];
          else v[ky][c] = (row_in && (unsigned)(rel_x + c) < (unsigned)g.in_w) ? row[rel_x + c] : 0.f;
        }
      }
#pragma unroll
      for (int o = 0; o < NX; ++o) {
        if (OP == CB200_POOL_MAX) {
          float acc = v[0][o * SX];
#pragma unroll
          for (int ky = 0; ky < KH; ++ky)
#pragma unroll
            for (int kx = 0; kx < KW; ++kx)
              if (ky + kx > 0) { const float x = v[ky][o * SX + kx]; acc = x > acc ? x : acc; }
          res[o] = acc;
        } else {
          int n_cols = 0;
#pragma unroll
          for (int kx = 0; kx < KW; ++kx) n_cols += (unsigned)(rel_x + o * SX + kx) < (unsigned)g.in_w ? 1 : 0;
          const double divisor = OP == CB200_POOL_AVG ? (double)(KW * KH) : (double)(n_rows * n_cols);
          float acc = 0.f;
          // padding positions add 0 / divisor: the identity, as in the reference's position-by-position sum
#pragma unroll
          for (int ky = 0; ky < KH; ++ky)
#pragma unroll
            for (int kx = 0; kx < KW; ++kx) acc = (float)((double)acc + (double)v[ky][o * SX + kx] / divisor);
          res[o] = acc;
        }
      }
    } else {
      bool row_ok[KH], col_ok[W_IN];
      int n_rows = 0;
#pragma unroll
      for (int ky = 0; ky < KH; ++ky) { row_ok[ky] = (unsigned)(rel_y + ky) < (unsigned)g.in_h; n_rows += row_ok[ky] ? 1 : 0; }
#pragma unroll
      for (int c = 0; c < W_IN; ++c) col_ok[c] = (unsigned)(rel_x + c) < (unsigned)g.in_w;
      float v[KH][W_IN];
#pragma unroll
      for (int ky = 0; ky < KH; ++ky) {
        const float* row = src + (rel_y + ky) * g.in_w;
        float seg[SEG];
#pragma unroll
        for (int q = 0; q < SEG / 4; ++q) {
          if (row_ok[ky] && seg_x + 4 * q + 3 < g.in_w) {
            const float4 t = *reinterpret_cast<const float4*>(row + seg_x + 4 * q);
            seg[4 * q] = t.x; seg[4 * q + 1] = t.y; seg[4 * q + 2] = t.z; seg[4 * q + 3] = t.w;
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              seg[4 * q + e] = (row_ok[ky] && seg_x + 4 * q + e < g.in_w) ? row[seg_x + 4 * q + e] : 0.f;
          }
        }
#pragma unroll
        for (int c = 0; c < W_IN; ++c) {
          if (c >= PX && c < PX + SEG) v[ky][c] = seg[c - PX];
          else v[ky][c] = (row_ok[ky] && col_ok[c]) ? row[rel_x + c] : 0.f;
        }
      }
      const int py1 = min(rel_y + KH, g.in_h + g.pad_y);
      const int rows_visited = max(0, py1 - rel_y);
#pragma unroll
      for (int o = 0; o < NX; ++o) {
        int n_cols = 0;
#pragma unroll
        for (int kx = 0; kx < KW; ++kx) n_cols += col_ok[o * SX + kx] ? 1 : 0;
        const int inside = n_rows * n_cols;
        const int rx = rel_x + o * SX;
        const int visited = rows_visited * max(0, min(rx + KW, g.in_w + g.pad_x) - rx);
        float acc = 0.f;
        if (OP == CB200_POOL_MAX) {
          bool first = true;
#pragma unroll
          for (int ky = 0; ky < KH; ++ky)
#pragma unroll
            for (int kx = 0; kx < KW; ++kx)
              if (row_ok[ky] && col_ok[o * SX + kx]) { const float x = v[ky][o * SX + kx]; if (first || x > acc) acc = x; first = false; }
          if (visited > inside && (first || 0.f > acc)) acc = 0.f;
        } else {
          const double divisor = OP == CB200_POOL_AVG ? (double)(KW * KH) : (double)inside;
#pragma unroll
          for (int ky = 0; ky < KH; ++ky)
#pragma unroll
            for (int kx = 0; kx < KW; ++kx)
              if (row_ok[ky] && col_ok[o * SX + kx]) acc = (float)((double)acc + (double)v[ky][o * SX + kx] / divisor);
          if (OP == CB200_POOL_AVG_EXC_PAD && inside == 0 && visited > 0) acc = (float)((double)acc + 0.0 / divisor);
        }
        res[o] = acc;
      }
    }
    if (out_vec && out_alpha == 0.0) {
      *reinterpret_cast<float4*>(dst) = make_float4(res[0], res[1], res[2], res[3]);
    } else {
#pragma unroll
      for (int o = 0; o < NX; ++o)
        if (ox0 + o < g.out_w) dst[o] = out_alpha == 0.0 ? res[o] : (float)((double)res[o] + out_alpha * (double)dst[o]);
    }
  }
}

template <typename T, int OP, int KH, int KW>
bool pooling_launch_vec(cb200_stream*, T*, const T*, const PoolGeom&, long long, double) { return false; }

template <int OP, int KH, int KW>
bool pooling_launch_vec_f(cb200_stream* s, float* out, const float* in, const PoolGeom& g, long long n_out, double out_alpha) {
  if ((g.stride_x != 1 && g.stride_x != 2) || g.pad_x > 1 || (g.in_w % 4) != 0 || ((((uintptr_t)in) & 15) != 0)) return false;
  const int groups_per_row = (g.out_w + 3) / 4;
  const long long planes = n_out / ((long long)g.out_w * g.out_h);
  const long long per_plane = (long long)g.out_h * groups_per_row;
  if (planes > 2147483647LL / ((per_plane + 255) / 256)) return false;
  // one block per 256 (row, group) pairs of a plane, no cap: with a capped grid every block walks 3-4 planes and
  // the ones with 4 set the kernel's duration
  long long blocks = planes * ((per_plane + 255) / 256);
  if (blocks > 1048576) blocks = 1048576;
#define CB_POOL_VEC(SX, PX) pooling_forward_vec_kernel<OP, KH, KW, SX, PX><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g, (int)planes, groups_per_row, out_alpha)
  if (g.stride_x == 2 && g.pad_x == 0) CB_POOL_VEC(2, 0);
  else if (g.stride_x == 2) CB_POOL_VEC(2, 1);
  else if (g.pad_x == 0) CB_POOL_VEC(1, 0);
  else CB_POOL_VEC(1, 1);
#undef CB_POOL_VEC
  return true;
}
template <> bool pooling_launch_vec<float, CB200_POOL_MAX, 3, 3>(cb200_stream* s, float* o, const float* i, const PoolGeom& g, long long n, double a) { return pooling_launch_vec_f<CB200_POOL_MAX, 3, 3>(s, o, i, g, n, a); }
template <> bool pooling_launch_vec<float, CB200_POOL_AVG, 3, 3>(cb200_stream* s, float* o, const float* i, const PoolGeom& g, long long n, double a) { return pooling_launch_vec_f<CB200_POOL_AVG, 3, 3>(s, o, i, g, n, a); }
template <> bool pooling_launch_vec<float, CB200_POOL_AVG_EXC_PAD, 3, 3>(cb200_stream* s, float* o, const float* i, const PoolGeom& g, long long n, double a) { return pooling_launch_vec_f<CB200_POOL_AVG_EXC_PAD, 3, 3>(s, o, i, g, n, a); }
template <> bool pooling_launch_vec<float, CB200_POOL_MAX, 2, 2>(cb200_stream* s, float* o, const float* i, const PoolGeom& g, long long n, double a) { return pooling_launch_vec_f<CB200_POOL_MAX, 2, 2>(s, o, i, g, n, a); }
template <> bool pooling_launch_vec<float, CB200_POOL_AVG, 2, 2>(cb200_stream* s, float* o, const float* i, const PoolGeom& g, long long n, double a) { return pooling_launch_vec_f<CB200_POOL_AVG, 2, 2>(s, o, i, g, n, a); }
template <> bool pooling_launch_vec<float, CB200_POOL_AVG_EXC_PAD, 2, 2>(cb200_stream* s, float* o, const float* i, const PoolGeom& g, long long n, double a) { return pooling_launch_vec_f<CB200_POOL_AVG_EXC_PAD, 2, 2>(s, o, i, g, n, a); }

template <typename T, int OP, int KH, int KW>
bool pooling_launch_quad(cb200_stream* s, T* out, const T* in, const PoolGeom& g, long long n_out, double out_alpha) {
  if (pooling_launch_vec<T, OP, KH, KW>(s, out, in, g, n_out, out_alpha)) return true;
  if (g.stride_x != 1 && g.stride_x != 2) return false;
  const int groups_per_row = (g.out_w + 3) / 4;
  const long long n_groups = (n_out / g.out_w) * groups_per_row;
  long long blocks = (n_groups + 255) / 256;
  const long long cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (g.stride_x == 2)
    pooling_forward_quad_kernel<T, OP, KH, KW, 2><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g, n_groups, groups_per_row, out_alpha);
  else
    pooling_forward_quad_kernel<T, OP, KH, KW, 1><<<(unsigned)blocks, 256, 0, s->stream>>>(out, in, g, n_groups, groups_per_row, out_alpha);
  return true;
}

template <typename T, int OP>
void pooling_launch_op(cb200_stream* s, T* out, const T* in, const PoolGeom& g, long long n_out, double out_alpha,
                       unsigned blocks) {
  if (g.kh == 3 && g.kw == 3) {
    if (!pooling_launch_quad<T, OP, 3, 3>(s, out, in, g, n_out, out_alpha))
      pooling_forward_small_kernel<T, OP, 3, 3><<<blocks, 256, 0, s->stream>>>(out, in, g, n_out, out_alpha);
  } else if (g.kh == 2 && g.kw == 2) {
    if (!pooling_launch_quad<T, OP, 2, 2>(s, out, in, g, n_out, out_alpha))
      pooling_forward_small_kernel<T, OP, 2, 2><<<blocks, 256, 0, s->stream>>>(out, in, g, n_out, out_alpha);
  }
  else
    pooling_forward_kernel<T, OP><<<blocks, 256, 0, s->stream>>>(out, in, g, n_out, out_alpha);
}

template <typename T>
void pooling_launch(cb200_stream* s, T* out, const T* in, const PoolGeom& g, long long n_out, double out_alpha, unsigned blocks) {
  if (g.op == CB200_POOL_MAX) pooling_launch_op<T, CB200_POOL_MAX>(s, out, in, g, n_out, out_alpha, blocks);
  else if (g.op == CB200_POOL_AVG) pooling_launch_op<T, CB200_POOL_AVG>(s, out, in, g, n_out, out_alpha, blocks);
  else pooling_launch_op<T, CB200_POOL_AVG_EXC_PAD>(s, out, in, g, n_out, out_alpha, blocks);
}

}  // namespace

extern "C" int cb200_pooling_forward(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, double out_alpha,
                                     const void* in, const cb200_dims* in_dims, const cb200_pool_desc* desc) {
  CB_REQUIRE(s && out && out_dims && in && in_dims && desc, "pooling_forward: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE, "pooling-forward! is only defined for float and double tensors");
  CB_REQUIRE(desc->pool_op >= CB200_POOL_MAX && desc->pool_op <= CB200_POOL_AVG_EXC_PAD, "pooling_forward: unknown pool op %d",
             desc->pool_op);
  CB_REQUIRE(desc->kernel_width >= 1 && desc->kernel_height >= 1 && desc->stride_x >= 1 && desc->stride_y >= 1 &&
                 desc->pad_x >= 0 && desc->pad_y >= 0, "pooling_forward: bad descriptor");
  int rc = cb200_check_dims(out_dims, "pooling_forward output");
  if (rc) return rc;
  rc = cb200_check_dims(in_dims, "pooling_forward input");
  if (rc) return rc;
  // [batch, channels, height, width], dense (rev order: w, h, c, n)
  for (const cb200_dims* d : {out_dims, in_dims}) {
    CB_REQUIRE(d->rev_shape[4] == 1, "pooling_forward: tensors must be 4-d [batch, channels, height, width]");
    long long expect = 1;
    for (int k = 0; k < 4; ++k) {
      CB_REQUIRE(!d->index[k], "pooling_forward: index arrays are not supported");
      CB_REQUIRE(d->rev_shape[k] == 1 || d->rev_strides[k] == expect, "pooling_forward: tensors must be dense");
      expect *= d->rev_shape[k];
    }
  }
  CB_REQUIRE(out_dims->rev_shape[3] == in_dims->rev_shape[3] && out_dims->rev_shape[2] == in_dims->rev_shape[2],
             "pooling_forward: batch / channel counts of input and output differ");
  PoolGeom g;
  g.channels = in_dims->rev_shape[2]; g.in_h = in_dims->rev_shape[1]; g.in_w = in_dims->rev_shape[0];
  g.out_h = out_dims->rev_shape[1]; g.out_w = out_dims->rev_shape[0];
  g.kw = desc->kernel_width; g.kh = desc->kernel_height; g.pad_x = desc->pad_x; g.pad_y = desc->pad_y;
  g.stride_x = desc->stride_x; g.stride_y = desc->stride_y; g.op = desc->pool_op;
  const long long n_out = (long long)out_dims->rev_shape[3] * out_dims->rev_shape[2] * g.out_h * g.out_w;
  if (n_out == 0) return CB200_OK;
  CB_REQUIRE(n_out <= 2147483647LL, "pooling_forward: output has more than 2^31 - 1 elements");
  DeviceGuard guard(s->device);
  long long blocks = (n_out + 255) / 256;
  const long long cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (dtype == CB200_FLOAT) pooling_launch<float>(s, (float*)out, (const float*)in, g, n_out, out_alpha, (unsigned)blocks);
  else pooling_launch<double>(s, (double*)out, (const double*)in, g, n_out, out_alpha, (unsigned)blocks);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}
