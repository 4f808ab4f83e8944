// convolution-backward-weights! and convolution-backward-data!
// (src/cortex/tensor.clj:1469-1493 -> tm/convolution-backward-weights! / -data!; CPU semantics
// src/cortex/compute/cpu/tensor_math.clj:1716-1800 and the roll / unroll kernels of src/cortex/nn/impl.clj).
//
//   weights:  W_grad[C_out, K] = alpha * W_grad + sum over images n of  OG_n[C_out, hw] . cols_n[hw, K]
//             with cols_n the unrolled (im2col) input of image n, K = C_in*kH*kW
//   data:     colsgrad_n[hw, K] = OG_n^T[hw, C_out] . W[C_out, K], rolled back (col2im) into
//             I_grad[n, C_in, H, W] = alpha * I_grad + sum of the colsgrad entries that came from that pixel
//
// The reference CPU backend reuses the unrolled input its forward pass left in the caller's workspace; here the
// unrolled matrix is rebuilt in the stream's own workspace (the forward pass keeps none: it gathers straight
// into the tensor-core tiles).  The data gradient is ONE product over all images (the output gradient is first
// transposed to pixel rows) through the same dispatch as gemm! (tcgen05 3xTF32 / DMMA / SIMT); the weight gradient is a split reduction of its own (conv_wgrad_kernel): its
// output is C_out x K small while the reduction runs over every pixel of the batch.  col2im is a gather: one thread per input
// pixel sums the (at most kH*kW) unrolled entries that read it, so there are no atomics and the sum order is
// fixed.  The CPU backend ignores input-gradient-alpha (it always clears the gradient); this backend applies it,
// as the reference's CUDA backend does -- the two agree for alpha = 0, which is what the layers pass.
#include "common.cuh"

int cb200_gemm_no_workspace(cb200_stream* s, int dtype, void* C, long long ldc, int trans_a, int trans_b, double alpha,
                            const void* A, long long a_rows, long long a_cols, long long lda, const void* B,
                            long long b_cols, long long ldb, double beta);

int cb200_gemm_tf32x3_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                             const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                             float beta, const float* bias, int act, int store_mode, int hw, int flags);
bool cb200_gemm_tf32x3_eligible(const float* A, long long lda, const float* B, long long ldb, int M, int N, int K);
bool cb200_conv_forward_f32_uses_tma(const cb200_stream* s, int batch, int cin, int in_h, int in_w, int cout, int out_h,
                                     int out_w, int kh, int kw, int stride_x, int stride_y);
int cb200_conv_forward_f32(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                           int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y, int stride_x,
                           int stride_y, float out_alpha);

namespace {

struct BwdGeom {
  int batch, cin, in_h, in_w, out_h, out_w, kh, kw, pad_x, pad_y, stride_x, stride_y;
  int kcols;   // cin*kh*kw
  int ld;      // row pitch of the unrolled matrix (kcols rounded up to 4)
};

// cols[(n*hw + p) * ld + c*kh*kw + ky*kw + kx] = in[n, c, oy*sy - py + ky, ox*sx - px + kx] (0 in the padding).
// One block walks whole rows of the unrolled matrix (one output pixel each): the pixel's coordinates are worked
// out once per row, a thread then needs two small divisions per element, and a warp writes 128 contiguous bytes.
template <typename T>
__global__ void __launch_bounds__(256) unroll_kernel(T* cols, const T* in, BwdGeom g, long long rows) {
  const int hw = g.out_h * g.out_w, taps = g.kh * g.kw;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const int n = (int)(row / hw), p = (int)(row - (long long)n * hw);
    const int oy = p / g.out_w, ox = p - oy * g.out_w;
    const int y0 = oy * g.stride_y - g.pad_y, x0 = ox * g.stride_x - g.pad_x;
    const T* img = in + (long long)n * g.cin * g.in_h * g.in_w;
    T* dst = cols + row * g.ld;
    for (int col = threadIdx.x; col < g.ld; col += blockDim.x) {
      T v = (T)0;
      if (col < g.kcols) {
        const int c = col / taps, t = col - c * taps;
        const int ky = t / g.kw, kx = t - ky * g.kw;
        const int iy = y0 + ky, ix = x0 + kx;
        if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w) v = img[((long long)c * g.in_h + iy) * g.in_w + ix];
      }
      dst[col] = v;
    }
  }
}

// in_grad[n, c, iy, ix] = alpha * in_grad + sum over taps (ky, kx) with (iy + py - ky) % sy == 0 etc. of
// colsgrad[(n*hw + oy*out_w + ox) * ld + c*kh*kw + ky*kw + kx]
template <typename T>
__global__ void __launch_bounds__(256) roll_kernel(T* in_grad, const T* colsgrad, BwdGeom g, T alpha, long long total) {
  typedef typename acc_of<T>::type A;
  const int hw = g.out_h * g.out_w;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ix = (int)(i % g.in_w);
    long long r = i / g.in_w;
    const int iy = (int)(r % g.in_h);
    r /= g.in_h;
    const int c = (int)(r % g.cin), n = (int)(r / g.cin);
    A acc = (A)0;
    for (int ky = 0; ky < g.kh; ++ky) {
      const int ty = iy + g.pad_y - ky;
      if (ty < 0 || ty % g.stride_y) continue;
      const int oy = ty / g.stride_y;
      if (oy >= g.out_h) continue;
      for (int kx = 0; kx < g.kw; ++kx) {
        const int tx = ix + g.pad_x - kx;
        if (tx < 0 || tx % g.stride_x) continue;
        const int ox = tx / g.stride_x;
        if (ox >= g.out_w) continue;
        acc += (A)colsgrad[((long long)n * hw + oy * g.out_w + ox) * g.ld + (c * g.kh + ky) * g.kw + kx];
      }
    }
    in_grad[i] = alpha == (T)0 ? (T)acc : (T)((A)alpha * (A)in_grad[i] + acc);
  }
}

// W_grad[C_out, K] += sum over the block's images of OG_n[C_out, hw] . cols_n[hw, K].  The output is tiny
// (C_out x K) and the reduction runs over batch * hw pixels, so the parallelism has to come from splitting that
// reduction: block = (64 x 64 output tile, group of images); 4 x 4 outputs per thread from 16-deep shared-memory
// tiles (fp32 / fp64 FMA: the reduction length per block is one or a few images, far too short per tile for the
// tensor-core kernel's pipeline to pay); one atomic add per output and block at the end.
template <typename T>
__global__ void __launch_bounds__(256)
conv_wgrad_kernel(T* wg, const T* og, const T* cols, int cout, int kcols, int ld, int hw, int batch, int imgs_per_block,
                  int vec_a) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ T As[TK][TM + 4];
  __shared__ T Bs[TK][TN];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * TN, m0 = blockIdx.y * TM;
  const int img0 = blockIdx.z * imgs_per_block, img1 = min(batch, img0 + imgs_per_block);
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = T();
  const int a_row = tid >> 2, a_kq = (tid & 3) * 4;      // A tile: 64 rows x 16 k, 4 consecutive k per thread
  const int b_k = tid >> 4, b_nq = (tid & 15) * 4;       // B tile: 16 k x 64 n, 4 consecutive n per thread
  for (int img = img0; img < img1; ++img) {
    const T* A = og + (long long)img * cout * hw;
    const T* B = cols + (long long)img * hw * ld;
    for (int k0 = 0; k0 < hw; k0 += TK) {
      T av[4] = {T(), T(), T(), T()}, bv[4] = {T(), T(), T(), T()};
      if (m0 + a_row < cout) {
        const T* src = A + (long long)(m0 + a_row) * hw + k0 + a_kq;
        if (vec_a && k0 + a_kq + 4 <= hw) {
          struct alignas(sizeof(T) * 4) V { T v[4]; };
          const V v = *reinterpret_cast<const V*>(src);
#pragma unroll
          for (int e = 0; e < 4; ++e) av[e] = v.v[e];
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) if (k0 + a_kq + e < hw) av[e] = src[e];
        }
      }
      if (k0 + b_k < hw && n0 + b_nq < ld) {
        // ld is a multiple of 4 and the workspace is 16-byte aligned; columns kcols .. ld-1 hold zeros
        struct alignas(sizeof(T) * 4) V { T v[4]; };
        const V v = *reinterpret_cast<const V*>(B + (long long)(k0 + b_k) * ld + n0 + b_nq);
#pragma unroll
        for (int e = 0; e < 4; ++e) bv[e] = v.v[e];
      }
      __syncthreads();          // the previous tile has been consumed
#pragma unroll
      for (int e = 0; e < 4; ++e) As[a_kq + e][a_row] = av[e];
#pragma unroll
      for (int e = 0; e < 4; ++e) Bs[b_k][b_nq + e] = bv[e];
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TK; ++kk) {
        T a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= cout) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < kcols) atomicAdd(wg + (long long)m * kcols + n, acc[i][j]);
    }
  }
}

// out[(n*hw + p) * ldo + c] = in[(n*C + c) * hw + p]: NCHW gradient -> one [batch*hw, C] matrix (pitch ldo)
template <typename T>
__global__ void __launch_bounds__(256) nchw_to_pixel_rows_kernel(T* out, const T* in, int C, int hw, int ldo) {
  __shared__ T t[32][33];
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32, n = blockIdx.z;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = c0 + ty + 8 * j, p_ = p0 + tx;
    if (c < C && p_ < hw) t[ty + 8 * j][tx] = in[((long long)n * C + c) * hw + p_];
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p_ = p0 + ty + 8 * j, c = c0 + tx;
    if (p_ < hw && c < ldo) out[((long long)n * hw + p_) * ldo + c] = c < C ? t[tx][ty + 8 * j] : T();
  }
}

// Operands of the weight gradient as ONE K-major product over all pixels of the batch (P = batch * hw, pitch ldp):
//   ogc[co][n*hw + p]               = out_grad[n, co, p]                       (gradient, channel-major)
//   ut[c*kh*kw + ky*kw + kx][n*hw + p] = in[n, c, oy*sy - py + ky, ox*sx - px + kx]  (the unrolled input, transposed)
// so that W_grad[co][k] = sum_P ogc[co][P] * ut[k][P] is a gemm! NT whose reduction runs over P.  Both kernels move
// whole pixel runs: adjacent threads read and write adjacent addresses.
// one block per (image, channel) run of hw pixels: a plain copy
__global__ void __launch_bounds__(256)
og_rows_copy_kernel(float* __restrict__ ogc, const float* __restrict__ og, int batch, int cout, int hw, long long ldp) {
  const long long runs = (long long)batch * cout;
  for (long long r = blockIdx.x; r < runs; r += gridDim.x) {
    const long long n = r / cout;
    const int co = (int)(r - n * cout);
    const float* src = og + r * hw;
    float* dst = ogc + (long long)co * ldp + n * hw;
    for (int p = threadIdx.x; p < hw; p += blockDim.x) dst[p] = src[p];
  }
}

// one block per (image, k row).  VEC4: four consecutive output columns per thread and one 16-byte store (out_w a
// multiple of 4, so that a group never straddles two output rows and every store is aligned); else one column per
// thread.  Reads are runs of one input row, writes runs of one output row.
template <bool VEC4>
__global__ void __launch_bounds__(256)
unroll_transposed_kernel(float* __restrict__ ut, const float* __restrict__ in, BwdGeom g, long long ldp) {
  const int hw = g.out_h * g.out_w, taps = g.kh * g.kw;
  const int k = blockIdx.x, n = blockIdx.y;
  const int c = k / taps, t = k - c * taps;
  const int ky = t / g.kw, kx = t - ky * g.kw;
  const float* plane = in + ((long long)n * g.cin + c) * g.in_h * g.in_w;
  float* dst = ut + (long long)k * ldp + (long long)n * hw;
  if (VEC4) {
    const int gpr = g.out_w >> 2, groups = g.out_h * gpr;
    for (int q = threadIdx.x; q < groups; q += blockDim.x) {
      const int oy = q / gpr, ox0 = (q - oy * gpr) << 2;
      const int iy = oy * g.stride_y - g.pad_y + ky;
      const bool row_in = iy >= 0 && iy < g.in_h;
      const float* src = plane + (long long)iy * g.in_w;
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ix = (ox0 + e) * g.stride_x - g.pad_x + kx;
        v[e] = (row_in && ix >= 0 && ix < g.in_w) ? src[ix] : 0.f;
      }
      *reinterpret_cast<float4*>(dst + (q << 2)) = make_float4(v[0], v[1], v[2], v[3]);
    }
  } else {
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int oy = ty; oy < g.out_h; oy += 8) {
      const int iy = oy * g.stride_y - g.pad_y + ky;
      const bool row_in = iy >= 0 && iy < g.in_h;
      const float* src = plane + (long long)iy * g.in_w;
      for (int ox = tx; ox < g.out_w; ox += 32) {
        const int ix = ox * g.stride_x - g.pad_x + kx;
        dst[oy * g.out_w + ox] = (row_in && ix >= 0 && ix < g.in_w) ? src[ix] : 0.f;
      }
    }
  }
}

// wg[co][k] = alpha * wg[co][k] + wt[k][co]   (the GEMM below produces the gradient transposed)
__global__ void __launch_bounds__(256)
wgrad_transpose_add_kernel(float* __restrict__ wg, const float* __restrict__ wt, int cout, int kcols, int ldt, float alpha) {
  const int total = cout * kcols;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int co = i / kcols, k = i - co * kcols;
    const float v = wt[(long long)k * ldt + co];
    wg[i] = alpha == 0.f ? v : alpha * wg[i] + v;
  }
}

template <typename T> __global__ void scale_kernel(T* p, T alpha, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    p[i] = alpha * p[i];
}

bool dense4(const cb200_dims* d) {
  long long e = 1;
  for (int i = 0; i < 4; ++i) {
    if (d->index[i]) return false;
    if (d->rev_shape[i] > 1 && d->rev_strides[i] != e) return false;
    e *= d->rev_shape[i];
  }
  return d->rev_shape[4] == 1;
}

// shared validation: fills the geometry from the input-side and output-side NCHW descriptors
int make_geom(BwdGeom& g, int& cout, const cb200_dims* in_dims, const cb200_dims* og_dims, const cb200_dims* w_dims,
              const cb200_conv_desc* desc, const char* who) {
  CB_REQUIRE(dense4(in_dims) && dense4(og_dims), "%s: Convolution arguments must be dense 4-d tensors", who);
  g.batch = in_dims->rev_shape[3]; g.cin = in_dims->rev_shape[2]; g.in_h = in_dims->rev_shape[1]; g.in_w = in_dims->rev_shape[0];
  g.out_h = og_dims->rev_shape[1]; g.out_w = og_dims->rev_shape[0];
  cout = og_dims->rev_shape[2];
  g.kh = desc->kernel_height; g.kw = desc->kernel_width;
  g.pad_x = desc->pad_x; g.pad_y = desc->pad_y; g.stride_x = desc->stride_x; g.stride_y = desc->stride_y;
  CB_REQUIRE(g.cin == desc->in_channels && cout == desc->out_channels && og_dims->rev_shape[3] == g.batch,
             "%s: tensor shapes do not match the descriptor", who);
  CB_REQUIRE(g.kh >= 1 && g.kw >= 1 && g.stride_x >= 1 && g.stride_y >= 1 && g.pad_x >= 0 && g.pad_y >= 0,
             "%s: bad descriptor", who);
  CB_REQUIRE(g.out_w == (g.in_w + 2 * g.pad_x - g.kw) / g.stride_x + 1 &&
             g.out_h == (g.in_h + 2 * g.pad_y - g.kh) / g.stride_y + 1,
             "%s: output extent does not match floor((in + 2*pad - k)/stride) + 1", who);
  g.kcols = g.cin * g.kh * g.kw;
  g.ld = (g.kcols + 3) & ~3;
  long long wec = 1;
  for (int i = 0; i < 5; ++i) wec *= w_dims->rev_shape[i];
  CB_REQUIRE(wec == (long long)cout * g.kcols, "%s: weight element count does not equal out-channels * kernel * in-channels", who);
  CB_REQUIRE((long long)g.batch * g.out_h * g.out_w <= 2147483647LL, "%s: more than 2^31-1 output pixels", who);
  return CB200_OK;
}

}  // namespace

extern "C" {

int cb200_convolution_backward_weights(cb200_stream* s, int dtype, void* w_grad, const cb200_dims* w_grad_dims,
                                       double w_grad_alpha, const void* out_grad, const cb200_dims* out_grad_dims,
                                       const void* in, const cb200_dims* in_dims, void* workspace,
                                       int64_t workspace_ecount, const cb200_conv_desc* desc) {
  (void)workspace; (void)workspace_ecount;
  CB_REQUIRE(s && w_grad && w_grad_dims && out_grad && out_grad_dims && in && in_dims && desc,
             "convolution_backward_weights: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE,
             "convolution-backward-weights! is only defined for float and double tensors");
  BwdGeom g;
  int cout = 0;
  int rc = make_geom(g, cout, in_dims, out_grad_dims, w_grad_dims, desc, "convolution_backward_weights");
  if (rc) return rc;
  const int hw = g.out_h * g.out_w;
  const long long rows = (long long)g.batch * hw;
  if (cout == 0 || g.kcols == 0) return CB200_OK;
  const size_t es = dtype == CB200_FLOAT ? 4 : 8;
  if (rows == 0) {
    // nothing to add: W_grad = alpha * W_grad is the caller's binary-op!; with no images leave it untouched
    return CB200_OK;
  }
  DeviceGuard guard(s->device);
  // fp32 with a reduction long enough to pay: ONE tensor-core gemm! NT over all pixels of the batch,
  // W_grad[C_out, K] = alpha * W_grad + ogc[C_out, P] . ut[K, P]^T, the reduction sliced over the SMs by the GEMM
  // itself (few output tiles, tens of thousands of k-blocks).  The sum order over P is fixed: deterministic.
  if (dtype == CB200_FLOAT && rows >= 4096 && g.kcols <= 65535 && g.batch <= 65535) {
    const long long ldp = (rows + 3) & ~3LL;
    const int ldt = (cout + 3) & ~3;
    void* ws = nullptr;
    const size_t operand_floats = (size_t)(cout + g.kcols) * ldp;
    if ((rc = cb200_scratch(s, (operand_floats + (size_t)g.kcols * ldt) * sizeof(float), &ws))) return rc;
    float* ogc = (float*)ws;
    float* ut = ogc + (size_t)cout * ldp;
    float* wt = ut + (size_t)g.kcols * ldp;           // the gradient transposed: [K][C_out]
    if (ldp != rows) CB_CUDA(cudaMemsetAsync(ws, 0, operand_floats * sizeof(float), s->stream));
    const long long runs = (long long)g.batch * cout;
    const long long cap16 = (long long)s->sm_count * 16;
    og_rows_copy_kernel<<<(unsigned)(runs < cap16 ? runs : cap16), 256, 0, s->stream>>>(ogc, (const float*)out_grad, g.batch,
                                                                                         cout, hw, ldp);
    CB_LAUNCH_CHECK(s);
    // 16-byte stores when every image's run of the k row starts aligned (hw % 4 == 0 follows from out_w % 4 == 0)
    if ((g.out_w % 4) == 0)
      unroll_transposed_kernel<true><<<dim3((unsigned)g.kcols, (unsigned)g.batch, 1), 256, 0, s->stream>>>(ut, (const float*)in, g, ldp);
    else
      unroll_transposed_kernel<false><<<dim3((unsigned)g.kcols, (unsigned)g.batch, 1), 256, 0, s->stream>>>(ut, (const float*)in, g, ldp);
    CB_LAUNCH_CHECK(s);
    // computed transposed, wt[K, C_out] = ut . ogc^T: the long dimension (K = C_in*kH*kW rows) fills the 128-row
    // tiles, C_out is one narrow column tile
    if (cb200_gemm_tf32x3_eligible(ut, ldp, ogc, ldp, g.kcols, cout, (int)rows)) {
      rc = cb200_gemm_tf32x3_launch(s, wt, ldt, 0, 1, 1.0f, ut, g.kcols, (int)rows, ldp, ogc, cout, ldp, 0.f, nullptr, 0, 0,
                                    1, 0);
      if (rc) return rc;
      const int n_out = cout * g.kcols;
      wgrad_transpose_add_kernel<<<(n_out + 255) / 256, 256, 0, s->stream>>>((float*)w_grad, wt, cout, g.kcols, ldt,
                                                                            (float)w_grad_alpha);
      CB_LAUNCH_CHECK(s);
      return CB200_OK;
    }
  }
  const long long total = rows * g.ld;
  void* cols = nullptr;
  if ((rc = cb200_scratch(s, (size_t)total * es, &cols))) return rc;
  const long long cap = (long long)s->sm_count * 32;
  const long long blocks = rows < cap ? rows : cap;
  if (dtype == CB200_FLOAT)
    unroll_kernel<float><<<(unsigned)blocks, 256, 0, s->stream>>>((float*)cols, (const float*)in, g, rows);
  else
    unroll_kernel<double><<<(unsigned)blocks, 256, 0, s->stream>>>((double*)cols, (const double*)in, g, rows);
  CB_LAUNCH_CHECK(s);
  // W_grad = alpha * W_grad first (alpha = 0: cleared without being read), then the split reduction adds onto it
  const long long wn = (long long)cout * g.kcols;
  if (w_grad_alpha == 0.0) {
    CB_CUDA(cudaMemsetAsync(w_grad, 0, (size_t)wn * es, s->stream));
  } else if (w_grad_alpha != 1.0) {
    const unsigned sb = (unsigned)((wn + 255) / 256 > cap ? cap : (wn + 255) / 256);
    if (dtype == CB200_FLOAT) scale_kernel<float><<<sb, 256, 0, s->stream>>>((float*)w_grad, (float)w_grad_alpha, wn);
    else scale_kernel<double><<<sb, 256, 0, s->stream>>>((double*)w_grad, w_grad_alpha, wn);
    CB_LAUNCH_CHECK(s);
  }
  const int tiles = ((g.kcols + 63) / 64) * ((cout + 63) / 64);
  // enough image groups for ~4 blocks per SM, at most one group per image
  int groups = (4 * s->sm_count + tiles - 1) / tiles;
  if (groups > g.batch) groups = g.batch;
  if (groups > 65535) groups = 65535;
  if (groups < 1) groups = 1;
  const int per = (g.batch + groups - 1) / groups;
  dim3 grid((unsigned)((g.kcols + 63) / 64), (unsigned)((cout + 63) / 64), (unsigned)((g.batch + per - 1) / per));
  const int vec_a = (hw % 4 == 0) && ((((uintptr_t)out_grad) & (4 * es - 1)) == 0);
  if (dtype == CB200_FLOAT)
    conv_wgrad_kernel<float><<<grid, 256, 0, s->stream>>>((float*)w_grad, (const float*)out_grad, (const float*)cols, cout,
                                                          g.kcols, g.ld, hw, g.batch, per, vec_a);
  else
    conv_wgrad_kernel<double><<<grid, 256, 0, s->stream>>>((double*)w_grad, (const double*)out_grad, (const double*)cols,
                                                           cout, g.kcols, g.ld, hw, g.batch, per, vec_a);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

// W[C_out][c*khkw + t]  ->  Wt[c][co*khkw + (khkw - 1 - t)]: the filter of the forward convolution that computes the
// data gradient (input and output channels swapped, taps mirrored)
__global__ void __launch_bounds__(256)
flip_weights_kernel(float* __restrict__ wt, const float* __restrict__ w, int cout, int cin, int khkw) {
  const int total = cout * cin * khkw;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int c = i / (cout * khkw), r = i - c * (cout * khkw);
    const int co = r / khkw, t = r - co * khkw;
    wt[i] = w[((long long)co * cin + c) * khkw + (khkw - 1 - t)];
  }
}

int cb200_convolution_backward_data(cb200_stream* s, int dtype, void* in_grad, const cb200_dims* in_grad_dims,
                                    double in_grad_alpha, const void* out_grad, const cb200_dims* out_grad_dims,
                                    const void* w, const cb200_dims* w_dims, void* workspace, int64_t workspace_ecount,
                                    const cb200_conv_desc* desc) {
  (void)workspace; (void)workspace_ecount;
  CB_REQUIRE(s && in_grad && in_grad_dims && out_grad && out_grad_dims && w && w_dims && desc,
             "convolution_backward_data: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE,
             "convolution-backward-data! is only defined for float and double tensors");
  BwdGeom g;
  int cout = 0;
  int rc = make_geom(g, cout, in_grad_dims, out_grad_dims, w_dims, desc, "convolution_backward_data");
  if (rc) return rc;
  const int hw = g.out_h * g.out_w;
  const long long rows = (long long)g.batch * hw;
  const long long in_total = (long long)g.batch * g.cin * g.in_h * g.in_w;
  if (in_total == 0) return CB200_OK;
  const size_t es = dtype == CB200_FLOAT ? 4 : 8;
  DeviceGuard guard(s->device);
  // Stride 1: the data gradient IS a forward convolution of the output gradient with the mirrored, channel-swapped
  // filter and padding k - 1 - pad:  in_grad[n, c, y, x] = sum over (co, ky, kx) of
  // out_grad[n, co, y + pad - ky, x + pad - kx] * W[co, c, ky, kx].  When that convolution qualifies for the TMA-fed
  // tensor-core kernels it runs there: no unrolled gradient matrix (K x pixels floats) is written or read back.
  if (dtype == CB200_FLOAT && rows > 0 && cout > 0 && g.stride_x == 1 && g.stride_y == 1 && g.pad_x <= g.kw - 1 &&
      g.pad_y <= g.kh - 1 &&
      cb200_conv_forward_f32_uses_tma(s, g.batch, cout, g.out_h, g.out_w, g.cin, g.in_h, g.in_w, g.kh, g.kw, 1, 1)) {
    // the forward launch takes (2 * its input + 2 * its weights) floats from the head of the stream's workspace:
    // the mirrored filter goes behind that
    const size_t og_elems = (size_t)rows * cout, w_elems = (size_t)cout * g.kcols;
    const size_t head = (2 * og_elems + 2 * w_elems) * sizeof(float);
    void* ws = nullptr;
    if ((rc = cb200_scratch(s, head + w_elems * sizeof(float), &ws))) return rc;
    float* wt = (float*)((char*)ws + head);
    int fb = (int)((w_elems + 255) / 256);
    if (fb > s->sm_count * 8) fb = s->sm_count * 8;
    flip_weights_kernel<<<fb, 256, 0, s->stream>>>(wt, (const float*)w, cout, g.cin, g.kh * g.kw);
    CB_LAUNCH_CHECK(s);
    return cb200_conv_forward_f32(s, (float*)in_grad, (const float*)out_grad, wt, g.batch, cout, g.out_h, g.out_w, g.cin,
                                  g.in_h, g.in_w, g.kh, g.kw, g.kw - 1 - g.pad_x, g.kh - 1 - g.pad_y, 1, 1,
                                  (float)in_grad_alpha);
  }
  void* colsgrad = nullptr;
  if (rows > 0 && cout > 0) {
    // all images in ONE product: the gradient is first laid out as pixel rows, OGt[batch*hw, C_out] (a 32 x 32
    // tile transpose per image), then colsgrad[batch*hw, K] = OGt . W
    const int ldt = (cout + 3) & ~3;
    const size_t cg_bytes = (size_t)rows * g.ld * es;
    if ((rc = cb200_scratch(s, cg_bytes + (size_t)rows * ldt * es, &colsgrad))) return rc;
    void* ogt = (char*)colsgrad + cg_bytes;
    CB_REQUIRE(g.batch <= 65535 && (ldt + 31) / 32 <= 65535, "convolution_backward_data: batch or channel count too large");
    dim3 tgrid((unsigned)((hw + 31) / 32), (unsigned)((ldt + 31) / 32), (unsigned)g.batch);
    if (dtype == CB200_FLOAT)
      nchw_to_pixel_rows_kernel<float><<<tgrid, 256, 0, s->stream>>>((float*)ogt, (const float*)out_grad, cout, hw, ldt);
    else
      nchw_to_pixel_rows_kernel<double><<<tgrid, 256, 0, s->stream>>>((double*)ogt, (const double*)out_grad, cout, hw, ldt);
    CB_LAUNCH_CHECK(s);
    rc = cb200_gemm_no_workspace(s, dtype, colsgrad, g.ld, 0, 0, 1.0, ogt, rows, cout, ldt, w, g.kcols, g.kcols, 0.0);
    if (rc) return rc;
  } else {
    // no output pixels: the sum is empty; a one-element dummy keeps the kernel's pointer valid
    if ((rc = cb200_scratch(s, 16, &colsgrad))) return rc;
    g.out_h = 0; g.out_w = 0;
  }
  long long blocks = (in_total + 255) / 256, cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (dtype == CB200_FLOAT)
    roll_kernel<float><<<(unsigned)blocks, 256, 0, s->stream>>>((float*)in_grad, (const float*)colsgrad, g,
                                                                (float)in_grad_alpha, in_total);
  else
    roll_kernel<double><<<(unsigned)blocks, 256, 0, s->stream>>>((double*)in_grad, (const double*)colsgrad, g,
                                                                 in_grad_alpha, in_total);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}

}  // extern "C"
