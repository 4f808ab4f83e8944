// convolution-forward! (src/cortex/tensor/math.clj:197-203): NCHW
// cross-correlation, out = conv(in, W) + out_alpha * out.
//
// Same decomposition as the reference CPU backend
// (src/cortex/compute/cpu/tensor_math.clj:1118-1131, 1682-1714,
//  src/cortex/nn/impl.clj:8-90): unroll the input into a
// [batch*outH*outW, C_in*kH*kW] matrix (column = c*kH*kW + ky*kW + kx, zeros in
// the padding), then multiply by W[C_out, C_in*kH*kW] transposed.  Unlike the
// reference, the whole batch is ONE GEMM with the output pixels as the M
// dimension; the tensor-core epilogue scatters its [pixel, channel] tile
// straight into NCHW (adjacent lanes = adjacent pixels, so stores coalesce).
// The unrolled matrix lives in the stream's scratch buffer, not in the caller's
// workspace.
#include "common.cuh"

int cb200_gemm_tf32x3_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                             const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                             float beta, const float* bias, int act, int store_mode, int hw, int flags);
int cb200_gemm_f64_launch(cb200_stream* s, double* C, long long ldc, int trans_a, int trans_b, double alpha,
                          const double* A, int M, int K, long long lda, const double* B, int N, long long ldb,
                          double beta, const double* bias, int act);
int cb200_gemm_simt_f32_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                               const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                               float beta);

namespace {

struct ConvGeom {
  int batch, cin, in_h, in_w, out_h, out_w, kh, kw, pad_x, pad_y, stride_x, stride_y;
  int kcols;   // cin*kh*kw
  int ld;      // row pitch of the unrolled matrix (kcols rounded up to 4)
};

template <typename T>
__global__ void __launch_bounds__(256)
im2col_kernel(T* cols, const T* in, ConvGeom g, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int col = (int)(i % g.ld);
    long long row = i / g.ld;
    T v = (T)0;
    if (col < g.kcols) {
      int kx = col % g.kw, ky = (col / g.kw) % g.kh, c = col / (g.kw * g.kh);
      int hw = g.out_h * g.out_w;
      int n = (int)(row / hw), p = (int)(row % hw);
      int oy = p / g.out_w, ox = p % g.out_w;
      int iy = oy * g.stride_y - g.pad_y + ky, ix = ox * g.stride_x - g.pad_x + kx;
      if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w)
        v = in[(((long long)n * g.cin + c) * g.in_h + iy) * g.in_w + ix];
    }
    cols[i] = v;
  }
}

}  // namespace

extern "C" {

int cb200_convolution_workspace_size(const cb200_conv_desc* desc, int in_w, int in_h, int out_w, int out_h, int batch,
                                     int64_t* n_elems) {
  CB_REQUIRE(desc && n_elems, "convolution_workspace_size: null argument");
  (void)in_w; (void)in_h; (void)out_w; (void)out_h; (void)batch;
  *n_elems = 1;
  return CB200_OK;
}

int cb200_convolution_forward(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, double out_alpha,
                              const void* in, const cb200_dims* in_dims, const void* w, const cb200_dims* w_dims,
                              void* workspace, int64_t workspace_ecount, const cb200_conv_desc* desc) {
  (void)workspace; (void)workspace_ecount;
  CB_REQUIRE(s && out && out_dims && in && in_dims && w && w_dims && desc, "convolution_forward: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE,
             "convolution-forward! is only defined for float and double tensors");
  // input / output are dense [batch, channels, height, width]
  ConvGeom g;
  g.batch = in_dims->rev_shape[3]; g.cin = in_dims->rev_shape[2]; g.in_h = in_dims->rev_shape[1]; g.in_w = in_dims->rev_shape[0];
  g.out_h = out_dims->rev_shape[1]; g.out_w = out_dims->rev_shape[0];
  g.kh = desc->kernel_height; g.kw = desc->kernel_width;
  g.pad_x = desc->pad_x; g.pad_y = desc->pad_y; g.stride_x = desc->stride_x; g.stride_y = desc->stride_y;
  const int cout = out_dims->rev_shape[2];
  CB_REQUIRE(in_dims->rev_shape[4] == 1 && out_dims->rev_shape[4] == 1, "convolution_forward: tensors must be 4-d");
  CB_REQUIRE(g.cin == desc->in_channels && cout == desc->out_channels && out_dims->rev_shape[3] == g.batch,
             "convolution_forward: tensor shapes do not match the descriptor");
  CB_REQUIRE(g.kh >= 1 && g.kw >= 1 && g.stride_x >= 1 && g.stride_y >= 1 && g.pad_x >= 0 && g.pad_y >= 0,
             "convolution_forward: bad descriptor");
  CB_REQUIRE(g.out_w == (g.in_w + 2 * g.pad_x - g.kw) / g.stride_x + 1 &&
             g.out_h == (g.in_h + 2 * g.pad_y - g.kh) / g.stride_y + 1,
             "convolution_forward: output extent does not match floor((in + 2*pad - k)/stride) + 1");
  auto dense_nchw = [](const cb200_dims* d) {
    long long e = 1;
    for (int i = 0; i < 4; ++i) { if (d->index[i]) return false; if (d->rev_shape[i] > 1 && d->rev_strides[i] != e) return false; e *= d->rev_shape[i]; }
    return true;
  };
  CB_REQUIRE(dense_nchw(in_dims) && dense_nchw(out_dims), "Convolution arguments must be dense tensors");
  g.kcols = g.cin * g.kh * g.kw;
  g.ld = (g.kcols + 3) & ~3;
  long long wec = 1;
  for (int i = 0; i < 5; ++i) wec *= w_dims->rev_shape[i];
  CB_REQUIRE(wec == (long long)cout * g.kcols, "Weight element count does not equal out-channels * kernel * in-channels");
  const int hw = g.out_h * g.out_w;
  const long long rows = (long long)g.batch * hw;
  CB_REQUIRE(rows <= 2147483647LL, "convolution_forward: more than 2^31-1 output pixels");
  if (rows == 0 || cout == 0) return CB200_OK;
  const size_t es = dtype == CB200_FLOAT ? 4 : 8;
  const long long total = rows * g.ld;
  void* cols = nullptr;
  int rc = cb200_scratch(s, (size_t)total * es, &cols);
  if (rc) return rc;
  DeviceGuard guard(s->device);
  long long blocks = (total + 255) / 256, cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (dtype == CB200_FLOAT) {
    im2col_kernel<float><<<(unsigned)blocks, 256, 0, s->stream>>>((float*)cols, (const float*)in, g, total);
    CB_LAUNCH_CHECK(s);
    if ((((uintptr_t)w) & 15) == 0 && (g.kcols % 4) == 0) {
      // out[pixel, co] = cols[pixel, :] . W[co, :]   stored as NCHW
      return cb200_gemm_tf32x3_launch(s, (float*)out, hw, 0, 1, 1.0f, (const float*)cols, (int)rows, g.kcols, g.ld,
                                      (const float*)w, cout, g.kcols, (float)out_alpha, nullptr, 0, 1, hw, 0);
    }
    for (int n = 0; n < g.batch; ++n) {
      rc = cb200_gemm_simt_f32_launch(s, (float*)out + (long long)n * cout * hw, hw, 0, 1, 1.0f, (const float*)w, cout,
                                      g.kcols, g.kcols, (const float*)cols + (long long)n * hw * g.ld, hw, g.ld,
                                      (float)out_alpha);
      if (rc) return rc;
    }
    return CB200_OK;
  }
  im2col_kernel<double><<<(unsigned)blocks, 256, 0, s->stream>>>((double*)cols, (const double*)in, g, total);
  CB_LAUNCH_CHECK(s);
  for (int n = 0; n < g.batch; ++n) {
    // per image, as the reference: out_n[C_out, hw] = W[C_out, K] * cols_n[hw, K]^T + out_alpha * out_n
    rc = cb200_gemm_f64_launch(s, (double*)out + (long long)n * cout * hw, hw, 0, 1, 1.0, (const double*)w, cout,
                               g.kcols, g.kcols, (const double*)cols + (long long)n * hw * g.ld, hw, g.ld, out_alpha,
                               nullptr, 0);
    if (rc) return rc;
  }
  return CB200_OK;
}

}  // extern "C"
