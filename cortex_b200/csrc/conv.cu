// convolution-forward! (src/cortex/tensor/math.clj:197-203): NCHW
// cross-correlation, out = conv(in, W) + out_alpha * out.
//
// Same decomposition as the reference CPU backend
// (src/cortex/compute/cpu/tensor_math.clj:1118-1131, 1682-1714,
//  src/cortex/nn/impl.clj:8-90): the input unrolled into a
// [batch*outH*outW, C_in*kH*kW] matrix (column = c*kH*kW + ky*kW + kx, zeros in
// the padding) times W[C_out, C_in*kH*kW] transposed.  Unlike the reference, the
// whole batch is ONE GEMM with the output pixels as the M dimension and an
// epilogue that scatters [pixel, channel] tiles straight into NCHW.
//   fp32: conv_igemm.cu gathers the unrolled rows directly into the tensor-core
//         operand tiles; the unrolled matrix is never materialised.  The only
//         scratch memory it takes from the stream is for re-ordered / zero-padded
//         hi and lo copies of the WEIGHTS (2 * C_out * K floats).
//   fp64: explicit im2col into the stream's scratch buffer, then one DMMA GEMM
//         per image as the reference does.
// The caller's workspace tensor is not used by either.
#include "common.cuh"
#include <mutex>

int cb200_gemm_tf32x3_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                             const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                             float beta, const float* bias, int act, int store_mode, int hw, int flags);
int cb200_gemm_f64_launch(cb200_stream* s, double* C, long long ldc, int trans_a, int trans_b, double alpha,
                          const double* A, int M, int K, long long lda, const double* B, int N, long long ldb,
                          double beta, const double* bias, int act, const PeerList* peers);
int cb200_gemm_simt_f32_launch(cb200_stream* s, float* C, long long ldc, int trans_a, int trans_b, float alpha,
                               const float* A, int M, int K, long long lda, const float* B, int N, long long ldb,
                               float beta);
int cb200_conv_igemm_launch(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                            int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y,
                            int stride_x, int stride_y, float out_alpha, const float* bias, int act);

bool cb200_conv_halo_eligible(int cin, int cout, int out_w, int out_h, int kh, int kw, int stride_x, int stride_y,
                              long long in_elems);
int cb200_conv_halo_launch(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                           int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y,
                           float out_alpha, const float* bias, int act);
bool cb200_conv_tma_eligible(int cin, int cout, int kh, int kw, int out_w, int out_h, int stride_x, int stride_y,
                             long long in_elems);
int cb200_conv_tma_launch(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                          int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y,
                          int stride_x, int stride_y, float out_alpha, const float* bias, int act);

// fp32 forward convolution on dense NCHW tensors, routed by geometry.  Layers with a multiple of 16 input
// channels: every operand tile by TMA -- stride 1: the input patch kept in shared memory across the filter taps
// (conv_halo.cu) where the 8 x 16 tiles fit the output, one shifted tile per tap otherwise (conv_tma.cu, which also
// takes stride-2 layers with enough products per input element through the tensor map's traversal stride); the rest:
// im2col rows gathered by threads (conv_igemm.cu).  opt_conv_route: 0 = by geometry, 1 = always gather, 2 = never
// the patch kernel, 3 = by geometry, but the patch kernel always behind its layout pre-pass.  Also the engine of convolution-backward-data! (conv_backward.cu).
bool cb200_conv_forward_f32_uses_tma(const cb200_stream* s, int batch, int cin, int in_h, int in_w, int cout, int out_h,
                                     int out_w, int kh, int kw, int stride_x, int stride_y) {
  const long long in_elems = (long long)batch * cin * in_h * in_w;
  if ((s->opt_conv_route == 0 || s->opt_conv_route == 3) && cb200_conv_halo_eligible(cin, cout, out_w, out_h, kh, kw, stride_x, stride_y, in_elems))
    return true;
  return s->opt_conv_route != 1 && cb200_conv_tma_eligible(cin, cout, kh, kw, out_w, out_h, stride_x, stride_y, in_elems);
}

// out = act(conv(in, w) + out_alpha * out + bias[channel]): bias (may be null) and the activation (enum cb200_act)
// are applied in the epilogue of whichever kernel runs the layer.
int cb200_conv_forward_f32_bias_act(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin,
                                    int in_h, int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x,
                                    int pad_y, int stride_x, int stride_y, float out_alpha, const float* bias, int act) {
  const long long in_elems = (long long)batch * cin * in_h * in_w;
  if ((s->opt_conv_route == 0 || s->opt_conv_route == 3) && cb200_conv_halo_eligible(cin, cout, out_w, out_h, kh, kw, stride_x, stride_y, in_elems))
    return cb200_conv_halo_launch(s, out, in, w, batch, cin, in_h, in_w, cout, out_h, out_w, kh, kw, pad_x, pad_y, out_alpha, bias, act);
  if (s->opt_conv_route != 1 && cb200_conv_tma_eligible(cin, cout, kh, kw, out_w, out_h, stride_x, stride_y, in_elems))
    return cb200_conv_tma_launch(s, out, in, w, batch, cin, in_h, in_w, cout, out_h, out_w, kh, kw, pad_x, pad_y, stride_x, stride_y, out_alpha, bias, act);
  return cb200_conv_igemm_launch(s, out, in, w, batch, cin, in_h, in_w, cout, out_h, out_w, kh, kw, pad_x, pad_y, stride_x,
                                 stride_y, out_alpha, bias, act);
}

int cb200_conv_forward_f32(cb200_stream* s, float* out, const float* in, const float* w, int batch, int cin, int in_h,
                           int in_w, int cout, int out_h, int out_w, int kh, int kw, int pad_x, int pad_y, int stride_x,
                           int stride_y, float out_alpha) {
  return cb200_conv_forward_f32_bias_act(s, out, in, w, batch, cin, in_h, in_w, cout, out_h, out_w, kh, kw, pad_x, pad_y,
                                         stride_x, stride_y, out_alpha, nullptr, 0);
}

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
    // rows < 2^31 and ld < 2^31 (checked by the caller): one 64-bit division, the rest 32-bit
    const unsigned row = (unsigned)(i / (unsigned)g.ld);
    const int col = (int)(i - (long long)row * g.ld);
    T v = (T)0;
    if (col < g.kcols) {
      int kx = col % g.kw, ky = (col / g.kw) % g.kh, c = col / (g.kw * g.kh);
      const unsigned hw = (unsigned)(g.out_h * g.out_w);
      int n = (int)(row / hw), p = (int)(row % hw);
      int oy = p / g.out_w, ox = p % g.out_w;
      int iy = oy * g.stride_y - g.pad_y + ky, ix = ox * g.stride_x - g.pad_x + kx;
      if (iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w)
        v = in[(((long long)n * g.cin + c) * g.in_h + iy) * g.in_w + ix];
    }
    cols[i] = v;
  }
}

// fp64 layers: bias per output channel and activation over the finished NCHW output
__global__ void __launch_bounds__(256)
conv_bias_act_f64_kernel(double* out, const double* bias, int act, unsigned hw, unsigned channels, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    double v = out[i];
    if (bias) v += bias[(unsigned)((i / hw) % channels)];
    if (act == CB200_ACT_RELU) v = v > 0.0 ? v : 0.0;
    else if (act == CB200_ACT_TANH) v = tanh(v);
    else if (act == CB200_ACT_LOGISTIC) v = 1.0 / (1.0 + exp(-v));
    out[i] = v;
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

static int convolution_forward_impl(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, double out_alpha,
                                    const void* in, const cb200_dims* in_dims, const void* w, const cb200_dims* w_dims,
                                    const cb200_conv_desc* desc, const void* bias, int act) {
  CB_REQUIRE(s && out && out_dims && in && in_dims && w && w_dims && desc, "convolution_forward: null argument");
  CB_REQUIRE(act >= CB200_ACT_NONE && act <= CB200_ACT_LOGISTIC, "convolution_forward: unknown activation %d", act);
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
  if (dtype == CB200_FLOAT)
    return cb200_conv_forward_f32_bias_act(s, (float*)out, (const float*)in, (const float*)w, g.batch, g.cin, g.in_h, g.in_w,
                                           cout, g.out_h, g.out_w, g.kh, g.kw, g.pad_x, g.pad_y, g.stride_x, g.stride_y,
                                           (float)out_alpha, (const float*)bias, act);
  const size_t es = 8;
  const long long total = rows * g.ld;
  void* cols = nullptr;
  int rc = cb200_scratch(s, (size_t)total * es, &cols);
  if (rc) return rc;
  DeviceGuard guard(s->device);
  long long blocks = (total + 255) / 256, cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  // fp64: im2col into the stream's scratch, then one DMMA GEMM per image as the reference does
  im2col_kernel<double><<<(unsigned)blocks, 256, 0, s->stream>>>((double*)cols, (const double*)in, g, total);
  CB_LAUNCH_CHECK(s);
  for (int n = 0; n < g.batch; ++n) {
    // per image, as the reference: out_n[C_out, hw] = W[C_out, K] * cols_n[hw, K]^T + out_alpha * out_n
    rc = cb200_gemm_f64_launch(s, (double*)out + (long long)n * cout * hw, hw, 0, 1, 1.0, (const double*)w, cout,
                               g.kcols, g.kcols, (const double*)cols + (long long)n * hw * g.ld, hw, g.ld, out_alpha,
                               nullptr, 0, nullptr);
    if (rc) return rc;
  }
  if (bias || act) {
    // fp64: one more pass over the output (the per-image GEMMs write whole [C_out, hw] blocks)
    const long long n_out = rows * cout;
    long long b2 = (n_out + 255) / 256;
    if (b2 > cap) b2 = cap;
    conv_bias_act_f64_kernel<<<(unsigned)b2, 256, 0, s->stream>>>((double*)out, (const double*)bias, act, (unsigned)hw,
                                                                   (unsigned)cout, n_out);
    CB_LAUNCH_CHECK(s);
  }
  return CB200_OK;
}

int cb200_convolution_forward(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, double out_alpha,
                              const void* in, const cb200_dims* in_dims, const void* w, const cb200_dims* w_dims,
                              void* workspace, int64_t workspace_ecount, const cb200_conv_desc* desc) {
  (void)workspace; (void)workspace_ecount;
  return convolution_forward_impl(s, dtype, out, out_dims, out_alpha, in, in_dims, w, w_dims, desc, nullptr, CB200_ACT_NONE);
}

int cb200_convolution_forward_bias_act(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims, double out_alpha,
                                       const void* in, const cb200_dims* in_dims, const void* w, const cb200_dims* w_dims,
                                       const cb200_conv_desc* desc, const void* bias, int act) {
  return convolution_forward_impl(s, dtype, out, out_dims, out_alpha, in, in_dims, w, w_dims, desc, bias, act);
}

// ---------------------------------------------------------------------------------------------
// convolution-forward! for callers that must not allocate.
//
// cb200_convolution_forward takes scratch memory from a per-stream buffer that it grows with
// cudaMalloc on demand (fp64: the unrolled input; fp32: split copies of the weights).  Some hosts of this library cannot tolerate that: a serving loop that has
// handed all device memory to its own pool, a process that forbids the implicit device-wide
// synchronisation of cudaMalloc / cudaFree on its latency path, or code that runs between two
// points where allocation is simply not allowed.  This variant keeps the unrolled matrix in a
// fixed array that is part of the library image instead.
//
//  * The array is CB200_STATIC_CONV_SCRATCH_BYTES (64 MiB) of device memory per GPU that loads the
//    library, held until the process exits whether or not this entry point is ever called.
//  * A problem whose unrolled matrix (batch*outH*outW rows x C_in*kH*kW columns, columns rounded up
//    to 4) does not fit is rejected with CB200_ERR_INVALID and a message; nothing is launched.
//  * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
//    that device current) and caches it.  Make that first call before any stream capture.
//    No call allocates or frees device or host memory, directly or through a library.
//  * All calls, on all streams of a device, share the one array, and it keeps the previous call's
//    contents.  im2col rewrites every element of the region a call uses (padding columns included),
//    so nothing needs clearing between calls; but two calls whose kernels overlap on the GPU
//    (different streams, no event between them) race on it.  Serialise them.
#define CB200_STATIC_CONV_SCRATCH_BYTES (64ull << 20)
static __device__ __align__(256) unsigned char g_static_conv_scratch[CB200_STATIC_CONV_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mutex;
void* g_static_scratch_ptr[64] = {nullptr};

// Device address of g_static_conv_scratch on `device` (which must be current).  In host code the
// array's name is only a handle for the runtime, never a pointer a kernel may be given.
int static_scratch_address(int device, void** out) {
  CB_REQUIRE(device >= 0 && device < 64, "convolution_forward_static: device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[device]) {
    void* p = nullptr;
    CB_CUDA(cudaGetSymbolAddress(&p, g_static_conv_scratch));
    CB_REQUIRE(p != nullptr, "convolution_forward_static: the static scratch array has no device address");
    g_static_scratch_ptr[device] = p;
  }
  *out = g_static_scratch_ptr[device];
  return CB200_OK;
}
}  // namespace

int cb200_convolution_forward_static(cb200_stream* s, int dtype, void* out, const cb200_dims* out_dims,
                                     double out_alpha, const void* in, const cb200_dims* in_dims, const void* w,
                                     const cb200_dims* w_dims, const cb200_conv_desc* desc) {
  CB_REQUIRE(s && out && out_dims && in && in_dims && w && w_dims && desc, "convolution_forward_static: null argument");
  CB_REQUIRE(dtype == CB200_FLOAT || dtype == CB200_DOUBLE,
             "convolution-forward! is only defined for float and double tensors");
  ConvGeom g;
  g.batch = in_dims->rev_shape[3]; g.cin = in_dims->rev_shape[2]; g.in_h = in_dims->rev_shape[1]; g.in_w = in_dims->rev_shape[0];
  g.out_h = out_dims->rev_shape[1]; g.out_w = out_dims->rev_shape[0];
  g.kh = desc->kernel_height; g.kw = desc->kernel_width;
  g.pad_x = desc->pad_x; g.pad_y = desc->pad_y; g.stride_x = desc->stride_x; g.stride_y = desc->stride_y;
  const int cout = out_dims->rev_shape[2];
  CB_REQUIRE(in_dims->rev_shape[4] == 1 && out_dims->rev_shape[4] == 1, "convolution_forward_static: tensors must be 4-d");
  CB_REQUIRE(g.cin == desc->in_channels && cout == desc->out_channels && out_dims->rev_shape[3] == g.batch,
             "convolution_forward_static: tensor shapes do not match the descriptor");
  CB_REQUIRE(g.kh >= 1 && g.kw >= 1 && g.stride_x >= 1 && g.stride_y >= 1 && g.pad_x >= 0 && g.pad_y >= 0,
             "convolution_forward_static: bad descriptor");
  CB_REQUIRE(g.out_w == (g.in_w + 2 * g.pad_x - g.kw) / g.stride_x + 1 &&
             g.out_h == (g.in_h + 2 * g.pad_y - g.kh) / g.stride_y + 1,
             "convolution_forward_static: output extent does not match floor((in + 2*pad - k)/stride) + 1");
  for (int i = 0; i < 4; ++i)
    CB_REQUIRE(!in_dims->index[i] && !out_dims->index[i], "Convolution arguments must be dense tensors");
  long long e_in = 1, e_out = 1;
  for (int i = 0; i < 4; ++i) {
    CB_REQUIRE(in_dims->rev_shape[i] == 1 || in_dims->rev_strides[i] == e_in, "Convolution arguments must be dense tensors");
    CB_REQUIRE(out_dims->rev_shape[i] == 1 || out_dims->rev_strides[i] == e_out, "Convolution arguments must be dense tensors");
    e_in *= in_dims->rev_shape[i];
    e_out *= out_dims->rev_shape[i];
  }
  g.kcols = g.cin * g.kh * g.kw;
  g.ld = (g.kcols + 3) & ~3;
  long long wec = 1;
  for (int i = 0; i < 5; ++i) wec *= w_dims->rev_shape[i];
  CB_REQUIRE(wec == (long long)cout * g.kcols, "Weight element count does not equal out-channels * kernel * in-channels");
  const int hw = g.out_h * g.out_w;
  const long long rows = (long long)g.batch * hw;
  CB_REQUIRE(rows <= 2147483647LL, "convolution_forward_static: more than 2^31-1 output pixels");
  if (rows == 0 || cout == 0) return CB200_OK;
  const size_t es = dtype == CB200_FLOAT ? 4 : 8;
  const long long total = rows * g.ld;
  if (total == 0) return CB200_OK;
  CB_REQUIRE((unsigned long long)total * es <= CB200_STATIC_CONV_SCRATCH_BYTES,
             "convolution_forward_static: the unrolled input needs %lld bytes but the static scratch array holds %llu; "
             "use cb200_convolution_forward (which allocates) for this size",
             (long long)(total * (long long)es), (unsigned long long)CB200_STATIC_CONV_SCRATCH_BYTES);
  DeviceGuard guard(s->device);
  CB_REQUIRE(guard.ok, "convolution_forward_static: cannot select device %d", s->device);
  void* cols = nullptr;
  int rc = static_scratch_address(s->device, &cols);
  if (rc) return rc;
  long long blocks = (total + 255) / 256, cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (dtype == CB200_FLOAT) {
    im2col_kernel<float><<<(unsigned)blocks, 256, 0, s->stream>>>((float*)cols, (const float*)in, g, total);
    CB_LAUNCH_CHECK(s);
    if ((((uintptr_t)w) & 15) == 0 && (g.kcols % 4) == 0)
      return cb200_gemm_tf32x3_launch(s, (float*)out, hw, 0, 1, 1.0f, (const float*)cols, (int)rows, g.kcols, g.ld,
                                      (const float*)w, cout, g.kcols, (float)out_alpha, nullptr, 0, 1, hw, 0);
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
    rc = cb200_gemm_f64_launch(s, (double*)out + (long long)n * cout * hw, hw, 0, 1, 1.0, (const double*)w, cout,
                               g.kcols, g.kcols, (const double*)cols + (long long)n * hw * g.ld, hw, g.ld, out_alpha,
                               nullptr, 0, nullptr);
    if (rc) return rc;
  }
  return CB200_OK;
}

}  // extern "C"
