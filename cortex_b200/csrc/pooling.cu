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

template <typename T>
__global__ void __launch_bounds__(256)
pooling_forward_kernel(T* out, const T* in, PoolGeom g, long long n_out, double out_alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_out; i += (long long)gridDim.x * blockDim.x) {
    const int ox = (int)(i % g.out_w);
    const long long t = i / g.out_w;
    const int oy = (int)(t % g.out_h);
    const long long plane = t / g.out_h;                 // batch * channels + channel
    const T* src = in + plane * (long long)g.in_h * g.in_w;
    const int rel_x = ox * g.stride_x - g.pad_x, rel_y = oy * g.stride_y - g.pad_y;
    const int over_x = max(0, rel_x + g.kw - g.in_w), over_y = max(0, rel_y + g.kh - g.in_h);
    const int under_x = min(rel_x, 0), under_y = min(rel_y, 0);
    const int exc_w = max(0, g.kw - over_x + under_x), exc_h = max(0, g.kh - over_y + under_y);
    const double divisor = g.op == CB200_POOL_AVG ? (double)(g.kw * g.kh) : (double)(exc_w * exc_h);
    T acc = (T)0;
    bool first = true;
    for (int ky = 0; ky < g.kh; ++ky) {
      const int iy = rel_y + ky;
      if (iy < -g.pad_y || iy >= g.in_h + g.pad_y) continue;
      for (int kx = 0; kx < g.kw; ++kx) {
        const int ix = rel_x + kx;
        if (ix < -g.pad_x || ix >= g.in_w + g.pad_x) continue;
        const bool inside = iy >= 0 && iy < g.in_h && ix >= 0 && ix < g.in_w;
        const T v = inside ? src[(long long)iy * g.in_w + ix] : (T)0;
        if (g.op == CB200_POOL_MAX) {
          if (first || v > acc) acc = v;
        } else {
          acc = (T)((double)acc + (double)v / divisor);
        }
        first = false;
      }
    }
    out[i] = out_alpha == 0.0 ? acc : (T)((double)acc + out_alpha * (double)out[i]);
  }
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
  DeviceGuard guard(s->device);
  long long blocks = (n_out + 255) / 256;
  const long long cap = (long long)s->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (dtype == CB200_FLOAT)
    pooling_forward_kernel<float><<<(unsigned)blocks, 256, 0, s->stream>>>((float*)out, (const float*)in, g, n_out, out_alpha);
  else
    pooling_forward_kernel<double><<<(unsigned)blocks, 256, 0, s->stream>>>((double*)out, (const double*)in, g, n_out, out_alpha);
  CB_LAUNCH_CHECK(s);
  return CB200_OK;
}
