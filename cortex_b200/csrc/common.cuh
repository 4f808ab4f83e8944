// Shared internals of libcortex_b200: stream object, error plumbing, the
// device-side restatement of cortex's index system and of the JVM arithmetic
// rules its CPU backend computes with.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>
#include <memory>
#include <vector>
#include "../../include/cortex_b200.h"

struct cb200_stream {
  int device;
  cudaStream_t stream;
  int sm_count;
  int* status_dev;     // device words {code, detail, wait limit in cycles >> 10 (0 = default), injected fault bits}
  int* status_host;    // pinned mirror used by cb200_stream_status
  void* scratch;       // lazily grown per-stream device workspace
  size_t scratch_bytes;
  int* tile_flags;     // zero-initialised device words, one per output tile of a K-split GEMM launch
  size_t tile_flags_count;
  void* partials;      // lazily grown block for partial accumulators of K-split tail tiles (pair GEMM kernel)
  size_t partials_bytes;
  std::atomic<int64_t> launches;
  int64_t capture_start;   // launch counter when the running capture began; -1 when not capturing
  // Graphs captured on this stream hold the workspace / flag pointers of their launches as kernel
  // arguments.  While any is alive a block that has to grow is retired (kept until the stream is
  // destroyed) instead of freed.  The counter is shared with the graphs, which may outlive the stream.
  std::shared_ptr<std::atomic<int>> live_graphs;
  std::vector<void*> retired;
  // per-stream routing options (cb200_stream_set_option); 0 = automatic
  int opt_gemm_auto_presplit, opt_presplit_variant, opt_f64_simple, opt_conv_route, opt_gemm_k_slices, opt_gemm_tile_n, opt_gemm_slice_handover;
};

// A captured sequence of this library's launches on one stream, replayable with one call.
struct cb200_graph {
  int device;
  cudaGraph_t graph;
  cudaGraphExec_t exec;
  int64_t kernels;      // launches recorded while capturing (added to the stream's counter per replay)
  std::shared_ptr<std::atomic<int>> live;   // the capturing stream's live-graph counter
};

struct cb200_event {
  int device;
  cudaEvent_t ev;
  cb200_stream* stream;
};

void cb200_set_error(const char* fmt, ...);
int cb200_cuda_fail(cudaError_t e, const char* what, const char* file, int line);
// make `bytes` of per-stream scratch available (grows, never shrinks)
int cb200_scratch(cb200_stream* s, size_t bytes, void** out);
// at least `count` zeroed flag words owned by the stream (kernels that use them leave them zero)
int cb200_tile_flags(cb200_stream* s, size_t count, int** out);
// at least `bytes` of a second workspace block that is independent of cb200_scratch (which callers may already
// hold operands in); contents undefined
int cb200_partials(cb200_stream* s, size_t bytes, void** out);

#define CB_CUDA(call)                                                     \
  do {                                                                    \
    cudaError_t e__ = (call);                                             \
    if (e__ != cudaSuccess) return cb200_cuda_fail(e__, #call, __FILE__, __LINE__); \
  } while (0)

#define CB_REQUIRE(cond, ...)                                             \
  do {                                                                    \
    if (!(cond)) { cb200_set_error(__VA_ARGS__); return CB200_ERR_INVALID; } \
  } while (0)

#define CB_LAUNCH_CHECK(s)                                                \
  do {                                                                    \
    (s)->launches.fetch_add(1, std::memory_order_relaxed);                \
    cudaError_t e__ = cudaGetLastError();                                 \
    if (e__ != cudaSuccess) return cb200_cuda_fail(e__, "kernel launch", __FILE__, __LINE__); \
  } while (0)

struct DeviceGuard {
  int prev;
  bool ok;
  explicit DeviceGuard(int dev) : prev(-1), ok(true) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

static inline size_t cb200_dtype_size(int dt) {
  switch (dt) {
    case CB200_BYTE: return 1; case CB200_SHORT: return 2; case CB200_INT: return 4;
    case CB200_LONG: return 8; case CB200_FLOAT: return 4; case CB200_DOUBLE: return 8;
  }
  return 0;
}

// ---------------------------------------------------------------------------
// Arithmetic rules of the reference CPU backend (src/cortex/compute/cpu/tensor_math.clj,
// compiled with *unchecked-math*): float views are widened to double for every
// operation and rounded once on store; byte/short/int/long views are widened to
// 64-bit long, wrap on overflow and are narrowed by truncation on store;
// double -> integer stores use the JVM's saturating narrowing (NaN -> 0).
// ---------------------------------------------------------------------------
template <typename T> struct acc_of { typedef long long type; };
template <> struct acc_of<float> { typedef double type; };
template <> struct acc_of<double> { typedef double type; };

__host__ __device__ inline int jvm_d2i(double v) {
  if (v != v) return 0;
  if (v >= 2147483647.0) return 2147483647;
  if (v <= -2147483648.0) return (-2147483647 - 1);
  return (int)v;
}
__host__ __device__ inline long long jvm_d2l(double v) {
  if (v != v) return 0;
  if (v >= 9223372036854775807.0) return 9223372036854775807LL;
  if (v <= -9223372036854775808.0) return (-9223372036854775807LL - 1);
  return (long long)v;
}

template <typename T> struct store_as;
template <> struct store_as<float> {
  __host__ __device__ static float from(double v) { return (float)v; }
  __host__ __device__ static float from(long long v) { return (float)v; }
};
template <> struct store_as<double> {
  __host__ __device__ static double from(double v) { return v; }
  __host__ __device__ static double from(long long v) { return (double)v; }
};
template <> struct store_as<int> {
  __host__ __device__ static int from(double v) { return jvm_d2i(v); }
  __host__ __device__ static int from(long long v) { return (int)v; }
};
template <> struct store_as<long long> {
  __host__ __device__ static long long from(double v) { return jvm_d2l(v); }
  __host__ __device__ static long long from(long long v) { return v; }
};
template <> struct store_as<short> {
  __host__ __device__ static short from(double v) { return (short)jvm_d2i(v); }
  __host__ __device__ static short from(long long v) { return (short)v; }
};
template <> struct store_as<signed char> {
  __host__ __device__ static signed char from(double v) { return (signed char)jvm_d2i(v); }
  __host__ __device__ static signed char from(long long v) { return (signed char)v; }
};

// scalar (alpha, beta, constants) cast to the element type before use
template <typename T> __host__ __device__ inline typename acc_of<T>::type scalar_as(double v) {
  return (typename acc_of<T>::type)store_as<T>::from(v);
}

// ---------------------------------------------------------------------------
// Index system: element index -> element offset for one operand
// (src/cortex/tensor/dimensions.clj:226-252, resources/index_system.h:42-52).
// ---------------------------------------------------------------------------
struct Operand {
  int shape[5];
  int stride[5];
  const int* index[5];
};

struct Geometry {
  int max_shape[5];
  int ndims;   // dimensions beyond ndims all have max_shape 1
};

// Element indexes are 32-bit in the tensor protocol (int n_elems), so the divisions stay 32-bit;
// only the resulting offset is widened.
__device__ __forceinline__ long long operand_offset(const Operand& o, const Geometry& g, long long idx) {
  unsigned i = (unsigned)idx;
  long long off = 0;
#pragma unroll
  for (int d = 0; d < 5; ++d) {
    if (d < g.ndims) {
      unsigned m = (unsigned)g.max_shape[d];
      unsigned q = i / m;
      unsigned c = i - q * m;
      i = q;
      unsigned sh = (unsigned)o.shape[d];
      if (sh != m) c = c % sh;
      if (o.index[d]) c = (unsigned)o.index[d][c];
      off += (long long)o.stride[d] * (long long)c;
    }
  }
  return off;
}

static inline void operand_from_dims(Operand& o, const cb200_dims* d) {
  for (int i = 0; i < 5; ++i) {
    o.shape[i] = d->rev_shape[i];
    o.stride[i] = d->rev_strides[i];
    o.index[i] = d->index[i];
  }
}

// Extra destinations of a GEMM epilogue: the finished C window is also stored at the same row-major
// position of each buffer (other GPUs' memory, reached by plain stores over NVLink).
enum { CB_MAX_PEERS = 7 };
struct PeerList {
  int n;
  void* p[CB_MAX_PEERS];
};

// validation shared by the elementwise entry points
int cb200_check_dims(const cb200_dims* d, const char* what);

#define CB_DISPATCH_DTYPE(dt, T, ...)                                     \
  switch (dt) {                                                           \
    case CB200_BYTE:   { typedef signed char T; __VA_ARGS__; break; }     \
    case CB200_SHORT:  { typedef short T; __VA_ARGS__; break; }           \
    case CB200_INT:    { typedef int T; __VA_ARGS__; break; }             \
    case CB200_LONG:   { typedef long long T; __VA_ARGS__; break; }       \
    case CB200_FLOAT:  { typedef float T; __VA_ARGS__; break; }           \
    case CB200_DOUBLE: { typedef double T; __VA_ARGS__; break; }          \
    default: cb200_set_error("unknown dtype %d", (int)(dt)); return CB200_ERR_INVALID; \
  }
