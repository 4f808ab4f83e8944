// Device / stream / buffer / event half of the C ABI: the B200 counterpart of
// the reference's CudaDriver / CudaDevice / CudaStream records
// (src/cortex/compute/cuda/driver.clj:725-733, 849-1045).
#include "common.cuh"
#include <ctype.h>
#include <errno.h>
#include <stdarg.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>
#include <map>
#include <mutex>
#include <new>

static thread_local char g_err[1024] = "";

void cb200_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cb200_cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  cb200_set_error("CUDA error %d (%s) in %s at %s:%d", (int)e, cudaGetErrorString(e), what, file, line);
  return e == cudaErrorMemoryAllocation ? CB200_ERR_NOMEM : CB200_ERR_CUDA;
}

int cb200_check_dims(const cb200_dims* d, const char* what) {
  if (!d) { cb200_set_error("%s: null dimensions", what); return CB200_ERR_INVALID; }
  for (int i = 0; i < 5; ++i) {
    if (d->rev_shape[i] < 1) {
      cb200_set_error("%s: rev_shape[%d] = %d must be >= 1", what, i, d->rev_shape[i]);
      return CB200_ERR_INVALID;
    }
    if (d->rev_strides[i] < 0) {
      cb200_set_error("%s: rev_strides[%d] = %d must be >= 0", what, i, d->rev_strides[i]);
      return CB200_ERR_INVALID;
    }
  }
  return CB200_OK;
}

// A per-stream block (workspace or tile flags) has to grow.  Kernels already enqueued, and graphs
// captured on the stream, still hold the old address: while capturing nothing may be allocated at
// all; with live graphs the old block is retired (freed with the stream); otherwise it is freed
// once the stream has drained.
static int release_for_growth(cb200_stream* s, void* old_block, const char* what) {
  if (s->capture_start >= 0) {
    cb200_set_error("%s has to grow while the stream is capturing: run the sequence once before capturing it", what);
    return CB200_ERR_INVALID;
  }
  if (!old_block) return CB200_OK;
  if (s->live_graphs && s->live_graphs->load() > 0) {
    s->retired.push_back(old_block);
    return CB200_OK;
  }
  CB_CUDA(cudaStreamSynchronize(s->stream));
  CB_CUDA(cudaFree(old_block));
  for (void* r : s->retired) cudaFree(r);      // no graph is left that could replay them
  s->retired.clear();
  return CB200_OK;
}

int cb200_scratch(cb200_stream* s, size_t bytes, void** out) {
  if (bytes > s->scratch_bytes) {
    DeviceGuard g(s->device);
    int rc = release_for_growth(s, s->scratch, "the stream's workspace");
    if (rc) return rc;
    s->scratch = nullptr;
    s->scratch_bytes = 0;
    size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    CB_CUDA(cudaMalloc(&s->scratch, want));
    s->scratch_bytes = want;
  }
  *out = s->scratch;
  return CB200_OK;
}

int cb200_tile_flags(cb200_stream* s, size_t count, int** out) {
  if (count > s->tile_flags_count) {
    DeviceGuard g(s->device);
    int rc = release_for_growth(s, s->tile_flags, "the stream's tile-flag block");
    if (rc) return rc;
    s->tile_flags = nullptr;
    s->tile_flags_count = 0;
    size_t want = (count + 4095) & ~(size_t)4095;
    CB_CUDA(cudaMalloc(&s->tile_flags, want * sizeof(int)));
    CB_CUDA(cudaMemsetAsync(s->tile_flags, 0, want * sizeof(int), s->stream));
    s->tile_flags_count = want;
  }
  *out = s->tile_flags;
  return CB200_OK;
}

int cb200_partials(cb200_stream* s, size_t bytes, void** out) {
  if (bytes > s->partials_bytes) {
    DeviceGuard g(s->device);
    int rc = release_for_growth(s, s->partials, "the stream's partial-sum block");
    if (rc) return rc;
    s->partials = nullptr;
    s->partials_bytes = 0;
    size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    CB_CUDA(cudaMalloc(&s->partials, want));
    s->partials_bytes = want;
  }
  *out = s->partials;
  return CB200_OK;
}

extern "C" {

const char* cb200_last_error(void) { return g_err; }

int cb200_unsupported(const char* method_name) {
  cb200_set_error("%s is outside the dense-inference path of this backend", method_name ? method_name : "?");
  return CB200_ERR_UNSUPPORTED;
}

int cb200_device_count(int* count) {
  CB_REQUIRE(count, "device_count: null out pointer");
  CB_CUDA(cudaGetDeviceCount(count));
  return CB200_OK;
}

int cb200_device_info(int device, char* name, int name_len, int* sm_count, int* cc_major, int* cc_minor) {
  cudaDeviceProp p;
  CB_CUDA(cudaGetDeviceProperties(&p, device));
  if (name && name_len > 0) { strncpy(name, p.name, name_len - 1); name[name_len - 1] = 0; }
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return CB200_OK;
}

int cb200_mem_info(int device, size_t* free_bytes, size_t* total_bytes) {
  DeviceGuard g(device);
  CB_REQUIRE(g.ok, "mem_info: cannot select device %d", device);
  size_t f = 0, t = 0;
  CB_CUDA(cudaMemGetInfo(&f, &t));
  if (free_bytes) *free_bytes = f;
  if (total_bytes) *total_bytes = t;
  return CB200_OK;
}

int cb200_stream_create(int device, cb200_stream** out) {
  CB_REQUIRE(out, "stream_create: null out pointer");
  DeviceGuard g(device);
  CB_REQUIRE(g.ok, "stream_create: cannot select device %d", device);
  cb200_stream* s = new (std::nothrow) cb200_stream();
  if (!s) { cb200_set_error("stream_create: out of host memory"); return CB200_ERR_NOMEM; }
  s->device = device;
  s->scratch = nullptr;
  s->scratch_bytes = 0;
  s->tile_flags = nullptr;
  s->tile_flags_count = 0;
  s->partials = nullptr;
  s->partials_bytes = 0;
  s->launches.store(0);
  s->capture_start = -1;
  s->live_graphs = std::make_shared<std::atomic<int>>(0);
  s->opt_gemm_auto_presplit = s->opt_presplit_variant = s->opt_f64_simple = s->opt_conv_route = s->opt_gemm_k_slices = s->opt_gemm_tile_n = s->opt_gemm_slice_handover = 0;
  cudaError_t e = cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e == cudaSuccess) e = cudaMalloc((void**)&s->status_dev, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(s->status_dev, 0, 4 * sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost((void**)&s->status_host, 4 * sizeof(int));
  if (e != cudaSuccess) { delete s; return cb200_cuda_fail(e, "stream_create", __FILE__, __LINE__); }
  s->status_host[0] = s->status_host[1] = 0;
  *out = s;
  return CB200_OK;
}

int cb200_stream_destroy(cb200_stream* s) {
  if (!s) return CB200_OK;
  DeviceGuard g(s->device);
  cudaStreamSynchronize(s->stream);
  if (s->scratch) cudaFree(s->scratch);
  if (s->tile_flags) cudaFree(s->tile_flags);
  if (s->partials) cudaFree(s->partials);
  for (void* r : s->retired) cudaFree(r);
  cudaFree(s->status_dev);
  cudaFreeHost(s->status_host);
  cudaStreamDestroy(s->stream);
  delete s;
  return CB200_OK;
}

void* cb200_stream_native(cb200_stream* s) { return s ? (void*)s->stream : nullptr; }
int cb200_stream_device(cb200_stream* s) { return s ? s->device : -1; }
int64_t cb200_launch_count(cb200_stream* s) { return s ? s->launches.load() : 0; }

int cb200_stream_set_option(cb200_stream* s, int option, int64_t value) {
  CB_REQUIRE(s, "stream_set_option: null stream");
  switch (option) {
    case CB200_OPT_GEMM_AUTO_PRESPLIT:
      CB_REQUIRE(value >= 0 && value <= 2, "stream_set_option: gemm routing %lld outside [0, 2]", (long long)value);
      s->opt_gemm_auto_presplit = (int)value;
      return CB200_OK;
    case CB200_OPT_PRESPLIT_VARIANT:
      CB_REQUIRE(value >= 0 && value <= 2, "stream_set_option: pre-split kernel %lld outside [0, 2]", (long long)value);
      s->opt_presplit_variant = (int)value;
      return CB200_OK;
    case CB200_OPT_F64_SIMPLE_KERNEL:
      s->opt_f64_simple = value != 0;
      return CB200_OK;
    case CB200_OPT_CONV_ROUTE:
      CB_REQUIRE(value >= 0 && value <= 3, "stream_set_option: convolution route %lld outside [0, 3]", (long long)value);
      s->opt_conv_route = (int)value;
      return CB200_OK;
    case CB200_OPT_GEMM_K_SLICES:
      CB_REQUIRE(value >= 0 && value <= 16, "stream_set_option: K slices %lld outside [0, 16]", (long long)value);
      s->opt_gemm_k_slices = (int)value;
      return CB200_OK;
    case CB200_OPT_GEMM_SLICE_HANDOVER:
      CB_REQUIRE(value == 0 || value == 1, "stream_set_option: slice hand-over %lld outside [0, 1]", (long long)value);
      s->opt_gemm_slice_handover = (int)value;
      return CB200_OK;
    case CB200_OPT_GEMM_TILE_N:
      CB_REQUIRE(value == 0 || value == 64 || value == 128 || value == 256,
                 "stream_set_option: tile width %lld is not 0, 64, 128 or 256", (long long)value);
      s->opt_gemm_tile_n = (int)value;
      return CB200_OK;
    case CB200_OPT_WAIT_LIMIT_CYCLES:
    case CB200_OPT_INJECT_FAULT: {
      CB_REQUIRE(value >= 0 && value < ((int64_t)1 << 40), "stream_set_option: value out of range");
      CB_REQUIRE(s->capture_start < 0, "stream_set_option: not while capturing");
      DeviceGuard g(s->device);
      // stream-ordered: launches already enqueued keep the old setting
      const int word = option == CB200_OPT_WAIT_LIMIT_CYCLES ? (int)((value + 1023) >> 10) : (int)value;
      s->status_host[2] = word;      // staging only; the device copy is what kernels read
      CB_CUDA(cudaMemcpyAsync(s->status_dev + (option == CB200_OPT_WAIT_LIMIT_CYCLES ? 2 : 3), &s->status_host[2],
                              sizeof(int), cudaMemcpyHostToDevice, s->stream));
      CB_CUDA(cudaStreamSynchronize(s->stream));
      return CB200_OK;
    }
  }
  cb200_set_error("stream_set_option: unknown option %d", option);
  return CB200_ERR_INVALID;
}

int cb200_stream_workspace_info(cb200_stream* s, size_t* workspace_bytes, int* retired_blocks, int* live_graphs) {
  CB_REQUIRE(s, "stream_workspace_info: null stream");
  if (workspace_bytes) *workspace_bytes = s->scratch_bytes + s->partials_bytes;
  if (retired_blocks) *retired_blocks = (int)s->retired.size();
  if (live_graphs) *live_graphs = s->live_graphs ? s->live_graphs->load() : 0;
  return CB200_OK;
}

int cb200_stream_status(cb200_stream* s, int* code, int* detail) {
  CB_REQUIRE(s, "stream_status: null stream");
  DeviceGuard g(s->device);
  CB_CUDA(cudaMemcpyAsync(s->status_host, s->status_dev, 2 * sizeof(int), cudaMemcpyDeviceToHost, s->stream));
  CB_CUDA(cudaMemsetAsync(s->status_dev, 0, 2 * sizeof(int), s->stream));
  CB_CUDA(cudaStreamSynchronize(s->stream));
  if (code) *code = s->status_host[0];
  if (detail) *detail = s->status_host[1];
  // a launch that gave up may have left tile flags set: later launches expect them zero
  if (s->status_host[0] != 0 && s->tile_flags)
    CB_CUDA(cudaMemsetAsync(s->tile_flags, 0, s->tile_flags_count * sizeof(int), s->stream));
  return CB200_OK;
}

int cb200_malloc(int device, size_t bytes, void** out) {
  CB_REQUIRE(out, "malloc: null out pointer");
  DeviceGuard g(device);
  CB_REQUIRE(g.ok, "malloc: cannot select device %d", device);
  CB_CUDA(cudaMalloc(out, bytes ? bytes : 1));
  return CB200_OK;
}

int cb200_free(int device, void* ptr) {
  if (!ptr) return CB200_OK;
  DeviceGuard g(device);
  CB_CUDA(cudaFree(ptr));
  return CB200_OK;
}

int cb200_host_alloc(size_t bytes, void** out) {
  CB_REQUIRE(out, "host_alloc: null out pointer");
  CB_CUDA(cudaMallocHost(out, bytes ? bytes : 1));
  return CB200_OK;
}

// NUMA node of the GPU's PCIe slot, from sysfs; -1 when the platform does not say
static int device_numa_node(int device) {
  char bus[32] = "";
  if (cudaDeviceGetPCIBusId(bus, (int)sizeof(bus), device) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
  for (char* c = bus; *c; ++c) *c = (char)tolower(*c);
  char path[128];
  snprintf(path, sizeof(path), "/sys/bus/pci/devices/%s/numa_node", bus);
  FILE* f = fopen(path, "r");
  if (!f) return -1;
  int node = -1;
  if (fscanf(f, "%d", &node) != 1) node = -1;
  fclose(f);
  return node;
}

namespace {
std::mutex g_near_mutex;
std::map<void*, size_t> g_near_blocks;     // mmap'ed + registered blocks of cb200_host_alloc_near
}

int cb200_device_numa_node(int device, int* node) {
  CB_REQUIRE(node, "device_numa_node: null out pointer");
  *node = device_numa_node(device);
  return CB200_OK;
}

int cb200_host_alloc_near(int device, size_t bytes, void** out, int* node_out) {
  CB_REQUIRE(out, "host_alloc_near: null out pointer");
  const int node = device_numa_node(device);
  if (node_out) *node_out = -1;
  if (node < 0 || node >= 1024) return cb200_host_alloc(bytes, out);
  const size_t page = (size_t)sysconf(_SC_PAGESIZE);
  const size_t len = ((bytes ? bytes : 1) + page - 1) / page * page;
  void* p = mmap(nullptr, len, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  if (p == MAP_FAILED) return cb200_host_alloc(bytes, out);
  // MPOL_PREFERRED (1): pages come from `node` while it has room; set before the first touch
  unsigned long mask[16] = {0};
  mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
  const long bound = syscall(SYS_mbind, p, len, 1 /* MPOL_PREFERRED */, mask, (unsigned long)(8 * sizeof(mask)), 0u);
  memset(p, 0, len);     // first touch: the pages exist, on the chosen node, before they are pinned
  DeviceGuard g(device);
  cudaError_t e = cudaHostRegister(p, len, cudaHostRegisterPortable);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    munmap(p, len);
    return cb200_host_alloc(bytes, out);
  }
  {
    std::lock_guard<std::mutex> lock(g_near_mutex);
    g_near_blocks[p] = len;
  }
  if (node_out && bound == 0) *node_out = node;
  *out = p;
  return CB200_OK;
}

int cb200_host_free(void* ptr) {
  if (!ptr) return CB200_OK;
  size_t len = 0;
  {
    std::lock_guard<std::mutex> lock(g_near_mutex);
    auto it = g_near_blocks.find(ptr);
    if (it != g_near_blocks.end()) { len = it->second; g_near_blocks.erase(it); }
  }
  if (len) {
    CB_CUDA(cudaHostUnregister(ptr));
    munmap(ptr, len);
    return CB200_OK;
  }
  CB_CUDA(cudaFreeHost(ptr));
  return CB200_OK;
}

int cb200_memcpy_h2d(cb200_stream* s, void* dst, const void* src, size_t bytes) {
  CB_REQUIRE(s && (bytes == 0 || (dst && src)), "memcpy_h2d: null argument");
  DeviceGuard g(s->device);
  CB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, s->stream));
  return CB200_OK;
}

int cb200_memcpy_d2h(cb200_stream* s, void* dst, const void* src, size_t bytes) {
  CB_REQUIRE(s && (bytes == 0 || (dst && src)), "memcpy_d2h: null argument");
  DeviceGuard g(s->device);
  CB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, s->stream));
  return CB200_OK;
}

int cb200_memcpy_d2d(cb200_stream* s, void* dst, const void* src, size_t bytes) {
  CB_REQUIRE(s && (bytes == 0 || (dst && src)), "memcpy_d2d: null argument");
  DeviceGuard g(s->device);
  CB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s->stream));
  return CB200_OK;
}

// ---- stream capture: a launch-bound sequence (a small-batch forward pass) replayed as one graph ----
int cb200_graph_capture_begin(cb200_stream* s) {
  CB_REQUIRE(s, "graph_capture_begin: null stream");
  CB_REQUIRE(s->capture_start < 0, "graph_capture_begin: this stream is already capturing");
  DeviceGuard g(s->device);
  CB_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
  s->capture_start = s->launches.load();
  return CB200_OK;
}

int cb200_graph_capture_end(cb200_stream* s, cb200_graph** out) {
  CB_REQUIRE(s && out, "graph_capture_end: null argument");
  CB_REQUIRE(s->capture_start >= 0, "graph_capture_end: this stream is not capturing");
  DeviceGuard g(s->device);
  const int64_t kernels = s->launches.load() - s->capture_start;
  s->capture_start = -1;
  s->launches.fetch_sub(kernels);     // the captured launches did not run
  cudaGraph_t graph = nullptr;
  CB_CUDA(cudaStreamEndCapture(s->stream, &graph));
  cb200_graph* gr = new (std::nothrow) cb200_graph();
  if (!gr) { cudaGraphDestroy(graph); cb200_set_error("graph_capture_end: out of host memory"); return CB200_ERR_NOMEM; }
  gr->device = s->device; gr->graph = graph; gr->exec = nullptr; gr->kernels = kernels;
  cudaError_t err = cudaGraphInstantiate(&gr->exec, graph, 0);
  if (err != cudaSuccess) {
    cudaGraphDestroy(graph);
    delete gr;
    return cb200_cuda_fail(err, "cudaGraphInstantiate", __FILE__, __LINE__);
  }
  gr->live = s->live_graphs;        // from now on the stream's blocks are retired, not freed, when they grow
  gr->live->fetch_add(1);
  *out = gr;
  return CB200_OK;
}

int cb200_graph_launch(cb200_graph* gr, cb200_stream* s) {
  CB_REQUIRE(gr && s, "graph_launch: null argument");
  CB_REQUIRE(gr->device == s->device, "graph_launch: graph captured on device %d, stream is on device %d", gr->device,
             s->device);
  DeviceGuard g(s->device);
  CB_CUDA(cudaGraphLaunch(gr->exec, s->stream));
  s->launches.fetch_add(gr->kernels);
  return CB200_OK;
}

int cb200_graph_destroy(cb200_graph* gr) {
  if (!gr) return CB200_OK;
  DeviceGuard g(gr->device);
  if (gr->exec) cudaGraphExecDestroy(gr->exec);
  if (gr->graph) cudaGraphDestroy(gr->graph);
  if (gr->live) gr->live->fetch_sub(1);
  delete gr;
  return CB200_OK;
}

// ---- multi-GPU plumbing: peer access inside one process, CUDA IPC across processes ------------
int cb200_peer_enable(int device, int peer_device) {
  CB_REQUIRE(device != peer_device, "peer_enable: a device is not its own peer");
  DeviceGuard g(device);
  int can = 0;
  CB_CUDA(cudaDeviceCanAccessPeer(&can, device, peer_device));
  if (!can) {
    cb200_set_error("peer_enable: device %d cannot address device %d", device, peer_device);
    return CB200_ERR_UNSUPPORTED;
  }
  cudaError_t err = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (err == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); return CB200_OK; }
  CB_CUDA(err);
  return CB200_OK;
}

int cb200_ipc_export(int device, void* device_ptr, unsigned char* handle_out) {
  CB_REQUIRE(device_ptr && handle_out, "ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == CB200_IPC_HANDLE_BYTES, "IPC handle size");
  DeviceGuard g(device);
  cudaIpcMemHandle_t h;
  CB_CUDA(cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle_out, &h, sizeof(h));
  return CB200_OK;
}

int cb200_ipc_import(int device, const unsigned char* handle, void** ptr_out) {
  CB_REQUIRE(handle && ptr_out, "ipc_import: null argument");
  DeviceGuard g(device);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  CB_CUDA(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return CB200_OK;
}

int cb200_ipc_close(int device, void* ptr) {
  if (!ptr) return CB200_OK;
  DeviceGuard g(device);
  CB_CUDA(cudaIpcCloseMemHandle(ptr));
  return CB200_OK;
}

int cb200_event_record(cb200_stream* s, int timing, cb200_event** out) {
  CB_REQUIRE(s && out, "event_record: null argument");
  DeviceGuard g(s->device);
  cb200_event* e = new (std::nothrow) cb200_event();
  if (!e) { cb200_set_error("event_record: out of host memory"); return CB200_ERR_NOMEM; }
  e->device = s->device;
  e->stream = s;
  cudaError_t err = cudaEventCreateWithFlags(&e->ev, timing ? cudaEventDefault : cudaEventDisableTiming);
  if (err == cudaSuccess) err = cudaEventRecord(e->ev, s->stream);
  if (err != cudaSuccess) { delete e; return cb200_cuda_fail(err, "event_record", __FILE__, __LINE__); }
  *out = e;
  return CB200_OK;
}

int cb200_stream_wait_event(cb200_stream* s, cb200_event* e) {
  CB_REQUIRE(s && e, "stream_wait_event: null argument");
  DeviceGuard g(s->device);
  CB_CUDA(cudaStreamWaitEvent(s->stream, e->ev, 0));
  return CB200_OK;
}

int cb200_event_wait(cb200_event* e) {
  CB_REQUIRE(e, "event_wait: null event");
  DeviceGuard g(e->device);
  CB_CUDA(cudaEventSynchronize(e->ev));
  return CB200_OK;
}

int cb200_event_elapsed_ms(cb200_event* start, cb200_event* stop, float* ms) {
  CB_REQUIRE(start && stop && ms, "event_elapsed_ms: null argument");
  DeviceGuard g(start->device);
  CB_CUDA(cudaEventElapsedTime(ms, start->ev, stop->ev));
  return CB200_OK;
}

int cb200_event_destroy(cb200_event* e) {
  if (!e) return CB200_OK;
  DeviceGuard g(e->device);
  cudaEventDestroy(e->ev);
  delete e;
  return CB200_OK;
}

int cb200_stream_sync(cb200_stream* s) {
  CB_REQUIRE(s, "stream_sync: null stream");
  DeviceGuard g(s->device);
  CB_CUDA(cudaStreamSynchronize(s->stream));
  int code = 0, detail = 0;
  int rc = cb200_stream_status(s, &code, &detail);
  if (rc != CB200_OK) return rc;
  if (code != 0) {
    cb200_set_error("device-side status %d (detail %d): a bounded wait ran out or a kernel rejected its arguments",
                    code, detail);
    return code == CB200_ERR_TIMEOUT ? CB200_ERR_TIMEOUT : CB200_ERR_CUDA;
  }
  return CB200_OK;
}

}  // extern "C"
