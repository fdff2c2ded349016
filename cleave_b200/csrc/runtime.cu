// Runtime half of libcleave_cuda: device context, pooled allocator, handle table, transfers,
// error channel.  Plays the part cleave_alloc / cleave_realloc / dynarray_* play in the
// reference runtime (cleave-rt/src/lib.rs:56-71, :146-213), for device memory.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

#include "common.cuh"

namespace cleave {

static std::recursive_mutex g_mu;
static Context g_ctx;
static std::unordered_set<Buf*> g_live;
typedef std::unordered_map<int64_t, std::vector<void*>> BlockCache;       // block size -> cached blocks
static BlockCache g_free_blocks;
// The cache allocations are served from.  While a step is being captured into a CUDA graph this points at the
// graph's private cache, so the captured kernels only ever name blocks that stay reserved for the graph.
static BlockCache* g_pool = &g_free_blocks;

// A captured step: the instantiated graph and the device blocks its kernels point at.
struct StepGraph {
  uint32_t magic;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  BlockCache blocks;
};
constexpr uint32_t kGraphMagic = 0x6EA9C1EAu;
static StepGraph* g_capturing = nullptr;
static std::unordered_set<StepGraph*> g_graphs;
static std::unordered_map<void*, int64_t> g_scratch_sizes;
static int64_t g_live_bytes = 0;
static int64_t g_cached_bytes = 0;
static int64_t g_launches = 0;

static thread_local int t_err_code = 0;
static thread_local char t_err_msg[512] = "";

Context& ctx() { return g_ctx; }
std::recursive_mutex& api_mutex() { return g_mu; }

int set_error(int code, const char* fmt, ...) {
  t_err_code = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err_msg, sizeof(t_err_msg), fmt, ap);
  va_end(ap);
  const char* abort_env = getenv("CLEAVE_CUDA_ABORT_ON_ERROR");
  if (abort_env && abort_env[0] == '1') {
    fprintf(stderr, "libcleave_cuda: fatal: %s\n", t_err_msg);
    abort();
  }
  return code;
}

bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  set_error(CLEAVE_CUDA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return false;
}

static bool init_device(int device) {
  if (g_ctx.ready && (device < 0 || device == g_ctx.device)) return true;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    set_error(CLEAVE_CUDA_ERR_NO_DEVICE, "no CUDA device available (%s); this library has no CPU fallback",
              e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    return false;
  }
  if (device < 0) {
    const char* env = getenv("CLEAVE_CUDA_DEVICE");
    device = env ? atoi(env) : 0;
  }
  if (device >= count) {
    set_error(CLEAVE_CUDA_ERR_ARG, "device %d requested but only %d present", device, count);
    return false;
  }
  if (g_ctx.ready) {
    set_error(CLEAVE_CUDA_ERR_ARG, "already initialised on device %d; one device per process", g_ctx.device);
    return false;
  }
  if (!cuda_ok(cudaSetDevice(device), "cudaSetDevice")) return false;
  cudaDeviceProp prop;
  if (!cuda_ok(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return false;
  if (prop.major != 10) {
    set_error(CLEAVE_CUDA_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
              prop.major, prop.minor);
    return false;
  }
  g_ctx.device = device;
  g_ctx.sm_count = prop.multiProcessorCount;
  if (!cuda_ok(cudaStreamCreateWithFlags(&g_ctx.own_stream, cudaStreamNonBlocking), "cudaStreamCreate")) return false;
  g_ctx.stream = g_ctx.own_stream;
  if (!cuda_ok(cudaHostAlloc((void**)&g_ctx.status_host, sizeof(DeviceStatus), cudaHostAllocMapped), "cudaHostAlloc"))
    return false;
  memset(g_ctx.status_host, 0, sizeof(DeviceStatus));
  if (!cuda_ok(cudaHostGetDevicePointer((void**)&g_ctx.status_dev, g_ctx.status_host, 0), "cudaHostGetDevicePointer"))
    return false;
  if (!cuda_ok(cudaHostAlloc((void**)&g_ctx.scalar_host, 64 * sizeof(float), cudaHostAllocMapped), "cudaHostAlloc"))
    return false;
  if (!cuda_ok(cudaHostGetDevicePointer((void**)&g_ctx.scalar_dev, g_ctx.scalar_host, 0), "cudaHostGetDevicePointer"))
    return false;
  g_ctx.ready = true;
  return true;
}

bool ensure_init() {
  if (g_ctx.ready) {
    // Calls may arrive on a host thread that never selected the device.
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur != g_ctx.device) cudaSetDevice(g_ctx.device);
    return true;
  }
  return init_device(-1);
}

int check_device_status() {
  if (!g_ctx.status_host) return CLEAVE_CUDA_OK;
  DeviceStatus s = *g_ctx.status_host;
  if (s.code == 0) return CLEAVE_CUDA_OK;
  memset(g_ctx.status_host, 0, sizeof(DeviceStatus));
  return set_error(CLEAVE_CUDA_ERR_DEVICE_TIMEOUT,
                   "a kernel gave up a bounded wait (code %d, location %d, block %d, detail %d); "
                   "results of the queued work are invalid",
                   s.code, s.where, s.block, s.detail);
}

void count_launch(int n) { g_launches += n; }

// ---- call trace (CLEAVE_CUDA_TRACE=1) -------------------------------------------------------------------
static int g_trace_mode = -1;     // -1: environment not read yet
static int g_trace_depth = 0;
static cudaEvent_t g_trace_ev[2] = {nullptr, nullptr};

Trace::Trace(const char* op, const char* fmt, ...) : on(false) {
  if (g_trace_mode < 0) {
    const char* e = getenv("CLEAVE_CUDA_TRACE");
    g_trace_mode = (e && e[0] == '1') ? 1 : 0;
  }
  if (!g_trace_mode || !g_ctx.ready) return;
  if (g_capturing) {   // a capture records work, it does not run it: nothing to time
    ++g_trace_depth;
    return;
  }
  if (g_trace_depth++ > 0) return;
  if (!g_trace_ev[0] && (cudaEventCreate(&g_trace_ev[0]) != cudaSuccess || cudaEventCreate(&g_trace_ev[1]) != cudaSuccess)) {
    cudaGetLastError();
    g_trace_ev[0] = nullptr;
    return;
  }
  int n = snprintf(text, sizeof(text), "%-16s ", op);
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(text + n, sizeof(text) - (size_t)n, fmt, ap);
  va_end(ap);
  on = cudaEventRecord(g_trace_ev[0], g_ctx.stream) == cudaSuccess;
}

Trace::~Trace() {
  if (!g_trace_mode || !g_ctx.ready) return;
  if (--g_trace_depth > 0 || !on) return;
  float ms = 0.f;
  if (cudaEventRecord(g_trace_ev[1], g_ctx.stream) == cudaSuccess && cudaEventSynchronize(g_trace_ev[1]) == cudaSuccess &&
      cudaEventElapsedTime(&ms, g_trace_ev[0], g_trace_ev[1]) == cudaSuccess)
    fprintf(stderr, "cleave_cuda trace: %s  %.1f us\n", text, ms * 1e3);
  else
    cudaGetLastError();
}

// ---- guard words behind every pool block (CLEAVE_CUDA_DEBUG=1) ----------------------------------------------
// In debug mode each block handed out by the pool is followed by kGuardBytes of a fixed pattern, written when the
// block is handed out and compared when it comes back: a kernel that wrote past the end of a tensor or of a
// scratch buffer is reported (error code CLEAVE_CUDA_ERR_CUDA, message naming the block) at the free that
// follows it.  The check waits for the stream, so a debug run is slow; nothing changes without the variable.
constexpr int64_t kGuardBytes = 512;
constexpr unsigned char kGuardByte = 0xA5;
static int g_debug_mode = -1;
static int64_t g_guard_failures = 0;
static bool debug_mode() {
  if (g_debug_mode < 0) {
    const char* e = getenv("CLEAVE_CUDA_DEBUG");
    g_debug_mode = (e && e[0] == '1') ? 1 : 0;
  }
  return g_debug_mode == 1;
}
static void guard_arm(void* block, int64_t bs) {
  if (debug_mode()) cudaMemsetAsync((char*)block + bs, kGuardByte, (size_t)kGuardBytes, g_ctx.stream);
}
static void guard_check(void* block, int64_t bs) {
  if (!debug_mode()) return;
  unsigned char host[kGuardBytes];
  if (cudaMemcpyAsync(host, (char*)block + bs, (size_t)kGuardBytes, cudaMemcpyDeviceToHost, g_ctx.stream) != cudaSuccess ||
      cudaStreamSynchronize(g_ctx.stream) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  for (int64_t i = 0; i < kGuardBytes; ++i)
    if (host[i] != kGuardByte) {
      ++g_guard_failures;
      set_error(CLEAVE_CUDA_ERR_CUDA, "debug: %lld-byte block at %p was overrun (guard byte %lld behind its end changed)",
                (long long)bs, block, (long long)i);
      fprintf(stderr, "libcleave_cuda: %s\n", t_err_msg);
      return;
    }
}

// ---- pool ----------------------------------------------------------------------------
static int64_t block_size_for(int64_t bytes) {
  if (bytes < 512) bytes = 512;
  if (bytes <= (1 << 20)) {
    int64_t b = 512;
    while (b < bytes) b <<= 1;
    return b;
  }
  const int64_t g = 2 << 20;
  return (bytes + g - 1) / g * g;
}

static void* pool_alloc(int64_t bytes, int64_t* block_bytes) {
  int64_t bs = block_size_for(bytes);
  *block_bytes = bs;
  auto it = g_pool->find(bs);
  if (it != g_pool->end() && !it->second.empty()) {
    void* p = it->second.back();
    it->second.pop_back();
    if (!g_capturing) g_cached_bytes -= bs;
    guard_arm(p, bs);
    return p;
  }
  const size_t real = (size_t)bs + (debug_mode() ? (size_t)kGuardBytes : 0);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, real);
  if (e != cudaSuccess && !g_capturing) {
    // Give cached blocks back to the driver and retry once.
    cudaGetLastError();
    cudaStreamSynchronize(g_ctx.stream);
    for (auto& kv : g_free_blocks) {
      for (void* q : kv.second) cudaFree(q);
      kv.second.clear();
    }
    g_cached_bytes = 0;
    e = cudaMalloc(&p, real);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(CLEAVE_CUDA_ERR_OOM, "device allocation of %lld bytes failed: %s", (long long)bs, cudaGetErrorString(e));
    return nullptr;
  }
  guard_arm(p, bs);
  return p;
}

// Blocks go straight back to the free list: all work of this library runs on one stream,
// so a later user of the block is ordered after every kernel that touched it.
static void pool_free(void* p, int64_t block_bytes) {
  if (!g_capturing) guard_check(p, block_bytes);   // the check waits for the stream, which a capture cannot do
  (*g_pool)[block_bytes].push_back(p);
  if (!g_capturing) g_cached_bytes += block_bytes;
}

Buf* new_buf(int64_t len, int dtype) {
  if (len <= 0) {
    set_error(CLEAVE_CUDA_ERR_ARG, "tensor length must be positive, got %lld", (long long)len);
    return nullptr;
  }
  if (!ensure_init()) return nullptr;
  int64_t bs = 0;
  void* p = pool_alloc(len * (int64_t)(dtype == DT_F64 ? sizeof(double) : sizeof(float)), &bs);
  if (!p) return nullptr;
  Buf* b = new Buf{kMagic, (float*)p, len, bs, nullptr, nullptr, false, dtype};
  g_live.insert(b);
  g_live_bytes += bs;
  return b;
}

Buf* lookup_buf(cleave_buf h, const char* what) {
  Buf* b = (Buf*)h;
  if (!b || g_live.find(b) == g_live.end() || b->magic != kMagic) {
    set_error(CLEAVE_CUDA_ERR_BAD_HANDLE, "%s: not a live tensor handle (%p)", what, (void*)h);
    return nullptr;
  }
  return b;
}

static void settle_transfer(Buf* b) {
  if (b->xfer_pending) {
    cudaStreamWaitEvent(g_ctx.stream, b->xfer_ev, 0);   // compute stream continues after the copy
    b->xfer_pending = false;
  }
}

Buf* as_buf(cleave_buf h, const char* what, int dtype) {
  Buf* b = lookup_buf(h, what);
  if (!b) return nullptr;
  if (b->dtype != dtype) {
    set_error(CLEAVE_CUDA_ERR_ARG, "%s: tensor holds %s elements, this entry point works on %s", what,
              b->dtype == DT_F64 ? "f64" : "f32", dtype == DT_F64 ? "f64" : "f32");
    return nullptr;
  }
  settle_transfer(b);
  return b;
}

void release_buf(Buf* b) {
  settle_transfer(b);   // the block returns to the pool in compute-stream order, after any copy in flight
  if (b->xfer_ev) cudaEventDestroy(b->xfer_ev);
  if (b->order_ev) cudaEventDestroy(b->order_ev);
  g_live.erase(b);
  if (b->cap_bytes) {
    pool_free(b->ptr, b->cap_bytes);
    g_live_bytes -= b->cap_bytes;
  }
  b->magic = 0;
  delete b;
}

float* scratch_alloc(int64_t bytes) {
  if (!ensure_init()) return nullptr;
  int64_t bs = 0;
  void* p = pool_alloc(bytes, &bs);
  if (p) g_scratch_sizes[p] = bs;
  return (float*)p;
}

void scratch_free(float* p) {
  if (!p) return;
  auto it = g_scratch_sizes.find(p);
  if (it == g_scratch_sizes.end()) return;
  pool_free(p, it->second);
  g_scratch_sizes.erase(it);
}

float read_scalar(const float* dev_scalar) {
  Context& c = g_ctx;
  if (!cuda_ok(cudaMemcpyAsync(c.scalar_host, dev_scalar, sizeof(float), cudaMemcpyDeviceToHost, c.stream),
               "cudaMemcpyAsync(scalar)"))
    return NAN;
  if (!cuda_ok(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize")) return NAN;
  if (check_device_status() != CLEAVE_CUDA_OK) return NAN;
  return c.scalar_host[0];
}

static bool g_profiling = false;
static std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_prof_events;
static size_t g_prof_used = 0;

cudaStream_t side_fork() {
  Context& c = g_ctx;
  if (!c.side_stream) {
    if (!cuda_ok(cudaStreamCreateWithFlags(&c.side_stream, cudaStreamNonBlocking), "cudaStreamCreate(side)") ||
        !cuda_ok(cudaEventCreateWithFlags(&c.side_fork_ev, cudaEventDisableTiming), "cudaEventCreate(fork)") ||
        !cuda_ok(cudaEventCreateWithFlags(&c.side_join_ev, cudaEventDisableTiming), "cudaEventCreate(join)"))
      return nullptr;
  }
  if (!cuda_ok(cudaEventRecord(c.side_fork_ev, c.stream), "cudaEventRecord(fork)") ||
      !cuda_ok(cudaStreamWaitEvent(c.side_stream, c.side_fork_ev, 0), "cudaStreamWaitEvent(fork)"))
    return nullptr;
  return c.side_stream;
}

bool side_join() {
  Context& c = g_ctx;
  return cuda_ok(cudaEventRecord(c.side_join_ev, c.side_stream), "cudaEventRecord(join)") &&
         cuda_ok(cudaStreamWaitEvent(c.stream, c.side_join_ev, 0), "cudaStreamWaitEvent(join)");
}

void profile_mark(bool begin) {
  if (!g_profiling) return;
  if (begin) {
    if (g_prof_used == g_prof_events.size()) {
      cudaEvent_t a, b;
      if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) {
        cudaGetLastError();
        return;
      }
      g_prof_events.emplace_back(a, b);
    }
    cudaEventRecord(g_prof_events[g_prof_used].first, g_ctx.stream);
  } else if (g_prof_used < g_prof_events.size()) {
    cudaEventRecord(g_prof_events[g_prof_used].second, g_ctx.stream);
    ++g_prof_used;
  }
}

void profile_begin() {
  g_profiling = true;
  g_prof_used = 0;
}

double profile_end(int* pairs) {
  double total = 0.0;
  g_profiling = false;
  for (size_t i = 0; i < g_prof_used; ++i) {
    float ms = 0.f;
    if (cudaEventSynchronize(g_prof_events[i].second) == cudaSuccess &&
        cudaEventElapsedTime(&ms, g_prof_events[i].first, g_prof_events[i].second) == cudaSuccess)
      total += ms;
    else
      cudaGetLastError();
  }
  if (pairs) *pairs = (int)g_prof_used;
  g_prof_used = 0;
  return total;
}

float* scalar_slot() { return g_ctx.scalar_dev + 1; }   // slot 0 is read_scalar's copy target

double* scalar_slot_f64() { return reinterpret_cast<double*>(g_ctx.scalar_dev + 2); }   // 8-byte aligned

double wait_scalar_f64() {
  Context& c = g_ctx;
  if (!cuda_ok(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize")) return NAN;
  if (check_device_status() != CLEAVE_CUDA_OK) return NAN;
  return *reinterpret_cast<volatile double*>(c.scalar_host + 2);
}

float wait_scalar() {
  Context& c = g_ctx;
  if (!cuda_ok(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize")) return NAN;
  if (check_device_status() != CLEAVE_CUDA_OK) return NAN;
  return ((volatile float*)c.scalar_host)[1];
}

}  // namespace cleave

using namespace cleave;

extern "C" {

int32_t cleave_cuda_init(int32_t device) {
  ApiLock lock;
  return init_device(device) ? CLEAVE_CUDA_OK : t_err_code;
}

int32_t cleave_cuda_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int32_t cleave_cuda_last_error(void) { return t_err_code; }
const char* cleave_cuda_last_error_message(void) { return t_err_msg; }
void cleave_cuda_clear_error(void) {
  t_err_code = 0;
  t_err_msg[0] = 0;
}

int32_t cleave_cuda_sync(void) {
  ApiLock lock;
  if (!ensure_init()) return t_err_code;
  if (!cuda_ok(cudaStreamSynchronize(g_ctx.stream), "cudaStreamSynchronize")) return t_err_code;
  return check_device_status();
}

void cleave_cuda_set_stream(void* s) {
  ApiLock lock;
  if (!ensure_init()) return;
  // Order the new stream after everything queued so far, so pooled blocks stay safe to reuse.
  cudaStreamSynchronize(g_ctx.stream);
  g_ctx.stream = s ? (cudaStream_t)s : g_ctx.own_stream;
}

void* cleave_cuda_get_stream(void) {
  ApiLock lock;
  if (!ensure_init()) return nullptr;
  return (void*)g_ctx.stream;
}

void cleave_cuda_reset(void) {
  ApiLock lock;
  std::vector<Buf*> all(g_live.begin(), g_live.end());
  for (Buf* b : all) release_buf(b);
}

void cleave_cuda_trim(void) {
  ApiLock lock;
  if (!g_ctx.ready) return;
  cudaStreamSynchronize(g_ctx.stream);
  for (auto& kv : g_free_blocks) {
    for (void* q : kv.second) cudaFree(q);
    kv.second.clear();
  }
  g_cached_bytes = 0;
}

int64_t cleave_cuda_live_bytes(void) {
  ApiLock lock;
  return g_live_bytes;
}

void cleave_cuda_profile_begin(void) {
  ApiLock lock;
  profile_begin();
}

double cleave_cuda_profile_end(int32_t* launches) {
  ApiLock lock;
  int n = 0;
  double ms = profile_end(&n);
  if (launches) *launches = n;
  return ms;
}

int64_t cleave_cuda_kernel_launches(void) {
  ApiLock lock;
  return g_launches;
}

int64_t cleave_cuda_test_hook(int32_t what, int64_t arg) {
  ApiLock lock;
  if (!ensure_init()) return -t_err_code;
  switch (what) {
    case CLEAVE_HOOK_SET_DEVICE_STATUS:
      // what a kernel does when a bounded wait runs out, done from the host
      g_ctx.status_host->where = 9000;
      g_ctx.status_host->block = 0;
      g_ctx.status_host->detail = 0;
      g_ctx.status_host->code = (int)arg;
      return 0;
    case CLEAVE_HOOK_POISON_NOALLOC_WORD:
      return noalloc_poke_completion_word((unsigned long long)arg) ? 0 : -t_err_code;
    case CLEAVE_HOOK_GUARD_FAILURES:
      return g_guard_failures;
    default:
      return -set_error(CLEAVE_CUDA_ERR_ARG, "test_hook: unknown selector %d", what);
  }
}

int32_t cleave_cuda_graph_begin(void) {
  ApiLock lock;
  if (!ensure_init()) return -t_err_code;
  if (g_capturing) return -set_error(CLEAVE_CUDA_ERR_ARG, "graph_begin: a capture is already open");
  // Relaxed mode: the pool may call cudaMalloc for a block the graph's private cache does not hold yet.
  if (!cuda_ok(cudaStreamBeginCapture(g_ctx.stream, cudaStreamCaptureModeRelaxed), "cudaStreamBeginCapture"))
    return -t_err_code;
  g_capturing = new StepGraph();
  g_capturing->magic = kGraphMagic;
  g_pool = &g_capturing->blocks;
  return CLEAVE_CUDA_OK;
}

void* cleave_cuda_graph_end(void) {
  ApiLock lock;
  if (!g_capturing) {
    set_error(CLEAVE_CUDA_ERR_ARG, "graph_end: no capture is open");
    return nullptr;
  }
  StepGraph* g = g_capturing;
  g_capturing = nullptr;
  g_pool = &g_free_blocks;
  bool ok = cuda_ok(cudaStreamEndCapture(g_ctx.stream, &g->graph), "cudaStreamEndCapture") && g->graph != nullptr &&
            cuda_ok(cudaGraphInstantiate(&g->exec, g->graph, 0), "cudaGraphInstantiate");
  if (!ok) {
    if (t_err_code == 0) set_error(CLEAVE_CUDA_ERR_CUDA, "graph_end: the capture produced no graph");
    if (g->graph) cudaGraphDestroy(g->graph);
    for (auto& kv : g->blocks)
      for (void* q : kv.second) cudaFree(q);
    delete g;
    cudaGetLastError();
    return nullptr;
  }
  g_graphs.insert(g);
  return (void*)g;
}

static StepGraph* as_graph(void* h, const char* what) {
  StepGraph* g = (StepGraph*)h;
  if (!g || g_graphs.find(g) == g_graphs.end() || g->magic != kGraphMagic) {
    set_error(CLEAVE_CUDA_ERR_BAD_HANDLE, "%s: not a live graph handle (%p)", what, h);
    return nullptr;
  }
  return g;
}

int32_t cleave_cuda_graph_launch(void* graph) {
  ApiLock lock;
  StepGraph* g = as_graph(graph, "graph_launch");
  if (!g) return -t_err_code;
  if (g_capturing) return -set_error(CLEAVE_CUDA_ERR_ARG, "graph_launch: a capture is open");
  if (!cuda_ok(cudaGraphLaunch(g->exec, g_ctx.stream), "cudaGraphLaunch")) return -t_err_code;
  return CLEAVE_CUDA_OK;
}

void cleave_cuda_graph_free(void* graph) {
  ApiLock lock;
  StepGraph* g = as_graph(graph, "graph_free");
  if (!g) return;
  cudaStreamSynchronize(g_ctx.stream);
  cudaGraphExecDestroy(g->exec);
  cudaGraphDestroy(g->graph);
  for (auto& kv : g->blocks)
    for (void* q : kv.second) cudaFree(q);
  g_graphs.erase(g);
  g->magic = 0;
  delete g;
}

void* cleave_cuda_host_alloc(int64_t bytes) {
  ApiLock lock;
  if (bytes <= 0) {
    set_error(CLEAVE_CUDA_ERR_ARG, "host_alloc: bytes must be positive");
    return nullptr;
  }
  if (!ensure_init()) return nullptr;
  void* p = nullptr;
  cudaError_t e = cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocDefault);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(CLEAVE_CUDA_ERR_OOM, "pinned host allocation of %lld bytes failed: %s", (long long)bytes,
              cudaGetErrorString(e));
    return nullptr;
  }
  return p;
}

void cleave_cuda_host_free(void* p) {
  ApiLock lock;
  if (p && g_ctx.ready) cudaFreeHost(p);
}

cleave_buf cleave_cuda_none(void) { return nullptr; }

cleave_buf cleave_cuda_alloc_f32(int64_t len) {
  ApiLock lock;
  return (cleave_buf)new_buf(len);
}

int32_t cleave_cuda_upload_into_f32(cleave_buf t, const float* host, int64_t len) {
  ApiLock lock;
  Buf* b = as_buf(t, "upload_into");
  if (!b) return -t_err_code;
  if (!host || len != b->len) return -set_error(CLEAVE_CUDA_ERR_SHAPE, "upload_into: %lld elements given, tensor has %lld",
                                                (long long)len, (long long)b->len);
  Trace tr("upload_into", "n=%lld", (long long)len);
  if (!cuda_ok(cudaMemcpyAsync(b->ptr, host, (size_t)len * sizeof(float), cudaMemcpyHostToDevice, g_ctx.stream),
               "cudaMemcpyAsync(H2D)"))
    return -t_err_code;
  return CLEAVE_CUDA_OK;
}

cleave_buf cleave_cuda_upload_f32(const float* host, int64_t len) {
  ApiLock lock;
  if (!host) {
    set_error(CLEAVE_CUDA_ERR_ARG, "upload: NULL host pointer");
    return nullptr;
  }
  Buf* b = new_buf(len);
  if (!b) return nullptr;
  Trace tr("upload", "n=%lld", (long long)len);
  if (!cuda_ok(cudaMemcpyAsync(b->ptr, host, (size_t)len * sizeof(float), cudaMemcpyHostToDevice, g_ctx.stream),
               "cudaMemcpyAsync(H2D)")) {
    release_buf(b);
    return nullptr;
  }
  // The caller's array may be a temporary (cleave passes a stack array): finish the copy
  // before returning unless the source is pinned memory, which this call cannot know, so
  // always wait.  Pinned sources still get the full-bandwidth DMA path.
  if (!cuda_ok(cudaStreamSynchronize(g_ctx.stream), "cudaStreamSynchronize")) {
    release_buf(b);
    return nullptr;
  }
  return (cleave_buf)b;
}

int64_t cleave_cuda_download_f32(cleave_buf t, float* host, int64_t len) {
  ApiLock lock;
  Buf* b = as_buf(t, "download");
  if (!b) return -t_err_code;
  if (!host || len != b->len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "download: room for %lld elements, tensor has %lld", (long long)len,
                      (long long)b->len);
  Trace tr("download", "n=%lld", (long long)len);
  if (!cuda_ok(cudaMemcpyAsync(host, b->ptr, (size_t)len * sizeof(float), cudaMemcpyDeviceToHost, g_ctx.stream),
               "cudaMemcpyAsync(D2H)"))
    return -t_err_code;
  if (!cuda_ok(cudaStreamSynchronize(g_ctx.stream), "cudaStreamSynchronize")) return -t_err_code;
  if (check_device_status() != CLEAVE_CUDA_OK) return -t_err_code;
  return len;
}

// ---- asynchronous transfers on the copy engines ------------------------------------------------
static cudaStream_t g_h2d_stream = nullptr, g_d2h_stream = nullptr;

static bool transfer_ready(Buf* b) {
  if (!g_h2d_stream) {
    if (!cuda_ok(cudaStreamCreateWithFlags(&g_h2d_stream, cudaStreamNonBlocking), "cudaStreamCreate(h2d)")) return false;
    if (!cuda_ok(cudaStreamCreateWithFlags(&g_d2h_stream, cudaStreamNonBlocking), "cudaStreamCreate(d2h)")) return false;
  }
  if (!b->xfer_ev) {
    if (!cuda_ok(cudaEventCreateWithFlags(&b->xfer_ev, cudaEventDisableTiming), "cudaEventCreate")) return false;
    if (!cuda_ok(cudaEventCreateWithFlags(&b->order_ev, cudaEventDisableTiming), "cudaEventCreate")) return false;
  }
  return true;
}

// Queues `copy` on `xs` after (a) all compute work queued so far and (b) any earlier async copy
// touching the same tensor, and leaves the tensor marked so that later compute waits for it.
static int32_t async_transfer(Buf* b, cudaStream_t xs, void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
  if (!cuda_ok(cudaEventRecord(b->order_ev, g_ctx.stream), "cudaEventRecord")) return -t_err_code;
  cudaStreamWaitEvent(xs, b->order_ev, 0);
  if (b->xfer_pending) cudaStreamWaitEvent(xs, b->xfer_ev, 0);
  if (!cuda_ok(cudaMemcpyAsync(dst, src, bytes, kind, xs), "cudaMemcpyAsync(async transfer)")) return -t_err_code;
  if (!cuda_ok(cudaEventRecord(b->xfer_ev, xs), "cudaEventRecord")) return -t_err_code;
  b->xfer_pending = true;
  return CLEAVE_CUDA_OK;
}

int32_t cleave_cuda_upload_async_f32(cleave_buf t, const float* pinned_host, int64_t len) {
  ApiLock lock;
  Buf* b = lookup_buf(t, "upload_async");
  if (!b) return -t_err_code;
  if (!pinned_host || len != b->len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "upload_async: %lld elements given, tensor has %lld", (long long)len,
                      (long long)b->len);
  if (!transfer_ready(b)) return -t_err_code;
  return async_transfer(b, g_h2d_stream, b->ptr, pinned_host, (size_t)len * sizeof(float), cudaMemcpyHostToDevice);
}

int32_t cleave_cuda_download_async_f32(cleave_buf t, float* pinned_host, int64_t len) {
  ApiLock lock;
  Buf* b = lookup_buf(t, "download_async");
  if (!b) return -t_err_code;
  if (!pinned_host || len != b->len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "download_async: room for %lld elements, tensor has %lld", (long long)len,
                      (long long)b->len);
  if (!transfer_ready(b)) return -t_err_code;
  return async_transfer(b, g_d2h_stream, pinned_host, b->ptr, (size_t)len * sizeof(float), cudaMemcpyDeviceToHost);
}

int32_t cleave_cuda_transfers_sync(void) {
  ApiLock lock;
  if (!g_h2d_stream) return CLEAVE_CUDA_OK;
  if (!cuda_ok(cudaStreamSynchronize(g_h2d_stream), "cudaStreamSynchronize(h2d)")) return -t_err_code;
  if (!cuda_ok(cudaStreamSynchronize(g_d2h_stream), "cudaStreamSynchronize(d2h)")) return -t_err_code;
  return check_device_status() == CLEAVE_CUDA_OK ? CLEAVE_CUDA_OK : -t_err_code;
}

float cleave_cuda_get_f32(cleave_buf t, int64_t i) {
  ApiLock lock;
  Buf* b = as_buf(t, "get");
  if (!b) return NAN;
  if (i < 0 || i >= b->len) {
    set_error(CLEAVE_CUDA_ERR_ARG, "get: index %lld outside [0, %lld)", (long long)i, (long long)b->len);
    return NAN;
  }
  return read_scalar(b->ptr + i);
}

int64_t cleave_cuda_len(cleave_buf t) {
  ApiLock lock;
  Buf* b = lookup_buf(t, "len");
  return b ? b->len : -t_err_code;
}

void cleave_cuda_free(cleave_buf t) {
  ApiLock lock;
  Buf* b = lookup_buf(t, "free");
  if (b) release_buf(b);
}

cleave_buf cleave_cuda_wrap_f32(void* device_ptr, int64_t len) {
  ApiLock lock;
  if (!device_ptr || len <= 0 || ((uintptr_t)device_ptr & 3u)) {
    set_error(CLEAVE_CUDA_ERR_ARG, "wrap: need a 4-byte aligned device pointer and a positive length");
    return nullptr;
  }
  if (!ensure_init()) return nullptr;
  Buf* b = new Buf{kMagic, (float*)device_ptr, len, 0, nullptr, nullptr, false, DT_F32};
  g_live.insert(b);
  return (cleave_buf)b;
}

void* cleave_cuda_data_ptr(cleave_buf t) {
  ApiLock lock;
  Buf* b = lookup_buf(t, "data_ptr");
  if (b) as_buf(t, "data_ptr", b->dtype);   // orders the compute stream after a pending async transfer
  return b ? (void*)b->ptr : nullptr;
}

}  // extern "C"
