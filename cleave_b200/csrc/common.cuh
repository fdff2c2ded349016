// Shared internals of libcleave_cuda: context, handle table, error channel, launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/cleave_cuda.h"

namespace cleave {

enum { DT_F32 = 0, DT_F64 = 1 };

// One device tensor: dense row-major, `len` elements of `dtype` at `ptr` (f64 entry points cast).
struct Buf {
  uint32_t magic;   // kMagic while live
  float* ptr;
  int64_t len;
  int64_t cap_bytes;  // pool block size; 0 for a non-owning view
  // Asynchronous transfers (copy-engine streams): xfer_ev marks the end of the last such copy
  // touching this tensor; while xfer_pending the next compute op that uses the handle first makes
  // the compute stream wait for it.  order_ev is scratch for ordering a copy after compute work.
  cudaEvent_t xfer_ev;
  cudaEvent_t order_ev;
  bool xfer_pending;
  int dtype;          // DT_F32 or DT_F64
};
constexpr uint32_t kMagic = 0xC1EA7E5Bu;

// Device-visible status word: kernels with bounded waits record a non-zero code here
// (pinned, mapped host memory), the host checks it at every synchronisation point.
struct DeviceStatus {
  int code;       // 0 = fine
  int where;      // kernel-specific location id
  int block;      // blockIdx.x of the reporter
  int detail;
};

struct Context {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;      // stream in use (own or caller's)
  DeviceStatus* status_host = nullptr;
  DeviceStatus* status_dev = nullptr;
  float* scalar_host = nullptr;       // pinned, mapped landing area for scalar results (64 floats)
  float* scalar_dev = nullptr;        // device alias of scalar_host: kernels write results straight to the host
  cudaStream_t side_stream = nullptr; // library-owned; used only between side_fork() and side_join()
  cudaEvent_t side_fork_ev = nullptr, side_join_ev = nullptr;
};

Context& ctx();

// ---- error channel -------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);   // records and returns `code`
bool ensure_init();                              // lazily initialises device 0 (or CLEAVE_CUDA_DEVICE)
bool cuda_ok(cudaError_t e, const char* what);   // records CLEAVE_CUDA_ERR_CUDA on failure
int check_device_status();                       // after a sync: translate the status word

// Every extern "C" entry point holds this lock for its whole body.
std::recursive_mutex& api_mutex();
struct ApiLock {
  std::lock_guard<std::recursive_mutex> g;
  ApiLock() : g(api_mutex()) {}
};

// ---- handles and memory ---------------------------------------------------------------
Buf* new_buf(int64_t len, int dtype = DT_F32);   // pooled device allocation; nullptr + error on failure
// Validates the handle and its element type, settles a pending async transfer; nullptr + error on failure.
Buf* as_buf(cleave_buf h, const char* what, int dtype = DT_F32);
Buf* lookup_buf(cleave_buf h, const char* what);   // validates liveness only
double* scalar_slot_f64();   // like scalar_slot(), for f64 results; read back with wait_scalar_f64()
double wait_scalar_f64();
void release_buf(Buf* b);
float* scratch_alloc(int64_t bytes);   // pooled scratch (stream-ordered reuse); pair with scratch_free
void scratch_free(float* p);
void count_launch(int n = 1);
bool noalloc_poke_completion_word(unsigned long long value);   // test hook: overwrite sum_noalloc's completion word

// Reads one f32 produced on the device at `dev_scalar`: copies to pinned memory, syncs,
// checks the status word.  Returns NaN on failure.
float read_scalar(const float* dev_scalar);
// Scalar results without a copy: a kernel writes the value to scalar_slot() (mapped host memory),
// wait_scalar() synchronises the stream, checks the status word and returns it (NaN on failure).
float* scalar_slot();
float wait_scalar();

// ---- a second queue inside one call ---------------------------------------------------------------
// side_fork() returns a library-owned stream that is ordered after everything queued on ctx().stream so far;
// side_join() orders ctx().stream after everything queued on that stream.  An entry point that has two
// independent kernels to run (a product that leaves SMs idle and a streaming pass) queues one on each between the two
// calls; to its caller all of it is ordered on ctx().stream as usual, so the pool's stream-ordered reuse stays valid:
// whatever is queued after the call follows the join.  Works while a graph is being captured (the side stream joins
// the capture through the fork event).  nullptr / false + error on failure.
cudaStream_t side_fork();
bool side_join();
// Column sums x[rows, cols] -> out[cols] on `stream` (reduce.cu).
bool colsum_launch(const float* x, float* out, int rows, int cols, cudaStream_t stream);

// ---- optional per-kernel timing -------------------------------------------------------------------
// Between profile_begin() and profile_end() every profile_mark(true) / profile_mark(false) pair
// records a CUDA event pair on the launching stream around the kernels in between (the tensor-core
// GEMM kernel, the linear-regression sweep); profile_end() waits for them and returns the summed
// duration in milliseconds and the number of pairs.  Outside begin/end the marks cost nothing.
void profile_begin();
double profile_end(int* pairs);
void profile_mark(bool begin);

// ---- optional call trace --------------------------------------------------------------------------
// With CLEAVE_CUDA_TRACE=1 in the environment every traced entry point prints one line to stderr when it
// returns: operation, shape, and the device time of what it queued (a CUDA event pair on the library's
// stream; the call then waits for its own work, so a traced run is serialised).  Nested scopes (an entry
// point implemented through another) print only the outermost.  Without the variable a Trace costs one
// load and a branch.
struct Trace {
  bool on;
  char text[120];
  Trace(const char* op, const char* fmt, ...);
  ~Trace();
};

// ---- launch geometry -------------------------------------------------------------------
inline int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// Grid for a grid-stride streaming kernel: enough CTAs for the work, capped at a multiple
// of the SM count so every SM holds the same number of resident CTAs.
inline int stream_grid(int64_t work_items, int threads, int ctas_per_sm) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)ctx().sm_count * ctas_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace cleave
