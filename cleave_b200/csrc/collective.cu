// Data-parallel SGD step as ONE kernel over NVLink / NVSwitch peer memory:
//   gradient sum over the G ranks  +  w -= lr * (sum / G)  +  replication of the new weights.
//
// Parameters and gradients of every rank live in symmetric memory (same size and layout on each
// GPU, every rank holds pointers to all peers' copies and, where the fabric supports it, one
// multicast address that reaches all of them through NVSwitch).  Rank r owns the r-th slice of
// the flat parameter vector.  For each 16-byte word of its slice it
//   multimem mode: reads the word SUMMED across all ranks in the switch (multimem.ld_reduce),
//                  updates it, and writes the new weights to all ranks at once (multimem.st);
//   peer mode:     loads the word from every rank's gradient buffer (plain peer loads, summed in
//                  rank order), updates it, and stores the result into every rank's parameters.
// Either way each gradient byte crosses NVLink once and each new weight once, there is no
// separate all-reduce, no packing pass and no second sweep for the update, and every replica
// receives bit-identical weights because one rank computes each element.
//
// The kernel carries its own cross-GPU barriers (signal words in symmetric memory, monotonic
// epochs, never reset): an entry barrier ("every rank's backward pass has finished writing its
// gradients") taken by CTA 0, which then releases the other CTAs, and an exit barrier ("every
// rank's writes have landed") taken by the last CTA to finish.  Every wait is bounded; a wait
// that gives up records a status code for the host and lets the kernel return.
//
// An entry barrier that gives up ABORTS the launch: CTA 0 tells every peer (an abort word in each
// rank's signal block) and its own CTAs (a local abort word published before the release), and no
// CTA then reads a gradient, writes a weight or waits at the exit barrier.  A rank that passes its own
// entry wait but finds a peer's abort mark for this epoch aborts as well.  So when a rank never
// arrives, every live rank returns with its weights exactly as they were; the host sees
// CLEAVE_CUDA_ERR_DEVICE_TIMEOUT at its next synchronisation.
//
// Ranks must be one process per GPU: kernels that wait on each other never share a GPU.
#include <cstdlib>

#include "common.cuh"

namespace cleave {

constexpr int kMaxRanks = 8;
constexpr int kDpThreads = 128;   // small CTAs: one fits beside a resident tensor-core GEMM CTA (registers)
constexpr unsigned long long kDpWaitLimitNs = 2000000000ull;   // 2 s across GPUs unless CLEAVE_CUDA_DP_WAIT_MS is set

// Signal-word layout inside each rank's flag buffer (uint32 words).
constexpr int kFlagFromRank = 0;    // [0, 8): last epoch signalled by rank s
constexpr int kFlagAbortFrom = 8;   // [8, 16): epoch of the last launch that rank s abandoned at its entry barrier
constexpr int kFlagGo = 16;         // CTA 0 -> other CTAs of the same launch
constexpr int kFlagDone = 17;       // CTAs finished in this launch
constexpr int kFlagAbort = 18;      // CTA 0 -> other CTAs: epoch of the last launch abandoned on this rank

struct DpArgs {
  float* params[kMaxRanks];         // every rank's parameter buffer (peer pointers)
  const float* grads[kMaxRanks];    // every rank's gradient buffer
  uint32_t* flags[kMaxRanks];       // every rank's signal words
  float* params_mc;                 // multicast address of the parameter buffers, or null
  const float* grads_mc;            // multicast address of the gradient buffers, or null
  int rank, world;
  int64_t word_lo, word_hi;         // this rank's slice, in 16-byte words
  float lr, gscale;
  uint32_t epoch;                   // entry barrier uses epoch, exit barrier epoch + 1
  unsigned long long wait_ns;       // limit of a cross-GPU wait; the CTAs' wait for CTA 0 gets twice that and a second
  DeviceStatus* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long dp_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Spin until *p has reached `want` (epochs only grow; the signed difference tolerates wrap-around).
template <bool kSys>
__device__ __forceinline__ bool wait_epoch(const uint32_t* p, uint32_t want, unsigned long long limit_ns) {
  const unsigned long long t0 = dp_timer_ns();
  uint32_t spins = 0;
  for (;;) {
    const uint32_t v = kSys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int32_t)(v - want) >= 0) return true;
    if ((++spins & 0x3Fu) == 0 && dp_timer_ns() - t0 > limit_ns) return false;
  }
}

__device__ __forceinline__ void dp_report(DeviceStatus* st, int code, int where, int detail) {
  volatile DeviceStatus* v = st;
  v->where = where;
  v->block = blockIdx.x;
  v->detail = detail;
  v->code = code;
  __threadfence_system();
}

__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_f4(float* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

// w - lr * (gscale * g), rounded step by step like the stand-alone SGD kernel.
__device__ __forceinline__ float sgd1(float w, float g, float lr, float gscale) {
  const float gg = gscale == 1.0f ? g : __fmul_rn(gscale, g);
  return __fsub_rn(w, __fmul_rn(lr, gg));
}

__global__ void __launch_bounds__(kDpThreads) dp_sgd_allreduce_kernel(DpArgs a) {
  uint32_t* mine = a.flags[a.rank];

  // ---- entry barrier: every rank's gradients are final ------------------------------------
  __shared__ int s_abort;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    if (threadIdx.x < a.world) {
      __threadfence_system();
      st_release_sys(a.flags[threadIdx.x] + kFlagFromRank + a.rank, a.epoch);
      if (!wait_epoch<true>(mine + kFlagFromRank + threadIdx.x, a.epoch, a.wait_ns)) {
        dp_report(a.status, 10, 1000 + threadIdx.x, (int)a.epoch);
        s_abort = 1;
      }
    }
    __syncthreads();
    const int entry_failed = s_abort;   // read by all threads before anyone may set it again below
    __syncthreads();
    if (entry_failed) {
      // tell every peer that this rank abandons the launch (a late rank must not update alone) ...
      if (threadIdx.x < a.world) st_release_sys(a.flags[threadIdx.x] + kFlagAbortFrom + a.rank, a.epoch);
    } else if (threadIdx.x < a.world && ld_acquire_sys(mine + kFlagAbortFrom + threadIdx.x) == a.epoch) {
      // ... and a rank whose own wait succeeded still stands down when a peer has given up on this epoch
      dp_report(a.status, 13, 1300 + threadIdx.x, (int)a.epoch);
      s_abort = 1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (s_abort) st_release_gpu(mine + kFlagAbort, a.epoch);
      st_release_gpu(mine + kFlagGo, a.epoch);   // always released, so that no CTA of this launch is left waiting
    }
  } else {
    if (threadIdx.x == 0) {
      s_abort = 0;
      if (!wait_epoch<false>(mine + kFlagGo, a.epoch, 2 * a.wait_ns + 1000000000ull)) {
        dp_report(a.status, 11, 1100, (int)a.epoch);
        s_abort = 1;
      } else if (ld_acquire_gpu(mine + kFlagAbort) == a.epoch) {
        s_abort = 1;
      }
    }
    __syncthreads();
  }
  const bool aborted = s_abort != 0;   // uniform over the CTA
  __threadfence_system();

  // ---- this rank's slice: reduce, update, replicate ------------------------------------------
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float* w_local = a.params[a.rank];
  if (aborted) {
    // nothing is read from or written to any rank
  } else if (a.grads_mc != nullptr && a.params_mc != nullptr) {
    // Four reduced loads in flight per thread: the round trip through the switch is long and the
    // grid is deliberately small.
    constexpr int kU = 4;
    for (int64_t base = a.word_lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < a.word_hi;
         base += stride * kU) {
      float4 g[kU], w[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = base + u * stride;
        if (i < a.word_hi) {
          g[u] = multimem_ld_reduce_f4(a.grads_mc + 4 * i);
          w[u] = *reinterpret_cast<const float4*>(w_local + 4 * i);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = base + u * stride;
        if (i < a.word_hi) {
          float4 r;
          r.x = sgd1(w[u].x, g[u].x, a.lr, a.gscale); r.y = sgd1(w[u].y, g[u].y, a.lr, a.gscale);
          r.z = sgd1(w[u].z, g[u].z, a.lr, a.gscale); r.w = sgd1(w[u].w, g[u].w, a.lr, a.gscale);
          multimem_st_f4(a.params_mc + 4 * i, r);
        }
      }
    }
  } else {
    for (int64_t i = a.word_lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.word_hi; i += stride) {
      float4 part[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world) part[r] = ld_peer_f4(a.grads[r] + 4 * i);
      float4 g = part[0];
#pragma unroll
      for (int r = 1; r < kMaxRanks; ++r)
        if (r < a.world) {
          g.x = __fadd_rn(g.x, part[r].x); g.y = __fadd_rn(g.y, part[r].y);
          g.z = __fadd_rn(g.z, part[r].z); g.w = __fadd_rn(g.w, part[r].w);
        }
      const float4 w = *reinterpret_cast<const float4*>(w_local + 4 * i);
      float4 o;
      o.x = sgd1(w.x, g.x, a.lr, a.gscale); o.y = sgd1(w.y, g.y, a.lr, a.gscale);
      o.z = sgd1(w.z, g.z, a.lr, a.gscale); o.w = sgd1(w.w, g.w, a.lr, a.gscale);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world) st_peer_f4(a.params[r] + 4 * i, o);
    }
  }

  // ---- exit barrier: taken by the last CTA of this launch ----------------------------------------
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(mine + kFlagDone, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) mine[kFlagDone] = 0;   // ready for the next launch, also after an abandoned one
    // The exit epoch is signalled even by an abandoned launch (a peer that did run must not wait out its limit
    // for this rank); an abandoned launch has written nothing and waits for nobody.
    if (threadIdx.x < a.world) {
      __threadfence_system();
      st_release_sys(a.flags[threadIdx.x] + kFlagFromRank + a.rank, a.epoch + 1u);
      if (!aborted && !wait_epoch<true>(mine + kFlagFromRank + threadIdx.x, a.epoch + 1u, a.wait_ns))
        dp_report(a.status, 12, 1200 + threadIdx.x, (int)a.epoch);
    }
  }
}

}  // namespace cleave

using namespace cleave;

extern "C" int32_t cleave_cuda_dp_sgd_allreduce_f32(void* const* params_peers, void* const* grads_peers,
                                                    void* const* flags_peers, void* params_multicast,
                                                    void* grads_multicast, int64_t offset, int64_t len, int32_t rank,
                                                    int32_t world, float lr, uint32_t epoch, void* cuda_stream) {
  ApiLock lock;
  if (!ensure_init()) return -cleave_cuda_last_error();
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return -set_error(CLEAVE_CUDA_ERR_ARG, "dp_sgd_allreduce: rank %d / world %d (at most %d ranks)", rank, world,
                      kMaxRanks);
  if (!params_peers || !grads_peers || !flags_peers || len <= 0 || len % 4 != 0 || offset < 0 || offset % 4 != 0)
    return -set_error(CLEAVE_CUDA_ERR_ARG, "dp_sgd_allreduce: need peer pointer tables and an offset and length that "
                                           "are multiples of 4 (got %lld, %lld)", (long long)offset, (long long)len);
  DpArgs a{};
  for (int r = 0; r < world; ++r) {
    if (!params_peers[r] || !grads_peers[r] || !flags_peers[r] || ((uintptr_t)params_peers[r] & 15u) ||
        ((uintptr_t)grads_peers[r] & 15u))
      return -set_error(CLEAVE_CUDA_ERR_ARG, "dp_sgd_allreduce: peer %d has a NULL or unaligned buffer", r);
    a.params[r] = (float*)params_peers[r] + offset;
    a.grads[r] = (const float*)grads_peers[r] + offset;
    a.flags[r] = (uint32_t*)flags_peers[r];
  }
  a.params_mc = params_multicast ? (float*)params_multicast + offset : nullptr;
  a.grads_mc = grads_multicast ? (const float*)grads_multicast + offset : nullptr;
  a.rank = rank;
  a.world = world;
  const int64_t words = len / 4, base = words / world, extra = words % world;
  a.word_lo = rank * base + (rank < extra ? rank : extra);
  a.word_hi = a.word_lo + base + (rank < extra ? 1 : 0);
  a.lr = lr;
  a.gscale = 1.0f / (float)world;
  a.epoch = epoch;
  // Cross-GPU wait limit: 2 s, or CLEAVE_CUDA_DP_WAIT_MS (1 .. 60000) read once.  Host-side skew between the
  // ranks' launches (module loading, a data loader, a garbage collection) counts against it.
  static const unsigned long long wait_ns = [] {
    const char* e = getenv("CLEAVE_CUDA_DP_WAIT_MS");
    const long ms = e ? atol(e) : 0;
    return (ms >= 1 && ms <= 60000) ? (unsigned long long)ms * 1000000ull : kDpWaitLimitNs;
  }();
  a.wait_ns = wait_ns;
  a.status = ctx().status_dev;
  // A light grid of small CTAs: the kernel is bound by NVLink round trips, not by SMs, and it is meant to run
  // BESIDE a tensor-core GEMM (whose persistent CTAs leave about 11 K registers per SM: room for one 128-thread
  // CTA of this kernel).  CTAs other than 0 wait only for CTA 0, which is dispatched first.
  static const int max_ctas = [] {
    const char* e = getenv("CLEAVE_CUDA_DP_CTAS");
    const int v = e ? atoi(e) : 0;
    return (v >= 1 && v <= 1024) ? v : 0;
  }();
  int grid = ceil_div(a.word_hi - a.word_lo, kDpThreads * 4);
  const int cap = max_ctas ? max_ctas : ctx().sm_count;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  cudaStream_t s = cuda_stream ? (cudaStream_t)cuda_stream : ctx().stream;
  Trace tr("dp_sgd_allreduce", "offset=%lld len=%lld rank=%d world=%d", (long long)offset, (long long)len, rank, world);
  dp_sgd_allreduce_kernel<<<grid, kDpThreads, 0, s>>>(a);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "dp_sgd_allreduce launch")) return -cleave_cuda_last_error();
  return CLEAVE_CUDA_OK;
}
