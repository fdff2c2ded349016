// Reductions: Sum / Mean / Max (stdlib/nn/nn.cleave:111-149 in the reference), column sums,
// fused mean-squared-error forward+backward, and the single-sweep linear-regression step.
//
// All of them are deterministic: the grid size is a fixed function of the problem size, each
// CTA reduces a fixed set of elements with warp shuffles and a shared-memory tree, writes one
// partial, and a second one-CTA kernel combines the partials in index order.  No atomics.
#include <cfloat>
#include <cmath>

#include "common.cuh"

namespace cleave {

constexpr int kRThreads = 256;
constexpr int kRWarps = kRThreads / 32;
constexpr int kMaxPartials = 148 * 8;   // upper bound on first-stage CTAs

struct SumRed {
  static __device__ float identity() { return 0.0f; }
  static __device__ float combine(float a, float b) { return __fadd_rn(a, b); }
};
// Maximum that skips NaN operands (fmaxf); the NaN-in-first-element rule of the reference's
// strict-> scan is applied when the partials are combined with v[0].
struct MaxRed {
  static __device__ float identity() { return -INFINITY; }
  static __device__ float combine(float a, float b) { return fmaxf(a, b); }
};

template <class R>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = R::combine(v, __shfl_down_sync(0xffffffffu, v, off));
  return v;
}

// Block-wide reduction; the result is valid in thread 0.
template <class R>
__device__ __forceinline__ float block_reduce(float v) {
  __shared__ float warp_part[kRWarps];
  v = warp_reduce<R>(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();   // protects warp_part across back-to-back calls
  if (lane == 0) warp_part[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < kRWarps ? warp_part[lane] : R::identity();
    v = warp_reduce<R>(v);
  }
  return v;
}

// What the last CTA of a reduction does with the per-CTA partials: thread t folds partials
// t, t+256, ... in ascending order, then a block tree.
// mode 0: out = total / divisor (divisor 1 skips the division).
// mode 1 (max_of): out = (total > first) ? total : first.
struct Finish {
  float* out;
  float divisor;
  int mode;
  const float* first;
  unsigned int* done;   // completion counter of this launch family: zero between launches
};

// Arrival on a completion counter with release + acquire semantics in ONE memory operation: the partial sums this
// thread stored before it are visible to whoever observes the count, and the CTA that observes the final count sees
// every other CTA's partials.  Replaces store; fence; atomic; fence -- two L2 round trips less on the kernel's tail.
__device__ __forceinline__ unsigned int arrive_acq_rel(unsigned int* counter) {
  unsigned int prev;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(counter) : "memory");
  return prev;
}

// Publishes partials[blockIdx.x] = value (thread 0's) and tells, in every thread, whether this CTA
// is the last of the grid to do so.  The last CTA re-arms the counter for the next launch.
__device__ __forceinline__ bool publish_and_check_last(float* partials, float value, const Finish& f) {
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = value;
    const unsigned int prev = arrive_acq_rel(f.done);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) *f.done = 0;
  }
  __syncthreads();
  return s_last != 0;
}

template <class R>
__device__ __forceinline__ void finish_reduction(const float* partials, int count, const Finish& f) {
  float acc = R::identity();
  for (int i = threadIdx.x; i < count; i += kRThreads) acc = R::combine(acc, __ldcg(partials + i));
  acc = block_reduce<R>(acc);
  if (threadIdx.x == 0) {
    if (f.mode == 0) {
      f.out[0] = f.divisor == 1.0f ? acc : __fdiv_rn(acc, f.divisor);
    } else {
      const float v0 = f.first[0];
      f.out[0] = acc > v0 ? acc : v0;
    }
  }
}

// One launch per reduction.  Each CTA owns a contiguous slab of the input (partial b covers
// elements [b*slab, (b+1)*slab)) and reads it as float4; the last CTA to finish combines the
// partials in index order, so the result does not depend on the order in which CTAs ran.
template <class R>
__global__ void __launch_bounds__(kRThreads) reduce_kernel(const float* __restrict__ v, int64_t n, int64_t slab,
                                                           float* __restrict__ partials, int vec, Finish fin) {
  const int64_t lo = (int64_t)blockIdx.x * slab;
  int64_t hi = lo + slab;
  if (hi > n) hi = n;
  float acc[4] = {R::identity(), R::identity(), R::identity(), R::identity()};
  if (vec) {   // slab is a multiple of 4 and v is 16-byte aligned
    const float4* v4 = reinterpret_cast<const float4*>(v);
    const int64_t lo4 = lo >> 2, hi4 = hi >> 2;
    int64_t i = lo4 + threadIdx.x;
    for (; i + 3 * kRThreads < hi4; i += 4 * kRThreads) {   // four independent 16-byte loads in flight
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) x[u] = __ldcs(v4 + i + u * kRThreads);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        acc[0] = R::combine(acc[0], x[u].x);
        acc[1] = R::combine(acc[1], x[u].y);
        acc[2] = R::combine(acc[2], x[u].z);
        acc[3] = R::combine(acc[3], x[u].w);
      }
    }
    for (; i < hi4; i += kRThreads) {
      float4 x = __ldcs(v4 + i);
      acc[0] = R::combine(acc[0], x.x);
      acc[1] = R::combine(acc[1], x.y);
      acc[2] = R::combine(acc[2], x.z);
      acc[3] = R::combine(acc[3], x.w);
    }
    for (int64_t j = (hi4 << 2) + threadIdx.x; j < hi; j += kRThreads) acc[0] = R::combine(acc[0], v[j]);
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kRThreads) acc[0] = R::combine(acc[0], v[i]);
  }
  float t = R::combine(R::combine(acc[0], acc[1]), R::combine(acc[2], acc[3]));
  t = block_reduce<R>(t);
  if (publish_and_check_last(partials, t, fin)) finish_reduction<R>(partials, gridDim.x, fin);
}

// Completion counters of the pooled entry points (one reduction runs at a time: single stream).
static __device__ unsigned int g_reduce_done = 0;

// ---- column sums: x[rows, cols] -> out[cols] ------------------------------------------------
// grid = (column strips of 128 floats, row splits).  Thread (tx, ty) owns one float4 column
// group and the rows ty, ty+8, ... of its split; the 8 row-threads are combined through
// shared memory in ty order; splits are combined by the second stage in split order.
constexpr int kCsTx = 32, kCsTy = 8;

constexpr int kCsMaxStrips = 2048;   // strips that can finish in the same launch (one completion counter each)
static __device__ unsigned int g_colsum_done[kCsMaxStrips];

// `out` != null: single launch -- the last CTA of a column strip to finish (a counter per strip, the
// only atomic) adds the strip's partial sums in split order and writes the result.  `out` == null:
// only the partials are written and colsum_stage2 combines them (more strips than counters).
__global__ void __launch_bounds__(kCsTx* kCsTy) colsum_stage1(const float* __restrict__ x, int rows, int cols,
                                                               int rows_per_split, float* __restrict__ partials,
                                                               int vec, float* __restrict__ out) {
  __shared__ float4 sm[kCsTy][kCsTx];
  __shared__ int is_last;
  const int tx = threadIdx.x % kCsTx, ty = threadIdx.x / kCsTx;
  const int c0 = (blockIdx.x * kCsTx + tx) * 4;
  const int r_lo = blockIdx.y * rows_per_split;
  int r_hi = r_lo + rows_per_split;
  if (r_hi > rows) r_hi = rows;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c0 < cols) {
    if (vec) {
      for (int r = r_lo + ty; r < r_hi; r += kCsTy) {
        float4 v = __ldcs(reinterpret_cast<const float4*>(x + (int64_t)r * cols + c0));
        acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
        acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
      }
    } else {
      for (int r = r_lo + ty; r < r_hi; r += kCsTy) {
        const float* p = x + (int64_t)r * cols + c0;
        acc.x = __fadd_rn(acc.x, p[0]);
        if (c0 + 1 < cols) acc.y = __fadd_rn(acc.y, p[1]);
        if (c0 + 2 < cols) acc.z = __fadd_rn(acc.z, p[2]);
        if (c0 + 3 < cols) acc.w = __fadd_rn(acc.w, p[3]);
      }
    }
  }
  sm[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && c0 < cols) {
    float4 t = sm[0][tx];
#pragma unroll
    for (int j = 1; j < kCsTy; ++j) {
      float4 u = sm[j][tx];
      t.x = __fadd_rn(t.x, u.x); t.y = __fadd_rn(t.y, u.y); t.z = __fadd_rn(t.z, u.z); t.w = __fadd_rn(t.w, u.w);
    }
    float* p = partials + (int64_t)blockIdx.y * cols + c0;
    p[0] = t.x;
    if (c0 + 1 < cols) p[1] = t.y;
    if (c0 + 2 < cols) p[2] = t.z;
    if (c0 + 3 < cols) p[3] = t.w;
  }
  if (out == nullptr) return;
  // ---- the strip's last CTA combines the splits
  __syncthreads();   // every thread's partial stores are ordered before thread 0's arrival below (CTA scope) ...
  if (threadIdx.x == 0) {
    __threadfence();   // ... and made visible device-wide (cumulativity: the fence covers what the barrier ordered)
    is_last = arrive_acq_rel(&g_colsum_done[blockIdx.x]) == gridDim.y - 1 ? 1 : 0;
  }
  __syncthreads();
  if (!is_last) return;
  const int splits = gridDim.y;
  float4 part = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c0 < cols) {
    // thread row ty takes splits ty, ty + 8, ... in increasing order; the 8 rows are then added in ty order
    for (int sidx = ty; sidx < splits; sidx += kCsTy) {
      const float* p = partials + (int64_t)sidx * cols + c0;
      part.x = __fadd_rn(part.x, __ldcg(p));
      if (c0 + 1 < cols) part.y = __fadd_rn(part.y, __ldcg(p + 1));
      if (c0 + 2 < cols) part.z = __fadd_rn(part.z, __ldcg(p + 2));
      if (c0 + 3 < cols) part.w = __fadd_rn(part.w, __ldcg(p + 3));
    }
  }
  sm[ty][tx] = part;
  __syncthreads();
  if (ty == 0 && c0 < cols) {
    float4 t = sm[0][tx];
#pragma unroll
    for (int j = 1; j < kCsTy; ++j) {
      float4 u = sm[j][tx];
      t.x = __fadd_rn(t.x, u.x); t.y = __fadd_rn(t.y, u.y); t.z = __fadd_rn(t.z, u.z); t.w = __fadd_rn(t.w, u.w);
    }
    out[c0] = t.x;
    if (c0 + 1 < cols) out[c0 + 1] = t.y;
    if (c0 + 2 < cols) out[c0 + 2] = t.z;
    if (c0 + 3 < cols) out[c0 + 3] = t.w;
  }
  if (threadIdx.x == 0) g_colsum_done[blockIdx.x] = 0;   // ready for the next launch (stream order)
}

__global__ void __launch_bounds__(kRThreads) colsum_stage2(const float* __restrict__ partials, int splits, int cols,
                                                           float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float acc = partials[c];
  for (int s = 1; s < splits; ++s) acc = __fadd_rn(acc, partials[(int64_t)s * cols + c]);
  out[c] = acc;
}

// ---- fused MSE: partial sums of (p-t)^2 and, optionally, dp = 2 (p-t) / n -----------------------
// With bwd_act != identity, p is the OUTPUT of that activation and the value written is the
// gradient with respect to the pre-activation: act'(p) * 2 (p - t) / n, each factor rounded as the
// separate mse and *_bwd entry points round it (so the fused result is bit-identical to the chain).
__device__ __forceinline__ float mse_grad(float p, float e, float fn, int bwd_act) {
  float d = __fdiv_rn(__fmul_rn(2.0f, e), fn);
  if (bwd_act == CLEAVE_ACT_SIGMOID) d = __fmul_rn(__fmul_rn(p, __fsub_rn(1.0f, p)), d);
  else if (bwd_act == CLEAVE_ACT_TANH) d = __fmul_rn(__fsub_rn(1.0f, __fmul_rn(p, p)), d);
  return d;
}

// Low split part of a value (the lo plane a following tensor-core GEMM needs; same function as split_lo in
// tc_common.cuh, repeated here because this file does not include the GEMM headers).
__device__ __forceinline__ float lo_part(float x) {
  const float d = __fsub_rn(x, __uint_as_float(__float_as_uint(x) & 0xFFFFE000u));
  return __uint_as_float(__float_as_uint(d) + 0x1000u);
}

__global__ void __launch_bounds__(kRThreads) mse_stage1(const float* __restrict__ p, const float* __restrict__ t,
                                                        float* __restrict__ dp, float* __restrict__ dlo, int64_t n,
                                                        int64_t slab, float fn, float* __restrict__ partials, int vec,
                                                        int bwd_act, Finish fin) {
  const int64_t lo = (int64_t)blockIdx.x * slab;
  int64_t hi = lo + slab;
  if (hi > n) hi = n;
  float acc = 0.0f;
  if (vec) {
    const float4* p4 = reinterpret_cast<const float4*>(p);
    const float4* t4 = reinterpret_cast<const float4*>(t);
    float4* d4 = reinterpret_cast<float4*>(dp);
    const int64_t lo4 = lo >> 2, hi4 = hi >> 2;
    for (int64_t i = lo4 + threadIdx.x; i < hi4; i += kRThreads) {
      float4 a = __ldcs(p4 + i), b = __ldcs(t4 + i);
      float e0 = __fsub_rn(a.x, b.x), e1 = __fsub_rn(a.y, b.y), e2 = __fsub_rn(a.z, b.z), e3 = __fsub_rn(a.w, b.w);
      acc = __fadd_rn(acc, __fadd_rn(__fadd_rn(__fmul_rn(e0, e0), __fmul_rn(e1, e1)),
                                     __fadd_rn(__fmul_rn(e2, e2), __fmul_rn(e3, e3))));
      if (dp) {
        float4 d;
        d.x = mse_grad(a.x, e0, fn, bwd_act); d.y = mse_grad(a.y, e1, fn, bwd_act);
        d.z = mse_grad(a.z, e2, fn, bwd_act); d.w = mse_grad(a.w, e3, fn, bwd_act);
        __stcs(d4 + i, d);
        if (dlo) __stcs(reinterpret_cast<float4*>(dlo) + i, make_float4(lo_part(d.x), lo_part(d.y), lo_part(d.z), lo_part(d.w)));
      }
    }
    for (int64_t i = (hi4 << 2) + threadIdx.x; i < hi; i += kRThreads) {
      float e = __fsub_rn(p[i], t[i]);
      acc = __fadd_rn(acc, __fmul_rn(e, e));
      if (dp) {
        const float d = mse_grad(p[i], e, fn, bwd_act);
        dp[i] = d;
        if (dlo) dlo[i] = lo_part(d);
      }
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kRThreads) {
      float e = __fsub_rn(p[i], t[i]);
      acc = __fadd_rn(acc, __fmul_rn(e, e));
      if (dp) {
        const float d = mse_grad(p[i], e, fn, bwd_act);
        dp[i] = d;
        if (dlo) dlo[i] = lo_part(d);
      }
    }
  }
  acc = block_reduce<SumRed>(acc);
  if (publish_and_check_last(partials, acc, fin)) finish_reduction<SumRed>(partials, gridDim.x, fin);
}

// ---- linear-regression step: one sweep over X[rows, feat] ------------------------------------
// Each thread owns whole rows: pred_i = sum_f X[i,f] w[f] (f ascending, multiply then add, so
// pred is bit-identical to the reference's matmul), e = pred - y, accumulates e^2 and
// X[i,f] * (2 e / rows) per feature.  Per-CTA partials: [feat] gradient sums, then the loss sum.
constexpr int kMaxFeat = 32;

// Completion counter of the linear-regression sweep: the last CTA to finish folds the per-CTA
// partials (second stage) in the same launch.  One sweep runs at a time (single stream).
static __device__ unsigned int g_linreg_done = 0;

// Second stage, run by the last CTA to finish.  Everything else has drained by then, so its
// latency is pure tail: all 256 threads first pull their share of every quantity's partials with
// batches of independent 16-byte loads (thread t owns partials 4t .. 4t+3, then 4t+1024 .., of
// each quantity, added in ascending order) into scratch[q][t]; then warp w finishes quantities
// w, w+8, ...: lane l adds scratch[q][l], scratch[q][l+32], ... in ascending order and a fixed
// shuffle tree combines the lanes.  partials[q] starts at q * pitch, pitch a multiple of 4.
// The order depends only on the number of CTAs, never on which CTA finished last.
// NQ = feat + 1 quantities (gradient components, then the loss); scratch holds NQ * 256 floats.
template <int NQ_MAX>
__device__ __forceinline__ void linreg_fold(const float* partials, int pitch, int ctas, int feat, float fn,
                                            float* grad, float* loss_out, float* scratch) {
  const int t = threadIdx.x, lane = t & 31, nwarps = blockDim.x >> 5;
  constexpr int kBatch = 9;   // 16-byte loads in flight per thread
  for (int q0 = 0; q0 < NQ_MAX; q0 += kBatch) {
    float acc[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) acc[j] = 0.0f;
    for (int c0 = 4 * t; c0 < ctas; c0 += 4 * kRThreads) {
      float4 v[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j)
        v[j] = (q0 + j <= feat) ? __ldcg(reinterpret_cast<const float4*>(partials + (int64_t)(q0 + j) * pitch + c0))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        acc[j] = __fadd_rn(acc[j], v[j].x);
        if (c0 + 1 < ctas) acc[j] = __fadd_rn(acc[j], v[j].y);
        if (c0 + 2 < ctas) acc[j] = __fadd_rn(acc[j], v[j].z);
        if (c0 + 3 < ctas) acc[j] = __fadd_rn(acc[j], v[j].w);
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (q0 + j <= feat) scratch[(q0 + j) * kRThreads + t] = acc[j];
  }
  __syncthreads();
  for (int q = t >> 5; q <= feat; q += nwarps) {
    const float* row = scratch + q * kRThreads;
    float acc = row[lane];
#pragma unroll
    for (int j = 1; j < kRThreads / 32; ++j) acc = __fadd_rn(acc, row[lane + 32 * j]);
    acc = warp_reduce<SumRed>(acc);
    if (lane == 0) {
      if (q < feat) grad[q] = acc;
      else loss_out[0] = __fdiv_rn(acc, fn);
    }
  }
}

// Publishes this CTA's partials and returns true in exactly one CTA: the last one to arrive.
__device__ __forceinline__ bool linreg_arrive_last() {
  __shared__ int s_last;
  __syncthreads();     // the partial stores of threads 0..feat are ordered before thread 0's arrival (CTA scope)
  if (threadIdx.x == 0) {
    __threadfence();   // cumulative: makes them visible device-wide before the count can be observed
    const unsigned int prev = arrive_acq_rel(&g_linreg_done);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) g_linreg_done = 0;   // ready for the next launch
  }
  __syncthreads();
  return s_last != 0;
}

constexpr int kLrStages = 3;   // row groups in flight per warp (cp.async ring)

template <int FEAT>
__global__ void __launch_bounds__(kRThreads, FEAT <= 16 ? 4 : 2) linreg_stage1(const float* __restrict__ X, const float* __restrict__ y,
                                                           const float* __restrict__ w, float* __restrict__ pred,
                                                           int64_t rows, int64_t slab, float fn,
                                                           float* __restrict__ partials, float* __restrict__ grad,
                                                           float* __restrict__ loss_out) {
  // Each warp takes 32 consecutive rows at a time.  The 32*FEAT floats of such a group are
  // contiguous in X, so the warp fetches them with fully coalesced 16-byte asynchronous copies
  // (cp.async, lane l takes 16-byte words l, l+32, ...) straight into a warp-private ring of
  // kLrStages shared tiles -- several groups are in flight per warp without holding registers --
  // and every lane then picks up ITS row.  Words of row r land at slot q ^ swz(r), which makes both
  // the copies and the row-wise 16-byte reads bank-conflict free.
  static_assert(FEAT % 4 == 0 && FEAT >= 4 && FEAT <= 32, "FEAT must be 4, 8, 16 or 32");
  constexpr int Q = FEAT / 4;                 // 16-byte words per row
  const int pitch = (gridDim.x + 3) & ~3;     // row pitch of partials[quantity][cta]
  constexpr int kRowsPerSwz = Q >= 8 ? 1 : 8 / Q;
  extern __shared__ __align__(16) unsigned char lr_smem[];
  float4* tile = reinterpret_cast<float4*>(lr_smem);                       // [kRWarps][kLrStages][32 * Q]
  float* sw = reinterpret_cast<float*>(tile + kRWarps * kLrStages * 32 * Q);   // [FEAT]
  float* red = sw + FEAT;                                                  // [kRWarps][FEAT + 1]
  if (threadIdx.x < FEAT) sw[threadIdx.x] = w[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t lo = (int64_t)blockIdx.x * slab;
  int64_t hi = lo + slab;
  if (hi > rows) hi = rows;
  float g[FEAT];
#pragma unroll
  for (int f = 0; f < FEAT; ++f) g[f] = 0.0f;
  float loss = 0.0f;
  float4* my_ring = tile + (size_t)warp * kLrStages * 32 * Q;
  const int my_swz = (lane / kRowsPerSwz) & (Q - 1);
  constexpr int64_t kStep = (int64_t)kRWarps * 32;
  const float two_over_n = __fdiv_rn(2.0f, fn);

  // Queue the copies of one row group into ring stage `stage` (rows past the slab end are zeroed).
  auto issue = [&](int stage, int64_t r0) {
    if (r0 < hi) {
      const float4* src = reinterpret_cast<const float4*>(X + r0 * FEAT);
      float4* dst = my_ring + stage * 32 * Q;
#pragma unroll
      for (int k = 0; k < Q; ++k) {
        const int idx = lane + 32 * k;
        const int r = idx / Q, q = idx % Q;
        float4* d = dst + r * Q + (q ^ ((r / kRowsPerSwz) & (Q - 1)));
        if (r0 + r < hi) {
          const unsigned sa = (unsigned)__cvta_generic_to_shared(d);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src + idx) : "memory");
        } else {
          *d = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // one group per call, possibly empty
  };

  const int64_t first = lo + (int64_t)warp * 32;
#pragma unroll
  for (int s = 0; s < kLrStages - 1; ++s) issue(s, first + s * kStep);
  int stage = 0;
  for (int64_t r0 = first; r0 < hi; r0 += kStep) {
    issue((stage + kLrStages - 1) % kLrStages, r0 + (kLrStages - 1) * kStep);
    const int64_t i = r0 + lane;
    const float yi = i < hi ? __ldcs(y + i) : 0.0f;
    asm volatile("cp.async.wait_group %0;" ::"n"(kLrStages - 1) : "memory");
    __syncwarp();
    float xr[FEAT];
    const float4* cur = my_ring + stage * 32 * Q;
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const float4 t = cur[lane * Q + (q ^ my_swz)];
      xr[4 * q] = t.x; xr[4 * q + 1] = t.y; xr[4 * q + 2] = t.z; xr[4 * q + 3] = t.w;
    }
    __syncwarp();   // every lane has its row: the stage may be refilled by the next iteration
    if (i < hi) {
      float acc = 0.0f;
#pragma unroll
      for (int f = 0; f < FEAT; ++f) acc = __fadd_rn(acc, __fmul_rn(xr[f], sw[f]));
      if (pred) pred[i] = acc;
      const float e = __fsub_rn(acc, yi);
      loss = __fadd_rn(loss, __fmul_rn(e, e));
      // Gradient terms x * (2 e / n): summed in a tree anyway, so fused multiply-adds are used
      // here (one rounding per term instead of two); only pred has to match the reference's chain.
      const float d = __fmul_rn(e, two_over_n);
#pragma unroll
      for (int f = 0; f < FEAT; ++f) g[f] = fmaf(xr[f], d, g[f]);
    }
    stage = (stage + 1) % kLrStages;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // CTA reduction with one barrier: shuffle tree inside each warp, then warps 0..7 in order.
#pragma unroll
  for (int f = 0; f < FEAT; ++f) {
    const float t = warp_reduce<SumRed>(g[f]);
    if (lane == 0) red[warp * (FEAT + 1) + f] = t;
  }
  {
    const float t = warp_reduce<SumRed>(loss);
    if (lane == 0) red[warp * (FEAT + 1) + FEAT] = t;
  }
  __syncthreads();
  if (threadIdx.x <= FEAT) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int wv = 1; wv < kRWarps; ++wv) t = __fadd_rn(t, red[wv * (FEAT + 1) + threadIdx.x]);
    partials[(int64_t)threadIdx.x * pitch + blockIdx.x] = t;
  }
  // the ring is idle now (all copies were waited for): reuse it as the fold's scratch
  if (linreg_arrive_last()) linreg_fold<FEAT + 1>(partials, pitch, gridDim.x, FEAT, fn, grad, loss_out, reinterpret_cast<float*>(lr_smem));
}

// Generic-feat fallback (feat <= 32, any value): same arithmetic, runtime loops.
__global__ void __launch_bounds__(kRThreads) linreg_stage1_any(const float* __restrict__ X, const float* __restrict__ y,
                                                               const float* __restrict__ w, float* __restrict__ pred,
                                                               int64_t rows, int feat, int64_t slab, float fn,
                                                               float* __restrict__ partials, float* __restrict__ grad,
                                                               float* __restrict__ loss_out) {
  __shared__ float sw[kMaxFeat];
  const int pitch = (gridDim.x + 3) & ~3;
  if (threadIdx.x < feat) sw[threadIdx.x] = w[threadIdx.x];
  __syncthreads();
  const int64_t lo = (int64_t)blockIdx.x * slab;
  int64_t hi = lo + slab;
  if (hi > rows) hi = rows;
  float g[kMaxFeat];
#pragma unroll
  for (int f = 0; f < kMaxFeat; ++f) g[f] = 0.0f;
  float loss = 0.0f;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kRThreads) {
    float acc = 0.0f;
    for (int f = 0; f < feat; ++f) acc = __fadd_rn(acc, __fmul_rn(X[i * feat + f], sw[f]));
    if (pred) pred[i] = acc;
    float e = __fsub_rn(acc, y[i]);
    loss = __fadd_rn(loss, __fmul_rn(e, e));
    float d = __fdiv_rn(__fmul_rn(2.0f, e), fn);
#pragma unroll
    for (int f = 0; f < kMaxFeat; ++f)
      if (f < feat) g[f] = __fadd_rn(g[f], __fmul_rn(X[i * feat + f], d));
  }
#pragma unroll
  for (int f = 0; f < kMaxFeat; ++f) {
    if (f < feat) {   // uniform across the block
      float t = block_reduce<SumRed>(g[f]);
      if (threadIdx.x == 0) partials[(int64_t)f * pitch + blockIdx.x] = t;
    }
  }
  loss = block_reduce<SumRed>(loss);
  if (threadIdx.x == 0) partials[(int64_t)feat * pitch + blockIdx.x] = loss;
  __shared__ float fold_scratch[(kMaxFeat + 1) * kRThreads];
  if (linreg_arrive_last()) linreg_fold<kMaxFeat + 1>(partials, pitch, gridDim.x, feat, fn, grad, loss_out, fold_scratch);
}

static size_t linreg_smem_bytes(int feat) {
  const int q = feat / 4;
  size_t ring = (size_t)kRWarps * kLrStages * 32 * q * sizeof(float4);
  const size_t fold = (size_t)(feat + 1) * kRThreads * sizeof(float);   // the fold reuses the ring as scratch
  if (ring < fold) ring = fold;
  return ring + (size_t)(feat + kRWarps * (feat + 1)) * sizeof(float);
}

// ---- host side -------------------------------------------------------------------------------
// Slab size (elements per first-stage CTA): at least 4096 elements, a multiple of 4, and no
// more CTAs than can be resident at once for the kernel in question (one wave: a second,
// partial wave would cost as much as the first).  A function of n and of the device model only,
// so the summation tree is reproducible.
template <class Kernel>
static int resident_ctas(Kernel kernel, size_t dyn_smem = 0) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kRThreads, dyn_smem) != cudaSuccess ||
      per_sm < 1) {
    cudaGetLastError();
    per_sm = 1;
  }
  int sms = ctx().sm_count;
  if (sms <= 0) {   // allocation-free entry point used before the library context exists
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
      cudaGetLastError();
      sms = 1;
    }
  }
  int64_t c = (int64_t)per_sm * sms;
  return (int)(c < kMaxPartials ? c : kMaxPartials);
}

static void slab_for(int64_t n, int max_ctas, int64_t* slab, int* ctas) {
  int64_t s = (n + max_ctas - 1) / max_ctas;
  if (s < 4096) s = 4096;
  s = (s + 3) / 4 * 4;
  *slab = s;
  *ctas = (int)((n + s - 1) / s);
}

template <class R>
static float reduce_scalar(const float* v, int64_t n, int64_t first, float divisor, int mode) {
  // Elements [first, n) are reduced; for max_of (mode 1) the result is combined with v[0].
  const float* base = v + first;
  int64_t cnt = n - first;
  Trace tr(mode == 1 ? "max_of" : (divisor == 1.0f ? "sum" : "mean"), "n=%lld", (long long)cnt);
  float* partials = scratch_alloc((kMaxPartials + 4) * sizeof(float));
  if (!partials) return NAN;
  float* out = scalar_slot();
  cudaStream_t s = ctx().stream;
  int64_t slab;
  int ctas;
  static const int max_ctas = resident_ctas(reduce_kernel<R>);
  slab_for(cnt, max_ctas, &slab, &ctas);
  unsigned int* done = nullptr;
  cudaGetSymbolAddress((void**)&done, g_reduce_done);
  reduce_kernel<R><<<ctas, kRThreads, 0, s>>>(base, cnt, slab, partials, aligned16(base) ? 1 : 0,
                                            Finish{out, divisor, mode, v, done});
  count_launch();
  float r = NAN;
  if (cuda_ok(cudaGetLastError(), "reduction launch")) r = wait_scalar();
  scratch_free(partials);
  return r;
}

}  // namespace cleave

using namespace cleave;

extern "C" {

float cleave_cuda_sum_f32(cleave_buf v) {
  ApiLock lock;
  Buf* a = as_buf(v, "sum");
  if (!a) return NAN;
  return reduce_scalar<SumRed>(a->ptr, a->len, 0, 1.0f, 0);
}

float cleave_cuda_mean_f32(cleave_buf v) {
  ApiLock lock;
  Buf* a = as_buf(v, "mean");
  if (!a) return NAN;
  // sum(v) / (f32)N with N an i32 (stdlib/nn/nn.cleave:135-138)
  return reduce_scalar<SumRed>(a->ptr, a->len, 0, (float)(int32_t)a->len, 0);
}

float cleave_cuda_max_f32(cleave_buf v) {
  ApiLock lock;
  Buf* a = as_buf(v, "max_of");
  if (!a) return NAN;
  // v[0] takes part in the NaN-skipping maximum as well: if it is NaN it is skipped there and
  // re-imposed by the final strict-> comparison, otherwise including it changes nothing.
  return reduce_scalar<MaxRed>(a->ptr, a->len, 0, 1.0f, 1);
}

}  // extern "C"

namespace cleave {
bool colsum_launch(const float* x, float* out, int rows, int cols, cudaStream_t s) {
  Trace tr("colsum", "rows=%d cols=%d", rows, cols);
  const int strips = ceil_div(cols, kCsTx * 4);
  // Row splits: enough CTAs to fill the machine, at least 64 rows each; a function of the shape only.
  int splits = ceil_div((int64_t)ctx().sm_count * 4, strips);
  int max_splits = ceil_div(rows, 64);
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  int rows_per_split = ceil_div(rows, splits);
  splits = ceil_div(rows, rows_per_split);
  float* partials = scratch_alloc((int64_t)splits * cols * sizeof(float));
  if (!partials) return false;
  int vec = (aligned16(x) && cols % 4 == 0) ? 1 : 0;
  if (strips <= kCsMaxStrips) {
    colsum_stage1<<<dim3(strips, splits), kCsTx * kCsTy, 0, s>>>(x, rows, cols, rows_per_split, partials, vec, out);
    count_launch(1);
  } else {
    colsum_stage1<<<dim3(strips, splits), kCsTx * kCsTy, 0, s>>>(x, rows, cols, rows_per_split, partials, vec,
                                                                  nullptr);
    colsum_stage2<<<ceil_div(cols, kRThreads), kRThreads, 0, s>>>(partials, splits, cols, out);
    count_launch(2);
  }
  bool ok = cuda_ok(cudaGetLastError(), "colsum launch");
  scratch_free(partials);
  return ok;
}
}  // namespace cleave

extern "C" {

cleave_buf cleave_cuda_colsum_f32(cleave_buf x, int32_t rows, int32_t cols) {
  ApiLock lock;
  Buf* a = as_buf(x, "colsum");
  if (!a) return nullptr;
  if (rows <= 0 || cols <= 0 || a->len != (int64_t)rows * cols) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "colsum: tensor has %lld elements, not %d x %d", (long long)a->len, rows, cols);
    return nullptr;
  }
  Buf* o = new_buf(cols);
  if (!o) return nullptr;
  if (!colsum_launch(a->ptr, o->ptr, rows, cols, ctx().stream)) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

int32_t cleave_cuda_colsum_into_f32(cleave_buf out, cleave_buf x, int32_t rows, int32_t cols) {
  ApiLock lock;
  Buf* a = as_buf(x, "colsum_into");
  Buf* o = as_buf(out, "colsum_into");
  if (!a || !o) return -cleave_cuda_last_error();
  if (rows <= 0 || cols <= 0 || a->len != (int64_t)rows * cols || o->len != cols)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "colsum_into: tensor has %lld elements, output %lld, for %d x %d",
                      (long long)a->len, (long long)o->len, rows, cols);
  return colsum_launch(a->ptr, o->ptr, rows, cols, ctx().stream) ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

// loss_dev == nullptr: the loss is returned (the call waits for it).  Otherwise it is written to
// that one-element device tensor, nothing is waited for, and 0 is returned on success.
static float mse_impl(cleave_buf p, cleave_buf t, cleave_buf dp, int bwd_act, const char* name,
                      cleave_buf loss_dev = nullptr, cleave_buf dp_lo = nullptr) {
  ApiLock lock;
  Buf* dl = nullptr;
  if (dp_lo) {
    dl = as_buf(dp_lo, name);
    if (!dl) return NAN;
  }
  Buf* lo = nullptr;
  if (loss_dev) {
    lo = as_buf(loss_dev, name);
    if (!lo) return NAN;
    if (lo->len != 1) {
      set_error(CLEAVE_CUDA_ERR_SHAPE, "%s: the loss output must be a one-element tensor", name);
      return NAN;
    }
  }
  Buf* a = as_buf(p, name);
  Buf* b = as_buf(t, name);
  if (!a || !b) return NAN;
  Buf* d = nullptr;
  if (dp) {
    d = as_buf(dp, name);
    if (!d) return NAN;
  }
  if (dl && (!d || dl->len != d->len || dl->ptr == d->ptr)) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "%s: the lo plane needs the gradient output and its length", name);
    return NAN;
  }
  if (a->len != b->len || (d && d->len != a->len)) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "%s: prediction, target and gradient tensors must have the same length", name);
    return NAN;
  }
  if (bwd_act != CLEAVE_ACT_IDENTITY && bwd_act != CLEAVE_ACT_SIGMOID && bwd_act != CLEAVE_ACT_TANH) {
    set_error(CLEAVE_CUDA_ERR_ARG, "%s: activation code %d has no output-form derivative (use identity, sigmoid or tanh)",
              name, bwd_act);
    return NAN;
  }
  const int64_t n = a->len;
  Trace tr(name, "n=%lld act=%d", (long long)n, bwd_act);
  float* partials = scratch_alloc((kMaxPartials + 4) * sizeof(float));
  if (!partials) return NAN;
  int64_t slab;
  int ctas;
  static const int max_ctas = resident_ctas(mse_stage1);
  slab_for(n, max_ctas, &slab, &ctas);
  unsigned int* done = nullptr;
  cudaGetSymbolAddress((void**)&done, g_reduce_done);
  int vec = (aligned16(a->ptr) && aligned16(b->ptr) && (!d || aligned16(d->ptr)) && (!dl || aligned16(dl->ptr))) ? 1 : 0;
  const float fn = (float)(int32_t)n;
  cudaStream_t s = ctx().stream;
  float* out = lo ? lo->ptr : scalar_slot();
  mse_stage1<<<ctas, kRThreads, 0, s>>>(a->ptr, b->ptr, d ? d->ptr : nullptr, dl ? dl->ptr : nullptr, n, slab, fn,
                                        partials, vec, bwd_act, Finish{out, fn, 0, nullptr, done});
  count_launch();
  float r = NAN;
  if (cuda_ok(cudaGetLastError(), "mse launch")) r = lo ? 0.0f : wait_scalar();
  scratch_free(partials);
  return r;
}

float cleave_cuda_mse_f32(cleave_buf p, cleave_buf t, cleave_buf dp) {
  return mse_impl(p, t, dp, CLEAVE_ACT_IDENTITY, "mse");
}

int32_t cleave_cuda_mse_act_bwd_dev_f32(cleave_buf y, cleave_buf t, cleave_buf dz, int32_t act, cleave_buf loss_out) {
  if (!dz || !loss_out) {
    ApiLock lock;
    return -set_error(CLEAVE_CUDA_ERR_ARG, "mse_act_bwd_dev: the gradient and loss output handles are required");
  }
  float r = mse_impl(y, t, dz, act, "mse_act_bwd_dev", loss_out);
  return r == 0.0f ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

int32_t cleave_cuda_mse_act_bwd_lo_f32(cleave_buf y, cleave_buf t, cleave_buf dz, int32_t act, cleave_buf loss_out,
                                       cleave_buf dz_lo) {
  if (!dz || !loss_out || !dz_lo) {
    ApiLock lock;
    return -set_error(CLEAVE_CUDA_ERR_ARG, "mse_act_bwd_lo: the gradient, loss and lo-plane output handles are required");
  }
  float r = mse_impl(y, t, dz, act, "mse_act_bwd_lo", loss_out, dz_lo);
  return r == 0.0f ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

float cleave_cuda_mse_act_bwd_f32(cleave_buf y, cleave_buf t, cleave_buf dz, int32_t act) {
  if (!dz) {
    ApiLock lock;
    set_error(CLEAVE_CUDA_ERR_ARG, "mse_act_bwd: the gradient output handle is required");
    return NAN;
  }
  return mse_impl(y, t, dz, act, "mse_act_bwd");
}

// loss_dev == nullptr: the loss is returned (the call waits for it).  Otherwise it is written to that one-element
// device tensor, nothing is waited for, and 0 is returned on success.
static float linreg_impl(cleave_buf x, cleave_buf y, cleave_buf w, cleave_buf pred_out, cleave_buf grad_out, int32_t rows,
                         int32_t feat, cleave_buf loss_dev) {
  ApiLock lock;
  Buf* LO = nullptr;
  if (loss_dev) {
    LO = as_buf(loss_dev, "linreg_step");
    if (!LO) return NAN;
    if (LO->len != 1) {
      set_error(CLEAVE_CUDA_ERR_SHAPE, "linreg_step: the loss output must be a one-element tensor");
      return NAN;
    }
  }
  Buf* X = as_buf(x, "linreg_step");
  Buf* Y = as_buf(y, "linreg_step");
  Buf* W = as_buf(w, "linreg_step");
  Buf* G = as_buf(grad_out, "linreg_step");
  if (!X || !Y || !W || !G) return NAN;
  Buf* P = nullptr;
  if (pred_out) {
    P = as_buf(pred_out, "linreg_step");
    if (!P) return NAN;
  }
  if (rows <= 0 || feat <= 0 || feat > kMaxFeat) {
    set_error(CLEAVE_CUDA_ERR_ARG, "linreg_step: need rows > 0 and 1 <= feat <= %d (got %d, %d)", kMaxFeat, rows, feat);
    return NAN;
  }
  if (X->len != (int64_t)rows * feat || Y->len != rows || W->len != feat || G->len != feat || (P && P->len != rows)) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "linreg_step: operand lengths do not match rows=%d feat=%d", rows, feat);
    return NAN;
  }
  Trace tr("linreg_step", "rows=%d feat=%d", rows, feat);
  // Row slabs: one resident wave of CTAs, at least 1024 rows each, a multiple of 256 rows (8 warps x 32).
  const bool fast = (feat == 4 || feat == 8 || feat == 16 || feat == 32) && aligned16(X->ptr);
  const size_t dyn = fast ? linreg_smem_bytes(feat) : 0;
  int max_ctas;
  if (fast) {
    static bool attr_done = false;
    if (!attr_done) {   // the FEAT = 32 ring exceeds the default 48 KiB dynamic shared memory limit
      cudaFuncSetAttribute(linreg_stage1<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)linreg_smem_bytes(32));
      cudaFuncSetAttribute(linreg_stage1<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)linreg_smem_bytes(16));
      attr_done = true;
    }
    switch (feat) {
      case 4: max_ctas = resident_ctas(linreg_stage1<4>, dyn); break;
      case 8: max_ctas = resident_ctas(linreg_stage1<8>, dyn); break;
      case 16: max_ctas = resident_ctas(linreg_stage1<16>, dyn); break;
      default: max_ctas = resident_ctas(linreg_stage1<32>, dyn); break;
    }
  } else {
    max_ctas = resident_ctas(linreg_stage1_any);
  }
  int64_t slab = ((int64_t)rows + max_ctas - 1) / max_ctas;
  if (slab < 1024) slab = 1024;
  slab = (slab + 255) / 256 * 256;
  int ctas = (int)(((int64_t)rows + slab - 1) / slab);
  float* partials = scratch_alloc(((int64_t)((ctas + 3) & ~3) * (feat + 1) + 4) * sizeof(float));
  if (!partials) return NAN;
  float* out = LO ? LO->ptr : scalar_slot();
  const float fn = (float)rows;
  cudaStream_t s = ctx().stream;
  float* pp = P ? P->ptr : nullptr;
  profile_mark(true);
  if (fast && feat == 16)
    linreg_stage1<16><<<ctas, kRThreads, dyn, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials, G->ptr, out);
  else if (fast && feat == 32)
    linreg_stage1<32><<<ctas, kRThreads, dyn, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials, G->ptr, out);
  else if (fast && feat == 8)
    linreg_stage1<8><<<ctas, kRThreads, dyn, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials, G->ptr, out);
  else if (fast && feat == 4)
    linreg_stage1<4><<<ctas, kRThreads, dyn, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials, G->ptr, out);
  else
    linreg_stage1_any<<<ctas, kRThreads, 0, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, feat, slab, fn, partials, G->ptr,
                                                 out);
  profile_mark(false);
  count_launch(1);
  float r = NAN;
  if (cuda_ok(cudaGetLastError(), "linreg launch")) r = LO ? 0.0f : wait_scalar();
  scratch_free(partials);
  return r;
}

float cleave_cuda_linreg_step_f32(cleave_buf x, cleave_buf y, cleave_buf w, cleave_buf pred_out, cleave_buf grad_out,
                                  int32_t rows, int32_t feat) {
  return linreg_impl(x, y, w, pred_out, grad_out, rows, feat, nullptr);
}

int32_t cleave_cuda_linreg_step_dev_f32(cleave_buf x, cleave_buf y, cleave_buf w, cleave_buf pred_out, cleave_buf grad_out,
                                        int32_t rows, int32_t feat, cleave_buf loss_out) {
  if (!loss_out) {
    ApiLock lock;
    return -set_error(CLEAVE_CUDA_ERR_ARG, "linreg_step_dev: the loss output handle is required");
  }
  const float r = linreg_impl(x, y, w, pred_out, grad_out, rows, feat, loss_out);
  return r == 0.0f ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free sum.
//
// Some callers may not allocate device memory at the moment they need a reduction: code that runs
// while another framework owns the device heap and forbids side allocations, latency-critical loops
// where a cudaMalloc (which can synchronise the whole device) is unacceptable, or processes that
// are already at their memory budget.  cleave_cuda_sum_f32 takes its partial-sum buffer from the
// library's pool, which may call cudaMalloc; the variant below keeps that buffer in a fixed
// device-resident array instead and touches neither the pool, the handle table nor the library
// context's memory (it reads the SM count and bumps the launch counter, nothing else).  The cost is that every
// GPU that loads the library carries the array until exit.
// ------------------------------------------------------------------------------------------------
namespace cleave {

constexpr int kNoAllocScratchFloats = kMaxPartials + 4;     // 1188 floats, 4752 bytes: partials, then the
                                                            // completion counter (byte offset 4736)

constexpr int64_t kNoAllocMaxLen = 2147483647ll;             // largest tensor an i32 shape can describe
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

// Device address of the array above, per device.  The symbol name is only a host-side stand-in;
// the address a kernel can use has to be asked for, once per device, with that device current.
static float* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};

static float* noalloc_scratch_for_current_device() {
  int dev = -1;
  if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return nullptr;
  if (dev < 0 || dev >= kNoAllocMaxDevices) {
    set_error(CLEAVE_CUDA_ERR_UNSUPPORTED, "sum_noalloc: device ordinal %d is outside the supported range [0, %d)", dev,
              kNoAllocMaxDevices);
    return nullptr;
  }
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    if (!cuda_ok(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)")) return nullptr;
    g_noalloc_ptr[dev] = p;
  }
  return g_noalloc_ptr[dev];
}

bool noalloc_poke_completion_word(unsigned long long value) {
  float* scratch = noalloc_scratch_for_current_device();
  if (!scratch) return false;
  return cuda_ok(cudaMemcpy(scratch + kMaxPartials, &value, sizeof(value), cudaMemcpyHostToDevice),
                 "cudaMemcpy(completion counter)");
}

}  // namespace cleave

extern "C" int32_t cleave_cuda_sum_noalloc_f32(const float* x_dev, int64_t len, float* out_dev, void* cuda_stream) {
  ApiLock lock;
  if (!x_dev || !out_dev)
    return -set_error(CLEAVE_CUDA_ERR_ARG, "sum_noalloc: input and output must be non-NULL device pointers");
  if (len <= 0)
    return -set_error(CLEAVE_CUDA_ERR_ARG, "sum_noalloc: length must be positive, got %lld", (long long)len);
  if (len > kNoAllocMaxLen)
    return -set_error(CLEAVE_CUDA_ERR_UNSUPPORTED,
                      "sum_noalloc: %lld elements exceed the maximum of %lld this entry point accepts",
                      (long long)len, (long long)kNoAllocMaxLen);
  if ((reinterpret_cast<uintptr_t>(x_dev) & 3u) || (reinterpret_cast<uintptr_t>(out_dev) & 3u))
    return -set_error(CLEAVE_CUDA_ERR_ARG, "sum_noalloc: pointers must be 4-byte aligned");
  float* scratch = noalloc_scratch_for_current_device();
  if (!scratch) return -cleave_cuda_last_error();
  cudaStream_t s = (cudaStream_t)cuda_stream;
  // Same slab rule and the same kernel as cleave_cuda_sum_f32, so the summation tree and
  // therefore the result are identical.  The CTAs write partials [0, ctas) and the last one to
  // finish reads exactly those, so no value left in the array by an earlier call is ever read.
  // The one word that must start at zero is the completion counter behind the partials.  It is cleared
  // on the caller's stream right before the kernel (a memset node: no allocation, ordered like the kernel
  // itself), so a value left behind by a call whose kernel never finished -- or by two calls that
  // overlapped, which is a caller error -- cannot make this call skip its final step.
  int64_t slab;
  int ctas;
  // The occupancy query reads kernel attributes only; it allocates nothing.
  static const int max_ctas = resident_ctas(reduce_kernel<SumRed>);
  slab_for(len, max_ctas, &slab, &ctas);
  unsigned int* done = reinterpret_cast<unsigned int*>(scratch + kMaxPartials);
  if (!cuda_ok(cudaMemsetAsync(done, 0, 2 * sizeof(unsigned int), s), "cudaMemsetAsync(completion counter)"))
    return -cleave_cuda_last_error();
  reduce_kernel<SumRed><<<ctas, kRThreads, 0, s>>>(x_dev, len, slab, scratch, aligned16(x_dev) ? 1 : 0,
                                                   Finish{out_dev, 1.0f, 0, nullptr, done});
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "sum_noalloc launch")) return -cleave_cuda_last_error();
  return CLEAVE_CUDA_OK;
}
