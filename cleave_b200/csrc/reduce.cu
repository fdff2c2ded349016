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

// Stage 1: each CTA owns a contiguous slab of the input (so partial b covers elements
// [b*slab, (b+1)*slab)), reads it as float4 with four loads in flight per thread.
// Elements are taken from index `first` on (max_of starts its scan at element 1).
template <class R>
__global__ void __launch_bounds__(kRThreads) reduce_stage1(const float* __restrict__ v, int64_t n, int64_t slab,
                                                           float* __restrict__ partials, int vec) {
  const int64_t lo = (int64_t)blockIdx.x * slab;
  int64_t hi = lo + slab;
  if (hi > n) hi = n;
  float acc[4] = {R::identity(), R::identity(), R::identity(), R::identity()};
  if (vec) {   // slab is a multiple of 4 and v is 16-byte aligned
    const float4* v4 = reinterpret_cast<const float4*>(v);
    const int64_t lo4 = lo >> 2, hi4 = hi >> 2;
    for (int64_t i = lo4 + threadIdx.x; i < hi4; i += kRThreads) {
      float4 x = __ldcs(v4 + i);
      acc[0] = R::combine(acc[0], x.x);
      acc[1] = R::combine(acc[1], x.y);
      acc[2] = R::combine(acc[2], x.z);
      acc[3] = R::combine(acc[3], x.w);
    }
    for (int64_t i = (hi4 << 2) + threadIdx.x; i < hi; i += kRThreads) acc[0] = R::combine(acc[0], v[i]);
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kRThreads) acc[0] = R::combine(acc[0], v[i]);
  }
  float t = R::combine(R::combine(acc[0], acc[1]), R::combine(acc[2], acc[3]));
  t = block_reduce<R>(t);
  if (threadIdx.x == 0) partials[blockIdx.x] = t;
}

// Stage 2: one CTA; thread t folds partials t, t+256, ... in ascending order, then a block tree.
// mode 0: out = total * scale.  mode 1 (max_of): out = (total > first) ? total : first.
template <class R>
__global__ void __launch_bounds__(kRThreads) reduce_stage2(const float* __restrict__ partials, int count,
                                                           float* __restrict__ out, float scale_or_unused, int mode,
                                                           const float* __restrict__ first) {
  float acc = R::identity();
  for (int i = threadIdx.x; i < count; i += kRThreads) acc = R::combine(acc, partials[i]);
  acc = block_reduce<R>(acc);
  if (threadIdx.x == 0) {
    if (mode == 0) {
      out[0] = scale_or_unused == 1.0f ? acc : __fdiv_rn(acc, scale_or_unused);
    } else {
      float f = first[0];
      out[0] = acc > f ? acc : f;
    }
  }
}

// ---- column sums: x[rows, cols] -> out[cols] ------------------------------------------------
// grid = (column strips of 128 floats, row splits).  Thread (tx, ty) owns one float4 column
// group and the rows ty, ty+8, ... of its split; the 8 row-threads are combined through
// shared memory in ty order; splits are combined by the second stage in split order.
constexpr int kCsTx = 32, kCsTy = 8;

__global__ void __launch_bounds__(kCsTx* kCsTy) colsum_stage1(const float* __restrict__ x, int rows, int cols,
                                                               int rows_per_split, float* __restrict__ partials,
                                                               int vec) {
  __shared__ float4 sm[kCsTy][kCsTx];
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

__global__ void __launch_bounds__(kRThreads) mse_stage1(const float* __restrict__ p, const float* __restrict__ t,
                                                        float* __restrict__ dp, int64_t n, int64_t slab, float fn,
                                                        float* __restrict__ partials, int vec, int bwd_act) {
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
      }
    }
    for (int64_t i = (hi4 << 2) + threadIdx.x; i < hi; i += kRThreads) {
      float e = __fsub_rn(p[i], t[i]);
      acc = __fadd_rn(acc, __fmul_rn(e, e));
      if (dp) dp[i] = mse_grad(p[i], e, fn, bwd_act);
    }
  } else {
    for (int64_t i = lo + threadIdx.x; i < hi; i += kRThreads) {
      float e = __fsub_rn(p[i], t[i]);
      acc = __fadd_rn(acc, __fmul_rn(e, e));
      if (dp) dp[i] = mse_grad(p[i], e, fn, bwd_act);
    }
  }
  acc = block_reduce<SumRed>(acc);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

// ---- linear-regression step: one sweep over X[rows, feat] ------------------------------------
// Each thread owns whole rows: pred_i = sum_f X[i,f] w[f] (f ascending, multiply then add, so
// pred is bit-identical to the reference's matmul), e = pred - y, accumulates e^2 and
// X[i,f] * (2 e / rows) per feature.  Per-CTA partials: [feat] gradient sums, then the loss sum.
constexpr int kMaxFeat = 32;

template <int FEAT>
__global__ void __launch_bounds__(kRThreads) linreg_stage1(const float* __restrict__ X, const float* __restrict__ y,
                                                           const float* __restrict__ w, float* __restrict__ pred,
                                                           int64_t rows, int64_t slab, float fn,
                                                           float* __restrict__ partials) {
  // Each warp takes 32 consecutive rows at a time.  The 32*FEAT floats of such a group are
  // contiguous in X, so the warp reads them with fully coalesced 16-byte loads (lane l takes
  // 16-byte words l, l+32, ...), parks them in a warp-private shared tile and every lane then
  // picks up ITS row.  Words of row r are stored at slot q ^ swz(r), which makes both the
  // coalesced writes and the row-wise 16-byte reads bank-conflict free.
  static_assert(FEAT % 4 == 0 && FEAT >= 4 && FEAT <= 32, "FEAT must be 4, 8, 16 or 32");
  constexpr int Q = FEAT / 4;                 // 16-byte words per row
  constexpr int kRowsPerSwz = Q >= 8 ? 1 : 8 / Q;
  __shared__ float sw[FEAT];
  __shared__ float4 tile[kRWarps][32 * Q];
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
  float4* my_tile = tile[warp];
  const int my_swz = (lane / kRowsPerSwz) & (Q - 1);
  for (int64_t r0 = lo + (int64_t)warp * 32; r0 < hi; r0 += (int64_t)kRWarps * 32) {
    const float4* src = reinterpret_cast<const float4*>(X + r0 * FEAT);
    float4 v[Q];
#pragma unroll
    for (int i = 0; i < Q; ++i) {
      const int idx = lane + 32 * i;
      v[i] = (r0 + idx / Q < hi) ? __ldcs(src + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < Q; ++i) {
      const int idx = lane + 32 * i;
      const int r = idx / Q, q = idx % Q;
      my_tile[r * Q + (q ^ ((r / kRowsPerSwz) & (Q - 1)))] = v[i];
    }
    __syncwarp();
    float xr[FEAT];
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const float4 t = my_tile[lane * Q + (q ^ my_swz)];
      xr[4 * q] = t.x; xr[4 * q + 1] = t.y; xr[4 * q + 2] = t.z; xr[4 * q + 3] = t.w;
    }
    __syncwarp();
    const int64_t i = r0 + lane;
    if (i < hi) {
      float acc = 0.0f;
#pragma unroll
      for (int f = 0; f < FEAT; ++f) acc = __fadd_rn(acc, __fmul_rn(xr[f], sw[f]));
      if (pred) pred[i] = acc;
      const float e = __fsub_rn(acc, __ldcs(y + i));
      loss = __fadd_rn(loss, __fmul_rn(e, e));
      const float d = __fdiv_rn(__fmul_rn(2.0f, e), fn);
#pragma unroll
      for (int f = 0; f < FEAT; ++f) g[f] = __fadd_rn(g[f], __fmul_rn(xr[f], d));
    }
  }
#pragma unroll
  for (int f = 0; f < FEAT; ++f) {
    float t = block_reduce<SumRed>(g[f]);
    if (threadIdx.x == 0) partials[(int64_t)f * gridDim.x + blockIdx.x] = t;
  }
  loss = block_reduce<SumRed>(loss);
  if (threadIdx.x == 0) partials[(int64_t)FEAT * gridDim.x + blockIdx.x] = loss;
}

// Generic-feat fallback (feat <= 32, any value): same arithmetic, runtime loops.
__global__ void __launch_bounds__(kRThreads) linreg_stage1_any(const float* __restrict__ X, const float* __restrict__ y,
                                                               const float* __restrict__ w, float* __restrict__ pred,
                                                               int64_t rows, int feat, int64_t slab, float fn,
                                                               float* __restrict__ partials) {
  __shared__ float sw[kMaxFeat];
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
      if (threadIdx.x == 0) partials[(int64_t)f * gridDim.x + blockIdx.x] = t;
    }
  }
  loss = block_reduce<SumRed>(loss);
  if (threadIdx.x == 0) partials[(int64_t)feat * gridDim.x + blockIdx.x] = loss;
}

// Stage 2: one warp per quantity (feat gradient components, then the loss).  The partials of
// quantity f are contiguous (partials[f][cta]); lane l folds entries l, l+32, ... in ascending
// order and the 32 lane sums are combined by a fixed shuffle tree: deterministic.
// grad[0..feat) = gradient, loss_out[0] = loss sum / rows.
__global__ void __launch_bounds__(1024) linreg_stage2(const float* __restrict__ partials, int ctas, int feat, float fn,
                                                     float* __restrict__ grad, float* __restrict__ loss_out) {
  const int lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int f = threadIdx.x >> 5; f <= feat; f += nwarps) {
    const float* col = partials + (int64_t)f * ctas;
    float acc = 0.0f;
    for (int b = lane; b < ctas; b += 32) acc = __fadd_rn(acc, col[b]);
    acc = warp_reduce<SumRed>(acc);
    if (lane == 0) {
      if (f < feat) grad[f] = acc;
      else loss_out[0] = __fdiv_rn(acc, fn);
    }
  }
}

// ---- host side -------------------------------------------------------------------------------
// Slab size (elements per first-stage CTA): at least 4096 elements, a multiple of 4, and no
// more CTAs than can be resident at once for the kernel in question (one wave: a second,
// partial wave would cost as much as the first).  A function of n and of the device model only,
// so the summation tree is reproducible.
template <class Kernel>
static int resident_ctas(Kernel kernel) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kRThreads, 0) != cudaSuccess || per_sm < 1) {
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
  float* partials = scratch_alloc((kMaxPartials + 4) * sizeof(float));
  if (!partials) return NAN;
  float* out = scalar_slot();
  cudaStream_t s = ctx().stream;
  int ctas = 0;
  if (cnt > 0) {
    int64_t slab;
    static const int max_ctas = resident_ctas(reduce_stage1<R>);
    slab_for(cnt, max_ctas, &slab, &ctas);
    int vec = aligned16(base) ? 1 : 0;
    reduce_stage1<R><<<ctas, kRThreads, 0, s>>>(base, cnt, slab, partials, vec);
    count_launch();
  }
  reduce_stage2<R><<<1, kRThreads, 0, s>>>(partials, ctas, out, divisor, mode, v);
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

static bool colsum_launch(const float* x, float* out, int rows, int cols) {
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
  cudaStream_t s = ctx().stream;
  colsum_stage1<<<dim3(strips, splits), kCsTx * kCsTy, 0, s>>>(x, rows, cols, rows_per_split, partials, vec);
  colsum_stage2<<<ceil_div(cols, kRThreads), kRThreads, 0, s>>>(partials, splits, cols, out);
  count_launch(2);
  bool ok = cuda_ok(cudaGetLastError(), "colsum launch");
  scratch_free(partials);
  return ok;
}

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
  if (!colsum_launch(a->ptr, o->ptr, rows, cols)) { release_buf(o); return nullptr; }
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
  return colsum_launch(a->ptr, o->ptr, rows, cols) ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

// loss_dev == nullptr: the loss is returned (the call waits for it).  Otherwise it is written to
// that one-element device tensor, nothing is waited for, and 0 is returned on success.
static float mse_impl(cleave_buf p, cleave_buf t, cleave_buf dp, int bwd_act, const char* name,
                      cleave_buf loss_dev = nullptr) {
  ApiLock lock;
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
  float* partials = scratch_alloc((kMaxPartials + 4) * sizeof(float));
  if (!partials) return NAN;
  int64_t slab;
  int ctas;
  static const int max_ctas = resident_ctas(mse_stage1);
  slab_for(n, max_ctas, &slab, &ctas);
  int vec = (aligned16(a->ptr) && aligned16(b->ptr) && (!d || aligned16(d->ptr))) ? 1 : 0;
  const float fn = (float)(int32_t)n;
  cudaStream_t s = ctx().stream;
  float* out = lo ? lo->ptr : scalar_slot();
  mse_stage1<<<ctas, kRThreads, 0, s>>>(a->ptr, b->ptr, d ? d->ptr : nullptr, n, slab, fn, partials, vec, bwd_act);
  reduce_stage2<SumRed><<<1, kRThreads, 0, s>>>(partials, ctas, out, fn, 0, nullptr);
  count_launch(2);
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

float cleave_cuda_mse_act_bwd_f32(cleave_buf y, cleave_buf t, cleave_buf dz, int32_t act) {
  if (!dz) {
    ApiLock lock;
    set_error(CLEAVE_CUDA_ERR_ARG, "mse_act_bwd: the gradient output handle is required");
    return NAN;
  }
  return mse_impl(y, t, dz, act, "mse_act_bwd");
}

float cleave_cuda_linreg_step_f32(cleave_buf x, cleave_buf y, cleave_buf w, cleave_buf pred_out, cleave_buf grad_out,
                                  int32_t rows, int32_t feat) {
  ApiLock lock;
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
  // Row slabs: one resident wave of CTAs, at least 1024 rows each, a multiple of 256 rows (8 warps x 32).
  int max_ctas;
  switch (feat) {
    case 4: max_ctas = resident_ctas(linreg_stage1<4>); break;
    case 8: max_ctas = resident_ctas(linreg_stage1<8>); break;
    case 16: max_ctas = resident_ctas(linreg_stage1<16>); break;
    case 32: max_ctas = resident_ctas(linreg_stage1<32>); break;
    default: max_ctas = resident_ctas(linreg_stage1_any); break;
  }
  int64_t slab = ((int64_t)rows + max_ctas - 1) / max_ctas;
  if (slab < 1024) slab = 1024;
  slab = (slab + 255) / 256 * 256;
  int ctas = (int)(((int64_t)rows + slab - 1) / slab);
  float* partials = scratch_alloc(((int64_t)ctas * (feat + 1) + 4) * sizeof(float));
  if (!partials) return NAN;
  float* out = scalar_slot();
  const float fn = (float)rows;
  cudaStream_t s = ctx().stream;
  float* pp = P ? P->ptr : nullptr;
  profile_mark(true);
  if (feat == 16 && aligned16(X->ptr))
    linreg_stage1<16><<<ctas, kRThreads, 0, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials);
  else if (feat == 32 && aligned16(X->ptr))
    linreg_stage1<32><<<ctas, kRThreads, 0, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials);
  else if (feat == 8 && aligned16(X->ptr))
    linreg_stage1<8><<<ctas, kRThreads, 0, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials);
  else if (feat == 4 && aligned16(X->ptr))
    linreg_stage1<4><<<ctas, kRThreads, 0, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, slab, fn, partials);
  else
    linreg_stage1_any<<<ctas, kRThreads, 0, s>>>(X->ptr, Y->ptr, W->ptr, pp, rows, feat, slab, fn, partials);
  linreg_stage2<<<1, 32 * (feat + 1 > 32 ? 32 : feat + 1), 0, s>>>(partials, ctas, feat, fn, G->ptr, out);
  profile_mark(false);
  count_launch(2);
  float r = NAN;
  if (cuda_ok(cudaGetLastError(), "linreg launch")) r = wait_scalar();
  scratch_free(partials);
  return r;
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
// context.  The cost is that every GPU that loads the library carries the array until exit.
// ------------------------------------------------------------------------------------------------
namespace cleave {

constexpr int kNoAllocScratchFloats = kMaxPartials + 4;     // 1188 floats, 4752 bytes
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
  // Same slab rule and the same two kernels as cleave_cuda_sum_f32, so the summation tree and
  // therefore the result are identical.  Stage 1 writes partials [0, ctas) and stage 2 reads
  // exactly those, so nothing left in the array by an earlier call is ever read and nothing has
  // to be cleared first.
  int64_t slab;
  int ctas;
  // The occupancy query reads kernel attributes only; it allocates nothing.
  static const int max_ctas = resident_ctas(reduce_stage1<SumRed>);
  slab_for(len, max_ctas, &slab, &ctas);
  reduce_stage1<SumRed><<<ctas, kRThreads, 0, s>>>(x_dev, len, slab, scratch, aligned16(x_dev) ? 1 : 0);
  reduce_stage2<SumRed><<<1, kRThreads, 0, s>>>(scratch, ctas, out_dev, 1.0f, 0, nullptr);
  count_launch(2);
  if (!cuda_ok(cudaGetLastError(), "sum_noalloc launch")) return -cleave_cuda_last_error();
  return CLEAVE_CUDA_OK;
}
