// f64 instances of the operator surface: the reference declares its tensor algebras for every
// `T: Float` (Ring<f64> stdlib/num/num.cleave:189-196, Activation<f64> stdlib/nn/nn.cleave:60-64,
// Tensor<T, Dims...> generic over T), so each f32 entry point has an f64 twin here.
//
// Streaming kernels move 128-bit words (two doubles) with the same structure as the f32 ones;
// reductions use the same single-launch, last-CTA-finishes scheme; matmul is the exact CUDA-core
// kernel (rounded multiply, then rounded add, k ascending: bit-identical to the reference loop --
// the tensor pipe has no f64 mode on this part).
#include <cmath>

#include "common.cuh"

namespace cleave {

constexpr int kT = 256;
constexpr int kCtas = 4;
constexpr int kU = 4;

struct DAdd { __device__ double operator()(double a, double b) const { return __dadd_rn(a, b); } };
struct DSub { __device__ double operator()(double a, double b) const { return __dsub_rn(a, b); } };
struct DMul { __device__ double operator()(double a, double b) const { return __dmul_rn(a, b); } };
struct DDiv { __device__ double operator()(double a, double b) const { return __ddiv_rn(a, b); } };
struct DNeg { __device__ double operator()(double a) const { return -a; } };
struct DRelu { __device__ double operator()(double x) const { return x != x ? x : (x > 0.0 ? x : 0.0); } };
struct DExp { __device__ double operator()(double x) const { return exp(x); } };
struct DSigmoid { __device__ double operator()(double x) const { return __ddiv_rn(1.0, __dadd_rn(1.0, exp(-x))); } };
struct DTanh { __device__ double operator()(double x) const { return tanh(x); } };
// Derivative rules times the upstream factor, each step rounded like the separate arith ops
// (stdlib/num/num.cleave:222-223; sigmoid through the chain of :123-136): y = forward output, x = forward input.
struct DTanhBwd { __device__ double operator()(double y, double g) const { return __dmul_rn(__dsub_rn(1.0, __dmul_rn(y, y)), g); } };
struct DSigmoidBwd { __device__ double operator()(double y, double g) const { return __dmul_rn(__dmul_rn(y, __dsub_rn(1.0, y)), g); } };
struct DReluBwd { __device__ double operator()(double x, double g) const { return x > 0.0 ? g : 0.0; } };
struct DSgd {   // w - lr * (gscale * g)
  double lr, gscale;
  __device__ double operator()(double w, double g) const {
    const double gg = gscale == 1.0 ? g : __dmul_rn(gscale, g);
    return __dsub_rn(w, __dmul_rn(lr, gg));
  }
};

template <class Op>
__global__ void __launch_bounds__(kT, kCtas) unary_f64_kernel(const double* __restrict__ a, double* __restrict__ o,
                                                               int64_t n, int vec, Op op) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n2 = n >> 1;
    const double2* a2 = reinterpret_cast<const double2*>(a);
    double2* o2 = reinterpret_cast<double2*>(o);
    for (int64_t base = tid; base < n2; base += nthreads * kU) {
      double2 v[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = base + u * nthreads;
        if (i < n2) v[u] = __ldcs(a2 + i);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = base + u * nthreads;
        if (i < n2) __stcs(o2 + i, make_double2(op(v[u].x), op(v[u].y)));
      }
    }
    for (int64_t i = (n2 << 1) + tid; i < n; i += nthreads) o[i] = op(a[i]);
  } else {
    for (int64_t i = tid; i < n; i += nthreads) o[i] = op(a[i]);
  }
}

template <class Op>
__global__ void __launch_bounds__(kT, kCtas) binary_f64_kernel(const double* a, const double* b, double* o, int64_t n,
                                                                int vec, Op op) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n2 = n >> 1;
    const double2* a2 = reinterpret_cast<const double2*>(a);
    const double2* b2 = reinterpret_cast<const double2*>(b);
    double2* o2 = reinterpret_cast<double2*>(o);
    for (int64_t base = tid; base < n2; base += nthreads * kU) {
      double2 va[kU], vb[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = base + u * nthreads;
        if (i < n2) { va[u] = __ldcs(a2 + i); vb[u] = __ldcs(b2 + i); }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int64_t i = base + u * nthreads;
        if (i < n2) __stcs(o2 + i, make_double2(op(va[u].x, vb[u].x), op(va[u].y, vb[u].y)));
      }
    }
    for (int64_t i = (n2 << 1) + tid; i < n; i += nthreads) o[i] = op(a[i], b[i]);
  } else {
    for (int64_t i = tid; i < n; i += nthreads) o[i] = op(a[i], b[i]);
  }
}

__global__ void __launch_bounds__(kT, kCtas) fill_f64_kernel(double* __restrict__ o, int64_t n, double v) {
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nthreads) o[i] = v;
}

// ---- reductions ------------------------------------------------------------------------------
struct DSum {
  static __device__ double identity() { return 0.0; }
  static __device__ double combine(double a, double b) { return __dadd_rn(a, b); }
};
struct DMax {   // skips NaN operands; the NaN-in-first-element rule is applied at the end
  static __device__ double identity() { return -INFINITY; }
  static __device__ double combine(double a, double b) { return fmax(a, b); }
};

template <class R>
__device__ __forceinline__ double warp_reduce_f64(double v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = R::combine(v, __shfl_down_sync(0xffffffffu, v, off));
  return v;
}
template <class R>
__device__ __forceinline__ double block_reduce_f64(double v) {
  __shared__ double part[kT / 32];
  v = warp_reduce_f64<R>(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) part[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < kT / 32 ? part[lane] : R::identity();
    v = warp_reduce_f64<R>(v);
  }
  return v;
}

constexpr int kMaxPartialsF64 = 148 * 8;
static __device__ unsigned int g_reduce_f64_done = 0;

// mode 0: out = total / divisor (1 skips the division); mode 1: out = total > v[0] ? total : v[0].
template <class R>
__global__ void __launch_bounds__(kT) reduce_f64_kernel(const double* __restrict__ v, int64_t n, int64_t slab,
                                                        double* __restrict__ partials, double* __restrict__ out,
                                                        double divisor, int mode, unsigned int* done) {
  const int64_t lo = (int64_t)blockIdx.x * slab;
  int64_t hi = lo + slab;
  if (hi > n) hi = n;
  double a0 = R::identity(), a1 = R::identity();
  const double2* v2 = reinterpret_cast<const double2*>(v);   // slab is even, v 16-byte aligned (pool block)
  const int64_t lo2 = lo >> 1, hi2 = hi >> 1;
  for (int64_t i = lo2 + threadIdx.x; i < hi2; i += kT) {
    const double2 x = __ldcs(v2 + i);
    a0 = R::combine(a0, x.x);
    a1 = R::combine(a1, x.y);
  }
  for (int64_t i = (hi2 << 1) + threadIdx.x; i < hi; i += kT) a0 = R::combine(a0, v[i]);
  double t = block_reduce_f64<R>(R::combine(a0, a1));
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = t;
    __threadfence();
    const unsigned int prev = atomicAdd(done, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) *done = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  double acc = R::identity();
  for (int i = threadIdx.x; i < (int)gridDim.x; i += kT) acc = R::combine(acc, __ldcg(partials + i));
  acc = block_reduce_f64<R>(acc);
  if (threadIdx.x == 0) {
    if (mode == 0) out[0] = divisor == 1.0 ? acc : __ddiv_rn(acc, divisor);
    else { const double f = v[0]; out[0] = acc > f ? acc : f; }
  }
}

// ---- exact matmul ----------------------------------------------------------------------------------
constexpr int kDM = 64, kDN = 64, kDK = 16;

// A is [m,k] (or [k,m] when ta), B is [k,n] (or [n,k] when tb); blockIdx.z walks the batch.
__global__ void __launch_bounds__(256) gemm_exact_f64_kernel(const double* __restrict__ A, const double* __restrict__ B,
                                                             double* __restrict__ C, int m, int n, int k, int ta, int tb) {
  __shared__ double As[kDK][kDM + 2];
  __shared__ double Bs[kDK][kDN + 2];
  A += (int64_t)blockIdx.z * m * k;
  B += (int64_t)blockIdx.z * k * n;
  C += (int64_t)blockIdx.z * m * n;
  const int m0 = blockIdx.y * kDM, n0 = blockIdx.x * kDN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  double acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;
  for (int k0 = 0; k0 < k; k0 += kDK) {
    for (int e = threadIdx.x; e < kDM * kDK; e += 256) {
      const int c = e % kDK, r = e / kDK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < m && gk < k) ? (ta ? A[(int64_t)gk * m + gm] : A[(int64_t)gm * k + gk]) : 0.0;
    }
    for (int e = threadIdx.x; e < kDN * kDK; e += 256) {
      const int c = e % kDN, r = e / kDN;
      const int gk = k0 + r, gn = n0 + c;
      Bs[r][c] = (gk < k && gn < n) ? (tb ? B[(int64_t)gn * k + gk] : B[(int64_t)gk * n + gn]) : 0.0;
    }
    __syncthreads();
    const int kmax = (k - k0) < kDK ? (k - k0) : kDK;
    for (int kk = 0; kk < kmax; ++kk) {
      double a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __dadd_rn(acc[i][j], __dmul_rn(a[i], b[j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < n) C[(int64_t)gm * n + gn] = acc[i][j];
    }
  }
}

// ---- column sums and the squared-error loss ---------------------------------------------------------------
// Column sums in two deterministic stages: stage 1 adds the rows of one split (rows r0, r0 + 1, ... in order)
// for one column per thread, stage 2 adds the splits in order.
__global__ void __launch_bounds__(256) colsum_f64_stage1(const double* __restrict__ x, int rows, int cols, int rows_per_split,
                                                         double* __restrict__ partials) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int r0 = blockIdx.y * rows_per_split;
  const int r1 = (r0 + rows_per_split) < rows ? (r0 + rows_per_split) : rows;
  double acc = 0.0;
  for (int r = r0; r < r1; ++r) acc = __dadd_rn(acc, x[(int64_t)r * cols + c]);
  partials[(int64_t)blockIdx.y * cols + c] = acc;
}
__global__ void __launch_bounds__(256) colsum_f64_stage2(const double* __restrict__ partials, int splits, int cols,
                                                         double* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  double acc = partials[c];
  for (int sp = 1; sp < splits; ++sp) acc = __dadd_rn(acc, partials[(int64_t)sp * cols + c]);
  out[c] = acc;
}
// e = p - t; sq = e * e; dp = (2 e) / n  -- the separate arith ops of the lowered program, one pass
__global__ void __launch_bounds__(kT, kCtas) mse_f64_kernel(const double* __restrict__ p, const double* __restrict__ t,
                                                            double* __restrict__ sq, double* __restrict__ dp, int64_t n,
                                                            double fn) {
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nthreads) {
    const double e = __dsub_rn(p[i], t[i]);
    sq[i] = __dmul_rn(e, e);
    if (dp) dp[i] = __ddiv_rn(__dmul_rn(2.0, e), fn);
  }
}

// ---- host side --------------------------------------------------------------------------------------
static inline double* dp(Buf* b) { return reinterpret_cast<double*>(b->ptr); }

static int grid_f64(int64_t n, bool vec) {
  const int64_t items = vec ? (n / 2 + kU - 1) / kU : n;
  return stream_grid(items, kT, kCtas);
}

template <class Op>
static cleave_buf unary_f64_api(cleave_buf x, const char* name, Op op) {
  ApiLock lock;
  Buf* a = as_buf(x, name, DT_F64);
  if (!a) return nullptr;
  Trace tr(name, "f64 n=%lld", (long long)a->len);
  Buf* o = new_buf(a->len, DT_F64);
  if (!o) return nullptr;
  const bool vec = aligned16(a->ptr) && aligned16(o->ptr) && a->len >= 2;
  unary_f64_kernel<Op><<<grid_f64(a->len, vec), kT, 0, ctx().stream>>>(dp(a), dp(o), a->len, vec ? 1 : 0, op);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "f64 unary launch")) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

template <class Op>
static cleave_buf binary_f64_api(cleave_buf x, cleave_buf y, const char* name, Op op) {
  ApiLock lock;
  Buf* a = as_buf(x, name, DT_F64);
  Buf* b = as_buf(y, name, DT_F64);
  if (!a || !b) return nullptr;
  if (a->len != b->len) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "%s: operands have %lld and %lld elements; shapes must match (no broadcasting)",
              name, (long long)a->len, (long long)b->len);
    return nullptr;
  }
  Trace tr(name, "f64 n=%lld", (long long)a->len);
  Buf* o = new_buf(a->len, DT_F64);
  if (!o) return nullptr;
  const bool vec = aligned16(a->ptr) && aligned16(b->ptr) && aligned16(o->ptr) && a->len >= 2;
  binary_f64_kernel<Op><<<grid_f64(a->len, vec), kT, 0, ctx().stream>>>(dp(a), dp(b), dp(o), a->len, vec ? 1 : 0, op);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "f64 binary launch")) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

template <class R>
static double reduce_f64_ptr(const double* data, int64_t n, double divisor_or_zero_for_len, int mode);

template <class R>
static double reduce_f64(cleave_buf v, const char* name, double divisor_or_zero_for_len, int mode) {
  ApiLock lock;
  Buf* a = as_buf(v, name, DT_F64);
  if (!a) return NAN;
  Trace tr(name, "f64 n=%lld", (long long)a->len);
  return reduce_f64_ptr<R>(dp(a), a->len, divisor_or_zero_for_len, mode);
}

template <class R>
static double reduce_f64_ptr(const double* data, int64_t n, double divisor_or_zero_for_len, int mode) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reduce_f64_kernel<R>, kT, 0) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    per_sm = 1;
  }
  int64_t max_ctas = (int64_t)per_sm * ctx().sm_count;
  if (max_ctas > kMaxPartialsF64) max_ctas = kMaxPartialsF64;
  int64_t slab = (n + max_ctas - 1) / max_ctas;
  if (slab < 2048) slab = 2048;
  slab = (slab + 1) / 2 * 2;
  const int ctas = (int)((n + slab - 1) / slab);
  double* partials = reinterpret_cast<double*>(scratch_alloc((kMaxPartialsF64 + 2) * sizeof(double)));
  if (!partials) return NAN;
  unsigned int* done = nullptr;
  cudaGetSymbolAddress((void**)&done, g_reduce_f64_done);
  const double divisor = divisor_or_zero_for_len == 0.0 ? (double)(int32_t)n : divisor_or_zero_for_len;
  reduce_f64_kernel<R><<<ctas, kT, 0, ctx().stream>>>(data, n, slab, partials, scalar_slot_f64(), divisor, mode, done);
  count_launch();
  double r = NAN;
  if (cuda_ok(cudaGetLastError(), "f64 reduction launch")) r = wait_scalar_f64();
  scratch_free(reinterpret_cast<float*>(partials));
  return r;
}

}  // namespace cleave

using namespace cleave;

extern "C" {

cleave_buf cleave_cuda_alloc_f64(int64_t len) {
  ApiLock lock;
  return (cleave_buf)new_buf(len, DT_F64);
}

cleave_buf cleave_cuda_upload_f64(const double* host, int64_t len) {
  ApiLock lock;
  if (!host) {
    set_error(CLEAVE_CUDA_ERR_ARG, "upload: NULL host pointer");
    return nullptr;
  }
  Buf* b = new_buf(len, DT_F64);
  if (!b) return nullptr;
  if (!cuda_ok(cudaMemcpyAsync(b->ptr, host, (size_t)len * sizeof(double), cudaMemcpyHostToDevice, ctx().stream),
               "cudaMemcpyAsync(H2D)") ||
      !cuda_ok(cudaStreamSynchronize(ctx().stream), "cudaStreamSynchronize")) {
    release_buf(b);
    return nullptr;
  }
  return (cleave_buf)b;
}

int64_t cleave_cuda_download_f64(cleave_buf t, double* host, int64_t len) {
  ApiLock lock;
  Buf* b = as_buf(t, "download", DT_F64);
  if (!b) return -cleave_cuda_last_error();
  if (!host || len != b->len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "download: room for %lld elements, tensor has %lld", (long long)len,
                      (long long)b->len);
  if (!cuda_ok(cudaMemcpyAsync(host, b->ptr, (size_t)len * sizeof(double), cudaMemcpyDeviceToHost, ctx().stream),
               "cudaMemcpyAsync(D2H)") ||
      !cuda_ok(cudaStreamSynchronize(ctx().stream), "cudaStreamSynchronize"))
    return -cleave_cuda_last_error();
  if (check_device_status() != CLEAVE_CUDA_OK) return -cleave_cuda_last_error();
  return len;
}

cleave_buf cleave_cuda_fill_f64(double value, int64_t len) {
  ApiLock lock;
  Buf* o = new_buf(len, DT_F64);
  if (!o) return nullptr;
  fill_f64_kernel<<<stream_grid(len, kT, kCtas), kT, 0, ctx().stream>>>(dp(o), len, value);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "f64 fill launch")) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

cleave_buf cleave_cuda_zeros_f64(int64_t len) { return cleave_cuda_fill_f64(0.0, len); }

double cleave_cuda_get_f64(cleave_buf t, int64_t i) {
  ApiLock lock;
  Buf* b = as_buf(t, "get", DT_F64);
  if (!b) return NAN;
  if (i < 0 || i >= b->len) {
    set_error(CLEAVE_CUDA_ERR_ARG, "get: index %lld outside [0, %lld)", (long long)i, (long long)b->len);
    return NAN;
  }
  double v = NAN;
  if (!cuda_ok(cudaMemcpyAsync(&v, dp(b) + i, sizeof(double), cudaMemcpyDeviceToHost, ctx().stream), "cudaMemcpyAsync") ||
      !cuda_ok(cudaStreamSynchronize(ctx().stream), "cudaStreamSynchronize"))
    return NAN;
  return v;
}

cleave_buf cleave_cuda_add_f64(cleave_buf a, cleave_buf b) { return binary_f64_api(a, b, "add", DAdd{}); }
cleave_buf cleave_cuda_sub_f64(cleave_buf a, cleave_buf b) { return binary_f64_api(a, b, "sub", DSub{}); }
cleave_buf cleave_cuda_mul_f64(cleave_buf a, cleave_buf b) { return binary_f64_api(a, b, "mul", DMul{}); }
cleave_buf cleave_cuda_div_f64(cleave_buf a, cleave_buf b) { return binary_f64_api(a, b, "div", DDiv{}); }
cleave_buf cleave_cuda_neg_f64(cleave_buf a) { return unary_f64_api(a, "neg", DNeg{}); }
cleave_buf cleave_cuda_relu_f64(cleave_buf x) { return unary_f64_api(x, "relu", DRelu{}); }
cleave_buf cleave_cuda_sigmoid_f64(cleave_buf x) { return unary_f64_api(x, "sigmoid", DSigmoid{}); }
cleave_buf cleave_cuda_tanh_f64(cleave_buf x) { return unary_f64_api(x, "tanh", DTanh{}); }
cleave_buf cleave_cuda_exp_f64(cleave_buf x) { return unary_f64_api(x, "exp", DExp{}); }

double cleave_cuda_sum_f64(cleave_buf v) { return reduce_f64<DSum>(v, "sum", 1.0, 0); }
double cleave_cuda_mean_f64(cleave_buf v) { return reduce_f64<DSum>(v, "mean", 0.0, 0); }
double cleave_cuda_max_f64(cleave_buf v) { return reduce_f64<DMax>(v, "max_of", 1.0, 1); }

static int gemm_f64_into(Buf* C, Buf* A, Buf* B, int batch, int m, int n, int k, int ta, int tb) {
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0)
    return set_error(CLEAVE_CUDA_ERR_ARG, "gemm_f64: batch, m, n, k must be positive (got %d, %d, %d, %d)", batch, m, n, k);
  if (A->len != (int64_t)batch * m * k || B->len != (int64_t)batch * k * n || C->len != (int64_t)batch * m * n)
    return set_error(CLEAVE_CUDA_ERR_SHAPE,
                     "gemm_f64: operand lengths %lld, %lld, %lld do not match batch %d of [%d x %d] * [%d x %d]",
                     (long long)A->len, (long long)B->len, (long long)C->len, batch, m, k, k, n);
  if (C->ptr == A->ptr || C->ptr == B->ptr)
    return set_error(CLEAVE_CUDA_ERR_ARG, "gemm_f64: the output must not alias an operand");
  if (batch > 65535 || ceil_div(m, kDM) > 65535)
    return set_error(CLEAVE_CUDA_ERR_UNSUPPORTED, "gemm_f64: batch %d / %d rows exceed the grid range", batch, m);
  Trace tr("gemm", "f64 batch=%d m=%d n=%d k=%d ta=%d tb=%d", batch, m, n, k, ta, tb);
  gemm_exact_f64_kernel<<<dim3(ceil_div(n, kDN), ceil_div(m, kDM), batch), 256, 0, ctx().stream>>>(dp(A), dp(B), dp(C), m, n,
                                                                                                  k, ta ? 1 : 0, tb ? 1 : 0);
  count_launch();
  return cuda_ok(cudaGetLastError(), "f64 GEMM launch") ? CLEAVE_CUDA_OK : cleave_cuda_last_error();
}

static cleave_buf gemm_f64_new(cleave_buf a, cleave_buf b, int batch, int m, int n, int k, int ta, int tb) {
  ApiLock lock;
  Buf* A = as_buf(a, "gemm_f64", DT_F64);
  Buf* B = as_buf(b, "gemm_f64", DT_F64);
  if (!A || !B) return nullptr;
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) {
    set_error(CLEAVE_CUDA_ERR_ARG, "gemm_f64: batch, m, n, k must be positive (got %d, %d, %d, %d)", batch, m, n, k);
    return nullptr;
  }
  Buf* C = new_buf((int64_t)batch * m * n, DT_F64);
  if (!C) return nullptr;
  if (gemm_f64_into(C, A, B, batch, m, n, k, ta, tb) != CLEAVE_CUDA_OK) { release_buf(C); return nullptr; }
  return (cleave_buf)C;
}

cleave_buf cleave_cuda_gemm_f64(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k) {
  return gemm_f64_new(a, b, 1, m, n, k, 0, 0);
}
cleave_buf cleave_cuda_gemm_nt_f64(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k) {
  return gemm_f64_new(a, b, 1, m, n, k, 0, 1);
}
cleave_buf cleave_cuda_gemm_tn_f64(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k) {
  return gemm_f64_new(a, b, 1, m, n, k, 1, 0);
}
cleave_buf cleave_cuda_gemm_batched_f64(cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n, int32_t k) {
  return gemm_f64_new(a, b, batch, m, n, k, 0, 0);
}

cleave_buf cleave_cuda_tanh_bwd_f64(cleave_buf y, cleave_buf g) { return binary_f64_api(y, g, "tanh_bwd", DTanhBwd{}); }
cleave_buf cleave_cuda_sigmoid_bwd_f64(cleave_buf y, cleave_buf g) {
  return binary_f64_api(y, g, "sigmoid_bwd", DSigmoidBwd{});
}
cleave_buf cleave_cuda_relu_bwd_f64(cleave_buf x, cleave_buf g) { return binary_f64_api(x, g, "relu_bwd", DReluBwd{}); }

int32_t cleave_cuda_sgd_f64(cleave_buf w, cleave_buf g, double lr, double gscale) {
  ApiLock lock;
  Buf* a = as_buf(w, "sgd", DT_F64);
  Buf* b = as_buf(g, "sgd", DT_F64);
  if (!a || !b) return -cleave_cuda_last_error();
  if (a->len != b->len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "sgd: weights have %lld elements, gradient %lld", (long long)a->len,
                      (long long)b->len);
  Trace tr("sgd", "f64 n=%lld", (long long)a->len);
  const bool vec = aligned16(a->ptr) && aligned16(b->ptr) && a->len >= 2;
  binary_f64_kernel<DSgd><<<grid_f64(a->len, vec), kT, 0, ctx().stream>>>(dp(a), dp(b), dp(a), a->len, vec ? 1 : 0,
                                                                          DSgd{lr, gscale});
  count_launch();
  return cuda_ok(cudaGetLastError(), "f64 sgd launch") ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

cleave_buf cleave_cuda_colsum_f64(cleave_buf x, int32_t rows, int32_t cols) {
  ApiLock lock;
  Buf* a = as_buf(x, "colsum", DT_F64);
  if (!a) return nullptr;
  if (rows <= 0 || cols <= 0 || a->len != (int64_t)rows * cols) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "colsum: tensor has %lld elements, not %d x %d", (long long)a->len, rows, cols);
    return nullptr;
  }
  Trace tr("colsum", "f64 rows=%d cols=%d", rows, cols);
  int splits = ceil_div(rows, 64);
  if (splits > 64) splits = 64;
  const int rows_per_split = ceil_div(rows, splits);
  splits = ceil_div(rows, rows_per_split);
  double* partials = reinterpret_cast<double*>(scratch_alloc((int64_t)splits * cols * sizeof(double)));
  if (!partials) return nullptr;
  Buf* o = new_buf(cols, DT_F64);
  if (!o) { scratch_free(reinterpret_cast<float*>(partials)); return nullptr; }
  colsum_f64_stage1<<<dim3(ceil_div(cols, 256), splits), 256, 0, ctx().stream>>>(dp(a), rows, cols, rows_per_split, partials);
  colsum_f64_stage2<<<ceil_div(cols, 256), 256, 0, ctx().stream>>>(partials, splits, cols, dp(o));
  count_launch(2);
  const bool ok = cuda_ok(cudaGetLastError(), "f64 colsum launch");
  scratch_free(reinterpret_cast<float*>(partials));
  if (!ok) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

double cleave_cuda_mse_f64(cleave_buf p, cleave_buf t, cleave_buf dpred) {
  ApiLock lock;
  Buf* a = as_buf(p, "mse", DT_F64);
  Buf* b = as_buf(t, "mse", DT_F64);
  if (!a || !b) return NAN;
  Buf* d = nullptr;
  if (dpred) {
    d = as_buf(dpred, "mse", DT_F64);
    if (!d) return NAN;
  }
  if (a->len != b->len || (d && d->len != a->len)) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "mse: prediction, target and gradient tensors must have the same length");
    return NAN;
  }
  const int64_t n = a->len;
  Trace tr("mse", "f64 n=%lld", (long long)n);
  double* sq = reinterpret_cast<double*>(scratch_alloc(n * (int64_t)sizeof(double)));
  if (!sq) return NAN;
  const double fn = (double)(int32_t)n;
  mse_f64_kernel<<<stream_grid(n, kT, kCtas), kT, 0, ctx().stream>>>(dp(a), dp(b), sq, d ? dp(d) : nullptr, n, fn);
  count_launch();
  double r = NAN;
  if (cuda_ok(cudaGetLastError(), "f64 mse launch")) r = reduce_f64_ptr<DSum>(sq, n, fn, 0);
  scratch_free(reinterpret_cast<float*>(sq));
  return r;
}

}  // extern "C"
