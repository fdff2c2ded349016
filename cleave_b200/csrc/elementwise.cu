// Streaming (HBM-bound) operators: Ring<Tensor> add/sub/mul/div/neg, activations, their
// derivative forms, bias + activation, SGD update, fill.
//
// Every kernel is a grid-stride loop over 128-bit words: each thread issues four independent
// 16-byte loads per operand before it touches the data, the grid is a whole number of CTAs
// per SM, and loads/stores carry streaming (evict-first) hints because nothing is re-read.
// Multi-step formulas use the non-contracting intrinsics (__fmul_rn, __fadd_rn, ...) so each
// step rounds exactly as the separate arith.* ops of the reference do.
#include <cmath>

#include "common.cuh"

namespace cleave {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 4;   // resident CTAs per SM the launch bounds guarantee (<= 64 registers/thread)
constexpr int kUnroll = 4;      // 16-byte loads in flight per operand per thread: 128 KiB per SM for a binary op

// ---- functors ---------------------------------------------------------------------------
struct AddOp { __device__ float operator()(float a, float b) const { return __fadd_rn(a, b); } };
struct SubOp { __device__ float operator()(float a, float b) const { return __fsub_rn(a, b); } };
struct MulOp { __device__ float operator()(float a, float b) const { return __fmul_rn(a, b); } };
struct DivOp { __device__ float operator()(float a, float b) const { return __fdiv_rn(a, b); } };
struct NegOp { __device__ float operator()(float a) const { return -a; } };
// arith.maximumf(x, 0): NaN propagates, max(-0, +0) = +0.
struct ReluOp { __device__ float operator()(float x) const { return x != x ? x : (x > 0.0f ? x : 0.0f); } };
struct ExpOp { __device__ float operator()(float x) const { return expf(x); } };
// negf -> exp -> addf(1, e) -> divf(1, denom), fused into one pass.
struct SigmoidOp {
  // 1/d as a correctly rounded reciprocal: the same value as the IEEE division 1.0f / d, cheaper
  __device__ float operator()(float x) const { return __frcp_rn(__fadd_rn(1.0f, expf(-x))); }
};
struct TanhOp { __device__ float operator()(float x) const { return tanhf(x); } };
struct IdentityOp { __device__ float operator()(float x) const { return x; } };
// (1 - y*y) * g
struct TanhBwdOp {
  __device__ float operator()(float y, float g) const { return __fmul_rn(__fsub_rn(1.0f, __fmul_rn(y, y)), g); }
};
// (y * (1 - y)) * g
struct SigmoidBwdOp {
  __device__ float operator()(float y, float g) const { return __fmul_rn(__fmul_rn(y, __fsub_rn(1.0f, y)), g); }
};
struct ReluBwdOp { __device__ float operator()(float x, float g) const { return x > 0.0f ? g : 0.0f; } };
// w - lr * (gscale * g); gscale == 1 is skipped so the plain form rounds like the reference's.
struct SgdOp {
  float lr, gscale;
  __device__ float operator()(float w, float g) const {
    float gg = gscale == 1.0f ? g : __fmul_rn(gscale, g);
    return __fsub_rn(w, __fmul_rn(lr, gg));
  }
};

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

template <class Op>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) unary_kernel(const float* __restrict__ a, float* __restrict__ o,
                                                         int64_t n, int vec, Op op) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    float4* o4 = reinterpret_cast<float4*>(o);
    for (int64_t base = tid; base < n4; base += nthreads * kUnroll) {
      float4 va[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int64_t i = base + u * nthreads;
        if (i < n4) va[u] = ld_stream(a4 + i);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int64_t i = base + u * nthreads;
        if (i < n4) {
          float4 r;
          r.x = op(va[u].x); r.y = op(va[u].y); r.z = op(va[u].z); r.w = op(va[u].w);
          st_stream(o4 + i, r);
        }
      }
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) o[i] = op(a[i]);
  } else {
    for (int64_t i = tid; i < n; i += nthreads) o[i] = op(a[i]);
  }
}

template <class Op>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) binary_kernel(const float* a, const float* b, float* o, int64_t n,
                                                          int vec, Op op) {
  // No __restrict__: the SGD update runs in place (o == a).
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(o);
    for (int64_t base = tid; base < n4; base += nthreads * kUnroll) {
      float4 va[kUnroll], vb[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int64_t i = base + u * nthreads;
        if (i < n4) { va[u] = ld_stream(a4 + i); vb[u] = ld_stream(b4 + i); }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int64_t i = base + u * nthreads;
        if (i < n4) {
          float4 r;
          r.x = op(va[u].x, vb[u].x); r.y = op(va[u].y, vb[u].y);
          r.z = op(va[u].z, vb[u].z); r.w = op(va[u].w, vb[u].w);
          st_stream(o4 + i, r);
        }
      }
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) o[i] = op(a[i], b[i]);
  } else {
    for (int64_t i = tid; i < n; i += nthreads) o[i] = op(a[i], b[i]);
  }
}

// o[r, c] = act(x[r, c] + bias[c]); vec requires cols % 4 == 0 and 16-byte aligned pointers.
template <class Act>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) bias_act_kernel(const float* __restrict__ x, const float* __restrict__ bias,
                                                            float* __restrict__ o, int64_t n, int cols, int vec,
                                                            Act act) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    const int cols4 = cols >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* b4 = reinterpret_cast<const float4*>(bias);
    float4* o4 = reinterpret_cast<float4*>(o);
    for (int64_t base = tid; base < n4; base += nthreads * kUnroll) {
      float4 vx[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int64_t i = base + u * nthreads;
        if (i < n4) vx[u] = ld_stream(x4 + i);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        int64_t i = base + u * nthreads;
        if (i < n4) {
          float4 vb = __ldg(b4 + (int)(i % cols4));
          float4 r;
          r.x = act(__fadd_rn(vx[u].x, vb.x)); r.y = act(__fadd_rn(vx[u].y, vb.y));
          r.z = act(__fadd_rn(vx[u].z, vb.z)); r.w = act(__fadd_rn(vx[u].w, vb.w));
          st_stream(o4 + i, r);
        }
      }
    }
  } else {
    for (int64_t i = tid; i < n; i += nthreads) o[i] = act(__fadd_rn(x[i], __ldg(bias + (int)(i % cols))));
  }
}

__global__ void __launch_bounds__(kThreads, kCtasPerSm) fill_kernel(float* __restrict__ o, int64_t n, float v, int vec) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec) {
    const int64_t n4 = n >> 2;
    float4* o4 = reinterpret_cast<float4*>(o);
    const float4 v4 = make_float4(v, v, v, v);
    for (int64_t i = tid; i < n4; i += nthreads) st_stream(o4 + i, v4);
    for (int64_t i = (n4 << 2) + tid; i < n; i += nthreads) o[i] = v;
  } else {
    for (int64_t i = tid; i < n; i += nthreads) o[i] = v;
  }
}

// ---- host-side launchers -------------------------------------------------------------------
static int grid_for(int64_t n, bool vec) {
  int64_t items = vec ? (n / 4 + kUnroll - 1) / kUnroll : n;
  return stream_grid(items, kThreads, kCtasPerSm);
}

template <class Op>
static bool launch_unary(const float* a, float* o, int64_t n, Op op) {
  bool vec = aligned16(a) && aligned16(o) && n >= 4;
  unary_kernel<Op><<<grid_for(n, vec), kThreads, 0, ctx().stream>>>(a, o, n, vec ? 1 : 0, op);
  count_launch();
  return cuda_ok(cudaGetLastError(), "unary kernel launch");
}

template <class Op>
static bool launch_binary(const float* a, const float* b, float* o, int64_t n, Op op) {
  bool vec = aligned16(a) && aligned16(b) && aligned16(o) && n >= 4;
  binary_kernel<Op><<<grid_for(n, vec), kThreads, 0, ctx().stream>>>(a, b, o, n, vec ? 1 : 0, op);
  count_launch();
  return cuda_ok(cudaGetLastError(), "binary kernel launch");
}

template <class Op>
static cleave_buf unary_api(cleave_buf x, const char* name, Op op) {
  ApiLock lock;
  Buf* a = as_buf(x, name);
  if (!a) return nullptr;
  Trace tr(name, "n=%lld", (long long)a->len);
  Buf* o = new_buf(a->len);
  if (!o) return nullptr;
  if (!launch_unary(a->ptr, o->ptr, a->len, op)) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

template <class Op>
static cleave_buf binary_api(cleave_buf x, cleave_buf y, const char* name, Op op) {
  ApiLock lock;
  Buf* a = as_buf(x, name);
  Buf* b = as_buf(y, name);
  if (!a || !b) return nullptr;
  if (a->len != b->len) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "%s: operands have %lld and %lld elements; shapes must match (no broadcasting)",
              name, (long long)a->len, (long long)b->len);
    return nullptr;
  }
  Trace tr(name, "n=%lld", (long long)a->len);
  Buf* o = new_buf(a->len);
  if (!o) return nullptr;
  if (!launch_binary(a->ptr, b->ptr, o->ptr, a->len, op)) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

bool launch_fill(float* o, int64_t n, float v) {
  bool vec = aligned16(o) && n >= 4;
  fill_kernel<<<stream_grid(vec ? n / 4 : n, kThreads, kCtasPerSm), kThreads, 0, ctx().stream>>>(o, n, v, vec ? 1 : 0);
  count_launch();
  return cuda_ok(cudaGetLastError(), "fill kernel launch");
}

bool launch_bias_act(const float* x, const float* bias, float* o, int64_t rows, int cols, int act) {
  int64_t n = rows * (int64_t)cols;
  bool vec = aligned16(x) && aligned16(bias) && aligned16(o) && (cols % 4 == 0);
  int grid = grid_for(n, vec);
  cudaStream_t s = ctx().stream;
  switch (act) {
    case CLEAVE_ACT_IDENTITY: bias_act_kernel<<<grid, kThreads, 0, s>>>(x, bias, o, n, cols, vec, IdentityOp{}); break;
    case CLEAVE_ACT_RELU: bias_act_kernel<<<grid, kThreads, 0, s>>>(x, bias, o, n, cols, vec, ReluOp{}); break;
    case CLEAVE_ACT_SIGMOID: bias_act_kernel<<<grid, kThreads, 0, s>>>(x, bias, o, n, cols, vec, SigmoidOp{}); break;
    case CLEAVE_ACT_TANH: bias_act_kernel<<<grid, kThreads, 0, s>>>(x, bias, o, n, cols, vec, TanhOp{}); break;
    default: set_error(CLEAVE_CUDA_ERR_ARG, "unknown activation code %d", act); return false;
  }
  count_launch();
  return cuda_ok(cudaGetLastError(), "bias_act kernel launch");
}

}  // namespace cleave

using namespace cleave;

extern "C" {

cleave_buf cleave_cuda_add_f32(cleave_buf a, cleave_buf b) { return binary_api(a, b, "add", AddOp{}); }
cleave_buf cleave_cuda_sub_f32(cleave_buf a, cleave_buf b) { return binary_api(a, b, "sub", SubOp{}); }
cleave_buf cleave_cuda_mul_f32(cleave_buf a, cleave_buf b) { return binary_api(a, b, "mul", MulOp{}); }
cleave_buf cleave_cuda_div_f32(cleave_buf a, cleave_buf b) { return binary_api(a, b, "div", DivOp{}); }
cleave_buf cleave_cuda_neg_f32(cleave_buf a) { return unary_api(a, "neg", NegOp{}); }

cleave_buf cleave_cuda_relu_f32(cleave_buf x) { return unary_api(x, "relu", ReluOp{}); }
cleave_buf cleave_cuda_sigmoid_f32(cleave_buf x) { return unary_api(x, "sigmoid", SigmoidOp{}); }
cleave_buf cleave_cuda_tanh_f32(cleave_buf x) { return unary_api(x, "tanh", TanhOp{}); }
cleave_buf cleave_cuda_exp_f32(cleave_buf x) { return unary_api(x, "exp", ExpOp{}); }

cleave_buf cleave_cuda_tanh_bwd_f32(cleave_buf y, cleave_buf g) { return binary_api(y, g, "tanh_bwd", TanhBwdOp{}); }
cleave_buf cleave_cuda_sigmoid_bwd_f32(cleave_buf y, cleave_buf g) {
  return binary_api(y, g, "sigmoid_bwd", SigmoidBwdOp{});
}
cleave_buf cleave_cuda_relu_bwd_f32(cleave_buf x, cleave_buf g) { return binary_api(x, g, "relu_bwd", ReluBwdOp{}); }

cleave_buf cleave_cuda_fill_f32(float value, int64_t len) {
  ApiLock lock;
  Buf* o = new_buf(len);
  if (!o) return nullptr;
  Trace tr("fill", "n=%lld", (long long)len);
  if (!launch_fill(o->ptr, len, value)) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

cleave_buf cleave_cuda_zeros_f32(int64_t len) { return cleave_cuda_fill_f32(0.0f, len); }

cleave_buf cleave_cuda_bias_act_f32(cleave_buf x, cleave_buf bias, int32_t rows, int32_t cols, int32_t act) {
  ApiLock lock;
  Buf* a = as_buf(x, "bias_act");
  Buf* b = as_buf(bias, "bias_act");
  if (!a || !b) return nullptr;
  if (rows <= 0 || cols <= 0 || a->len != (int64_t)rows * cols || b->len != cols) {
    set_error(CLEAVE_CUDA_ERR_SHAPE, "bias_act: x has %lld elements, bias %lld, for a %d x %d tensor",
              (long long)a->len, (long long)b->len, rows, cols);
    return nullptr;
  }
  Trace tr("bias_act", "rows=%d cols=%d act=%d", rows, cols, act);
  Buf* o = new_buf(a->len);
  if (!o) return nullptr;
  if (!launch_bias_act(a->ptr, b->ptr, o->ptr, rows, cols, act)) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

int32_t cleave_cuda_sgd_f32(cleave_buf w, cleave_buf g, float lr, float gscale) {
  ApiLock lock;
  Buf* a = as_buf(w, "sgd");
  Buf* b = as_buf(g, "sgd");
  if (!a || !b) return -cleave_cuda_last_error();
  if (a->len != b->len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "sgd: weights have %lld elements, gradient %lld", (long long)a->len,
                      (long long)b->len);
  Trace tr("sgd", "n=%lld", (long long)a->len);
  if (!launch_binary(a->ptr, b->ptr, a->ptr, a->len, SgdOp{lr, gscale})) return -cleave_cuda_last_error();
  return CLEAVE_CUDA_OK;
}

}  // extern "C"
