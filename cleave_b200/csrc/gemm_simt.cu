// Exact f32 GEMM on the CUDA cores: every output element is the chain
//   acc = +0;  acc = acc + (a * b)  for k = 0, 1, ...   (rounded multiply, then rounded add)
// which is the arithmetic of the reference's linalg.matmul region (mlir_lower.rs:2089-2120)
// after convert-linalg-to-loops, so results are bit-identical to the CPU path.  Used for small
// and oddly shaped problems and as the on-device cross-check of the tensor-core path.
#include "common.cuh"
#include "gemm.cuh"

namespace cleave {

constexpr int kTM = 64, kTN = 64, kTK = 16;

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case CLEAVE_ACT_RELU: return v != v ? v : (v > 0.0f ? v : 0.0f);
    case CLEAVE_ACT_SIGMOID: return __frcp_rn(__fadd_rn(1.0f, expf(-v)));
    case CLEAVE_ACT_TANH: return tanhf(v);
    default: return v;
  }
}

// A is [m,k] (or [k,m] when ta), B is [k,n] (or [n,k] when tb); 256 threads, 4x4 outputs each.
__global__ void __launch_bounds__(256) gemm_exact_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                         float* __restrict__ C, int m, int n, int k, int ta, int tb,
                                                         const float* __restrict__ bias, int act,
                                                         const float* __restrict__ dact_y, int dact) {
  __shared__ float As[kTK][kTM + 4];
  __shared__ float Bs[kTK][kTN + 4];
  const int64_t batch = blockIdx.z;
  A += batch * (int64_t)m * k;
  B += batch * (int64_t)k * n;
  C += batch * (int64_t)m * n;
  if (dact_y) dact_y += batch * (int64_t)m * n;
  const int m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < k; k0 += kTK) {
    // Cooperative loads: 64x16 elements of each operand, 4 per thread.  Positions outside the
    // problem are zero-filled; they only feed outputs that are never stored, and the k tail is
    // cut off below, so padding never enters a stored result.
    for (int e = threadIdx.x; e < kTM * kTK; e += 256) {
      int r, c;
      if (ta) { r = e % kTM; c = e / kTM; } else { c = e % kTK; r = e / kTK; }
      int gm = m0 + r, gk = k0 + c;
      float v = 0.0f;
      if (gm < m && gk < k) v = ta ? A[(int64_t)gk * m + gm] : A[(int64_t)gm * k + gk];
      As[c][r] = v;
    }
    for (int e = threadIdx.x; e < kTN * kTK; e += 256) {
      int r, c;   // r: k index within tile, c: n index within tile
      if (tb) { r = e % kTK; c = e / kTK; } else { c = e % kTN; r = e / kTN; }
      int gk = k0 + r, gn = n0 + c;
      float v = 0.0f;
      if (gk < k && gn < n) v = tb ? B[(int64_t)gn * k + gk] : B[(int64_t)gk * n + gn];
      Bs[r][c] = v;
    }
    __syncthreads();
    const int kmax = (k - k0) < kTK ? (k - k0) : kTK;
    for (int kk = 0; kk < kmax; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= n) continue;
      float v = acc[i][j];
      if (bias) v = __fadd_rn(v, bias[gn]);
      v = apply_act(v, act);
      if (dact_y) v = dact_apply(dact_y[(int64_t)gm * n + gn], v, dact);
      C[(int64_t)gm * n + gn] = v;
    }
  }
}

bool launch_gemm_exact(const GemmArgs& g) {
  // gridDim.y and .z hold at most 65535: a tall problem is cut into row bands (whole 64-row tiles, so every
  // element is computed exactly as in one launch) and a long batch into runs of entries.
  constexpr int kMaxGridYZ = 65535;
  const int band_rows = kMaxGridYZ * kTM;
  for (int b0 = 0; b0 < g.batch; b0 += kMaxGridYZ) {
    const int nb = (g.batch - b0) < kMaxGridYZ ? (g.batch - b0) : kMaxGridYZ;
    if (g.m > band_rows && nb > 1) {
      set_error(CLEAVE_CUDA_ERR_UNSUPPORTED, "exact GEMM: %d rows with a batch of %d is out of range", g.m, g.batch);
      return false;
    }
    for (int r0 = 0; r0 < g.m; r0 += band_rows) {
      const int rows = (g.m - r0) < band_rows ? (g.m - r0) : band_rows;
      // A band of a transposed A ([k, m], rows contiguous) is a column range: same leading dimension, so the
      // kernel would need a stride argument; such a shape (m > 4 Mi rows, trans_a) is refused instead.
      if (r0 > 0 && g.trans_a) {
        set_error(CLEAVE_CUDA_ERR_UNSUPPORTED, "exact GEMM: a transposed A with more than %d rows is out of range",
                  band_rows);
        return false;
      }
      const int64_t a_off = (int64_t)b0 * g.m * g.k + (int64_t)r0 * g.k;
      const int64_t c_off = (int64_t)b0 * g.m * g.n + (int64_t)r0 * g.n;
      dim3 grid(ceil_div(g.n, kTN), ceil_div(rows, kTM), nb);
      gemm_exact_kernel<<<grid, 256, 0, ctx().stream>>>(g.a + a_off, g.b + (int64_t)b0 * g.k * g.n, g.c + c_off, rows,
                                                        g.n, g.k, g.trans_a, g.trans_b, g.bias, g.act,
                                                        g.dact_y ? g.dact_y + c_off : nullptr, g.dact);
      count_launch();
    }
  }
  return cuda_ok(cudaGetLastError(), "exact GEMM launch");
}

}  // namespace cleave
