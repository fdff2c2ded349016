// Internal GEMM interface shared by the exact (SIMT) and tensor-core (tcgen05) paths.
#pragma once
#include <stdint.h>

#include "common.cuh"

namespace cleave {

// C[batch][m,n] = op(A) * op(B) (+ bias[n] per row, then activation).
// A is stored [m,k] (trans_a == 0) or [k,m]; B is stored [k,n] (trans_b == 0) or [n,k].
struct GemmArgs {
  const float* a;
  const float* b;
  float* c;
  int batch, m, n, k;
  int trans_a, trans_b;
  const float* bias;   // may be null
  int act;             // CLEAVE_ACT_*
  // Backward form: C = act'(y) (.) (op(A) * op(B)), the derivative of activation `dact` evaluated from its
  // OUTPUT y (same shape as C); null for a plain product.  Not combined with bias / act.
  const float* dact_y;
  int dact;
  // Optional low split parts (see split_lo in tc_common.cuh), each the shape of its tensor.  a_lo / b_lo: planes
  // the caller already holds for the operands (written by an earlier GEMM's c_lo or by split_lo_plane), so the
  // tensor-core path needs no operand pre-pass; c_lo: receives the low part of every value stored to C.
  const float* a_lo = nullptr;
  const float* b_lo = nullptr;
  float* c_lo = nullptr;
};

// Derivative of an activation, from the activation's output y, times the upstream value g: the same
// operation sequence as the elementwise tanh_bwd / sigmoid_bwd / relu_bwd kernels, so fusing it into a
// GEMM epilogue changes no bit.
__device__ __forceinline__ float dact_apply(float y, float g, int dact) {
  switch (dact) {
    case CLEAVE_ACT_TANH: return __fmul_rn(__fsub_rn(1.0f, __fmul_rn(y, y)), g);
    case CLEAVE_ACT_SIGMOID: return __fmul_rn(__fmul_rn(y, __fsub_rn(1.0f, y)), g);
    case CLEAVE_ACT_RELU: return y > 0.0f ? g : 0.0f;
    default: return g;
  }
}

bool launch_gemm_exact(const GemmArgs& g);
// dst[i] = low split part of src[i]; on_stream = nullptr: the library's stream
bool split_lo_plane(const float* src, float* dst, int64_t n, cudaStream_t on_stream = nullptr);
bool launch_gemm_3xtf32(const GemmArgs& g);   // false + error if the problem cannot use this path
bool gemm_3xtf32_supported(const GemmArgs& g);
// Cut of a partly filled last wave of 256 x 256 tiles (gemm_tc_pair.cu): returns the tiles of the wave that are cut along K
// and stores the K-runs per tile in *slices; 0 / 0 when the wave is left whole.  Host arithmetic only.
int gemm_cut_plan(int tiles, int num_kb, int sm_pairs, int* slices);
int gemm_batch_chunk(int64_t bytes_per_entry, int batch);   // batch entries per pass (workspace and grid limits)

}  // namespace cleave
