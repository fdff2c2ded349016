// Internal GEMM interface shared by the exact (SIMT) and tensor-core (tcgen05) paths.
#pragma once
#include <stdint.h>

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
};

bool launch_gemm_exact(const GemmArgs& g);
bool launch_gemm_3xtf32(const GemmArgs& g);   // false + error if the problem cannot use this path
bool gemm_3xtf32_supported(const GemmArgs& g);

}  // namespace cleave
