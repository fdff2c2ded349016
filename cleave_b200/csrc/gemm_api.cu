// C-ABI entry points of the MatMul family and the choice between the two GEMM paths.
#include <cstdlib>

#include "common.cuh"
#include "gemm.cuh"

namespace cleave {

// Below this many multiply-adds the exact CUDA-core kernel is used: the pre-pass and pipeline
// fill of the tensor-core path cost more than they save, and the result is bit-identical to
// the reference's loop.
constexpr int64_t kTensorCoreMinMacs = 1ll << 24;

static bool run_gemm(const GemmArgs& g, int algo) {
  if (algo == CLEAVE_GEMM_AUTO) {
    const int64_t macs = (int64_t)g.batch * g.m * g.n * g.k;
    algo = (macs >= kTensorCoreMinMacs && g.m >= 64 && g.n >= 64 && gemm_3xtf32_supported(g)) ? CLEAVE_GEMM_3XTF32
                                                                                              : CLEAVE_GEMM_EXACT;
  }
  // The exact kernel has no lo-plane output of its own: the plane is written by a pass over the finished C.
  if (algo == CLEAVE_GEMM_EXACT)
    return launch_gemm_exact(g) && (!g.c_lo || split_lo_plane(g.c, g.c_lo, (int64_t)g.batch * g.m * g.n));
  if (algo == CLEAVE_GEMM_3XTF32) return launch_gemm_3xtf32(g);
  set_error(CLEAVE_CUDA_ERR_ARG, "gemm: unknown algorithm code %d", algo);
  return false;
}

static int gemm_into(Buf* C, Buf* A, Buf* B, int batch, int m, int n, int k, int ta, int tb, int algo, Buf* bias,
                     int act, Buf* dact_y = nullptr, int dact = CLEAVE_ACT_IDENTITY, Buf* a_lo = nullptr,
                     Buf* b_lo = nullptr, Buf* c_lo = nullptr) {
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0)
    return set_error(CLEAVE_CUDA_ERR_ARG, "gemm: batch, m, n, k must be positive (got %d, %d, %d, %d)", batch, m, n, k);
  if (A->len != (int64_t)batch * m * k || B->len != (int64_t)batch * k * n || C->len != (int64_t)batch * m * n)
    return set_error(CLEAVE_CUDA_ERR_SHAPE,
                     "gemm: operand lengths %lld, %lld, %lld do not match batch %d of [%d x %d] * [%d x %d]",
                     (long long)A->len, (long long)B->len, (long long)C->len, batch, m, k, k, n);
  if (bias && bias->len != n)
    return set_error(CLEAVE_CUDA_ERR_SHAPE, "gemm: bias has %lld elements, n is %d", (long long)bias->len, n);
  if (act < CLEAVE_ACT_IDENTITY || act > CLEAVE_ACT_TANH)
    return set_error(CLEAVE_CUDA_ERR_ARG, "gemm: unknown activation code %d", act);
  if (C->ptr == A->ptr || C->ptr == B->ptr)
    return set_error(CLEAVE_CUDA_ERR_ARG, "gemm: the output must not alias an operand");
  if (dact_y) {
    if (dact_y->len != C->len)
      return set_error(CLEAVE_CUDA_ERR_SHAPE, "gemm_dact: y has %lld elements, the product %lld",
                       (long long)dact_y->len, (long long)C->len);
    if (dact < CLEAVE_ACT_IDENTITY || dact > CLEAVE_ACT_TANH)
      return set_error(CLEAVE_CUDA_ERR_ARG, "gemm_dact: unknown activation code %d", dact);
    if (dact_y->ptr == C->ptr)
      return set_error(CLEAVE_CUDA_ERR_ARG, "gemm_dact: the output must not alias y");
  }
  Trace tr(dact_y ? "gemm_dact" : "gemm", "batch=%d m=%d n=%d k=%d ta=%d tb=%d algo=%d act=%d", batch, m, n, k, ta ? 1 : 0,
           tb ? 1 : 0, algo, dact_y ? dact : act);
  if ((a_lo && a_lo->len != A->len) || (b_lo && b_lo->len != B->len) || (c_lo && c_lo->len != C->len))
    return set_error(CLEAVE_CUDA_ERR_SHAPE, "gemm_fused: a lo plane must have as many elements as its tensor");
  if (c_lo && (c_lo->ptr == C->ptr || c_lo->ptr == A->ptr || c_lo->ptr == B->ptr))
    return set_error(CLEAVE_CUDA_ERR_ARG, "gemm_fused: the output lo plane must not alias C or an operand");
  GemmArgs g{A->ptr, B->ptr, C->ptr, batch, m, n, k, ta ? 1 : 0, tb ? 1 : 0, bias ? bias->ptr : nullptr, act,
             dact_y ? dact_y->ptr : nullptr, dact};
  g.a_lo = a_lo ? a_lo->ptr : nullptr;
  g.b_lo = b_lo ? b_lo->ptr : nullptr;
  g.c_lo = c_lo ? c_lo->ptr : nullptr;
  if (!run_gemm(g, algo)) return cleave_cuda_last_error();
  return CLEAVE_CUDA_OK;
}

static cleave_buf gemm_new(cleave_buf a, cleave_buf b, int batch, int m, int n, int k, int ta, int tb) {
  ApiLock lock;
  Buf* A = as_buf(a, "gemm");
  Buf* B = as_buf(b, "gemm");
  if (!A || !B) return nullptr;
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) {
    set_error(CLEAVE_CUDA_ERR_ARG, "gemm: batch, m, n, k must be positive (got %d, %d, %d, %d)", batch, m, n, k);
    return nullptr;
  }
  Buf* C = new_buf((int64_t)batch * m * n);
  if (!C) return nullptr;
  if (gemm_into(C, A, B, batch, m, n, k, ta, tb, CLEAVE_GEMM_AUTO, nullptr, CLEAVE_ACT_IDENTITY) != CLEAVE_CUDA_OK) {
    release_buf(C);
    return nullptr;
  }
  return (cleave_buf)C;
}

}  // namespace cleave

using namespace cleave;

extern "C" {

cleave_buf cleave_cuda_gemm_f32(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k) {
  return gemm_new(a, b, 1, m, n, k, 0, 0);
}
cleave_buf cleave_cuda_gemm_nt_f32(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k) {
  return gemm_new(a, b, 1, m, n, k, 0, 1);
}
cleave_buf cleave_cuda_gemm_tn_f32(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k) {
  return gemm_new(a, b, 1, m, n, k, 1, 0);
}
cleave_buf cleave_cuda_gemm_batched_f32(cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n, int32_t k) {
  return gemm_new(a, b, batch, m, n, k, 0, 0);
}

int32_t cleave_cuda_gemm_ex_f32(cleave_buf c, cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n,
                                int32_t k, int32_t trans_a, int32_t trans_b, int32_t algo, cleave_buf bias,
                                int32_t act) {
  ApiLock lock;
  Buf* C = as_buf(c, "gemm_ex");
  Buf* A = as_buf(a, "gemm_ex");
  Buf* B = as_buf(b, "gemm_ex");
  if (!C || !A || !B) return -cleave_cuda_last_error();
  Buf* bi = nullptr;
  if (bias) {
    bi = as_buf(bias, "gemm_ex");
    if (!bi) return -cleave_cuda_last_error();
  }
  int r = gemm_into(C, A, B, batch, m, n, k, trans_a, trans_b, algo, bi, act);
  return r == CLEAVE_CUDA_OK ? CLEAVE_CUDA_OK : -r;
}

int32_t cleave_cuda_gemm_dact_f32(cleave_buf c, cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n,
                                  int32_t k, int32_t trans_a, int32_t trans_b, int32_t algo, cleave_buf y,
                                  int32_t act) {
  ApiLock lock;
  Buf* C = as_buf(c, "gemm_dact");
  Buf* A = as_buf(a, "gemm_dact");
  Buf* B = as_buf(b, "gemm_dact");
  Buf* Y = as_buf(y, "gemm_dact");
  if (!C || !A || !B || !Y) return -cleave_cuda_last_error();
  int r = gemm_into(C, A, B, batch, m, n, k, trans_a, trans_b, algo, nullptr, CLEAVE_ACT_IDENTITY, Y, act);
  return r == CLEAVE_CUDA_OK ? CLEAVE_CUDA_OK : -r;
}

int32_t cleave_cuda_gemm_fused_f32(cleave_buf c, cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n,
                                   int32_t k, int32_t trans_a, int32_t trans_b, int32_t algo, cleave_buf bias,
                                   int32_t act, cleave_buf y, int32_t dact, cleave_buf a_lo, cleave_buf b_lo,
                                   cleave_buf c_lo) {
  ApiLock lock;
  Buf* C = as_buf(c, "gemm_fused");
  Buf* A = as_buf(a, "gemm_fused");
  Buf* B = as_buf(b, "gemm_fused");
  if (!C || !A || !B) return -cleave_cuda_last_error();
  Buf* opt[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  cleave_buf given[5] = {bias, y, a_lo, b_lo, c_lo};
  for (int i = 0; i < 5; ++i)
    if (given[i]) {
      opt[i] = as_buf(given[i], "gemm_fused");
      if (!opt[i]) return -cleave_cuda_last_error();
    }
  if (opt[0] && opt[1])
    return -set_error(CLEAVE_CUDA_ERR_ARG, "gemm_fused: bias + activation and the backward form exclude each other");
  if (opt[1] && act != CLEAVE_ACT_IDENTITY)
    return -set_error(CLEAVE_CUDA_ERR_ARG, "gemm_fused: the backward form takes no forward activation");
  int r = gemm_into(C, A, B, batch, m, n, k, trans_a, trans_b, algo, opt[0], act, opt[1], opt[1] ? dact : CLEAVE_ACT_IDENTITY,
                    opt[2], opt[3], opt[4]);
  return r == CLEAVE_CUDA_OK ? CLEAVE_CUDA_OK : -r;
}

int32_t cleave_cuda_dense_grads_f32(cleave_buf dw, cleave_buf db, cleave_buf x, cleave_buf dz, int32_t rows, int32_t d_in,
                                    int32_t d_out, cleave_buf x_lo, cleave_buf dz_lo) {
  ApiLock lock;
  Trace tr("dense_grads", "rows=%d d_in=%d d_out=%d", rows, d_in, d_out);
  Buf* DW = as_buf(dw, "dense_grads");
  Buf* DB = as_buf(db, "dense_grads");
  Buf* X = as_buf(x, "dense_grads");
  Buf* DZ = as_buf(dz, "dense_grads");
  if (!DW || !DB || !X || !DZ) return -cleave_cuda_last_error();
  Buf* XL = nullptr;
  Buf* DZL = nullptr;
  if (x_lo && !(XL = as_buf(x_lo, "dense_grads"))) return -cleave_cuda_last_error();
  if (dz_lo && !(DZL = as_buf(dz_lo, "dense_grads"))) return -cleave_cuda_last_error();
  if (rows <= 0 || d_in <= 0 || d_out <= 0 || DB->len != d_out || DZ->len != (int64_t)rows * d_out)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "dense_grads: db has %lld elements, dz %lld, for rows %d, d_out %d",
                      (long long)DB->len, (long long)DZ->len, rows, d_out);
  // The bias gradient only needs dz, which is complete before this call: it runs on the side queue, beside the product
  // (which is queued first so that its CTAs are placed first; a product with fewer tiles than SMs leaves the rest
  // to the column sums, otherwise they fill in as the product's CTAs retire).
  cudaStream_t side = side_fork();
  if (!side) return -cleave_cuda_last_error();
  int r = gemm_into(DW, X, DZ, 1, d_in, d_out, rows, 1, 0, CLEAVE_GEMM_AUTO, nullptr, CLEAVE_ACT_IDENTITY, nullptr,
                    CLEAVE_ACT_IDENTITY, XL, DZL, nullptr);
  const bool ok = colsum_launch(DZ->ptr, DB->ptr, rows, d_out, side);
  if (!side_join()) return -cleave_cuda_last_error();   // always rejoin: a captured graph must not end forked
  if (r != CLEAVE_CUDA_OK) return -r;
  return ok ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

cleave_buf cleave_cuda_split_lo_f32(cleave_buf x) {
  ApiLock lock;
  Buf* a = as_buf(x, "split_lo");
  if (!a) return nullptr;
  Trace tr("split_lo", "n=%lld", (long long)a->len);
  Buf* o = new_buf(a->len);
  if (!o) return nullptr;
  if (!split_lo_plane(a->ptr, o->ptr, a->len)) { release_buf(o); return nullptr; }
  return (cleave_buf)o;
}

int32_t cleave_cuda_gemm_batch_chunk(int64_t workspace_bytes_per_entry, int32_t batch) {
  return gemm_batch_chunk(workspace_bytes_per_entry, batch);
}

int32_t cleave_cuda_gemm_cut_plan(int32_t tiles, int32_t k_blocks, int32_t sm_pairs, int32_t* runs_per_tile) {
  int runs = 0;
  const int cut = gemm_cut_plan(tiles, k_blocks, sm_pairs, &runs);
  if (runs_per_tile) *runs_per_tile = runs;
  return cut;
}

int32_t cleave_cuda_split_lo_into_f32(cleave_buf lo, cleave_buf x, void* cuda_stream) {
  ApiLock lock;
  Buf* a = as_buf(x, "split_lo_into");
  Buf* o = as_buf(lo, "split_lo_into");
  if (!a || !o) return -cleave_cuda_last_error();
  if (a->len != o->len || a->ptr == o->ptr)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "split_lo_into: the plane must be a distinct tensor of the same length");
  return split_lo_plane(a->ptr, o->ptr, a->len, (cudaStream_t)cuda_stream) ? CLEAVE_CUDA_OK : -cleave_cuda_last_error();
}

}  // extern "C"
