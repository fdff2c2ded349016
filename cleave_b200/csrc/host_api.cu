// Host-array forms of the operators: the entry points a lowering hook in cleave's MLIR lowering calls for
// operations on NATIVE cleave tensors.  A `Tensor<f32, Dims...>` value is a host memref after bufferisation
// (cleave/src/mlir_lower.rs:223-226); the hook passes each operand the way every array crosses an extern call,
// as (pointer, i64 total length) (mlir_lower.rs:1096-1113, :1720-1751), plus the static dims as i32 scalars.
// Each call copies its operands to the device, runs the same kernels as the handle-based entry points and
// copies the result back into the caller's output array; it returns when the output is complete.
//
// The matmul form pipelines large products: B is uploaded once, then row blocks of A are uploaded on the copy
// engine while the previous block is multiplied and the block before that is downloaded, so the call costs
// about the longer of its transfers and its arithmetic rather than their sum.
#include "common.cuh"

using namespace cleave;

namespace {

struct Guard {   // frees the handles a call collected, on every exit path
  cleave_buf h[8];
  int n = 0;
  void add(cleave_buf b) { if (b && n < 8) h[n++] = b; }
  ~Guard() { for (int i = 0; i < n; ++i) cleave_cuda_free(h[i]); }
};

bool is_pinned(const void* p) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeHost;
}

}  // namespace

extern "C" {

int64_t cleave_cuda_host_gemm_f32(const float* a, int64_t a_len, const float* b, int64_t b_len, float* c, int64_t c_len,
                                  int32_t m, int32_t n, int32_t k) {
  ApiLock lock;
  if (!ensure_init()) return -cleave_cuda_last_error();
  if (!a || !b || !c || m <= 0 || n <= 0 || k <= 0)
    return -set_error(CLEAVE_CUDA_ERR_ARG, "host_gemm: need three arrays and positive m, n, k (got %d, %d, %d)", m, n, k);
  if (a_len != (int64_t)m * k || b_len != (int64_t)k * n || c_len != (int64_t)m * n)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "host_gemm: array lengths %lld, %lld, %lld do not match [%d x %d] * [%d x %d]",
                      (long long)a_len, (long long)b_len, (long long)c_len, m, k, k, n);
  Trace tr("host_gemm", "m=%d n=%d k=%d", m, n, k);
  Guard g;
  // Row blocks: whole 256-row tiles, at most 8 blocks, each at least 16 Mi multiply-adds per row block column;
  // small products and pageable arrays (whose copies the driver stages and serialises anyway) go in one piece.
  int blocks = 1;
  if ((int64_t)m * n * k >= (1ll << 33) && m >= 2048 && is_pinned(a) && is_pinned(c)) {
    blocks = m / 1024;
    if (blocks > 8) blocks = 8;
  }
  cleave_buf tb = cleave_cuda_upload_f32(b, b_len);
  g.add(tb);
  if (!tb) return -cleave_cuda_last_error();
  if (blocks == 1) {
    cleave_buf ta = cleave_cuda_upload_f32(a, a_len);
    g.add(ta);
    if (!ta) return -cleave_cuda_last_error();
    cleave_buf tc = cleave_cuda_gemm_f32(ta, tb, m, n, k);
    g.add(tc);
    if (!tc) return -cleave_cuda_last_error();
    const int64_t r = cleave_cuda_download_f32(tc, c, c_len);
    return r < 0 ? r : c_len;
  }
  const int rows_per = ((m + blocks - 1) / blocks + 255) / 256 * 256;
  cleave_buf ta[2] = {cleave_cuda_alloc_f32((int64_t)rows_per * k), cleave_cuda_alloc_f32((int64_t)rows_per * k)};
  cleave_buf tc[2] = {cleave_cuda_alloc_f32((int64_t)rows_per * n), cleave_cuda_alloc_f32((int64_t)rows_per * n)};
  for (int i = 0; i < 2; ++i) { g.add(ta[i]); g.add(tc[i]); }
  if (!ta[0] || !ta[1] || !tc[0] || !tc[1]) return -cleave_cuda_last_error();
  // Views of exactly the rows a block holds (the last block may be shorter), so lengths always match.
  auto rows_of = [&](int blk) { const int r0 = blk * rows_per; return (m - r0) < rows_per ? (m - r0) : rows_per; };
  bool ok = true;
  auto upload_block = [&](int blk) {
    Buf* t = lookup_buf(ta[blk & 1], "host_gemm");
    // the async copy is tracked on the full-size handle; only the block's rows are written
    const int rows = rows_of(blk);
    const int64_t saved = t->len;
    t->len = (int64_t)rows * k;
    ok = ok && cleave_cuda_upload_async_f32(ta[blk & 1], a + (int64_t)blk * rows_per * k, t->len) == CLEAVE_CUDA_OK;
    t->len = saved;
  };
  const int nblk = (m + rows_per - 1) / rows_per;
  upload_block(0);
  for (int blk = 0; ok && blk < nblk; ++blk) {
    if (blk + 1 < nblk) upload_block(blk + 1);
    const int rows = rows_of(blk);
    Buf* A = as_buf(ta[blk & 1], "host_gemm");   // orders the compute stream after this block's upload
    Buf* C = as_buf(tc[blk & 1], "host_gemm");   // ... and after the download that last read this output buffer
    if (!A || !C) { ok = false; break; }
    cleave_buf va = cleave_cuda_wrap_f32(A->ptr, (int64_t)rows * k);
    cleave_buf vc = cleave_cuda_wrap_f32(C->ptr, (int64_t)rows * n);
    ok = va && vc &&
         cleave_cuda_gemm_ex_f32(vc, va, tb, 1, rows, n, k, 0, 0, CLEAVE_GEMM_AUTO, nullptr, CLEAVE_ACT_IDENTITY) ==
             CLEAVE_CUDA_OK;
    if (va) cleave_cuda_free(va);
    if (vc) cleave_cuda_free(vc);
    if (!ok) break;
    const int64_t saved = C->len;
    C->len = (int64_t)rows * n;
    ok = cleave_cuda_download_async_f32(tc[blk & 1], c + (int64_t)blk * rows_per * n, C->len) == CLEAVE_CUDA_OK;
    C->len = saved;
  }
  if (cleave_cuda_transfers_sync() != CLEAVE_CUDA_OK) ok = false;
  if (ok && cleave_cuda_sync() != CLEAVE_CUDA_OK) ok = false;
  return ok ? c_len : -cleave_cuda_last_error();
}

int64_t cleave_cuda_host_binary_f32(int32_t op, const float* a, int64_t a_len, const float* b, int64_t b_len, float* out,
                                    int64_t out_len) {
  ApiLock lock;
  if (!a || !b || !out || a_len <= 0 || a_len != b_len || a_len != out_len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "host_binary: the three arrays must be non-NULL and of equal length "
                                             "(%lld, %lld, %lld)", (long long)a_len, (long long)b_len, (long long)out_len);
  typedef cleave_buf (*Fn)(cleave_buf, cleave_buf);
  Fn fn = nullptr;
  switch (op) {
    case CLEAVE_OP_ADD: fn = cleave_cuda_add_f32; break;
    case CLEAVE_OP_SUB: fn = cleave_cuda_sub_f32; break;
    case CLEAVE_OP_MUL: fn = cleave_cuda_mul_f32; break;
    case CLEAVE_OP_DIV: fn = cleave_cuda_div_f32; break;
    default: return -set_error(CLEAVE_CUDA_ERR_ARG, "host_binary: unknown operation code %d", op);
  }
  Guard g;
  cleave_buf ta = cleave_cuda_upload_f32(a, a_len);
  g.add(ta);
  cleave_buf tb = ta ? cleave_cuda_upload_f32(b, b_len) : nullptr;
  g.add(tb);
  if (!ta || !tb) return -cleave_cuda_last_error();
  cleave_buf to = fn(ta, tb);
  g.add(to);
  if (!to) return -cleave_cuda_last_error();
  const int64_t r = cleave_cuda_download_f32(to, out, out_len);
  return r < 0 ? r : out_len;
}

int64_t cleave_cuda_host_unary_f32(int32_t op, const float* a, int64_t a_len, float* out, int64_t out_len) {
  ApiLock lock;
  if (!a || !out || a_len <= 0 || a_len != out_len)
    return -set_error(CLEAVE_CUDA_ERR_SHAPE, "host_unary: both arrays must be non-NULL and of equal length (%lld, %lld)",
                      (long long)a_len, (long long)out_len);
  typedef cleave_buf (*Fn)(cleave_buf);
  Fn fn = nullptr;
  switch (op) {
    case CLEAVE_OP_NEG: fn = cleave_cuda_neg_f32; break;
    case CLEAVE_OP_EXP: fn = cleave_cuda_exp_f32; break;
    case CLEAVE_OP_TANH: fn = cleave_cuda_tanh_f32; break;
    case CLEAVE_OP_RELU: fn = cleave_cuda_relu_f32; break;
    case CLEAVE_OP_SIGMOID: fn = cleave_cuda_sigmoid_f32; break;
    default: return -set_error(CLEAVE_CUDA_ERR_ARG, "host_unary: unknown operation code %d", op);
  }
  Guard g;
  cleave_buf ta = cleave_cuda_upload_f32(a, a_len);
  g.add(ta);
  if (!ta) return -cleave_cuda_last_error();
  cleave_buf to = fn(ta);
  g.add(to);
  if (!to) return -cleave_cuda_last_error();
  const int64_t r = cleave_cuda_download_f32(to, out, out_len);
  return r < 0 ? r : out_len;
}

}  // extern "C"
