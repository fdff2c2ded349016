/* libcleave_cuda -- C ABI of the B200 (sm_100a) tensor backend for cleave.
 *
 * Every entry point uses only what cleave's extern-call lowering can pass
 * (cleave/src/mlir_lower.rs:1061-1130, :1720-1751, :2127-2160 in the reference):
 *   - scalars i32 / i64 / f32 by value,
 *   - an opaque struct handle as ONE pointer (mlir_lower.rs:145), here `cleave_buf`,
 *   - an array `[T; ...]` as the pair (T* ptr, int64_t total_len),
 *   - one scalar / handle result, or void.
 * A `cleave_buf` plays the role `RawBuf` plays for DynArray
 * (stdlib/dynarray/dynarray.cleave:29, cleave-rt/src/lib.rs:169-213): it is produced by an
 * extern function, only ever passed back to extern functions, and owns a dense, row-major,
 * contiguous f32 device array -- the layout of `Tensor<T, Dims...>`
 * (stdlib/linalg/tensor.cleave:40, mlir_lower.rs:276-295).  Shapes stay in the cleave type
 * system (const generics are i32) and are passed as i32 scalars where an op needs them.
 *
 * Value semantics: tensor values in cleave are immutable SSA values, so every op returns a
 * NEW handle; the `_into` forms write into a handle the caller already owns.
 *
 * Errors: the reference runtime has no error channel (it panics: cleave-rt/src/lib.rs:69).
 * Here a failing call returns NULL (handle), NaN (f32 scalar) or a negative code (i32/i64)
 * and records a thread-local code + message readable with cleave_cuda_last_error*().
 * With CLEAVE_CUDA_ABORT_ON_ERROR=1 in the environment a failing call aborts the process
 * instead, which is the reference's behaviour.  There is no CPU fallback: without a CUDA
 * device every compute call fails with CLEAVE_CUDA_ERR_NO_DEVICE.
 *
 * Threads: calls may come from several host threads; they are serialised on one device
 * stream per process.  Work is asynchronous until a scalar-returning op, a download or
 * cleave_cuda_sync().
 */
#ifndef CLEAVE_CUDA_H
#define CLEAVE_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cleave_buf_s* cleave_buf; /* opaque device tensor handle ("DevBuf") */

enum {
  CLEAVE_CUDA_OK = 0,
  CLEAVE_CUDA_ERR_NO_DEVICE = 1,   /* no usable CUDA device / driver */
  CLEAVE_CUDA_ERR_BAD_HANDLE = 2,  /* NULL, freed or foreign handle */
  CLEAVE_CUDA_ERR_SHAPE = 3,       /* lengths / dims inconsistent with the operands */
  CLEAVE_CUDA_ERR_ARG = 4,         /* other invalid argument */
  CLEAVE_CUDA_ERR_OOM = 5,         /* device or pinned-host allocation failed */
  CLEAVE_CUDA_ERR_CUDA = 6,        /* a CUDA runtime call failed (message has the text) */
  CLEAVE_CUDA_ERR_DEVICE_TIMEOUT = 7, /* a bounded in-kernel wait gave up; results invalid */
  CLEAVE_CUDA_ERR_UNSUPPORTED = 8
};

/* activation codes for the fused entry points */
enum { CLEAVE_ACT_IDENTITY = 0, CLEAVE_ACT_RELU = 1, CLEAVE_ACT_SIGMOID = 2, CLEAVE_ACT_TANH = 3 };

/* GEMM algorithm selector for cleave_cuda_gemm_ex_f32 */
enum {
  CLEAVE_GEMM_AUTO = 0,   /* tensor-core path for large problems, exact path for small ones */
  CLEAVE_GEMM_EXACT = 1,  /* SIMT f32, k-ascending multiply-then-add: bit-identical to the CPU path */
  CLEAVE_GEMM_3XTF32 = 2  /* tcgen05 + TMEM + TMA, split-precision TF32 (3 MMAs per product).  Finite operands only:
                             an infinite operand yields NaN (inf * 0 from the split) where the reference loop may
                             yield +-inf; NaN operands propagate as NaN on both paths */
};

/* ------------------------------------------------------------------ runtime
 * No counterpart in cleave-rt (it has no device); modelled on its allocation pair
 * cleave_alloc / cleave_realloc (cleave-rt/src/lib.rs:56-71, :146-155). */
int32_t cleave_cuda_init(int32_t device);            /* select device, create the stream; idempotent */
int32_t cleave_cuda_device_count(void);
int32_t cleave_cuda_last_error(void);                /* code of this thread's last failing call */
const char* cleave_cuda_last_error_message(void);    /* its message (thread-local storage) */
void cleave_cuda_clear_error(void);
int32_t cleave_cuda_sync(void);                      /* wait for all queued work; returns a code */
void cleave_cuda_set_stream(void* cuda_stream);      /* run on a caller-owned cudaStream_t (NULL: own stream) */
void* cleave_cuda_get_stream(void);
void cleave_cuda_reset(void);                        /* invalidate every handle, keep memory cached */
void cleave_cuda_trim(void);                         /* return cached device memory to the driver */
int64_t cleave_cuda_live_bytes(void);                /* bytes held by live handles */
int64_t cleave_cuda_kernel_launches(void);           /* kernels launched by this library so far */
/* Measurement aid: between begin and end every tensor-core GEMM kernel launch (operand pre-pass
 * excluded) and every linear-regression sweep (both of its kernels) is bracketed by a CUDA event
 * pair on the launching stream; end waits for them and returns their total duration in
 * milliseconds and, through `launches`, how many pairs there were. */
void cleave_cuda_profile_begin(void);
double cleave_cuda_profile_end(int32_t* launches);
/* Diagnostics (environment, read once):
 *   CLEAVE_CUDA_TRACE=1  every compute / transfer entry point prints "operation shape microseconds" to stderr
 *                        (device time of what the call queued; the call waits for it, so the run is serialised)
 *   CLEAVE_CUDA_DEBUG=1  every pool block is followed by guard bytes that are checked when the block is freed;
 *                        an overrun is reported through the error channel and on stderr
 * Test hook: lets a test put the library into states that otherwise need a misbehaving kernel.  It never
 * launches anything.  Selectors: */
enum {
  CLEAVE_HOOK_SET_DEVICE_STATUS = 1,   /* arg = status code: as if a kernel's bounded wait had run out */
  CLEAVE_HOOK_POISON_NOALLOC_WORD = 2, /* arg = 64-bit value stored over cleave_cuda_sum_noalloc_f32's completion counter */
  CLEAVE_HOOK_GUARD_FAILURES = 3       /* returns the number of guard-byte mismatches seen so far (debug mode) */
};
int64_t cleave_cuda_test_hook(int32_t what, int64_t arg);
/* Host arithmetic of the batched GEMM paths, exposed so that it can be checked without a device: how many batch
 * entries one pass processes given the operand workspace one entry needs (bounded by the workspace limit, by
 * `batch`, and by the 65535 entries a grid's z dimension can index). */
int32_t cleave_cuda_gemm_batch_chunk(int64_t workspace_bytes_per_entry, int32_t batch);
/* Host arithmetic of the CTA-pair GEMM's last wave, likewise exposed for checking without a device: for a product of
 * `tiles` 256 x 256 tiles and `k_blocks` K-blocks of 32 on `sm_pairs` SM pairs, returns how many tiles of the last,
 * partly filled wave are cut along K (0: none) and stores the equal K-runs per cut tile in *runs_per_tile.  The cut
 * keeps tiles x runs <= sm_pairs and runs of at least 8 K-blocks, and applies only when it saves at least 16 K-blocks. */
int32_t cleave_cuda_gemm_cut_plan(int32_t tiles, int32_t k_blocks, int32_t sm_pairs, int32_t* runs_per_tile);
/* A step captured once and replayed (CUDA graph): everything queued between begin and end is recorded instead of
 * run, and cleave_cuda_graph_launch replays it on the library's stream without the per-kernel launch gaps (the
 * 13 kernels of a perceptron step: 0.77 -> 0.73 ms).  Only entry points that do not wait may be called inside a
 * capture (no scalar-returning op, no download, no sync); call the step once before capturing it, so that one-time
 * kernel set-up has happened.  Tensors allocated inside the capture come from a cache that belongs to the graph:
 * the replays keep using exactly those blocks, nothing else is handed them, and cleave_cuda_graph_free returns them.
 * A handle created inside the capture and still alive afterwards (an output) is overwritten by every replay.
 * No counterpart in the reference (it has no device and no launch overhead to hide). */
int32_t cleave_cuda_graph_begin(void);
void* cleave_cuda_graph_end(void);                   /* the graph handle, NULL on failure */
int32_t cleave_cuda_graph_launch(void* graph);
void cleave_cuda_graph_free(void* graph);
void* cleave_cuda_host_alloc(int64_t bytes);         /* pinned host memory for fast transfers */
void cleave_cuda_host_free(void* p);

/* ------------------------------------------------------------------ construction / readback
 * Replaces tensor.from_elements (mlir_lower.rs:1447-1476), the array-repeat fill behind
 * Ring::zero (stdlib/linalg/tensor.cleave:79, mlir_lower.rs:1176-1272) and tensor.extract
 * (stdlib/linalg/tensor.cleave:129-133, mlir_lower.rs:1972-2002). */
cleave_buf cleave_cuda_none(void);   /* the absent operand: NULL.  cleave has no null literal for an opaque struct, so
                                        optional handles (a bias, a lo plane) are spelled with this call */
cleave_buf cleave_cuda_alloc_f32(int64_t len);                              /* uninitialised */
cleave_buf cleave_cuda_upload_f32(const float* host, int64_t len);          /* [f32; len] -> device */
int64_t cleave_cuda_download_f32(cleave_buf t, float* host, int64_t len);   /* returns len or <0 */
int32_t cleave_cuda_upload_into_f32(cleave_buf t, const float* host, int64_t len);
/* Transfers on the copy engines, overlapping compute.  The host buffer must be pinned
 * (cleave_cuda_host_alloc) and stay untouched until cleave_cuda_transfers_sync().  An upload is
 * ordered after all compute queued so far (which may still read the tensor); compute queued later
 * that uses the SAME handle waits for the copy.  A download is ordered after all compute queued
 * so far; later compute that writes the tensor waits for it.  Tracking is per handle: views made
 * with cleave_cuda_wrap_f32 do not inherit it.  To overlap step i's compute with step i+1's
 * upload, alternate between two tensors and issue the upload before queueing step i. */
int32_t cleave_cuda_upload_async_f32(cleave_buf t, const float* pinned_host, int64_t len);
int32_t cleave_cuda_download_async_f32(cleave_buf t, float* pinned_host, int64_t len);
int32_t cleave_cuda_transfers_sync(void);
cleave_buf cleave_cuda_fill_f32(float value, int64_t len);
cleave_buf cleave_cuda_zeros_f32(int64_t len);
float cleave_cuda_get_f32(cleave_buf t, int64_t flat_index);                /* row-major flat index */
int64_t cleave_cuda_len(cleave_buf t);
void cleave_cuda_free(cleave_buf t);
cleave_buf cleave_cuda_wrap_f32(void* device_ptr, int64_t len);             /* non-owning view of caller memory */
void* cleave_cuda_data_ptr(cleave_buf t);

/* ------------------------------------------------------------------ Ring<Tensor<T, Dims...>>
 * stdlib/linalg/tensor.cleave:66-80: add/sub/mul/div/neg = arith.addf/subf/mulf/divf/negf on
 * same-shape tensors (no broadcasting).  One IEEE-754 operation per element. */
cleave_buf cleave_cuda_add_f32(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_sub_f32(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_mul_f32(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_div_f32(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_neg_f32(cleave_buf a);

/* ------------------------------------------------------------------ Activation / Transcendental
 * stdlib/nn/nn.cleave:82-95 (tensor) and :54-64 (scalar); stdlib/num/num.cleave:227-233.
 * relu = NaN-propagating max(x, 0); sigmoid = 1/(1+exp(-x)) in ONE pass instead of the
 * reference's four; tanh, exp. */
cleave_buf cleave_cuda_relu_f32(cleave_buf x);
cleave_buf cleave_cuda_sigmoid_f32(cleave_buf x);
cleave_buf cleave_cuda_tanh_f32(cleave_buf x);
cleave_buf cleave_cuda_exp_f32(cleave_buf x);
/* Derivative rules applied to a whole tensor, fused with the upstream factor
 * (stdlib/num/num.cleave:222-223; sigmoid through the chain of :123-136).
 * y = forward OUTPUT for tanh/sigmoid, x = forward INPUT for relu, g = upstream gradient. */
cleave_buf cleave_cuda_tanh_bwd_f32(cleave_buf y, cleave_buf g);     /* (1 - y*y) * g */
cleave_buf cleave_cuda_sigmoid_bwd_f32(cleave_buf y, cleave_buf g);  /* y*(1 - y) * g */
cleave_buf cleave_cuda_relu_bwd_f32(cleave_buf x, cleave_buf g);     /* x > 0 ? g : 0 */

/* ------------------------------------------------------------------ Sum / Mean / Max
 * stdlib/nn/nn.cleave:111-149.  sum is a deterministic tree (fixed grid, fixed order), not
 * the reference's left-to-right chain: equal within rounding, reproducible run to run.
 * max_of keeps the reference's strict-> scan semantics for NaN (NaN in v[0] wins, later
 * NaNs are skipped). */
float cleave_cuda_sum_f32(cleave_buf v);
float cleave_cuda_mean_f32(cleave_buf v);
float cleave_cuda_max_f32(cleave_buf v);
/* Sum without any allocation.  No counterpart in the reference (its runtime only ever
 * allocates, cleave-rt/src/lib.rs:56-71); added for callers that cannot allocate device memory
 * when they need the reduction: hosts where another framework owns the device heap, loops
 * where a cudaMalloc stall is not acceptable, processes already at their memory budget.
 * x_dev (len f32 values) and out_dev (one f32) are raw device pointers owned by the caller; the
 * kernel is queued on cuda_stream (NULL = the default stream) of the CURRENT device and the
 * call returns without waiting.  The partial sums and a completion word live in a 4752-byte array that is
 * part of the library image on every GPU; len may be at most 2^31 - 1 (larger is rejected with
 * CLEAVE_CUDA_ERR_UNSUPPORTED).  The first call on each device looks up the array's device
 * address, so make that first call outside any stream capture.  All calls on one device share
 * the array: calls whose kernels may overlap on the GPU (different streams) race on it and their
 * results are undefined; calls on one stream do not.  Every call clears its completion counter on its own
 * stream before the kernel (a memset node, no allocation), so a call that was cut short (or an overlapped
 * pair) leaves nothing behind that a later, properly ordered call could trip over.  The value equals
 * cleave_cuda_sum_f32 of the same data bit for bit.
 * It uses no handle and no pool, never calls cudaMalloc or cudaFree, and takes from the library context
 * only the SM count.  x_dev must stay valid until the kernel has run: when it comes from
 * cleave_cuda_data_ptr and the call is on a stream other than the library's, do not free the handle
 * before that stream has been synchronised (the pool hands freed blocks to later library work at once). */
int32_t cleave_cuda_sum_noalloc_f32(const float* x_dev, int64_t len, float* out_dev, void* cuda_stream);
/* Sum applied to each column of a rows x cols matrix (bias gradients). */
cleave_buf cleave_cuda_colsum_f32(cleave_buf x, int32_t rows, int32_t cols);
int32_t cleave_cuda_colsum_into_f32(cleave_buf out, cleave_buf x, int32_t rows, int32_t cols);

/* ------------------------------------------------------------------ MatMul
 * stdlib/linalg/matrix.cleave:22-62: MatMul<Tensor<T,N,M>, Tensor<T,M,K>, Tensor<T,N,K>>,
 * linalg.matmul into a zero tensor (region mlir_lower.rs:2089-2120).  Here the dims are named
 * BLAS-style: C[m,n] = A[m,k] * B[k,n]  (cleave's N,M,K are m,k,n). */
cleave_buf cleave_cuda_gemm_f32(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k);
/* Transposed-operand forms needed by the derivative rule matmul(da,b) + matmul(a,db)
 * (stdlib/linalg/matrix.cleave:24) evaluated in reverse mode:
 *   nt: C[m,n] = A[m,k] * B[n,k]^T        tn: C[m,n] = A[k,m]^T * B[k,n] */
cleave_buf cleave_cuda_gemm_nt_f32(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k);
cleave_buf cleave_cuda_gemm_tn_f32(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k);
/* `batch` independent products, operands stacked along a leading batch dimension.
 * (Named in the reference only as a comment, mlir_lower.rs:2078.) */
cleave_buf cleave_cuda_gemm_batched_f32(cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n,
                                        int32_t k);
/* General form: writes C (caller-owned, batch*m*n elements).  trans_a / trans_b select the
 * stored layout of the operands as above; algo is a CLEAVE_GEMM_* value; bias (may be NULL,
 * n elements) is added to every row and act (CLEAVE_ACT_*) applied before the store.  On the tensor-core path
 * the sigmoid of the epilogue uses the hardware exponential and reciprocal: within a few ulp (3e-7 relative) of
 * cleave_cuda_sigmoid_f32 applied to the same sums, not bit-identical to it; tanh and relu are the same functions. */
int32_t cleave_cuda_gemm_ex_f32(cleave_buf c, cleave_buf a, cleave_buf b, int32_t batch, int32_t m,
                                int32_t n, int32_t k, int32_t trans_a, int32_t trans_b, int32_t algo,
                                cleave_buf bias, int32_t act);
/* Backward form of a layer: C = act'(y) (.) (op(A) * op(B)), elementwise product of the matrix product with the
 * derivative of activation `act` taken from that activation's forward OUTPUT y (batch*m*n elements): tanh 1 - y^2,
 * sigmoid y (1 - y), relu y > 0 (stdlib/num/num.cleave:222-223 exp / tanh rules, stdlib/nn/nn.cleave:54-64).  It is
 * dZ = act'(H) (.) (dZ_next * W^T) of reverse mode in one pass; the result is bit-identical to
 * cleave_cuda_gemm_ex_f32 followed by cleave_cuda_tanh_bwd_f32 / sigmoid_bwd / relu_bwd. */
int32_t cleave_cuda_gemm_dact_f32(cleave_buf c, cleave_buf a, cleave_buf b, int32_t batch, int32_t m,
                                  int32_t n, int32_t k, int32_t trans_a, int32_t trans_b, int32_t algo,
                                  cleave_buf y, int32_t act);

/* Chained form for graphs in which one product feeds the next (the lowered perceptron: H = act(X W1 + b1) feeds
 * H W2 and H^T dZ2; dZ1 feeds X^T dZ1).  The tensor-core path multiplies x as hi + lo; with the lo parts handed
 * over between calls no operand pre-pass runs at all:
 *   a_lo / b_lo  (may be NULL) lo planes of the operands, same shape as a / b, obtained from an earlier call's
 *                c_lo, from cleave_cuda_split_lo_f32, or from cleave_cuda_mse_act_bwd_lo_f32; a plane must belong
 *                to the CURRENT contents of its tensor -- the library cannot check that;
 *   c_lo         (may be NULL) receives the lo plane of the values stored to c, written by the same epilogue.
 * bias + act, or y + dact (the backward form), as in the two entry points above; not both.  The result is
 * bit-identical to cleave_cuda_gemm_ex_f32 / cleave_cuda_gemm_dact_f32 on the same tensor-core route.
 * No counterpart in the reference (its matmul is one linalg op, stdlib/linalg/matrix.cleave:59-60). */
int32_t cleave_cuda_gemm_fused_f32(cleave_buf c, cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n,
                                   int32_t k, int32_t trans_a, int32_t trans_b, int32_t algo, cleave_buf bias,
                                   int32_t act, cleave_buf y, int32_t dact, cleave_buf a_lo, cleave_buf b_lo,
                                   cleave_buf c_lo);
/* Both gradients of a dense layer y = x W + b from the gradient dz of its output, in one call (the derivative rule of
 * MatMul and of the broadcast bias add: stdlib/linalg/matrix.cleave:59-60 reversed, and the column sum that undoes the
 * row broadcast of stdlib/nn/nn.cleave:72-74):
 *   dw[d_in, d_out] = x[rows, d_in]^T * dz[rows, d_out],    db[d_out] = sum over rows of dz.
 * The two are independent, so the library queues the column sums beside the product on a second stream of its own and
 * rejoins before returning: a product with fewer tiles than SMs leaves the idle SMs to the sums.  Results are bit-identical
 * to cleave_cuda_gemm_fused_f32(dw, x, dz, trans_a = 1, ...) followed by cleave_cuda_colsum_into_f32(db, dz, ...).
 * x_lo / dz_lo (may be NULL): lo planes of the operands, as in cleave_cuda_gemm_fused_f32. */
int32_t cleave_cuda_dense_grads_f32(cleave_buf dw, cleave_buf db, cleave_buf x, cleave_buf dz, int32_t rows, int32_t d_in,
                                    int32_t d_out, cleave_buf x_lo, cleave_buf dz_lo);
/* The lo plane of a tensor in one streaming pass: lo[i] = tf32-rounded (x[i] - x[i] with its 13 low mantissa
 * bits cleared), the part of x the tensor pipe drops when it reads x as tf32. */
cleave_buf cleave_cuda_split_lo_f32(cleave_buf x);
/* The same into a plane the caller owns, queued on cuda_stream (NULL = the library's stream): a data-parallel
 * driver refreshes the weights' planes on the stream of its exchange kernel, off the training step's critical
 * path.  On a foreign stream the caller orders the call against the library's work (events), as for
 * cleave_cuda_dp_sgd_allreduce_f32. */
int32_t cleave_cuda_split_lo_into_f32(cleave_buf lo, cleave_buf x, void* cuda_stream);

/* ------------------------------------------------------------------ compositions the programs spell out
 * bias add: a rows x cols tensor plus a tensor whose rows all equal `bias`
 * (arith.addf does not broadcast: stdlib/nn/nn.cleave:72-74), then an activation. */
cleave_buf cleave_cuda_bias_act_f32(cleave_buf x, cleave_buf bias, int32_t rows, int32_t cols, int32_t act);
/* mean((p - t)^2) (examples/linear_regression.cleave:20-30 with Mean, nn.cleave:119-139).
 * If dp is non-NULL it receives 2*(p - t)/len, the gradient with respect to p. */
float cleave_cuda_mse_f32(cleave_buf p, cleave_buf t, cleave_buf dp);
/* The same loss for y = act(z), with the chain through the activation folded in: dz receives
 * act'(y) * 2*(y - t)/len, the gradient with respect to the PRE-activation z, in one pass
 * (mse followed by sigmoid_bwd / tanh_bwd, bit for bit).  act: identity, sigmoid or tanh. */
float cleave_cuda_mse_act_bwd_f32(cleave_buf y, cleave_buf t, cleave_buf dz, int32_t act);
/* Same, but the loss goes to the one-element tensor loss_out and the call does not wait: a
 * training loop can queue many steps and read the loss only when it wants to log it. */
int32_t cleave_cuda_mse_act_bwd_dev_f32(cleave_buf y, cleave_buf t, cleave_buf dz, int32_t act, cleave_buf loss_out);
/* cleave_cuda_mse_act_bwd_dev_f32 that also writes the lo plane of dz (see cleave_cuda_gemm_fused_f32). */
int32_t cleave_cuda_mse_act_bwd_lo_f32(cleave_buf y, cleave_buf t, cleave_buf dz, int32_t act, cleave_buf loss_out,
                                       cleave_buf dz_lo);
/* w = w - lr * (gscale * g) in place (examples/xor.cleave:67-70); gscale folds the 1/G of a
 * gradient mean over G data-parallel ranks into the same pass. */
int32_t cleave_cuda_sgd_f32(cleave_buf w, cleave_buf g, float lr, float gscale);
/* One linear-regression batch-gradient step in a single sweep over X[rows, feat]:
 * pred = X w, loss = mean((pred - y)^2), grad = dloss/dw.  pred_out (rows) and grad_out
 * (feat) are caller-owned handles; pred_out may be NULL.  feat <= 32.  Returns the loss. */
float cleave_cuda_linreg_step_f32(cleave_buf x, cleave_buf y, cleave_buf w, cleave_buf pred_out,
                                  cleave_buf grad_out, int32_t rows, int32_t feat);
/* Same, but the loss goes to the one-element tensor loss_out and the call does not wait: gradient-descent loops
 * queue step after step (grad_out feeds cleave_cuda_sgd_f32) and read the loss only when they log it. */
int32_t cleave_cuda_linreg_step_dev_f32(cleave_buf x, cleave_buf y, cleave_buf w, cleave_buf pred_out,
                                        cleave_buf grad_out, int32_t rows, int32_t feat, cleave_buf loss_out);

/* ------------------------------------------------------------------ host-array forms (the lowering hook's targets)
 * What a name-based exception in lower_raw_mlir_op (cleave/src/mlir_lower.rs:2004-2068; the two existing ones
 * are at :2031-2039 and :2062-2064) calls for an operation on NATIVE tensors: `linalg.matmul`, and tensor-typed
 * `arith.addf/subf/mulf/divf/negf` and `math.exp/tanh` (stdlib/linalg/matrix.cleave:59-60,
 * stdlib/linalg/tensor.cleave:66-80, stdlib/nn/nn.cleave:82-95).  A native tensor is a host memref after
 * bufferisation (mlir_lower.rs:223-226) and crosses the call as every array does, (pointer, i64 total length)
 * (mlir_lower.rs:1096-1113, :1720-1751); static dims follow as i32.  Each call uploads its operands, runs the
 * same kernels as the handle forms above, writes the result into the caller's `out` array and returns its
 * length (or a negative error code) once the array is complete.  The matmul form pipelines products of 2^33
 * multiply-adds and more over row blocks (upload, product and download of consecutive blocks overlap) when
 * a and c are pinned host memory (cleave_cuda_host_alloc). */
enum { CLEAVE_OP_ADD = 1, CLEAVE_OP_SUB = 2, CLEAVE_OP_MUL = 3, CLEAVE_OP_DIV = 4,              /* binary */
       CLEAVE_OP_NEG = 5, CLEAVE_OP_EXP = 6, CLEAVE_OP_TANH = 7, CLEAVE_OP_RELU = 8, CLEAVE_OP_SIGMOID = 9 };
int64_t cleave_cuda_host_gemm_f32(const float* a, int64_t a_len, const float* b, int64_t b_len, float* c, int64_t c_len,
                                  int32_t m, int32_t n, int32_t k);
int64_t cleave_cuda_host_binary_f32(int32_t op, const float* a, int64_t a_len, const float* b, int64_t b_len, float* out,
                                    int64_t out_len);
int64_t cleave_cuda_host_unary_f32(int32_t op, const float* a, int64_t a_len, float* out, int64_t out_len);

/* ------------------------------------------------------------------ f64 instances
 * The reference's algebras are declared for every T: Float (Ring<f64> stdlib/num/num.cleave:189-196,
 * Activation<f64> stdlib/nn/nn.cleave:60-64, Tensor<T, Dims...> stdlib/linalg/tensor.cleave:40), so
 * the operator surface exists for f64 tensors too.  Same semantics as the f32 entry points above;
 * a handle remembers its element type and the two families reject each other's tensors.
 * Matmul is the exact kernel only (bit-identical to the reference loop; no f64 tensor-core mode). */
cleave_buf cleave_cuda_alloc_f64(int64_t len);
cleave_buf cleave_cuda_upload_f64(const double* host, int64_t len);
int64_t cleave_cuda_download_f64(cleave_buf t, double* host, int64_t len);
cleave_buf cleave_cuda_fill_f64(double value, int64_t len);
cleave_buf cleave_cuda_zeros_f64(int64_t len);
double cleave_cuda_get_f64(cleave_buf t, int64_t flat_index);
cleave_buf cleave_cuda_add_f64(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_sub_f64(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_mul_f64(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_div_f64(cleave_buf a, cleave_buf b);
cleave_buf cleave_cuda_neg_f64(cleave_buf a);
cleave_buf cleave_cuda_relu_f64(cleave_buf x);
cleave_buf cleave_cuda_sigmoid_f64(cleave_buf x);
cleave_buf cleave_cuda_tanh_f64(cleave_buf x);
cleave_buf cleave_cuda_exp_f64(cleave_buf x);
double cleave_cuda_sum_f64(cleave_buf v);
double cleave_cuda_mean_f64(cleave_buf v);
double cleave_cuda_max_f64(cleave_buf v);
cleave_buf cleave_cuda_gemm_f64(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k);
/* What derive() over f64 tensors emits beyond the above (the algebras and their derivative rules are declared for
 * every T: Float, stdlib/num/num.cleave:189-196, :222-223, :231-234; stdlib/linalg/matrix.cleave:24): transposed
 * and batched products (exact kernel), the derivative forms, column sums, the squared-error loss, the SGD update. */
cleave_buf cleave_cuda_gemm_nt_f64(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k);
cleave_buf cleave_cuda_gemm_tn_f64(cleave_buf a, cleave_buf b, int32_t m, int32_t n, int32_t k);
cleave_buf cleave_cuda_gemm_batched_f64(cleave_buf a, cleave_buf b, int32_t batch, int32_t m, int32_t n, int32_t k);
cleave_buf cleave_cuda_tanh_bwd_f64(cleave_buf y, cleave_buf g);
cleave_buf cleave_cuda_sigmoid_bwd_f64(cleave_buf y, cleave_buf g);
cleave_buf cleave_cuda_relu_bwd_f64(cleave_buf x, cleave_buf g);
cleave_buf cleave_cuda_colsum_f64(cleave_buf x, int32_t rows, int32_t cols);
double cleave_cuda_mse_f64(cleave_buf p, cleave_buf t, cleave_buf dp);      /* dp may be NULL */
int32_t cleave_cuda_sgd_f64(cleave_buf w, cleave_buf g, double lr, double gscale);

/* ------------------------------------------------------------------ data-parallel step over peer memory
 * No counterpart in the reference (distribution is "named as a goal but not designed",
 * doc/hld.md:250).  One kernel per step does what a gradient all-reduce followed by the SGD update
 * (examples/xor.cleave:67-70 on tensors) would do: every rank owns 1/world of the flat parameter
 * vector, sums that slice of the gradients over all ranks -- in the NVSwitch when multicast
 * addresses are given (multimem.ld_reduce), else with plain peer loads in rank order -- applies
 * w -= lr * (sum / world) and writes the new weights into every rank's parameter buffer.
 * params_peers / grads_peers / flags_peers: `world` device pointers each, the same symmetric
 * allocations as seen from this rank (flags: >= 32 zero-initialised uint32 words per rank, used
 * for the kernel's own bounded cross-GPU barriers).  The call covers elements
 * [offset, offset + len) of the flat vectors (both multiples of 4), so a training step can
 * exchange the gradients in several buckets as the backward pass completes them; calls that
 * may be in flight at the same time must use different flag words (pass flags pointers that
 * are 32 words apart).  epoch: 1 for the first call on a set of flag words, then += 2 per call,
 * identical on every rank.  cuda_stream: the stream to launch on (NULL = the library's), so a
 * bucket can overlap the rest of the backward pass.  Every rank must make the same calls, one
 * process per GPU.  A bucket may only be exchanged once no rank reads its WEIGHTS any more in
 * this step.  A barrier that times out is reported as CLEAVE_CUDA_ERR_DEVICE_TIMEOUT at the next
 * synchronisation; when it is the ENTRY barrier (a rank's gradients never arrived, limit 2 s, or
 * CLEAVE_CUDA_DP_WAIT_MS milliseconds if that is set when the library initialises) the kernel
 * touches neither weights nor gradients on any rank: every replica still holds the weights it had
 * before the call.  Buffers passed here on a stream other than the library's must stay alive until
 * that stream has been synchronised.  The pointer tables are host arrays: this entry point is meant
 * for a host framework, it has no cleave-source binding (no cleave type lowers to a bare pointer table). */
int32_t cleave_cuda_dp_sgd_allreduce_f32(void* const* params_peers, void* const* grads_peers,
                                         void* const* flags_peers, void* params_multicast, void* grads_multicast,
                                         int64_t offset, int64_t len, int32_t rank, int32_t world, float lr,
                                         uint32_t epoch, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* CLEAVE_CUDA_H */
