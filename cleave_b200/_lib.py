"""ctypes binding of ``libcleave_cuda.so`` -- the same symbols, argument order and calling
convention that cleave's ``extern(cleave_cuda_*) fn`` declarations bind.

There is no fallback: if the shared library is missing this module raises at import of the
library handle, and every compute call fails loudly when no CUDA device is present.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcleave_cuda.so")

c_buf = ctypes.c_void_p
c_f32p = ctypes.POINTER(ctypes.c_float)
c_f64p = ctypes.POINTER(ctypes.c_double)
f64 = ctypes.c_double
i32, i64, f32 = ctypes.c_int32, ctypes.c_int64, ctypes.c_float

# name -> (restype, argtypes); mirrors include/cleave_cuda.h declaration by declaration.
SIGNATURES = {
    "cleave_cuda_init": (i32, [i32]),
    "cleave_cuda_device_count": (i32, []),
    "cleave_cuda_last_error": (i32, []),
    "cleave_cuda_last_error_message": (ctypes.c_char_p, []),
    "cleave_cuda_clear_error": (None, []),
    "cleave_cuda_sync": (i32, []),
    "cleave_cuda_set_stream": (None, [ctypes.c_void_p]),
    "cleave_cuda_get_stream": (ctypes.c_void_p, []),
    "cleave_cuda_reset": (None, []),
    "cleave_cuda_trim": (None, []),
    "cleave_cuda_live_bytes": (i64, []),
    "cleave_cuda_kernel_launches": (i64, []),
    "cleave_cuda_test_hook": (i64, [i32, i64]),
    "cleave_cuda_gemm_batch_chunk": (i32, [i64, i32]),
    "cleave_cuda_gemm_cut_plan": (i32, [i32, i32, i32, ctypes.POINTER(ctypes.c_int32)]),
    "cleave_cuda_profile_begin": (None, []),
    "cleave_cuda_profile_end": (ctypes.c_double, [ctypes.POINTER(i32)]),
    "cleave_cuda_graph_begin": (i32, []),
    "cleave_cuda_graph_end": (ctypes.c_void_p, []),
    "cleave_cuda_graph_launch": (i32, [ctypes.c_void_p]),
    "cleave_cuda_graph_free": (None, [ctypes.c_void_p]),
    "cleave_cuda_host_alloc": (ctypes.c_void_p, [i64]),
    "cleave_cuda_host_free": (None, [ctypes.c_void_p]),
    "cleave_cuda_none": (c_buf, []),
    "cleave_cuda_alloc_f32": (c_buf, [i64]),
    "cleave_cuda_upload_f32": (c_buf, [c_f32p, i64]),
    "cleave_cuda_download_f32": (i64, [c_buf, c_f32p, i64]),
    "cleave_cuda_upload_into_f32": (i32, [c_buf, c_f32p, i64]),
    "cleave_cuda_upload_async_f32": (i32, [c_buf, c_f32p, i64]),
    "cleave_cuda_download_async_f32": (i32, [c_buf, c_f32p, i64]),
    "cleave_cuda_transfers_sync": (i32, []),
    "cleave_cuda_fill_f32": (c_buf, [f32, i64]),
    "cleave_cuda_zeros_f32": (c_buf, [i64]),
    "cleave_cuda_get_f32": (f32, [c_buf, i64]),
    "cleave_cuda_len": (i64, [c_buf]),
    "cleave_cuda_free": (None, [c_buf]),
    "cleave_cuda_wrap_f32": (c_buf, [ctypes.c_void_p, i64]),
    "cleave_cuda_data_ptr": (ctypes.c_void_p, [c_buf]),
    "cleave_cuda_add_f32": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_sub_f32": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_mul_f32": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_div_f32": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_neg_f32": (c_buf, [c_buf]),
    "cleave_cuda_relu_f32": (c_buf, [c_buf]),
    "cleave_cuda_sigmoid_f32": (c_buf, [c_buf]),
    "cleave_cuda_tanh_f32": (c_buf, [c_buf]),
    "cleave_cuda_exp_f32": (c_buf, [c_buf]),
    "cleave_cuda_tanh_bwd_f32": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_sigmoid_bwd_f32": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_relu_bwd_f32": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_sum_f32": (f32, [c_buf]),
    "cleave_cuda_mean_f32": (f32, [c_buf]),
    "cleave_cuda_max_f32": (f32, [c_buf]),
    "cleave_cuda_sum_noalloc_f32": (i32, [ctypes.c_void_p, i64, ctypes.c_void_p, ctypes.c_void_p]),
    "cleave_cuda_colsum_f32": (c_buf, [c_buf, i32, i32]),
    "cleave_cuda_colsum_into_f32": (i32, [c_buf, c_buf, i32, i32]),
    "cleave_cuda_gemm_f32": (c_buf, [c_buf, c_buf, i32, i32, i32]),
    "cleave_cuda_gemm_nt_f32": (c_buf, [c_buf, c_buf, i32, i32, i32]),
    "cleave_cuda_gemm_tn_f32": (c_buf, [c_buf, c_buf, i32, i32, i32]),
    "cleave_cuda_gemm_batched_f32": (c_buf, [c_buf, c_buf, i32, i32, i32, i32]),
    "cleave_cuda_gemm_ex_f32": (i32, [c_buf, c_buf, c_buf, i32, i32, i32, i32, i32, i32, i32, c_buf, i32]),
    "cleave_cuda_gemm_dact_f32": (i32, [c_buf, c_buf, c_buf, i32, i32, i32, i32, i32, i32, i32, c_buf, i32]),
    "cleave_cuda_gemm_fused_f32": (i32, [c_buf, c_buf, c_buf, i32, i32, i32, i32, i32, i32, i32, c_buf, i32, c_buf, i32,
                                         c_buf, c_buf, c_buf]),
    "cleave_cuda_dense_grads_f32": (i32, [c_buf, c_buf, c_buf, c_buf, i32, i32, i32, c_buf, c_buf]),
    "cleave_cuda_split_lo_f32": (c_buf, [c_buf]),
    "cleave_cuda_split_lo_into_f32": (i32, [c_buf, c_buf, ctypes.c_void_p]),
    "cleave_cuda_bias_act_f32": (c_buf, [c_buf, c_buf, i32, i32, i32]),
    "cleave_cuda_mse_f32": (f32, [c_buf, c_buf, c_buf]),
    "cleave_cuda_mse_act_bwd_f32": (f32, [c_buf, c_buf, c_buf, i32]),
    "cleave_cuda_mse_act_bwd_dev_f32": (i32, [c_buf, c_buf, c_buf, i32, c_buf]),
    "cleave_cuda_mse_act_bwd_lo_f32": (i32, [c_buf, c_buf, c_buf, i32, c_buf, c_buf]),
    "cleave_cuda_sgd_f32": (i32, [c_buf, c_buf, f32, f32]),
    "cleave_cuda_host_gemm_f32": (i64, [c_f32p, i64, c_f32p, i64, c_f32p, i64, i32, i32, i32]),
    "cleave_cuda_host_binary_f32": (i64, [i32, c_f32p, i64, c_f32p, i64, c_f32p, i64]),
    "cleave_cuda_host_unary_f32": (i64, [i32, c_f32p, i64, c_f32p, i64]),
    "cleave_cuda_alloc_f64": (c_buf, [i64]),
    "cleave_cuda_upload_f64": (c_buf, [c_f64p, i64]),
    "cleave_cuda_download_f64": (i64, [c_buf, c_f64p, i64]),
    "cleave_cuda_fill_f64": (c_buf, [f64, i64]),
    "cleave_cuda_zeros_f64": (c_buf, [i64]),
    "cleave_cuda_get_f64": (f64, [c_buf, i64]),
    "cleave_cuda_add_f64": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_sub_f64": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_mul_f64": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_div_f64": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_neg_f64": (c_buf, [c_buf]),
    "cleave_cuda_relu_f64": (c_buf, [c_buf]),
    "cleave_cuda_sigmoid_f64": (c_buf, [c_buf]),
    "cleave_cuda_tanh_f64": (c_buf, [c_buf]),
    "cleave_cuda_exp_f64": (c_buf, [c_buf]),
    "cleave_cuda_sum_f64": (f64, [c_buf]),
    "cleave_cuda_mean_f64": (f64, [c_buf]),
    "cleave_cuda_max_f64": (f64, [c_buf]),
    "cleave_cuda_gemm_f64": (c_buf, [c_buf, c_buf, i32, i32, i32]),
    "cleave_cuda_gemm_nt_f64": (c_buf, [c_buf, c_buf, i32, i32, i32]),
    "cleave_cuda_gemm_tn_f64": (c_buf, [c_buf, c_buf, i32, i32, i32]),
    "cleave_cuda_gemm_batched_f64": (c_buf, [c_buf, c_buf, i32, i32, i32, i32]),
    "cleave_cuda_tanh_bwd_f64": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_sigmoid_bwd_f64": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_relu_bwd_f64": (c_buf, [c_buf, c_buf]),
    "cleave_cuda_colsum_f64": (c_buf, [c_buf, i32, i32]),
    "cleave_cuda_mse_f64": (f64, [c_buf, c_buf, c_buf]),
    "cleave_cuda_sgd_f64": (i32, [c_buf, c_buf, f64, f64]),
    "cleave_cuda_dp_sgd_allreduce_f32": (i32, [ctypes.POINTER(ctypes.c_void_p)] * 3 + [ctypes.c_void_p, ctypes.c_void_p,
                                                i64, i64, i32, i32, f32, ctypes.c_uint32, ctypes.c_void_p]),
    "cleave_cuda_linreg_step_f32": (f32, [c_buf, c_buf, c_buf, c_buf, c_buf, i32, i32]),
    "cleave_cuda_linreg_step_dev_f32": (i32, [c_buf, c_buf, c_buf, c_buf, c_buf, i32, i32, c_buf]),
}

_lib = None


class CleaveCudaError(RuntimeError):
    """A libcleave_cuda call failed; ``code`` is the CLEAVE_CUDA_ERR_* value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libcleave_cuda error {code}: {message}")
        self.code = code


def lib() -> ctypes.CDLL:
    """The loaded library with typed signatures.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m cleave_b200.build` "
                "(there is no CPU or PyTorch fallback for the tensor operators)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def raise_last_error(what: str = ""):
    L = lib()
    code = L.cleave_cuda_last_error()
    msg = (L.cleave_cuda_last_error_message() or b"").decode(errors="replace")
    L.cleave_cuda_clear_error()
    raise CleaveCudaError(code, f"{what}: {msg}" if what else msg)
