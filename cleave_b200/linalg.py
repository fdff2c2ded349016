"""Host-side mirror of cleave's ``stdlib/linalg`` over device tensors.

``Tensor`` corresponds to ``struct Tensor<T: Float, const Dims...: i32>``
(stdlib/linalg/tensor.cleave:40): dense, row-major, static shape, immutable value.  Its
operators are the ``Ring<Tensor<T, Dims...>>`` impl (tensor.cleave:66-80) -- ``+ - * /`` and unary
``-`` are elementwise on same-shape operands, ``zero`` is the zero tensor -- ``t[i, j]`` is
``Index::index`` (tensor.cleave:129-133) and ``matmul`` is ``MatMul::matmul``
(stdlib/linalg/matrix.cleave:22-62).  Each method is one call into ``libcleave_cuda`` with
exactly the arguments the matching ``extern(cleave_cuda_*) fn`` would pass.

Where cleave rejects a program at compile time (shape mismatch, wrong index rank) these
functions raise ``TypeError``; a failing library call raises ``CleaveCudaError``.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from ._lib import c_f32p, c_f64p, lib, raise_last_error

_NP = {"f32": np.float32, "f64": np.float64}
_PTR = {"f32": c_f32p, "f64": c_f64p}


def _prod(dims) -> int:
    return int(math.prod(dims))


class Tensor:
    """``Tensor<T, Dims...>`` for ``T`` = f32 (default) or f64: a device-resident array with a static shape."""

    __slots__ = ("_h", "dims", "dtype", "_owner")

    def __init__(self, data=None, *, dims=None, dtype: str = "f32", _handle=None):
        """``Tensor(data)`` uploads a nested list / array, like ``Tensor::<f32, ...>(data: [...])``."""
        if dtype not in _NP:
            raise TypeError(f"Tensor element type must be f32 or f64, not {dtype!r}")
        self.dtype = dtype
        if _handle is not None:
            self._h, self.dims = _handle, tuple(int(d) for d in dims)
            return
        a = np.ascontiguousarray(data, dtype=_NP[dtype])
        if dims is not None and tuple(dims) != a.shape:
            raise TypeError(f"data has shape {a.shape}, declared dims are {tuple(dims)}")
        if a.ndim < 1 or a.size == 0:
            raise TypeError("a Tensor needs rank >= 1 and at least one element")
        h = self._fn("upload")(a.ctypes.data_as(_PTR[dtype]), a.size)
        if not h:
            raise_last_error("Tensor upload")
        self._h, self.dims = h, a.shape

    def _fn(self, op: str):
        """The library entry point of ``op`` for this tensor's element type."""
        return getattr(lib(), f"cleave_cuda_{op}_{self.dtype}")

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def _wrap(cls, handle, dims, what="op", dtype: str = "f32"):
        if not handle:
            raise_last_error(what)
        return cls(dims=dims, dtype=dtype, _handle=handle)

    @classmethod
    def zero(cls, *dims, dtype: str = "f32") -> "Tensor":
        """``Ring::zero()`` for ``Tensor<T, dims...>`` (tensor.cleave:79)."""
        return cls._wrap(getattr(lib(), f"cleave_cuda_zeros_{dtype}")(_prod(dims)), dims, "zero", dtype)

    @classmethod
    def filled(cls, value: float, *dims, dtype: str = "f32") -> "Tensor":
        """``Tensor::<T, Dims...>(data: [value; Dims...])``."""
        return cls._wrap(getattr(lib(), f"cleave_cuda_fill_{dtype}")(float(value), _prod(dims)), dims, "fill", dtype)

    @classmethod
    def empty(cls, *dims, dtype: str = "f32") -> "Tensor":
        return cls._wrap(getattr(lib(), f"cleave_cuda_alloc_{dtype}")(_prod(dims)), dims, "alloc", dtype)

    @classmethod
    def from_device_ptr(cls, ptr: int, *dims) -> "Tensor":
        """Non-owning view of caller-owned device memory (e.g. a torch CUDA tensor's data_ptr)."""
        return cls._wrap(lib().cleave_cuda_wrap_f32(ctypes.c_void_p(ptr), _prod(dims)), dims, "wrap")

    # ---- readback -----------------------------------------------------------------------
    @property
    def numel(self) -> int:
        return _prod(self.dims)

    @property
    def data_ptr(self) -> int:
        return int(lib().cleave_cuda_data_ptr(self._h) or 0)

    def numpy(self, out: np.ndarray | None = None) -> np.ndarray:
        if out is None:
            out = np.empty(self.dims, _NP[self.dtype])
        assert out.dtype == _NP[self.dtype] and out.size == self.numel and out.flags.c_contiguous
        if self._fn("download")(self._h, out.ctypes.data_as(_PTR[self.dtype]), out.size) < 0:
            raise_last_error("download")
        return out

    def reshape(self, *dims) -> "Tensor":
        """Same storage, new static shape (row-major flattening is the identity on memory)."""
        if _prod(dims) != self.numel:
            raise TypeError(f"cannot view {self.dims} as {dims}")
        if self.dtype != "f32":
            raise TypeError("views are available for f32 tensors only")
        t = Tensor.from_device_ptr(self.data_ptr, *dims)
        t._owner = self   # keep the storage alive
        return t

    def __getitem__(self, idx) -> float:
        """``t[i, j, ...]`` -> scalar; the index count must equal the rank (tensor.cleave:129-133)."""
        idx = idx if isinstance(idx, tuple) else (idx,)
        if len(idx) != len(self.dims):
            raise TypeError(f"tensor of rank {len(self.dims)} indexed with {len(idx)} indices")
        flat = 0
        for i, d in zip(idx, self.dims):
            if not 0 <= int(i) < d:
                raise IndexError(f"index {idx} out of bounds for dims {self.dims}")
            flat = flat * d + int(i)
        v = self._fn("get")(self._h, flat)
        if math.isnan(v) and lib().cleave_cuda_last_error():
            raise_last_error("index")
        return float(_NP[self.dtype](v))

    # ---- Ring<Tensor> -------------------------------------------------------------------
    def _binary(self, other, name):
        if not isinstance(other, Tensor):
            raise TypeError(f"{name}: operand is not a Tensor (a bare scalar is not broadcast)")
        if other.dims != self.dims or other.dtype != self.dtype:
            raise TypeError(f"{name}: mismatched types {self!r} and {other!r}")
        return Tensor._wrap(self._fn(name)(self._h, other._h), self.dims, name, self.dtype)

    def __add__(self, o): return self._binary(o, "add")
    def __sub__(self, o): return self._binary(o, "sub")
    def __mul__(self, o): return self._binary(o, "mul")
    def __truediv__(self, o): return self._binary(o, "div")
    def __neg__(self): return Tensor._wrap(self._fn("neg")(self._h), self.dims, "neg", self.dtype)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                lib().cleave_cuda_free(h)
            except Exception:  # interpreter shutdown
                pass

    def __repr__(self):
        return f"Tensor<{self.dtype}, {', '.join(map(str, self.dims))}>"


def matmul(a: Tensor, b: Tensor) -> Tensor:
    """``MatMul<Tensor<T,N,M>, Tensor<T,M,K>, Tensor<T,N,K>>::matmul`` (matrix.cleave:27-62)."""
    if len(a.dims) != 2 or len(b.dims) != 2 or a.dims[1] != b.dims[0] or a.dtype != b.dtype:
        raise TypeError(f"matmul: no impl for {a!r} x {b!r}")
    (m, k), n = a.dims, b.dims[1]
    return Tensor._wrap(a._fn("gemm")(a._h, b._h, m, n, k), (m, n), "matmul", a.dtype)


def matmul_nt(a: Tensor, b: Tensor) -> Tensor:
    """``a @ b^T`` with b stored [n, k]: the ``matmul(d(a), b)`` half of the derivative rule
    (matrix.cleave:24) pulled back to the first operand."""
    if len(a.dims) != 2 or len(b.dims) != 2 or a.dims[1] != b.dims[1]:
        raise TypeError(f"matmul_nt: no impl for Tensor<f32,{a.dims}> x Tensor<f32,{b.dims}>^T")
    (m, k), n = a.dims, b.dims[0]
    return Tensor._wrap(lib().cleave_cuda_gemm_nt_f32(a._h, b._h, m, n, k), (m, n), "matmul_nt")


def matmul_tn(a: Tensor, b: Tensor) -> Tensor:
    """``a^T @ b`` with a stored [k, m]: the ``matmul(a, d(b))`` half pulled back to the second operand."""
    if len(a.dims) != 2 or len(b.dims) != 2 or a.dims[0] != b.dims[0]:
        raise TypeError(f"matmul_tn: no impl for Tensor<f32,{a.dims}>^T x Tensor<f32,{b.dims}>")
    (k, m), n = a.dims, b.dims[1]
    return Tensor._wrap(lib().cleave_cuda_gemm_tn_f32(a._h, b._h, m, n, k), (m, n), "matmul_tn")


def batched_matmul(a: Tensor, b: Tensor) -> Tensor:
    """``batch`` independent products: a is [batch, m, k], b is [batch, k, n]."""
    if len(a.dims) != 3 or len(b.dims) != 3 or a.dims[0] != b.dims[0] or a.dims[2] != b.dims[1]:
        raise TypeError(f"batched_matmul: no impl for Tensor<f32,{a.dims}> x Tensor<f32,{b.dims}>")
    batch, m, k = a.dims
    n = b.dims[2]
    return Tensor._wrap(lib().cleave_cuda_gemm_batched_f32(a._h, b._h, batch, m, n, k), (batch, m, n),
                        "batched_matmul")


GEMM_AUTO, GEMM_EXACT, GEMM_3XTF32 = 0, 1, 2
ACT = {"identity": 0, "relu": 1, "sigmoid": 2, "tanh": 3}


def dense_grads(dw: Tensor, db: Tensor, x: Tensor, dz: Tensor, x_lo: Tensor | None = None,
                dz_lo: Tensor | None = None) -> None:
    """Both gradients of a dense layer from the gradient ``dz`` [rows, d_out] of its output: ``dw = x^T dz`` and
    ``db = colsum(dz)``, the column sums queued beside the product (``cleave_cuda_dense_grads_f32``)."""
    rows, d_in = x.dims
    if dz.dims[0] != rows or dw.dims != (d_in, dz.dims[1]) or db.dims != (dz.dims[1],):
        raise TypeError(f"dense_grads: x {x.dims}, dz {dz.dims} -> dw {dw.dims}, db {db.dims} do not agree")
    h = lambda t: t._h if t is not None else None  # noqa: E731
    if lib().cleave_cuda_dense_grads_f32(dw._h, db._h, x._h, dz._h, rows, d_in, dz.dims[1], h(x_lo), h(dz_lo)) != 0:
        raise_last_error("dense_grads")


def split_lo(x: Tensor) -> Tensor:
    """The lo plane of ``x`` (``cleave_cuda_split_lo_f32``): what the tensor-core path needs beside ``x`` itself."""
    return Tensor._wrap(lib().cleave_cuda_split_lo_f32(x._h), x.dims, "split_lo")


def gemm_into(c: Tensor, a: Tensor, b: Tensor, *, trans_a=False, trans_b=False, algo=GEMM_AUTO,
              bias: Tensor | None = None, act: str = "identity", dact_of: Tensor | None = None,
              dact: str = "identity", a_lo: Tensor | None = None, b_lo: Tensor | None = None,
              c_lo: Tensor | None = None) -> Tensor:
    """General product written into ``c`` (``cleave_cuda_gemm_ex_f32``).  Shapes follow the stored
    layouts: a is [m,k] ([k,m] if trans_a), b is [k,n] ([n,k] if trans_b); a leading batch
    dimension on all three runs independent products.

    ``dact_of=y, dact=name`` selects the backward form ``c = name'(y) * (a @ b)`` elementwise, the
    derivative taken from the activation's forward output ``y`` (``cleave_cuda_gemm_dact_f32``).

    ``a_lo`` / ``b_lo``: lo planes of the operands the caller already holds; ``c_lo``: tensor that receives the lo
    plane of the result (``cleave_cuda_gemm_fused_f32``), so a chain of products runs without operand pre-passes."""
    batched = len(c.dims) == 3
    batch = c.dims[0] if batched else 1
    ad, bd, cd = (t.dims[1:] if batched else t.dims for t in (a, b, c))
    m, k = (ad[1], ad[0]) if trans_a else ad
    k2, n = (bd[1], bd[0]) if trans_b else bd
    if k != k2 or tuple(cd) != (m, n) or (batched and not (a.dims[0] == b.dims[0] == batch)):
        raise TypeError(f"gemm_into: shapes {a.dims}, {b.dims} -> {c.dims} do not agree")
    if dact_of is not None:
        if bias is not None or act != "identity":
            raise TypeError("gemm_into: the backward form takes no bias and no forward activation")
        if dact_of.dims != c.dims:
            raise TypeError(f"gemm_into: dact_of has shape {dact_of.dims}, the product {c.dims}")
    if a_lo is not None or b_lo is not None or c_lo is not None:
        for t, lo, what in ((a, a_lo, "a_lo"), (b, b_lo, "b_lo"), (c, c_lo, "c_lo")):
            if lo is not None and lo.numel != t.numel:
                raise TypeError(f"gemm_into: {what} has {lo.numel} elements, its tensor {t.numel}")
        h = lambda t: t._h if t is not None else None  # noqa: E731
        r = lib().cleave_cuda_gemm_fused_f32(c._h, a._h, b._h, batch, m, n, k, int(trans_a), int(trans_b), algo, h(bias),
                                             ACT[act], h(dact_of), ACT[dact], h(a_lo), h(b_lo), h(c_lo))
        if r != 0:
            raise_last_error("gemm_into")
        return c
    if dact_of is not None:
        r = lib().cleave_cuda_gemm_dact_f32(c._h, a._h, b._h, batch, m, n, k, int(trans_a), int(trans_b), algo,
                                            dact_of._h, ACT[dact])
        if r != 0:
            raise_last_error("gemm_into")
        return c
    r = lib().cleave_cuda_gemm_ex_f32(c._h, a._h, b._h, batch, m, n, k, int(trans_a), int(trans_b), algo,
                                      bias._h if bias is not None else None, ACT[act])
    if r != 0:
        raise_last_error("gemm_into")
    return c
