"""Reverse-mode evaluation of the gradients cleave's ``derive()`` defines, on device tensors.

``derive()`` in the reference is forward-mode symbolic differentiation by e-graph rewriting: one
partial per scalar parameter, built from the declared rules
  add/sub/mul/div/neg   stdlib/num/num.cleave:123-136
  exp, tanh             stdlib/num/num.cleave:222-223
  matmul                stdlib/linalg/matrix.cleave:24   d matmul(a,b) = matmul(da,b) + matmul(a,db)
  index                 stdlib/linalg/tensor.cleave:126
The values are the mathematical gradient; for tensor-sized parameter sets the same numbers are
obtained in one backward sweep:  for  Y = act(X W + b):
  dZ = act'(.) * dY,   dW = X^T dZ,   db = colsum(dZ),   dX = dZ W^T
and for L = mean((Y - T)^2):  dY = 2 (Y - T) / numel.
Each step below is one libcleave_cuda call; bias + activation ride in the GEMM epilogue and the
weight gradients are written straight into one contiguous bucket (so a data-parallel run
all-reduces a single buffer with no packing pass).
"""
from __future__ import annotations

import math

import numpy as np

from . import nn
from ._lib import lib, raise_last_error
from .linalg import Tensor, gemm_into

_ACT_BWD = {"tanh": nn.tanh_bwd, "sigmoid": nn.sigmoid_bwd}


class MLP2:
    """Two-layer perceptron ``Y = act2(act1(X W1 + b1) W2 + b2)`` with an MSE loss.

    Parameters live in one contiguous device buffer ``params`` = [W1 | b1 | W2 | b2] and gradients
    in a buffer ``grads`` with the same layout; ``W1`` ... ``db2`` are views into them.
    """

    def __init__(self, d_in: int, d_hid: int, d_out: int, act1: str = "tanh", act2: str = "sigmoid",
                 params: Tensor | None = None, grads: Tensor | None = None):
        """``params`` / ``grads``: optional caller-provided flat buffers (e.g. views of symmetric
        memory shared with the other data-parallel ranks); allocated here when omitted."""
        if act1 not in _ACT_BWD or act2 not in _ACT_BWD:
            raise ValueError("activations with a declared derivative rule: tanh, sigmoid")
        self.d_in, self.d_hid, self.d_out, self.act1, self.act2 = d_in, d_hid, d_out, act1, act2
        sizes = [d_in * d_hid, d_hid, d_hid * d_out, d_out]
        shapes = [(d_in, d_hid), (d_hid,), (d_hid, d_out), (d_out,)]
        self.n_params = sum(sizes)
        for given in (params, grads):
            if given is not None and given.numel != self.n_params:
                raise TypeError(f"flat buffer has {given.numel} elements, the network has {self.n_params}")
        self.params = params if params is not None else Tensor.zero(self.n_params)
        self.grads = grads if grads is not None else Tensor.zero(self.n_params)
        offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        self._offsets = offs

        def views(buf):
            out = []
            for o, shp in zip(offs[:-1], shapes):
                v = Tensor.from_device_ptr(buf.data_ptr + 4 * int(o), *shp)
                v._owner = buf
                out.append(v)
            return out

        self.W1, self.b1, self.W2, self.b2 = views(self.params)
        self.dW1, self.db1, self.dW2, self.db2 = views(self.grads)

    def load(self, W1, b1, W2, b2) -> None:
        flat = np.concatenate([np.asarray(a, np.float32).ravel() for a in (W1, b1, W2, b2)])
        assert flat.size == self.n_params
        from ._lib import c_f32p
        if lib().cleave_cuda_upload_into_f32(self.params._h, flat.ctypes.data_as(c_f32p), flat.size) != 0:
            raise_last_error("MLP2.load")
        lib().cleave_cuda_sync()

    def forward(self, X: Tensor):
        batch = X.dims[0]
        H = gemm_into(Tensor.empty(batch, self.d_hid), X, self.W1, bias=self.b1, act=self.act1)
        Y = gemm_into(Tensor.empty(batch, self.d_out), H, self.W2, bias=self.b2, act=self.act2)
        return H, Y

    def forward_backward(self, X: Tensor, T: Tensor, keep: bool = False, on_grads_ready=None,
                         loss_out: Tensor | None = None):
        """One forward + backward pass; gradients land in ``self.grads``.  Returns the loss
        (and, with ``keep``, the intermediates for inspection).  ``on_grads_ready(i)`` is called
        when a gradient bucket is final: 0 = [dW2 | db2], 1 = [dW1 | db1].  With ``loss_out`` (a
        one-element tensor) the loss is left on the device, nothing waits and ``None`` is returned."""
        H, Y = self.forward(X)
        loss, dZ2 = nn.mse_act_bwd(Y, T, self.act2, loss_out)   # dY and act2'(Y) * dY in one pass
        # dH first: it is the last reader of W2 in this step, so once [dW2 | db2] are announced a
        # data-parallel exchange may already overwrite W2 and b2 while the rest of the pass runs.
        # Without ``keep`` dH is never stored: dZ1 = act1'(H) * (dZ2 W2^T) leaves the GEMM's epilogue directly
        # (bit-identical to the two-step form, one pass over H instead of three over H-sized tensors).
        dH = None
        if keep:
            dH = gemm_into(Tensor.empty(*H.dims), dZ2, self.W2, trans_b=True)   # dZ2 W2^T
            dZ1 = None
        else:
            dZ1 = gemm_into(Tensor.empty(*H.dims), dZ2, self.W2, trans_b=True, dact_of=H, dact=self.act1)
        gemm_into(self.dW2, H, dZ2, trans_a=True)            # H^T dZ2
        self._colsum_into(self.db2, dZ2)
        if on_grads_ready:
            on_grads_ready(0)
        if dZ1 is None:
            dZ1 = _ACT_BWD[self.act1](H, dH)
        gemm_into(self.dW1, X, dZ1, trans_a=True)            # X^T dZ1
        self._colsum_into(self.db1, dZ1)
        if on_grads_ready:
            on_grads_ready(1)
        if keep:
            return loss, dict(H=H, Y=Y, dZ2=dZ2, dH=dH, dZ1=dZ1)
        return loss

    @staticmethod
    def _colsum_into(out: Tensor, x: Tensor) -> None:
        if lib().cleave_cuda_colsum_into_f32(out._h, x._h, x.dims[0], x.dims[1]) != 0:
            raise_last_error("colsum_into")

    def sgd(self, lr: float, gscale: float = 1.0) -> None:
        """``p = p - lr * gscale * g`` over the whole parameter buffer in one pass."""
        nn.sgd_step(self.params, self.grads, lr, gscale)


def linreg_step(X: Tensor, y: Tensor, w: Tensor, want_pred: bool = True):
    """Linear-regression batch gradient step in one sweep over ``X`` [rows, feat]:
    returns ``(loss, grad, pred)`` with loss = mean((X w - y)^2) and grad = dloss/dw
    (examples/linear_regression.cleave:15-33 scaled to a real batch)."""
    rows, feat = X.dims
    if y.dims != (rows,) or w.dims != (feat,):
        raise TypeError(f"linreg_step: X {X.dims}, y {y.dims}, w {w.dims}")
    grad = Tensor.empty(feat)
    pred = Tensor.empty(rows) if want_pred else None
    loss = lib().cleave_cuda_linreg_step_f32(X._h, y._h, w._h, pred._h if pred is not None else None, grad._h,
                                             rows, feat)
    if math.isnan(loss) and lib().cleave_cuda_last_error():
        raise_last_error("linreg_step")
    return loss, grad, pred
