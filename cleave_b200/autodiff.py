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
from .linalg import Tensor, dense_grads, gemm_into, split_lo

_ACT_BWD = {"tanh": nn.tanh_bwd, "sigmoid": nn.sigmoid_bwd}


class MLP2:
    """Two-layer perceptron ``Y = act2(act1(X W1 + b1) W2 + b2)`` with an MSE loss.

    Parameters live in one contiguous device buffer ``params`` = [W1 | b1 | W2 | b2] and gradients
    in a buffer ``grads`` with the same layout; ``W1`` ... ``db2`` are views into them.
    """

    def __init__(self, d_in: int, d_hid: int, d_out: int, act1: str = "tanh", act2: str = "sigmoid",
                 params: Tensor | None = None, grads: Tensor | None = None, chain_lo: bool | None = None):
        """``params`` / ``grads``: optional caller-provided flat buffers (e.g. views of symmetric
        memory shared with the other data-parallel ranks); allocated here when omitted.
        ``chain_lo``: hand the lo planes of the tensor-core split from one product to the next (each GEMM's
        epilogue writes the plane its consumer needs) instead of letting every product split its operands
        again; default: on for layer sizes that are multiples of 32 (what the tensor-core route needs to read
        the tensors in place).  The gradients are bit-identical either way."""
        if act1 not in _ACT_BWD or act2 not in _ACT_BWD:
            raise ValueError("activations with a declared derivative rule: tanh, sigmoid")
        self.d_in, self.d_hid, self.d_out, self.act1, self.act2 = d_in, d_hid, d_out, act1, act2
        self.chain_lo = all(d % 32 == 0 for d in (d_in, d_hid, d_out)) if chain_lo is None else bool(chain_lo)
        self.weights_version = 0   # bumped by every method of this class that rewrites the weights (load, sgd)
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
        self.weights_version += 1
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
                         loss_out: Tensor | None = None, before_layer=None, weight_planes=None):
        """One forward + backward pass; gradients land in ``self.grads``.  Returns the loss
        (and, with ``keep``, the intermediates for inspection).  ``on_grads_ready(i)`` is called
        when a gradient bucket is final and its weights are no longer read in this pass:
        1 = [dW1 | db1] first, then 0 = [dW2 | db2].  ``before_layer(i)`` is called just before the
        first kernel that reads layer i's weights (1: W1, b1; 2: W2, b2), so a data-parallel driver can
        let the previous step's exchange of that layer run beside the kernels queued before it.
        ``weight_planes = (W1_lo, W2_lo)``: lo planes of the CURRENT weights that the caller maintains (either
        may be ``None``); without them the step splits the weights itself when it chains planes.
        With ``loss_out`` (a one-element tensor) the loss is left on the device, nothing waits and
        ``None`` is returned."""
        if before_layer:
            before_layer(1)
        batch = X.dims[0]
        # Lo planes travel with their tensors through the chain when the products are large enough for the
        # tensor cores (each plane is one extra store in a producer's epilogue, or one streaming pass).
        chain = self.chains_planes(batch)
        lo = (lambda t: split_lo(t)) if chain else (lambda t: None)
        new = (lambda *dims: Tensor.empty(*dims)) if chain else (lambda *dims: None)
        given1, given2 = weight_planes if weight_planes else (None, None)
        X_lo = lo(X)
        W1_lo = given1 if (chain and given1 is not None) else lo(self.W1)
        H_lo = new(batch, self.d_hid)
        H = gemm_into(Tensor.empty(batch, self.d_hid), X, self.W1, bias=self.b1, act=self.act1,
                      a_lo=X_lo, b_lo=W1_lo, c_lo=H_lo)
        if before_layer:
            before_layer(2)
        W2_lo = given2 if (chain and given2 is not None) else lo(self.W2)
        Y = gemm_into(Tensor.empty(batch, self.d_out), H, self.W2, bias=self.b2, act=self.act2, a_lo=H_lo, b_lo=W2_lo)
        if chain:
            dev_loss = loss_out if loss_out is not None else Tensor.empty(1)
            dZ2, dZ2_lo = nn.mse_act_bwd_lo(Y, T, self.act2, dev_loss)
            loss = None if loss_out is not None else dev_loss[0]
        else:
            loss, dZ2 = nn.mse_act_bwd(Y, T, self.act2, loss_out)   # dY and act2'(Y) * dY in one pass
            dZ2_lo = None
        # Without ``keep`` dH is never stored: dZ1 = act1'(H) * (dZ2 W2^T) leaves the GEMM's epilogue directly
        # (bit-identical to the two-step form, one pass over H instead of three over H-sized tensors).
        dH = None
        dZ1_lo = None
        if keep:
            dH = gemm_into(Tensor.empty(*H.dims), dZ2, self.W2, trans_b=True, a_lo=dZ2_lo, b_lo=W2_lo)   # dZ2 W2^T
            dZ1 = _ACT_BWD[self.act1](H, dH)
        else:
            dZ1_lo = new(*H.dims)
            dZ1 = gemm_into(Tensor.empty(*H.dims), dZ2, self.W2, trans_b=True, dact_of=H, dact=self.act1,
                            a_lo=dZ2_lo, b_lo=W2_lo, c_lo=dZ1_lo)
        # Layer 1's gradients first: W1 was last read by the forward product, so its exchange can run beside
        # the dW2 product, and layer 2's exchange beside the NEXT step's first forward product (which needs
        # only W1).  dZ1 above was the last reader of W2 in this pass.
        # Each layer's weight and bias gradient in one call: X^T dZ on the tensor cores, colsum(dZ) beside it.
        dense_grads(self.dW1, self.db1, X, dZ1, X_lo, dZ1_lo)
        if on_grads_ready:
            on_grads_ready(1)
        dense_grads(self.dW2, self.db2, H, dZ2, H_lo, dZ2_lo)
        if on_grads_ready:
            on_grads_ready(0)
        if keep:
            return loss, dict(H=H, Y=Y, dZ2=dZ2, dH=dH, dZ1=dZ1)
        return loss

    def chains_planes(self, batch: int) -> bool:
        """Whether a step at this batch size hands lo planes from product to product."""
        return bool(self.chain_lo and batch % 32 == 0 and batch * self.d_in * self.d_hid >= (1 << 24))

    def sgd(self, lr: float, gscale: float = 1.0) -> None:
        """``p = p - lr * gscale * g`` over the whole parameter buffer in one pass."""
        self.weights_version += 1
        nn.sgd_step(self.params, self.grads, lr, gscale)


def linreg_step(X: Tensor, y: Tensor, w: Tensor, want_pred: bool = True, loss_out: Tensor | None = None,
                grad_out: Tensor | None = None, pred_out: Tensor | None = None):
    """Linear-regression batch gradient step in one sweep over ``X`` [rows, feat]:
    returns ``(loss, grad, pred)`` with loss = mean((X w - y)^2) and grad = dloss/dw
    (examples/linear_regression.cleave:15-33 scaled to a real batch).  With ``loss_out`` (a one-element tensor)
    the loss stays on the device, the call does not wait and the returned loss is ``None``; ``grad_out`` /
    ``pred_out`` reuse the caller's tensors instead of allocating."""
    rows, feat = X.dims
    if y.dims != (rows,) or w.dims != (feat,):
        raise TypeError(f"linreg_step: X {X.dims}, y {y.dims}, w {w.dims}")
    grad = grad_out if grad_out is not None else Tensor.empty(feat)
    pred = pred_out if pred_out is not None else (Tensor.empty(rows) if want_pred else None)
    if loss_out is not None:
        if lib().cleave_cuda_linreg_step_dev_f32(X._h, y._h, w._h, pred._h if pred is not None else None, grad._h,
                                                 rows, feat, loss_out._h) != 0:
            raise_last_error("linreg_step_dev")
        return None, grad, pred
    loss = lib().cleave_cuda_linreg_step_f32(X._h, y._h, w._h, pred._h if pred is not None else None, grad._h,
                                             rows, feat)
    if math.isnan(loss) and lib().cleave_cuda_last_error():
        raise_last_error("linreg_step")
    return loss, grad, pred
