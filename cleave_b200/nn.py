"""Host-side mirror of cleave's ``stdlib/nn`` over device tensors.

``relu`` / ``sigmoid`` / ``tanh`` are ``Activation<Tensor<T, N>>`` (stdlib/nn/nn.cleave:82-95),
``exp`` is ``Transcendental::exp`` applied elementwise (stdlib/num/num.cleave:227), ``sum`` /
``mean`` / ``max_of`` are the ``Sum`` / ``Mean`` / ``Max`` algebras (nn.cleave:111-149).  The
reference declares the tensor impls for rank 1 only and applies them to matrices element by
element (examples/xor_tensor.cleave:38-40); here every rank is accepted and reduced over the
row-major flattening, which is the same sequence of elements.
"""
from __future__ import annotations

import math

from ._lib import lib, raise_last_error
from .linalg import ACT, Tensor


def _unary(what: str):
    def f(x: Tensor) -> Tensor:
        return Tensor._wrap(x._fn(what)(x._h), x.dims, what, x.dtype)

    f.__name__ = what
    return f


relu = _unary("relu")
sigmoid = _unary("sigmoid")
tanh = _unary("tanh")
exp = _unary("exp")


def _scalar(op: str, what: str):
    def f(v: Tensor) -> float:
        r = v._fn(op)(v._h)
        if math.isnan(r) and lib().cleave_cuda_last_error():
            raise_last_error(what)
        return r

    f.__name__ = what
    return f


sum = _scalar("sum", "sum")  # noqa: A001 - the reference's name
mean = _scalar("mean", "mean")
max_of = _scalar("max", "max_of")


# ---- derivative forms (what derive() emits for the activations, applied to a whole tensor) ------
def _bwd(fn_name: str, what: str):
    def f(y_or_x: Tensor, upstream: Tensor) -> Tensor:
        if y_or_x.dims != upstream.dims:
            raise TypeError(f"{what}: mismatched types {y_or_x!r} and {upstream!r}")
        return Tensor._wrap(getattr(lib(), fn_name)(y_or_x._h, upstream._h), upstream.dims, what)

    f.__name__ = what
    return f


tanh_bwd = _bwd("cleave_cuda_tanh_bwd_f32", "tanh_bwd")          # (1 - y*y) * g, y = tanh(x)
sigmoid_bwd = _bwd("cleave_cuda_sigmoid_bwd_f32", "sigmoid_bwd")  # y*(1-y) * g, y = sigmoid(x)
relu_bwd = _bwd("cleave_cuda_relu_bwd_f32", "relu_bwd")          # x > 0 ? g : 0


def colsum(x: Tensor) -> Tensor:
    """``sum`` of each column of a matrix: the gradient of a row-broadcast bias."""
    if len(x.dims) != 2:
        raise TypeError("colsum needs a rank-2 tensor")
    return Tensor._wrap(lib().cleave_cuda_colsum_f32(x._h, x.dims[0], x.dims[1]), (x.dims[1],), "colsum")


def bias_act(x: Tensor, bias: Tensor, act: str = "identity") -> Tensor:
    """``act(x + B)`` where every row of B equals ``bias`` (arith.addf does not broadcast, nn.cleave:72-74)."""
    if len(x.dims) != 2 or bias.dims != (x.dims[1],):
        raise TypeError(f"bias_act: {x!r} with bias {bias!r}")
    return Tensor._wrap(lib().cleave_cuda_bias_act_f32(x._h, bias._h, x.dims[0], x.dims[1], ACT[act]), x.dims,
                        "bias_act")


def mse(pred: Tensor, target: Tensor, want_grad: bool = True):
    """``mean((pred - target)^2)`` and, if asked, its gradient ``2 (pred - target) / numel``."""
    if pred.dims != target.dims:
        raise TypeError(f"mse: mismatched types {pred!r} and {target!r}")
    d = Tensor.empty(*pred.dims) if want_grad else None
    loss = lib().cleave_cuda_mse_f32(pred._h, target._h, d._h if d is not None else None)
    if math.isnan(loss) and lib().cleave_cuda_last_error():
        raise_last_error("mse")
    return (loss, d) if want_grad else loss


def mse_act_bwd(y: Tensor, target: Tensor, act: str, loss_out: Tensor | None = None):
    """Loss ``mean((y - target)^2)`` for ``y = act(z)`` and the gradient with respect to ``z``
    (``act'(y) * 2 (y - target) / numel``) in one pass; equals ``mse`` followed by ``*_bwd``.
    With ``loss_out`` (a one-element tensor) the loss stays on the device, the call does not wait
    and the returned loss is ``None``."""
    if y.dims != target.dims:
        raise TypeError(f"mse_act_bwd: mismatched types {y!r} and {target!r}")
    dz = Tensor.empty(*y.dims)
    if loss_out is not None:
        if lib().cleave_cuda_mse_act_bwd_dev_f32(y._h, target._h, dz._h, ACT[act], loss_out._h) != 0:
            raise_last_error("mse_act_bwd_dev")
        return None, dz
    loss = lib().cleave_cuda_mse_act_bwd_f32(y._h, target._h, dz._h, ACT[act])
    if math.isnan(loss) and lib().cleave_cuda_last_error():
        raise_last_error("mse_act_bwd")
    return loss, dz


def mse_act_bwd_lo(y: Tensor, target: Tensor, act: str, loss_out: Tensor):
    """``mse_act_bwd`` with the loss left in ``loss_out`` that also returns the lo plane of the gradient
    (``cleave_cuda_mse_act_bwd_lo_f32``): ``(dz, dz_lo)``."""
    if y.dims != target.dims:
        raise TypeError(f"mse_act_bwd_lo: mismatched types {y!r} and {target!r}")
    dz, dz_lo = Tensor.empty(*y.dims), Tensor.empty(*y.dims)
    if lib().cleave_cuda_mse_act_bwd_lo_f32(y._h, target._h, dz._h, ACT[act], loss_out._h, dz_lo._h) != 0:
        raise_last_error("mse_act_bwd_lo")
    return dz, dz_lo


def sgd_step(w: Tensor, g: Tensor, lr: float, gscale: float = 1.0) -> None:
    """``w = w - lr * (gscale * g)`` in place (examples/xor.cleave:67-70)."""
    if w.dims != g.dims:
        raise TypeError(f"sgd_step: mismatched types {w!r} and {g!r}")
    if lib().cleave_cuda_sgd_f32(w._h, g._h, float(lr), float(gscale)) != 0:
        raise_last_error("sgd")
