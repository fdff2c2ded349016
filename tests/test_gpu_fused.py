"""Fused entry points equal the chains of primitive ops they replace, bit for bit."""
import numpy as np
import pytest

from cleave_b200 import linalg, nn
from oracle import ref

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
@pytest.mark.parametrize("act", ["identity", "sigmoid", "tanh"])
def test_mse_act_bwd_equals_mse_then_activation_backward(n, act):
    rng = np.random.default_rng(n)
    z = rng.standard_normal(n).astype(f32)
    y = z if act == "identity" else getattr(ref, act)(z)
    t = rng.uniform(0, 1, n).astype(f32)
    ty, tt = linalg.Tensor(y), linalg.Tensor(t)
    loss, dz = nn.mse_act_bwd(ty, tt, act)
    loss2, dy = nn.mse(ty, tt)
    chain = dy if act == "identity" else getattr(nn, act + "_bwd")(ty, dy)
    assert loss == loss2
    assert np.array_equal(dz.numpy(), chain.numpy())
    # and both equal the oracle's chain
    _, dy_ref = ref.mse(y, t)
    want = dy_ref if act == "identity" else getattr(ref, act + "_bwd")(y, dy_ref)
    assert np.array_equal(dz.numpy(), want)


def test_mse_act_bwd_rejects_relu():
    import cleave_b200 as cb
    y = linalg.Tensor(np.ones(4, f32))
    with pytest.raises(cb.CleaveCudaError):
        nn.mse_act_bwd(y, y, "relu")


def test_device_resident_loss_equals_the_returned_loss():
    rng = np.random.default_rng(3)
    y = rng.uniform(0, 1, 50001).astype(f32)
    t = rng.uniform(0, 1, 50001).astype(f32)
    ty, tt = linalg.Tensor(y), linalg.Tensor(t)
    loss, dz = nn.mse_act_bwd(ty, tt, "sigmoid")
    out = linalg.Tensor.zero(1)
    none, dz2 = nn.mse_act_bwd(ty, tt, "sigmoid", loss_out=out)
    assert none is None
    assert out[0] == loss
    assert np.array_equal(dz.numpy(), dz2.numpy())
