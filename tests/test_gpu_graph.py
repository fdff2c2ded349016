"""A step captured into a CUDA graph through the C ABI replays to the same bits as the eager step, keeps its own
blocks, and refuses calls that would wait inside a capture."""
import numpy as np
import pytest

import cleave_b200 as cb
from cleave_b200 import autodiff, linalg, nn, workloads

pytestmark = pytest.mark.gpu
f32 = np.float32


def test_captured_perceptron_step_replays_bit_identically():
    X, W1, b1, W2, b2, T = workloads.mlp_inputs(512, 256, 1024, 256)
    net = autodiff.MLP2(256, 1024, 256)
    net.load(W1, b1, W2, b2)
    tX, tT = linalg.Tensor(X), linalg.Tensor(T)
    loss_dev = linalg.Tensor.zero(1)
    net.forward_backward(tX, tT, loss_out=loss_dev)
    cb.sync()
    want_loss, want_grads = loss_dev[0], net.grads.numpy().copy()
    L = cb.lib()
    live = L.cleave_cuda_live_bytes()
    g = cb.StepGraph(lambda: net.forward_backward(tX, tT, loss_out=loss_dev))
    # between replays other work allocates and frees: it must not be handed the graph's blocks
    for i in range(3):
        scratch = [linalg.Tensor(workloads.normal(70 + i, 1 << 18)) for _ in range(4)]
        linalg.Tensor.filled(0.0, net.n_params)      # a fresh tensor of the gradients' size
        nn.sgd_step(net.grads, net.grads, 1.0)       # wipe the gradients: g - 1 * g
        loss_dev2 = nn.sum(scratch[0])
        g.replay()
        cb.sync()
        assert loss_dev[0] == want_loss
        assert np.array_equal(net.grads.numpy(), want_grads)
        assert loss_dev2 == nn.sum(scratch[0])
        del scratch
    g.close()
    assert L.cleave_cuda_live_bytes() == live
    # the eager path still works and agrees
    net.forward_backward(tX, tT, loss_out=loss_dev)
    cb.sync()
    assert np.array_equal(net.grads.numpy(), want_grads)


def test_capture_misuse_is_reported():
    L = cb.lib()
    assert L.cleave_cuda_graph_end() is None and L.cleave_cuda_last_error() == 4        # no capture open
    assert L.cleave_cuda_graph_launch(None) == -2                                       # not a graph handle
    L.cleave_cuda_clear_error()
    a = linalg.Tensor(np.ones(1024, f32))
    assert L.cleave_cuda_graph_begin() == 0
    assert L.cleave_cuda_graph_begin() == -4                                            # one capture at a time
    b = a + a                                                                           # recorded, not run
    h = L.cleave_cuda_graph_end()
    assert h
    L.cleave_cuda_clear_error()
    assert L.cleave_cuda_graph_launch(h) == 0
    cb.sync()
    assert b[5] == 2.0
    L.cleave_cuda_graph_free(h)
    L.cleave_cuda_graph_free(h)                                                         # a stale handle is ignored
    assert L.cleave_cuda_last_error() == 2
    L.cleave_cuda_clear_error()
