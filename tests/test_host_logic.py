"""Host-side logic that needs no device: static-shape checks that mirror cleave's compile-time
type errors, and the seeded workload generators."""
import numpy as np
import pytest

from cleave_b200 import linalg, nn, workloads


def fake(*dims):
    # A Tensor with a handle the library has never issued: shape checks must fire before any call.
    return linalg.Tensor(dims=dims, _handle=0)


def test_ring_ops_reject_mismatched_shapes_like_a_type_error():
    a, b = fake(2, 3), fake(3, 2)
    for op in (lambda: a + b, lambda: a - b, lambda: a * b, lambda: a / b):
        with pytest.raises(TypeError):
            op()
    with pytest.raises(TypeError):
        a + 1.0   # a bare scalar is not broadcast (nn.cleave:72-74)


def test_matmul_requires_matching_inner_dimension():
    with pytest.raises(TypeError):
        linalg.matmul(fake(2, 3), fake(2, 3))
    with pytest.raises(TypeError):
        linalg.matmul(fake(6), fake(6))
    with pytest.raises(TypeError):
        linalg.matmul_nt(fake(2, 3), fake(4, 5))
    with pytest.raises(TypeError):
        linalg.matmul_tn(fake(2, 3), fake(4, 5))
    with pytest.raises(TypeError):
        linalg.batched_matmul(fake(2, 3, 4), fake(3, 4, 5))


def test_index_rank_must_equal_tensor_rank():
    # cleave rejects m[i,j,k] on a rank-2 tensor (tests/mlir_lower.rs, "3 indices on a rank-2 Tensor")
    with pytest.raises(TypeError):
        fake(2, 2)[0, 1, 0]
    with pytest.raises(TypeError):
        fake(2, 2, 2)[0]
    with pytest.raises(IndexError):
        fake(2, 2)[0, 2]


def test_bias_and_loss_helpers_check_shapes():
    with pytest.raises(TypeError):
        nn.bias_act(fake(4, 8), fake(4))
    with pytest.raises(TypeError):
        nn.mse(fake(4, 8), fake(8, 4))
    with pytest.raises(TypeError):
        nn.sgd_step(fake(8), fake(9), 0.1)
    with pytest.raises(TypeError):
        nn.colsum(fake(8))


def test_workloads_are_reproducible_and_distributed_as_stated():
    a1, b1 = workloads.gemm_inputs(64, 48, 32)
    a2, b2 = workloads.gemm_inputs(64, 48, 32)
    assert np.array_equal(a1, a2) and np.array_equal(b1, b2) and not np.array_equal(a1[:32, :32], b1[:32, :32])
    assert a1.dtype == np.float32 and a1.min() >= -1 and a1.max() < 1
    X, y, w = workloads.linreg_inputs(4096, 16)
    assert X.shape == (4096, 16) and y.shape == (4096,) and w.shape == (16,)
    noise = y - X @ w
    assert 0.08 < noise.std() < 0.12          # sigma 0.1 (variance 0.01)
    X, W1, b1_, W2, b2_, T = workloads.mlp_inputs(32, 16, 64, 8)
    lim = np.sqrt(6.0 / (16 + 64))
    assert np.abs(W1).max() <= lim and not b1_.any() and not b2_.any()
    assert T.min() >= 0 and T.max() < 1


def test_shard_properties_hold_for_arbitrary_sizes():
    from hypothesis import given, settings, strategies as st

    from cleave_b200 import dp

    @settings(max_examples=200, deadline=None)
    @given(st.integers(0, 10**7), st.integers(1, 16))
    def check(n, world):
        spans = [dp.shard(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert all(s >= 0 for s in sizes) and max(sizes) - min(sizes) <= 1
        blocks = [dp.row_block(n, r, world) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        owned = sorted(b for r in range(world) for b in dp.batch_shard(min(n, 500), r, world))
        assert owned == list(range(min(n, 500)))

    check()


def test_batch_chunking_respects_workspace_batch_and_grid_limits():
    # entries per pass = min(workspace limit / bytes per entry, batch, 65535), at least 1
    import os

    import cleave_b200 as cb
    L = cb.lib()
    os.environ.pop("CLEAVE_CUDA_GEMM_WORKSPACE_MB", None)
    gib = 1 << 30
    assert L.cleave_cuda_gemm_batch_chunk(128 << 20, 64) == 32          # 4 GiB / 128 MiB
    assert L.cleave_cuda_gemm_batch_chunk(128 << 20, 20) == 20          # never more than the batch
    assert L.cleave_cuda_gemm_batch_chunk(16 * gib, 7) == 1             # an entry larger than the limit still runs
    assert L.cleave_cuda_gemm_batch_chunk(1024, 1 << 20) == 65535       # gridDim.z
    assert L.cleave_cuda_gemm_batch_chunk(0, 5) == 5
    os.environ["CLEAVE_CUDA_GEMM_WORKSPACE_MB"] = "1"
    try:
        assert L.cleave_cuda_gemm_batch_chunk(300 << 10, 64) == 3       # 1 MiB / 300 KiB
    finally:
        del os.environ["CLEAVE_CUDA_GEMM_WORKSPACE_MB"]


def test_the_absent_operand_is_a_null_handle():
    import cleave_b200 as cb
    assert cb.lib().cleave_cuda_none() is None
