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


def test_cut_plan_of_a_partly_filled_last_wave():
    # host arithmetic of the CTA-pair GEMM: which tiles of the last wave are cut along K, and into how many runs
    import ctypes

    import cleave_b200 as cb
    L = cb.lib()
    runs = ctypes.c_int32(-1)

    def plan(tiles, k_blocks, pairs=74):
        cut = L.cleave_cuda_gemm_cut_plan(tiles, k_blocks, pairs, ctypes.byref(runs))
        return cut, runs.value

    assert plan(256, 128) == (34, 2)        # 4096^3: three waves + 34 tiles, cut in two
    assert plan(256, 32) == (34, 2)         # 4096 x 4096 x K1024: saves 16 K-blocks, just enough
    assert plan(256, 16) == (0, 0)          # K = 512: the second pass would cost what the cut saves
    assert plan(1024, 256) == (0, 0)        # 8192^3: the last wave has 62 of 74 tiles, nothing to share out
    assert plan(4096, 512) == (26, 2)       # 16384^3
    assert plan(80, 64) == (6, 8)           # a nearly empty wave: at most 8 runs
    assert plan(80, 32) == (6, 4)           # ... of at least 8 K-blocks each
    assert plan(80, 24) == (6, 3)
    assert plan(64, 128) == (0, 0)          # fewer tiles than SM pairs: a single wave is never cut
    assert plan(148, 128) == (0, 0)         # whole waves
    assert plan(0, 128) == (0, 0) and plan(100, 0) == (0, 0)
    for tiles in range(75, 400, 7):
        for kb in (16, 24, 32, 48, 64, 100, 128, 512):
            cut, r = plan(tiles, kb)
            if cut:
                assert cut == tiles % 74 and 2 <= r <= 8 and cut * r <= 74 and kb // r >= 8 and kb * (r - 1) >= 16 * r
                # the runs floor(kb * j / r) .. floor(kb * (j + 1) / r) partition the K-blocks
                edges = [kb * j // r for j in range(r + 1)]
                assert edges[0] == 0 and edges[-1] == kb and all(b > a for a, b in zip(edges, edges[1:]))
            else:
                assert r == 0
