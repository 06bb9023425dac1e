"""The block projection kernel on the tensor pipe (2..256 tokens, weights streamed once) through the
per-operator C ABI, against the CPU oracle's row-by-row mat-vec."""
import numpy as np
import pytest

from nerva_b200 import ops, synth

pytestmark = pytest.mark.gpu

# bf16 products accumulated in fp32 by the MMA in its own order: rounding noise of partial sums,
# the same bound as the single-token projection tests
PROJ_ATOL = 2e-3


def _weights(rows, cols, tid=77):
    return ops.synth_normal_bf16(0, tid, rows * cols, 0.02)


def _acts(cols, tokens, tid=synth.T_ACTIVATION):
    return ops.synth_normal_bf16(0, tid, tokens * cols, 1.0)


def _oracle_rows(oracle_mod, w, x, rows, cols, tokens, sample=None):
    wm = w.reshape(rows, cols)
    if sample is not None:
        wm = np.ascontiguousarray(wm[sample])
    return np.stack([oracle_mod.matvec(wm, synth.bf16_to_f32(x[m * cols:(m + 1) * cols]), wm.shape[0], cols)
                     for m in range(tokens)])


@pytest.mark.parametrize("rows,cols,tokens", [
    (768, 512, 2), (512, 512, 4), (3072, 512, 16), (512, 1536, 64),   # tiny-config shapes
    (1000, 1408, 5), (37, 4096, 3), (130, 64, 7),                     # ragged row counts, one 64-wide slice
    (4096, 4096, 100), (6144, 4096, 256), (4096, 12288, 33),          # Qwen3-8B O, QKV, down
])
def test_block_projection_matches_oracle(built_lib, oracle_mod, rows, cols, tokens):
    w, x = _weights(rows, cols), _acts(cols, tokens)
    y, _ = ops.projection(w, x, rows, cols, tokens=tokens)
    ref = _oracle_rows(oracle_mod, w, x, rows, cols, tokens)
    assert np.isfinite(y).all()
    assert np.abs(y - ref).max() <= PROJ_ATOL
    # bit-stable run to run (partials of split tiles are added in a fixed order)
    y2, _ = ops.projection(w, x, rows, cols, tokens=tokens)
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("rows,cols", [(24576, 4096), (151936, 4096)])
@pytest.mark.parametrize("tokens", [4, 16, 64])
def test_block_projection_full_size_row_sample(built_lib, oracle_mod, rows, cols, tokens):
    """Gate/up and lm_head at full size: every 997th row of every token against the oracle."""
    w, x = _weights(rows, cols), _acts(cols, tokens)
    y, _ = ops.projection(w, x, rows, cols, tokens=tokens)
    sample = np.arange(0, rows, 997)
    ref = _oracle_rows(oracle_mod, w, x, rows, cols, tokens, sample)
    assert np.abs(y[:, sample] - ref).max() <= PROJ_ATOL


def test_a_tokens_result_does_not_depend_on_its_block(built_lib):
    """The same activation row alone with one neighbour, in a block of 16 and in a block of 64:
    identical bits (the work partition depends on the matrix shape only)."""
    rows, cols = 4096, 4096
    w = _weights(rows, cols)
    x = _acts(cols, 64)
    y64, _ = ops.projection(w, x, rows, cols, tokens=64)
    y16, _ = ops.projection(w, x[:16 * cols], rows, cols, tokens=16)
    y2, _ = ops.projection(w, x[:2 * cols], rows, cols, tokens=2)
    assert np.array_equal(y64[:16], y16)
    assert np.array_equal(y16[:2], y2)
    # and it is the single-token kernel's result within the operator bound
    y1, _ = ops.projection(w, x[:cols], rows, cols, tokens=1)
    assert np.abs(y1[0] - y2[0]).max() <= PROJ_ATOL


def test_reference_projection_bench_entry_point_with_a_block(built_lib):
    """nerva_cuda_projection_bench with block_tokens: the reference's own check (deterministic
    inputs, 0.25 absolute) plus this library's fp64 check of every token of the block."""
    import ctypes as C
    from nerva_b200 import ffi
    req = ffi.ProjectionBenchRequest(dtype=1, rows=4096, cols=4096, iterations=5, warmup_iterations=2, block_tokens=8)
    out = ffi.ProjectionBenchResult()
    rc = ffi.lib().nerva_cuda_projection_bench(C.byref(req), C.byref(out))
    assert rc == 0 and out.status == 0, (out.cuda_error, out.mismatch_count, ffi.last_error())
    assert out.mismatch_count == 0 and out.block_tokens == 8
    assert out.custom_avg_ns > 0 and out.block_cublaslt_avg_ns > 0 and out.block_cublaslt_graph_avg_ns > 0
    # eight tokens for less than eight single-token passes over the weights
    assert out.block_cublaslt_graph_avg_ns < 8 * out.custom_graph_avg_ns
