"""GPU parity of the individual operators, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

from nerva_b200 import ops, synth

pytestmark = pytest.mark.gpu

# fp32 accumulation in a different order than the oracle's serial sum: the
# difference is rounding noise of the partial sums.  Bound used for projections
# with |y| = O(1): 2e-3 absolute (the end-to-end logit bound is 2e-2).
PROJ_ATOL = 2e-3
ATTN_ATOL = 2e-3


def _weights(rows, cols, tid=77):
    return ops.synth_normal_bf16(0, tid, rows * cols, 0.02)


def _acts(cols, tokens=1, tid=synth.T_ACTIVATION):
    return ops.synth_normal_bf16(0, tid, tokens * cols, 1.0)


@pytest.mark.parametrize("rows,cols", [
    (768, 512), (512, 512), (3072, 512), (512, 1536), (32000, 512),  # tiny-config shapes
    (6144, 4096), (4096, 12288),                                      # Qwen3-8B QKV and down
    (37, 4096), (1000, 1408), (5, 8), (3, 24576 // 2),                # ragged row counts / odd widths
])
def test_projection_matches_oracle(built_lib, oracle_mod, rows, cols):
    w, x = _weights(rows, cols), _acts(cols)
    y, _ = ops.projection(w, x, rows, cols)
    ref = oracle_mod.matvec(w, synth.bf16_to_f32(x), rows, cols)
    assert np.abs(y[0] - ref).max() <= PROJ_ATOL
    # bit-stable run to run
    y2, _ = ops.projection(w, x, rows, cols)
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("rows,cols", [(24576, 4096), (151936, 4096)])
def test_projection_full_size_row_sample(built_lib, oracle_mod, rows, cols):
    """Full-size gate-up and lm_head shapes: every 97th row against the oracle,
    plus linearity in x (a size-independent property): W(2x) == 2 W(x) exactly."""
    w, x = _weights(rows, cols), _acts(cols)
    y, _ = ops.projection(w, x, rows, cols)
    xf = synth.bf16_to_f32(x)
    sample = np.arange(0, rows, 97)
    ref = oracle_mod.matvec(np.ascontiguousarray(w.reshape(rows, cols)[sample]), xf, sample.size, cols)
    assert np.abs(y[0][sample] - ref).max() <= PROJ_ATOL
    x2 = synth.f32_to_bf16(xf * 2.0)
    y2, _ = ops.projection(w, x2, rows, cols)
    assert np.array_equal(y2, y * 2.0)


def test_projection_multiple_tokens_odd_width(built_lib, oracle_mod):
    """A width that is not a multiple of 64 keeps the token-by-token path."""
    rows, cols, tokens = 1024, 4096 + 8, 4
    w, x = _weights(rows, cols), _acts(cols, tokens)
    y, _ = ops.projection(w, x, rows, cols, tokens=tokens)
    for m in range(tokens):
        ref = oracle_mod.matvec(w, synth.bf16_to_f32(x[m * cols:(m + 1) * cols]), rows, cols)
        assert np.abs(y[m] - ref).max() <= PROJ_ATOL


def _paged_kv(batch, context, kv_heads, head_dim, seed=0, permute=True):
    pages = (context + 15) // 16
    kv_hidden = kv_heads * head_dim
    n = batch * pages * 16 * kv_hidden
    k = ops.synth_normal_bf16(seed, synth.layer_tensor_id(0, synth.L_K), n, 1.0)
    v = ops.synth_normal_bf16(seed, synth.layer_tensor_id(0, synth.L_V), n, 1.0)
    table = np.stack([synth.permutation(seed + b, synth.T_PAGE_TABLE, pages) if permute
                      else np.arange(pages, dtype=np.uint32) for b in range(batch)])
    return k, v, table


@pytest.mark.parametrize("batch,context,heads,kv_heads,head_dim", [
    (1, 1, 32, 8, 128), (1, 17, 32, 8, 128), (1, 769, 32, 8, 128), (2, 2048, 32, 8, 128),
    (1, 8192, 32, 8, 128),
    (1, 97, 8, 2, 64), (3, 333, 8, 2, 64),
    (1, 50, 4, 4, 32), (1, 9, 1, 1, 2), (2, 40, 6, 2, 96),   # generic path: other group sizes / head dims
])
def test_gqa_decode_attention_matches_oracle(built_lib, oracle_mod, batch, context, heads, kv_heads, head_dim):
    k, v, table = _paged_kv(batch, context, kv_heads, head_dim)
    q = synth.normal_f32(0, synth.layer_tensor_id(0, synth.L_Q), batch * heads * head_dim, 1.0)
    out, _ = ops.gqa_decode_attention(q, k, v, table, batch, context, heads, kv_heads, head_dim)
    pages = (context + 15) // 16
    per_seq = pages * 16 * kv_heads * head_dim
    for b in range(batch):
        ref = oracle_mod.attention_paged(q[b * heads * head_dim:(b + 1) * heads * head_dim],
                                         k[b * per_seq:(b + 1) * per_seq], v[b * per_seq:(b + 1) * per_seq],
                                         table[b], context, heads, kv_heads, head_dim)
        assert np.abs(out[b] - ref).max() <= ATTN_ATOL


def test_gqa_attention_invariant_to_page_permutation(built_lib):
    """Any placement of the 16-token pages gives bit-identical output."""
    batch, context, heads, kv_heads, d = 1, 1000, 32, 8, 128
    k, v, table = _paged_kv(batch, context, kv_heads, d, permute=False)
    q = synth.normal_f32(0, synth.layer_tensor_id(0, synth.L_Q), heads * d, 1.0)
    base, _ = ops.gqa_decode_attention(q, k, v, table, batch, context, heads, kv_heads, d)
    pages = table.shape[1]
    perm = synth.permutation(5, synth.T_PAGE_TABLE, pages)
    kp = np.empty_like(k).reshape(pages, -1)
    vp = np.empty_like(v).reshape(pages, -1)
    kp[perm] = k.reshape(pages, -1)
    vp[perm] = v.reshape(pages, -1)
    moved, _ = ops.gqa_decode_attention(q, kp, vp, perm[None, :], batch, context, heads, kv_heads, d)
    assert np.array_equal(base, moved)


def test_gqa_attention_rejects_bad_page_index(built_lib):
    batch, context, heads, kv_heads, d = 1, 64, 32, 8, 128
    k, v, table = _paged_kv(batch, context, kv_heads, d, permute=False)
    table = table.copy()
    table[0, 1] = 1000  # outside the 4 pages: recorded by the kernel, never dereferenced
    q = np.zeros(heads * d, dtype=np.float32)
    with pytest.raises(RuntimeError):
        ops.gqa_decode_attention(q, k, v, table, batch, context, heads, kv_heads, d)


@pytest.mark.parametrize("case", ["plain", "ties", "nonfinite", "all_nonfinite", "negative"])
def test_greedy_argmax_bit_exact(built_lib, oracle_mod, case):
    rng = np.random.default_rng(3)
    logits = rng.standard_normal(151936).astype(np.float32)
    if case == "ties":
        logits[[70000, 5, 140000]] = 9.5
    elif case == "nonfinite":
        logits[11] = np.inf
        logits[12] = np.nan
        logits[13] = -np.inf
    elif case == "all_nonfinite":
        logits[:] = np.nan
    elif case == "negative":
        logits = -np.abs(logits) - 1.0
    assert ops.greedy_argmax(logits) == oracle_mod.argmax(logits, oracle_mod.MODE_CUDA)
    small = logits[:7].copy()
    assert ops.greedy_argmax(small) == oracle_mod.argmax(small, oracle_mod.MODE_CUDA)


def test_projection_bench_entry_point(built_lib):
    rc, out = ops.projection_bench(4096, 4096, iterations=5, warmup=2)
    assert rc == 0 and out.status == 0 and out.mismatch_count == 0
    assert out.custom_avg_ns > 0 and out.custom_graph_avg_ns > 0 and out.hot_path_allocations == 0
    assert out.matrix_bytes == 4096 * 4096 * 2
