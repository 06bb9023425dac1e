"""The allocation-free attention entry point against the allocating one and the CPU oracle, through the C ABI.

Collected last on purpose (the file name sorts after the other test files): the
entry point keeps its split partials in one device array that every call shares,
so it has to give the right answer both in a fresh process and after everything
else has used the device.
"""
import numpy as np
import pytest

from nerva_b200 import ops, synth

pytestmark = pytest.mark.gpu

ATTN_ATOL = 2e-3  # the operator tests' bound for attention


def _inputs(batch, context, heads, kv_heads, head_dim, seed):
    pages = (context + 15) // 16
    n = batch * pages * 16 * kv_heads * head_dim
    k = ops.synth_normal_bf16(seed, synth.layer_tensor_id(0, synth.L_K), n, 1.0)
    v = ops.synth_normal_bf16(seed, synth.layer_tensor_id(0, synth.L_V), n, 1.0)
    table = np.stack([synth.permutation(seed + b, synth.T_PAGE_TABLE, pages) for b in range(batch)])
    q = synth.normal_f32(seed, synth.layer_tensor_id(0, synth.L_Q), batch * heads * head_dim, 1.0)
    return q, k, v, table


def _static_scratch(q, k, v, table, batch, context, heads, kv_heads, head_dim):
    import torch
    dev = torch.device("cuda:0")
    d_q = torch.from_numpy(q).to(dev)
    d_k = torch.from_numpy(k.view(np.int16)).to(dev)
    d_v = torch.from_numpy(v.view(np.int16)).to(dev)
    d_t = torch.from_numpy(np.ascontiguousarray(table).view(np.int32)).to(dev)
    d_out = torch.full((batch, heads * head_dim), float("nan"), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    ops.gqa_decode_attention_static_scratch(d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_t.data_ptr(),
                                            d_out.data_ptr(), batch, context, heads, kv_heads, head_dim,
                                            stream=0)
    return d_out.cpu().numpy()


# Two calls in a row: the second runs over whatever the first left in the shared
# array, with another shape, so slots of the first call are reused at other offsets.
CASES = [(2, 2048, 32, 8, 128), (1, 769, 8, 2, 64)]


def _oracle(oracle_mod, q, k, v, table, batch, context, heads, kv_heads, head_dim):
    pages = (context + 15) // 16
    seq = pages * 16 * kv_heads * head_dim
    rows = [oracle_mod.attention_paged(q[b * heads * head_dim:(b + 1) * heads * head_dim], k[b * seq:(b + 1) * seq],
                                       v[b * seq:(b + 1) * seq], table[b], context, heads, kv_heads, head_dim)
            for b in range(batch)]
    return np.stack(rows)


def test_static_scratch_attention_matches_allocating_entry_point(built_lib, oracle_mod):
    for seed, (batch, context, heads, kv_heads, head_dim) in enumerate(CASES):
        q, k, v, table = _inputs(batch, context, heads, kv_heads, head_dim, seed)
        got = _static_scratch(q, k, v, table, batch, context, heads, kv_heads, head_dim)
        want, _ = ops.gqa_decode_attention(q, k, v, table, batch, context, heads, kv_heads, head_dim)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= ATTN_ATOL
        assert np.abs(got - _oracle(oracle_mod, q, k, v, table, batch, context, heads, kv_heads, head_dim)).max() \
            <= ATTN_ATOL


def test_static_scratch_attention_lowers_the_split_count_to_fit(built_lib, oracle_mod):
    """64 query heads of 256 dims on one KV head: the split count the launcher would pick (64) needs
    more than the fixed array holds (63 splits of 64 x 258 floats), so the entry point lowers it;
    the result must not change."""
    batch, context, heads, kv_heads, head_dim = 1, 8200, 64, 1, 256
    q, k, v, table = _inputs(batch, context, heads, kv_heads, head_dim, 7)
    got = _static_scratch(q, k, v, table, batch, context, heads, kv_heads, head_dim)
    want = _oracle(oracle_mod, q, k, v, table, batch, context, heads, kv_heads, head_dim)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= ATTN_ATOL


def test_static_scratch_attention_rejects_misaligned_views(built_lib):
    import torch
    # a K view that starts 2 bytes into a 16-byte piece: refused on the host, nothing is launched
    buf = torch.zeros(1 << 16, dtype=torch.int16, device="cuda:0")
    q = torch.zeros(8 * 64, dtype=torch.float32, device="cuda:0")
    table = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    out = torch.zeros(8 * 64, dtype=torch.float32, device="cuda:0")
    with pytest.raises(RuntimeError, match="misaligned buffer"):
        ops.gqa_decode_attention_static_scratch(q.data_ptr(), buf.data_ptr() + 2, buf.data_ptr(), table.data_ptr(),
                                                out.data_ptr(), 1, 48, 8, 2, 64)


def test_static_scratch_attention_repeats_bit_exactly(built_lib):
    batch, context, heads, kv_heads, head_dim = CASES[0]
    q, k, v, table = _inputs(batch, context, heads, kv_heads, head_dim, 3)
    first = _static_scratch(q, k, v, table, batch, context, heads, kv_heads, head_dim)
    second = _static_scratch(q, k, v, table, batch, context, heads, kv_heads, head_dim)
    assert np.array_equal(first, second)


def test_static_scratch_attention_rejects_oversize(built_lib):
    import torch
    # 64 * 128 * (128 + 2) floats of partials do not fit the 1 Mi-float array even unsplit;
    # the call returns before it touches any buffer.
    dummy = torch.zeros(64, dtype=torch.float32, device="cuda:0")
    with pytest.raises(RuntimeError, match="static scratch too small"):
        ops.gqa_decode_attention_static_scratch(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                                dummy.data_ptr(), dummy.data_ptr(), 64, 16, 128, 8, 128)
