"""The CPU oracle against the reference's own known answers and the committed golden vectors.

These run without a GPU.  They pin the checker that the GPU parity tests trust.
"""
import numpy as np
import pytest

from nerva_b200 import synth


# ---- codecs (crates/nerva-model/src/tests/precision.rs:19-32) ----

def test_f16_and_bf16_conversions_round_known_values(oracle_mod):
    L = oracle_mod.lib()
    assert L.oracle_f32_to_f16(1.0) == 0x3c00
    assert L.oracle_f32_to_f16(-2.0) == 0xc000
    assert L.oracle_f32_to_f16(0.5) == 0x3800
    assert L.oracle_f32_to_f16(65504.0) == 0x7bff
    assert L.oracle_f16_to_f32(0x3c00) == 1.0
    assert L.oracle_f16_to_f32(0xc000) == -2.0
    assert L.oracle_f32_to_bf16(1.0) == 0x3f80
    assert L.oracle_f32_to_bf16(-2.0) == 0xc000
    assert L.oracle_f32_to_bf16(0.5) == 0x3f00
    assert L.oracle_bf16_to_f32(0x3f80) == 1.0
    assert L.oracle_bf16_to_f32(0xc000) == -2.0


def test_bf16_round_to_nearest_even_matches_numpy_twin(oracle_mod):
    L = oracle_mod.lib()
    rng = np.random.default_rng(7)
    bits = rng.integers(0, 2**32, size=4096, dtype=np.uint64).astype(np.uint32)
    # ties exactly between two bf16 values, both parities, and values next to them
    bits[:6] = [0x3f808000, 0x3f818000, 0x3f807fff, 0x3f808001, 0x7f7fffff, 0x00008000]
    values = bits.view(np.float32)
    finite = np.isfinite(values)
    twin = synth.f32_to_bf16(values)
    for v, t, ok in zip(values, twin, finite):
        if ok:
            assert L.oracle_f32_to_bf16(float(v)) == int(t)
    assert int(twin[0]) == 0x3f80 and int(twin[1]) == 0x3f82  # ties go to the even mantissa
    back = synth.bf16_to_f32(twin[finite])
    for b, f in zip(twin[finite][:256], back[:256]):
        assert L.oracle_bf16_to_f32(int(b)) == float(f)


# ---- the token-cycle known-answer test (crates/nerva-cuda/src/tests/decode_sequence.rs:123-200,
# decode_sequence_qk_norm.rs:12-91): embeddings and lm_head chosen so that token t -> t+1 mod 4 ----

class _Checkpoint:
    pass


def _token_cycle_checkpoint(qk_norm: bool):
    one, zero, neg = 0x3c00, 0, 0xbc00  # f16
    cfg = synth.DecoderConfig("kat", layers=1, hidden=2, heads=1, kv_heads=1, head_dim=2, intermediate=2, vocab=4,
                              rms_eps=1e-5, rope_theta=0.0, qk_norm=qk_norm)
    ck = _Checkpoint()
    ck.config = cfg
    ck.embeddings = np.array([one, zero, zero, one, neg, zero, zero, neg], dtype=np.uint16)
    ck.final_norm = np.array([one, one], dtype=np.uint16)
    ck.lm_head = np.array([zero, neg, one, zero, zero, one, neg, zero], dtype=np.uint16)
    m = np.zeros(4, dtype=np.uint16)
    rms = np.array([one, one], dtype=np.uint16)
    layer = dict(rms_attn=rms, rms_mlp=rms, w_q=m, w_k=m, w_v=m, w_o=m, w_gate=m, w_up=m, w_down=m)
    if qk_norm:
        layer.update(q_norm=rms, k_norm=rms)
    ck.layers = [layer]
    return ck


@pytest.mark.parametrize("qk_norm", [False, True])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_token_cycle_known_answer(oracle_mod, qk_norm, mode):
    ck = _token_cycle_checkpoint(qk_norm)
    dec = oracle_mod.Decoder(ck, 16, mode=mode, dtype=oracle_mod.DTYPE_F16)
    assert dec.decode_greedy([0], 4).tolist() == [1, 2, 3, 0]
    dec.reset()
    assert dec.decode_greedy([2, 3], 3).tolist() == [0, 1, 2]


# ---- attention against the dense formula (crates/nerva-model/src/tests/attention.rs,
# tests/support.rs:99-142) ----

def _dense_attention(q, k, v, heads, kv_heads, d):
    out = np.zeros(heads * d, dtype=np.float64)
    group = heads // kv_heads
    for h in range(heads):
        kv = h // group
        qh = q[h * d:(h + 1) * d].astype(np.float64)
        kh = k[:, kv * d:(kv + 1) * d].astype(np.float64)
        vh = v[:, kv * d:(kv + 1) * d].astype(np.float64)
        s = kh @ qh / np.sqrt(d)
        p = np.exp(s - s.max())
        out[h * d:(h + 1) * d] = (p / p.sum()) @ vh
    return out


@pytest.mark.parametrize("tokens,heads,kv_heads,d", [(1, 4, 2, 8), (37, 8, 2, 64), (300, 32, 8, 128), (5, 3, 3, 6)])
def test_attention_matches_dense_softmax(oracle_mod, tokens, heads, kv_heads, d):
    rng = np.random.default_rng(tokens)
    q = rng.standard_normal(heads * d).astype(np.float32)
    k = rng.standard_normal((tokens, kv_heads * d)).astype(np.float32)
    v = rng.standard_normal((tokens, kv_heads * d)).astype(np.float32)
    got = oracle_mod.attention(q, k, v, tokens, heads, kv_heads, d)
    assert np.abs(got - _dense_attention(q, k, v, heads, kv_heads, d)).max() < 1e-5


def test_paged_attention_equals_contiguous_attention_under_any_page_placement(oracle_mod):
    tokens, heads, kv_heads, d = 75, 8, 2, 64
    pages = (tokens + 15) // 16
    kvh = kv_heads * d
    k_bits = synth.normal_bf16(3, 11, pages * 16 * kvh, 1.0)
    v_bits = synth.normal_bf16(3, 12, pages * 16 * kvh, 1.0)
    q = synth.normal_f32(3, 13, heads * d, 1.0)
    identity = np.arange(pages, dtype=np.uint32)
    base = oracle_mod.attention_paged(q, k_bits, v_bits, identity, tokens, heads, kv_heads, d)
    dense = oracle_mod.attention(q, synth.bf16_to_f32(k_bits).reshape(-1, kvh)[:tokens],
                                 synth.bf16_to_f32(v_bits).reshape(-1, kvh)[:tokens], tokens, heads, kv_heads, d)
    assert np.array_equal(base, dense)
    perm = synth.permutation(9, synth.T_PAGE_TABLE, pages)
    kp = np.empty_like(k_bits).reshape(pages, -1)
    vp = np.empty_like(v_bits).reshape(pages, -1)
    kp[perm] = k_bits.reshape(pages, -1)
    vp[perm] = v_bits.reshape(pages, -1)
    moved = oracle_mod.attention_paged(q, kp.reshape(-1), vp.reshape(-1), perm, tokens, heads, kv_heads, d)
    assert np.array_equal(base, moved)


# ---- RoPE (crates/nerva-model/src/common/rope.rs:54-79): pairs (i, i + d/2), angle pos / theta^(2i/d) ----

def test_rope_rotates_half_split_pairs(oracle_mod):
    heads, d, pos, theta = 2, 8, 5, 10000.0
    x = np.arange(1, heads * d + 1, dtype=np.float32)
    got = oracle_mod.rope(x, heads, d, pos, theta)
    want = x.astype(np.float64).copy()
    for h in range(heads):
        for i in range(d // 2):
            ang = pos / theta ** (2 * i / d)
            a, b = x[h * d + i], x[h * d + i + d // 2]
            want[h * d + i] = a * np.cos(ang) - b * np.sin(ang)
            want[h * d + i + d // 2] = a * np.sin(ang) + b * np.cos(ang)
    assert np.abs(got - want).max() < 1e-4
    assert np.array_equal(oracle_mod.rope(x, heads, d, 0, theta), x)  # position 0 is the identity


# ---- greedy arg-max (common/token.rs:33-58 for the CPU rule; sampler.cu:35-40,89-119 for CUDA) ----

def test_argmax_first_maximum_wins(oracle_mod):
    logits = np.array([0.5, 3.0, -1.0, 3.0, 2.0], dtype=np.float32)
    assert oracle_mod.argmax(logits, oracle_mod.MODE_CPU) == 1
    assert oracle_mod.argmax(logits, oracle_mod.MODE_CUDA) == 1


def test_argmax_non_finite_rules(oracle_mod):
    logits = np.array([0.5, np.nan, np.inf, 2.0, -np.inf], dtype=np.float32)
    assert oracle_mod.argmax(logits, oracle_mod.MODE_CPU) < 0        # the CPU decoder reports an error
    assert oracle_mod.argmax(logits, oracle_mod.MODE_CUDA) == 3      # the CUDA sampler skips non-finite values
    all_bad = np.full(4, np.nan, dtype=np.float32)
    assert oracle_mod.argmax(all_bad, oracle_mod.MODE_CUDA) == 0     # nothing finite: token 0


# ---- softmax top-k routing (precision/block/moe.rs:1303-1326): weight descending, index ascending ----

def test_softmax_topk_route_order_ties_and_renormalisation(oracle_mod):
    logits = np.array([1.0, 3.0, 3.0, -2.0, 0.5, 3.0], dtype=np.float32)
    ids, w = oracle_mod.route_softmax_topk(logits, 4, norm_topk_prob=False)
    assert ids.tolist() == [1, 2, 5, 0]
    p = np.exp(logits.astype(np.float64) - 3.0)
    p /= p.sum()
    assert np.allclose(w, p[[1, 2, 5, 0]], atol=1e-6)
    ids_n, w_n = oracle_mod.route_softmax_topk(logits, 4, norm_topk_prob=True)
    assert ids_n.tolist() == [1, 2, 5, 0]
    assert abs(float(w_n.sum()) - 1.0) < 1e-6
    assert np.allclose(w_n, p[[1, 2, 5, 0]] / p[[1, 2, 5, 0]].sum(), atol=1e-6)


# ---- mat-vec and norms against numpy ----

def test_matvec_is_the_serial_fp32_row_sum(oracle_mod):
    rows, cols = 9, 40
    w = synth.normal_bf16(0, 77, rows * cols, 0.02)
    x = synth.normal_f32(0, 78, cols, 1.0)
    got = oracle_mod.matvec(w, x, rows, cols)
    wf = synth.bf16_to_f32(w).reshape(rows, cols)
    want = np.zeros(rows, dtype=np.float32)
    for r in range(rows):
        acc = np.float32(0.0)
        for c in range(cols):
            acc = np.float32(acc + np.float32(wf[r, c] * x[c]))
        want[r] = acc
    assert np.array_equal(got, want)


def test_rms_norm_matches_formula(oracle_mod):
    n, eps = 64, 1e-6
    x = synth.normal_f32(0, 5, n, 1.0)
    w = synth.f32_to_bf16(np.linspace(0.5, 1.5, n).astype(np.float32))
    got = oracle_mod.rms_norm(x, w, eps)
    xd = x.astype(np.float64)
    want = xd / np.sqrt((xd * xd).mean() + eps) * synth.bf16_to_f32(w)
    assert np.abs(got - want).max() < 1e-5


# ---- the tiny Qwen3-architecture configuration against the committed golden file ----

@pytest.mark.parametrize("name,mode", [("cpu", 0), ("cuda", 1)])
def test_tiny_decoder_reproduces_golden_tokens_and_logits(oracle_mod, tiny_golden, name, mode):
    cfg = synth.TINY_QWEN3
    ck = synth.dense_checkpoint(cfg)
    prompt = synth.prompt_ids(cfg)
    assert prompt.tolist() == tiny_golden["prompt"]
    dec = oracle_mod.Decoder(ck, cfg.prompt_tokens + cfg.decode_tokens, mode=mode)
    tokens, logits = dec.decode_greedy(prompt, cfg.decode_tokens, want_logits=True)
    gold = tiny_golden[name]
    assert tokens.tolist() == gold["tokens"]
    assert oracle_mod.hash_tokens(tokens) == gold["token_hash"]
    samples = logits[:, tiny_golden["sample_indices"]]
    assert np.array_equal(samples, np.array(gold["logit_samples"], dtype=np.float32))
    assert np.array_equal(logits.max(axis=1), np.array(gold["max_logit"], dtype=np.float32))


def test_summation_order_probe_changes_logits_only_slightly_on_tiny(oracle_mod):
    """The floor the GPU logit tests add to their tolerance: the oracle against itself
    with another fp32 summation order stays inside the stated 2e-2 on the tiny model."""
    cfg = synth.TINY_QWEN3
    ck = synth.dense_checkpoint(cfg)
    prompt = synth.prompt_ids(cfg)[:8]
    dec = oracle_mod.Decoder(ck, 16, mode=oracle_mod.MODE_CUDA)
    _, ref = dec.decode_greedy(prompt, 2, want_logits=True)
    oracle_mod.set_sum_lanes(8)
    try:
        dec2 = oracle_mod.Decoder(ck, 16, mode=oracle_mod.MODE_CUDA)
        _, alt = dec2.decode_greedy(prompt, 2, want_logits=True)
    finally:
        oracle_mod.set_sum_lanes(1)
    d = float(np.abs(alt - ref).max())
    assert 0.0 < d < 2e-2


# ---- the full-size fixture: its cheapest row is regenerated here ----

def test_one_layer_cut_of_the_full_size_fixture_is_reproduced(oracle_mod):
    """tests/golden/qwen3_8b.json takes an hour to make; its depth-1 row (one Qwen3-8B layer between
    the full embedding table and lm_head, 16-token prompt) takes seconds, so it is recomputed and
    compared bit for bit, under both summation orders: the committed file and this oracle agree."""
    import dataclasses
    import json
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", "qwen3_8b.json")
    with open(path) as f:
        sweep = json.load(f)["depth_sweep"]
    assert sweep["depths"][0] == 1
    cfg = dataclasses.replace(synth.QWEN3_8B, layers=1, name="qwen3-8b cut to 1")
    ck = synth.dense_checkpoint(cfg, fill=oracle_mod.synth_normal_bf16)
    prompt = synth.prompt_ids(synth.QWEN3_8B, count=sweep["prompt_tokens"])
    idx = sweep["sample_indices"]
    try:
        for lanes, key in ((1, "serial_samples"), (8, "lanes8_samples")):
            oracle_mod.set_sum_lanes(lanes)
            dec = oracle_mod.Decoder(ck, sweep["prompt_tokens"], mode=oracle_mod.MODE_CUDA)
            for token in prompt[:-1]:
                dec.step(int(token), want_logits=False)
            logits = dec.step(int(prompt[-1]), want_logits=True)
            dec.close()
            assert np.array_equal(logits[idx], np.array(sweep[key][0], dtype=np.float32))
            if lanes == 1:
                assert int(np.argmax(logits)) == sweep["serial_argmax"][0]
    finally:
        oracle_mod.set_sum_lanes(1)
