"""The oracle's composed DeepSeek-V2-Lite-architecture decoder (latent attention in absorbed form +
softmax top-k MoE with always-on shared experts, one dense first layer) against an independent numpy
restatement in float64 that uses the EXPANDED attention formula of the DeepSeek-V2 paper: per-head
keys and values decompressed from the cached latent rows (k_nope = W_UK c, v = W_UV c), ordinary
softmax attention over them.  The restatement rounds to bf16 at the points of the CUDA numeric
contract (normalised hidden state into dense mat-vecs, cache rows, attention output, dense SwiGLU
output) and nowhere else, like the oracle (oracle/nerva_oracle.c: layer_forward, mla_attention,
sparse_moe_mlp)."""
import dataclasses

import numpy as np

from nerva_b200 import synth


def _cfg():
    return dataclasses.replace(synth.DEEPSEEK_V2_LITE, name="v2-lite-toy", layers=3, vocab=640, prompt_tokens=9,
                               decode_tokens=4, hidden=192, heads=4, kv_heads=4, head_dim=32, intermediate=320,
                               num_experts=8, top_k=3, moe_intermediate=48, shared_intermediate=96, dense_layers=1,
                               kv_lora_rank=64, qk_nope_head_dim=24, qk_rope_head_dim=16)


def _bf16(x):
    return synth.bf16_to_f32(synth.f32_to_bf16(np.asarray(x, np.float32))).astype(np.float64)


def _w(bits, *shape):
    return synth.bf16_to_f32(bits).astype(np.float64).reshape(*shape)


def _rms_norm(x, weight_bits, eps):
    return x / np.sqrt((x * x).mean() + eps) * _w(weight_bits, -1)


def _rope_interleaved(v, position, theta):
    out = v.copy()
    dim = v.shape[-1]
    for pair in range(dim // 2):
        angle = position * theta ** (-(2.0 * pair) / dim)
        c, s = np.cos(angle), np.sin(angle)
        left, right = v[..., 2 * pair], v[..., 2 * pair + 1]
        out[..., 2 * pair] = left * c - right * s
        out[..., 2 * pair + 1] = right * c + left * s
    return out


def _silu(x):
    return x / (1.0 + np.exp(-x))


def _expanded_latent_attention(cfg, layer, a, cache, position):
    """a: the bf16-rounded normalised hidden state.  Appends this token's cache row, returns heads * v."""
    rank, nope, rope, v = cfg.kv_lora_rank, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.head_dim
    q = _w(layer["w_q"], cfg.heads, nope + rope, cfg.hidden) @ a
    kv = _w(layer["w_kv_a"], rank + rope, cfg.hidden) @ a
    latent = _bf16(_rms_norm(kv[:rank], layer["kv_a_norm"], cfg.rms_eps))
    k_pe = _bf16(_rope_interleaved(_bf16(kv[rank:]), position, cfg.rope_theta))
    cache.append((latent, k_pe))
    w_kv_b = _w(layer["w_kv_b"], cfg.heads, nope + v, rank)
    q_pe = _rope_interleaved(q[:, nope:], position, cfg.rope_theta)
    out = np.zeros((cfg.heads, v))
    for h in range(cfg.heads):
        w_uk, w_uv = w_kv_b[h, :nope], w_kv_b[h, nope:]
        keys = np.stack([w_uk @ c for c, _ in cache])     # [tokens, nope]
        values = np.stack([w_uv @ c for c, _ in cache])   # [tokens, v]
        rotary = np.stack([r for _, r in cache])          # [tokens, rope]
        s = (keys @ q[h, :nope] + rotary @ q_pe[h]) / np.sqrt(nope + rope)
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ values
    return out.reshape(-1)


def _moe(cfg, layer, m):
    """m: the unrounded normalised hidden state (the reference's MoE kernel does not round it)."""
    e, mi, hidden = cfg.num_experts, cfg.moe_intermediate, cfg.hidden
    logits = _w(layer["w_router"], e, hidden) @ m
    weights = np.exp(logits - logits.max())
    weights /= weights.sum()
    order = sorted(range(e), key=lambda i: (-weights[i], i))[:cfg.top_k]
    chosen = weights[order] / (weights[order].sum() if cfg.norm_topk_prob else 1.0)
    gate_up = _w(layer["w_expert_gate_up"], e, 2, mi, hidden)
    down_w = _w(layer["w_expert_down"], e, hidden, mi)
    down = np.zeros(hidden)
    for weight, i in zip(chosen, order):
        down += weight * (down_w[i] @ (_silu(gate_up[i, 0] @ m) * (gate_up[i, 1] @ m)))
    si = cfg.shared_intermediate
    shared = _silu(_w(layer["w_shared_expert_gate"], si, hidden) @ m) * (_w(layer["w_shared_expert_up"], si, hidden) @ m)
    return down + _w(layer["w_shared_expert_down"], hidden, si) @ shared, order


def _decode(cfg, ck, tokens):
    """Logits after every token of `tokens`, and the experts every sparse layer chose."""
    caches = [[] for _ in range(cfg.layers)]
    embeddings = _w(ck.embeddings, cfg.vocab, cfg.hidden)
    lm_head = _w(ck.lm_head, cfg.vocab, cfg.hidden)
    all_logits, routes = [], []
    for position, token in enumerate(tokens):
        x = embeddings[token]
        for l, layer in enumerate(ck.layers):
            a = _bf16(_rms_norm(x, layer["rms_attn"], cfg.rms_eps))
            attn = _bf16(_expanded_latent_attention(cfg, layer, a, caches[l], position))
            r = _w(layer["w_o"], cfg.hidden, cfg.heads * cfg.head_dim) @ attn + x
            m = _rms_norm(r, layer["rms_mlp"], cfg.rms_eps)
            if "w_router" in layer:
                down, order = _moe(cfg, layer, m)
                routes.append(order)
            else:
                mb = _bf16(m)
                ff = _bf16(_silu(_w(layer["w_gate"], cfg.intermediate, cfg.hidden) @ mb) *
                           (_w(layer["w_up"], cfg.intermediate, cfg.hidden) @ mb))
                down = _w(layer["w_down"], cfg.hidden, cfg.intermediate) @ ff
            x = r + down
        all_logits.append(lm_head @ _bf16(_rms_norm(x, ck.final_norm, cfg.rms_eps)))
    return np.stack(all_logits), routes


def test_composed_oracle_equals_the_expanded_formulas(oracle_mod):
    cfg = _cfg()
    ck = synth.dense_checkpoint(cfg, std=0.08)  # large enough weights for attention and routing to matter
    tokens = [int(t) for t in synth.prompt_ids(cfg)]
    dec = oracle_mod.Decoder(ck, len(tokens) + 1, mode=oracle_mod.MODE_CUDA)
    got = []
    for token in tokens:
        got.append(np.array(dec.step(token, want_logits=True), np.float64))
    got = np.stack(got)
    want, routes = _decode(cfg, ck, tokens)
    # two sparse layers per token, top_k distinct experts each, and not always the same ones
    assert len(routes) == 2 * len(tokens) and all(len(set(r)) == cfg.top_k for r in routes)
    assert len({tuple(r) for r in routes}) > 1
    # attention has something to weigh: the logits of the last position depend on the earlier tokens
    alone, _ = _decode(cfg, ck, tokens[-1:])
    assert np.abs(alone[0] - want[-1]).max() > 1e-2
    # fp32 serial sums against float64, with a handful of bf16 roundings that may fall the other way
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-3 * scale, (np.abs(got - want).max(), scale)
    assert (got.argmax(axis=1) == want.argmax(axis=1)).all()
