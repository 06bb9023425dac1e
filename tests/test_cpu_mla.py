"""The MLA decode oracle against the expanded (per-head K/V) attention formula, on the reference's
own fixture (native/cuda/deepseek/nerva_cuda_deepseek_mla.cu:10-47, checked there against the same
expanded form, :65-90) and on DeepSeek-V2-Lite shapes."""
import numpy as np
import pytest

FIXTURE = dict(
    heads=2, tokens=3, rank=3, nope=2, rope=1, v=2, scale=0.7,
    q_nope=[0.2, -0.3, 0.4, 0.1], q_pe=[0.15, -0.25],
    kv_c=[0.3, -0.1, 0.2, -0.4, 0.5, 0.1, 0.2, 0.4, -0.3], k_pe=[0.05, -0.2, 0.3],
    w_uk=[0.3, -0.2, 0.1, 0.4, -0.5, 0.2, 0.6, -0.1, 0.7, 0.3, -0.2, 0.5],
    w_uv=[0.2, -0.4, 0.5, 0.1, -0.3, 0.6, 0.4, -0.2, 0.7, 0.2, -0.1, 0.3])


def expanded_mha(q_nope, q_pe, kv_c, k_pe, w_uk, w_uv, heads, tokens, rank, nope, rope, v, scale):
    """k_nope[t][h] = kv_c[t] W_UK[:, h], value[t][h] = kv_c[t] W_UV[:, h]; ordinary softmax attention."""
    q_nope = np.asarray(q_nope, np.float64).reshape(heads, nope)
    q_pe = np.asarray(q_pe, np.float64).reshape(heads, rope)
    kv_c = np.asarray(kv_c, np.float64).reshape(tokens, rank)
    k_pe = np.asarray(k_pe, np.float64).reshape(tokens, rope)
    w_uk = np.asarray(w_uk, np.float64).reshape(rank, heads, nope)
    w_uv = np.asarray(w_uv, np.float64).reshape(rank, heads, v)
    out = np.zeros((heads, v))
    for h in range(heads):
        k_nope = kv_c @ w_uk[:, h, :]            # [tokens, nope]
        value = kv_c @ w_uv[:, h, :]             # [tokens, v]
        s = (k_nope @ q_nope[h] + k_pe @ q_pe[h]) * scale
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ value
    return out.reshape(-1)


def test_reference_fixture(oracle_mod):
    f = FIXTURE
    rc, out = oracle_mod.mla_decode(f["q_nope"], f["q_pe"], f["kv_c"], f["k_pe"], f["w_uk"], f["w_uv"], f["heads"],
                                    f["tokens"], f["rank"], f["nope"], f["rope"], f["v"], f["scale"])
    want = expanded_mha(f["q_nope"], f["q_pe"], f["kv_c"], f["k_pe"], f["w_uk"], f["w_uv"], f["heads"], f["tokens"],
                        f["rank"], f["nope"], f["rope"], f["v"], f["scale"])
    assert rc == 0
    assert np.abs(out - want).max() <= 1e-6  # the reference's own smoke tolerance


def mla_case(heads, tokens, rank, nope, rope, v, seed):
    rng = np.random.default_rng(seed)
    return dict(heads=heads, tokens=tokens, rank=rank, nope=nope, rope=rope, v=v, scale=float((nope + rope) ** -0.5),
                q_nope=rng.standard_normal(heads * nope).astype(np.float32),
                q_pe=rng.standard_normal(heads * rope).astype(np.float32),
                kv_c=rng.standard_normal(tokens * rank).astype(np.float32),
                k_pe=rng.standard_normal(tokens * rope).astype(np.float32),
                w_uk=(rng.standard_normal(rank * heads * nope) * 0.05).astype(np.float32),
                w_uv=(rng.standard_normal(rank * heads * v) * 0.05).astype(np.float32))


@pytest.mark.parametrize("shape", [(16, 300, 512, 128, 64, 128), (4, 1, 64, 16, 8, 16), (3, 77, 40, 6, 0, 5)])
def test_absorbed_form_equals_expanded_attention(oracle_mod, shape):
    f = mla_case(*shape, seed=shape[1])
    rc, out = oracle_mod.mla_decode(f["q_nope"], f["q_pe"] if f["rope"] else np.zeros(1, np.float32), f["kv_c"],
                                    f["k_pe"] if f["rope"] else np.zeros(1, np.float32), f["w_uk"], f["w_uv"],
                                    f["heads"], f["tokens"], f["rank"], f["nope"], f["rope"], f["v"], f["scale"])
    want = expanded_mha(f["q_nope"], f["q_pe"], f["kv_c"], f["k_pe"], f["w_uk"], f["w_uv"], f["heads"], f["tokens"],
                        f["rank"], f["nope"], f["rope"], f["v"], f["scale"])
    assert rc == 0
    assert np.abs(out - want).max() <= 2e-5


def test_bad_shapes_are_rejected(oracle_mod):
    z = np.zeros(4, np.float32)
    assert oracle_mod.mla_decode(z, z, z, z, z, z, 0, 1, 1, 1, 1, 1, 1.0)[0] == -1
    assert oracle_mod.mla_decode(z, z, z, z, z, z, 1, 1, 2048, 1, 1, 1, 1.0)[0] == -1
