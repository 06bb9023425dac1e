"""The fp32 expert-MLP oracle against the formula in float64 (per-operator interface of
native/cuda/deepseek/nerva_cuda_deepseek_moe.cu:456-510)."""
import numpy as np
import pytest


def moe_case(hidden, intermediate, experts, top_k, seed):
    rng = np.random.default_rng(seed)
    return dict(hidden=hidden, intermediate=intermediate, experts=experts,
                x=rng.standard_normal(hidden).astype(np.float32),
                ids=rng.choice(experts, size=top_k, replace=False).astype(np.uint32),
                weights=rng.uniform(0.05, 0.6, size=top_k).astype(np.float32),
                w_gate=(rng.standard_normal((experts, intermediate, hidden)) * 0.1).astype(np.float32),
                w_up=(rng.standard_normal((experts, intermediate, hidden)) * 0.1).astype(np.float32),
                w_down=(rng.standard_normal((experts, hidden, intermediate)) * 0.1).astype(np.float32))


def formula(c, clamp=False, limit=0.0):
    x = c["x"].astype(np.float64)
    out = np.zeros(c["hidden"])
    for e, w in zip(c["ids"], c["weights"]):
        gate = c["w_gate"][e].astype(np.float64) @ x
        up = c["w_up"][e].astype(np.float64) @ x
        if clamp:
            gate = np.minimum(gate, limit)
            up = np.clip(up, -limit, limit)
        act = gate / (1.0 + np.exp(-gate)) * up
        out += float(w) * (c["w_down"][e].astype(np.float64) @ act)
    return out


@pytest.mark.parametrize("clamp", [False, True])
def test_expert_mlp_matches_formula(oracle_mod, clamp):
    c = moe_case(96, 40, 6, 3, seed=4)
    rc, out = oracle_mod.moe_forward(c["x"], c["ids"], c["weights"], c["w_gate"], c["w_up"], c["w_down"], c["hidden"],
                                     c["intermediate"], c["experts"], clamp_swiglu=clamp, swiglu_limit=0.5)
    assert rc == 0
    assert np.abs(out - formula(c, clamp, 0.5)).max() <= 1e-5


def test_expert_id_out_of_range(oracle_mod):
    c = moe_case(16, 8, 4, 2, seed=1)
    rc, _ = oracle_mod.moe_forward(c["x"], [1, 4], c["weights"], c["w_gate"], c["w_up"], c["w_down"], 16, 8, 4)
    assert rc == -2
