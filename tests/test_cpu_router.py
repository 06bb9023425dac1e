"""The router oracle against the reference's known answers and against the reference's own
router header compiled for the host (oracle/_ref, built where the reference checkout exists)."""
import numpy as np
import pytest

V3 = dict(logits=[-2.0, 0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -3.0], bias=[0.0, 0.0, 0.0, 4.0, 0.0, 0.0, -4.0, 0.0])
V4 = dict(logits=[-2.0, 0.0, 1.0, 3.0], bias=[0.0, 3.0, 0.0, -3.0])
HASH = dict(logits=[4.0, -1.0, 0.0, 2.0], table=[0, 1, 3, 2, 1, 3, 3, 0, 2])


def _sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def _sqrt_softplus(v):
    return np.sqrt(np.log1p(np.exp(v)))


# crates/nerva-cuda/src/tests/deepseek_router.rs:84-127 and
# native/cuda/deepseek/nerva_cuda_deepseek_router.cu:20-31
@pytest.mark.parametrize("ref", [False, True])
def test_reference_known_answers(oracle_mod, ref):
    if ref and oracle_mod.ref_router_lib() is None:
        pytest.skip("the reference's router header has not been compiled here")
    rc, ids, w = oracle_mod.route_v3_grouped_sigmoid(V3["logits"], V3["bias"], 2, 1, 2, True, 2.5, ref=ref)
    assert rc == 0 and ids.tolist() == [3, 2]
    s = _sigmoid(-1.0) + _sigmoid(1.0)
    assert np.allclose(w, [_sigmoid(-1.0) * 2.5 / s, _sigmoid(1.0) * 2.5 / s], atol=1e-6)
    rc, ids, w = oracle_mod.route_v4_sqrtsoftplus(V4["logits"], V4["bias"], 2, True, 1.5, ref=ref)
    assert rc == 0 and ids.tolist() == [1, 2]
    w1, w2 = _sqrt_softplus(0.0), _sqrt_softplus(1.0)
    assert np.allclose(w, [w1 * 1.5 / (w1 + w2), w2 * 1.5 / (w1 + w2)], atol=1e-6)
    rc, ids, w = oracle_mod.route_v4_hash(HASH["logits"], HASH["table"], 1, 3, True, 1.0, ref=ref)
    assert rc == 0 and ids.tolist() == [2, 1, 3]
    e = np.array([_sqrt_softplus(0.0), _sqrt_softplus(-1.0), _sqrt_softplus(2.0)])
    assert np.allclose(w, e / e.sum(), atol=1e-6)


def _random_cases(count=200):
    rng = np.random.default_rng(11)
    for i in range(count):
        groups = int(rng.choice([1, 2, 4, 8]))
        per_group = int(rng.integers(1, 33))
        experts = groups * per_group
        top_k = int(rng.integers(1, min(16, experts) + 1))
        top_groups = int(rng.integers(1, groups + 1))
        logits = rng.standard_normal(experts).astype(np.float32) * 3.0
        if i % 7 == 0:
            logits[rng.integers(0, experts, size=max(1, experts // 4))] = 0.25   # exact ties
        if i % 11 == 0:
            logits[int(rng.integers(0, experts))] = -np.inf
        if i % 13 == 0:
            logits[int(rng.integers(0, experts))] = 30.0                          # softplus linear branch
        bias = None if i % 3 == 0 else (rng.standard_normal(experts).astype(np.float32) * 0.5)
        yield logits, bias, groups, top_groups, top_k, bool(i % 2), float(rng.uniform(0.5, 3.0))


def test_restatement_is_bit_identical_to_the_reference_header(oracle_mod):
    """Same libm, same order of operations: ids and weight bits must be equal, ties, -inf
    and the large-argument branch included."""
    if oracle_mod.ref_router_lib() is None:
        pytest.skip("the reference's router header has not been compiled here")
    for logits, bias, groups, top_groups, top_k, norm, scaling in _random_cases():
        a = oracle_mod.route_v3_grouped_sigmoid(logits, bias, groups, top_groups, top_k, norm, scaling)
        b = oracle_mod.route_v3_grouped_sigmoid(logits, bias, groups, top_groups, top_k, norm, scaling, ref=True)
        assert a[0] == b[0] and np.array_equal(a[1], b[1]) and np.array_equal(a[2].view(np.uint32), b[2].view(np.uint32))
        a = oracle_mod.route_v4_sqrtsoftplus(logits, bias, top_k, norm, scaling)
        b = oracle_mod.route_v4_sqrtsoftplus(logits, bias, top_k, norm, scaling, ref=True)
        assert a[0] == b[0] and np.array_equal(a[1], b[1]) and np.array_equal(a[2].view(np.uint32), b[2].view(np.uint32))


def test_invalid_routes_are_rejected(oracle_mod):
    logits = np.zeros(8, dtype=np.float32)
    assert oracle_mod.route_v4_sqrtsoftplus(logits, None, 17, True, 1.0)[0] == -1       # more than 16 ranks
    assert oracle_mod.route_v4_sqrtsoftplus(logits[:2], None, 3, True, 1.0)[0] == -1    # top_k > experts
    assert oracle_mod.route_v3_grouped_sigmoid(logits, None, 3, 1, 2, True, 1.0)[0] == -1  # 8 % 3 != 0
    assert oracle_mod.route_v3_grouped_sigmoid(logits, None, 2, 3, 2, True, 1.0)[0] == -1  # more groups than exist
    assert oracle_mod.route_v4_hash(logits, [0, 1, 2], 1, 2, True, 1.0)[0] == -2         # table too short
    assert oracle_mod.route_v4_hash(logits, [0, 9], 0, 2, True, 1.0)[0] == -3            # expert id out of range
