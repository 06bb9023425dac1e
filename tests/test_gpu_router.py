"""nerva_cuda_deepseek_router_route on the GPU against the CPU oracle: expert ids bit-exact, weights
within 1e-6 (device and host libm may differ in the last place)."""
import numpy as np
import pytest

from nerva_b200 import ops
from tests.test_cpu_router import HASH, V3, V4, _random_cases

pytestmark = pytest.mark.gpu


def test_router_known_answers(built_lib):
    rc, ids, w, out = ops.deepseek_router_route(ops.ROUTER_V3_GROUPED_SIGMOID, V3["logits"], 2, bias=V3["bias"],
                                                num_groups=2, top_k_groups=1, routed_scaling_factor=2.5)
    assert rc == 0 and out.status == 0 and ids.tolist() == [3, 2]
    assert (out.kernel_launches, out.sync_calls, out.hot_path_allocations) == (1, 1, 0) and out.output_hash != 0
    rc, ids, w, out = ops.deepseek_router_route(ops.ROUTER_V4_SQRTSOFTPLUS, V4["logits"], 2, bias=V4["bias"],
                                                routed_scaling_factor=1.5)
    assert rc == 0 and ids.tolist() == [1, 2]
    rc, ids, w, out = ops.deepseek_router_route(ops.ROUTER_V4_HASH, HASH["logits"], 3, hash_route_table=HASH["table"],
                                                route_token=1)
    assert rc == 0 and ids.tolist() == [2, 1, 3]
    assert abs(float(w.sum()) - 1.0) < 1e-6


def test_router_matches_oracle_on_random_routes(built_lib, oracle_mod):
    for logits, bias, groups, top_groups, top_k, norm, scaling in _random_cases(120):
        if not np.isfinite(logits).all():
            continue  # -inf scores: exercised on the CPU against the reference header
        want = oracle_mod.route_v3_grouped_sigmoid(logits, bias, groups, top_groups, top_k, norm, scaling)
        rc, ids, w, out = ops.deepseek_router_route(ops.ROUTER_V3_GROUPED_SIGMOID, logits, top_k, bias=bias,
                                                    num_groups=groups, top_k_groups=top_groups,
                                                    norm_topk_prob=norm, routed_scaling_factor=scaling)
        assert rc == want[0] == 0
        assert np.array_equal(ids, want[1])
        assert np.allclose(w, want[2], rtol=2e-6, atol=1e-6)
        want = oracle_mod.route_v4_sqrtsoftplus(logits, bias, top_k, norm, scaling)
        rc, ids, w, out = ops.deepseek_router_route(ops.ROUTER_V4_SQRTSOFTPLUS, logits, top_k, bias=bias,
                                                    norm_topk_prob=norm, routed_scaling_factor=scaling)
        assert rc == 0 and np.array_equal(ids, want[1])
        assert np.allclose(w, want[2], rtol=2e-6, atol=1e-6)


def test_router_deepseek_v3_sized_route(built_lib, oracle_mod):
    rng = np.random.default_rng(5)
    logits = rng.standard_normal(256).astype(np.float32)
    bias = (rng.standard_normal(256) * 0.1).astype(np.float32)
    want = oracle_mod.route_v3_grouped_sigmoid(logits, bias, 8, 4, 8, True, 2.5)
    rc, ids, w, out = ops.deepseek_router_route(ops.ROUTER_V3_GROUPED_SIGMOID, logits, 8, bias=bias, num_groups=8,
                                                top_k_groups=4, routed_scaling_factor=2.5)
    assert rc == 0 and np.array_equal(ids, want[1]) and np.allclose(w, want[2], rtol=2e-6, atol=1e-6)


def test_router_rejects_bad_requests(built_lib):
    rc, _, _, out = ops.deepseek_router_route(ops.ROUTER_V4_SQRTSOFTPLUS, np.zeros(4, np.float32), 17)
    assert rc == -1 and out.status == -1 and out.route_error == -1
    rc, _, _, out = ops.deepseek_router_route(ops.ROUTER_V4_HASH, np.zeros(4, np.float32), 2, hash_route_table=[0, 1],
                                              route_token=1)
    assert rc == -1
    rc, _, _, out = ops.deepseek_router_route(ops.ROUTER_V4_HASH, np.zeros(4, np.float32), 2, hash_route_table=[0, 9])
    assert rc == -1 and out.route_error == -3
