"""nerva_cuda_deepseek_moe_forward on the GPU against the CPU oracle (fp32; summation orders differ)."""
import numpy as np
import pytest

from nerva_b200 import ops
from tests.test_cpu_moe_forward import moe_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,clamp", [((96, 40, 6, 3), False), ((96, 40, 6, 3), True),
                                         ((2048, 1408, 8, 6), False), ((33, 7, 3, 1), False)])
def test_moe_forward_matches_oracle(built_lib, oracle_mod, shape, clamp):
    c = moe_case(*shape, seed=shape[0])
    rc, got, out = ops.deepseek_moe_forward(c["x"], c["ids"], c["weights"], c["w_gate"], c["w_up"], c["w_down"],
                                            c["hidden"], c["intermediate"], c["experts"], clamp_swiglu=clamp,
                                            swiglu_limit=0.5)
    want_rc, want = oracle_mod.moe_forward(c["x"], c["ids"], c["weights"], c["w_gate"], c["w_up"], c["w_down"],
                                           c["hidden"], c["intermediate"], c["experts"], clamp_swiglu=clamp,
                                           swiglu_limit=0.5)
    assert rc == want_rc == 0 and out.status == 0 and out.moe_error == 0 and out.kernel_launches == 2
    scale = max(1.0, float(np.abs(want).max()))
    assert np.abs(got - want).max() <= 2e-5 * scale


def test_moe_forward_rejects_bad_expert(built_lib):
    c = moe_case(16, 8, 4, 2, seed=1)
    rc, _, out = ops.deepseek_moe_forward(c["x"], [1, 4], c["weights"], c["w_gate"], c["w_up"], c["w_down"], 16, 8, 4)
    assert rc == -1 and out.status == -1 and out.moe_error == -2
