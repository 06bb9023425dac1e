"""nerva_cuda_deepseek_mla_decode on the GPU against the CPU oracle (fp32 both; the summation orders
differ, so the bound is the reference's own smoke tolerance scaled to the problem size)."""
import numpy as np
import pytest

from nerva_b200 import ops
from tests.test_cpu_mla import FIXTURE, mla_case

pytestmark = pytest.mark.gpu


def _run(f, oracle_mod):
    q_pe = f["q_pe"] if f["rope"] else np.zeros(1, np.float32)
    k_pe = f["k_pe"] if f["rope"] else np.zeros(1, np.float32)
    rc, got, out = ops.deepseek_mla_decode(f["q_nope"], q_pe, f["kv_c"], k_pe, f["w_uk"], f["w_uv"], f["heads"],
                                           f["tokens"], f["rank"], f["nope"], f["rope"], f["v"], f["scale"])
    want_rc, want = oracle_mod.mla_decode(f["q_nope"], q_pe, f["kv_c"], k_pe, f["w_uk"], f["w_uv"], f["heads"],
                                          f["tokens"], f["rank"], f["nope"], f["rope"], f["v"], f["scale"])
    return rc, got, out, want_rc, want


def test_mla_reference_fixture(built_lib, oracle_mod):
    rc, got, out, want_rc, want = _run(FIXTURE, oracle_mod)
    assert rc == want_rc == 0 and out.status == 0 and out.decode_error == 0
    assert np.abs(got - want).max() <= 1e-6
    assert out.output_hash != 0 and out.hot_path_allocations == 0 and out.sync_calls == 1


@pytest.mark.parametrize("shape", [
    (16, 1024, 512, 128, 64, 128),   # DeepSeek-V2-Lite: 16 heads, latent 512, rope 64
    (16, 1, 512, 128, 64, 128), (16, 65, 512, 128, 64, 128), (16, 5000, 512, 128, 64, 128),
    (20, 333, 96, 24, 8, 40), (3, 77, 40, 6, 0, 5), (128, 200, 512, 128, 64, 128), (2, 50, 1024, 16, 16, 16)])
def test_mla_matches_oracle(built_lib, oracle_mod, shape):
    f = mla_case(*shape, seed=shape[1] + shape[0])
    rc, got, out, want_rc, want = _run(f, oracle_mod)
    assert rc == want_rc == 0
    assert np.abs(got - want).max() <= 2e-5
    rc2, again, _, _, _ = _run(f, oracle_mod)
    assert np.array_equal(got, again)  # bit-stable run to run


def test_mla_rejects_bad_requests(built_lib):
    z = np.zeros(8, np.float32)
    rc, _, out = ops.deepseek_mla_decode(z, z, z, z, z, z, 0, 1, 1, 1, 1, 1, 1.0)
    assert rc == -1 and out.status == -1
    rc, _, out = ops.deepseek_mla_decode(z, z, z, z, z, z, 1, 1, 2048, 1, 1, 1, 1.0)
    assert rc == -1
