import ctypes
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _has_gpu() -> bool:
    try:
        cudart = ctypes.CDLL("libcudart.so")
    except OSError:
        try:
            cudart = ctypes.CDLL("/usr/local/cuda/lib64/libcudart.so")
        except OSError:
            return False
    count = ctypes.c_int(0)
    return cudart.cudaGetDeviceCount(ctypes.byref(count)) == 0 and count.value > 0


def pytest_collection_modifyitems(config, items):
    # GPU tests fail loudly on a box without a device only when explicitly selected
    # with -m gpu; in an unfiltered run on a CPU machine they are skipped.
    if config.getoption("-m") and "gpu" in config.getoption("-m"):
        return
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    from nerva_b200 import build, ffi
    build.build()
    return ffi.lib()


@pytest.fixture(scope="session")
def oracle_mod():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def tiny_checkpoint(built_lib):
    from nerva_b200 import ops, synth
    return synth.dense_checkpoint(synth.TINY_QWEN3, fill=ops.synth_normal_bf16)


@pytest.fixture(scope="session")
def tiny_golden():
    with open(os.path.join(GOLDEN, "tiny_qwen3.json")) as f:
        return json.load(f)


def contract_self_distance(oracle_mod, checkpoint, max_context, prompt, steps, ref_logits) -> float:
    """max |logit difference| between two exact restatements of the same numeric
    contract that differ only in fp32 summation order (serial vs 8 interleaved
    partial sums per row).  Rounding projection inputs to bf16 makes deep/wide
    models sensitive to that order, so this is the floor under any logit bound."""
    oracle_mod.set_sum_lanes(8)
    try:
        dec = oracle_mod.Decoder(checkpoint, max_context, mode=oracle_mod.MODE_CUDA)
        _, alt = dec.decode_greedy(prompt, steps, want_logits=True)
    finally:
        oracle_mod.set_sum_lanes(1)
    return float(np.abs(alt[-1] - ref_logits[-1]).max())


def bf16_bits(values) -> np.ndarray:
    from nerva_b200 import synth
    return synth.f32_to_bf16(np.asarray(values, dtype=np.float32))


def first_divergence(got, want):
    """Index of the first position where two token streams differ, or None."""
    for i, (a, b) in enumerate(zip(got, want)):
        if int(a) != int(b):
            return i
    return None


def assert_stream_matches_or_ties(got, want, margins, tie_bound, what=""):
    """Greedy streams of two correct implementations may part only where the reference's own
    top-1 / top-2 margin is below what a change of fp32 summation order can move a logit by
    (tie_bound).  Everything before that position must be identical; returns the position of the
    tie (None when the streams are identical)."""
    at = first_divergence(got, want)
    if at is None:
        assert len(got) == len(want), f"{what}: {len(got)} tokens against {len(want)}"
        return None
    assert margins[at] <= tie_bound, (
        f"{what}: streams differ at step {at} ({got[at]} vs {want[at]}) where the reference margin "
        f"{margins[at]:.4g} is above the tie bound {tie_bound:.4g}")
    return at
