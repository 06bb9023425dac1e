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


def bf16_bits(values) -> np.ndarray:
    from nerva_b200 import synth
    return synth.f32_to_bf16(np.asarray(values, dtype=np.float32))
