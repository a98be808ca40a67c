import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def bf16_bits_to_f32(u16):
    return (np.asarray(u16).astype(np.uint32) << 16).view(np.float32)


@pytest.fixture(scope="session")
def golden_nvfp4_quantize():
    return load_golden("nvfp4_quantize.npz")


@pytest.fixture(scope="session")
def golden_nvfp4_linear():
    return load_golden("nvfp4_linear.npz")


@pytest.fixture(scope="session")
def golden_mxfp8_quantize():
    return load_golden("mxfp8_quantize.npz")
