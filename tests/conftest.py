"""Shared fixtures of the test suite.

`-m "not gpu"` tests cover the CPU restatement against the golden vectors, the host logic and the
exported C ABI; `-m gpu` tests are the parity tests proper and call the sm_100a kernels through the
C ABI.  Only the tests (never the product) import anything under oracle/.
"""
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import __graft_entry__ as entry  # noqa: E402

entry.load_package()

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box)")


def pytest_collection_modifyitems(config, items):
    # keep the allocation-free entry point's test last (a run that stops at the first failure has
    # then already run everything else)
    items.sort(key=lambda item: 1 if "test_zz_" in item.nodeid else 0)


@pytest.fixture(scope="session")
def oracle():
    import oracle_py

    oracle_py.build_oracle()
    return oracle_py


@pytest.fixture(scope="session")
def golden_index():
    with open(os.path.join(GOLDEN_DIR, "index.json")) as f:
        return json.load(f)


def load_golden(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between two fp16 arrays (sign-magnitude aware)."""
    a = a.view(np.int16).astype(np.int32)
    b = b.view(np.int16).astype(np.int32)
    a = np.where(a < 0, -(a & 0x7FFF), a)
    b = np.where(b < 0, -(b & 0x7FFF), b)
    return np.abs(a - b)


def psnr_db(test: np.ndarray, reference: np.ndarray) -> float:
    """PSNR of `test` against `reference`, peak = the reference's value range."""
    t = test.astype(np.float64)
    r = reference.astype(np.float64)
    peak = max(float(r.max() - r.min()), 1e-12)
    mse = float(((t - r) ** 2).mean())
    if mse == 0.0:
        return float("inf")
    return 10.0 * np.log10(peak * peak / mse)


def reference_chain(oracle, data, use_int8):
    """The unmodified reference's decode of every mip of a synthetic set (oracle/_ref, through its
    public API: Decompress, then ReadChannels(FLOAT16, AddressSpace::Device) per mip), as one flat
    CUDA tensor in the interleaved order [mip][y][x][c]."""
    import torch

    geo = data.geometry
    decoder = oracle.ReferenceDecoder(data.container, geo.channels)
    try:
        decoder.decompress(use_int8)
        chain = torch.empty(geo.total_texels * geo.channels, dtype=torch.float16, device="cuda:0")
        for mip, cm in enumerate(geo.color_mips):
            decoder.read_mip_into(mip, cm.width, cm.height, chain.data_ptr() + cm.texel_offset * geo.channels * 2, True)
        torch.cuda.synchronize()
    finally:
        decoder.close()
    return chain
