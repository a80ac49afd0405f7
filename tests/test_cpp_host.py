"""The C++ host interface (include/ntcb_host.h) used from a C++ program, as a client of the
reference's ntc::IContext / ITextureSet would use it: tests/cpp/host_example.cpp is compiled against
the header, linked with the library and run.  Without a GPU it must fail loudly at CreateContext;
on a GPU its texels and BC4 blocks must be the ones the Python binding gets through the C ABI."""
import os
import subprocess

import numpy as np
import pytest

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, synthetic  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE = os.path.join(ROOT, "rtxntc-library_b200")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _build(tmp_path) -> str:
    binary = str(tmp_path / "host_example")
    subprocess.run([NVCC, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "host_example.cpp"),
                    "-o", binary, "-L", PACKAGE, "-lntcb200", "-Xlinker", "-rpath", "-Xlinker", PACKAGE], check=True)
    return binary


def _fnv1a(data: bytes) -> int:
    value = 1469598103934665603
    for chunk in np.frombuffer(data, dtype=np.uint8):
        value = ((value ^ int(chunk)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return value


def _container(tmp_path):
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(48, 24, 4, 0, 2, 8, seed=17, network="unit", weights="fp8"))
    data.textures = [{"name": "Height", "firstChannel": 0, "numChannels": 1, "bcFormat": "BC4"},
                     {"name": "Mask", "firstChannel": 1, "numChannels": 3, "bcFormat": "BC7",
                      "bcModeBuffers": [{"mipLevel": 0, "data": _mode_bitmap(12, 6).tobytes()}]}]
    path = tmp_path / "set.ntc"
    path.write_bytes(data.container)
    return data, str(path)


def _mode_bitmap(blocks_x: int, blocks_y: int) -> np.ndarray:
    """A BC7 mode bitmap for a blocks_x x blocks_y mip: seeded modes and partitions, 9 bits per block."""
    rng = np.random.default_rng(4)
    limits = (15, 63, 63, 63, 7, 3, 0, 63)
    bits = np.zeros(binding.bc7_mode_buffer_size(blocks_x, blocks_y), dtype=np.uint8)
    for k in range(blocks_x * blocks_y):
        mode = int(rng.integers(0, 8))
        entry = (mode << 6 | int(rng.integers(0, limits[mode] + 1))) or 0x1BF
        byte, shift = (k * 9) // 8, (k * 9) % 8
        bits[byte] |= (entry << shift) & 0xFF
        bits[byte + 1] |= (entry >> (8 - shift)) & 0xFF
    return bits


def test_cpp_client_builds_and_fails_loudly_without_a_gpu(tmp_path):
    import torch

    binary = _build(tmp_path)
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: covered by the GPU test")
    _, path = _container(tmp_path)
    result = subprocess.run([binary, path], capture_output=True, text=True)
    assert result.returncode == 2, result.stderr
    assert "CreateContext" in result.stderr and "cuda" in result.stderr.lower()


@pytest.mark.gpu
def test_cpp_client_matches_the_c_abi(tmp_path):
    binary = _build(tmp_path)
    data, path = _container(tmp_path)
    result = subprocess.run([binary, path], capture_output=True, text=True)
    assert result.returncode == 0, result.stderr
    lines = result.stdout.splitlines()
    assert lines[0] == "texture 0: Height channels 0+1 bc 4" and lines[1] == "texture 1: Mask channels 1+3 bc 7"
    bc7 = lines[2].split()
    fields = lines[3].split()
    with binding.Context() as context:
        texture_set = context.create_texture_set(data.container)
        texture_set.decompress(False)
        texels = texture_set.read_mip(0)
        blocks = texture_set.block_compress(0, binding.BLOCK_FORMAT_BC4, 0).cpu().numpy()
        blocks7 = texture_set.block_compress_texture(1, 0).cpu().numpy()
        texture_set.close()
    assert int(bc7[1], 16) == _fnv1a(blocks7.tobytes()) and bc7[3] == str(_mode_bitmap(12, 6).nbytes) and bc7[5] == "same" and bc7[7] == "same"
    assert np.array_equal(binding.make_bc7_mode_buffer(blocks7), _mode_bitmap(12, 6))  # every block in the mode it was given
    assert int(fields[1], 16) == _fnv1a(np.ascontiguousarray(texels).tobytes())
    assert int(fields[3], 16) == _fnv1a(blocks.tobytes())
    assert fields[5] == "48x24x4"
