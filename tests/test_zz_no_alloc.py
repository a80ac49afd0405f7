"""The allocation-free host read (ntcb_read_channels_to_host_noalloc).

It exists for callers that must not reach cudaMalloc - frame or streaming threads, fixed memory
budgets, hosts that forbid allocation in some regions - and stages through an array built into
the library instead of the buffer ntcb_texture_set_read_channels grows on demand.  The test calls
it through the C ABI twice in a row (a padded channel subset, then a full read that reuses the
same staging bytes) and compares with the existing entry point bit for bit (the copy is
FLOAT16 -> FLOAT16, so the tolerance is zero, as in the other read-channels tests).

The file sorts last so that a run stopping at the first failure has already run everything else;
it does not depend on any other test having run.
"""
import ctypes

import numpy as np
import pytest

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, synthetic  # noqa: E402

pytestmark = pytest.mark.gpu


def _read_noalloc(pointer, layout, width, height, channels, first, count, pixel_stride, row_pitch, fill):
    out = np.full(height * row_pitch // 2, fill, dtype=np.float16)
    binding.check(binding.lib().ntcb_read_channels_to_host_noalloc(
        pointer, layout, width, height, channels, first, count, out.ctypes.data, pixel_stride, row_pitch, None))
    return out


@pytest.mark.parametrize("layout", [binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS])
def test_noalloc_read_matches_read_channels(layout):
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(160, 72, 6, 0, 2, 8, seed=41, network="unit"))
    context = binding.Context(0)
    texture_set = context.create_texture_set(data.container, layout)
    try:
        texture_set.decompress(True)
        texture_set.synchronize()
        channels = texture_set.desc.channels
        for mip in (0, 1):
            width, height = texture_set.mip_size(mip)
            pointer, size = texture_set.device_mip(mip)
            assert size == width * height * channels * 2

            # call 1: three channels with padding between pixels and rows (gaps must read as zeros)
            pixel_stride, row_pitch = 10, (width + 5) * 10
            expected = np.full(height * row_pitch // 2, 9.0, dtype=np.float16)
            texture_set.read_channels_into(mip, expected.ctypes.data, False, 2, 3, pixel_stride, row_pitch)
            got = _read_noalloc(pointer, layout, width, height, channels, 2, 3, pixel_stride, row_pitch, 7.0)
            assert np.array_equal(got.view(np.uint16), expected.view(np.uint16))

            # call 2, straight after: every channel, tightly packed, over the same staging bytes
            pixel_stride, row_pitch = channels * 2, width * channels * 2
            expected = texture_set.read_mip(mip).reshape(-1)
            got = _read_noalloc(pointer, layout, width, height, channels, 0, channels, pixel_stride, row_pitch, 7.0)
            assert np.array_equal(got.view(np.uint16), expected.view(np.uint16))

        # the property the entry point exists for: once the first call on the device has looked up the
        # array's address, a call takes no device memory - not even for a padded channel subset, the
        # request that makes ntcb_texture_set_read_channels grow its staging buffer
        import torch

        width, height = texture_set.mip_size(1)
        pointer, _ = texture_set.device_mip(1)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        for first, count, pixel_stride in ((1, 4, 12), (0, channels, channels * 2), (3, 2, 4)):
            _read_noalloc(pointer, layout, width, height, channels, first, count, pixel_stride, (width + 3) * pixel_stride, 1.0)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the allocation-free read took %d bytes of device memory" % (free_before - free_after)

        # a mip address that is not 4-byte aligned is refused on the host (nothing is launched)
        code = binding.lib().ntcb_read_channels_to_host_noalloc(
            pointer + 2, layout, width, height, channels, 0, channels, got.ctypes.data, channels * 2, width * channels * 2, None)
        assert code == -1

        # requests beyond the built-in staging area are refused, not truncated
        width, height = texture_set.mip_size(0)
        pointer, _ = texture_set.device_mip(0)
        huge = np.zeros(8, dtype=np.float16)
        code = binding.lib().ntcb_read_channels_to_host_noalloc(
            pointer, layout, width, height, channels, 0, channels, huge.ctypes.data, channels * 2, 1 << 20, None)
        assert code == -9 and b"staging" in binding.lib().ntcb_last_error()
        code = binding.lib().ntcb_read_channels_to_host_noalloc(
            pointer, layout, width, height, channels, 4, 3, huge.ctypes.data, 6, width * 6, None)
        assert code == -9
    finally:
        texture_set.close()
        context.close()
