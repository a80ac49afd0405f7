"""The decoder behind the reference's own public API.

oracle/_ref/libntc_ref_ntcb.so is LibNTC built from its own sources with ONE translation unit
changed: TextureSet::Decompress hands a set loaded from a file to libntcb200.so (ntcb_decode into
the reference's own texture-data buffer, oracle/texture_set_ntcb.inl) instead of running
UnpackLatents, ConvertNetworkFromQuantizedToFp16 and the per-mip cuda::Inference loop
(src/TextureSet.cpp:1691-1864).  The same harness drives it and the stock library through
ntc::CreateContext -> IContext::CreateCompressedTextureSetFromMemory -> ITextureSet::Decompress ->
ITextureSet::ReadChannels (include/libntc/ntc.h:1330, 1171, 933, 902); the bytes that come back
must be identical, for both weight sets, as FLOAT16 and as UNORM8 pixels.
"""
import numpy as np
import pytest

from conftest import load_golden

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import container, synthetic  # noqa: E402

pytestmark = pytest.mark.gpu

GOLDEN_CASES = ["sq64_g2_f8_unit", "sq64_g2_f8_bench", "r96x40_g3_f12_unit", "sq128_g4_f12_2bit_bench",
                "sq128_g4_f12_2bit_unit", "r128x64_g4_f16_unit", "r33x17_g1_f4_unit", "sq128_g6_f8_unit",
                "sq64_g5_f16_mip0_unit"]
UNORM8, FLOAT16 = 1, 3  # ntc::ChannelFormat


@pytest.fixture(scope="module")
def both(oracle):
    if not (oracle.reference_available() and oracle.reference_ntcb_available()):
        pytest.skip("oracle/_ref/libntc_ref.so and libntc_ref_ntcb.so are not both built")
    return oracle


def _compare(oracle, image, geo, modes):
    stock = oracle.ReferenceDecoder(image, geo.channels)
    routed = oracle.ReferenceDecoder(image, geo.channels, library=oracle.REF_NTCB_LIB)
    try:
        for use_int8 in modes:
            stock.decompress(use_int8)
            milliseconds = routed.decompress(use_int8)
            assert milliseconds > 0  # DecompressionStats::gpuTimeMilliseconds keeps working
            for mip, cm in enumerate(geo.color_mips):
                theirs = stock.read_mip(mip, cm.width, cm.height)
                ours = routed.read_mip(mip, cm.width, cm.height)
                assert np.array_equal(ours.view(np.uint16), theirs.view(np.uint16)), (use_int8, mip)
                theirs = stock.read_channels(mip, cm.width, cm.height, UNORM8)
                ours = routed.read_channels(mip, cm.width, cm.height, UNORM8)
                assert np.array_equal(ours, theirs), (use_int8, mip)
    finally:
        stock.close()
        routed.close()


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_reference_api_with_this_decoder_behind_it_gives_the_stock_bytes(both, golden_index, name):
    fixture = load_golden(name)
    image = fixture["container"].tobytes()
    geo, _, _, _ = container.read_container(image)
    _compare(both, image, geo, [mode == "int8" for mode in golden_index[name]["modes"]])
    # and the stock bytes are the committed fixture
    stock = both.ReferenceDecoder(image, geo.channels, library=both.REF_NTCB_LIB)
    try:
        for mode in golden_index[name]["modes"]:
            stock.decompress(mode == "int8")
            for mip, cm in enumerate(geo.color_mips):
                assert np.array_equal(stock.read_mip(mip, cm.width, cm.height).view(np.uint16), fixture["%s_mip%d" % (mode, mip)])
    finally:
        stock.close()


def test_reference_api_with_this_decoder_on_the_benchmark_set(both):
    """Configuration 1 at full size (4096 x 4096, 12 channels, 13 mips), both weight sets."""
    data = synthetic.make_texture_set(synthetic.config_spec(1))
    _compare(both, data.container, data.geometry, (False, True))
