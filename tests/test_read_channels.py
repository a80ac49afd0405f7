"""Output formats of the decode path: ReadChannels (channel formats, colour spaces, dithering) as a
separate pass, and the same conversion fused into the decode kernel's epilogue.

The fixtures `tests/golden/readchannels_*.npz` hold fp16 texels decoded by the unmodified reference
and what its `ITextureSet::ReadChannels` made of them for a list of requests.

Bars:
  * conversion kernel vs the reference on the same texels: identical bytes, every format, colour
    space and dither setting (the kernel spells out the reference's fast-math arithmetic);
  * fused epilogue vs decode followed by ReadChannels: identical bytes;
  * CPU restatement (C library transfer functions, IEEE division) vs the reference: identical for
    linear channels and for every UNORM8 request of the fixtures; for sRGB / HLG channels at most
    one code in UNORM16, one unit in the last place in FLOAT16 and 4e-6 relative in FLOAT32.
"""
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN_DIR, load_golden

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, container, synthetic  # noqa: E402

CASE = "readchannels_r64x48_g2_f8"
UNORM8, UNORM16, FLOAT16, FLOAT32, UINT32 = 1, 2, 3, 4, 5
LINEAR, SRGB, HLG = 0, 1, 2


@pytest.fixture(scope="module")
def case():
    with open(os.path.join(GOLDEN_DIR, "readchannels_index.json")) as f:
        index = json.load(f)[CASE]
    return index, load_golden(CASE)


def _requests(index):
    return sorted(index["requests"].items())


def _bytes(array):
    return np.ascontiguousarray(array).view(np.uint8)


# ---------------------------------------------------------------------------------------------
# CPU: the restatement against the reference's outputs, and known answers
# ---------------------------------------------------------------------------------------------

def test_restatement_against_reference_outputs(oracle, case):
    index, fixture = case
    spaces = index["channel_spaces"]
    for mip in index["mips"]:
        texels = fixture["texels_mip%d" % mip].view(np.float16)
        for name, r in _requests(index):
            reference = fixture["%s_mip%d" % (name, mip)]
            restated = oracle.read_channels(texels, r["format"], r["first"], r["count"], r["components"], spaces,
                                            r["dst"], r["dither"])
            assert restated.shape == reference.shape and restated.dtype == reference.dtype, name
            nonlinear = any(spaces[r["first"] + c] != LINEAR or (r["dst"] and r["dst"][c] != LINEAR) for c in range(r["count"]))
            if r["format"] in (UNORM8, UINT32) or not nonlinear:
                assert np.array_equal(_bytes(restated), _bytes(reference)), name
            elif r["format"] == UNORM16:
                distance = np.abs(restated.astype(np.int64) - reference.astype(np.int64))
                assert distance.max() <= 1 and (distance > 0).mean() < 0.01, name
            elif r["format"] == FLOAT16:
                a, b = restated.astype(np.float64), reference.astype(np.float64)
                assert np.all(np.abs(a - b) <= 1e-3 * np.abs(b) + 1e-7), name
                assert (_bytes(restated) != _bytes(reference)).mean() < 0.005, name
            else:
                a, b = restated.astype(np.float64), reference.astype(np.float64)
                assert np.all(np.abs(a - b) <= 4e-6 * np.abs(b) + 1e-9), name


def test_restatement_known_answers(oracle):
    values = np.array([[[0.0, 0.5, 1.0, 2.0], [-1.0, 0.25, 0.0031308, 0.75]]], dtype=np.float16)  # [1][2][4]
    linear = oracle.read_channels(values, UNORM8)
    assert linear.tolist() == [[[0, 128, 255, 255], [0, 64, 1, 191]]]  # round half away from zero, clamped
    srgb = oracle.read_channels(values, UNORM8, dst_color_spaces=[SRGB] * 4)
    # sRGB transfer function: 0.5 -> 0.7354, 0.25 -> 0.5371, 0.75 -> 0.8807; the linear toe below 0.0031308
    assert srgb.tolist() == [[[0, 188, 255, 255], [0, 137, 10, 225]]]
    back = oracle.read_channels(values, FLOAT32, src_color_spaces=[SRGB] * 4)
    assert abs(float(back[0, 0, 1]) - 0.21404114) < 1e-6 and float(back[0, 0, 2]) == 1.0
    hlg = oracle.read_channels(values, FLOAT32, dst_color_spaces=[HLG] * 4)
    assert abs(float(hlg[0, 0, 2]) - 0.5) < 1e-6 and abs(float(hlg[0, 1, 1]) - 0.25) < 1e-6  # sqrt branch
    assert abs(float(hlg[0, 0, 3]) - (0.17883277 * np.log(2.0 - 0.28466892) + 0.55991073)) < 1e-6
    assert float(hlg[0, 1, 0]) == -0.5  # odd extension
    # components past the requested channels: 0, and 1 in component 3
    padded = oracle.read_channels(values, UNORM16, first_channel=1, num_channels=2, components=5)
    assert padded[0, 0].tolist() == [32768, 65535, 0, 65535, 0]
    wide = oracle.read_channels(values, UINT32, first_channel=2, num_channels=2)
    assert wide[0, 0].tolist() == [1, 2] and wide[0, 1].tolist() == [0, 0]
    large = np.array([[[np.inf, -40000.0, -np.inf, 65504.0]]], dtype=np.float16)
    assert oracle.read_channels(large, FLOAT16)[0, 0].tolist() == [65504.0, -40000.0, -65504.0, 65504.0]  # +-65504 clamp


def test_restatement_dither_is_a_bounded_deterministic_offset(oracle):
    rng = np.random.default_rng(5)
    texels = rng.uniform(-0.1, 1.1, size=(24, 40, 4)).astype(np.float16)
    plain = oracle.read_channels(texels, UNORM8).astype(np.int32)
    first = oracle.read_channels(texels, UNORM8, use_dithering=True).astype(np.int32)
    again = oracle.read_channels(texels, UNORM8, use_dithering=True).astype(np.int32)
    assert np.array_equal(first, again)
    assert np.abs(first - plain).max() <= 1 and 0.1 < (first != plain).mean() < 0.4  # flips with probability E|offset| = 1/4
    # the offsets average out: the dithered mean tracks the exact value
    exact = np.clip(texels.astype(np.float64), 0, 1) * 255
    assert abs(float((first - exact).mean())) < 0.02
    # channels draw different offsets, pixels too
    subset = oracle.read_channels(texels, UNORM8, first_channel=1, num_channels=2, use_dithering=True).astype(np.int32)
    assert not np.array_equal(subset, first[:, :, 1:3])


def test_container_carries_channel_colour_spaces():
    spec = synthetic.TextureSetSpec(32, 16, 4, 1, 2, 8, seed=2, network="unit")
    tagged = synthetic.make_texture_set(spec)
    tagged.channel_color_spaces = [SRGB, LINEAR, HLG, SRGB]
    document_start = tagged.container.index(b'{"schemaVersion"')
    text = tagged.container[document_start:tagged.container.index(b"\0", document_start)].decode()
    assert json.loads(text)["channels"] == [{"colorSpace": "sRGB"}, {}, {"colorSpace": "HLG"}, {"colorSpace": "sRGB"}]
    desc = binding.probe_container(tagged.container)
    assert desc.channels == 4
    broken = tagged.container.replace(b'"colorSpace":"HLG"', b'"colorSpace":"XYZ"')
    with pytest.raises(binding.NtcbError) as failure:
        binding.probe_container(broken)
    assert "color space" in str(failure.value)


# ---------------------------------------------------------------------------------------------
# GPU
# ---------------------------------------------------------------------------------------------

def _conversion(index, r, with_source_spaces=True):
    source = [index["channel_spaces"][r["first"] + c] for c in range(r["count"])] if with_source_spaces else None
    return binding.make_conversion(r["format"], r["count"], r["first"], r["components"], source, r["dst"], r["dither"])


@pytest.mark.gpu
@pytest.mark.parametrize("layout", [binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS])
def test_conversion_kernel_reproduces_reference_bytes(case, layout):
    import torch

    index, fixture = case
    for mip in index["mips"]:
        texels = fixture["texels_mip%d" % mip].view(np.float16)
        height, width, channels = texels.shape
        if layout == binding.LAYOUT_PLANAR_PAIRS:
            # the reference's internal layout: per row, channel pairs as planes of (x, pair member)
            arranged = texels.reshape(height, width, channels // 2, 2).transpose(0, 2, 1, 3)
        else:
            arranged = texels
        device = torch.from_numpy(np.ascontiguousarray(arranged)).cuda()
        for name, r in _requests(index):
            reference = fixture["%s_mip%d" % (name, mip)]
            converted = binding.convert_channels(device, _conversion(index, r), layout, width, height, channels)
            assert np.array_equal(_bytes(converted.cpu().numpy()), _bytes(reference)), (name, mip)


@pytest.mark.gpu
@pytest.mark.parametrize("layout", [binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS])
def test_read_channels_and_fused_epilogue_agree_with_the_restatement(oracle, case, layout):
    """Texture-set level: ReadChannels of our own decode equals the CPU restatement applied to our
    own fp16 texels (same tolerances as above), and the fused decode writes the same bytes."""
    index, fixture = case
    spaces = index["channel_spaces"]
    tagged = fixture["container"].tobytes()
    geo, latents, int8_blob, fp8_blob = container.read_container(tagged)
    plain = container.write_container(geo, latents, int8_blob, fp8_blob)
    use_int8 = index["mode"] == "int8"
    with binding.Context(0) as context:
        raw_set = context.create_texture_set(plain, layout)
        raw_set.decompress(use_int8)
        texture_set = context.create_texture_set(tagged, layout)
        texture_set.decompress(use_int8)
        for name, r in _requests(index):
            two_pass = [texture_set.read_mip(mip, r["first"], r["count"], r["format"], r["dst"], r["dither"], r["components"])
                        for mip in range(geo.mips)]
            for mip in (0, geo.mips - 1):
                restated = oracle.read_channels(raw_set.read_mip(mip), r["format"], r["first"], r["count"], r["components"],
                                                spaces, r["dst"], r["dither"])
                if restated.dtype.kind == "u":
                    distance = np.abs(restated.astype(np.int64) - two_pass[mip].astype(np.int64))
                    assert distance.max() <= 1 and (distance > 0).mean() < 0.02, (name, mip)
                else:
                    a, b = restated.astype(np.float64), two_pass[mip].astype(np.float64)
                    assert np.all(np.abs(a - b) <= 1e-3 * np.abs(b) + 1e-7), (name, mip)
            fused, milliseconds = texture_set.decompress_converted(_conversion(index, r, False), use_int8, True)
            assert milliseconds > 0
            for mip in range(geo.mips):
                assert np.array_equal(_bytes(fused[mip]), _bytes(two_pass[mip])), (name, mip)
            texture_set.decompress(use_int8)
        raw_set.close()
        texture_set.close()


@pytest.mark.gpu
@pytest.mark.parametrize("numerics", [binding.NUMERICS_REFERENCE, binding.NUMERICS_EXACT], ids=["reference", "exact"])
def test_fused_epilogue_on_ragged_shapes_row_ranges_and_fp8(oracle, numerics):
    """Kernel level: the converting epilogue through ntcb_decode on sizes that are no multiple of
    the tile, in FP8 mode, in two row bands; against the conversion kernel run on the fp16 decode."""
    import torch

    spec = synthetic.TextureSetSpec(203, 77, 10, 0, 3, 12, seed=31, network="unit")
    data = synthetic.make_texture_set(spec)
    geo = data.geometry
    resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
    for use_int8 in (False, True):
        resident.decode(use_int8)
        torch.cuda.synchronize()
        resident.check_status()
        for conversion in (binding.make_conversion(UNORM8, 3, 2, 4, [SRGB] * 3, [SRGB] * 3, True),
                           binding.make_conversion(UNORM8, 10, 0, 10, None, None, False),
                           binding.make_conversion(UNORM16, 1, 9, 1, None, None, True),
                           binding.make_conversion(FLOAT32, 5, 5, 5, [LINEAR, SRGB, HLG, LINEAR, SRGB], [HLG] * 5, False),
                           binding.make_conversion(UNORM8, 3, 7, 3, None, [SRGB] * 3, True)):
            whole = resident.decode_converted(use_int8, conversion)
            bands = {mip: (0, geo.color_mips[mip].height // 2) for mip in range(geo.mips)}
            rest = {mip: (geo.color_mips[mip].height // 2, geo.color_mips[mip].height) for mip in range(geo.mips)}
            banded = resident.decode_converted(use_int8, conversion, row_ranges=bands)
            params = resident.params(use_int8, out=banded, row_ranges=rest, conversion=conversion)
            resident.launch(params)
            torch.cuda.synchronize()
            resident.check_status()
            assert torch.equal(whole, banded)
            for mip in range(geo.mips):
                cm = geo.color_mips[mip]
                texels = resident.out[cm.texel_offset * geo.channels:(cm.texel_offset + cm.width * cm.height) * geo.channels]
                expected = binding.convert_channels(texels.view(cm.height, cm.width, geo.channels), conversion)
                start = cm.texel_offset * conversion.components
                got = whole[start:start + cm.width * cm.height * conversion.components].view(cm.height, cm.width, -1)
                assert torch.equal(got, expected), (use_int8, mip)


@pytest.mark.gpu
def test_read_channels_argument_checks(case):
    index, fixture = case
    with binding.Context(0) as context:
        texture_set = context.create_texture_set(fixture["container"].tobytes())
        texture_set.decompress(True)
        width, height = texture_set.mip_size(0)
        out = np.zeros(width * height * 64, dtype=np.uint8)
        for kwargs, code in (({"channel_format": 0}, -1), ({"channel_format": 6}, -1),
                             ({"channel_format": UNORM16, "pixel_stride": 3}, -1),
                             ({"channel_format": FLOAT32, "pixel_stride": 2}, -1),
                             ({"dst_color_spaces": [0, 1, 3, 0, 0, 0]}, -1),
                             ({"channel_format": UNORM8, "pixel_stride": 4, "row_pitch": 4 * width - 1}, -1)):
            with pytest.raises(binding.NtcbError) as failure:
                texture_set.read_channels_into(0, out.ctypes.data, **kwargs)
            assert failure.value.code == code, kwargs
        with pytest.raises(binding.NtcbError):
            texture_set.decompress_converted(binding.make_conversion(UNORM8, 7), True)
        with pytest.raises(binding.NtcbError):
            texture_set.decompress_converted(binding.make_conversion(UNORM8, 2, components=17), True)
        with pytest.raises(binding.NtcbError):
            texture_set.decompress_converted(binding.make_conversion(9, 2), True)
        texture_set.close()


@pytest.mark.gpu
def test_conversion_against_a_live_reference_run(oracle):
    """When the reference library travels with the repository (oracle/_ref): a larger set, decoded
    and read back by the reference, against the conversion kernel on the reference's texels."""
    import torch

    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libntc_ref.so is not built")
    spec = synthetic.TextureSetSpec(320, 200, 8, 0, 2, 8, seed=44, network="unit")
    plain = synthetic.make_texture_set(spec)
    tagged = synthetic.make_texture_set(spec)
    spaces = [SRGB, SRGB, SRGB, LINEAR, HLG, HLG, LINEAR, SRGB]
    tagged.channel_color_spaces = spaces
    geo = plain.geometry
    raw = oracle.ReferenceDecoder(plain.container, geo.channels)
    raw.decompress(False)
    reference = oracle.ReferenceDecoder(tagged.container, geo.channels, staging_bytes_per_pixel=64)
    reference.decompress(False)
    requests = [(UNORM8, 0, 4, 4, [SRGB, SRGB, SRGB, LINEAR], True), (UNORM16, 4, 2, 2, [HLG, LINEAR], True),
                (FLOAT16, 0, 8, 8, None, False), (FLOAT32, 3, 5, 6, [SRGB] * 5, False), (UNORM8, 7, 1, 1, [SRGB], False),
                (UINT32, 0, 8, 8, None, False)]
    for mip in (0, 1, 4):
        cm = geo.color_mips[mip]
        texels = torch.from_numpy(raw.read_mip(mip, cm.width, cm.height).copy()).cuda()
        for channel_format, first, count, components, dst, dither in requests:
            expected = reference.read_channels(mip, cm.width, cm.height, channel_format, first, count, components, dst, dither)
            conversion = binding.make_conversion(channel_format, count, first, components, spaces[first:first + count], dst, dither)
            got = binding.convert_channels(texels, conversion).cpu().numpy()
            assert np.array_equal(_bytes(got), _bytes(expected)), (mip, channel_format, first)
    raw.close()
    reference.close()


# ---------------------------------------------------------------------------------------------
# ReadChannels with a size other than the mip's: the reference's bilinear resize
# (fixture: tests/golden/readchannels_resize.npz, generator tests/golden/make_golden_resize.py)
# ---------------------------------------------------------------------------------------------

RESIZE_SPACES = [SRGB, SRGB, SRGB, LINEAR, HLG, LINEAR]
RESIZE_SIZES = [(0, (32, 24)), (0, (100, 70)), (0, (65, 47)), (0, (1, 1)), (1, (9, 40)), (1, (32, 25))]
RESIZE_REQUESTS = {
    "f16_all_linear": (FLOAT16, 0, 6, 6, None, False),
    "u8_rgba_srgb_dither": (UNORM8, 0, 4, 4, [SRGB, SRGB, SRGB, LINEAR], True),
    "f32_mixed": (FLOAT32, 2, 4, 4, [LINEAR, SRGB, HLG, LINEAR], False),
    "u16_pair_plus_default": (UNORM16, 4, 2, 4, None, True),
}


def test_restated_resize_against_reference_outputs(oracle):
    """The CPU restatement divides exactly where the reference's GPU code divides approximately and
    uses the C library's transfer functions: UNORM8 within 1 code, UNORM16 within 8, floating point
    within 1 % (of the value, or of 0.001 for smaller ones), at most 1 % of UNORM values differing."""
    golden = load_golden("readchannels_resize")
    for mip, (width, height) in RESIZE_SIZES:
        texels = golden["texels_mip%d" % mip].view(np.float16)
        for name, (channel_format, first, count, components, dst, dither) in RESIZE_REQUESTS.items():
            expected = golden["%s_mip%d_%dx%d" % (name, mip, width, height)]
            got = oracle.read_channels(texels, channel_format, first, count, components, RESIZE_SPACES, dst, dither, size=(width, height))
            assert got.shape == expected.shape == (height, width, components)
            if channel_format in (UNORM8, UNORM16):
                distance = np.abs(got.astype(np.int64) - expected.astype(np.int64))
                assert distance.max() <= (1 if channel_format == UNORM8 else 8), (name, mip, width, height)
                assert (distance > 0).mean() <= 0.01, (name, mip, width, height)
            else:
                a, b = got.astype(np.float64), expected.astype(np.float64)
                assert (np.abs(a - b) <= 0.01 * np.maximum(np.abs(b), 1e-3)).all(), (name, mip, width, height)


@pytest.mark.gpu
def test_resized_read_matches_reference_outputs():
    """The library on the fixture's container: identical bytes for every size and request."""
    golden = load_golden("readchannels_resize")
    with binding.Context() as context:
        texture_set = context.create_texture_set(golden["container"].tobytes())
        texture_set.decompress(False)
        for mip, size in RESIZE_SIZES:
            for name, (channel_format, first, count, components, dst, dither) in RESIZE_REQUESTS.items():
                expected = golden["%s_mip%d_%dx%d" % (name, mip, size[0], size[1])]
                got = texture_set.read_mip(mip, first, count, channel_format, dst, dither, components, size=size)
                assert np.array_equal(_bytes(got), _bytes(expected)), (name, mip, size)
        # the same kernel on texels the caller holds (ntcb_convert_channels with a destination size)
        import torch

        texels = torch.from_numpy(golden["texels_mip0"].view(np.float16).copy()).cuda()
        name, (channel_format, first, count, components, dst, dither) = "u8_rgba_srgb_dither", RESIZE_REQUESTS["u8_rgba_srgb_dither"]
        conversion = binding.make_conversion(channel_format, count, first, components, RESIZE_SPACES[first:first + count], dst, dither)
        got = binding.convert_channels(texels, conversion, size=(100, 70)).cpu().numpy()
        assert np.array_equal(_bytes(got), _bytes(golden["%s_mip0_100x70" % name]))
        # the mip's own size is the 1:1 path; a non-positive size is refused as in the reference
        width, height = texture_set.mip_size(1)
        assert np.array_equal(texture_set.read_mip(1, size=(width, height)), texture_set.read_mip(1))
        with pytest.raises(binding.NtcbError) as error:
            texture_set.read_mip(0, size=(0, 8))
        assert error.value.code == -9 and "must be positive" in str(error.value)
        texture_set.close()


@pytest.mark.gpu
def test_resized_read_against_a_live_reference_run(oracle):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libntc_ref.so is not built")
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(160, 96, 8, 0, 2, 8, seed=45, network="unit"))
    spaces = [SRGB, SRGB, SRGB, LINEAR, HLG, HLG, LINEAR, SRGB]
    data.channel_color_spaces = spaces
    reference = oracle.ReferenceDecoder(data.container, data.geometry.channels, staging_bytes_per_pixel=256)
    reference.decompress(True)
    requests = [(FLOAT16, 0, 8, 8, None, False), (UNORM8, 0, 4, 4, [SRGB, SRGB, SRGB, LINEAR], True),
                (FLOAT32, 3, 5, 6, [SRGB] * 5, False), (UNORM16, 4, 2, 2, [HLG, LINEAR], True), (UINT32, 6, 2, 2, None, False)]
    with binding.Context() as context:
        texture_set = context.create_texture_set(data.container)
        texture_set.decompress(True)
        for mip, size in ((0, (80, 48)), (0, (213, 131)), (0, (161, 95)), (2, (7, 5)), (3, (33, 64)), (0, (160, 97)), (1, (1, 1))):
            for channel_format, first, count, components, dst, dither in requests:
                expected = reference.read_channels(mip, size[0], size[1], channel_format, first, count, components, dst, dither)
                got = texture_set.read_mip(mip, first, count, channel_format, dst, dither, components, size=size)
                assert np.array_equal(_bytes(got), _bytes(expected)), (mip, size, channel_format)
        texture_set.close()
    reference.close()
