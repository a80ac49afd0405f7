"""BC1 - BC5 encoding of decoded texels (`ntcb_block_compress`).

PARITY PINNED to the reference's own shader source.  The reference's encoders are compute shaders
(src/shaders/CompressBC1-5.hlsl, BlockCompressCommon.hlsli) that it only runs through a graphics
API, which is unavailable here - but the shader source itself compiles as C++ once HLSL's vector
types are supplied (oracle/hlsl_shim.h; oracle/transform_hlsl.py changes parameter qualifiers,
literal suffixes and attributes, nothing of the arithmetic), and oracle/build_ref.sh builds it that
way, without floating-point contraction, into oracle/_ref/libntc_ref_bc.so.  Its output on seeded
images is committed as tests/golden/block_compress_ref.npz (generator:
tests/golden/make_golden_block_compress.py).  What is tested:
  * the CPU restatement of the encoders (oracle/ntc_oracle.c) against that fixture, and against a
    live run of the compiled shader source where it is built: IDENTICAL BYTES;
  * the CUDA kernels against the fixture: IDENTICAL BYTES; and against the CPU restatement on
    more images, both layouts, offsets, ragged edges, NaN / infinity: IDENTICAL BYTES;
  * the format itself, through BC1 / BC4 decoders written from the formats' definitions: constant
    blocks and blocks of 0 / 255 decode exactly, ramps and noise within the bounds the palette
    allows, and the encoder never does worse than its own starting endpoints.
One deviation, outside what the reference defines: the shader indexes its single-colour tables
with the unclamped 8-bit average of a block, so a block whose average lies outside [0, 1] reads
beyond them; both implementations here clamp the index.  The pinned images stay inside [0, 1].
"""
import os

import numpy as np
import pytest

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, synthetic  # noqa: E402


def decode_bc4(blocks: np.ndarray) -> np.ndarray:
    """[by][bx][8] bytes -> [by*4][bx*4] values in 0..255 (float64), per the format's definition."""
    by, bx, _ = blocks.shape
    out = np.zeros((by * 4, bx * 4))
    for y in range(by):
        for x in range(bx):
            block = blocks[y, x]
            a0, a1 = int(block[0]), int(block[1])
            bits = int.from_bytes(bytes(block[2:8]), "little")
            if a0 > a1:
                palette = [a0, a1] + [((7 - k) * a0 + k * a1) / 7 for k in range(1, 7)]
            else:
                palette = [a0, a1] + [((5 - k) * a0 + k * a1) / 5 for k in range(1, 5)] + [0, 255]
            for i in range(16):
                out[y * 4 + (i >> 2), x * 4 + (i & 3)] = palette[(bits >> (3 * i)) & 7]
    return out


def decode_bc1(blocks: np.ndarray):
    """[by][bx][8] bytes -> ([by*4][bx*4][3] colours in 0..1, [by*4][bx*4] alpha), per the format's definition."""
    by, bx, _ = blocks.shape
    rgb, alpha = np.zeros((by * 4, bx * 4, 3)), np.ones((by * 4, bx * 4))

    def expand(w):
        return np.array([((w >> 11) & 31) / 31.0, ((w >> 5) & 63) / 63.0, (w & 31) / 31.0])

    for y in range(by):
        for x in range(bx):
            block = blocks[y, x]
            c0, c1 = int(block[0]) | int(block[1]) << 8, int(block[2]) | int(block[3]) << 8
            bits = int.from_bytes(bytes(block[4:8]), "little")
            e0, e1 = expand(c0), expand(c1)
            if c0 > c1:
                palette = [(e0, 1), (e1, 1), ((2 * e0 + e1) / 3, 1), ((e0 + 2 * e1) / 3, 1)]
            else:
                palette = [(e0, 1), (e1, 1), ((e0 + e1) / 2, 1), (np.zeros(3), 0)]
            for i in range(16):
                colour, a = palette[(bits >> (2 * i)) & 3]
                rgb[y * 4 + (i >> 2), x * 4 + (i & 3)] = colour
                alpha[y * 4 + (i >> 2), x * 4 + (i & 3)] = a
    return rgb, alpha


def color_images():
    rng = np.random.default_rng(31)
    h, w = 24, 40
    smooth = np.zeros((h, w, 4))
    smooth[..., 0] = np.linspace(0.1, 0.9, w)[None, :]
    smooth[..., 1] = np.linspace(0.8, 0.2, h)[:, None]
    smooth[..., 2] = 0.5 + 0.3 * np.sin(np.arange(w) / 5.0)[None, :]
    smooth[..., 3] = 1.0
    noise = rng.uniform(-0.05, 1.05, (h, w, 4))
    cutout = smooth + rng.normal(0, 0.02, (h, w, 4))
    cutout[..., 3] = (rng.uniform(size=(h, w)) < 0.6).astype(np.float64)
    cutout[:8, :8, 3] = 0
    flat = np.zeros((h, w, 4))
    flat[...] = rng.integers(0, 256, (h // 4, w // 4, 4)).repeat(4, axis=0).repeat(4, axis=1) / 255.0
    flat[..., 3] = 1.0
    extremes = rng.integers(0, 2, (h, w, 4)).astype(np.float64)
    return {name: image.astype(np.float16) for name, image in
            (("smooth", smooth), ("noise", noise), ("cutout", cutout), ("flat", flat), ("extremes", extremes))}


def quantised(texels: np.ndarray) -> np.ndarray:
    """What the encoder sees: round-half-even of the saturated value times 255 (NaN as 0)."""
    return np.rint(np.clip(np.nan_to_num(texels.astype(np.float32), nan=0.0), 0, 1) * np.float32(255)).astype(np.float64)


def images():
    rng = np.random.default_rng(12)
    noise = rng.uniform(-0.1, 1.1, (24, 40, 3)).astype(np.float16)
    ramp = (np.linspace(0.1, 0.9, 40)[None, :, None] + np.linspace(0, 0.08, 24)[:, None, None] + np.zeros((24, 40, 3)))
    ramp[..., 1] = ramp[..., 1][:, ::-1] * 0.5
    ramp[..., 2] = np.where(rng.uniform(size=(24, 40)) < 0.3, rng.integers(0, 2, (24, 40)), ramp[..., 2])
    binary = rng.integers(0, 2, (24, 40, 3)).astype(np.float16)
    binary[:8, :8] = 0
    binary[8:16, :8] = 1
    special = noise.copy()
    special[::5, ::3, 0] = np.nan
    special[1::5, ::3, 0] = np.inf
    special[2::5, ::3, 0] = -np.inf
    return {"noise": noise, "ramp": ramp.astype(np.float16), "binary": binary, "special": special}


# ---------------------------------------------------------------------------------------------
# The pin: blocks produced by the reference's own shader source compiled for the CPU
# ---------------------------------------------------------------------------------------------

PIN_IMAGES = ["smooth", "noise", "cutout", "flat", "extremes", "gentle", "two_tone"]
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "block_compress_ref.npz")


@pytest.fixture(scope="module")
def pinned():
    return np.load(GOLDEN)


def _restated(oracle, block_format, texels, **window):
    """The CPU restatement on the channels the shader of `block_format` reads."""
    if block_format in (4, 5):
        window = {k: v for k, v in window.items() if k != "alpha_threshold"}
        return oracle.block_compress(texels, 0, block_format - 3, **window)
    return oracle.block_compress_color(texels, block_format, 0, 4, **window)


@pytest.mark.parametrize("name", PIN_IMAGES)
def test_restatement_reproduces_the_reference_shader_source(oracle, pinned, name):
    """oracle/ntc_oracle.c against what src/shaders/CompressBC1-5.hlsl computed on the same texels."""
    texels = pinned["image_" + name]
    for block_format in (1, 2, 3, 4, 5):
        assert np.array_equal(_restated(oracle, block_format, texels), pinned["bc%d_%s" % (block_format, name)]), block_format
    window = dict(src_left=3, src_top=5, width_in_blocks=13, height_in_blocks=8)
    assert np.array_equal(_restated(oracle, 1, texels, **window), pinned["bc1_window_" + name])
    assert np.array_equal(_restated(oracle, 4, texels, **window), pinned["bc4_window_" + name])
    assert np.array_equal(_restated(oracle, 1, texels, alpha_threshold=-1.0), pinned["bc1_opaque_" + name])


def test_live_reference_shader_source_on_more_images(oracle):
    """Where the compiled shader source is present: it and the restatement on fresh random images
    (inside [0, 1], the range the reference defines), every format."""
    if not oracle.reference_bc_available():
        pytest.skip("oracle/_ref/libntc_ref_bc.so is not built")
    rng = np.random.default_rng(77)
    for trial in range(6):
        h, w = int(rng.integers(4, 40)), int(rng.integers(4, 60))
        base = rng.random((h, w, 4))
        if trial % 2:
            base = np.clip(rng.random((1, 1, 4)) + 0.1 * rng.standard_normal((h, w, 4)), 0, 1)
        if trial % 3 == 0:
            base[..., 3] = rng.random((h, w)) < 0.5
        texels = base.astype(np.float16)
        for block_format in (1, 2, 3, 4, 5):
            rgba = np.zeros((h, w, 4), dtype=np.float32)
            count = {4: 1, 5: 2}.get(block_format, 4)
            rgba[..., :count] = texels[..., :count].astype(np.float32)
            assert np.array_equal(_restated(oracle, block_format, texels), oracle.reference_block_compress(block_format, rgba)), \
                (trial, block_format)


@pytest.mark.gpu
@pytest.mark.parametrize("name", PIN_IMAGES)
def test_kernels_reproduce_the_reference_shader_source(pinned, name):
    """The CUDA kernels against what src/shaders/CompressBC1-5.hlsl computed on the same texels."""
    import torch

    texels = torch.from_numpy(pinned["image_" + name]).cuda()
    for block_format in (1, 2, 3, 4, 5):
        channels = 0 if block_format in (4, 5) else 4
        blocks = binding.block_compress(texels, block_format, 0, num_channels=channels)
        assert np.array_equal(blocks.cpu().numpy(), pinned["bc%d_%s" % (block_format, name)]), block_format
    window = dict(src_left=3, src_top=5, width_in_blocks=13, height_in_blocks=8)
    assert np.array_equal(binding.block_compress(texels, 1, 0, num_channels=4, **window).cpu().numpy(), pinned["bc1_window_" + name])
    assert np.array_equal(binding.block_compress(texels, 4, 0, **window).cpu().numpy(), pinned["bc4_window_" + name])
    assert np.array_equal(binding.block_compress(texels, 1, 0, num_channels=4, alpha_threshold=-1.0).cpu().numpy(),
                          pinned["bc1_opaque_" + name])


# ---------------------------------------------------------------------------------------------
# CPU: the restated encoder against the format
# ---------------------------------------------------------------------------------------------

def test_constant_blocks_decode_exactly(oracle):
    values = np.arange(256, dtype=np.float32) / np.float32(255)
    image = np.repeat(np.repeat(values.reshape(16, 16), 4, axis=0), 4, axis=1)[..., None].astype(np.float32)
    # fp16 cannot hold every k/255 exactly; what counts is the 8-bit value the encoder derives
    texels = image.astype(np.float16)
    blocks = oracle.block_compress(texels, 0, 1)
    assert np.array_equal(decode_bc4(blocks), quantised(texels[..., 0]))


def test_blocks_of_extremes_decode_exactly(oracle):
    texels = images()["binary"]
    for channel in range(3):
        blocks = oracle.block_compress(texels, channel, 1)
        assert np.array_equal(decode_bc4(blocks)[:24, :40], quantised(texels[..., channel]))


def test_error_bounds(oracle):
    for name, bound in (("ramp", 0.0), ("noise", 0.0)):
        texels = images()[name]
        for channel in range(3):
            source = quantised(texels[..., channel])
            decoded = decode_bc4(oracle.block_compress(texels, channel, 1))[:24, :40]
            for y in range(0, 24, 4):
                for x in range(0, 40, 4):
                    tile, got = source[y:y + 4, x:x + 4], decoded[y:y + 4, x:x + 4]
                    spread = tile.max() - tile.min()
                    # eight palette entries over the spread: no texel farther than half a step, plus
                    # the rounding of the interpolants and the 1/34 inset of the starting endpoints
                    assert np.abs(tile - got).max() <= spread / 14 + spread / 34 + 1.0, (name, channel, y, x)


def test_ragged_edges_and_special_values(oracle):
    texels = images()["special"][:22, :37]
    blocks = oracle.block_compress(texels, 0, 1)
    assert blocks.shape == (6, 10, 8)
    padded = np.zeros((24, 40), np.float16)
    padded[:22, :37] = texels[..., 0]
    padded = np.nan_to_num(padded.astype(np.float32), nan=0.0, posinf=1.0, neginf=0.0).astype(np.float16)
    expected = oracle.block_compress(padded[..., None], 0, 1)
    assert np.array_equal(blocks, expected)


def test_bc5_is_two_bc4_blocks(oracle):
    texels = images()["noise"]
    bc5 = oracle.block_compress(texels, 1, 2)
    assert np.array_equal(bc5[..., :8], oracle.block_compress(texels, 1, 1))
    assert np.array_equal(bc5[..., 8:], oracle.block_compress(texels, 2, 1))


def test_source_window(oracle):
    texels = images()["ramp"]
    window = oracle.block_compress(texels, 0, 1, src_left=8, src_top=4, width_in_blocks=3, height_in_blocks=2)
    assert np.array_equal(window, oracle.block_compress(texels, 0, 1)[1:3, 2:5])


def test_match_tables_are_the_reference_ones(oracle):
    """The single-colour match tables are generated, not stored; their digests are those of the
    tables in BlockCompressCommon.hlsli:40-80 (taken where the reference's sources are at hand)."""
    import hashlib

    assert hashlib.sha256(oracle.color_match_table(5).astype("<u2").tobytes()).hexdigest() == \
        "51207020db025e90c3a7b985b0b78d4eff317eb74b68e21329fff7db3f22d196"
    assert hashlib.sha256(oracle.color_match_table(6).astype("<u2").tobytes()).hexdigest() == \
        "db2ca3aa978ed0f5b3aa05a2e4efb53f44d6741014dd578498f4e50a05a0576c"


def test_bc1_flat_blocks_and_error_bounds(oracle):
    images = color_images()
    flat = images["flat"]
    rgb, alpha = decode_bc1(oracle.block_compress_color(flat, 1, 0, 4))
    assert (alpha == 1).all()
    # one colour per block: the match tables land within 2/255 per component (3 % rule included)
    assert np.abs(rgb - flat[..., :3].astype(np.float64)).max() <= 2.5 / 255
    for name, bound in (("smooth", 33.0), ("noise", 12.0)):
        source = np.clip(images[name][..., :3].astype(np.float64), 0, 1)
        rgb, alpha = decode_bc1(oracle.block_compress_color(images[name], 1, 0, 3))
        assert (alpha == 1).all(), name
        psnr = -10 * np.log10(np.mean((rgb - source) ** 2))
        assert psnr >= bound, (name, psnr)


def test_bc1_transparency(oracle):
    image = color_images()["cutout"]
    blocks = oracle.block_compress_color(image, 1, 0, 4)
    rgb, alpha = decode_bc1(blocks)
    source_alpha = image[..., 3].astype(np.float64)
    # a fully transparent block is the reference's fixed pattern
    assert (blocks[0, 0] == np.array([0, 0, 0, 0, 255, 255, 255, 255], np.uint8)).all()
    # where the encoder chose the transparent mode, exactly the transparent texels carry index 3
    by, bx = blocks.shape[:2]
    chosen = 0
    for y in range(by):
        for x in range(bx):
            c0 = int(blocks[y, x, 0]) | int(blocks[y, x, 1]) << 8
            c1 = int(blocks[y, x, 2]) | int(blocks[y, x, 3]) << 8
            tile = source_alpha[y * 4:y * 4 + 4, x * 4:x * 4 + 4]
            if c0 <= c1 and 0 < (tile == 0).sum() < 16:
                chosen += 1
                assert np.array_equal(alpha[y * 4:y * 4 + 4, x * 4:x * 4 + 4] == 0, tile == 0), (y, x)
    assert chosen >= 10
    opaque = source_alpha == 1
    error = np.abs(rgb - np.clip(image[..., :3].astype(np.float64), 0, 1))[opaque & (alpha == 1)]
    assert np.sqrt(np.mean(error ** 2)) <= 0.05


def test_bc2_and_bc3_share_the_colour_block(oracle):
    image = color_images()["cutout"]
    bc2, bc3 = oracle.block_compress_color(image, 2, 0, 4), oracle.block_compress_color(image, 3, 0, 4)
    assert np.array_equal(bc2[..., 8:], bc3[..., 8:])
    # BC2 alpha: 4 bits per texel, round(15 a); BC3 alpha: the BC4 block of the alpha channel
    nibbles = np.rint(np.clip(image[..., 3].astype(np.float32), 0, 1) * np.float32(15)).astype(np.uint8)
    for y in range(bc2.shape[0]):
        for x in range(bc2.shape[1]):
            bits = int.from_bytes(bytes(bc2[y, x, :8]), "little")
            got = np.array([(bits >> (4 * i)) & 15 for i in range(16)]).reshape(4, 4)
            assert np.array_equal(got, nibbles[y * 4:y * 4 + 4, x * 4:x * 4 + 4])
    assert np.array_equal(bc3[..., :8], oracle.block_compress(image, 3, 1))
    # the colour block ignores alpha: the same as BC1 of the opaque image whenever that is a four-colour block
    opaque = image.copy()
    opaque[..., 3] = 1
    bc1 = oracle.block_compress_color(opaque, 1, 0, 4)
    c0 = bc1[..., 0].astype(np.int32) | bc1[..., 1].astype(np.int32) << 8
    c1 = bc1[..., 2].astype(np.int32) | bc1[..., 3].astype(np.int32) << 8
    four = c0 > c1
    assert four.sum() > 30 and np.array_equal(bc1[four], bc3[..., 8:][four])


def test_arguments_are_checked():
    lib = binding.lib()
    assert lib.ntcb_block_compress(None, None) == -1
    params = binding.BlockCompressParams()
    params.deviceMip, params.deviceBlocks = 4096, 8192  # never dereferenced: the checks come first
    params.layout, params.width, params.height, params.channels = binding.LAYOUT_INTERLEAVED, 8, 8, 2
    params.widthInBlocks, params.heightInBlocks, params.rowPitch = 2, 2, 16
    params.format = 6
    assert lib.ntcb_block_compress(params, None) == -5  # BC6: a valid format of the reference, not built here
    params.format, params.deviceModeBuffer = binding.BLOCK_FORMAT_BC4, 4096
    assert lib.ntcb_block_compress(params, None) == -1 and b"Mode buffer" in lib.ntcb_last_error()
    params.format, params.rowPitch, params.numChannels = binding.BLOCK_FORMAT_BC7, 32, 2
    assert lib.ntcb_block_compress(params, None) == -1 and b"modeMapWidthInBlocks" in lib.ntcb_last_error()
    params.modeMapWidthInBlocks = params.modeMapHeightInBlocks = 2
    params.deviceModeBuffer = 4097
    assert lib.ntcb_block_compress(params, None) == -1 and b"aligned" in lib.ntcb_last_error()
    params.deviceModeBuffer, params.rowPitch, params.numChannels = None, 16, 0
    params.format, params.numChannels = binding.BLOCK_FORMAT_BC1, 5
    assert lib.ntcb_block_compress(params, None) == -9 and b"numChannels" in lib.ntcb_last_error()
    params.numChannels = 0
    params.format = 9
    assert lib.ntcb_block_compress(params, None) == -9
    params.format, params.firstChannel = binding.BLOCK_FORMAT_BC5, 1
    assert lib.ntcb_block_compress(params, None) == -9 and b"firstChannel" in lib.ntcb_last_error()
    params.firstChannel, params.rowPitch = 0, 24
    assert lib.ntcb_block_compress(params, None) == -1 and b"rowPitch" in lib.ntcb_last_error()
    params.format, params.rowPitch, params.srcLeft = binding.BLOCK_FORMAT_BC4, 16, -4
    assert lib.ntcb_block_compress(params, None) == -9 and b"srcLeft" in lib.ntcb_last_error()


# ---------------------------------------------------------------------------------------------
# BC7: mode buffers (host), then the kernels against the reference's shader source
# ---------------------------------------------------------------------------------------------

def _entries_of(mode_buffer: np.ndarray, count: int) -> np.ndarray:
    """The 9-bit entries of a mode buffer, unpacked in numpy."""
    bits = np.unpackbits(np.asarray(mode_buffer, dtype=np.uint8), bitorder="little")[:count * 9].reshape(count, 9)
    return (bits.astype(np.uint32) << np.arange(9, dtype=np.uint32)).sum(axis=1)


@pytest.mark.parametrize("name", PIN_IMAGES)
def test_bc7_mode_buffer_is_what_the_reference_extracts(pinned, name):
    """ntcb_make_bc7_mode_buffer against ntc::MakeBC7ModeBuffer on the blocks of the reference's full
    search, and on the blocks its one-mode-per-block path wrote: those carry the mode and partition the
    mode buffer asked for, so extracting them gives the mode buffer back."""
    blocks = pinned["bc7_opaque_" + name]
    assert np.array_equal(binding.make_bc7_mode_buffer(blocks), pinned["bc7_extracted_" + name])
    assert binding.bc7_mode_buffer_size(blocks.shape[1], blocks.shape[0]) == pinned["bc7_extracted_" + name].nbytes
    asked = _entries_of(pinned["bc7_modebuffer_" + name], blocks.shape[0] * blocks.shape[1])
    got = _entries_of(binding.make_bc7_mode_buffer(pinned["bc7_modes_" + name]), asked.size)
    stored = asked != 0
    assert stored.sum() > 100 and np.array_equal(got[stored], asked[stored])
    # blocks without an entry: the shader's four coloured squares
    missing = pinned["bc7_modes_" + name].reshape(-1, 16)[~stored]
    assert len(missing) and all(bytes(b) == bytes.fromhex("0400f80000f001001f00f03f00009e1f") for b in missing)


def test_bc7_mode_buffer_on_random_blocks_and_its_checks(oracle):
    rng = np.random.default_rng(3)
    blocks = rng.integers(0, 256, (9, 13, 16), dtype=np.uint8)
    blocks[0, 0, :4] = 0            # no mode bit in the first word: read as mode 7
    blocks[0, 1, :4] = (1, 0, 0, 0)  # mode 0, partition 0: stored as 0x1bf
    ours = binding.make_bc7_mode_buffer(blocks)
    entries = _entries_of(ours, 9 * 13)
    assert entries[0] >> 6 == 7 and entries[1] == 0x1BF and ours.nbytes == ((9 * 13 * 9 + 31) // 32) * 4
    if oracle.reference_available():
        assert np.array_equal(ours, oracle.reference_make_bc7_mode_buffer(blocks))
    lib = binding.lib()
    out = np.zeros(ours.nbytes, dtype=np.uint8)
    call = lambda *a: lib.ntcb_make_bc7_mode_buffer(*a)  # noqa: E731
    assert call(13, 9, None, blocks.nbytes, 13 * 16, out.ctypes.data, out.nbytes) == -1
    assert call(13, 9, blocks.ctypes.data, blocks.nbytes, 13 * 16, None, out.nbytes) == -1
    assert call(13, 9, blocks.ctypes.data, blocks.nbytes, 13 * 16 - 8, out.ctypes.data, out.nbytes) == -1 and b"rowPitch" in lib.ntcb_last_error()
    assert call(13, 9, blocks.ctypes.data, blocks.nbytes - 1, 13 * 16, out.ctypes.data, out.nbytes) == -1 and b"block data" in lib.ntcb_last_error()
    assert call(13, 9, blocks.ctypes.data, blocks.nbytes, 13 * 16, out.ctypes.data, out.nbytes - 4) == -1 and b"mode buffer" in lib.ntcb_last_error()
    assert call(0, 9, blocks.ctypes.data, blocks.nbytes, 13 * 16, out.ctypes.data, out.nbytes) == -9


@pytest.mark.gpu
@pytest.mark.parametrize("name", PIN_IMAGES)
def test_bc7_kernels_reproduce_the_reference_shader_source(pinned, name):
    """Both BC7 kernels against what src/shaders/CompressBC7.hlsl computed on the same texels: the full
    search (every mode wins somewhere in these images) and the mode-buffer path (every mode, seeded
    partitions, missing entries, a window into a larger mode map)."""
    import torch

    texels = torch.from_numpy(pinned["image_" + name]).cuda()
    assert np.array_equal(binding.block_compress(texels, 7).cpu().numpy(), pinned["bc7_" + name])
    assert np.array_equal(binding.block_compress(texels, 7, num_channels=3).cpu().numpy(), pinned["bc7_opaque_" + name])
    modes = torch.from_numpy(pinned["bc7_modebuffer_" + name]).cuda()
    assert np.array_equal(binding.block_compress(texels, 7, mode_buffer=modes).cpu().numpy(), pinned["bc7_modes_" + name])
    blocks_y, blocks_x = pinned["bc7_" + name].shape[:2]
    wide = torch.from_numpy(pinned["bc7_widemodebuffer_" + name]).cuda()
    window = binding.block_compress(texels, 7, mode_buffer=wide, mode_map_size=(blocks_x + 5, blocks_y + 3), mode_map_offset=(4, 2),
                                    src_left=3, src_top=5, width_in_blocks=blocks_x, height_in_blocks=blocks_y - 1)
    assert np.array_equal(window.cpu().numpy(), pinned["bc7_window_" + name])


@pytest.mark.gpu
def test_bc7_kernels_against_the_live_shader_source_on_larger_images(oracle):
    """Images of several CTAs (a CTA covers 32 x 8 blocks), both layouts, channels taken from the middle of a
    wider mip, against the reference's shader source run on the CPU on the same texels."""
    import sys

    import torch

    sys.path.insert(0, os.path.dirname(GOLDEN))
    from make_golden_block_compress import bc7_mode_entries, pack_mode_entries

    if not oracle.reference_bc_available():
        pytest.skip("oracle/_ref/libntc_ref_bc.so is not built")
    rng = np.random.default_rng(11)
    for trial, (h, w, channels, first) in enumerate([(70, 150, 4, 0), (37, 261, 6, 1), (132, 64, 8, 2)]):
        base = np.clip(rng.random((1, 1, channels)) + (0.05 + 0.2 * trial) * rng.standard_normal((h, w, channels)), 0, 1)
        base[..., first + 3] = np.where(rng.random((h, w)) < 0.7, 1.0, rng.random((h, w)))
        texels = base.astype(np.float16)
        rgba = np.ascontiguousarray(texels[..., first:first + 4].astype(np.float32))
        bh, bw = (h + 3) // 4, (w + 3) // 4
        modes = pack_mode_entries(bc7_mode_entries(bh, bw, seed=trial))
        want_full = oracle.reference_block_compress_bc7(rgba)
        want_modes = oracle.reference_block_compress_bc7(rgba, mode_buffer=modes)
        device_modes = torch.from_numpy(modes).cuda()
        for layout in (binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS):
            if layout == binding.LAYOUT_PLANAR_PAIRS:
                source = torch.from_numpy(np.ascontiguousarray(
                    texels.reshape(h, w, channels // 2, 2).transpose(0, 2, 1, 3))).cuda()
            else:
                source = torch.from_numpy(texels).cuda()
            common = dict(first_channel=first, layout=layout, width=w, height=h, channels=channels, num_channels=4)
            assert np.array_equal(binding.block_compress(source, 7, **common).cpu().numpy(), want_full), (trial, layout)
            assert np.array_equal(binding.block_compress(source, 7, mode_buffer=device_modes, **common).cpu().numpy(), want_modes), \
                (trial, layout)


# ---------------------------------------------------------------------------------------------
# GPU: the kernel against the restatement
# ---------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("name", ["noise", "ramp", "binary", "special"])
def test_kernel_matches_the_restated_encoder(oracle, name):
    import torch

    texels = images()[name]
    device = torch.from_numpy(texels).cuda()
    for channel in range(3):
        got = binding.block_compress(device, binding.BLOCK_FORMAT_BC4, channel).cpu().numpy()
        assert np.array_equal(got, oracle.block_compress(texels, channel, 1)), (name, channel)
    got = binding.block_compress(device, binding.BLOCK_FORMAT_BC5, 1).cpu().numpy()
    assert np.array_equal(got, oracle.block_compress(texels, 1, 2)), name


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["smooth", "noise", "cutout", "flat", "extremes"])
def test_colour_kernels_match_the_restated_encoders(oracle, name):
    import torch

    image = color_images()[name]
    device = torch.from_numpy(image).cuda()
    for block_format in (binding.BLOCK_FORMAT_BC1, binding.BLOCK_FORMAT_BC2, binding.BLOCK_FORMAT_BC3):
        for channels in (3, 4):
            got = binding.block_compress(device, block_format, 0, num_channels=channels).cpu().numpy()
            expected = oracle.block_compress_color(image, block_format, 0, channels)
            assert np.array_equal(got, expected), (name, block_format, channels, int((got != expected).any(axis=-1).sum()))
    ragged = image[:22, :37]
    got = binding.block_compress(torch.from_numpy(np.ascontiguousarray(ragged)).cuda(), binding.BLOCK_FORMAT_BC1, 0, num_channels=4,
                                 alpha_threshold=0.5).cpu().numpy()
    assert np.array_equal(got, oracle.block_compress_color(ragged, 1, 0, 4, alpha_threshold=0.5))


@pytest.mark.gpu
def test_colour_kernels_with_odd_channel_offsets_and_the_planar_layout(oracle):
    """Channel pairs are read as 32-bit words when the first channel and the channel count are even;
    every other combination takes single-channel reads."""
    import torch

    rng = np.random.default_rng(8)
    for channels in (5, 6):
        image = rng.uniform(0, 1, (26, 45, channels)).astype(np.float16)
        image[..., -1] = (rng.uniform(size=(26, 45)) < 0.7)
        device = torch.from_numpy(image).cuda()
        for first, count in ((0, 4), (1, 4), (2, 3), (1, 3), (channels - 1, 1), (2, 2)):
            if first + count > channels:
                continue
            for block_format in (binding.BLOCK_FORMAT_BC1, binding.BLOCK_FORMAT_BC3):
                got = binding.block_compress(device, block_format, first, num_channels=count).cpu().numpy()
                assert np.array_equal(got, oracle.block_compress_color(image, block_format, first, count)), (channels, first, count)
    image = rng.uniform(0, 1, (26, 45, 6)).astype(np.float16)
    h, w, c = image.shape
    planar = np.zeros(h * w * c, np.float16)
    for ch in range(c):
        for y in range(h):
            planar[y * w * c + (ch & ~1) * w + (ch & 1):y * w * c + (ch & ~1) * w + 2 * w:2] = image[y, :, ch]
    for first, count in ((0, 4), (2, 4), (1, 3)):
        got = binding.block_compress(torch.from_numpy(planar).cuda(), binding.BLOCK_FORMAT_BC1, first, layout=binding.LAYOUT_PLANAR_PAIRS,
                                     width=w, height=h, channels=c, num_channels=count).cpu().numpy()
        assert np.array_equal(got, oracle.block_compress_color(image, 1, first, count)), (first, count)


@pytest.mark.gpu
def test_kernel_on_ragged_images_windows_and_the_planar_layout(oracle):
    import torch

    rng = np.random.default_rng(5)
    texels = rng.uniform(0, 1, (37, 61, 4)).astype(np.float16) ** 2
    device = torch.from_numpy(texels).cuda()
    assert np.array_equal(binding.block_compress(device, binding.BLOCK_FORMAT_BC5, 2).cpu().numpy(),
                          oracle.block_compress(texels, 2, 2))
    window = binding.block_compress(device, binding.BLOCK_FORMAT_BC4, 3, src_left=12, src_top=8, width_in_blocks=5,
                                    height_in_blocks=4).cpu().numpy()
    assert np.array_equal(window, oracle.block_compress(texels, 3, 1, 12, 8, 5, 4))
    # planar pairs: half index = y*W*C + (c & ~1)*W + 2*x + (c & 1)
    h, w, c = texels.shape
    planar = np.zeros(h * w * c, np.float16)
    for ch in range(c):
        for y in range(h):
            planar[y * w * c + (ch & ~1) * w + (ch & 1):y * w * c + (ch & ~1) * w + 2 * w:2] = texels[y, :, ch]
    got = binding.block_compress(torch.from_numpy(planar).cuda(), binding.BLOCK_FORMAT_BC5, 2, layout=binding.LAYOUT_PLANAR_PAIRS,
                                 width=w, height=h, channels=c).cpu().numpy()
    assert np.array_equal(got, oracle.block_compress(texels, 2, 2))


@pytest.mark.gpu
def test_decoded_texture_set_to_bc5(oracle):
    """Decode on load, then block-compress: every mip of a decoded set, two channels as BC5, from the
    decode kernel's own output buffer; checked against the restatement and through the BC decoder."""
    import torch

    data = synthetic.make_texture_set(synthetic.TextureSetSpec(128, 64, 6, 0, 4, 12, seed=2, network="unit"))
    resident = binding.ResidentTextureSet.from_synthetic(data)
    resident.decode(False)
    torch.cuda.synchronize()
    resident.check_status()
    geo = data.geometry
    for mip in range(geo.mips):
        view = resident.mip_view(mip)
        texels = resident.mip_numpy(mip)
        blocks = binding.block_compress(view, binding.BLOCK_FORMAT_BC5, 2).cpu().numpy()
        assert np.array_equal(blocks, oracle.block_compress(texels, 2, 2)), mip
        h, w = texels.shape[:2]
        for k in range(2):
            source = quantised(texels[..., 2 + k])
            decoded = decode_bc4(np.ascontiguousarray(blocks[..., 8 * k:8 * k + 8]))[:h, :w]
            mse = np.mean((decoded - source) ** 2)
            assert mse <= 40.0, (mip, k, mse)  # > 32 dB on noise-like synthetic texels


@pytest.mark.gpu
def test_texture_set_block_compress(oracle):
    """The texture-set level call: NTCB_ERR_INVALID_STATE before Decompress, then the same blocks as
    the restated encoder makes of the texels ReadChannels hands back."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(72, 40, 6, 0, 2, 8, seed=4, network="unit"))
    with binding.Context() as context:
        texture_set = context.create_texture_set(data.container)
        with pytest.raises(binding.NtcbError) as error:
            texture_set.block_compress(0, binding.BLOCK_FORMAT_BC4, 1)
        assert error.value.code == -8
        texture_set.decompress(False)
        for mip in (0, 2):
            texels = texture_set.read_mip(mip)
            assert np.array_equal(texture_set.block_compress(mip, binding.BLOCK_FORMAT_BC4, 1).cpu().numpy(),
                                  oracle.block_compress(texels, 1, 1))
            assert np.array_equal(texture_set.block_compress(mip, binding.BLOCK_FORMAT_BC3, 0, 4).cpu().numpy(),
                                  oracle.block_compress_color(texels, 3, 0, 4))
        texture_set.close()


@pytest.mark.gpu
def test_transcode_every_texture_by_its_header(oracle):
    """The SDK's "decompress on load, then BCn" flow driven by the container's own texture headers:
    each texture's channel range is encoded in the block format its header names."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 32, 6, 0, 2, 8, seed=6, network="unit"))
    data.textures = [
        {"name": "Albedo", "firstChannel": 0, "numChannels": 3, "rgbColorSpace": "sRGB", "bcFormat": "BC1"},
        {"name": "Normal", "firstChannel": 3, "numChannels": 2, "bcFormat": "BC5"},
        {"name": "Roughness", "firstChannel": 5, "numChannels": 1, "bcFormat": "BC4"},
    ]
    with binding.Context() as context:
        texture_set = context.create_texture_set(data.container)
        headers = texture_set.textures()
        assert [h["name"] for h in headers] == ["Albedo", "Normal", "Roughness"]
        texture_set.decompress(False)
        texels = texture_set.read_mip(0)
        for header in headers:
            block_format, first, count = header["blockCompressedFormat"], header["firstChannel"], header["numChannels"]
            blocks = texture_set.block_compress(0, block_format, first, count if block_format <= 3 else 0).cpu().numpy()
            if block_format <= 3:
                expected = oracle.block_compress_color(texels, block_format, first, count)
            else:
                expected = oracle.block_compress(texels, first, count)
            assert np.array_equal(blocks, expected), header["name"]
        texture_set.close()


def _set_with_bc7_textures(mode_buffers=None):
    """A 72 x 40, 8-channel set with a full mip chain with an RGBA texture and an RGB texture, both headed for BC7."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(72, 40, 8, 0, 2, 8, seed=12, network="unit"))
    data.textures = [
        {"name": "Albedo", "firstChannel": 0, "numChannels": 4, "rgbColorSpace": "sRGB", "bcFormat": "BC7"},
        {"name": "Emissive", "firstChannel": 5, "numChannels": 3, "bcFormat": "BC7"},
    ]
    for (texture, mip), bits in (mode_buffers or {}).items():
        data.textures[texture].setdefault("bcModeBuffers", []).append({"mipLevel": mip, "data": bits.tobytes()})
    return data


def test_stored_bc7_mode_buffers_are_found_where_the_reference_finds_them(oracle):
    """The container's "bcModeBuffers": the loader reports the byte range the Python writer gave them, and the
    reference's own metadata loader reports the same range (no GPU needed for either)."""
    rng = np.random.default_rng(8)
    buffers = {(0, 0): rng.integers(0, 256, binding.bc7_mode_buffer_size(18, 10), dtype=np.uint8),
               (0, 2): rng.integers(0, 256, binding.bc7_mode_buffer_size(5, 3), dtype=np.uint8),
               (1, 1): rng.integers(0, 256, binding.bc7_mode_buffer_size(9, 5), dtype=np.uint8)}
    container = _set_with_bc7_textures(buffers).container
    for texture in (0, 1):
        for mip in range(3):
            offset, stored, compressed = binding.probe_bc7_mode_buffer(container, texture, mip)
            bits = buffers.get((texture, mip))
            if bits is None:
                assert (offset, stored, compressed) == (0, 0, False)
            else:
                assert stored == bits.nbytes and not compressed and container[offset:offset + stored] == bits.tobytes()
            if oracle.reference_available():
                assert oracle.reference_mode_buffer_footprint(container, texture, mip) == (offset, stored, 0)
    lib = binding.lib()
    assert lib.ntcb_probe_container_bc7_mode_buffer(container, len(container), 2, 0, None, None, None) == -9
    assert lib.ntcb_probe_container_bc7_mode_buffer(container, len(container), 0, 99, None, None, None) == -9
    # an entry that names a view the file does not have
    broken = _set_with_bc7_textures()
    broken.textures[0]["bcModeBuffers"] = [{"mipLevel": 0, "view": 999}]
    assert lib.ntcb_probe_container_bc7_mode_buffer(broken.container, len(broken.container), 0, 0, None, None, None) == -3
    assert b"BC7 mode buffer" in lib.ntcb_last_error()


@pytest.mark.gpu
def test_transcode_to_bc7_from_the_mode_buffers_a_set_carries(oracle):
    """Decompress on load, then BC7 by the stored mode bitmap (BlockCompressionModeBufferSource::TextureSet):
    an offline pass (here: this library's full search) chooses the modes, the set carries them, and the
    run-time pass encodes every block in its mode.  Checked against the explicit-mode-buffer call, against the
    reference's shader source where it is built, and for the modes the blocks end up with."""
    import torch

    plain = _set_with_bc7_textures()
    with binding.Context() as context:
        offline = context.create_texture_set(plain.container)
        offline.decompress(False)
        searched = {(t, m): offline.block_compress_texture(t, m).cpu().numpy() for t in (0, 1) for m in (0, 1)}
        texels = {m: offline.read_mip(m) for m in (0, 1)}
        assert offline.bc7_mode_buffer(0, 0) is None
        # the same through MakeAndStoreBC7ModeBuffer on the loaded set
        offline.make_and_store_bc7_mode_buffer(0, 0, searched[(0, 0)])
        stored = offline.bc7_mode_buffer(0, 0)
        assert np.array_equal(stored, binding.make_bc7_mode_buffer(searched[(0, 0)]))
        from_stored = offline.block_compress_texture(0, 0).cpu().numpy()
        with pytest.raises(binding.NtcbError):
            offline.make_and_store_bc7_mode_buffer(0, 1, searched[(0, 0)])  # blocks of another mip's size
        offline.close()

        buffers = {key: binding.make_bc7_mode_buffer(blocks) for key, blocks in searched.items()}
        shipped = context.create_texture_set(_set_with_bc7_textures(buffers).container)
        shipped.decompress(False)
        for (texture, mip), bits in buffers.items():
            assert np.array_equal(shipped.bc7_mode_buffer(texture, mip), bits)
            blocks = shipped.block_compress_texture(texture, mip).cpu().numpy()
            header = shipped.textures()[texture]
            first, count = header["firstChannel"], header["numChannels"]
            mip_texels = torch.from_numpy(texels[mip]).cuda()
            explicit = binding.block_compress(mip_texels, 7, first, num_channels=count, mode_buffer=torch.from_numpy(bits).cuda())
            assert np.array_equal(blocks, explicit.cpu().numpy()), (texture, mip)
            assert np.array_equal(binding.make_bc7_mode_buffer(blocks), bits), (texture, mip)  # every block in its mode
            if (texture, mip) == (0, 0):
                assert np.array_equal(blocks, from_stored)
            if oracle.reference_bc_available():
                rgba = np.zeros(texels[mip].shape[:2] + (4,), dtype=np.float32)
                rgba[..., 3] = 1.0
                rgba[..., :count] = texels[mip][..., first:first + count].astype(np.float32)
                assert np.array_equal(blocks, oracle.reference_block_compress_bc7(rgba, mode_buffer=bits)), (texture, mip)
                assert np.array_equal(searched[(texture, mip)], oracle.reference_block_compress_bc7(rgba)), (texture, mip)
        assert shipped.bc7_mode_buffer(1, 2) is None  # no bitmap for that mip: the full search runs
        assert shipped.block_compress_texture(1, 2).shape == (3, 5, 16)
        shipped.close()


@pytest.mark.gpu
def test_flat_and_binary_blocks_decode_exactly_at_full_size():
    """Size-independent property on a 4096 x 4096 channel (1 M blocks): blocks of one value and blocks
    holding only 0 and 1 decode, through the format's definition, to exactly the encoder's 8-bit values."""
    import torch

    side = 4096
    blocks_per_side = side // 4
    generator = torch.Generator(device="cuda").manual_seed(5)
    flat = torch.randint(0, 256, (blocks_per_side, blocks_per_side), device="cuda", generator=generator)
    flat = flat.repeat_interleave(4, 0).repeat_interleave(4, 1).to(torch.float32) / 255.0
    binary = torch.randint(0, 2, (side, side), device="cuda", generator=generator).to(torch.float32)
    chooser = torch.randint(0, 2, (blocks_per_side, blocks_per_side), device="cuda", generator=generator)
    chooser = chooser.repeat_interleave(4, 0).repeat_interleave(4, 1).bool()
    image = torch.where(chooser, flat, binary).to(torch.float16)
    texels = torch.stack([image, image.flip(0)], dim=-1).contiguous()
    blocks = binding.block_compress(texels, binding.BLOCK_FORMAT_BC5, 0)

    def decode(block_bytes):
        wide = block_bytes.to(torch.int64)
        a0, a1 = wide[..., 0], wide[..., 1]
        bits = sum(wide[..., 2 + k] << (8 * k) for k in range(6))
        eight = a0 > a1
        palette = [a0.double(), a1.double()]
        for k in range(1, 7):
            interpolant8 = ((7 - k) * a0 + k * a1).double() / 7
            interpolant6 = ((5 - k) * a0 + k * a1).double() / 5 if k <= 4 else torch.full_like(interpolant8, 0.0 if k == 5 else 255.0)
            palette.append(torch.where(eight, interpolant8, interpolant6))
        palette = torch.stack(palette, dim=-1)                                    # [by][bx][8]
        indices = torch.stack([(bits >> (3 * i)) & 7 for i in range(16)], dim=-1)  # [by][bx][16]
        values = torch.gather(palette, -1, indices)                               # [by][bx][16]
        by, bx = values.shape[:2]
        return values.view(by, bx, 4, 4).permute(0, 2, 1, 3).reshape(by * 4, bx * 4)

    for channel in range(2):
        expected = torch.round(texels[..., channel].to(torch.float32).clamp(0, 1) * 255.0).double()
        assert torch.equal(decode(blocks[..., 8 * channel:8 * channel + 8]), expected), channel
