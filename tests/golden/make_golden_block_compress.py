#!/usr/bin/env python
"""Generates tests/golden/block_compress_ref.npz: BC1 - BC5 and BC7 blocks produced by the REFERENCE'S OWN
shader source (src/shaders/CompressBC1-5.hlsl, CompressBC7.hlsl, BlockCompressCommon.hlsli) compiled for the CPU by
oracle/build_ref.sh (oracle/_ref/libntc_ref_bc.so), over small seeded images.  Run where the
reference sources are present; the fixture then pins the CPU restatement and the CUDA kernels
wherever the tests run.

    python tests/golden/make_golden_block_compress.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import oracle_py  # noqa: E402


def pin_images():
    """fp16 RGBA images inside [0, 1] (the shader's single-colour path indexes its tables with the
    unclamped 8-bit average, so values outside that range are outside what the reference defines)."""
    rng = np.random.default_rng(2024)
    h, w = 36, 52
    y, x = np.mgrid[0:h, 0:w]
    smooth = np.stack([x / w, y / h, (x + y) / (w + h), 0.5 + 0.5 * np.sin(x / 7.0)], -1)
    noise = rng.random((h, w, 4))
    cutout = np.clip(smooth + rng.normal(0, 0.02, (h, w, 4)), 0, 1)
    cutout[..., 3] = (rng.random((h, w)) < 0.6) * rng.random((h, w))
    cutout[:8, :8, 3] = 0
    flat = (rng.integers(0, 256, (h // 4, w // 4, 4)).repeat(4, axis=0).repeat(4, axis=1) / 255.0)
    extremes = rng.integers(0, 2, (h, w, 4)).astype(np.float64)
    gentle = np.clip(0.5 + 0.04 * rng.standard_normal((h, w, 4)), 0, 1)
    two_tone = np.where(rng.random((h, w, 1)) < 0.5, rng.random((1, 1, 4)), rng.random((1, 1, 4))) + np.zeros((h, w, 4))
    return {name: image.astype(np.float16) for name, image in
            (("smooth", smooth), ("noise", noise), ("cutout", cutout), ("flat", flat), ("extremes", extremes),
             ("gentle", gentle), ("two_tone", two_tone))}


def rgba_for(block_format: int, texels: np.ndarray) -> np.ndarray:
    """The shader's input texture for a format: BC4 reads .r, BC5 .r and .g, the colour formats all four."""
    rgba = np.zeros(texels.shape[:2] + (4,), dtype=np.float32)
    count = {4: 1, 5: 2}.get(block_format, 4)
    rgba[..., :count] = texels[..., :count].astype(np.float32)
    return rgba


PARTITION_MASK = (15, 63, 63, 63, 7, 3, 0, 63)  # what the partition field of each BC7 mode can hold


def bc7_mode_entries(blocks_y: int, blocks_x: int, seed: int) -> np.ndarray:
    """A mode-buffer entry (mode << 6 | partition) per block: every mode, random partitions (for modes 4
    and 5: rotation and index selector), a few blocks without an entry (0) and mode 0, partition 0."""
    rng = np.random.default_rng(seed)
    mode = rng.integers(0, 8, (blocks_y, blocks_x))
    partition = np.array([[rng.integers(0, PARTITION_MASK[m] + 1) for m in row] for row in mode])
    entries = (mode << 6 | partition).astype(np.uint32)
    entries[0, 0] = 0x1BF         # how mode 0, partition 0 is stored
    entries[1, 1::5] = 0          # nothing stored: the shader writes its four-squares block
    return entries


def pack_mode_entries(entries: np.ndarray) -> np.ndarray:
    """9 bits per entry, entry k at bit 9 k, little-endian, rounded up to whole 32-bit words."""
    flat = entries.ravel()
    bits = np.zeros(((flat.size * 9 + 31) // 32) * 4, dtype=np.uint8)
    for k, entry in enumerate(int(e) for e in flat):
        byte, shift = (k * 9) // 8, (k * 9) % 8
        bits[byte] |= (entry << shift) & 0xFF
        bits[byte + 1] |= (entry >> (8 - shift)) & 0xFF
    return bits


def main() -> int:
    if not oracle_py.reference_bc_available():
        print("oracle/_ref/libntc_ref_bc.so is not built (oracle/build_ref.sh)", file=sys.stderr)
        return 1
    arrays = {}
    for name, texels in pin_images().items():
        arrays["image_" + name] = texels
        for block_format in (1, 2, 3, 4, 5):
            arrays["bc%d_%s" % (block_format, name)] = oracle_py.reference_block_compress(block_format, rgba_for(block_format, texels))
        # a source window with an offset, blocks hanging over the right and bottom edges
        arrays["bc1_window_" + name] = oracle_py.reference_block_compress(1, rgba_for(1, texels), src_left=3, src_top=5,
                                                                          width_in_blocks=13, height_in_blocks=8)
        arrays["bc4_window_" + name] = oracle_py.reference_block_compress(4, rgba_for(4, texels), src_left=3, src_top=5,
                                                                          width_in_blocks=13, height_in_blocks=8)
        arrays["bc1_opaque_" + name] = oracle_py.reference_block_compress(1, rgba_for(1, texels), alpha_threshold=-1.0)
        # BC7: the full search on the image as it is and with alpha 1 (only then the three-channel modes
        # compete), and the one-mode-per-block path on seeded mode buffers, also through a window of a
        # larger mode map
        rgba = rgba_for(7, texels)
        opaque = rgba.copy()
        opaque[..., 3] = 1.0
        arrays["bc7_" + name] = oracle_py.reference_block_compress_bc7(rgba)
        arrays["bc7_opaque_" + name] = oracle_py.reference_block_compress_bc7(opaque)
        blocks_y, blocks_x = arrays["bc7_" + name].shape[:2]
        modes = pack_mode_entries(bc7_mode_entries(blocks_y, blocks_x, seed=len(arrays)))
        arrays["bc7_modebuffer_" + name] = modes
        arrays["bc7_modes_" + name] = oracle_py.reference_block_compress_bc7(rgba, mode_buffer=modes)
        wide = pack_mode_entries(bc7_mode_entries(blocks_y + 3, blocks_x + 5, seed=len(arrays)))
        arrays["bc7_widemodebuffer_" + name] = wide
        arrays["bc7_window_" + name] = oracle_py.reference_block_compress_bc7(
            rgba, mode_buffer=wide, mode_map_size=(blocks_x + 5, blocks_y + 3), mode_map_offset=(4, 2), src_left=3, src_top=5,
            width_in_blocks=blocks_x, height_in_blocks=blocks_y - 1)
        # the mode bitmap the reference's host function extracts from its own blocks
        if oracle_py.reference_available():
            arrays["bc7_extracted_" + name] = oracle_py.reference_make_bc7_mode_buffer(arrays["bc7_opaque_" + name])
    np.savez_compressed(os.path.join(HERE, "block_compress_ref.npz"), **arrays)
    print("wrote %d arrays" % len(arrays))
    return 0


if __name__ == "__main__":
    sys.exit(main())
