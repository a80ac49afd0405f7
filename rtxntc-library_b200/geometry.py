"""Texture-set geometry of the NTC decode path (host-side mirror used by the container writer,
the synthetic workloads and the multi-GPU sharder).

Follows the reference's integer rules:
  * neural mip count, grid dimensions, colour-mip -> neural-LOD map:
    src/FeatureGridMath.cpp:47-76, src/FeatureGridHost.cpp:27-52
  * colour mip sizes and texel offsets: src/TextureSet.cpp:88-101
  * positional-encoding constants per colour mip: src/TextureSet.cpp:450-463
The C++ host library computes the same values itself; this module exists so that Python tooling
can lay out buffers and files without calling into native code.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List

import numpy as np

MAX_MIPS = 16            # include/libntc/shaders/InferenceConstants.h:22
MAX_CHANNELS = 16
MAX_NEURAL_MIPS = 8
FEATURES_PER_LAYER = 4   # one BGRA4 pixel holds four 4-bit features
MLP_LAYER_INPUTS = (48, 64, 48, 32)
MLP_LAYER_OUTPUTS = (64, 48, 32, 16)
INT8_BLOB_BYTES = 9472
FP8_BLOB_BYTES = 8608

_SHARED_MIPS_FOR_GRID_SCALE = (2, 3, 3, 3, 4, 4)


def lod_to_neural_lod(lod: int, grid_scale: int, neural_lods: int) -> int:
    """Colour mip -> index of the high-resolution latent image (always even)."""
    shared = _SHARED_MIPS_FOR_GRID_SCALE[grid_scale - 1]
    neural = (lod - shared + 2) & ~1
    return max(0, min(neural, neural_lods - 2))


def grid_dimension(image_dimension: int, neural_lod: int, grid_scale: int) -> int:
    return max((image_dimension // grid_scale) >> neural_lod, 1)


def num_neural_mips(width: int, height: int, mips: int, grid_scale: int) -> int:
    min_grid = int(np.float32(min(width, height)) / np.float32(grid_scale))
    theoretical = max(2, int(1 + math.floor(math.log2(min_grid))) if min_grid >= 1 else 2) & ~1
    last = lod_to_neural_lod(mips - 1, grid_scale, MAX_NEURAL_MIPS)
    return min(theoretical, last + 2)


def full_mip_count(width: int, height: int) -> int:
    return int(math.floor(math.log2(max(width, height)))) + 1


@dataclass
class ColorMip:
    width: int
    height: int
    neural_lod: int
    position_scale: float
    position_lod: float
    texel_offset: int


@dataclass
class Geometry:
    width: int
    height: int
    channels: int          # rounded up to even, as the texture set stores it
    mips: int
    grid_scale: int
    num_features: int
    num_layers: int = 0
    latent_width: List[int] = field(default_factory=list)
    latent_height: List[int] = field(default_factory=list)
    latent_pixel_offset: List[int] = field(default_factory=list)  # per-layer pixels, cumulative
    color_mips: List[ColorMip] = field(default_factory=list)

    @property
    def num_neural_mips(self) -> int:
        return len(self.latent_width)

    @property
    def total_latent_pixels(self) -> int:
        return self.latent_pixel_offset[-1]

    @property
    def total_texels(self) -> int:
        last = self.color_mips[-1]
        return last.texel_offset + last.width * last.height

    @property
    def encoded_latent_bytes(self) -> int:
        return self.total_latent_pixels * self.num_layers * 2


def make_geometry(width: int, height: int, channels: int, mips: int, grid_scale: int, num_features: int) -> Geometry:
    if not (1 <= grid_scale <= 6):
        raise ValueError("gridSizeScale must be 1..6")
    if num_features not in (4, 8, 12, 16):
        raise ValueError("numFeatures must be 4, 8, 12 or 16")
    if not (1 <= mips <= MAX_MIPS) or not (1 <= channels <= MAX_CHANNELS):
        raise ValueError("invalid mip or channel count")
    geo = Geometry(width, height, (channels + 1) & ~1, mips, grid_scale, num_features)
    geo.num_layers = (num_features + FEATURES_PER_LAYER - 1) // FEATURES_PER_LAYER
    offset = 0
    for m in range(num_neural_mips(width, height, mips, grid_scale)):
        w, h = grid_dimension(width, m, grid_scale), grid_dimension(height, m, grid_scale)
        geo.latent_width.append(w)
        geo.latent_height.append(h)
        geo.latent_pixel_offset.append(offset)
        offset += w * h
    geo.latent_pixel_offset.append(offset)
    texels = 0
    f32 = np.float32
    for mip in range(mips):
        w, h = max(1, width >> mip), max(1, height >> mip)
        lod = lod_to_neural_lod(mip, grid_scale, geo.num_neural_mips)
        ws = f32(geo.latent_width[lod]) / f32(w)
        hs = f32(geo.latent_height[lod]) / f32(h)
        scale = f32(0.5) * max(ws, hs)
        plod = max(f32(-1), min(f32(1), f32(0.25) * f32(np.log2(scale))))
        geo.color_mips.append(ColorMip(w, h, lod, float(scale), float(plod), texels))
        texels += w * h
    return geo
