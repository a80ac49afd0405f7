"""Seeded synthetic compressed texture sets.

The reference ships no assets and names no dataset, so the workloads are generated: shapes, sizes
and value distributions are the ones the benchmark configurations state, expressed in what the
container format can hold (one latent array, 4 bits per feature, `gridSizeScale` 1..6 and 4/8/12/16
features; a 2-bit grid is embedded exactly as the nibbles {0, 5, 10, 15} on the even neural mips).
Everything is a pure function of the seed (numpy Philox streams).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from .container import write_container
from .geometry import (FP8_BLOB_BYTES, INT8_BLOB_BYTES, MLP_LAYER_INPUTS, MLP_LAYER_OUTPUTS, Geometry,
                       full_mip_count, make_geometry)


# ---------------------------------------------------------------------------------------------
# e4m3 helpers (finite-only FP8: 1 sign, 4 exponent, 3 mantissa bits, bias 7, max 448)
# ---------------------------------------------------------------------------------------------

def _e4m3_table() -> np.ndarray:
    codes = np.arange(128, dtype=np.int32)
    exponent, mantissa = codes >> 3, codes & 7
    value = np.where(exponent == 0, mantissa * 2.0 ** -9, (1 + mantissa / 8.0) * 2.0 ** (exponent - 7.0))
    value[127] = np.nan
    return value


_E4M3_POSITIVE = _e4m3_table()


def float_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, saturating to +-448; returns the byte patterns."""
    x = np.asarray(x, dtype=np.float64)
    magnitude = np.minimum(np.abs(x), 448.0)
    table = _E4M3_POSITIVE[:127]
    hi = np.clip(np.searchsorted(table, magnitude, side="left"), 0, 126)
    lo = np.maximum(hi - 1, 0)
    d_hi, d_lo = np.abs(table[hi] - magnitude), np.abs(magnitude - table[lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & ((lo & 1) == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    return code | np.where(np.signbit(x), 0x80, 0).astype(np.uint8)


def e4m3_to_float(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    value = _E4M3_POSITIVE[codes & 0x7F]
    return np.where(codes & 0x80, -value, value)


# ---------------------------------------------------------------------------------------------
# Workload description
# ---------------------------------------------------------------------------------------------

@dataclass
class TextureSetSpec:
    width: int
    height: int
    channels: int
    mips: int                    # 0 = full chain
    grid_scale: int
    num_features: int
    seed: int
    weights: str = "int8"        # weight set the workload decodes with: "int8" or "fp8"
    latent_alphabet: str = "4bit"  # "4bit": uniform 0..15 everywhere; "2bit-even": {0,5,10,15} on even neural mips
    network: str = "benchmark"   # "benchmark": the distributions the configurations state;
                                 # "unit": scaled so that pre-activations are O(1) (exercises the
                                 # unsaturated part of the activation; used by parity tests)

    def geometry(self) -> Geometry:
        mips = self.mips if self.mips > 0 else full_mip_count(self.width, self.height)
        return make_geometry(self.width, self.height, self.channels, mips, self.grid_scale, self.num_features)


@dataclass
class SyntheticSet:
    spec: TextureSetSpec
    geometry: Geometry
    latents: List[np.ndarray]    # per neural mip: u16 [layers][h][w]
    int8_blob: bytes
    fp8_blob: bytes
    _container: Optional[bytes] = None
    channel_color_spaces: Optional[List[int]] = None  # ntc::ColorSpace per channel; None = all Linear
    textures: Optional[List[dict]] = None             # texture headers as the container's JSON holds them

    @property
    def container(self) -> bytes:
        if self._container is None:
            self._container = write_container(self.geometry, self.latents, self.int8_blob, self.fp8_blob,
                                              self.channel_color_spaces, self.textures)
        return self._container

    @property
    def use_int8(self) -> bool:
        return self.spec.weights == "int8"

    def packed_latents(self) -> np.ndarray:
        """All latent planes in device order: per neural mip, per layer, rows of pixels."""
        return np.concatenate([p.reshape(-1) for p in self.latents]).astype("<u2")


def _int8_layer(rng: np.random.Generator, nin: int, nout: int, network: str, input_layer: bool):
    weights = rng.integers(-127, 128, size=(nout, nin), dtype=np.int64).astype(np.int8)
    if network == "benchmark":
        scale = (np.abs(rng.normal(0.0, 0.02, size=nout)) + 1e-3).astype(np.float32)
        bias = rng.normal(0.0, 0.1, size=nout)
    else:
        # codes have a spread of roughly 70 (inputs) or 60 (activation codes): aim at unit variance
        spread = 73.0 * (70.0 if input_layer else 60.0) * np.sqrt(nin)
        scale = (np.abs(rng.normal(1.0, 0.25, size=nout)) / spread + 1e-7).astype(np.float32)
        bias = rng.normal(0.3, 0.5, size=nout)
    if not input_layer:
        # the stored bias also carries the -113 code offset (src/Quantizer.cu:176-181)
        bias = bias + 113.0 * weights.astype(np.float64).sum(axis=1) * scale.astype(np.float64)
    bias_i32 = np.rint(bias / scale.astype(np.float64)).astype(np.int32)  # src/Quantizer.cu:200-205
    return weights, scale, bias_i32


def _make_int8_blob(rng: np.random.Generator, network: str) -> bytes:
    layers = [_int8_layer(rng, nin, nout, network, i == 0)
              for i, (nin, nout) in enumerate(zip(MLP_LAYER_INPUTS, MLP_LAYER_OUTPUTS))]
    blob = (b"".join(l[0].tobytes() for l in layers) + b"".join(l[1].astype("<f4").tobytes() for l in layers)
            + b"".join(l[2].astype("<i4").tobytes() for l in layers))
    assert len(blob) == INT8_BLOB_BYTES
    return blob


def _make_fp8_blob(rng: np.random.Generator, network: str) -> bytes:
    weights, biases = [], []
    for i in range(3):
        nin, nout = MLP_LAYER_INPUTS[i], MLP_LAYER_OUTPUTS[i]
        sigma = 0.05 if network == "benchmark" else 2.0 / np.sqrt(nin)
        weights.append(float_to_e4m3(rng.normal(0.0, sigma, size=(nout, nin))).tobytes())
        bias_sigma = 0.05 if network == "benchmark" else 0.5
        biases.append(rng.normal(0.0 if network == "benchmark" else 0.3, bias_sigma, size=nout).astype("<f2").tobytes())
    last_w, last_scale, last_bias = _int8_layer(rng, MLP_LAYER_INPUTS[3], MLP_LAYER_OUTPUTS[3], network, False)
    blob = (b"".join(weights) + last_w.tobytes() + b"".join(biases) + last_scale.astype("<f4").tobytes()
            + last_bias.astype("<i4").tobytes())
    assert len(blob) == FP8_BLOB_BYTES
    return blob


def make_texture_set(spec: TextureSetSpec) -> SyntheticSet:
    geo = spec.geometry()
    latent_rng = np.random.Generator(np.random.Philox(key=spec.seed, counter=0))
    latents = []
    for m in range(geo.num_neural_mips):
        shape = (geo.num_layers, geo.latent_height[m], geo.latent_width[m], 4)
        if spec.latent_alphabet == "2bit-even" and (m & 1) == 0:
            nibbles = latent_rng.integers(0, 4, size=shape, dtype=np.uint16) * 5
        else:
            nibbles = latent_rng.integers(0, 16, size=shape, dtype=np.uint16)
        packed = nibbles[..., 0] | (nibbles[..., 1] << 4) | (nibbles[..., 2] << 8) | (nibbles[..., 3] << 12)
        latents.append(packed.astype(np.uint16))
    weight_rng = np.random.Generator(np.random.Philox(key=spec.seed, counter=1 << 64))
    int8_blob = _make_int8_blob(weight_rng, spec.network)
    fp8_blob = _make_fp8_blob(weight_rng, spec.network)
    return SyntheticSet(spec, geo, latents, int8_blob, fp8_blob)


# ---------------------------------------------------------------------------------------------
# The benchmark configurations
# ---------------------------------------------------------------------------------------------

def config_spec(index: int, set_index: int = 0) -> TextureSetSpec:
    """Configurations 0..4 as the benchmark definition lists them."""
    if index == 0:    # 1024^2, 4 channels, mip 0 only, 8 features, scale 2, int8
        return TextureSetSpec(1024, 1024, 4, 1, 2, 8, seed=0, weights="int8")
    if index in (1, 4):  # 4096^2 PBR set, 12 channels, full chain, 12 features, FP8 hidden + int8 last layer
        return TextureSetSpec(4096, 4096, 12, 0, 4, 12, seed=1, weights="fp8", latent_alphabet="2bit-even")
    if index == 2:    # one of 64 sets: 2048^2, 8 channels, full chain, 8 features, int8
        return TextureSetSpec(2048, 2048, 8, 0, 4, 8, seed=100 + set_index, weights="int8", latent_alphabet="2bit-even")
    if index == 3:    # 8192^2, 16 channels, full chain, 16 features, scale 4, int8
        return TextureSetSpec(8192, 8192, 16, 0, 4, 16, seed=7, weights="int8")
    raise ValueError("unknown configuration")


def make_queries(count: int, max_lod: float = 12.0, seed: int = 9) -> np.ndarray:
    """Inference-on-sample queries: (u, v) uniform in [0,1)^2, LOD uniform in [0, max_lod]."""
    rng = np.random.Generator(np.random.Philox(key=seed))
    q = rng.random(size=(count, 3), dtype=np.float32)
    q[:, 2] *= np.float32(max_lod)
    return q
