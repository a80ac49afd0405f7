"""Generates `producers.npz` by running two internal kernels of the UNMODIFIED reference library
(oracle/_ref/libntc_ref.so, through oracle/ref_harness_producers.cu) on a GPU:
`cuda::PackLatents` and `cuda::QuantizeNetwork` (src/Quantizer.cu), the producers of the packed
latents and of the GenericInt8 / GenericFP8 network blobs that the decoder consumes.

Stored: the seeded inputs and the reference's outputs.
  pack_all_codes          the reference's 4-bit code for each of the 65536 fp16 bit patterns
  pack<i>_latents/_shape/_packed   ragged and padded latent arrays (shape = width, height, layers, stride)
  q<i>_weights/_biases/_scale/_bias    fp16 network, optimal-to-linear scale and bias per output channel
  q<i>_blob_int8/_blob_fp8/_rounded_int8/_rounded_fp8   the reference's blobs and its fp16 copy afterwards

Run on a machine with a GPU, from the repository root:
    python tests/golden/make_golden_producers.py [output-dir]
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import oracle_py  # noqa: E402

WEIGHTS = 48 * 64 + 64 * 48 + 48 * 32 + 32 * 16
COLUMNS = 64 + 48 + 32 + 16


def network(seed: int):
    """Three families: trained-looking normal weights, wide uniform ones, and a mix of magnitudes
    with an all-zero column, an all-negative column and a constant output channel (zero scale)."""
    rng = np.random.default_rng(1000 + seed)
    kind = seed % 3
    if kind == 0:
        w = rng.normal(0, 0.3, WEIGHTS)
    elif kind == 1:
        w = rng.uniform(-2, 2, WEIGHTS)
    else:
        w = rng.normal(0, 0.05, WEIGHTS) * rng.choice([1, 10, 0.001], WEIGHTS)
    bias = rng.normal(0, 0.5, COLUMNS)
    scale = rng.uniform(0.2, 3, 16)
    obias = rng.normal(0, 0.4, 16)
    if kind == 2:
        scale[3] = 0.0
        w[:48] = 0
        w[48:96] = -np.abs(w[48:96])
    return w.astype(np.float16), bias.astype(np.float16), scale.astype(np.float32), obias.astype(np.float32)


PACK_CASES = [(37, 19, 4, 5), (64, 32, 3, 0), (1, 1, 2, 3)]  # width, height, layers, padding of the stride


def latents(case):
    width, height, layers, pad = case
    rng = np.random.default_rng(width * 131 + height)
    stride = width * height * 2 + pad
    values = (rng.integers(0, 16, layers * stride * 2) / 15.0).astype(np.float16)
    values[::7] = rng.uniform(-0.3, 1.3, values[::7].size).astype(np.float16)
    values[::11] = 0.5
    return values, stride


def main() -> int:
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    data = {}
    every = np.arange(65536, dtype=np.uint16).view(np.float16)
    side = 256
    flat = np.zeros(side * side * 4, np.float16)
    flat[0:side * side * 2:2] = every
    words = oracle_py.reference_pack_latents(flat, side, side, 1, side * side * 2).reshape(-1)
    data["pack_all_codes"] = (words & 15).astype(np.uint8)
    for i, case in enumerate(PACK_CASES):
        values, stride = latents(case)
        data[f"pack{i}_latents"] = values
        data[f"pack{i}_shape"] = np.array([case[0], case[1], case[2], stride], dtype=np.int64)
        data[f"pack{i}_packed"] = oracle_py.reference_pack_latents(values, case[0], case[1], case[2], stride)
    for i in range(6):
        w, bias, scale, obias = network(i)
        data[f"q{i}_weights"], data[f"q{i}_biases"], data[f"q{i}_scale"], data[f"q{i}_bias"] = w, bias, scale, obias
        for fp8, tag in ((False, "int8"), (True, "fp8")):
            blob, rounded = oracle_py.reference_quantize_network(w, bias, fp8, scale, obias)
            data[f"q{i}_blob_{tag}"] = np.frombuffer(blob, dtype=np.uint8)
            data[f"q{i}_rounded_{tag}"] = rounded
    path = os.path.join(out_dir, "producers.npz")
    np.savez_compressed(path, **data)
    print("wrote", path, os.path.getsize(path), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
