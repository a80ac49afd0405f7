"""Generates the golden fixtures in this directory by running the UNMODIFIED reference library
(oracle/_ref/libntc_ref.so, built from the reference sources by oracle/build_ref.sh) on a GPU.

For each case below a seeded synthetic compressed texture set is written as an NTC container,
loaded through the reference's public API, decompressed with its CUDA decoder and read back as
fp16.  The container bytes and the reference's outputs are stored together, so the fixtures do
not depend on the generator staying unchanged.

Run on a machine with a GPU, from the repository root:
    python tests/golden/make_golden.py [output-dir]
The reference's own timing of configuration-like workloads is printed as a side effect.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
from rtxntc_library_b200.synthetic import TextureSetSpec, make_texture_set  # noqa: E402
import oracle_py  # noqa: E402

# name -> (spec, weight modes to decode with)
CASES = {
    "sq64_g2_f8_unit": (TextureSetSpec(64, 64, 4, 0, 2, 8, seed=3, network="unit"), ("int8", "fp8")),
    "sq64_g2_f8_bench": (TextureSetSpec(64, 64, 4, 0, 2, 8, seed=4, network="benchmark"), ("int8", "fp8")),
    "r96x40_g3_f12_unit": (TextureSetSpec(96, 40, 6, 0, 3, 12, seed=5, network="unit"), ("int8", "fp8")),
    "sq128_g4_f12_2bit_bench": (TextureSetSpec(128, 128, 12, 0, 4, 12, seed=1, network="benchmark",
                                               latent_alphabet="2bit-even"), ("fp8",)),
    "sq128_g4_f12_2bit_unit": (TextureSetSpec(128, 128, 12, 0, 4, 12, seed=11, network="unit",
                                              latent_alphabet="2bit-even"), ("fp8", "int8")),
    "r128x64_g4_f16_unit": (TextureSetSpec(128, 64, 16, 0, 4, 16, seed=7, network="unit"), ("int8",)),
    "r33x17_g1_f4_unit": (TextureSetSpec(33, 17, 2, 0, 1, 4, seed=8, network="unit"), ("int8", "fp8")),
    "sq128_g6_f8_unit": (TextureSetSpec(128, 128, 8, 0, 6, 8, seed=9, network="unit"), ("int8",)),
    "sq64_g5_f16_mip0_unit": (TextureSetSpec(64, 64, 3, 1, 5, 16, seed=10, network="unit"), ("int8", "fp8")),
}


def main() -> int:
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out_dir, exist_ok=True)
    index = {}
    for name, (spec, modes) in CASES.items():
        synthetic = make_texture_set(spec)
        geo = synthetic.geometry
        arrays = {"container": np.frombuffer(synthetic.container, dtype=np.uint8)}
        decoder = oracle_py.ReferenceDecoder(synthetic.container, geo.channels)
        for mode in modes:
            decoder.decompress(mode == "int8")
            for mip, cm in enumerate(geo.color_mips):
                arrays["%s_mip%d" % (mode, mip)] = decoder.read_mip(mip, cm.width, cm.height).view(np.uint16)
        decoder.close()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **arrays)
        index[name] = {"width": spec.width, "height": spec.height, "channels": geo.channels, "mips": geo.mips,
                       "grid_scale": spec.grid_scale, "num_features": spec.num_features, "seed": spec.seed,
                       "network": spec.network, "latent_alphabet": spec.latent_alphabet, "modes": list(modes)}
        print("golden", name, "ok")
    with open(os.path.join(out_dir, "index.json"), "w") as f:
        json.dump(index, f, indent=1, sort_keys=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
