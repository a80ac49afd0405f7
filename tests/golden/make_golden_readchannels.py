"""Generates the ReadChannels fixtures (`readchannels_*.npz`, `readchannels_index.json`) by running
the UNMODIFIED reference library (oracle/_ref/libntc_ref.so) on a GPU.

A seeded synthetic texture set whose channels are stored in a mix of colour spaces is decompressed
by the reference; for two mips its fp16 texels are stored together with what the reference's
`ITextureSet::ReadChannels` hands back for a list of requests (channel format, channel range,
component count, destination colour spaces, dithering).  The fixtures pin the conversion stage on
identical inputs: the fp16 texels in, the client's bytes out.  ReadChannels takes every channel out
of its stored colour space even for a plain FLOAT16 read, so the raw texels are read from a second
container that is identical except that it declares no colour spaces.

Run on a machine with a GPU, from the repository root:
    python tests/golden/make_golden_readchannels.py [output-dir]
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

UNORM8, UNORM16, FLOAT16, FLOAT32, UINT32 = 1, 2, 3, 4, 5
LINEAR, SRGB, HLG = 0, 1, 2

# the colour space each of the six channels is stored in
CHANNEL_SPACES = [SRGB, SRGB, SRGB, LINEAR, LINEAR, HLG]

# name -> request: format, first channel, channel count, components, destination spaces (None = Linear), dithering
REQUESTS = {
    "u8_all_linear": dict(format=UNORM8, first=0, count=6, components=6, dst=None, dither=False),
    "u8_rgb_to_rgba_srgb": dict(format=UNORM8, first=0, count=3, components=4, dst=[SRGB, SRGB, SRGB], dither=False),
    "u8_rgb_to_rgba_srgb_dither": dict(format=UNORM8, first=0, count=3, components=4, dst=[SRGB, SRGB, SRGB], dither=True),
    "u8_rgb8_linear_dither": dict(format=UNORM8, first=1, count=3, components=3, dst=None, dither=True),
    "u8_single": dict(format=UNORM8, first=4, count=1, components=1, dst=None, dither=False),
    "u16_pair_dither": dict(format=UNORM16, first=3, count=2, components=2, dst=None, dither=True),
    "u16_all_mixed": dict(format=UNORM16, first=0, count=6, components=6, dst=[SRGB, SRGB, SRGB, LINEAR, HLG, HLG], dither=False),
    "f16_hlg_single": dict(format=FLOAT16, first=5, count=1, components=1, dst=[HLG], dither=False),
    "f16_all_linear": dict(format=FLOAT16, first=0, count=6, components=8, dst=None, dither=False),
    "f32_all_mixed": dict(format=FLOAT32, first=0, count=6, components=6, dst=[LINEAR, SRGB, HLG, LINEAR, SRGB, HLG], dither=False),
    "u32_pair": dict(format=UINT32, first=0, count=2, components=2, dst=None, dither=False),
}

CASES = {
    "readchannels_r64x48_g2_f8": (TextureSetSpec(64, 48, 6, 0, 2, 8, seed=21, network="unit"), "int8", (0, 2)),
}


def main() -> int:
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out_dir, exist_ok=True)
    index = {}
    for name, (spec, mode, mips) in CASES.items():
        plain = make_texture_set(spec)
        synthetic = make_texture_set(spec)
        synthetic.channel_color_spaces = list(CHANNEL_SPACES)
        geo = synthetic.geometry
        arrays = {"container": np.frombuffer(synthetic.container, dtype=np.uint8)}
        raw_decoder = oracle_py.ReferenceDecoder(plain.container, geo.channels)
        raw_decoder.decompress(mode == "int8")
        decoder = oracle_py.ReferenceDecoder(synthetic.container, geo.channels, staging_bytes_per_pixel=64)
        decoder.decompress(mode == "int8")
        for mip in mips:
            cm = geo.color_mips[mip]
            arrays["texels_mip%d" % mip] = raw_decoder.read_mip(mip, cm.width, cm.height).view(np.uint16)
            for request_name, r in REQUESTS.items():
                arrays["%s_mip%d" % (request_name, mip)] = decoder.read_channels(
                    mip, cm.width, cm.height, r["format"], r["first"], r["count"], r["components"], r["dst"], r["dither"])
        decoder.close()
        raw_decoder.close()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **arrays)
        index[name] = {"width": spec.width, "height": spec.height, "channels": geo.channels, "mode": mode, "mips": list(mips),
                       "channel_spaces": CHANNEL_SPACES, "requests": REQUESTS}
        print("golden", name, "ok")
    with open(os.path.join(out_dir, "readchannels_index.json"), "w") as f:
        json.dump(index, f, indent=1, sort_keys=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
