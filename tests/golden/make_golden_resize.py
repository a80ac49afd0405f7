"""Generates `readchannels_resize.npz` by running the UNMODIFIED reference library
(oracle/_ref/libntc_ref.so) on a GPU: `ITextureSet::ReadChannels` with a width and height other than
the mip's, which makes the reference's copy kernel resize bilinearly (src/ImageProcessing.cu:24-71,
220-266).

A seeded 64x48, 6-channel set whose channels are stored in a mix of colour spaces is decompressed
by the reference.  Stored: the container, the raw fp16 texels of mips 0 and 1 (read from a twin
container that declares no colour spaces, because ReadChannels takes every channel out of its
stored colour space even for a plain FLOAT16 read) and, for every (mip, size, request) of the
lists below, what the reference handed back, under the key "<request>_mip<m>_<width>x<height>".

Run on a machine with a GPU, from the repository root:
    python tests/golden/make_golden_resize.py [output-dir]
"""
from __future__ import annotations

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

SPEC = TextureSetSpec(64, 48, 6, 0, 2, 8, seed=33, network="unit")
CHANNEL_SPACES = [SRGB, SRGB, SRGB, LINEAR, HLG, LINEAR]
# (mip, (width, height)): shrink, enlarge, off by one, a single pixel, another aspect, one axis unchanged
SIZES = [(0, (32, 24)), (0, (100, 70)), (0, (65, 47)), (0, (1, 1)), (1, (9, 40)), (1, (32, 25))]
REQUESTS = {
    "f16_all_linear": dict(format=FLOAT16, first=0, count=6, components=6, dst=None, dither=False),
    "u8_rgba_srgb_dither": dict(format=UNORM8, first=0, count=4, components=4, dst=[SRGB, SRGB, SRGB, LINEAR], dither=True),
    "f32_mixed": dict(format=FLOAT32, first=2, count=4, components=4, dst=[LINEAR, SRGB, HLG, LINEAR], dither=False),
    "u16_pair_plus_default": dict(format=UNORM16, first=4, count=2, components=4, dst=None, dither=True),
}


def main() -> int:
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    plain = make_texture_set(SPEC)
    tagged = make_texture_set(SPEC)
    tagged.channel_color_spaces = list(CHANNEL_SPACES)
    geo = tagged.geometry
    arrays = {"container": np.frombuffer(tagged.container, dtype=np.uint8)}
    raw = oracle_py.ReferenceDecoder(plain.container, geo.channels)
    raw.decompress(False)
    decoder = oracle_py.ReferenceDecoder(tagged.container, geo.channels, staging_bytes_per_pixel=256)
    decoder.decompress(False)
    for mip in (0, 1):
        cm = geo.color_mips[mip]
        arrays["texels_mip%d" % mip] = raw.read_mip(mip, cm.width, cm.height).view(np.uint16)
    for mip, (width, height) in SIZES:
        for name, r in REQUESTS.items():
            arrays["%s_mip%d_%dx%d" % (name, mip, width, height)] = decoder.read_channels(
                mip, width, height, r["format"], r["first"], r["count"], r["components"], r["dst"], r["dither"])
    decoder.close()
    raw.close()
    path = os.path.join(out_dir, "readchannels_resize.npz")
    np.savez_compressed(path, **arrays)
    print("wrote", path, os.path.getsize(path), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
