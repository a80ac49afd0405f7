"""Writer (and a small reader) for the NTC container the decode path consumes.

Layout (all little-endian), as the reference reads it:
  * 40-byte header: u32 signature "NTEX" (0x5845544E), u32 version 0x100, u64 JSON offset,
    u64 JSON size (with the terminating NUL), u64 binary chunk offset, u64 binary chunk size
    (src/JsonFileFormat.h:26-38, checks in src/TextureSetMetadata.cpp:1210-1264);
  * JSON document, schema version 3 (field names: src/JsonFileFormat.cpp:25-185);
  * binary chunk addressed through `views` (offset relative to the chunk, multiple of 4).
Latent planes are BGRA4: one u16 per latent pixel per layer, nibble j = feature 4*layer + j
(src/Quantizer.cu:497-527).  Weights come as two MLP versions, Int8 and FloatE4M3, each split in
per-layer weight / scale / bias views in the GenericInt8 / GenericFP8 order
(src/WeightLayout.cpp:142-268, src/TextureSetMetadata.cpp:676-784, 1000-1135).

The writer exists to produce inputs for the decoder (synthetic workloads, tests); no buffer is
compressed (`compression: None`).
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .geometry import (FP8_BLOB_BYTES, INT8_BLOB_BYTES, MLP_LAYER_INPUTS, MLP_LAYER_OUTPUTS, Geometry,
                       make_geometry)

SIGNATURE = 0x5845544E
VERSION = 0x100
HEADER_BYTES = 40


def split_int8_blob(blob: bytes) -> List[Dict[str, bytes]]:
    """GenericInt8: all weight matrices, then all fp32 scale vectors, then all int32 bias vectors."""
    assert len(blob) == INT8_BLOB_BYTES
    layers = []
    w_off = 0
    s_off = 8192
    b_off = 8192 + 640
    for nin, nout in zip(MLP_LAYER_INPUTS, MLP_LAYER_OUTPUTS):
        layers.append({"weights": blob[w_off:w_off + nin * nout], "scale": blob[s_off:s_off + 4 * nout],
                       "bias": blob[b_off:b_off + 4 * nout]})
        w_off += nin * nout
        s_off += 4 * nout
        b_off += 4 * nout
    return layers


def split_fp8_blob(blob: bytes) -> List[Dict[str, bytes]]:
    """GenericFP8: weights (layers 0-2 e4m3, layer 3 int8), fp16 biases of layers 0-2, then the
    fp32 scale and int32 bias of layer 3."""
    assert len(blob) == FP8_BLOB_BYTES
    layers = []
    w_off = 0
    b_off = 8192
    for i, (nin, nout) in enumerate(zip(MLP_LAYER_INPUTS, MLP_LAYER_OUTPUTS)):
        entry = {"weights": blob[w_off:w_off + nin * nout]}
        w_off += nin * nout
        if i < 3:
            entry["bias"] = blob[b_off:b_off + 2 * nout]
            b_off += 2 * nout
        else:
            entry["scale"] = blob[b_off:b_off + 4 * nout]
            entry["bias"] = blob[b_off + 4 * nout:b_off + 8 * nout]
        layers.append(entry)
    return layers


class _BinaryChunk:
    def __init__(self) -> None:
        self.data = bytearray()
        self.views: List[Dict[str, int]] = []

    def add(self, payload: bytes) -> int:
        while len(self.data) % 4:
            self.data.append(0)
        self.views.append({"offset": len(self.data), "storedSize": len(payload)})
        self.data += payload
        return len(self.views) - 1

    def finish(self) -> bytes:
        while len(self.data) % 4:
            self.data.append(0)
        return bytes(self.data)


COLOR_SPACE_NAMES = ("Linear", "sRGB", "HLG")  # ntc::ColorSpace values 0, 1, 2


def write_container(geo: Geometry, latents: Sequence[np.ndarray], int8_blob: bytes, fp8_blob: bytes,
                    channel_color_spaces: Optional[Sequence[int]] = None, textures: Optional[Sequence[dict]] = None) -> bytes:
    """Serialises one compressed texture set.

    latents[m] is the u16 array [layers][height][width] of neural mip m.  channel_color_spaces, when
    given, holds one ntc::ColorSpace value per channel (the colour space the channel was stored in).
    textures, when given, holds the documents of the texture headers (the schema's own field names:
    name, firstChannel, numChannels and optionally channelFormat, rgbColorSpace, alphaColorSpace,
    bcFormat as the schema's strings).  A header's "bcModeBuffers" may hold {"mipLevel": m, "data": bytes}
    entries: the bytes go into the binary chunk and the entry becomes the schema's {"mipLevel", "view"}.
    """
    chunk = _BinaryChunk()
    latent_entries = []
    for m, planes in enumerate(latents):
        planes = np.ascontiguousarray(planes, dtype="<u2")
        assert planes.shape == (geo.num_layers, geo.latent_height[m], geo.latent_width[m]), planes.shape
        layer_views = [chunk.add(planes[layer].tobytes()) for layer in range(geo.num_layers)]
        latent_entries.append({"width": geo.latent_width[m], "height": geo.latent_height[m], "layerViews": layer_views})

    def mlp_entry(parts: List[Dict[str, bytes]], fp8: bool) -> Dict:
        layers = []
        for i, (nin, nout) in enumerate(zip(MLP_LAYER_INPUTS, MLP_LAYER_OUTPUTS)):
            part = parts[i]
            layer = {"inputChannels": nin, "outputChannels": nout, "weightView": chunk.add(part["weights"])}
            if fp8 and i < 3:
                layer.update({"biasView": chunk.add(part["bias"]), "weightType": "FloatE4M3", "biasType": "Float16"})
            else:
                layer.update({"scaleView": chunk.add(part["scale"]), "biasView": chunk.add(part["bias"]),
                              "weightType": "Int8", "scaleType": "Float32", "biasType": "Int32"})
            layers.append(layer)
        return {"layers": layers, "activation": "HGELUClamp", "weightLayout": "RowMajor"}

    mlp_versions = [mlp_entry(split_int8_blob(int8_blob), False), mlp_entry(split_fp8_blob(fp8_blob), True)]
    color_mips = [{"width": cm.width, "height": cm.height, "latentMip": cm.neural_lod,
                   "positionLod": cm.position_lod, "positionScale": cm.position_scale} for cm in geo.color_mips]
    channel_entries = []
    if channel_color_spaces is not None:
        assert len(channel_color_spaces) == geo.channels
        channel_entries = [{} if space == 0 else {"colorSpace": COLOR_SPACE_NAMES[space]} for space in channel_color_spaces]
    texture_entries = []
    for header in (textures or []):
        if not isinstance(header, dict):  # a malformed entry, written as it is (loader tests)
            texture_entries.append(header)
            continue
        header = dict(header)
        if isinstance(header.get("bcModeBuffers"), list):
            header["bcModeBuffers"] = [
                {"mipLevel": item["mipLevel"], "view": chunk.add(bytes(item["data"]))} if isinstance(item, dict) and "data" in item else item
                for item in header["bcModeBuffers"]]
        texture_entries.append(header)
    document = {
        "schemaVersion": 3,
        "width": geo.width,
        "height": geo.height,
        "numChannels": geo.channels,
        "numColorMips": geo.mips,
        "latentShape": {"numFeatures": geo.num_features},
        "mlpVersions": mlp_versions,
        "textures": texture_entries,
        "channels": channel_entries,
        "latents": latent_entries,
        "colorMips": color_mips,
        "views": chunk.views,
    }
    text = json.dumps(document, separators=(",", ":")).encode("ascii") + b"\0"
    binary = chunk.finish()
    json_offset = HEADER_BYTES
    binary_offset = (json_offset + len(text) + 3) & ~3
    header = struct.pack("<IIQQQQ", SIGNATURE, VERSION, json_offset, len(text), binary_offset, len(binary))
    out = bytearray(header)
    out += text
    while len(out) < binary_offset:
        out.append(0)
    out += binary
    return bytes(out)


def read_container(data: bytes) -> Tuple[Geometry, List[np.ndarray], bytes, bytes]:
    """Parses a container written by write_container (or by the reference with no compressed
    views) back into geometry, latent planes and the two weight blobs."""
    signature, version, json_offset, json_size, binary_offset, binary_size = struct.unpack_from("<IIQQQQ", data, 0)
    if signature != SIGNATURE or version != VERSION:
        raise ValueError("not an NTC container")
    document = json.loads(data[json_offset:json_offset + json_size].rstrip(b"\0").decode("ascii"))
    if document["schemaVersion"] != 3:
        raise ValueError("unsupported schema version")
    binary = memoryview(data)[binary_offset:binary_offset + binary_size]

    def view(index: int) -> bytes:
        v = document["views"][index]
        if v.get("compression", "None") != "None":
            raise ValueError("compressed views are not supported")
        return bytes(binary[v["offset"]:v["offset"] + v["storedSize"]])

    lat0 = document["latents"][0]
    grid_scale = int(round(min(document["width"] / lat0["width"], document["height"] / lat0["height"])))
    geo = make_geometry(document["width"], document["height"], document["numChannels"],
                        document.get("numColorMips", 1), grid_scale, document["latentShape"]["numFeatures"])
    latents = []
    for m, entry in enumerate(document["latents"]):
        planes = [np.frombuffer(view(i), dtype="<u2", count=entry["width"] * entry["height"]) for i in entry["layerViews"]]
        latents.append(np.stack(planes).reshape(len(planes), entry["height"], entry["width"]).copy())
    int8_blob = fp8_blob = None
    for mlp in document["mlpVersions"]:
        layers = mlp["layers"]
        if layers[0]["weightType"] == "Int8":
            int8_blob = (b"".join(view(l["weightView"]) for l in layers) + b"".join(view(l["scaleView"]) for l in layers)
                         + b"".join(view(l["biasView"]) for l in layers))
        else:
            fp8_blob = (b"".join(view(l["weightView"]) for l in layers) + b"".join(view(l["biasView"]) for l in layers[:3])
                        + view(layers[3]["scaleView"]) + view(layers[3]["biasView"]))
    return geo, latents, int8_blob, fp8_blob
