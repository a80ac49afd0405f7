"""TEST INFRASTRUCTURE ONLY: ctypes bindings for the CPU restatement (libntc_oracle.so) and for
the unmodified reference library built by build_ref.sh (oracle/_ref/libntc_ref.so).

Only tests, the smoke check and the benchmark's baseline legs may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import List, Optional

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(HERE, "libntc_oracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libntc_ref.so")

MAX_MIPS = 16
MAX_NEURAL_MIPS = 8


class _TextureSet(ctypes.Structure):
    _fields_ = [("width", ctypes.c_int), ("height", ctypes.c_int), ("channels", ctypes.c_int),
                ("numMips", ctypes.c_int), ("gridSizeScale", ctypes.c_int), ("numFeatures", ctypes.c_int),
                ("latents", ctypes.c_void_p), ("int8Blob", ctypes.c_void_p), ("fp8Blob", ctypes.c_void_p)]


class Geometry(ctypes.Structure):
    _fields_ = [("numNeuralMips", ctypes.c_int), ("numLayers", ctypes.c_int),
                ("latentWidth", ctypes.c_int * MAX_NEURAL_MIPS), ("latentHeight", ctypes.c_int * MAX_NEURAL_MIPS),
                ("latentPixelOffset", ctypes.c_uint64 * (MAX_NEURAL_MIPS + 1)),
                ("mipWidth", ctypes.c_int * MAX_MIPS), ("mipHeight", ctypes.c_int * MAX_MIPS),
                ("neuralLod", ctypes.c_int * MAX_MIPS), ("positionScale", ctypes.c_float * MAX_MIPS),
                ("positionLod", ctypes.c_float * MAX_MIPS), ("mipTexelOffset", ctypes.c_uint64 * (MAX_MIPS + 1))]


class Options(ctypes.Structure):
    _fields_ = [("weights", ctypes.c_int), ("numerics", ctypes.c_int), ("threads", ctypes.c_int),
                ("refBlendFma", ctypes.c_int), ("refQuantFma", ctypes.c_int), ("refAccChunk", ctypes.c_int),
                ("refAccMode", ctypes.c_int), ("refActFma", ctypes.c_int)]


WEIGHTS_INT8, WEIGHTS_FP8 = 0, 1
NUMERICS_SPEC, NUMERICS_REF = 0, 1

_oracle = None


class ReadChannels(ctypes.Structure):
    _fields_ = [("width", ctypes.c_int), ("height", ctypes.c_int), ("channels", ctypes.c_int),
                ("firstChannel", ctypes.c_int), ("numChannels", ctypes.c_int), ("channelFormat", ctypes.c_int),
                ("pixelStride", ctypes.c_size_t), ("rowPitch", ctypes.c_size_t),
                ("srcColorSpaces", ctypes.POINTER(ctypes.c_int)), ("dstColorSpaces", ctypes.POINTER(ctypes.c_int)),
                ("useDithering", ctypes.c_int)]


FORMAT_DTYPES = {1: np.uint8, 2: np.uint16, 3: np.float16, 4: np.float32, 5: np.uint32}  # ntc::ChannelFormat


def read_channels(texels: np.ndarray, channel_format: int, first_channel: int = 0, num_channels: Optional[int] = None,
                  components: Optional[int] = None, src_color_spaces=None, dst_color_spaces=None,
                  use_dithering: bool = False, size=None) -> np.ndarray:
    """ReadChannels restated on the CPU: `texels` is a decoded mip [h][w][channels] (float16);
    returns [h][w][components] in the channel format's dtype; `size` = (width, height) other than
    the mip's resizes bilinearly."""
    texels = np.ascontiguousarray(texels, dtype=np.float16)
    h, w, channels = texels.shape
    n = channels - first_channel if num_channels is None else num_channels
    count = n if components is None else components
    dtype = np.dtype(FORMAT_DTYPES[channel_format])
    dw, dh = (w, h) if size is None else size
    out = np.zeros((dh, dw, count), dtype=dtype)
    p = ReadChannels()
    p.width, p.height, p.channels, p.firstChannel, p.numChannels, p.channelFormat = w, h, channels, first_channel, n, channel_format
    p.pixelStride, p.rowPitch = count * dtype.itemsize, count * dtype.itemsize * dw
    keep = []
    if src_color_spaces is not None:
        keep.append((ctypes.c_int * channels)(*src_color_spaces))
        p.srcColorSpaces = ctypes.cast(keep[-1], ctypes.POINTER(ctypes.c_int))
    if dst_color_spaces is not None:
        keep.append((ctypes.c_int * n)(*dst_color_spaces))
        p.dstColorSpaces = ctypes.cast(keep[-1], ctypes.POINTER(ctypes.c_int))
    p.useDithering = 1 if use_dithering else 0
    if oracle_lib().ntco_read_channels_resized(texels.ctypes.data, ctypes.byref(p), dw, dh, out.ctypes.data) != 0:
        raise ValueError("ntco_read_channels rejected its arguments")
    return out


def pack_latents(latents: np.ndarray, width: int, height: int, num_layers: int, latent_stride: int) -> np.ndarray:
    """PackLatents restated on the CPU: a flat float16 array in the reference's latent layout to
    uint16 words [num_layers][height][width]."""
    latents = np.ascontiguousarray(latents, dtype=np.float16)
    out = np.empty((num_layers, height, width), dtype=np.uint16)
    if oracle_lib().ntco_pack_latents(latents.ctypes.data, width, height, num_layers, latent_stride, out.ctypes.data) != 0:
        raise ValueError("ntco_pack_latents rejected its arguments")
    return out


def quantize_network(weights: np.ndarray, biases: np.ndarray, use_fp8: bool, output_scale=None, output_bias=None):
    """QuantizeNetwork restated on the CPU; returns (blob bytes, rounded fp16 weights)."""
    weights = np.ascontiguousarray(weights, dtype=np.float16)
    biases = np.ascontiguousarray(biases, dtype=np.float16)
    scale = np.ascontiguousarray(np.ones(16) if output_scale is None else output_scale, dtype=np.float32)
    bias = np.ascontiguousarray(np.zeros(16) if output_bias is None else output_bias, dtype=np.float32)
    blob = np.zeros(8608 if use_fp8 else 9472, dtype=np.uint8)
    rounded = np.empty_like(weights)
    if oracle_lib().ntco_quantize_network(weights.ctypes.data, biases.ctypes.data, scale.ctypes.data, bias.ctypes.data,
                                          int(use_fp8), blob.ctypes.data, rounded.ctypes.data) != 0:
        raise ValueError("ntco_quantize_network rejected its arguments")
    return blob.tobytes(), rounded


def block_compress(texels: np.ndarray, first_channel: int, format_channels: int, src_left: int = 0, src_top: int = 0,
                   width_in_blocks: Optional[int] = None, height_in_blocks: Optional[int] = None) -> np.ndarray:
    """BC4 (format_channels 1) / BC5 (2) encoding restated on the CPU (parity unpinned: the
    reference's encoders are compute shaders).  `texels`: [h][w][channels] float16.  Returns uint8
    [blocks_y][blocks_x][8 * format_channels]."""
    texels = np.ascontiguousarray(texels, dtype=np.float16)
    h, w, channels = texels.shape
    bw = (w - src_left + 3) // 4 if width_in_blocks is None else width_in_blocks
    bh = (h - src_top + 3) // 4 if height_in_blocks is None else height_in_blocks
    out = np.zeros((bh, bw, 8 * format_channels), dtype=np.uint8)
    if oracle_lib().ntco_block_compress(texels.ctypes.data, w, h, channels, first_channel, format_channels, src_left, src_top,
                                        bw, bh, out.ctypes.data) != 0:
        raise ValueError("ntco_block_compress rejected its arguments")
    return out


def block_compress_color(texels: np.ndarray, block_format: int, first_channel: int = 0, num_channels: Optional[int] = None,
                         alpha_threshold: float = 1.0 / 255.0, src_left: int = 0, src_top: int = 0,
                         width_in_blocks: Optional[int] = None, height_in_blocks: Optional[int] = None) -> np.ndarray:
    """BC1 / BC2 / BC3 (block_format 1 / 2 / 3) restated on the CPU (parity unpinned).  Returns uint8
    [blocks_y][blocks_x][8 or 16]."""
    texels = np.ascontiguousarray(texels, dtype=np.float16)
    h, w, channels = texels.shape
    n = (3 if block_format == 1 else 4) if num_channels is None else num_channels
    bw = (w - src_left + 3) // 4 if width_in_blocks is None else width_in_blocks
    bh = (h - src_top + 3) // 4 if height_in_blocks is None else height_in_blocks
    out = np.zeros((bh, bw, 8 if block_format == 1 else 16), dtype=np.uint8)
    if oracle_lib().ntco_block_compress_color(texels.ctypes.data, w, h, channels, first_channel, n, block_format,
                                              alpha_threshold, src_left, src_top, bw, bh, out.ctypes.data) != 0:
        raise ValueError("ntco_block_compress_color rejected its arguments")
    return out


def color_match_table(bits: int) -> np.ndarray:
    table = np.zeros(256, dtype=np.uint16)
    if oracle_lib().ntco_color_match_table(bits, table.ctypes.data) != 0:
        raise ValueError("bits must be 5 or 6")
    return table


def build_oracle() -> None:
    subprocess.run(["make", "-s", "-C", HERE, "libntc_oracle.so"], check=True)


def oracle_lib():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_LIB):
            build_oracle()
        lib = ctypes.CDLL(ORACLE_LIB)
        lib.ntco_geometry.argtypes = [ctypes.POINTER(_TextureSet), ctypes.POINTER(Geometry)]
        lib.ntco_decode_mip.argtypes = [ctypes.POINTER(_TextureSet), ctypes.POINTER(Options), ctypes.c_int,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.ntco_sample.argtypes = [ctypes.POINTER(_TextureSet), ctypes.POINTER(Options), ctypes.c_void_p,
                                    ctypes.c_size_t, ctypes.c_void_p]
        lib.ntco_read_channels.argtypes = [ctypes.c_void_p, ctypes.POINTER(ReadChannels), ctypes.c_void_p]
        lib.ntco_read_channels_resized.argtypes = [ctypes.c_void_p, ctypes.POINTER(ReadChannels), ctypes.c_int, ctypes.c_int,
                                                   ctypes.c_void_p]
        lib.ntco_pack_latents.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t,
                                          ctypes.c_void_p]
        lib.ntco_quantize_network.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        lib.ntco_block_compress.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 9 + [ctypes.c_void_p]
        lib.ntco_block_compress_color.argtypes = ([ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_float] + [ctypes.c_int] * 4
                                                  + [ctypes.c_void_p])
        lib.ntco_color_match_table.argtypes = [ctypes.c_int, ctypes.c_void_p]
        lib.ntco_float_to_half.restype = ctypes.c_uint16
        lib.ntco_float_to_half.argtypes = [ctypes.c_float]
        lib.ntco_half_to_float.restype = ctypes.c_float
        lib.ntco_half_to_float.argtypes = [ctypes.c_uint16]
        lib.ntco_half_to_e4m3.restype = ctypes.c_uint8
        lib.ntco_half_to_e4m3.argtypes = [ctypes.c_uint16]
        lib.ntco_e4m3_to_float.restype = ctypes.c_float
        lib.ntco_e4m3_to_float.argtypes = [ctypes.c_uint8]
        lib.ntco_hgelu_clamp_half.restype = ctypes.c_uint16
        lib.ntco_hgelu_clamp_half.argtypes = [ctypes.c_uint16]
        _oracle = lib
    return _oracle


class OracleSet:
    """A compressed texture set as the oracle sees it (arrays kept alive by this object)."""

    def __init__(self, geometry, packed_latents: np.ndarray, int8_blob: bytes, fp8_blob: bytes):
        self.geometry = geometry
        self._latents = np.ascontiguousarray(packed_latents, dtype=np.uint16)
        self._int8 = np.frombuffer(int8_blob, dtype=np.uint8).copy()
        self._fp8 = np.frombuffer(fp8_blob, dtype=np.uint8).copy()
        self.c = _TextureSet(geometry.width, geometry.height, geometry.channels, geometry.mips,
                             geometry.grid_scale, geometry.num_features, self._latents.ctypes.data,
                             self._int8.ctypes.data, self._fp8.ctypes.data)

    @classmethod
    def from_synthetic(cls, synthetic_set) -> "OracleSet":
        return cls(synthetic_set.geometry, synthetic_set.packed_latents(), synthetic_set.int8_blob,
                   synthetic_set.fp8_blob)

    def c_geometry(self) -> Geometry:
        out = Geometry()
        if oracle_lib().ntco_geometry(ctypes.byref(self.c), ctypes.byref(out)) != 0:
            raise ValueError("ntco_geometry rejected the texture set")
        return out

    def decode_mip(self, mip: int, use_int8: bool, numerics: int = NUMERICS_SPEC, y0: int = 0,
                   y1: Optional[int] = None, threads: int = 0, **ref_switches) -> np.ndarray:
        cm = self.geometry.color_mips[mip]
        y1 = cm.height if y1 is None else y1
        out = np.empty((y1 - y0, cm.width, self.geometry.channels), dtype=np.uint16)
        opt = make_options(use_int8, numerics, threads, **ref_switches)
        rc = oracle_lib().ntco_decode_mip(ctypes.byref(self.c), ctypes.byref(opt), mip, y0, y1, out.ctypes.data)
        if rc != 0:
            raise ValueError("ntco_decode_mip failed")
        return out.view(np.float16)

    def decode_all(self, use_int8: bool, numerics: int = NUMERICS_SPEC, threads: int = 0, **ref_switches) -> List[np.ndarray]:
        return [self.decode_mip(m, use_int8, numerics, threads=threads, **ref_switches) for m in range(self.geometry.mips)]

    def sample(self, queries: np.ndarray, use_int8: bool, numerics: int = NUMERICS_SPEC, threads: int = 0) -> np.ndarray:
        queries = np.ascontiguousarray(queries, dtype=np.float32)
        out = np.empty((queries.shape[0], self.geometry.channels), dtype=np.uint16)
        opt = make_options(use_int8, numerics, threads)
        rc = oracle_lib().ntco_sample(ctypes.byref(self.c), ctypes.byref(opt), queries.ctypes.data,
                                      queries.shape[0], out.ctypes.data)
        if rc != 0:
            raise ValueError("ntco_sample failed")
        return out.view(np.float16)


# Switches of the reference-emulating numerics that reproduce the reference kernel's outputs
# (see tests/golden/README.md for how they were pinned).
REF_DEFAULTS = dict(refBlendFma=2, refQuantFma=1, refAccChunk=16, refAccMode=25, refActFma=0)


def make_options(use_int8: bool, numerics: int, threads: int = 0, **ref_switches) -> Options:
    switches = dict(REF_DEFAULTS)
    switches.update(ref_switches)
    return Options(WEIGHTS_INT8 if use_int8 else WEIGHTS_FP8, numerics, threads, switches["refBlendFma"],
                   switches["refQuantFma"], switches["refAccChunk"], switches["refAccMode"], switches["refActFma"])


# ---------------------------------------------------------------------------------------------
# The unmodified reference library (needs a GPU to decode)
# ---------------------------------------------------------------------------------------------

# The reference with its CUDA decompression routed through libntcb200.so (build_ref.sh --with-ntcb):
# the same public API, the same harness, this repository's decoder behind ITextureSet::Decompress.
REF_NTCB_LIB = os.path.join(HERE, "_ref", "libntc_ref_ntcb.so")

# The reference's BC1 - BC5 compute shaders compiled for the CPU (build_ref.sh; no graphics API).
REF_BC_LIB = os.path.join(HERE, "_ref", "libntc_ref_bc.so")

_ref = {}
_ref_bc = None


def reference_bc_available() -> bool:
    return os.path.exists(REF_BC_LIB)


def reference_block_compress(block_format: int, rgba: np.ndarray, alpha_threshold: float = 1.0 / 255.0, src_left: int = 0,
                             src_top: int = 0, width_in_blocks: Optional[int] = None,
                             height_in_blocks: Optional[int] = None) -> np.ndarray:
    """Runs the reference's own CompressBC<n>.hlsl (n = block_format, 1..5) on the CPU over an RGBA binary32
    image [h][w][4] - what the shader's input texture holds - and returns uint8 [blocks_y][blocks_x][8 or 16]."""
    global _ref_bc
    if _ref_bc is None:
        _ref_bc = ctypes.CDLL(REF_BC_LIB)
    rgba = np.ascontiguousarray(rgba, dtype=np.float32)
    h, w, four = rgba.shape
    assert four == 4
    bw = (w - src_left + 3) // 4 if width_in_blocks is None else width_in_blocks
    bh = (h - src_top + 3) // 4 if height_in_blocks is None else height_in_blocks
    out = np.zeros((bh, bw, 8 if block_format in (1, 4) else 16), dtype=np.uint8)
    function = getattr(_ref_bc, "ntcref_block_compress_bc%d" % block_format)
    function.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_void_p]
    function(rgba.ctypes.data, w, h, src_left, src_top, bw, bh, alpha_threshold, out.ctypes.data)
    return out



def reference_block_compress_bc7(rgba: np.ndarray, mode_buffer: Optional[np.ndarray] = None, mode_buffer_byte_offset: int = 0,
                                 mode_map_size=None, mode_map_offset=(0, 0), src_left: int = 0, src_top: int = 0,
                                 width_in_blocks: Optional[int] = None, height_in_blocks: Optional[int] = None) -> np.ndarray:
    """Runs the reference's own CompressBC7.hlsl on the CPU over an RGBA binary32 image [h][w][4]: the
    full search, or with `mode_buffer` (uint8, the layout ntc::MakeBC7ModeBuffer writes) the shader built
    with USE_MODE_BUFFER.  Returns uint8 [blocks_y][blocks_x][16]."""
    global _ref_bc
    if _ref_bc is None:
        _ref_bc = ctypes.CDLL(REF_BC_LIB)
    rgba = np.ascontiguousarray(rgba, dtype=np.float32)
    h, w, four = rgba.shape
    assert four == 4
    bw = (w - src_left + 3) // 4 if width_in_blocks is None else width_in_blocks
    bh = (h - src_top + 3) // 4 if height_in_blocks is None else height_in_blocks
    out = np.zeros((bh, bw, 16), dtype=np.uint8)
    if mode_buffer is None:
        function = _ref_bc.ntcref_block_compress_bc7
        function.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_void_p]
        function(rgba.ctypes.data, w, h, src_left, src_top, bw, bh, 0.0, out.ctypes.data)
        return out
    # the shader reads whole 32-bit words, the second one of an entry also past the last entry's byte
    words = np.zeros((mode_buffer.nbytes + 3) // 4 + 2, dtype=np.uint32)
    words.view(np.uint8)[:mode_buffer.nbytes] = np.ascontiguousarray(mode_buffer, dtype=np.uint8).ravel()
    map_w, map_h = mode_map_size if mode_map_size is not None else (bw, bh)
    function = _ref_bc.ntcref_block_compress_bc7_modes
    function.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32,
                                                                 ctypes.c_uint32, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    function(rgba.ctypes.data, w, h, src_left, src_top, bw, bh, words.ctypes.data, mode_buffer_byte_offset, map_w, map_h,
             mode_map_offset[0], mode_map_offset[1], out.ctypes.data)
    return out


def reference_available() -> bool:
    return os.path.exists(REF_LIB)


def reference_ntcb_available() -> bool:
    return os.path.exists(REF_NTCB_LIB)


def reference_lib(path: str = REF_LIB):
    if path not in _ref:
        lib = ctypes.CDLL(path)
        lib.ntcref_last_error.restype = ctypes.c_char_p
        lib.ntcref_open.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                    ctypes.POINTER(ctypes.c_void_p)]
        lib.ntcref_probe_metadata.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_int)]
        lib.ntcref_decompress.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
        lib.ntcref_read_mip.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
        lib.ntcref_read_channels.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t,
                                             ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_void_p]
        lib.ntcref_close.argtypes = [ctypes.c_void_p]
        if hasattr(lib, "ntcref_probe_mode_buffer_footprint"):
            lib.ntcref_probe_mode_buffer_footprint.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                                               ctypes.POINTER(ctypes.c_uint64)]
        if hasattr(lib, "ntcref_make_bc7_mode_buffer"):
            lib.ntcref_bc7_mode_buffer_size.argtypes = [ctypes.c_int, ctypes.c_int]
            lib.ntcref_bc7_mode_buffer_size.restype = ctypes.c_size_t
            lib.ntcref_make_bc7_mode_buffer.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                                        ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t]
        lib.ntcref_producers_last_error.restype = ctypes.c_char_p
        lib.ntcref_pack_latents.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p,
                                            ctypes.c_size_t, ctypes.c_void_p]
        lib.ntcref_quantize_network.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        _ref[path] = lib
    return _ref[path]


def reference_probe(container: bytes) -> List[int]:
    out = (ctypes.c_int * 8)()
    lib = reference_lib()
    rc = lib.ntcref_probe_metadata(container, len(container), out)
    if rc != 0:
        raise RuntimeError("reference loader rejected the container: %s" % lib.ntcref_last_error().decode())
    return list(out)


def reference_mode_buffer_footprint(container: bytes, texture_index: int, mip_level: int):
    """(offset in the container, stored size, compression type) of a texture's BC7 mode bitmap as the
    reference's metadata loader reports it (no GPU needed)."""
    out = (ctypes.c_uint64 * 3)()
    lib = reference_lib()
    rc = lib.ntcref_probe_mode_buffer_footprint(container, len(container), texture_index, mip_level, out)
    if rc != 0:
        raise RuntimeError("reference loader: status %d %s" % (rc, lib.ntcref_last_error().decode()))
    return int(out[0]), int(out[1]), int(out[2])


def reference_make_bc7_mode_buffer(blocks: np.ndarray) -> np.ndarray:
    """ntc::MakeBC7ModeBuffer of the reference library on uint8 [blocks_y][blocks_x][16]."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    bh, bw = blocks.shape[:2]
    lib = reference_lib()
    out = np.zeros(lib.ntcref_bc7_mode_buffer_size(bw, bh), dtype=np.uint8)
    rc = lib.ntcref_make_bc7_mode_buffer(bw, bh, blocks.ctypes.data, blocks.nbytes, bw * 16, out.ctypes.data, out.nbytes)
    if rc != 0:
        raise RuntimeError("MakeBC7ModeBuffer failed: %s" % lib.ntcref_last_error().decode())
    return out


def reference_pack_latents(latents: np.ndarray, width: int, height: int, num_layers: int, latent_stride: int) -> np.ndarray:
    """The reference's own PackLatents kernel on a flat float16 array; uint16 [layers][height][width]."""
    latents = np.ascontiguousarray(latents, dtype=np.float16)
    out = np.empty((num_layers, height, width), dtype=np.uint16)
    lib = reference_lib()
    rc = lib.ntcref_pack_latents(width, height, num_layers, latent_stride, latents.ctypes.data, latents.size, out.ctypes.data)
    if rc != 0:
        raise RuntimeError("reference PackLatents failed: %s" % lib.ntcref_producers_last_error().decode())
    return out


def reference_quantize_network(weights: np.ndarray, biases: np.ndarray, use_fp8: bool, output_scale=None, output_bias=None):
    """The reference's own QuantizeNetwork kernel.  `weights` / `biases`: float16, the blob's order.
    Returns (blob bytes, rounded fp16 weights)."""
    weights = np.ascontiguousarray(weights, dtype=np.float16)
    biases = np.ascontiguousarray(biases, dtype=np.float16)
    scale = np.ascontiguousarray(np.ones(16) if output_scale is None else output_scale, dtype=np.float32)
    bias = np.ascontiguousarray(np.zeros(16) if output_bias is None else output_bias, dtype=np.float32)
    blob = np.zeros(8608 if use_fp8 else 9472, dtype=np.uint8)
    rounded = np.empty_like(weights)
    lib = reference_lib()
    rc = lib.ntcref_quantize_network(weights.ctypes.data, biases.ctypes.data, scale.ctypes.data, bias.ctypes.data,
                                     int(use_fp8), blob.ctypes.data, blob.size, rounded.ctypes.data)
    if rc != 0:
        raise RuntimeError("reference QuantizeNetwork failed: %s" % lib.ntcref_producers_last_error().decode())
    return blob.tobytes(), rounded


class ReferenceDecoder:
    """The reference's CUDA decompression of one container, through its public API."""

    def __init__(self, container: bytes, channels: int, device: int = 0, staging_bytes_per_pixel: Optional[int] = None,
                 library: str = REF_LIB):
        self._lib = reference_lib(library)
        self._container = container
        self._handle = ctypes.c_void_p()
        # the reference sizes its ReadChannels staging buffer from TextureSetFeatures::stagingBytesPerPixel
        staging = channels * 2 if staging_bytes_per_pixel is None else staging_bytes_per_pixel
        rc = self._lib.ntcref_open(container, len(container), device, staging, ctypes.byref(self._handle))
        if rc != 0:
            raise RuntimeError("reference open failed: %s" % self._lib.ntcref_last_error().decode())
        self.channels = channels

    def decompress(self, use_int8: bool) -> float:
        ms = ctypes.c_float()
        rc = self._lib.ntcref_decompress(self._handle, 1 if use_int8 else 0, ctypes.byref(ms))
        if rc != 0:
            raise RuntimeError("reference Decompress failed: %s" % self._lib.ntcref_last_error().decode())
        return float(ms.value)

    def read_mip_into(self, mip: int, width: int, height: int, address: int, to_device: bool) -> None:
        rc = self._lib.ntcref_read_mip(self._handle, mip, 0, self.channels, width, height, address, 1 if to_device else 0)
        if rc != 0:
            raise RuntimeError("reference ReadChannels failed: %s" % self._lib.ntcref_last_error().decode())

    def read_mip(self, mip: int, width: int, height: int) -> np.ndarray:
        out = np.empty((height, width, self.channels), dtype=np.float16)
        self.read_mip_into(mip, width, height, out.ctypes.data, False)
        return out

    def read_channels_into(self, mip: int, width: int, height: int, channel_format: int, components: int, address: int) -> None:
        """ReadChannels of every channel, linear, undithered, tightly packed, to host memory at `address`."""
        item = np.dtype(FORMAT_DTYPES[channel_format]).itemsize
        rc = self._lib.ntcref_read_channels(self._handle, mip, 0, self.channels, width, height, channel_format,
                                            components * item, components * item * width, None, 0, address)
        if rc != 0:
            raise RuntimeError("reference ReadChannels failed: %s" % self._lib.ntcref_last_error().decode())

    def read_channels(self, mip: int, width: int, height: int, channel_format: int, first_channel: int = 0,
                      num_channels: Optional[int] = None, components: Optional[int] = None, dst_color_spaces=None,
                      use_dithering: bool = False) -> np.ndarray:
        """ITextureSet::ReadChannels of the reference in any channel format, to host memory."""
        n = self.channels - first_channel if num_channels is None else num_channels
        count = n if components is None else components
        dtype = np.dtype(FORMAT_DTYPES[channel_format])
        out = np.zeros((height, width, count), dtype=dtype)
        spaces = None
        if dst_color_spaces is not None:
            spaces = (ctypes.c_int * n)(*dst_color_spaces)
        rc = self._lib.ntcref_read_channels(self._handle, mip, first_channel, n, width, height, channel_format,
                                            count * dtype.itemsize, count * dtype.itemsize * width, spaces,
                                            1 if use_dithering else 0, out.ctypes.data)
        if rc != 0:
            raise RuntimeError("reference ReadChannels failed: %s" % self._lib.ntcref_last_error().decode())
        return out

    def close(self) -> None:
        if self._handle:
            self._lib.ntcref_close(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
