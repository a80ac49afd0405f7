"""ctypes bindings of the C ABI in include/ntcb.h (libntcb200.so) and a thin decoder object that
keeps a texture set resident on one GPU.

PyTorch is used only for device memory and streams; every computation goes through the C ABI.
If the shared library is missing or cannot be loaded the import of this module fails: there is no
fallback path.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence, Tuple

import numpy as np

from .geometry import FP8_BLOB_BYTES, INT8_BLOB_BYTES, Geometry

_HERE = os.path.dirname(os.path.abspath(__file__))
# NTCB_LIBRARY selects another build of the library (the profiling variants `make ablations` produces)
LIBRARY_PATH = os.environ.get("NTCB_LIBRARY") or os.path.join(_HERE, "libntcb200.so")

MAX_MIPS = 16
DEFAULT_WAIT_POLLS = 1 << 20  # NTCB_DEFAULT_WAIT_POLLS
STAGED_NETWORK_BYTES = 14864
STAGED_REFERENCE_NETWORK_BYTES = 21504
LATENTS_PLANAR, LATENTS_INTERLEAVED = 0, 1
NUMERICS_REFERENCE, NUMERICS_EXACT = 0, 1  # NtcbNumerics: the reference's binary16 accumulation (default) / exact accumulation
STATUS_WORDS = 4
WEIGHTS_INT8, WEIGHTS_FP8 = 0, 1
LAYOUT_PLANAR_PAIRS, LAYOUT_INTERLEAVED = 0, 1


class MipDesc(ctypes.Structure):
    _fields_ = [("width", ctypes.c_int32), ("height", ctypes.c_int32),
                ("hiWidth", ctypes.c_int32), ("hiHeight", ctypes.c_int32),
                ("loWidth", ctypes.c_int32), ("loHeight", ctypes.c_int32),
                ("hiOffset", ctypes.c_uint64), ("loOffset", ctypes.c_uint64),
                ("hiPlane", ctypes.c_uint64), ("loPlane", ctypes.c_uint64),
                ("positionScale", ctypes.c_float), ("positionLod", ctypes.c_float),
                ("outOffset", ctypes.c_uint64),
                ("rowBegin", ctypes.c_int32), ("rowEnd", ctypes.c_int32)]


class OutputConversion(ctypes.Structure):
    _fields_ = [("channelFormat", ctypes.c_int32), ("components", ctypes.c_int32),
                ("firstChannel", ctypes.c_int32), ("numChannels", ctypes.c_int32),
                ("useDithering", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("srcColorSpaces", ctypes.c_uint8 * 16), ("dstColorSpaces", ctypes.c_uint8 * 16)]


def make_conversion(channel_format: int, num_channels: int, first_channel: int = 0, components: Optional[int] = None,
                    src_color_spaces=None, dst_color_spaces=None, use_dithering: bool = False) -> OutputConversion:
    """Channels [first_channel, first_channel + num_channels) -> pixels of `components` values
    (default num_channels) of `channel_format`; colour spaces are given per requested channel."""
    conversion = OutputConversion()
    conversion.channelFormat = channel_format
    conversion.components = num_channels if components is None else components
    conversion.firstChannel, conversion.numChannels = first_channel, num_channels
    conversion.useDithering = 1 if use_dithering else 0
    for i, space in enumerate(src_color_spaces or []):
        conversion.srcColorSpaces[i] = space
    for i, space in enumerate(dst_color_spaces or []):
        conversion.dstColorSpaces[i] = space
    return conversion


class DecodeParams(ctypes.Structure):
    _fields_ = [("latents", ctypes.c_void_p), ("network", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("status", ctypes.c_void_p),
                ("numMips", ctypes.c_int32), ("numFeatures", ctypes.c_int32), ("channels", ctypes.c_int32),
                ("weightMode", ctypes.c_int32), ("outputLayout", ctypes.c_int32), ("numerics", ctypes.c_int32),
                ("mips", MipDesc * MAX_MIPS), ("conversion", ctypes.POINTER(OutputConversion))]


class ConvertParams(ctypes.Structure):
    _fields_ = [("deviceMip", ctypes.c_void_p), ("layout", ctypes.c_int32), ("width", ctypes.c_int32),
                ("height", ctypes.c_int32), ("channels", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("deviceDestination", ctypes.c_void_p), ("pixelStride", ctypes.c_size_t), ("rowPitch", ctypes.c_size_t),
                ("conversion", OutputConversion), ("dstWidth", ctypes.c_int32), ("dstHeight", ctypes.c_int32)]


class SampleParams(ctypes.Structure):
    _fields_ = [("latents", ctypes.c_void_p), ("network", ctypes.c_void_p), ("queries", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("status", ctypes.c_void_p), ("numQueries", ctypes.c_uint64),
                ("numMips", ctypes.c_int32), ("numFeatures", ctypes.c_int32), ("channels", ctypes.c_int32),
                ("weightMode", ctypes.c_int32), ("numerics", ctypes.c_int32), ("latentLayout", ctypes.c_int32),
                ("mips", MipDesc * MAX_MIPS)]


class TextureSetDesc(ctypes.Structure):
    _fields_ = [("width", ctypes.c_int32), ("height", ctypes.c_int32), ("channels", ctypes.c_int32),
                ("mips", ctypes.c_int32), ("gridSizeScale", ctypes.c_int32), ("numFeatures", ctypes.c_int32),
                ("numNeuralMips", ctypes.c_int32), ("numLayers", ctypes.c_int32), ("totalTexels", ctypes.c_uint64)]


class TextureDesc(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 128), ("firstChannel", ctypes.c_int32), ("numChannels", ctypes.c_int32),
                ("channelFormat", ctypes.c_int32), ("blockCompressedFormat", ctypes.c_int32),
                ("rgbColorSpace", ctypes.c_int32), ("alphaColorSpace", ctypes.c_int32)]

    def as_dict(self) -> dict:
        return {"name": self.name.decode(), "firstChannel": self.firstChannel, "numChannels": self.numChannels,
                "channelFormat": self.channelFormat, "blockCompressedFormat": self.blockCompressedFormat,
                "rgbColorSpace": self.rgbColorSpace, "alphaColorSpace": self.alphaColorSpace}


class TextureSetFeatures(ctypes.Structure):
    _fields_ = [("outputLayout", ctypes.c_int32), ("numerics", ctypes.c_int32)]


class DecompressionStats(ctypes.Structure):
    _fields_ = [("gpuTimeMilliseconds", ctypes.c_float)]


class ReadChannelsParams(ctypes.Structure):
    _fields_ = [("mipLevel", ctypes.c_int32), ("firstChannel", ctypes.c_int32), ("numChannels", ctypes.c_int32),
                ("addressSpace", ctypes.c_int32), ("pOutData", ctypes.c_void_p),
                ("width", ctypes.c_int32), ("height", ctypes.c_int32),
                ("channelFormat", ctypes.c_int32), ("useDithering", ctypes.c_int32),
                ("pixelStride", ctypes.c_size_t), ("rowPitch", ctypes.c_size_t),
                ("dstColorSpaces", ctypes.POINTER(ctypes.c_int32))]


ADDRESS_SPACE_HOST, ADDRESS_SPACE_DEVICE = 0, 1
# ntc::ChannelFormat and ntc::ColorSpace values
CHANNEL_FORMAT_UNORM8, CHANNEL_FORMAT_UNORM16, CHANNEL_FORMAT_FLOAT16, CHANNEL_FORMAT_FLOAT32, CHANNEL_FORMAT_UINT32 = 1, 2, 3, 4, 5
COLOR_SPACE_LINEAR, COLOR_SPACE_SRGB, COLOR_SPACE_HLG = 0, 1, 2
CHANNEL_FORMAT_DTYPES = {CHANNEL_FORMAT_UNORM8: np.uint8, CHANNEL_FORMAT_UNORM16: np.uint16, CHANNEL_FORMAT_FLOAT16: np.float16,
                         CHANNEL_FORMAT_FLOAT32: np.float32, CHANNEL_FORMAT_UINT32: np.uint32}


class BatchItem(ctypes.Structure):
    """NtcbBatchItem: one texture set of a multi-device batch."""
    _fields_ = [("container", ctypes.c_void_p), ("containerBytes", ctypes.c_size_t), ("hostTexels", ctypes.c_void_p),
                ("hostTexelsBytes", ctypes.c_size_t), ("useInt8Weights", ctypes.c_int32), ("status", ctypes.c_int32)]


class BatchUnit(ctypes.Structure):
    """NtcbBatchUnit: rows [rowBegin[m], rowEnd[m]) of every mip m of one item."""
    _fields_ = [("item", ctypes.c_int32), ("device", ctypes.c_int32), ("attempts", ctypes.c_int32), ("status", ctypes.c_int32),
                ("rowBegin", ctypes.c_int32 * MAX_MIPS), ("rowEnd", ctypes.c_int32 * MAX_MIPS), ("texels", ctypes.c_uint64)]


BATCH_WORKER = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(BatchUnit))


class BatchOptions(ctypes.Structure):
    """NtcbBatchOptions."""
    _fields_ = [("numerics", ctypes.c_int32), ("maxAttempts", ctypes.c_int32), ("unitsPerDevice", ctypes.c_int32),
                ("workersPerDevice", ctypes.c_int32), ("worker", BATCH_WORKER), ("workerUser", ctypes.c_void_p)]


class NtcbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__("%s (%d): %s" % (lib().ntcb_status_string(code).decode(), code, message))
        self.code = code


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise ImportError("libntcb200.so is not built; run __graft_entry__.build() "
                              "(make -C rtxntc-library_b200/csrc)")
        handle = ctypes.CDLL(LIBRARY_PATH)
        handle.ntcb_last_error.restype = ctypes.c_char_p
        handle.ntcb_status_string.restype = ctypes.c_char_p
        handle.ntcb_status_string.argtypes = [ctypes.c_int]
        handle.ntcb_launch_count.restype = ctypes.c_uint64
        handle.ntcb_debug_set_network_wait_polls.restype = ctypes.c_uint32
        handle.ntcb_debug_set_network_wait_polls.argtypes = [ctypes.c_uint32]
        handle.ntcb_stage_network.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        handle.ntcb_stage_network_reference.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
        handle.ntcb_decode.argtypes = [ctypes.POINTER(DecodeParams), ctypes.c_void_p]
        handle.ntcb_sample.argtypes = [ctypes.POINTER(SampleParams), ctypes.c_void_p]
        handle.ntcb_texture_set_sample.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int]
        handle.ntcb_interleave_latents.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(MipDesc), ctypes.c_int,
                                                   ctypes.c_int, ctypes.c_void_p]
        handle.ntcb_decode_resident_ctas.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        handle.ntcb_probe_container.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(TextureSetDesc)]
        handle.ntcb_probe_container_texture.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.POINTER(TextureDesc),
                                                        ctypes.POINTER(ctypes.c_int)]
        handle.ntcb_texture_set_get_texture.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(TextureDesc),
                                                        ctypes.POINTER(ctypes.c_int)]
        handle.ntcb_context_create.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]
        handle.ntcb_context_destroy.argtypes = [ctypes.c_void_p]
        handle.ntcb_context_destroy.restype = None
        handle.ntcb_batch_decoder_create.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.POINTER(BatchOptions),
                                                     ctypes.POINTER(ctypes.c_void_p)]
        handle.ntcb_batch_decoder_run.argtypes = [ctypes.c_void_p, ctypes.POINTER(BatchItem), ctypes.c_int, ctypes.POINTER(BatchUnit),
                                                  ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        handle.ntcb_batch_decoder_destroy.argtypes = [ctypes.c_void_p]
        handle.ntcb_batch_decoder_destroy.restype = None
        handle.ntcb_texture_set_load_from_memory.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
        handle.ntcb_texture_set_create_from_memory.argtypes = [
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(TextureSetFeatures),
            ctypes.POINTER(ctypes.c_void_p)]
        handle.ntcb_texture_set_create_from_file.argtypes = [
            ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(TextureSetFeatures), ctypes.POINTER(ctypes.c_void_p)]
        handle.ntcb_texture_set_destroy.argtypes = [ctypes.c_void_p]
        handle.ntcb_texture_set_destroy.restype = None
        handle.ntcb_texture_set_get_desc.argtypes = [ctypes.c_void_p, ctypes.POINTER(TextureSetDesc)]
        handle.ntcb_texture_set_decompress.argtypes = [ctypes.c_void_p, ctypes.POINTER(DecompressionStats), ctypes.c_int]
        handle.ntcb_texture_set_decompress_rows.argtypes = [
            ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(DecompressionStats), ctypes.c_int]
        handle.ntcb_texture_set_read_channels.argtypes = [ctypes.c_void_p, ctypes.POINTER(ReadChannelsParams)]
        handle.ntcb_texture_set_decompress_converted.argtypes = [
            ctypes.c_void_p, ctypes.POINTER(DecompressionStats), ctypes.c_int, ctypes.POINTER(OutputConversion), ctypes.c_int,
            ctypes.c_void_p, ctypes.c_size_t]
        handle.ntcb_convert_channels.argtypes = [ctypes.POINTER(ConvertParams), ctypes.c_void_p]
        handle.ntcb_pack_latents.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t,
                                             ctypes.c_void_p, ctypes.c_void_p]
        handle.ntcb_quantize_network.argtypes = [ctypes.POINTER(QuantizeNetworkParams), ctypes.c_void_p]
        handle.ntcb_block_compress.argtypes = [ctypes.POINTER(BlockCompressParams), ctypes.c_void_p]
        handle.ntcb_probe_container_bc7_mode_buffer.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                                                ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64),
                                                                ctypes.POINTER(ctypes.c_int)]
        handle.ntcb_texture_set_get_bc7_mode_buffer.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                                                ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_size_t)]
        handle.ntcb_texture_set_make_and_store_bc7_mode_buffer.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                                           ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
        handle.ntcb_texture_set_block_compress_texture.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                                                   ctypes.c_void_p, ctypes.c_size_t]
        handle.ntcb_bc7_mode_buffer_size.argtypes = [ctypes.c_int, ctypes.c_int]
        handle.ntcb_bc7_mode_buffer_size.restype = ctypes.c_size_t
        handle.ntcb_make_bc7_mode_buffer.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t,
                                                     ctypes.c_void_p, ctypes.c_size_t]
        handle.ntcb_texture_set_block_compress.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                           ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t]
        handle.ntcb_texture_set_device_mip.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_size_t)]
        handle.ntcb_texture_set_synchronize.argtypes = [ctypes.c_void_p]
        handle.ntcb_read_channels_to_host_noalloc.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p]
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise NtcbError(code, lib().ntcb_last_error().decode())


def stage_network(blob: bytes, weight_mode: int, numerics: int = NUMERICS_REFERENCE) -> np.ndarray:
    """Host-side conversion of a GenericInt8 / GenericFP8 blob into the image of the kernel that
    implements `numerics`."""
    source = np.frombuffer(blob, dtype=np.uint8)
    if numerics == NUMERICS_REFERENCE:
        staged = np.zeros(STAGED_REFERENCE_NETWORK_BYTES, dtype=np.uint8)
        check(lib().ntcb_stage_network_reference(source.ctypes.data, len(blob), weight_mode, staged.ctypes.data))
        return staged
    staged = np.zeros(STAGED_NETWORK_BYTES, dtype=np.uint8)
    check(lib().ntcb_stage_network(source.ctypes.data, len(blob), weight_mode, staged.ctypes.data))
    return staged


def probe_container(container: bytes) -> TextureSetDesc:
    """Host-only validation of an NTC container; raises NtcbError with the loader's message."""
    desc = TextureSetDesc()
    buffer = np.frombuffer(container, dtype=np.uint8)
    check(lib().ntcb_probe_container(buffer.ctypes.data, len(container), ctypes.byref(desc)))
    return desc


def probe_bc7_mode_buffer(container: bytes, texture_index: int, mip_level: int):
    """(offset in the container, stored size, compressed?) of a texture's BC7 mode bitmap; (0, 0, False) when the
    container keeps none.  No GPU needed."""
    offset, stored, compressed = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_int()
    check(lib().ntcb_probe_container_bc7_mode_buffer(container, len(container), texture_index, mip_level, ctypes.byref(offset),
                                                     ctypes.byref(stored), ctypes.byref(compressed)))
    return int(offset.value), int(stored.value), bool(compressed.value)


def probe_textures(container: bytes) -> list:
    """The texture headers of a container (host only): a list of dictionaries."""
    buffer = np.frombuffer(container, dtype=np.uint8)
    count = ctypes.c_int()
    code = lib().ntcb_probe_container_texture(buffer.ctypes.data, len(container), -1, None, ctypes.byref(count))
    if code != -9:  # index -1 is out of range by design once the container has loaded
        check(code)
    textures = []
    for index in range(count.value):
        desc = TextureDesc()
        check(lib().ntcb_probe_container_texture(buffer.ctypes.data, len(container), index, ctypes.byref(desc), None))
        textures.append(desc.as_dict())
    return textures


def out_elements(geo: Geometry) -> int:
    return geo.total_texels * geo.channels


def fill_params(geo: Geometry, latents_ptr: int, network_ptr: int, out_ptr: int, status_ptr: int, weight_mode: int,
                layout: int = LAYOUT_INTERLEAVED, mips: Optional[Sequence[int]] = None,
                row_ranges: Optional[dict] = None, conversion: Optional[OutputConversion] = None) -> DecodeParams:
    """Describes a decode of `mips` (default: all) of a texture set whose latents are resident in
    the reference's encoded-pixel order.  `row_ranges` maps mip -> (rowBegin, rowEnd).  With
    `conversion` the kernel writes converted pixels (mip after mip, no padding) instead of fp16."""
    params = DecodeParams()
    if conversion is not None:
        params._conversion = conversion  # keeps the pointee alive as long as the parameters
        params.conversion = ctypes.pointer(conversion)
    params.latents = latents_ptr
    params.network = network_ptr
    params.out = out_ptr
    params.status = status_ptr
    params.numFeatures = geo.num_features
    params.channels = geo.channels
    params.weightMode = weight_mode
    params.outputLayout = layout
    selected = list(range(geo.mips)) if mips is None else list(mips)
    params.numMips = len(selected)
    for slot, mip in enumerate(selected):
        cm = geo.color_mips[mip]
        lod = cm.neural_lod
        d = params.mips[slot]
        d.width, d.height = cm.width, cm.height
        d.hiWidth, d.hiHeight = geo.latent_width[lod], geo.latent_height[lod]
        d.loWidth, d.loHeight = geo.latent_width[lod + 1], geo.latent_height[lod + 1]
        d.hiOffset = geo.latent_pixel_offset[lod] * geo.num_layers
        d.loOffset = geo.latent_pixel_offset[lod + 1] * geo.num_layers
        d.hiPlane = d.hiWidth * d.hiHeight
        d.loPlane = d.loWidth * d.loHeight
        d.positionScale, d.positionLod = cm.position_scale, cm.position_lod
        d.outOffset = cm.texel_offset * (geo.channels if conversion is None else conversion.components)
        begin, end = (0, cm.height) if not row_ranges or mip not in row_ranges else row_ranges[mip]
        d.rowBegin, d.rowEnd = begin, end
    return params


def convert_channels(texels, conversion: OutputConversion, layout: int = LAYOUT_INTERLEAVED, width: Optional[int] = None,
                     height: Optional[int] = None, channels: Optional[int] = None, size: Optional[Tuple[int, int]] = None):
    """Runs the ReadChannels conversion kernel on decoded texels that the caller holds: `texels` is
    a CUDA float16 tensor, [height][width][channels] for the interleaved layout (the sizes are then
    taken from its shape).  Returns a CUDA tensor [height][width][components] of the channel
    format's element type (uint16 / uint32 data as int16 / int32 bit patterns)."""
    import torch

    if layout == LAYOUT_INTERLEAVED and width is None:
        height, width, channels = texels.shape
    dtype = {CHANNEL_FORMAT_UNORM8: torch.uint8, CHANNEL_FORMAT_UNORM16: torch.int16, CHANNEL_FORMAT_FLOAT16: torch.float16,
             CHANNEL_FORMAT_FLOAT32: torch.float32, CHANNEL_FORMAT_UINT32: torch.int32}[conversion.channelFormat]
    out_width, out_height = (width, height) if size is None else size  # another size: bilinear resize
    out = torch.zeros((out_height, out_width, conversion.components), dtype=dtype, device=texels.device)
    params = ConvertParams()
    params.deviceMip = texels.data_ptr()
    params.layout, params.width, params.height, params.channels = layout, width, height, channels
    params.deviceDestination = out.data_ptr()
    params.pixelStride = conversion.components * out.element_size()
    params.rowPitch = params.pixelStride * out_width
    params.conversion = conversion
    if size is not None:
        params.dstWidth, params.dstHeight = size
    with torch.cuda.device(texels.device):
        stream = torch.cuda.current_stream(texels.device).cuda_stream
        check(lib().ntcb_convert_channels(ctypes.byref(params), ctypes.c_void_p(stream)))
    return out


class QuantizeNetworkParams(ctypes.Structure):
    _fields_ = [("weights", ctypes.c_void_p), ("biases", ctypes.c_void_p),
                ("outputScale", ctypes.POINTER(ctypes.c_float)), ("outputBias", ctypes.POINTER(ctypes.c_float)),
                ("weightMode", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("blob", ctypes.c_void_p), ("roundedWeights", ctypes.c_void_p)]


NETWORK_WEIGHT_COUNT = 48 * 64 + 64 * 48 + 48 * 32 + 32 * 16
NETWORK_COLUMN_COUNT = 64 + 48 + 32 + 16


def pack_latents(latents, width: int, height: int, num_layers: int, latent_stride: int):
    """Packs quantised fp16 latents (a flat CUDA float16 tensor in the reference's layout: layer z,
    texel t has features 0-1 at z * latent_stride * 2 + t * 2 and features 2-3 latent_stride
    elements later) into 16-bit words; returns a CUDA int16 tensor [num_layers][height][width]."""
    import torch

    needed = (num_layers - 1) * latent_stride * 2 + latent_stride + width * height * 2
    if latents.dtype != torch.float16 or latents.numel() < needed:
        raise ValueError(f"latents must be float16 with at least {needed} elements")
    out = torch.empty((num_layers, height, width), dtype=torch.int16, device=latents.device)
    with torch.cuda.device(latents.device):
        stream = torch.cuda.current_stream(latents.device).cuda_stream
        check(lib().ntcb_pack_latents(ctypes.c_void_p(latents.data_ptr()), width, height, num_layers, latent_stride,
                                      ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream)))
    return out


def quantize_network(weights, biases, weight_mode: int, output_scale=None, output_bias=None, want_rounded: bool = False):
    """Quantises fp16 network weights (CUDA float16 tensors: NETWORK_WEIGHT_COUNT weights, per layer
    outputs x inputs with one output's inputs together, and NETWORK_COLUMN_COUNT biases) to a
    GenericInt8 / GenericFP8 blob.  Returns the blob as a CUDA uint8 tensor, and with `want_rounded`
    also the fp16 weights as the decoder will apply them."""
    import torch

    if weights.dtype != torch.float16 or weights.numel() != NETWORK_WEIGHT_COUNT:
        raise ValueError("weights must be float16 with NETWORK_WEIGHT_COUNT elements")
    if biases.dtype != torch.float16 or biases.numel() != NETWORK_COLUMN_COUNT:
        raise ValueError("biases must be float16 with NETWORK_COLUMN_COUNT elements")
    blob_bytes = INT8_BLOB_BYTES if weight_mode == WEIGHTS_INT8 else FP8_BLOB_BYTES
    blob = torch.zeros(blob_bytes, dtype=torch.uint8, device=weights.device)
    rounded = torch.empty_like(weights) if want_rounded else None
    params = QuantizeNetworkParams()
    params.weights, params.biases = weights.data_ptr(), biases.data_ptr()
    keep = []
    for name, values in (("outputScale", output_scale), ("outputBias", output_bias)):
        if values is not None:
            array = (ctypes.c_float * 16)(*[float(v) for v in values])
            keep.append(array)
            setattr(params, name, array)
    params.weightMode = weight_mode
    params.blob = blob.data_ptr()
    params.roundedWeights = rounded.data_ptr() if want_rounded else None
    with torch.cuda.device(weights.device):
        stream = torch.cuda.current_stream(weights.device).cuda_stream
        check(lib().ntcb_quantize_network(ctypes.byref(params), ctypes.c_void_p(stream)))
    return (blob, rounded) if want_rounded else blob


BLOCK_FORMAT_BC1, BLOCK_FORMAT_BC2, BLOCK_FORMAT_BC3, BLOCK_FORMAT_BC4, BLOCK_FORMAT_BC5 = 1, 2, 3, 4, 5
BLOCK_FORMAT_BC7 = 7


class BlockCompressParams(ctypes.Structure):
    _fields_ = [("deviceMip", ctypes.c_void_p), ("layout", ctypes.c_int32), ("width", ctypes.c_int32),
                ("height", ctypes.c_int32), ("channels", ctypes.c_int32), ("firstChannel", ctypes.c_int32),
                ("format", ctypes.c_int32), ("srcLeft", ctypes.c_int32), ("srcTop", ctypes.c_int32),
                ("widthInBlocks", ctypes.c_int32), ("heightInBlocks", ctypes.c_int32), ("numChannels", ctypes.c_int32),
                ("deviceBlocks", ctypes.c_void_p), ("rowPitch", ctypes.c_size_t), ("alphaThreshold", ctypes.c_float),
                ("reserved", ctypes.c_int32), ("deviceModeBuffer", ctypes.c_void_p),
                ("modeBufferByteOffset", ctypes.c_uint32), ("modeMapWidthInBlocks", ctypes.c_uint32),
                ("modeMapHeightInBlocks", ctypes.c_uint32), ("modeMapOffsetX", ctypes.c_int32),
                ("modeMapOffsetY", ctypes.c_int32), ("reserved2", ctypes.c_int32)]


def bc7_mode_buffer_size(width_in_blocks: int, height_in_blocks: int) -> int:
    return int(lib().ntcb_bc7_mode_buffer_size(width_in_blocks, height_in_blocks))


def make_bc7_mode_buffer(blocks: np.ndarray, row_pitch: Optional[int] = None) -> np.ndarray:
    """The 9-bit-per-block mode bitmap of BC7 blocks (uint8 [blocks_y][blocks_x][16], or rows of `row_pitch`
    bytes): uint8 of bc7_mode_buffer_size() bytes (ntc::MakeBC7ModeBuffer)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    bh, bw = blocks.shape[0], blocks.shape[1] if blocks.ndim == 3 else blocks.shape[1] // 16
    if blocks.ndim == 3:
        row_pitch = bw * 16
    out = np.full(bc7_mode_buffer_size(bw, bh), 0xAA, dtype=np.uint8)  # the call clears it
    check(lib().ntcb_make_bc7_mode_buffer(bw, bh, blocks.ctypes.data, blocks.nbytes, row_pitch, out.ctypes.data, out.nbytes))
    return out


def block_compress(texels, block_format: int, first_channel: int = 0, layout: int = LAYOUT_INTERLEAVED,
                   width: Optional[int] = None, height: Optional[int] = None, channels: Optional[int] = None,
                   src_left: int = 0, src_top: int = 0, width_in_blocks: Optional[int] = None,
                   height_in_blocks: Optional[int] = None, num_channels: int = 0, alpha_threshold: float = 1.0 / 255.0,
                   mode_buffer=None, mode_buffer_byte_offset: int = 0, mode_map_size=None, mode_map_offset=(0, 0)):
    """BC1 - BC5 and BC7 encoding of decoded texels the caller holds: `texels` is a CUDA float16 tensor,
    [height][width][channels] for the interleaved layout (sizes then come from its shape).  Returns a
    CUDA uint8 tensor [blocks_y][blocks_x][8 or 16].  BC7: `mode_buffer` (a CUDA uint8 tensor laid out as
    make_bc7_mode_buffer does, for a block grid of `mode_map_size` = (width, height) in blocks, default the
    destination's) selects the one-mode-per-block path."""
    import torch

    if layout == LAYOUT_INTERLEAVED and width is None:
        height, width, channels = texels.shape
    bw = (width - src_left + 3) // 4 if width_in_blocks is None else width_in_blocks
    bh = (height - src_top + 3) // 4 if height_in_blocks is None else height_in_blocks
    block_bytes = 8 if block_format in (BLOCK_FORMAT_BC1, BLOCK_FORMAT_BC4) else 16
    out = torch.zeros((bh, bw, block_bytes), dtype=torch.uint8, device=texels.device)
    params = BlockCompressParams()
    params.deviceMip = texels.data_ptr()
    params.layout, params.width, params.height, params.channels = layout, width, height, channels
    params.firstChannel, params.format = first_channel, block_format
    params.srcLeft, params.srcTop, params.widthInBlocks, params.heightInBlocks = src_left, src_top, bw, bh
    params.deviceBlocks = out.data_ptr()
    params.rowPitch = bw * block_bytes
    params.numChannels, params.alphaThreshold = num_channels, alpha_threshold
    if mode_buffer is not None:
        params.deviceModeBuffer = mode_buffer.data_ptr()
        params.modeBufferByteOffset = mode_buffer_byte_offset
        params.modeMapWidthInBlocks, params.modeMapHeightInBlocks = mode_map_size if mode_map_size is not None else (bw, bh)
        params.modeMapOffsetX, params.modeMapOffsetY = mode_map_offset
    with torch.cuda.device(texels.device):
        stream = torch.cuda.current_stream(texels.device).cuda_stream
        check(lib().ntcb_block_compress(ctypes.byref(params), ctypes.c_void_p(stream)))
    return out


class ResidentTextureSet:
    """A compressed texture set uploaded to one GPU: packed latents, both staged networks, an
    output buffer for the whole mip chain and the status words."""

    def __init__(self, geo: Geometry, packed_latents: np.ndarray, int8_blob: bytes, fp8_blob: bytes,
                 device: str = "cuda:0", layout: int = LAYOUT_INTERLEAVED, allocate_output: bool = True,
                 numerics: int = NUMERICS_REFERENCE):
        import torch

        self.torch = torch
        self.geometry = geo
        self.device = torch.device(device)
        self.layout = layout
        lib()
        self.latents = torch.from_numpy(np.ascontiguousarray(packed_latents).view(np.int16)).to(self.device)
        self.numerics = numerics
        self.networks = {
            WEIGHTS_INT8: torch.from_numpy(stage_network(int8_blob, WEIGHTS_INT8, numerics)).to(self.device),
            WEIGHTS_FP8: torch.from_numpy(stage_network(fp8_blob, WEIGHTS_FP8, numerics)).to(self.device),
        }
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=self.device)
        self.out = torch.empty(out_elements(geo), dtype=torch.float16, device=self.device) if allocate_output else None

    @classmethod
    def from_synthetic(cls, synthetic_set, **kwargs) -> "ResidentTextureSet":
        return cls(synthetic_set.geometry, synthetic_set.packed_latents(), synthetic_set.int8_blob,
                   synthetic_set.fp8_blob, **kwargs)

    def params(self, use_int8: bool, out=None, mips=None, row_ranges=None, conversion=None) -> DecodeParams:
        mode = WEIGHTS_INT8 if use_int8 else WEIGHTS_FP8
        out = self.out if out is None else out
        params = fill_params(self.geometry, self.latents.data_ptr(), self.networks[mode].data_ptr(), out.data_ptr(),
                             self.status.data_ptr(), mode, self.layout, mips, row_ranges, conversion)
        params.numerics = self.numerics
        return params

    def decode_converted(self, use_int8: bool, conversion: OutputConversion, mips=None, row_ranges=None):
        """Decode with the converting epilogue into a fresh device buffer covering the whole mip
        chain; returns it as a flat CUDA tensor of the channel format's element type (uint32 data
        comes back as int32 bit patterns)."""
        torch = self.torch
        dtype = {CHANNEL_FORMAT_UNORM8: torch.uint8, CHANNEL_FORMAT_UNORM16: torch.int16, CHANNEL_FORMAT_FLOAT16: torch.float16,
                 CHANNEL_FORMAT_FLOAT32: torch.float32, CHANNEL_FORMAT_UINT32: torch.int32}[conversion.channelFormat]
        out = torch.zeros(self.geometry.total_texels * conversion.components, dtype=dtype, device=self.device)
        with torch.cuda.device(self.device):
            self.launch(self.params(use_int8, out=out, mips=mips, row_ranges=row_ranges, conversion=conversion))
        return out

    def launch(self, params: DecodeParams) -> None:
        """Queues one decode on torch's current stream of this device."""
        stream = self.torch.cuda.current_stream(self.device).cuda_stream
        check(lib().ntcb_decode(ctypes.byref(params), ctypes.c_void_p(stream)))

    def decode(self, use_int8: bool, mips=None, row_ranges=None) -> None:
        with self.torch.cuda.device(self.device):
            self.launch(self.params(use_int8, mips=mips, row_ranges=row_ranges))

    def interleave_latents(self):
        """ntcb_interleave_latents: the pixel-major copy of the latents (a slot of 1, 2 or 4 elements per latent
        pixel; 12 features are padded to 4) for `sample(..., interleaved=True)`.  Made once and kept; queued on
        torch's current stream."""
        if getattr(self, "interleaved_latents", None) is None:
            torch = self.torch
            layers = self.geometry.num_features // 4
            slot = 4 if layers == 3 else layers
            self.interleaved_latents = torch.zeros(self.latents.numel() // layers * slot, dtype=self.latents.dtype,
                                                   device=self.device)
            # (only the mip descriptions of these parameters are used)
            decode = fill_params(self.geometry, self.latents.data_ptr(), self.networks[WEIGHTS_INT8].data_ptr(),
                                 self.status.data_ptr(), self.status.data_ptr(), WEIGHTS_INT8)
            with torch.cuda.device(self.device):
                stream = torch.cuda.current_stream(self.device).cuda_stream
                check(lib().ntcb_interleave_latents(ctypes.c_void_p(self.latents.data_ptr()),
                                                    ctypes.c_void_p(self.interleaved_latents.data_ptr()), decode.mips,
                                                    decode.numMips, decode.numFeatures, ctypes.c_void_p(stream)))
        return self.interleaved_latents

    def sample(self, queries, use_int8: bool, interleaved: bool = False):
        """Inference on sample: `queries` is a float32 CUDA tensor [n][3] of (u, v, lod); returns a
        float16 CUDA tensor [n][channels].  Queued on torch's current stream.  `interleaved`: read the
        latents from the copy `interleave_latents()` makes (same answers, fewer memory requests)."""
        torch = self.torch
        mode = WEIGHTS_INT8 if use_int8 else WEIGHTS_FP8
        queries = queries.contiguous()
        out = torch.empty((queries.shape[0], self.geometry.channels), dtype=torch.float16, device=self.device)
        network = self.networks[mode]
        latents = self.interleave_latents() if interleaved else self.latents
        decode = fill_params(self.geometry, latents.data_ptr(), network.data_ptr(), out.data_ptr(),
                             self.status.data_ptr(), mode)
        params = SampleParams()
        params.latentLayout = LATENTS_INTERLEAVED if interleaved else LATENTS_PLANAR
        params.latents, params.network, params.queries = decode.latents, decode.network, queries.data_ptr()
        params.out, params.status, params.numQueries = out.data_ptr(), decode.status, queries.shape[0]
        params.numMips, params.numFeatures, params.channels = decode.numMips, decode.numFeatures, decode.channels
        params.weightMode = mode
        params.numerics = self.numerics
        for i in range(decode.numMips):
            params.mips[i] = decode.mips[i]
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            check(lib().ntcb_sample(ctypes.byref(params), ctypes.c_void_p(stream)))
        return out

    def check_status(self) -> None:
        words = self.status.cpu().numpy()
        if words[0] != 0:
            raise NtcbError(-7, "a bounded wait in the decode kernel expired (tile %d, layer %d)" % (words[1], words[2]))

    def mip_view(self, mip: int):
        """The decoded fp16 texels of one mip as a tensor: [H][W][C] (interleaved layout) or
        [H][C/2][W][2] (planar-pair layout)."""
        cm = self.geometry.color_mips[mip]
        c = self.geometry.channels
        flat = self.out[cm.texel_offset * c:(cm.texel_offset + cm.width * cm.height) * c]
        if self.layout == LAYOUT_INTERLEAVED:
            return flat.view(cm.height, cm.width, c)
        return flat.view(cm.height, c // 2, cm.width, 2)

    def mip_numpy(self, mip: int) -> np.ndarray:
        """One decoded mip as a numpy array [H][W][C] regardless of the device layout."""
        view = self.mip_view(mip).cpu().numpy()
        if self.layout == LAYOUT_INTERLEAVED:
            return view
        h, pairs, w, _ = view.shape
        return view.transpose(0, 2, 1, 3).reshape(h, w, pairs * 2)


class Context:
    """ntcb_context_*: a decoder context on one CUDA device (the counterpart of ntc::IContext)."""

    def __init__(self, device: int = 0):
        self.handle = ctypes.c_void_p()
        check(lib().ntcb_context_create(device, ctypes.byref(self.handle)))
        self.device = device

    def create_texture_set(self, container: bytes, layout: int = LAYOUT_INTERLEAVED,
                           numerics: int = NUMERICS_REFERENCE) -> "TextureSet":
        return TextureSet(self, container, layout, numerics)

    def close(self) -> None:
        if self.handle:
            lib().ntcb_context_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __enter__(self) -> "Context":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


class TextureSet:
    """ntcb_texture_set_*: a compressed texture set loaded from an NTC container (the counterpart
    of ntc::ITextureSet for decompression)."""

    def __init__(self, context: Context, container: bytes, layout: int = LAYOUT_INTERLEAVED, numerics: int = NUMERICS_REFERENCE):
        self.context = context
        self.handle = ctypes.c_void_p()
        features = TextureSetFeatures(layout, numerics)
        buffer = np.frombuffer(container, dtype=np.uint8)
        check(lib().ntcb_texture_set_create_from_memory(context.handle, buffer.ctypes.data, len(container),
                                                        ctypes.byref(features), ctypes.byref(self.handle)))
        self.desc = TextureSetDesc()
        check(lib().ntcb_texture_set_get_desc(self.handle, ctypes.byref(self.desc)))

    def mip_size(self, mip: int) -> Tuple[int, int]:
        return max(1, self.desc.width >> mip), max(1, self.desc.height >> mip)

    def decompress(self, use_int8: bool, with_stats: bool = False, row_ranges=None) -> Optional[float]:
        stats = DecompressionStats()
        stats_ref = ctypes.byref(stats) if with_stats else None
        if row_ranges is None:
            check(lib().ntcb_texture_set_decompress(self.handle, stats_ref, 1 if use_int8 else 0))
        else:
            flat = (ctypes.c_int32 * (2 * self.desc.mips))(*[v for pair in row_ranges for v in pair])
            check(lib().ntcb_texture_set_decompress_rows(self.handle, flat, stats_ref, 1 if use_int8 else 0))
        return float(stats.gpuTimeMilliseconds) if with_stats else None

    def read_channels_into(self, mip: int, address: int, to_device: bool = False, first_channel: int = 0,
                           num_channels: Optional[int] = None, pixel_stride: Optional[int] = None,
                           row_pitch: Optional[int] = None, channel_format: int = CHANNEL_FORMAT_FLOAT16,
                           dst_color_spaces=None, use_dithering: bool = False, size: Optional[Tuple[int, int]] = None) -> None:
        w, h = self.mip_size(mip) if size is None else size
        n = self.desc.channels - first_channel if num_channels is None else num_channels
        component = np.dtype(CHANNEL_FORMAT_DTYPES.get(channel_format, np.float16)).itemsize
        params = ReadChannelsParams()
        params.mipLevel, params.firstChannel, params.numChannels = mip, first_channel, n
        params.addressSpace = ADDRESS_SPACE_DEVICE if to_device else ADDRESS_SPACE_HOST
        params.pOutData = address
        params.width, params.height = w, h
        params.channelFormat = channel_format
        params.useDithering = 1 if use_dithering else 0
        params.pixelStride = component * n if pixel_stride is None else pixel_stride
        params.rowPitch = params.pixelStride * w if row_pitch is None else row_pitch
        spaces = None
        if dst_color_spaces is not None:
            spaces = (ctypes.c_int32 * len(dst_color_spaces))(*dst_color_spaces)
            params.dstColorSpaces = ctypes.cast(spaces, ctypes.POINTER(ctypes.c_int32))
        check(lib().ntcb_texture_set_read_channels(self.handle, ctypes.byref(params)))

    def read_mip(self, mip: int, first_channel: int = 0, num_channels: Optional[int] = None,
                 channel_format: int = CHANNEL_FORMAT_FLOAT16, dst_color_spaces=None, use_dithering: bool = False,
                 components: Optional[int] = None, size: Optional[Tuple[int, int]] = None) -> np.ndarray:
        """One decoded mip as [height][width][components] in the given channel format; `components`
        (default: the number of channels read) above that number adds the default components;
        `size` = (width, height) other than the mip's resizes bilinearly, as the reference does."""
        w, h = self.mip_size(mip) if size is None else size
        n = self.desc.channels - first_channel if num_channels is None else num_channels
        dtype = np.dtype(CHANNEL_FORMAT_DTYPES[channel_format])
        count = n if components is None else components
        out = np.empty((h, w, count), dtype=dtype)
        self.read_channels_into(mip, out.ctypes.data, False, first_channel, n, count * dtype.itemsize, None, channel_format,
                                dst_color_spaces, use_dithering, size)
        return out

    def decompress_converted(self, conversion: OutputConversion, use_int8: bool = False, want_stats: bool = False,
                             device_address: Optional[int] = None):
        """Decompress + ReadChannels of every mip in one launch.  Returns (list of per-mip host arrays
        [h][w][components], gpu milliseconds or None); with `device_address` the pixels go to that
        device buffer instead and the list is empty."""
        dtype = np.dtype(CHANNEL_FORMAT_DTYPES.get(conversion.channelFormat, np.uint8))  # the library rejects unknown formats
        total = self.desc.totalTexels * max(conversion.components, 1)
        stats = DecompressionStats()
        stats_ref = ctypes.byref(stats) if want_stats else None
        if device_address is not None:
            check(lib().ntcb_texture_set_decompress_converted(self.handle, stats_ref, 1 if use_int8 else 0,
                                                               ctypes.byref(conversion), ADDRESS_SPACE_DEVICE, device_address,
                                                               total * dtype.itemsize))
            return [], (stats.gpuTimeMilliseconds if want_stats else None)
        flat = np.empty(total, dtype=dtype)
        check(lib().ntcb_texture_set_decompress_converted(self.handle, stats_ref, 1 if use_int8 else 0, ctypes.byref(conversion),
                                                           ADDRESS_SPACE_HOST, flat.ctypes.data, flat.nbytes))
        mips, offset = [], 0
        for mip in range(self.desc.mips):
            w, h = self.mip_size(mip)
            count = w * h * conversion.components
            mips.append(flat[offset:offset + count].reshape(h, w, conversion.components))
            offset += count
        return mips, (stats.gpuTimeMilliseconds if want_stats else None)

    def block_compress(self, mip: int, block_format: int, first_channel: int = 0, num_channels: int = 0,
                       alpha_threshold: float = 1.0 / 255.0):
        """One decoded mip as BC1 - BC5 blocks: a CUDA uint8 tensor [blocks_y][blocks_x][8 or 16]
        (waits for the texture set's stream)."""
        import torch

        width, height = self.mip_size(mip)
        bw, bh = (width + 3) // 4, (height + 3) // 4
        block_bytes = 8 if block_format in (BLOCK_FORMAT_BC1, BLOCK_FORMAT_BC4) else 16
        out = torch.zeros((bh, bw, block_bytes), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        check(lib().ntcb_texture_set_block_compress(self.handle, mip, first_channel, num_channels, block_format,
                                                    alpha_threshold, ctypes.c_void_p(out.data_ptr()), bw * block_bytes))
        self.synchronize()
        return out

    def load_from_memory(self, container: bytes) -> None:
        """Another compressed set of the same shape into this one's buffers (ITextureSet::LoadFromMemory)."""
        check(lib().ntcb_texture_set_load_from_memory(self.handle, container, len(container)))

    def bc7_mode_buffer(self, texture_index: int, mip_level: int) -> Optional[np.ndarray]:
        """The BC7 mode bitmap the set keeps for a texture's mip level (a copy, uint8), or None."""
        data, size = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().ntcb_texture_set_get_bc7_mode_buffer(self.handle, texture_index, mip_level, ctypes.byref(data), ctypes.byref(size)))
        if not data.value:
            return None
        return np.frombuffer(ctypes.string_at(data.value, size.value), dtype=np.uint8).copy()

    def make_and_store_bc7_mode_buffer(self, texture_index: int, mip_level: int, blocks: np.ndarray):
        """Stores the mode bitmap of BC7 blocks (uint8 [blocks_y][blocks_x][16]) for a texture's mip level."""
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        check(lib().ntcb_texture_set_make_and_store_bc7_mode_buffer(self.handle, texture_index, mip_level, blocks.shape[1],
                                                                    blocks.shape[0], blocks.ctypes.data, blocks.nbytes,
                                                                    blocks.shape[1] * 16))

    def block_compress_texture(self, texture_index: int, mip_level: int, alpha_threshold: float = 1.0 / 255.0):
        """One mip of one texture in the block format its header names (BC7: from its stored mode bitmap when it
        has one): a CUDA uint8 tensor [blocks_y][blocks_x][8 or 16] (waits for the texture set's stream)."""
        import torch

        block_format = self.textures()[texture_index]["blockCompressedFormat"]
        width, height = self.mip_size(mip_level)
        bw, bh = (width + 3) // 4, (height + 3) // 4
        block_bytes = 8 if block_format in (BLOCK_FORMAT_BC1, BLOCK_FORMAT_BC4) else 16
        out = torch.zeros((bh, bw, block_bytes), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        check(lib().ntcb_texture_set_block_compress_texture(self.handle, texture_index, mip_level, alpha_threshold,
                                                            ctypes.c_void_p(out.data_ptr()), bw * block_bytes))
        self.synchronize()
        return out

    def textures(self) -> list:
        """The texture headers of the set: a list of dictionaries (see TextureDesc)."""
        count = ctypes.c_int()
        lib().ntcb_texture_set_get_texture(self.handle, -1, None, ctypes.byref(count))
        result = []
        for index in range(count.value):
            desc = TextureDesc()
            check(lib().ntcb_texture_set_get_texture(self.handle, index, ctypes.byref(desc), None))
            result.append(desc.as_dict())
        return result

    def device_mip(self, mip: int) -> Tuple[int, int]:
        """Device address and size in bytes of one decoded mip in the internal layout."""
        pointer, size = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().ntcb_texture_set_device_mip(self.handle, mip, ctypes.byref(pointer), ctypes.byref(size)))
        return int(pointer.value), int(size.value)

    def sample(self, queries, use_int8: bool):
        """ntcb_texture_set_sample: `queries` is a float32 CUDA tensor [n][3] of (u, v, lod) on the set's device;
        returns a float16 CUDA tensor [n][channels] with the bits a decompress would write to the selected texels.
        The call waits for the answers."""
        import torch

        queries = queries.contiguous()
        out = torch.empty((queries.shape[0], self.desc.channels), dtype=torch.float16, device=queries.device)
        check(lib().ntcb_texture_set_sample(self.handle, ctypes.c_void_p(queries.data_ptr()), queries.shape[0],
                                            ctypes.c_void_p(out.data_ptr()), 1 if use_int8 else 0))
        return out

    def synchronize(self) -> None:
        check(lib().ntcb_texture_set_synchronize(self.handle))

    def close(self) -> None:
        if self.handle:
            lib().ntcb_texture_set_destroy(self.handle)
            self.handle = ctypes.c_void_p()


# ---------------------------------------------------------------------------------------------
# Several GPUs of one machine
# ---------------------------------------------------------------------------------------------

def plan_batch(shapes: Sequence[Tuple[int, int, int]], num_devices: int, units_per_device: int = 0) -> List[BatchUnit]:
    """ntcb_plan_batch for items given as (width, height, mips): the work units, largest first."""
    descs = (TextureSetDesc * len(shapes))()
    for desc, (width, height, mips) in zip(descs, shapes):
        desc.width, desc.height, desc.mips = width, height, mips
        desc.totalTexels = sum(max(width >> m, 1) * max(height >> m, 1) for m in range(mips))
    count = ctypes.c_int()
    check(lib().ntcb_plan_batch(descs, len(shapes), num_devices, units_per_device, None, 0, ctypes.byref(count)))
    units = (BatchUnit * count.value)()
    check(lib().ntcb_plan_batch(descs, len(shapes), num_devices, units_per_device, units, count.value, ctypes.byref(count)))
    return list(units)


def _batch_items(containers: Sequence[bytes], use_int8, host_images):
    items = (BatchItem * len(containers))()
    keep = []
    flags = [use_int8] * len(containers) if isinstance(use_int8, (bool, int)) else list(use_int8)
    for index, (item, container) in enumerate(zip(items, containers)):
        pointer = ctypes.c_char_p(container)  # the bytes object's own storage: nothing is copied
        keep.append((container, pointer))
        item.container = ctypes.cast(pointer, ctypes.c_void_p)
        item.containerBytes = len(container)
        item.useInt8Weights = 1 if flags[index] else 0
        if host_images is not None:
            image = host_images[index]
            item.hostTexels = image.data_ptr() if hasattr(image, "data_ptr") else image.ctypes.data
            item.hostTexelsBytes = image.numel() * image.element_size() if hasattr(image, "numel") else image.nbytes
    return items, keep


def _batch_options(numerics, worker, max_attempts, units_per_device, workers_per_device):
    options = BatchOptions()
    options.numerics, options.maxAttempts = numerics, max_attempts
    options.unitsPerDevice, options.workersPerDevice = units_per_device, workers_per_device
    callback = None
    if worker is not None:
        callback = BATCH_WORKER(lambda user, device, unit: int(worker(device, unit.contents)))
        options.worker = callback
    return options, callback


def decode_batch(containers: Sequence[bytes], devices: Sequence[int], use_int8, host_images=None, numerics: int = NUMERICS_REFERENCE,
                 worker=None, max_attempts: int = 0, units_per_device: int = 0, workers_per_device: int = 0):
    """ntcb_decode_batch: decodes the sets on the listed devices and gathers every set's mip chain in
    `host_images[i]` (a writable buffer object exposing its address as .data_ptr() or .ctypes.data;
    None with a fake `worker`).  `use_int8`: one flag, or one per set.  `worker(device, unit) -> status`
    replaces the GPU work (tests).  Returns (status code, item statuses, units as BatchUnit list)."""
    items, keep = _batch_items(containers, use_int8, host_images)
    options, callback = _batch_options(numerics, worker, max_attempts, units_per_device, workers_per_device)
    device_list = (ctypes.c_int * len(devices))(*devices)
    units = (BatchUnit * 8192)()
    count = ctypes.c_int()
    code = lib().ntcb_decode_batch(items, len(containers), device_list, len(devices), ctypes.byref(options), units, 8192,
                                   ctypes.byref(count))
    return code, [item.status for item in items], list(units)[:count.value]


class BatchDecoder:
    """ntcb_batch_decoder_*: the worker threads of decode_batch, their contexts and texture sets kept between runs."""

    def __init__(self, devices: Sequence[int], numerics: int = NUMERICS_REFERENCE, worker=None, max_attempts: int = 0,
                 units_per_device: int = 0, workers_per_device: int = 0):
        options, self._callback = _batch_options(numerics, worker, max_attempts, units_per_device, workers_per_device)
        device_list = (ctypes.c_int * len(devices))(*devices)
        self.handle = ctypes.c_void_p()
        check(lib().ntcb_batch_decoder_create(device_list, len(devices), ctypes.byref(options), ctypes.byref(self.handle)))

    def run(self, containers: Sequence[bytes], use_int8, host_images=None):
        """One batch; returns (status code, item statuses, units) like decode_batch."""
        items, keep = _batch_items(containers, use_int8, host_images)
        units = (BatchUnit * 8192)()
        count = ctypes.c_int()
        code = lib().ntcb_batch_decoder_run(self.handle, items, len(containers), units, 8192, ctypes.byref(count))
        return code, [item.status for item in items], list(units)[:count.value]

    def close(self) -> None:
        if self.handle:
            lib().ntcb_batch_decoder_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
