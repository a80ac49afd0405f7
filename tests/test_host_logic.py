"""Host-side logic that needs no GPU: geometry, the container writer/reader pair, the C ABI's
exports and argument checking, and weight staging."""
import ctypes
import os
import re

import numpy as np
import pytest

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, container, geometry, synthetic  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SHAPES = [(64, 64, 4, 0, 2, 8), (96, 40, 6, 0, 3, 12), (4096, 4096, 12, 0, 4, 12), (2048, 2048, 8, 0, 4, 8),
          (8192, 8192, 16, 0, 4, 16), (1024, 1024, 4, 1, 2, 8), (33, 17, 1, 0, 1, 4), (7, 300, 3, 0, 6, 16),
          (1, 1, 2, 1, 1, 4), (500, 500, 5, 3, 5, 8)]


@pytest.mark.parametrize("shape", SHAPES)
def test_python_geometry_matches_c_restatement(oracle, shape):
    w, h, c, mips, g, f = shape
    spec = synthetic.TextureSetSpec(w, h, c, mips, g, f, seed=0)
    geo = spec.geometry()
    dummy = np.zeros(geo.total_latent_pixels * geo.num_layers, dtype=np.uint16)
    cgeo = oracle.OracleSet(geo, dummy, bytes(geometry.INT8_BLOB_BYTES), bytes(geometry.FP8_BLOB_BYTES)).c_geometry()
    assert cgeo.numNeuralMips == geo.num_neural_mips and cgeo.numLayers == geo.num_layers
    assert list(cgeo.latentWidth[:geo.num_neural_mips]) == geo.latent_width
    assert list(cgeo.latentHeight[:geo.num_neural_mips]) == geo.latent_height
    for mip, cm in enumerate(geo.color_mips):
        assert (cgeo.mipWidth[mip], cgeo.mipHeight[mip], cgeo.neuralLod[mip]) == (cm.width, cm.height, cm.neural_lod)
        assert cgeo.positionScale[mip] == np.float32(cm.position_scale)
        assert abs(cgeo.positionLod[mip] - cm.position_lod) <= 1e-6
        assert cgeo.mipTexelOffset[mip] == cm.texel_offset


def test_known_geometry_of_the_pbr_configuration():
    """4096x4096, grid scale 4: eight neural mips from 1024^2 down; mips 0-2 read neural LOD 0,
    3-4 LOD 2, 5-6 LOD 4, 7-12 LOD 6 (src/FeatureGridMath.cpp:47-76)."""
    geo = synthetic.config_spec(1).geometry()
    assert geo.mips == 13 and geo.num_neural_mips == 8 and geo.num_layers == 3
    assert geo.latent_width == [1024, 512, 256, 128, 64, 32, 16, 8]
    assert [cm.neural_lod for cm in geo.color_mips] == [0, 0, 0, 2, 2, 4, 4, 6, 6, 6, 6, 6, 6]
    assert [cm.position_scale for cm in geo.color_mips[:3]] == [0.125, 0.25, 0.5]
    assert geo.total_texels == 22369621
    assert geo.encoded_latent_bytes == 8388480


def test_container_round_trip_and_probe():
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(96, 40, 5, 0, 3, 12, seed=5, network="unit"))
    geo, latents, int8_blob, fp8_blob = container.read_container(data.container)
    assert (geo.width, geo.height, geo.channels, geo.mips) == (96, 40, 6, 7)
    assert int8_blob == data.int8_blob and fp8_blob == data.fp8_blob
    assert all(np.array_equal(a, b) for a, b in zip(latents, data.latents))
    desc = binding.probe_container(data.container)
    assert (desc.width, desc.height, desc.channels, desc.mips) == (96, 40, 6, 7)
    assert (desc.gridSizeScale, desc.numFeatures, desc.numNeuralMips, desc.numLayers) == (3, 12, 4, 3)
    assert desc.totalTexels == geo.total_texels


def test_reference_loader_accepts_the_container(oracle):
    """Needs oracle/_ref (built where the reference sources are); metadata only, no GPU."""
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libntc_ref.so is not built")
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 0, 2, 8, seed=3))
    assert oracle.reference_probe(data.container) == [64, 64, 4, 7, 2, 8, 6, 0]


def patch_document(data: bytes, edit) -> bytes:
    """Rewrites a container with its JSON document passed through `edit` (header sizes updated)."""
    import json
    import struct

    signature, version, json_offset, json_size, binary_offset, binary_size = struct.unpack_from("<IIQQQQ", data, 0)
    document = json.loads(data[json_offset:json_offset + json_size].rstrip(b"\0"))
    edit(document)
    text = json.dumps(document, separators=(",", ":")).encode() + b"\0"
    new_binary_offset = (40 + len(text) + 3) & ~3
    out = bytearray(struct.pack("<IIQQQQ", signature, version, 40, len(text), new_binary_offset, binary_size))
    out += text
    out += bytes(new_binary_offset - len(out))
    out += data[binary_offset:binary_offset + binary_size]
    return bytes(out)


def _set(path, value):
    def edit(document):
        node = document
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
    return edit


@pytest.mark.parametrize("damage,code", [
    (lambda b: b[:30], -3),
    (lambda b: b"XXXX" + b[4:], -3),
    (lambda b: b[:4] + b"\x01\x02\x00\x00" + b[8:], -3),
    (lambda b: b[:len(b) - 100], -3),
    (lambda b: patch_document(b, _set(["schemaVersion"], 2)), -3),
    (lambda b: patch_document(b, _set(["latentShape", "numFeatures"], 9)), -9),
    (lambda b: patch_document(b, _set(["mlpVersions", 0, "weightLayout"], "ColumnMajor")), -3),
    (lambda b: patch_document(b, _set(["mlpVersions", 1, "layers", 0, "biasType"], "Int32")), -3),
    (lambda b: patch_document(b, _set(["mlpVersions", 0, "layers", 0, "inputChannels"], 32)), -3),
    (lambda b: patch_document(b, _set(["colorMips", 0, "latentMip"], 4)), -3),
    (lambda b: patch_document(b, _set(["latents", 1, "width"], 17)), -3),
    (lambda b: patch_document(b, _set(["views", 3, "offset"], 2)), -3),
    (lambda b: patch_document(b, _set(["views", 3, "storedSize"], 1 << 40)), -3),
    (lambda b: patch_document(b, _set(["width"], 0)), -9),
])
def test_container_errors_are_reported(damage, code):
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 0, 2, 8, seed=3)).container
    with pytest.raises(binding.NtcbError) as error:
        binding.probe_container(damage(data))
    assert error.value.code == code
    assert str(error.value)


def test_patch_document_keeps_a_valid_container_valid():
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 0, 2, 8, seed=3)).container
    assert binding.probe_container(patch_document(data, lambda document: None)).width == 64


def test_smaller_hidden_layers_are_zero_expanded():
    """A file may carry narrower hidden layers; they land in the top-left corner of the full
    matrices (src/TextureSetMetadata.cpp:660-713)."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 0, 2, 8, seed=3)).container

    def narrow(document):
        layers = document["mlpVersions"][0]["layers"]
        layers[0]["outputChannels"] = 48
        layers[1]["inputChannels"] = 48
    assert binding.probe_container(patch_document(data, narrow)).width == 64


def test_compressed_views_are_refused():
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 0, 2, 8, seed=3)).container
    damaged = patch_document(data, _set(["views", 0, "compression"], "GDeflate"))
    with pytest.raises(binding.NtcbError) as error:
        binding.probe_container(damaged)
    assert error.value.code == -5  # Unsupported


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "ntcb.h")).read()
    declared = set(re.findall(r"\b(ntcb_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 15
    lib = binding.lib()
    for name in sorted(declared):
        assert hasattr(lib, name), "libntcb200.so does not export " + name


STAGED_WEIGHT_OFFSETS = [0, 4096, 8704, 11776]
STAGED_K = [64, 96, 96, 64]          # real inputs, then the slots that carry an int8 layer's bias
STAGED_SCALES, STAGED_BIASES, STAGED_FLAGS = 12800, 13824, 14848


def _staged_matrix(staged, layer, nout):
    k = np.arange(STAGED_K[layer])
    n = np.arange(nout)[:, None]
    index = STAGED_WEIGHT_OFFSETS[layer] + (k // 16) * nout * 16 + n * 16 + k % 16
    return staged[index].view(np.int8).astype(np.int64)


def _file_biases(source, mode):
    """int32 biases of the int8 layers as the weight blob stores them: {layer: values}."""
    if mode == binding.WEIGHTS_INT8:
        table = source[8192 + 640:8192 + 1280].view(np.int32)
        bounds = np.cumsum([0] + list(geometry.MLP_LAYER_OUTPUTS))
        return {layer: table[bounds[layer]:bounds[layer + 1]].astype(np.int64) for layer in range(4)}
    return {3: source[8544:8608].view(np.int32).astype(np.int64)}


def test_weight_staging_layout():
    """K-major core-matrix order: byte (n, k) of layer l at (k / 16) * (N * 16) + n * 16 + k % 16;
    the K slots past an int8 layer's inputs hold a decomposition of its bias over the constant
    inputs 127 (1 in the last slot of each 32-slot K step)."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 1, 2, 8, seed=3))
    for blob, mode in ((data.int8_blob, binding.WEIGHTS_INT8), (data.fp8_blob, binding.WEIGHTS_FP8)):
        staged = binding.stage_network(blob, mode, binding.NUMERICS_EXACT)
        assert staged.size == binding.STAGED_NETWORK_BYTES
        source = np.frombuffer(blob, dtype=np.uint8)
        # Int8 networks carry their biases in the matrix product (every bias of this set fits its slots);
        # the FP8 network's single int8 layer keeps the table
        biases = _file_biases(source, mode) if mode == binding.WEIGHTS_INT8 else {}
        assert staged[STAGED_FLAGS:STAGED_FLAGS + 4].view(np.uint32)[0] == (0 if mode == binding.WEIGHTS_INT8 else 1)
        position = 0
        for layer, (nin, nout) in enumerate(zip(geometry.MLP_LAYER_INPUTS, geometry.MLP_LAYER_OUTPUTS)):
            weights = source[position:position + nin * nout].view(np.int8).reshape(nout, nin)
            position += nin * nout
            matrix = _staged_matrix(staged, layer, nout)
            assert np.array_equal(matrix[:, :nin], weights)
            constants = np.where(np.arange(STAGED_K[layer]) % 32 == 31, 1, 127)[nin:]
            if layer in biases:
                assert np.array_equal(matrix[:, nin:] @ constants, biases[layer]), layer
                assert np.abs(matrix[:, nin:]).max() <= 127
            else:
                assert not matrix[:, nin:].any()  # e4m3 layers: zero padding
        scales = staged[STAGED_SCALES:STAGED_SCALES + 1024].view(np.float32).reshape(4, 64)
        if mode == binding.WEIGHTS_INT8:
            assert np.array_equal(scales[0], source[8192:8192 + 256].view(np.float32))
            assert not staged[STAGED_BIASES:STAGED_BIASES + 1024].any()  # the table is only the fallback
        else:
            assert np.array_equal(scales[3, :16], source[8480:8544].view(np.float32))
            assert np.array_equal(staged[STAGED_BIASES:STAGED_BIASES + 128].view(np.float16), source[8192:8320].view(np.float16))
            assert np.array_equal(staged[STAGED_BIASES + 768:STAGED_BIASES + 832].view(np.int32), source[8544:8608].view(np.int32))


def test_weight_staging_falls_back_to_the_bias_table():
    """A bias too large for its slots switches the whole network to the table."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 1, 2, 8, seed=3))
    blob = bytearray(data.int8_blob)
    table = np.frombuffer(bytes(blob[8192 + 640:8192 + 1280]), dtype=np.int32).copy()
    table[64 + 5] = 127 * 127 * 31 + 64  # one more than layer 1's 32 slots can carry
    blob[8192 + 640:8192 + 1280] = table.tobytes()
    staged = binding.stage_network(bytes(blob), binding.WEIGHTS_INT8, binding.NUMERICS_EXACT)
    assert staged[STAGED_FLAGS:STAGED_FLAGS + 4].view(np.uint32)[0] == 1
    stored = staged[STAGED_BIASES:STAGED_BIASES + 1024].view(np.int32).reshape(4, 64)
    assert np.array_equal(stored[1, :48], table[64:112]) and np.array_equal(stored[3, :16], table[144:160])
    for layer, (nin, nout) in enumerate(zip(geometry.MLP_LAYER_INPUTS, geometry.MLP_LAYER_OUTPUTS)):
        assert not _staged_matrix(staged, layer, nout)[:, nin:].any()
    table[64 + 5] -= 1  # the largest value that still fits
    blob[8192 + 640:8192 + 1280] = table.tobytes()
    staged = binding.stage_network(bytes(blob), binding.WEIGHTS_INT8, binding.NUMERICS_EXACT)
    assert staged[STAGED_FLAGS:STAGED_FLAGS + 4].view(np.uint32)[0] == 0
    constants = np.where(np.arange(96) % 32 == 31, 1, 127)[64:]
    assert (_staged_matrix(staged, 1, 48)[5, 64:] @ constants) == table[64 + 5]


def test_reference_network_staging():
    """The image of the reference-numerics kernels: binary16 weights rebuilt as the reference's
    ConvertNetworkFromQuantizedToFp16 does, in K-major core matrices of 8 halves (element (n, k) of
    layer l at byte (k / 8) * (N * 16) + n * 16 + (k % 8) * 2), and per layer an N x 16 bias-step operand
    with the binary16 bias in column 0 (FP8 networks) or one 64 x 8 matrix whose column l is the bias of
    layer l (Int8 networks).  The e4m3 layers of an FP8 network keep their bytes: one
    N x 32 byte matrix per 16-wide K step with the step's weights at their place inside the 32-wide
    chunk and zeros in the other half."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 1, 2, 8, seed=3))
    weight_offsets, bias_offsets = [0, 6144, 12288, 15360], [16384, 18432, 19968, 20992]
    for blob, mode in ((data.int8_blob, binding.WEIGHTS_INT8), (data.fp8_blob, binding.WEIGHTS_FP8)):
        staged = binding.stage_network(blob, mode)  # the default numerics are the reference's
        assert staged.size == binding.STAGED_REFERENCE_NETWORK_BYTES == 21504
        halves = staged.view(np.float16)
        source = np.frombuffer(blob, dtype=np.uint8)
        position = 0
        for layer, (nin, nout) in enumerate(zip(geometry.MLP_LAYER_INPUTS, geometry.MLP_LAYER_OUTPUTS)):
            raw = source[position:position + nin * nout].reshape(nout, nin)
            position += nin * nout
            k = np.arange(nin)
            n = np.arange(nout)[:, None]
            layer_is_fp8 = mode == binding.WEIGHTS_FP8 and layer < 3
            if layer_is_fp8:
                region = staged[weight_offsets[layer]:weight_offsets[layer] + nin * nout * 2]
                steps = region.reshape(nin // 16, 2, nout, 16)  # [K step][16-byte column group of the 32-wide chunk][n][byte]
                for step in range(nin // 16):
                    group = step % 2
                    assert np.array_equal(steps[step, group], raw[:, 16 * step:16 * step + 16]), (layer, step)
                    assert not steps[step, 1 - group].any(), (layer, step)
                bias = source[8192 + 2 * sum(geometry.MLP_LAYER_OUTPUTS[:layer]):][:2 * nout].view(np.float16)
                matrix = expected = None
            else:
                matrix = halves[(weight_offsets[layer] + (k // 8) * nout * 16 + n * 16 + (k % 8) * 2) // 2].astype(np.float32)
                if mode == binding.WEIGHTS_INT8:
                    first = sum(geometry.MLP_LAYER_OUTPUTS[:layer])
                    scale = source[8192 + 4 * first:][:4 * nout].view(np.float32)
                    integer_bias = source[8192 + 640 + 4 * first:][:4 * nout].view(np.int32)
                else:
                    scale = source[8480:8544].view(np.float32)
                    integer_bias = source[8544:8608].view(np.int32)
                # src/Quantizer.cu:325-382, the same fp32 operation order
                layer_bias = integer_bias.astype(np.float32) * scale
                step = np.float32(3.1875) / np.float32(255)
                layer_scale = scale * (np.float32(127.5) if layer == 0 else np.float32(1) / step)
                weights = raw.view(np.int8).astype(np.float32)
                expected = (weights * layer_scale[:, None]).astype(np.float16).astype(np.float32)
                if layer != 0:
                    sums = raw.view(np.int8).astype(np.int64).sum(axis=1)
                    product = (sums * -113).astype(np.float32) * layer_scale
                    layer_bias = (product.astype(np.float64) * np.float64(step) + layer_bias.astype(np.float64)).astype(np.float32)  # one rounding: fma
                bias = layer_bias.astype(np.float16)
            assert matrix is None or np.array_equal(matrix, expected), (mode, layer)
            if mode == binding.WEIGHTS_INT8:
                bias_matrix = halves[16384 // 2:17408 // 2].reshape(64, 8)
                assert np.array_equal(bias_matrix[:nout, layer].view(np.uint16), bias.view(np.uint16)), (mode, layer)
                assert not bias_matrix[nout:, layer].any() and not bias_matrix[:, 4:].any()
                assert not staged[17408:].any()
            else:
                step_operand = halves[bias_offsets[layer] // 2:bias_offsets[layer] // 2 + nout * 16].reshape(2, nout, 8)
                assert np.array_equal(step_operand[0, :, 0].view(np.uint16), bias.view(np.uint16)), (mode, layer)
                assert not step_operand[0, :, 1:].any() and not step_operand[1].any()


def test_stage_network_rejects_wrong_sizes():
    for numerics in (binding.NUMERICS_REFERENCE, binding.NUMERICS_EXACT):
        with pytest.raises(binding.NtcbError) as error:
            binding.stage_network(bytes(100), binding.WEIGHTS_INT8, numerics)
        assert error.value.code == -1


def test_decode_validates_arguments_before_touching_the_gpu():
    lib = binding.lib()
    params = binding.DecodeParams()
    assert lib.ntcb_decode(ctypes.byref(params), None) == -1
    assert b"NULL" in lib.ntcb_last_error()
    geo = synthetic.TextureSetSpec(64, 64, 4, 1, 2, 8, seed=0).geometry()
    good = binding.fill_params(geo, 0x1000, 0x2000, 0x3000, 0x4000, binding.WEIGHTS_INT8)
    good.channels = 5
    assert lib.ntcb_decode(ctypes.byref(good), None) == -1
    good.channels = 4
    good.mips[0].rowEnd = 100
    assert lib.ntcb_decode(ctypes.byref(good), None) == -1


def test_sample_and_interleave_validate_arguments_before_touching_the_gpu():
    lib = binding.lib()
    geo = synthetic.TextureSetSpec(64, 64, 4, 1, 2, 8, seed=0).geometry()
    decode = binding.fill_params(geo, 0x1000, 0x2000, 0x3000, 0x4000, binding.WEIGHTS_INT8)
    params = binding.SampleParams()
    params.latents, params.network, params.queries, params.out, params.status = 0x1000, 0x2000, 0x5000, 0x3000, 0x4000
    params.numQueries, params.numMips, params.numFeatures, params.channels = 16, decode.numMips, 8, 4
    params.weightMode, params.numerics = binding.WEIGHTS_INT8, binding.NUMERICS_REFERENCE
    for i in range(decode.numMips):
        params.mips[i] = decode.mips[i]
    params.latentLayout = 2
    assert lib.ntcb_sample(ctypes.byref(params), None) == -1
    assert b"latent layout" in lib.ntcb_last_error()
    params.latentLayout = binding.LATENTS_INTERLEAVED
    params.latents = 0x1004
    assert lib.ntcb_sample(ctypes.byref(params), None) == -1
    assert b"8-byte aligned" in lib.ntcb_last_error()
    # ntcb_interleave_latents: NULL, aliased or misaligned buffers, bad counts, a grid larger than its plane,
    # an offset that is not a multiple of the layer count
    mips = decode.mips
    assert lib.ntcb_interleave_latents(None, ctypes.c_void_p(0x1000), mips, 1, 8, None) == -1
    assert lib.ntcb_interleave_latents(ctypes.c_void_p(0x1000), ctypes.c_void_p(0x1000), mips, 1, 8, None) == -1
    assert lib.ntcb_interleave_latents(ctypes.c_void_p(0x1000), ctypes.c_void_p(0x9004), mips, 1, 8, None) == -1
    assert lib.ntcb_interleave_latents(ctypes.c_void_p(0x1000), ctypes.c_void_p(0x9000), mips, 0, 8, None) == -1
    assert lib.ntcb_interleave_latents(ctypes.c_void_p(0x1000), ctypes.c_void_p(0x9000), mips, 1, 6, None) == -1
    broken = (binding.MipDesc * 1)(decode.mips[0])
    broken[0].hiPlane = 1
    assert lib.ntcb_interleave_latents(ctypes.c_void_p(0x1000), ctypes.c_void_p(0x9000), broken, 1, 8, None) == -1
    assert b"between its layers" in lib.ntcb_last_error()
    broken = (binding.MipDesc * 1)(decode.mips[0])
    broken[0].loOffset = decode.mips[0].loOffset + 1
    assert lib.ntcb_interleave_latents(ctypes.c_void_p(0x1000), ctypes.c_void_p(0x9000), broken, 1, 8, None) == -1
    assert b"multiple of the layer count" in lib.ntcb_last_error()


def test_misaligned_and_oversized_requests_are_refused_on_the_host():
    """Requests that would make a kernel issue a misaligned vector access, or overflow its 32-bit
    element index, are refused before anything is launched (the addresses here are never touched)."""
    import torch

    gpu_present = torch.cuda.is_available()
    lib = binding.lib()
    geo = synthetic.TextureSetSpec(64, 64, 4, 1, 2, 8, seed=0).geometry()
    # converting epilogue: a pixel of 16 (8) bytes is stored as one 16-byte (8-byte) vector
    for channel_format, components, misaligned, aligned in (
            (binding.CHANNEL_FORMAT_FLOAT32, 4, 0x3004, 0x3010), (binding.CHANNEL_FORMAT_FLOAT16, 8, 0x3008, 0x3020),
            (binding.CHANNEL_FORMAT_FLOAT16, 4, 0x3004, 0x3008), (binding.CHANNEL_FORMAT_UNORM8, 16, 0x3004, 0x3030)):
        conversion = binding.make_conversion(channel_format, 4, components=components)
        params = binding.fill_params(geo, 0x1000, 0x2000, misaligned, 0x4000, binding.WEIGHTS_INT8, conversion=conversion)
        assert lib.ntcb_decode(ctypes.byref(params), None) == -1
        assert b"multiple of" in lib.ntcb_last_error()
        if not gpu_present:
            # the aligned request passes the argument checks and fails only for want of a GPU (never tried
            # where a GPU is present: the addresses are made up)
            params = binding.fill_params(geo, 0x1000, 0x2000, aligned, 0x4000, binding.WEIGHTS_INT8, conversion=conversion)
            assert lib.ntcb_decode(ctypes.byref(params), None) == -2
    # a mip of 2^32 values or more
    params = binding.fill_params(geo, 0x1000, 0x2000, 0x3000, 0x4000, binding.WEIGHTS_INT8)
    params.mips[0].width, params.mips[0].height, params.mips[0].rowEnd = 65536, 16384, 16384
    assert lib.ntcb_decode(ctypes.byref(params), None) == -9
    # ntcb_convert_channels and the allocation-free read take channel pairs as 32-bit words
    convert = binding.ConvertParams()
    convert.deviceMip, convert.layout, convert.width, convert.height, convert.channels = 0x5002, binding.LAYOUT_INTERLEAVED, 8, 8, 4
    convert.deviceDestination, convert.pixelStride, convert.rowPitch = 0x6000, 8, 64
    convert.conversion = binding.make_conversion(binding.CHANNEL_FORMAT_FLOAT16, 4)
    assert lib.ntcb_convert_channels(ctypes.byref(convert), None) == -1
    host = np.zeros(8 * 8 * 4, dtype=np.float16)
    assert lib.ntcb_read_channels_to_host_noalloc(0x5002, binding.LAYOUT_INTERLEAVED, 8, 8, 4, 0, 4, host.ctypes.data, 8, 64, None) == -1


def test_no_cpu_fallback():
    """Without a usable GPU the compute entry points fail with a CUDA error instead of computing
    on the host."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = binding.lib()
    handle = ctypes.c_void_p()
    assert lib.ntcb_context_create(0, ctypes.byref(handle)) == -2
    geo = synthetic.TextureSetSpec(64, 64, 4, 1, 2, 8, seed=0).geometry()
    params = binding.fill_params(geo, 0x1000, 0x2000, 0x3000, 0x4000, binding.WEIGHTS_INT8)
    assert lib.ntcb_decode(ctypes.byref(params), None) == -2


TEXTURES = [
    {"name": "Albedo", "firstChannel": 0, "numChannels": 3, "channelFormat": "UNORM8", "rgbColorSpace": "sRGB", "bcFormat": "BC1"},
    {"name": "Normal", "firstChannel": 3, "numChannels": 2, "bcFormat": "BC5"},
    {"name": "Emissive HDR with a rather long name " + "x" * 120, "firstChannel": 5, "numChannels": 1,
     "channelFormat": "FLOAT16", "rgbColorSpace": "HLG", "alphaColorSpace": "Linear", "bcFormat": "BC6"},
]


def _set_with_textures(textures=TEXTURES):
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 6, 0, 2, 8, seed=3))
    data.textures = textures
    return data


def test_texture_headers_are_read_with_the_reference_defaults():
    """ITextureSetMetadata::GetTexture: name, channel range and intended formats; a field the file
    leaves out takes the default the reference's loader gives it (UNORM8, Linear, no block format)."""
    textures = binding.probe_textures(_set_with_textures().container)
    assert [t["name"] for t in textures[:2]] == ["Albedo", "Normal"]
    assert textures[2]["name"] == TEXTURES[2]["name"][:127]  # the C structure holds 127 characters
    assert [(t["firstChannel"], t["numChannels"]) for t in textures] == [(0, 3), (3, 2), (5, 1)]
    assert [t["channelFormat"] for t in textures] == [1, 1, 3]
    assert [t["blockCompressedFormat"] for t in textures] == [1, 5, 6]
    assert [(t["rgbColorSpace"], t["alphaColorSpace"]) for t in textures] == [(1, 0), (0, 0), (2, 0)]
    assert binding.probe_textures(synthetic.make_texture_set(synthetic.TextureSetSpec(64, 64, 4, 0, 2, 8, seed=3)).container) == []


def test_texture_header_errors():
    lib = binding.lib()
    for bad in ([{"name": "A", "firstChannel": 0, "numChannels": 3, "bcFormat": "BC9"}],
                [{"firstChannel": 0, "numChannels": 3}],
                [{"name": "A", "numChannels": 3}],
                ["Albedo"]):
        container = _set_with_textures(bad).container
        buffer = np.frombuffer(container, dtype=np.uint8)
        assert lib.ntcb_probe_container_texture(buffer.ctypes.data, len(container), 0, None, None) == -3, bad
    container = _set_with_textures().container
    buffer = np.frombuffer(container, dtype=np.uint8)
    desc = binding.TextureDesc()
    assert lib.ntcb_probe_container_texture(buffer.ctypes.data, len(container), 3, ctypes.byref(desc), None) == -9


def test_reference_loader_accepts_the_texture_headers(oracle):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libntc_ref.so is not built")
    probed = oracle.reference_probe(_set_with_textures().container)
    assert probed[:6] == [64, 64, 6, 7, 2, 8]
    assert probed[7] == 0b111111  # the reference's valid-channel mask: the channels the textures cover
