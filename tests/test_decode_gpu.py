"""Parity of the sm_100a decode path, through the C ABI, against outputs of the unmodified reference
decoder and against the CPU restatement.

The library decodes with one of two numerics (NtcbNumerics):
  * REFERENCE (the default): binary16 weights, activations and accumulators, as the reference's CUDA
    decoder.  Bar: IDENTICAL BITS to what the reference decoded - every value of every golden
    fixture, and a live run of the reference library when oracle/_ref is present.  (The CPU
    restatement of these numerics models the tensor core's internal rounding and agrees with the
    reference in 99.998 % of values; against it the kernel is allowed 2 differences in 10,000.)
  * EXACT: exact accumulation, the reference's integer-path arithmetic.

Bars for EXACT (integer / byte work is bit-exact; floating point carries its tolerance here):
  * kernel vs the CPU restatement of its arithmetic contract (exact accumulation): identical bits,
    both weight modes (the FP8 layers accumulate e4m3 products in fp32 inside the tensor core; an
    occasional last-bit difference in that sum may flip one binary16 rounding, so FP8 mode allows
    <= 1 value in 100,000 to differ - none did on the fixtures);
  * kernel vs the reference's own CUDA decode (golden fixtures and a live run when oracle/_ref is
    present): >= 50 dB PSNR (peak = the reference's value range) on networks with O(1)
    pre-activations.  The reference accumulates in binary16 and rounds after every 16 products;
    that rounding flips 8-bit activation codes, which bounds the agreement any exact-accumulating
    decoder can reach (the CPU restatement shows the same distance, test_oracle_golden.py).
"""
import ctypes

import numpy as np
import pytest

from conftest import load_golden, psnr_db, reference_chain

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, container, synthetic  # noqa: E402

pytestmark = pytest.mark.gpu

GOLDEN_CASES = ["sq64_g2_f8_unit", "sq64_g2_f8_bench", "r96x40_g3_f12_unit", "sq128_g4_f12_2bit_bench",
                "sq128_g4_f12_2bit_unit", "r128x64_g4_f16_unit", "r33x17_g1_f4_unit", "sq128_g6_f8_unit",
                "sq64_g5_f16_mip0_unit"]


def _sync():
    import torch

    torch.cuda.synchronize()


EXACT, REFERENCE = binding.NUMERICS_EXACT, binding.NUMERICS_REFERENCE
BOTH_NUMERICS = pytest.mark.parametrize("numerics", [REFERENCE, EXACT], ids=["reference", "exact"])


def _assert_matches_contract(decoded, expected, use_int8, what):
    different = int((decoded.view(np.uint16) != expected.view(np.uint16)).sum())
    allowed = 0 if use_int8 else max(0, decoded.size // 100000)
    assert different <= allowed, "%s: %d of %d values differ from the CPU restatement" % (what, different, decoded.size)


def _restated(oracle, checker, mip, use_int8, numerics):
    """The CPU restatement of the kernel that implements `numerics`."""
    if numerics == EXACT:
        return checker.decode_mip(mip, use_int8, oracle.NUMERICS_SPEC)
    return checker.decode_mip(mip, use_int8, oracle.NUMERICS_REF, **oracle.REF_DEFAULTS)


class _Tally:
    """Mismatch budget of a whole test against the CPU restatement: none for exact int8 work, one in
    100,000 for exact FP8 work, two in 10,000 for the emulated reference numerics."""

    def __init__(self, numerics):
        self.numerics, self.values, self.different = numerics, 0, 0

    def add(self, decoded, expected, use_int8, what):
        if self.numerics == EXACT:
            _assert_matches_contract(decoded, expected, use_int8, what)
            return
        assert decoded.shape == expected.shape, what
        self.values += decoded.size
        self.different += int((decoded.view(np.uint16) != expected.view(np.uint16)).sum())

    def check(self):
        assert self.different <= max(2, self.values * 2e-4), "%d of %d values differ" % (self.different, self.values)


@pytest.mark.parametrize("layout", [binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_reference_numerics_reproduce_the_reference_bit_for_bit(golden_index, name, layout):
    """Every value the unmodified reference decoded (both weight modes, every mip) comes out of the
    default kernel with identical bits."""
    fixture = load_golden(name)
    geo, latents, int8_blob, fp8_blob = container.read_container(fixture["container"].tobytes())
    packed = np.concatenate([p.reshape(-1) for p in latents])
    resident = binding.ResidentTextureSet(geo, packed, int8_blob, fp8_blob, layout=layout)
    assert resident.numerics == REFERENCE
    for mode in golden_index[name]["modes"]:
        resident.out.fill_(float("nan"))
        resident.decode(mode == "int8")
        _sync()
        resident.check_status()
        for mip in range(geo.mips):
            reference = fixture["%s_mip%d" % (mode, mip)]
            assert np.array_equal(resident.mip_numpy(mip).view(np.uint16), reference), "%s %s mip %d" % (name, mode, mip)


@pytest.mark.parametrize("layout", [binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS])
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_kernel_matches_contract_and_reference_on_golden_sets(oracle, golden_index, name, layout):
    fixture = load_golden(name)
    geo, latents, int8_blob, fp8_blob = container.read_container(fixture["container"].tobytes())
    packed = np.concatenate([p.reshape(-1) for p in latents])
    checker = oracle.OracleSet(geo, packed, int8_blob, fp8_blob)
    resident = binding.ResidentTextureSet(geo, packed, int8_blob, fp8_blob, layout=layout, numerics=EXACT)
    for mode in golden_index[name]["modes"]:
        use_int8 = mode == "int8"
        resident.out.fill_(float("nan"))
        resident.decode(use_int8)
        _sync()
        resident.check_status()
        for mip in range(geo.mips):
            decoded = resident.mip_numpy(mip)
            _assert_matches_contract(decoded, checker.decode_mip(mip, use_int8, oracle.NUMERICS_SPEC), use_int8,
                                     "%s %s mip %d" % (name, mode, mip))
        if golden_index[name]["network"] == "unit":
            reference = fixture["%s_mip0" % mode].view(np.float16)
            assert psnr_db(resident.mip_numpy(0), reference) >= 50.0


RANDOM_SPECS = [
    # width, height, channels, mips (0 = full chain), grid scale, features
    (1, 1, 2, 1, 1, 4), (2, 3, 1, 0, 1, 8), (31, 5, 3, 0, 2, 12), (32, 4, 4, 1, 3, 16), (33, 9, 5, 0, 4, 4),
    (100, 37, 7, 0, 5, 8), (257, 129, 9, 0, 6, 12), (64, 256, 11, 0, 1, 16), (512, 64, 13, 0, 2, 4),
    (320, 200, 15, 0, 3, 8), (200, 320, 16, 0, 4, 12), (96, 96, 12, 4, 5, 16), (1000, 10, 2, 0, 6, 16),
]


@BOTH_NUMERICS
@pytest.mark.parametrize("shape", RANDOM_SPECS)
@pytest.mark.parametrize("network", ["unit", "benchmark"])
def test_kernel_matches_contract_on_ragged_shapes(oracle, shape, network, numerics):
    """Every grid scale and feature count, odd channel counts, sizes that are not multiples of the
    32x4 tile, one-texel mips, width != height."""
    w, h, c, mips, g, f = shape
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(w, h, c, mips, g, f, seed=w * 7 + h, network=network))
    geo = data.geometry
    checker = oracle.OracleSet.from_synthetic(data)
    resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
    # the default numerics are held to the reference itself wherever it can answer: identical bits to a
    # live run of the unmodified reference on this GPU; the CPU model of its rounding (2 differences in
    # 10,000 allowed, because the model is 99.998 % exact) is only the fallback
    live = numerics == REFERENCE and oracle.reference_available()
    tally = _Tally(numerics)
    for use_int8 in (True, False):
        resident.out.fill_(float("nan"))
        resident.decode(use_int8)
        _sync()
        resident.check_status()
        if live:
            chain = reference_chain(oracle, data, use_int8).cpu().numpy()
        for mip in range(geo.mips):
            if live:
                cm = geo.color_mips[mip]
                theirs = chain[cm.texel_offset * geo.channels:(cm.texel_offset + cm.width * cm.height) * geo.channels]
                assert np.array_equal(resident.mip_numpy(mip).reshape(-1).view(np.uint16), theirs.view(np.uint16)), \
                    "%s mip %d differs from the live reference" % (shape, mip)
            else:
                tally.add(resident.mip_numpy(mip), _restated(oracle, checker, mip, use_int8, numerics), use_int8,
                          "%s mip %d" % (shape, mip))
    tally.check()


def test_biases_too_large_for_the_matrix_product_come_from_the_table(oracle):
    """Exact numerics.  The layers of an Int8 network normally carry their bias in spare K slots of the matrix product;
    a bias that does not fit there switches the network to the bias table.  Both paths must give the
    contract's bits, also at the largest bias that still fits and at negative extremes (the FP8
    network, decoded alongside, always takes its int8 output layer's bias from the table)."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(96, 40, 6, 0, 3, 12, seed=77, network="unit"))
    geo = data.geometry
    packed = data.packed_latents()
    limit = 127 * 127 * 31 + 63  # what the 32 bias slots of layers 1 and 3 can carry
    for delta in (limit, limit + 1, -limit, -limit - 1):
        int8_blob = bytearray(data.int8_blob)
        table = np.frombuffer(bytes(int8_blob[8192 + 640:8192 + 1280]), dtype=np.int32).copy()
        table[64 + 5] = delta      # layer 1, output 5
        table[144 + 2] = -delta    # layer 3, output 2
        int8_blob[8192 + 640:8192 + 1280] = table.tobytes()
        fp8_blob = bytearray(data.fp8_blob)
        last = np.frombuffer(bytes(fp8_blob[8544:8608]), dtype=np.int32).copy()
        last[3] = delta
        fp8_blob[8544:8608] = last.tobytes()
        staged = binding.stage_network(bytes(int8_blob), binding.WEIGHTS_INT8, EXACT)
        assert staged[14848:14852].view(np.uint32)[0] == (1 if abs(delta) > limit else 0)
        checker = oracle.OracleSet(geo, packed, bytes(int8_blob), bytes(fp8_blob))
        resident = binding.ResidentTextureSet(geo, packed, bytes(int8_blob), bytes(fp8_blob), numerics=EXACT)
        for use_int8 in (True, False):
            resident.out.fill_(float("nan"))
            resident.decode(use_int8)
            _sync()
            resident.check_status()
            for mip in (0, geo.mips - 1):
                _assert_matches_contract(resident.mip_numpy(mip), checker.decode_mip(mip, use_int8, oracle.NUMERICS_SPEC),
                                         use_int8, "bias %d mip %d" % (delta, mip))


@BOTH_NUMERICS
def test_row_ranges_tile_rows_and_guard_bands(oracle, numerics):
    """Decoding a mip in row bands (the unit of tile-row sharding) gives the same bits as one
    whole decode, writes nothing outside its band, and leaves canaries around the buffer intact."""
    import torch

    data = synthetic.make_texture_set(synthetic.TextureSetSpec(160, 90, 6, 0, 2, 8, seed=21, network="unit"))
    geo = data.geometry
    resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
    resident.decode(True)
    _sync()
    whole = resident.out.clone()

    elements = binding.out_elements(geo)
    guard = 4096
    padded = torch.full((elements + 2 * guard,), -7.0, dtype=torch.float16, device=resident.device)
    band = padded[guard:guard + elements]
    bands = {0: [(0, 13), (13, 14), (14, 64), (64, 90)], 1: [(0, 45)], 2: [(5, 22)]}
    for mip, ranges in bands.items():
        for begin, end in ranges:
            params = resident.params(True, out=band, mips=[mip], row_ranges={mip: (begin, end)})
            resident.launch(params)
    _sync()
    resident.check_status()
    result = padded.cpu().numpy()
    assert (result[:guard] == -7.0).all() and (result[guard + elements:] == -7.0).all()
    expected = whole.cpu().numpy()
    c = geo.channels
    for mip, cm in enumerate(geo.color_mips):
        rows = np.zeros(cm.height, dtype=bool)
        for begin, end in bands.get(mip, []):
            rows[begin:end] = True
        got = result[guard + cm.texel_offset * c:guard + (cm.texel_offset + cm.width * cm.height) * c].reshape(cm.height, -1)
        want = expected[cm.texel_offset * c:(cm.texel_offset + cm.width * cm.height) * c].reshape(cm.height, -1)
        assert np.array_equal(got[rows].view(np.uint16), want[rows].view(np.uint16))
        assert (got[~rows] == -7.0).all()


def test_texture_set_api_decompress_and_read_channels(oracle):
    """The texture-set level of the C ABI: load from a container in host memory, Decompress,
    ReadChannels with full, subset and padded requests, to host and to device memory, for both
    internal layouts."""
    import torch

    data = synthetic.make_texture_set(synthetic.TextureSetSpec(96, 40, 6, 0, 3, 12, seed=5, network="unit"))
    geo = data.geometry
    checker = oracle.OracleSet.from_synthetic(data)
    context = binding.Context(0)
    try:
        for layout in (binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS):
            # the default numerics are the reference's: same bits as the kernel-level decode
            default_set = context.create_texture_set(data.container, layout)
            resident = binding.ResidentTextureSet.from_synthetic(data)
            for use_int8 in (True, False):
                default_set.decompress(use_int8)
                resident.decode(use_int8)
                _sync()
                for mip in range(geo.mips):
                    assert np.array_equal(default_set.read_mip(mip).view(np.uint16), resident.mip_numpy(mip).view(np.uint16))
            default_set.close()
            texture_set = context.create_texture_set(data.container, layout, EXACT)
            assert (texture_set.desc.width, texture_set.desc.channels, texture_set.desc.mips) == (96, 6, geo.mips)
            with pytest.raises(binding.NtcbError) as error:
                texture_set.read_mip(0)
            assert error.value.code == -8  # InvalidState: nothing decompressed yet
            for use_int8 in (True, False):
                milliseconds = texture_set.decompress(use_int8, with_stats=True)
                assert milliseconds > 0
                for mip in range(geo.mips):
                    expected = checker.decode_mip(mip, use_int8, oracle.NUMERICS_SPEC)
                    assert np.array_equal(texture_set.read_mip(mip).view(np.uint16), expected.view(np.uint16))
                expected = checker.decode_mip(0, use_int8, oracle.NUMERICS_SPEC)
                # channel subset
                assert np.array_equal(texture_set.read_mip(0, 1, 3).view(np.uint16), expected[:, :, 1:4].view(np.uint16))
                # padded strides into host memory: the components past the requested channels and the row gaps are zeros
                w, h = texture_set.mip_size(0)
                padded = np.full((h, w + 3, 8), 5.0, dtype=np.float16)
                texture_set.read_channels_into(0, padded.ctypes.data, False, 2, 4, pixel_stride=16, row_pitch=(w + 3) * 16)
                assert np.array_equal(padded[:, :w, :4].view(np.uint16), expected[:, :, 2:6].view(np.uint16))
                assert (padded[:, :w, 4:] == 0).all() and (padded[:, w:, :] == 0).all()
                # device destination
                target = torch.zeros((h, w, geo.channels), dtype=torch.float16, device="cuda:0")
                texture_set.read_channels_into(0, target.data_ptr(), True)
                assert np.array_equal(target.cpu().numpy().view(np.uint16), expected.view(np.uint16))
            # argument errors follow the reference's conventions
            for kwargs, code in (({"first_channel": 6}, -9), ({"num_channels": 7}, -9), ({"pixel_stride": 1}, -1),
                                 ({"pixel_stride": 6, "row_pitch": 5}, -1)):
                with pytest.raises(binding.NtcbError) as error:
                    texture_set.read_channels_into(0, target.data_ptr(), True, **kwargs)
                assert error.value.code == code
            with pytest.raises(binding.NtcbError):
                texture_set.read_channels_into(geo.mips, target.data_ptr(), True)
            # row-sharded decompress
            ranges = [(0, cm.height // 2) for cm in geo.color_mips]
            texture_set.decompress(True, row_ranges=ranges)
            texture_set.synchronize()
            texture_set.close()
    finally:
        context.close()


def test_large_sets_decode_in_row_bands_with_pipelined_readback():
    """A set whose mip 0 has 512 rows or more is decoded by the texture-set API in four row-band
    launches plus one for the other mips, and a host read of mip 0 copies band by band: same bits
    as the single launch, for fp16 and for converted pixels, in both numerics."""
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(200, 530, 6, 0, 2, 8, seed=12, network="unit"))
    geo = data.geometry
    with binding.Context(0) as context:
        for numerics in (REFERENCE, EXACT):
            resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
            texture_set = context.create_texture_set(data.container, numerics=numerics)
            for use_int8 in (True, False):
                resident.decode(use_int8)
                _sync()
                resident.check_status()
                texture_set.decompress(use_int8)
                for mip in range(geo.mips):
                    assert np.array_equal(texture_set.read_mip(mip).view(np.uint16), resident.mip_numpy(mip).view(np.uint16)), mip
                # a second read, a sub-range read and a converted decode see the same texels
                assert np.array_equal(texture_set.read_mip(0, 1, 3).view(np.uint16), resident.mip_numpy(0)[:, :, 1:4].view(np.uint16))
                conversion = binding.make_conversion(binding.CHANNEL_FORMAT_UNORM8, 6)
                fused, _ = texture_set.decompress_converted(conversion, use_int8)
                texture_set.decompress(use_int8)
                for mip in (0, 1, geo.mips - 1):
                    two_pass = texture_set.read_mip(mip, 0, 6, binding.CHANNEL_FORMAT_UNORM8)
                    assert np.array_equal(fused[mip], two_pass), mip
            texture_set.close()


def test_live_reference_comparison(oracle):
    """Runs the unmodified reference decoder (oracle/_ref) on this GPU next to ours on a set the
    fixtures do not contain."""
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libntc_ref.so is not built")
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(256, 192, 8, 0, 4, 8, seed=77, network="unit"))
    geo = data.geometry
    reference = oracle.ReferenceDecoder(data.container, geo.channels)
    resident = binding.ResidentTextureSet.from_synthetic(data, numerics=EXACT)
    identical = binding.ResidentTextureSet.from_synthetic(data, numerics=REFERENCE)
    checker = oracle.OracleSet.from_synthetic(data)
    try:
        for use_int8 in (True, False):
            reference.decompress(use_int8)
            resident.decode(use_int8)
            identical.decode(use_int8)
            _sync()
            for mip in range(geo.mips):
                cm = geo.color_mips[mip]
                theirs = reference.read_mip(mip, cm.width, cm.height)
                # the reference's numerics: identical bits
                assert np.array_equal(identical.mip_numpy(mip).view(np.uint16), theirs.view(np.uint16))
            for mip in (0, 1, 2):
                cm = geo.color_mips[mip]
                theirs = reference.read_mip(mip, cm.width, cm.height)
                ours = resident.mip_numpy(mip)
                assert psnr_db(ours, theirs) >= 50.0
                # and the reference-emulating CPU numerics reproduce the live reference
                emulated = checker.decode_mip(mip, use_int8, oracle.NUMERICS_REF)
                different = int((emulated.view(np.uint16) != theirs.view(np.uint16)).sum())
                assert different <= max(2, theirs.size * 2e-4)
    finally:
        reference.close()


@BOTH_NUMERICS
def test_full_size_properties_of_the_pbr_configuration(oracle, numerics):
    """4096x4096, 12 channels, 13 mips, FP8: the CPU restatement cannot decode 22 M texels in
    seconds, so the full-size check uses properties: a second decode reproduces the first bit for
    bit, a row-banded decode reproduces the whole decode, and 20,000 randomly chosen texels over all
    mips agree with the CPU restatement."""
    import torch

    data = synthetic.make_texture_set(synthetic.config_spec(1))
    geo = data.geometry
    resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
    resident.decode(False)
    _sync()
    resident.check_status()
    first = resident.out.clone()
    resident.out.zero_()
    bands = {mip: (0, cm.height) for mip, cm in enumerate(geo.color_mips)}
    for part in range(8):  # mip 0..2 in eight row bands, as eight GPUs would share them
        ranges = {}
        for mip in (0, 1, 2):
            h = geo.color_mips[mip].height
            ranges[mip] = (part * h // 8, (part + 1) * h // 8)
        resident.launch(resident.params(False, mips=[0, 1, 2], row_ranges=ranges))
    resident.launch(resident.params(False, mips=list(range(3, geo.mips)), row_ranges=bands))
    _sync()
    resident.check_status()
    assert torch.equal(first.view(torch.int16), resident.out.view(torch.int16))

    checker = oracle.OracleSet.from_synthetic(data)
    queries = synthetic.make_queries(20000, max_lod=geo.mips - 0.001, seed=9)
    expected = (checker.sample(queries, False, oracle.NUMERICS_SPEC) if numerics == EXACT
                else checker.sample(queries, False, oracle.NUMERICS_REF))
    c = geo.channels
    flat = first.cpu().numpy()
    mismatched = 0
    for q, want in zip(queries, expected):
        mip = int(np.floor(q[2]))
        cm = geo.color_mips[mip]
        x = min(cm.width - 1, int(np.floor(np.float32(q[0]) * np.float32(cm.width))))
        y = min(cm.height - 1, int(np.floor(np.float32(q[1]) * np.float32(cm.height))))
        start = (cm.texel_offset + y * cm.width + x) * c
        mismatched += int(not np.array_equal(flat[start:start + c].view(np.uint16), want.view(np.uint16)))
    assert mismatched <= (0 if numerics == EXACT else 8)  # the CPU model of the reference's rounding is 99.998 % exact


@BOTH_NUMERICS
@pytest.mark.parametrize("shape", [(96, 40, 6, 0, 3, 12), (256, 256, 12, 0, 4, 12), (33, 17, 2, 0, 1, 4)])
def test_inference_on_sample_matches_contract(oracle, shape, numerics):
    """Random (u, v, lod) queries: every answer equals the entry of the fully decoded mip chain (so,
    with the default numerics, the reference's bits) and the CPU restatement of the selected texel
    (bit-exact for exact accumulation, within the CPU model's accuracy for the reference numerics)."""
    import torch

    w, h, c, mips, g, f = shape
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(w, h, c, mips, g, f, seed=3, network="unit"))
    geo = data.geometry
    checker = oracle.OracleSet.from_synthetic(data)
    resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
    queries = synthetic.make_queries(5000, max_lod=geo.mips + 0.5, seed=9)
    queries[:8] = [[0, 0, 0], [0.999999, 0.999999, 0], [0.5, 0.5, -1.0], [0.25, 0.75, 99.0], [1.0, 1.0, 1.0],
                   [0.0, 1.0, geo.mips - 1], [0.3, 0.6, 1.999], [0.7, 0.1, 2.0]]
    device_queries = torch.from_numpy(queries).cuda()
    for use_int8 in (True, False):
        got = resident.sample(device_queries, use_int8).cpu().numpy()
        _sync()
        resident.check_status()
        if numerics == EXACT:
            expected = checker.sample(queries, use_int8, oracle.NUMERICS_SPEC)
            assert np.array_equal(got.view(np.uint16), expected.view(np.uint16))
        elif oracle.reference_available():
            # identical bits to a gather from the live reference's decoded mip chain
            chain = reference_chain(oracle, data, use_int8).cpu().numpy().reshape(-1, geo.channels)
            for q in range(queries.shape[0]):
                mip = int(max(0, min(geo.mips - 1, np.floor(queries[q, 2]))))
                cm = geo.color_mips[mip]
                x = int(max(0, min(cm.width - 1, np.floor(np.float32(queries[q, 0]) * np.float32(cm.width)))))
                y = int(max(0, min(cm.height - 1, np.floor(np.float32(queries[q, 1]) * np.float32(cm.height)))))
                assert np.array_equal(got[q].view(np.uint16), chain[cm.texel_offset + y * cm.width + x].view(np.uint16)), (q, mip, x, y)
        else:
            expected = checker.sample(queries, use_int8, oracle.NUMERICS_REF)
            different = int((got.view(np.uint16) != expected.view(np.uint16)).sum())
            assert different <= max(2, got.size * 2e-4)
        resident.decode(use_int8)
        _sync()
        for q in range(0, 5000, 7):
            mip = int(max(0, min(geo.mips - 1, np.floor(queries[q, 2]))))
            cm = geo.color_mips[mip]
            x = int(max(0, min(cm.width - 1, np.floor(np.float32(queries[q, 0]) * np.float32(cm.width)))))
            y = int(max(0, min(cm.height - 1, np.floor(np.float32(queries[q, 1]) * np.float32(cm.height)))))
            assert np.array_equal(resident.mip_numpy(mip)[y, x].view(np.uint16), got[q].view(np.uint16))
    # zero queries is a no-op
    assert resident.sample(device_queries[:0], True).shape[0] == 0


@BOTH_NUMERICS
@pytest.mark.parametrize("shape", [(256, 256, 12, 0, 4, 16), (512, 384, 12, 0, 4, 12), (200, 136, 6, 0, 2, 8), (96, 40, 6, 0, 3, 12),
                                   (33, 17, 2, 0, 1, 4)])
def test_inference_on_sample_reads_interleaved_latents(shape, numerics):
    """ntcb_interleave_latents makes the pixel-major copy - layer l of pixel p of the grid at `offset` at element
    offset / layers * slot + p * slot + l, slot = 1, 2, 4, 4 elements for 1 - 4 layers, a zero behind three - and a
    query answered from that copy (NTCB_LATENTS_INTERLEAVED: one aligned load per tap) has the bits of the query
    answered from the file's planes.  Enough queries for several tiles per CTA."""
    import torch

    w, h, c, mips, g, f = shape
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(w, h, c, mips, g, f, seed=5, network="unit"))
    geo = data.geometry
    resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
    planar = resident.latents.cpu().numpy()
    relaid = resident.interleave_latents().cpu().numpy()
    _sync()
    layers = f // 4
    slot = 4 if layers == 3 else layers
    assert relaid.size == planar.size // layers * slot
    params = binding.fill_params(geo, 0, 0, 0, 0, binding.WEIGHTS_INT8)
    seen = set()
    for m in range(params.numMips):
        mip = params.mips[m]
        for offset, plane, gw, gh in ((mip.hiOffset, mip.hiPlane, mip.hiWidth, mip.hiHeight),
                                      (mip.loOffset, mip.loPlane, mip.loWidth, mip.loHeight)):
            if offset in seen:
                continue
            seen.add(offset)
            pixels = gw * gh
            want = np.zeros((pixels, slot), dtype=planar.dtype)
            for l in range(layers):
                want[:, l] = planar[offset + l * plane:offset + l * plane + pixels]
            first = offset // layers * slot
            assert np.array_equal(relaid[first:first + pixels * slot].reshape(pixels, slot), want), (m, offset)
    queries = synthetic.make_queries(700000, max_lod=geo.mips + 0.5, seed=11)
    queries[:4] = [[0, 0, 0], [0.999999, 0.999999, 0], [1.0, 1.0, 1.0], [0.0, 1.0, geo.mips - 1]]
    device_queries = torch.from_numpy(queries).cuda()
    for use_int8 in (True, False):
        for count in (700000, 1000, 1):
            from_planes = resident.sample(device_queries[:count], use_int8).cpu().numpy()
            from_copy = resident.sample(device_queries[:count], use_int8, interleaved=True).cpu().numpy()
            _sync()
            resident.check_status()
            assert np.array_equal(from_planes.view(np.uint16), from_copy.view(np.uint16)), (use_int8, count)


@BOTH_NUMERICS
def test_texture_set_sample_answers_with_the_decompressed_texels(numerics):
    """ntcb_texture_set_sample: before any decompress (the call uploads the compressed data and makes its
    pixel-major copy), after one, and after LoadFromMemory put another set into the same buffers (both copies
    stale) - every answer is the texel a decompress of the set currently loaded writes."""
    import torch

    specs = [synthetic.TextureSetSpec(200, 136, 6, 0, 2, 12, seed=41, network="unit"),
             synthetic.TextureSetSpec(200, 136, 6, 0, 2, 12, seed=42, network="unit")]
    sets = [synthetic.make_texture_set(spec) for spec in specs]
    geo = sets[0].geometry
    queries = synthetic.make_queries(30000, max_lod=geo.mips + 0.5, seed=13)
    queries[:3] = [[0, 0, 0], [0.999999, 0.999999, 0], [1.0, 1.0, geo.mips - 1]]
    device_queries = torch.from_numpy(queries).cuda()

    def expected(texture_set, use_int8):
        texture_set.decompress(use_int8)
        mips = [texture_set.read_mip(m) for m in range(geo.mips)]
        want = np.zeros((queries.shape[0], geo.channels), dtype=np.float16)
        for q in range(queries.shape[0]):
            mip = int(max(0, min(geo.mips - 1, np.floor(queries[q, 2]))))
            cm = geo.color_mips[mip]
            x = int(max(0, min(cm.width - 1, np.floor(np.float32(queries[q, 0]) * np.float32(cm.width)))))
            y = int(max(0, min(cm.height - 1, np.floor(np.float32(queries[q, 1]) * np.float32(cm.height)))))
            want[q] = mips[mip][y, x]
        return want

    with binding.Context() as context:
        texture_set = context.create_texture_set(sets[0].container, numerics=numerics)
        first = {use_int8: texture_set.sample(device_queries, use_int8).cpu().numpy() for use_int8 in (True, False)}
        for use_int8 in (True, False):
            assert np.array_equal(first[use_int8].view(np.uint16), expected(texture_set, use_int8).view(np.uint16))
            again = texture_set.sample(device_queries, use_int8).cpu().numpy()
            assert np.array_equal(again.view(np.uint16), first[use_int8].view(np.uint16))
        texture_set.load_from_memory(sets[1].container)
        other = texture_set.sample(device_queries, True).cpu().numpy()
        assert not np.array_equal(other.view(np.uint16), first[True].view(np.uint16))
        assert np.array_equal(other.view(np.uint16), expected(texture_set, True).view(np.uint16))
        assert texture_set.sample(device_queries[:0], True).shape[0] == 0
        texture_set.close()


@pytest.mark.parametrize("numerics", [binding.NUMERICS_REFERENCE, binding.NUMERICS_EXACT], ids=["reference", "exact"])
def test_decode_launches_replay_from_a_cuda_graph(numerics):
    """ntcb_decode only queues work on the stream it is given, so a batch of decodes can be captured once
    in a CUDA graph and replayed (after one eager call per kernel: its first use on a device sets a function
    attribute).  Three sets, both weight modes, replayed twice: the same bits as the eager launches."""
    import torch

    specs = [synthetic.TextureSetSpec(200, 136, 6, 0, 2, 8, seed=31, network="unit"),
             synthetic.TextureSetSpec(96, 40, 12, 0, 4, 12, seed=32, network="unit"),
             synthetic.TextureSetSpec(64, 64, 4, 0, 3, 16, seed=33, network="unit")]
    residents = [binding.ResidentTextureSet.from_synthetic(synthetic.make_texture_set(spec), numerics=numerics) for spec in specs]
    for use_int8 in (True, False):
        eager = []
        for resident in residents:
            resident.decode(use_int8)
            torch.cuda.synchronize()
            resident.check_status()
            eager.append(resident.out.clone())
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for resident in residents:
                    resident.decode(use_int8)
        for _ in range(2):
            for resident in residents:
                resident.out.fill_(float("nan"))
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            for resident, expected in zip(residents, eager):
                resident.check_status()
                assert torch.equal(resident.out.view(torch.int16), expected.view(torch.int16))


def test_an_expired_wait_is_reported_and_leaves_the_gpu_usable():
    """The kernels' timeout path, walked without hanging or faulting anything: the test hook makes
    the FIRST wait of every CTA - for the network image, before any tile is touched and with no
    tensor-core work in flight - run out at once.  Every kernel must then report the wait in the
    status words ({1, no tile, no layer}), the host must turn it into NTCB_ERR_DEVICE_TIMEOUT, and
    the next ordinary decode on the same objects must be bit-correct again."""
    import torch

    lib = binding.lib()
    data = synthetic.make_texture_set(synthetic.TextureSetSpec(200, 72, 6, 0, 2, 8, seed=31, network="unit"))
    geo = data.geometry
    queries = torch.from_numpy(synthetic.make_queries(3000, max_lod=geo.mips - 0.001, seed=5)).cuda()
    with binding.Context(0) as context:
        for numerics in (REFERENCE, EXACT):
            resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
            texture_set = context.create_texture_set(data.container, numerics=numerics)
            for use_int8 in (True, False):
                resident.decode(use_int8)
                good_samples = resident.sample(queries, use_int8)
                _sync()
                resident.check_status()
                good = resident.out.clone()

                assert lib.ntcb_debug_set_network_wait_polls(0) == binding.DEFAULT_WAIT_POLLS
                try:
                    resident.out.fill_(float("nan"))
                    resident.decode(use_int8)
                    _sync()
                    assert resident.status.cpu().numpy().view(np.uint32).tolist()[:3] == [1, 0xFFFFFFFF, 0xFFFFFFFF]
                    with pytest.raises(binding.NtcbError) as error:
                        resident.check_status()
                    assert error.value.code == -7
                    assert bool(torch.isnan(resident.out).all())  # the CTAs left before touching a tile
                    resident.status.zero_()
                    resident.sample(queries, use_int8)
                    _sync()
                    assert resident.status.cpu().numpy().view(np.uint32).tolist()[:3] == [1, 0xFFFFFFFF, 0xFFFFFFFF]
                    resident.status.zero_()
                    # the texture-set level reports it as a status code with a message
                    with pytest.raises(binding.NtcbError) as error:
                        texture_set.decompress(use_int8, with_stats=True)
                    assert error.value.code == -7 and "wait" in str(error.value)
                finally:
                    assert lib.ntcb_debug_set_network_wait_polls(binding.DEFAULT_WAIT_POLLS) == 0

                resident.decode(use_int8)
                again = resident.sample(queries, use_int8)
                _sync()
                resident.check_status()
                assert torch.equal(resident.out.view(torch.int16), good.view(torch.int16))
                assert torch.equal(again.view(torch.int16), good_samples.view(torch.int16))
                texture_set.decompress(use_int8, with_stats=True)
                for mip in range(geo.mips):
                    assert np.array_equal(texture_set.read_mip(mip).view(np.uint16), resident.mip_numpy(mip).view(np.uint16))
            texture_set.close()
