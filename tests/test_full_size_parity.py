"""Full-size parity of the benchmark configurations against a LIVE run of the unmodified reference.

Every configuration the benchmark names is decoded twice on the same GPU - by the reference's own
CUDA decoder (oracle/_ref, driven through ntc::CreateContext -> CreateCompressedTextureSetFromMemory
-> ITextureSet::Decompress -> ITextureSet::ReadChannels(FLOAT16, AddressSpace::Device);
src/TextureSet.cpp:1664-1897, :915-985) and by this library's default numerics through the C ABI -
and EVERY texel of EVERY mip is compared on the device.  The bar is identical bits, in both output
layouts.  Inference on sample (configuration 4) is compared with a gather from the reference's
decoded mip chain.

The small golden fixtures (tests/golden) pin the bits on shapes of at most 128 x 128; these tests pin
them on the shapes that are benchmarked, which exercise other tile counts, footprint sizes, the
row-band path and the direct (unstaged) latent reads of strongly minified mips.
"""
import pytest

from conftest import reference_chain

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, synthetic  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def live(oracle):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref/libntc_ref.so is not built")
    return oracle


def _assert_identical(resident, chain, what):
    """Every value of every mip, compared on the device as 16-bit patterns."""
    import torch

    geo = resident.geometry
    c = geo.channels
    for mip, cm in enumerate(geo.color_mips):
        ours = resident.mip_view(mip)
        if resident.layout == binding.LAYOUT_PLANAR_PAIRS:
            ours = ours.permute(0, 2, 1, 3).reshape(cm.height, cm.width, c)
        theirs = chain[cm.texel_offset * c:(cm.texel_offset + cm.width * cm.height) * c].view(cm.height, cm.width, c)
        if not torch.equal(ours.view(torch.int16), theirs.view(torch.int16)):
            different = int((ours.view(torch.int16) != theirs.view(torch.int16)).sum())
            raise AssertionError("%s, mip %d: %d of %d values differ from the reference's decode"
                                 % (what, mip, different, theirs.numel()))


def _check_configuration(oracle, spec, modes, what):
    import torch

    data = synthetic.make_texture_set(spec)
    for use_int8 in modes:
        chain = reference_chain(oracle, data, use_int8)
        for layout in (binding.LAYOUT_INTERLEAVED, binding.LAYOUT_PLANAR_PAIRS):
            resident = binding.ResidentTextureSet.from_synthetic(data, layout=layout)
            assert resident.numerics == binding.NUMERICS_REFERENCE
            resident.out.fill_(float("nan"))
            resident.decode(use_int8)
            torch.cuda.synchronize()
            resident.check_status()
            _assert_identical(resident, chain, "%s, %s weights, layout %d" % (what, "int8" if use_int8 else "fp8", layout))
            del resident
        del chain
        torch.cuda.empty_cache()


def test_configuration_0_matches_the_live_reference(live):
    """1024 x 1024, 4 channels, mip 0 only, latent shape {2, 8}, int8 weights, seed 0."""
    _check_configuration(live, synthetic.config_spec(0), (True,), "configuration 0")


@pytest.mark.parametrize("grid_scale", [4, 2])
def test_configuration_1_matches_the_live_reference(live, grid_scale):
    """4096 x 4096, 12 channels, 13 mips, 12 features, FP8 hidden layers (the metric's workload) and
    the set's Int8 network; grid scale 4 (the benchmark's) and 2."""
    spec = synthetic.config_spec(1)
    spec.grid_scale = grid_scale
    _check_configuration(live, spec, (False, True), "configuration 1, grid scale %d" % grid_scale)


@pytest.mark.parametrize("set_index", [0, 63])
def test_configuration_2_matches_the_live_reference(live, set_index):
    """One set of the batch: 2048 x 2048, 8 channels, 12 mips, latent shape {4, 8}, int8 (seeds 100 and 163)."""
    _check_configuration(live, synthetic.config_spec(2, set_index), (True,), "configuration 2, set %d" % set_index)


def test_configuration_3_matches_the_live_reference(live):
    """8192 x 8192, 16 channels, 14 mips, latent shape {4, 16}, int8, seed 7 (2.9 GB of texels per decode)."""
    _check_configuration(live, synthetic.config_spec(3), (True,), "configuration 3")


def test_configuration_4_matches_a_gather_from_the_live_reference(live):
    """16,777,216 random (u, v, lod) queries on the configuration-1 set: every answer of ntcb_sample
    equals the texel the query selects in the REFERENCE's decoded mip chain."""
    import torch

    data = synthetic.make_texture_set(synthetic.config_spec(4))
    geo = data.geometry
    c = geo.channels
    chain = reference_chain(live, data, False).view(-1, c)
    queries = torch.from_numpy(synthetic.make_queries(1 << 24, max_lod=12.0, seed=9)).cuda()
    resident = binding.ResidentTextureSet.from_synthetic(data, allocate_output=False)
    got = resident.sample(queries, False)
    torch.cuda.synchronize()
    resident.check_status()

    # the selection rule of ntcb_sample, in the same binary32 operations
    mip = queries[:, 2].floor().clamp(0, geo.mips - 1).to(torch.int64)
    widths = torch.tensor([cm.width for cm in geo.color_mips], device="cuda:0")
    heights = torch.tensor([cm.height for cm in geo.color_mips], device="cuda:0")
    offsets = torch.tensor([cm.texel_offset for cm in geo.color_mips], device="cuda:0")
    w, h = widths[mip], heights[mip]
    x = torch.minimum((queries[:, 0] * w.to(torch.float32)).floor().to(torch.int64), w - 1).clamp_(min=0)
    y = torch.minimum((queries[:, 1] * h.to(torch.float32)).floor().to(torch.int64), h - 1).clamp_(min=0)
    expected = chain[offsets[mip] + y * w + x]
    assert torch.equal(got.view(torch.int16), expected.view(torch.int16)), \
        "%d of %d values differ" % (int((got.view(torch.int16) != expected.view(torch.int16)).sum()), got.numel())
    # the same from the pixel-major copy of the latents (12 features: slots of four elements, one load per tap)
    again = resident.sample(queries, False, interleaved=True)
    torch.cuda.synchronize()
    resident.check_status()
    assert torch.equal(again.view(torch.int16), expected.view(torch.int16))
