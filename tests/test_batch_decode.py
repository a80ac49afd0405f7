"""Decoding on several devices (ntcb_plan_batch / ntcb_decode_batch).

The scheduler - cutting a job into units, handing them out largest first, trying a failed unit on
another device, retiring a device that keeps failing - is independent of the GPU work, so it is
tested here on the CPU with workers that the test supplies: a worker that fails, one that fails
once, one that is slow.  No GPU is faulted, hung or even touched by these tests.  The GPU tests at
the end run the real path and compare the gathered host images with a plain single-launch decode.
"""
import collections
import threading
import time

import numpy as np
import pytest

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import binding, synthetic  # noqa: E402

SHAPES = [
    ([(2048, 2048, 12)] * 64, 8),      # the batch configuration: 64 sets on 8 devices
    ([(8192, 8192, 14)], 8),           # one large set cut into bands of tile rows
    ([(4096, 4096, 13)], 1),
    ([(100, 37, 7), (513, 1025, 11), (64, 64, 1)], 3),
    ([(1, 1, 1)], 4),
]


@pytest.mark.parametrize("shapes,devices", SHAPES)
def test_plan_covers_every_row_exactly_once(shapes, devices):
    units = binding.plan_batch(shapes, devices)
    covered = collections.Counter()
    for unit in units:
        texels = 0
        for mip in range(binding.MAX_MIPS):
            begin, end = unit.rowBegin[mip], unit.rowEnd[mip]
            assert 0 <= begin <= end
            width, height, mips = shapes[unit.item]
            if end > begin:
                assert mip < mips and end <= max(height >> mip, 1)
                # bands start on tile rows, so that no tile of the decode kernel straddles two units
                assert begin % 8 == 0
                texels += (end - begin) * max(width >> mip, 1)
                for row in range(begin, end):
                    covered[(unit.item, mip, row)] += 1
        assert texels == unit.texels
    assert set(covered.values()) == {1}
    assert len(covered) == sum(max(h >> m, 1) for (w, h, mips) in shapes for m in range(mips))
    assert [u.texels for u in units] == sorted((u.texels for u in units), reverse=True)  # largest first


def test_plan_balances_the_benchmark_jobs():
    # one 8192 x 8192 set on 8 devices: four units per device, none much larger than the others
    units = binding.plan_batch([(8192, 8192, 14)], 8)
    assert len(units) == 32
    assert units[0].texels <= 1.4 * units[-1].texels
    # 64 sets on 8 devices: enough items to balance, every set stays whole (one parse and upload per set)
    units = binding.plan_batch([(2048, 2048, 12)] * 64, 8)
    assert len(units) == 64 and units[0].texels == 5592405
    # 24 sets on 8 devices: (mip 0) and (the rest) of every set
    units = binding.plan_batch([(2048, 2048, 12)] * 24, 8)
    assert len(units) == 48 and units[0].texels == 2048 * 2048
    # 8 sets on 8 devices: four bands of tile rows each
    assert len(binding.plan_batch([(2048, 2048, 12)] * 8, 8)) == 32


@pytest.fixture(scope="module")
def containers():
    return [synthetic.make_texture_set(synthetic.TextureSetSpec(256, 256, 4, 0, 2, 8, seed=s)).container for s in range(6)]


def _run(containers, worker, devices=(0, 1, 2, 3), **kwargs):
    log, lock = [], threading.Lock()

    def logged(device, unit):
        result = worker(device, unit)
        with lock:
            log.append((device, unit.item, result))
        return result

    code, statuses, units = binding.decode_batch(containers, devices, True, worker=logged, **kwargs)
    return code, statuses, units, log


def test_every_unit_runs_once_when_nothing_fails(containers):
    code, statuses, units, log = _run(containers, lambda device, unit: 0)
    assert code == 0 and statuses == [0] * 6
    assert len(log) == len(units) == 18  # each 256 x 256 set: three bands
    assert all(unit.attempts == 1 and unit.status == 0 for unit in units)


def test_a_failing_device_is_retired_and_its_units_run_elsewhere(containers):
    code, statuses, units, log = _run(containers, lambda device, unit: -2 if device == 1 else 0)
    assert code == 0 and statuses == [0] * 6
    failures = [entry for entry in log if entry[2] != 0]
    assert 1 <= len(failures) <= 4 and all(device == 1 for device, _, _ in failures)  # two in a row retire it (two threads may overlap)
    assert all(unit.status == 0 and unit.device != 1 for unit in units)
    assert max(unit.attempts for unit in units) == 2


def test_a_transient_failure_is_retried_on_another_device(containers):
    calls = {"n": 0}
    lock = threading.Lock()

    def flaky(device, unit):
        with lock:
            calls["n"] += 1
            return -7 if calls["n"] in (2, 7) else 0  # NTCB_ERR_DEVICE_TIMEOUT twice, far enough apart not to retire a device

    code, statuses, units, log = _run(containers, flaky)
    assert code == 0 and statuses == [0] * 6
    # two extra attempts in all (the second failure may hit the unit that failed first, when it comes back)
    assert sum(unit.attempts - 1 for unit in units) == 2 and len(log) == len(units) + 2
    assert all(unit.status == 0 for unit in units)


def test_failure_on_every_device_is_reported_not_waited_for(containers):
    start = time.time()
    code, statuses, units, log = _run(containers, lambda device, unit: -2)
    assert time.time() - start < 5.0
    assert code == -2 and statuses == [-2] * 6
    assert b"could not be decoded" in binding.lib().ntcb_last_error()
    assert all(unit.status != 0 for unit in units if unit.attempts)
    assert len(log) <= 2 * 4 * 2  # every device is retired after two failures (per thread at most two more)


def test_the_attempt_limit_is_respected(containers):
    code, statuses, units, log = _run(containers, lambda device, unit: -2 if unit.item == 3 else 0, max_attempts=2,
                                      devices=(0, 1, 2, 3, 4, 5))
    assert code == -2
    assert [s == 0 for s in statuses] == [True, True, True, False, True, True]
    assert all(unit.attempts <= 2 for unit in units)


def test_a_slow_device_gets_less_work(containers):
    def slow(device, unit):
        time.sleep(0.08 if device == 0 else 0.004)
        return 0

    code, statuses, units, log = _run(containers, slow)
    assert code == 0
    per_device = collections.Counter(device for device, _, _ in log)
    assert per_device[0] <= 2 and sum(per_device.values()) == 18


def test_a_decoder_runs_batch_after_batch_with_the_same_workers(containers):
    """ntcb_batch_decoder_*: the threads survive the runs; a run in which a device keeps failing retires it for
    that run only."""
    seen = collections.Counter()
    lock = threading.Lock()
    failing = {"device": None}

    def worker(device, unit):
        with lock:
            seen[(threading.get_ident(), device)] += 1
        return -2 if device == failing["device"] else 0

    with binding.BatchDecoder([0, 1, 2], worker=worker) as decoder:
        code, statuses, units = decoder.run(containers, True)
        assert code == 0 and statuses == [0] * 6 and all(unit.attempts == 1 for unit in units)
        threads_after_first = {ident for ident, _ in seen}
        failing["device"] = 1
        code, statuses, units = decoder.run(containers[:3], True)
        assert code == 0 and statuses == [0] * 3 and all(unit.device != 1 and unit.status == 0 for unit in units)
        failing["device"] = None
        code, statuses, units = decoder.run(containers, True)
        assert code == 0 and any(unit.device == 1 for unit in units)  # back in the next run
        assert {ident for ident, _ in seen} == threads_after_first and len(threads_after_first) == 3
        assert decoder.run([b"not a container"], True)[0] == -3 and b"item 0" in binding.lib().ntcb_last_error()


def test_arguments_are_checked(containers):
    assert binding.decode_batch([], [0], True, worker=lambda d, u: 0)[0] == -1
    assert binding.decode_batch(containers[:1], [], True, worker=lambda d, u: 0)[0] == -1
    assert binding.decode_batch([b"not a container" * 10], [0], True, worker=lambda d, u: 0)[0] == -3
    # without the test hook every item needs a host image
    assert binding.decode_batch(containers[:1], [0], True)[0] == -1


@pytest.mark.gpu
@pytest.mark.parametrize("numerics", [binding.NUMERICS_REFERENCE, binding.NUMERICS_EXACT], ids=["reference", "exact"])
def test_gathered_host_images_equal_a_plain_decode(numerics):
    """The real path on the GPUs that are there (one device listed twice when there is only one): a
    batch of small sets plus one set large enough to be cut into row bands; every byte of every
    host image equals what one ordinary launch decodes."""
    import torch

    # two sets share a shape: a worker that meets both loads the second into the buffers of the first
    specs = [synthetic.TextureSetSpec(200, 136, 6, 0, 2, 8, seed=11, network="unit"),
             synthetic.TextureSetSpec(64, 64, 4, 0, 4, 12, seed=12, network="unit"),
             synthetic.TextureSetSpec(1024, 768, 8, 0, 4, 8, seed=13, network="unit"),
             synthetic.TextureSetSpec(200, 136, 6, 0, 2, 8, seed=14, network="unit")]
    sets = [synthetic.make_texture_set(spec) for spec in specs]
    devices = list(range(min(torch.cuda.device_count(), 4)))
    if len(devices) == 1:
        devices = [0, 0]
    images = [torch.full((data.geometry.total_texels * data.geometry.channels,), -5.0, dtype=torch.float16).pin_memory()
              for data in sets]
    flags = [True, False, True, True]
    code, statuses, units = binding.decode_batch([data.container for data in sets], devices, flags, images, numerics=numerics)
    assert code == 0, binding.lib().ntcb_last_error()
    assert statuses == [0, 0, 0, 0] and all(unit.status == 0 and unit.attempts == 1 for unit in units)
    assert len({unit.item for unit in units}) == 4 and len(units) > 4
    for data, image, use_int8 in zip(sets, images, flags):
        resident = binding.ResidentTextureSet.from_synthetic(data, numerics=numerics)
        resident.decode(use_int8)
        torch.cuda.synchronize()
        resident.check_status()
        assert torch.equal(resident.out.cpu().view(torch.int16), image.view(torch.int16))


@pytest.mark.gpu
def test_a_texture_set_reloaded_in_place_decodes_like_a_fresh_one():
    """ITextureSet::LoadFromMemory: a second set of the same shape goes into the buffers of the first (what a
    batch worker does between items); a set of another shape is refused and nothing changes."""
    import torch

    first = synthetic.make_texture_set(synthetic.TextureSetSpec(200, 136, 6, 0, 2, 8, seed=21, network="unit"))
    second = synthetic.make_texture_set(synthetic.TextureSetSpec(200, 136, 6, 0, 2, 8, seed=22, network="unit"))
    other = synthetic.make_texture_set(synthetic.TextureSetSpec(200, 136, 6, 0, 4, 8, seed=23, network="unit"))
    with binding.Context() as context:
        fresh = {}
        for name, data in (("first", first), ("second", second)):
            texture_set = context.create_texture_set(data.container)
            texture_set.decompress(True)
            fresh[name] = [texture_set.read_mip(m) for m in range(data.geometry.mips)]
            texture_set.close()
        assert not np.array_equal(fresh["first"][0], fresh["second"][0])
        texture_set = context.create_texture_set(first.container)
        texture_set.decompress(True)
        texture_set.load_from_memory(second.container)
        with pytest.raises(binding.NtcbError):
            texture_set.read_mip(0)  # decoded texels of the previous set are not handed out
        texture_set.decompress(True)
        assert all(np.array_equal(texture_set.read_mip(m), fresh["second"][m]) for m in range(second.geometry.mips))
        with pytest.raises(binding.NtcbError) as refused:
            texture_set.load_from_memory(other.container)
        assert refused.value.code == -4
        texture_set.decompress(True)
        assert all(np.array_equal(texture_set.read_mip(m), fresh["second"][m]) for m in range(second.geometry.mips))
        texture_set.load_from_memory(first.container)
        texture_set.decompress(True)
        assert all(np.array_equal(texture_set.read_mip(m), fresh["first"][m]) for m in range(first.geometry.mips))
        texture_set.close()


@pytest.mark.gpu
def test_a_device_that_does_not_exist_is_retired_and_the_job_completes():
    """A listed device whose context cannot be created (an index beyond the machine's GPUs: a host-side
    failure, nothing is launched on it) takes no work; the other device decodes everything."""
    import torch

    data = synthetic.make_texture_set(synthetic.TextureSetSpec(256, 256, 4, 0, 2, 8, seed=3, network="unit"))
    image = torch.zeros(data.geometry.total_texels * data.geometry.channels, dtype=torch.float16).pin_memory()
    code, statuses, units = binding.decode_batch([data.container], [0, 4096], True, [image])
    assert code == 0 and statuses == [0]
    assert all(unit.device == 0 for unit in units)
    resident = binding.ResidentTextureSet.from_synthetic(data)
    resident.decode(True)
    torch.cuda.synchronize()
    assert torch.equal(resident.out.cpu().view(torch.int16), image.view(torch.int16))
