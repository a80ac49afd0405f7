"""Multi-GPU partitioning: plan properties, and the N > 1 path end to end on CPU with two gloo
ranks (each rank "decodes" its share with the CPU restatement standing in for the GPU, rank 0
gathers and the result must equal a single-process decode)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import __graft_entry__ as entry

entry.load_package()
from rtxntc_library_b200 import sharding, synthetic  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_batch_plan_covers_everything_once_and_balances():
    geometries = [synthetic.config_spec(2, i).geometry() for i in range(64)]
    for world in (1, 2, 4, 8):
        plan = sharding.plan_batch(geometries, world)
        seen = sorted((u.set_index, m) for rank in plan for u in rank for m in u.mips)
        assert seen == sorted((i, m) for i, g in enumerate(geometries) for m in range(g.mips))
        loads = [sum(u.texels for u in rank) for rank in plan]
        assert sum(loads) == sum(g.total_texels for g in geometries)
        assert max(loads) <= min(loads) * 1.02  # 64 equal sets split evenly


def test_batch_plan_with_unequal_sets():
    geometries = [synthetic.TextureSetSpec(s, s, 4, 0, 4, 8, seed=0).geometry() for s in (4096, 2048, 2048, 1024, 512, 512, 256)]
    plan = sharding.plan_batch(geometries, 3)
    loads = [sum(u.texels for u in rank) for rank in plan]
    assert sum(loads) == sum(g.total_texels for g in geometries)
    # the largest unit (mip 0 of the 4096^2 set) bounds the makespan
    assert max(loads) == 4096 * 4096


@pytest.mark.parametrize("shape", [(8192, 8192, 16, 0, 4, 16), (4096, 4096, 12, 0, 4, 12), (1000, 3000, 3, 0, 2, 8), (64, 64, 4, 0, 2, 8)])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_row_plan_partitions_every_mip(shape, world):
    geo = synthetic.TextureSetSpec(*shape, seed=0).geometry()
    plan = sharding.plan_rows(geo, world)
    for mip, cm in enumerate(geo.color_mips):
        bands = sorted(plan[rank][mip] for rank in range(world) if plan[rank][mip][1] > plan[rank][mip][0])
        assert bands[0][0] == 0 and bands[-1][1] == cm.height
        for (b0, e0), (b1, e1) in zip(bands, bands[1:]):
            assert e0 == b1                      # contiguous, disjoint
        for begin, end in bands[:-1]:
            assert begin % sharding.TILE_ROWS == 0 and end % sharding.TILE_ROWS == 0
    assert sum(sharding.texels_of_rows(geo, plan[r]) for r in range(world)) == geo.total_texels
    if geo.color_mips[0].height >= world * sharding.MIN_ROWS_PER_RANK:
        loads = [sharding.texels_of_rows(geo, plan[r]) for r in range(world)]
        assert max(loads) <= 1.4 * geo.total_texels / world  # the small mips go whole to single ranks


WORKER = r'''
import os, sys
import numpy as np
import torch.distributed as dist
sys.path.insert(0, os.environ["NTCB_ROOT"]); sys.path.insert(0, os.path.join(os.environ["NTCB_ROOT"], "oracle"))
import __graft_entry__ as entry
entry.load_package()
from rtxntc_library_b200 import sharding, synthetic
import oracle_py

dist.init_process_group(backend="gloo")
rank, world = dist.get_rank(), dist.get_world_size()
data = synthetic.make_texture_set(synthetic.TextureSetSpec(96, 160, 4, 0, 2, 8, seed=31, network="unit"))
geo = data.geometry
checker = oracle_py.OracleSet.from_synthetic(data)

# --- tile-row sharding of one set: every rank decodes its bands, rank 0 gathers --------------------
old_min = sharding.MIN_ROWS_PER_RANK
sharding.MIN_ROWS_PER_RANK = 16          # make the small test set worth splitting
plan = sharding.plan_rows(geo, world)
mine = []
for mip, (begin, end) in enumerate(plan[rank]):
    if end > begin:
        mine.append((mip, begin, checker.decode_mip(mip, True, oracle_py.NUMERICS_SPEC, y0=begin, y1=end, threads=1)))
gathered = [None] * world
dist.gather_object(mine, gathered if rank == 0 else None, dst=0)
ok = True
if rank == 0:
    images = [np.zeros((cm.height, cm.width, geo.channels), dtype=np.float16) for cm in geo.color_mips]
    for part in gathered:
        for mip, begin, rows in part:
            images[mip][begin:begin + rows.shape[0]] = rows
    for mip in range(geo.mips):
        whole = checker.decode_mip(mip, True, oracle_py.NUMERICS_SPEC, threads=1)
        ok = ok and np.array_equal(images[mip].view(np.uint16), whole.view(np.uint16))
    ok = ok and any(len(part) > 0 for part in gathered[1:])   # the other rank really had work

# --- batch sharding: the ranks agree on the plan without talking --------------------------------
geometries = [synthetic.TextureSetSpec(64, 64, 4, 0, 2, 8, seed=s).geometry() for s in range(5)]
plans = [None] * world
dist.all_gather_object(plans, [(u.set_index, u.mips) for u in sharding.plan_batch(geometries, world)[rank]])
if rank == 0:
    flat = sorted(x for p in plans for x in p)
    ok = ok and flat == sorted((i, m) for i, g in enumerate(geometries) for m in [(0,), tuple(range(1, g.mips))])
result = [ok]
dist.broadcast_object_list(result, src=0)
dist.destroy_process_group()
sys.exit(0 if result[0] else 1)
'''


def test_two_rank_gloo_decode_and_gather(tmp_path, oracle):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NTCB_ROOT=ROOT, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", "29517", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stdout[-2000:] + result.stderr[-4000:]
