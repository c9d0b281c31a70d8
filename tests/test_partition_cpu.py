"""Host-side logic of the multi-GPU partitioner on CPU: shard arithmetic, and the column all-gather run as two gloo
ranks (the collective and the re-tiling; the arithmetic on each shard is the GPU library's and is tested there)."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT


def test_shard_range_covers_every_unit_once():
    from neurotensor_b200.partition import column_shard, shard_range
    for total in (0, 1, 7, 64, 65, 1000):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                s, c = shard_range(total, world, r)
                seen += list(range(s, s + c))
            assert seen == list(range(total))
            counts = [shard_range(total, world, r)[1] for r in range(world)]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)
    # column shards are multiples of 8 columns (16-byte rows for 2-byte dtypes) and tile [0, n)
    for n in (8, 100, 4096, 16384):
        for world in (1, 2, 4, 8):
            edges = [column_shard(n, world, r) for r in range(world)]
            assert edges[0][0] == 0 and sum(c for _, c in edges) == n
            assert all(s % 8 == 0 for s, _ in edges)


def test_c_abi_shard_agrees_with_the_python_mirror():
    """ntb200_dist_shard (what a C++ caller uses) and partition.shard_range / column_shard give the same ranges."""
    import ctypes
    from neurotensor_b200 import _lib
    from neurotensor_b200.partition import c_shard, column_shard, shard_range
    for total in (0, 1, 7, 64, 65, 1000, 16384):
        for world in (1, 2, 3, 8):
            for r in range(world):
                assert c_shard(total, world, r) == shard_range(total, world, r)
                assert c_shard(total, world, r, 8) == column_shard(total, world, r)
    s, c = ctypes.c_int64(), ctypes.c_int64()
    L = _lib.lib()
    assert L.ntb200_dist_shard(10, 2, 2, 1, ctypes.byref(s), ctypes.byref(c)) == _lib.ERR_INVALID_ARG
    assert L.ntb200_dist_shard(10, 0, 0, 1, ctypes.byref(s), ctypes.byref(c)) == _lib.ERR_INVALID_ARG
    assert L.ntb200_dist_shard(10, 2, 0, 0, ctypes.byref(s), ctypes.byref(c)) == _lib.ERR_INVALID_ARG
    assert L.ntb200_dist_shard(10, 2, 0, 1, None, None) == _lib.ERR_INVALID_ARG
    # more ranks than a NVLink domain holds, or no way to exchange buffer records: refused before any device work
    h = ctypes.c_void_p()
    assert L.ntb200_dist_init(ctypes.byref(h), 0, 9, _lib.ALLGATHER_FN(0), None) == _lib.ERR_INVALID_ARG
    assert L.ntb200_dist_init(ctypes.byref(h), 0, 2, _lib.ALLGATHER_FN(0), None) == _lib.ERR_INVALID_ARG
    assert L.ntb200_dist_barrier(None, None) == _lib.ERR_INVALID_ARG


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NTB_ROOT"])
from neurotensor_b200 import partition
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, world = dist.get_rank(), dist.get_world_size()
m, n = 6, 16
full = torch.arange(m * n, dtype=torch.float32).reshape(m, n)
c0, cn = partition.column_shard(n, world, rank)
assert (c0, cn) == partition.c_shard(n, world, rank, 8)          # the C ABI's arithmetic, in every rank
out = partition.all_gather_columns(full[:, c0:c0 + cn].contiguous())
assert torch.equal(out, full), (rank, out)
# batch sharding: every rank multiplies only its own items; gathering along the batch restores the whole
start, count = partition.shard_range(6, world, rank)
a = torch.arange(6 * 3 * 4, dtype=torch.float32).reshape(6, 3, 4)
b = torch.ones(6, 4, 2)
mine = torch.matmul(a[start:start + count], b[start:start + count])   # stand-in arithmetic: the collective is the subject
sizes = [partition.shard_range(6, world, r)[1] for r in range(world)]
bufs = [torch.empty((s, 3, 2)) for s in sizes]
dist.all_gather(bufs, mine)
assert torch.equal(torch.cat(bufs), torch.matmul(a, b))
# conv2d shards its images the same way (weights replicated, no exchange for the forward pass): every image has
# exactly one owner and gathering the owners' outputs along the batch restores the whole
imgs = torch.arange(5 * 2 * 4 * 4, dtype=torch.float32).reshape(5, 2, 4, 4)
w = torch.ones(3, 2, 3, 3)
s0, sc = partition.conv2d_image_shard(imgs.shape[0], world, rank)
mine = torch.nn.functional.conv2d(imgs[s0:s0 + sc], w, padding=1)   # stand-in arithmetic again
parts = [None] * world                                   # 5 images on 2 ranks: ragged shares (3 + 2)
dist.all_gather_object(parts, mine)
assert [p.shape[0] for p in parts] == [partition.conv2d_image_shard(5, world, r)[1] for r in range(world)]
assert torch.equal(torch.cat(parts), torch.nn.functional.conv2d(imgs, w, padding=1))
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_column_all_gather_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = 29400 + os.getpid() % 500
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NTB_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                      text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o
