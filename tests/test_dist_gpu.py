"""The multi-GPU partitioner behind the C ABI (ntb200_dist_*).

On one GPU: a one-rank communicator runs the same entry points (gather into a buffer at a column offset, Linear + ReLU
with the pre-activation kept, gather of an existing block), checked against the plain GEMM and the oracle.

On two or more GPUs (skipped otherwise): two processes, one per GPU, exchange their buffer records through gloo and
then use nothing but this library's kernels: the epilogue stores cross NVLink into the peer's buffer, the flag
exchange orders the ranks.  Every rank checks the gathered matrix against the unsharded product, bit for bit, over
many alternating steps; and a barrier whose peer stays away gives up after its limit, reports NTB200_ERR_TIMEOUT,
leaves the context usable and falls back into step once the peer arrives."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT
from gpu_util import dev, host, normal

pytestmark = pytest.mark.gpu


def test_one_rank_communicator(oracle):
    from neurotensor_b200 import _lib, api, partition
    rng = np.random.default_rng(31)
    comm = partition.DistComm()
    assert (comm.rank, comm.world) == (0, 1)
    # small problem: the copy-kernel fallback; large problem (>= 74 tiles of 256 x 256): the TMA-store epilogue
    for m, k, n, width, col0 in ((200, 96, 136, 400, 128), (2304, 128, 2096, 4608, 2048)):
        x, w, b = normal(rng, (m, k), np.float16, 0.5), normal(rng, (k, n), np.float16, 0.5), normal(rng, (n,), np.float16)
        xd, wd, bd = dev(x), dev(w), dev(b)
        buf = comm.buffer(m, width, torch.float16)
        buf.local.fill_(7.0)
        exp = api.linear(xd, wd, bd)
        got = comm.gemm_allgather(xd, wd, buf, col0, bias=bd)
        assert torch.equal(got[:, col0:col0 + n], exp)
        assert bool((got[:, :col0] == 7).all()) and bool((got[:, col0 + n:] == 7).all())
        assert oracle.rel_fro(host(exp[:64]), oracle.linear(x[:64], w, b)) <= 2e-3
        buf.local.fill_(7.0)
        h = comm.gemm_allgather(xd, wd, buf, col0, bias=bd, relu=True)
        assert torch.equal(h, exp)                                            # the owner keeps the pre-activation
        assert torch.equal(buf.local[:, col0:col0 + n], torch.clamp(exp, min=0))
        assert bool((buf.local[:, :col0] == 7).all()) and bool((buf.local[:, col0 + n:] == 7).all())
        buf.local.fill_(7.0)
        comm.allgather_columns(exp, buf, col0)
        assert torch.equal(buf.local[:, col0:col0 + n], exp)
        comm.barrier()                                                        # one rank: nothing to wait for
        buf.close()
    _lib.check(_lib.lib().ntb200_check_device_status(None))
    comm.close()


WORKER = r"""
import ctypes, os, sys, time, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NTB_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", rank=rank, world_size=world)
from neurotensor_b200 import _lib, api, partition
L = _lib.lib()
comm = partition.DistComm()
gen = torch.Generator(device="cuda").manual_seed(5)                  # same seed: replicated operands agree
rn = lambda shape, s=1.0: (torch.randn(shape, generator=gen, device="cuda") * s).bfloat16()
for m, k, n in ((256, 128, 512), (4096, 512, 4096)):               # copy-kernel fallback; TMA-store epilogue
    x, w, b = rn((m, k)), rn((k, n), k ** -0.5), rn((n,), 0.1)
    full = api.linear(x, w, b)
    c0, cn = partition.c_shard(n, world, rank, 8)
    bufs = [comm.buffer(m, n, torch.bfloat16) for _ in range(2)]
    for step in range(20):
        buf = bufs[step & 1]
        got = comm.gemm_allgather(x, w[:, c0:c0 + cn], buf, c0, bias=b[c0:c0 + cn])
        assert torch.equal(got, full), ("gather", m, step)
    for step in range(20):
        buf = bufs[step & 1]
        h = comm.gemm_allgather(x, w[:, c0:c0 + cn], buf, c0, bias=b[c0:c0 + cn], relu=True)
        assert torch.equal(h, full[:, c0:c0 + cn]) and torch.equal(buf.local, torch.clamp(full, min=0)), ("relu", m, step)
    blk = full[:, c0:c0 + cn].contiguous()
    assert torch.equal(comm.allgather_columns(blk, bufs[0], c0), full)
    comm.barrier(); torch.cuda.synchronize()
    for b_ in bufs:
        b_.close()
_lib.check(L.ntb200_check_device_status(None))
# two row blocks of one gathered matrix on two streams, each with its own communicator (its own flags), into a buffer
# that belongs to the first: ntb200_dist_gemm_allgather_at
comm2 = partition.DistComm()
side = torch.cuda.Stream()
m, k, n = 4096, 512, 4096
x, w, b = rn((m, k)), rn((k, n), k ** -0.5), rn((n,), 0.1)
full = api.linear(x, w, b)
c0, cn = partition.c_shard(n, world, rank, 8)
bufs = [comm.buffer(m, n, torch.bfloat16) for _ in range(2)]
for step in range(10):
    buf = bufs[step & 1]
    h = torch.empty((m, cn), dtype=torch.bfloat16, device="cuda")
    main = torch.cuda.current_stream()
    side.wait_stream(main)
    comm.gemm_allgather(x[:1920], w[:, c0:c0 + cn], buf, c0, bias=b[c0:c0 + cn], relu=True, row0=0, h_out=h[:1920])
    with torch.cuda.stream(side):
        comm2.gemm_allgather(x[1920:], w[:, c0:c0 + cn], buf, c0, bias=b[c0:c0 + cn], relu=True, row0=1920, h_out=h[1920:])
    main.wait_stream(side)
    assert torch.equal(h, full[:, c0:c0 + cn]) and torch.equal(buf.local, torch.clamp(full, min=0)), ("row blocks", step)
    # the gather without its closing flag exchange: the own block is there at once (in stream order), everybody's after
    # a barrier of the same communicator
    comm.barrier()          # every rank is through comparing this buffer
    got = comm.gemm_allgather(x, w[:, c0:c0 + cn], buf, c0, bias=b[c0:c0 + cn], barrier=False)
    assert torch.equal(got[:, c0:c0 + cn], full[:, c0:c0 + cn]), ("own block", step)
    comm.barrier()
    assert torch.equal(buf.local, full), ("after the barrier", step)
    comm.barrier()          # nobody overwrites the buffer (next step) while a slower rank still compares it
torch.cuda.synchronize()
for b_ in bufs:
    b_.close()
comm2.close()
_lib.check(L.ntb200_check_device_status(None))
# a barrier whose peer stays away: rank 0 gives up after 100 ms and says so; rank 1 arrives late and completes at
# once against the count rank 0 left behind; afterwards the two are in step again
_lib.check(L.ntb200_dist_set_barrier_limit_ms(comm._h, 100))
dist.barrier()
if rank == 0:
    comm.barrier()
    rc = L.ntb200_check_device_status(None)
    assert rc == _lib.ERR_TIMEOUT, rc
    assert L.ntb200_check_device_status(None) == _lib.OK              # reported once; the context is usable
    dist.barrier()                                                   # now let rank 1 go
else:
    dist.barrier()
    comm.barrier()
    _lib.check(L.ntb200_check_device_status(None))
_lib.check(L.ntb200_dist_set_barrier_limit_ms(comm._h, 2000))
dist.barrier()
comm.barrier()
_lib.check(L.ntb200_check_device_status(None))
comm.close()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_real_peers(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = 29900 + os.getpid() % 90
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NTB_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                      text=True))
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0] + "\n(timed out)")
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o
