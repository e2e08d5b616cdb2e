"""GPU (needs two devices): the peer-store all-gather equals NCCL's all-gather bit for bit."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ms_custom_ops_b200 import sharding
        shape = (64, 16, 128)
        pg = sharding.PeerGather(shape, torch.bfloat16, dev)
        ok = True
        for step in range(5):  # both buffers of the double buffer, several rounds
            g = torch.Generator(device=dev)
            g.manual_seed(1000 * step + rank)
            local = torch.randn(shape, generator=g, device=dev).to(torch.bfloat16)
            got = pg.gather(local)
            torch.cuda.synchronize()
            pg.check()
            want = sharding.all_gather_outputs(local)
            torch.cuda.synchronize()
            ok = ok and torch.equal(got.view(torch.int16), want.view(torch.int16))
            full = sharding.assemble_gathered(got)
            ok = ok and full.shape == (64, 16 * world, 128)
        ret[rank] = ok
        dist.barrier()
        pg.release()
    finally:
        dist.destroy_process_group()


def test_peer_store_allgather_matches_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    for p in procs:
        if p.is_alive():
            p.kill()
        assert p.exitcode == 0, "a rank failed or timed out"
    assert dict(ret) == {0: True, 1: True}
