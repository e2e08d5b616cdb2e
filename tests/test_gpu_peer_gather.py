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


def test_bounded_wait_for_a_peer_runs_out_and_reports_timeout():
    """One GPU stands in for rank 0 of a two-rank gather whose second rank never shows up: nobody
    ever writes the second flag word.  The wait is bounded (shortened here through the descriptor),
    so the kernel gives up, leaves MSCO_ERR_TIMEOUT in the status word and returns; the context
    stays usable.  Nothing faults, nothing hangs."""
    import ctypes as C

    from ms_custom_ops_b200 import _abi
    dev = torch.device("cuda", 0)
    slice_bytes = 4096
    gathered = [torch.zeros(2 * slice_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
    words = torch.zeros(2, dtype=torch.int32, device=dev)  # ticket, status
    local = torch.arange(slice_bytes, dtype=torch.int32, device=dev).to(torch.uint8)
    d = _abi.MscoGatherDesc()
    d.world, d.rank, d.slice_bytes = 2, 0, slice_bytes
    d.ticket, d.status = words.data_ptr(), words.data_ptr() + 4
    d.wait_polls = 20000   # a few milliseconds
    for r in range(2):
        d.gathered[r], d.flags[r] = gathered[r].data_ptr(), flags[r].data_ptr()
    _abi.check(_abi.lib().msco_peer_allgather(C.byref(d), C.c_void_p(local.data_ptr()), C.c_uint32(1),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert int(words[1].item()) == _abi.ERR_TIMEOUT
    # the local push happened, the flag of this rank was published to both "ranks"
    assert torch.equal(gathered[0][:slice_bytes], local) and torch.equal(gathered[1][:slice_bytes], local)
    assert int(flags[0][0].item()) == 1 and int(flags[1][0].item()) == 1 and int(flags[0][1].item()) == 0
    # the context is alive: the same launch with the missing flag provided completes cleanly
    words.zero_()
    flags[0][1] = 2
    _abi.check(_abi.lib().msco_peer_allgather(C.byref(d), C.c_void_p(local.data_ptr()), C.c_uint32(2),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert int(words[1].item()) == 0


@pytest.mark.parametrize("lens", [[700, 1500, 33, 0, 5000, 129], [40, 17, 300, 511]])
def test_decode_step_gather_pushes_the_finished_rows(lens):
    """msco_decode_step_gather on one GPU standing in for rank 1 of two: the flag of the absent rank 0 is
    provided by the test, so nothing waits on another launch.  The step's output must equal the plain
    msco_decode_step's bit for bit, and slot 1 of BOTH gathered buffers must hold it -- rows that were
    merged from splits and rows the attention kernel wrote itself alike (the second case has no split
    at all: the finishing kernel runs only for the exchange)."""
    import ctypes as C

    import numpy as np

    from ms_custom_ops_b200 import _abi, kernels, workloads
    dev = torch.device("cuda", 0)
    spec = workloads.DecodeSpec("gather", len(lens), 8, kv_heads=2, seed=5, len_lo=1, len_hi=1)
    rng = np.random.default_rng(3)
    lens_np = np.array(lens, dtype=np.int32)
    nb, tables, slots = workloads.layout(spec, lens_np, rng)
    g = torch.Generator(device=dev)
    g.manual_seed(9)
    kc = torch.randn((nb, 128, 2, 128), generator=g, device=dev).to(torch.bfloat16)
    vc = torch.randn((nb, 128, 2, 128), generator=g, device=dev).to(torch.bfloat16)
    q = torch.randn((len(lens), 8, 128), generator=g, device=dev).to(torch.bfloat16)
    key = torch.randn((len(lens), 256), generator=g, device=dev).to(torch.bfloat16)
    val = torch.randn((len(lens), 256), generator=g, device=dev).to(torch.bfloat16)
    bt = torch.from_numpy(tables).to(dev)
    sl = torch.from_numpy(slots).to(dev)
    desc = kernels.make_pa_desc(q, kc, bt, spec.qk_scale, 0)
    plan = _abi.PaPlan(desc, [int(x) for x in lens])
    ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device=dev)
    want = torch.empty_like(q)
    kernels.decode_step(plan, key, val, kc, vc, sl, q, bt, want, ws)
    torch.cuda.synchronize()

    slice_bytes = q.numel() * 2
    gathered = [torch.zeros(2 * slice_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
    words = torch.zeros(2, dtype=torch.int32, device=dev)
    d = _abi.MscoGatherDesc()
    d.world, d.rank, d.slice_bytes = 2, 1, slice_bytes
    d.ticket, d.status = words.data_ptr(), words.data_ptr() + 4
    d.wait_polls = 20000
    for r in range(2):
        d.gathered[r], d.flags[r] = gathered[r].data_ptr(), flags[r].data_ptr()
    flags[1][0] = 1  # "rank 0 has pushed step 1": written by the test, rank 0 does not exist

    class OneStep:
        def next_step(self):
            return C.byref(d), C.c_uint32(1), None
    got = torch.empty_like(q)
    kernels.decode_step(plan, key, val, kc, vc, sl, q, bt, got, ws, gather=OneStep())
    torch.cuda.synchronize()
    kernels.pa_status(plan, ws)
    assert int(words[1].item()) == 0 and int(words[0].item()) == 0  # no timeout, ticket back at zero
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    mine = got.view(torch.uint8).reshape(-1)
    for r in range(2):
        assert torch.equal(gathered[r][slice_bytes:], mine), f"slot 1 of rank {r}'s buffer"
        assert int(gathered[r][:slice_bytes].max().item()) == 0
        assert int(flags[r][1].item()) == 1
    # a slice of the wrong size is refused before anything is launched
    d.slice_bytes = slice_bytes + 16
    with pytest.raises(_abi.MscoError):
        kernels.decode_step(plan, key, val, kc, vc, sl, q, bt, got, ws, gather=OneStep())
    plan.close()


def _step_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import numpy as np

        from ms_custom_ops_b200 import _abi, kernels, sharding, workloads
        lens = [700, 1500, 33, 5000, 129, 2048]
        hq, hkv = 8, 2                      # per rank
        spec = workloads.DecodeSpec("gather2", len(lens), hq, kv_heads=hkv, seed=5, len_lo=1, len_hi=1)
        rng = np.random.default_rng(3)      # same tables on every rank
        nb, tables, slots = workloads.layout(spec, np.array(lens, dtype=np.int32), rng)
        g = torch.Generator(device=dev)
        g.manual_seed(100 + rank)           # every rank its own heads
        kc = torch.randn((nb, 128, hkv, 128), generator=g, device=dev).to(torch.bfloat16)
        vc = torch.randn((nb, 128, hkv, 128), generator=g, device=dev).to(torch.bfloat16)
        q = torch.randn((len(lens), hq, 128), generator=g, device=dev).to(torch.bfloat16)
        key = torch.randn((len(lens), hkv * 128), generator=g, device=dev).to(torch.bfloat16)
        val = torch.randn((len(lens), hkv * 128), generator=g, device=dev).to(torch.bfloat16)
        bt, sl = torch.from_numpy(tables).to(dev), torch.from_numpy(slots).to(dev)
        desc = kernels.make_pa_desc(q, kc, bt, spec.qk_scale, 0)
        plan = _abi.PaPlan(desc, lens)
        ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device=dev)
        pg = sharding.PeerGather(q.shape, q.dtype, dev)
        out = torch.empty_like(q)
        ok = True
        for step in range(4):  # both gathered buffers, twice
            got = kernels.decode_step(plan, key, val, kc, vc, sl, q, bt, out, ws, gather=pg)
            torch.cuda.synchronize()
            pg.check()
            kernels.pa_status(plan, ws)
            want = sharding.all_gather_outputs(out)
            torch.cuda.synchronize()
            ok = ok and torch.equal(got.view(torch.int16), want.view(torch.int16))
            q = (q.float() * 0.5 + 0.1).to(torch.bfloat16)  # another query next step
        ret[rank] = ok
        dist.barrier()
        plan.close()
        pg.release()
    finally:
        dist.destroy_process_group()


def test_decode_step_gather_on_two_gpus_matches_nccl():
    """The decode step whose finishing kernel pushes the rows to the peer, on two real ranks: the gathered
    buffer of every rank equals NCCL's all-gather of the two local outputs, bit for bit, step after step."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_step_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    for p in procs:
        if p.is_alive():
            p.kill()
        assert p.exitcode == 0, "a rank failed or timed out"
    assert dict(ret) == {0: True, 1: True}


def _packets_of(data_u8, step):
    """Packet image of a byte tensor: every 4 data bytes followed by the step number (uint32)."""
    words = data_u8.view(torch.int32).reshape(-1, 1)
    return torch.cat([words, torch.full_like(words, step)], dim=1).reshape(-1).view(torch.uint8)


@pytest.mark.parametrize("peer_sends", [True, False])
def test_decode_step_gather_packet_form(peer_sends):
    """The packet form of the exchange on one GPU standing in for rank 1 of two.  The absent rank 0's
    packets are written by the test (or not at all: then the bounded wait must run out, the status word
    must read MSCO_ERR_TIMEOUT and the context must stay usable).  What rank 1 sends must be the packet
    image of its output in slot 1 of rank 0's packet buffer; its own gathered buffer must hold rank 0's
    slice in slot 0 and its own output in slot 1."""
    import ctypes as C

    import numpy as np

    from ms_custom_ops_b200 import _abi, kernels, workloads
    dev = torch.device("cuda", 0)
    lens = [700, 1500, 33, 0, 5000, 129]
    spec = workloads.DecodeSpec("packets", len(lens), 8, kv_heads=2, seed=5, len_lo=1, len_hi=1)
    rng = np.random.default_rng(3)
    nb, tables, slots = workloads.layout(spec, np.array(lens, dtype=np.int32), rng)
    g = torch.Generator(device=dev)
    g.manual_seed(9)
    kc = torch.randn((nb, 128, 2, 128), generator=g, device=dev).to(torch.bfloat16)
    vc = torch.randn((nb, 128, 2, 128), generator=g, device=dev).to(torch.bfloat16)
    q = torch.randn((len(lens), 8, 128), generator=g, device=dev).to(torch.bfloat16)
    key = torch.randn((len(lens), 256), generator=g, device=dev).to(torch.bfloat16)
    val = torch.randn((len(lens), 256), generator=g, device=dev).to(torch.bfloat16)
    bt, sl = torch.from_numpy(tables).to(dev), torch.from_numpy(slots).to(dev)
    desc = kernels.make_pa_desc(q, kc, bt, spec.qk_scale, 0)
    plan = _abi.PaPlan(desc, [int(x) for x in lens])
    ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device=dev)
    want = torch.empty_like(q)
    kernels.decode_step(plan, key, val, kc, vc, sl, q, bt, want, ws)
    torch.cuda.synchronize()

    slice_bytes = q.numel() * 2
    gathered = [torch.zeros(2 * slice_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
    packets = [torch.zeros(4 * slice_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    words = torch.zeros(2, dtype=torch.int32, device=dev)
    d = _abi.MscoGatherDesc()
    d.world, d.rank, d.slice_bytes = 2, 1, slice_bytes
    d.ticket, d.status = words.data_ptr(), words.data_ptr() + 4
    d.wait_polls = 2000
    for r in range(2):
        d.gathered[r], d.flags[r], d.packets[r] = gathered[r].data_ptr(), flags[r].data_ptr(), packets[r].data_ptr()
    step = 3
    theirs = torch.randint(0, 256, (slice_bytes,), dtype=torch.uint8, device=dev, generator=g)
    if peer_sends:
        packets[1][:2 * slice_bytes] = _packets_of(theirs, step)   # rank 0's slice, slot 0 of MY packet buffer

    class OneStep:
        def next_step(self):
            return C.byref(d), C.c_uint32(step), None
    got = torch.empty_like(q)
    kernels.decode_step(plan, key, val, kc, vc, sl, q, bt, got, ws, gather=OneStep())
    torch.cuda.synchronize()
    kernels.pa_status(plan, ws)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    mine = got.view(torch.uint8).reshape(-1)
    # what was sent: slot 1 of rank 0's packet buffer is the packet image of my output
    assert torch.equal(packets[0][2 * slice_bytes:], _packets_of(mine, step))
    assert int(packets[0][:2 * slice_bytes].max().item()) == 0
    assert torch.equal(gathered[1][slice_bytes:], mine)          # my own slot, stored directly
    assert int(flags[0].abs().max().item()) == 0 and int(flags[1].abs().max().item()) == 0  # no flags in this form
    if peer_sends:
        assert int(words[1].item()) == 0
        assert torch.equal(gathered[1][:slice_bytes], theirs)
    else:
        assert int(words[1].item()) == _abi.ERR_TIMEOUT          # nobody sent: reported, not hung
        words.zero_()
        packets[1][:2 * slice_bytes] = _packets_of(theirs, step + 1)
        step += 1                                                # the context is alive: the next step completes
        kernels.decode_step(plan, key, val, kc, vc, sl, q, bt, got, ws, gather=OneStep())
        torch.cuda.synchronize()
        assert int(words[1].item()) == 0
        assert torch.equal(gathered[1][:slice_bytes], theirs)
    plan.close()
