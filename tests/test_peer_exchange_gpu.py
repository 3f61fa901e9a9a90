"""The peer-memory all-gather (``ssd_b200_xchg_*``) and the sequence-sharded forward on top of it, on two GPUs of
one node (one process per GPU).  Skipped on a single-GPU box.

NVLS is switched off for the helper collectives and the library's kernel uses plain peer stores; the timeout test
makes its failure on the host (a rank that never calls the exchange), every device wait is bounded."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

needs_two = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                               reason="needs two GPUs")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _init(rank, world, port):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    return dist


def _run(world, target, *args):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            rank, val = q.get(timeout=300)
            out[rank] = val
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return out


def _exchange_worker(rank, world, port, q):
    dist = _init(rank, world, port)
    try:
        from workloadsuite_b200.peer_exchange import PeerExchange
        from workloadsuite_b200 import ssd

        dev = torch.device(f"cuda:{rank}")
        numel = 3 * 1000 + 2                      # not a multiple of 4: the slot is padded
        ex = PeerExchange(numel, device=dev)
        send = torch.zeros(ex.slot, device=dev)
        ok = True
        for step in range(5):                     # eager launches, fresh values each time
            send[:numel] = torch.arange(numel, device=dev) * 0.5 + 1000.0 * rank + step
            recv = ex.all_gather(send, status=ssd._status_word(dev))
            torch.cuda.synchronize()
            for r in range(world):
                want = torch.arange(numel, device=dev) * 0.5 + 1000.0 * r + step
                ok = ok and bool(torch.equal(recv[r, :numel], want))
        # one captured launch, replayed: the exchange counter lives on the device
        g = torch.cuda.CUDAGraph()
        cap = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(cap):
            with torch.cuda.graph(g, stream=cap):
                ex.all_gather(send, status=ssd._status_word(dev))
        for step in range(4):
            send[:numel] = -7.0 * rank - step
            g.replay()
            torch.cuda.synchronize()
            for r in range(world):
                ok = ok and bool((ex.recv[r, :numel] == -7.0 * r - step).all())
        status = ssd.device_status(dev)
        ex.close()
        q.put((rank, (ok, status)))
    finally:
        dist.destroy_process_group()


@needs_two
def test_all_gather_through_peer_memory():
    out = _run(2, _exchange_worker)
    assert out[0] == (True, 0) and out[1] == (True, 0)


def _sharded_worker(rank, world, port, q):
    dist = _init(rank, world, port)
    try:
        from oracle import ssd_oracle as O
        from workloadsuite_b200 import sharded, ssd

        dev = torch.device(f"cuda:{rank}")
        s_loc = 1024
        inp = O.make_inputs(b=1, s=s_loc * world, h=4, p=64, n=128, g=1, dtype=torch.bfloat16, init=True, seed=11,
                            decay_scale=0.02)
        sl = slice(s_loc * rank, s_loc * (rank + 1))
        loc = {k: inp[k][:, sl].contiguous().to(dev) for k in ("X", "A", "B", "C")}
        init = inp["initial_states"].to(dev)
        res = {}
        for mode in ("peer", "collective"):
            eng = sharded.SequenceShardedSSD(exchange=mode, cuda_graphs=(mode == "peer"))
            for _ in range(3):                      # first call eager + capture, then replays
                Y = eng.forward(loc["X"], loc["A"], loc["B"], loc["C"], 256, initial_states=init)
            torch.cuda.synchronize()
            res[mode] = (Y.clone(), eng.exchange_mode())
        Yref = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"])[:, sl]
        err = O.error_metrics(res["peer"][0].cpu(), Yref)[0]
        same = bool(torch.equal(res["peer"][0], res["collective"][0]))
        q.put((rank, (err, same, res["peer"][1], res["collective"][1], ssd.device_status(dev))))
    finally:
        dist.destroy_process_group()


@needs_two
def test_sequence_sharded_forward_over_peer_memory():
    """Same result, bit for bit, as with the collective library's all-gather, and within tolerance of the
    unsharded float64 recurrence (slow decay: the state that crosses the shard boundary matters)."""
    out = _run(2, _sharded_worker)
    for rank in (0, 1):
        err, same, mode_peer, mode_coll, status = out[rank]
        assert err < 2e-2 and same and status == 0
        assert mode_peer.startswith("peer-memory") and mode_coll.startswith("torch.distributed")


def _timeout_worker(rank, world, port, q):
    dist = _init(rank, world, port)
    try:
        from workloadsuite_b200.peer_exchange import PeerExchange
        from workloadsuite_b200 import ssd

        dev = torch.device(f"cuda:{rank}")
        ex = PeerExchange(1024, device=dev, wait_limit_ms=200)
        send = torch.ones(ex.slot, device=dev)
        status = 0
        if rank == 0:                      # rank 1 never enters the exchange
            ex.all_gather(send, status=ssd._status_word(dev))
            status = ssd.device_status(dev)
        usable = float((torch.ones(8, device=dev) * 2).sum().item()) == 16.0      # the context survived
        dist.barrier()
        ex.close()
        q.put((rank, (status, usable)))
    finally:
        dist.destroy_process_group()


@needs_two
def test_exchange_gives_up_when_a_rank_never_arrives():
    out = _run(2, _timeout_worker)
    assert out[0] == (7, True) and out[1] == (0, True)
