"""The multi-GPU partitioning logic on CPU ranks (gloo, world size 2 and 4).

The CUDA compute callables are replaced by the CPU oracle, so these tests cover
the host side only: slicing, the single all-gather, the fold and the seeding."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ssd_oracle as O
from workloadsuite_b200 import sharded


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_scan(X, A, B, C, chunk, dt=None, initial_states=None, state_only=False):
    Y, H = O.ssd_recurrence(X, A, B, C, dt=dt, initial_states=initial_states, return_final_state=True)
    if state_only:
        return H.float(), O.total_logdecay(A).float()
    return Y.to(X.dtype)


def _oracle_fold(states, lds, rank, initial=None):
    return O.fold_incoming_state(states, lds, rank, initial).float()


def _seq_worker(rank, world, port, with_init, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        inp = O.make_inputs(b=2, s=64 * world, h=4, p=8, n=6, g=2, dtype=torch.float32, init=with_init, seed=7,
                            decay_scale=0.02)
        init = inp.get("initial_states")
        sl = slice(64 * rank, 64 * (rank + 1))
        eng = sharded.SequenceShardedSSD(scan_fn=_oracle_scan, fold_fn=_oracle_fold)
        Y = eng.forward(inp["X"][:, sl], inp["A"][:, sl], inp["B"][:, sl], inp["C"][:, sl], 32, initial_states=init)
        Yfull = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=init)
        err = O.error_metrics(Y, Yfull[:, sl])[0]
        q.put((rank, err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,with_init", [(2, False), (2, True), (4, True)])
def test_sequence_sharded_matches_unsharded(world, with_init):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_seq_worker, args=(r, world, port, with_init, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == list(range(world))
    # fp32 exchange of fp64-computed states: errors at fp32 rounding level
    assert max(e for _, e in res) < 1e-5, res


def _withholding_worker(rank, world, port, q):
    """Rank 1 scans its shard but never joins the exchange (it leaves between steps, nothing of its in flight)."""
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    torch.set_num_threads(1)
    inp = O.make_inputs(b=1, s=64 * world, h=2, p=8, n=6, g=1, dtype=torch.float32, seed=8, decay_scale=0.02)
    sl = slice(64 * rank, 64 * (rank + 1))
    def report(msg):
        q.put((rank, msg))
        q.close()
        q.join_thread()                  # the message is in the pipe before the process ends
        os._exit(0)                      # no destroy_process_group: a peer must find out by itself

    if rank == 1:
        report("left")
    eng = sharded.SequenceShardedSSD(scan_fn=_oracle_scan, fold_fn=_oracle_fold)
    try:
        eng.forward(inp["X"][:, sl], inp["A"][:, sl], inp["B"][:, sl], inp["C"][:, sl], 32)
        msg = "no error"
    except Exception as exc:             # the collective fails: by its timeout, or at once on the closed connection
        msg = "error: " + type(exc).__name__
    report(msg)


def test_a_rank_that_withholds_its_state_ends_the_exchange_with_an_error():
    """Failure detection on the host: the sequence-sharded forward has one collective; when a rank never joins it,
    the others must get an exception from that collective (a short process-group timeout), not a result."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_withholding_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert res[1] == "left"
    assert res[0].startswith("error"), res


def test_head_shard_bounds_cover_all_heads_and_keep_groups_whole():
    for h, g, world in [(80, 1, 8), (80, 1, 4), (48, 8, 8), (48, 8, 2), (128, 8, 4), (24, 1, 2)]:
        seen = []
        for r in range(world):
            h0, h1, g0, g1 = sharded.head_shard_bounds(h, g, r, world)
            seen += list(range(h0, h1))
            hpg = h // g
            assert {j // hpg for j in range(h0, h1)} == set(range(g0, g1))
        assert seen == list(range(h))
    with pytest.raises(ValueError):
        sharded.head_shard_bounds(80, 1, 0, 3)
    with pytest.raises(ValueError):
        sharded.head_shard_bounds(48, 8, 0, 12)  # 4 heads per rank straddle groups of 6


def test_head_sharded_results_concatenate_to_the_full_result():
    inp = O.make_inputs(b=1, s=64, h=8, p=4, n=4, g=4, dtype=torch.float64, seed=9, decay_scale=0.1)
    Yfull = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"])
    parts = []
    for r in range(4):
        sh = sharded.shard_heads(inp["X"], inp["A"], inp["B"], inp["C"], r, 4)
        parts.append(O.ssd_recurrence(sh["X"], sh["A"], sh["B"], sh["C"]))
    assert torch.equal(torch.cat(parts, dim=2), Yfull)
