"""Multi-GPU partitioning of the SSD forward: one process per GPU.

Two partitionings, neither present in the single-device reference:

* **heads** -- every (batch, head) pair is an independent scan, so heads are split
  across ranks with no data-path collective; B/C of a group travel with its heads.
* **sequence** -- the recurrence is linear in the state, so each rank scans its
  token shard from a zero state, the ranks exchange only that final state and the
  shard's summed log-decay (one NCCL all-gather over NVLink; 1 MiB per rank at
  h=32, n=128, p=64), and each rank re-scans its shard seeded with the folded
  state of its predecessors.

The compute callables are injectable so that the exchange algebra runs on CPU
``gloo`` ranks in the tests; the defaults are the CUDA kernels and never fall back.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def head_shard_bounds(n_heads: int, n_groups: int, rank: int, world: int) -> Tuple[int, int, int, int]:
    """(h0, h1, g0, g1): heads [h0,h1) and B/C groups [g0,g1) owned by ``rank``.

    Heads are split evenly; a rank's heads are whole groups, or lie inside one group.
    """
    if n_heads % n_groups != 0:
        raise ValueError("n_heads must be divisible by n_groups")
    if n_heads % world != 0:
        raise ValueError(f"n_heads={n_heads} is not divisible by world size {world}")
    hl = n_heads // world
    hpg = n_heads // n_groups
    if not (hl % hpg == 0 or hpg % hl == 0):
        raise ValueError(f"{hl} heads per rank do not align with groups of {hpg} heads")
    h0, h1 = rank * hl, (rank + 1) * hl
    g0 = h0 // hpg
    g1 = max(g0 + 1, h1 // hpg)
    return h0, h1, g0, g1


def shard_heads(X, A, B, C, rank: int, world: int, dt=None, initial_states=None):
    """Slice full tensors to the head shard of ``rank`` (views, no copies)."""
    h, g = X.shape[2], B.shape[2]
    h0, h1, g0, g1 = head_shard_bounds(h, g, rank, world)
    out = dict(X=X[:, :, h0:h1], A=A[:, :, h0:h1], B=B[:, :, g0:g1], C=C[:, :, g0:g1])
    if dt is not None:
        out["dt"] = dt[:, :, h0:h1]
    if initial_states is not None:
        out["initial_states"] = initial_states[:, h0:h1]
    return out


def _cuda_scan(X, A, B, C, chunk, dt=None, initial_states=None, state_only=False, **kw):
    from .ssd import ssd_forward

    if state_only:
        kw = {k: v for k, v in kw.items() if k != "out"}      # (the state-only phase writes no Y)
        return ssd_forward(X, A, B, C, chunk, dt=dt, initial_states=initial_states, state_only=True,
                           return_logdecay=True, **kw)       # (kw may carry out_final_state / out_logdecay)
    # the state-only call that precedes this one left its per-segment states in the workspace
    return ssd_forward(X, A, B, C, chunk, dt=dt, initial_states=initial_states, reuse_segments=True, **kw)


def _cuda_fold(states, logdecays, rank, initial=None):
    from .ssd import fold_states

    return fold_states(states, logdecays, rank, initial)


class SequenceShardedSSD:
    """SSD forward over a sequence split evenly across the ranks of ``group``.

    Rank r holds tokens ``[r*s/R, (r+1)*s/R)`` of every tensor.  ``forward`` returns
    the local Y shard.  Buffers for the exchange are allocated once per shape.

    With ``cuda_graphs=True`` the whole step (local scan, all-gather, fold, seeded scan) is
    captured into one CUDA graph the first time a given set of tensors is seen and replayed
    afterwards; if the collective cannot be captured, the two local phases are captured and the
    collective is launched normally between them.  The returned Y is then the same tensor on
    every call with those inputs.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, scan_fn: Callable = _cuda_scan,
                 fold_fn: Callable = _cuda_fold, cuda_graphs: bool = False, exchange: str = "auto"):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.scan_fn = scan_fn
        self.fold_fn = fold_fn
        self.cuda_graphs = cuda_graphs
        # "peer": this library's all-gather kernel over NVLink peer memory (CUDA tensors, one process per GPU of one
        # node); "collective": torch.distributed's all_gather_into_tensor (NCCL, or gloo for the CPU tests);
        # "auto": peer when the tensors are on CUDA devices and the ranks can map each other's buffers
        if exchange not in ("auto", "peer", "collective"):
            raise ValueError("exchange must be 'auto', 'peer' or 'collective'")
        self.exchange = exchange
        self._peer = None
        self._send = None
        self._recv = None
        self._graphs = {}
        self._one_graph = None      # None: not tried yet; True/False: the collective is / is not inside the graph
        self._last = None

    def _buffers(self, numel: int, device):
        slot = (numel + 3) // 4 * 4          # (the peer kernel moves 16-byte pieces)
        if self._send is None or self._send.numel() != slot or self._send.device != device:
            self._graphs.clear()
            if self._peer is not None:
                self._peer.close()
                self._peer = None
            self._send = torch.zeros(slot, dtype=torch.float32, device=device)
            self._recv = None
            if self.exchange != "collective" and device.type == "cuda" and self.world > 1:
                from .peer_exchange import PeerExchange
                try:
                    self._peer = PeerExchange(numel, group=self.group, device=device)
                    self._recv = self._peer.recv
                except RuntimeError:
                    if self.exchange == "peer":
                        raise
            if self._recv is None:
                self._recv = torch.empty((self.world, slot), dtype=torch.float32, device=device)
        return self._send, self._recv

    # phase 1: local scan from zero, final state and summed log-decay only, packed for the exchange
    def _phase_local(self, X, A, B, C, chunk, dt, kw):
        b, s_loc, h, p = X.shape
        n = B.shape[3]
        ns, nd = b * h * n * p, b * h
        send, recv = self._buffers(ns + nd, X.device)
        if self.scan_fn is _cuda_scan:
            # the kernels write the shard's final state and log-decay sum straight into the send buffer
            self.scan_fn(X, A, B, C, chunk, dt=dt, initial_states=None, state_only=True,
                         out_final_state=send[:ns].view(b, h, n, p), out_logdecay=send[ns:ns + nd].view(b, h), **kw)
        else:
            F, D = self.scan_fn(X, A, B, C, chunk, dt=dt, initial_states=None, state_only=True, **kw)
            send[:ns].copy_(F.reshape(-1))
            send[ns:ns + nd].copy_(D.reshape(-1))
        return (b, h, n, p, ns, nd)

    # phase 3: fold the predecessors, then the real scan seeded with the result
    def _phase_seeded(self, X, A, B, C, chunk, dt, initial_states, dims, kw):
        b, h, n, p, ns, nd = dims
        recv = self._recv
        states = recv[:, :ns].unflatten(1, (b, h, n, p))
        lds = recv[:, ns:ns + nd].unflatten(1, (b, h))
        # (initial_states, the state before token 0 of the whole sequence, is replicated on all ranks)
        h_in = initial_states if self.rank == 0 else self.fold_fn(states, lds, self.rank, initial_states)
        return self.scan_fn(X, A, B, C, chunk, dt=dt, initial_states=h_in, state_only=False, **kw)

    def _exchange(self):
        # phase 2: the only exchange -- every rank's (state, log-decay) lands in every rank's own memory
        if self._peer is not None:
            from .ssd import _status_word
            self._peer.all_gather(self._send, status=_status_word(self._send.device))
        else:
            dist.all_gather_into_tensor(self._recv.view(-1), self._send, group=self.group)

    def close(self):
        """Releases the peer-memory exchange buffers (collective: every rank calls it).  Optional: a process that
        exits leaves the clean-up to the driver."""
        self._graphs.clear()
        if self._peer is not None:
            self._peer.close()
            self._peer = None
            self._send = self._recv = None

    def exchange_mode(self) -> str:
        if self._send is None:
            return "not run yet"
        return "peer-memory kernel (NVLink stores + flags)" if self._peer is not None else "torch.distributed all-gather"

    def forward(self, X, A, B, C, chunk, dt=None, initial_states=None, **kw):
        self._last = (X, A, B, C, chunk, dt, initial_states, dict(kw))
        if self.cuda_graphs and X.is_cuda:
            return self._forward_graphed(X, A, B, C, chunk, dt, initial_states, kw)
        dims = self._phase_local(X, A, B, C, chunk, dt, kw)
        self._exchange()
        return self._phase_seeded(X, A, B, C, chunk, dt, initial_states, dims, kw)

    def _forward_graphed(self, X, A, B, C, chunk, dt, initial_states, kw):
        out = kw.get("out")
        key = (X.data_ptr(), A.data_ptr(), B.data_ptr(), C.data_ptr(), chunk,
               None if dt is None else dt.data_ptr(), None if initial_states is None else initial_states.data_ptr(),
               None if out is None else out.data_ptr(), tuple(sorted((k, str(v)) for k, v in kw.items() if k != "out")))
        entry = self._graphs.get(key)
        if entry is None:
            # one ordinary run first: allocates workspaces and exchange buffers and warms the communicator
            # outside any capture
            dims = self._phase_local(X, A, B, C, chunk, dt, kw)
            self._exchange()
            self._phase_seeded(X, A, B, C, chunk, dt, initial_states, dims, kw)
            torch.cuda.synchronize(X.device)
            cap = torch.cuda.Stream(device=X.device)
            entry = None
            if self._one_graph is not False:
                # the whole step -- local scan, all-gather, fold, seeded scan -- as ONE graph: a step is one replay
                try:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(cap):
                        with torch.cuda.graph(g, stream=cap):
                            dims = self._phase_local(X, A, B, C, chunk, dt, kw)
                            self._exchange()
                            Y = self._phase_seeded(X, A, B, C, chunk, dt, initial_states, dims, kw)
                    torch.cuda.synchronize(X.device)
                    entry = ((g,), Y)
                    self._one_graph = True
                except Exception:          # the collective could not be captured: keep it outside the graphs
                    self._one_graph = False
                    torch.cuda.synchronize(X.device)
            if entry is None:
                g1, g2 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
                with torch.cuda.stream(cap):
                    with torch.cuda.graph(g1, stream=cap):
                        dims = self._phase_local(X, A, B, C, chunk, dt, kw)
                    with torch.cuda.graph(g2, stream=cap):
                        Y = self._phase_seeded(X, A, B, C, chunk, dt, initial_states, dims, kw)
                torch.cuda.synchronize(X.device)
                entry = ((g1, g2), Y)
            self._graphs[key] = entry
        graphs, Y = entry
        if len(graphs) == 1:
            graphs[0].replay()
        else:
            graphs[0].replay()
            self._exchange()
            graphs[1].replay()
        return Y

    # ---- accounting for the benchmark -------------------------------------------------------------------
    def launch_mode(self) -> str:
        if not self.cuda_graphs:
            return "eager"
        if self._one_graph:
            return "cuda_graph (local scan + all-gather + fold + seeded scan in one graph)"
        if self._one_graph is False:
            return "cuda_graph (local phases) + eager all-gather"
        return "cuda_graph"

    def launches_per_step(self, X, A, B, C, chunk, **kw) -> int:
        """Kernels of this library per step and rank (the collective's own kernel and the two small copies
        into the send buffer are not counted)."""
        from .ssd import plan

        kw = {k: v for k, v in kw.items() if k in ("kernel", "nsegments")}
        p_state = plan(X, A, B, C, chunk, state_only=True, **kw)
        p_seeded = plan(X, A, B, C, chunk, reuse_segments=True, **kw)   # (already net of the reused first pass)
        fold = 1 if self.rank > 0 else 0
        return p_state["launches"] + fold + p_seeded["launches"]

    def phase_times_ms(self, repeats: int = 10):
        """CUDA-event times of the phases of the last ``forward`` (this rank, median over ``repeats``): local
        state-only scan, exchange, fold + seeded scan.  Each phase is captured into a CUDA graph of its own and the
        three are replayed back to back, so the figures hold device time and one graph launch each, not the Python
        launch overhead of the eager path (which is several times the kernels' own time here).  Falls back to eager
        launches when the collective cannot be captured.  Collective on every rank."""
        if getattr(self, "_last", None) is None:
            return None
        X, A, B, C, chunk, dt, initial_states, kw = self._last
        if not X.is_cuda:
            return None
        dims = self._phase_local(X, A, B, C, chunk, dt, kw)
        self._exchange()
        self._phase_seeded(X, A, B, C, chunk, dt, initial_states, dims, kw)
        torch.cuda.synchronize(X.device)
        steps = [lambda: self._phase_local(X, A, B, C, chunk, dt, kw), self._exchange,
                 lambda: self._phase_seeded(X, A, B, C, chunk, dt, initial_states, dims, kw)]
        how = "eager launches with events between the phases"
        if self._one_graph is not False:
            try:
                cap = torch.cuda.Stream(device=X.device)
                graphs = []
                with torch.cuda.stream(cap):
                    for fn in steps:
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, stream=cap):
                            fn()
                        graphs.append(g)
                torch.cuda.synchronize(X.device)
                steps = [g.replay for g in graphs]
                how = "one CUDA graph per phase, replayed back to back with events in between"
            except Exception:
                torch.cuda.synchronize(X.device)
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(repeats)]
        for r in range(repeats):
            dist.barrier(group=self.group)
            ev[r][0].record()
            for k, fn in enumerate(steps):
                fn()
                ev[r][k + 1].record()
        torch.cuda.synchronize(X.device)
        med = lambda i: sorted(e[i].elapsed_time(e[i + 1]) for e in ev)[repeats // 2]
        return {"local_state_scan": med(0), "all_gather": med(1), "fold_and_seeded_scan": med(2), "note": how}


def sequence_sharded_forward(X, A, B, C, chunk, group=None, dt=None, initial_states=None, **kw):
    """Functional form of :class:`SequenceShardedSSD` (allocates its buffers per call).

    ``initial_states`` (the state before token 0 of the whole sequence) must be
    passed identically on every rank, or be None.
    """
    return SequenceShardedSSD(group).forward(X, A, B, C, chunk, dt=dt, initial_states=initial_states, **kw)
