"""The reference's per-slice all-reduce pipeline, replayed with the same NCCL
primitives through ``torch.distributed`` -- a comparison arm for groupings the
reference itself cannot be given on one box (it tells machines apart by boot
id, fairring/machine.cc:25-32, so eight GPUs of one host are always 1 x 8).

Per all-reduce, with the tensor viewed as ``[D][M][X]`` (fairring/device.cc:461-467):

1. reduce-scatter inside the machine, in place            (ncclReduceScatter, :47-54)
2. collect: shard ``[d][m']`` goes to machine ``m'`` on the rail of device ``d``,
   into the neighbour's slot of the tensor as scratch      (grouped ncclSend/ncclRecv, :88-105)
3. add: ``sum`` over the M collected copies                 (at::sum_out, :123-130)
4. diffuse: the reduced shard goes to every rail peer       (grouped ncclSend/ncclRecv, :149-172)
5. all-gather inside the machine, in place                  (ncclAllGather, :188-194)

Each stage has its own stream and its own communicator family (four NCCL
groups here, as in fairring/machine.cc:290-382), chained by events, so stages of
consecutive all-reduces overlap as they do in the reference.  The enqueueing is
Python here and C++ there: for small messages this arm pays more host time than
the reference would; from a few MiB on the GPU time dominates.

This is NOT the reference; the real thing is timed by ``baseline/ref_sweep.py``
(1 x N only).  Results of this arm are labelled ``refseq``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class ReferenceSequence:
    def __init__(self, world: int, rank: int, gpus_per_machine: int, device: torch.device,
                 favorable: bool = False):
        self.W, self.D = world, gpus_per_machine
        assert world % gpus_per_machine == 0
        self.M = world // gpus_per_machine
        self.rank, self.dev = rank, device
        D, M = self.D, self.M
        self.rank_of = (lambda m, d: d * M + m) if favorable else (lambda m, d: m * D + d)
        self.m, self.d = (rank % M, rank // M) if favorable else (rank // D, rank % D)
        # Four communicator families; every rank creates every group, in one order.
        self.rs = self.ag = self.collect = self.diffuse = None
        for mm in range(M):
            ranks = [self.rank_of(mm, dd) for dd in range(D)]
            a, b = dist.new_group(ranks, backend="nccl"), dist.new_group(ranks, backend="nccl")
            if mm == self.m:
                self.rs, self.ag = a, b
        for dd in range(D):
            ranks = [self.rank_of(mm, dd) for mm in range(M)]
            a, b = dist.new_group(ranks, backend="nccl"), dist.new_group(ranks, backend="nccl")
            if dd == self.d:
                self.collect, self.diffuse = a, b
        self.rail = [self.rank_of(mm, self.d) for mm in range(M)]
        lo, hi = torch.cuda.Stream.priority_range()
        self.streams = [torch.cuda.Stream(device=device, priority=hi) for _ in range(5)]
        self.staging = None  # only for D == 1 (no neighbour slot to borrow)

    def _slice(self, t3: torch.Tensor, caller_event: torch.cuda.Event) -> torch.cuda.Event:
        D, M, d, m = self.D, self.M, self.d, self.m
        X = t3.shape[2]
        flat = t3.view(-1)
        s_rs, s_collect, s_add, s_diffuse, s_ag = self.streams
        ev = caller_event
        with torch.cuda.stream(s_rs):
            s_rs.wait_event(ev)
            if D > 1:
                dist.reduce_scatter_tensor(t3[d].view(-1), flat, group=self.rs, async_op=True).wait()
            ev = torch.cuda.Event()
            ev.record(s_rs)
        if M > 1:
            if D > 1:
                staging = t3[(d + 1) % D]
            else:
                if self.staging is None or self.staging.numel() < M * X or self.staging.dtype != t3.dtype:
                    self.staging = torch.empty(M * X, device=self.dev, dtype=t3.dtype)
                staging = self.staging[:M * X].view(M, X)
            with torch.cuda.stream(s_collect):
                s_collect.wait_event(ev)
                ops = []
                for mm in range(M):
                    if mm == m:
                        continue
                    ops.append(dist.P2POp(dist.isend, t3[d][mm], self.rail[mm], group=self.collect))
                    ops.append(dist.P2POp(dist.irecv, staging[mm], self.rail[mm], group=self.collect))
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
                staging[m].copy_(t3[d][m])  # the self send/recv of the reference
                ev = torch.cuda.Event()
                ev.record(s_collect)
            with torch.cuda.stream(s_add):
                s_add.wait_event(ev)
                torch.sum(staging, dim=0, out=t3[d][m])
                ev = torch.cuda.Event()
                ev.record(s_add)
            with torch.cuda.stream(s_diffuse):
                s_diffuse.wait_event(ev)
                ops = []
                for mm in range(M):
                    if mm == m:
                        continue
                    ops.append(dist.P2POp(dist.isend, t3[d][m], self.rail[mm], group=self.diffuse))
                    ops.append(dist.P2POp(dist.irecv, t3[d][mm], self.rail[mm], group=self.diffuse))
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
                ev = torch.cuda.Event()
                ev.record(s_diffuse)
        with torch.cuda.stream(s_ag):
            s_ag.wait_event(ev)
            if D > 1:
                dist.all_gather_into_tensor(flat, t3[d].view(-1), group=self.ag, async_op=True).wait()
            ev = torch.cuda.Event()
            ev.record(s_ag)
        return ev

    def all_reduce(self, t: torch.Tensor) -> None:
        """In-place sum over all ranks; the caller's current stream waits for the result."""
        assert t.is_contiguous() and t.dim() == 1
        DM = self.D * self.M
        n = t.numel() // DM * DM
        cur = torch.cuda.current_stream(self.dev)
        start = torch.cuda.Event()
        start.record(cur)
        done = None
        if n:
            done = self._slice(t[:n].view(self.D, self.M, n // DM), start)
        if n < t.numel():
            # ragged tail through a padding slot, like fairring/device.cc:468-475,511-521
            pad = torch.zeros(DM, device=self.dev, dtype=t.dtype)
            with torch.cuda.stream(self.streams[0]):
                self.streams[0].wait_event(start)
                pad[: t.numel() - n].copy_(t[n:])
                e = torch.cuda.Event()
                e.record(self.streams[0])
            e = self._slice(pad.view(self.D, self.M, 1), e)
            with torch.cuda.stream(self.streams[4]):
                t[n:].copy_(pad[: t.numel() - n])
                done = torch.cuda.Event()
                done.record(self.streams[4])
            pad.record_stream(self.streams[4])
        for s in self.streams:
            t.record_stream(s)
        if done is not None:
            cur.wait_event(done)
