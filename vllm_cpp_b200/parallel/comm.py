"""Communicators: the collective surface the models call.

* ``SingleComm``   world size 1, every collective is the identity.
* ``TorchComm``    one process per GPU over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).
                   This is the baseline mode ("GEMM kernel + NCCL call") and the bootstrap for
                   the symmetric-memory fused kernels.
* ``FakeComm``     ranks are threads of one process and collectives are a barrier plus a sum
                   over shared host tensors, so sharding math and the multi-rank engine
                   contract are testable on a CPU-only machine.

The reference has no distributed runtime at all; its design note
(``.agents/specs/tensor-parallelism.md:422-476``) proposes exactly this host-mock
communicator for tests.
"""
from __future__ import annotations

import threading
from typing import Optional

import torch


class SingleComm:
    rank = 0
    world = 1

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def all_gather(self, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
        return t

    def reduce_scatter(self, t: torch.Tensor, dim: int = 0) -> torch.Tensor:
        return t

    def broadcast_object(self, obj, src: int = 0):
        return obj

    def all_gather_object(self, obj) -> list:
        return [obj]

    def exchange(self, sends, recvs) -> None:
        """Point-to-point batch: ``sends`` [(dst rank, tensor)], ``recvs`` [(src rank, buffer)];
        between a pair of ranks tensors arrive in the order they were listed."""
        assert not sends and not recvs

    def barrier(self) -> None:
        pass


class TorchComm:
    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def all_reduce(self, t):
        self.dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t, dim=-1):
        outs = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(outs, t.contiguous(), group=self.group)
        return torch.cat(outs, dim=dim)

    def all_gather_into(self, out, t):
        self.dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def reduce_scatter(self, t, dim=0):
        assert dim == 0
        n = t.shape[0] // self.world
        out = torch.empty((n, *t.shape[1:]), dtype=t.dtype, device=t.device)
        self.dist.reduce_scatter_tensor(out, t.contiguous(), group=self.group)
        return out

    def all_to_all_single(self, out, inp, out_splits=None, in_splits=None):
        self.dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)
        return out

    def exchange(self, sends, recvs) -> None:
        ops = [self.dist.P2POp(self.dist.isend, t, self._global(dst), self.group) for dst, t in sends]
        ops += [self.dist.P2POp(self.dist.irecv, buf, self._global(src), self.group) for src, buf in recvs]
        if ops:
            for w in self.dist.batch_isend_irecv(ops):
                w.wait()

    def _global(self, r: int) -> int:
        return self.dist.get_global_rank(self.group, r) if self.group is not None else r

    def broadcast_object(self, obj, src=0):
        box = [obj]
        self.dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def all_gather_object(self, obj) -> list:
        outs = [None] * self.world
        self.dist.all_gather_object(outs, obj, group=self.group)
        return outs

    def barrier(self):
        self.dist.barrier(group=self.group)


class _FakeWorld:
    def __init__(self, world: int):
        self.world = world
        self.barrier = threading.Barrier(world)
        self.slots: list = [None] * world
        self.lock = threading.Lock()
        self.failed = False


class FakeComm:
    """Thread-rank communicator. Create one world, hand ``FakeComm(world, r)`` to thread r."""

    def __init__(self, world: _FakeWorld, rank: int, timeout: float = 10.0):
        self._w = world
        self.rank = rank
        self.world = world.world
        self.timeout = timeout

    @staticmethod
    def make_world(world: int) -> _FakeWorld:
        return _FakeWorld(world)

    def _sync(self):
        try:
            self._w.barrier.wait(self.timeout)
        except threading.BrokenBarrierError as e:
            self._w.failed = True
            raise RuntimeError("FakeComm: a rank failed to join the collective") from e

    def _exchange(self, t):
        self._w.slots[self.rank] = t
        self._sync()
        vals = list(self._w.slots)
        self._sync()
        return vals

    def all_reduce(self, t):
        vals = self._exchange(t.clone())
        acc = vals[0].float().clone()
        for v in vals[1:]:
            acc += v.float()          # fixed rank order => bit-identical on every rank
        t.copy_(acc.to(t.dtype))
        return t

    def all_gather(self, t, dim=-1):
        vals = self._exchange(t.clone())
        return torch.cat(vals, dim=dim)

    def reduce_scatter(self, t, dim=0):
        vals = self._exchange(t.clone())
        acc = vals[0].float().clone()
        for v in vals[1:]:
            acc += v.float()
        n = t.shape[0] // self.world
        return acc[self.rank * n:(self.rank + 1) * n].to(t.dtype)

    def exchange(self, sends, recvs) -> None:
        vals = self._exchange([(dst, t.clone()) for dst, t in sends])
        pending = {src: [t for dst, t in vals[src] if dst == self.rank] for src in range(self.world)}
        for src, buf in recvs:
            buf.copy_(pending[src].pop(0))
        assert not any(pending.values()), "FakeComm.exchange: sends without a matching receive"

    def broadcast_object(self, obj, src=0):
        vals = self._exchange(obj)
        return vals[src]

    def all_gather_object(self, obj) -> list:
        return self._exchange(obj)

    def barrier(self):
        self._sync()

    def abort(self):
        """A failing rank calls this so its peers' next collective raises instead of waiting."""
        self._w.failed = True
        self._w.barrier.abort()


def make_comm(world: int = 1, group=None):
    if world <= 1:
        return SingleComm()
    return TorchComm(group)
