"""Expert-parallel load balancing (EPLB).

Expert parallelism gives every rank whole experts. With a fixed contiguous split the rank that
happens to hold the popular experts bounds the step. EPLB keeps a window of per-layer expert loads
(token counts taken from the router's top-k ids), and every ``interval`` steps computes a new
placement of ``num_experts + num_redundant`` physical slots on the ranks: hot experts get replicas,
slots are packed so that ranks carry equal load (policy in ``csrc/engine/parallel/eplb.cpp``), and
the expert weight tensors are rearranged between the ranks to match. Between rebalances the only
cost on the step path is a table lookup that turns the router's logical expert ids into physical
slot ids (a replica is picked by token position, so replicas share an expert's tokens evenly) and
one scatter-add into the load window.

Slots ``[r * S, (r + 1) * S)`` belong to rank ``r``; the grouped-GEMM path is unchanged because it
already selects the (token, expert) pairs whose id falls in its rank's range.

The reference project is single-GPU and has no expert parallelism (its ``.agents/engine-matrix.md``
lists EP and EPLB as not implemented); this component follows the serving-stack design its
tensor-parallel specification points to.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class EplbConfig:
    num_redundant_experts: int = 0     # physical slots beyond one per expert (total must divide over the ranks)
    interval: int = 3000               # steps between rebalances
    window: int = 1000                 # steps of load history a rebalance looks at
    num_groups: int = 1                # expert groups of group-limited routing (kept on one node)
    num_nodes: int = 1


def rebalance(loads, num_physical: int, num_groups: int = 1, num_nodes: int = 1, num_ranks: int = 1) -> dict:
    """{phy2log [L, P], phy_rank [L, P], log2phy [L, E, R], logcnt [L, E]} as int32 numpy arrays."""
    from .. import _engine as E
    arr = np.ascontiguousarray(np.asarray(loads, dtype=np.float64))
    if arr.ndim == 1:
        arr = arr[None]
    return E.eplb_rebalance(arr, num_physical, num_groups, num_nodes, num_ranks)


def contiguous_placement(num_layers: int, num_experts: int) -> np.ndarray:
    """The placement expert parallelism starts from: slot i holds expert i."""
    return np.tile(np.arange(num_experts, dtype=np.int32), (num_layers, 1))


def rank_loads(phy2log: np.ndarray, logcnt: np.ndarray, loads: np.ndarray, num_ranks: int) -> np.ndarray:
    """Load per rank [L, ranks] under a placement (an expert's load splits evenly over its replicas)."""
    L, P = phy2log.shape
    per_slot = np.take_along_axis(loads / np.maximum(logcnt, 1), phy2log.astype(np.int64), axis=1)
    return per_slot.reshape(L, num_ranks, P // num_ranks).sum(-1)


class ExpertLoadWindow:
    """Token counts per (layer, expert) over the last ``window`` steps, on the model's device. The
    counters are updated by device ops only (no host sync), so recording is safe inside a captured
    graph."""

    def __init__(self, num_layers: int, num_experts: int, window: int, device):
        self.window = max(1, window)
        self.hist = torch.zeros((self.window, num_layers, num_experts), dtype=torch.float32, device=device)
        self.cur = torch.zeros((num_layers, num_experts), dtype=torch.float32, device=device)
        self.pos = 0
        self._ones: dict[int, torch.Tensor] = {}

    def record(self, layer: int, ids: torch.Tensor) -> None:
        flat = ids.reshape(-1).long()
        ones = self._ones.get(flat.numel())
        if ones is None:
            ones = self._ones[flat.numel()] = torch.ones(flat.numel(), dtype=torch.float32, device=flat.device)
        self.cur[layer].scatter_add_(0, flat, ones)

    def end_step(self) -> None:
        self.hist[self.pos % self.window].copy_(self.cur)
        self.cur.zero_()
        self.pos += 1

    def loads(self) -> np.ndarray:
        return self.hist.sum(0).cpu().numpy().astype(np.float64)


def plan_moves(old_p2l: np.ndarray, new_p2l: np.ndarray, num_ranks: int):
    """For one layer: where each new slot's weights come from. Returns a list of
    (dst_slot, src_slot) over all new slots; the source is a slot on the destination's own rank when
    one holds the expert already, else the lowest-numbered old slot that does. Every rank computes
    the same plan from the same tables."""
    S_old, S_new = len(old_p2l) // num_ranks, len(new_p2l) // num_ranks
    holders: dict[int, list[int]] = {}
    for s, e in enumerate(old_p2l.tolist()):
        holders.setdefault(e, []).append(s)
    moves = []
    for d, e in enumerate(new_p2l.tolist()):
        src = holders.get(e)
        if not src:
            raise ValueError(f"expert {e} is held by no slot of the old placement")
        r = d // S_new
        local = [s for s in src if s // S_old == r]
        moves.append((d, local[0] if local else src[0]))
    return moves


def rearrange_layer(comm, old_p2l: np.ndarray, new_p2l: np.ndarray, tensors: list[torch.Tensor]) -> list[torch.Tensor]:
    """Moves one layer's expert tensors (each ``[S_old, ...]`` on every rank) to the new placement;
    returns ``[S_new, ...]`` tensors. Local copies where the rank already holds the expert,
    point-to-point transfers otherwise."""
    world, rank = comm.world, comm.rank
    S_old, S_new = len(old_p2l) // world, len(new_p2l) // world
    moves = plan_moves(old_p2l, new_p2l, world)
    outs = [torch.empty((S_new, *t.shape[1:]), dtype=t.dtype, device=t.device) for t in tensors]
    sends, recvs = [], []
    for d, s in moves:
        dr, sr = d // S_new, s // S_old
        if dr == rank and sr == rank:
            for o, t in zip(outs, tensors):
                o[d - rank * S_new].copy_(t[s - rank * S_old])
        elif sr == rank:
            for t in tensors:
                sends.append((dr, t[s - rank * S_old].contiguous()))
        elif dr == rank:
            for o in outs:
                recvs.append((sr, o[d - rank * S_new]))
    comm.exchange(sends, recvs)
    return outs


class EplbState:
    """Placement tables of a model's MoE layers plus the load window and the rebalance schedule."""

    def __init__(self, cfg: EplbConfig, comm, num_layers: int, num_experts: int, device):
        self.cfg, self.comm = cfg, comm
        self.L, self.E = num_layers, num_experts
        self.world = comm.world
        self.P = num_experts + cfg.num_redundant_experts
        if self.P % self.world:
            raise ValueError(f"{self.P} physical expert slots do not divide over {self.world} ranks")
        self.S = self.P // self.world
        self.device = device
        self.window = ExpertLoadWindow(num_layers, num_experts, cfg.window, device)
        self.steps = 0
        self.rebalances = 0
        self.phy2log = None
        self.log2phy = None       # device int64 [L, E, R]
        self.logcnt = None        # device int64 [L, E]

    # ---- placement
    def _install(self, plc: dict) -> None:
        self.phy2log = plc["phy2log"].copy()
        l2p = torch.from_numpy(plc["log2phy"].astype(np.int64))
        cnt = torch.from_numpy(plc["logcnt"].astype(np.int64))
        if self.log2phy is not None and self.log2phy.shape == l2p.shape:
            self.log2phy.copy_(l2p)           # in place: a captured graph keeps reading these
            self.logcnt.copy_(cnt)
        else:
            self.log2phy, self.logcnt = l2p.to(self.device), cnt.to(self.device)

    def _compute(self, loads: np.ndarray) -> dict:
        plc = rebalance(loads, self.P, self.cfg.num_groups, self.cfg.num_nodes, self.world)
        # a fixed table width, so that the device tables never change shape after the first install
        R = self.P - self.E + 1
        l2p = np.full((self.L, self.E, R), -1, dtype=np.int32)
        l2p[:, :, : plc["log2phy"].shape[2]] = plc["log2phy"]
        plc["log2phy"] = l2p
        return plc

    def initial(self, layers_tensors: list[list[torch.Tensor]]) -> list[list[torch.Tensor]]:
        """From the contiguous split the weights were loaded with to a first placement (uniform
        loads: replicas spread evenly). Returns the rearranged per-layer tensors."""
        plc = self._compute(np.ones((self.L, self.E)))
        old = contiguous_placement(self.L, self.E)
        out = [rearrange_layer(self.comm, old[l], plc["phy2log"][l], layers_tensors[l]) for l in range(self.L)]
        self._install(plc)
        return out

    # ---- step path
    def remap(self, layer: int, ids: torch.Tensor) -> torch.Tensor:
        """Logical expert ids [T, k] -> physical slot ids; replica = (token + choice) mod replicas."""
        self.window.record(layer, ids)
        T, k = ids.shape
        idl = ids.long()
        cnt = self.logcnt[layer][idl]
        pos = torch.arange(T, device=ids.device).unsqueeze(1) + torch.arange(k, device=ids.device).unsqueeze(0)
        rep = pos % cnt
        return self.log2phy[layer][idl, rep].to(ids.dtype)

    def end_step(self) -> bool:
        """Closes the step's load counters; True when a rebalance is due."""
        self.window.end_step()
        self.steps += 1
        return self.cfg.interval > 0 and self.steps % self.cfg.interval == 0

    def rebalance_now(self, layers_tensors: list[list[torch.Tensor]]) -> list[list[torch.Tensor]]:
        """New placement from the load window, weights moved to match. Collective: every rank calls
        it at the same step (they all saw the same router outputs, so they compute the same plan;
        the loads are summed over ranks anyway for engines whose ranks see different tokens)."""
        loads = torch.from_numpy(self.window.loads()).to(self.device, torch.float32)
        self.comm.all_reduce(loads)
        plc = self._compute(loads.cpu().numpy().astype(np.float64))
        old = self.phy2log
        out = [rearrange_layer(self.comm, old[l], plc["phy2log"][l], layers_tensors[l]) for l in range(self.L)]
        self._install(plc)
        self.rebalances += 1
        return out

    def imbalance(self, loads: np.ndarray | None = None) -> float:
        """max over layers of (heaviest rank / mean rank) under the current placement."""
        loads = self.window.loads() if loads is None else loads
        cnt = self.logcnt.cpu().numpy()
        rl = rank_loads(self.phy2log, cnt, loads, self.world)
        mean = np.maximum(rl.mean(1), 1e-9)
        return float((rl.max(1) / mean).max())
