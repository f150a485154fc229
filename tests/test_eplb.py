"""Expert-parallel load balancing: the placement policy (native), weight rearrangement between
ranks (thread ranks), and a MoE engine whose tokens do not change when its experts move."""
import threading

import numpy as np
import pytest
import torch

from vllm_cpp_b200.parallel import eplb as EP
from vllm_cpp_b200.parallel.comm import FakeComm


def _check_placement(plc, loads, P, ranks):
    L, E = loads.shape
    p2l, cnt, l2p = plc["phy2log"], plc["logcnt"], plc["log2phy"]
    assert p2l.shape == (L, P) and cnt.shape == (L, E)
    for l in range(L):
        assert sorted(set(p2l[l].tolist())) == list(range(E))                 # every expert is held somewhere
        assert np.bincount(p2l[l], minlength=E).tolist() == cnt[l].tolist()
        for e in range(E):
            slots = [s for s in l2p[l, e].tolist() if s >= 0]
            assert len(slots) == cnt[l, e] and all(p2l[l, s] == e for s in slots)
            assert sorted(plc["phy_rank"][l, slots].tolist()) == list(range(cnt[l, e]))


def test_published_example():
    """The two-layer, twelve-expert example of the EPLB write-up (16 slots, 4 groups, 2 nodes, 8 GPUs)."""
    w = np.array([[90, 132, 40, 61, 104, 165, 39, 4, 73, 56, 183, 86],
                  [20, 107, 104, 64, 19, 197, 187, 157, 172, 86, 16, 27]], dtype=float)
    plc = EP.rebalance(w, 16, num_groups=4, num_nodes=2, num_ranks=8)
    assert plc["phy2log"].tolist() == [[5, 6, 5, 7, 8, 4, 3, 4, 10, 9, 10, 2, 0, 1, 11, 1],
                                       [7, 10, 6, 8, 6, 11, 8, 9, 2, 4, 5, 1, 5, 0, 3, 1]]
    _check_placement(plc, w, 16, 8)
    # groups stay on their node: slots 0..7 (node 0) hold experts of two groups only
    for l in range(2):
        assert len({e // 3 for e in plc["phy2log"][l, :8].tolist()}) == 2


@pytest.mark.parametrize("E,P,ranks,groups,nodes", [(64, 64, 8, 1, 1), (64, 72, 8, 8, 1), (128, 160, 8, 8, 2),
                                                    (60, 64, 4, 1, 1), (8, 8, 2, 1, 1)])
def test_balance_beats_the_contiguous_split(E, P, ranks, groups, nodes):
    rng = np.random.default_rng(E + P)
    loads = rng.zipf(1.4, size=(3, E)).astype(float).clip(max=5000)            # a few hot experts
    plc = EP.rebalance(loads, P, groups, nodes, ranks)
    _check_placement(plc, loads, P, ranks)
    rl = EP.rank_loads(plc["phy2log"], plc["logcnt"], loads, ranks)
    new = (rl.max(1) / rl.mean(1)).max()
    base = loads.reshape(3, ranks, E // ranks).sum(-1)
    old = (base.max(1) / base.mean(1)).max()
    assert new <= old + 1e-9
    if P > E:
        # with spare slots the heaviest rank is within the heaviest slot of the mean
        per_slot = np.take_along_axis(loads / plc["logcnt"], plc["phy2log"].astype(np.int64), 1)
        assert (rl.max(1) <= rl.mean(1) + per_slot.max(1) + 1e-9).all()


def test_bad_sizes_are_refused():
    w = np.ones((1, 8))
    with pytest.raises(ValueError):
        EP.rebalance(w, 9, 1, 1, 2)          # slots do not divide over the ranks
    with pytest.raises(ValueError):
        EP.rebalance(w, 4, 1, 1, 2)          # fewer slots than experts
    with pytest.raises(ValueError):
        EP.rebalance(w, 8, 3, 1, 2)          # experts do not divide into groups


def _run_ranks(world, fn):
    w = FakeComm.make_world(world)
    out, err = [None] * world, []

    def body(r):
        try:
            out[r] = fn(FakeComm(w, r), r)
        except Exception as e:                # noqa: BLE001
            err.append(e)
            FakeComm(w, r).abort()

    ts = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    if err:
        raise err[0]
    return out


def test_rearrangement_moves_every_expert_to_its_new_slots():
    world, E, P = 4, 8, 12
    full = [torch.arange(E, dtype=torch.float32).reshape(E, 1, 1).expand(E, 3, 2).contiguous(),
            (torch.arange(E, dtype=torch.float32) * 10).reshape(E, 1).expand(E, 5).contiguous()]
    loads = np.array([[50, 1, 1, 1, 30, 1, 1, 20.0]])
    plc = EP.rebalance(loads, P, 1, 1, world)
    old = EP.contiguous_placement(1, E)[0]

    def rank_fn(comm, r):
        S = E // world
        mine = [t[r * S:(r + 1) * S].clone() for t in full]
        return EP.rearrange_layer(comm, old, plc["phy2log"][0], mine)

    outs = _run_ranks(world, rank_fn)
    S_new = P // world
    for r in range(world):
        for j in range(S_new):
            e = plc["phy2log"][0][r * S_new + j]
            assert outs[r][0][j].eq(float(e)).all() and outs[r][1][j].eq(float(e) * 10).all()
    # and a second move, from that placement to another one
    loads2 = np.array([[1, 1, 40, 1, 1, 60, 1, 1.0]])
    plc2 = EP.rebalance(loads2, P, 1, 1, world)
    outs2 = _run_ranks(world, lambda comm, r: EP.rearrange_layer(comm, plc["phy2log"][0], plc2["phy2log"][0], outs[r]))
    for r in range(world):
        for j in range(S_new):
            assert outs2[r][0][j].eq(float(plc2["phy2log"][0][r * S_new + j])).all()


def test_remap_spreads_an_experts_tokens_over_its_replicas():
    from vllm_cpp_b200.parallel.comm import SingleComm
    st = EP.EplbState(EP.EplbConfig(num_redundant_experts=4, interval=0, window=4), SingleComm(), 1, 4, "cpu")
    w = [[torch.arange(4.0).reshape(4, 1).clone()]]
    new = st.initial(w)
    assert new[0][0].shape == (8, 1) and sorted(new[0][0].flatten().tolist()) == [0, 0, 1, 1, 2, 2, 3, 3]
    ids = torch.zeros((16, 2), dtype=torch.int32)
    ids[:, 1] = 3
    phys = st.remap(0, ids)
    p2l = torch.from_numpy(st.phy2log[0]).long()
    assert torch.equal(p2l[phys.long()], ids.long())                           # every slot holds the asked expert
    assert len(set(phys[:, 0].tolist())) == 2 and len(set(phys[:, 1].tolist())) == 2
    assert not st.end_step()                                                   # interval 0: never due
    assert st.window.loads()[0].tolist() == [16.0, 0.0, 0.0, 16.0]


@pytest.mark.parametrize("shape", ["tiny-moe", "tiny-gdn-moe", "tiny-mla"])
def test_engine_tokens_do_not_change_when_experts_move(shape):
    """Two expert-parallel ranks with redundant slots, rebalancing every third step: the same greedy
    tokens as the engine without EPLB (the experts compute the same thing wherever they live)."""
    from vllm_cpp_b200.config import EngineArgs, ParallelConfig, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    cfg = synthetic_config(shape)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (21, 5, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)

    def engine(par, comm=None):
        return LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                              max_num_seqs=4, max_num_batched_tokens=128, parallel=par), comm=comm)

    want = [o.outputs[0].token_ids for o in engine(ParallelConfig()).generate(prompts, sp)]

    def rank_fn(comm, r):
        par = ParallelConfig(tensor_parallel_size=2, rank=r, enable_expert_parallel=True, enable_eplb=True,
                             eplb_redundant_experts=4, eplb_interval=3, eplb_window=3)
        llm = engine(par, comm)
        toks = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        return toks, llm.model.eplb.rebalances, llm.model.eplb.S

    outs = _run_ranks(2, rank_fn)
    for toks, rebalances, S in outs:
        assert toks == want
        assert rebalances >= 2 and S == (cfg.num_experts + 4) // 2
