"""KV offloading: eviction policies, host and disk tiers, tiering (promotion, cascade
demotion, identity checks) and the connector end to end through the engine on CPU."""
import os

import torch

from vllm_cpp_b200 import _engine as E


def k(i):
    return bytes([i % 256, i // 256]) + b"\0" * 30


def test_lru_and_arc_policies():
    p = E.CachePolicy.make("lru", 4)
    for i in range(4):
        p.insert(k(i))
    p.touch(k(0))
    assert p.victim() == k(1)                    # 0 was refreshed
    a = E.CachePolicy.make("arc", 4)
    for i in range(4):
        a.insert(k(i))
    a.touch(k(0)); a.touch(k(1))                 # 0, 1 move to the frequency list
    v1 = a.victim(); v2 = a.victim()
    assert {v1, v2} == {k(2), k(3)}              # recency list is drained first: scan resistant
    a.insert(k(2))                               # ghost hit: comes back as a frequent key
    assert len(a) == 3 and a.victim() in (k(0), k(1), k(2))
    try:
        E.CachePolicy.make("nope", 1)
        assert False
    except ValueError:
        pass


def test_tiering_promotion_demotion_and_identity(tmp_path):
    bb = 4096
    host = torch.zeros(2, bb, dtype=torch.uint8)
    ident = E.CacheIdentity("m", 16, bb, "bf16")
    t = E.TieringManager(2, "lru", host.data_ptr(), bb, str(tmp_path), ident, 0)
    assert t.lookup(k(1)) == E.OffloadLookup.MISS
    s1 = t.reserve_for_store(k(1)); host[s1] = 11
    s2 = t.reserve_for_store(k(2)); host[s2] = 22
    assert t.lookup(k(1)) == E.OffloadLookup.HIT and t.fs_blocks == 0
    s3 = t.reserve_for_store(k(3))               # evicts the LRU block (2) -> demoted to disk
    assert s3 == s2 and t.fs_blocks == 1 and os.path.exists(t.fs_path(k(2)))
    host[s3] = 33
    assert t.lookup(k(2)) == E.OffloadLookup.RETRY        # promoted back (evicting 1 to disk)
    assert t.lookup(k(2)) == E.OffloadLookup.HIT
    assert int(host[t.cpu_slot(k(2))][0]) == 22 and t.fs_blocks == 2
    # a cache directory written for another layout is never served
    other = E.TieringManager(2, "lru", host.data_ptr(), bb, str(tmp_path), E.CacheIdentity("m", 32, bb, "bf16"), 0)
    assert other.fs_blocks == 2 and other.lookup(k(1)) == E.OffloadLookup.MISS and other.fs_blocks == 1
    # corrupt file: rejected and removed
    with open(t.fs_path(k(2)), "r+b") as f:
        f.seek(200); f.write(b"\xff\xff\xff")
    t2 = E.TieringManager(2, "lru", host.data_ptr(), bb, str(tmp_path), ident, 0)
    n = t2.fs_blocks
    assert n >= 1 and t2.lookup(k(2)) == E.OffloadLookup.MISS and t2.fs_blocks == n - 1
    # size budget
    small = E.TieringManager(1, "lru", host.data_ptr(), bb, str(tmp_path / "b"), ident, 3 * (bb + 88))
    for i in range(10, 20):
        small.reserve_for_store(k(i))
    assert small.fs_blocks <= 3 and small.fs_stats.evictions >= 5


def test_engine_reuses_offloaded_prefix():
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    cfg = synthetic_config("tiny-dense")
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, cfg.vocab_size, (96,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)

    def make(offload):
        return LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=12, max_model_len=256,
                              max_num_seqs=2, max_num_batched_tokens=128, enable_prefix_caching=True,
                              kv_transfer_config={"cpu_blocks": 64} if offload else None))

    base = make(False)
    want = base.generate([shared + [1, 2, 3]], sp)[0].outputs[0].token_ids
    llm = make(True)
    first = llm.generate([shared + [1, 2, 3]], sp)[0]
    assert first.outputs[0].token_ids == want
    # push the shared prefix out of the small GPU cache with unrelated prompts
    for s in range(3):
        other = torch.randint(0, cfg.vocab_size, (150,), generator=g).tolist()
        llm.generate([other], sp)
    assert llm.offload.stored_blocks > 0
    again = llm.generate([shared + [1, 2, 3]], sp)[0]
    assert again.outputs[0].token_ids == want           # same answer from reloaded blocks
    assert llm.offload.loaded_blocks > 0                # and they really came from the host tier
