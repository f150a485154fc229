"""Block pool, block hashing and KVCacheManager behaviour (host only).

Restates the behaviours pinned by the reference's tests/vllm/v1/test_block_pool.cpp,
test_kv_cache_utils.cpp and test_kv_cache_manager.cpp."""
import hashlib

import pytest

from vllm_cpp_b200 import _engine as E


def _req(rid, toks, **kw):
    sp = E.SamplingParams(max_tokens=kw.pop("max_tokens", 16))
    return E.Request(E.EngineCoreRequest(rid, list(toks), sp, None, 0.0, 0))


def _cfg(num_blocks=11, block_size=4, kind=None, **kw):
    spec = E.KVCacheSpec(kind=kind or E.KVSpecKind.FULL_ATTENTION, block_size=block_size,
                         num_kv_heads=2, head_size=8, dtype_bytes=2, **kw)
    return E.KVCacheConfig(num_blocks, [E.KVCacheGroupSpec(["l0"], spec)])


def test_sha256_matches_hashlib():
    for msg in (b"", b"abc", b"a" * 55, b"a" * 56, b"a" * 64, b"x" * 1000):
        assert E.sha256_hex(msg) == hashlib.sha256(msg).hexdigest()


def test_block_hash_is_sha256_of_canonical_cbor():
    parent = bytes(range(32))
    toks = [1, 23, 24, 255, 256, 65535, 65536, 151935]
    # canonical CBOR of [parent, toks, null]
    def cbor_uint(v, major=0):
        m = major << 5
        if v < 24:
            return bytes([m | v])
        if v < 256:
            return bytes([m | 24, v])
        if v < 65536:
            return bytes([m | 25]) + v.to_bytes(2, "big")
        return bytes([m | 26]) + v.to_bytes(4, "big")
    enc = bytes([0x83]) + cbor_uint(32, 2) + parent + cbor_uint(len(toks), 4)
    enc += b"".join(cbor_uint(t) for t in toks) + bytes([0xF6])
    assert E.hash_block_tokens(parent, toks) == hashlib.sha256(enc).digest()
    # extra keys change the hash; chaining changes the hash
    assert E.hash_block_tokens(parent, toks, ["salt"]) != E.hash_block_tokens(parent, toks)
    assert E.hash_block_tokens(E.none_hash(), toks) != E.hash_block_tokens(parent, toks)


def test_none_hash_deterministic_by_seed():
    E.reset_none_hash_for_test("7")
    a = E.none_hash()
    E.reset_none_hash_for_test("8")
    b = E.none_hash()
    E.reset_none_hash_for_test("7")
    assert E.none_hash() == a and a != b and len(a) == 32
    E.reset_none_hash_for_test("0")


def test_pool_null_block_and_distinct_blocks():
    p = E.BlockPool(8, True)
    assert p.null_block().is_null and p.null_block().block_id == 0
    assert p.get_num_free_blocks() == 7
    bl = p.get_new_blocks(7)
    assert sorted(b.block_id for b in bl) == list(range(1, 8))
    assert all(b.ref_cnt == 1 for b in bl)
    with pytest.raises(RuntimeError):
        p.get_new_blocks(1)


def test_pool_free_order_and_lru_eviction():
    p = E.BlockPool(6, True)
    r = _req("a", range(8))
    m = E.KVCacheManager(_cfg(6, 4), 64, True)
    # through the manager: cache two full blocks, free, and check they are evicted last
    blocks = m.allocate_slots(r, 8)
    ids = blocks.block_ids()[0]
    assert len(ids) == 2
    m.free(r)
    pool = m.pool()
    # unhashed blocks are reused first: a new request gets the never-used blocks before the cached ones
    r2 = _req("b", range(100, 112))
    got = m.allocate_slots(r2, 12).block_ids()[0]
    assert not (set(got) & set(ids))
    # now the pool is short: the next allocation evicts the cached blocks (LRU: tail block first)
    r3 = _req("c", range(200, 208))
    got3 = m.allocate_slots(r3, 8).block_ids()[0]
    assert set(got3) == set(ids)
    assert pool.block(ids[0]).block_hash != None  # re-cached under request c's hashes


def test_touch_protects_from_eviction_and_prefix_hit():
    m = E.KVCacheManager(_cfg(8, 4), 64, True)
    r = _req("a", range(10))
    m.allocate_slots(r, 10)
    m.free(r)
    r2 = _req("b", list(range(8)) + [99, 98, 97])
    computed, n = m.get_computed_blocks(r2)
    assert n == 8 and len(computed.block_ids()[0]) == 2
    free_before = m.num_free_blocks()
    nb = m.allocate_slots(r2, 3, n, computed)
    assert nb is not None
    # two cached blocks left the free list (touch) + one new block
    assert m.num_free_blocks() == free_before - 3
    assert m.get_block_ids("b")[0][:2] == computed.block_ids()[0]


def test_full_prompt_hit_leaves_last_token_to_compute():
    m = E.KVCacheManager(_cfg(8, 4), 64, True)
    r = _req("a", range(8))
    m.allocate_slots(r, 8)
    m.free(r)
    r2 = _req("b", range(8))
    _, n = m.get_computed_blocks(r2)
    assert n == 4  # the block holding the last token is recomputed so logits exist


def test_allocate_returns_none_when_short_and_reset_prefix_cache():
    m = E.KVCacheManager(_cfg(4, 4), 64, True)  # 3 usable blocks
    a = _req("a", range(8))
    assert m.allocate_slots(a, 8) is not None
    b = _req("b", range(50, 58))
    assert m.allocate_slots(b, 8) is None
    assert not m.reset_prefix_cache()  # blocks in use
    m.free(a)
    assert m.reset_prefix_cache()
    _, n = m.get_computed_blocks(_req("c", range(8)))
    assert n == 0


def test_caching_disabled_never_hits():
    m = E.KVCacheManager(_cfg(8, 4), 64, False)
    a = _req("a", range(8))
    m.allocate_slots(a, 8)
    m.free(a)
    _, n = m.get_computed_blocks(_req("b", range(8)))
    assert n == 0


def test_lookahead_tokens_reserve_blocks():
    m = E.KVCacheManager(_cfg(8, 4), 64, True)
    a = _req("a", range(4))
    nb = m.allocate_slots(a, 4, num_lookahead_tokens=5)
    assert len(nb.block_ids()[0]) == 3  # ceil((4 + 5) / 4)


def test_common_prefix_blocks():
    m = E.KVCacheManager(_cfg(12, 4), 64, True)
    a = _req("a", list(range(8)) + [1])
    m.allocate_slots(a, 9)
    b = _req("b", list(range(8)) + [2])
    comp, n = m.get_computed_blocks(b)
    m.allocate_slots(b, 1, n, comp)
    assert m.get_num_common_prefix_blocks(a, 2) == [2]


def test_hybrid_full_plus_mamba_groups():
    full = E.KVCacheSpec(kind=E.KVSpecKind.FULL_ATTENTION, block_size=4, num_kv_heads=1, head_size=8)
    mamba = E.KVCacheSpec(kind=E.KVSpecKind.MAMBA, block_size=4, mamba_state_bytes=1024)
    cfg = E.KVCacheConfig(10, [E.KVCacheGroupSpec(["a0"], full), E.KVCacheGroupSpec(["g0"], mamba)])
    m = E.KVCacheManager(cfg, 64, True)
    a = _req("a", range(9))
    nb = m.allocate_slots(a, 9).block_ids()
    assert len(nb[0]) == 3 and len(nb[1]) == 1   # one state block per request
    a.num_computed_tokens = 9
    a.append_output_token(5)
    nb2 = m.allocate_slots(a, 1).block_ids()
    assert nb2[1] == []                           # state block is not re-allocated
    m.free(a)
    # recurrent state cannot be prefix-cached: the hybrid coordinator reports a miss
    _, n = m.get_computed_blocks(_req("b", range(9)))
    assert n == 0
    assert m.num_free_blocks() == 9


def test_sliding_window_frees_blocks_behind_the_window():
    cfg = _cfg(16, 4, kind=E.KVSpecKind.SLIDING_WINDOW, sliding_window=8)
    m = E.KVCacheManager(cfg, 256, True)
    a = _req("a", range(32))
    m.allocate_slots(a, 32)
    assert m.num_free_blocks() == 15 - 8
    a.num_computed_tokens = 32
    a.append_output_token(1)
    m.allocate_slots(a, 1)
    ids = m.get_block_ids("a")[0]
    # blocks wholly before position 32 - 8 + 1 were swapped for the null block and freed
    assert ids[:6] == [0] * 6
    assert m.num_free_blocks() == 15 - 3
