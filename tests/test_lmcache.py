"""LMCache client: hashing, keys and wire bytes against vectors produced by LMCache itself
(blake3 package / lmcache.v1 protocol classes), and the TCP client against an in-process server
that parses the messages independently with ``struct``."""
import socket
import struct
import threading

import pytest
import torch

from vllm_cpp_b200 import _engine as E

lm = E.lmcache


def test_blake3_known_answers():
    def pat(n):
        return bytes(i % 251 for i in range(n))
    # official BLAKE3 test vectors (input byte i = i mod 251)
    assert lm.blake3(pat(0)).hex() == "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"
    assert lm.blake3(pat(1)).hex() == "2d3adedff11b61f14c886e35afa036736dcd87a74d27b5c1510225d0f592e213"
    assert lm.blake3(pat(1024)).hex() == "42214739f095a406f3fc83deb889744ac00df831c10daa55189b5d121c855af7"
    assert lm.blake3(pat(1025)).hex() == "d00278ae47eb27b34faecf67b4fe263f82d5412916c1ffd97c8cb7fb814b8444"
    assert lm.blake3(pat(2048)).hex() == "e776b6028c7cd22a4d0ba182a8bf62205d2ef576467e838ed6f2529b85fba24a"


def test_token_hasher_matches_lmcache():
    h = lm.TokenHasher(4)
    assert h.none_hash.hex() == "7e3eff9ef7613a50340eb12677ee03b83ac759fcba9bb32705f07248d56d473b"
    assert h.hash_tokens([0]).hex() == "2eddf2cbf072f71f8e6b766cdd3096880ba606cf90e505269042228550c9eeb0"
    assert h.hash_tokens([1, 2, 3]).hex() == "d1d19ba2c9dd11f963a9e18fbcb6c37bca3f0c719444f0170aba741f2d68d838"
    assert h.hash_tokens([65536, 4294967295, 0]).hex() == \
        "e6704efd16a87f8888fe6c7f43f4dab9bc6a3f1a1871b115ca3414b6c346212a"
    d0 = h.hash_tokens([1, 2, 3, 4])
    assert d0.hex() == "6309ed506b8721905753f5c73c070bb21c3aafbd9b474b1e231f41368b71123c"
    assert h.hash_tokens([5, 6, 7, 8], d0).hex() == \
        "98efc76eafb06cfe774c31ff151f300b61a614c27982a211bb8cdbd83a8c0e19"
    assert [x.hex() for x in h.chunk_hashes(list(range(12)))] == [
        "a2981a4d792b45f791d784bfd025148836ce3032f546cc490ef9fb7db9e639de",
        "f76a7280af54e664fff4e1239c4a72936fedc49ba027e3a969a314ae980dbfd5",
        "52cde0b920e22a78324ccefea623c5707678d56033320a60ba85eb2d7e13532e"]
    assert len(h.chunk_hashes(list(range(10)))) == 2          # the partial tail is dropped
    assert lm.TokenHasher.fold(h.hash_tokens([0])) == 3377122253324089119


def test_vllm_sha256_cbor_chunk_keys_agree_with_a_peer():
    """Keys derived by a real vLLM + LMCache pair (ChunkedTokenDatabase, sha256_cbor, seed 0)."""
    assert lm.vllm_none_hash("0") == 5625442194607170974
    assert [(a, b, f"{h:x}") for a, b, h in lm.vllm_chunk_hashes(list(range(1, 257)))] == \
        [(0, 256, "b44cfe1cb25a9be0")]
    assert [f"{h:x}" for _, _, h in lm.vllm_chunk_hashes(list(range(1000, 1512)))] == \
        ["33d6862800fff40c", "893ec9ccb64be34a"]
    assert [(a, b, f"{h:x}") for a, b, h in lm.vllm_chunk_hashes([10, 11, 12, 13, 14, 15], 4, True)] == \
        [(0, 4, "3b0e6619ff2ca93b"), (4, 6, "eeaac88b910fc20b")]
    assert lm.vllm_chunk_hashes([10, 11, 12, 13, 14, 15], 4, False)[-1][:2] == (0, 4)
    assert lm.vllm_chunk_hashes([7, 8, 9]) == []
    h = lm.vllm_chunk_hashes(list(range(8)), 8)[0][2]
    assert lm.CacheKey("some/model", 4, 3, h, lm.Dtype.FLOAT32).to_string() == "some/model@4@3@1edac42a0285a5f9@float"


def test_cache_key_strings():
    k = lm.CacheKey("gpt2", 1, 0, 3735928559, lm.Dtype.BFLOAT16)
    assert k.to_string() == "gpt2@1@0@deadbeef@bfloat16"
    assert lm.CacheKey("meta-llama/Llama-3.1-8B", 2, 1, 81985529216486895, lm.Dtype.FLOAT16).to_string() == \
        "meta-llama/Llama-3.1-8B@2@1@123456789abcdef@half"
    assert lm.CacheKey("Qwen/Qwen3-27B", 8, 7, 0, lm.Dtype.FLOAT32).to_string() == "Qwen/Qwen3-27B@8@7@0@float"
    back = lm.CacheKey.from_string("m@2@1@ff00@half@tenant%a")
    assert (back.model, back.world_size, back.worker_id, back.chunk_hash, back.dtype) == \
        ("m", 2, 1, 0xff00, lm.Dtype.FLOAT16)
    assert back.tags == [("tenant", "a")] and back.to_string() == "m@2@1@ff00@half@tenant%a"


def test_wire_messages_byte_exact():
    m = lm.ClientMeta()
    m.command, m.key, m.length = lm.Command.PUT, "gpt2@1@0@deadbeef@bfloat16", 4096
    m.fmt, m.dtype, m.shape = lm.MemFormat.KV_2LTD, lm.Dtype.BFLOAT16, [2, 24, 256, 128]
    raw = m.serialize()
    assert len(raw) == 186
    assert raw.hex().startswith("010000000010000001000000030000000000000002000000180000000001000080000000"
                                "67707432403140304064656164626565664062666c6f61743136" + "20" * 8)
    assert raw[36 + len(m.key):] == b" " * (150 - len(m.key))
    back = lm.ClientMeta.deserialize(raw)
    assert (back.command, back.key, back.length, back.shape) == (lm.Command.PUT, m.key, 4096, [2, 24, 256, 128])
    m2 = lm.ClientMeta()
    m2.command, m2.key, m2.fmt, m2.dtype = lm.Command.EXIST, "m@2@1@ff00@half", lm.MemFormat.KV_2LTD, lm.Dtype.FLOAT16
    m2.shape, m2.location = [2, 12, 64, 64], lm.Location.LOCAL_CPU
    assert m2.serialize().hex().startswith("0300000000000000010000000200000001000000020000000c0000004000000040000000"
                                           "6d4032403140666630304068616c66")
    s = lm.ServerMeta()
    s.code, s.length, s.fmt, s.dtype, s.shape = lm.ReturnCode.SUCCESS, 4096, lm.MemFormat.KV_2LTD, lm.Dtype.BFLOAT16, \
        [2, 24, 256, 128]
    assert s.serialize().hex() == "c80000000010000001000000030000000200000018000000000100008000000000000000"
    f = lm.ServerMeta()
    f.code, f.shape = lm.ReturnCode.FAIL, [0]
    assert f.serialize().hex() == "9001" + "00" * 34
    ok = lm.ServerMeta.deserialize(bytes.fromhex(
        "c8000000400000000100000002000000020000000c000000400000004000000001000000"))
    assert (ok.code, ok.length, ok.dtype, ok.shape, ok.location) == \
        (lm.ReturnCode.SUCCESS, 64, lm.Dtype.FLOAT16, [2, 12, 64, 64], lm.Location.LOCAL_CPU)


def test_kv2ltd_layout():
    L, T, D = 2, 3, 4
    vals = torch.arange(2 * L * T * D, dtype=torch.float32).reshape(2, L, T, D)
    k = [vals[0, l].numpy().tobytes() for l in range(L)]
    v = [vals[1, l].numpy().tobytes() for l in range(L)]
    packed = lm.pack_kv2ltd(L, T, D, 4, k, v)
    assert packed == vals.numpy().tobytes()
    assert packed.hex().startswith("000000000000803f0000004000004040000080400000a040")
    k2, v2 = lm.unpack_kv2ltd(L, T, D, 4, packed)
    assert k2 == k and v2 == v


class MockServer(threading.Thread):
    """Speaks the server side with struct / bytes only."""

    def __init__(self):
        super().__init__(daemon=True)
        self.sock = socket.socket()
        self.sock.bind(("127.0.0.1", 0))
        self.sock.listen(8)
        self.port = self.sock.getsockname()[1]
        self.store = {}

    @staticmethod
    def _recv(c, n):
        b = b""
        while len(b) < n:
            chunk = c.recv(n - len(b))
            if not chunk:
                return None
            b += chunk
        return b

    def run(self):
        while True:
            c, _ = self.sock.accept()
            threading.Thread(target=self._serve, args=(c,), daemon=True).start()

    def _serve(self, c):
        while True:
            hdr = self._recv(c, 186)
            if hdr is None:
                break
            cmd, length, fmt, dtype, loc, s0, s1, s2, s3 = struct.unpack("<9i", hdr[:36])
            key = hdr[36:].decode().strip()
            if cmd == 1:
                self.store[key] = (self._recv(c, length), fmt, dtype, (s0, s1, s2, s3))
            elif cmd == 2:
                if key in self.store:
                    data, f, d, sh = self.store[key]
                    c.sendall(struct.pack("<9i", 200, len(data), f, d, *sh, 0) + data)
                else:
                    c.sendall(struct.pack("<9i", 400, 0, 0, 0, 0, 0, 0, 0, 0))
            elif cmd == 3:
                c.sendall(struct.pack("<9i", 200 if key in self.store else 400, 0, 0, 0, 0, 0, 0, 0, 0))
            elif cmd == 5:
                c.sendall(struct.pack("<9i", 200, 0, 0, 0, 0, 0, 0, 0, 0))
        c.close()


def test_client_against_mock_server_and_store_roundtrip():
    from vllm_cpp_b200.worker.lmcache import LMCacheStore, parse_url
    assert parse_url("lm://cache.local:65432") == ("cache.local", 65432)
    with pytest.raises(ValueError):
        parse_url("http://x:1")
    srv = MockServer()
    srv.start()
    torch.manual_seed(0)
    layers, bs, hkv, d, chunk = 3, 4, 2, 8, 8
    caches = [torch.randn(16, 2, bs, hkv, d).to(torch.bfloat16) for _ in range(layers)]
    store = LMCacheStore(f"lm://127.0.0.1:{srv.port}", "tiny", caches, bs, chunk_size=chunk)
    assert store.client.health()
    tokens = list(range(100, 121))                    # 21 tokens: two complete chunks
    blocks = [5, 2, 9, 11, 3, 7]
    assert store.lookup(tokens) == 0
    assert store.client.get("absent@1@0@0@bfloat16") is None       # absent keys are not an error
    assert store.store(tokens, blocks) == 2
    assert store.store(tokens, blocks) == 0           # already there
    assert store.lookup(tokens) == 16
    assert store.lookup(tokens[:8] + [1] * 8) == 8    # a different second chunk shares the first
    key0 = store.chunk_keys(tokens)[0]
    data, fmt, dtype, shape = srv.store[key0][0], *srv.store[key0][1:3], srv.store[key0][3]
    assert (fmt, dtype, shape) == (1, 3, (2, layers, chunk, hkv * d)) and len(data) == 2 * layers * chunk * hkv * d * 2
    # a second engine with empty caches gets the same KV in its own blocks
    caches2 = [torch.zeros_like(c) for c in caches]
    store2 = LMCacheStore(f"lm://127.0.0.1:{srv.port}", "tiny", caches2, bs, chunk_size=chunk, connect=False)
    store2.client = store.client                      # the mock accepts one connection
    blocks2 = [1, 4, 6, 8]
    assert store2.load(tokens, blocks2, 16) == 16
    for c1, c2 in zip(caches, caches2):
        for t in range(16):
            b1, o = blocks[t // bs], t % bs
            b2 = blocks2[t // bs]
            assert torch.equal(c1[b1, :, o], c2[b2, :, o])
    store.client.close()


def test_engine_reuses_kv_from_lmcache_server():
    """Engine A serves a prompt and stores its KV chunks; engine B (fresh process state, same
    weights) finds them at admission, loads them into its own blocks and produces the same
    tokens while computing only the tail of the prompt."""
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    srv = MockServer()
    srv.start()
    cfg = synthetic_config("tiny-dense")
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=g).tolist()
    ktc = {"kv_connector": "LMCacheConnector", "url": f"lm://127.0.0.1:{srv.port}", "chunk_size": 32}

    def engine(with_cache):
        return LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, max_model_len=128, max_num_seqs=2,
                              max_num_batched_tokens=128, num_blocks=32, seed=0,
                              kv_transfer_config=ktc if with_cache else None))

    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    plain = engine(False).generate([prompt], sp)[0].outputs[0].token_ids
    a = engine(True)
    assert a.generate([prompt], sp)[0].outputs[0].token_ids == plain
    assert a.offload.stored_chunks == 2                                  # 64 of the 75 computed tokens
    import time
    deadline = time.monotonic() + 5.0                                    # the server thread files them on its own time
    while len(srv.store) < 2 and time.monotonic() < deadline:
        time.sleep(0.01)
    assert len(srv.store) == 2
    b = engine(True)
    out = b.generate([prompt], sp)[0]
    assert out.outputs[0].token_ids == plain
    assert b.offload.loaded_tokens == 64 and out.num_cached_tokens == 64
    assert b.offload.stored_chunks == 0                                  # nothing new to send
