"""Host-side properties of the kernel wrappers that need no GPU."""
import torch


def test_workspace_never_releases_an_outgrown_buffer():
    """A CUDA graph captured while a smaller scratch buffer was current keeps its address, so growing
    a workspace must keep the old buffer alive."""
    from vllm_cpp_b200 import ops
    dev = torch.device("cpu")
    a = ops.workspace(dev, 1 << 20, "retire-test")
    addr = a.data_ptr()
    b = ops.workspace(dev, 4 << 20, "retire-test")
    assert b.numel() >= 4 << 20 and b.data_ptr() != addr
    assert any(t.data_ptr() == addr for t in ops._retired_workspaces)
    assert ops.workspace(dev, 1 << 20, "retire-test") is b


def test_attention_backend_registry_priorities():
    from vllm_cpp_b200.config import synthetic_config
    from vllm_cpp_b200.models import attention_backends as AB
    assert AB.select("decode", head_dim=128, group=4, block_size=16).name == "tcgen05-decode"
    assert AB.select("decode", head_dim=256, group=6, block_size=32).name == "tcgen05-decode"
    assert AB.select("decode", head_dim=64, group=4, block_size=16).name == "cuda-core-decode"
    assert AB.select("decode", head_dim=128, group=32, block_size=16).name == "cuda-core-decode"
    assert AB.select("decode", head_dim=128, group=4, block_size=48).name == "cuda-core-decode"
    b = AB.select("decode", head_dim=128, group=4, block_size=16, exclude=("tcgen05-decode",))
    assert b.name == "cuda-core-decode"
    assert AB.select("decode", head_dim=96, group=4, block_size=16) is None
    assert AB.select("prefill", head_dim=256, group=1, block_size=16).name == "tcgen05-prefill"
    d = AB.describe(synthetic_config("qwen3.6-27b"), 32)
    assert d["paged"] == {"decode": "tcgen05-decode", "prefill": "tcgen05-prefill"}
    assert d["gdn"] == {"decode": "gdn-packed-decode", "prefill": "gdn-chunk-scan"}
    assert AB.describe(synthetic_config("deepseek-v2-lite"), 64)["mla"]["decode"] == "mla-absorbed-decode"
    from vllm_cpp_b200 import ops
    assert ops._decode_uses_tc(128, 4, 16) and not ops._decode_uses_tc(64, 4, 16)


def test_validation_layer_names_the_broken_rule():
    import pytest
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.ops.validate import OpArgumentError, validate
    a = torch.zeros(4, 64, dtype=torch.bfloat16)
    w = torch.zeros(8, 64, dtype=torch.bfloat16)
    validate("gemm", a=a, w=w)
    with pytest.raises(OpArgumentError, match="same K"):
        validate("gemm", a=a, w=torch.zeros(8, 32, dtype=torch.bfloat16))
    with pytest.raises(OpArgumentError, match="are bf16"):
        ops.gemm(a.float(), w)                  # raised before any launcher (or library) is touched
    with pytest.raises(OpArgumentError, match="rows are contiguous"):
        validate("gemm", a=a[:, ::2], w=w[:, ::2])
    with pytest.raises(OpArgumentError, match="multiple of 256"):
        validate("gemm_nvfp4", aq=torch.zeros(4, 64, dtype=torch.uint8), wq=torch.zeros(8, 64, dtype=torch.uint8),
                 sfa=torch.zeros(1), sfw=torch.zeros(1), g_a=torch.ones(1), g_w=torch.ones(1))
    with pytest.raises(OpArgumentError, match="head_dim is 64, 128 or 256"):
        validate("attn_decode", q=torch.zeros(2, 4 * 96, dtype=torch.bfloat16), num_q_heads=4, num_kv_heads=2,
                 head_dim=96, block_size=16, kv_cache=torch.zeros(3, 2, 16, 2, 96, dtype=torch.bfloat16),
                 block_table=torch.zeros(2, 4, dtype=torch.int32), seq_lens=torch.zeros(2, dtype=torch.int32))
    e = None
    try:
        validate("rmsnorm", x=torch.zeros(3, 8, dtype=torch.bfloat16), weight=torch.zeros(7))
    except OpArgumentError as ex:
        e = ex
    assert e is not None and e.op == "rmsnorm" and "weight" in e.rule and "(3, 8)" in str(e)


def test_nvfp4_plan_file_round_trip(tmp_path, monkeypatch):
    """The W4A4 tile plans survive a restart through B200_NVFP4_PLAN_FILE; a damaged file is ignored."""
    from vllm_cpp_b200.ops import quant as Q
    path = str(tmp_path / "plans.json")
    monkeypatch.setenv("B200_NVFP4_PLAN_FILE", path)
    saved = dict(Q._NVFP4_PLANS)
    try:
        Q._NVFP4_PLANS.clear()
        Q._NVFP4_PLANS[(64, 34816, 5120)] = 256
        Q._NVFP4_PLANS[(64, 5120, 17408)] = 128
        Q.save_nvfp4_plans()
        Q._NVFP4_PLANS.clear()
        Q._NVFP4_PLANS[(64, 5120, 17408)] = 256              # already in memory: kept
        assert Q.load_nvfp4_plans() == 1
        assert Q._NVFP4_PLANS == {(64, 34816, 5120): 256, (64, 5120, 17408): 256}
        with open(path, "w") as f:
            f.write("{not json")
        Q._NVFP4_PLANS.clear()
        assert Q.load_nvfp4_plans() == 0 and not Q._NVFP4_PLANS
        with open(path, "w") as f:
            f.write('{"1,2": 256, "a,b,c": 128, "64,8,256": 64, "16,512,256": 128}')
        assert Q.load_nvfp4_plans() == 1 and Q._NVFP4_PLANS == {(16, 512, 256): 128}
    finally:
        Q._NVFP4_PLANS.clear()
        Q._NVFP4_PLANS.update(saved)
