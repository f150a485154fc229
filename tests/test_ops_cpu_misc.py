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
