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
