"""Failure detection on one GPU, without faulting it: a wait on a counter that nothing raises
runs out after a short, runtime-set limit, the kernel records the reason in the status word and
returns, the context stays usable, and the engine turns the status into EngineDeadError.

Reference behaviour: a runner failure ends the engine for every waiter
(src/vllm/v1/engine/core_proc.cpp:140-146)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_FLAG_TIMEOUT = 2


@pytest.fixture
def short_peer_wait():
    from vllm_cpp_b200.ops import _lib
    prev = _lib.lib().b200_set_peer_wait_cycles(2_000_000)      # about a millisecond
    yield
    _lib.lib().b200_set_peer_wait_cycles(prev)


def _timed_out_reduce(device):
    """Launches the owner-side reduce of the fused tensor-parallel path with an arrival count
    that never comes: local buffers stand in for the peers, nothing scatters into them."""
    from vllm_cpp_b200.parallel.comm import SingleComm
    from vllm_cpp_b200.parallel.tp_fused import TpFusedContext
    H, T = 512, 64
    tpf = TpFusedContext(SingleComm(), device, H, T)
    w = torch.ones(H, dtype=torch.bfloat16, device=device)
    hidden = torch.randn(T, H, device=device).to(torch.bfloat16)
    tpf.first_norm(hidden, w, 1e-6, False)
    tpf.reduce_norm_gather(T, expected_rs=4, weight=w, eps=1e-6, gemma=False)
    torch.cuda.synchronize()
    return tpf


def test_peer_wait_runs_out_and_the_context_survives(short_peer_wait):
    from vllm_cpp_b200 import ops
    dev = torch.device("cuda", 0)
    assert ops.read_status() == 0
    tpf = _timed_out_reduce(dev)
    assert ops.read_status() == ERR_FLAG_TIMEOUT          # recorded, then cleared by the read
    assert ops.read_status() == 0
    # the next launches work: same context, a plain kernel against fp32
    x = torch.randn(64, 512, device=dev).to(torch.bfloat16)
    w = (torch.rand(512, device=dev) + 0.5).to(torch.bfloat16)
    got = ops.rmsnorm(x, w, 1e-6)
    xf = x.float()
    want = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (got.float() - want).abs().max().item() < 3e-2
    assert ops.read_status() == 0
    tpf.close()


def test_engine_raises_engine_dead_after_a_kernel_gave_up(short_peer_wait):
    from vllm_cpp_b200 import _engine as E
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.config import EngineArgs, synthetic_config
    from vllm_cpp_b200.engine import LLM, SamplingParams
    cfg = synthetic_config("tiny-qwen3")
    cfg.head_dim = 128
    llm = LLM(EngineArgs(model_config=cfg, device="cuda", block_size=16, num_blocks=64,
                         max_model_len=256, max_num_seqs=2, max_num_batched_tokens=128))
    llm.add_request(list(range(1, 20)), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    llm.step()                                   # a healthy step
    tpf = _timed_out_reduce(llm.device)          # a kernel of this process gives up a wait
    with pytest.raises(E.EngineDeadError):
        for _ in range(3):                       # async scheduling may deliver one step late
            llm.step()
    assert ops.read_status() == ERR_FLAG_TIMEOUT
    tpf.close()


def test_oneshot_allreduce_norm_on_one_gpu_with_a_stand_in_peer():
    """The one-shot all-reduce + residual + RMSNorm kernel with local buffers standing in for a
    second rank: numerics against fp32, monotonic counters over several ops, and an arrival that
    never comes makes the bounded wait report kErrFlagTimeout and leave the engine usable."""
    import ctypes
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.ops import reference as ref
    from vllm_cpp_b200.ops._lib import check, lib, ptr, stream_ptr
    from vllm_cpp_b200.parallel.tp_fused import B200TpOneShot, _declare
    _declare()
    dev = torch.device("cuda")
    T, H = 37, 512
    torch.manual_seed(0)
    mine = (torch.randn(T, H, device=dev)).to(torch.bfloat16)
    peer = (torch.randn(T, H, device=dev)).to(torch.bfloat16)
    resid = (torch.randn(T, H, device=dev)).to(torch.bfloat16)
    w = (torch.rand(H, device=dev) + 0.5).to(torch.bfloat16)
    out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros(64, dtype=torch.int32, device=dev)          # [2 counters | ... | seq @32 | done @48]
    peer_flags = torch.zeros(64, dtype=torch.int32, device=dev)     # what this rank signals on the "peer"

    def launch(res):
        a = B200TpOneShot()
        a.world, a.rank, a.M, a.H = 2, 0, T, H
        a.peer_partial[0], a.peer_partial[1] = ptr(mine), ptr(peer)
        a.peer_flags[0], a.peer_flags[1] = ptr(flags), ptr(peer_flags)
        a.seq, a.done_counter = flags.data_ptr() + 128, flags.data_ptr() + 192
        a.residual, a.norm_w, a.out = ptr(res), ptr(w), ptr(out)
        a.eps, a.gemma = 1e-6, 0
        check(lib().b200_tp_oneshot_allreduce_norm(ctypes.byref(a), stream_ptr()), "oneshot")

    old = lib().b200_set_peer_wait_cycles(2_000_000)       # about a millisecond
    try:
        for op in range(3):
            flags[1] = op + 1                       # the stand-in peer's arrival for this op
            r = resid.clone()
            launch(r)
            torch.cuda.synchronize()
            s = (mine.float() + peer.float() + resid.float()).to(torch.bfloat16)
            exp, _ = ref.rmsnorm(s, w, 1e-6)
            assert torch.equal(r, s)
            assert ((out.float() - exp.float()).norm() / exp.float().norm()).item() < 5e-3
            assert int(flags[0]) == op + 1 and int(peer_flags[0]) == op + 1 and int(flags[32]) == op + 1
            assert ops.read_status() == 0
        # no arrival for op 4: the wait runs out, the kernel returns and reports it
        launch(resid.clone())
        torch.cuda.synchronize()
        assert ops.read_status() == 2
        # and the next launch works once the peer has caught up
        flags[1] = 5
        launch(resid.clone())
        torch.cuda.synchronize()
        assert ops.read_status() == 0
    finally:
        lib().b200_set_peer_wait_cycles(old)
