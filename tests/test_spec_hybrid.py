"""Speculative decoding on the hybrid (Gated DeltaNet + attention) models: n-gram drafts and the
multi-token-prediction head, with the recurrent state saved before a verifying step and restored
when a draft is rejected (the kept tokens of that step then run again with the next one)."""
import pytest
import torch

from vllm_cpp_b200.config import EngineArgs, synthetic_config
from vllm_cpp_b200.engine import LLM, SamplingParams
from vllm_cpp_b200.spec_decode import SpeculativeConfig


def _prompts(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    lens = (70, 5, 33, 120)
    # a small alphabet, so that n-grams recur and prompt lookup proposes both right and wrong tokens
    return [torch.randint(0, 24, (n,), generator=g).tolist() for n in lens]


def _run(cfg, prompts, spec, budget=256, n=14, spoil=False):
    llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=160, max_model_len=512,
                         max_num_seqs=4, max_num_batched_tokens=budget, speculative_config=spec))
    if spoil:
        # every other step the first draft of each request is replaced by a token the trunk will not
        # choose, so rejections happen whatever the proposer finds
        orig, step = llm.runner._build_output, [0]

        def spoiled(info, ids_host):
            out = orig(info, ids_host)
            step[0] += 1
            if step[0] % 2:
                for d in llm.runner._drafts.values():
                    if d:
                        d[0] = (d[0] + 1) % cfg.vocab_size
            return out
        llm.runner._build_output = spoiled
    # Random-weight tiny models mostly repeat one token, which a wrong recurrent state would not
    # change; so besides the tokens the test keeps, for every token a request emitted, the gap
    # between the two largest logits of the row that produced it, and compares those too.
    trace: dict = {}
    inner = llm.runner._build_output

    def traced(info, ids_host):
        lg = llm.runner._logits
        out = inner(info, ids_host)
        row = 0
        for r, p in enumerate(info.produces_token):
            if not p:
                continue
            kept = len(out.sampled_token_ids[r])
            top = lg[row: row + kept].float().topk(2, -1).values
            trace.setdefault(info.req_ids[r], []).extend((top[:, 0] - top[:, 1]).tolist())
            row += info.num_draft[r] + 1
        return out
    llm.runner._build_output = traced
    sp = SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)
    toks = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    llm.logit_gaps = [trace[k][: len(t)] for k, t in zip(sorted(trace, key=lambda x: int(x.split("-")[-1]) if x.split("-")[-1].isdigit() else x), toks)]
    return toks, llm


def _same(got, llm_got, base, llm_base, tol=0.03):
    assert got == base
    for a, b in zip(llm_got.logit_gaps, llm_base.logit_gaps):
        assert len(a) == len(b) and all(abs(x - y) <= tol for x, y in zip(a, b)), (a, b)


@pytest.mark.parametrize("shape", ["tiny-gdn", "tiny-gdn-moe"])
def test_ngram_drafts_on_a_hybrid_keep_the_greedy_tokens(shape):
    cfg = synthetic_config(shape)
    drafted = accepted = 0
    for seed in (1, 2, 3):
        prompts = _prompts(cfg, seed)
        base, lb = _run(cfg, prompts, None)
        for k, budget in ((1, 256), (3, 48)):
            spec = SpeculativeConfig(method="ngram", num_speculative_tokens=k, prompt_lookup_min=1, prompt_lookup_max=2)
            got, llm = _run(cfg, prompts, spec, budget)
            _same(got, llm, base, lb)
            drafted += llm.runner.spec_stats["drafted"]
            accepted += llm.runner.spec_stats["accepted"]
    assert 0 < accepted <= drafted
    # and with drafts spoiled on purpose: rejections restore the saved state and the kept tokens of
    # the step run again, so the tokens still do not change
    prompts = _prompts(cfg, 4)
    base, lb = _run(cfg, prompts, None)
    spec = SpeculativeConfig(method="ngram", num_speculative_tokens=2, prompt_lookup_min=1, prompt_lookup_max=2)
    got, llm = _run(cfg, prompts, spec, 64, spoil=True)
    _same(got, llm, base, lb)
    st = llm.runner.spec_stats
    assert 0 < st["accepted"] < st["drafted"]


def test_mtp_head_drafts_keep_the_greedy_tokens():
    cfg = synthetic_config("tiny-gdn")
    prompts = _prompts(cfg, 5)
    base, lb = _run(cfg, prompts, None)
    for k, budget in ((1, 256), (1, 32), (3, 48)):
        got, llm = _run(cfg, prompts, SpeculativeConfig(method="mtp", num_speculative_tokens=k), budget)
        _same(got, llm, base, lb)
        assert llm.runner.spec_stats["drafted"] > 0 and llm.runner.mtp is not None
        # chains of k drafts: the head continues from its own hidden state for drafts two to k
        assert all(len(d) % k == 0 for d in llm.runner.mtp_proposed.values())
    # the head's cache does not depend on how the prompt was chunked: the same drafts either way
    def drafts(budget):
        _, llm = _run(cfg, prompts[:1], SpeculativeConfig(method="mtp", num_speculative_tokens=1), budget, n=3)
        return list(llm.runner.mtp_proposed.values())
    a, b = drafts(256), drafts(16)
    assert a and a[0] and a == b


def test_mtp_head_weights_load_from_a_checkpoint_stream():
    """``mtp.*`` tensors of a checkpoint go to the head (input-stage tensors kept, blocks and final
    norm renamed to the trunk's names); a checkpoint without them is refused."""
    from vllm_cpp_b200.models.gdn_mtp import Qwen35MTP
    cfg = synthetic_config("tiny-gdn")
    llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=32, max_model_len=128,
                         max_num_seqs=2, max_num_batched_tokens=64))
    ref = Qwen35MTP(llm.model)
    ref.init_random(3)
    H = cfg.hidden_size
    named = {"mtp.fc.weight": ref.w["fc"], "mtp.pre_fc_norm_embedding.weight": ref.w["pre_fc_norm_embedding"],
             "mtp.pre_fc_norm_hidden.weight": ref.w["pre_fc_norm_hidden"], "mtp.norm.weight": torch.zeros(H)}
    D = cfg.head_dim
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.empty(*s).normal_(0, 0.02, generator=g).to(torch.bfloat16)
    p = "mtp.layers.0."
    named.update({p + "input_layernorm.weight": torch.zeros(H), p + "post_attention_layernorm.weight": torch.zeros(H),
                  p + "self_attn.q_proj.weight": rn(cfg.num_heads * D * 2, H), p + "self_attn.k_proj.weight": rn(cfg.num_kv_heads * D, H),
                  p + "self_attn.v_proj.weight": rn(cfg.num_kv_heads * D, H), p + "self_attn.o_proj.weight": rn(H, cfg.num_heads * D),
                  p + "self_attn.q_norm.weight": torch.zeros(D), p + "self_attn.k_norm.weight": torch.zeros(D),
                  p + "mlp.gate_proj.weight": rn(cfg.intermediate_size, H), p + "mlp.up_proj.weight": rn(cfg.intermediate_size, H),
                  p + "mlp.down_proj.weight": rn(H, cfg.intermediate_size)})
    head = Qwen35MTP(llm.model)
    head.load_weights(iter(named.items()))
    assert torch.equal(head.w["fc"], ref.w["fc"]) and head.inner.w["embed"] is llm.model.w["embed"]
    assert head.inner.layers[0]["qkv"].shape[1] == H and "final_norm" in head.inner.w
    with pytest.raises(ValueError):
        Qwen35MTP(llm.model).load_weights(iter({"model.embed_tokens.weight": torch.zeros(4, H)}.items()))


def test_mtp_chains_are_accepted_when_the_head_agrees_with_the_trunk():
    """A head rigged to repeat the trunk's own choice (fc passes the trunk's hidden state through,
    its block adds nothing): on a model that repeats tokens its chains are accepted, which runs the
    accepting path with several drafts per step; tokens and logit gaps stay those of plain decoding."""
    cfg = synthetic_config("tiny-gdn")
    prompts = _prompts(cfg, 1)
    base, lb = _run(cfg, prompts, None)
    H = cfg.hidden_size

    def rig(llm):
        m = llm.runner.mtp
        m.w["fc"] = torch.cat([torch.zeros(H, H), torch.eye(H)], 1).to(torch.bfloat16)
        m.inner.layers[0]["o"].zero_()
        m.inner.layers[0]["down"].zero_()

    for k in (1, 3):
        llm = LLM(EngineArgs(model_config=cfg, device="cpu", block_size=16, num_blocks=160, max_model_len=512,
                             max_num_seqs=4, max_num_batched_tokens=64,
                             speculative_config=SpeculativeConfig(method="mtp", num_speculative_tokens=k)))
        rig(llm)
        sp = SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True)
        got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        assert got == base
        st = llm.runner.spec_stats
        assert st["accepted"] > 0.5 * st["drafted"] > 0, st
        # fewer trunk steps than tokens: accepted drafts really shorten the loop
        assert llm.runner.num_kernel_steps < 14 + 4
