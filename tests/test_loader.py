"""Checkpoint loading end to end on CPU: a synthetic HF directory (config + safetensors +
tokenizer) through the public LLM API with text prompts; quantised-layout expansion against
the format definitions."""
import json
import os

import torch

from vllm_cpp_b200 import loader
from vllm_cpp_b200.config import EngineArgs, synthetic_config
from vllm_cpp_b200.engine import LLM, SamplingParams
from vllm_cpp_b200.loader.safetensors import save_file


def test_synthetic_checkpoint_round_trip(tmp_path):
    cfg = synthetic_config("tiny-qwen3")
    d = loader.write_synthetic_checkpoint(str(tmp_path / "ckpt"), cfg, seed=3)
    assert {"config.json", "model.safetensors", "tokenizer.json"} <= set(os.listdir(d))
    llm = LLM(EngineArgs(model=d, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                         max_num_seqs=4, max_num_batched_tokens=128))
    assert llm.tokenizer is not None and llm.tokenizer.vocab_size <= cfg.vocab_size
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = llm.generate(["The quick brown fox", "and then there was"], sp)
    assert all(len(o.outputs[0].token_ids) == 6 for o in outs)
    assert all(isinstance(o.outputs[0].text, str) for o in outs)
    # same weights created in memory give the same greedy tokens
    ref = LLM(EngineArgs(model_config=cfg, seed=3, device="cpu", block_size=16, num_blocks=64,
                         max_model_len=256, max_num_seqs=4, max_num_batched_tokens=128))
    ids = [llm.tokenizer.encode(p) for p in ["The quick brown fox", "and then there was"]]
    want = ref.generate(ids, sp)
    assert [o.outputs[0].token_ids for o in outs] == [o.outputs[0].token_ids for o in want]


def test_nvfp4_layouts_expand_to_the_same_weights(tmp_path):
    torch.manual_seed(0)
    n, k = 8, 64
    codes = torch.randint(0, 16, (n, k), dtype=torch.uint8)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    bscale = (torch.rand(n, k // 16) * 3 + 0.25).to(torch.float8_e4m3fn)
    g = torch.tensor([448.0 * 6.0 / 3.0])
    val = loader._FP4_VALUES[codes.long()]
    want = (val.reshape(n, -1, 16) * (bscale.float() / g).reshape(n, -1, 1)).reshape(n, k)
    got = loader.dequant_nvfp4(packed, bscale, g, True)
    assert torch.allclose(got.float(), want, rtol=1e-2, atol=1e-6)
    got2 = loader.dequant_nvfp4(packed, bscale, 1.0 / g, False)
    assert torch.equal(got, got2)
    # through the directory loader: compressed-tensors and ModelOpt names
    d = tmp_path / "q"
    d.mkdir()
    cfg = synthetic_config("tiny-qwen3")
    with open(d / "config.json", "w") as f:
        json.dump(loader.hf_config_dict(cfg), f)
    save_file({"a.weight_packed": packed, "a.weight_scale": bscale, "a.weight_global_scale": g,
               "b.weight": packed, "b.weight_scale": bscale, "b.weight_scale_2": 1.0 / g,
               "c.weight": torch.ones(2, 2, dtype=torch.bfloat16)}, str(d / "model.safetensors"))
    _, it, tok = loader.load_model_dir(str(d))
    t = dict(it)
    assert tok is None and set(t) == {"a.weight", "b.weight", "c.weight"}
    assert torch.equal(t["a.weight"], got) and torch.equal(t["b.weight"], got)


def test_fp8_scales(tmp_path):
    torch.manual_seed(1)
    w = torch.randn(256, 384)
    for scale in (torch.tensor(0.5), torch.rand(256, 1) + 0.5, torch.rand(2, 3) + 0.5):
        if scale.numel() == 1 or scale.shape == (256, 1):
            full = scale.expand(256, 384) if scale.numel() > 1 else scale
        else:
            full = scale.repeat_interleave(128, 0).repeat_interleave(128, 1)
        q = (w / full).to(torch.float8_e4m3fn)
        got = loader.dequant_fp8(q, scale, (128, 128))
        assert torch.allclose(got.float(), q.float() * full, rtol=1e-2, atol=1e-3)
        assert (got.float() - w).abs().max() < 0.3


def test_native_layer_binding_matches_the_c_structs():
    """The ctypes mirror of the per-layer launch entry has the C structs' size and layout (the
    kernel library loads without a GPU)."""
    import ctypes
    from vllm_cpp_b200.ops import _lib
    from vllm_cpp_b200.ops.layer import DenseLayerWeights, DenseStep
    if not _lib.available():
        import pytest
        pytest.skip("kernel library not built")
    out = (ctypes.c_int * 4)()
    _lib.lib().b200_dense_layer_abi(out)
    assert list(out) == [ctypes.sizeof(DenseLayerWeights), ctypes.sizeof(DenseStep),
                         DenseLayerWeights.down_scale.offset, DenseStep.fp8_scales.offset]


def test_fp8_checkpoint_loads_into_w8a8_layers(tmp_path):
    """A checkpoint whose projections are e4m3 with per-tensor scales (ModelOpt / compressed-tensors
    fp8 layout) loads into Fp8Weight layers holding the checkpoint's own codes, and generates."""
    import json
    from vllm_cpp_b200.loader.safetensors import SafetensorsFile, save_file
    from vllm_cpp_b200.models.backend import Fp8Weight
    cfg = synthetic_config("tiny-dense")
    d = loader.write_synthetic_checkpoint(str(tmp_path / "ckpt"), cfg, seed=5)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors, codes = {}, {}
    for k in f.keys():
        t = f.get(k).clone()
        if k.endswith("_proj.weight"):
            s = (t.float().abs().max() / 448.0).reshape(1)
            q = (t.float() / s).to(torch.float8_e4m3fn)
            tensors[k], tensors[k[:-len(".weight")] + ".weight_scale"] = q, s
            codes[k] = q
        else:
            tensors[k] = t
    f.close()
    save_file(tensors, os.path.join(d, "model.safetensors"), {"format": "pt"})
    with open(os.path.join(d, "config.json")) as fh:
        hf = json.load(fh)
    hf["quantization_config"] = {"quant_method": "fp8", "activation_scheme": "dynamic"}
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(hf, fh)
    llm = LLM(EngineArgs(model=d, device="cpu", block_size=16, num_blocks=64, max_model_len=256,
                         max_num_seqs=4, max_num_batched_tokens=128))
    down = llm.model.layers[0]["down"]
    assert isinstance(down, Fp8Weight)
    c = codes["model.layers.0.mlp.down_proj.weight"].float()
    ratio = torch.where(c == 0, torch.ones_like(c), down.w8.float() / c)
    assert torch.equal(ratio, ratio.amax(1, keepdim=True).expand_as(ratio))      # the same codes, row by row
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    outs = llm.generate(["The quick brown fox"], sp)
    assert len(outs[0].outputs[0].token_ids) == 5
