"""Architecture name -> model class, with vLLM-style messages for unsupported names.

Reference: ``include/vllm/model_executor/models/model_registry.h:137-220`` and
``model_registry.cpp`` (self-registering factories, unsupported-architecture messages).
"""
from __future__ import annotations

_DENSE = ("LlamaForCausalLM", "MistralForCausalLM", "Qwen3ForCausalLM", "Qwen2ForCausalLM",
          "GemmaForCausalLM", "Gemma2ForCausalLM", "Gemma3ForCausalLM", "Glm4ForCausalLM",
          "Olmo2ForCausalLM", "Olmo3ForCausalLM", "Phi3ForCausalLM", "GraniteForCausalLM")

_REGISTRY: dict[str, tuple[str, str]] = {a: ("dense", "DenseModel") for a in _DENSE}
_REGISTRY.update({
    "Qwen3MoeForCausalLM": ("moe", "MoeModel"),
    "DeepseekV2ForCausalLM": ("mla", "DeepseekV2Model"),
    "Glm4MoeLiteForCausalLM": ("mla", "DeepseekV2Model"),
    "Qwen3_5ForConditionalGeneration": ("gdn", "Qwen35Model"),
    "Qwen3_5MoeForConditionalGeneration": ("gdn", "Qwen35Model"),
    "Qwen3NextForCausalLM": ("gdn", "Qwen35Model"),
    "OPTForCausalLM": ("opt", "OPTModel"),
})


def supported_architectures() -> list[str]:
    return sorted(_REGISTRY)


def register_model(arch: str, module: str, cls: str) -> None:
    _REGISTRY[arch] = (module, cls)


def resolve(architectures) -> tuple[str, type]:
    """First supported architecture in ``architectures`` (a name or a list of names)."""
    import importlib
    names = [architectures] if isinstance(architectures, str) else list(architectures)
    for a in names:
        if a in _REGISTRY:
            mod, cls = _REGISTRY[a]
            m = importlib.import_module(f"vllm_cpp_b200.models.{mod}")
            return a, getattr(m, cls)
    raise ValueError(
        f"Model architectures {names} are not supported for now. Supported architectures: "
        f"{supported_architectures()}")
