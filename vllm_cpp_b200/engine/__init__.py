from .llm import LLM, CompletionOutput, RequestOutput, SamplingParams  # noqa: F401
