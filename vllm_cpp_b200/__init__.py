"""B200-native LLM inference engine (sm_100a kernels + C++ host runtime + torch.distributed)."""
__version__ = "0.1.0"
