"""zllm_b200: B200-native (sm_100a) GGUF block-quantized linear layer behind zLLM's backend operator surface."""
from .ffi import BF16, F16, F32, IQ4_NL, Q4_0, Q4_K, Q5_K, Q6_K, Q8_0, ZqFailure  # noqa: F401

__all__ = ["B200Context", "Weight", "Q4_0", "Q8_0", "Q4_K", "Q5_K", "Q6_K", "IQ4_NL", "F32", "F16", "BF16", "ZqFailure"]


def __getattr__(name):
    if name in ("B200Context", "Weight"):
        from . import backend

        return getattr(backend, name)
    raise AttributeError(name)
