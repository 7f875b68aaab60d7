"""gemm_b200 — a Blackwell-native (B200, sm_100a) LLM / MoE inference framework.

Layout:  ``ops`` (CUDA kernels + PyTorch references), ``models`` (Qwen2/3 dense, Qwen3-MoE, Qwen3.5 hybrid),
``parallel`` (TP / EP / PP / DP groups and the NVLink fabric), ``utils`` (GGUF / safetensors / tokenizer / profiler /
checkpoints), ``serve`` (engine, scheduler, HTTP front end).
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "LLM":
        from .serve.llm import LLM
        return LLM
    if name == "SamplingParams":
        from .serve.engine import SamplingParams
        return SamplingParams
    if name == "Engine":
        from .serve.engine import Engine
        return Engine
    raise AttributeError(name)
