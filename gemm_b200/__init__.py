"""gemm_b200 — a Blackwell-native (B200, sm_100a) LLM / MoE inference framework.

Layout:  ``ops`` (CUDA kernels + PyTorch references), ``models`` (Qwen2/3 dense, Qwen3-MoE, Qwen3.5 hybrid),
``parallel`` (TP / EP / PP / DP groups and the NVLink fabric), ``utils`` (GGUF / safetensors / tokenizer / profiler /
checkpoints), ``serve`` (engine, scheduler, HTTP front end).
"""
__version__ = "0.1.0"
