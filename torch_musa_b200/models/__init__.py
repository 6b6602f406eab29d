"""Reference model families used by the benchmarks and tests: Llama-style decoder, Mixtral-style MoE
decoder and ResNet-50, written against stock ``torch.nn`` plus the backend's fused operators."""
from .llama import LlamaConfig, Llama, llama_7b_config, llama_tiny_config  # noqa: F401
