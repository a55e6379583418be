"""Model families that exercise the library: the TP+SP Llama-3-shaped decoder stack and the MoE expert-parallel layer."""
from .llama import DecoderLayer, LlamaConfig, LlamaStack  # noqa: F401
