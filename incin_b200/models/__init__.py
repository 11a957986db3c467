"""Model families built on the op surface: GPT-2 (pre-LN, GELU) and Llama (RMSNorm, RoPE, GQA, SwiGLU), MLP."""
from .gpt2 import GPT2, GPT2Config  # noqa: F401
