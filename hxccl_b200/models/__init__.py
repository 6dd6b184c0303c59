from .gpt2 import GPT2, GPT2Config  # noqa: F401
