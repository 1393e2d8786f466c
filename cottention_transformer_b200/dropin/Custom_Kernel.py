"""Import shim: ``from Custom_Kernel import CustomAttention`` (the reference's
``GPT_Trainer/GPTCosAttention.py:17-18``) resolves to the B200 implementation."""
from cottention_transformer_b200.custom_kernel import CustomAttention  # noqa: F401
