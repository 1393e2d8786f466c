"""Import shim for the older package name of the reference's extension (its README still uninstalls
``FastAttention``; ``Cuda_Kernel/Custom_Kernel.py:2`` imports ``FastAttention2 as FastAttention``): the same module
as ``FastAttention2``."""
from cottention_transformer_b200 import kernel  # noqa: F401
