"""Import shim: ``import FastAttention2`` / ``from FastAttention2 import kernel`` (the reference's
``Cuda_Kernel/Custom_Kernel.py:2-3``) resolve to the B200 implementation when the ``dropin``
directory is on ``sys.path`` in place of the reference's ``Cuda_Kernel``."""
from cottention_transformer_b200 import kernel  # noqa: F401
