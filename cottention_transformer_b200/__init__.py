"""cottention_transformer_b200: B200 (sm_100a) kernels for Cottention's cosine linear attention,
behind the reference's own extension API (``FastAttention2.kernel`` / ``CustomAttention``)."""
from . import _lib, kernel  # noqa: F401
from .custom_kernel import CustomAttention  # noqa: F401
from .cos_attention import (cos_attn_bidirectional, cos_attn_bidirectional_packed, cos_attn_causal,  # noqa: F401
                            cos_attn_causal_packed, rotary_packed_)
from .decode import CosAttnDecodeState  # noqa: F401

__version__ = "0.1.0"
