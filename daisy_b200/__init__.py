"""daisy_b200 -- the Daisy attention hot path on B200 (sm_100a): windowed prefill, ring-cache decode
and KDA, as hand-written CUDA behind the reference's CausalSelfAttention / KVCache / chunk_kda API."""
from .attention import (B200CausalSelfAttention, WindowMask, BlockWindowMask, Rotary,   # noqa: F401
                        create_blockmasks, doc_starts)
from .kv_cache import B200KVCache, ring_segment                       # noqa: F401
from .generate import StepRunner                                      # noqa: F401
from .kda import B200KimiLinearSelfAttention, B200ShortConvolution, B200FusedRMSNormGated   # noqa: F401
from . import ops                                                      # noqa: F401
from .autograd import swa_attention                                   # noqa: F401

__all__ = ["B200CausalSelfAttention", "B200KVCache", "WindowMask", "BlockWindowMask", "create_blockmasks", "doc_starts",
           "Rotary", "ring_segment", "StepRunner", "B200KimiLinearSelfAttention", "B200ShortConvolution",
           "B200FusedRMSNormGated", "ops", "swa_attention"]
