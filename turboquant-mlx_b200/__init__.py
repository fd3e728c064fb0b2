"""B200-native TurboQuant / PolarQuant KV-cache hot path: hand-written sm_100a
CUDA kernels in libtqb200.so behind the reference's Python names (reference
turboquant_mlx/__init__.py:1-24).  All tensors are CUDA `torch.Tensor`s."""

from .cache import TurboQuantKVCache
from .v_only_cache import VOnlyTurboQuantCache, v_only_attention
from .adaptive import make_adaptive_cache
from .patch import apply_patch, remove_patch
from .quantizer import PolarQuantizer
from .kernels import (
    fused_quantize,
    dequant_fp16,
    packed_dequantize,
    packed_fused_qk_scores,
    prerotate_query,
    prerot_fused_qk_scores,
    prerot_packed_dequantize,
    sparse_v_matvec,
    count_active_positions,
    flash_attention_turboquant,
    flash_decode,
    merge_partials,
    FlashDecodePlan,
    MergePlan,
    prefill_attention,
)
from .fused_attention import turboquant_attention
from .packing import pack_indices, unpack_indices, packed_dim
from .rotation import (
    walsh_hadamard_transform,
    randomized_hadamard_transform,
    inverse_randomized_hadamard,
    random_diagonal_sign,
)
from .base import KVCache, scaled_dot_product_attention
from .mixed_cache import MixedQuantKVCache
from .hybrid_cache import HybridQuantCache, hybrid_quantized_attention

__version__ = "0.5.0"
