"""B200-native kernels for the rollout-forward hot path of verl-project/vexact.

Public surface (same names as `vexact.batch_invariant_ops`):
    enable_batch_invariant_mode, disable_batch_invariant_mode, set_batch_invariant_mode,
    is_batch_invariant_mode_enabled, matmul_persistent, log_softmax, mean_dim, triton_bmm,
    batch_invariant_rms_norm, get_batch_invariant_attention_block_size, AttentionBlockSize,
    flash_attention_forward, flash_attention_forward_cute, triton_flash_attention_forward,
    triton_flash_attn_varlen_func
plus store_kvcache / set_kv_cache_context, fused_moe_forward and
logprobs_from_logits_flash_attn from the sibling modules of the reference package.
"""
from .batch_invariant_ops import (  # noqa: F401
    AttentionBlockSize,
    add_rms_norm,
    batch_invariant_rms_norm,
    disable_batch_invariant_mode,
    enable_batch_invariant_mode,
    get_batch_invariant_attention_block_size,
    hf_rms_norm,
    is_batch_invariant_mode_enabled,
    linear,
    log_softmax,
    matmul_persistent,
    mean_dim,
    set_batch_invariant_mode,
    triton_bmm,
)
from .attention import flash_attention_forward, flash_attn_varlen_func, paged_attention  # noqa: F401
from .attention import flash_attention_forward as flash_attention_forward_cute  # noqa: F401
from .attention import flash_attention_forward as triton_flash_attention_forward  # noqa: F401
from .attention import flex_attention_forward  # noqa: F401
from .attention import flash_attn_varlen_func as triton_flash_attn_varlen_func  # noqa: F401
from .fused_moe import fused_moe_forward, route_sigmoid_group_topk, route_softmax_topk  # noqa: F401
from .kv_cache_context import (  # noqa: F401
    KVCacheContext,
    KVCacheManager,
    KVCacheStore,
    get_kv_cache_context,
    set_kv_cache_context,
    store_kvcache,
)
from .standalone_logprobs import logprobs_from_logits_flash_attn  # noqa: F401

__version__ = "0.1.0"
