"""kernel_collections_b200 — B200 (sm_100a) decode-attention kernels behind the entry-point
names of the xKV experiment repository: dense / factorized GQA decode, fused key
reconstruction with RoPE, split-KV flash decoding and MLA absorbed decode.

The work runs in libxkv.so (hand-written CUDA, C ABI in include/xkv.h); there is no CPU or
eager fallback — tensors must live on a CUDA device.
"""
from .attention import (  # noqa: F401
    group_query_attention,
    group_query_attention_fa,
    group_query_attention_sdpa,
    group_query_attentionv2,
    group_query_attention_factorized,
    group_query_attention_factorized_v_only,
    group_query_attention_factorized_RoPE,
    recon_rope_decode,
    rope_query,
    latent_append,
    xkv_group_decode,
    xkv_group_decode_v_only,
    mla_absorbed_decode,
)
from . import flash_recontruction, flash_decoding  # noqa: F401

__version__ = "0.1.0"
