"""MLA decode with separate latent and RoPE tensors; the output stays in latent space.
Reference: flash_decoding/mla2/__init__.py:1, mla_flash_decoding.py, ref.py."""
from __future__ import annotations

from ... import _C, ops

__all__ = ["mla_decode_attention_fwd", "mla_decode_attention_fwd_ref", "mla_decode_attention_xKV"]


def _core(q_nope, q_rope, kv_nope, k_rope, scale, k_proj=None, v_proj=None):
    assert kv_nope.shape[2] == 1 and k_rope.shape[2] == 1
    return ops.decode(entry="xkv_mla_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT,
                      q=q_nope, k=kv_nope[:, :, 0, :], v=kv_nope[:, :, 0, :], q_tail=q_rope,
                      k_tail=k_rope[:, :, 0, :], k_proj=k_proj, v_proj=v_proj, sm_scale=scale,
                      num_kv_heads=1)


def mla_decode_attention_fwd(q_nope, q_rope, kv_nope, k_rope, sm_scale=1.0):
    """softmax((q_nope . c^T + q_rope . k_rope^T) * sm_scale) . c -> (batch, num_q_heads, lora_rank).
    q_nope (batch, H, lora_rank) already absorbed; kv_nope (batch, kv_len, 1, lora_rank);
    k_rope (batch, kv_len, 1, rope_dim).  The latent is read once for logits and values.
    Reference: flash_decoding/mla2/mla_flash_decoding.py:6-62."""
    return _core(q_nope, q_rope, kv_nope, k_rope, sm_scale)


def mla_decode_attention_fwd_ref(q_nope, q_rope, kv_nope, k_rope, sm_scale=1.0):
    """The reference's eager check function, which DIVIDES by sm_scale (mla2/ref.py:28)."""
    return _core(q_nope, q_rope, kv_nope, k_rope, 1.0 / sm_scale)


def mla_decode_attention_xKV(q_nope, q_rope, kv_A_nope, kv_B_nope, k_rope, sm_scale=1.0):
    """The MLA latent itself factorized, c = kv_A @ kv_B: kv_A_nope (batch, kv_len, 1, rank),
    kv_B_nope (batch, 1, rank, lora_rank).  kv_B is folded into q before and applied to the
    output after the split-KV pass.  Reference: mla2/mla_flash_decoding.py:66-130."""
    assert kv_A_nope.shape[2] == 1
    assert kv_B_nope.shape[1] == 1
    return _core(q_nope, q_rope, kv_A_nope, k_rope, sm_scale, k_proj=kv_B_nope, v_proj=kv_B_nope)
