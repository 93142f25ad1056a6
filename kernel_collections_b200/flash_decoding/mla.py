"""Split-KV decode attention over a packed MLA cache (keys carry a RoPE tail; values are a
prefix of the keys or a separate buffer).  Reference: flash_decoding/mla.py."""
from __future__ import annotations

from .. import _C, ops


def decode_attention_fwd(q, k_buffer, v_buffer, o, sm_scale=1.0, logit_cap=0.0):
    """q (batch, num_q_heads, Dk); k_buffer (batch, kv_len, num_kv_heads, Dk), e.g. Dk = 576 =
    512 latent + 64 rope; v_buffer (batch, kv_len, num_kv_heads, Dv); o (batch, num_q_heads, Dv)
    is filled in place and nothing is returned, as in the reference.  Logits are multiplied by
    sm_scale; logit_cap > 0 applies cap * tanh(x / cap).  Reference: flash_decoding/mla.py:388-440."""
    assert q.shape[1] // k_buffer.shape[2] >= 1
    ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE,
               q=q, k=k_buffer, v=v_buffer, out=o, sm_scale=sm_scale, logit_cap=logit_cap)


def decode_attention_reference(q, k_buffer, v_buffer, o, sm_scale):
    """The reference's eager check function (flash_decoding/mla.py:442-471): it DIVIDES the
    logits by sm_scale and returns a new tensor.  Kept under its name with that convention."""
    return ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE,
                      q=q, k=k_buffer, v=v_buffer, sm_scale=1.0 / sm_scale)
