"""Split-KV decode attention over a dense GQA cache.  Reference: flash_decoding/gqa.py."""
from __future__ import annotations

from .. import _C, ops


def decode_attention_fwd(q, k_buffer, v_buffer, o, num_kv_splits, max_kv_splits, sm_scale=1.0):
    """q, o (batch, num_q_heads, head_dim); k_buffer / v_buffer (batch, kv_len, num_kv_heads,
    head_dim); logits are MULTIPLIED by sm_scale.  Fills and returns `o`.  num_kv_splits (int32
    (batch,)) and max_kv_splits are validated and used as a hint only.
    Reference: flash_decoding/gqa.py:339-434."""
    if num_kv_splits is not None and (num_kv_splits.dim() != 1 or num_kv_splits.shape[0] != q.shape[0]):
        raise ValueError("num_kv_splits must have shape (batch,)")
    if int(max_kv_splits) <= 0:
        raise ValueError("max_kv_splits must be positive")
    assert q.shape[1] // v_buffer.shape[2] >= 1
    return ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE,
                      q=q, k=k_buffer, v=v_buffer, out=o, sm_scale=sm_scale, num_splits=int(max_kv_splits))
