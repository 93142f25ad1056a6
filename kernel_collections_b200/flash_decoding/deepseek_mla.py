"""Decode over prefill / decode-separated buffers: a long prefill cache (dense, or factorized with
the projections absorbed) plus a short dense buffer of freshly decoded tokens.  Each part is one
decode call that also returns its log-sum-exp; the parts are then merged exactly.

Reference: flash_decoding/deepseek_mla/flash_decoding.py:66-255 (`mla_decode_attention_fwd_pd_sep`,
`mla_decode_attention_fwd_pd_sep_xKV`).  There the partial buffers of the two parts are concatenated
and stage 2 re-derives which splits are valid from the MERGED length, which can drop trailing
partials that hold real data; here validity travels with each part's own log-sum-exp."""
from __future__ import annotations

from .. import _C, ops


def _part(q, k_buffer, v_buffer, sm_scale, logit_cap=0.0):
    return ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=q,
                      k=k_buffer, v=v_buffer, sm_scale=sm_scale, logit_cap=logit_cap, return_lse=True)


def mla_decode_attention_fwd_pd_sep(q, k_buffer, v_buffer, k_buffer_decoded, v_buffer_decoded, sm_scale=1.0,
                                    logit_cap=0.0):
    """q (batch, num_q_heads, head_dim); prefill K/V (batch, prefill_kv_len, num_kv_heads, head_dim | v_dim);
    decoded K/V (batch, decode_kv_len, num_kv_heads, ...).  Logits are multiplied by sm_scale.  Returns
    (batch, num_q_heads, v_dim).  Reference: deepseek_mla/flash_decoding.py:66-157."""
    o1, l1 = _part(q, k_buffer, v_buffer, sm_scale, logit_cap)
    o2, l2 = _part(q, k_buffer_decoded, v_buffer_decoded, sm_scale, logit_cap)
    return ops.merge_segments([o1, o2], [l1, l2])


def mla_decode_attention_fwd_pd_sep_xKV(q, k_A_buffer, k_B_buffer, v_A_buffer, v_B_buffer, k_buffer_decoded,
                                        v_buffer_decoded, sm_scale=1.0):
    """Prefill cache factorized (k_A (batch, prefill_kv_len, rank), k_B (batch, num_kv_heads, rank, head_dim),
    likewise v_A / v_B), decoded tokens dense.  The projections are absorbed: q.k_B^T before and .v_B after
    the latent pass.  Reference: deepseek_mla/flash_decoding.py:160-254."""
    o1, l1 = ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=q,
                        k=k_A_buffer, k_proj=k_B_buffer, v=v_A_buffer, v_proj=v_B_buffer, sm_scale=sm_scale,
                        return_lse=True)
    o2, l2 = _part(q, k_buffer_decoded, v_buffer_decoded, sm_scale)
    return ops.merge_segments([o1, o2], [l1, l2])
