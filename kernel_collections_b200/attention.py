"""Drop-in equivalents of the reference's eager decode functions (attention.py there).

Same names, argument order, shapes and return values; the work runs in libxkv's CUDA
kernels.  All functions are single decode steps (q_len == 1).  `attn_mask` is the reference's
additive mask (added to the scaled logits before the softmax, attention.py:60-64), any shape
that broadcasts to (bsz, num_kv_heads, group, 1, kv_len) / (bsz, num_heads, 1, kv_len); masked
calls run on the portable kernels.  `dropout_p` other than 0.0 raises NotImplementedError
(training-only; there is no CPU or eager fallback).

Keyword-only extras, defaulting to the reference's behaviour: `sm_scale` (multiplies the
logits), `theta`, `k_position_offset` (RoPE position of key row 0), `kv_lens` (int32 (bsz,)
device tensor: row b attends to its first kv_lens[b] cache rows only — ragged batches; the
reference's kernels take one length for the whole batch).
"""
from __future__ import annotations

import torch

from . import _C, ops


def _no_mask(attn_mask, dropout_p):
    if attn_mask is not None or dropout_p != 0.0:
        raise NotImplementedError("attn_mask / dropout are not supported by this entry point")


def _mask3(attn_mask, dropout_p, bsz, num_heads, num_kv_heads, kv_len):
    """The reference adds attn_mask to logits shaped (bsz, num_kv_heads, group, kv_len) (attention.py:63,
    q_len == 1 folded away); return it as something that broadcasts to (bsz, num_heads, kv_len)."""
    if dropout_p != 0.0:
        raise NotImplementedError("dropout is training-only and not supported by the decode kernels")
    if attn_mask is None:
        return None
    m = attn_mask
    G = num_heads // num_kv_heads
    if m.dim() == 5:                       # (bsz|1, kvh|1, G|1, 1, L)
        m = m.expand(m.shape[0], num_kv_heads, G, 1, m.shape[-1]).reshape(m.shape[0], num_heads, m.shape[-1])
    elif m.dim() == 4:                     # (bsz|1, heads|1, 1, L)
        m = m[:, :, 0, :]
    elif m.dim() == 2:                     # (q_len = 1, L)
        m = m[None]
    if m.dim() != 3:
        raise ValueError(f"unsupported attn_mask shape {tuple(attn_mask.shape)}")
    return m


def _q3(query):
    if query.dim() != 4:
        raise ValueError(f"query must be (bsz, num_heads, 1, head_dim); got {tuple(query.shape)}")
    if query.shape[2] != 1:
        raise AssertionError("q_len must be 1")
    return query[:, :, 0, :]


def group_query_attention(query, key, value, attn_mask=None, dropout_p=0.0, *, sm_scale=None, kv_lens=None):
    """Dense GQA decode.  Reference: attention.py:7-90.

    query (bsz, num_heads, 1, head_dim); key/value (bsz, num_kv_heads, kv_len, head_dim)
    -> (bsz, num_heads, 1, head_dim).  Logits are divided by sqrt(head_dim) as there."""
    bsz, num_heads, _, head_dim = query.shape
    mask = _mask3(attn_mask, dropout_p, bsz, num_heads, key.shape[1], key.shape[2])
    if key.shape[0] != bsz or value.shape[0] != bsz:
        raise AssertionError("Batch size mismatch among Q, K, V.")
    if key.shape[1] != value.shape[1]:
        raise AssertionError("num_kv_heads mismatch between K, V.")
    if key.shape[3] != head_dim or value.shape[3] != head_dim:
        raise AssertionError("head_dim mismatch among Q, K, V.")
    if key.shape[2] != value.shape[2]:
        raise AssertionError("kv_len mismatch between K, V.")
    if num_heads % key.shape[1] != 0:
        raise AssertionError("num_heads must be multiple of num_kv_heads.")
    scale = head_dim ** -0.5 if sm_scale is None else sm_scale
    o = ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE,
                   q=_q3(query), k=key.transpose(1, 2), v=value.transpose(1, 2), sm_scale=scale, kv_lens=kv_lens,
                   mask=mask)
    return o.unsqueeze(2)


def _fold_query_tokens(query, num_kv_heads):
    """(bsz, H, q_len, D) -> (bsz, H * q_len, 1, D): the q_len tokens of a head become q_len more heads of
    the same KV head (head h, token t -> row h * q_len + t, which keeps rows of one KV head together), so
    several query tokens ride on the M dimension of the same MMAs that serve the GQA group."""
    bsz, H, q_len, D = query.shape
    return query.reshape(bsz, H * q_len, 1, D)


def group_query_attentionv2(query, key, value, attn_mask=None, dropout_p=0.0, *, kv_lens=None):
    """The reference's second formulation (attention.py:93-182), which also takes q_len > 1 query
    tokens per sequence (speculative / multi-token decode): every query token attends to the whole
    cache, and `attn_mask` (additive, broadcastable to (bsz, num_kv_heads, group, q_len, kv_len) or
    (bsz, num_heads, q_len, kv_len)) carries any causal structure among the new tokens.  Returns
    (bsz, num_heads, q_len, head_dim).  The query tokens are folded into the head dimension, so they
    share one pass over K and V; up to 16 rows per KV head (group x q_len) stay on the tensor-core
    kernel, more run on the portable one."""
    if query.dim() != 4:
        raise ValueError(f"query must be (bsz, num_heads, q_len, head_dim); got {tuple(query.shape)}")
    bsz, H, q_len, D = query.shape
    if q_len == 1:
        return group_query_attention(query, key, value, attn_mask, dropout_p, kv_lens=kv_lens)
    KVH, L = key.shape[1], key.shape[2]
    if H % KVH != 0:
        raise AssertionError("num_heads must be multiple of num_kv_heads.")
    mask = None
    if attn_mask is not None:
        if dropout_p != 0.0:
            raise NotImplementedError("dropout is training-only and not supported by the decode kernels")
        m = attn_mask
        if m.dim() == 5:                   # (bsz|1, kvh|1, G|1, q_len|1, L)
            m = m.expand(m.shape[0], KVH, H // KVH, q_len, m.shape[-1]).reshape(m.shape[0], H * q_len, 1, m.shape[-1])
        elif m.dim() == 4:                 # (bsz|1, heads|1, q_len|1, L)
            m = m.expand(m.shape[0], H, q_len, m.shape[-1]).reshape(m.shape[0], H * q_len, 1, m.shape[-1])
        elif m.dim() == 2:                 # (q_len, L)
            m = m[None, None].expand(1, H, q_len, m.shape[-1]).reshape(1, H * q_len, 1, m.shape[-1])
        else:
            raise ValueError(f"unsupported attn_mask shape {tuple(attn_mask.shape)}")
        mask = m
    out = group_query_attention(_fold_query_tokens(query, KVH), key, value, mask, dropout_p, kv_lens=kv_lens)
    return out.reshape(bsz, H, q_len, D)


def group_query_attention_sdpa(query, key, value, attn_mask=None, dropout_p=0.0):
    """Reference: attention.py:193-200, F.scaled_dot_product_attention(..., enable_gqa=True): the same
    math with the default 1/sqrt(head_dim) scale and an additive float mask."""
    return group_query_attention(query, key, value, attn_mask, dropout_p)


def group_query_attention_fa(query, key, value, attn_mask=None, dropout_p=0.0):
    """Flash-decoding layout of the same op.  Reference: attention.py:184-191, which forwards to
    flash_attn_with_kvcache(q, k, v, causal=True): query (bsz, 1, num_heads, head_dim),
    key/value (bsz, kv_len, num_kv_heads, head_dim) -> (bsz, 1, num_heads, head_dim); the
    softmax scale is 1/sqrt(head_dim) and, with one query token, causal means "attend to all".
    The mask / dropout arguments are ignored there and here."""
    if query.dim() != 4 or query.shape[1] != 1:
        raise ValueError(f"query must be (bsz, 1, num_heads, head_dim); got {tuple(query.shape)}")
    o = ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE,
                   q=query[:, 0], k=key, v=value, sm_scale=query.shape[-1] ** -0.5)
    return o.unsqueeze(1)


def group_query_attention_factorized_v_only(query, key, value_A, value_B, attn_mask=None, dropout_p=0.0):
    """Dense K, V = value_A @ value_B.  Reference: attention.py:202-274.

    key (bsz, num_kv_heads, kv_len, head_dim); value_A (bsz, kv_len, v_rank);
    value_B (bsz, num_kv_heads, v_rank, head_dim)."""
    mask = _mask3(attn_mask, dropout_p, query.shape[0], query.shape[1], key.shape[1], key.shape[2])
    if value_A.shape[-1] != value_B.shape[2]:
        raise AssertionError("Rank mismatch between value_A and value_B")
    if query.shape[1] % key.shape[1] != 0:
        raise AssertionError("num_heads must be divisible by num_kv_heads")
    o = ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_LATENT,
                   q=_q3(query), k=key.transpose(1, 2), v=value_A, v_proj=value_B,
                   sm_scale=query.shape[-1] ** -0.5, mask=mask)
    return o.unsqueeze(2)


def group_query_attention_factorized(query, key_A, key_B, value_A, value_B, attn_mask=None,
                                     dropout_p=0.0, *, sm_scale=None, kv_lens=None):
    """K = key_A @ key_B, V = value_A @ value_B in absorbed form.  Reference: attention.py:276-357.

    key_A (bsz, kv_len, k_rank); key_B (bsz, num_kv_heads, k_rank, head_dim); value_A / value_B
    alike.  Logits are divided by sqrt(head_dim)."""
    mask = _mask3(attn_mask, dropout_p, query.shape[0], query.shape[1], key_B.shape[1], key_A.shape[1])
    if key_A.shape[-1] != key_B.shape[2]:
        raise AssertionError("Rank mismatch between key_A and key_B")
    if value_A.shape[-1] != value_B.shape[2]:
        raise AssertionError("Rank mismatch between value_A and value_B")
    if query.shape[1] % key_B.shape[1] != 0:
        raise AssertionError("num_heads must be divisible by num_kv_heads")
    scale = query.shape[-1] ** -0.5 if sm_scale is None else sm_scale
    o = ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT,
                   q=_q3(query), k=key_A, k_proj=key_B, v=value_A, v_proj=value_B, sm_scale=scale,
                   kv_lens=kv_lens, mask=mask)
    return o.unsqueeze(2)


def group_query_attention_factorized_RoPE(query, key_A, key_B, value_A, value_B, attn_mask=None,
                                          dropout_p=0.0, *, theta=10000000.0, sm_scale=1.0,
                                          k_position_offset=0):
    """Factorized K with RoPE applied to the rebuilt keys, factorized V.  Reference:
    attention.py:360-431 — logits q . RoPE_l(key_A[l] @ key_B) with theta 1e7 and NO 1/sqrt(d)
    scaling (:393-396), key position = row index, q used as given."""
    mask = _mask3(attn_mask, dropout_p, query.shape[0], query.shape[1], key_B.shape[1], key_A.shape[1])
    if key_A.shape[-1] != key_B.shape[2]:
        raise AssertionError("Rank mismatch between key_A and key_B")
    if value_A.shape[-1] != value_B.shape[2]:
        raise AssertionError("Rank mismatch between value_A and value_B")
    o = ops.decode(entry="xkv_recon_rope_decode", score_mode=_C.SCORE_RECON_ROPE,
                   value_mode=_C.VALUE_LATENT, q=_q3(query), k=key_A, k_proj=key_B, v=value_A,
                   v_proj=value_B, sm_scale=sm_scale, theta=theta, pos_offset=k_position_offset, mask=mask)
    return o.unsqueeze(2)


# ---- entry points the reference does not have but its benchmark configurations need -------------
def recon_rope_decode(query, key_A, key_B, value, value_B=None, *, theta, sm_scale=None,
                      k_position_offset=0, num_splits=0, force_generic=False, kv_lens=None, cta_pair=None,
                      pv_mma_sync=False, check_status=None):
    """Factorized K + RoPE with dense V (bsz, num_kv_heads, kv_len, head_dim), or factorized V
    when value_B is given (then `value` is the value latent).  key_B may be (bsz|1, num_kv_heads,
    k_rank, head_dim) or a shared (k_rank, num_kv_heads*head_dim) matrix.  Default scale
    1/sqrt(head_dim).  Per call this is attention.py:7-90 on K = RoPE(A.B)."""
    q = _q3(query)
    D = q.shape[-1]
    key_B = as_key_proj(key_B, D)
    scale = D ** -0.5 if sm_scale is None else sm_scale
    flags = 0
    if cta_pair is not None:     # None: the library chooses; True / False pin the CTA-pair or single-CTA kernel
        flags |= _C.FLAG_RECON_PAIR if cta_pair else _C.FLAG_RECON_SINGLE_CTA
    if pv_mma_sync:              # factorized values: second pass on the mma.sync kernel (cross-checks)
        flags |= _C.FLAG_PV_MMA_SYNC
    kw = dict(score_mode=_C.SCORE_RECON_ROPE, q=q, k=key_A, k_proj=key_B, sm_scale=scale, theta=theta,
              pos_offset=k_position_offset, num_splits=num_splits, force_generic=force_generic, kv_lens=kv_lens,
              extra_flags=flags, check_status=check_status)
    if value_B is None:
        o = ops.decode(entry="xkv_recon_rope_decode", value_mode=_C.VALUE_DENSE, v=value.transpose(1, 2), **kw)
    else:
        o = ops.decode(entry="xkv_recon_rope_decode", value_mode=_C.VALUE_LATENT, v=value,
                       v_proj=as_key_proj(value_B, D), **kw)
    return o.unsqueeze(2)


def as_key_proj(B, head_dim):
    """Accept the per-batch (bsz, KVH, R, D) form or a shared (R, KVH*D) matrix."""
    if B.dim() == 2:
        R = B.shape[0]
        return B.view(R, -1, head_dim).permute(1, 0, 2).unsqueeze(0)
    return B


def rope_query(query, theta, position, out=None):
    """Rotate a decode-step query (bsz, num_heads, 1, head_dim) to `position` (half-split RoPE,
    flash_recontruction/rope/rope_ref.py:11-21) with the library's kernel (xkv_rope_query).
    `position` is an int, or an int32 device tensor (bsz,) of per-sequence positions."""
    _C.require_cuda(query)
    q = query if query.stride(-1) == 1 else query.contiguous()
    if q.dim() != 4 or q.shape[2] != 1:
        raise ValueError(f"query must be (bsz, num_heads, 1, head_dim); got {tuple(query.shape)}")
    b, H, _, D = q.shape
    if out is None:
        out = torch.empty((b, H, 1, D), dtype=q.dtype, device=q.device)
    f = _C.inv_freq(D, theta, q.device)
    pos_t, pos_i = None, 0
    if isinstance(position, torch.Tensor):
        if position.dtype != torch.int32 or tuple(position.shape) != (b,) or not position.is_cuda:
            raise ValueError("per-sequence positions must be an int32 device tensor of shape (bsz,)")
        pos_t = position.contiguous()
    else:
        pos_i = int(position)
    with torch.cuda.device(q.device):
        rc = _C.load().xkv_rope_query(q.data_ptr(), out.data_ptr(), _C.dtype_code(q), b, H, D, q.stride(0), q.stride(1),
                                      out.stride(0), out.stride(1), pos_i, pos_t.data_ptr() if pos_t is not None else None,
                                      float(theta), f.data_ptr(), torch.cuda.current_stream(q.device).cuda_stream)
    _C.check(rc, "xkv_rope_query")
    return out


def latent_append(latent, new_rows, proj, position):
    """Append one token per sequence to a factorized cache, in place: latent[b, pos_b] = new_rows[b] @ proj.

    latent (bsz, capacity, rank) is the cache's A; new_rows (bsz, num_kv_heads * head_dim) the new key (or
    value) rows; proj (num_kv_heads * head_dim, rank) the map into latent space, i.e. the pseudo-inverse of
    the cache's (rank, num_kv_heads * head_dim) B matrix; `position` an int or an int32 device tensor
    (bsz,) — typically the kv_lens of the step before.  Returns `latent`."""
    _C.require_cuda(latent, new_rows, proj)
    if latent.dim() != 3 or new_rows.dim() != 2 or proj.dim() != 2:
        raise ValueError("latent (bsz, capacity, rank), new_rows (bsz, in_dim), proj (in_dim, rank) expected")
    b, cap, R = latent.shape
    if new_rows.shape[0] != b or proj.shape != (new_rows.shape[1], R):
        raise ValueError("shape mismatch among latent, new_rows and proj")
    if latent.stride(2) != 1 or not (latent.dtype == new_rows.dtype == proj.dtype):
        raise ValueError("latent needs a contiguous last dim and all tensors one dtype")
    x = new_rows if new_rows.stride(1) == 1 else new_rows.contiguous()
    pos_t, pos_i = None, 0
    if isinstance(position, torch.Tensor):
        if position.dtype != torch.int32 or tuple(position.shape) != (b,) or not position.is_cuda:
            raise ValueError("per-sequence positions must be an int32 device tensor of shape (bsz,)")
        pos_t = position.contiguous()
    else:
        pos_i = int(position)
    with torch.cuda.device(latent.device):
        rc = _C.load().xkv_latent_append(x.data_ptr(), x.stride(0), proj.data_ptr(), proj.stride(0), proj.stride(1),
                                         latent.data_ptr(), latent.stride(0), latent.stride(1),
                                         pos_t.data_ptr() if pos_t is not None else None, pos_i, _C.dtype_code(latent),
                                         b, x.shape[1], R, cap, torch.cuda.current_stream(latent.device).cuda_stream)
    _C.check(rc, "xkv_latent_append")
    return latent


def xkv_group_decode(queries, key_A, key_Bs, value, value_Bs=None, *, theta, sm_scale=None,
                     k_position_offset=0, kv_lens=None):
    """Cross-layer group: NL layers share key_A (and the value latent when value_Bs is given).

    queries: sequence of (bsz, H, 1, D); key_Bs: per-layer key projections; value: the shared
    value latent (bsz, L, Rv) with value_Bs, or a per-layer sequence of dense V
    (bsz, KVH, L, D).  Returns a list of (bsz, H, 1, D)."""
    D = queries[0].shape[-1]
    scale = D ** -0.5 if sm_scale is None else sm_scale
    layers = []
    for i, q in enumerate(queries):
        kw = dict(score_mode=_C.SCORE_RECON_ROPE, q=_q3(q), k=key_A, k_proj=as_key_proj(key_Bs[i], D),
                  sm_scale=scale, theta=theta, pos_offset=k_position_offset, kv_lens=kv_lens)
        if value_Bs is None:
            kw.update(value_mode=_C.VALUE_DENSE, v=value[i].transpose(1, 2))
        else:
            kw.update(value_mode=_C.VALUE_LATENT, v=value, v_proj=as_key_proj(value_Bs[i], D))
        layers.append(kw)
    return [o.unsqueeze(2) for o in ops.group_decode(layers)]


def xkv_group_decode_v_only(queries, keys, value_A, value_Bs, *, sm_scale=None, kv_lens=None):
    """Cross-layer group of the V-only-factorized form: every layer has its own dense keys
    (bsz, KVH, L, D) and value projection, all layers share one value latent value_A (bsz, L, Rv).  Per
    layer this is attention.py:202-274; as a group the shared latent is streamed ONCE, with the heads of
    all layers stacked for the softmax + P.A_v pass.  Returns a list of (bsz, H, 1, D)."""
    D = queries[0].shape[-1]
    scale = D ** -0.5 if sm_scale is None else sm_scale
    layers = [dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_LATENT, q=_q3(q), k=keys[i].transpose(1, 2), v=value_A,
                   v_proj=as_key_proj(value_Bs[i], D), sm_scale=scale, kv_lens=kv_lens) for i, q in enumerate(queries)]
    return [o.unsqueeze(2) for o in ops.group_decode(layers)]


def mla_absorbed_decode(q_nope, q_rope, c_kv, k_rope, W_uk, W_uv, sm_scale, *, kv_lens=None):
    """MLA absorbed decode.  q_nope (b,H,nope); q_rope (b,H,rope); c_kv (b,L,lora);
    k_rope (b,L,rope); W_uk (H,nope,lora); W_uv (H,lora,v) -> (b,H,v).  W_uk is folded into q,
    the latent is streamed once for both logits and values, W_uv is applied after the merge.
    The attention core is flash_decoding/mla2/mla_flash_decoding.py:6-62."""
    kp = W_uk.permute(0, 2, 1).unsqueeze(0)      # (1, H, lora, nope): element [h, r, d] = W_uk[h, d, r]
    vp = W_uv.unsqueeze(0)                       # (1, H, lora, v)
    return ops.decode(entry="xkv_mla_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT,
                      q=q_nope, k=c_kv, k_proj=kp, v=c_kv, v_proj=vp, q_tail=q_rope, k_tail=k_rope,
                      sm_scale=sm_scale, num_kv_heads=1, kv_lens=kv_lens)
