"""Drop-in names of the reference's `flash_recontruction` package (spelling kept):
fused key reconstruction q . (A @ B)^T with and without RoPE, and the fused xKV decode
attention over factorized K / V.  Reference: flash_recontruction/__init__.py:1-35."""
from __future__ import annotations

import torch

from .. import _C, ops

__all__ = [
    "qAB_no_pe_v1", "qAB_no_pe_v2", "qAB_no_pe_ref",
    "qAB_rope_v1", "qAB_rope_v2", "qAB_rope_v3", "qAB_rope_v4",
    "gqa_xKV_no_pe_ref", "gqa_xKV_no_pe_k_only_ref", "gqa_xKV_no_pe_k_only",
    "gqa_xKV_no_pe", "gqa_xKV_no_pe_v2",
]


def _check_qab(q, Ak, Bk):
    assert q.dim() == 4, f"Expected q to be 4D, got {q.dim()}D"
    assert Ak.dim() == 3, f"Expected Ak to be 3D, got {Ak.dim()}D"
    assert Bk.dim() == 4, f"Expected Bk to be 4D, got {Bk.dim()}D"
    assert q.shape[0] == Ak.shape[0] == Bk.shape[0], "Batch size mismatch"
    assert Ak.shape[2] == Bk.shape[2], "Rank mismatch"
    assert q.shape[3] == Bk.shape[3], "Head dimension mismatch"
    assert q.shape[2] == 1, "Only supporting q_len=1 for now"
    assert q.shape[1] % Bk.shape[1] == 0, "num_heads must be divisible by num_kv_heads"


def _qab_no_pe(q: torch.Tensor, Ak: torch.Tensor, Bk: torch.Tensor) -> torch.Tensor:
    """Unscaled logits q . (Ak @ Bk)^T, (bsz, num_heads, 1, kv_len).  Without RoPE the product
    is evaluated in absorbed order ((q . Bk^T) . Ak^T): the rebuilt K never exists and the latent
    is streamed once.  Reference: flash_recontruction/qAB_no_pe/v1.py:78-135, v2.py:72-130,
    ref.py:4-26."""
    _check_qab(q, Ak, Bk)
    out = ops.decode(entry="xkv_qab_logits", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_DENSE,
                     q=q[:, :, 0, :], k=Ak, k_proj=Bk, logits_only=True, sm_scale=1.0)
    return out.unsqueeze(2)


qAB_no_pe_v1 = _qab_no_pe
qAB_no_pe_v2 = _qab_no_pe
qAB_no_pe_ref = _qab_no_pe


def _qab_rope(q: torch.Tensor, Ak: torch.Tensor, Bk: torch.Tensor, theta: float = 10000000.0) -> torch.Tensor:
    """Unscaled logits q . RoPE_l(Ak[l] @ Bk)^T, (bsz, num_heads, 1, kv_len); key position is
    the row index, q is used as given (the caller rotates it).  The four reference variants
    differ only in loop order / accumulator type and share one kernel here.  Reference:
    flash_recontruction/qAB/v1.py:90-148, v3.py:84-142, v4.py:85-143."""
    _check_qab(q, Ak, Bk)
    out = ops.decode(entry="xkv_qab_logits", score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE,
                     q=q[:, :, 0, :], k=Ak, k_proj=Bk, logits_only=True, sm_scale=1.0, theta=theta)
    return out.unsqueeze(2)


qAB_rope_v1 = _qab_rope
qAB_rope_v3 = _qab_rope
qAB_rope_v4 = _qab_rope


def qAB_rope_v2(q: torch.Tensor, Ak: torch.Tensor, Bk: torch.Tensor, sin_cos: torch.Tensor) -> torch.Tensor:
    """As qAB_rope_v1 with a caller-made table sin_cos (kv_len, head_dim): [:, :D/2] = sin,
    [:, D/2:] = cos.  Reference: flash_recontruction/qAB/v2.py:132-187."""
    _check_qab(q, Ak, Bk)
    L, D = Ak.shape[1], q.shape[3]
    if tuple(sin_cos.shape) != (L, D):
        raise ValueError(f"sin_cos must be (kv_len, head_dim) = ({L}, {D}); got {tuple(sin_cos.shape)}")
    half = D // 2
    table = torch.stack((sin_cos[:, half:], sin_cos[:, :half]), dim=-1).float().contiguous()
    out = ops.decode(entry="xkv_qab_logits", score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE,
                     q=q[:, :, 0, :], k=Ak, k_proj=Bk, logits_only=True, sm_scale=1.0, rope_table=table)
    return out.unsqueeze(2)


def _check_splits(q, num_kv_splits, max_kv_splits):
    if num_kv_splits is not None:
        if num_kv_splits.dim() != 1 or num_kv_splits.shape[0] != q.shape[0]:
            raise ValueError("num_kv_splits must have shape (batch,)")
    if int(max_kv_splits) <= 0:
        raise ValueError("max_kv_splits must be positive")
    return int(max_kv_splits)


def gqa_xKV_no_pe(q, k_A_buffer, k_B_buffer, v_A_buffer, v_B_buffer, o, num_kv_splits, max_kv_splits,
                  sm_scale=1.0):
    """Fused decode over factorized K and V; fills and returns `o` (batch, num_q_heads, head_dim).
    The split counts are accepted as a hint; the split geometry is chosen from the SM count.
    Reference: flash_recontruction/fused_attention/no_pe/v1.py:365-474."""
    hint = _check_splits(q, num_kv_splits, max_kv_splits)
    return ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT,
                      q=q, k=k_A_buffer, k_proj=k_B_buffer, v=v_A_buffer, v_proj=v_B_buffer, out=o,
                      sm_scale=sm_scale, num_splits=hint)


def gqa_xKV_no_pe_v2(q, k_A_buffer, k_B_buffer, v_A_buffer, v_B_buffer, num_kv_splits, max_kv_splits,
                     sm_scale=1.0):
    """As gqa_xKV_no_pe but allocates and returns the output (the splits are merged in rank space
    and B_v is applied once).  Reference: fused_attention/no_pe/v2.py:364-474."""
    hint = _check_splits(q, num_kv_splits, max_kv_splits)
    return ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT,
                      q=q, k=k_A_buffer, k_proj=k_B_buffer, v=v_A_buffer, v_proj=v_B_buffer,
                      sm_scale=sm_scale, num_splits=hint)


def gqa_xKV_no_pe_k_only(q, k_A_buffer, k_B_buffer, v_buffer, o, num_kv_splits, max_kv_splits, sm_scale=1.0):
    """Factorized K, dense V (batch, kv_len, num_kv_heads, head_dim); fills and returns `o`.
    Reference: fused_attention/no_pe/v1_k_only.py:368-465."""
    hint = _check_splits(q, num_kv_splits, max_kv_splits)
    return ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_DENSE,
                      q=q, k=k_A_buffer, k_proj=k_B_buffer, v=v_buffer, out=o, sm_scale=sm_scale,
                      num_splits=hint)


def gqa_xKV_no_pe_ref(query, key_A, key_B, value_A, value_B, attn_mask=None, dropout_p=0.0):
    """Unscaled factorized decode, q (bsz, num_heads, head_dim).  Reference:
    fused_attention/no_pe/ref.py:4-87 (an eager function there; the same kernels here)."""
    if attn_mask is not None or dropout_p != 0.0:
        raise NotImplementedError("attn_mask / dropout are not supported by the decode kernels")
    return ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT,
                      q=query, k=key_A, k_proj=key_B, v=value_A, v_proj=value_B, sm_scale=1.0)


def gqa_xKV_no_pe_k_only_ref(query, key_A, key_B, value, attn_mask=None, dropout_p=0.0):
    """Unscaled factorized-K / dense-V decode.  Reference: fused_attention/no_pe/ref.py:92-161."""
    if attn_mask is not None or dropout_p != 0.0:
        raise NotImplementedError("attn_mask / dropout are not supported by the decode kernels")
    return ops.decode(entry="xkv_absorbed_decode", score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_DENSE,
                      q=query, k=key_A, k_proj=key_B, v=value, sm_scale=1.0)
