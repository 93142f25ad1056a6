"""CPU oracle for the xKV decode-attention path.  TEST INFRASTRUCTURE ONLY.

A plain-PyTorch (CPU, eager) restatement of the reference's eager decode
functions.  Every function names the reference file:line it follows.  It is
imported by tests/, by the smoke check and by the bench's CPU-baseline leg
only; nothing in the product package may import it.

Parity status: PINNED.  tests/golden/*.npz were produced by importing the
reference's own eager functions (tests/golden/make_golden.py) and
tests/test_oracle_golden.py checks every function here against them.

Conventions (the reference's):
  * single decode step, q_len == 1
  * softmax in fp32, probabilities cast back to the working dtype before P.V
    (attention.py:68,247,330)
  * RoPE is the half-split "rotate_half" form with pairs (j, j + D/2) and
    angle = float32(pos) * float32(theta ** (-2j/D))   (rope/rope_ref.py:3-21)
  * scale conventions differ per entry point: eager GQA divides logits by
    sqrt(D); the fused / flash entry points multiply by a caller sm_scale.

``compute_dtype`` is the dtype every matmul runs in.  The primary oracle is
fp32 on the (already dtype-rounded) inputs; passing the tensors' own dtype
replays the reference's native rounding.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _up(x, dt):
    return x if x is None or x.dtype == dt else x.to(dt)


# --------------------------------------------------------------------------- RoPE
def rope_cos_sin(dim: int, end: int, theta: float = 10000.0):
    """cos/sin tables of shape (end, dim), fp32.  flash_recontruction/rope/rope_ref.py:3-9."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    t = torch.arange(end, dtype=torch.int64).type_as(inv_freq)
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x):
    """flash_recontruction/rope/rope_ref.py:11-15."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x, cos, sin):
    """x * cos + rotate_half(x) * sin, broadcast over leading dims.  rope_ref.py:17-21."""
    return x * cos + rotate_half(x) * sin


# --------------------------------------------------------------------------- core
def _softmax_pv(logits, value, work_dtype):
    """fp32 softmax, cast to the working dtype, then P.V.  attention.py:66-79."""
    p = F.softmax(logits, dim=-1, dtype=torch.float32).to(work_dtype)
    return torch.matmul(p, value)


def gqa_dense(query, key, value, compute_dtype=torch.float32, scale=None):
    """Dense GQA decode.  attention.py:7-90.

    query (b,H,1,D); key/value (b,KVH,L,D) -> (b,H,1,D).  ``scale`` multiplies
    the logits; None means the reference default 1/sqrt(D).
    """
    b, H, q_len, D = query.shape
    _, KVH, L, _ = key.shape
    assert q_len == 1 and H % KVH == 0
    G = H // KVH
    q = _up(query, compute_dtype).reshape(b, KVH, G, D)
    k = _up(key, compute_dtype)
    v = _up(value, compute_dtype)
    s = torch.matmul(q, k.transpose(-1, -2))
    s = s / (D ** 0.5) if scale is None else s * scale
    o = _softmax_pv(s, v, compute_dtype)
    return o.reshape(b, H, 1, D)


def gqa_dense_multi(query, key, value, attn_mask=None, compute_dtype=torch.float32):
    """Dense GQA with q_len >= 1 query tokens per sequence and an optional additive mask
    broadcastable to (b, KVH, G, q_len, L).  attention.py:93-182 (group_query_attentionv2)."""
    b, H, q_len, D = query.shape
    _, KVH, L, _ = key.shape
    G = H // KVH
    q = _up(query, compute_dtype).reshape(b, KVH, G, q_len, D)
    k = _up(key, compute_dtype).unsqueeze(2)
    v = _up(value, compute_dtype).unsqueeze(2)
    s = torch.matmul(q, k.transpose(-1, -2)) / (D ** 0.5)
    if attn_mask is not None:
        s = s + attn_mask.to(s.dtype)
    p = F.softmax(s, dim=-1, dtype=torch.float32).to(compute_dtype)
    return torch.matmul(p, v).reshape(b, H, q_len, D)


def gqa_factorized_v_only(query, key, value_A, value_B, compute_dtype=torch.float32):
    """Dense K, V = value_A @ value_B.  attention.py:202-274."""
    b, H, q_len, D = query.shape
    _, KVH, L, _ = key.shape
    Rv = value_A.shape[-1]
    assert q_len == 1 and H % KVH == 0 and value_B.shape[2] == Rv
    G = H // KVH
    q = _up(query, compute_dtype).reshape(b, KVH, G, D)
    s = torch.matmul(q, _up(key, compute_dtype).transpose(-1, -2)) / (D ** 0.5)
    p = F.softmax(s, dim=-1, dtype=torch.float32).to(compute_dtype)
    t = torch.matmul(p.reshape(b, H, L), _up(value_A, compute_dtype))          # (b,H,Rv)
    o = torch.matmul(t.reshape(b, KVH, G, Rv), _up(value_B, compute_dtype))    # (b,KVH,G,D)
    return o.reshape(b, H, 1, D)


def gqa_factorized(query, key_A, key_B, value_A, value_B, compute_dtype=torch.float32,
                   scale=None):
    """K = key_A @ key_B, V = value_A @ value_B, absorbed form.  attention.py:276-357.

    ``scale=None`` is the reference default 1/sqrt(D); the fused kernels'
    eager reference (fused_attention/no_pe/ref.py:4-87) is the same math with
    scale = 1.
    """
    b, H, q_len, D = query.shape
    _, L, Rk = key_A.shape
    KVH = key_B.shape[1]
    Rv = value_A.shape[-1]
    assert q_len == 1 and H % KVH == 0
    G = H // KVH
    q = _up(query, compute_dtype).reshape(b, KVH, G, D)
    lat = torch.matmul(q, _up(key_B, compute_dtype).transpose(-1, -2)).reshape(b, H, Rk)
    s = torch.matmul(lat, _up(key_A, compute_dtype).transpose(-1, -2))          # (b,H,L)
    s = s / (D ** 0.5) if scale is None else s * scale
    p = F.softmax(s, dim=-1, dtype=torch.float32).to(compute_dtype)
    t = torch.matmul(p, _up(value_A, compute_dtype))                            # (b,H,Rv)
    o = torch.matmul(t.reshape(b, KVH, G, Rv), _up(value_B, compute_dtype))
    return o.reshape(b, H, 1, D)


def qab_no_pe(q, Ak, Bk, compute_dtype=torch.float32):
    """Unscaled logits q . (Ak @ Bk)^T -> (b,H,1,L).  flash_recontruction/qAB_no_pe/ref.py:4-26."""
    b, H, q_len, D = q.shape
    _, L, R = Ak.shape
    KVH = Bk.shape[1]
    G = H // KVH
    qq = _up(q, compute_dtype).reshape(b, KVH, G * q_len, D)
    K = torch.matmul(_up(Ak, compute_dtype).unsqueeze(1), _up(Bk, compute_dtype))
    out = torch.matmul(qq, K.transpose(-1, -2))
    return out.reshape(b, H, q_len, L)


def reconstruct_rope_keys(Ak, Bk, theta, compute_dtype=torch.float32, position_offset=0):
    """K = RoPE_l(Ak[l] @ Bk), key position = row index.  test_qAB_rope.py:29-36 with the
    rotary tables of rope/rope_ref.py in place of the HF module (same formula)."""
    b, L, R = Ak.shape
    D = Bk.shape[-1]
    K = torch.matmul(_up(Ak, compute_dtype).unsqueeze(1), _up(Bk, compute_dtype))   # (b,KVH,L,D)
    cos, sin = rope_cos_sin(D, L + position_offset, theta)
    cos = cos[position_offset:].to(compute_dtype)
    sin = sin[position_offset:].to(compute_dtype)
    return apply_rope(K, cos, sin)


def qab_rope(q_pe, Ak, Bk, theta=10000000.0, compute_dtype=torch.float32):
    """Unscaled logits q_pe . RoPE(Ak @ Bk)^T -> (b,H,1,L); q is used as given.
    test_qAB_rope.py:19-43 (qAB_rope_ref)."""
    b, H, q_len, D = q_pe.shape
    KVH = Bk.shape[1]
    G = H // KVH
    L = Ak.shape[1]
    K = reconstruct_rope_keys(Ak, Bk, theta, compute_dtype)
    qq = _up(q_pe, compute_dtype).reshape(b, KVH, G * q_len, D)
    out = torch.matmul(qq, K.transpose(-1, -2))
    return out.reshape(b, H, q_len, L)


def gqa_factorized_rope(query, key_A, key_B, value_A, value_B, theta=10000000.0,
                        compute_dtype=torch.float32):
    """attention.py:360-431: logits from the RoPE qAB op, NOT scaled (:396), then the
    factorized P.V of :404-429."""
    b, H, q_len, D = query.shape
    KVH = key_B.shape[1]
    G = H // KVH
    Rv = value_A.shape[-1]
    s = qab_rope(query, key_A, key_B, theta, compute_dtype)                    # (b,H,1,L)
    p = F.softmax(s, dim=-1, dtype=torch.float32).to(compute_dtype)
    L = s.shape[-1]
    t = torch.matmul(p.reshape(b, H, L), _up(value_A, compute_dtype))
    o = torch.matmul(t.reshape(b, KVH, G, Rv), _up(value_B, compute_dtype))
    return o.reshape(b, H, 1, D)


def xkv_fused(query, key_A, key_B, value_A, value_B, sm_scale=1.0, compute_dtype=torch.float32):
    """q 3-D (b,H,D); factorized K and V; logits multiplied by sm_scale (the kernels'
    convention).  flash_recontruction/fused_attention/no_pe/ref.py:4-87 (which is scale 1)."""
    o = gqa_factorized(query.unsqueeze(2), key_A, key_B, value_A, value_B, compute_dtype,
                       scale=sm_scale)
    return o.squeeze(2)


def xkv_fused_k_only(query, key_A, key_B, value, sm_scale=1.0, compute_dtype=torch.float32):
    """q (b,H,D); factorized K; dense V (b,L,KVH,D).  fused_attention/no_pe/ref.py:92-161."""
    b, H, D = query.shape
    _, L, Rk = key_A.shape
    KVH = key_B.shape[1]
    G = H // KVH
    q = _up(query, compute_dtype).reshape(b, KVH, G, D)
    lat = torch.matmul(q, _up(key_B, compute_dtype).transpose(-1, -2)).reshape(b, H, Rk)
    s = torch.matmul(lat, _up(key_A, compute_dtype).transpose(-1, -2)) * sm_scale
    p = F.softmax(s, dim=-1, dtype=torch.float32).to(compute_dtype)
    v = _up(value, compute_dtype).transpose(1, 2)                               # (b,KVH,L,D)
    o = torch.matmul(p.reshape(b, KVH, G, L), v)
    return o.reshape(b, H, D)


def flash_decode_gqa(q, k_buffer, v_buffer, sm_scale=1.0, compute_dtype=torch.float32,
                     logit_cap=0.0):
    """q (b,H,D); K/V (b,L,KVH,Dk|Dv); logits MULTIPLIED by sm_scale as the kernels do
    (flash_decoding/gqa.py:122); eager form from flash_decoding/mla.py:442-471.  Optional
    tanh cap as flash_decoding/mla.py:157-158."""
    b, H, Dk = q.shape
    _, L, KVH, _ = k_buffer.shape
    Dv = v_buffer.shape[-1]
    G = H // KVH
    k = _up(k_buffer, compute_dtype).transpose(1, 2)
    v = _up(v_buffer, compute_dtype).transpose(1, 2)
    s = torch.matmul(_up(q, compute_dtype).reshape(b, KVH, G, Dk), k.transpose(-1, -2)) * sm_scale
    if logit_cap > 0:
        s = logit_cap * torch.tanh(s / logit_cap)
    o = _softmax_pv(s, v, compute_dtype)
    return o.reshape(b, H, Dv)


def mla_decode(q_nope, q_rope, kv_nope, k_rope, sm_scale=1.0, compute_dtype=torch.float32):
    """softmax((q_nope.c^T + q_rope.k_rope^T) * sm_scale) . c, output in latent space.
    flash_decoding/mla2/ref.py:3-33 with the kernels' multiply convention
    (mla2/stage1.py:128-150)."""
    b, H, lora = q_nope.shape
    assert kv_nope.shape[2] == 1
    c = _up(kv_nope, compute_dtype).squeeze(2)
    kr = _up(k_rope, compute_dtype).squeeze(2)
    s = torch.matmul(_up(q_nope, compute_dtype), c.transpose(-1, -2))
    s = s + torch.matmul(_up(q_rope, compute_dtype), kr.transpose(-1, -2))
    s = s * sm_scale
    p = F.softmax(s, dim=-1, dtype=torch.float32).to(compute_dtype)
    return torch.matmul(p, c).reshape(b, H, lora)


def mla_decode_xkv(q_nope, q_rope, kv_A_nope, kv_B_nope, k_rope, sm_scale=1.0,
                   compute_dtype=torch.float32):
    """Latent itself factorized: c = kv_A @ kv_B.  mla2/mla_flash_decoding.py:66-130."""
    B = _up(kv_B_nope, compute_dtype).squeeze(1)                                # (b,r,lora)
    qf = torch.matmul(_up(q_nope, compute_dtype), B.transpose(1, 2))            # :82
    o = mla_decode(qf, q_rope, kv_A_nope, k_rope, sm_scale, compute_dtype)
    return torch.matmul(o, B)                                                   # :128


def mla_absorbed(q_nope, q_rope, c_kv, k_rope, W_uk, W_uv, sm_scale, compute_dtype=torch.float32):
    """MLA absorbed decode: W_uk folded into q, W_uv applied after attention.

    q_nope (b,H,nope); q_rope (b,H,rope); c_kv (b,L,lora); k_rope (b,L,rope);
    W_uk (H,nope,lora); W_uv (H,lora,v) -> (b,H,v).  The attention core is
    mla2/ref.py:3-33; the two einsums are the standard absorption (the reference
    receives q_nope already absorbed).  q_rope / k_rope are taken as already rotated.
    """
    q_lat = torch.einsum("bhd,hdr->bhr", _up(q_nope, compute_dtype), _up(W_uk, compute_dtype))
    o_lat = mla_decode(q_lat, q_rope, c_kv.unsqueeze(2), k_rope.unsqueeze(2), sm_scale, compute_dtype)
    return torch.einsum("bhr,hrv->bhv", o_lat, _up(W_uv, compute_dtype))


# --------------------------------------------------------------------------- benchmark configurations
def rope_query(q, theta, position):
    """Rotate a decode-step query (b,H,1,D) to ``position``.  rope_ref.py:17-21."""
    D = q.shape[-1]
    cos, sin = rope_cos_sin(D, position + 1, theta)
    return apply_rope(q.float(), cos[position], sin[position]).to(q.dtype)


def recon_rope_decode(query, key_A, key_B, value, theta, sm_scale=None,
                      compute_dtype=torch.float32, value_B=None):
    """Factorized K with RoPE + dense V (b,KVH,L,D) (or factorized V when value_B is given):
    K = RoPE(A.B) as test_qAB_rope.py:29-36, then attention.py:7-90 on it.  ``query`` is used
    as given (already rotated to its position)."""
    b, H, _, D = query.shape
    KVH = key_B.shape[1]
    G = H // KVH
    K = reconstruct_rope_keys(key_A, key_B, theta, compute_dtype)
    if value_B is None:
        return gqa_dense(query, K, value, compute_dtype, scale=sm_scale)
    q = _up(query, compute_dtype).reshape(b, KVH, G, D)
    s = torch.matmul(q, K.transpose(-1, -2))
    s = s / (D ** 0.5) if sm_scale is None else s * sm_scale
    L = s.shape[-1]
    p = F.softmax(s, dim=-1, dtype=torch.float32).to(compute_dtype)
    t = torch.matmul(p.reshape(b, H, L), _up(value, compute_dtype))
    Rv = t.shape[-1]
    o = torch.matmul(t.reshape(b, KVH, G, Rv), _up(value_B, compute_dtype))
    return o.reshape(b, H, 1, D)


def group_decode(queries, key_A, key_Bs, value, value_Bs, theta, sm_scale=None,
                 compute_dtype=torch.float32):
    """Cross-layer group: NL layers share key_A; per layer its own query and key_B.  With
    ``value_Bs`` given, ``value`` is the shared value latent (b,L,Rv) and each layer has its
    own value_B; otherwise ``value`` is a per-layer sequence of dense V (b,KVH,L,D).
    Returns (NL,b,H,1,D).  Per layer this is recon_rope_decode."""
    outs = []
    for i in range(len(key_Bs)):
        if value_Bs is None:
            v, vB = value[i], None
        else:
            v, vB = value, value_Bs[i]
        outs.append(recon_rope_decode(queries[i], key_A, key_Bs[i], v, theta, sm_scale,
                                      compute_dtype, value_B=vB))
    return torch.stack(outs)


def error_metrics(got, want):
    """(max-abs error, relative L2 error) in fp64."""
    g = got.detach().double().cpu()
    w = want.detach().double().cpu()
    max_abs = (g - w).abs().max().item() if g.numel() else 0.0
    den = w.norm().item()
    rel_l2 = ((g - w).norm().item() / den) if den > 0 else 0.0
    return max_abs, rel_l2
