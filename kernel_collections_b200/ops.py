"""Host-side assembly of xkv_decode_params from torch tensors.

`decode()` is the one place that talks to the C ABI; the reference-named entry points in
attention.py, flash_recontruction/ and flash_decoding/ only reshape their arguments into it.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _C


def _inner_contig(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """Kernels address the innermost dimension with stride 1; everything else by stride."""
    if t is None:
        return None
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        return t.contiguous()
    return t


def _stride(t: torch.Tensor, dim: int) -> int:
    return t.stride(dim)


def build_params(
    *,
    score_mode: int,
    value_mode: int,
    q: torch.Tensor,                      # (b, H, D)
    k: torch.Tensor,                      # dense (b, L, KVH, D) view, or latent (b, L, R)
    v: Optional[torch.Tensor] = None,     # dense (b, L, KVH, Dv) view, or latent (b, L, Rv)
    k_proj: Optional[torch.Tensor] = None,   # (b|1, heads, R, D) view
    v_proj: Optional[torch.Tensor] = None,   # (b|1, heads, Rv, Dv) view
    q_tail: Optional[torch.Tensor] = None,   # (b, H, Dt)
    k_tail: Optional[torch.Tensor] = None,   # (b, L, Dt)
    sm_scale: float = 1.0,
    theta: float = 0.0,
    pos_offset: int = 0,
    logit_cap: float = 0.0,
    logits_only: bool = False,
    out: Optional[torch.Tensor] = None,   # (b, H, Dv) view to fill
    num_splits: int = 0,
    force_generic: bool = False,
    num_kv_heads: Optional[int] = None,
    rope_table: Optional[torch.Tensor] = None,   # (L, D/2, 2) fp32 {cos, sin}
    kv_lens: Optional[torch.Tensor] = None,      # (b,) int32: per-row cache lengths (ragged batches)
    return_lse: bool = False,                    # also return the (b, H) fp32 log-sum-exp of the scaled logits
    mask: Optional[torch.Tensor] = None,         # additive, broadcastable to (b, H, L), same dtype
    extra_flags: int = 0,                        # XKV_FLAG_* bits beyond logits-only / force-generic
):
    """Validate shapes and fill one xkv_decode_params block.  Returns (params, result tensor)."""
    _C.require_cuda(q, k, v, k_proj, v_proj, q_tail, k_tail, out, rope_table, kv_lens, mask)
    # projections are addressed with a full set of strides; the streamed tensors need a
    # contiguous innermost dimension
    q, k, v, q_tail, k_tail = map(_inner_contig, (q, k, v, q_tail, k_tail))
    for t in (k, v, k_proj, v_proj, q_tail, k_tail):
        if t is not None and t.dtype != q.dtype:
            raise ValueError("all tensors of one call must share a dtype")
    dev = q.device
    p = _C.DecodeParams()
    p.dtype = _C.dtype_code(q)
    p.score_mode, p.value_mode = score_mode, value_mode
    p.flags = (_C.FLAG_LOGITS_ONLY if logits_only else 0) | (_C.FLAG_FORCE_GENERIC if force_generic else 0) \
        | int(extra_flags)
    b, H, D = q.shape
    L = k.shape[1]
    p.batch, p.num_heads, p.kv_len, p.head_dim = b, H, L, D
    p.q, p.q_sb, p.q_sh = q.data_ptr(), _stride(q, 0), _stride(q, 1)
    p.sm_scale, p.theta, p.logit_cap = float(sm_scale), float(theta), float(logit_cap)
    p.pos_offset, p.num_splits = int(pos_offset), int(num_splits)

    if score_mode == _C.SCORE_DENSE:
        if k.dim() != 4 or k.shape[0] != b or k.shape[3] != D:
            raise ValueError(f"dense keys must be (b, L, KVH, D); got {tuple(k.shape)} for q {tuple(q.shape)}")
        KVH = k.shape[2]
        p.k, p.k_sb, p.k_sl, p.k_sh = k.data_ptr(), _stride(k, 0), _stride(k, 1), _stride(k, 2)
    else:
        if k.dim() != 3 or k.shape[0] != b:
            raise ValueError(f"key latent must be (b, L, R); got {tuple(k.shape)}")
        p.k_rank = k.shape[2]
        p.k, p.k_sb, p.k_sl = k.data_ptr(), _stride(k, 0), _stride(k, 1)
        KVH = num_kv_heads
        if k_proj is not None:
            if k_proj.dim() != 4 or k_proj.shape[2] != p.k_rank or k_proj.shape[3] != D:
                raise ValueError(f"key projection must be (b, heads, R, D); got {tuple(k_proj.shape)}")
            if k_proj.shape[0] not in (1, b):
                raise ValueError("Batch size mismatch between q and the key projection")
            p.k_proj_heads = k_proj.shape[1]
            p.k_proj = k_proj.data_ptr()
            p.kp_sb, p.kp_sh, p.kp_sr, p.kp_sd = (_stride(k_proj, i) for i in range(4))
            if k_proj.shape[0] == 1:
                p.kp_sb = 0          # one matrix shared by the whole batch
            if p.kp_sd == 0:
                p.kp_sd = 1
            if KVH is None:
                KVH = k_proj.shape[1]
    if q_tail is not None:
        p.tail_dim = q_tail.shape[-1]
        p.q_tail, p.qt_sb, p.qt_sh = q_tail.data_ptr(), _stride(q_tail, 0), _stride(q_tail, 1)
        p.k_tail, p.kt_sb, p.kt_sl = k_tail.data_ptr(), _stride(k_tail, 0), _stride(k_tail, 1)

    if not logits_only:
        if v is None:
            raise ValueError("values are required unless logits_only")
        if v.shape[0] != b or v.shape[1] != L:
            raise ValueError("kv_len / batch mismatch between keys and values")
        if value_mode == _C.VALUE_DENSE:
            if v.dim() != 4:
                raise ValueError(f"dense values must be (b, L, KVH, Dv); got {tuple(v.shape)}")
            if KVH is None:
                KVH = v.shape[2]
            if v.shape[2] != KVH:
                raise ValueError("num_kv_heads mismatch between K and V")
            p.value_dim = v.shape[3]
            p.v, p.v_sb, p.v_sl, p.v_sh = v.data_ptr(), _stride(v, 0), _stride(v, 1), _stride(v, 2)
        else:
            if v.dim() != 3:
                raise ValueError(f"value latent must be (b, L, Rv); got {tuple(v.shape)}")
            p.v_rank = v.shape[2]
            p.v, p.v_sb, p.v_sl = v.data_ptr(), _stride(v, 0), _stride(v, 1)
            if v_proj is not None:
                if v_proj.dim() != 4 or v_proj.shape[2] != p.v_rank or v_proj.shape[0] not in (1, b):
                    raise ValueError(f"value projection must be (b, heads, Rv, Dv); got {tuple(v_proj.shape)}")
                p.v_proj_heads = v_proj.shape[1]
                p.value_dim = v_proj.shape[3]
                p.v_proj = v_proj.data_ptr()
                p.vp_sb, p.vp_sh, p.vp_sr, p.vp_sd = (_stride(v_proj, i) for i in range(4))
                if v_proj.shape[0] == 1:
                    p.vp_sb = 0
                if p.vp_sd == 0:
                    p.vp_sd = 1
                if KVH is None:
                    KVH = v_proj.shape[1]
            else:
                p.value_dim = p.v_rank
    if KVH is None:
        KVH = 1
    if H % KVH != 0:
        raise ValueError("num_heads must be divisible by num_kv_heads")
    p.num_kv_heads = KVH

    keep = []
    if score_mode == _C.SCORE_RECON_ROPE:
        if rope_table is not None:
            if tuple(rope_table.shape) != (L, D // 2, 2) or rope_table.dtype != torch.float32 \
                    or not rope_table.is_contiguous():
                raise ValueError("rope_table must be a contiguous fp32 (kv_len, head_dim/2, 2) tensor")
            keep.append(rope_table)
            p.rope_table = rope_table.data_ptr()
        else:
            f = _C.inv_freq(D, theta, dev)
            keep.append(f)
            p.inv_freq = f.data_ptr()

    if mask is not None:
        _C.require_cuda(mask)
        if mask.dtype != q.dtype:
            mask = mask.to(q.dtype)
        try:
            m3 = mask.expand(b, H, L)
        except RuntimeError:
            raise ValueError(f"attn_mask of shape {tuple(mask.shape)} does not broadcast to ({b}, {H}, {L})") from None
        if m3.stride(2) != 1 and L != 1:
            m3 = m3.contiguous()
        keep.append(m3)
        p.mask, p.mask_sb, p.mask_sh = m3.data_ptr(), m3.stride(0), m3.stride(1)
    if kv_lens is not None:
        _C.require_cuda(kv_lens)
        if kv_lens.dtype != torch.int32 or tuple(kv_lens.shape) != (b,) or not kv_lens.is_contiguous():
            raise ValueError("kv_lens must be a contiguous int32 tensor of shape (batch,)")
        keep.append(kv_lens)
        p.kv_lens = kv_lens.data_ptr()

    result = None
    if logits_only:
        result = torch.empty((b, H, L), dtype=q.dtype, device=dev)
        p.logits, p.lg_sb, p.lg_sh = result.data_ptr(), result.stride(0), result.stride(1)
    else:
        if out is None:
            out = torch.empty((b, H, p.value_dim), dtype=q.dtype, device=dev)
        elif out.stride(-1) != 1 or tuple(out.shape) != (b, H, p.value_dim) or out.dtype != q.dtype:
            raise ValueError(f"output must be a ({b}, {H}, {p.value_dim}) {q.dtype} tensor with a contiguous last dim")
        p.out, p.o_sb, p.o_sh = out.data_ptr(), _stride(out, 0), _stride(out, 1)
        result = out
    if return_lse:
        if logits_only:
            raise ValueError("return_lse needs a softmax: not available with logits_only")
        lse = torch.empty((b, H), dtype=torch.float32, device=dev)
        keep.append(lse)
        p.lse_out, p.lse_sb = lse.data_ptr(), lse.stride(0)
        result = (result, lse)
    p._keepalive = (q, k, v, k_proj, v_proj, q_tail, k_tail, keep)   # contiguous copies made above
    return p, result


def decode(*, entry: str = "xkv_decode", check_status=None, **kw):
    """One decode-attention call through the C ABI entry point `entry`.  check_status=True
    synchronises after the call and raises _C.DeviceTimeout if a bounded device-side wait expired
    (default: the process-wide setting, see _C.set_check_status)."""
    p, result = build_params(**kw)
    _C.run_decode(p, kw["q"].device, entry, check_status)
    return result


def decode_builtin_scratch(**kw):
    """Same call as decode(), for hosts that must not allocate device memory: the library's
    built-in scratch array replaces the workspace (see xkv_decode_builtin_scratch in
    include/xkv.h for the size limit and the sharing rules).  The output tensor must be passed
    in (`out=` or, for logits, it is still created here by the caller's allocator)."""
    p, result = build_params(**kw)
    _C.run_decode_builtin_scratch(p, kw["q"].device)
    return result


def merge_segments(outs, lses):
    """Exact merge of decode results over disjoint parts of a cache (e.g. a factorized prefill cache
    and a dense tail): outs[i] (b, H, dim) with lses[i] (b, H) from decode(..., return_lse=True).
    Runs the library's split-merge kernel (xkv_merge); empty parts (lse = -inf) drop out."""
    o0 = outs[0]
    b, H, dim = o0.shape
    part = torch.stack([o.float() for o in outs], dim=2).contiguous()          # (b, H, S, dim)
    lse = torch.stack(list(lses), dim=2).contiguous()                          # (b, H, S)
    out = torch.empty((b, H, dim), dtype=o0.dtype, device=o0.device)
    lib = _C.load()
    rc = lib.xkv_merge(part.data_ptr(), lse.data_ptr(), out.data_ptr(), _C.dtype_code(o0), b, H, len(outs), dim,
                       out.stride(0), out.stride(1), torch.cuda.current_stream(o0.device).cuda_stream)
    _C.check(rc, "xkv_merge")
    return out


def plan(**kw):
    """Name of the kernel family the library would run for these arguments."""
    p, _ = build_params(**kw)
    return _C.plan_name(p, kw["q"].device)


def group_decode(layer_kwargs: list, check_status=None):
    """Run xkv_group_decode over per-layer keyword sets of decode() (same shapes, shared latents).
    Returns the list of per-layer outputs."""
    blocks, outs = [], []
    for kw in layer_kwargs:
        p, result = build_params(**kw)
        blocks.append(p)
        outs.append(result)
    n = len(blocks)
    arr = (_C.DecodeParams * n)(*blocks)
    lib = _C.load()
    dev = layer_kwargs[0]["q"].device
    with torch.cuda.device(dev):
        nbytes = lib.xkv_group_decode_workspace_bytes(arr, n)
        if nbytes == 0:
            _C.check(lib.xkv_group_decode(arr, n, None, 0, None) or -2, "xkv_group_decode")
        ws = _C.workspace(dev, nbytes)
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = lib.xkv_group_decode(arr, n, ws.data_ptr(), ws.numel(), stream)
        _C.check(rc, "xkv_group_decode")
        if _C._check_status if check_status is None else check_status:
            _C.raise_on_status(ws.data_ptr(), stream, "xkv_group_decode")
    return outs
