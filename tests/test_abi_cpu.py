"""CPU-only checks of the C-ABI library: it loads, exports every symbol include/xkv.h declares,
its parameter block matches the ctypes mirror, and host-side validation returns the documented
status codes without touching a GPU."""
import ctypes as C
import os
import re

import pytest
import torch

from kernel_collections_b200 import _C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "xkv.h")).read()
    return sorted(set(re.findall(r"XKV_API[^;(]*?\b(xkv_\w+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = _C.load()
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/xkv.h but not exported"
    assert sorted(_C.EXPORTS) == names


def test_params_mirror_matches():
    lib = _C.load()
    assert lib.xkv_decode_params_size() == C.sizeof(_C.DecodeParams)
    assert lib.xkv_version() == 1


def test_strerror():
    assert _C.strerror(0) == "ok"
    for rc in range(-7, 0):
        assert _C.strerror(rc) and "unknown" not in _C.strerror(rc)
    assert "unknown" in _C.strerror(-99)


def _valid_dense():
    p = _C.DecodeParams()
    p.dtype, p.score_mode, p.value_mode = _C.XKV_BF16, _C.SCORE_DENSE, _C.VALUE_DENSE
    p.batch, p.num_heads, p.num_kv_heads, p.kv_len = 2, 8, 2, 100
    p.head_dim = p.value_dim = 64
    p.q = p.k = p.v = p.out = 0x1000   # never dereferenced on the host
    p.sm_scale = 1.0
    return p


def test_validation_status_codes():
    lib = _C.load()
    p = _valid_dense()
    assert lib.xkv_decode_workspace_bytes(C.byref(p)) > 0
    assert lib.xkv_decode_plan(C.byref(p)) == b"generic"
    # workspace missing
    assert lib.xkv_decode(C.byref(p), None, 0, None) == -4
    # null params
    assert lib.xkv_decode(None, None, 0, None) == -1
    for field, bad in [("batch", 0), ("kv_len", 0), ("num_kv_heads", 3), ("dtype", 7), ("q", None),
                       ("head_dim", 0), ("out", None), ("score_mode", 9)]:
        p = _valid_dense()
        setattr(p, field, bad)
        assert lib.xkv_decode(C.byref(p), None, 0, None) == -1, field
        assert lib.xkv_decode_workspace_bytes(C.byref(p)) == 0
    # named entry points refuse parameter blocks of another operation
    p = _valid_dense()
    assert lib.xkv_mla_decode(C.byref(p), None, 0, None) == -1
    assert lib.xkv_qab_logits(C.byref(p), None, 0, None) == -1
    assert lib.xkv_recon_rope_decode(C.byref(p), None, 0, None) == -1
    assert lib.xkv_dense_decode(C.byref(p), None, 0, None) == -4
    # too wide for any kernel
    p = _valid_dense()
    p.head_dim = 1 << 20
    assert lib.xkv_decode(C.byref(p), None, 0, None) == -2


def test_cpu_tensors_are_rejected_loudly():
    import kernel_collections_b200 as K
    q = torch.randn(1, 4, 1, 16)
    kv = torch.randn(1, 2, 8, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        K.group_query_attention(q, kv, kv)
    with pytest.raises(RuntimeError, match="CUDA"):
        K.group_query_attention(q, kv, kv, attn_mask=torch.zeros(1, 1, 1, 8))
    with pytest.raises(NotImplementedError):
        K.group_query_attention(q, kv, kv, dropout_p=0.1)


def _blk(**kw):
    p = _C.DecodeParams()
    p.dtype = _C.XKV_BF16
    p.batch, p.num_heads, p.num_kv_heads, p.kv_len = 4, 32, 8, 4096
    p.head_dim = p.value_dim = 128
    p.sm_scale = 1.0
    p.q = p.k = p.v = p.out = 0x10000          # aligned dummies, never dereferenced on the host
    p.q_sb, p.q_sh = 32 * 128, 128
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_kernel_selection_is_host_side_and_follows_the_shape():
    """xkv_decode_plan launches nothing: which kernel family serves which call."""
    lib = _C.load()
    plan = lambda p: lib.xkv_decode_plan(C.byref(p))
    dense = dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, k_sb=4096 * 1024, k_sl=1024, k_sh=128,
                 v_sb=4096 * 1024, v_sl=1024, v_sh=128)
    assert plan(_blk(**dense)) == b"dense_tc"
    assert plan(_blk(**dense, dtype=_C.XKV_F32)) == b"generic"
    assert plan(_blk(**dense, flags=_C.FLAG_FORCE_GENERIC)) == b"generic"
    assert plan(_blk(**dense, k=0x10002)) == b"generic"                      # unaligned cache pointer
    recon = dict(score_mode=_C.SCORE_RECON_ROPE, k_rank=512, k_sb=4096 * 512, k_sl=512, k_proj=0x20000, k_proj_heads=8,
                 kp_sb=0, kp_sh=128, kp_sr=1024, kp_sd=1, theta=5e5)
    vdense = dict(value_mode=_C.VALUE_DENSE, v_sb=4096 * 1024, v_sl=1024, v_sh=128)
    assert plan(_blk(**recon, **vdense)) == b"recon_tc"
    assert plan(_blk(**{**recon, "k_rank": 500, "k_sl": 500, "k_sb": 4096 * 500}, **vdense)) == b"generic"
    vlat = dict(value_mode=_C.VALUE_LATENT, v_rank=512, v_sb=4096 * 512, v_sl=512, v_proj=0x30000, v_proj_heads=8,
                vp_sb=0, vp_sh=128, vp_sr=1024, vp_sd=1)
    assert plan(_blk(**recon, **vlat)) == b"two_pass"
    assert plan(_blk(**dense | vlat)) == b"two_pass"
    lat = dict(score_mode=_C.SCORE_LATENT, k_rank=256, k_sb=4096 * 256, k_sl=256, k_proj=0x20000, k_proj_heads=8,
               kp_sb=0, kp_sh=256 * 128, kp_sr=128, kp_sd=1)
    assert plan(_blk(**lat, **vlat)) == b"latent_tc"
    assert plan(_blk(**lat, **{**vlat, "v_rank": 100, "v_sl": 100})) == b"generic"
    # packed MLA cache: one KV head, 576-wide keys, values = their 512-wide prefix
    packed = dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, num_kv_heads=1, head_dim=576, value_dim=512,
                  k_sb=4096 * 576, k_sl=576, k_sh=576, v_sb=4096 * 576, v_sl=576, v_sh=576, q_sb=32 * 576, q_sh=576)
    assert plan(_blk(**packed)) == b"latent_tc"
    # 64 or more heads: the tcgen05 CTA-pair kernel (heads on the M dimension); a flag keeps the mma.sync one
    many = dict(packed, num_heads=128, q_sb=128 * 576)
    assert plan(_blk(**many)) == b"latent_pair"
    assert plan(_blk(**many, flags=_C.FLAG_LATENT_MMA_SYNC)) == b"latent_tc"
    assert plan(_blk(**packed, logit_cap=5.0)) == b"generic"
