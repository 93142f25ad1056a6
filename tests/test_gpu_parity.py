"""GPU parity: every reference-named entry point (through the C ABI) against the CPU oracle on
the same seeded inputs.  Primary oracle = eager math in fp32 on the dtype-rounded inputs.

Tolerances: fp32 max-abs and rel-L2 <= 1e-4; bf16 / fp16 max-abs <= 2e-2 and rel-L2 <= 1e-2
(max-abs is taken relative to max(1, |ref|max) so unscaled logits of magnitude ~10 are judged
in their own units)."""
import os

import numpy as np
import pytest
import torch

import kernel_collections_b200 as K
from kernel_collections_b200 import flash_recontruction as FR
from kernel_collections_b200 import flash_decoding as FD
from kernel_collections_b200 import _C, ops
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16, torch.float16]
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_eager.npz"))


def tol(dtype):
    return (1e-4, 1e-4) if dtype == torch.float32 else (2e-2, 1e-2)


def check(got, want, dtype, what=""):
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert got.dtype == dtype, (what, got.dtype)
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite output"
    max_abs, rel = O.error_metrics(got, want)
    ta, tr = tol(dtype)
    scale = max(1.0, want.abs().max().item())
    assert max_abs <= ta * scale and rel <= tr, f"{what}: max_abs={max_abs:.3e} (scale {scale:.2f}) rel_l2={rel:.3e}"


def mk(shape, dtype, scale=1.0, gen=None):
    """Seeded CPU fp32 normal, rounded to dtype; returns (cpu tensor in dtype, cuda copy)."""
    x = (torch.randn(shape, generator=gen) * scale).to(dtype)
    return x, x.to(DEV)


def g(seed):
    return torch.Generator().manual_seed(seed)


SHAPES = [  # b, H, KVH, D, L
    (2, 8, 2, 64, 100),
    (1, 4, 4, 128, 1),
    (1, 32, 8, 128, 1000),
    (3, 7, 1, 32, 17),
    (2, 16, 2, 16, 16),
    (1, 6, 2, 80, 333),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_dense_gqa(dtype, shape):
    b, H, KVH, D, L = shape
    gen = g(1)
    q, qd = mk((b, H, 1, D), dtype, gen=gen)
    k, kd = mk((b, KVH, L, D), dtype, gen=gen)
    v, vd = mk((b, KVH, L, D), dtype, gen=gen)
    check(K.group_query_attention(qd, kd, vd), O.gqa_dense(q, k, v), dtype, "group_query_attention")
    # flash layout: (b,1,H,D) / (b,L,KVH,D)
    out = K.group_query_attention_fa(qd.transpose(1, 2), kd.transpose(1, 2).contiguous(),
                                     vd.transpose(1, 2).contiguous())
    check(out.transpose(1, 2), O.gqa_dense(q, k, v), dtype, "group_query_attention_fa")
    # flash_decoding.gqa with explicit scale and in-place output
    o = torch.zeros(b, H, D, dtype=dtype, device=DEV)
    splits = torch.full((b,), 8, dtype=torch.int32, device=DEV)
    r = FD.gqa.decode_attention_fwd(qd[:, :, 0], kd.transpose(1, 2), vd.transpose(1, 2), o, splits, 8, 0.3)
    assert r is o
    check(o, O.flash_decode_gqa(q[:, :, 0], k.transpose(1, 2), v.transpose(1, 2), 0.3), dtype, "gqa.decode_attention_fwd")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 8, 2, 64, 100, 24, 40), (1, 32, 8, 128, 700, 256, 384), (2, 4, 1, 32, 9, 5, 3)])
def test_factorized_family(dtype, shape):
    b, H, KVH, D, L, Rk, Rv = shape
    gen = g(2)
    q, qd = mk((b, H, 1, D), dtype, gen=gen)
    k, kd = mk((b, KVH, L, D), dtype, gen=gen)
    v, vd = mk((b, L, KVH, D), dtype, gen=gen)
    Ak, Akd = mk((b, L, Rk), dtype, gen=gen)
    Bk, Bkd = mk((b, KVH, Rk, D), dtype, Rk ** -0.5, gen=gen)
    Av, Avd = mk((b, L, Rv), dtype, gen=gen)
    Bv, Bvd = mk((b, KVH, Rv, D), dtype, Rv ** -0.5, gen=gen)
    check(K.group_query_attention_factorized_v_only(qd, kd, Avd, Bvd),
          O.gqa_factorized_v_only(q, k, Av, Bv), dtype, "factorized_v_only")
    check(K.group_query_attention_factorized(qd, Akd, Bkd, Avd, Bvd),
          O.gqa_factorized(q, Ak, Bk, Av, Bv), dtype, "factorized")
    check(FR.qAB_no_pe_v1(qd, Akd, Bkd), O.qab_no_pe(q, Ak, Bk), dtype, "qAB_no_pe_v1")
    check(FR.qAB_no_pe_v2(qd, Akd, Bkd), O.qab_no_pe(q, Ak, Bk), dtype, "qAB_no_pe_v2")
    # fused xKV entry points, q 3-D, explicit multiply scale
    q3, q3d = q[:, :, 0], qd[:, :, 0]
    splits = torch.full((b,), 16, dtype=torch.int32, device=DEV)
    s = 0.11
    want = O.xkv_fused(q3, Ak, Bk, Av, Bv, s)
    o = torch.zeros(b, H, D, dtype=dtype, device=DEV)
    assert FR.gqa_xKV_no_pe(q3d, Akd, Bkd, Avd, Bvd, o, splits, 16, s) is o
    check(o, want, dtype, "gqa_xKV_no_pe")
    check(FR.gqa_xKV_no_pe_v2(q3d, Akd, Bkd, Avd, Bvd, splits, 16, s), want, dtype, "gqa_xKV_no_pe_v2")
    o2 = torch.zeros(b, H, D, dtype=dtype, device=DEV)
    FR.gqa_xKV_no_pe_k_only(q3d, Akd, Bkd, vd, o2, splits, 16, s)
    check(o2, O.xkv_fused_k_only(q3, Ak, Bk, v, s), dtype, "gqa_xKV_no_pe_k_only")
    s1 = 1.0 if dtype == torch.float32 else None
    if s1:  # the unscaled *_ref names (scale 1 makes bf16 softmax very peaked; fp32 only)
        check(FR.gqa_xKV_no_pe_ref(q3d * 0.2, Akd, Bkd, Avd, Bvd), O.xkv_fused(q3 * 0.2, Ak, Bk, Av, Bv, 1.0), dtype, "xKV_ref")
        check(FR.gqa_xKV_no_pe_k_only_ref(q3d * 0.2, Akd, Bkd, vd), O.xkv_fused_k_only(q3 * 0.2, Ak, Bk, v, 1.0), dtype, "xKV_k_only_ref")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 8, 2, 64, 100, 24, 10000.0), (1, 32, 8, 128, 520, 64, 500000.0),
                                   (1, 4, 1, 128, 130, 32, 1e7), (2, 4, 4, 16, 5, 3, 10000.0)])
def test_qab_rope_and_recon_decode(dtype, shape):
    b, H, KVH, D, L, R, theta = shape
    gen = g(3)
    q, qd = mk((b, H, 1, D), dtype, gen=gen)
    A, Ad = mk((b, L, R), dtype, gen=gen)
    B, Bd = mk((b, KVH, R, D), dtype, R ** -0.5, gen=gen)
    v, vd = mk((b, KVH, L, D), dtype, gen=gen)
    Av, Avd = mk((b, L, 20), dtype, gen=gen)
    Bv, Bvd = mk((b, KVH, 20, D), dtype, 20 ** -0.5, gen=gen)
    want = O.qab_rope(q, A, B, theta)
    for fn in (FR.qAB_rope_v1, FR.qAB_rope_v3, FR.qAB_rope_v4):
        check(fn(qd, Ad, Bd, theta=theta), want, dtype, fn.__name__)
    cos, sin = O.rope_cos_sin(D, L, theta)
    table = torch.cat([sin[:, : D // 2], cos[:, : D // 2]], dim=-1).to(DEV)
    check(FR.qAB_rope_v2(qd, Ad, Bd, table), want, dtype, "qAB_rope_v2")
    # fused decode: dense V and factorized V, default 1/sqrt(D) scale
    check(K.recon_rope_decode(qd, Ad, Bd, vd, theta=theta), O.recon_rope_decode(q, A, B, v, theta), dtype, "recon_rope_decode dense V")
    check(K.recon_rope_decode(qd, Ad, Bd, Avd, Bvd, theta=theta),
          O.recon_rope_decode(q, A, B, Av, theta, value_B=Bv), dtype, "recon_rope_decode factorized V")
    # the reference's own RoPE entry point: unscaled logits (scaled-down q keeps softmax sane)
    qs, qsd = (q * D ** -0.5).to(dtype), (qd * D ** -0.5).to(dtype)
    check(K.group_query_attention_factorized_RoPE(qsd, Ad, Bd, Avd, Bvd, theta=theta),
          O.gqa_factorized_rope(qs, A, B, Av, Bv, theta), dtype, "factorized_RoPE")


def test_rope_query_matches_oracle():
    q, qd = mk((2, 8, 1, 128), torch.bfloat16, gen=g(4))
    got = K.rope_query(qd, 500000.0, 16384)
    want = O.rope_query(q, 500000.0, 16384)
    # (the device's cos / sin may differ from the host's in the last fp32 bit: one unit in the last place at most)
    assert ((got.cpu().float() - want.float()).abs() <= 2.0 ** -7 * want.float().abs().clamp(min=1.0)).all()
    assert (got.cpu() != want).float().mean().item() < 0.01


@pytest.mark.parametrize("dtype", DTYPES)
def test_shared_B_matrix_and_strided_views(dtype):
    """Shared B as in the benchmark configurations (R, KVH*D) broadcast over the batch, and non-contiguous K/V views."""
    b, H, KVH, D, L, R, theta = 3, 8, 2, 64, 75, 32, 500000.0
    gen = g(5)
    q, qd = mk((b, H, 1, D), dtype, gen=gen)
    A, Ad = mk((b, L, R), dtype, gen=gen)
    B2, B2d = mk((R, KVH * D), dtype, R ** -0.5, gen=gen)
    v, vd = mk((b, L, KVH, D), dtype, gen=gen)         # stored token-major, passed as a transposed view
    B4 = B2.view(R, KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1)
    want = O.recon_rope_decode(q, A, B4, v.transpose(1, 2), theta)
    check(K.recon_rope_decode(qd, Ad, B2d, vd.transpose(1, 2), theta=theta), want, dtype, "shared B, strided V")
    # A as a slice of a wider buffer (row stride != R)
    wide = torch.zeros(b, L, R + 8, dtype=dtype, device=DEV)
    wide[..., :R] = Ad
    check(K.recon_rope_decode(qd, wide[..., :R], B2d, vd.transpose(1, 2), theta=theta), want, dtype, "strided A")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mla_family(dtype):
    b, H, lora, rope, L = 2, 16, 64, 16, 203
    gen = g(6)
    qn, qnd = mk((b, H, lora), dtype, 1 / 3, gen=gen)
    qr, qrd = mk((b, H, rope), dtype, 1 / 3, gen=gen)
    c, cd = mk((b, L, 1, lora), dtype, 1 / 3, gen=gen)
    kr, krd = mk((b, L, 1, rope), dtype, 1 / 3, gen=gen)
    check(FD.mla2.mla_decode_attention_fwd(qnd, qrd, cd, krd, 0.7), O.mla_decode(qn, qr, c, kr, 0.7), dtype, "mla2 fwd")
    check(FD.mla2.mla_decode_attention_fwd_ref(qnd, qrd, cd, krd, 2.0), O.mla_decode(qn, qr, c, kr, 0.5), dtype, "mla2 ref (divide)")
    # factorized latent
    r = 24
    kA, kAd = mk((b, L, 1, r), dtype, 1 / 3, gen=gen)
    kB, kBd = mk((b, 1, r, lora), dtype, 1 / 3, gen=gen)
    check(FD.mla2.mla_decode_attention_xKV(qnd, qrd, kAd, kBd, krd, 0.7),
          O.mla_decode_xkv(qn, qr, kA, kB, kr, 0.7), dtype, "mla2 xKV")
    # packed 576-style cache (here 64+16 = 80), value = the latent prefix, optional logit cap
    kbuf = torch.cat([c, kr], dim=-1)
    kbufd = kbuf.to(DEV)
    qfull, qfulld = torch.cat([qn, qr], dim=-1), torch.cat([qnd, qrd], dim=-1)
    for cap in (0.0, 5.0):
        o = torch.zeros(b, H, lora, dtype=dtype, device=DEV)
        assert FD.mla.decode_attention_fwd(qfulld, kbufd, kbufd[..., :lora], o, 0.9, cap) is None
        check(o, O.flash_decode_gqa(qfull, kbuf, kbuf[..., :lora], 0.9, logit_cap=cap), dtype, f"mla.decode cap={cap}")
    check(FD.mla.decode_attention_reference(qfulld, kbufd, kbufd[..., :lora], None, 2.0),
          O.flash_decode_gqa(qfull, kbuf, kbuf[..., :lora], 0.5), dtype, "mla.decode_attention_reference")
    # absorbed form with W_uk / W_uv
    nope, vdim = 32, 48
    qq, qqd = mk((b, H, nope), dtype, gen=gen)
    Wk, Wkd = mk((H, nope, lora), dtype, lora ** -0.5, gen=gen)
    Wv, Wvd = mk((H, lora, vdim), dtype, lora ** -0.5, gen=gen)
    sc = (nope + rope) ** -0.5
    check(K.mla_absorbed_decode(qqd, qrd, cd[:, :, 0], krd[:, :, 0], Wkd, Wvd, sc),
          O.mla_absorbed(qq, qr, c[:, :, 0], kr[:, :, 0], Wk, Wv, sc), dtype, "mla_absorbed_decode")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("factorized_v", [False, True])
def test_group_decode(dtype, factorized_v):
    NL, b, H, KVH, D, L, R, Rv, theta = 3, 2, 8, 2, 64, 90, 32, 24, 500000.0
    gen = g(7)
    A, Ad = mk((b, L, R), dtype, gen=gen)
    qs, Bs, Vs, Bvs = [], [], [], []
    Av, Avd = mk((b, L, Rv), dtype, gen=gen)
    for _ in range(NL):
        qs.append(mk((b, H, 1, D), dtype, gen=gen))
        Bs.append(mk((R, KVH * D), dtype, R ** -0.5, gen=gen))
        Vs.append(mk((b, KVH, L, D), dtype, gen=gen))
        Bvs.append(mk((Rv, KVH * D), dtype, Rv ** -0.5, gen=gen))
    expand = lambda B2, r: B2.view(r, KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1)
    if factorized_v:
        got = K.xkv_group_decode([x[1] for x in qs], Ad, [x[1] for x in Bs], Avd, [x[1] for x in Bvs], theta=theta)
        want = O.group_decode([x[0] for x in qs], A, [expand(x[0], R) for x in Bs], Av,
                              [expand(x[0], Rv) for x in Bvs], theta)
    else:
        got = K.xkv_group_decode([x[1] for x in qs], Ad, [x[1] for x in Bs], [x[1] for x in Vs], theta=theta)
        want = O.group_decode([x[0] for x in qs], A, [expand(x[0], R) for x in Bs], [x[0] for x in Vs], None, theta)
    for i in range(NL):
        check(got[i], want[i], dtype, f"group layer {i}")


def test_golden_fixtures_through_cuda():
    """The committed outputs of the reference's own eager code, reproduced by the CUDA path."""
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_eager.npz"))
    t = lambda k: torch.from_numpy(G[k])
    d = lambda k: torch.from_numpy(G[k]).to(DEV)
    f32 = torch.float32
    for name in ("a", "b", "c"):
        p = f"gqa/{name}/"
        check(K.group_query_attention(d(p + "q"), d(p + "K"), d(p + "V")), t(p + "dense"), f32, p + "dense")
        check(K.group_query_attention_factorized_v_only(d(p + "q"), d(p + "K"), d(p + "Av"), d(p + "Bv")), t(p + "v_only"), f32, p + "v_only")
        check(K.group_query_attention_factorized(d(p + "q"), d(p + "Ak"), d(p + "Bk"), d(p + "Av"), d(p + "Bv")), t(p + "factorized"), f32, p + "factorized")
        check(FR.qAB_no_pe_ref(d(p + "q"), d(p + "Ak"), d(p + "Bk")), t(p + "qab_no_pe"), f32, p + "qab_no_pe")
        check(FR.gqa_xKV_no_pe_ref(d(p + "q")[:, :, 0], d(p + "Ak"), d(p + "Bk"), d(p + "Av"), d(p + "Bv")), t(p + "fused"), f32, p + "fused")
        check(FR.gqa_xKV_no_pe_k_only_ref(d(p + "q")[:, :, 0], d(p + "Ak"), d(p + "Bk"), d(p + "V").transpose(1, 2)), t(p + "fused_k_only"), f32, p + "k_only")
    for name in ("r1", "r2"):
        p = f"qab_rope/{name}/"
        theta = float(G[p + "theta"])
        check(FR.qAB_rope_v1(d(p + "q"), d(p + "Ak"), d(p + "Bk"), theta=theta), t(p + "logits"), f32, p + "logits")
        check(K.recon_rope_decode(d(p + "q"), d(p + "Ak"), d(p + "Bk"), d(p + "V"), theta=theta), t(p + "decode"), f32, p + "decode")
    for name in ("m1", "m2"):
        p = f"mla/{name}/"
        check(FD.mla2.mla_decode_attention_fwd(d(p + "q_nope"), d(p + "q_rope"), d(p + "kv_nope"), d(p + "k_rope"), 1.0), t(p + "out_scale1"), f32, p)
        check(FD.mla2.mla_decode_attention_fwd(d(p + "q_nope"), d(p + "q_rope"), d(p + "kv_nope"), d(p + "k_rope"), 0.25), t(p + "out_mul_quarter"), f32, p)


def test_split_count_independence_and_determinism():
    """Size-independent properties: the result does not depend on the KV split count beyond
    rounding, and repeated calls are bit-identical (fixed merge order)."""
    dtype = torch.float32
    b, H, KVH, D, L = 2, 8, 2, 64, 4000
    gen = g(8)
    q, qd = mk((b, H, D), dtype, gen=gen)
    k, kd = mk((b, L, KVH, D), dtype, gen=gen)
    v, vd = mk((b, L, KVH, D), dtype, gen=gen)
    outs = []
    for s in (1, 3, 64, 250):
        kw = dict(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE,
                  q=qd, k=kd, v=vd, sm_scale=D ** -0.5, num_splits=s)
        o1 = ops.decode(**kw)
        o2 = ops.decode(**kw)
        assert torch.equal(o1, o2)
        outs.append(o1)
    for o in outs[1:]:
        assert (o - outs[0]).abs().max().item() < 2e-6
    check(outs[0], O.flash_decode_gqa(q, k, v, D ** -0.5), dtype, "split invariance")


def test_softmax_shift_invariance_and_extreme_logits():
    """Large logits must not overflow (online softmax); adding a constant key direction that
    shifts every logit equally leaves the output unchanged."""
    dtype = torch.float32
    b, H, KVH, D, L = 1, 4, 1, 32, 300
    gen = g(9)
    q, qd = mk((b, H, 1, D), dtype, 30.0, gen=gen)      # logits of magnitude ~ 1e2-1e3
    k, kd = mk((b, KVH, L, D), dtype, gen=gen)
    v, vd = mk((b, KVH, L, D), dtype, gen=gen)
    got = K.group_query_attention(qd, kd, vd)
    check(got, O.gqa_dense(q, k, v), dtype, "extreme logits")


def test_error_behaviour_on_gpu():
    q = torch.randn(1, 4, 1, 16, device=DEV)
    kv = torch.randn(1, 2, 8, 16, device=DEV)
    with pytest.raises(NotImplementedError):
        K.group_query_attention(q, kv, kv, dropout_p=0.5)
    with pytest.raises(ValueError):
        K.group_query_attention(q, kv, kv, attn_mask=torch.zeros(1, 1, 1, 9, device=DEV))
    with pytest.raises(ValueError):
        K.group_query_attention(q, kv.half(), kv.half())
    with pytest.raises(AssertionError):
        K.group_query_attention(torch.randn(1, 4, 2, 16, device=DEV), kv, kv)
    with pytest.raises(ValueError):
        K.group_query_attention(q.double(), kv.double(), kv.double())
    with pytest.raises(AssertionError):
        FR.qAB_rope_v1(q, torch.randn(1, 8, 5, device=DEV), torch.randn(1, 2, 6, 16, device=DEV))


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_decode_separated_buffers(dtype):
    """deepseek_mla pd_sep entry points: one cache split into a prefill part and a decoded tail must
    equal attention over the concatenated cache, including a tail that a merged-length split table
    would have dropped."""
    b, H, KVH, D, Lp, Ld = 2, 16, 1, 128, 1000, 37
    gen = g(10)
    q, qd = mk((b, H, D), dtype, 0.5, gen=gen)
    kp, kpd = mk((b, Lp, KVH, D), dtype, gen=gen)
    vp, vpd = mk((b, Lp, KVH, D), dtype, gen=gen)
    kdn, kdd = mk((b, Ld, KVH, D), dtype, gen=gen)
    vdn, vdd = mk((b, Ld, KVH, D), dtype, gen=gen)
    got = FD.deepseek_mla.mla_decode_attention_fwd_pd_sep(qd, kpd, vpd, kdd, vdd, 0.2)
    want = O.flash_decode_gqa(q, torch.cat([kp, kdn], 1), torch.cat([vp, vdn], 1), 0.2)
    check(got, want, dtype, "pd_sep")
    # factorized prefill cache
    R = 64
    kA, kAd = mk((b, Lp, R), dtype, gen=gen)
    kB, kBd = mk((b, KVH, R, D), dtype, R ** -0.5, gen=gen)
    vA, vAd = mk((b, Lp, R), dtype, gen=gen)
    vB, vBd = mk((b, KVH, R, D), dtype, R ** -0.5, gen=gen)
    got = FD.deepseek_mla.mla_decode_attention_fwd_pd_sep_xKV(qd, kAd, kBd, vAd, vBd, kdd, vdd, 0.2)
    Kp = torch.matmul(kA.float().unsqueeze(1), kB.float()).transpose(1, 2)      # (b, Lp, KVH, D)
    Vp = torch.matmul(vA.float().unsqueeze(1), vB.float()).transpose(1, 2)
    want = O.flash_decode_gqa(q, torch.cat([Kp, kdn.float()], 1), torch.cat([Vp, vdn.float()], 1), 0.2)
    check(got, want, dtype, "pd_sep_xKV")
    # the log-sum-exp itself
    o, lse = ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=qd, k=kpd,
                        v=vpd, sm_scale=0.2, return_lse=True)
    s = torch.einsum("bhd,blkd->bhl", q.float(), kp.float()) * 0.2
    assert (lse.cpu() - torch.logsumexp(s, -1)).abs().max().item() < (2e-2 if dtype != torch.float32 else 1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_additive_attention_mask(dtype):
    """attn_mask is added to the scaled logits before the softmax (attention.py:60-64), in every
    broadcast form the reference accepts; also on factorized caches and on head_dim-128 shapes,
    where masked calls leave the tensor-core kernels for the portable ones."""
    b, H, KVH, D, L, R = 2, 8, 2, 128, 200, 64
    gen = g(11)
    q, qd = mk((b, H, 1, D), dtype, gen=gen)
    k, kd = mk((b, KVH, L, D), dtype, gen=gen)
    v, vd = mk((b, KVH, L, D), dtype, gen=gen)
    G = H // KVH

    def ref_dense(mask5):
        qq = q.float().view(b, KVH, G, D)
        s = torch.matmul(qq, k.float().transpose(-1, -2)) / D ** 0.5 + mask5.float()[:, :, :, 0]
        p = torch.softmax(s, -1)
        return torch.matmul(p, v.float()).view(b, H, 1, D)

    for shape in [(b, 1, 1, 1, L), (b, KVH, G, 1, L), (1, 1, 1, 1, L)]:
        m, md = mk(shape, dtype, 2.0, gen=gen)
        m5 = m.expand(b, KVH, G, 1, L)
        check(K.group_query_attention(qd, kd, vd, attn_mask=md), ref_dense(m5), dtype, f"mask {shape}")
    m4, m4d = mk((b, H, 1, L), dtype, 2.0, gen=gen)
    check(K.group_query_attention_sdpa(qd, kd, vd, attn_mask=m4d), ref_dense(m4.view(b, KVH, G, 1, L)), dtype, "mask 4-D")
    # a padding-style mask equals truncating the cache
    pad = torch.zeros(b, 1, 1, L)
    pad[0, ..., 150:] = float("-inf")
    got = K.group_query_attentionv2(qd, kd, vd, attn_mask=pad.to(dtype).to(DEV))
    lens = torch.tensor([150, L], dtype=torch.int32, device=DEV)
    check(got, K.group_query_attention(qd, kd, vd, kv_lens=lens).float().cpu(), dtype, "-inf mask vs kv_lens")
    # factorized cache
    Ak, Akd = mk((b, L, R), dtype, gen=gen)
    Bk, Bkd = mk((b, KVH, R, D), dtype, R ** -0.5, gen=gen)
    Av, Avd = mk((b, L, R), dtype, gen=gen)
    Bv, Bvd = mk((b, KVH, R, D), dtype, R ** -0.5, gen=gen)
    m, md = mk((b, 1, 1, 1, L), dtype, 2.0, gen=gen)
    Kf = torch.matmul(Ak.float().unsqueeze(1), Bk.float())
    Vf = torch.matmul(Av.float().unsqueeze(1), Bv.float())
    qq = q.float().view(b, KVH, G, D)
    s = torch.matmul(qq, Kf.transpose(-1, -2)) / D ** 0.5 + m.float()[:, :, :, 0]
    want = torch.matmul(torch.softmax(s, -1), Vf).view(b, H, 1, D)
    check(K.group_query_attention_factorized(qd, Akd, Bkd, Avd, Bvd, attn_mask=md), want, dtype, "masked factorized")


@pytest.mark.parametrize("dtype", DTYPES)
def test_leading_minus_inf_mask_single_split(dtype):
    """A left-padding mask: the first 40 tokens are -inf, so whole 16-token tiles are masked before
    the split has seen a finite logit.  With one KV split nothing may be dropped: the result equals
    attention over the unmasked suffix."""
    b, H, KVH, D, L, pad = 2, 8, 2, 64, 200, 40
    gen = g(12)
    q, qd = mk((b, H, D), dtype, gen=gen)
    k, kd = mk((b, L, KVH, D), dtype, gen=gen)
    v, vd = mk((b, L, KVH, D), dtype, gen=gen)
    mask = torch.zeros(b, 1, L)
    mask[:, :, :pad] = float("-inf")
    for splits in (1, 0):
        got = ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=qd, k=kd, v=vd,
                         sm_scale=D ** -0.5, mask=mask.to(dtype).to(DEV), num_splits=splits)
        want = O.flash_decode_gqa(q, k[:, pad:], v[:, pad:], sm_scale=D ** -0.5)
        check(got, want, dtype, f"leading -inf mask, num_splits={splits}")
    # the most negative finite fp32 value rounds to -inf in bf16: same result
    big = torch.zeros(b, 1, L)
    big[:, :, :pad] = torch.finfo(torch.float32).min
    got = ops.decode(entry="xkv_dense_decode", score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=qd, k=kd, v=vd,
                     sm_scale=D ** -0.5, mask=big.to(DEV), num_splits=1)
    check(got, want, dtype, "finfo.min mask")


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_query_kernel_positions(dtype):
    """xkv_rope_query: one position for the batch or one per sequence, in place or into a new tensor,
    against the reference's rotation (flash_recontruction/rope/rope_ref.py:11-21).  The angles are formed
    as in the oracle; the device's cos / sin may differ from the host's in the last fp32 bit, so a result
    may land on the neighbouring value of the working dtype: at most one unit in the last place, on a
    small fraction of the elements."""
    b, H, D = 3, 8, 128
    q, qd = mk((b, H, 1, D), dtype, gen=g(14))
    ulp = {torch.float32: 2e-6, torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}[dtype]

    def same(got, want):
        diff = (got.float().cpu() - want.float()).abs()
        assert (diff <= ulp * want.float().abs().clamp(min=1.0)).all(), diff.max().item()
        if dtype != torch.float32:
            assert (diff > 0).float().mean().item() < 0.01

    for theta, pos in [(5e5, 16384), (1e7, 131072), (1e4, 0)]:
        same(K.rope_query(qd, theta, pos), O.rope_query(q, theta, pos))
    positions = torch.tensor([5, 70000, 131071], dtype=torch.int32, device=DEV)
    got = K.rope_query(qd, 5e5, positions)
    for i, pz in enumerate(positions.tolist()):
        same(got[i:i + 1], O.rope_query(q[i:i + 1], 5e5, pz))
    buf = qd.clone()
    assert K.rope_query(buf, 5e5, positions, out=buf) is buf and torch.equal(buf, got)
    with pytest.raises(ValueError):
        K.rope_query(qd, 5e5, positions.long())


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_append_roundtrip(dtype):
    """xkv_latent_append: the new token's key row projected with the pseudo-inverse of B lands in row
    pos_b of the latent; with keys that lie in B's row space the appended row rebuilds the key, and a
    decode over the grown cache equals the oracle on the cache extended on the CPU."""
    b, KVH, D, R, cap, H = 3, 2, 64, 48, 40, 8
    gen = g(15)
    lens = [17, 0, 39]
    Bm = torch.randn(R, KVH * D, generator=gen) / R ** 0.5
    pinv = torch.linalg.pinv(Bm)                                         # (KVH*D, R)
    A, Ad = mk((b, cap, R), dtype, gen=gen)
    a_new = torch.randn(b, R, generator=gen)
    k_new = (a_new @ Bm).to(dtype)                                       # in the row space of B (up to rounding)
    pos = torch.tensor(lens, dtype=torch.int32, device=DEV)
    pinv_t = pinv.to(dtype)
    out = K.latent_append(Ad, k_new.to(DEV), pinv_t.to(DEV), pos)
    assert out is Ad
    want_rows = (k_new.float() @ pinv_t.float())
    ta = 1e-4 if dtype == torch.float32 else 2e-2
    for i, n in enumerate(lens):
        assert (Ad[i, n].float().cpu() - want_rows[i]).abs().max().item() <= ta * max(1.0, want_rows[i].abs().max().item())
        keep = torch.ones(cap, dtype=torch.bool)
        keep[n] = False
        assert torch.equal(Ad[i, keep].cpu(), A[i, keep])              # nothing else was touched
    if dtype == torch.float32:
        assert (Ad[0, 17].cpu() @ Bm - k_new[0]).abs().max().item() < 1e-3   # the appended row rebuilds the key
    # a position outside the cache appends nothing; a scalar position applies to every row
    before = Ad.clone()
    K.latent_append(Ad, k_new.to(DEV), pinv_t.to(DEV), torch.tensor([cap, -1, cap + 5], dtype=torch.int32, device=DEV))
    assert torch.equal(before, Ad)
    K.latent_append(Ad, k_new.to(DEV), pinv_t.to(DEV), 3)
    assert (Ad[:, 3].float().cpu() - want_rows).abs().max().item() <= ta * max(1.0, want_rows.abs().max().item())
    # decode over the grown cache (lengths + 1) against the oracle on the same latent bits
    Bk = Bm.view(R, KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1).contiguous().to(dtype)
    q, qd = mk((b, H, 1, D), dtype, gen=gen)
    V, Vd = mk((b, cap, R), dtype, gen=gen)
    new_lens = torch.tensor([n + 1 for n in lens], dtype=torch.int32, device=DEV)
    got = K.group_query_attention_factorized(qd, Ad, Bk.to(DEV), Vd, Bk.to(DEV), kv_lens=new_lens)
    Ac = Ad.cpu()
    for i, n in enumerate(lens):
        want = O.gqa_factorized(q[i:i + 1], Ac[i:i + 1, :n + 1], Bk[i:i + 1], V[i:i + 1, :n + 1], Bk[i:i + 1])
        check(got[i:i + 1], want, dtype, f"decode after append, row {i}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_several_query_tokens_v2(dtype):
    """group_query_attentionv2 with q_len > 1 (attention.py:93-182): the reference's own outputs on the
    golden inputs, then a speculative-decode shape (4 new tokens, causal among themselves through the
    additive mask) on head_dim 128 where group x q_len = 16 rows stay on the tensor-core kernel, and a
    longer burst that goes to the portable kernel."""
    if dtype == torch.float32:
        for name in ("v1", "v2"):
            p = f"gqa_v2/{name}/"
            q, Kc, V, mask = (torch.from_numpy(GOLD[p + k]) for k in ["q", "K", "V", "mask"])
            got = K.group_query_attentionv2(q.to(DEV), Kc.to(DEV), V.to(DEV))
            check(got, torch.from_numpy(GOLD[p + "plain"]), dtype, f"golden v2 {name}")
            got = K.group_query_attentionv2(q.to(DEV), Kc.to(DEV), V.to(DEV), attn_mask=mask.to(DEV))
            check(got, torch.from_numpy(GOLD[p + "masked"]), dtype, f"golden v2 {name} masked")
    b, H, KVH, D, L = 2, 32, 8, 128, 700
    gen = g(16)
    k, kd = mk((b, KVH, L, D), dtype, gen=gen)
    v, vd = mk((b, KVH, L, D), dtype, gen=gen)
    for q_len in (4, 7):
        q, qd = mk((b, H, q_len, D), dtype, gen=gen)
        got = K.group_query_attentionv2(qd, kd, vd)
        check(got, O.gqa_dense_multi(q, k, v), dtype, f"q_len {q_len}")
        # the last q_len cache rows are the new tokens: token t may not see the ones after it
        causal = torch.zeros(q_len, L)
        for t_ in range(q_len):
            causal[t_, L - q_len + t_ + 1:] = float("-inf")
        got = K.group_query_attentionv2(qd, kd, vd, attn_mask=causal.to(dtype).to(DEV))
        check(got, O.gqa_dense_multi(q, k, v, causal), dtype, f"q_len {q_len} causal")
        # each query token alone is the single-step call
        one = K.group_query_attention(qd[:, :, 1:2].contiguous(), kd, vd)
        check(K.group_query_attentionv2(qd, kd, vd)[:, :, 1:2], one.float().cpu(), dtype, "one token of the burst")
    if dtype != torch.float32:
        q4 = torch.zeros(b, H * 4, D, dtype=dtype, device=DEV)
        assert ops.plan(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=q4, k=kd.transpose(1, 2), v=vd.transpose(1, 2),
                        sm_scale=1.0) == "dense_tc"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("case", [(3, 32, 16, 128), (2, 5, 3, 512), (1, 7, 1, 64)])
def test_merge_warp_kernel_agrees_with_block_kernel_bit_for_bit(dtype, case):
    """xkv_merge without a value projection runs one warp per row when the partial rows are 16-byte aligned and the
    block-per-row kernel otherwise: same weights, same order of additions, so the two give the same bits.  The
    misaligned copy of the same partials (shifted by one float inside a larger buffer) takes the block kernel.
    Also against the plain formula."""
    b, H, S, dim = case
    g = torch.Generator(device="cuda").manual_seed(5)
    part = torch.randn(b, H, S, dim, generator=g, device="cuda")
    lse = torch.randn(b, H, S, generator=g, device="cuda") * 3
    if S > 2:
        lse[:, :, 1] = float("-inf")                       # an empty split drops out
    lib = _C.load()
    stream = torch.cuda.current_stream().cuda_stream

    def run(p):
        out = torch.empty(b, H, dim, dtype=dtype, device="cuda")
        rc = lib.xkv_merge(p.data_ptr(), lse.data_ptr(), out.data_ptr(), _C.dtype_code(out), b, H, S, dim,
                           out.stride(0), out.stride(1), stream)
        _C.check(rc, "xkv_merge")
        return out

    aligned = run(part)
    buf = torch.empty(part.numel() + 1, device="cuda")
    shifted = buf[1:].view_as(part)
    shifted.copy_(part)
    assert shifted.data_ptr() % 16 != 0 and part.data_ptr() % 16 == 0
    assert torch.equal(aligned, run(shifted))
    w = torch.softmax(lse.double(), dim=-1)
    want = (w.unsqueeze(-1) * part.double()).sum(2)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (aligned.double() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())


def test_decode_call_replays_from_a_cuda_graph():
    """A decode call allocates nothing, reads no status and launches a fixed sequence of kernels, so it can be
    captured in a CUDA graph after one eager warm-up call and replayed: the replay works on the tensors' CURRENT
    contents (new queries written into the same buffers) and matches the eager call bit for bit."""
    b, H, KVH, L, D, R = 4, 32, 8, 1024, 128, 256
    g = torch.Generator(device="cuda").manual_seed(9)
    q = torch.randn(b, H, 1, D, generator=g, device="cuda").bfloat16()
    A = torch.randn(b, L, R, generator=g, device="cuda").bfloat16()
    B = (torch.randn(R, KVH * D, generator=g, device="cuda") / R ** 0.5).bfloat16()
    V = torch.randn(b, KVH, L, D, generator=g, device="cuda").bfloat16()
    f = lambda: K.recon_rope_decode(q, A, B, V, theta=5e5)
    f()                                              # eager warm-up: per-device look-ups happen here
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        f()                                          # the workspace of the capture stream exists before capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = f()
    q.copy_(torch.randn(b, H, 1, D, generator=g, device="cuda").bfloat16())     # a new step's queries, same buffer
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, f())
    rc, detail = _C.last_status(torch.device("cuda"))
    assert rc == 0, detail
