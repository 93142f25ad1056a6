"""GPU parity of the two-pass decode (tensor-core logits pass + shared-latent P.V pass): factorized
values behind RoPE-reconstructed keys (single layer and cross-layer groups) and behind dense keys."""
import pytest
import torch

import kernel_collections_b200 as K
from kernel_collections_b200 import _C, ops
from kernel_collections_b200.attention import as_key_proj
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
KVH, D = 8, 128


def close(got, want, what, ta=2e-2, tr=1e-2):
    assert torch.isfinite(got.float()).all(), what
    ma, rel = O.error_metrics(got, want)
    assert ma <= ta * max(1.0, want.abs().max().item()) and rel <= tr, f"{what}: max_abs={ma:.3e} rel_l2={rel:.3e}"


def b4(B, b):
    return B.view(B.shape[0], KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(2, 4, 700, 128, 256), (1, 8, 1029, 256, 128), (3, 4, 31, 64, 1024)])
def test_recon_rope_with_factorized_values(dtype, case):
    b, G, L, R, Rv = case
    theta = 500000.0
    g = torch.Generator().manual_seed(51)
    H = KVH * G
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    A = torch.randn(b, L, R, generator=g).to(dtype)
    B = (torch.randn(R, KVH * D, generator=g) / R ** 0.5).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    Bv = (torch.randn(Rv, KVH * D, generator=g) / Rv ** 0.5).to(dtype)
    qd, Ad, Bd, Avd, Bvd = (x.to(DEV) for x in (q, A, B, Av, Bv))
    kw = dict(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_LATENT, q=qd[:, :, 0], k=Ad, k_proj=as_key_proj(Bd, D),
              v=Avd, v_proj=as_key_proj(Bvd, D), sm_scale=D ** -0.5, theta=theta)
    assert ops.plan(**kw) == "two_pass"
    got = K.recon_rope_decode(qd, Ad, Bd, Avd, Bvd, theta=theta)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    want = O.recon_rope_decode(q, A, b4(B, b), Av, theta, value_B=b4(Bv, b))
    close(got, want, "two-pass vs oracle")
    gen = K.recon_rope_decode(qd, Ad, Bd, Avd, Bvd, theta=theta, force_generic=True)
    close(got, gen.float().cpu(), "two-pass vs portable kernel", 1e-2, 6e-3)
    assert torch.equal(got, K.recon_rope_decode(qd, Ad, Bd, Avd, Bvd, theta=theta))
    # the reference's own entry point for this mode (unscaled logits; q scaled down by the caller)
    qs = (q * D ** -0.5).to(dtype)
    Bb, Bvb = b4(B, b).contiguous(), b4(Bv, b).contiguous()
    got2 = K.group_query_attention_factorized_RoPE(qs.to(DEV), Ad, Bb.to(DEV), Avd, Bvb.to(DEV), theta=theta)
    close(got2, O.gqa_factorized_rope(qs, A, Bb, Av, Bvb, theta), "group_query_attention_factorized_RoPE")


@pytest.mark.parametrize("dtype", [torch.bfloat16])
@pytest.mark.parametrize("NL,b,L,R,Rv,G", [(4, 2, 600, 128, 256, 4), (2, 1, 1500, 64, 512, 8)])
def test_group_with_shared_value_latent(dtype, NL, b, L, R, Rv, G):
    theta = 500000.0
    g = torch.Generator().manual_seed(52)
    H = KVH * G
    A = torch.randn(b, L, R, generator=g).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    qs = [torch.randn(b, H, 1, D, generator=g).to(dtype) for _ in range(NL)]
    Bs = [(torch.randn(R, KVH * D, generator=g) / R ** 0.5).to(dtype) for _ in range(NL)]
    Bvs = [(torch.randn(Rv, KVH * D, generator=g) / Rv ** 0.5).to(dtype) for _ in range(NL)]
    got = K.xkv_group_decode([x.to(DEV) for x in qs], A.to(DEV), [x.to(DEV) for x in Bs], Av.to(DEV),
                             [x.to(DEV) for x in Bvs], theta=theta)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    want = O.group_decode(qs, A, [b4(x, b) for x in Bs], Av, [b4(x, b) for x in Bvs], theta)
    for i in range(NL):
        close(got[i], want[i], f"group layer {i}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(2, 32, 8, 900, 384), (1, 16, 2, 64, 128), (2, 8, 8, 2049, 512)])
def test_dense_keys_with_factorized_values(dtype, case):
    b, H, kvh, L, Rv = case
    g = torch.Generator().manual_seed(53)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    k = torch.randn(b, kvh, L, D, generator=g).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    Bv = (torch.randn(b, kvh, Rv, D, generator=g) / Rv ** 0.5).to(dtype)
    qd, kd, Avd, Bvd = (x.to(DEV) for x in (q, k, Av, Bv))
    kw = dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_LATENT, q=qd[:, :, 0], k=kd.transpose(1, 2), v=Avd,
              v_proj=Bvd, sm_scale=D ** -0.5)
    assert ops.plan(**kw) == "two_pass"
    got = K.group_query_attention_factorized_v_only(qd, kd, Avd, Bvd)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    close(got, O.gqa_factorized_v_only(q, k, Av, Bv), "v_only two-pass vs oracle")
    assert torch.equal(got, K.group_query_attention_factorized_v_only(qd, kd, Avd, Bvd))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Rv", [128, 384, 512, 1024])
def test_rising_logits_force_the_tmem_rescale(dtype, Rv):
    """Logits that climb along the context, each 64-token tile topping the previous one by about 12 log2
    units: the second pass's lazily updated reference maximum has to move on nearly every tile, so
    the in-place rescale of the output rows held in tensor memory runs throughout.  Value ranks 128
    (one narrow MMA per k-step), 384 (a wide and a narrow one), 512 and 1024 (two column blocks)."""
    b, H, kvh, L = 2, 32, 8, 1000
    g = torch.Generator().manual_seed(54)
    u = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
    q = (4.0 * u + 0.05 * torch.randn(b, H, 1, D, generator=g)).to(dtype)
    ramp = (torch.arange(L, dtype=torch.float32) / 64.0 * 23.5)[None, None, :, None]
    k = (ramp * u + 0.05 * torch.randn(b, kvh, L, D, generator=g)).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    Bv = (torch.randn(b, kvh, Rv, D, generator=g) / Rv ** 0.5).to(dtype)
    qd, kd, Avd, Bvd = (x.to(DEV) for x in (q, k, Av, Bv))
    s = (k[0, 0].float() @ q[0, 0, 0].float()) * D ** -0.5 * 1.4427              # head 0, log2 units
    assert s[64:128].max() - s[:64].max() > 8.0 and s[-64:].max() - s[-128:-64].max() > 8.0   # the premise of the test
    got = K.group_query_attention_factorized_v_only(qd, kd, Avd, Bvd)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    close(got, O.gqa_factorized_v_only(q, k, Av, Bv), f"rising logits, value rank {Rv}")
    assert torch.equal(got, K.group_query_attention_factorized_v_only(qd, kd, Avd, Bvd))


def test_group_with_more_than_128_stacked_heads():
    """Eight layers of 32 heads share one value latent: 256 stacked head rows, i.e. two head blocks of
    the second pass, each streaming the latent once."""
    NL, b, L, R, Rv, G, theta = 8, 2, 700, 64, 256, 4, 500000.0
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(55)
    H = KVH * G
    A = torch.randn(b, L, R, generator=g).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    qs = [torch.randn(b, H, 1, D, generator=g).to(dtype) for _ in range(NL)]
    Bs = [(torch.randn(R, KVH * D, generator=g) / R ** 0.5).to(dtype) for _ in range(NL)]
    Bvs = [(torch.randn(Rv, KVH * D, generator=g) / Rv ** 0.5).to(dtype) for _ in range(NL)]
    got = K.xkv_group_decode([x.to(DEV) for x in qs], A.to(DEV), [x.to(DEV) for x in Bs], Av.to(DEV),
                             [x.to(DEV) for x in Bvs], theta=theta)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    want = O.group_decode(qs, A, [b4(x, b) for x in Bs], Av, [b4(x, b) for x in Bvs], theta)
    for i in range(NL):
        close(got[i], want[i], f"8-layer group, layer {i}")


def test_second_pass_kernels_agree():
    """The tcgen05 second pass (default) against the mma.sync one (XKV_FLAG_PV_MMA_SYNC) on one call."""
    b, G, L, R, Rv, theta = 2, 4, 1500, 128, 512, 500000.0
    g = torch.Generator().manual_seed(56)
    H = KVH * G
    q = torch.randn(b, H, 1, D, generator=g).bfloat16().to(DEV)
    A = torch.randn(b, L, R, generator=g).bfloat16().to(DEV)
    B = (torch.randn(R, KVH * D, generator=g) / R ** 0.5).bfloat16().to(DEV)
    Av = torch.randn(b, L, Rv, generator=g).bfloat16().to(DEV)
    Bv = (torch.randn(Rv, KVH * D, generator=g) / Rv ** 0.5).bfloat16().to(DEV)
    got = K.recon_rope_decode(q, A, B, Av, Bv, theta=theta)
    alt = K.recon_rope_decode(q, A, B, Av, Bv, theta=theta, pv_mma_sync=True)
    close(got, alt.float().cpu(), "tcgen05 vs mma.sync second pass", 4e-3, 3e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(1, 32, 8, 4096, 256), (3, 64, 8, 1000, 128), (2, 8, 8, 130, 512), (2, 32, 2, 777, 192)])
def test_factorized_keys_with_dense_values(dtype, case):
    """Factorized K without RoPE in front of dense V (the reference's k_only fused kernel,
    flash_recontruction/fused_attention/no_pe/v1_k_only.py:368-465; configuration 1's dataflow): logits on
    the shared-latent tensor-core kernel in absorbed order, softmax and P.V on the dense-value kernel."""
    from kernel_collections_b200 import flash_recontruction as FR
    b, H, kvh, L, R = case
    g = torch.Generator().manual_seed(57)
    q = torch.randn(b, H, D, generator=g).to(dtype)
    A = torch.randn(b, L, R, generator=g).to(dtype)
    Bk = (torch.randn(b, kvh, R, D, generator=g) / R ** 0.5).to(dtype)
    V = torch.randn(b, L, kvh, D, generator=g).to(dtype)
    qd, Ad, Bd, Vd = (x.to(DEV) for x in (q, A, Bk, V))
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_DENSE, q=qd, k=Ad, k_proj=Bd, v=Vd, sm_scale=D ** -0.5)
    assert ops.plan(**kw) == "two_pass"
    o = torch.empty(b, H, D, dtype=dtype, device=DEV)
    got = FR.gqa_xKV_no_pe_k_only(qd, Ad, Bd, Vd, o, torch.full((b,), 4, dtype=torch.int32, device=DEV), 4, sm_scale=D ** -0.5)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    assert got is o
    close(got, O.xkv_fused_k_only(q, A, Bk, V, sm_scale=D ** -0.5), "k_only two-pass vs oracle")
    gen = ops.decode(entry="xkv_absorbed_decode", force_generic=True, **kw)
    close(got, gen.float().cpu(), "k_only two-pass vs portable kernel", 1e-2, 6e-3)
    assert torch.equal(got, ops.decode(entry="xkv_absorbed_decode", **kw))
    # ragged rows, NaN past each row's length
    lens = [L, 1, L // 2 + 3][:b]
    Ap, Vp = A.clone(), V.clone()
    for i, n in enumerate(lens):
        Ap[i, n:] = float("nan")
        Vp[i, n:] = float("nan")
    got_r = ops.decode(entry="xkv_absorbed_decode", **dict(kw, k=Ap.to(DEV), v=Vp.to(DEV),
                                                           kv_lens=torch.tensor(lens, dtype=torch.int32, device=DEV)))
    for i, n in enumerate(lens):
        close(got_r[i:i + 1], O.xkv_fused_k_only(q[i:i + 1], A[i:i + 1, :n], Bk[i:i + 1], V[i:i + 1, :n], sm_scale=D ** -0.5),
              f"k_only ragged row {i}")


def test_v_only_group_streams_the_shared_latent_once():
    """Four layers with their own dense keys and one shared value latent as ONE group call (the heads of all
    layers stacked for the value pass): every layer against the oracle and against its single-layer call."""
    NL, b, H, kvh, L, Rv = 4, 2, 32, 8, 900, 256
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(58)
    qs = [torch.randn(b, H, 1, D, generator=g).to(dtype) for _ in range(NL)]
    ks = [torch.randn(b, kvh, L, D, generator=g).to(dtype) for _ in range(NL)]
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    Bvs = [(torch.randn(Rv, kvh * D, generator=g) / Rv ** 0.5).to(dtype) for _ in range(NL)]
    Avd = Av.to(DEV)
    got = K.xkv_group_decode_v_only([x.to(DEV) for x in qs], [x.to(DEV) for x in ks], Avd, [x.to(DEV) for x in Bvs])
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    for i in range(NL):
        Bv4 = b4(Bvs[i], b).contiguous()
        close(got[i], O.gqa_factorized_v_only(qs[i], ks[i], Av, Bv4), f"v-only group layer {i}")
        single = K.group_query_attention_factorized_v_only(qs[i].to(DEV), ks[i].to(DEV), Avd, Bv4.to(DEV))
        close(got[i], single.float().cpu(), f"v-only group layer {i} vs single-layer call", 4e-3, 3e-3)
