"""GPU parity of the shared-latent decode kernel (absorbed factorized K / V and MLA; bf16 / fp16,
ranks in multiples of 64 / 128): against the CPU oracle and the portable kernel."""
import pytest
import torch

import kernel_collections_b200 as K
from kernel_collections_b200 import flash_recontruction as FR
from kernel_collections_b200 import flash_decoding as FD
from kernel_collections_b200 import _C, ops
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(got, want, what, ta=2e-2, tr=1e-2):
    assert torch.isfinite(got.float()).all(), what
    ma, rel = O.error_metrics(got, want)
    assert ma <= ta * max(1.0, want.abs().max().item()) and rel <= tr, f"{what}: max_abs={ma:.3e} rel_l2={rel:.3e}"


def status_ok():
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail


FACT = [  # b, H, KVH, D, L, Rk, Rv
    (2, 32, 8, 128, 1000, 256, 384), (1, 32, 8, 128, 33, 64, 128), (3, 16, 4, 64, 257, 128, 128),
    (1, 64, 8, 128, 2048, 512, 512), (2, 8, 2, 128, 700, 768, 512), (1, 40, 8, 128, 31, 192, 256),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", FACT)
def test_factorized_absorbed(dtype, case):
    b, H, KVH, D, L, Rk, Rv = case
    g = torch.Generator().manual_seed(41)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    Ak = torch.randn(b, L, Rk, generator=g).to(dtype)
    Bk = (torch.randn(b, KVH, Rk, D, generator=g) / Rk ** 0.5).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    Bv = (torch.randn(b, KVH, Rv, D, generator=g) / Rv ** 0.5).to(dtype)
    qd, Akd, Bkd, Avd, Bvd = (x.to(DEV) for x in (q, Ak, Bk, Av, Bv))
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=qd[:, :, 0], k=Akd, k_proj=Bkd, v=Avd,
              v_proj=Bvd, sm_scale=D ** -0.5)
    assert ops.plan(**kw) == "latent_tc"
    got = K.group_query_attention_factorized(qd, Akd, Bkd, Avd, Bvd)
    status_ok()
    close(got, O.gqa_factorized(q, Ak, Bk, Av, Bv), "factorized (latent_tc) vs oracle")
    gen = ops.decode(entry="xkv_absorbed_decode", force_generic=True, **kw)
    close(got[:, :, 0], gen.float().cpu(), "latent_tc vs portable kernel", 1e-2, 6e-3)
    assert torch.equal(got, K.group_query_attention_factorized(qd, Akd, Bkd, Avd, Bvd))
    # fused xKV entry point with its own scale and in-place output
    o = torch.zeros(b, H, D, dtype=dtype, device=DEV)
    FR.gqa_xKV_no_pe(qd[:, :, 0], Akd, Bkd, Avd, Bvd, o, torch.full((b,), 8, dtype=torch.int32, device=DEV), 8, 0.07)
    close(o, O.xkv_fused(q[:, :, 0], Ak, Bk, Av, Bv, 0.07), "gqa_xKV_no_pe (latent_tc)")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(8, 32, 8, 128, 700, 256, 384), (5, 16, 4, 64, 257, 128, 128), (16, 32, 8, 128, 3000, 256, 256)])
def test_factorized_absorbed_with_projections_shared_by_the_batch(dtype, case):
    """B_k / B_v as model weights (one copy, stride 0 over the batch) and 4 or more rows: both projections run as
    tensor-core products over the whole batch, the value one merging the KV splits as it stages them."""
    b, H, KVH, D, L, Rk, Rv = case
    g = torch.Generator().manual_seed(48)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    Ak = torch.randn(b, L, Rk, generator=g).to(dtype)
    Bk = (torch.randn(1, KVH, Rk, D, generator=g) / Rk ** 0.5).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    Bv = (torch.randn(1, KVH, Rv, D, generator=g) / Rv ** 0.5).to(dtype)
    qd, Akd, Avd = (x.to(DEV) for x in (q, Ak, Av))
    Bkd, Bvd = Bk.to(DEV).expand(b, -1, -1, -1), Bv.to(DEV).expand(b, -1, -1, -1)
    got = K.group_query_attention_factorized(qd, Akd, Bkd, Avd, Bvd)
    status_ok()
    close(got, O.gqa_factorized(q, Ak, Bk.expand(b, -1, -1, -1), Av, Bv.expand(b, -1, -1, -1)), "factorized, shared B, vs oracle")
    per_row = K.group_query_attention_factorized(qd, Akd, Bkd.contiguous(), Avd, Bvd.contiguous())
    close(got, per_row.float().cpu(), "shared B vs per-row B", 4e-3, 3e-3)
    assert torch.equal(got, K.group_query_attention_factorized(qd, Akd, Bkd, Avd, Bvd))


MLA = [  # b, H, lora, rope, L
    (2, 16, 128, 64, 203), (1, 128, 512, 64, 1500), (3, 64, 256, 64, 64), (1, 32, 512, 64, 4097),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", MLA)
def test_mla(dtype, case):
    b, H, lora, rope, L = case
    g = torch.Generator().manual_seed(42)
    qn = (torch.randn(b, H, lora, generator=g) / 3).to(dtype)
    qr = (torch.randn(b, H, rope, generator=g) / 3).to(dtype)
    c = (torch.randn(b, L, 1, lora, generator=g) / 3).to(dtype)
    kr = (torch.randn(b, L, 1, rope, generator=g) / 3).to(dtype)
    qnd, qrd, cd, krd = (x.to(DEV) for x in (qn, qr, c, kr))
    got = FD.mla2.mla_decode_attention_fwd(qnd, qrd, cd, krd, 0.3)
    status_ok()
    close(got, O.mla_decode(qn, qr, c, kr, 0.3), "mla2 fwd (latent_tc)")
    # absorbed form with W_uk / W_uv
    nope, vd = 128, 128
    qq = torch.randn(b, H, nope, generator=g).to(dtype)
    Wk = (torch.randn(H, nope, lora, generator=g) / lora ** 0.5).to(dtype)
    Wv = (torch.randn(H, lora, vd, generator=g) / lora ** 0.5).to(dtype)
    sc = (nope + rope) ** -0.5
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=qq.to(DEV), k=cd[:, :, 0], v=cd[:, :, 0],
              k_proj=Wk.to(DEV).permute(0, 2, 1).unsqueeze(0), v_proj=Wv.to(DEV).unsqueeze(0), q_tail=qrd,
              k_tail=krd[:, :, 0], sm_scale=sc, num_kv_heads=1)
    assert ops.plan(**kw) == ("latent_pair" if H >= 64 else "latent_tc")
    got2 = K.mla_absorbed_decode(qq.to(DEV), qrd, cd[:, :, 0], krd[:, :, 0], Wk.to(DEV), Wv.to(DEV), sc)
    status_ok()
    close(got2, O.mla_absorbed(qq, qr, c[:, :, 0], kr[:, :, 0], Wk, Wv, sc), "mla_absorbed_decode (latent_tc)")
    assert torch.equal(got2, K.mla_absorbed_decode(qq.to(DEV), qrd, cd[:, :, 0], krd[:, :, 0], Wk.to(DEV), Wv.to(DEV), sc))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("k_major", [False, True])
@pytest.mark.parametrize("case", [(5, 64, 256, 64, 300), (70, 128, 512, 64, 130), (16, 72, 128, 0, 90), (60, 128, 512, 64, 1280)])
def test_mla_absorbed_with_batch_wide_projections(dtype, k_major, case):
    """W_uk folded into the queries and W_uv applied to the merged latent rows as tensor-core products over the
    whole batch (projection matrices shared by the batch, 4 rows or more): batches that do not fill a 64-row
    strip and ones that need two, head counts off the block size, and both memory orders of the matrices
    (contraction index contiguous or output column contiguous), against the oracle.  The batch of 5 is cut into
    several KV splits per row, which the value projection merges while it stages the partial rows."""
    b, H, lora, rope, L = case
    g = torch.Generator().manual_seed(46)
    nope, vd = 128, 128
    qq = torch.randn(b, H, nope, generator=g).to(dtype)
    qr = (torch.randn(b, H, rope, generator=g) / 3).to(dtype) if rope else None
    c = (torch.randn(b, L, lora, generator=g) / 3).to(dtype)
    kr = (torch.randn(b, L, rope, generator=g) / 3).to(dtype) if rope else None
    Wk = (torch.randn(H, nope, lora, generator=g) / lora ** 0.5).to(dtype)
    Wv = (torch.randn(H, lora, vd, generator=g) / lora ** 0.5).to(dtype)
    sc = (nope + rope) ** -0.5
    dev = lambda x: None if x is None else x.to(DEV)
    # k_proj is indexed (batch, head, rank, head_dim), v_proj (batch, head, rank, value_dim)
    if k_major:     # the contraction index is the contiguous one: head_dim for W_uk, rank for W_uv
        kp = Wk.permute(0, 2, 1).contiguous().to(DEV).unsqueeze(0)
        vp = Wv.permute(0, 2, 1).contiguous().to(DEV).permute(0, 2, 1).unsqueeze(0)
    else:           # the output column is the contiguous one
        kp = Wk.to(DEV).permute(0, 2, 1).unsqueeze(0)
        vp = Wv.to(DEV).unsqueeze(0)
    cd = dev(c)
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=dev(qq), k=cd, v=cd, k_proj=kp, v_proj=vp,
              q_tail=dev(qr), k_tail=dev(kr), sm_scale=sc, num_kv_heads=1)
    assert ops.plan(**kw) == "latent_pair"
    got = ops.decode(entry="xkv_mla_decode", **kw)
    status_ok()
    zr = torch.zeros(b, H, 0, dtype=dtype)
    zk = torch.zeros(b, L, 0, dtype=dtype)
    want = O.mla_absorbed(qq, qr if rope else zr, c, kr if rope else zk, Wk, Wv, sc)
    close(got, want, "latent_pair with batch-wide projections")
    assert torch.equal(got, ops.decode(entry="xkv_mla_decode", **kw))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(2, 32, 576, 512, 1100), (1, 16, 320, 256, 70), (1, 128, 576, 512, 333)])
def test_packed_single_kv_head_cache(dtype, case):
    """The packed MLA layout of flash_decoding.mla (keys = [latent | rope], values = a prefix of the
    keys, one KV head) is served by the shared-latent kernel; the aliased rows are read once."""
    b, H, Dk, Dv, L = case
    g = torch.Generator().manual_seed(43)
    q = (torch.randn(b, H, Dk, generator=g) / 3).to(dtype)
    kbuf = (torch.randn(b, L, 1, Dk, generator=g) / 3).to(dtype)
    qd, kd = q.to(DEV), kbuf.to(DEV)
    kw = dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=qd, k=kd, v=kd[..., :Dv], sm_scale=0.4)
    assert ops.plan(**kw) == ("latent_pair" if H >= 64 else "latent_tc")
    o = torch.zeros(b, H, Dv, dtype=dtype, device=DEV)
    assert FD.mla.decode_attention_fwd(qd, kd, kd[..., :Dv], o, 0.4) is None
    status_ok()
    close(o, O.flash_decode_gqa(q, kbuf, kbuf[..., :Dv], 0.4), "packed MLA cache (latent_tc)")
    # a separate value buffer of another width goes the same way
    vbuf = (torch.randn(b, L, 1, 128, generator=g) / 3).to(dtype)
    o2 = torch.zeros(b, H, 128, dtype=dtype, device=DEV)
    FD.mla.decode_attention_fwd(qd, kd, vbuf.to(DEV), o2, 0.4)
    close(o2, O.flash_decode_gqa(q, kbuf, vbuf, 0.4), "separate V buffer (latent_tc)")
    # the logit cap is not covered by the fast kernel and must still be right
    o3 = torch.zeros(b, H, Dv, dtype=dtype, device=DEV)
    FD.mla.decode_attention_fwd(qd, kd, kd[..., :Dv], o3, 0.4, 3.0)
    close(o3, O.flash_decode_gqa(q, kbuf, kbuf[..., :Dv], 0.4, logit_cap=3.0), "logit cap (portable)")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(2, 32, 8, 128, 1000, 256), (1, 64, 8, 128, 77, 128), (3, 8, 2, 64, 300, 512)])
def test_qab_no_pe_logits(dtype, case):
    """qAB without RoPE: absorbed logits q.(A.B)^T straight from the latent stream."""
    b, H, kvh, D, L, R = case
    g = torch.Generator().manual_seed(44)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    Ak = torch.randn(b, L, R, generator=g).to(dtype)
    Bk = (torch.randn(b, kvh, R, D, generator=g) / R ** 0.5).to(dtype)
    qd, Akd, Bkd = q.to(DEV), Ak.to(DEV), Bk.to(DEV)
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_DENSE, q=qd[:, :, 0], k=Akd, k_proj=Bkd,
              logits_only=True, sm_scale=1.0)
    assert ops.plan(**kw) == "latent_tc"
    want = O.qab_no_pe(q, Ak, Bk)
    for fn in (FR.qAB_no_pe_v1, FR.qAB_no_pe_v2, FR.qAB_no_pe_ref):
        got = fn(qd, Akd, Bkd)
        status_ok()
        close(got, want, fn.__name__ if hasattr(fn, "__name__") else "qAB_no_pe")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", [(2, 128, 512, 64, 5000, 512), (1, 64, 256, 64, 47, 256), (3, 100, 512, 64, 1000, 512),
                                  (1, 200, 384, 0, 777, 384), (2, 128, 256, 0, 300, 128)])
def test_cta_pair_kernel_against_oracle_and_mma_sync_kernel(dtype, case):
    """The tcgen05 CTA-pair kernel for shared latents (heads on M, the pair splitting the score
    contraction and the value columns, partial scores exchanged through distributed shared memory)
    against the oracle and against the mma.sync kernel on the same inputs: 128 heads, fewer than a
    block, more than a block, with and without the decoupled RoPE part, value columns that are a
    prefix of the key latent, ragged lengths, and logits that climb so the lazy rescale runs."""
    b, H, lora, rope, L, Rv = case
    g = torch.Generator().manual_seed(44)
    qn = (torch.randn(b, H, lora, generator=g) / 3).to(dtype)
    c = (torch.randn(b, L, lora, generator=g) / 3).to(dtype)
    qr = (torch.randn(b, H, rope, generator=g) / 3).to(dtype) if rope else None
    kr = (torch.randn(b, L, rope, generator=g) / 3).to(dtype) if rope else None
    dev = lambda x: None if x is None else x.to(DEV)
    cd = dev(c)                                  # values are a prefix of the key latent: one tensor, read once
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=dev(qn), k=cd, v=cd[..., :Rv], q_tail=dev(qr),
              k_tail=dev(kr), sm_scale=0.3, num_kv_heads=1)
    assert ops.plan(**kw) == "latent_pair"
    got = ops.decode(entry="xkv_mla_decode", **kw)
    status_ok()

    def ref(qn_, qr_, c_, kr_):
        s = torch.matmul(qn_.float(), c_.float().transpose(-1, -2))
        if qr_ is not None:
            s = s + torch.matmul(qr_.float(), kr_.float().transpose(-1, -2))
        return torch.matmul(torch.softmax(s * 0.3, -1), c_.float()[..., :Rv])

    close(got, ref(qn, qr, c, kr), "latent_pair vs eager math")
    alt = ops.decode(entry="xkv_mla_decode", extra_flags=_C.FLAG_LATENT_MMA_SYNC, **kw)
    close(got, alt.float().cpu(), "latent_pair vs mma.sync kernel", 4e-3, 3e-3)
    assert torch.equal(got, ops.decode(entry="xkv_mla_decode", **kw))
    # ragged lengths, NaN past each row's length
    lens = [L, 1, max(1, L // 2 + 5)][:b]
    cp = c.clone()
    krp = None if kr is None else kr.clone()
    for i, n in enumerate(lens):
        cp[i, n:] = float("nan")
        if krp is not None:
            krp[i, n:] = float("nan")
    cpd = dev(cp)
    kwr = dict(kw, k=cpd, v=cpd[..., :Rv], k_tail=dev(krp), kv_lens=torch.tensor(lens, dtype=torch.int32, device=DEV))
    got_r = ops.decode(entry="xkv_mla_decode", **kwr)
    status_ok()
    for i, n in enumerate(lens):
        want = ref(qn[i:i + 1], None if qr is None else qr[i:i + 1], c[i:i + 1, :n], None if kr is None else kr[i:i + 1, :n])
        close(got_r[i:i + 1], want, f"latent_pair ragged row {i}")
    # climbing logits: keys grow along the context in the direction all queries share
    u = torch.nn.functional.normalize(torch.randn(lora, generator=g), dim=0)
    q2 = (3.0 * u + 0.05 * torch.randn(b, H, lora, generator=g)).to(dtype)
    c2 = ((torch.arange(L, dtype=torch.float32) / 48.0 * 9.0)[None, :, None] * u + 0.05 * torch.randn(b, L, lora, generator=g)).to(dtype)
    c2d = dev(c2)
    kw2 = dict(kw, q=dev(q2), k=c2d, v=c2d[..., :Rv], sm_scale=0.4)
    got2 = ops.decode(entry="xkv_mla_decode", **kw2)
    status_ok()
    close(got2, torch.matmul(torch.softmax((torch.matmul(q2.float(), c2.float().transpose(-1, -2))
                                            + (0 if qr is None else torch.matmul(qr.float(), kr.float().transpose(-1, -2)))) * 0.4, -1),
                             c2.float()[..., :Rv]), "latent_pair with climbing logits")


def test_cta_pair_kernel_with_nearly_as_many_rows_as_pair_slots():
    """60 rows on the GPU's 74 CTA-pair slots: one KV split per row, one wave."""
    b, H, lora, rope, L = 60, 128, 512, 64, 1280
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(47)
    qn = (torch.randn(b, H, lora, generator=g) / 3).to(dtype)
    c = (torch.randn(b, L, lora, generator=g) / 3).to(dtype)
    qr = (torch.randn(b, H, rope, generator=g) / 3).to(dtype)
    kr = (torch.randn(b, L, rope, generator=g) / 3).to(dtype)
    cd = c.to(DEV)
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=qn.to(DEV), k=cd, v=cd, q_tail=qr.to(DEV),
              k_tail=kr.to(DEV), sm_scale=0.3, num_kv_heads=1)
    assert ops.plan(**kw) == "latent_pair"
    got = ops.decode(entry="xkv_mla_decode", **kw)
    status_ok()
    s = (torch.matmul(qn.float(), c.float().transpose(-1, -2)) + torch.matmul(qr.float(), kr.float().transpose(-1, -2))) * 0.3
    close(got, torch.matmul(torch.softmax(s, -1), c.float()), "latent_pair with uneven splits")
    assert torch.equal(got, ops.decode(entry="xkv_mla_decode", **kw))


@pytest.mark.parametrize("case", [(2, 64, 256, 0, 900, 256), (1, 96, 256, 64, 400, 128)])
def test_cta_pair_kernel_with_a_separate_value_latent(case):
    """Key latent and value latent as two tensors (absorbed factorized cache with 64 or more heads): the
    pair splits the value columns and deals the key blocks out between its CTAs."""
    b, H, rk, rope, L, Rv = case
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(45)
    qn = (torch.randn(b, H, rk, generator=g) / 3).to(dtype)
    Ak = (torch.randn(b, L, rk, generator=g) / 3).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    qr = (torch.randn(b, H, rope, generator=g) / 3).to(dtype) if rope else None
    kr = (torch.randn(b, L, rope, generator=g) / 3).to(dtype) if rope else None
    dev = lambda x: None if x is None else x.to(DEV)
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=dev(qn), k=dev(Ak), v=dev(Av), q_tail=dev(qr),
              k_tail=dev(kr), sm_scale=0.3, num_kv_heads=1)
    assert ops.plan(**kw) == "latent_pair"
    got = ops.decode(entry="xkv_mla_decode", **kw)
    status_ok()
    s = torch.matmul(qn.float(), Ak.float().transpose(-1, -2))
    if rope:
        s = s + torch.matmul(qr.float(), kr.float().transpose(-1, -2))
    close(got, torch.matmul(torch.softmax(s * 0.3, -1), Av.float()), "latent_pair, separate value latent")
