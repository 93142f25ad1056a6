"""GPU parity of the tcgen05 key-reconstruction kernel (the path aligned bf16 / fp16 shapes take):
against the CPU oracle, against the portable kernel on the same inputs, over tails, ranks, split
counts, head groupings and layouts, plus the bounded-wait status word."""
import pytest
import torch

import kernel_collections_b200 as K
from kernel_collections_b200 import flash_recontruction as FR
from kernel_collections_b200 import _C, ops
from kernel_collections_b200.attention import as_key_proj
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
KVH, D = 8, 128


def make(b, L, R, G, dtype, seed, batched_B=False):
    g = torch.Generator().manual_seed(seed)
    H = KVH * G
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    A = torch.randn(b, L, R, generator=g).to(dtype)
    if batched_B:
        B = (torch.randn(b, KVH, R, D, generator=g) / R ** 0.5).to(dtype)
    else:
        B = (torch.randn(R, KVH * D, generator=g) / R ** 0.5).to(dtype)
    V = torch.randn(b, L, KVH, D, generator=g).to(dtype)
    return q, A, B, V


def b4(B, b):
    return B if B.dim() == 4 else B.view(B.shape[0], KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1)


def assert_close(got, want, what, max_abs_tol=2e-2, rel_tol=1e-2):
    assert torch.isfinite(got.float()).all(), what
    ma, rel = O.error_metrics(got, want)
    scale = max(1.0, want.abs().max().item())
    assert ma <= max_abs_tol * scale and rel <= rel_tol, f"{what}: max_abs={ma:.3e} rel_l2={rel:.3e}"


def status_ok():
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, f"device status {rc} detail {detail}"


CASES = [  # b, L, R, G
    (1, 1, 64, 4), (1, 127, 64, 4), (2, 128, 64, 4), (1, 129, 128, 4), (3, 1000, 192, 4),
    (2, 4101, 512, 4), (2, 700, 128, 8), (1, 2048, 1024, 8),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_logits_tc(dtype, case):
    b, L, R, G = case
    theta = 500000.0
    q, A, B, V = make(b, L, R, G, dtype, seed=11)
    kw = dict(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=q[:, :, 0].to(DEV), k=A.to(DEV),
              k_proj=as_key_proj(B.to(DEV), D), logits_only=True, sm_scale=1.0, theta=theta)
    assert ops.plan(**kw) == "recon_tc"
    got = ops.decode(entry="xkv_qab_logits", **kw)
    status_ok()
    want = O.qab_rope(q, A, b4(B, b), theta)[:, :, 0]
    assert_close(got, want, "tc logits vs oracle")
    gen = ops.decode(entry="xkv_qab_logits", force_generic=True, **kw)
    assert_close(got, gen.float().cpu(), "tc logits vs portable kernel")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_fused_decode_tc(dtype, case):
    b, L, R, G = case
    theta = 500000.0
    q, A, B, V = make(b, L, R, G, dtype, seed=12, batched_B=(R == 128))
    qd, Ad, Bd, Vd = q.to(DEV), A.to(DEV), B.to(DEV), V.to(DEV)
    got = K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=theta)
    status_ok()
    want = O.recon_rope_decode(q, A, b4(B, b), V.transpose(1, 2), theta)
    assert_close(got, want, "tc fused decode vs oracle")
    gen = K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=theta, force_generic=True)
    assert_close(got, gen.float().cpu(), "tc fused decode vs portable kernel", 1e-2, 5e-3)
    # head-major V layout (b, KVH, L, D) contiguous
    got2 = K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2).contiguous(), theta=theta)
    assert torch.equal(got, got2)
    # bit-identical on repeat (fixed merge order)
    assert torch.equal(got, K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=theta))


def test_tc_path_is_selected_for_the_benchmark_shape():
    q = torch.zeros(16, 32, 128, dtype=torch.bfloat16, device=DEV)
    A = torch.zeros(16, 256, 512, dtype=torch.bfloat16, device=DEV)
    B = torch.zeros(512, 1024, dtype=torch.bfloat16, device=DEV)
    V = torch.zeros(16, 256, 8, 128, dtype=torch.bfloat16, device=DEV)
    kw = dict(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=q, k=A, k_proj=as_key_proj(B, 128), v=V,
              sm_scale=1.0, theta=5e5)
    assert ops.plan(**kw) == "recon_tc"
    assert ops.plan(force_generic=True, **kw) == "generic"
    # fp32 and odd ranks stay on the portable kernel
    assert ops.plan(**{**kw, "q": q.float(), "k": A.float(), "k_proj": as_key_proj(B.float(), 128), "v": V.float()}) == "generic"
    assert ops.plan(**{**kw, "k": A[..., :500], "k_proj": as_key_proj(B[:500], 128)}) == "generic"


def test_rope_positions_and_user_table():
    """k_position_offset shifts the key positions; a caller-made table gives the same logits."""
    dtype, b, L, R, G, theta = torch.bfloat16, 2, 300, 128, 4, 1e7
    q, A, B, V = make(b, L, R, G, dtype, seed=13)
    qd, Ad, Bd = q.to(DEV), A.to(DEV), B.to(DEV)
    B4 = b4(B, b)
    want = O.qab_rope(q, A, B4, theta)
    got = FR.qAB_rope_v1(qd, Ad, as_key_proj(Bd, D).expand(b, -1, -1, -1), theta=theta)
    assert_close(got, want, "qAB_rope_v1 (tc)")
    cos, sin = O.rope_cos_sin(D, L, theta)
    table = torch.cat([sin[:, : D // 2], cos[:, : D // 2]], dim=-1).to(DEV)
    got2 = FR.qAB_rope_v2(qd, Ad, as_key_proj(Bd, D).expand(b, -1, -1, -1), table)
    assert_close(got2, want, "qAB_rope_v2 (tc, user table)")
    off = 4096
    Kr = O.reconstruct_rope_keys(A, B4, theta, position_offset=off)
    want_off = O.gqa_dense(q, Kr, V.transpose(1, 2))
    got_off = K.recon_rope_decode(qd, Ad, Bd, V.to(DEV).transpose(1, 2), theta=theta, k_position_offset=off)
    assert_close(got_off, want_off, "k_position_offset")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("NL,b,L,R,G", [(4, 2, 700, 128, 4), (3, 1, 2048, 256, 8), (8, 1, 130, 64, 4)])
def test_group_decode_single_launch(dtype, NL, b, L, R, G):
    """Cross-layer group on the tensor-core kernel: one launch, layers fastest over the grid; every
    layer must match its own single-layer result bit for bit and the oracle within tolerance."""
    theta = 500000.0
    g = torch.Generator().manual_seed(21)
    H = KVH * G
    A = torch.randn(b, L, R, generator=g).to(dtype)
    qs = [torch.randn(b, H, 1, D, generator=g).to(dtype) for _ in range(NL)]
    Bs = [(torch.randn(R, KVH * D, generator=g) / R ** 0.5).to(dtype) for _ in range(NL)]
    Vs = [torch.randn(b, L, KVH, D, generator=g).to(dtype) for _ in range(NL)]
    Ad = A.to(DEV)
    qd, Bd, Vd = [x.to(DEV) for x in qs], [x.to(DEV) for x in Bs], [x.to(DEV) for x in Vs]
    got = K.xkv_group_decode(qd, Ad, Bd, [v.transpose(1, 2) for v in Vd], theta=theta)
    status_ok()
    for i in range(NL):
        want = O.recon_rope_decode(qs[i], A, b4(Bs[i], b), Vs[i].transpose(1, 2), theta)
        assert_close(got[i], want, f"group layer {i} vs oracle")
        single = K.recon_rope_decode(qd[i], Ad, Bd[i], Vd[i].transpose(1, 2), theta=theta)
        # same math, possibly a different split count: equal up to the merge's fp32 rounding
        assert_close(got[i], single.float().cpu(), f"group layer {i} vs single-layer call", 4e-3, 2e-3)
    again = K.xkv_group_decode(qd, Ad, Bd, [v.transpose(1, 2) for v in Vd], theta=theta)
    for i in range(NL):
        assert torch.equal(got[i], again[i])


@pytest.mark.parametrize("case", [(2, 700, 128, 4), (1, 2048, 512, 8), (3, 129, 64, 4), (2, 4101, 256, 4)])
def test_cta_pair_variant(case):
    """The CTA-pair variant (tcgen05 cta_group::2: two CTAs share every MMA, each loading half
    of the B chunk) must agree with the oracle and with the single-CTA kernel, odd tile counts and
    phantom tiles included."""
    b, L, R, G = case
    dtype, theta = torch.bfloat16, 500000.0
    q, A, B, V = make(b, L, R, G, dtype, seed=17)
    qd, Ad, Bd, Vd = q.to(DEV), A.to(DEV), B.to(DEV), V.to(DEV)
    single = K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=theta, cta_pair=False)
    got = K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=theta, cta_pair=True)
    status_ok()
    want = O.recon_rope_decode(q, A, b4(B, b), V.transpose(1, 2), theta)
    assert_close(got, want, "pair variant vs oracle")
    assert_close(got, single.float().cpu(), "pair variant vs single-CTA kernel", 4e-3, 2e-3)
    assert torch.equal(got, K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=theta, cta_pair=True))
    logits = ops.decode(entry="xkv_qab_logits", score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE,
                        q=qd[:, :, 0], k=Ad, k_proj=as_key_proj(Bd, D), logits_only=True, sm_scale=1.0, theta=theta,
                        extra_flags=_C.FLAG_RECON_PAIR)
    status_ok()
    assert_close(logits, O.qab_rope(q, A, b4(B, b), theta)[:, :, 0], "pair variant logits")
