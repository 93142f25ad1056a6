"""GPU parity at the five benchmark configurations' own sizes, through the C ABI, against the CPU
oracle in fp32 on the dtype-rounded inputs.

Split selection, tiles per CTA and the length of the online-softmax recurrences all depend on the
problem size, so the shapes here are the full ones: configuration 1 exactly (fp32), configuration
2 with every batch row on the GPU and four rows checked, configurations 3, 4 and 5 at full context /
rank / head count with the batch cut to what the CPU oracle checks in seconds (batch rows are
independent).  Tolerances: fp32 max-abs and relative L2 <= 1e-4; bf16 max-abs <= 2e-2 (relative to
max(1, |want|max)) and relative L2 <= 1e-2.
"""
import math

import pytest
import torch

import kernel_collections_b200 as K
from kernel_collections_b200 import _C, ops
from kernel_collections_b200 import flash_recontruction as FR
from kernel_collections_b200.attention import as_key_proj
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
KVH, D = 8, 128


def close(got, want, what, ta=2e-2, tr=1e-2):
    assert torch.isfinite(got.float()).all(), what
    ma, rel = O.error_metrics(got, want)
    assert ma <= ta * max(1.0, want.abs().max().item()) and rel <= tr, f"{what}: max_abs={ma:.3e} rel_l2={rel:.3e}"
    return ma, rel


def status_ok():
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, f"device status {rc} detail {detail}"


def b4(B, b=1):
    """Shared (R, KVH*D) projection as the reference's (b, KVH, R, D)."""
    return B.view(B.shape[0], KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1)


def dev_randn(gen, *shape, dtype=torch.bfloat16, scale=1.0):
    t = torch.randn(*shape, generator=gen, device=DEV, dtype=torch.float32 if scale != 1.0 else dtype)
    return (t * scale).to(dtype) if scale != 1.0 else t


def test_config1_factorized_k_dense_v_fp32():
    """Configuration 1 exactly: fp32, batch 1, 32 / 8 heads, head_dim 128, context 4096, rank 256, no
    RoPE, dense V; inputs from torch.manual_seed(0) in the order A, B, V, q."""
    b, H, L, R = 1, 32, 4096, 256
    torch.manual_seed(0)
    A = torch.randn(b, L, R)
    B = torch.randn(R, KVH * D) / math.sqrt(R)
    V = torch.randn(b, L, KVH, D)
    q = torch.randn(b, H, D)
    B4 = b4(B).contiguous()
    # oracle: the reference's absorbed function with dense V written as an identity factorization
    eye = torch.eye(KVH * D).view(KVH * D, KVH, D).permute(1, 0, 2)[None].contiguous()
    want = O.gqa_factorized(q[:, :, None], A, B4, V.reshape(b, L, KVH * D), eye)[:, :, 0]
    want2 = O.xkv_fused_k_only(q, A, B4, V, sm_scale=D ** -0.5)
    assert O.error_metrics(want2, want)[1] < 1e-6
    qd, Ad, Bd, Vd = q.to(DEV), A.to(DEV), B4.to(DEV), V.to(DEV)
    o = torch.empty(b, H, D, device=DEV)
    got = FR.gqa_xKV_no_pe_k_only(qd, Ad, Bd, Vd, o, torch.full((b,), 8, dtype=torch.int32, device=DEV), 8,
                                  sm_scale=D ** -0.5)
    assert got is o
    close(got, want, "c1 via gqa_xKV_no_pe_k_only", 1e-4, 1e-4)
    got2 = K.group_query_attention_factorized(qd[:, :, None], Ad, Bd, Vd.reshape(b, L, KVH * D), eye.to(DEV))
    close(got2[:, :, 0], want, "c1 via group_query_attention_factorized (identity value factorization)", 1e-4, 1e-4)
    # the same shape in bf16 runs on a tensor-core path
    got3 = FR.gqa_xKV_no_pe_k_only_ref(qd.bfloat16(), Ad.bfloat16(), Bd.bfloat16(), Vd.bfloat16())
    want3 = O.xkv_fused_k_only(q.bfloat16(), A.bfloat16(), B4.bfloat16(), V.bfloat16(), sm_scale=1.0)
    close(got3, want3, "c1 shape in bf16 (unscaled eager name)")


def test_config2_full_size_sampled_rows():
    """Configuration 2 at full size (batch 16, context 16384, rank 512, bf16, theta 5e5, key positions
    0..L-1, query position L): every row runs on the GPU, rows 0, 15 and two seeded-random rows are
    checked against the oracle; both the single-CTA and the CTA-pair kernel."""
    from kernel_collections_b200 import synthetic
    cfg = synthetic.ReconRopeConfig()
    A, B, q, V = synthetic.recon_rope_inputs(cfg, seed=0)
    qr = O.rope_query(q, cfg.theta, cfg.kv_len)
    Ad, Bd, Vd, qd = A.to(DEV), B.to(DEV), V.to(DEV), qr.to(DEV)
    qk = K.rope_query(q.to(DEV), cfg.theta, cfg.kv_len).cpu()      # the library's own rotation: same up to one ulp
    assert ((qk.float() - qr.float()).abs() <= 2.0 ** -7 * qr.float().abs().clamp(min=1.0)).all()
    assert (qk != qr).float().mean().item() < 0.01
    rows = sorted({0, 15, *torch.randint(1, 15, (2,), generator=torch.Generator().manual_seed(2)).tolist()})
    want = {r: O.recon_rope_decode(qr[r:r + 1], A[r:r + 1], b4(B), V[r:r + 1].transpose(1, 2), cfg.theta) for r in rows}
    for pair in (False, True):
        got = K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=cfg.theta, cta_pair=pair)
        status_ok()
        for r in rows:
            close(got[r:r + 1], want[r], f"c2 row {r} (cta_pair={pair})")
    # logits of the same call (qAB_rope) on one row
    lg = FR.qAB_rope_v1(qd[:1], Ad[:1], as_key_proj(Bd, D), theta=cfg.theta)
    close(lg, O.qab_rope(qr[:1], A[:1], b4(B), cfg.theta), "c2 qAB_rope logits, row 0")


def test_config3_group_full_context():
    """Configuration 3 at full context / rank / layer count (4 layers share one key latent and one
    value latent of rank 1024, context 32768, 32 / 8 heads, theta 5e5), batch 2: the K+V-factorized
    group and the V-only-factorized variant with dense keys."""
    b, NL, L, R, G, theta = 2, 4, 32768, 1024, 4, 500000.0
    H = KVH * G
    gen = torch.Generator(device=DEV).manual_seed(3)
    A = dev_randn(gen, b, L, R)
    Av = dev_randn(gen, b, L, R)
    qs = [dev_randn(gen, b, H, 1, D) for _ in range(NL)]
    Bs = [dev_randn(gen, R, KVH * D, scale=R ** -0.5) for _ in range(NL)]
    Bvs = [dev_randn(gen, R, KVH * D, scale=R ** -0.5) for _ in range(NL)]
    qs = [K.rope_query(x, theta, L) for x in qs]
    got = K.xkv_group_decode(qs, A, Bs, Av, Bvs, theta=theta)
    status_ok()
    Ac, Avc = A.cpu(), Av.cpu()
    for i in range(NL):
        want = O.recon_rope_decode(qs[i].cpu(), Ac, b4(Bs[i].cpu(), b), Avc, theta, value_B=b4(Bvs[i].cpu(), b))
        close(got[i], want, f"c3 group layer {i}")
    # V-only variant: dense keys per layer, the shared value latent, one layer checked per call
    Kd = dev_randn(gen, b, KVH, L, D)
    Bv4 = b4(Bvs[0], b).contiguous()
    got_v = K.group_query_attention_factorized_v_only(qs[0], Kd, Av, Bv4)
    status_ok()
    close(got_v, O.gqa_factorized_v_only(qs[0].cpu(), Kd.cpu(), Avc, Bv4.cpu()), "c3 V-only variant")


def test_config4_mla_full_shape_sampled_rows():
    """Configuration 4 at full shape (batch 64, 128 heads, kv_lora_rank 512, nope 128, rope 64, v 128,
    context 8192, scale 1/sqrt(192)); four batch rows are checked against the oracle."""
    b, H, L, lora, nope, rope, vd = 64, 128, 8192, 512, 128, 64, 128
    gen = torch.Generator(device=DEV).manual_seed(4)
    c = dev_randn(gen, b, L, lora)
    kr = dev_randn(gen, b, L, rope)
    Wk = dev_randn(gen, H, nope, lora, scale=lora ** -0.5)
    Wv = dev_randn(gen, H, lora, vd, scale=lora ** -0.5)
    qn = dev_randn(gen, b, H, nope)
    qr = dev_randn(gen, b, H, rope)
    scale = 1.0 / math.sqrt(192.0)
    got = K.mla_absorbed_decode(qn, qr, c, kr, Wk, Wv, scale)
    status_ok()
    for r in (0, 63, 17, 40):
        want = O.mla_absorbed(qn[r:r + 1].cpu(), qr[r:r + 1].cpu(), c[r:r + 1].cpu(), kr[r:r + 1].cpu(), Wk.cpu(),
                              Wv.cpu(), scale)
        close(got[r:r + 1], want, f"c4 row {r}")
    assert torch.equal(got, K.mla_absorbed_decode(qn, qr, c, kr, Wk, Wv, scale))


@pytest.mark.parametrize("pair", [False, True])
def test_config5_long_context_rows(pair):
    """Configuration 5's per-row shape (64 / 8 heads, rank 1024, context 131072, dense V, theta 5e5,
    query position 131072), two batch rows, on the single-CTA and the CTA-pair kernel."""
    b, L, R, G, theta = 2, 131072, 1024, 8, 500000.0
    H = KVH * G
    gen = torch.Generator(device=DEV).manual_seed(5)
    A = dev_randn(gen, b, L, R)
    V = dev_randn(gen, b, L, KVH, D)
    B = dev_randn(gen, R, KVH * D, scale=R ** -0.5)
    q = K.rope_query(dev_randn(gen, b, H, 1, D), theta, L)
    got = K.recon_rope_decode(q, A, B, V.transpose(1, 2), theta=theta, cta_pair=pair)
    status_ok()
    Bc = b4(B.cpu())
    for r in range(b):
        want = O.recon_rope_decode(q[r:r + 1].cpu(), A[r:r + 1].cpu(), Bc, V[r:r + 1].cpu().transpose(1, 2), theta)
        close(got[r:r + 1], want, f"c5 row {r} (cta_pair={pair})")


@pytest.mark.parametrize("theta", [1e4, 5e5, 1e7])
def test_rope_at_long_positions(theta):
    """Key positions up to 131071 (k_position_offset = 131072 - L): the tensor-core epilogue reduces the
    angle with a three-constant Cody-Waite step before the SFU sin / cos, which must hold out there."""
    b, L, R, G = 2, 300, 128, 4
    off = 131072 - L
    g = torch.Generator().manual_seed(31)
    H = KVH * G
    q = torch.randn(b, H, 1, D, generator=g).bfloat16()
    A = torch.randn(b, L, R, generator=g).bfloat16()
    B = (torch.randn(R, KVH * D, generator=g) / R ** 0.5).bfloat16()
    V = torch.randn(b, L, KVH, D, generator=g).bfloat16()
    qd, Ad, Bd, Vd = q.to(DEV), A.to(DEV), B.to(DEV), V.to(DEV)
    Kr = O.reconstruct_rope_keys(A, b4(B, b), theta, position_offset=off)
    want = O.gqa_dense(q, Kr, V.transpose(1, 2))
    for pair in (False, True):
        got = K.recon_rope_decode(qd, Ad, Bd, Vd.transpose(1, 2), theta=theta, k_position_offset=off, cta_pair=pair)
        status_ok()
        close(got, want, f"decode at positions {off}..{off + L - 1}, theta {theta:g}, pair={pair}")
    kw = dict(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=qd[:, :, 0], k=Ad, k_proj=as_key_proj(Bd, D),
              logits_only=True, sm_scale=1.0, theta=theta, pos_offset=off)
    assert ops.plan(**kw) == "recon_tc"
    lg = ops.decode(entry="xkv_qab_logits", **kw)
    want_lg = torch.matmul(q.float().view(b, KVH, G, D), Kr.transpose(-1, -2)).view(b, H, L)
    close(lg, want_lg, f"logits at long positions, theta {theta:g}")
    gen = ops.decode(entry="xkv_qab_logits", force_generic=True, **kw)
    close(gen, want_lg, f"portable kernel at long positions, theta {theta:g}")


def test_rope_table_kernel_matches_oracle():
    """xkv_rope_table against the reference's table formula (flash_recontruction/rope/sin_cos.py:72-99
    in half-table form): {cos, sin}(float(pos) * inv_freq[j]).  The reference accepts 1e-3 for its own
    fast-math kernel; the angles here are formed exactly as in the oracle, so the bound is 1e-6."""
    lib = _C.load()
    for L, half, off, theta in [(1000, 64, 0, 1e7), (300, 64, 131072 - 300, 5e5), (257, 32, 5, 1e4)]:
        cos, sin = O.rope_cos_sin(2 * half, L + off, theta)
        want = torch.stack((cos[off:, :half], sin[off:, :half]), dim=-1)
        for use_inv in (True, False):
            out = torch.empty(L, half, 2, device=DEV)
            f = _C.inv_freq(2 * half, theta, torch.device(DEV))
            rc = lib.xkv_rope_table(out.data_ptr(), L, half, off, theta, f.data_ptr() if use_inv else None,
                                    torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            err = (out.cpu() - want).abs().max().item()
            # without inv_freq the kernel derives the frequencies itself (powf): angles differ in the last
            # bits, which at position 1e5 is visible in sin / cos
            assert err <= (1e-6 if use_inv else 2e-2 if off > 1000 else 5e-4), (L, half, off, theta, use_inv, err)
    assert lib.xkv_rope_table(None, 4, 4, 0, 1e4, None, None) == -1


def test_status_check_raises_on_a_timeout_word():
    """The opt-in status check: a call that ends with a time-out code in its status words raises.  The
    code is written into the workspace by the test (host-side injection, no device wait is made to
    expire); a healthy call passes the same check."""
    q = torch.randn(2, 32, 1, D, device=DEV).bfloat16()
    A = torch.randn(2, 256, 64, device=DEV).bfloat16()
    B = (torch.randn(64, KVH * D, device=DEV) / 8).bfloat16()
    V = torch.randn(2, KVH, 256, D, device=DEV).bfloat16()
    out = K.recon_rope_decode(q, A, B, V, theta=1e4, check_status=True)      # healthy: no raise
    assert torch.isfinite(out.float()).all()
    dev = torch.device(DEV)
    ws = _C.workspace(dev, 256)
    stream = torch.cuda.current_stream().cuda_stream
    ws[:32].view(torch.int32).copy_(torch.tensor([-6, 4, 17, 2, 1, 0, 0, 0], dtype=torch.int32))
    with pytest.raises(_C.DeviceTimeout, match="role 4, tile 17, chunk 2"):
        _C.raise_on_status(ws.data_ptr(), stream, "injected")
    ws[:32].zero_()
    prev = _C.set_check_status(True)
    try:
        K.recon_rope_decode(q, A, B, V, theta=1e4)
    finally:
        _C.set_check_status(prev)
