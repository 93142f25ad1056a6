"""Ragged batches: per-row cache lengths (kv_lens) on every kernel family, against the oracle
evaluated row by row on the truncated caches."""
import pytest
import torch

import kernel_collections_b200 as K
from kernel_collections_b200 import _C
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
KVH, D = 8, 128


def close(got, want, what, dtype):
    ta, tr = (1e-4, 1e-4) if dtype == torch.float32 else (2e-2, 1e-2)
    assert torch.isfinite(got.float()).all(), what
    ma, rel = O.error_metrics(got, want)
    assert ma <= ta * max(1.0, want.abs().max().item()) and rel <= tr, f"{what}: max_abs={ma:.3e} rel_l2={rel:.3e}"


def rows(fn, lens, *tensors):
    """Oracle row by row: tensors are (b, ...) with the cache length on the axis given per tensor."""
    outs = []
    for i, n in enumerate(lens):
        outs.append(fn(i, n))
    return torch.cat(outs, dim=0)


LENS = [1000, 1, 517, 128, 999]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_ragged_dense(dtype):
    b, H, L = len(LENS), 32, 1000
    g = torch.Generator().manual_seed(61)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    k = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    v = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    lens = torch.tensor(LENS, dtype=torch.int32, device=DEV)
    got = K.group_query_attention(q.to(DEV), k.to(DEV), v.to(DEV), kv_lens=lens)
    want = rows(lambda i, n: O.gqa_dense(q[i:i + 1], k[i:i + 1, :, :n], v[i:i + 1, :, :n]), LENS)
    close(got, want, "ragged dense", dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("factorized_v", [False, True])
def test_ragged_recon_rope(dtype, factorized_v):
    b, G, L, R, Rv, theta = len(LENS), 4, 1000, 128, 256, 500000.0
    H = KVH * G
    g = torch.Generator().manual_seed(62)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    A = torch.randn(b, L, R, generator=g).to(dtype)
    B = (torch.randn(R, KVH * D, generator=g) / R ** 0.5).to(dtype)
    B4 = B.view(R, KVH, D).permute(1, 0, 2)[None]
    lens = torch.tensor(LENS, dtype=torch.int32, device=DEV)
    if factorized_v:
        Av = torch.randn(b, L, Rv, generator=g).to(dtype)
        Bv = (torch.randn(Rv, KVH * D, generator=g) / Rv ** 0.5).to(dtype)
        Bv4 = Bv.view(Rv, KVH, D).permute(1, 0, 2)[None]
        got = K.recon_rope_decode(q.to(DEV), A.to(DEV), B.to(DEV), Av.to(DEV), Bv.to(DEV), theta=theta, kv_lens=lens)
        want = rows(lambda i, n: O.recon_rope_decode(q[i:i + 1], A[i:i + 1, :n], B4, Av[i:i + 1, :n], theta, value_B=Bv4), LENS)
    else:
        V = torch.randn(b, KVH, L, D, generator=g).to(dtype)
        got = K.recon_rope_decode(q.to(DEV), A.to(DEV), B.to(DEV), V.to(DEV), theta=theta, kv_lens=lens)
        want = rows(lambda i, n: O.recon_rope_decode(q[i:i + 1], A[i:i + 1, :n], B4, V[i:i + 1, :, :n], theta), LENS)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    close(got, want, f"ragged recon rope (factorized_v={factorized_v})", dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_ragged_factorized_and_mla(dtype):
    b, H, L, R = len(LENS), 32, 1000, 128
    g = torch.Generator().manual_seed(63)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    Ak = torch.randn(b, L, R, generator=g).to(dtype)
    Bk = (torch.randn(b, KVH, R, D, generator=g) / R ** 0.5).to(dtype)
    Av = torch.randn(b, L, R, generator=g).to(dtype)
    Bv = (torch.randn(b, KVH, R, D, generator=g) / R ** 0.5).to(dtype)
    lens = torch.tensor(LENS, dtype=torch.int32, device=DEV)
    got = K.group_query_attention_factorized(q.to(DEV), Ak.to(DEV), Bk.to(DEV), Av.to(DEV), Bv.to(DEV), kv_lens=lens)
    want = rows(lambda i, n: O.gqa_factorized(q[i:i + 1], Ak[i:i + 1, :n], Bk[i:i + 1], Av[i:i + 1, :n], Bv[i:i + 1]), LENS)
    close(got, want, "ragged factorized", dtype)
    # MLA absorbed
    Hm, lora, rope, nope, vd = 16, 128, 64, 64, 64
    qn = torch.randn(b, Hm, nope, generator=g).to(dtype)
    qr = (torch.randn(b, Hm, rope, generator=g) / 3).to(dtype)
    c = (torch.randn(b, L, lora, generator=g) / 3).to(dtype)
    kr = (torch.randn(b, L, rope, generator=g) / 3).to(dtype)
    Wk = (torch.randn(Hm, nope, lora, generator=g) / lora ** 0.5).to(dtype)
    Wv = (torch.randn(Hm, lora, vd, generator=g) / lora ** 0.5).to(dtype)
    got = K.mla_absorbed_decode(qn.to(DEV), qr.to(DEV), c.to(DEV), kr.to(DEV), Wk.to(DEV), Wv.to(DEV), 0.1, kv_lens=lens)
    want = rows(lambda i, n: O.mla_absorbed(qn[i:i + 1], qr[i:i + 1], c[i:i + 1, :n], kr[i:i + 1, :n], Wk, Wv, 0.1), LENS)
    close(got, want, "ragged mla", dtype)


def test_zero_length_row_gives_zeros():
    b, H, L = 3, 32, 300
    g = torch.Generator().manual_seed(64)
    q = torch.randn(b, H, 1, D, generator=g).bfloat16().to(DEV)
    k = torch.randn(b, KVH, L, D, generator=g).bfloat16().to(DEV)
    lens = torch.tensor([300, 0, 17], dtype=torch.int32, device=DEV)
    got = K.group_query_attention(q, k, k, kv_lens=lens)
    assert torch.isfinite(got.float()).all()
    assert (got[1] == 0).all() and (got[0] != 0).any() and (got[2] != 0).any()
    with pytest.raises(ValueError):
        K.group_query_attention(q, k, k, kv_lens=lens.long())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tails_past_the_row_length_may_hold_nan(dtype):
    """Cache rows at or past kv_lens[b] are outside the call: filling them with NaN must not change
    any result, on every tensor-core kernel family (0 * NaN inside an MMA would poison the row)."""
    LN = [1000, 1, 517, 128, 999, 64, 65]
    b, G, L, R, Rv, theta = len(LN), 4, 1000, 128, 256, 500000.0
    H = KVH * G
    g = torch.Generator().manual_seed(65)
    nan = float("nan")

    def poisoned(t, axis):
        t = t.clone()
        for i, n in enumerate(LN):
            idx = [slice(None)] * t.dim()
            idx[0], idx[axis] = i, slice(n, None)
            t[tuple(idx)] = nan
        return t

    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    A = torch.randn(b, L, R, generator=g).to(dtype)
    B = (torch.randn(R, KVH * D, generator=g) / R ** 0.5).to(dtype)
    Bb = B.view(R, KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1).contiguous()
    V = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    Kd = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    Av = torch.randn(b, L, Rv, generator=g).to(dtype)
    Bv = (torch.randn(Rv, KVH * D, generator=g) / Rv ** 0.5).to(dtype)
    Bvb = Bv.view(Rv, KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1).contiguous()
    lens = torch.tensor(LN, dtype=torch.int32, device=DEV)
    qd, Bd, Bvd, Bbd, Bvbd = (x.to(DEV) for x in (q, B, Bv, Bb, Bvb))
    cases = {
        "recon_tc (dense V)": lambda a, v, k, av: K.recon_rope_decode(qd, a, Bd, v, theta=theta, kv_lens=lens),
        "recon_tc pair (dense V)": lambda a, v, k, av: K.recon_rope_decode(qd, a, Bd, v, theta=theta, kv_lens=lens, cta_pair=True),
        "two-pass, tcgen05 second pass": lambda a, v, k, av: K.recon_rope_decode(qd, a, Bd, av, Bvd, theta=theta, kv_lens=lens),
        "two-pass, mma.sync second pass": lambda a, v, k, av: K.recon_rope_decode(qd, a, Bd, av, Bvd, theta=theta, kv_lens=lens,
                                                                                   pv_mma_sync=True),
        "dense_tc": lambda a, v, k, av: K.group_query_attention(qd, k, v, kv_lens=lens),
        "latent_tc": lambda a, v, k, av: K.group_query_attention_factorized(qd, a, Bbd, av, Bvbd, kv_lens=lens),
    }
    clean = (A.to(DEV), V.to(DEV), Kd.to(DEV), Av.to(DEV))
    dirty = (poisoned(A, 1).to(DEV), poisoned(V, 2).to(DEV), poisoned(Kd, 2).to(DEV), poisoned(Av, 1).to(DEV))
    for name, fn in cases.items():
        want = fn(*clean)
        got = fn(*dirty)
        assert torch.isfinite(got.float()).all(), f"{name}: NaN leaked from rows past kv_lens"
        assert torch.equal(got, want), f"{name}: rows past kv_lens changed the result"
    # MLA (values alias the key latent) on the shared-latent kernel
    Hm, lora, rope = 64, 128, 64
    qn = torch.randn(b, Hm, lora, generator=g).to(dtype).to(DEV)
    qr = (torch.randn(b, Hm, rope, generator=g) / 3).to(dtype).to(DEV)
    c = (torch.randn(b, L, lora, generator=g) / 3).to(dtype)
    kr = (torch.randn(b, L, rope, generator=g) / 3).to(dtype)
    from kernel_collections_b200 import ops
    kw = dict(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=qn, q_tail=qr, sm_scale=0.1, num_kv_heads=1,
              kv_lens=lens)
    cd, krd = c.to(DEV), kr.to(DEV)
    want = ops.decode(entry="xkv_mla_decode", k=cd, v=cd, k_tail=krd, **kw)
    pc, pk = poisoned(c, 1).to(DEV), poisoned(kr, 1).to(DEV)
    got = ops.decode(entry="xkv_mla_decode", k=pc, v=pc, k_tail=pk, **kw)
    assert torch.isfinite(got.float()).all() and torch.equal(got, want), "MLA latent with NaN tails"
