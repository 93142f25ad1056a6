"""Pins the CPU oracle against outputs of the reference's own eager code
(tests/golden/reference_eager.npz, written by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import xkv_oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_eager.npz"))


def t(key):
    return torch.from_numpy(G[key])


def close(a, b, tol=2e-5):
    a, b = a.double(), b.double()
    assert a.shape == b.shape
    assert (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item())


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_gqa_family(name):
    p = f"gqa/{name}/"
    q, K, V, Ak, Bk, Av, Bv = (t(p + k) for k in ["q", "K", "V", "Ak", "Bk", "Av", "Bv"])
    close(O.gqa_dense(q, K, V), t(p + "dense"))
    close(O.gqa_factorized_v_only(q, K, Av, Bv), t(p + "v_only"))
    close(O.gqa_factorized(q, Ak, Bk, Av, Bv), t(p + "factorized"))
    close(O.qab_no_pe(q, Ak, Bk), t(p + "qab_no_pe"))
    close(O.xkv_fused(q.squeeze(2), Ak, Bk, Av, Bv, 1.0), t(p + "fused"))
    close(O.xkv_fused_k_only(q.squeeze(2), Ak, Bk, V.transpose(1, 2).contiguous(), 1.0),
          t(p + "fused_k_only"))
    close(O.flash_decode_gqa(q.squeeze(2), K.transpose(1, 2).contiguous(),
                             V.transpose(1, 2).contiguous(), 1.0), t(p + "flash_gqa"))


@pytest.mark.parametrize("name", ["t1", "t2", "t3"])
def test_rope_tables(name):
    p = f"rope/{name}/"
    D, L, theta = int(G[p + "D"]), int(G[p + "L"]), float(G[p + "theta"])
    cos, sin = O.rope_cos_sin(D, L, theta)
    assert torch.equal(cos, t(p + "cos")) and torch.equal(sin, t(p + "sin"))
    close(O.apply_rope(t(p + "x"), cos, sin), t(p + "x_rot"), 1e-6)


@pytest.mark.parametrize("name", ["r1", "r2"])
def test_qab_rope(name):
    p = f"qab_rope/{name}/"
    q, Ak, Bk, V = (t(p + k) for k in ["q", "Ak", "Bk", "V"])
    theta = float(G[p + "theta"])
    got = O.qab_rope(q, Ak, Bk, theta)
    close(got, t(p + "logits"))
    close(got, t(p + "logits_intree"))
    close(O.recon_rope_decode(q, Ak, Bk, V, theta), t(p + "decode"))


@pytest.mark.parametrize("name", ["m1", "m2"])
def test_mla(name):
    p = f"mla/{name}/"
    qn, qr, c, kr = (t(p + k) for k in ["q_nope", "q_rope", "kv_nope", "k_rope"])
    close(O.mla_decode(qn, qr, c, kr, 1.0), t(p + "out_scale1"))
    close(O.mla_decode(qn, qr, c, kr, 0.25), t(p + "out_mul_quarter"))


def test_dense_v_as_identity_factorization():
    """Dense V expressed as an identity factorization reproduces the k-only form: the
    construction used for the fp32 CPU-runnable configuration."""
    torch.manual_seed(0)
    b, H, KVH, D, L, R = 1, 8, 2, 16, 33, 12
    q = torch.randn(b, H, 1, D)
    A = torch.randn(b, L, R)
    B = torch.randn(b, KVH, R, D) / R ** 0.5
    V = torch.randn(b, L, KVH, D)
    vA = V.reshape(b, L, KVH * D)
    vB = torch.eye(KVH * D).view(KVH * D, KVH, D).permute(1, 0, 2)[None].contiguous()
    ref = O.gqa_factorized(q, A, B, vA, vB)
    got = O.xkv_fused_k_only(q.squeeze(2), A, B, V, D ** -0.5)
    close(got, ref.squeeze(2), 1e-5)


@pytest.mark.parametrize("name", ["v1", "v2"])
def test_gqa_v2_several_query_tokens(name):
    p = f"gqa_v2/{name}/"
    q, K, V, mask = (t(p + k) for k in ["q", "K", "V", "mask"])
    close(O.gqa_dense_multi(q, K, V), t(p + "plain"))
    close(O.gqa_dense_multi(q, K, V, mask), t(p + "masked"))
    # one query token at a time is the single-step function
    close(O.gqa_dense_multi(q, K, V)[:, :, 1:2], O.gqa_dense(q[:, :, 1:2], K, V))
