"""GPU parity of the dense GQA decode kernel (TMA ring + mma.sync; head_dim 128, bf16 / fp16):
against the CPU oracle and the portable kernel, over tails, groupings, layouts and splits."""
import pytest
import torch

import kernel_collections_b200 as K
from kernel_collections_b200 import flash_decoding as FD
from kernel_collections_b200 import _C, ops
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
D = 128

CASES = [  # b, H, KVH, L
    (1, 4, 4, 1), (2, 8, 2, 63), (1, 32, 8, 64), (3, 16, 1, 65), (2, 32, 8, 1000), (1, 8, 8, 5000),
    (2, 64, 8, 777), (1, 7, 1, 300), (4, 12, 4, 4096),
]


def close(got, want, what, ta=2e-2, tr=1e-2):
    assert torch.isfinite(got.float()).all(), what
    ma, rel = O.error_metrics(got, want)
    assert ma <= ta * max(1.0, want.abs().max().item()) and rel <= tr, f"{what}: max_abs={ma:.3e} rel_l2={rel:.3e}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_dense_tc(dtype, case):
    b, H, KVH, L = case
    g = torch.Generator().manual_seed(31)
    q = torch.randn(b, H, 1, D, generator=g).to(dtype)
    k = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    v = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    kw = dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=qd[:, :, 0], k=kd.transpose(1, 2),
              v=vd.transpose(1, 2), sm_scale=D ** -0.5)
    assert ops.plan(**kw) == "dense_tc"
    want = O.gqa_dense(q, k, v)
    got = K.group_query_attention(qd, kd, vd)
    rc, detail = _C.last_status(torch.device(DEV))
    assert rc == 0, detail
    close(got, want, "dense_tc vs oracle")
    gen = ops.decode(entry="xkv_dense_decode", force_generic=True, **kw)
    close(got[:, :, 0], gen.float().cpu(), "dense_tc vs portable kernel", 1e-2, 5e-3)
    assert torch.equal(got, K.group_query_attention(qd, kd, vd))          # repeatable
    # token-major cache layout (b, L, KVH, D) through the flash-decoding entry point
    o = torch.empty(b, H, D, dtype=dtype, device=DEV)
    FD.gqa.decode_attention_fwd(qd[:, :, 0], kd.transpose(1, 2).contiguous(), vd.transpose(1, 2).contiguous(), o,
                                torch.full((b,), 4, dtype=torch.int32, device=DEV), 4, D ** -0.5)
    close(o, want[:, :, 0], "dense_tc token-major layout")
    # fa layout
    out = K.group_query_attention_fa(qd.transpose(1, 2), kd.transpose(1, 2).contiguous(), vd.transpose(1, 2).contiguous())
    close(out.transpose(1, 2), want, "group_query_attention_fa")


def test_dense_tc_extreme_logits_and_masked_warps():
    """Large logits and a tail tile in which whole warps see only masked tokens."""
    dtype = torch.bfloat16
    b, H, KVH, L = 1, 8, 2, 64 + 3
    g = torch.Generator().manual_seed(32)
    q = (torch.randn(b, H, 1, D, generator=g) * 6).to(dtype)
    k = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    v = torch.randn(b, KVH, L, D, generator=g).to(dtype)
    got = K.group_query_attention(q.to(DEV), k.to(DEV), v.to(DEV))
    close(got, O.gqa_dense(q, k, v), "extreme logits")
