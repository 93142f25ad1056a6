"""Generate tests/golden/reference_eager.npz by running the REFERENCE's own eager code.

Run once, in a container where the reference checkout is mounted:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The reference is Python and cannot travel to the GPU box, so its outputs on small
seeded inputs are committed as fixtures; tests/test_oracle_golden.py pins the CPU
oracle against them.  Everything stored is float32 numpy.
"""
import os
import sys

import numpy as np
import torch

if len(sys.argv) != 2:
    sys.exit("usage: make_golden.py /path/to/reference")
ref_root = sys.argv[1]
sys.path.insert(0, ref_root)
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
sys.dont_write_bytecode = True

import attention as ref_attention  # noqa: E402
from flash_recontruction.qAB_no_pe.ref import qAB_ref  # noqa: E402
from flash_recontruction.rope import rope_ref  # noqa: E402
from flash_recontruction.fused_attention.no_pe import ref as fused_ref  # noqa: E402
from flash_decoding.mla2.ref import mla_decode_attention_fwd_ref  # noqa: E402
from flash_decoding.mla import decode_attention_reference  # noqa: E402
from transformers.models.qwen2.modeling_qwen2 import apply_rotary_pos_emb as hf_rope  # noqa: E402

out = {}


def put(prefix, **kw):
    for k, v in kw.items():
        out[f"{prefix}/{k}"] = v.detach().float().numpy() if torch.is_tensor(v) else np.asarray(v)


def case_shapes():
    # (name, b, H, KVH, D, L, Rk, Rv)
    return [("a", 2, 8, 2, 16, 37, 12, 20), ("b", 1, 6, 6, 32, 64, 8, 8), ("c", 3, 4, 1, 8, 5, 3, 7)]


torch.manual_seed(1234)
for name, b, H, KVH, D, L, Rk, Rv in case_shapes():
    q = torch.randn(b, H, 1, D)
    K = torch.randn(b, KVH, L, D)
    V = torch.randn(b, KVH, L, D)
    Ak = torch.randn(b, L, Rk)
    Bk = torch.randn(b, KVH, Rk, D) / Rk ** 0.5
    Av = torch.randn(b, L, Rv)
    Bv = torch.randn(b, KVH, Rv, D) / Rv ** 0.5
    put(f"gqa/{name}", q=q, K=K, V=V, Ak=Ak, Bk=Bk, Av=Av, Bv=Bv)
    put(f"gqa/{name}",
        dense=ref_attention.group_query_attention(q, K, V),
        v_only=ref_attention.group_query_attention_factorized_v_only(q, K, Av, Bv),
        factorized=ref_attention.group_query_attention_factorized(q, Ak, Bk, Av, Bv),
        qab_no_pe=qAB_ref(q, Ak, Bk),
        fused=fused_ref.group_query_attention_xKV(q.squeeze(2), Ak, Bk, Av, Bv),
        fused_k_only=fused_ref.group_query_attention_xKV_k_only(
            q.squeeze(2), Ak, Bk, V.transpose(1, 2).contiguous()),
        flash_gqa=decode_attention_reference(
            q.squeeze(2), K.transpose(1, 2).contiguous(), V.transpose(1, 2).contiguous(), None, 1.0),
    )

# RoPE tables and the rotate-half application (rope_ref.py), plus the qAB-with-RoPE eager
# reference of test_qAB_rope.py fed with those tables.
for name, D, L, theta in [("t1", 16, 40, 10000.0), ("t2", 128, 300, 500000.0), ("t3", 64, 17, 1e7)]:
    cos, sin = rope_ref.LlamaRotaryEmbedding(D, L, theta)
    x = torch.randn(1, 2, L, D)
    put(f"rope/{name}", D=D, L=L, theta=theta, cos=cos, sin=sin, x=x,
        x_rot=rope_ref.apply_rotary_pos_emb_pytorch(x, cos, sin))

for name, b, H, KVH, D, L, R, theta in [("r1", 2, 8, 2, 16, 33, 10, 10000.0),
                                        ("r2", 1, 4, 1, 128, 70, 24, 500000.0)]:
    q = torch.randn(b, H, 1, D)
    Ak = torch.randn(b, L, R)
    Bk = torch.randn(b, KVH, R, D) / R ** 0.5
    cos, sin = rope_ref.LlamaRotaryEmbedding(D, L, theta)
    # The steps of qAB_rope_ref (test_qAB_rope.py:19-43) with the rotary function it imports
    # from transformers; the installed transformers dropped the position_ids argument that
    # the reference script still passes, so the five lines are replayed here rather than
    # called.  cos/sin of shape (b, L, D) as the HF function expects.
    Kh = torch.matmul(Ak.unsqueeze(1), Bk)
    Kh, _ = hf_rope(Kh, Kh, cos[None].expand(b, -1, -1), sin[None].expand(b, -1, -1))
    logits = torch.matmul(q.view(b, KVH, H // KVH, D).contiguous(),
                          Kh.transpose(-1, -2)).view(b, H, 1, L)
    # the same built only from in-tree reference pieces (no HF): rebuild, rotate, dot
    K = torch.matmul(Ak.unsqueeze(1), Bk)
    K = rope_ref.apply_rotary_pos_emb_pytorch(K, cos, sin)
    logits2 = torch.matmul(q.view(b, KVH, H // KVH, D), K.transpose(-1, -2)).view(b, H, 1, L)
    V = torch.randn(b, KVH, L, D)
    put(f"qab_rope/{name}", q=q, Ak=Ak, Bk=Bk, theta=theta, logits=logits, logits_intree=logits2,
        V=V, decode=ref_attention.group_query_attention(q, K, V))

for name, b, H, lora, rope, L in [("m1", 2, 4, 16, 8, 29), ("m2", 1, 16, 32, 16, 50)]:
    qn = torch.randn(b, H, lora) / 3
    qr = torch.randn(b, H, rope) / 3
    c = torch.randn(b, L, 1, lora) / 3
    kr = torch.randn(b, L, 1, rope) / 3
    import contextlib
    import io
    with contextlib.redirect_stdout(io.StringIO()):      # the reference prints shapes
        o1 = mla_decode_attention_fwd_ref(qn, qr, c, kr, sm_scale=1.0)
        # the eager reference DIVIDES by sm_scale; 1/0.25 therefore means "multiply by 0.25"
        o2 = mla_decode_attention_fwd_ref(qn, qr, c, kr, sm_scale=4.0)
    put(f"mla/{name}", q_nope=qn, q_rope=qr, kv_nope=c, k_rope=kr, out_scale1=o1, out_mul_quarter=o2)

# group_query_attentionv2 with several query tokens per sequence (attention.py:93-182), with and
# without an additive mask; its own seed, so the arrays above do not move when cases are added here
torch.manual_seed(4321)
for name, b, H, KVH, D, L, QL in [("v1", 2, 8, 2, 16, 37, 3), ("v2", 1, 4, 4, 32, 20, 5)]:
    q = torch.randn(b, H, QL, D)
    K = torch.randn(b, KVH, L, D)
    V = torch.randn(b, KVH, L, D)
    mask = torch.randn(b, 1, 1, QL, L)
    put(f"gqa_v2/{name}", q=q, K=K, V=V, mask=mask,
        plain=ref_attention.group_query_attentionv2(q, K, V),
        masked=ref_attention.group_query_attentionv2(q, K, V, attn_mask=mask))

dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_eager.npz")
np.savez_compressed(dst, **out)
print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")
