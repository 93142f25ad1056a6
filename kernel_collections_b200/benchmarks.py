"""Device-timed runs of the secondary configurations (everything bench.py does not cover).

    python -m kernel_collections_b200.benchmarks [--workload NAME ...] [--reps N]

One JSON line per workload: kernel family, ms per call, tokens/s, algorithmic bytes / flops and the
fractions of the measured HBM / bf16 peaks (MEASURED_PEAKS.json at the repository root when
present).  Inputs are drawn on the device; timing uses CUDA events after warm-up calls, and every
workload streams far more than the 126 MB L2 per call.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import _C, ops
from . import attention as A
from . import flash_recontruction as FR
from .flash_decoding import mla2

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timed(fn, reps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def rnd(*shape, dtype=torch.bfloat16, scale=1.0, dev="cuda"):
    return (torch.randn(*shape, device=dev) * scale).to(dtype)


SMALL = False      # --small: quarter contexts, for profiler captures


def ctx(L):
    return L // 4 if SMALL else L


def w_dense(reps):
    """Dense GQA decode at the c2 cache shape (group_query_attention / flash_decoding.gqa)."""
    b, H, KVH, D, L = 16, 32, 8, 128, ctx(16384)
    q, k, v = rnd(b, H, 1, D), rnd(b, L, KVH, D), rnd(b, L, KVH, D)
    fn = lambda: A.group_query_attention(q, k.transpose(1, 2), v.transpose(1, 2))
    plan = ops.plan(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=q[:, :, 0], k=k, v=v, sm_scale=1.0)
    return dict(workload="dense_gqa_b16_L16384", plan=plan, tokens=b, ms=timed(fn, reps),
                bytes=2 * (2 * b * L * KVH * D + 2 * b * H * D), flops=4 * b * H * L * D)


def w_qab_logits(reps):
    """qAB_rope logits only (c2 shape): key rebuild + RoPE + q-dot, logits written to HBM."""
    b, H, KVH, D, L, R = 16, 32, 8, 128, 16384, 512
    q, Ak = rnd(b, H, 1, D), rnd(b, L, R)
    Bk = A.as_key_proj(rnd(R, KVH * D, scale=R ** -0.5), D).expand(b, -1, -1, -1)
    fn = lambda: FR.qAB_rope_v1(q, Ak, Bk, theta=5e5)
    plan = ops.plan(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=q[:, :, 0], k=Ak, k_proj=Bk,
                    logits_only=True, sm_scale=1.0, theta=5e5)
    return dict(workload="qab_rope_logits_c2", plan=plan, tokens=b, ms=timed(fn, reps),
                bytes=2 * (b * L * R + R * KVH * D + b * H * D + b * H * L), flops=2 * b * L * R * KVH * D + 2 * b * H * L * D)


def w_group(reps):
    """c3, dense-V flavour: 4 layers share one latent (b32, L32768, R1024), one launch for the group."""
    NL, b, H, KVH, D, L, R = 4, 32, 32, 8, 128, 32768, 1024
    Ak = rnd(b, L, R)
    qs = [rnd(b, H, 1, D) for _ in range(NL)]
    Bs = [rnd(R, KVH * D, scale=R ** -0.5) for _ in range(NL)]
    Vs = [rnd(b, L, KVH, D).transpose(1, 2) for _ in range(NL)]
    fn = lambda: A.xkv_group_decode(qs, Ak, Bs, Vs, theta=5e5)
    return dict(workload="c3_group4_dense_v_b32_L32768_R1024", plan="recon_tc (one launch)", tokens=b * NL,
                ms=timed(fn, max(3, reps // 4)),
                bytes=2 * (b * L * R + NL * (b * L * KVH * D + R * KVH * D + 2 * b * H * D)),
                flops=NL * (2 * b * L * R * KVH * D + 4 * b * H * L * D))


def w_group_kv(reps):
    """c3 as specified: 4 layers share the key latent AND the value latent (b32, L32768, R1024 each),
    per-layer B_k / B_v.  Two passes: grouped tcgen05 logits, then one P.A_v pass over 128 stacked heads."""
    NL, b, H, KVH, D, L, R = 4, 32, 32, 8, 128, ctx(32768), 1024
    Ak, Av = rnd(b, L, R), rnd(b, L, R)
    qs = [rnd(b, H, 1, D) for _ in range(NL)]
    Bs = [rnd(R, KVH * D, scale=R ** -0.5) for _ in range(NL)]
    Bvs = [rnd(R, KVH * D, scale=R ** -0.5) for _ in range(NL)]
    fn = lambda: A.xkv_group_decode(qs, Ak, Bs, Av, Bvs, theta=5e5)
    return dict(workload="c3_group4_kv_factorized_b32_L32768_R1024", plan="two_pass (grouped)", tokens=b * NL,
                ms=timed(fn, max(3, reps // 4)),
                bytes=2 * (2 * b * L * R + NL * (2 * R * KVH * D + 2 * b * H * D)),
                flops=NL * (2 * b * L * R * KVH * D + 2 * b * H * L * (D + R) + 2 * b * H * R * D))


def w_v_only(reps):
    """c3, V-only-factorized variant: per layer dense K (b32, L32768) + the shared value latent (R1024)."""
    b, H, KVH, D, L, R = 32, 32, 8, 128, ctx(32768), 1024
    q, k, Av = rnd(b, H, 1, D), rnd(b, L, KVH, D), rnd(b, L, R)
    Bv = rnd(b, KVH, R, D, scale=R ** -0.5)
    fn = lambda: A.group_query_attention_factorized_v_only(q, k.transpose(1, 2), Av, Bv)
    plan = ops.plan(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_LATENT, q=q[:, :, 0], k=k, v=Av, v_proj=Bv, sm_scale=1.0)
    return dict(workload="c3_v_only_one_layer_b32_L32768_R1024", plan=plan, tokens=b, ms=timed(fn, max(3, reps // 4)),
                bytes=2 * (b * L * (KVH * D + R) + b * KVH * R * D + 2 * b * H * D),
                flops=2 * b * H * L * (D + R) + 2 * b * H * R * D)


def w_factorized(reps):
    """Absorbed factorized K and V without RoPE (group_query_attention_factorized), c1 shape in bf16
    at a serving-sized batch."""
    b, H, KVH, D, L, R = 16, 32, 8, 128, ctx(16384), 256
    q, Ak, Av = rnd(b, H, 1, D), rnd(b, L, R), rnd(b, L, R)
    Bk, Bv = rnd(b, KVH, R, D, scale=R ** -0.5), rnd(b, KVH, R, D, scale=R ** -0.5)
    fn = lambda: A.group_query_attention_factorized(q, Ak, Bk, Av, Bv)
    plan = ops.plan(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=q[:, :, 0], k=Ak, k_proj=Bk, v=Av,
                    v_proj=Bv, sm_scale=1.0)
    return dict(workload="factorized_absorbed_b16_L16384_R256", plan=plan, tokens=b, ms=timed(fn, max(2, reps // 5)),
                bytes=2 * (2 * b * L * R + 2 * b * KVH * R * D + 2 * b * H * D), flops=2 * b * H * L * 2 * R + 4 * b * H * R * D)


def w_mla(reps):
    """c4: MLA absorbed decode, DeepSeek-V3 attention shape (b64, 128 heads, L8192)."""
    b, H, lora, rope, nope, vd, L = 64, 128, 512, 64, 128, 128, ctx(8192)
    qn, qr = rnd(b, H, nope), rnd(b, H, rope)
    c, kr = rnd(b, L, lora), rnd(b, L, rope)
    Wk, Wv = rnd(H, nope, lora, scale=lora ** -0.5), rnd(H, lora, vd, scale=lora ** -0.5)
    fn = lambda: A.mla_absorbed_decode(qn, qr, c, kr, Wk, Wv, (nope + rope) ** -0.5)
    return dict(workload="c4_mla_absorbed_b64_H128_L8192", plan="see plan of xkv_mla_decode", tokens=b,
                ms=timed(fn, max(2, reps // 10)),
                bytes=2 * (b * L * (lora + rope) + 2 * H * nope * lora + b * H * (nope + rope + vd)),
                flops=b * L * H * (2 * (lora + rope) + 2 * lora) + 4 * b * H * nope * lora)


WORKLOADS = {"dense": w_dense, "qab_logits": w_qab_logits, "group": w_group, "group_kv": w_group_kv,
             "v_only": w_v_only, "factorized": w_factorized, "mla": w_mla}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", nargs="*", default=list(WORKLOADS), choices=list(WORKLOADS))
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--small", action="store_true", help="quarter contexts (profiler-sized cases)")
    args = ap.parse_args()
    global SMALL
    SMALL = args.small
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    hbm, tc, src = peaks()
    for name in args.workload:
        r = WORKLOADS[name](args.reps)
        ms = r["ms"]
        r.update(tokens_per_s=r["tokens"] / ms * 1e3, gbs=r["bytes"] / ms / 1e6, tflops=r["flops"] / ms / 1e9,
                 hbm_frac=r["bytes"] / ms / 1e6 / hbm, tensor_frac=r["flops"] / ms / 1e9 / tc, peaks=src)
        print(json.dumps(r))
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
