#!/usr/bin/env python
"""Decode-attention benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--graph on] [--gather MODE]

Default workload `c5`: the long-context sweep the headline metric is quoted on — factorized-K + RoPE
GQA decode with dense V, 64 query / 8 KV heads, head_dim 128, rank 1024, context 131072, bf16, GLOBAL
batch 128 (strong scaling: each of the N GPUs holds 128 / N batch rows, outputs are all-gathered over
NCCL inside the timed step).  One step = one decode-attention call over the whole batch (one new token
per sequence, one layer).  Other workloads (same JSON schema): c2 (qAB_rope configuration, batch 16,
context 16384, rank 512), c3 (cross-layer group of 4, K and V factorized), c3_vonly, c4 (MLA absorbed
decode; --shard batch|heads), dense, absorbed, k_only.

Rank 0 prints ONE JSON line.  `value` is tokens/s with inputs resident in HBM (CUDA events on the
launching stream, max over ranks); `e2e` is the same call through the public Python API with every
input copied from pinned host memory and the output read back inside the timed region; `parity` is the
error of sampled batch rows of the very tensors that were timed against the CPU oracle; `cpu_baseline`
is that oracle's own speed on the host cores (N = 1 only).

--graph on (N = 1) replays one captured step from a CUDA graph in the timed region (the plain call leaves
the GPU idle between the three to five launches of a sub-millisecond step); --gather nccl|peer|auto picks
how the outputs are gathered at N > 1 (auto: the library's peer-store kernel for steps under 2 ms when
symmetric memory is available and it agrees with NCCL, else NCCL).

--impl reference times the reference's eager CPU math (the oracle port: the reference is Python that
does not exist on the GPU box) on the host cores, one batch row at full context per step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_attn_tokens_per_s"
UNIT = "tokens/s"

# DRAM bytes moved per algorithmic byte, from ncu captures of profiling-sized cases of the same kernels
# (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the captured launch; the
# traffic of these streaming kernels grows in proportion to the rows processed).  profiles/ has the captures.
DRAM_PER_ALGORITHMIC_BYTE = {
    "recon_tc": (1.03, "profiles/recon_tc_kernel_c5_and_c2_cutdown.md"),
    "latent_pair": (1.03, "profiles/latent_pair_kernel_c4_cutdown.md"),
    "dense_tc": (1.004, "profiles/dense_tc_and_latent_tc_kernels_quarter_context.md"),
    "latent_tc": (1.063, "profiles/dense_tc_and_latent_tc_kernels_quarter_context.md"),
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.3)          # let the first samples come before the timed region starts
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------
# Workloads.  Each draws its inputs from seeded normal distributions as the configuration states
# (on the device when `dev` is a CUDA device: tens of GB; per-rank seed), knows its algorithmic bytes
# and flops, runs one step through the public API, and can check sampled batch rows against the
# CPU oracle.
class Workload:
    name = ""
    dtype = torch.bfloat16
    bound_hint = "tensor"

    def __init__(self, args, world, rank):
        self.args, self.world, self.rank = args, world, rank

    def local_batch(self, global_batch):
        if global_batch % self.world:
            raise SystemExit(f"global batch {global_batch} is not divisible by {self.world} GPUs")
        return global_batch // self.world

    def rnd(self, gen, *shape, scale=1.0, dev=None):
        dev = dev if dev is not None else self.dev
        if scale == 1.0:
            return torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32 if dev.type == "cpu" else self.dtype
                               ).to(self.dtype)
        return (torch.randn(*shape, generator=gen, device=dev) * scale).to(self.dtype)

    def big_rnd(self, gen, rows, *shape):
        """(rows, *shape) standard normal in the working dtype, drawn row by row (bounded temporaries)."""
        out = torch.empty((rows,) + tuple(shape), dtype=self.dtype, device=self.dev)
        for r in range(rows):
            out[r] = self.rnd(gen, *shape)
        return out


class ReconRope(Workload):
    """Factorized K + RoPE, dense V (configurations 2 and 5)."""

    def __init__(self, args, world, rank, *, name, global_batch, H, L, R, strong):
        super().__init__(args, world, rank)
        self.KVH, self.D, self.theta = 8, 128, 500000.0
        self.H, self.L, self.R = H, (args.kv_len or L), R
        self.strong = strong
        gb = args.rows * world if args.rows else global_batch
        self.b = self.local_batch(gb) if strong else (args.rows or global_batch)
        self.global_batch = gb if strong else self.b * world
        self.name = name if not (args.rows or args.kv_len) else f"{name}_cut_b{self.global_batch}_L{self.L}"
        self.scaling = "strong" if strong else "weak"
        self.launches = 3
        self.kernel = "recon_tc"

    def alloc(self, dev, seed):
        self.dev = dev
        g = torch.Generator(device=dev).manual_seed(seed)
        KD = self.KVH * self.D
        self.A = self.big_rnd(g, self.b, self.L, self.R)
        self.V = self.big_rnd(g, self.b, self.L, self.KVH, self.D)
        self.B = self.rnd(g, self.R, KD, scale=self.R ** -0.5)
        self.q_raw = self.rnd(g, self.b, self.H, 1, self.D)
        return self

    def prepare(self):
        import kernel_collections_b200 as K
        self.q = K.rope_query(self.q_raw, self.theta, self.L)     # query position = context length
        self.streamed = [self.A, self.V]
        self.small = [self.B, self.q]

    def step(self, A=None, V=None, B=None, q=None):
        import kernel_collections_b200 as K
        pair = {"auto": None, "on": True, "off": False}[self.args.pair]
        return K.recon_rope_decode(self.q if q is None else q, self.A if A is None else A, self.B if B is None else B,
                                   (self.V if V is None else V).transpose(1, 2), theta=self.theta, cta_pair=pair,
                                   force_generic=self.args.force_generic)

    def plan(self):
        from kernel_collections_b200 import _C, ops, attention
        return ops.plan(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=self.q[:, :, 0], k=self.A,
                        k_proj=attention.as_key_proj(self.B, self.D), v=self.V, sm_scale=self.D ** -0.5, theta=self.theta,
                        force_generic=self.args.force_generic)

    def alg_bytes(self):
        b, L, R, KD = self.b, self.L, self.R, self.KVH * self.D
        return 2 * (b * L * (R + KD) + R * KD + 2 * b * self.H * self.D)

    def alg_flops(self):
        b, L, R = self.b, self.L, self.R
        return 2 * b * L * R * self.KVH * self.D + 4 * b * self.H * L * self.D

    def config(self):
        return {"num_heads": self.H, "num_kv_heads": self.KVH, "head_dim": self.D, "kv_len": self.L, "rank": self.R,
                "rope_theta": self.theta, "value": "dense", "query_position": self.L}

    def oracle_row(self, r, tensors=None):
        from oracle import xkv_oracle as O
        A, V, B, q = tensors if tensors is not None else (self.A, self.V, self.B, self.q)
        B4 = B.cpu().view(self.R, self.KVH, self.D).permute(1, 0, 2)[None]
        return O.recon_rope_decode(q[r:r + 1].cpu(), A[r:r + 1].cpu(), B4, V[r:r + 1].cpu().transpose(1, 2), self.theta)

    def cpu_inputs(self, seed=0):
        """One batch row of the same distributions drawn on the CPU (for --impl reference)."""
        self.dev = torch.device("cpu")
        g = torch.Generator().manual_seed(seed)
        A = self.rnd(g, 1, self.L, self.R)
        V = self.rnd(g, 1, self.L, self.KVH, self.D)
        B = self.rnd(g, self.R, self.KVH * self.D, scale=self.R ** -0.5)
        from oracle import xkv_oracle as O
        q = O.rope_query(self.rnd(g, 1, self.H, 1, self.D), self.theta, self.L)
        return A, V, B, q


class Group(Workload):
    """Configuration 3: four consecutive layers share one key latent and one value latent (rank 1024
    each, context 32768, batch 32), per-layer B_k / B_v; or its V-only-factorized variant (dense K per
    layer, the shared value latent)."""

    def __init__(self, args, world, rank, v_only=False):
        super().__init__(args, world, rank)
        self.KVH, self.D, self.theta, self.H, self.NL = 8, 128, 500000.0, 32, 4
        self.L, self.R = args.kv_len or 32768, 1024
        self.v_only = v_only
        gb = args.rows * world if args.rows else 32
        self.b = self.local_batch(gb)
        self.global_batch = gb
        base = "c3_vonly_b32_L32768_Rv1024_x4layers" if v_only else "c3_group4_kv_factorized_b32_L32768_R1024"
        self.name = base if not (args.rows or args.kv_len) else f"{base}_cut_b{gb}_L{self.L}"
        self.scaling = "strong"
        self.bound_hint = "hbm" if v_only else "tensor"
        self.kernel = "two_pass"
        self.launches = (3 * self.NL + 1 + self.NL) if v_only else (2 + 1 + self.NL)

    def alloc(self, dev, seed):
        self.dev = dev
        g = torch.Generator(device=dev).manual_seed(seed)
        KD = self.KVH * self.D
        self.Av = self.big_rnd(g, self.b, self.L, self.R)
        self.Bvs = [self.rnd(g, self.R, KD, scale=self.R ** -0.5) for _ in range(self.NL)]
        self.q_raw = [self.rnd(g, self.b, self.H, 1, self.D) for _ in range(self.NL)]
        if self.v_only:
            self.Ks = [self.big_rnd(g, self.b, self.L, self.KVH, self.D) for _ in range(self.NL)]
        else:
            self.A = self.big_rnd(g, self.b, self.L, self.R)
            self.Bs = [self.rnd(g, self.R, KD, scale=self.R ** -0.5) for _ in range(self.NL)]
        return self

    def prepare(self):
        import kernel_collections_b200 as K
        if self.v_only:
            self.q = self.q_raw
            self.Bv4 = [x.view(self.R, self.KVH, self.D).permute(1, 0, 2)[None].expand(self.b, -1, -1, -1) for x in self.Bvs]
            self.streamed = [self.Av] + self.Ks
            self.small = self.Bvs + self.q
        else:
            self.q = [K.rope_query(x, self.theta, self.L) for x in self.q_raw]
            self.streamed = [self.A, self.Av]
            self.small = self.Bs + self.Bvs + self.q

    def step(self, *over):
        import kernel_collections_b200 as K
        if self.v_only:
            outs = K.xkv_group_decode_v_only(self.q, [k.transpose(1, 2) for k in self.Ks], self.Av, self.Bvs)
        else:
            outs = K.xkv_group_decode(self.q, self.A, self.Bs, self.Av, self.Bvs, theta=self.theta)
        return torch.stack(outs, dim=1)          # (b, NL, H, 1, D)

    def plan(self):
        return "two_pass"

    def alg_bytes(self):
        b, L, R, KD, NL = self.b, self.L, self.R, self.KVH * self.D, self.NL
        if self.v_only:
            return 2 * (b * L * R + NL * (b * L * KD + R * KD + 2 * b * self.H * self.D))
        return 2 * (2 * b * L * R + NL * (2 * R * KD + 2 * b * self.H * self.D))

    def alg_flops(self):
        b, L, R, NL, H, D = self.b, self.L, self.R, self.NL, self.H, self.D
        pv = 2 * b * H * L * R + 2 * b * H * R * D
        if self.v_only:
            return NL * (2 * b * H * L * D + pv)
        return NL * (2 * b * L * R * self.KVH * D + 2 * b * H * L * D + pv)

    def config(self):
        return {"layers": self.NL, "num_heads": self.H, "num_kv_heads": self.KVH, "head_dim": self.D, "kv_len": self.L,
                "rank": self.R, "rope_theta": self.theta, "value": "factorized (shared latent)",
                "key": "dense per layer" if self.v_only else "factorized (shared latent) + RoPE",
                "tokens_counted": "batch x layers per step"}

    def tokens_per_row(self):
        return self.NL

    def oracle_row(self, r, tensors=None):
        from oracle import xkv_oracle as O
        outs = []
        Avc = self.Av[r:r + 1].cpu()
        for i in range(self.NL):
            Bv4 = self.Bvs[i].cpu().view(self.R, self.KVH, self.D).permute(1, 0, 2)[None]
            if self.v_only:
                outs.append(O.gqa_factorized_v_only(self.q[i][r:r + 1].cpu(), self.Ks[i][r:r + 1].cpu().transpose(1, 2), Avc, Bv4))
            else:
                B4 = self.Bs[i].cpu().view(self.R, self.KVH, self.D).permute(1, 0, 2)[None]
                outs.append(O.recon_rope_decode(self.q[i][r:r + 1].cpu(), self.A[r:r + 1].cpu(), B4, Avc, self.theta, value_B=Bv4))
        return torch.stack(outs, dim=1)


class Mla(Workload):
    """Configuration 4: MLA absorbed decode, DeepSeek-V3 attention shape.  --shard batch cuts the batch
    across the GPUs (each streams its own latents); --shard heads cuts the 128 heads (every GPU streams
    the whole latent)."""
    bound_hint = "hbm"

    def __init__(self, args, world, rank):
        super().__init__(args, world, rank)
        self.H, self.lora, self.nope, self.rope, self.vd = 128, 512, 128, 64, 128
        self.L = args.kv_len or 8192
        self.shard = args.shard
        gb = args.rows * (world if self.shard == "batch" else 1) if args.rows else 64
        self.global_batch = gb
        self.b = self.local_batch(gb) if self.shard == "batch" else gb
        self.Hl = self.H if self.shard == "batch" else self.H // world
        self.scale = 1.0 / math.sqrt(self.nope + self.rope)
        base = "c4_mla_absorbed_b64_H128_L8192"
        self.name = (base if not (args.rows or args.kv_len) else f"{base}_cut_b{gb}_L{self.L}") + \
            (f"_{self.shard}_sharded" if world > 1 else "")
        self.scaling = "strong"
        self.kernel = "latent_tc"
        self.launches = 4

    def alloc(self, dev, seed):
        self.dev = dev
        # head sharding: every rank draws the same latents (seed without the rank) and its own heads
        g = torch.Generator(device=dev).manual_seed(seed if self.shard == "batch" else 12345)
        self.c = self.big_rnd(g, self.b, self.L, self.lora)
        self.kr = self.big_rnd(g, self.b, self.L, self.rope)
        Wk = self.rnd(g, self.H, self.nope, self.lora, scale=self.lora ** -0.5)
        Wv = self.rnd(g, self.H, self.lora, self.vd, scale=self.lora ** -0.5)
        qn = self.rnd(g, self.b, self.H, self.nope)
        qr = self.rnd(g, self.b, self.H, self.rope)
        h0 = 0 if self.shard == "batch" else self.rank * self.Hl
        self.Wk, self.Wv = Wk[h0:h0 + self.Hl].contiguous(), Wv[h0:h0 + self.Hl].contiguous()
        self.qn, self.qr = qn[:, h0:h0 + self.Hl].contiguous(), qr[:, h0:h0 + self.Hl].contiguous()
        return self

    def prepare(self):
        self.streamed = [self.c, self.kr]
        self.small = [self.Wk, self.Wv, self.qn, self.qr]

    def step(self, *over):
        import kernel_collections_b200 as K
        return K.mla_absorbed_decode(self.qn, self.qr, self.c, self.kr, self.Wk, self.Wv, self.scale)

    def plan(self):
        from kernel_collections_b200 import _C, ops
        return ops.plan(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=self.qn, k=self.c,
                        k_proj=self.Wk.permute(0, 2, 1).unsqueeze(0), v=self.c, v_proj=self.Wv.unsqueeze(0),
                        q_tail=self.qr, k_tail=self.kr, sm_scale=self.scale, num_kv_heads=1)

    def alg_bytes(self):
        b, L, H = self.b, self.L, self.Hl
        return 2 * (b * L * (self.lora + self.rope) + 2 * H * self.nope * self.lora + b * H * (self.nope + self.rope + self.vd))

    def alg_flops(self):
        b, L, H = self.b, self.L, self.Hl
        return b * L * H * (2 * (self.lora + self.rope) + 2 * self.lora) + 4 * b * H * self.nope * self.lora

    def config(self):
        return {"num_heads": self.H, "heads_per_gpu": self.Hl, "kv_lora_rank": self.lora, "qk_nope_head_dim": self.nope,
                "qk_rope_head_dim": self.rope, "v_head_dim": self.vd, "kv_len": self.L, "sm_scale": self.scale,
                "rope": "q_rope / k_rope taken as already rotated (the mla2 API)", "shard": self.shard}

    def oracle_row(self, r, tensors=None):
        from oracle import xkv_oracle as O
        return O.mla_absorbed(self.qn[r:r + 1].cpu(), self.qr[r:r + 1].cpu(), self.c[r:r + 1].cpu(), self.kr[r:r + 1].cpu(),
                              self.Wk.cpu(), self.Wv.cpu(), self.scale)


class Simple(Workload):
    """Secondary single-GPU shapes at the configuration-2 cache size: dense GQA decode, absorbed
    factorized K and V (rank 256, no RoPE), and factorized K with dense V without RoPE (k_only)."""
    bound_hint = "hbm"

    def __init__(self, args, world, rank, kind):
        super().__init__(args, world, rank)
        self.kind = kind
        self.H, self.KVH, self.D, self.R = 32, 8, 128, 256
        self.L = args.kv_len or 16384
        gb = args.rows * world if args.rows else 16
        self.b = self.local_batch(gb)
        self.global_batch = gb
        self.name = {"dense": "dense_gqa_b16_L16384", "absorbed": "factorized_absorbed_b16_L16384_R256",
                     "k_only": "factorized_k_dense_v_b16_L16384_R256"}[kind] + \
            ("" if not (args.rows or args.kv_len) else f"_cut_b{gb}_L{self.L}")
        self.scaling = "strong"
        self.kernel = {"dense": "dense_tc", "absorbed": "latent_tc", "k_only": "two_pass"}[kind]
        self.launches = {"dense": 3, "absorbed": 4, "k_only": 5}[kind]

    def alloc(self, dev, seed):
        self.dev = dev
        g = torch.Generator(device=dev).manual_seed(seed)
        b, L, H, KVH, D, R = self.b, self.L, self.H, self.KVH, self.D, self.R
        self.q = self.rnd(g, b, H, 1, D)
        if self.kind == "dense":
            self.k, self.v = self.big_rnd(g, b, L, KVH, D), self.big_rnd(g, b, L, KVH, D)
        else:
            self.Ak = self.big_rnd(g, b, L, R)
            self.Bk = self.rnd(g, 1, KVH, R, D, scale=R ** -0.5).expand(b, -1, -1, -1)
            if self.kind == "absorbed":
                self.Av = self.big_rnd(g, b, L, R)
                self.Bv = self.rnd(g, 1, KVH, R, D, scale=R ** -0.5).expand(b, -1, -1, -1)
            else:
                self.v = self.big_rnd(g, b, L, KVH, D)
        return self

    def prepare(self):
        self.streamed = {"dense": lambda: [self.k, self.v], "absorbed": lambda: [self.Ak, self.Av],
                         "k_only": lambda: [self.Ak, self.v]}[self.kind]()
        self.small = [self.q]

    def step(self, *over):
        import kernel_collections_b200 as K
        from kernel_collections_b200 import flash_recontruction as FR
        if self.kind == "dense":
            return K.group_query_attention(self.q, self.k.transpose(1, 2), self.v.transpose(1, 2))
        if self.kind == "absorbed":
            return K.group_query_attention_factorized(self.q, self.Ak, self.Bk, self.Av, self.Bv)
        return FR.gqa_xKV_no_pe_k_only_ref(self.q[:, :, 0], self.Ak, self.Bk, self.v)

    def plan(self):
        from kernel_collections_b200 import _C, ops
        q = self.q[:, :, 0]
        if self.kind == "dense":
            return ops.plan(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=q, k=self.k, v=self.v, sm_scale=1.0)
        if self.kind == "absorbed":
            return ops.plan(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_LATENT, q=q, k=self.Ak, k_proj=self.Bk, v=self.Av,
                            v_proj=self.Bv, sm_scale=1.0)
        return ops.plan(score_mode=_C.SCORE_LATENT, value_mode=_C.VALUE_DENSE, q=q, k=self.Ak, k_proj=self.Bk, v=self.v,
                        sm_scale=1.0)

    def alg_bytes(self):
        b, L, H, KD, D, R = self.b, self.L, self.H, self.KVH * self.D, self.D, self.R
        io = 2 * b * H * D
        if self.kind == "dense":
            return 2 * (2 * b * L * KD + io)
        if self.kind == "absorbed":
            return 2 * (2 * b * L * R + 2 * R * KD + io)
        return 2 * (b * L * (R + KD) + R * KD + io)

    def alg_flops(self):
        b, L, H, D, R = self.b, self.L, self.H, self.D, self.R
        if self.kind == "dense":
            return 4 * b * H * L * D
        if self.kind == "absorbed":
            return 4 * b * H * L * R + 4 * b * H * R * D
        return 2 * b * H * L * (R + D) + 2 * b * H * R * D

    def config(self):
        return {"num_heads": self.H, "num_kv_heads": self.KVH, "head_dim": self.D, "kv_len": self.L,
                "rank": None if self.kind == "dense" else self.R, "kind": self.kind}

    def oracle_row(self, r, tensors=None):
        from oracle import xkv_oracle as O
        q = self.q[r:r + 1].cpu()
        if self.kind == "dense":
            return O.gqa_dense(q, self.k[r:r + 1].cpu().transpose(1, 2), self.v[r:r + 1].cpu().transpose(1, 2))
        if self.kind == "absorbed":
            return O.gqa_factorized(q, self.Ak[r:r + 1].cpu(), self.Bk[r:r + 1].cpu(), self.Av[r:r + 1].cpu(), self.Bv[r:r + 1].cpu())
        return O.xkv_fused_k_only(q[:, :, 0], self.Ak[r:r + 1].cpu(), self.Bk[r:r + 1].cpu(), self.v[r:r + 1].cpu(), 1.0)


def make_workload(args, world, rank):
    w = args.workload
    if w == "c5":
        return ReconRope(args, world, rank, name="c5_long_context_b128_L131072_R1024_H64", global_batch=128, H=64,
                         L=131072, R=1024, strong=True)
    if w == "c2":
        return ReconRope(args, world, rank, name="c2_qab_rope_b16_L16384_R512", global_batch=16, H=32, L=16384, R=512,
                         strong=False)
    if w in ("c3", "c3_vonly"):
        return Group(args, world, rank, v_only=(w == "c3_vonly"))
    if w == "c4":
        return Mla(args, world, rank)
    return Simple(args, world, rank, w)


def time_oracle_rows(wl, rows):
    """Oracle outputs of the given local rows and the seconds each took on the host cores."""
    torch.set_num_threads(os.cpu_count() or 1)
    outs, secs = [], []
    for r in rows:
        t0 = time.perf_counter()
        outs.append(wl.oracle_row(r))
        secs.append(time.perf_counter() - t0)
    return outs, secs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c5", "c2", "c3", "c3_vonly", "c4", "dense", "absorbed", "k_only"])
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"], help="c4 only: what the GPUs split")
    ap.add_argument("--rows", type=int, default=0, help="batch rows per GPU (cut-down case for profiler captures)")
    ap.add_argument("--kv-len", type=int, default=0, help="context length override (cut-down case)")
    ap.add_argument("--pair", default="auto", choices=["auto", "on", "off"], help="key reconstruction: CTA-pair kernel")
    ap.add_argument("--graph", default="off", choices=["off", "on"],
                    help="N = 1: capture one step (all of its launches) in a CUDA graph after the warm-up and replay it in the "
                         "timed region, as a serving loop would; the end-to-end figure stays the plain call")
    ap.add_argument("--gather", default="auto", choices=["auto", "nccl", "peer"],
                    help="N > 1: how the outputs are gathered.  peer = the library's peer-store kernel over symmetric memory; "
                         "auto = peer for steps under 2 ms when it can be set up and agrees with NCCL, else NCCL")
    ap.add_argument("--parity-rows", type=int, default=2, help="batch rows checked against the CPU oracle (0 = skip)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the oracle legs (parity and CPU baseline)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--force-generic", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = make_workload(args, world if args.impl == "ours" else 1, rank)
    tokens_per_row = getattr(wl, "tokens_per_row", lambda: 1)()
    config = {"workload": wl.name, "global_batch": wl.global_batch, "batch_per_gpu": wl.b, **wl.config(),
              "parallelism": (f"{args.shard if args.workload == 'c4' else 'batch'}-shard x{world}"
                              + (" + NCCL all-gather of outputs" if world > 1 else "")),
              "l2_policy": f"inputs ({wl.alg_bytes() / 1e9:.2f} GB per GPU per step) exceed the 126 MB L2"}

    if args.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)
        if not hasattr(wl, "cpu_inputs"):
            raise SystemExit("--impl reference covers the c5 and c2 workloads")
        A, V, B, q = wl.cpu_inputs()
        warm = min(args.warmup, 1)
        reps = max(1, min(args.steps, 3))
        ts = []
        for i in range(warm + reps):
            t0 = time.perf_counter()
            wl.oracle_row(0, (A, V, B, q))
            if i >= warm:
                ts.append(time.perf_counter() - t0)
        sec = statistics.median(ts)
        v = 1.0 / sec
        cores = torch.get_num_threads()
        sample = (f"1 of {wl.global_batch} batch rows at full context per step (fp32 math on the bf16-rounded inputs), "
                  f"median of {reps}; the whole batch is a linear extrapolation")
        line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": reps,
                "warmup": warm, "ms_per_step": 1e3 * sec, "rows_per_step": 1, "higher_is_better": True,
                "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
                "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    from kernel_collections_b200 import dist as xdist
    from oracle import xkv_oracle as O
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    wl.alloc(dev, seed=1000 + rank)
    wl.prepare()
    gather_dim = 1 if (args.workload == "c4" and args.shard == "heads") else 0
    total_gather = (wl.H if gather_dim == 1 else wl.b * world) if world > 1 else 0

    # how the outputs come together at N > 1: NCCL all-gather, or the library's peer-store kernel (batch shards only)
    peer_gather, gather_kind = None, "nccl"
    if world > 1 and gather_dim == 0 and args.gather in ("auto", "peer"):
        def all_ranks(flag: bool) -> bool:                    # every rank takes the same branch
            t = torch.tensor([1 if flag else 0], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
            return bool(int(t.item()))

        probe = wl.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(3):
            wl.step()
        torch.cuda.synchronize()
        if all_ranks(args.gather == "peer" or (time.perf_counter() - t0) / 3 < 2e-3):
            pg = None
            try:
                pg = xdist.PeerAllGather(tuple(probe.shape), probe.dtype, dev)
            except Exception as e:        # symmetric memory not available here: the collective stays
                sys.stderr.write(f"peer gather not used: {e!r}\n")
            if all_ranks(pg is not None):
                same = torch.equal(pg(probe), xdist.all_gather_outputs(probe, total_gather)) and pg.status()[0] == 0
                if all_ranks(same):
                    peer_gather, gather_kind = pg, "peer stores (xkv_peer_allgather)"
    if world > 1:
        config["parallelism"] = config["parallelism"].replace("NCCL all-gather of outputs", f"all-gather of outputs by {gather_kind}")

    def gather(o):
        if peer_gather is not None:
            return peer_gather(o)
        return xdist.all_gather_outputs(o if gather_dim == 0 else o.contiguous(), total_gather, dim=gather_dim)

    def step():
        o = wl.step()
        if world > 1:
            o = gather(o)
        return o

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    plan = wl.plan()
    stream = torch.cuda.current_stream()

    # ---- device-resident timing ---------------------------------------------------------------
    warm = max(args.warmup, 3)
    for _ in range(warm):
        out = step()
    barrier()
    run_step = step
    if args.graph == "on" and world == 1:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = step()
        torch.cuda.synchronize()

        def run_step():
            graph.replay()
            return graph_out
        for _ in range(3):
            run_step()
        barrier()
        config["cuda_graph"] = "one step captured after the warm-up and replayed in the timed region"
    sampler = ClockSampler(local_rank)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record(stream)
    for i in range(args.steps):
        out = run_step()
        ev[i + 1].record(stream)
    barrier()
    clocks = sampler.stop()
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    total_ms = ev[0].elapsed_time(ev[-1])

    # ---- the collective on its own (N > 1) -----------------------------------------------------
    gather_ms = 0.0
    if world > 1:
        local = wl.step()
        local = local if gather_dim == 0 else local.contiguous()
        for _ in range(3):
            gather(local)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(20):
            gather(local)
        g1.record(stream)
        barrier()
        gather_ms = g0.elapsed_time(g1) / 20

    # ---- parity of the timed tensors + CPU baseline (rank 0) --------------------------------------
    parity, cpu_baseline = None, None
    if rank == 0 and not args.no_cpu_baseline and args.parity_rows > 0:
        local_out = wl.step()
        torch.cuda.synchronize()
        rows = sorted({0, wl.b - 1, *range(1, max(1, min(args.parity_rows, wl.b) - 1))})[:max(1, args.parity_rows)]
        want, secs = time_oracle_rows(wl, rows)
        ma = rel = 0.0
        mag = 1.0
        for r, w_ in zip(rows, want):
            a_, r_ = O.error_metrics(local_out[r:r + 1], w_)
            ma, rel, mag = max(ma, a_), max(rel, r_), max(mag, w_.abs().max().item())
        parity = {"max_abs": ma, "rel_l2": rel, "rows": rows, "against": "CPU oracle, fp32 math on the timed bf16 inputs",
                  "tolerance": {"max_abs": 2e-2 * mag, "rel_l2": 1e-2,
                                "note": "max-abs bound is 2e-2 x max(1, largest |expected| value), as in the tests"},
                  "ok": bool(ma <= 2e-2 * mag and rel <= 1e-2)}
        if world == 1:
            sec = statistics.median(secs)
            cpu_baseline = {"value": tokens_per_row / sec, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                            "dtype": "f32",
                            "sample": f"{len(rows)} of {wl.global_batch} batch rows at full context, median row time "
                                      f"{sec:.2f} s; the whole batch is a linear extrapolation"}
    barrier()

    # ---- end to end: pinned host -> device, call, result -> host ---------------------------------
    e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    e2e_ms, e2e_steps = float("nan"), 0
    if not args.no_e2e:
        # every streamed tensor is refilled row by row from ONE pinned host row buffer per tensor (a
        # cudaMemcpyAsync per batch row: the bytes a full host copy would move, without holding tens of GB
        # of pinned memory); small tensors (projections, queries) are copied whole.
        host_rows = [t[0].cpu().pin_memory() for t in wl.streamed]
        host_small = [t.contiguous().cpu().pin_memory() for t in wl.small]
        dev_small = [t for t in wl.small]
        h2d = sum(t.numel() * t.element_size() for t in wl.streamed) + sum(t.numel() * t.element_size() for t in host_small)
        out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        d2h = out_host.numel() * out_host.element_size()

        def e2e_step():
            for t, h in zip(wl.streamed, host_rows):
                for r in range(t.shape[0]):
                    t[r].copy_(h, non_blocking=True)
            for t, h in zip(dev_small, host_small):
                if t.is_contiguous():
                    t.copy_(h, non_blocking=True)
            o = step()
            out_host.copy_(o, non_blocking=True)

        e2e_steps = 3 if wl.alg_bytes() > 8e9 else max(3, min(args.steps, 10))
        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1)
        e2e.update(h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, steps=e2e_steps,
                   note="every input copied from pinned host memory each step (streamed tensors row by row from one "
                        "reusable pinned row buffer per tensor, same bytes as a whole copy), output read back")

    t = torch.tensor([total_ms, e2e_ms, gather_ms], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    total_ms, e2e_ms, gather_ms = t.tolist()
    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    tokens = wl.global_batch * tokens_per_row
    value = tokens / (ms_per_step * 1e-3)
    if e2e_steps:
        e2e["value"] = tokens / (e2e_ms / e2e_steps * 1e-3)
    peaks = load_peaks()
    kern_ms = statistics.mean(per_step) - (gather_ms if world > 1 else 0.0)   # whole step charged to the dominant kernel
    tflops = wl.alg_flops() / (kern_ms * 1e-3) / 1e12
    gbs = wl.alg_bytes() / (kern_ms * 1e-3) / 1e9
    t_hbm = wl.alg_bytes() / (peaks["hbm_gbs"] * 1e9)
    t_tc = wl.alg_flops() / (peaks["bf16_tflops"] * 1e12)
    bound = "tensor" if t_tc >= t_hbm else "hbm"
    ratio, src = DRAM_PER_ALGORITHMIC_BYTE.get(plan if plan in DRAM_PER_ALGORITHMIC_BYTE else wl.kernel, (None, None))
    # tensor peak: the burst figure for a kernel timed alone, the sustained one when the clock sampler saw the power
    # cap bite during the timed region (tens of milliseconds of back-to-back tensor work); both fractions are reported
    capped = "sw_power_cap" in (clocks.get("reasons") or []) and peaks.get("bf16_tflops_sustained")
    tc_peak = peaks["bf16_tflops_sustained"] if capped else peaks["bf16_tflops"]
    roof = {"bound": bound, "kernel": plan,
            "achieved": tflops if bound == "tensor" else gbs,
            "peak": tc_peak if bound == "tensor" else peaks["hbm_gbs"],
            "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
            "frac": (tflops / tc_peak) if bound == "tensor" else gbs / peaks["hbm_gbs"],
            "traffic": None if ratio is None else ratio * wl.alg_bytes(),
            "traffic_source": None if ratio is None else
            f"{src}: DRAM bytes per algorithmic byte {ratio} of a cut-down capture, scaled to this launch",
            "peak_source": peaks["source"] + (" (sustained bf16 figure: sw_power_cap was active during the timed region)"
                                              if (capped and bound == "tensor") else " (burst figure)"),
            "hbm_gbs": gbs, "hbm_frac": gbs / peaks["hbm_gbs"], "tensor_tflops": tflops,
            "tensor_frac": tflops / peaks["bf16_tflops"],
            "tensor_frac_of_sustained_peak": (tflops / peaks["bf16_tflops_sustained"]) if peaks.get("bf16_tflops_sustained") else None,
            "algorithmic_bytes": wl.alg_bytes(), "algorithmic_flops": wl.alg_flops(), "per": "GPU and step",
            "timed": "CUDA events around each step on the launching stream; step time (minus the all-gather's own "
                     "time at N > 1) charged to the dominant kernel"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": wl.scaling, "vs_baseline": None, "dtype": {"bfloat16": "bf16", "float16": "f16", "float32": "f32"}.get(str(wl.dtype).replace("torch.", ""), str(wl.dtype)),
            "data": "synthetic", "config": config, "clocks": clocks, "e2e": e2e,
            "gpu_launches": wl.launches * args.steps, "roofline": roof}
    if world > 1:
        line["all_gather_ms"] = gather_ms
        line["all_gather"] = gather_kind
    if parity is not None:
        line["parity"] = parity
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
