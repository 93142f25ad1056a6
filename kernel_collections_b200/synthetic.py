"""Seeded synthetic inputs of the benchmark configurations, with their algorithmic byte and
flop counts.  Inputs are drawn on the CPU in fp32 from torch.manual_seed(seed), in the order
the configuration lists them, then rounded to the working dtype — so a CPU checker and the GPU
kernels see identical bits."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class ReconRopeConfig:
    """Factorized K with RoPE + dense V, one decode step (the 'qAB_rope' configuration)."""
    name: str = "c2_qab_rope_b16_L16384_R512"
    batch: int = 16
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    kv_len: int = 16384
    rank: int = 512
    theta: float = 500000.0
    dtype: torch.dtype = torch.bfloat16

    @property
    def elem(self) -> int:
        return 2 if self.dtype in (torch.bfloat16, torch.float16) else 4

    def algorithmic_bytes(self) -> int:
        """Latent A + dense V streamed once, B once, q in and o out."""
        b, L, R, KD = self.batch, self.kv_len, self.rank, self.num_kv_heads * self.head_dim
        return self.elem * (b * L * (R + KD) + R * KD + 2 * b * self.num_heads * self.head_dim)

    def latent_bytes(self) -> int:
        return self.elem * self.batch * self.kv_len * self.rank

    def algorithmic_flops(self) -> int:
        """Key rebuild 2.b.L.R.KVH.D plus attention 4.b.H.L.D."""
        b, L, R = self.batch, self.kv_len, self.rank
        return 2 * b * L * R * self.num_kv_heads * self.head_dim + 4 * b * self.num_heads * L * self.head_dim

    def scaled(self, **kw) -> "ReconRopeConfig":
        d = dict(self.__dict__)
        d.update(kw)
        return ReconRopeConfig(**d)


def recon_rope_inputs(cfg: ReconRopeConfig, seed: int = 0, batch_rows=None):
    """CPU tensors (A, B, q, V) in cfg.dtype: A (b,L,R) ~ N(0,1); B (R, KVH*D) ~ N(0,1/R);
    q (b,H,1,D) ~ N(0,1); V (b,L,KVH,D) ~ N(0,1) stored token-major.  `batch_rows` draws only
    the first rows of the batch (a bounded sample of the same distribution)."""
    b = cfg.batch if batch_rows is None else batch_rows
    g = torch.Generator().manual_seed(seed)
    KD = cfg.num_kv_heads * cfg.head_dim
    A = torch.randn(b, cfg.kv_len, cfg.rank, generator=g).to(cfg.dtype)
    B = (torch.randn(cfg.rank, KD, generator=g) / cfg.rank ** 0.5).to(cfg.dtype)
    q = torch.randn(b, cfg.num_heads, 1, cfg.head_dim, generator=g).to(cfg.dtype)
    V = torch.randn(b, cfg.kv_len, cfg.num_kv_heads, cfg.head_dim, generator=g).to(cfg.dtype)
    return A, B, q, V
