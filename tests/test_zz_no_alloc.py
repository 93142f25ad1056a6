"""The allocation-free entry point, xkv_decode_builtin_scratch.

It exists for hosts that may not allocate device memory when they call into the library — a
plugin inside a serving process whose memory pool was carved up at start-up, a latency-critical
loop that must stay out of the allocator, a process whose device memory another runtime owns.
Such a caller hands over its inputs and a preallocated output and nothing else; the split-KV
scratch lives in an 8 MiB array compiled into libxkv.so.

The checks run through the C ABI and compare against the regular entry point (xkv_decode with a
caller workspace, portable kernels) on the same inputs: the two run the same kernels on the
same split plan, so the outputs must be bit-identical.  Two calls in a row with different
inputs show that what one call leaves in the shared array does not leak into the next, and an
over-sized request must be refused with the dedicated status code before anything launches.

This file is collected last on purpose; it must pass on its own and after the other tests.
"""
import ctypes as C

import pytest
import torch

from kernel_collections_b200 import _C, ops
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(seed, b, H, KVH, D, L, dtype):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, H, D, generator=g).to(dtype).to(DEV)
    k = torch.randn(b, L, KVH, D, generator=g).to(dtype).to(DEV)
    v = torch.randn(b, L, KVH, D, generator=g).to(dtype).to(DEV)
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_builtin_scratch_matches_workspace_path_twice_in_a_row(dtype):
    b, H, KVH, D, L = 2, 8, 2, 64, 3000
    for seed in (101, 202):           # two calls in a row, different data, same shared array
        q, k, v = _inputs(seed, b, H, KVH, D, L, dtype)
        kw = dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=q, k=k, v=v, sm_scale=D ** -0.5)
        want = ops.decode(entry="xkv_decode", force_generic=True, **kw)
        out = torch.full((b, H, D), float("nan"), dtype=dtype, device=DEV)   # caller-owned output
        got = ops.decode_builtin_scratch(out=out, **kw)
        torch.cuda.synchronize()
        assert got is out
        assert torch.isfinite(out.float()).all()
        assert torch.equal(out, want), f"seed {seed}: max diff {(out.float() - want.float()).abs().max().item():.3e}"
        # and against the CPU restatement of the reference's math, within the library's tolerances
        ref = O.flash_decode_gqa(q.cpu(), k.cpu(), v.cpu(), sm_scale=D ** -0.5)
        ma, rel = O.error_metrics(out, ref)
        tol = (1e-4, 1e-4) if dtype == torch.float32 else (2e-2, 1e-2)
        assert ma <= tol[0] and rel <= tol[1], f"seed {seed}: max_abs={ma:.3e} rel_l2={rel:.3e} against the oracle"


def test_builtin_scratch_factorized_rope_path():
    """Not only the dense mode: factorized K with RoPE and a factorized V through the same entry."""
    b, H, KVH, D, L, R, Rv = 2, 8, 2, 64, 500, 32, 24
    g = torch.Generator().manual_seed(7)
    q = torch.randn(b, H, D, generator=g).to(DEV)
    A = torch.randn(b, L, R, generator=g).to(DEV)
    B = (torch.randn(b, KVH, R, D, generator=g) / R ** 0.5).to(DEV)
    Av = torch.randn(b, L, Rv, generator=g).to(DEV)
    Bv = (torch.randn(b, KVH, Rv, D, generator=g) / Rv ** 0.5).to(DEV)
    kw = dict(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_LATENT, q=q, k=A, k_proj=B, v=Av, v_proj=Bv,
              sm_scale=D ** -0.5, theta=10000.0)
    want = ops.decode(entry="xkv_decode", force_generic=True, **kw)
    out = torch.empty(b, H, D, device=DEV)
    ops.decode_builtin_scratch(out=out, **kw)
    assert torch.equal(out, want)


def test_builtin_scratch_rejects_oversized_requests():
    # 8 x 64 heads x 512 splits x 512 value columns of fp32 partials is far beyond 8 MiB
    b, H, KVH, D, L = 8, 64, 64, 512, 8192
    q = torch.zeros(b, H, D, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(b, L, KVH, D, dtype=torch.bfloat16, device=DEV)
    kw = dict(score_mode=_C.SCORE_DENSE, value_mode=_C.VALUE_DENSE, q=q, k=k, v=k, sm_scale=1.0, num_splits=512)
    p, _ = ops.build_params(**kw)
    lib = _C.load()
    assert lib.xkv_decode_workspace_bytes(C.byref(p)) > _C.BUILTIN_SCRATCH_BYTES
    rc = lib.xkv_decode_builtin_scratch(C.byref(p), torch.cuda.current_stream().cuda_stream)
    assert rc == -8
    assert "built-in" in _C.strerror(rc)
    with pytest.raises(ValueError, match="built-in"):
        ops.decode_builtin_scratch(**kw)
    # and a bad parameter block is still a bad-argument error, not a scratch error
    assert lib.xkv_decode_builtin_scratch(None, None) == -1
