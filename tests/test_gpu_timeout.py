"""The bounded device-side waits, exercised on purpose.

libxkv_faulttest.so is the library compiled with -DXKV_FAULT_TEST: every mbarrier wait gives up after
20 ms instead of a second, and the flag bit 0x80000000 makes the key-reconstruction kernel's TMA producer
announce one stage and never load it.  The MMA issuer's wait for that stage then runs out: the CTA raises
its abort flag, records role / tile / chunk / step in the workspace status words, every role drains to
the common exit, tensor memory is released and the call returns.  Nothing faults, traps or spins without
a bound; the context stays usable, which the follow-up calls on the same library check."""
import ctypes as C
import os

import pytest
import torch

from kernel_collections_b200 import _C, build as xbuild, ops
from kernel_collections_b200.attention import as_key_proj
from oracle import xkv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
FLAG_TEST_DROP_LOAD = 0x80000000


def _fault_lib():
    path = xbuild.FAULT_TEST_LIB
    if not os.path.exists(path):
        path = xbuild.build_fault_test()
    lib = C.CDLL(path)
    lib.xkv_decode_workspace_bytes.restype = C.c_size_t
    lib.xkv_decode_workspace_bytes.argtypes = [C.POINTER(_C.DecodeParams)]
    lib.xkv_decode.restype = C.c_int
    lib.xkv_decode.argtypes = [C.POINTER(_C.DecodeParams), C.c_void_p, C.c_size_t, C.c_void_p]
    lib.xkv_workspace_status.restype = C.c_int
    lib.xkv_workspace_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
    return lib


def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_correct():
    lib = _fault_lib()
    b, H, KVH, D, L, R, theta = 2, 32, 8, 128, 1000, 128, 500000.0
    g = torch.Generator().manual_seed(71)
    q = torch.randn(b, H, 1, D, generator=g).bfloat16()
    A = torch.randn(b, L, R, generator=g).bfloat16()
    B = (torch.randn(R, KVH * D, generator=g) / R ** 0.5).bfloat16()
    V = torch.randn(b, L, KVH, D, generator=g).bfloat16()
    qd, Ad, Bd, Vd = q.to(DEV), A.to(DEV), B.to(DEV), V.to(DEV)
    stream = torch.cuda.current_stream().cuda_stream

    def run(flags):
        p, out = ops.build_params(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=qd[:, :, 0], k=Ad,
                                  k_proj=as_key_proj(Bd, D), v=Vd, sm_scale=D ** -0.5, theta=theta,
                                  extra_flags=_C.FLAG_RECON_SINGLE_CTA | flags)
        ws = torch.empty(lib.xkv_decode_workspace_bytes(C.byref(p)), dtype=torch.uint8, device=DEV)
        rc = lib.xkv_decode(C.byref(p), ws.data_ptr(), ws.numel(), stream)
        assert rc == 0                                    # the launch itself succeeds: the failure is device-side
        detail = (C.c_int32 * 8)()
        return lib.xkv_workspace_status(ws.data_ptr(), stream, detail), list(detail), out

    want = O.recon_rope_decode(q, A, B.view(R, KVH, D).permute(1, 0, 2)[None].expand(b, -1, -1, -1), V.transpose(1, 2), theta)
    rc, detail, out = run(0)
    assert rc == 0, detail
    ma, rel = O.error_metrics(out.unsqueeze(2), want)
    assert ma <= 2e-2 and rel <= 1e-2
    rc, detail, _ = run(FLAG_TEST_DROP_LOAD)
    assert rc == -6, (rc, detail)                         # XKV_ERR_TIMEOUT
    # whoever waited longest reports first: the MMA issuer (role 1) waiting for the stage that never fills, or
    # the TMA producer (role 0) waiting, three stages on, for that same stage to be consumed; both in chunk 1
    assert detail[0] == -6 and detail[1] in (0, 1) and detail[3] == 1, detail
    # the context is intact and tensor memory was released: the same library runs the call correctly again
    for _ in range(2):
        rc, detail, out = run(0)
        assert rc == 0, detail
        ma, rel = O.error_metrics(out.unsqueeze(2), want)
        assert ma <= 2e-2 and rel <= 1e-2
    # and the Python layer's opt-in check turns such a status into an exception (host-side injection covered
    # in test_gpu_reference_configs.py); the regular library ignores the test-only flag bit
    p, out = ops.build_params(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=qd[:, :, 0], k=Ad,
                              k_proj=as_key_proj(Bd, D), v=Vd, sm_scale=D ** -0.5, theta=theta,
                              extra_flags=FLAG_TEST_DROP_LOAD)
    _C.run_decode(p, torch.device(DEV), "xkv_decode", check_status=True)
    ma, rel = O.error_metrics(out.unsqueeze(2), want)
    assert ma <= 2e-2 and rel <= 1e-2
