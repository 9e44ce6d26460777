"""Allocation-free LayerNorm backward (``pnm_layernorm_bwd_noalloc``).

Some users of the kernel library cannot ask for device memory at call time (fixed memory
budget already handed out, buffers owned by a foreign allocator, or a loop that must not
hit the device synchronisation of ``cudaMalloc``).  For them the library keeps the scratch
of the LayerNorm backward in a static device array.  This test drives that entry point
through its exported C symbol, twice in a row, and checks it against the regular entry
point that takes a caller-provided scratch buffer.
"""
import ctypes

import pytest
import torch

from physicsnemo_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _bind(lib):
    c = ctypes
    fn = lib.pnm_layernorm_bwd_noalloc
    fn.argtypes = [c.c_void_p] * 9 + [c.c_longlong, c.c_int, c.c_void_p]
    fn.restype = c.c_int
    return fn


@pytest.mark.parametrize("M,C,with_dres", [(4099, 256, False), (777, 768, False), (1531, 8, False), (613, 1024, True),
                                            (2050, 256, True)])
def test_noalloc_matches_regular_entry_point_twice(M, C, with_dres):
    lib = _lib.load(required=True)
    noalloc = _bind(lib)
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream().cuda_stream
    gamma = (torch.rand(C, device=dev) + 0.5).float()
    for trial in range(2):  # the second call reuses the scratch left by the first
        torch.manual_seed(100 + trial)
        x = torch.randn(M, C, device=dev).to(torch.bfloat16)
        dy = torch.randn(M, C, device=dev).to(torch.bfloat16)
        dres = torch.randn(M, C, device=dev).to(torch.bfloat16) if with_dres else None
        dres_ptr = None if dres is None else dres.data_ptr()
        xf = x.float()
        mean = xf.mean(1).contiguous()
        rstd = torch.rsqrt(xf.var(1, unbiased=False) + 1e-5).contiguous()
        # regular entry point (caller-provided scratch)
        dx_ref = torch.empty_like(x)
        dg_ref = torch.empty(C, device=dev)
        db_ref = torch.empty(C, device=dev)
        scratch = torch.empty(lib.pnm_layernorm_bwd_scratch_floats(M, C), device=dev)
        rc = lib.pnm_layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                   dres_ptr, dx_ref.data_ptr(), dg_ref.data_ptr(), db_ref.data_ptr(), scratch.data_ptr(),
                                   M, C, stream)
        assert rc == 0
        # allocation-free entry point: outputs are pre-allocated here, nothing is allocated inside
        dx = torch.empty_like(x)
        dg = torch.empty(C, device=dev)
        db = torch.empty(C, device=dev)
        rc = noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dres_ptr,
                     dx.data_ptr(), dg.data_ptr(), db.data_ptr(), M, C, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)  # per-row math is identical
        scale = max(1.0, dg_ref.abs().max().item())
        assert (dg - dg_ref).abs().max().item() <= 2e-2 * scale
        assert (db - db_ref).abs().max().item() <= 2e-2 * max(1.0, db_ref.abs().max().item())


def test_noalloc_rejects_oversize():
    lib = _lib.load(required=True)
    noalloc = _bind(lib)
    t = torch.zeros(8, device="cuda")
    rc = noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(),
                 t.data_ptr(), t.data_ptr(), 16, 2048, None)
    assert rc == -101
    rc = noalloc(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(),
                 t.data_ptr(), t.data_ptr(), 16, 12, None)
    assert rc == -101
