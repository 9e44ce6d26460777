"""ctypes bindings of the four small-algebra kernels of the fused physics attention (``csrc/physics_attn_small.cu``)."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import _lib
from . import gemm as _g

S = 64  # slices per head covered by the kernels


def _lib_pa():
    lib = _lib.load(required=True)
    if not getattr(lib, "_pasmall_declared", False):
        c = ctypes
        vp, i, u, ll, f, d = c.c_void_p, c.c_int, c.c_uint, c.c_longlong, c.c_float, c.c_double
        lib.pnm_pa_prepare_fwd.argtypes = [vp] * 11 + [i, i, i, vp]
        lib.pnm_pa_tokens_fwd.argtypes = [vp, i, i, ll, i, vp, vp, vp, vp, i, i, i, f, vp, i, u, ll, d, vp, vp]
        lib.pnm_pa_tokens_bwd.argtypes = [vp, i, i, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, f, f, vp, i, u, ll, d, vp, vp]
        lib.pnm_pa_prepare_bwd.argtypes = [vp] * 12 + [i, i, i, vp]
        for n in ("pnm_pa_prepare_fwd", "pnm_pa_tokens_fwd", "pnm_pa_tokens_bwd", "pnm_pa_prepare_bwd"):
            getattr(lib, n).restype = i
        lib._pasmall_declared = True
    return lib


def _st():
    return torch.cuda.current_stream().cuda_stream


def _ptr_array(ptrs: Sequence[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def supported(H: int, D: int, slices: int, C: int, params: Sequence[torch.Tensor]) -> bool:
    return (slices == S and 0 < D <= 64 and 256 % D == 0 and (H * D) % 8 == 0 and C % 8 == 0
            and all(p.dtype == torch.float32 and p.is_cuda for p in params))


def prepare_fwd(Wx, bx, Wfx, Ws, bs, temp, H: int, D: int):
    """``(Wc bf16 [H*S, C], bc [H*S], inv_t [H*S], Wfx bf16, Wback bf16 [C, H*S + H*D])``."""
    C = Wx.shape[1]
    dev = Wx.device
    HS, inner = H * S, H * D
    Wc = torch.empty(HS, C, dtype=torch.bfloat16, device=dev)
    bc = torch.empty(HS, dtype=torch.float32, device=dev)
    inv_t = torch.empty(HS, dtype=torch.float32, device=dev)
    Wfx16 = torch.empty(inner, C, dtype=torch.bfloat16, device=dev)
    Wback = torch.empty(C, HS + inner, dtype=torch.bfloat16, device=dev)
    err = _lib_pa().pnm_pa_prepare_fwd(Wx.data_ptr(), bx.data_ptr(), Wfx.data_ptr(), Ws.data_ptr(), bs.data_ptr(),
                                       temp.data_ptr(), Wc.data_ptr(), bc.data_ptr(), inv_t.data_ptr(), Wfx16.data_ptr(),
                                       Wback.data_ptr(), H, D, C, _st())
    _g._check(err, "pnm_pa_prepare_fwd")
    _g.launch_count += 1
    return Wc, bc, inv_t, Wfx16, Wback


def new_saved(H: int, D: int, Cout: int, dev) -> List[torch.Tensor]:
    f = dict(dtype=torch.float32, device=dev)
    return [torch.empty(H, S, D, **f), torch.empty(H, S, **f), torch.empty(H, S, D, **f), torch.empty(H, S, D, **f),
            torch.empty(H, S, D, **f), torch.empty(H, S, S, **f), torch.empty(H, S, D, **f), torch.empty(Cout, H * S, **f)]


def tokens_fwd(src_ptrs: Sequence[int], norm_off: int, ld_tok: int, Wqkv, Wo, H: int, D: int, peer: Optional[tuple] = None):
    """``(Wcomb bf16 [Cout, H*S], saved)``; ``src_ptrs``: per rank the address of the [H*S, ld_tok] token-sum matrix.

    ``peer``: ``PeerRuntime.peer_args(epoch)`` when the sources are peers' buffers whose flags must be awaited.
    """
    Cout = Wo.shape[0]
    dev = Wo.device
    saved = new_saved(H, D, Cout, dev)
    wcomb16 = torch.empty(Cout, H * S, dtype=torch.bfloat16, device=dev)
    world = len(src_ptrs)
    use_flags = int(peer is not None)
    bases, rank, _w, epoch, cap, budget, ebase = peer if peer is not None else (None, 0, 1, 0, 0, 1.0, None)
    err = _lib_pa().pnm_pa_tokens_fwd(_ptr_array(src_ptrs), world, use_flags, norm_off, ld_tok, Wqkv.data_ptr(), Wo.data_ptr(),
                                      wcomb16.data_ptr(), _ptr_array([t.data_ptr() for t in saved]), H, D, Cout,
                                      float(D) ** -0.5, bases, rank, epoch, cap, budget, ebase, _st())
    _g._check(err, "pnm_pa_tokens_fwd")
    _g.launch_count += 1
    return wcomb16, saved


def tokens_bwd(src_ptrs: Sequence[int], Wqkv, Wo, saved, H: int, D: int, share: float, peer: Optional[tuple] = None):
    """``(dWo, dWqkv, d_norm [H*S], Bcat bf16 [H*S, Cout + H*D], BdT bf16 [H*D, H*S])``."""
    Cout = Wo.shape[0]
    dev = Wo.device
    inner = H * D
    dWo = torch.empty(Cout, inner, dtype=torch.float32, device=dev)
    dWqkv = torch.zeros(3 * D, D, dtype=torch.float32, device=dev)
    d_norm = torch.empty(H * S, dtype=torch.float32, device=dev)
    Bcat = torch.empty(H * S, Cout + inner, dtype=torch.bfloat16, device=dev)
    BdT = torch.empty(inner, H * S, dtype=torch.bfloat16, device=dev)
    world = len(src_ptrs)
    use_flags = int(peer is not None)
    bases, rank, _w, epoch, cap, budget, ebase = peer if peer is not None else (None, 0, 1, 0, 0, 1.0, None)
    err = _lib_pa().pnm_pa_tokens_bwd(_ptr_array(src_ptrs), world, use_flags, Wqkv.data_ptr(), Wo.data_ptr(),
                                      _ptr_array([t.data_ptr() for t in saved]), dWo.data_ptr(), dWqkv.data_ptr(),
                                      d_norm.data_ptr(), Bcat.data_ptr(), BdT.data_ptr(), H, D, Cout, float(D) ** -0.5,
                                      float(share), bases, rank, epoch, cap, budget, ebase, _st())
    _g._check(err, "pnm_pa_tokens_bwd")
    _g.launch_count += 1
    return dWo, dWqkv, d_norm, Bcat, BdT


def prepare_bwd(dWc, dbc, grp, Wx, bx, Ws, temp, H: int, D: int):
    """``(dWx, dbx, dWs, dbs, dtemp)`` from the gradients of the combined projection."""
    C = Wx.shape[1]
    dev = Wx.device
    f = dict(dtype=torch.float32, device=dev)
    dWx, dbx = torch.empty(H * D, C, **f), torch.empty(H * D, **f)
    dWs, dbs, dtemp = torch.empty(S, D, **f), torch.empty(S, **f), torch.empty(H, **f)
    err = _lib_pa().pnm_pa_prepare_bwd(dWc.data_ptr(), dbc.data_ptr(), grp.data_ptr(), Wx.data_ptr(), bx.data_ptr(),
                                       Ws.data_ptr(), temp.data_ptr(), dWx.data_ptr(), dbx.data_ptr(), dWs.data_ptr(),
                                       dbs.data_ptr(), dtemp.data_ptr(), H, D, C, _st())
    _g._check(err, "pnm_pa_prepare_bwd")
    _g.launch_count += 1
    return dWx, dbx, dWs, dbs, dtemp
