"""Python face of the sm_100a kernel library (``csrc/``): GEMM family, norms, fused blocks."""
from . import _lib
from .gemm import (
    ACT_GELU, ACT_NONE, ACT_RELU, ACT_SILU, ACT_SOFTMAX64,
    AUX_ADD, AUX_DGELU, AUX_DRELU, AUX_DSILU, AUX_DSOFTMAX, AUX_NONE,
    fused_path_enabled, gemm_nt, gemm_tn, gemm_tn_reference, linear, mlp_chain,
)
from .norm import layer_norm
from .graph import SegmentIndex, gather_rows, segment_reduce
from .patch_loss import squared_error, unpatchify


def library_available() -> bool:
    return _lib.available()


def kernel_launches() -> int:
    """Number of kernels of this library launched so far by this process."""
    from . import gemm

    return gemm.launch_count


def device_error() -> int:
    """Synchronising read of the library's device error word (0 = no bounded wait ran out)."""
    lib = _lib.load(required=True)
    return lib.pnm_get_error()
