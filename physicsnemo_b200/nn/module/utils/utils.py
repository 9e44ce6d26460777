"""Small shared helpers of the layer library (parity: ``physicsnemo/nn/module/utils/utils.py``)."""
import torch


def _validate_amp(amp_mode: bool) -> None:
    """With ``amp_mode=False`` the layers cast parameters themselves, which conflicts with autocast."""
    if not amp_mode and (torch.is_autocast_enabled() or torch.is_autocast_enabled("cpu")):
        raise ValueError(
            "amp_mode is False, but torch autocast is enabled. Set `amp_mode=True` on the model "
            "(e.g. `model.amp_mode = True`) to run under automatic mixed precision."
        )


def _recursive_property(name: str, typ: type, doc: str):
    """Property that, when set, also sets the same attribute on every sub-module that has it."""
    private = "_" + name

    def getter(self):
        return getattr(self, private)

    def setter(self, value):
        if not isinstance(value, typ):
            raise TypeError(f"{name} must be a {typ.__name__} value.")
        setattr(self, private, value)
        for sub in self.children():
            if hasattr(sub, name):
                setattr(sub, name, value)

    return property(getter, setter, doc=doc)


# ----------------------------------------------------------------- earth-window helpers
def get_earth_position_index(window_size, ndim=3):
    """Index into the earth-specific position-bias table for every (query, key) pair of a window.

    Parity: ``physicsnemo/nn/module/utils/utils.py:20-76``.  Pressure-level and latitude offsets are *absolute*
    pairs (``i + j·W``: the bias depends on both heights / latitudes), the longitude offset is relative
    (``i − j + W − 1``: longitude is periodic).
    """
    import torch

    sizes = tuple(window_size)
    if len(sizes) != ndim:
        raise ValueError(f"window_size must have {ndim} entries")
    *abs_axes, w_lon = sizes
    grids_q = [torch.arange(w) for w in abs_axes] + [torch.arange(w_lon)]
    grids_k = [-torch.arange(w) * w for w in abs_axes] + [torch.arange(w_lon)]
    cq = torch.stack(torch.meshgrid(grids_q, indexing="ij")).flatten(1)
    ck = torch.stack(torch.meshgrid(grids_k, indexing="ij")).flatten(1)
    rel = (cq[:, :, None] - ck[:, None, :]).permute(1, 2, 0).contiguous()
    rel[:, :, -1] += w_lon - 1
    stride = 2 * w_lon - 1
    for a in range(len(abs_axes) - 1, -1, -1):
        rel[:, :, a] *= stride
        stride *= abs_axes[a] * abs_axes[a]
    return rel.sum(-1)


def _split_pad(total):
    lo = total // 2
    return lo, total - lo


def get_pad3d(input_resolution, window_size):
    """``(left, right, top, bottom, front, back)`` zero padding that makes every extent a multiple of its window."""
    pads = []
    for n, w in zip(input_resolution, window_size):
        pads.append(_split_pad((w - n % w) % w))
    (front, back), (top, bottom), (left, right) = pads
    return left, right, top, bottom, front, back


def get_pad2d(input_resolution, window_size):
    return get_pad3d([2, *input_resolution], [2, *window_size])[:4]


def _center_crop(x, resolution):
    sl = [slice(None), slice(None)]
    for have, want in zip(x.shape[2:], resolution):
        lo, hi = _split_pad(have - want)
        sl.append(slice(lo, have - hi))
    return x[tuple(sl)]


def crop2d(x, resolution):
    return _center_crop(x, resolution[:2])


def crop3d(x, resolution):
    return _center_crop(x, resolution[:3])
