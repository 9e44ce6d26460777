"""Window partitioning for earth-specific (longitude-periodic) shifted-window attention.

Parity: ``physicsnemo/nn/module/utils/shift_window_mask.py``.  Windows are grouped *longitude-major*:
``window_partition`` returns ``[B·n_lon, n_other, *window, C]`` so that the position bias (which depends on the
pressure / latitude window but not on the longitude window) broadcasts over the first axis.
"""
import torch


def window_partition(x: torch.Tensor, window_size, ndim=3):
    if ndim == 3:
        B, Pl, Lat, Lon, C = x.shape
        wp, wl, wo = window_size
        x = x.view(B, Pl // wp, wp, Lat // wl, wl, Lon // wo, wo, C).permute(0, 5, 1, 3, 2, 4, 6, 7)
        return x.contiguous().view(-1, (Pl // wp) * (Lat // wl), wp, wl, wo, C)
    B, Lat, Lon, C = x.shape
    wl, wo = window_size
    x = x.view(B, Lat // wl, wl, Lon // wo, wo, C).permute(0, 3, 1, 2, 4, 5)
    return x.contiguous().view(-1, Lat // wl, wl, wo, C)


def window_reverse(windows, window_size, Pl=1, Lat=1, Lon=1, ndim=3):
    if ndim == 3:
        wp, wl, wo = window_size
        B = windows.shape[0] // (Lon // wo)
        x = windows.view(B, Lon // wo, Pl // wp, Lat // wl, wp, wl, wo, -1).permute(0, 2, 4, 3, 5, 1, 6, 7)
        return x.contiguous().view(B, Pl, Lat, Lon, -1)
    wl, wo = window_size
    B = windows.shape[0] // (Lon // wo)
    x = windows.view(B, Lon // wo, Lat // wl, wl, wo, -1).permute(0, 2, 3, 1, 4, 5)
    return x.contiguous().view(B, Lat, Lon, -1)


def get_shift_window_mask(input_resolution, window_size, shift_size, ndim=3):
    """Additive mask (0 / −100) that forbids attention between tokens brought together by the cyclic shift along
    pressure and latitude; longitude wraps physically, so only its seam region (computed on an extended strip)
    is labelled."""
    *lead, Lon = input_resolution
    *wlead, w_lon = window_size
    *slead, s_lon = shift_size
    labels = torch.zeros((1, *lead, Lon + s_lon, 1))
    bands = [(slice(0, -w), slice(-w, -s), slice(-s, None)) for w, s in zip(window_size, shift_size)]
    cnt = 0
    import itertools

    for combo in itertools.product(*bands):
        labels[(slice(None), *combo, slice(None))] = cnt
        cnt += 1
    labels = labels[..., :Lon, :]
    win = window_partition(labels, window_size, ndim=ndim)
    win = win.view(win.shape[0], win.shape[1], -1)
    diff = win.unsqueeze(2) - win.unsqueeze(3)
    return torch.where(diff != 0, torch.full_like(diff, -100.0), torch.zeros_like(diff))
