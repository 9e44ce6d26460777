from .patch_embed import PatchEmbed2D, PatchEmbed3D, PatchRecovery2D, PatchRecovery3D
from .shift_window_mask import get_shift_window_mask, window_partition, window_reverse
from .utils import _validate_amp, crop2d, crop3d, get_earth_position_index, get_pad2d, get_pad3d
from .weight_init import _weight_init, shrink_and_perturb_
