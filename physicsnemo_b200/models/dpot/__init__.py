from .dpot import DPOTNet, DPOTNet3D, checkpoint_filter_fn, resize_pos_embed  # noqa: F401
