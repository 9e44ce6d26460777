from .patching import BasePatching2D, GridPatching2D, RandomPatching2D, image_batching, image_fuse

__all__ = ["BasePatching2D", "GridPatching2D", "RandomPatching2D", "image_batching", "image_fuse"]
