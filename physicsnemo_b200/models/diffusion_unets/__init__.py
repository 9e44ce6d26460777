from .song_unet import SongUNet, SongUNetPosEmbd, SongUNetPosLtEmbd

__all__ = ["SongUNet", "SongUNetPosEmbd", "SongUNetPosLtEmbd"]
