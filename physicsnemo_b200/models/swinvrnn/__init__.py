from .swinvrnn import SwinRNN
