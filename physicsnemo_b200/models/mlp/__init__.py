from .fully_connected import FullyConnected
