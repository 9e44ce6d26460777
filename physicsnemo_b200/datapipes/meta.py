"""Datapipe capability record (parity: ``physicsnemo/datapipes/meta.py``)."""
from dataclasses import dataclass


@dataclass
class DatapipeMetaData:
    name: str = "BaseDatapipe"
    auto_device: bool = False
    cuda_graphs: bool = False
    ddp_sharding: bool = False
