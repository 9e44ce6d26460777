"""Legacy ``Datapipe`` base used by the generator-style pipes (parity: ``physicsnemo/datapipes/datapipe.py``)."""
import logging

from .meta import DatapipeMetaData


class Datapipe:
    def __init__(self, meta: DatapipeMetaData = None):
        self.logger = logging.getLogger("core.datapipe")
        if not meta or not isinstance(meta, DatapipeMetaData):
            self.meta = DatapipeMetaData()
        else:
            self.meta = meta
        self.logger.info(f"Datapipe {self.meta.name} initialized")

    def debug(self):
        self.logger.setLevel(logging.DEBUG)
