"""HEALPix time-series datapipes (parity: ``physicsnemo/datapipes/healpix``)."""
from .coupledtimeseries_dataset import CoupledTimeSeriesDataset
from .couplers import ConstantCoupler, TrailingAverageCoupler
from .timeseries_dataset import ArrayStore, TimeSeriesDataset, to_timedelta

__all__ = ["ArrayStore", "ConstantCoupler", "CoupledTimeSeriesDataset", "TimeSeriesDataset", "TrailingAverageCoupler", "to_timedelta"]
