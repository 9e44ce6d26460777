"""HEALPix time-series datapipes (parity: ``physicsnemo/datapipes/healpix``)."""
from .coupledtimeseries_dataset import CoupledTimeSeriesDataset
from .couplers import ConstantCoupler, TrailingAverageCoupler
from .timeseries_dataset import ArrayStore, TimeSeriesDataset, to_timedelta
from .data_modules import (CoupledTimeSeriesDataModule, TimeSeriesDataModule, create_time_series_dataset_classic,
                           open_time_series_dataset_classic_on_the_fly, open_time_series_dataset_classic_prebuilt)

__all__ = ["CoupledTimeSeriesDataModule", "TimeSeriesDataModule", "create_time_series_dataset_classic",
           "open_time_series_dataset_classic_on_the_fly", "open_time_series_dataset_classic_prebuilt", "ArrayStore", "ConstantCoupler", "CoupledTimeSeriesDataset", "TimeSeriesDataset", "TrailingAverageCoupler", "to_timedelta"]
