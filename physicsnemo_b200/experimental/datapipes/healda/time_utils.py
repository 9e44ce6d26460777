"""Conversions between the time types the pipeline meets (``datetime``, ``numpy.datetime64``, ``pandas.Timestamp``,
``cftime`` when installed) and the scalar encodings the models take.

Parity: ``physicsnemo/experimental/datapipes/healda/time_utils.py``.  ``cftime`` is optional here:
``as_cftime`` returns a timezone-aware ``datetime`` when the package is missing, and every function
accepts either kind of object.
"""
from __future__ import annotations

import datetime

import numpy as np

try:  # pragma: no cover - optional dependency
    import cftime
except ImportError:  # pragma: no cover
    cftime = None

_UTC = datetime.timezone.utc


def _is_cftime(t) -> bool:
    return cftime is not None and isinstance(t, cftime.datetime)


def as_pydatetime(time) -> datetime.datetime:
    if _is_cftime(time):
        return datetime.datetime(time.year, time.month, time.day, time.hour, time.minute, time.second, tzinfo=_UTC)
    if isinstance(time, datetime.datetime):            # includes pandas.Timestamp
        return time
    if isinstance(time, np.datetime64):
        return datetime.datetime.fromtimestamp(int(time.astype("datetime64[s]").astype(np.int64)), tz=_UTC)
    raise NotImplementedError(type(time))


def as_numpy(time) -> np.ndarray:
    """1-D ``datetime64`` array from a scalar or a sequence of any supported time type."""
    if hasattr(time, "values"):
        return np.asarray(time.values)
    if isinstance(time, np.datetime64):
        return np.array([time])
    if _is_cftime(time) or isinstance(time, datetime.datetime):
        return np.array([np.datetime64(as_pydatetime(time).replace(tzinfo=None))])
    return np.array([as_numpy(t)[0] for t in time])


def as_timestamp(time) -> np.ndarray:
    """Whole seconds since the epoch."""
    return as_numpy(time).astype("datetime64[s]").astype(np.int64)


def as_cftime(timestamp):
    """Gregorian ``cftime`` object for a timestamp-like; a UTC ``datetime`` when ``cftime`` is not installed."""
    t = as_pydatetime(timestamp)
    if cftime is None:
        return t.replace(tzinfo=_UTC) if t.tzinfo is None else t
    return cftime.DatetimeGregorian(t.year, t.month, t.day, t.hour, t.minute, t.second)


def cftime_to_timestamp(time) -> float:
    t = as_pydatetime(time)
    return (t.replace(tzinfo=_UTC) if t.tzinfo is None else t).timestamp()


def compute_timestamp(time) -> int:
    return int(cftime_to_timestamp(time))


def _start_of_day(time):
    return time.replace(hour=0, minute=0, second=0, microsecond=0) if isinstance(time, datetime.datetime) else \
        time.replace(hour=0, minute=0, second=0)


def compute_second_of_day(time) -> float:
    return (time - _start_of_day(time)) / datetime.timedelta(seconds=1)


second_of_day = compute_second_of_day


def compute_day_of_year(time) -> float:
    """Days since 1 January 00:00 of the same year, fractional."""
    return (time - _start_of_day(time).replace(month=1, day=1)) / datetime.timedelta(days=1)
