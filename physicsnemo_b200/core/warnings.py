"""Warning categories (parity: ``physicsnemo/core/warnings.py``)."""


class ExperimentalFeatureWarning(UserWarning):
    """Raised when an experimental feature is used."""


class FutureFeatureWarning(FutureWarning):
    """Raised when a feature is scheduled to change."""


class LegacyFeatureWarning(DeprecationWarning):
    """Raised when a legacy feature is used."""
