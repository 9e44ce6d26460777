from .meta import ModelMetaData
from .registry import ModelRegistry
from .module import Module
from .function_spec import FunctionSpec
from .filesystem import Package
from .version_check import OptionalImport, check_version_spec, require_version_spec
from .warnings import ExperimentalFeatureWarning, FutureFeatureWarning, LegacyFeatureWarning

__all__ = [
    "ModelMetaData", "ModelRegistry", "Module", "FunctionSpec", "Package", "OptionalImport",
    "check_version_spec", "require_version_spec",
    "ExperimentalFeatureWarning", "FutureFeatureWarning", "LegacyFeatureWarning",
]
