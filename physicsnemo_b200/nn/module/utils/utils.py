"""Small shared helpers of the layer library (parity: ``physicsnemo/nn/module/utils/utils.py``)."""
import torch


def _validate_amp(amp_mode: bool) -> None:
    """With ``amp_mode=False`` the layers cast parameters themselves, which conflicts with autocast."""
    if not amp_mode and (torch.is_autocast_enabled() or torch.is_autocast_enabled("cpu")):
        raise ValueError(
            "amp_mode is False, but torch autocast is enabled. Set `amp_mode=True` on the model "
            "(e.g. `model.amp_mode = True`) to run under automatic mixed precision."
        )


def _recursive_property(name: str, typ: type, doc: str):
    """Property that, when set, also sets the same attribute on every sub-module that has it."""
    private = "_" + name

    def getter(self):
        return getattr(self, private)

    def setter(self, value):
        if not isinstance(value, typ):
            raise TypeError(f"{name} must be a {typ.__name__} value.")
        setattr(self, private, value)
        for sub in self.children():
            if hasattr(sub, name):
                setattr(sub, name, value)

    return property(getter, setter, doc=doc)
