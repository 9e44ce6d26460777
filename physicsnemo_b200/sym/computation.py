"""A named node of the symbolic graph: which keys it reads, which it writes, and the callable.

Parity: ``physicsnemo/sym/computation.py`` (``Computation``; inputs containing the derivative
separator are kept apart as ``derivatives`` so the scheduler can ask a gradient node for them).
"""
from __future__ import annotations

from typing import Callable, Sequence

from .constants import diff_str


class Computation:
    def __init__(self, inputs: Sequence[str] | str, outputs: Sequence[str], evaluate: Callable,
                 name: str = "Computation"):
        if isinstance(inputs, str):
            inputs = [inputs]
        names = [str(x) for x in inputs]
        self._inputs = [n for n in names if diff_str not in n]
        self._derivatives = [n for n in names if diff_str in n]
        self._outputs = [str(x) for x in outputs]
        self.evaluate = evaluate
        self._name = name

    @classmethod
    def from_sympy(cls, eq, out_name: str, freeze_terms=None, detach_names=None) -> "Computation":
        from .utils.sympy.torch_printer import SympyToTorch, _subs_derivatives

        module = SympyToTorch(_subs_derivatives(eq), out_name, list(freeze_terms or []), list(detach_names or []))
        return cls(list(module.keys), [out_name], module, name="Sympy Computation: " + out_name)

    name = property(lambda self: self._name)
    outputs = property(lambda self: self._outputs)
    inputs = property(lambda self: self._inputs)
    derivatives = property(lambda self: self._derivatives)

    def __str__(self) -> str:
        return (f"computation: {self.name}\n  inputs: {self.inputs}\n  derivatives: {self.derivatives}\n"
                f"  outputs: {self.outputs}")
