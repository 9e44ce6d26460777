"""Base class for symbolic PDE systems.

Parity: ``physicsnemo/sym/eq/pde.py`` (``PDE``: an ``equations`` dictionary of SymPy expressions,
``subs``, ``pprint``, ``make_computations``).  A subclass sets ``self.dim`` and fills
``self.equations`` in its constructor; each entry becomes one ``Computation`` whose inputs are the
symbols and derivative keys of the expression.
"""
from __future__ import annotations

from ...core.version_check import OptionalImport
from ..computation import Computation

sympy = OptionalImport("sympy")


class PDE:
    name = "PDE"

    def pprint(self, print_latex: bool = False) -> None:
        from ..utils.sympy.torch_printer import _subs_derivatives

        for key, value in self.equations.items():
            print(f"{key}: {_subs_derivatives(value)}")
        if print_latex:
            for key, value in self.equations.items():
                print(f"{key} = {sympy.latex(value)}")

    def subs(self, x, y) -> None:
        for name, eq in self.equations.items():
            self.equations[name] = eq.subs(x, y).doit()

    def make_computations(self, detach_names: list[str] | None = None) -> list[Computation]:
        return [Computation.from_sympy(eq, str(name), detach_names=list(detach_names or []))
                for name, eq in self.equations.items()]
