"""Package-level names that resolve on first use.

A package lists ``public name -> (module, attribute)`` and gets a module ``__getattr__`` / ``__dir__`` pair
(PEP 562): ``from research_b200.optim import build_optimizer`` works, yet importing the package does not import its
submodules, so packages that refer to one another do not form import cycles and ``import research_b200`` stays cheap.
"""

from __future__ import annotations

import importlib
from typing import Mapping


def lazy_exports(package: str, table: Mapping[str, tuple[str, str]], eager: tuple[str, ...] = ()):
    """Returns ``(__getattr__, __dir__, __all__)`` for ``package``; ``eager`` are names it already defines."""

    names = sorted(set(table) | set(eager))

    def __getattr__(name: str):
        try:
            module, attr = table[name]
        except KeyError:
            raise AttributeError(f"module {package!r} has no attribute {name!r}") from None
        value = getattr(importlib.import_module(module), attr)
        import sys

        setattr(sys.modules[package], name, value)          # next time it is a plain attribute
        return value

    def __dir__():
        return names

    return __getattr__, __dir__, names
