"""A read-only, prefix-addressable view of named tensors.

Parts ask for their tensors by names relative to their own prefix.  The view
resolves a name on demand, so the source can be a dict of loaded tensors or a
generator that draws a random tensor only when it is asked for (at real sizes
that keeps a single layer's temporaries alive instead of the whole model's).
A checkpoint whose names differ from the parts' by a rule is read through
``renamed``.
"""

from __future__ import annotations

from typing import Callable, Iterable, Mapping

import torch


class TensorView:
    def __init__(self, names: Iterable[str], get: Callable[[str], torch.Tensor], prefix: str = "",
                 stored_name: Callable[[str], str] | None = None) -> None:
        self._names = names if isinstance(names, frozenset) else frozenset(names)
        self._get = get
        self._prefix = prefix
        self._stored_name = stored_name

    @classmethod
    def of(cls, tensors: "Mapping[str, torch.Tensor] | TensorView") -> "TensorView":
        if isinstance(tensors, TensorView):
            return tensors
        return cls(tensors.keys(), tensors.__getitem__)

    def renamed(self, stored_name: Callable[[str], str]) -> "TensorView":
        """The same tensors under the names a model's parts use: the source knows the tensor a part calls
        ``name`` as ``stored_name(name)``."""

        return TensorView(self._names, self._get, self._prefix, stored_name)

    def sub(self, prefix: str) -> "TensorView":
        return TensorView(self._names, self._get, f"{self._prefix}{prefix}.", self._stored_name)

    def _source(self, name: str) -> str:
        full = f"{self._prefix}{name}"
        return self._stored_name(full) if self._stored_name is not None else full

    def __contains__(self, name: str) -> bool:
        return self._source(name) in self._names

    def __getitem__(self, name: str) -> torch.Tensor:
        source = self._source(name)
        if source not in self._names:
            raise KeyError(source)
        return self._get(source)

    def keys(self) -> list[str]:
        """Names below the prefix, as the source spells them."""

        cut = len(self._prefix)
        return sorted(n[cut:] for n in self._names if n.startswith(self._prefix))
