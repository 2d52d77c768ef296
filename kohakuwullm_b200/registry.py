"""String-keyed component registries and the one ``build`` entry point.

"Select, don't dispatch": a config names a component once, ``build`` turns that name into a
concrete object at construction time, and nothing branches on configuration afterwards.

A *spec* may be
  * ``None``                         -> ``None``
  * an already built object          -> returned as is
  * a registered name / dotted path  -> looked up (or imported) and called with the defaults
  * ``{"name": ..., **kwargs}``      -> looked up and called with defaults overridden by kwargs
  * a class or factory               -> called with the defaults
  * an object exposing ``.build()``  -> ``spec.build(**defaults)``

Same contract as the reference's src/kohakuwullm/registry.py:12-94.
"""

from __future__ import annotations

from typing import Any, Callable, Iterator

from kohakuwullm_b200.utils.misc import import_class


class Registry:
    """Name -> factory table. Registering a name twice is an error."""

    def __init__(self, kind: str):
        self.kind = kind
        self._table: dict[str, Callable[..., Any]] = {}

    def register(self, name: str, obj: Callable[..., Any] | None = None):
        def _put(target):
            if name in self._table:
                raise KeyError(f"{self.kind} {name!r} is already registered")
            self._table[name] = target
            return target

        return _put if obj is None else _put(obj)

    def get(self, name: str) -> Callable[..., Any]:
        try:
            return self._table[name]
        except KeyError:
            known = ", ".join(sorted(self._table)) or "<none>"
            raise KeyError(f"unknown {self.kind} {name!r}; registered: {known}") from None

    def __contains__(self, name: str) -> bool:
        return name in self._table

    def __iter__(self) -> Iterator[str]:
        return iter(sorted(self._table))

    def __len__(self) -> int:
        return len(self._table)


NORM = Registry("norm")
MLP = Registry("mlp")
ATTENTION = Registry("attention")
POSENC = Registry("posenc")
ROUTER = Registry("router")
DATASET = Registry("dataset")
RENDERER = Registry("renderer")
OPTIMIZER = Registry("optimizer")
LOADER = Registry("loader")


def resolve(name: str, registry: Registry | None) -> Callable[..., Any]:
    """A registered name wins; anything containing a dot or colon is imported."""
    if registry is not None and name in registry:
        return registry.get(name)
    if "." in name or ":" in name:
        return import_class(name)
    if registry is None:
        raise KeyError(f"cannot resolve {name!r} without a registry")
    return registry.get(name)  # raises with the list of known names


def build(spec: Any, registry: Registry | None = None, **defaults: Any) -> Any:
    if spec is None:
        return None
    if isinstance(spec, str):
        return resolve(spec, registry)(**defaults)
    if isinstance(spec, dict):
        cfg = dict(spec)
        try:
            name = cfg.pop("name")
        except KeyError:
            raise KeyError(f"a dict spec needs a 'name' key, got {sorted(spec)}") from None
        target = resolve(name, registry) if isinstance(name, str) else name
        return target(**{**defaults, **cfg})
    if isinstance(spec, type) or (callable(spec) and not hasattr(spec, "forward")):
        if hasattr(spec, "build") and not isinstance(spec, type):
            return spec.build(**defaults)
        return spec(**defaults)
    if hasattr(spec, "build") and callable(spec.build) and not hasattr(spec, "forward"):
        return spec.build(**defaults)
    return spec
