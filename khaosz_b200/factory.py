"""Name -> class registries with decorator registration.

Capability parity with the reference's ``astrai/factory.py:10-223`` (``Registry`` and
``BaseFactory``): every ``BaseFactory`` subclass owns a private registry; ``create`` drops
keyword arguments the target constructor does not accept (unless it takes ``**kwargs``) so
one bag of options can be offered to interchangeable components.
"""

from __future__ import annotations

import inspect
from typing import Callable, Dict, Generic, List, Optional, Tuple, Type, TypeVar

T = TypeVar("T")


class Registry:
    """Ordered mapping ``name -> (class, category, priority)``."""

    def __init__(self) -> None:
        self._items: Dict[str, Tuple[type, Optional[str], int]] = {}

    def register(self, name: str, component_cls: type, category: Optional[str] = None, priority: int = 0) -> None:
        if name in self._items:
            raise ValueError(f"Component '{name}' is already registered")
        self._items[name] = (component_cls, category, priority)

    def get(self, name: str) -> type:
        return self.get_with_metadata(name)[0]

    def get_with_metadata(self, name: str) -> Tuple[type, Optional[str], int]:
        try:
            return self._items[name]
        except KeyError:
            raise KeyError(f"Component '{name}' not found in registry") from None

    def contains(self, name: str) -> bool:
        return name in self._items

    def list_names(self) -> List[str]:
        return sorted(self._items)

    def list_by_category(self, category: str) -> List[str]:
        return sorted(n for n, (_, c, _) in self._items.items() if c == category)

    def list_by_priority(self, reverse: bool = False) -> List[str]:
        return sorted(self._items, key=lambda n: self._items[n][2], reverse=reverse)

    def entries(self) -> Dict[str, Tuple[type, Optional[str], int]]:
        return dict(self._items)


class BaseFactory(Generic[T]):
    """Subclass to get an independent registry::

        class NormFactory(BaseFactory[nn.Module]): ...

        @NormFactory.register("rms")
        class RMSNorm(nn.Module): ...

        NormFactory.create("rms", dim=64, unrelated_option=1)   # unrelated_option is dropped
    """

    _registry: Registry

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        cls._registry = Registry()

    # -- registration ---------------------------------------------------------------
    @classmethod
    def register(cls, name: str, category: Optional[str] = None, priority: int = 0) -> Callable[[Type[T]], Type[T]]:
        def wrap(component_cls: Type[T]) -> Type[T]:
            cls._validate_component(component_cls)
            cls._registry.register(name, component_cls, category=category, priority=priority)
            return component_cls

        return wrap

    @classmethod
    def _validate_component(cls, component_cls: Type[T]) -> None:
        """Hook for subclasses; raise ``TypeError`` to refuse a class."""

    # -- lookup ---------------------------------------------------------------------
    @classmethod
    def _require(cls, name: str) -> type:
        if not cls._registry.contains(name):
            raise ValueError(f"Unknown component: '{name}'. Supported types: {cls._registry.list_names()}")
        return cls._registry.get(name)

    @classmethod
    def get_component_class(cls, name: str) -> Type[T]:
        return cls._require(name)

    @classmethod
    def create(cls, name: str, *args, **kwargs) -> T:
        target = cls._require(name)
        params = inspect.signature(target.__init__).parameters
        if not any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()):
            kwargs = {k: v for k, v in kwargs.items() if k in params and k != "self"}
        return target(*args, **kwargs)

    @classmethod
    def list_registered(cls) -> List[str]:
        return cls._registry.list_names()

    @classmethod
    def is_registered(cls, name: str) -> bool:
        return cls._registry.contains(name)

    @classmethod
    def list_by_category(cls, category: str) -> List[str]:
        return cls._registry.list_by_category(category)

    @classmethod
    def list_by_priority(cls, reverse: bool = False) -> List[str]:
        return cls._registry.list_by_priority(reverse)


__all__ = ["Registry", "BaseFactory"]
