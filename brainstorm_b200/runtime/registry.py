"""String-keyed class registries behind ``make_router`` / ``make_protocol`` / ``make_fabric``.

Same class methods as the reference's ``Registry`` (python/brt/runtime/registry.py:12-89):
sub-classes are registered per base class under a type name, and plain classes can be
collected under a tag.
"""
from typing import Callable, Dict, List, Optional, Type

from . import log

logger = log.get_logger(__file__)


class Registry:
    sub_cls_registries: Dict[type, Dict[str, type]] = {}
    func_registries: Dict[str, Callable] = {}
    cls_registries: Dict[str, List[type]] = {}

    @classmethod
    def register_sub_cls(cls, sub_cls_type: str, base_cls: type) -> Callable[[type], type]:
        table = cls.sub_cls_registries.setdefault(base_cls, {})

        def decorator(sub_cls: type) -> type:
            if not issubclass(sub_cls, base_cls):
                raise ValueError(f"{sub_cls} is not a subclass of {base_cls}.")
            if sub_cls_type in table:
                logger.warning("%s is already registered, overwrite it.", sub_cls_type)
            sub_cls.brt_abs_type = sub_cls_type
            table[sub_cls_type] = sub_cls
            return sub_cls

        return decorator

    @classmethod
    def get_sub_cls(cls, sub_cls_type: str, base_cls: type) -> Optional[Type]:
        try:
            table = cls.sub_cls_registries[base_cls]
        except KeyError:
            raise ValueError(f"{base_cls} is not registered.") from None
        return table.get(sub_cls_type)

    @classmethod
    def sub_cls_exists_and_registered(cls, sub_cls: type, base_cls: type) -> bool:
        if base_cls not in cls.sub_cls_registries:
            raise ValueError(
                f"No base class of {base_cls} exists in the registry, register the base class "
                "first.")
        return issubclass(sub_cls, base_cls) and any(
            sub_cls is c for c in cls.sub_cls_registries[base_cls].values())

    @classmethod
    def register_cls(cls, cls_type: str) -> Callable[[type], type]:
        def decorator(registered_cls: type) -> type:
            bucket = cls.cls_registries.setdefault(cls_type, [])
            if registered_cls in bucket:
                logger.warning("%s is already registered, overwrite it.", cls_type)
            bucket.append(registered_cls)
            return registered_cls

        return decorator

    @classmethod
    def register_cls_type(cls, cls_type: str) -> None:
        cls.cls_registries.setdefault(cls_type, [])

    @classmethod
    def cls_exists_and_registered(cls, registered_cls: type, cls_type: str) -> bool:
        return registered_cls in cls.cls_registries.setdefault(cls_type, [])
