"""Patch registry: which HF attribute each kernel-backed replacement stands in for.

Same surface and observable behaviour as the reference registry
(src/bastile/registry.py:18-142): ``PatchInfo`` records, a process-global
``PatchRegistry`` that remembers registration order and the applied set, and
the module-level ``register_patch`` / ``list_patches`` / ``get_registry``.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any

log = logging.getLogger(__name__)


@dataclass
class PatchInfo:
    """One replacement: ``target_module.target_attr`` -> ``replacement``."""

    name: str
    description: str
    target_module: str
    target_attr: str
    replacement: Any
    has_backward: bool
    original: Any = None
    is_applied: bool = False
    priority: int = 0
    models: list[str] = field(default_factory=list)


class PatchRegistry:
    def __init__(self) -> None:
        self._patches: dict[str, PatchInfo] = {}
        self._applied: list[str] = []

    def register(self, name: str, description: str, target_module: str, target_attr: str, replacement: Any,
                 has_backward: bool = True, priority: int = 0, models: list[str] | None = None) -> None:
        if name in self._patches:
            log.warning("Patch '%s' already registered, overwriting", name)
        self._patches[name] = PatchInfo(name, description, target_module, target_attr, replacement, has_backward,
                                        priority=priority, models=list(models) if models else [])

    def get(self, name: str) -> PatchInfo | None:
        return self._patches.get(name)

    def list_all(self) -> list[str]:
        return list(self._patches)

    def list_with_backward(self) -> list[str]:
        return [n for n, p in self._patches.items() if p.has_backward]

    def get_for_model(self, model_type: str) -> list[PatchInfo]:
        hits = [p for p in self._patches.values() if not p.models or model_type in p.models]
        hits.sort(key=lambda p: -p.priority)  # stable: registration order within one priority
        return hits

    def mark_applied(self, name: str, original: Any) -> None:
        p = self._patches.get(name)
        if p is None:
            return
        p.original, p.is_applied = original, True
        if name not in self._applied:
            self._applied.append(name)

    def mark_reset(self, name: str) -> None:
        p = self._patches.get(name)
        if p is None:
            return
        p.is_applied = False
        if name in self._applied:
            self._applied.remove(name)

    def get_applied(self) -> list[str]:
        return list(self._applied)


_registry = PatchRegistry()


def register_patch(name: str, description: str, target_module: str, target_attr: str, replacement: Any,
                   has_backward: bool = True, priority: int = 0, models: list[str] | None = None) -> None:
    _registry.register(name, description, target_module, target_attr, replacement, has_backward, priority, models)


def list_patches() -> list[str]:
    return _registry.list_all()


def get_registry() -> PatchRegistry:
    return _registry
