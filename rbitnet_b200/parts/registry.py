"""Registries of part kinds, one per role.  A new mixer, feed-forward, norm, position
encoding or block arrangement is one ``register_part`` call; specs name parts by kind."""
from __future__ import annotations

from typing import Callable, Dict

ROLES = ("mixer", "feed_forward", "norm", "position", "block")
_PARTS: Dict[str, Dict[str, Callable]] = {r: {} for r in ROLES}
_ALIASES = {"mixer_norm": "norm", "ffn_norm": "norm"}


def register_part(role: str, kind: str, factory: Callable, replace: bool = False) -> None:
    role = _ALIASES.get(role, role)
    if role not in _PARTS:
        raise ValueError(f"unknown part role {role!r}; roles: {', '.join(ROLES)}")
    if kind in _PARTS[role] and not replace:
        raise ValueError(f"{role} kind {kind!r} is already registered")
    _PARTS[role][kind] = factory


def unregister_part(role: str, kind: str) -> None:
    _PARTS[_ALIASES.get(role, role)].pop(kind, None)


def known_parts(role: str):
    return sorted(_PARTS[_ALIASES.get(role, role)])


def build_part(role: str, spec):
    role = _ALIASES.get(role, role)
    kinds = _PARTS[role]
    if spec.kind not in kinds:
        raise ValueError(f"unknown {role} kind {spec.kind!r}; known: {', '.join(sorted(kinds))}")
    return kinds[spec.kind](**spec.params)


def build_block(block_spec):
    kinds = _PARTS["block"]
    if block_spec.arrangement not in kinds:
        raise ValueError(f"unknown block arrangement {block_spec.arrangement!r}; "
                         f"known: {', '.join(sorted(kinds))}")
    return kinds[block_spec.arrangement](block_spec)
