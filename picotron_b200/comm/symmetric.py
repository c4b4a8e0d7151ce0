"""Registry of symmetric-memory workspaces (see :mod:`.workspace`), keyed by process group."""
from __future__ import annotations

from typing import Dict, Optional

_WORKSPACES: Dict[object, object] = {}


def _key(group):
    return group if isinstance(group, tuple) else id(group)


def register(group, workspace) -> None:
    _WORKSPACES[_key(group)] = workspace


def workspace_for(group) -> Optional[object]:
    return _WORKSPACES.get(_key(group))


def clear() -> None:
    _WORKSPACES.clear()
