"""Registry of per-group symmetric-memory workspaces (see :mod:`.workspace`)."""
from __future__ import annotations

from typing import Dict, Optional

_WORKSPACES: Dict[int, object] = {}


def register(group, workspace) -> None:
    _WORKSPACES[id(group)] = workspace


def workspace_for(group) -> Optional[object]:
    return _WORKSPACES.get(id(group))


def clear() -> None:
    _WORKSPACES.clear()
