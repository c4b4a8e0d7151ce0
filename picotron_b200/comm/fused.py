"""Switches the parallel modules from NCCL collectives to the peer-memory kernels of this package."""
from __future__ import annotations


def enable_fused_collectives(model) -> bool:
    """Attach symmetric-memory workspaces to the groups ``model`` communicates on. Returns True when active."""
    return False
