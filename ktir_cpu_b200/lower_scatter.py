"""Lowering of indirect (gather / scatter) statements."""
from __future__ import annotations

from .trace import Unsupported


def lower_indirect_store(dev, store, arena, stmt_id):
    raise Unsupported("indirect ktdp.store")
