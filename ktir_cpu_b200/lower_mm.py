"""Lowering of matmul loops and attention loops (tensor-core statements)."""
from __future__ import annotations


def try_lower_matmul(dev, store, arena, stmt_id):
    return None
