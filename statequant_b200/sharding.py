"""Slot sharding across GPUs: every (slot, layer) is independent, so N GPUs are N independent shards.

Rank r of N owns the slots ``{s : s mod N == r}``; inside the shard slot ``s`` has the local number ``s // N``
shifted by one so that local slot 0 stays the padding slot.  A step's slot table is split per rank with padding
preserved: rows of other ranks become padding rows (local index 0), whose output the kernels zero, so a gather of
the per-rank outputs is a plain sum or a row select.  There is no data-path collective and no peer access.
"""
from __future__ import annotations

import torch


def owner(slot, world):
    """Rank that owns a (positive) global slot number."""
    return (slot - 1) % world


def to_local(idx, rank, world):
    """Global slot table int32 [rows] -> this rank's table: local slot numbers for the rows it owns, 0 elsewhere
    (padding; non-positive entries stay padding)."""
    idx = idx.to(torch.int32)
    mine = (idx > 0) & (((idx - 1) % world) == rank)
    return torch.where(mine, (idx - 1) // world + 1, torch.zeros_like(idx))


def local_slots(num_slots, rank, world):
    """Number of slots (padding slot included) a rank needs for a global table of ``num_slots`` slots (slot 0 =
    padding)."""
    n = num_slots - 1
    return (n - rank + world - 1) // world + 1 if n > rank else 1


def rows_of(idx, rank, world):
    """Row indices of a global slot table that rank ``rank`` serves."""
    idx = idx.to(torch.int64)
    return torch.nonzero((idx > 0) & (((idx - 1) % world) == rank)).flatten()
