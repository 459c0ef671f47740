"""Flat parameter layout for element-granular, evenly sharded ZeRO.

The reference lays all parameters out flat and gives every *whole* parameter to one owner rank
(model/ZeRO3.py:903-933), which (a) turns every gather into a broadcast from one rank and every
reduction into a reduce to one rank — one GPU's links carry the whole message — and (b) breaks
when a parameter is larger than a shard (a 32000x768 embedding on 8 ranks). Here parameters are
grouped into *units* (one transformer block, the embedding table, the final norm, ...). A unit's
parameters are packed back to back (each start aligned to ``ALIGN`` elements), the unit is padded
to a multiple of ``world * ALIGN`` and every rank owns the same 1/world slice of every unit:

    full unit buffer   : [ rank0 slice | rank1 slice | ... | rank(W-1) slice ]   (P_u elements)
    rank r's shard     : concat over units of its slice of each unit

so gathering a unit is one balanced all-gather of P_u/W elements per rank into the unit buffer, and
reducing its gradient is one balanced reduce-scatter — both map 1:1 onto NVSwitch-friendly
collectives and onto the fused peer-memory kernels.

Parameters may also be marked *replicated* (ZeRO-2.5): they are left out of the unit buffers and
packed into one separate flat replica buffer that every rank holds in full; only their gradients
and optimizer state are sharded.
"""
from __future__ import annotations

from dataclasses import dataclass, field

ALIGN = 128  # elements; 256 bytes in bf16, keeps every parameter start TMA-legal (16 B) and more


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class ParamSlot:
    index: int                 # position in model.params
    shape: tuple
    size: int
    unit: int                  # unit id, or -1 when replicated
    offset: int                # element offset inside the unit buffer (or inside the replica buffer)


@dataclass
class Unit:
    name: str
    param_indices: list
    padded: int = 0            # P_u, multiple of world * ALIGN
    shard_offset: int = 0      # offset of this unit's slice inside a rank's shard
    full_offset: int = 0       # offset of the unit inside the (virtual) concatenation of all units

    @property
    def empty(self) -> bool:
        return self.padded == 0


@dataclass
class FlatLayout:
    world_size: int
    slots: list = field(default_factory=list)
    units: list = field(default_factory=list)
    shard_size: int = 0            # elements of the sharded set per rank
    padded_total: int = 0          # shard_size * world_size
    replica_total: int = 0         # elements of the replicated set (unpadded end)
    replica_padded_total: int = 0  # multiple of world * ALIGN
    replicated_param_indices: list = field(default_factory=list)

    # ------------------------------------------------------------------ construction
    @classmethod
    def build(cls, param_shapes, unit_defs, world_size: int, replicated=()):
        """``param_shapes``: list of shapes in model.params order. ``unit_defs``: list of
        (name, [param indices]) covering every parameter exactly once."""
        rep = set(int(i) for i in replicated)
        lay = cls(world_size=world_size, replicated_param_indices=sorted(rep))
        sizes = []
        for shp in param_shapes:
            n = 1
            for d in shp:
                n *= int(d)
            sizes.append(n)
        lay.slots = [None] * len(param_shapes)
        seen = set()
        shard_off = 0
        full_off = 0
        for uid, (name, idxs) in enumerate(unit_defs):
            unit = Unit(name=name, param_indices=list(idxs))
            off = 0
            for i in idxs:
                if i in seen:
                    raise ValueError(f"parameter {i} is in two units")
                seen.add(i)
                if i in rep:
                    continue
                off = _round_up(off, ALIGN)
                lay.slots[i] = ParamSlot(i, tuple(param_shapes[i]), sizes[i], uid, off)
                off += sizes[i]
            unit.padded = _round_up(off, world_size * ALIGN) if off > 0 else 0
            unit.shard_offset = shard_off
            unit.full_offset = full_off
            shard_off += unit.padded // world_size
            full_off += unit.padded
            lay.units.append(unit)
        if len(seen) != len(param_shapes):
            missing = sorted(set(range(len(param_shapes))) - seen)
            raise ValueError(f"parameters {missing} belong to no unit")
        lay.shard_size = shard_off
        lay.padded_total = shard_off * world_size
        roff = 0
        for i in sorted(rep):
            roff = _round_up(roff, ALIGN)
            lay.slots[i] = ParamSlot(i, tuple(param_shapes[i]), sizes[i], -1, roff)
            roff += sizes[i]
        lay.replica_total = roff
        lay.replica_padded_total = _round_up(roff, world_size * ALIGN) if roff > 0 else 0
        return lay

    # ------------------------------------------------------------------ queries
    @property
    def replica_opt_shard_size(self) -> int:
        return self.replica_padded_total // self.world_size

    def unit_slice_len(self, uid: int) -> int:
        return self.units[uid].padded // self.world_size

    def unit_shard_range(self, uid: int) -> tuple:
        u = self.units[uid]
        return u.shard_offset, u.shard_offset + u.padded // self.world_size

    def param_full_offset(self, i: int) -> int:
        """Offset of parameter i in the concatenation of all full unit buffers."""
        s = self.slots[i]
        if s.unit < 0:
            raise ValueError("replicated parameter has no sharded offset")
        return self.units[s.unit].full_offset + s.offset

    def full_to_shard(self, full_pos: int) -> tuple:
        """(rank, position inside that rank's shard) of an element of the full concatenation."""
        for u in self.units:
            if u.full_offset <= full_pos < u.full_offset + u.padded:
                rel = full_pos - u.full_offset
                sl = u.padded // self.world_size
                return rel // sl, u.shard_offset + rel % sl
        raise IndexError(full_pos)

    def describe(self) -> dict:
        """Plain-python description stored in checkpoints (enough to re-shard offline)."""
        return {
            "layout": "unit_even",
            "align": ALIGN,
            "world_size": self.world_size,
            "shard_size": self.shard_size,
            "padded_total": self.padded_total,
            "units": [{"name": u.name, "param_indices": list(u.param_indices), "padded": u.padded,
                       "shard_offset": u.shard_offset, "full_offset": u.full_offset} for u in self.units],
            "param_offsets": [(-1 if s.unit < 0 else self.param_full_offset(s.index)) for s in self.slots],
            "param_unit": [s.unit for s in self.slots],
            "param_unit_offsets": [s.offset for s in self.slots],
            "param_shapes": [tuple(s.shape) for s in self.slots],
            "param_sizes": [s.size for s in self.slots],
            "replicated_param_indices": list(self.replicated_param_indices),
            "replica_offsets": [(s.offset if s.unit < 0 else -1) for s in self.slots],
            "replica_total": self.replica_total,
            "replica_padded_total": self.replica_padded_total,
            "replica_opt_shard_size": self.replica_opt_shard_size,
        }


def select_replicated_params(sizes, unit_of_embedding_params, ratio: float, policy: str = "largest_first"):
    """Choose parameters to replicate until ``ratio`` of all elements is covered.

    Policies and stopping rule as in the reference (model/ZeRO2_5.py:863-892): ``largest_first``
    (default), ``first``, ``last``, ``embedding_first``; parameters are taken in the policy's order
    until the running total has REACHED ``ratio * total``, so the last one taken may overshoot the
    target and any ``ratio`` > 0 replicates at least one parameter. ``ratio`` >= 1 replicates
    everything (ZeRO-2).
    """
    n = len(sizes)
    total = sum(sizes)
    if ratio <= 0 or total == 0:
        return []
    if ratio >= 1.0:
        return list(range(n))
    if policy == "largest_first":
        order = sorted(range(n), key=lambda i: (-sizes[i], i))
    elif policy == "first":
        order = list(range(n))
    elif policy == "last":
        order = list(range(n - 1, -1, -1))
    elif policy == "embedding_first":
        emb = [i for i in unit_of_embedding_params]
        rest = sorted((i for i in range(n) if i not in set(emb)), key=lambda i: (-sizes[i], i))
        order = emb + rest
    else:
        raise ValueError(f"unknown zero25_replica_policy {policy!r}")
    target = int(total * ratio)
    chosen, acc = [], 0
    for i in order:
        if acc >= target:
            break
        chosen.append(i)
        acc += sizes[i]
    return sorted(chosen)
