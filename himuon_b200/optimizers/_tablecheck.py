"""Host-side bounds checking of the device entry tables (debug aid).

The multi-tensor optimizer kernels (``momentum_tile``, ``untile_apply``, ``adamw_multi``) receive raw pointers, shapes,
strides and work-unit offsets in packed tables; nothing on the device knows where an allocation ends, so a wrong table
is an out-of-bounds access that no kernel-side check could attribute.  This module validates a table on the host,
where the extents are known, right after it is built: every pointer range an entry makes the kernel touch must lie
inside one of the tensors the table was built from, tile ranges must stay inside the tile buffer and must not overlap,
tile grids must match the shapes, work units must be numbered without gaps, hyper-parameter rows must exist.

It is off by default (tables are built once per plan, but a check walks every entry): set ``HIMUON_CHECK_TABLES=1`` or
call ``enable(True)``.  ``ShardedEngine(debug=True)`` switches it on together with its other race / overrun checks.
A failed check raises ``TableError`` naming the entry and the field.  Pure host code: the tests build good and bad
tables by hand and need no GPU.
"""

from __future__ import annotations

import math
import os
import struct

import torch

MOM_FMT = "<8QQq6i"        # MomTileEntry: grad[8], mom, tile_base, h, w, R, C, unit_begin, ld
APPLY_FMT = "<Qq6ifi"      # ApplyEntry:   param, tile_base, h, w, R, C, unit_begin, group, scale, ld
ADAM_FMT = "<4Qqq2i"       # AdamEntry:    param, grad, m, v, numel, unit_begin, group, pad
ADAM_UNIT = 4096

_enabled = os.environ.get("HIMUON_CHECK_TABLES") == "1"


class TableError(ValueError):
    pass


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


class Extents:
    """Address ranges of live allocations: ``covers(ptr, nbytes)`` is true when ``[ptr, ptr + nbytes)`` lies inside one."""

    def __init__(self, tensors=()):
        self.ranges: list[tuple[int, int]] = []
        for t in tensors:
            self.add(t)

    def add(self, t) -> None:
        if isinstance(t, torch.Tensor):
            st = t.untyped_storage()
            self.ranges.append((st.data_ptr(), st.data_ptr() + st.nbytes()))
        else:                                       # an explicit (pointer, nbytes) pair
            self.ranges.append((int(t[0]), int(t[0]) + int(t[1])))

    def covers(self, ptr: int, nbytes: int) -> bool:
        return any(lo <= ptr and ptr + nbytes <= hi for lo, hi in self.ranges)


def _fail(kind: str, i: int, what: str):
    raise TableError(f"{kind} table, entry {i}: {what}")


def _check_matrix(kind, i, name, ptr, h, w, ld, esize, extents):
    if ptr == 0:
        _fail(kind, i, f"{name} pointer is null")
    if ptr % esize:
        _fail(kind, i, f"{name} pointer {ptr:#x} is not aligned to its {esize}-byte elements")
    if ld < w:
        _fail(kind, i, f"row stride {ld} is smaller than the row length {w}")
    span = ((h - 1) * ld + w) * esize
    if not extents.covers(ptr, span):
        _fail(kind, i, f"{name} range [{ptr:#x}, +{span}) ({h}x{w}, stride {ld}) leaves every known allocation")


def _check_tiling(kind, i, h, w, R, C, th, tw, tile_base, n_tiles_total, taken):
    if h <= 0 or w <= 0:
        _fail(kind, i, f"empty matrix {h}x{w}")
    if R != math.ceil(h / th) or C != math.ceil(w / tw):
        _fail(kind, i, f"tile grid {R}x{C} does not match {h}x{w} in tiles of {th}x{tw}")
    if tile_base < 0 or tile_base + R * C > n_tiles_total:
        _fail(kind, i, f"tiles [{tile_base}, {tile_base + R * C}) leave the tile buffer of {n_tiles_total} tiles")
    for lo, hi, j in taken:
        if tile_base < hi and lo < tile_base + R * C:
            _fail(kind, i, f"tiles [{tile_base}, {tile_base + R * C}) overlap those of entry {j}")
    taken.append((tile_base, tile_base + R * C, i))


def check_momentum_table(raw, n: int, th: int, tw: int, n_tiles_total: int, units_of, total_units: int, n_src: int,
                         grad_esize: int, extents: Extents) -> None:
    """``raw``: the packed ``MomTileEntry`` array; ``units_of(R, C)``: work units of one entry; ``extents``: the
    gradient replicas and momentum buffers the table points into."""
    size = struct.calcsize(MOM_FMT)
    if len(raw) < n * size:
        raise TableError(f"momentum table: {len(raw)} bytes for {n} entries of {size}")
    if not 1 <= n_src <= 8:
        raise TableError(f"momentum table: {n_src} gradient replicas (1..8 supported)")
    unit, taken = 0, []
    for i in range(n):
        *grads, mom, tile_base, h, w, R, C, unit_begin, ld = struct.unpack_from(MOM_FMT, raw, i * size)
        _check_tiling("momentum", i, h, w, R, C, th, tw, tile_base, n_tiles_total, taken)
        for s in range(n_src):
            _check_matrix("momentum", i, f"gradient replica {s}", grads[s], h, w, ld, grad_esize, extents)
        _check_matrix("momentum", i, "momentum buffer", mom, h, w, ld, grad_esize, extents)
        if unit_begin != unit:
            _fail("momentum", i, f"work units start at {unit_begin}, expected {unit}")
        unit += units_of(R, C)
    if unit != total_units:
        raise TableError(f"momentum table: {total_units} work units launched, the entries add up to {unit}")


def check_apply_table(raw, n: int, th: int, tw: int, n_tiles_total: int, units_of, total_units: int, n_groups: int,
                      param_esize: int, extents: Extents) -> None:
    size = struct.calcsize(APPLY_FMT)
    if len(raw) < n * size:
        raise TableError(f"apply table: {len(raw)} bytes for {n} entries of {size}")
    unit, taken = 0, []
    for i in range(n):
        param, tile_base, h, w, R, C, unit_begin, group, scale, ld = struct.unpack_from(APPLY_FMT, raw, i * size)
        _check_tiling("apply", i, h, w, R, C, th, tw, tile_base, n_tiles_total, taken)
        _check_matrix("apply", i, "parameter", param, h, w, ld, param_esize, extents)
        if not 0 <= group < n_groups:
            _fail("apply", i, f"hyper-parameter row {group} of {n_groups}")
        if not math.isfinite(scale):
            _fail("apply", i, f"learning-rate multiplier {scale}")
        if unit_begin != unit:
            _fail("apply", i, f"work units start at {unit_begin}, expected {unit}")
        unit += units_of(R, C)
    if unit != total_units:
        raise TableError(f"apply table: {total_units} work units launched, the entries add up to {unit}")


def check_adam_table(raw, n: int, total_units: int, n_groups: int, param_esize: int, state_esize: int,
                     extents: Extents) -> None:
    size = struct.calcsize(ADAM_FMT)
    if len(raw) < n * size:
        raise TableError(f"adam table: {len(raw)} bytes for {n} entries of {size}")
    unit = 0
    for i in range(n):
        param, grad, m, v, numel, unit_begin, group, _ = struct.unpack_from(ADAM_FMT, raw, i * size)
        if numel <= 0:
            _fail("adam", i, f"{numel} elements")
        for name, ptr, es in (("parameter", param, param_esize), ("gradient", grad, state_esize),
                              ("first moment", m, state_esize), ("second moment", v, state_esize)):
            _check_matrix("adam", i, name, ptr, 1, numel, numel, es, extents)
        if not 0 <= group < n_groups:
            _fail("adam", i, f"hyper-parameter row {group} of {n_groups}")
        if unit_begin != unit:
            _fail("adam", i, f"work units start at {unit_begin}, expected {unit}")
        unit += (numel + ADAM_UNIT - 1) // ADAM_UNIT
    if unit != total_units:
        raise TableError(f"adam table: {total_units} work units launched, the entries add up to {unit}")
