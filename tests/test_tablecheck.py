"""Host-side bounds checks of the optimizers' device tables: good tables pass, every kind of bad entry is named."""

import struct

import pytest
import torch

from himuon_b200.optimizers import _tablecheck as tc

TH = TW = 64
UNITS = lambda R, C: R * C * 2                       # noqa: E731  (two row blocks per tile in this toy numbering)


def _mom_entry(grads, mom, tile_base, h, w, unit_begin, ld, R=None, C=None):
    R = -(-h // TH) if R is None else R
    C = -(-w // TW) if C is None else C
    ptrs = list(grads) + [0] * (8 - len(grads))
    return struct.pack(tc.MOM_FMT, *ptrs, mom, tile_base, h, w, R, C, unit_begin, ld)


def _setup():
    g0, g1 = torch.zeros(2, 100, 130, dtype=torch.bfloat16), torch.zeros(2, 100, 130, dtype=torch.bfloat16)
    mom = torch.zeros(2, 100, 130, dtype=torch.bfloat16)
    return g0, g1, mom, tc.Extents([g0, g1, mom])


def test_good_momentum_and_apply_tables_pass():
    g0, g1, mom, ext = _setup()
    per = 2 * 3                                       # 100x130 in 64x64 tiles
    raw = b"".join(_mom_entry([g0[i].data_ptr(), g1[i].data_ptr()], mom[i].data_ptr(), i * per, 100, 130, i * UNITS(2, 3), 130)
                   for i in range(2))
    tc.check_momentum_table(raw, 2, TH, TW, 2 * per, UNITS, 2 * UNITS(2, 3), 2, 2, ext)
    par = torch.zeros(2, 100, 130, dtype=torch.float32)
    raw = b"".join(struct.pack(tc.APPLY_FMT, par[i].data_ptr(), i * per, 100, 130, 2, 3, i * UNITS(2, 3), 0, 0.5, 130)
                   for i in range(2))
    tc.check_apply_table(raw, 2, TH, TW, 2 * per, UNITS, 2 * UNITS(2, 3), 1, 4, tc.Extents([par]))


@pytest.mark.parametrize("what,kwargs,match", [
    ("past the end of the gradient", dict(h=101), "leaves every known allocation"),
    ("row stride shorter than a row", dict(ld=128), "row stride"),
    ("wrong tile grid", dict(R=1), "tile grid"),
    ("tiles past the tile buffer", dict(tile_base=8), "leave the tile buffer"),
    ("gap in the work units", dict(unit_begin=3), "work units start"),
])
def test_bad_momentum_entries_are_named(what, kwargs, match):
    g0, g1, mom, ext = _setup()
    args = dict(tile_base=0, h=100, w=130, unit_begin=0, ld=130)
    args.update(kwargs)
    # the last matrix of each allocation: one row too many runs past the end of the storage
    raw = _mom_entry([g0[1].data_ptr(), g1[1].data_ptr()], mom[1].data_ptr(), **args)
    with pytest.raises(tc.TableError, match=match):
        tc.check_momentum_table(raw, 1, TH, TW, 12, UNITS, UNITS(2, 3), 2, 2, ext)


def test_more_bad_tables():
    g0, g1, mom, ext = _setup()
    ok = _mom_entry([g0[0].data_ptr(), g1[0].data_ptr()], mom[0].data_ptr(), 0, 100, 130, 0, 130)
    with pytest.raises(tc.TableError, match="null"):                       # second replica missing
        tc.check_momentum_table(_mom_entry([g0[0].data_ptr()], mom[0].data_ptr(), 0, 100, 130, 0, 130), 1, TH, TW, 12, UNITS,
                                UNITS(2, 3), 2, 2, ext)
    with pytest.raises(tc.TableError, match="overlap"):                    # two matrices on the same tiles
        tc.check_momentum_table(ok + _mom_entry([g0[1].data_ptr(), g1[1].data_ptr()], mom[1].data_ptr(), 3, 100, 130,
                                                UNITS(2, 3), 130), 2, TH, TW, 12, UNITS, 2 * UNITS(2, 3), 2, 2, ext)
    with pytest.raises(tc.TableError, match="add up"):                     # launch covers fewer units than the table
        tc.check_momentum_table(ok, 1, TH, TW, 12, UNITS, UNITS(2, 3) - 1, 2, 2, ext)
    with pytest.raises(tc.TableError, match="bytes for"):                  # truncated table
        tc.check_momentum_table(ok[:-4], 1, TH, TW, 12, UNITS, UNITS(2, 3), 2, 2, ext)
    with pytest.raises(tc.TableError, match="not aligned"):
        tc.check_momentum_table(_mom_entry([g0[0].data_ptr() + 1, g1[0].data_ptr()], mom[0].data_ptr(), 0, 100, 130, 0, 130),
                                1, TH, TW, 12, UNITS, UNITS(2, 3), 2, 2, ext)
    par = torch.zeros(100, 130)
    bad_group = struct.pack(tc.APPLY_FMT, par.data_ptr(), 0, 100, 130, 2, 3, 0, 2, 0.5, 130)
    with pytest.raises(tc.TableError, match="hyper-parameter row"):
        tc.check_apply_table(bad_group, 1, TH, TW, 6, UNITS, UNITS(2, 3), 2, 4, tc.Extents([par]))
    nan_scale = struct.pack(tc.APPLY_FMT, par.data_ptr(), 0, 100, 130, 2, 3, 0, 0, float("nan"), 130)
    with pytest.raises(tc.TableError, match="multiplier"):
        tc.check_apply_table(nan_scale, 1, TH, TW, 6, UNITS, UNITS(2, 3), 1, 4, tc.Extents([par]))


def test_adam_table():
    p, g, m, v = (torch.zeros(5000, dtype=torch.bfloat16) for _ in range(4))
    p2, g2, m2, v2 = (torch.zeros(17, dtype=torch.bfloat16) for _ in range(4))
    ext = tc.Extents([p, g, m, v, p2, g2, m2, v2])
    raw = struct.pack(tc.ADAM_FMT, p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), 5000, 0, 0, 0) + \
        struct.pack(tc.ADAM_FMT, p2.data_ptr(), g2.data_ptr(), m2.data_ptr(), v2.data_ptr(), 17, 2, 1, 0)
    tc.check_adam_table(raw, 2, 3, 2, 2, 2, ext)
    with pytest.raises(tc.TableError, match="second moment range"):     # the second moment is shorter than the parameter
        short = torch.zeros(16, dtype=torch.bfloat16)
        tc.check_adam_table(struct.pack(tc.ADAM_FMT, p2.data_ptr(), g2.data_ptr(), m2.data_ptr(), short.data_ptr(), 17, 0, 0, 0),
                            1, 1, 1, 2, 2, tc.Extents([p2, g2, m2, short]))
    with pytest.raises(tc.TableError, match="work units start"):
        tc.check_adam_table(raw[:struct.calcsize(tc.ADAM_FMT)] +
                            struct.pack(tc.ADAM_FMT, p2.data_ptr(), g2.data_ptr(), m2.data_ptr(), v2.data_ptr(), 17, 1, 1, 0),
                            2, 3, 2, 2, 2, ext)


def test_adamw_builds_checked_tables_on_cpu_items():
    """AdamTable.build runs the check when it is switched on (host code: no device needed for the validation itself)."""
    from himuon_b200.optimizers._multi import AdamTable

    tc.enable(True)
    try:
        par, g, m, v = (torch.zeros(300) for _ in range(4))
        t = AdamTable()
        t.build([(par, g, m, v, 0)], 1, "cpu")
        assert t.recs[0]["n"] == 1 and t.recs[0]["units"] == 1
        with pytest.raises(tc.TableError):
            t.build([(par, g, m, v, 3)], 1, "cpu")         # group row that does not exist
    finally:
        tc.enable(False)
