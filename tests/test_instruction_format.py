"""The reference interpreter's instruction rows and barrier formulas, bit-exact against numbers
recorded from the reference's own classes (tests/golden/make_format_golden.py), plus the inverse."""

import json
import os

import pytest

from machete_b200.megakernel.instruction_format import END_OF_STREAM, INSTRUCTION_WORDS, BarrierFormula, TileInstruction

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "format_reference.json")))


def _tuples(args):
    return {k: tuple(v) if isinstance(v, list) else v for k, v in args.items()}


def test_instruction_rows_match_the_reference_bit_for_bit():
    assert TileInstruction.end_instruction().pack() == GOLD["end"] == [END_OF_STREAM, 0, 0, 0, 0]
    for case in GOLD["pack"]:
        ins = TileInstruction(**_tuples(case["args"]))
        row = ins.pack(case["meta"])
        assert row == case["row"] and len(row) == INSTRUCTION_WORDS, case["args"]
        assert all(-(1 << 31) <= w < (1 << 31) for w in row)
        back, meta = TileInstruction.unpack(row)
        assert meta == case["meta"] and back.op_idx == ins.op_idx
        assert back.tiles[:len(ins.tiles)] == tuple(ins.tiles) and not any(back.tiles[len(ins.tiles):])
        if ins.is_range:
            assert (back.range_axis, back.range_end_axis, back.range_end) == (ins.range_axis, ins.range_end_axis, ins.range_end)
        else:
            assert not back.is_range
    end, _ = TileInstruction.unpack(GOLD["end"])
    assert end.op_idx == TileInstruction.END_MARKER and end.logical_tiles() == []


def test_instruction_field_limits_are_the_reference_errors():
    for bad in (dict(op_idx=0xFFFF, tiles=(0,)), dict(op_idx=-2, tiles=(0,)), dict(op_idx=1, tiles=(0x10000,)),
                dict(op_idx=1, tiles=(0, 0, 0, 0, 0)), dict(op_idx=1, tiles=(0,), range_axis=4, range_end_axis=0),
                dict(op_idx=1, tiles=(0,), range_axis=0, range_end_axis=15),
                dict(op_idx=1, tiles=(0,), range_axis=0, range_end_axis=0, range_end=0x10000)):
        with pytest.raises(ValueError):
            TileInstruction(**bad).pack()
    with pytest.raises(ValueError):
        TileInstruction(1, (0,)).pack(barrier_meta_idx=1 << 31)


def test_range_instruction_covers_its_tiles_in_order():
    ins = TileInstruction(4, (2, 5), range_axis=1, range_end_axis=1, range_end=8)
    assert ins.logical_tiles() == [(2, 5, 0, 0), (2, 6, 0, 0), (2, 7, 0, 0)]
    assert TileInstruction(4, (2, 5)).logical_tiles() == [(2, 5)]
    assert TileInstruction(4, (2, 9), range_axis=1, range_end_axis=1, range_end=8).logical_tiles() == [(2, 9)]


def test_barrier_formulas_match_the_reference():
    for case in GOLD["formula"]:
        f = BarrierFormula(**_tuples(case["args"]))
        assert [f.compute_index(tuple(t)) for t in case["tiles"]] == case["index"], case["args"]
        assert [f.is_guarded(tuple(t)) for t in case["tiles"]] == case["guard"], case["args"]
        assert f.has_guard == case["has_guard"]
    plain = BarrierFormula(base=10, coeffs=(4, 1, 0, 0), divs=(1, 2, 1, 1))
    assert plain.compute_index((3, 5)) == 10 + 12 + 2 and not plain.has_guard and plain.is_guarded((100, 100))
