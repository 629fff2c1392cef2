"""Record the reference's instruction-row packing and barrier-formula arithmetic on seeded cases (run
once, with the reference's ``src`` on PYTHONPATH):
``python tests/golden/make_format_golden.py tests/golden/format_reference.json``."""

import json
import random
import sys

from machete.megakernel.scheduling import BarrierFormula, TileInstruction

rng = random.Random(7)
out = {"pack": [], "formula": []}
cases = [dict(op_idx=0, tiles=(0,)), dict(op_idx=0xFFFE, tiles=(0xFFFF, 0xFFFF, 0xFFFF, 0xFFFF)),
         dict(op_idx=3, tiles=(1, 2), range_axis=1, range_end_axis=1, range_end=9),
         dict(op_idx=40000, tiles=(40000, 3, 50000), range_axis=0, range_end_axis=14, range_end=0xFFFF),
         dict(op_idx=7, tiles=(5, 6, 7, 8), range_axis=3, range_end_axis=0, range_end=12),
         dict(op_idx=9, tiles=(1,), range_axis=0, range_end_axis=-1, range_end=5)]
for _ in range(40):
    n = rng.randint(1, 4)
    c = dict(op_idx=rng.randint(0, 0xFFFE), tiles=tuple(rng.randint(0, 0xFFFF) for _ in range(n)))
    if rng.random() < 0.5:
        c.update(range_axis=rng.randint(0, 3), range_end_axis=rng.randint(0, 14), range_end=rng.randint(0, 0xFFFF))
    cases.append(c)
for c in cases:
    meta = rng.randint(0, 0x7FFFFFFF)
    out["pack"].append({"args": {k: list(v) if isinstance(v, tuple) else v for k, v in c.items()}, "meta": meta,
                        "row": TileInstruction(**c).pack(meta)})
out["end"] = TileInstruction.end_instruction().pack()
for _ in range(40):
    f = dict(base=rng.randint(0, 5000), coeffs=tuple(rng.randint(0, 64) for _ in range(4)),
             divs=tuple(rng.randint(1, 8) for _ in range(4)), offset=rng.randint(0, 100), expected=rng.randint(1, 64))
    if rng.random() < 0.5:
        f.update(guard_min=rng.randint(0, 50), guard_max=rng.randint(51, 4000))
    if rng.random() < 0.3:
        f.update(guard_coeffs=tuple(rng.randint(0, 16) for _ in range(4)))
    bf = BarrierFormula(**f)
    tiles = [tuple(rng.randint(0, 200) for _ in range(rng.randint(1, 4))) for _ in range(6)]
    out["formula"].append({"args": {k: list(v) if isinstance(v, tuple) else v for k, v in f.items()},
                           "tiles": [list(t) for t in tiles], "index": [bf.compute_index(t) for t in tiles],
                           "guard": [bf.is_guarded(t) for t in tiles], "has_guard": bf.has_guard})
json.dump(out, open(sys.argv[1], "w"))
