"""The dependency edges this build infers equal the reference builder's on the same op lists.

Three views of one fact, all host-only:

* live differential: ``tests/dep_edges_driver.py`` runs in a subprocess against the reference
  package (found through ``MACHETE_REFERENCE_SRC`` or the usual checkout location; skipped when
  absent) and in-process against this package; the (producer, consumer) sets must be identical;
* the same comparison against ``tests/golden/dep_edges_reference.json``, the driver's output for the
  reference recorded once (regenerate: ``PYTHONPATH=<reference>/src python tests/dep_edges_driver.py
  reference tests/golden/dep_edges_reference.json``), so the check also runs where no checkout is;
* the lowered program: ``infer_dependencies`` (which reduces every kind of edge and splits them into
  op-entry waits, per-unit waits and loader waits) imposes exactly the reference's ordering: equal
  transitive closures on the unfused layer.
"""

import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import dep_edges_driver as driver  # noqa: E402

from machete_b200.megakernel import Megakernel, MegakernelConfig  # noqa: E402
from machete_b200.megakernel.scheduling import closure_of, infer_dependencies, resolve_dep_pairs  # noqa: E402

GOLDEN = os.path.join(HERE, "golden", "dep_edges_reference.json")
REFERENCE_SRC = os.environ.get("MACHETE_REFERENCE_SRC", os.path.join(os.sep, "root", "reference", "src"))


def _ours(tmp_path):
    out = tmp_path / "ours.json"
    driver.main("ours", str(out))
    return json.loads(out.read_text())


def _assert_same(ours, ref):
    assert set(ours) == set(ref)
    for case in ref:
        assert "error" not in ref[case] and "error" not in ours[case], (case, ref[case], ours[case])
        assert ours[case]["ops"] == ref[case]["ops"], case
        assert ours[case]["pairs"] == ref[case]["pairs"], case


def test_edges_equal_the_recorded_reference_edges(tmp_path):
    _assert_same(_ours(tmp_path), json.load(open(GOLDEN)))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_SRC, "machete")), reason="no reference checkout")
def test_edges_equal_the_reference_builder_live(tmp_path):
    out = tmp_path / "ref.json"
    env = dict(os.environ, PYTHONPATH=REFERENCE_SRC, CUDA_VISIBLE_DEVICES="")
    run = subprocess.run([sys.executable, os.path.join(HERE, "dep_edges_driver.py"), "reference", str(out)],
                         env=env, cwd=str(tmp_path), capture_output=True, text=True, timeout=900)
    if run.returncode != 0 and "ModuleNotFoundError" in run.stderr:
        pytest.skip("the reference package does not import here: " + run.stderr.strip().splitlines()[-1])
    assert run.returncode == 0, run.stderr[-2000:]
    ref = json.loads(out.read_text())
    _assert_same(_ours(tmp_path), ref)
    assert ref == json.load(open(GOLDEN)), "the recorded fixture is stale"


@pytest.mark.parametrize("cache_pos,splits", [(1008, 4), (2047, 8)])
def test_lowered_program_imposes_the_same_ordering(cache_pos, splits):
    ops, keep = driver._layer_ops("machete_b200", 1, cache_pos, splits)
    pairs = {(p, c) for p, c, _, _ in resolve_dep_pairs(ops)}
    mk = Megakernel(ops, config=MegakernelConfig(fuse=False))
    assert len(mk.native_ops) == len(ops)            # unfused: one native op per scheduled op
    deps, closure = infer_dependencies(mk.native_ops)
    assert closure == closure_of(pairs, len(ops))
    # every edge the lowered program keeps is a reference edge (it keeps fewer: read-after-write
    # pairs implied by another path are reduced away as well)
    kept = {(i, j) for j, d in enumerate(deps) for i in list(d.coarse) + list(d.fine)}
    assert kept <= pairs and kept
    own_closure = closure_of(kept, len(ops))
    assert [c | 0 for c in own_closure] == [c for c in closure_of(pairs, len(ops))]
