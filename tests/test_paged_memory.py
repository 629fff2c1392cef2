"""Shared-memory layout arithmetic: the reference ring's offsets (bit-exact against numbers recorded
from the reference's own classes, tests/golden/make_layout_golden.py) and this build's plan."""

import json
import os

import pytest

from machete_b200.megakernel import Megakernel
from machete_b200.megakernel.megakernel import CTRL_BYTES
from machete_b200.megakernel.paged_memory import (B200_SMEM_OPTIN, NativeSmemPlan, NPageLayout, PipelinePageLayout)

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "layout_reference.json")))


def test_npage_layout_offsets_match_the_reference():
    for g in GOLD["npage"]:
        pages, size, slots = g["args"]
        l = NPageLayout(num_pages=pages, page_size=size, num_slots=slots)
        got = {"flags": l.flags_offset, "iq": l.iq_offset, "mbar": l.mbarrier_offset, "scratch": l.scratch_size,
               "aligned": l.aligned_page_size, "start": l.pages_start, "total": l.total_size, "slots": l.num_slots,
               "wn": l.work_notify_mbar_offset(l.num_slots - 1), "cd": l.compute_done_mbar_offset(l.num_slots - 1)}
        assert got == {k: g[k] for k in got}, g["args"]
        assert l.pages_start % 128 == 0 and l.mbarrier_offset % 8 == 0
        assert l.page_offset(pages - 1) + l.aligned_page_size == l.total_size
    for bad in ({"num_pages": 0}, {"num_pages": 17}, {"num_pages": 2, "num_slots": 0}, {"num_pages": 2, "num_slots": 17}):
        with pytest.raises(ValueError):
            NPageLayout(**bad)


def test_for_device_picks_the_reference_page_counts():
    for g in GOLD["for_device"]:
        size, smem = g["args"]
        l = NPageLayout.for_device(page_size=size, max_smem=smem)
        assert (l.num_pages, l.total_size) == (g["pages"], g["total"]), g["args"]
    # B200: 227 KB opt-in gives four 48 KB pages or seven 32 KB pages
    assert NPageLayout.for_device(page_size=49152, max_smem=B200_SMEM_OPTIN).num_pages == 4
    assert NPageLayout.for_device(page_size=32768, max_smem=B200_SMEM_OPTIN).num_pages == 7
    with pytest.raises(ValueError):
        NPageLayout.for_device(page_size=200 * 1024, max_smem=B200_SMEM_OPTIN)


def test_pipeline_page_layout_matches_the_reference_and_checks_bounds():
    for g in GOLD["pipeline"]:
        pc, pb, sc, sb = g["args"]
        l = PipelinePageLayout(page_count=pc, page_bytes=pb, semaphore_count=sc, scratch_bytes=sb)
        got = {"sem": l.semaphores_offset, "scratch": l.scratch_offset, "total": l.total_size,
               "last_page": l.page_offset(pc - 1), "out1of2": l.output_scratch_offset(output_stage=1, output_stages=2)}
        assert got == {k: g[k] for k in got}, g["args"]
    l = PipelinePageLayout(page_count=3, page_bytes=1024, semaphore_count=5, scratch_bytes=96)
    # semaphore numbering: 1 activations, then input stages (arrived, finished), then output stages
    assert (l.activations_arrived_sem(), l.weights_arrived_sem(2), l.weights_finished_sem(3, 2)) == (0, 3, 6)
    assert (l.outputs_arrived_sem(3, 1), l.outputs_finished_sem(3, 3, 2)) == (8, 12)
    assert l.weight_page_offset(input_stage=0, page_in_stage=1, input_stages=1, stage_pages=2) == 2 * 1024
    assert l.semaphore_offset(4) == l.semaphores_offset + 32 and l.scratch_offset % 16 == 0 and l.total_size % 128 == 0
    for call in (lambda: l.page_offset(3), lambda: l.semaphore_offset(5), lambda: l.page_offset(-1),
                 lambda: l.output_scratch_offset(output_stage=2, output_stages=2),
                 lambda: l.weight_page_offset(input_stage=1, page_in_stage=0, input_stages=1, stage_pages=2)):
        with pytest.raises(IndexError):
            call()
    with pytest.raises(ValueError):
        PipelinePageLayout(page_count=0, page_bytes=16)
    with pytest.raises(ValueError):
        PipelinePageLayout(page_count=1, page_bytes=-1)


def test_native_plan_is_what_the_megakernel_sizes_its_launch_with():
    import sys
    sys.path.insert(0, os.path.dirname(__file__))
    import dep_edges_driver as driver

    ops, keep = driver._layer_ops("machete_b200", 1, 1008, 4)
    mk = Megakernel(ops)
    plan = NativeSmemPlan(CTRL_BYTES, mk._act_bytes, mk.page_bytes, smem_optin=mk._smem_optin, max_pages=32)
    assert plan.num_pages == mk.num_pages and plan.total_size == mk.smem_size
    assert plan.pages_offset % 1024 == 0 and plan.total_size <= mk._smem_optin
    # 32 KB pages next to 4 KB of staged activations: six pages in 227 KB
    p = NativeSmemPlan(CTRL_BYTES, 4096, 32768)
    assert p.num_pages == 6 and p.act_offset == CTRL_BYTES and p.pages_offset == CTRL_BYTES + 4096
    assert NativeSmemPlan(CTRL_BYTES, 220 * 1024, 32768).num_pages == 0
