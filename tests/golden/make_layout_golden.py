"""Record the reference's shared-memory layout numbers (run once, with the reference's ``src`` on
PYTHONPATH): ``python tests/golden/make_layout_golden.py tests/golden/layout_reference.json``."""

import json
import sys

from machete.megakernel.paged_memory import NPageLayout, PipelinePageLayout

out = {"npage": [], "pipeline": [], "for_device": []}
for pages, size, slots in [(1, 4096, None), (2, 16384, None), (4, 49152, None), (6, 32768, None), (7, 32768, 3),
                           (16, 1000, None), (3, 16400, 16), (5, 18432, 8)]:
    l = NPageLayout(num_pages=pages, page_size=size, num_slots=slots)
    out["npage"].append({"args": [pages, size, slots], "flags": l.flags_offset, "iq": l.iq_offset, "mbar": l.mbarrier_offset,
                         "scratch": l.scratch_size, "aligned": l.aligned_page_size, "start": l.pages_start,
                         "total": l.total_size, "slots": l.num_slots, "wn": l.work_notify_mbar_offset(l.num_slots - 1),
                         "cd": l.compute_done_mbar_offset(l.num_slots - 1)})
for size, smem in [(16384, 232448), (32768, 232448), (49152, 232448), (49152, 101376), (8192, 232448), (65536, 232448)]:
    l = NPageLayout.for_device(page_size=size, max_smem=smem)
    out["for_device"].append({"args": [size, smem], "pages": l.num_pages, "total": l.total_size})
for pc, pb, sc, sb in [(3, 1024, 5, 96), (1, 0, 0, 0), (13, 4096, 9, 1000), (2, 1001, 3, 17), (4, 8192, 0, 4096)]:
    l = PipelinePageLayout(page_count=pc, page_bytes=pb, semaphore_count=sc, scratch_bytes=sb)
    out["pipeline"].append({"args": [pc, pb, sc, sb], "sem": l.semaphores_offset, "scratch": l.scratch_offset,
                            "total": l.total_size, "last_page": l.page_offset(pc - 1),
                            "out1of2": l.output_scratch_offset(output_stage=1, output_stages=2)})
json.dump(out, open(sys.argv[1], "w"), indent=1)
