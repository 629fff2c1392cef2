"""Runtime surface of the handle on the GPU: op updates, tracing, variant bookkeeping, recovery."""

import json

import pytest
import torch

import oracle
from machete_b200 import _native as N
from machete_b200.kernels.allreduce import AllReduceSm100Op
from machete_b200.kernels.attention import flash_decoding_schedule
from machete_b200.kernels.decode_matvec import MatvecSm100Op
from machete_b200.megakernel import Megakernel, MegakernelConfig
from machete_b200.megakernel.lowering import LowerCtx
from machete_b200.megakernel.peer import PeerBuffers
from tests.util import assert_parity

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def test_update_op_advances_the_kv_window_across_a_page_boundary():
    """One handle, four cache positions: the attention op record is replaced through mk_update_op
    (longer window: more tokens per split, and from 64 to 65 tokens a second ring page), and every
    step must equal a program scheduled from scratch for that position and the oracle."""
    B, H, Hkv, D, T = 1, 8, 2, 64, 256
    g = torch.Generator().manual_seed(21)
    q = torch.randn(B, 1, H, D, generator=g).to(BF).cuda()
    kc = torch.randn(B, T, Hkv, D, generator=g).to(BF).cuda()
    vc = torch.randn(B, T, Hkv, D, generator=g).to(BF).cuda()
    o = torch.full_like(q, float("nan"))
    n0 = 62
    ops, _ = flash_decoding_schedule(q, kc[:, :n0], vc[:, :n0], o, num_splits=1, kv_group_size=H // Hkv)
    mk = Megakernel(ops)
    mk.run()
    ctx = LowerCtx(num_sms=mk.num_sms, page_bytes=mk.page_bytes, smem_optin=232448)
    for n in (63, 64, 65, 130):
        new_ops, _ = flash_decoding_schedule(q, kc[:, :n], vc[:, :n], torch.empty_like(o), num_splits=1,
                                             kv_group_size=H // Hkv)
        fresh = Megakernel(new_ops)
        rec = fresh.native_ops[0]
        # keep this handle's own output, lse and arrival buffers; take the new window from the fresh lowering
        mine = mk.native_ops[0]
        for key in (N.AT_P_O, N.AT_P_LSE, N.AT_P_ARRIVE, N.AT_P_OPART, N.AT_P_LSEPART):
            rec.p[key] = mine.p[key]
        mk.update_op(0, rec)
        o.fill_(float("nan"))
        mk.run()
        want = oracle.attention_bshd(q.cpu().float(), kc[:, :n].cpu().float(), vc[:, :n].cpu().float())
        assert_parity(o, want, f"window of {n} tokens after update_op")
        assert mk.status()[0] == 0 and (mk.read_counters() == 0).all()
    del ctx
    # an update that changes the unit count is refused with a message
    bad, _ = flash_decoding_schedule(q, kc[:, :200], vc[:, :200], torch.empty_like(o), num_splits=3,
                                     kv_group_size=H // Hkv)
    with pytest.raises(ValueError, match="unit count"):
        mk.update_op(0, Megakernel(bad).native_ops[0])


def test_trace_records_and_chrome_export(tmp_path):
    a = torch.randn(1, 1, 512, device="cuda").to(BF)
    w = (torch.randn(1024, 512, device="cuda") * 0.02).to(BF)
    y = torch.zeros(1, 1, 1024, dtype=BF, device="cuda")
    mk = Megakernel(MatvecSm100Op.schedule(a=a, weight=w, y=y))
    mk.run()
    plain = y.clone()
    mk.enable_trace(256)
    mk.run()
    assert torch.equal(plain, y)                       # the traced kernel variant computes the same bits
    tr = mk.read_trace()
    assert len(tr) == mk.program.num_ctas * 8
    codes = {int(c) for arr in tr.values() for c in arr["code"]}
    assert {1, 2, 3, 4, 5, 6, 7, 8, 9} <= codes        # loads, pages, units and the op-entry event
    for arr in tr.values():
        t = arr["t"].astype("int64")
        assert (t[1:] >= t[:-1]).all()                 # one time base, monotonic per warp
    path = tmp_path / "trace.json"
    mk.export_chrome_trace(str(path), ctas=(0, 1))
    events = json.loads(path.read_text())["traceEvents"]
    assert events and all(e["ph"] == "X" and e["dur"] >= 0 for e in events)
    assert {e["name"].split()[0] for e in events} >= {"load", "page", "unit"}
    # the per-op table of the same launch: one op, all of its units, a positive span inside the launch
    (row,) = mk.stage_table()
    assert row["name"] == "MatvecSm100Op" and row["units"] == 64 and 0 < row["span"] < 1000
    assert row["begin"] >= 0 and row["end"] == pytest.approx(row["begin"] + row["span"]) and row["page"] > 0
    mk.disable_trace()
    mk.run()
    assert torch.equal(plain, y)


def test_large_program_still_runs_after_a_smaller_one_was_compiled():
    """The shared-memory limit belongs to the kernel function, not to a handle: a later, smaller
    program of the same variant must not lower it under a live larger one."""
    g = torch.Generator().manual_seed(22)
    x8 = torch.randn(1, 1, 8192, generator=g).to(BF).cuda()
    w8 = (torch.randn(256, 8192, generator=g) * 0.02).to(BF).cuda()
    y8 = torch.zeros(1, 1, 256, dtype=BF, device="cuda")
    big = Megakernel(MatvecSm100Op.schedule(a=x8, weight=w8, y=y8), config=MegakernelConfig(native_kc=1024))
    big.run()
    x1 = torch.randn(1, 1, 256, generator=g).to(BF).cuda()
    w1 = (torch.randn(64, 256, generator=g) * 0.02).to(BF).cuda()
    y1 = torch.zeros(1, 1, 64, dtype=BF, device="cuda")
    small = Megakernel(MatvecSm100Op.schedule(a=x1, weight=w1, y=y1), config=MegakernelConfig(native_kc=256, num_pages=2))
    assert small.smem_size < big.smem_size
    small.run()
    y8.zero_()
    big.run()
    assert_parity(y8.view(1, 256), oracle.matvec(x8.cpu().view(1, 8192), w8.cpu()), "large program, second run")


def test_grid_larger_than_the_device_is_refused():
    a = torch.randn(1, 1, 256, device="cuda").to(BF)
    w = (torch.randn(16 * 400, 256, device="cuda") * 0.02).to(BF)
    y = torch.zeros(1, 1, 16 * 400, dtype=BF, device="cuda")
    mk = Megakernel(MatvecSm100Op.schedule(a=a, weight=w, y=y), config=MegakernelConfig(num_sms=400))
    with pytest.raises(RuntimeError, match="multiprocessors"):
        mk.compile()


def test_peer_that_never_writes_times_out_and_the_launch_count_survives_the_reset():
    """Rank 0 of a 2-rank all-reduce whose peer buffer is a local allocation nobody writes: the wait for
    the peer's words gives up after timeout_ms with a status, the context stays usable, and the
    reset that follows keeps the launch count (the exchange's message epoch)."""
    peers = PeerBuffers.local(1 << 20, rank=0, world_size=2, device="cuda")
    x = torch.randn(1, 1, 2048, device="cuda")
    y = torch.zeros(1, 1, 2048, dtype=BF, device="cuda")
    mk = Megakernel(AllReduceSm100Op.schedule(peers=peers, x=x, y=y), config=MegakernelConfig(timeout_ms=50))
    assert mk.launch_count() == 0
    with pytest.raises(RuntimeError, match="peer rank"):
        mk.run()
    assert mk.status()[0] == 0            # wait() reset the handle before raising
    assert mk.launch_count() == 1         # ... but the aborted launch still counts
    # play the peer on the host: put rank 1's words for the NEXT launch (epoch base + 2) into rank 0's inbox
    nat = mk.native_ops[0]
    epoch = nat.i[N.AR_EPOCH_BASE] + mk.launch_count() + 1
    n, P = 2048, 2
    half = -(-P * n * 8 // 16) * 16
    inbox = peers.buffer[nat.s[N.AR_S_INBOX] + (epoch & 1) * half:][:P * n * 8].view(torch.int32).view(P, n, 2)
    peer_x = torch.randn(n, device="cuda")
    inbox[1, :, 0] = peer_x.view(torch.int32)
    inbox[1, :, 1] = epoch
    torch.cuda.synchronize()
    mk.run()
    assert_parity(y.view(-1), (x.view(-1) + peer_x).cpu(), "sum with the host-played peer")
    assert mk.launch_count() == 2
    mk.set_launch_count(7)
    assert mk.launch_count() == 7
