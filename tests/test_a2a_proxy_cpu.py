"""The all-to-all host proxy on CPU: two one-rank "nodes" with host-memory regions and host-only
transfer engines, Python playing the kernels' part (it writes what the kernels would stage and
raises the words they would raise). Checks what the proxy moves where, that a flag never arrives
before the data it announces, and that an injected write failure marks the proxy failed
(reference p2p-all-to-all/src/a2a_worker.rs:340-455, a2a_context.rs:332-334)."""

from __future__ import annotations

import time

import pytest
import torch

from pplx_garden import _native
from pplx_garden.fabric_lib import TransferEngine
from pplx_garden.native.p2p_all_to_all import AllToAllContext

WORLD, TOKENS, EXPERTS, HIDDEN, TOPK = 2, 8, 4, 64, 2
ARGS = dict(hidden_dim=HIDDEN, in_elemsize=2, out_elemsize=2, max_num_tokens=TOKENS, num_experts=EXPERTS,
            num_experts_per_token=TOPK, world_size=WORLD)
# words of the proxy block (A2AProxyWord in csrc/a2a/a2a_types.h)
DISPATCH_SENT, COMBINE_SENT, RECORDS, ROWS, ROW_BASE = 0, 1, 8, 16, 24
FLAG_STRIDE, MAX_RANKS = 128, 8
FLAG_DISPATCH_STARTED, FLAG_REMOTE_COMBINE = 0, 3


class Rank:
    def __init__(self, rank: int) -> None:
        self.rank = rank
        self.layout = AllToAllContext.layout(wire="plain", node_mask=1 << rank, **ARGS)
        self.engine = TransferEngine(1, [-1])
        L = self.layout
        self.sync = torch.zeros(L["sync_bytes"], dtype=torch.uint8)
        self.recv = torch.zeros(L["recv_bytes"], dtype=torch.uint8)
        _, self.sync_desc = self.engine.register_tensor(self.sync)
        _, self.recv_desc = self.engine.register_tensor(self.recv)
        other = 1 - rank
        self.shadow_sync = torch.zeros(L["sync_bytes"], dtype=torch.uint8)
        self.shadow_recv = torch.zeros(L["drecv_group_stride"], dtype=torch.uint8)
        self.stage = torch.zeros(L["max_recv_rows"] * L["combine_record_bytes"], dtype=torch.uint8)
        self.flag_source = torch.zeros(4096, dtype=torch.uint8)
        self.words = torch.zeros(32, dtype=torch.int32)
        self.slots = torch.zeros(L["max_recv_rows"], dtype=torch.int32)
        for t in (self.shadow_sync, self.shadow_recv, self.stage, self.flag_source):
            self.engine.register_tensor(t)
        self.other = other
        self.probe = None

    def start(self, peer: "Rank", wait_limit_ms: int = 3000) -> None:
        self.probe = _native._A2AProxyProbe(
            dict(ARGS, node_mask=1 << self.rank, wait_limit_ms=wait_limit_ms), self.rank, self.engine,
            [(peer.rank, peer.sync_desc, peer.recv_desc)], {peer.rank: self.shadow_sync.data_ptr()},
            {peer.rank: self.shadow_recv.data_ptr()}, self.stage.data_ptr(), self.flag_source.data_ptr(),
            self.words.data_ptr(), self.slots.data_ptr())

    def flag(self, row: int, src: int) -> int:
        off = (row * MAX_RANKS + src) * FLAG_STRIDE
        return int(self.sync[off:off + 4].view(torch.int32).item())

    def close(self) -> None:
        if self.probe is not None:
            self.probe.close()
        self.engine.stop()


def _wait(cond, timeout=5.0) -> bool:
    end = time.monotonic() + timeout
    while time.monotonic() < end:
        if cond():
            return True
        time.sleep(0.002)
    return False


@pytest.fixture()
def ranks():
    r = [Rank(0), Rank(1)]
    r[0].start(r[1])
    r[1].start(r[0])
    yield r
    for x in r:
        x.close()


def test_proxy_forwards_dispatch_then_combine(ranks) -> None:
    a, b = ranks                      # a = rank 0 sends, b = rank 1 receives
    L = a.layout
    d_stride, c_stride = L["dispatch_record_bytes"], L["combine_record_bytes"]
    tag, par, group = 1, 0, 0

    # ---- dispatch 1: three records for rank 1, and the counts the kernel would have written ----
    records = torch.randint(1, 255, (3 * d_stride,), dtype=torch.uint8)
    a.shadow_recv[:3 * d_stride] = records
    counts_off = L["off_counts"] + 4 * (par * L["counts_bank_words"] + group * L["counts_stride"])
    counts = torch.arange(1, L["counts_stride"] + 1, dtype=torch.int32)
    a.shadow_sync[counts_off:counts_off + 4 * L["counts_stride"]] = counts.view(torch.uint8)
    a.words[RECORDS + 1] = 3
    a.words[DISPATCH_SENT] = tag
    assert _wait(lambda: b.flag(FLAG_DISPATCH_STARTED, 0) == tag), a.probe.error()
    # the flag is there: counts and records must already be, at the same places in the real regions
    dst = L["off_drecv"] + group * L["drecv_group_stride"]
    assert torch.equal(b.recv[dst:dst + 3 * d_stride], records)
    assert int(b.recv[dst + 3 * d_stride:dst + 4 * d_stride].count_nonzero()) == 0
    assert torch.equal(b.sync[counts_off:counts_off + 4 * L["counts_stride"]].view(torch.int32), counts)
    # the proxy counts a phase once its own write of the flag has completed: just after the flag is visible
    assert _wait(lambda: a.probe.counters() == (1, 0))

    # ---- combine 1: rows for origin group 1 sit in the second segment of the staging buffer ----
    first, rows = 5, 4                # five rows of group 0 come first (they stay on this rank)
    slots = [7, 0, 12, 3]             # combine slots (token * topk + k) at the origin
    payload = torch.randint(1, 255, (rows, c_stride), dtype=torch.uint8)
    a.stage.view(-1, c_stride)[first:first + rows] = payload
    a.slots[first:first + rows] = torch.tensor(slots, dtype=torch.int32)
    a.words[ROW_BASE + 1] = first
    a.words[ROWS + 1] = rows
    a.words[COMBINE_SENT] = tag
    assert _wait(lambda: b.flag(FLAG_REMOTE_COMBINE, 0) == tag), a.probe.error()
    crecv = b.recv[L["off_crecv"]:].view(-1)[:TOKENS * TOPK * c_stride].view(TOKENS * TOPK, c_stride)
    for i, slot in enumerate(slots):
        assert torch.equal(crecv[slot], payload[i])
    untouched = [s for s in range(TOKENS * TOPK) if s not in slots]
    assert int(crecv[untouched].count_nonzero()) == 0
    assert _wait(lambda: a.probe.counters() == (1, 1)) and not a.probe.failed()

    # ---- a second dispatch with nothing for rank 1: the flag still travels ----
    a.words[RECORDS + 1] = 0
    a.words[DISPATCH_SENT] = 2
    assert _wait(lambda: b.flag(FLAG_DISPATCH_STARTED, 0) == 2)


def test_proxy_reports_an_injected_write_failure(ranks) -> None:
    a, b = ranks
    a.engine._inject_write_failure(-1, 1)
    a.words[RECORDS + 1] = 1
    a.words[DISPATCH_SENT] = 1
    assert _wait(lambda: a.probe.failed())
    assert "fabric-lib transfer error" in a.probe.error()
    assert b.flag(FLAG_DISPATCH_STARTED, 0) == 0      # no flag for a dispatch that did not arrive


def test_proxy_gives_up_on_a_lost_write() -> None:
    r = [Rank(0), Rank(1)]
    try:
        r[0].start(r[1], wait_limit_ms=300)
        r[1].start(r[0], wait_limit_ms=300)
        r[0].engine._inject_fault(-1, "drop", 1)
        r[0].words[RECORDS + 1] = 2
        r[0].words[DISPATCH_SENT] = 1
        assert _wait(lambda: r[0].probe.failed(), timeout=3.0)
        assert "did not complete" in r[0].probe.error()
    finally:
        for x in r:
            x.close()
