"""Multi-rank dispatch/combine on ONE GPU: every rank is a slice of one launch.
Shapes follow the reference's parametrisation table
(tests/p2p_all_to_all/test_p2p_all_to_all.py:240-557) plus cases for the split phases,
bound_m, accumulate, repeated iterations, pre-reduced combine and fused quantisation."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import pytest
import torch

from pplx_garden.kernels import oracle
from tests.a2a_data import act, make_rank_data

pytestmark = pytest.mark.gpu


@dataclass
class Cfg:
    world: int
    dp_size: int = 1
    tokens: int = 128
    experts: int = 16
    hidden: int = 128
    hidden_scale: Optional[int] = None
    topk: int = 2
    in_dtype: torch.dtype = torch.float32
    out_dtype: torch.dtype = torch.float32
    padding: int = 1
    combine_mode: str = "per_route"
    wire: Optional[str] = None


CONFIGS = {
    "W1-FP32": Cfg(world=1),
    "W2-FP32": Cfg(world=2),
    "W2-BF16": Cfg(world=2, in_dtype=torch.bfloat16, out_dtype=torch.bfloat16),
    "W2-BF16-PADDED": Cfg(world=2, tokens=8, hidden=16, in_dtype=torch.bfloat16,
                          out_dtype=torch.bfloat16, padding=16),
    "W2-SCALES": Cfg(world=2, tokens=2, hidden_scale=16, in_dtype=torch.bfloat16,
                     out_dtype=torch.bfloat16),
    "W4-FP32-K8": Cfg(world=4, experts=128, topk=8),
    "W4-BF16-H7168": Cfg(world=4, experts=256, hidden=7168, topk=8, in_dtype=torch.bfloat16,
                         out_dtype=torch.bfloat16),
    "W4-DP2-TINY": Cfg(world=4, dp_size=2, tokens=1, experts=4, hidden=8, topk=1,
                       in_dtype=torch.bfloat16, out_dtype=torch.bfloat16),
    "W4-DP2": Cfg(world=4, dp_size=2, tokens=64, experts=32, hidden=256, topk=4,
                  in_dtype=torch.bfloat16, out_dtype=torch.bfloat16),
    "W8-BF16": Cfg(world=8, experts=128, hidden=7168, topk=8, in_dtype=torch.bfloat16,
                   out_dtype=torch.bfloat16),
    "W8-FP8": Cfg(world=8, tokens=256, experts=128, hidden=7168, hidden_scale=56, topk=8,
                  in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16),
    "W8-UNEVEN-EXPERTS": Cfg(world=8, tokens=32, experts=60, hidden=256, topk=6,
                             in_dtype=torch.bfloat16, out_dtype=torch.bfloat16, padding=4),
    "W8-PRE-REDUCE": Cfg(world=8, experts=64, hidden=1024, topk=8, in_dtype=torch.bfloat16,
                         out_dtype=torch.bfloat16, combine_mode="pre_reduce"),
    "W2-PRE-REDUCE-FP32": Cfg(world=2, combine_mode="pre_reduce"),
    "W8-F16-OUT": Cfg(world=8, tokens=16, experts=64, hidden=512, topk=4,
                      in_dtype=torch.bfloat16, out_dtype=torch.float16),
}


def _make_group(cfg: Cfg, device, **kw):
    from pplx_garden.kernels.local_all_to_all import LocalAllToAllGroup

    return LocalAllToAllGroup(
        world_size=cfg.world, dp_size=cfg.dp_size, max_num_tokens=cfg.tokens,
        num_experts=cfg.experts, expert_padding=cfg.padding, hidden_dim=cfg.hidden,
        hidden_dim_scale=cfg.hidden_scale, in_dtype=cfg.in_dtype, out_dtype=cfg.out_dtype,
        scale_dtype=torch.float32 if cfg.hidden_scale else None,
        num_experts_per_token=cfg.topk, device=device, combine_mode=cfg.combine_mode,
        wait_limit_ms=2000, wire=cfg.wire, **kw)


def _inputs(cfg: Cfg, device, seed_offset: int = 0):
    groups = cfg.world // cfg.dp_size
    data = [make_rank_data(seed=g + seed_offset, num_experts=cfg.experts, topk=cfg.topk,
                           num_tokens=cfg.tokens, hidden_dim=cfg.hidden,
                           hidden_dim_scale=cfg.hidden_scale,
                           in_dtype=torch.float32 if cfg.in_dtype == torch.float8_e4m3fn else cfg.in_dtype,
                           device=device) for g in range(groups)]
    if cfg.in_dtype == torch.float8_e4m3fn:
        for d in data:
            d.dp_x = d.dp_x.clamp(-400, 400).to(torch.float8_e4m3fn)
    return data


def _outputs(cfg: Cfg, group, device):
    L = group.num_local_experts
    rows = group.max_recv_rows
    W = cfg.world
    num = [torch.full((L,), -1, dtype=torch.int32, device=device) for _ in range(W)]
    ox = [torch.zeros((rows, cfg.hidden), dtype=torch.float32, device=device).to(cfg.in_dtype)
          for _ in range(W)]
    os_ = None
    if cfg.hidden_scale:
        os_ = [torch.zeros((rows, cfg.hidden_scale), dtype=torch.float32, device=device)
               for _ in range(W)]
    out = [torch.zeros((cfg.tokens, cfg.hidden), dtype=cfg.out_dtype, device=device)
           for _ in range(W)]
    return num, ox, os_, out


def _run_once(cfg: Cfg, group, data, device, *, split=False, bound=None, accumulate=False,
              out_prev=None):
    W = cfg.world
    per_rank = [data[r // cfg.dp_size] for r in range(W)]
    num, ox, os_, out = _outputs(cfg, group, device)
    if out_prev is not None:
        for o, p in zip(out, out_prev):
            o.copy_(p)
    xs = [d.dp_x for d in per_rank]
    scales = [d.dp_x_scale for d in per_rank] if cfg.hidden_scale else None
    idx = [d.indices for d in per_rank]
    wts = [d.weights for d in per_rank]
    bm = None
    if bound is not None:
        bm = [torch.tensor([bound], dtype=torch.int32, device=device) for _ in range(W)]
    if split:
        group.dispatch(num, ox, os_, xs, scales, idx, wts, bm, do_send=True, do_recv=False)
        group.dispatch(num, ox, os_, xs, scales, idx, wts, bm, do_send=False, do_recv=True)
    else:
        group.dispatch(num, ox, os_, xs, scales, idx, wts, bm)
    ys = [act(ox[r], None if os_ is None else os_[r]).to(cfg.out_dtype) for r in range(W)]
    if split:
        group.combine(out, idx, wts, ys, bm, do_send=True, do_recv=False, accumulate=accumulate)
        group.combine(out, idx, wts, ys, bm, do_send=False, do_recv=True, accumulate=accumulate)
    else:
        group.combine(out, idx, wts, ys, bm, accumulate=accumulate)
    torch.cuda.synchronize()
    group.check()
    return num, ox, os_, out


def _verify(cfg: Cfg, data, num, ox, os_, out, *, bound=None, out_prev=None):
    groups = cfg.world // cfg.dp_size
    n_tok = None if bound is None else [bound] * groups
    for r in range(cfg.world):
        exp = oracle.expected_dispatch(
            r, cfg.world, cfg.experts, cfg.padding,
            [d.dp_x.cpu() for d in data],
            [d.dp_x_scale.cpu() for d in data] if cfg.hidden_scale else None,
            [d.indices.cpu() for d in data], n_tok)
        oracle.check_dispatch(exp, num[r], ox[r], None if os_ is None else os_[r])
        d = data[r // cfg.dp_size]
        T = cfg.tokens if bound is None else bound
        want = act(d.dp_x[:T].cpu().to(torch.float32) if cfg.hidden_scale is None else d.dp_x[:T].cpu(),
                   None if d.dp_x_scale is None else d.dp_x_scale[:T].cpu())
        want = want.to(cfg.out_dtype).to(torch.float32)
        if out_prev is not None:
            want = want + out_prev[r][:T].cpu().to(torch.float32)
        got = out[r][:T].cpu().to(torch.float32)
        tol = dict(rtol=2e-2, atol=2e-2) if cfg.out_dtype != torch.float32 else dict(rtol=1e-5, atol=1e-5)
        if cfg.hidden_scale:
            tol = dict(rtol=3e-2, atol=0.5)
        torch.testing.assert_close(got, want, **tol, msg=lambda m, r=r: f"rank {r} combine: {m}")


@pytest.mark.parametrize("wire", ["ll", "plain"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_dispatch_combine(name: str, wire: str) -> None:
    """Every shape in both wire formats: flagged 128-byte lines and plain records."""
    from dataclasses import replace

    cfg = replace(CONFIGS[name], wire=wire)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device)
    try:
        data = _inputs(cfg, device)
        num, ox, os_, out = _run_once(cfg, group, data, device)
        _verify(cfg, data, num, ox, os_, out)
    finally:
        group.destroy()


@pytest.mark.parametrize("wire", ["ll", "plain"])
def test_repeated_iterations_and_split_phases(wire: str) -> None:
    """Tags advance and cursors are double-buffered: many iterations with new routing
    each time, alternating fused and split launches, must all be exact."""
    cfg = Cfg(world=4, tokens=48, experts=32, hidden=512, topk=4, in_dtype=torch.bfloat16,
              out_dtype=torch.bfloat16, padding=8, wire=wire)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device)
    try:
        for it in range(6):
            data = _inputs(cfg, device, seed_offset=100 * it)
            num, ox, os_, out = _run_once(cfg, group, data, device, split=bool(it % 2))
            _verify(cfg, data, num, ox, os_, out)
        iters = group.context.iterations(0)
        assert list(iters) == [6, 6]
    finally:
        group.destroy()


@pytest.mark.parametrize("wire", ["ll", "plain"])
def test_bound_m_and_accumulate(wire: str) -> None:
    cfg = Cfg(world=2, tokens=64, experts=16, hidden=256, topk=4, wire=wire)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device)
    try:
        data = _inputs(cfg, device)
        num, ox, os_, out = _run_once(cfg, group, data, device, bound=17)
        _verify(cfg, data, num, ox, os_, out, bound=17)
        for r in range(cfg.world):
            assert torch.count_nonzero(out[r][17:]) == 0, "rows past bound_m must stay untouched"
        prev = [torch.randn((cfg.tokens, cfg.hidden), device=device) for _ in range(cfg.world)]
        num, ox, os_, out = _run_once(cfg, group, data, device, accumulate=True, out_prev=prev)
        _verify(cfg, data, num, ox, os_, out, out_prev=prev)
    finally:
        group.destroy()


def test_zero_tokens() -> None:
    cfg = Cfg(world=2, tokens=4, experts=8, hidden=64, topk=2)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device)
    try:
        data = _inputs(cfg, device)
        num, ox, os_, out = _run_once(cfg, group, data, device, bound=0)
        for r in range(cfg.world):
            assert num[r].sum().item() == 0
    finally:
        group.destroy()


@pytest.mark.parametrize("wire", ["ll", "plain"])
@pytest.mark.parametrize("pow2", [False, True])
def test_fused_quantisation_matches_reference_quantiser(wire: str, pow2: bool) -> None:
    """bf16 tokens in, e4m3 + one fp32 scale per 1x128 block at the experts; with ``pow2_scales``
    every scale is the next power of two."""
    cfg = Cfg(world=4, tokens=32, experts=32, hidden=1024, hidden_scale=8, topk=4,
              in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16, wire=wire)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device, pow2_scales=pow2)
    try:
        groups = cfg.world
        raw = [make_rank_data(seed=g, num_experts=cfg.experts, topk=cfg.topk, num_tokens=cfg.tokens,
                              hidden_dim=cfg.hidden, hidden_dim_scale=None, in_dtype=torch.bfloat16,
                              device=device) for g in range(groups)]
        num, ox, os_, out = _outputs(cfg, group, device)
        group.dispatch(num, ox, os_, [d.dp_x for d in raw], None, [d.indices for d in raw],
                       [d.weights for d in raw])
        torch.cuda.synchronize()
        group.check()
        quant = [oracle.quantize_1x128(d.dp_x.cpu().to(torch.float32), pow2=pow2) for d in raw]
        for r in range(cfg.world):
            exp = oracle.expected_dispatch(
                r, cfg.world, cfg.experts, cfg.padding,
                [q[0].to(torch.float32) for q in quant], [q[1] for q in quant],
                [d.indices.cpu() for d in raw])
            torch.testing.assert_close(num[r].cpu(), exp.num_tokens, rtol=0, atol=0)
            # de-quantised rows must agree with the float reference quantiser
            for le, (start, want, ws) in enumerate(zip(exp.block_start, exp.rows, exp.scales)):
                n = want.shape[0]
                got = ox[r][start:start + n].cpu().to(torch.float32)
                gs = os_[r][start:start + n].cpu()
                if pow2:
                    assert (torch.frexp(gs)[0] == 0.5).all(), "scales must be powers of two"
                deq_got = got * gs.repeat_interleave(128, dim=1)
                deq_want = want * ws.repeat_interleave(128, dim=1)
                key_g = deq_got.sum(dim=1).argsort()
                key_w = deq_want.sum(dim=1).argsort()
                torch.testing.assert_close(deq_got[key_g], deq_want[key_w], rtol=0.07, atol=1e-3)
        ys = [(ox[r].to(torch.float32) * os_[r].repeat_interleave(128, dim=1) * 2).to(cfg.out_dtype)
              for r in range(cfg.world)]
        group.combine(out, [d.indices for d in raw], [d.weights for d in raw], ys)
        torch.cuda.synchronize()
        group.check()
        for r in range(cfg.world):
            want = raw[r].dp_x.cpu().to(torch.float32) * 2
            torch.testing.assert_close(out[r].cpu().to(torch.float32), want, rtol=0.08, atol=0.08)
    finally:
        group.destroy()


@pytest.mark.parametrize("wire", ["ll", "plain"])
def test_wait_timeout_reports_status_without_hanging(wire: str) -> None:
    """A receive whose sources never signalled must give up after the configured limit,
    leave the context marked failed and keep the CUDA context usable."""
    cfg = Cfg(world=2, tokens=4, experts=8, hidden=64, topk=2)
    device = torch.device("cuda", 0)
    from pplx_garden.kernels.local_all_to_all import LocalAllToAllGroup

    group = LocalAllToAllGroup(
        world_size=cfg.world, max_num_tokens=cfg.tokens, num_experts=cfg.experts,
        expert_padding=1, hidden_dim=cfg.hidden, hidden_dim_scale=None, in_dtype=torch.float32,
        out_dtype=torch.float32, scale_dtype=None, num_experts_per_token=cfg.topk, device=device,
        wait_limit_ms=200, wire=wire)
    try:
        num, ox, os_, out = _outputs(cfg, group, device)
        # recv without any send: the arrival flags stay at zero
        group.context._set_next_phase(1)
        with pytest.raises((TimeoutError, RuntimeError)):
            group.context.dispatch_multi(None, [
                (num[r].data_ptr(), ox[r].data_ptr(), ox[r].stride(0) * 4, None, None, None,
                 ox[r].shape[0]) for r in range(cfg.world)], torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            group.check()
        code, phase, who, detail, message = group.context.status(0)
        assert code == 1 and phase == 1, message
        # the device is still healthy
        assert torch.ones(8, device=device).sum().item() == 8
    finally:
        group.destroy()


def test_cuda_graph_replay_of_a_whole_layer() -> None:
    """dispatch -> expert -> combine captured once in a CUDA graph and replayed with new tokens and
    routing each time: the protocol keeps its epochs on the device, so a replay is a layer like any
    other (this is how a serving loop would launch it)."""
    cfg = Cfg(world=4, tokens=32, experts=16, hidden=256, topk=4, in_dtype=torch.bfloat16,
              out_dtype=torch.bfloat16)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device)
    try:
        W = cfg.world
        num, ox, os_, out = _outputs(cfg, group, device)
        data = _inputs(cfg, device)
        xs = [d.dp_x.clone() for d in data]
        idx = [d.indices.clone() for d in data]
        wts = [d.weights.clone() for d in data]
        ys = [torch.zeros((group.max_recv_rows, cfg.hidden), dtype=cfg.out_dtype, device=device) for _ in range(W)]

        def layer() -> None:
            group.dispatch(num, ox, None, xs, None, idx, wts)
            for r in range(W):
                ys[r].copy_(act(ox[r], None).to(cfg.out_dtype))
            group.combine(out, idx, wts, ys)

        layer()   # eager once: everything that allocates or loads modules happens here
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                layer()
        torch.cuda.synchronize()
        for it in range(4):
            fresh = _inputs(cfg, device, seed_offset=1000 * (it + 1))
            for r in range(W):
                xs[r].copy_(fresh[r].dp_x)
                idx[r].copy_(fresh[r].indices)
                wts[r].copy_(fresh[r].weights)
            graph.replay()
            torch.cuda.synchronize()
            group.check()
            _verify(cfg, fresh, num, ox, None, out)
        assert list(group.context.iterations(0)) == [5, 5]   # 1 eager + 4 replays (capturing runs nothing)
    finally:
        group.destroy()


def test_barrier_and_rejected_call_leaves_phase_order_intact() -> None:
    """The device barrier returns on every emulated rank; a dispatch that the host rejects
    (too many tokens) does not advance the phase order, so a corrected call may follow."""
    cfg = Cfg(world=4, tokens=8, experts=8, hidden=64, topk=2)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device)
    try:
        for _ in range(3):
            group.barrier()
        torch.cuda.synchronize()
        group.check()
        data = _inputs(cfg, device)
        num, ox, os_, out = _outputs(cfg, group, device)
        too_many = [torch.zeros((cfg.tokens + 1, cfg.hidden), device=device) for _ in range(cfg.world)]
        with pytest.raises((ValueError, RuntimeError)):
            group.dispatch(num, ox, os_, too_many, None, [d.indices for d in data],
                           [d.weights for d in data])
        num, ox, os_, out = _run_once(cfg, group, data, device)
        _verify(cfg, data, num, ox, os_, out)
        group.barrier()
        torch.cuda.synchronize()
        group.check()
    finally:
        group.destroy()


@pytest.mark.parametrize("wire", ["ll", "plain"])
@pytest.mark.parametrize("experts,topk,with_bias,bf16_logits", [(64, 4, False, False), (256, 8, True, False),
                                                                 (288, 6, True, True)])
def test_routing_fused_into_dispatch(wire: str, experts: int, topk: int, with_bias: bool, bf16_logits: bool) -> None:
    """dispatch(logits=...) picks the experts itself: the indices and weights it writes equal
    torch.topk + softmax (choice on logit + bias, weight from the plain logits), and the layer it
    drives gives the same tokens as routing first and dispatching with the result."""
    world, tokens, hidden = 4, 40, 256
    cfg = Cfg(world=world, tokens=tokens, experts=experts, hidden=hidden, topk=topk, in_dtype=torch.bfloat16,
              out_dtype=torch.bfloat16, wire=wire)
    device = torch.device("cuda", 0)
    group = _make_group(cfg, device)
    try:
        gen = torch.Generator(device="cpu").manual_seed(5)
        xs = [torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16).to(device) for _ in range(world)]
        logits = [torch.randn((tokens, experts), generator=gen) for _ in range(world)]
        if bf16_logits:
            logits = [lg.to(torch.bfloat16) for lg in logits]
        bias = [torch.randn(experts, generator=gen).to(device) if with_bias else None for _ in range(world)]
        logits = [lg.to(device) for lg in logits]
        idx = [torch.zeros((tokens, topk), dtype=torch.int32, device=device).view(torch.uint32) for _ in range(world)]
        wts = [torch.zeros((tokens, topk), dtype=torch.float32, device=device) for _ in range(world)]
        num, ox, _, out = _outputs(cfg, group, device)
        group.dispatch(num, ox, None, xs, None, idx, wts, logits=logits, logits_bias=bias if with_bias else None)
        ys = [act(ox[r], None).to(cfg.out_dtype) for r in range(world)]
        group.combine(out, idx, wts, ys)
        torch.cuda.synchronize()
        group.check()
        for r in range(world):
            lg = logits[r].float()
            key = lg + bias[r] if with_bias else lg
            want_idx = torch.topk(key, topk, dim=-1).indices
            want_w = torch.softmax(torch.gather(lg, 1, want_idx), dim=-1)
            got_idx = idx[r].view(torch.int32).long()
            assert torch.equal(got_idx.sort(dim=-1).values, want_idx.sort(dim=-1).values), f"rank {r}: experts differ"
            order_g, order_w = got_idx.argsort(dim=-1), want_idx.argsort(dim=-1)
            torch.testing.assert_close(torch.gather(wts[r], 1, order_g), torch.gather(want_w, 1, order_w),
                                       rtol=1e-4, atol=1e-6)
        # the same layer with the routing given: identical counts and tokens
        num2, ox2, _, out2 = _outputs(cfg, group, device)
        group.dispatch(num2, ox2, None, xs, None, idx, wts)
        ys2 = [act(ox2[r], None).to(cfg.out_dtype) for r in range(world)]
        group.combine(out2, idx, wts, ys2)
        torch.cuda.synchronize()
        group.check()
        for r in range(world):
            assert torch.equal(num[r], num2[r])
            assert torch.equal(out[r], out2[r]), f"rank {r}: fused routing changed the combined tokens"
    finally:
        group.destroy()
