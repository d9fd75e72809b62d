"""The fused MoE layer against a float32 PyTorch statement of the same layer (with the same
quantisation points), on one GPU and across GPUs."""

from __future__ import annotations

import pytest
import torch

from pplx_garden.distributed import ParallelLaunch
from pplx_garden.ops import dequantize_128x128, dequantize_1x128, quantize_1x128

pytestmark = pytest.mark.gpu


def _reference(x, indices, weights, w13_q, w13_s, w2_q, w2_s, experts_per_rank_offset=0, pow2=True):
    """out[t] = sum_k w[t,k] * FFN_{e(t,k)}(x[t]) with fp8 quantisation at the same places."""
    xq, xs = quantize_1x128(x.float().cpu(), pow2=pow2)
    xd = dequantize_1x128(xq, xs)
    w13 = dequantize_128x128(w13_q.cpu(), w13_s.cpu())
    w2 = dequantize_128x128(w2_q.cpu(), w2_s.cpu())
    I = w2.shape[-1]
    out = torch.zeros_like(xd)
    idx = indices.cpu().to(torch.int64)
    for t in range(x.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            d = w13[e] @ xd[t]
            act = torch.nn.functional.silu(d[:I]) * d[I:]
            aq, a_s = quantize_1x128(act.unsqueeze(0), pow2=pow2)
            y = (w2[e] @ dequantize_1x128(aq, a_s)[0]).to(torch.bfloat16).float()
            out[t] += weights[t, k].item() * y
    return out


@pytest.mark.parametrize("scale_format", ["pow2", "fp32"])
def test_single_gpu_layer_matches_reference(scale_format: str) -> None:
    from pplx_garden.models import ExpertParallelMoE, route_topk

    dev = torch.device("cuda", 0)
    H, I, E, K, T = 512, 256, 8, 2, 48
    layer = ExpertParallelMoE(hidden_dim=H, intermediate_dim=I, num_experts=E, num_experts_per_token=K,
                              max_num_tokens=T, device=dev, global_group=None, init_std=0.05,
                              scale_format=scale_format)
    try:
        gen = torch.Generator(device="cpu").manual_seed(3)
        x = torch.randn((T, H), generator=gen).to(torch.bfloat16).to(dev)
        indices, weights = route_topk(torch.randn((T, E), generator=gen).to(dev), K)
        out = layer(x, indices, weights)
        torch.cuda.synchronize()
        layer.check()
        want = _reference(x, indices.view(torch.int32), weights.cpu(), layer.w13, layer.w13_scale, layer.w2, layer.w2_scale,
                          pow2=scale_format == "pow2")
        got = out.float().cpu()
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 1e-3, f"max abs error {err} vs scale {want.abs().max().item()}"
    finally:
        layer.destroy()


def test_fused_combine_equals_unfused_on_one_gpu() -> None:
    """The down projection that writes its rows straight into the combine buffers must give
    bit-identical tokens to GEMM -> expert_y -> combine_send: the rows are the same bf16 values."""
    from pplx_garden.models import ExpertParallelMoE, route_topk

    dev = torch.device("cuda", 0)
    H, I, E, K, T = 512, 256, 8, 2, 300
    gen = torch.Generator(device="cpu").manual_seed(5)
    w13 = torch.randn((E, 2 * I, H), generator=gen) * 0.05
    w2 = torch.randn((E, H, I), generator=gen) * 0.05
    x = torch.randn((T, H), generator=gen).to(torch.bfloat16).to(dev)
    indices, weights = route_topk(torch.randn((T, E), generator=gen).to(dev), K)
    outs = []
    for fused, bulk in ((False, False), (True, False), (True, True)):
        layer = ExpertParallelMoE(hidden_dim=H, intermediate_dim=I, num_experts=E, num_experts_per_token=K,
                                  max_num_tokens=T, device=dev, global_group=None, w13=w13, w2=w2,
                                  fused_combine=fused, fused_bulk=bulk)
        try:
            for _ in range(3):   # several layers in a row: epochs, the done counter's reset
                out = layer(x, indices, weights)
            torch.cuda.synchronize()
            layer.check()
            outs.append(out.float().cpu())
        finally:
            layer.destroy()
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0], outs[2])


def test_fused_combine_with_four_emulated_ranks() -> None:
    """Four ranks in one process: every rank's scatter GEMM writes into the other ranks' combine
    buffers (all on this GPU) and signals them; the receive phase then reduces as usual."""
    from pplx_garden.kernels.local_all_to_all import LocalAllToAllGroup
    from pplx_garden.ops import (MODE_BF16, MODE_BF16_SCATTER, MODE_SWIGLU_QUANT, grouped_fp8_gemm,
                                 quantize_128x128, topk_route)

    dev = torch.device("cuda", 0)
    world, T, E, H, I, K = 4, 96, 16, 512, 256, 4
    group = LocalAllToAllGroup(
        world_size=world, max_num_tokens=T, num_experts=E, expert_padding=1, hidden_dim=H,
        hidden_dim_scale=H // 128, in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16,
        scale_dtype=torch.float32, num_experts_per_token=K, device=dev, wait_limit_ms=2000,
        wire="plain")   # the GEMM writes plain rows
    try:
        gen = torch.Generator(device="cpu").manual_seed(9)
        L, rows = group.num_local_experts, group.max_recv_rows
        q13 = [[t.to(dev) for t in quantize_128x128(torch.randn((L, 2 * I, H), generator=gen) * 0.05)] for _ in range(world)]
        q2 = [[t.to(dev) for t in quantize_128x128(torch.randn((L, H, I), generator=gen) * 0.05)] for _ in range(world)]
        xs = [torch.randn((T, H), generator=gen).to(torch.bfloat16).to(dev) for _ in range(world)]
        routed = [topk_route(torch.randn((T, E), generator=gen).to(dev), K) for _ in range(world)]
        idx, wts = [r[0] for r in routed], [r[1] for r in routed]
        num = [torch.zeros(L, dtype=torch.int32, device=dev) for _ in range(world)]
        ox = [torch.zeros((rows, H), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn) for _ in range(world)]
        osc = [torch.zeros((rows, H // 128), dtype=torch.float32, device=dev) for _ in range(world)]
        act = [torch.zeros((rows, I), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn) for _ in range(world)]
        act_s = [torch.zeros((rows, I // 128), dtype=torch.float32, device=dev) for _ in range(world)]
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        results = []
        for fused, bulk in ((False, False), (True, False), (True, True)):
            out = [torch.zeros((T, H), dtype=torch.bfloat16, device=dev) for _ in range(world)]
            group.dispatch(num, ox, osc, xs, None, idx, wts)
            for r in range(world):
                grouped_fp8_gemm(ox[r], osc[r], q13[r][0], q13[r][1], num[r], act[r], act_s[r],
                                 mode=MODE_SWIGLU_QUANT, error_flag=flag)
            if fused:
                descs = group.combine_send_external(bulk)
                for r in range(world):
                    grouped_fp8_gemm(act[r], act_s[r], q2[r][0], q2[r][1], num[r], None, mode=MODE_BF16_SCATTER,
                                     error_flag=flag, scatter=descs[r])
                group.combine(out, idx, wts, None, do_send=False, do_recv=True)
            else:
                ys = [torch.zeros((rows, H), dtype=torch.bfloat16, device=dev) for _ in range(world)]
                for r in range(world):
                    grouped_fp8_gemm(act[r], act_s[r], q2[r][0], q2[r][1], num[r], ys[r], mode=MODE_BF16,
                                     error_flag=flag)
                group.combine(out, idx, wts, ys)
            torch.cuda.synchronize()
            group.check()
            assert int(flag.item()) == 0
            results.append([o.float().cpu() for o in out])
        for r in range(world):
            assert results[0][r].abs().max() > 0
            assert torch.equal(results[0][r], results[1][r]), f"rank {r}"
            assert torch.equal(results[0][r], results[2][r]), f"rank {r} (bulk copies)"
    finally:
        group.destroy()


def _worker(device, dp_group, global_group, seed, fused=False):
    from pplx_garden.models import ExpertParallelMoE, route_topk

    H, I, E, K, T = 512, 256, 16, 4, 64
    world, rank = global_group.size, global_group.rank
    L = E // world
    gen = torch.Generator(device="cpu").manual_seed(seed)
    w13_all = torch.randn((E, 2 * I, H), generator=gen) * 0.05
    w2_all = torch.randn((E, H, I), generator=gen) * 0.05
    layer = ExpertParallelMoE(hidden_dim=H, intermediate_dim=I, num_experts=E, num_experts_per_token=K,
                              max_num_tokens=T, device=device, global_group=global_group,
                              w13=w13_all[rank * L:(rank + 1) * L], w2=w2_all[rank * L:(rank + 1) * L],
                              fused_combine=fused)
    try:
        g2 = torch.Generator(device="cpu").manual_seed(seed + 1 + rank)
        x = torch.randn((T, H), generator=g2).to(torch.bfloat16).to(device)
        indices, weights = route_topk(torch.randn((T, E), generator=g2).to(device), K)
        out = layer(x, indices, weights)
        torch.cuda.synchronize()
        layer.check()
        from pplx_garden.ops import quantize_128x128

        w13_q, w13_s = quantize_128x128(w13_all, pow2=True)
        w2_q, w2_s = quantize_128x128(w2_all, pow2=True)
        want = _reference(x, indices.view(torch.int32), weights.cpu(), w13_q, w13_s, w2_q, w2_s)
        got = out.float().cpu()
        err = (got - want).abs().max().item()
        assert err <= 0.06 * want.abs().max().item() + 1e-3, f"rank {rank}: max abs error {err}"
    finally:
        layer.destroy()
    return True


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_layer_matches_reference(world: int, fused: bool) -> None:
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    assert all(ParallelLaunch(world_size=world).run(_worker, 11, fused))
