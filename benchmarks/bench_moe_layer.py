#!/usr/bin/env python
"""Fused expert-parallel MoE layer, Qwen3-30B-A3B-like: 2048 tokens per rank, hidden 2048,
128 experts, top-8, SwiGLU experts with intermediate 768, fp8 e4m3 weights with 128x128 block
scales, fp8 activations with 1x128 scales.

Two arms on the same inputs, one process per GPU:

* ours      route (top-k kernel) -> dispatch with fused fp8 quantisation over NVLink peer
            stores -> tcgen05 grouped GEMM gate/up with SwiGLU + requantise -> grouped GEMM
            down -> weighted combine (`pplx_garden.models.ExpertParallelMoE`)
* fused     as ours, but the down projection's epilogue writes every row over NVLink into the
            combine receive buffer of the GPU its token came from and signals the receivers
            (no expert_y round trip, no combine send kernel)
* library   the same layer from library parts only: torch top-k, NCCL all_to_all_single
            dispatch / combine (`NcclAllToAll`), per-expert cuBLAS bf16 matmuls on the
            dequantised weights. The reference's own kernels cannot be built here, so this is
            the baseline that runs.

Times are CUDA-event times per phase and for the whole layer, max over ranks, with an L2 flush
before every timed layer. Launch with torchrun (one rank per GPU) or alone on one GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 benchmarks/bench_moe_layer.py --steps 20 --warmup 5
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from pplx_garden.distributed import ProcessGroup
from pplx_garden.kernels.nccl_all_to_all import NcclAllToAll
from pplx_garden.models import ExpertParallelMoE
from pplx_garden.ops import dequantize_128x128, topk_route, topk_route_reference


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--intermediate", type=int, default=768)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--scales", choices=["pow2", "fp32"], default="pow2",
                    help="pow2: power-of-two scales applied by the tensor cores; fp32: any scales, folded in by the epilogue")
    ap.add_argument("--no-library", action="store_true")
    ap.add_argument("--no-fused", action="store_true", help="skip the arm whose down projection sends the rows itself")
    ap.add_argument("--bulk", action="store_true", help="also time the fused arm with bulk copies (cp.async.bulk) as the sender")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    pg = ProcessGroup.from_env(device) if world > 1 else None
    group = pg.create_group() if pg is not None else None
    rank = group.rank if group is not None else 0
    T, H, I, E, K = args.tokens, args.hidden, args.intermediate, args.experts, args.topk

    layer = ExpertParallelMoE(hidden_dim=H, intermediate_dim=I, num_experts=E, num_experts_per_token=K,
                              max_num_tokens=T, device=device, global_group=group, seed=1, scale_format=args.scales)
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    x = torch.randn((T, H), generator=gen).to(torch.bfloat16).to(device)
    logits = torch.randn((T, E), generator=gen).to(device)
    out = torch.empty_like(x)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    sync = torch.zeros(1, device=device)

    def align() -> None:
        flush.fill_(1)
        if group is not None:
            torch.distributed.all_reduce(sync)

    def reduce_max(v: float) -> float:
        if group is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    def timed_phases(phases) -> dict:
        """phases: list of (name, fn). Returns mean microseconds per phase and in total."""
        acc = {name: 0.0 for name, _ in phases}
        acc["layer"] = 0.0
        for step in range(args.warmup + args.steps):
            align()
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(phases) + 1)]
            evs[0].record()
            for i, (_, fn) in enumerate(phases):
                fn()
                evs[i + 1].record()
            torch.cuda.synchronize(device)
            if step >= args.warmup:
                for i, (name, _) in enumerate(phases):
                    acc[name] += evs[i].elapsed_time(evs[i + 1]) * 1e3
                acc["layer"] += evs[0].elapsed_time(evs[-1]) * 1e3
        return {k: reduce_max(v / args.steps) for k, v in acc.items()}

    # ------------------------------------------------------------------ ours
    st: dict = {}

    def o_route() -> None:
        st["idx"], st["w"] = topk_route(logits, K)

    def o_dispatch() -> None:
        layer.a2a.dispatch(layer.expert_num_tokens, layer.expert_x, layer.expert_x_scale, x, None, st["idx"], st["w"])

    def o_gemm1() -> None:
        layer.gate_up()

    def o_gemm2() -> None:
        layer.down()

    def o_combine() -> None:
        layer.a2a.combine(out, st["idx"], st["w"], layer.expert_y)

    ours = timed_phases([("route", o_route), ("dispatch", o_dispatch), ("gate_up_swiglu", o_gemm1),
                         ("down", o_gemm2), ("combine", o_combine)])
    layer.check()
    ours_out = out.float().clone()

    # the same layer with the routing made inside the dispatch kernel: one launch instead of two
    r_idx = torch.zeros((T, K), dtype=torch.int32, device=device).view(torch.uint32)
    r_w = torch.zeros((T, K), dtype=torch.float32, device=device)

    def r_dispatch() -> None:
        layer.a2a.dispatch(layer.expert_num_tokens, layer.expert_x, layer.expert_x_scale, x, None, r_idx, r_w,
                           logits=logits)

    def r_combine() -> None:
        layer.a2a.combine(out, r_idx, r_w, layer.expert_y)

    routed = timed_phases([("route_and_dispatch", r_dispatch), ("gate_up_swiglu", o_gemm1), ("down", o_gemm2),
                           ("combine", r_combine)])
    layer.check()
    routed["equal_to_unfused"] = bool(torch.equal(out.float(), ours_out))

    # the same layer with the down projection writing its rows into the peers' combine buffers
    fused = fused_bulk = None
    if not args.no_fused:
        def f_down_send() -> None:
            layer.down_and_send()

        def f_recv() -> None:
            layer.a2a.combine(out, st["idx"], st["w"], None, do_send=False, do_recv=True)

        fused = timed_phases([("route", o_route), ("dispatch", o_dispatch), ("gate_up_swiglu", o_gemm1),
                              ("down_and_combine_send", f_down_send), ("combine_recv", f_recv)])
        layer.check()
        fused["equal_to_unfused"] = bool(torch.equal(out.float(), ours_out))

        # ... and with the rows handed to the bulk-copy engine instead of stored by the epilogue warps
        if args.bulk:
            layer.fused_bulk = True
            fused_bulk = timed_phases([("route", o_route), ("dispatch", o_dispatch), ("gate_up_swiglu", o_gemm1),
                                       ("down_and_combine_send", f_down_send), ("combine_recv", f_recv)])
            layer.check()
            fused_bulk["equal_to_unfused"] = bool(torch.equal(out.float(), ours_out))
            layer.fused_bulk = False
    rows = int(layer.expert_num_tokens.sum().item())
    flops = 2.0 * rows * (2 * I * H + H * I)
    ours["expert_rows_this_rank"] = rows
    ours["ffn_tflops_per_gpu"] = flops / (ours["gate_up_swiglu"] + ours["down"]) / 1e6

    # ------------------------------------------------------------------ library parts
    lib = None
    max_err = None
    if not args.no_library:
        L = layer.num_local_experts
        a2a = NcclAllToAll(max_num_tokens=T, num_experts=E, expert_padding=1, hidden_dim=H, hidden_dim_scale=None,
                           in_dtype=torch.bfloat16, out_dtype=torch.bfloat16, scale_dtype=None,
                           num_experts_per_token=K, device=device, global_group=group)
        w13 = dequantize_128x128(layer.w13, layer.w13_scale).to(torch.bfloat16)
        w2 = dequantize_128x128(layer.w2, layer.w2_scale).to(torch.bfloat16)
        max_rows = layer.a2a.max_recv_rows
        num_tokens = torch.zeros(L, dtype=torch.int32, device=device)
        ex = torch.zeros((max_rows, H), dtype=torch.bfloat16, device=device)
        ey = torch.zeros((max_rows, H), dtype=torch.bfloat16, device=device)
        lout = torch.empty_like(x)

        def l_route() -> None:
            st["idx"], st["w"] = topk_route_reference(logits, K)

        def l_dispatch() -> None:
            a2a.dispatch(num_tokens, ex, None, x, None, st["idx"], st["w"])

        def l_ffn() -> None:
            counts = num_tokens.tolist()
            r0 = 0
            for e, n in enumerate(counts):
                if n:
                    h = ex[r0:r0 + n] @ w13[e].T
                    h = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
                    ey[r0:r0 + n] = h @ w2[e].T
                r0 += n

        def l_combine() -> None:
            a2a.combine(lout, st["idx"], st["w"], ey)

        lib = timed_phases([("route", l_route), ("dispatch", l_dispatch), ("ffn", l_ffn), ("combine", l_combine)])
        # the two arms differ by the fp8 quantisation of the activations only
        ref = lout.float()
        max_err = reduce_max(((ours_out - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item())
        a2a.destroy()

    if rank == 0:
        print(json.dumps({
            "config": {"model": "Qwen3-30B-A3B-like MoE layer", "tokens_per_rank": T, "hidden": H, "intermediate": I,
                       "experts": E, "topk": K, "n_gpus": world, "scales": args.scales, "l2": "flushed before each layer",
                       "steps": args.steps, "warmup": args.warmup},
            "unit": "us, max over ranks",
            "ours": ours, "ours_route_in_dispatch": routed, "ours_fused_combine": fused, "ours_fused_combine_bulk": fused_bulk, "library": lib, "max_rel_err_ours_vs_library": max_err,
            "speedup_layer": None if lib is None else lib["layer"] / ours["layer"],
            "speedup_layer_fused": None if lib is None or fused is None else lib["layer"] / fused["layer"],
        }))
    layer.destroy()
    if pg is not None:
        pg.destroy()


if __name__ == "__main__":
    main()
