#!/usr/bin/env python
"""All-to-all benchmark with the reference's flag set and report
(benchmarks/bench_all_to_all.py:269-516 there: six timings per iteration, dispatch and
combine fused and split into send / recv, a "wait" between phases that stands for the other
layers, results gathered from every rank and summarised as mean, spread and percentiles, plus
the NCCL all_to_all_single time for the same bytes).

    python -m benchmarks.bench_all_to_all --world-size 8 --num-warmup 50 --num-repeats 200

Differences that follow from the design: --nets-per-gpu and --max-private-tokens are accepted
and ignored (no NIC takes part inside one NVSwitch domain, and there is no private/overflow
split because record slots are fixed); with --world-size 1 nothing crosses a link. Times are
CUDA-event times on each rank's stream, in microseconds.
"""

from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Optional

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from pplx_garden.distributed import ParallelGroup, ParallelLaunch
from pplx_garden.kernels.p2p_all_to_all import P2PAllToAll
from pplx_garden.utils.math import Statistics, ceil_div, round_up
from pplx_garden.utils.torch import profile_range, str_to_dtype


@dataclass
class Config:
    max_num_tokens: int
    num_experts: int
    hidden_dim: int
    hidden_dim_scale: Optional[int]
    num_experts_per_token: int
    in_dtype: torch.dtype
    out_dtype: torch.dtype
    scale_dtype: Optional[torch.dtype]
    nets_per_gpu: int
    max_private_tokens: int
    combine_mode: str

    def dispatch_bytes(self) -> int:
        per_token = self.hidden_dim * self.in_dtype.itemsize
        if self.hidden_dim_scale and self.scale_dtype is not None:
            per_token += self.hidden_dim_scale * self.scale_dtype.itemsize
        return self.max_num_tokens * self.num_experts_per_token * per_token

    def combine_bytes(self) -> int:
        return self.max_num_tokens * self.num_experts_per_token * self.hidden_dim * self.out_dtype.itemsize


def _rank_inputs(cfg: Config, seed: int, device: torch.device):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    scores = torch.randn((cfg.max_num_tokens, cfg.num_experts), generator=gen).abs() + 1
    indices = torch.topk(scores, cfg.num_experts_per_token, dim=-1).indices
    x = torch.randn((cfg.max_num_tokens, cfg.hidden_dim), generator=gen)
    scale = None
    if cfg.hidden_dim_scale:
        scale = torch.rand((cfg.max_num_tokens, cfg.hidden_dim_scale), generator=gen) + 0.5
    weights = torch.rand((cfg.max_num_tokens, cfg.num_experts_per_token), generator=gen)
    weights = weights / weights.sum(dim=-1, keepdim=True)
    return (indices.to(torch.uint32).to(device), weights.to(device), x.to(cfg.in_dtype).to(device),
            None if scale is None else scale.to(device))


def _check(cfg: Config, a2a: P2PAllToAll, bufs: dict, inputs, device: torch.device) -> None:
    """dispatch -> expert = 2 * dequantised x -> combine must give back 2 * dequantised x, because the
    weights of a token add up to one (tests/p2p_all_to_all/test_p2p_all_to_all.py:44-50 there)."""
    indices, weights, x, scale = inputs
    a2a.dispatch(bufs["num_tokens"], bufs["expert_x"], bufs["expert_x_scale"], x, scale, indices, weights)
    ex = bufs["expert_x"].to(torch.float32)
    if scale is not None:
        rep = cfg.hidden_dim // cfg.hidden_dim_scale
        ex = ex * bufs["expert_x_scale"].repeat_interleave(rep, dim=1)
    bufs["expert_y"].copy_((ex * 2).to(cfg.out_dtype))
    a2a.combine(bufs["out_tokens"], indices, weights, bufs["expert_y"])
    torch.cuda.synchronize(device)
    ref = x.to(torch.float32)
    if scale is not None:
        ref = ref * scale.repeat_interleave(cfg.hidden_dim // cfg.hidden_dim_scale, dim=1)
    ref = ref * 2
    got = bufs["out_tokens"].to(torch.float32)
    err = (got - ref).abs().max().item()
    tol = 0.05 * ref.abs().max().item() + 1e-3
    if not err <= tol:
        raise AssertionError(f"round trip mismatch: max abs error {err} > {tol}")


def _worker(device: torch.device, dp_group: Optional[ParallelGroup], global_group: Optional[ParallelGroup],
            cfg: Config, num_warmup: int, num_repeats: int, output: str, check: bool) -> Optional[dict]:
    torch.cuda.set_device(device)
    rank = global_group.rank if global_group is not None else 0
    world = global_group.size if global_group is not None else 1
    dp_size = dp_group.size if dp_group is not None else 1
    dp_rank = rank // dp_size
    a2a = P2PAllToAll(
        max_num_tokens=cfg.max_num_tokens, num_experts=cfg.num_experts, expert_padding=1,
        hidden_dim=cfg.hidden_dim, hidden_dim_scale=cfg.hidden_dim_scale, in_dtype=cfg.in_dtype,
        out_dtype=cfg.out_dtype, scale_dtype=cfg.scale_dtype, num_experts_per_token=cfg.num_experts_per_token,
        nets_per_gpu=cfg.nets_per_gpu, max_private_tokens=cfg.max_private_tokens, device=device,
        dp_group=dp_group, global_group=global_group, combine_mode=cfg.combine_mode)
    try:
        rows = a2a.max_recv_rows
        bufs = {
            "num_tokens": torch.zeros(a2a.num_local_experts, dtype=torch.int32, device=device),
            "expert_x": torch.zeros((rows, cfg.hidden_dim), dtype=torch.uint8 if cfg.in_dtype.itemsize == 1 else cfg.in_dtype,
                                    device=device).view(cfg.in_dtype),
            "expert_x_scale": None if not cfg.hidden_dim_scale else torch.zeros(
                (rows, cfg.hidden_dim_scale), dtype=cfg.scale_dtype, device=device),
            "expert_y": torch.zeros((rows, cfg.hidden_dim), dtype=cfg.out_dtype, device=device),
            "out_tokens": torch.zeros((cfg.max_num_tokens, cfg.hidden_dim), dtype=cfg.out_dtype, device=device),
        }
        inputs = _rank_inputs(cfg, dp_rank, device)
        indices, weights, x, scale = inputs
        if check:
            _check(cfg, a2a, bufs, inputs, device)

        dummy = torch.zeros(1, dtype=torch.float32, device=device)
        n = 2048 if cfg.max_num_tokens <= 128 else 8192
        gemm = torch.empty((n, n), dtype=torch.float32, device=device).normal_()

        def wait() -> None:
            # the other layers of the model, and a loose alignment of the ranks
            if global_group is not None:
                torch.distributed.all_reduce(dummy)
            _ = gemm @ gemm
            if global_group is not None:
                torch.distributed.all_reduce(dummy)

        def dispatch(do_send: bool, do_recv: bool) -> None:
            a2a.dispatch(bufs["num_tokens"], bufs["expert_x"], bufs["expert_x_scale"], x, scale, indices, weights,
                         do_send=do_send, do_recv=do_recv)

        def combine(do_send: bool, do_recv: bool) -> None:
            a2a.combine(bufs["out_tokens"], indices, weights, bufs["expert_y"], do_send=do_send, do_recv=do_recv)

        # NCCL reference for the same payloads (what torch_group.py:239 there offers)
        d_rows = cfg.max_num_tokens * cfg.num_experts_per_token
        nccl_d = torch.zeros(round_up(ceil_div(cfg.dispatch_bytes(), world), 16) * world, dtype=torch.uint8, device=device)
        nccl_c = torch.zeros(round_up(ceil_div(cfg.combine_bytes(), world), 16) * world, dtype=torch.uint8, device=device)
        nccl_d_out, nccl_c_out = torch.empty_like(nccl_d), torch.empty_like(nccl_c)

        names = ("dispatch", "combine", "dispatch_send", "dispatch_recv", "combine_send", "combine_recv",
                 "overlap_dispatch_send", "overlap_work", "overlap_dispatch_recv",
                 "overlap_combine_send", "overlap_combine_recv", "overlap_step",
                 "nccl_dispatch", "nccl_combine")
        # "other work" that a micro-batched model runs between the send and the receive half of a
        # phase (the reference's overlap section: benchmarks/bench_all_to_all.py:406-425)
        fake_n = 1024 if cfg.max_num_tokens <= 128 else 4096
        fake = torch.empty((fake_n, fake_n), dtype=torch.bfloat16, device=device).normal_()
        times: dict[str, list[float]] = {k: [] for k in names}

        def timed(fn) -> torch.cuda.Event:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            return s, e

        for it in range(num_warmup + num_repeats):
            if it == max(num_warmup - 1, 0):
                # capture range for `nsys --capture-range=cudaProfilerApi` (reference :359-361)
                torch.cuda.profiler.start()
            ev = {}
            wait()
            ev["dispatch"] = timed(lambda: dispatch(True, True))
            wait()
            ev["combine"] = timed(lambda: combine(True, True))
            wait()
            ev["dispatch_send"] = timed(lambda: dispatch(True, False))
            wait()
            ev["dispatch_recv"] = timed(lambda: dispatch(False, True))
            wait()
            ev["combine_send"] = timed(lambda: combine(True, False))
            wait()
            ev["combine_recv"] = timed(lambda: combine(False, True))
            # overlap section: send half, other work, receive half, all on one stream
            wait()
            ov_start = torch.cuda.Event(enable_timing=True)
            ov_end = torch.cuda.Event(enable_timing=True)
            ov_start.record()
            with profile_range("overlap"):
                ev["overlap_dispatch_send"] = timed(lambda: dispatch(True, False))
                ev["overlap_work"] = timed(lambda: torch.matmul(fake, fake))
                ev["overlap_dispatch_recv"] = timed(lambda: dispatch(False, True))
                ev["overlap_combine_send"] = timed(lambda: combine(True, False))
                _ = fake @ fake
                ev["overlap_combine_recv"] = timed(lambda: combine(False, True))
            ov_end.record()
            ev["overlap_step"] = (ov_start, ov_end)
            if global_group is not None:
                wait()
                ev["nccl_dispatch"] = timed(lambda: torch.distributed.all_to_all_single(nccl_d_out, nccl_d))
                wait()
                ev["nccl_combine"] = timed(lambda: torch.distributed.all_to_all_single(nccl_c_out, nccl_c))
            torch.cuda.synchronize(device)
            if it >= num_warmup:
                for k, (s, e) in ev.items():
                    times[k].append(s.elapsed_time(e) * 1000.0)

        torch.cuda.profiler.stop()
        if global_group is not None:
            for k in names:
                times[k] = sum(global_group.all_gather_object(times[k]), [])
        if rank != 0:
            return None
        report = {
            "config": {**{k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in asdict(cfg).items()},
                       "world_size": world, "dp_size": dp_size, "num_warmup": num_warmup, "num_repeats": num_repeats,
                       "dispatch_bytes": cfg.dispatch_bytes(), "combine_bytes": cfg.combine_bytes(), "rows": d_rows},
            "unit": "us",
        }
        for k in names:
            if times[k]:
                st = Statistics.create(times[k])
                report[k] = {f: getattr(st, f) for f in st.__dataclass_fields__}
                print(f"{k:>14}: {st}", file=sys.stderr)
        with open(output, "w") as f:
            f.write(json.dumps(report) + "\n")
        return report
    finally:
        if global_group is not None:
            global_group.barrier()
        a2a.destroy()


def main() -> None:
    p = argparse.ArgumentParser(description="All-to-all benchmark")
    p.add_argument("--world-size", type=int, required=True)
    p.add_argument("--init-method", type=str, default=None)
    p.add_argument("--dp-size", type=int, default=1)
    p.add_argument("--node-rank", type=int, default=0)
    p.add_argument("--num-warmup", type=int, default=100)
    p.add_argument("--num-repeats", type=int, default=1000)
    p.add_argument("--nets-per-gpu", type=int, default=0)
    p.add_argument("--max-num-tokens", type=int, default=128)
    p.add_argument("--max-private-tokens", type=int, default=256)
    p.add_argument("--num-experts", type=int, default=256)
    p.add_argument("--hidden-dim", type=int, default=7168)
    p.add_argument("--hidden-dim-scale", type=int, default=56)
    p.add_argument("--num-experts-per-token", type=int, default=8)
    p.add_argument("--in-dtype", type=str_to_dtype, default=torch.float8_e4m3fn)
    p.add_argument("--out-dtype", type=str_to_dtype, default=torch.bfloat16)
    p.add_argument("--scale-dtype", type=str_to_dtype, default=torch.float32)
    p.add_argument("--nvlink", type=int, default=None, help="accepted for compatibility: all ranks share one NVLink domain")
    p.add_argument("--combine-mode", choices=("per_route", "pre_reduce"), default="per_route")
    p.add_argument("--output", type=Path, default=Path("/dev/stdout"))
    p.add_argument("--check", type=bool, default=True, action=argparse.BooleanOptionalAction)
    args = p.parse_args()
    scaled = args.hidden_dim_scale and args.hidden_dim_scale > 0
    cfg = Config(
        max_num_tokens=args.max_num_tokens, num_experts=args.num_experts, hidden_dim=args.hidden_dim,
        hidden_dim_scale=args.hidden_dim_scale if scaled else None,
        num_experts_per_token=args.num_experts_per_token, in_dtype=args.in_dtype, out_dtype=args.out_dtype,
        scale_dtype=args.scale_dtype if scaled else None, nets_per_gpu=args.nets_per_gpu,
        max_private_tokens=args.max_private_tokens, combine_mode=args.combine_mode)
    ParallelLaunch(world_size=args.world_size, init_method=args.init_method, dp_size=args.dp_size,
                   node_rank=args.node_rank).run(
        _worker, cfg, args.num_warmup, args.num_repeats, str(args.output), args.check)


if __name__ == "__main__":
    main()
