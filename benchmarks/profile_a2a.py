#!/usr/bin/env python
"""Small dispatch+combine workload for profilers: eight expert-parallel ranks played on ONE
GPU (DeepSeek-V3 decode shape: 128 tokens per rank, hidden 7168, 256 experts, top-8, fp8
dispatch, bf16 combine), a few iterations, then exit. Holds well under 1 GB on the device.

    python -m benchmarks.profile_a2a [--iters 4] [--tokens 128] [--world 8] [--combine-mode per_route]
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from pplx_garden.kernels.local_all_to_all import LocalAllToAllGroup


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--combine-mode", default="per_route")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    H, E, K, W, T = 7168, 256, 8, args.world, args.tokens
    group = LocalAllToAllGroup(
        world_size=W, max_num_tokens=T, num_experts=E, expert_padding=1, hidden_dim=H,
        hidden_dim_scale=H // 128, in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16,
        scale_dtype=torch.float32, num_experts_per_token=K, device=dev, combine_mode=args.combine_mode)
    L, rows = group.num_local_experts, group.max_recv_rows
    xs = [torch.randn(T, H, device=dev).to(torch.float8_e4m3fn) for _ in range(W)]
    sc = [torch.rand(T, H // 128, device=dev) for _ in range(W)]
    tops = [torch.topk(torch.randn(T, E, device=dev), K) for _ in range(W)]
    idx = [t.indices.to(torch.int32).view(torch.uint32) for t in tops]
    wts = [torch.softmax(t.values, -1) for t in tops]
    num = [torch.zeros(L, dtype=torch.int32, device=dev) for _ in range(W)]
    ox = [torch.zeros(rows, H, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn) for _ in range(W)]
    osc = [torch.zeros(rows, H // 128, device=dev) for _ in range(W)]
    out = [torch.zeros(T, H, dtype=torch.bfloat16, device=dev) for _ in range(W)]
    ys = [torch.randn(rows, H, device=dev).to(torch.bfloat16) for _ in range(W)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(args.iters):
        if it == args.iters - 1:
            start.record()
        group.dispatch(num, ox, osc, xs, sc, idx, wts)
        group.combine(out, idx, wts, ys)
    end.record()
    torch.cuda.synchronize()
    group.check()
    print(f"last iteration: {start.elapsed_time(end) * 1000:.1f} us for {W} ranks on one GPU; "
          f"rows per rank {int(num[0].sum())}")
    group.destroy()


if __name__ == "__main__":
    main()
