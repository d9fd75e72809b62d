#!/usr/bin/env python
"""Top-k routing kernel against torch.topk + softmax on the shapes the MoE benchmarks use
(tokens x experts, k = 8), CUDA-event timed after warm-up, logits rotated through copies larger
than L2 for the big shape.

    python -m benchmarks.bench_router
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from pplx_garden.ops import topk_route, topk_route_reference


def time_us(fn, iters: int = 50, warmup: int = 5) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / iters


def main() -> None:
    dev = torch.device("cuda", 0)
    out = []
    for tokens, experts, k in ((128, 256, 8), (4096, 256, 8), (2048, 128, 8), (262144, 256, 8)):
        copies = max(1, min(8, (256 << 20) // (tokens * experts * 4)))
        logits = [torch.randn((tokens, experts), device=dev) for _ in range(copies)]
        idx = torch.empty((tokens, k), dtype=torch.int32, device=dev).view(torch.uint32)
        w = torch.empty((tokens, k), dtype=torch.float32, device=dev)
        state = {"i": 0}

        def ours() -> None:
            state["i"] += 1
            topk_route(logits[state["i"] % copies], k, None, idx, w)

        def ref() -> None:
            state["i"] += 1
            topk_route_reference(logits[state["i"] % copies], k)

        t_ours, t_ref = time_us(ours), time_us(ref)
        bytes_moved = tokens * experts * 4 + tokens * k * 8
        out.append({"tokens": tokens, "experts": experts, "k": k, "ours_us": t_ours, "torch_us": t_ref,
                    "ours_gb_s": bytes_moved / t_ours / 1e3, "speedup": t_ref / t_ours})
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
