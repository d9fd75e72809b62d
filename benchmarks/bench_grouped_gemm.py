#!/usr/bin/env python
"""Throughput of the tcgen05 grouped fp8 GEMM on the expert FFN shapes of a Qwen3-30B-A3B-like
layer (hidden 2048, intermediate 768, 16 local experts, ~1024 rows per expert) and of a
DeepSeek-V3-like layer, device-timed with CUDA events after warm-up, inputs larger than L2
rotated between iterations. Reports TFLOP/s and the fraction of the measured cuBLAS bf16 peak
doubled for fp8 (MEASURED_PEAKS.json if present). `--scales pow2` (default) quantises with
power-of-two scales and runs the kernel whose tensor cores apply them; `--scales fp32` runs the
kernel that folds arbitrary scales in per K block and also reports where its pipeline waits.

    python -m benchmarks.bench_grouped_gemm [--rows-per-expert 1024] [--experts 16] [--scales pow2|fp32]
    python -m benchmarks.bench_grouped_gemm --experts 8 --hidden 7168 --intermediate 2048    # DeepSeek-V3-like
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from pplx_garden.ops import MODE_BF16, MODE_SWIGLU_QUANT, grouped_fp8_gemm, quantize_128x128, quantize_1x128


def time_op(fn, warmup: int = 5, iters: int = 20) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / iters  # us


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--rows-per-expert", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--intermediate", type=int, default=768)
    ap.add_argument("--copies", type=int, default=4, help="operand sets rotated to defeat L2")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tile-rows", type=int, default=0, help="256 = CTA pairs, 128 = single CTAs, 0 = automatic")
    ap.add_argument("--num-ctas", type=int, default=0, help="CTAs to launch (0 = one per SM)")
    ap.add_argument("--scales", choices=["fp32", "pow2"], default="pow2",
                    help="pow2: power-of-two scales applied by the tensor cores (block-scaled MMA); "
                         "fp32: any scales, folded in by the epilogue per K block")
    ap.add_argument("--ablate", action="store_true", help="also time the kernel with one pipeline stage removed")
    args = ap.parse_args()
    pow2 = args.scales == "pow2"
    dev = torch.device("cuda", 0)
    E, M, H, I = args.experts, args.rows_per_expert, args.hidden, args.intermediate
    rows = E * M
    peaks_file = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    bf16_peak = json.loads(peaks_file.read_text())["bf16_tflops"] if peaks_file.exists() else 1590.0
    peak_kind = "measured" if peaks_file.exists() else "fallback"
    cnt = torch.full((E,), M, dtype=torch.int32, device=dev)
    sets = []
    for c in range(args.copies):
        g = torch.Generator(device="cpu").manual_seed(c)
        x, xs = quantize_1x128(torch.randn(rows, H, generator=g), pow2=pow2)
        w13, w13s = quantize_128x128(torch.randn(E, 2 * I, H, generator=g) * H ** -0.5, pow2=pow2)
        w2, w2s = quantize_128x128(torch.randn(E, H, I, generator=g) * I ** -0.5, pow2=pow2)
        sets.append([t.to(dev) for t in (x, xs, w13, w13s, w2, w2s)])
    act = torch.zeros(rows, I, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    act_s = torch.zeros(rows, I // 128, dtype=torch.float32, device=dev)
    y = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    state = {"i": 0}

    def gemm1() -> None:
        x, xs, w13, w13s, _, _ = sets[state["i"] % args.copies]
        state["i"] += 1
        grouped_fp8_gemm(x, xs, w13, w13s, cnt, act, act_s, mode=MODE_SWIGLU_QUANT, error_flag=flag,
                         tile_rows=args.tile_rows, scale_format=args.scales, num_ctas=args.num_ctas)

    def gemm2() -> None:
        _, _, _, _, w2, w2s = sets[state["i"] % args.copies]
        state["i"] += 1
        grouped_fp8_gemm(act, act_s, w2, w2s, cnt, y, mode=MODE_BF16, error_flag=flag, tile_rows=args.tile_rows,
                         scale_format=args.scales, num_ctas=args.num_ctas)

    def both() -> None:
        gemm1()
        gemm2()

    t1, t2, t12 = time_op(gemm1, iters=args.iters), time_op(gemm2, iters=args.iters), time_op(both, iters=args.iters)
    assert flag.item() == 0
    # where the pipeline waits (one instrumented launch per GEMM)
    waits = {}
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    for name, run in (("gate_up", 0), ("down", 1)) if not pow2 else ():
        wc = torch.zeros((sms, 4), dtype=torch.int64, device=dev)
        x, xs, w13, w13s, w2, w2s = sets[0]
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        if run == 0:
            grouped_fp8_gemm(x, xs, w13, w13s, cnt, act, act_s, mode=MODE_SWIGLU_QUANT, error_flag=flag, wait_cycles=wc)
        else:
            grouped_fp8_gemm(act, act_s, w2, w2s, cnt, y, mode=MODE_BF16, error_flag=flag, wait_cycles=wc)
        c1.record()
        torch.cuda.synchronize()
        m = wc.float().mean(dim=0).tolist()
        waits[name] = {"kernel_us": c0.elapsed_time(c1) * 1e3, "mean_wait_cycles": {
            "producer_for_free_stage": m[0], "mma_for_free_accumulator": m[1], "mma_for_operands": m[2],
            "epilogue_for_partial_sums": m[3]}}
    # what the remaining stages sustain with one stage removed (results are garbage, timing only)
    ablation = {}
    if args.ablate and not pow2:
        for label, skip in (("no_epilogue_reads", 1), ("no_mma", 2), ("no_tma", 4), ("tma_only", 3), ("mma_only", 5)):
            def g1() -> None:
                x, xs, w13, w13s, _, _ = sets[state["i"] % args.copies]
                state["i"] += 1
                grouped_fp8_gemm(x, xs, w13, w13s, cnt, act, act_s, mode=MODE_SWIGLU_QUANT, error_flag=flag,
                                 debug_skip=skip)

            def g2() -> None:
                _, _, _, _, w2, w2s = sets[state["i"] % args.copies]
                state["i"] += 1
                grouped_fp8_gemm(act, act_s, w2, w2s, cnt, y, mode=MODE_BF16, error_flag=flag, debug_skip=skip)

            ablation[label] = {"gate_up_us": time_op(g1, iters=args.iters), "down_us": time_op(g2, iters=args.iters)}
    f1, f2 = 2.0 * rows * 2 * I * H, 2.0 * rows * H * I
    out = {
        "shape": {"experts": E, "rows_per_expert": M, "hidden": H, "intermediate": I},
        "scales": args.scales, "num_ctas": args.num_ctas,
        "gate_up_swiglu_us": t1, "gate_up_tflops": f1 / t1 / 1e6,
        "down_us": t2, "down_tflops": f2 / t2 / 1e6,
        "ffn_us": t12, "ffn_tflops": (f1 + f2) / t12 / 1e6,
        "fp8_roofline_tflops": 2 * bf16_peak,
        "ffn_fraction_of_roofline": (f1 + f2) / t12 / 1e6 / (2 * bf16_peak),
        "roofline_note": f"2 x cuBLAS bf16 burst peak ({peak_kind})",
        "waits": waits,
        "ablation": ablation,
    }
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
