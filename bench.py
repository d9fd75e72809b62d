#!/usr/bin/env python
"""Headline benchmark: MoE dispatch + combine latency on DeepSeek-V3 shapes.

    python bench.py --gpus 1 --steps 200 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 200 --warmup 20

One *step* is one ``dispatch`` followed by one ``combine`` of an expert-parallel MoE layer
with EP = number of GPUs: 128 tokens per rank (decode), hidden 7168, 256 experts, top-8,
fp8-e4m3 dispatch with 56 fp32 scales per token, bf16 combine, identity expert (the
combine input is a pre-filled bf16 buffer), which is the configuration of the reference's
benchmarks/bench_all_to_all.py:578-590 behind its published EP8 numbers
(docs/fabric-lib.md:100-119). ``--tokens 4096`` gives the prefill shape.

Timing: every step is bracketed by CUDA events on the launching stream; an L2 flush
(a 256 MiB device write followed by a read of the same buffer) and, with several ranks, a
tiny all-reduce that lines the ranks up run before the start event, outside the timed
interval. The reported value is the
maximum over ranks of the mean step time. The ``e2e`` entry times the same step through
the public API including the host->device copy of the step's inputs from pinned memory and
the device->host read of its result, with the host clock.

Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

PUBLISHED_US = {  # reference EP8 dispatch+combine, pplx-EFA column (docs/fabric-lib.md:109,119)
    128: 49.7 + 64.2,
    4096: 1052.4 + 1396.7,
}


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "nccl", "reference"], default="ours")
    ap.add_argument("--tokens", type=int, default=128, help="tokens per rank (128 decode, 4096 prefill)")
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--combine-mode", choices=["per_route", "pre_reduce"], default="per_route")
    ap.add_argument("--no-prefill", action="store_true", help="skip the secondary prefill measurement")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def reference_unavailable() -> str | None:
    """Why the unmodified reference cannot run here (None if it can)."""
    ref = ROOT / "baseline" / "_ref" / "pplx_garden"
    if not ref.exists():
        return "baseline/_ref is empty: the offline pip install of the reference was not done on this machine"
    if not list(ref.glob("_rust*.so")):
        return ("reference installed as pure Python only: its native module pplx_garden._rust is a Rust "
                "crate (cargo/rustc absent) that also needs libibverbs/libfabric, GDRCopy and an RDMA NIC per GPU")
    return None


def run_reference_arm(args: argparse.Namespace) -> None:
    """The unmodified reference through its own benchmark module (only reachable when its native
    module could be built, which needs cargo, libibverbs/libfabric, GDRCopy and a NIC per GPU)."""
    import glob

    ref_root = ROOT / "baseline" / "_ref"
    bench_mod = glob.glob(str(ref_root / "**" / "bench_all_to_all.py"), recursive=True)
    rank0 = int(os.environ.get("RANK", "0")) == 0
    if not bench_mod:
        if rank0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "reference installed without its benchmarks/bench_all_to_all.py"}))
        return
    if not rank0:
        return  # the reference's benchmark spawns its own ranks (ParallelLaunch)
    out = Path(tempfile.mkdtemp()) / "ref.json"
    env = dict(os.environ, PYTHONPATH=f"{ref_root}:{Path(bench_mod[0]).parent.parent}")
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    cmd = [sys.executable, bench_mod[0], "--world-size", str(args.gpus), "--nvlink", str(args.gpus),
           "--num-warmup", str(max(args.warmup, 3)), "--num-repeats", str(args.steps),
           "--max-num-tokens", str(args.tokens), "--output", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if proc.returncode != 0 or not out.exists():
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
        print(json.dumps({"impl": "reference", "unavailable": f"reference benchmark failed: {tail[0][:200]}"}))
        return
    data = json.loads(out.read_text())
    disp = data.get("dispatch", {}).get("both", {}).get("mean")
    comb = data.get("combine", {}).get("both", {}).get("mean")
    if disp is None or comb is None:
        print(json.dumps({"impl": "reference", "unavailable": "reference benchmark output has no dispatch/combine mean"}))
        return
    value = float(disp) + float(comb)
    print(json.dumps({"impl": "reference", "metric": "EP dispatch+combine latency per step (us), DeepSeek-V3 shape",
                      "value": value, "unit": "us", "n_gpus": args.gpus, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": value / 1000.0,
                      "higher_is_better": False}))


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a block runs. Reads only:
    NVML queries from a background thread every few milliseconds (nvidia-smi as a
    fallback), never a setting."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_s: float = 0.005) -> None:
        import threading

        self._clocks: list[float] = []
        self._max = None
        self._reasons: set[str] = set()
        self._stop = threading.Event()
        self._thread = None
        self._proc = None
        self._file = None
        try:
            import pynvml

            pynvml.nvmlInit()
            # NVML enumerates physical devices; honour CUDA_VISIBLE_DEVICES when it lists indices
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if visible:
                try:
                    phys = int(visible.split(",")[gpu_index])
                except (ValueError, IndexError):
                    phys = gpu_index
            handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            masks = {
                "hw_slowdown": pynvml.nvmlClocksThrottleReasonHwSlowdown,
                "hw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonHwThermalSlowdown,
                "sw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonSwThermalSlowdown,
                "sw_power_cap": pynvml.nvmlClocksThrottleReasonSwPowerCap,
            }

            def loop() -> None:
                while not self._stop.is_set():
                    try:
                        self._clocks.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        bits = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                        for name, mask in masks.items():
                            if bits & mask:
                                self._reasons.add(name)
                    except Exception:
                        pass
                    self._stop.wait(period_s)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
            self._file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            try:
                self._proc = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                     "-lms", "20", "-i", str(gpu_index)],
                    stdout=self._file, stderr=subprocess.DEVNULL)
            except OSError:
                self._proc = None

    def mark(self) -> int:
        """Number of samples so far (to select the ones taken inside an interval)."""
        return len(self._clocks)

    def stop(self, first: int = 0, last: int | None = None) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            clocks = self._clocks[first:last] or self._clocks
            if clocks:
                out.update(sm_mhz=statistics.median(clocks), sm_max_mhz=self._max,
                           reasons=sorted(self._reasons), samples=len(clocks))
            return out
        if self._proc is None:
            return out
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        self._file.flush()
        self._file.seek(0)
        clocks, max_clocks, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self._file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clocks.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self._file.close()
        try:
            os.unlink(self._file.name)
        except OSError:
            pass
        if clocks:
            out.update(sm_mhz=statistics.median(clocks), sm_max_mhz=max(max_clocks),
                       reasons=sorted(reasons), samples=len(clocks))
        return out


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        why = reference_unavailable()
        if why is not None:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": why}))
            return
        # reference_unavailable() returned None: the reference's native module exists. Drive its own
        # benchmark (benchmarks/bench_all_to_all.py of the reference, its public entry point) in a
        # child process with baseline/_ref first on the path, and relay its numbers.
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    import pplx_garden  # noqa: F401
    from pplx_garden.distributed import ProcessGroup
    from pplx_garden.kernels.nccl_all_to_all import NcclAllToAll
    from pplx_garden.kernels.p2p_all_to_all import P2PAllToAll

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    # Run this process (and first-touch its pinned staging buffers) on cores of the GPU's own
    # NUMA node, as the reference does for its worker threads
    # (python/pplx_garden/kernels/p2p_all_to_all.py:120-134).
    affinity = "unchanged"
    try:
        from pplx_garden.fabric_lib import TransferEngine

        for group in TransferEngine.detect_topology():
            if group.cuda_device == device.index and group.cpus:
                os.sched_setaffinity(0, set(group.cpus))
                affinity = f"{len(group.cpus)} cores of NUMA node {group.numa}"
    except Exception as exc:  # topology is best effort: a container may hide sysfs
        affinity = f"unchanged ({type(exc).__name__})"
    process_group = global_group = None
    if world > 1:
        process_group = ProcessGroup.from_env(device)
        global_group = process_group.create_group()

    def run_shape(tokens: int, steps: int, warmup: int, with_e2e: bool) -> dict:
        H, E, K = args.hidden, args.experts, args.topk
        hs = H // 128
        kw = dict(max_num_tokens=tokens, num_experts=E, expert_padding=1, hidden_dim=H,
                  hidden_dim_scale=hs, in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16,
                  scale_dtype=torch.float32, num_experts_per_token=K, device=device,
                  global_group=global_group)
        if args.impl == "ours":
            a2a = P2PAllToAll(dp_group=None, node_group=None, nets_per_gpu=0, max_private_tokens=None,
                              combine_mode=args.combine_mode, **kw)
            rows = a2a.max_recv_rows
        else:
            a2a = NcclAllToAll(**kw)
            rows = tokens * world * min(K, -(-E // world))
        L = -(-E // world)
        gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
        pool = 4
        host = []
        bias = torch.randn(E, generator=gen) * 0.5 if tokens >= 1024 else torch.zeros(E)
        for _ in range(pool):
            x = torch.randn((tokens, H), generator=gen)
            blocks = x.reshape(tokens, hs, 128)
            scale = blocks.abs().amax(-1).clamp_min(1e-10) / 448.0
            xq = (blocks / scale.unsqueeze(-1)).reshape(tokens, H).to(torch.float8_e4m3fn)
            logits = torch.randn((tokens, E), generator=gen) + bias
            top = torch.topk(logits, K, dim=-1)
            w = torch.softmax(top.values, dim=-1)
            host.append(tuple(t.pin_memory() for t in (xq.view(torch.uint8), scale.contiguous(),
                                                       top.indices.to(torch.int32).contiguous(), w.contiguous())))
        dev_inputs = [tuple(t.to(device) for t in h) for h in host]

        def views(tup):
            xq, sc, idx, w = tup
            return xq.view(torch.float8_e4m3fn), sc, idx.view(torch.uint32), w

        num = torch.zeros(L, dtype=torch.int32, device=device)
        ox = torch.zeros((rows, H), dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)
        osc = torch.zeros((rows, hs), dtype=torch.float32, device=device)
        out = torch.zeros((tokens, H), dtype=torch.bfloat16, device=device)
        expert_y = torch.randn((rows, H), device=device).to(torch.bfloat16)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        flush_words = flush.view(torch.int32)
        flush_sum = torch.zeros((), dtype=torch.int64, device=device)
        dummy = torch.zeros(1, device=device)

        def step(inp) -> None:
            xq, sc, idx, w = views(inp)
            a2a.dispatch(num, ox, osc, xq, sc, idx, w)
            a2a.combine(out, idx, w, expert_y)

        def all_counts_idx(i32: torch.Tensor) -> torch.Tensor:
            return i32.view(torch.int32).to(torch.int64).flatten()

        def line_up() -> None:
            # cold L2 without a cache full of dirty lines: write 256 MiB, then read it back
            flush.zero_()
            torch.sum(flush_words, dim=0, out=flush_sum)
            if world > 1:
                dist.all_reduce(dummy)
                if args.impl == "ours":
                    # NCCL lets the ranks leave its all-reduce several microseconds apart; the
                    # library's own device barrier lines them up to well under one
                    a2a.barrier()

        # Correctness of the path that is about to be timed, against what the routing tables of
        # ALL ranks say (outside the timed region): per-expert counts equal the bincount of the
        # gathered indices, every token routed to a local expert is present in that expert's rows
        # with its scales (decode shape; compared as multisets of row hashes), and the weighted
        # round trip returns dequant(x) within bf16 tolerance.
        xq, sc, idx, w = views(dev_inputs[0])
        a2a.dispatch(num, ox, osc, xq, sc, idx, w)
        y = (ox.to(torch.float32) * osc.repeat_interleave(128, dim=1)).to(torch.bfloat16)
        a2a.combine(out, idx, w, y)
        torch.cuda.synchronize()
        idx64 = idx.view(torch.int32).to(torch.int64)
        if world > 1:
            all_idx = torch.empty((world,) + tuple(idx64.shape), dtype=torch.int64, device=device)
            dist.all_gather_into_tensor(all_idx, idx64.contiguous())
        else:
            all_idx = idx64[None]
        want_counts = torch.bincount(all_idx.flatten(), minlength=E)[rank * L:(rank + 1) * L]
        assert torch.equal(num.to(torch.int64), want_counts), (
            f"rank {rank}: per-expert token counts differ from the gathered routing tables")
        assert int(want_counts.sum()) <= rows
        if tokens <= 512:
            xb = dev_inputs[0][0]
            if world > 1:
                all_x = torch.empty((world,) + tuple(xb.shape), dtype=torch.uint8, device=device)
                dist.all_gather_into_tensor(all_x, xb.contiguous())
                all_s = torch.empty((world,) + tuple(sc.shape), dtype=torch.float32, device=device)
                dist.all_gather_into_tensor(all_s, sc.contiguous())
            else:
                all_x, all_s = xb[None], sc[None]
            hgen = torch.Generator(device="cpu").manual_seed(99)
            hx = torch.randint(1, 1 << 20, (H,), generator=hgen).to(device)
            hsc = torch.randint(1, 1 << 20, (hs,), generator=hgen).to(device)

            def row_hash(xrows: torch.Tensor, srows: torch.Tensor) -> torch.Tensor:
                return ((xrows.to(torch.int64) * hx).sum(-1) +
                        (srows.contiguous().view(torch.int32).to(torch.int64) * hsc).sum(-1))

            src_hash = row_hash(all_x.reshape(-1, H), all_s.reshape(-1, hs))   # [world * tokens]
            flat_tok = torch.arange(world * tokens, device=device).repeat_interleave(K)
            flat_e = all_idx.reshape(-1)
            start = 0
            got_hash = row_hash(ox.view(torch.uint8), osc)
            for le in range(L):
                n = int(want_counts[le])
                sel = flat_tok[flat_e == rank * L + le]
                want_h = src_hash[sel].sort().values
                got_h = got_hash[start:start + n].sort().values
                assert torch.equal(want_h, got_h), f"rank {rank}: rows of local expert {le} are not the routed tokens"
                start += n
        want = (xq.to(torch.float32) * sc.repeat_interleave(128, dim=1)).to(torch.bfloat16).to(torch.float32)
        torch.testing.assert_close(out.to(torch.float32), want, rtol=2e-2, atol=2e-2,
                                   msg=lambda m: f"rank {rank}: dispatch/combine round trip: {m}")

        # nvidia-smi needs a moment to start: sample from the warm-up on
        sampler = ClockSampler(device.index)
        for i in range(warmup):
            line_up()
            step(dev_inputs[i % pool])
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(device_ids=[device.index])
        torch.cuda.synchronize()
        first_sample = sampler.mark()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        dstarts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        t_wall = time.perf_counter()
        for i in range(steps):
            inp = dev_inputs[i % pool]
            xq, sc, idx, w = views(inp)
            line_up()
            starts[i].record()
            a2a.dispatch(num, ox, osc, xq, sc, idx, w)
            dstarts[i].record()
            a2a.combine(out, idx, w, expert_y)
            ends[i].record()
        torch.cuda.synchronize()
        t_wall = time.perf_counter() - t_wall
        if world > 1:
            dist.barrier(device_ids=[device.index])
        torch.cuda.synchronize()
        step_us = [s.elapsed_time(e) * 1000 for s, e in zip(starts, ends)]
        disp_us = [s.elapsed_time(e) * 1000 for s, e in zip(starts, dstarts)]
        comb_us = [s.elapsed_time(e) * 1000 for s, e in zip(dstarts, ends)]

        # back-to-back (no flush, no line-up): K steps inside one event pair
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(device_ids=[device.index])
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for i in range(steps):
            step(dev_inputs[i % pool])
        b1.record()
        torch.cuda.synchronize()
        b2b_us = b0.elapsed_time(b1) * 1000 / steps
        clocks = sampler.stop(first_sample, sampler.mark())

        e2e = None
        if with_e2e:
            # One step as a caller sees it: the step's inputs start in pinned host memory (one
            # packed staging buffer: tokens, scales, expert ids, weights), go to the device, run
            # through dispatch + combine, and the whole combined tensor plus the per-expert
            # counts come back to pinned host memory. Host clock around all of it.
            sizes = [t.numel() * t.element_size() for t in host[0]]
            offs = [0]
            for n in sizes:
                offs.append(offs[-1] + (n + 255) // 256 * 256)
            packed_host = []
            for h in host:
                buf = torch.empty(offs[-1], dtype=torch.uint8).pin_memory()
                for t, o, n in zip(h, offs, sizes):
                    buf[o:o + n].copy_(t.contiguous().view(torch.uint8).reshape(-1))
                packed_host.append(buf)
            packed_dev = torch.empty(offs[-1], dtype=torch.uint8, device=device)
            d_in = tuple(packed_dev[o:o + n].view(t.dtype).view(t.shape)
                         for t, o, n in zip(host[0], offs, sizes))
            res_num = torch.empty(L, dtype=torch.int32).pin_memory()
            res_out = torch.empty((tokens, H), dtype=torch.bfloat16).pin_memory()
            h2d = offs[-1]
            d2h = res_num.numel() * 4 + res_out.numel() * 2
            xq, sc, idx, w = views(d_in)

            def eager_step(i: int) -> None:
                packed_dev.copy_(packed_host[i % pool], non_blocking=True)
                a2a.dispatch(num, ox, osc, xq, sc, idx, w)
                a2a.combine(out, idx, w, expert_y)
                res_num.copy_(num, non_blocking=True)
                res_out.copy_(out, non_blocking=True)

            def measure(run_step) -> tuple[float, float]:
                """(device-timed, host-clock) mean microseconds of one step. Device: CUDA events
                around [copy in ... copy out] on the launching stream, the ranks lined up by the
                untimed barrier just before, the host enqueuing ahead of the GPU as a serving loop
                does. Host clock: from an idle GPU to the result being readable on the host."""
                dev_us, host_us = [], []
                for i in range(warmup + steps):
                    ev0 = torch.cuda.Event(enable_timing=True)
                    ev1 = torch.cuda.Event(enable_timing=True)
                    line_up()
                    ev0.record()
                    run_step(i)
                    ev1.record()
                    torch.cuda.current_stream().synchronize()    # the result is on the host now
                    if i >= warmup:
                        dev_us.append(ev0.elapsed_time(ev1) * 1000)
                for i in range(warmup + steps):
                    line_up()
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                    run_step(i)
                    torch.cuda.current_stream().synchronize()
                    if i >= warmup:
                        host_us.append((time.perf_counter() - t0) * 1e6)
                return statistics.fmean(dev_us), statistics.fmean(host_us)

            eager_dev, eager_host = measure(eager_step)
            e2e = {"mean_us": eager_dev, "host_clock_us": eager_host, "h2d": h2d, "d2h": d2h,
                   "mode": "eager calls"}
            # The same step as a serving loop launches it: captured once per staging buffer in a
            # CUDA graph (copy in, dispatch, combine, copy out) and replayed. Epochs and cursors
            # live on the device, so a replay is a step like any other.
            # Across ranks the replay bought nothing (EP8, host clock: 209.1 us replayed against
            # 203.6 us eager) and its device-timed form has only run on one GPU: there it is off
            # unless PPLX_BENCH_GRAPH=1 asks for it, and the eager figure stands.
            if args.impl == "ours" and (world == 1 or os.environ.get("PPLX_BENCH_GRAPH") == "1"):
                try:
                    side = torch.cuda.Stream(device)
                    graphs = []
                    torch.cuda.synchronize()
                    for buf in packed_host:
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.stream(side):
                            with torch.cuda.graph(g, stream=side):
                                packed_dev.copy_(buf, non_blocking=True)
                                a2a.dispatch(num, ox, osc, xq, sc, idx, w)
                                a2a.combine(out, idx, w, expert_y)
                                res_num.copy_(num, non_blocking=True)
                                res_out.copy_(out, non_blocking=True)
                        graphs.append(g)
                    torch.cuda.synchronize()
                    graph_dev, graph_host = measure(lambda i: graphs[i % pool].replay())
                    a2a.check()
                    if world == 1:   # the replay really ran the step: its counts match the routing it was given
                        assert torch.equal(res_num.to(torch.int64),
                                           torch.bincount(all_counts_idx(idx), minlength=E)[:L].cpu())
                    e2e.update(eager_mean_us=eager_dev, eager_host_clock_us=eager_host,
                               graph_mean_us=graph_dev, graph_host_clock_us=graph_host)
                    if graph_dev < eager_dev:
                        e2e.update(mean_us=graph_dev, host_clock_us=graph_host,
                                   mode="CUDA graph replay of [copy in, dispatch, combine, copy out]")
                except Exception as exc:  # capture is an optimisation of the measurement, not a requirement
                    e2e["graph_error"] = f"{type(exc).__name__}: {exc}"[:200]

        if args.impl == "ours":
            a2a.check()
        result = {
            "mean_us": statistics.fmean(step_us), "p50_us": statistics.median(step_us),
            "dispatch_p50_us": statistics.median(disp_us), "combine_p50_us": statistics.median(comb_us),
            "b2b_us": b2b_us, "wall_s": t_wall, "clocks": clocks, "e2e": e2e,
        }
        a2a.destroy()
        return result

    def reduce_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    main_res = run_shape(args.tokens, args.steps, max(args.warmup, 3), not args.no_e2e)
    value = reduce_max(main_res["mean_us"])
    extra = {
        "p50_us_max_rank": reduce_max(main_res["p50_us"]),
        "dispatch_p50_us_max_rank": reduce_max(main_res["dispatch_p50_us"]),
        "combine_p50_us_max_rank": reduce_max(main_res["combine_p50_us"]),
        "back_to_back_us_per_step": reduce_max(main_res["b2b_us"]),
    }
    e2e_val = reduce_max(main_res["e2e"]["mean_us"]) if main_res["e2e"] else None
    e2e_host = reduce_max(main_res["e2e"]["host_clock_us"]) if main_res["e2e"] else None
    other_tokens = 4096 if args.tokens == 128 else 128
    if not args.no_prefill:
        other_steps = max(10, min(args.steps, 40)) if other_tokens > 128 else args.steps
        other = run_shape(other_tokens, other_steps, 3, False)
        extra[f"tokens{other_tokens}_step_us"] = reduce_max(other["mean_us"])
        extra[f"tokens{other_tokens}_dispatch_p50_us"] = reduce_max(other["dispatch_p50_us"])
        extra[f"tokens{other_tokens}_combine_p50_us"] = reduce_max(other["combine_p50_us"])
        pub = PUBLISHED_US.get(other_tokens)
        if pub:
            extra[f"tokens{other_tokens}_vs_published_ep8"] = extra[f"tokens{other_tokens}_step_us"] / pub

    if rank == 0:
        published = PUBLISHED_US.get(args.tokens)
        line = {
            "metric": "EP dispatch+combine latency per step (us), DeepSeek-V3 shape",
            "value": value,
            "unit": "us",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": value / 1000.0,
            "higher_is_better": False,
            "scaling": "weak",
            "vs_baseline": (value / published) if published else None,
            "dtype": "fp8_e4m3 dispatch (1x128 fp32 scales) / bf16 combine",
            "data": "synthetic",
            "impl": args.impl,
            "config": {
                "model": "DeepSeek-V3 MoE layer communication (identity expert)",
                "tokens_per_rank": args.tokens,
                "global_batch": args.tokens * world,
                "seq_len": 1,
                "hidden": args.hidden,
                "experts": args.experts,
                "topk": args.topk,
                "parallelism": f"ep{world}",
                "combine_mode": args.combine_mode,
                "l2": "flushed between timed steps (256 MiB device write, then read, before each start event)",
                "cpu_affinity": affinity,
                "line_up": "before each start event: NCCL all-reduce, then the library's device barrier (untimed)",
                "baseline_note": "vs_baseline divides by the reference's published EP8 dispatch+combine "
                                 "(113.9 us decode / 2449.1 us prefill), whatever n_gpus is",
            },
            "clocks": {k: main_res["clocks"][k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "gpu_launches": 2 * args.steps if args.impl == "ours" else 0,
            "extra": extra,
        }
        if e2e_val is not None:
            line["e2e"] = {
                "value": e2e_val,
                "unit": "us",
                "h2d_bytes_per_step": main_res["e2e"]["h2d"],
                "d2h_bytes_per_step": main_res["e2e"]["d2h"],
                "readback": "the whole combined tensor [tokens, hidden] bf16 + per-expert token counts, to pinned host memory",
                "mode": main_res["e2e"].get("mode"),
                "timing": "CUDA events around [copy in ... copy out], max over ranks of the mean; "
                          "host_clock_value is the same step by the host clock from an idle GPU",
                "host_clock_value": e2e_host,
                "eager_value": main_res["e2e"].get("eager_mean_us"),
                "eager_host_clock_value": main_res["e2e"].get("eager_host_clock_us"),
                "graph_value": main_res["e2e"].get("graph_mean_us"),
                "graph_host_clock_value": main_res["e2e"].get("graph_host_clock_us"),
                "graph_error": main_res["e2e"].get("graph_error"),
            }
        print(json.dumps(line))

    if global_group is not None:
        global_group.destroy()
    if process_group is not None:
        process_group.destroy()


if __name__ == "__main__":
    main()
