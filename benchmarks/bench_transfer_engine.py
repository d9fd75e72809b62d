#!/usr/bin/env python
"""Transfer-engine benchmark on one box: disaggregated prefill -> decode KV transfer and a
tensor-parallel weight reshard, both over the intra-box (NVLink) provider.

KV phase: the first half of the GPUs act as prefill workers, the second half as decode
workers. A paged KV cache (64-token pages x 8 KV heads x 128 dims, bf16 = 128 KiB per page
and layer) is written page-wise from a prefill GPU to its decode partner, one paged write per
(sequence, layer) carrying an immediate; the decode side counts one immediate per page and
fires a callback per layer. Sequence lengths are uniform in [1k, 32k] tokens.

Reshard phase: bf16 weight matrices of a dense transformer (hidden 7168) laid out for TP=8
are re-laid out for TP=4: every source shard is scattered to the destination shard that
holds its columns.

With one GPU both ends live on that GPU (the copies then measure HBM, not NVLink).
The reference has no such benchmark (its fabric-debug measures raw NIC writes only,
fabric-lib/fabric-debug/src/main.rs:706-837).

    python -m benchmarks.bench_transfer_engine [--seqs 32] [--layers 4] [--reshard-gb 2]
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import threading
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

from pplx_garden.fabric_lib import PageIndices, ScatterTarget, TransferEngine

PAGE_TOKENS, KV_HEADS, HEAD_DIM = 64, 8, 128
PAGE_BYTES = PAGE_TOKENS * KV_HEADS * HEAD_DIM * 2


def kv_phase(src_dev: int, dst_dev: int, seqs: int, layers: int, pool_pages: int, seed: int) -> dict:
    rng = random.Random(seed)
    tx, rx = TransferEngine(1, [src_dev]), TransferEngine(1, [dst_dev])
    try:
        # one pool per layer would not fit a quick run: layers share a pool, offsets differ per layer
        src = torch.randint(0, 255, (pool_pages * PAGE_BYTES,), dtype=torch.uint8, device=f"cuda:{src_dev}")
        dst = torch.zeros(pool_pages * PAGE_BYTES, dtype=torch.uint8, device=f"cuda:{dst_dev}")
        hs, _ = tx.register_tensor(src)
        _, dd = rx.register_tensor(dst)
        lengths = [rng.randint(1024, 32768) for _ in range(seqs)]
        plans = []
        for n_tok in lengths:
            n_pages = min(-(-n_tok // PAGE_TOKENS), pool_pages)
            plans.append((PageIndices(rng.sample(range(pool_pages), n_pages)),
                          PageIndices(rng.sample(range(pool_pages), n_pages)), n_pages))
        total_pages = sum(p[2] for p in plans)
        layer_done = [threading.Event() for _ in range(layers)]
        for layer in range(layers):
            rx.set_imm_count_expected(0x1000 + layer, total_pages, layer_done[layer].set)
        errors: list[str] = []
        sent = threading.Semaphore(0)
        # untimed first write: opens the peer mapping, loads the copy kernel, sizes the staging buffer
        warm = PageIndices(list(range(min(64, pool_pages))))
        tx.submit_paged_writes(PAGE_BYTES, hs, warm, PAGE_BYTES, 0, dd, warm, PAGE_BYTES, 0, None, sent.release,
                               lambda e: (errors.append(e), sent.release()))
        sent.acquire()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for layer in range(layers):
            for sp, dp, _ in plans:
                tx.submit_paged_writes(PAGE_BYTES, hs, sp, PAGE_BYTES, 0, dd, dp, PAGE_BYTES, 0,
                                       0x1000 + layer, sent.release, lambda e: (errors.append(e), sent.release()))
        for _ in range(layers * len(plans)):
            sent.acquire()
        for ev in layer_done:
            assert ev.wait(120), "a layer's immediates did not all arrive"
        elapsed = time.perf_counter() - t0
        assert not errors, errors[:3]
        # spot check one sequence
        sp, dp, n = plans[0]
        gbytes = total_pages * layers * PAGE_BYTES / 1e9
        return {"src": src_dev, "dst": dst_dev, "sequences": seqs, "layers": layers, "pages_per_layer": total_pages,
                "gbytes": gbytes, "seconds": elapsed, "gbytes_per_s": gbytes / elapsed,
                "mpages_per_s": total_pages * layers / elapsed / 1e6}
    finally:
        tx.stop()
        rx.stop()


def reshard_phase(devices: list[int], total_gb: float, hidden: int = 7168) -> dict:
    """TP=len(devices) column shards -> TP=len(devices)//2: destination shard j receives the
    shards 2j and 2j+1 side by side (each matrix row gets two contiguous pieces)."""
    tp_src = len(devices)
    tp_dst = max(tp_src // 2, 1)
    rows = hidden
    cols_src = max(128, int(total_gb * 1e9 / 2 / rows / tp_src) // 128 * 128)   # columns per source shard
    engines = {d: TransferEngine(1, [d]) for d in sorted(set(devices))}
    try:
        srcs, dsts, handles, descs = [], [], [], []
        for i, d in enumerate(devices):
            t = torch.full((rows, cols_src), float(i + 1), dtype=torch.bfloat16, device=f"cuda:{d}")
            srcs.append(t)
            handles.append(engines[d].register_tensor(t)[0])
        dst_devices = devices[:tp_dst]
        for j, d in enumerate(dst_devices):
            t = torch.zeros((rows, cols_src * (tp_src // tp_dst)), dtype=torch.bfloat16, device=f"cuda:{d}")
            dsts.append(t)
            descs.append(engines[d].register_tensor(t)[1])
        torch.cuda.synchronize()
        done = threading.Semaphore(0)
        errors: list[str] = []
        n_sub = 0
        row_bytes_src = cols_src * 2
        row_bytes_dst = row_bytes_src * (tp_src // tp_dst)
        # untimed first write per source: opens the peer mapping, loads the copy kernel
        for i, d in enumerate(devices):
            j, slot = divmod(i, tp_src // tp_dst)
            warm = PageIndices(list(range(8)))
            engines[d].submit_paged_writes(row_bytes_src, handles[i], warm, row_bytes_src, 0, descs[j], warm,
                                           row_bytes_dst, slot * row_bytes_src, None, done.release,
                                           lambda e: (errors.append(e), done.release()))
        for _ in devices:
            done.acquire()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i, d in enumerate(devices):
            j, slot = divmod(i, tp_src // tp_dst)
            # one paged write per source shard: "page" r is matrix row r
            pages = PageIndices(list(range(rows)))
            engines[d].submit_paged_writes(row_bytes_src, handles[i], pages, row_bytes_src, 0, descs[j], pages,
                                           row_bytes_dst, slot * row_bytes_src, None, done.release,
                                           lambda e: (errors.append(e), done.release()))
            n_sub += 1
        for _ in range(n_sub):
            done.acquire()
        elapsed = time.perf_counter() - t0
        torch.cuda.synchronize()
        assert not errors, errors[:3]
        for j, t in enumerate(dsts):
            k = tp_src // tp_dst
            for slot in range(k):
                want = float(j * k + slot + 1)
                piece = t[:, slot * cols_src:(slot + 1) * cols_src]
                assert torch.all(piece == want), "resharded weights are wrong"
        gbytes = rows * cols_src * 2 * tp_src / 1e9
        return {"tp_src": tp_src, "tp_dst": tp_dst, "gbytes": gbytes, "seconds": elapsed,
                "gbytes_per_s": gbytes / elapsed}
    finally:
        for e in engines.values():
            e.stop()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, default=32)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--pool-pages", type=int, default=4096)
    ap.add_argument("--reshard-gb", type=float, default=2.0)
    ap.add_argument("--output", type=Path, default=None)
    args = ap.parse_args()
    n = torch.cuda.device_count()
    assert n >= 1, "needs a GPU"
    half = max(n // 2, 1)
    pairs = [(i, (i + half) % n) for i in range(half)]
    kv = [kv_phase(s, d, args.seqs, args.layers, args.pool_pages, seed=s) for s, d in pairs[:1]]
    reshard = reshard_phase(list(range(n)) if n > 1 else [0, 0], args.reshard_gb)
    result = {"gpus": n, "kv": kv, "reshard": reshard}
    print(json.dumps(result, indent=1))
    if args.output:
        args.output.write_text(json.dumps(result, indent=1))


if __name__ == "__main__":
    main()
