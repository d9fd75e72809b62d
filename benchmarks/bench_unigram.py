#!/usr/bin/env python
"""Unigram encode throughput (MB/s) at 1 and N threads, with HuggingFace `tokenizers` on
the same vocabulary and corpus as the CPU baseline.

Workload: 32,000-piece vocabulary (256 byte pieces + generated pieces, Zipf(1.1) scores),
1,024 documents of ~10,000 characters of Zipf-distributed random words.
The reference only ships a one-string timing loop (pplx-unigram/examples/encode.rs:48-57).

    python -m benchmarks.bench_unigram [--docs 1024] [--threads N] [--output out.json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--docs", type=int, default=1024)
    ap.add_argument("--chars", type=int, default=10000)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--threads", type=int, default=os.cpu_count() or 1)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--output", type=Path, default=None)
    args = ap.parse_args()

    from pplx_garden.unigram import Engine
    from tests import unigram_data

    vocab = unigram_data.make_vocab(args.vocab, seed=0)
    spec = unigram_data.tokenizer_json(vocab)
    docs = unigram_data.make_corpus(args.docs, args.chars, seed=0)
    total_mb = sum(len(d.encode()) for d in docs) / 1e6

    t0 = time.perf_counter()
    engine = Engine.from_hf_json_bytes(spec)
    load_s = time.perf_counter() - t0

    def best(fn) -> float:
        times = []
        for _ in range(args.repeats):
            t = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t)
        return min(times)

    ours_1 = total_mb / best(lambda: engine.encode_batch_flat(docs, 1))
    ours_n = total_mb / best(lambda: engine.encode_batch_flat(docs, args.threads))
    lists_n = total_mb / best(lambda: engine.encode_batch(docs, args.threads))
    result = {
        "corpus_mb": total_mb, "docs": len(docs), "vocab": len(vocab), "load_s": load_s,
        "ours_mb_s_1_thread": ours_1, f"ours_mb_s_{args.threads}_threads": ours_n,
        f"ours_mb_s_{args.threads}_threads_python_lists": lists_n,
    }
    try:
        import tokenizers

        hf = tokenizers.Tokenizer.from_str(spec)
        sample = docs[: max(8, len(docs) // 16)]
        assert [e.ids for e in hf.encode_batch(sample, add_special_tokens=False)] == \
            engine.encode_batch(sample, args.threads), "outputs differ from HuggingFace tokenizers"
        os.environ["TOKENIZERS_PARALLELISM"] = "false"
        os.environ["RAYON_NUM_THREADS"] = "1"
        hf_1 = total_mb / best(lambda: [hf.encode(d, add_special_tokens=False) for d in docs])
        os.environ["TOKENIZERS_PARALLELISM"] = "true"
        os.environ.pop("RAYON_NUM_THREADS", None)
        hf_n = total_mb / best(lambda: hf.encode_batch(docs, add_special_tokens=False))
        result.update(hf_mb_s_1_thread=hf_1, hf_mb_s_all_threads=hf_n,
                      speedup_1_thread=ours_1 / hf_1, speedup_threads=ours_n / hf_n,
                      verified_against_hf=True)
    except ImportError:
        result["verified_against_hf"] = False
    print(json.dumps(result, indent=1))
    if args.output:
        args.output.write_text(json.dumps(result, indent=1))


if __name__ == "__main__":
    main()
