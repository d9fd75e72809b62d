"""Synthetic Unigram tokenizer and corpus for tests and benchmarks.

Vocabulary: 256 byte pieces ``<0xNN>`` + generated pieces ('▁'-prefixed with probability
0.5, 1-12 lowercase letters) with Zipf(1.1) log-probabilities; corpus: documents of random
words drawn Zipf(1.1) from a lexicon. The normaliser uses the ``nmt_nfkc`` precompiled
charsmap that the installed ``sentencepiece`` package compiles in (obtained by training a
throw-away model), so no file has to be downloaded.
"""

from __future__ import annotations

import functools
import json
import math
import os
import random
import tempfile


@functools.lru_cache(maxsize=1)
def nmt_nfkc_charsmap() -> bytes:
    import sentencepiece as spm
    from sentencepiece import sentencepiece_model_pb2 as pb

    with tempfile.TemporaryDirectory() as tmp:
        corpus = os.path.join(tmp, "corpus.txt")
        with open(corpus, "w") as f:
            rng = random.Random(0)
            for _ in range(400):
                f.write(" ".join("".join(rng.choice("abcdefghij") for _ in range(rng.randint(1, 6)))
                                 for _ in range(12)) + "\n")
        prefix = os.path.join(tmp, "m")
        spm.SentencePieceTrainer.train(input=corpus, model_prefix=prefix, vocab_size=30, hard_vocab_limit=False,
                                       model_type="unigram", normalization_rule_name="nmt_nfkc",
                                       minloglevel=2)
        proto = pb.ModelProto()
        with open(prefix + ".model", "rb") as f:
            proto.ParseFromString(f.read())
        return bytes(proto.normalizer_spec.precompiled_charsmap)


def make_vocab(size: int = 32000, seed: int = 0) -> list[tuple[str, float]]:
    rng = random.Random(seed)
    pieces: list[str] = [f"<0x{i:02X}>" for i in range(256)]
    seen = set(pieces)
    # single characters and the bare metaspace first, so that plain ASCII never needs UNK
    for ch in "▁abcdefghijklmnopqrstuvwxyz":
        if ch not in seen:
            pieces.append(ch)
            seen.add(ch)
    while len(pieces) < size:
        body = "".join(rng.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rng.randint(1, 12)))
        piece = ("▁" + body) if rng.random() < 0.5 else body
        if piece not in seen:
            seen.add(piece)
            pieces.append(piece)
    # Zipf(1.1) over a random rank order, normalised to log-probabilities
    ranks = list(range(1, size + 1))
    rng.shuffle(ranks)
    weights = [r ** -1.1 for r in ranks]
    total = math.fsum(weights)
    return [(p, math.log(w / total)) for p, w in zip(pieces, weights)]


def tokenizer_json(vocab: list[tuple[str, float]], *, unk_id: int = 0,
                   added_tokens: list[dict] | None = None, legacy_metaspace: bool = False) -> str:
    import base64

    metaspace = {"type": "Metaspace", "replacement": "▁", "prepend_scheme": "always", "split": True}
    if legacy_metaspace:
        metaspace = {"type": "Metaspace", "replacement": "▁", "add_prefix_space": True}
    doc = {
        "version": "1.0",
        "truncation": None,
        "padding": None,
        "added_tokens": added_tokens or [],
        "normalizer": {
            "type": "Sequence",
            "normalizers": [
                {"type": "Precompiled",
                 "precompiled_charsmap": base64.b64encode(nmt_nfkc_charsmap()).decode("ascii")},
                {"type": "Replace", "pattern": {"Regex": " {2,}"}, "content": " "},
            ],
        },
        "pre_tokenizer": metaspace,
        "post_processor": None,
        "decoder": metaspace,
        "model": {"type": "Unigram", "unk_id": unk_id, "vocab": [[p, s] for p, s in vocab],
                  "byte_fallback": False},
    }
    return json.dumps(doc, ensure_ascii=False)


def make_corpus(num_docs: int = 1024, chars_per_doc: int = 10000, seed: int = 0,
                lexicon_size: int = 50000) -> list[str]:
    rng = random.Random(seed + 1)
    lexicon = ["".join(rng.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rng.randint(2, 10)))
               for _ in range(lexicon_size)]
    weights = [(i + 1) ** -1.1 for i in range(lexicon_size)]
    docs = []
    for _ in range(num_docs):
        words = rng.choices(lexicon, weights=weights, k=chars_per_doc // 6)
        text = " ".join(words)
        docs.append(text[:chars_per_doc])
    return docs
