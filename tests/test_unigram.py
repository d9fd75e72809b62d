"""Unigram encoder: differential tests against HuggingFace `tokenizers` (the behaviour the
reference matches, docs/unigram.md) plus direct checks of the pieces that HF resolves
differently by design (special tokens are matched on normalised text here)."""

from __future__ import annotations

import json

import pytest

from pplx_garden import _native
from pplx_garden.unigram import Engine
from tests import unigram_data


@pytest.fixture(scope="module")
def small_vocab():
    return unigram_data.make_vocab(4000, seed=3)


@pytest.fixture(scope="module")
def pair(small_vocab):
    import tokenizers

    text = unigram_data.tokenizer_json(small_vocab)
    return Engine.from_hf_json_bytes(text), tokenizers.Tokenizer.from_str(text)


CASES = [
    "", " ", "a", "hello world", "  leading and   multiple   spaces  ", "tab\tseparated\nlines\r\nwith crlf",
    "ＦＵＬＬＷＩＤＴＨ ｔｅｘｔ", "ligature ﬁ and ﬂ", "accents: café naïve résumé", "unknown: 你好 世界 こんにちは",
    "emoji 👨‍👩‍👧‍👦 family and 🇫🇷 flag", "combining é and ǟ", "zero​width‍joiners",
    "hangul 한국어 jamo 각", "devanagari क्षत्रिय", "x" * 300, "thequickbrownfoxjumpsoverthelazydog",
    "nbsp and　ideographic space", "control \x01\x02 chars", "ｶﾀｶﾅ half width", "①②③ circled ㎏ ㍻",
]


@pytest.mark.parametrize("text", CASES)
def test_matches_huggingface_on_cases(pair, text: str) -> None:
    ours, hf = pair
    assert ours.encode(text) == hf.encode(text, add_special_tokens=False).ids


def test_matches_huggingface_on_random_text(pair) -> None:
    from hypothesis import given, settings, strategies as st

    ours, hf = pair
    alphabet = st.one_of(
        st.sampled_from(list("abcdefghijklmnopqrstuvwxyz     \t\n")),
        st.characters(min_codepoint=0x20, max_codepoint=0x2FFF, blacklist_categories=("Cs",)),
        st.sampled_from(["́", "‍", "👍", "🇩🇪", "\r\n", "ｱ", "é", "ﬃ", "한", "क्ष"]),
    )

    @settings(max_examples=400, deadline=None)
    @given(st.lists(alphabet, max_size=60).map("".join))
    def check(text: str) -> None:
        assert ours.encode(text) == hf.encode(text, add_special_tokens=False).ids, repr(text)

    check()


def test_normalizer_matches_huggingface(pair) -> None:
    ours, hf = pair
    for text in CASES:
        assert ours.normalize(text) == hf.normalizer.normalize_str(text), repr(text)


def test_grapheme_segmentation_matches_regex_module() -> None:
    import regex

    samples = CASES + ["🇫🇷🇩🇪🇯", "à́b", "\r\n\r\n", "क्‍ष", "👩🏽‍🚀", "؀a", "각ᆨ"]
    for text in samples:
        want, pos = [], 0
        for cluster in regex.findall(r"\X", text):
            pos += len(cluster.encode("utf-8"))
            want.append(pos)
        assert _native._grapheme_breaks(text) == want, repr(text)


def test_batch_equals_single_and_is_thread_safe(pair) -> None:
    ours, _ = pair
    docs = unigram_data.make_corpus(num_docs=64, chars_per_doc=500, seed=5)
    single = [ours.encode(d) for d in docs]
    for threads in (1, 2, 8):
        assert ours.encode_batch(docs, threads) == single


def test_special_tokens_split_on_normalised_text(small_vocab) -> None:
    n = len(small_vocab)
    added = [
        {"id": n, "content": "</s>", "single_word": False, "lstrip": False, "rstrip": False,
         "normalized": False, "special": True},
        {"id": n + 1, "content": "</", "single_word": False, "lstrip": False, "rstrip": False,
         "normalized": False, "special": True},
        {"id": n + 2, "content": "<mask>", "single_word": False, "lstrip": True, "rstrip": True,
         "normalized": False, "special": True},
        {"id": n + 3, "content": "<w>", "single_word": True, "lstrip": False, "rstrip": False,
         "normalized": False, "special": True},
    ]
    eng = Engine.from_hf_json_bytes(unigram_data.tokenizer_json(small_vocab, added_tokens=added))
    assert eng.vocab_size == n + 4
    ids = eng.encode("ab</s>cd")
    assert n in ids and n + 1 not in ids          # the longer token wins at the same position
    assert eng.encode("</s>") == [n]
    ids = eng.encode("ab   <mask>   cd")
    k = ids.index(n + 2)
    assert ids[:k] == eng.encode("ab") and ids[k + 1:] == eng.encode("cd")   # spaces were stripped
    assert n + 3 not in eng.encode("x<w>y") and n + 3 in eng.encode("x <w> y")
    native = eng._native
    assert native.split_special("a</s>b") == [(0, 1, None), (1, 5, n), (5, 6, None)]


def test_unknown_characters_fuse_and_legacy_metaspace(small_vocab) -> None:
    eng = Engine.from_hf_json_bytes(unigram_data.tokenizer_json(small_vocab, legacy_metaspace=True))
    unk = eng.unk_id
    ids = eng.encode("你好世界")
    assert ids.count(unk) == 1                     # four unknown characters, one UNK
    assert eng.encode("ab") == eng.encode("ab ")[: len(eng.encode("ab"))]


@pytest.mark.parametrize("mutate, message", [
    (lambda d: d["model"].__setitem__("byte_fallback", True), "byte_fallback"),
    (lambda d: d["model"].__setitem__("type", "BPE"), "not supported"),
    (lambda d: d.__setitem__("normalizer", {"type": "NFKC"}), "Precompiled"),
    (lambda d: d.__setitem__("pre_tokenizer", {"type": "WhitespaceSplit"}), "Metaspace"),
    (lambda d: d["model"].__setitem__("unk_id", 10 ** 6), "unk_id"),
    (lambda d: d["model"].__setitem__("vocab", []), "empty"),
    (lambda d: d.__setitem__("added_tokens", [{"id": 1, "content": "x", "special": False}]), "non-special"),
    (lambda d: d["decoder"].__setitem__("replacement", "_"), "mismatch"),
])
def test_rejected_configurations(small_vocab, mutate, message) -> None:
    doc = json.loads(unigram_data.tokenizer_json(small_vocab[:300]))
    mutate(doc)
    with pytest.raises(ValueError, match=message):
        Engine.from_hf_json_bytes(json.dumps(doc))


def test_malformed_json_is_reported() -> None:
    with pytest.raises(ValueError):
        Engine.from_hf_json_bytes(b'{"model": ')


def test_equal_score_paths_break_ties_like_huggingface() -> None:
    """On a 32,000-piece vocabulary with 17-digit scores some words have two segmentations whose
    scores differ only in the last bit of the running sum ('l' + 'll' against 'll' + 'l'). Which one
    wins depends on where the sum restarts (at every word) and on how the score literals were
    converted to doubles (serde_json's one-multiply conversion, not strtod): both must match."""
    tokenizers = pytest.importorskip("tokenizers")
    vocab = unigram_data.make_vocab(32000, seed=0)
    spec = unigram_data.tokenizer_json(vocab)
    docs = unigram_data.make_corpus(32, 10000, seed=0)
    engine = Engine.from_hf_json_bytes(spec)
    hf = tokenizers.Tokenizer.from_str(spec)
    want = [e.ids for e in hf.encode_batch(docs, add_special_tokens=False)]
    assert engine.encode_batch(docs, 2) == want


def test_number_literals_convert_like_serde_json() -> None:
    # integer literals are exact, short decimals are exact, and a 17-digit literal goes through
    # u64 -> double -> one division by a power of ten
    model = {"a": 1, "b": -0.5, "c": 1e3, "d": -12.143931267304547, "e": 12345678901234567890123, "f": 2.5E-3}
    text = json.dumps(model)
    got = _native._json_numbers(text) if hasattr(_native, "_json_numbers") else None
    if got is None:
        pytest.skip("number parser is not exposed")
    assert got["a"] == 1.0 and got["b"] == -0.5 and got["c"] == 1000.0 and got["f"] == 0.0025
    assert got["d"] == -(float(12143931267304547) / 1e15)
    assert got["e"] == pytest.approx(1.2345678901234568e22, rel=1e-15)


def test_flat_batch_equals_list_batch(pair) -> None:
    engine, _ = pair
    texts = ["hello world", "", "a  b   c", "ünïcödé ▁ text", "x" * 300]
    ids, offsets = engine.encode_batch_flat(texts, 2)
    lists = engine.encode_batch(texts, 2)
    assert offsets.tolist() == [0] + [sum(len(l) for l in lists[:i + 1]) for i in range(len(lists))]
    for i, want in enumerate(lists):
        assert ids[offsets[i]:offsets[i + 1]].tolist() == want


def test_word_cache_does_not_change_results(pair) -> None:
    # the same words again and again, in different neighbourhoods and beside special tokens: hits of
    # the per-thread word cache must give what a first encounter gives
    engine, hf = pair
    texts = ["the cat and the hat and the cat", "cat the", "the", " the  the", "x" * 100 + " the " + "x" * 100]
    first = [engine.encode(t) for t in texts]
    again = [engine.encode(t) for t in texts]
    assert first == again
    for t, ids in zip(texts, first):
        assert ids == hf.encode(t, add_special_tokens=False).ids
