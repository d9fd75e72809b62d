#include "engine.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <fstream>
#include <limits>
#include <sstream>
#include <thread>

#include "json.h"
#include "unicode.h"

namespace pplx::unigram {

namespace {

constexpr double kUnkPenalty = 10.0;
constexpr double kNegInf = -std::numeric_limits<double>::infinity();

[[noreturn]] void unsupported(const std::string& what) {
  throw UnigramError(ErrorKind::kUnsupportedConfig, what);
}
[[noreturn]] void invalid(const std::string& what) {
  throw UnigramError(ErrorKind::kInvalidConfig, what);
}

const json::Value& member(const json::Value& obj, const char* key, const char* where) {
  const json::Value* v = obj.find(key);
  if (v == nullptr) invalid(std::string("missing field `") + key + "` in " + where);
  return *v;
}

bool bool_or(const json::Value& obj, const char* key, bool fallback) {
  const json::Value* v = obj.find(key);
  return (v != nullptr && v->is_bool()) ? v->as_bool() : fallback;
}

std::string type_of(const json::Value& obj) {
  const json::Value* t = obj.find("type");
  return (t != nullptr && t->is_string()) ? t->as_string() : std::string();
}

struct MetaspaceConfig {
  std::string replacement;
  bool add_prefix_space = true;
  bool split = true;   // HuggingFace's default: the pre-tokenizer cuts the text into words
};

// Reads {"type":"Metaspace","replacement":"▁","add_prefix_space":true} or the newer
// spelling with "prepend_scheme": "always" | "first" | "never".
MetaspaceConfig read_metaspace(const json::Value& v) {
  MetaspaceConfig m;
  const json::Value& rep = member(v, "replacement", "Metaspace");
  if (!rep.is_string() || rep.as_string().empty()) invalid("Metaspace.replacement must be a character");
  m.replacement = rep.as_string();
  {
    int len = 0;
    unicode::decode(reinterpret_cast<const uint8_t*>(m.replacement.data()), m.replacement.size(), 0, &len);
    if (static_cast<size_t>(len) != m.replacement.size()) invalid("Metaspace.replacement must be one character");
  }
  if (const json::Value* aps = v.find("add_prefix_space"); aps != nullptr && aps->is_bool()) {
    m.add_prefix_space = aps->as_bool();
  } else if (const json::Value* ps = v.find("prepend_scheme"); ps != nullptr && ps->is_string()) {
    m.add_prefix_space = ps->as_string() != "never";
  } else {
    invalid("Metaspace needs add_prefix_space or prepend_scheme");
  }
  if (const json::Value* sp = v.find("split"); sp != nullptr && sp->is_bool()) m.split = sp->as_bool();
  return m;
}

// Finds the step of `type` either at the top level or inside a Sequence (field `list_key`).
const json::Value* find_step(const json::Value& cfg, const char* type, const char* list_key) {
  if (!cfg.is_object()) return nullptr;
  if (type_of(cfg) == type) return &cfg;
  if (type_of(cfg) == "Sequence") {
    const json::Value* list = cfg.find(list_key);
    if (list != nullptr && list->is_array()) {
      for (const json::Value& step : list->as_array()) {
        if (step.is_object() && type_of(step) == type) return &step;
      }
    }
  }
  return nullptr;
}

// ---- helpers on valid UTF-8 ----

inline size_t next_char_boundary(const uint8_t* s, size_t n, size_t from) {
  size_t nxt = from + 1;
  while (nxt < n && (s[nxt] & 0xC0) == 0x80) ++nxt;
  return nxt;
}

bool is_word_char(uint32_t cp) { return cp == '_' || unicode::is_alphanumeric(cp); }

}  // namespace

// ---------------------------------------------------------------------------
// special tokens
// ---------------------------------------------------------------------------

SpecialTokenMatcher::SpecialTokenMatcher(std::vector<SpecialToken> tokens) : tokens_(std::move(tokens)) {
  std::stable_sort(tokens_.begin(), tokens_.end(), [](const SpecialToken& l, const SpecialToken& r) {
    if (l.content.size() != r.content.size()) return l.content.size() > r.content.size();
    return l.id < r.id;
  });
}

void SpecialTokenMatcher::split(std::string_view text, std::vector<Segment>* out) const {
  out->clear();
  if (text.empty()) return;
  if (tokens_.empty()) {
    out->push_back(Segment{0, text.size(), false, 0});
    return;
  }
  const uint8_t* s = reinterpret_cast<const uint8_t*>(text.data());
  const size_t n = text.size();
  size_t cursor = 0;
  while (cursor < n) {
    bool have = false;
    size_t best_start = 0, best_end = 0, best_len = 0;
    TokenId best_id = 0;
    for (const SpecialToken& tok : tokens_) {
      if (tok.content.empty()) continue;
      const size_t found = text.find(tok.content, cursor);
      if (found == std::string_view::npos) continue;
      size_t start = found;
      size_t end = found + tok.content.size();
      if (tok.single_word) {
        int len = 0;
        const bool left_ok = start == 0 || !is_word_char(unicode::decode_before(s, start, &len));
        const bool right_ok = end == n || !is_word_char(unicode::decode(s, n, end, &len));
        if (!(left_ok && right_ok)) continue;
      }
      if (tok.lstrip) {
        while (start > 0) {
          int len = 0;
          const uint32_t cp = unicode::decode_before(s, start, &len);
          if (!unicode::is_white_space(cp)) break;
          start -= static_cast<size_t>(len);
        }
        start = std::max(start, cursor);
      }
      if (tok.rstrip) {
        while (end < n) {
          int len = 0;
          const uint32_t cp = unicode::decode(s, n, end, &len);
          if (!unicode::is_white_space(cp)) break;
          end += static_cast<size_t>(len);
        }
      }
      // earliest start wins; on a tie the longer content (tokens_ is sorted that way,
      // so the first candidate at a given start is kept)
      if (!have || start < best_start || (start == best_start && tok.content.size() > best_len)) {
        have = true;
        best_start = start;
        best_end = end;
        best_len = tok.content.size();
        best_id = tok.id;
      }
    }
    if (!have) {
      out->push_back(Segment{cursor, n, false, 0});
      break;
    }
    if (cursor < best_start) out->push_back(Segment{cursor, best_start, false, 0});
    out->push_back(Segment{best_start, best_end, true, best_id});
    cursor = best_end;
  }
}

// ---------------------------------------------------------------------------
// loading
// ---------------------------------------------------------------------------

std::shared_ptr<Engine> Engine::from_hf_json_path(const std::string& path) {
  std::ifstream in(path, std::ios::binary);
  if (!in) throw UnigramError(ErrorKind::kIo, "cannot open " + path);
  std::ostringstream buf;
  buf << in.rdbuf();
  return from_hf_json_bytes(buf.str());
}

std::shared_ptr<Engine> Engine::from_hf_json_bytes(std::string_view bytes) {
  json::Value root;
  try {
    root = json::parse(bytes);
  } catch (const std::exception& e) {
    invalid(e.what());
  }
  if (!root.is_object()) invalid("tokenizer.json must hold an object");
  std::shared_ptr<Engine> eng(new Engine());

  // normaliser: a Precompiled charsmap, alone or inside a Sequence
  const json::Value* pre = find_step(member(root, "normalizer", "tokenizer.json"), "Precompiled", "normalizers");
  if (pre == nullptr) unsupported("normalizer must include a Precompiled charsmap step");
  const json::Value& charsmap = member(*pre, "precompiled_charsmap", "Precompiled");
  if (!charsmap.is_string()) invalid("precompiled_charsmap must be a base64 string");
  try {
    eng->normalizer_ = PrecompiledNormalizer::from_base64(charsmap.as_string());
  } catch (const std::exception& e) {
    invalid(e.what());
  }

  // Metaspace in the pre-tokenizer and in the decoder must agree
  const json::Value* ms = find_step(member(root, "pre_tokenizer", "tokenizer.json"), "Metaspace", "pretokenizers");
  if (ms == nullptr) unsupported("pre_tokenizer must include a Metaspace step");
  const MetaspaceConfig pre_ms = read_metaspace(*ms);
  const json::Value& decoder = member(root, "decoder", "tokenizer.json");
  const json::Value* dec = find_step(decoder, "Metaspace", "decoders");
  if (dec == nullptr) unsupported("decoder must be Metaspace");
  const MetaspaceConfig dec_ms = read_metaspace(*dec);
  if (pre_ms.replacement != dec_ms.replacement) unsupported("metaspace replacement mismatch");
  if (pre_ms.add_prefix_space != dec_ms.add_prefix_space) unsupported("metaspace add_prefix_space mismatch");
  eng->replacement_ = pre_ms.replacement;
  eng->add_prefix_space_ = pre_ms.add_prefix_space;
  eng->split_words_ = pre_ms.split;

  // model
  const json::Value& model = member(root, "model", "tokenizer.json");
  if (const json::Value* ty = model.find("type"); ty != nullptr && ty->is_string() && ty->as_string() != "Unigram") {
    unsupported("model type \"" + ty->as_string() + "\" is not supported (only Unigram)");
  }
  if (bool_or(model, "byte_fallback", false)) unsupported("byte_fallback unigram models are not supported");
  const json::Value& unk = member(model, "unk_id", "model");
  if (!unk.is_number()) invalid("model.unk_id must be a number");
  const json::Value& vocab = member(model, "vocab", "model");
  if (!vocab.is_array() || vocab.as_array().empty()) invalid("unigram vocab cannot be empty");
  std::vector<std::string> pieces;
  std::vector<double> scores;
  pieces.reserve(vocab.as_array().size());
  scores.reserve(vocab.as_array().size());
  double min_score = std::numeric_limits<double>::infinity();
  for (const json::Value& entry : vocab.as_array()) {
    if (!entry.is_array() || entry.as_array().size() != 2 || !entry.as_array()[0].is_string() ||
        !entry.as_array()[1].is_number()) {
      invalid("vocab entries must be [piece, score] pairs");
    }
    pieces.push_back(entry.as_array()[0].as_string());
    scores.push_back(entry.as_array()[1].as_number());
    min_score = std::min(min_score, scores.back());
  }
  if (unk.as_number() < 0 || static_cast<size_t>(unk.as_number()) >= pieces.size()) invalid("unk_id out of range");
  eng->unk_id_ = static_cast<TokenId>(unk.as_number());
  eng->unk_score_ = min_score - kUnkPenalty;

  // added tokens: only special ones are understood
  std::vector<SpecialToken> specials;
  size_t total = pieces.size();
  if (const json::Value* added = root.find("added_tokens"); added != nullptr && added->is_array()) {
    for (const json::Value& t : added->as_array()) {
      if (!t.is_object()) invalid("added_tokens entries must be objects");
      if (!bool_or(t, "special", false)) unsupported("non-special added tokens are not supported");
      SpecialToken s;
      const json::Value& id = member(t, "id", "added_tokens");
      const json::Value& content = member(t, "content", "added_tokens");
      if (!id.is_number() || !content.is_string()) invalid("added token needs a numeric id and a string content");
      s.id = static_cast<TokenId>(id.as_number());
      s.content = content.as_string();
      s.single_word = bool_or(t, "single_word", false);
      s.lstrip = bool_or(t, "lstrip", false);
      s.rstrip = bool_or(t, "rstrip", false);
      total = std::max(total, static_cast<size_t>(s.id) + 1);
      specials.push_back(std::move(s));
    }
  }
  eng->special_ = SpecialTokenMatcher(std::move(specials));
  eng->vocab_size_ = total;

  try {
    eng->trie_ = VocabTrie::build(pieces, scores);
  } catch (const std::exception& e) {
    invalid(e.what());
  }
  return eng;
}

// ---------------------------------------------------------------------------
// encoding
// ---------------------------------------------------------------------------

void Engine::encode(std::string_view text, EncodeState* st) const {
  st->tokens.clear();
  normalizer_.normalize_into(text, &st->normalized);
  special_.split(st->normalized, &st->segments);
  for (const Segment& seg : st->segments) {
    if (seg.special) {
      st->tokens.push_back(seg.special_id);
    } else if (seg.end > seg.start) {
      encode_segment(std::string_view(st->normalized).substr(seg.start, seg.end - seg.start), st);
    }
  }
}

void Engine::encode_segment(std::string_view text, EncodeState* st) const {
  // Metaspace: optional prefix, every space becomes the replacement character.
  std::string& prep = st->prep;
  prep.clear();
  if (text.empty()) return;
  if (add_prefix_space_ && text.front() != ' ') prep.append(replacement_);
  size_t run = 0;
  while (run < text.size()) {
    const void* hit = std::memchr(text.data() + run, ' ', text.size() - run);
    if (hit == nullptr) break;
    const size_t i = static_cast<size_t>(static_cast<const char*>(hit) - text.data());
    prep.append(text.data() + run, i - run);
    prep.append(replacement_);
    run = i + 1;
  }
  prep.append(text.data() + run, text.size() - run);

  const size_t n = prep.size();
  if (st->best_score.size() < n + 1) {
    st->best_score.resize(n + 1);
    st->best_start.resize(n + 1);
    st->best_id.resize(n + 1);
  }
  if (n == 0) return;
  const uint8_t* bytes = reinterpret_cast<const uint8_t*>(prep.data());
  if (!split_words_) {
    viterbi(bytes, n, st);
    return;
  }
  // One Viterbi pass per word, a word starting at each replacement character: what the model
  // sees behind HuggingFace's Metaspace pre-tokenizer. The best path of the whole text is the
  // concatenation of the words' best paths except where two paths tie, and there the rounding
  // of the running sum decides; sums that restart at every word round as the original's do.
  // (The reference runs one pass over the whole segment: pplx-unigram/src/engine.rs:88-165.)
  const size_t rl = replacement_.size();
  if (st->words_owner != this) {   // a state that served another engine starts over
    st->words = WordCache();
    st->words_owner = this;
  }
  auto encode_word = [&](size_t begin, size_t len) {
    if (len > WordCache::kMaxWordBytes) {
      viterbi(bytes + begin, len, st);
      return;
    }
    const uint64_t h = WordCache::hash_bytes(bytes + begin, len);
    if (const WordCache::Entry* hit = st->words.find(bytes + begin, len, h)) {
      const TokenId* t = st->words.tokens_of(*hit);
      st->tokens.insert(st->tokens.end(), t, t + hit->num_tokens);
      return;
    }
    const size_t first = st->tokens.size();
    viterbi(bytes + begin, len, st);
    st->words.insert(bytes + begin, len, h, st->tokens.data() + first, st->tokens.size() - first);
  };
  size_t word = 0;
  if (rl > 0) {
    // jump from one candidate first byte of the replacement character to the next
    const uint8_t first = static_cast<uint8_t>(replacement_[0]);
    size_t i = 1;
    while (i + rl <= n) {
      const void* hit = std::memchr(bytes + i, first, n - rl + 1 - i);
      if (hit == nullptr) break;
      i = static_cast<size_t>(static_cast<const uint8_t*>(hit) - bytes);
      if (std::memcmp(bytes + i, replacement_.data(), rl) == 0) {
        encode_word(word, i - word);
        word = i;
        i += rl;
      } else {
        ++i;
      }
    }
  }
  encode_word(word, n - word);
}

void Engine::viterbi(const uint8_t* prep, size_t n, EncodeState* st) const {
  double* best_score = st->best_score.data();
  uint32_t* best_start = st->best_start.data();
  TokenId* best_id = st->best_id.data();
  std::fill(best_score, best_score + n + 1, kNegInf);
  best_score[0] = 0.0;
  const TrieNode* nodes = trie_.nodes();

  for (size_t pos = 0; pos < n; ++pos) {
    if ((prep[pos] & 0xC0) == 0x80) continue;  // inside a code point
    const double s0 = best_score[pos];
    if (s0 == kNegInf) continue;
    const size_t char_end = next_char_boundary(prep, n, pos);
    bool single_char_piece = false;
    const TrieNode* node = &nodes[0];
    for (size_t end = pos; end < n; ++end) {
      const uint8_t b = prep[end];
      if (!node->has_child(b)) break;
      node = &nodes[node->child_index(b)];
      if (node->token_id >= 0) {
        const size_t ep = end + 1;
        const double total = s0 + node->score;
        if (total > best_score[ep]) {
          best_score[ep] = total;
          best_start[ep] = static_cast<uint32_t>(pos);
          best_id[ep] = static_cast<TokenId>(node->token_id);
        }
        if (ep == char_end) single_char_piece = true;
      }
    }
    if (!single_char_piece) {
      const double total = s0 + unk_score_;
      if (total > best_score[char_end]) {
        best_score[char_end] = total;
        best_start[char_end] = static_cast<uint32_t>(pos);
        best_id[char_end] = unk_id_;
      }
    }
  }

  st->backtrack.clear();
  size_t end = n;
  while (end > 0) {
    if (best_score[end] == kNegInf) throw UnigramError(ErrorKind::kEncodeFailed, "backtrack failed");
    st->backtrack.push_back(best_id[end]);
    end = best_start[end];
  }
  const size_t first = st->tokens.size();
  for (size_t i = st->backtrack.size(); i-- > 0;) {
    const TokenId id = st->backtrack[i];
    // consecutive unknowns inside one segment collapse into one
    if (id == unk_id_ && st->tokens.size() > first && st->tokens.back() == unk_id_) continue;
    st->tokens.push_back(id);
  }
}

std::vector<std::vector<TokenId>> Engine::encode_batch(const std::vector<std::string_view>& texts,
                                                       int num_threads) const {
  std::vector<std::vector<TokenId>> out(texts.size());
  if (texts.empty()) return out;
  int threads = num_threads > 0 ? num_threads : static_cast<int>(std::thread::hardware_concurrency());
  threads = std::max(1, std::min<int>(threads, static_cast<int>(texts.size())));
  std::atomic<size_t> next{0};
  std::atomic<bool> failed{false};
  std::string failure;
  auto work = [&] {
    EncodeState st;
    try {
      for (;;) {
        const size_t i = next.fetch_add(1, std::memory_order_relaxed);
        if (i >= texts.size() || failed.load(std::memory_order_relaxed)) break;
        encode(texts[i], &st);
        out[i] = st.tokens;
      }
    } catch (const std::exception& e) {
      if (!failed.exchange(true)) failure = e.what();
    }
  };
  if (threads == 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    pool.reserve(static_cast<size_t>(threads));
    for (int t = 0; t < threads; ++t) pool.emplace_back(work);
    for (std::thread& t : pool) t.join();
  }
  if (failed.load()) throw UnigramError(ErrorKind::kEncodeFailed, failure);
  return out;
}

}  // namespace pplx::unigram
