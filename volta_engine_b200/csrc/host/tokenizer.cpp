// Byte-level BPE tokenizer (Qwen / GLM / DeepSeek / GPT-2 families) with special tokens, a word cache and
// byte-exact decode. Loads Hugging Face `tokenizer.json` or `vocab.json` + `merges.txt`.
// Behavioural counterpart of the reference tokenizer (inc/engine/loader/tokenizer.h:11-88,
// src/loader/tokenizer.cpp): pre-tokenisation follows the published split patterns of those families,
// implemented as a hand-written scanner over code points instead of a regex engine.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <mutex>
#include <queue>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "json.h"

namespace vh {

enum PretokMode { kQwen = 0, kGpt2 = 1, kLlama3 = 2, kDeepseek = 3, kSpm = 4 };

static uint32_t next_cp(const std::string& s, size_t& i) {
  unsigned char c = (unsigned char)s[i];
  if (c < 0x80) { ++i; return c; }
  const int n = (c >> 5) == 6 ? 1 : (c >> 4) == 14 ? 2 : (c >> 3) == 30 ? 3 : 0;
  if (n == 0 || i + (size_t)n >= s.size()) { ++i; return 0xFFFD; }   // stray or truncated sequence: one byte
  uint32_t cp = c & (0xFF >> (n + 2));
  for (int k = 1; k <= n; ++k) {
    unsigned char cc = (unsigned char)s[i + k];
    if ((cc & 0xC0) != 0x80) { ++i; return 0xFFFD; }
    cp = (cp << 6) | (cc & 0x3F);
  }
  i += n + 1;
  return cp;
}
static void put_cp(uint32_t cp, std::string& out) {
  if (cp < 0x80) out.push_back((char)cp);
  else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) {
    out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back((char)(0x80 | (cp & 0x3F)));
  } else {
    out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
    out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F)));
  }
}

static bool is_space(uint32_t c) {
  return c == ' ' || (c >= 9 && c <= 13) || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
         c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
static bool is_digit(uint32_t c) {
  return (c >= '0' && c <= '9') || (c >= 0x660 && c <= 0x669) || (c >= 0x6F0 && c <= 0x6F9) ||
         (c >= 0x966 && c <= 0x96F) || (c >= 0xFF10 && c <= 0xFF19) || c == 0xB2 || c == 0xB3 || c == 0xB9 ||
         (c >= 0xBC && c <= 0xBE) || (c >= 0x2070 && c <= 0x2079) || (c >= 0x2080 && c <= 0x2089) ||
         (c >= 0x2150 && c <= 0x218B) || (c >= 0x2460 && c <= 0x249B);
}
static bool is_letter(uint32_t c) {
  if (c < 0x80) return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z');
  if (c == 0xAA || c == 0xB5 || c == 0xBA) return true;
  if (c < 0xC0) return false;
  if (c == 0xD7 || c == 0xF7) return false;
  if (is_space(c) || is_digit(c)) return false;
  if (c >= 0x2000 && c <= 0x2BFF) return false;   // punctuation, symbols, arrows, math, box drawing
  if (c >= 0x3000 && c <= 0x303F) return false;   // CJK punctuation
  if (c >= 0xFE10 && c <= 0xFE6F) return false;
  if (c >= 0xFF00 && c <= 0xFF0F) return false;
  if (c >= 0xFF1A && c <= 0xFF20) return false;
  if (c >= 0xFF3B && c <= 0xFF40) return false;
  if (c >= 0xFF5B && c <= 0xFF65) return false;
  if (c >= 0x1F000 && c <= 0x1FAFF) return false;  // emoji and pictographs
  if (c >= 0xE000 && c <= 0xF8FF) return false;    // private use
  if (c >= 0x300 && c <= 0x36F) return false;      // combining marks
  return true;
}

// Splits `text` into pre-tokens according to the family's pattern.
static void pretokenize(const std::string& text, int mode, std::vector<std::string>& out) {
  std::vector<uint32_t> cps;
  std::vector<size_t> offs;
  for (size_t i = 0; i < text.size();) {
    offs.push_back(i);
    cps.push_back(next_cp(text, i));
  }
  offs.push_back(text.size());
  const size_t n = cps.size();
  auto emit = [&](size_t a, size_t b) { if (b > a) out.emplace_back(text.substr(offs[a], offs[b] - offs[a])); };
  auto lower = [](uint32_t c) { return c >= 'A' && c <= 'Z' ? c + 32 : c; };
  const int max_digits = (mode == kQwen) ? 1 : (mode == kGpt2 ? 1 << 30 : 3);
  size_t i = 0;
  while (i < n) {
    uint32_t c = cps[i];
    // contractions
    if (c == '\'' && i + 1 < n) {
      uint32_t d = mode == kGpt2 ? cps[i + 1] : lower(cps[i + 1]);
      if (d == 's' || d == 't' || d == 'm' || d == 'd') { emit(i, i + 2); i += 2; continue; }
      if (i + 2 < n) {
        uint32_t e = mode == kGpt2 ? cps[i + 2] : lower(cps[i + 2]);
        if ((d == 'r' && e == 'e') || (d == 'v' && e == 'e') || (d == 'l' && e == 'l')) { emit(i, i + 3); i += 3; continue; }
      }
    }
    // [^\r\n\p{L}\p{N}]?\p{L}+   (GPT-2: " ?\p{L}+")
    {
      size_t j = i;
      bool prefix_ok = mode == kGpt2 ? (c == ' ') : (c != '\r' && c != '\n' && !is_letter(c) && !is_digit(c));
      if (prefix_ok && j + 1 < n && is_letter(cps[j + 1])) ++j;
      if (is_letter(cps[j])) {
        size_t k = j;
        while (k < n && is_letter(cps[k])) ++k;
        emit(i, k);
        i = k;
        continue;
      }
    }
    // numbers
    if (is_digit(c) || (mode == kGpt2 && c == ' ' && i + 1 < n && is_digit(cps[i + 1]))) {
      size_t k = i + (is_digit(c) ? 0 : 1);
      int cnt = 0;
      while (k < n && is_digit(cps[k]) && cnt < max_digits) { ++k; ++cnt; }
      emit(i, k);
      i = k;
      continue;
    }
    //  ?[^\s\p{L}\p{N}]+[\r\n]*
    {
      size_t j = i;
      if (c == ' ' && j + 1 < n) ++j;
      auto is_punct = [&](uint32_t x) { return !is_space(x) && !is_letter(x) && !is_digit(x); };
      if (is_punct(cps[j])) {
        size_t k = j;
        while (k < n && is_punct(cps[k])) ++k;
        if (mode != kGpt2) while (k < n && (cps[k] == '\r' || cps[k] == '\n')) ++k;
        emit(i, k);
        i = k;
        continue;
      }
    }
    // whitespace: \s*[\r\n]+ | \s+(?!\S) | \s+
    if (is_space(c)) {
      size_t k = i;
      while (k < n && is_space(cps[k])) ++k;
      if (mode != kGpt2) {
        size_t last_nl = (size_t)-1;
        for (size_t q = i; q < k; ++q) if (cps[q] == '\r' || cps[q] == '\n') last_nl = q;
        if (last_nl != (size_t)-1) { emit(i, last_nl + 1); i = last_nl + 1; continue; }
      }
      if (k < n && k - i > 1) { emit(i, k - 1); i = k - 1; continue; }   // \s+(?!\S): leave one space for the word
      if (k < n && k - i == 1 && c == ' ' ) {
        // single space before a non-space: it attaches as the optional prefix handled above; reaching here
        // means the next char cannot take a prefix (e.g. digit in non-GPT2 modes)
        emit(i, k); i = k; continue;
      }
      emit(i, k);
      i = k;
      continue;
    }
    emit(i, i + 1);
    ++i;
  }
}

struct PairHash {
  size_t operator()(const std::pair<int, int>& p) const { return ((size_t)p.first << 32) ^ (size_t)(uint32_t)p.second; }
};

class Tokenizer {
 public:
  std::vector<std::string> id_to_bytes;                    // raw bytes of every token
  std::unordered_map<std::string, int> piece_to_id;        // byte-unicode piece -> id
  std::unordered_map<std::pair<int, int>, int, PairHash> merge_rank;   // (id, id) -> rank
  std::unordered_map<std::pair<int, int>, int, PairHash> merge_to;     // (id, id) -> merged id
  std::vector<std::pair<std::string, int>> specials;       // sorted by length desc
  std::vector<char> is_special;
  int byte_id[256];
  int mode = kQwen;
  std::string byte_enc[256];                               // byte -> utf8 of its stand-in code point
  std::unordered_map<uint32_t, int> cp_to_byte;
  std::unordered_map<std::string, std::vector<int>> cache;
  std::mutex mu;

  Tokenizer() {
    // GPT-2 bytes <-> printable code points
    std::vector<int> bs;
    for (int b = '!'; b <= '~'; ++b) bs.push_back(b);
    for (int b = 0xA1; b <= 0xAC; ++b) bs.push_back(b);
    for (int b = 0xAE; b <= 0xFF; ++b) bs.push_back(b);
    std::vector<int> cs(bs.begin(), bs.end());
    int extra = 0;
    for (int b = 0; b < 256; ++b)
      if (std::find(bs.begin(), bs.end(), b) == bs.end()) { bs.push_back(b); cs.push_back(256 + extra++); }
    for (size_t k = 0; k < bs.size(); ++k) {
      std::string u;
      put_cp((uint32_t)cs[k], u);
      byte_enc[bs[k]] = u;
      cp_to_byte[(uint32_t)cs[k]] = bs[k];
    }
    for (int b = 0; b < 256; ++b) byte_id[b] = -1;
  }

  // SentencePiece-style vocabularies (Gemma): pieces are plain UTF-8 with U+2581 standing for a space, bytes that have no
  // piece are spelled <0xNN>, merges run over the whole text between special tokens (no pre-token split), ranked by the
  // merge list or, when the file carries scores instead, by the score of the merged piece.
  std::vector<float> scores;                               // per id; empty when merges are ranked by the list
  int spm_byte_id[256];
  int unk_id = -1;

  std::string piece_to_bytes(const std::string& piece) const {
    std::string out;
    if (mode == kSpm) {
      unsigned v = 0;
      if (piece.size() == 6 && piece.compare(0, 3, "<0x") == 0 && piece[5] == '>' && sscanf(piece.c_str() + 3, "%2x", &v) == 1) {
        out.push_back((char)v);
        return out;
      }
      for (size_t i = 0; i < piece.size();) {
        if (piece.compare(i, 3, "\xE2\x96\x81") == 0) { out.push_back(' '); i += 3; }
        else out.push_back(piece[i++]);
      }
      return out;
    }
    for (size_t i = 0; i < piece.size();) {
      uint32_t cp = next_cp(piece, i);
      auto it = cp_to_byte.find(cp);
      if (it != cp_to_byte.end()) out.push_back((char)it->second);
      else put_cp(cp, out);
    }
    return out;
  }

  void add_piece(const std::string& piece, int id, bool special) {
    if (id < 0) return;
    if ((size_t)id >= id_to_bytes.size()) { id_to_bytes.resize(id + 1); is_special.resize(id + 1, 0); }
    if (special) {
      id_to_bytes[id] = piece;
      is_special[id] = 1;
      specials.emplace_back(piece, id);
    } else {
      piece_to_id[piece] = id;
      id_to_bytes[id] = piece_to_bytes(piece);
      if (mode == kSpm) {
        if ((size_t)id >= id_to_piece.size()) id_to_piece.resize(id + 1);
        id_to_piece[id] = piece;
        raw_to_id[piece] = id;
      }
    }
  }

  void finish() {
    std::sort(specials.begin(), specials.end(),
              [](const auto& a, const auto& b) { return a.first.size() > b.first.size(); });
    for (int b = 0; b < 256; ++b) {
      auto it = piece_to_id.find(byte_enc[b]);
      byte_id[b] = it == piece_to_id.end() ? -1 : it->second;
      char name[8];
      snprintf(name, sizeof(name), "<0x%02X>", b);
      auto jt = piece_to_id.find(name);
      spm_byte_id[b] = jt == piece_to_id.end() ? -1 : jt->second;
    }
    auto u = piece_to_id.find("<unk>");
    if (u != piece_to_id.end()) unk_id = u->second;
  }

  // Whole-text BPE for the SentencePiece mode: linked list of symbols + a heap of candidate merges (lazy invalidation),
  // O(n log n) instead of the per-word quadratic loop.
  void bpe_spm(const std::string& text, std::vector<int>& out) {
    std::string norm;
    norm.reserve(text.size() + 8);
    for (char c : text) {
      if (c == ' ') norm += "\xE2\x96\x81";
      else norm.push_back(c);
    }
    struct Sym { int id; int prev, next; bool alive; };
    std::vector<Sym> sy;
    for (size_t i = 0; i < norm.size();) {
      const size_t a = i;
      next_cp(norm, i);
      auto it = piece_to_id.find(norm.substr(a, i - a));
      if (it != piece_to_id.end()) {
        sy.push_back({it->second, 0, 0, true});
      } else {
        for (size_t b = a; b < i; ++b) {
          const int id = spm_byte_id[(unsigned char)norm[b]];
          sy.push_back({id >= 0 ? id : unk_id, 0, 0, true});
        }
      }
    }
    const int n = (int)sy.size();
    for (int k = 0; k < n; ++k) { sy[k].prev = k - 1; sy[k].next = k + 1 < n ? k + 1 : -1; }
    struct Cand { double pri; int pos; int left, right, merged; };
    auto worse = [](const Cand& a, const Cand& b) { return a.pri != b.pri ? a.pri > b.pri : a.pos > b.pos; };
    std::priority_queue<Cand, std::vector<Cand>, decltype(worse)> heap(worse);
    auto consider = [&](int k) {
      if (k < 0 || sy[k].next < 0) return;
      const int a = sy[k].id, b = sy[sy[k].next].id;
      if (a < 0 || b < 0) return;
      if (scores.empty()) {
        auto it = merge_rank.find({a, b});
        if (it != merge_rank.end()) heap.push({(double)it->second, k, a, b, merge_to[{a, b}]});
      } else {
        auto it = raw_to_id.find(id_to_piece[a] + id_to_piece[b]);
        if (it != raw_to_id.end()) heap.push({-(double)scores[it->second], k, a, b, it->second});
      }
    };
    for (int k = 0; k < n; ++k) consider(k);
    while (!heap.empty()) {
      const Cand c = heap.top();
      heap.pop();
      if (!sy[c.pos].alive || sy[c.pos].id != c.left) continue;
      const int r = sy[c.pos].next;
      if (r < 0 || !sy[r].alive || sy[r].id != c.right) continue;
      sy[c.pos].id = c.merged;
      sy[r].alive = false;
      sy[c.pos].next = sy[r].next;
      if (sy[r].next >= 0) sy[sy[r].next].prev = c.pos;
      consider(sy[c.pos].prev);
      consider(c.pos);
    }
    for (int k = 0; k >= 0 && k < n; k = sy[k].next)
      if (sy[k].id >= 0) out.push_back(sy[k].id);
  }
  std::vector<std::string> id_to_piece;                     // SentencePiece mode: the piece text of every id
  std::unordered_map<std::string, int> raw_to_id;

  void add_merge(const std::string& a, const std::string& b, int rank) {
    auto ia = piece_to_id.find(a), ib = piece_to_id.find(b), ic = piece_to_id.find(a + b);
    if (ia == piece_to_id.end() || ib == piece_to_id.end() || ic == piece_to_id.end()) return;
    auto key = std::make_pair(ia->second, ib->second);
    if (merge_rank.find(key) == merge_rank.end()) {
      merge_rank[key] = rank;
      merge_to[key] = ic->second;
    }
  }

  void bpe_word(const std::string& word, std::vector<int>& out) {
    {
      std::lock_guard<std::mutex> g(mu);
      auto it = cache.find(word);
      if (it != cache.end()) { out.insert(out.end(), it->second.begin(), it->second.end()); return; }
    }
    std::vector<int> ids;
    ids.reserve(word.size());
    for (unsigned char c : word) {
      if (byte_id[c] >= 0) ids.push_back(byte_id[c]);
    }
    while (ids.size() > 1) {
      int best = -1, best_rank = 1 << 30;
      for (size_t k = 0; k + 1 < ids.size(); ++k) {
        auto it = merge_rank.find({ids[k], ids[k + 1]});
        if (it != merge_rank.end() && it->second < best_rank) { best_rank = it->second; best = (int)k; }
      }
      if (best < 0) break;
      const int a = ids[best], b = ids[best + 1], m = merge_to[{a, b}];
      std::vector<int> nxt;
      nxt.reserve(ids.size());
      for (size_t k = 0; k < ids.size(); ++k) {
        if (k + 1 < ids.size() && ids[k] == a && ids[k + 1] == b) { nxt.push_back(m); ++k; }
        else nxt.push_back(ids[k]);
      }
      ids.swap(nxt);
    }
    {
      std::lock_guard<std::mutex> g(mu);
      if (cache.size() < (1u << 18)) cache[word] = ids;
    }
    out.insert(out.end(), ids.begin(), ids.end());
  }

  void encode_plain(const std::string& text, std::vector<int>& out) {
    if (mode == kSpm) { bpe_spm(text, out); return; }
    std::vector<std::string> words;
    pretokenize(text, mode, words);
    for (auto& w : words) bpe_word(w, out);
  }

  void encode(const std::string& text, bool allow_special, std::vector<int>& out) {
    if (!allow_special || specials.empty()) { encode_plain(text, out); return; }
    size_t pos = 0, start = 0;
    while (pos < text.size()) {
      int hit = -1;
      size_t hit_len = 0;
      if (text[pos] == '<' || !specials.empty()) {
        for (auto& sp : specials) {
          if (sp.first.size() <= text.size() - pos && text.compare(pos, sp.first.size(), sp.first) == 0) {
            hit = sp.second;
            hit_len = sp.first.size();
            break;
          }
        }
      }
      if (hit >= 0) {
        if (pos > start) encode_plain(text.substr(start, pos - start), out);
        out.push_back(hit);
        pos += hit_len;
        start = pos;
      } else {
        ++pos;
      }
    }
    if (start < text.size()) encode_plain(text.substr(start), out);
  }
};

static std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

static Tokenizer* load_tokenizer_json(const std::string& path, int mode) {
  Json j = json_parse(read_file(path));
  auto* t = new Tokenizer();
  t->mode = mode;
  const Json* model = j.find("model");
  if (!model) throw std::runtime_error("tokenizer.json: no model");
  const Json* vocab = model->find("vocab");
  if (vocab && vocab->is_object())
    for (auto& kv : vocab->obj) t->add_piece(kv.first, (int)kv.second.as_int(), false);
  if (vocab && vocab->is_array()) {                 // unigram-style list of [piece, score]: merges ranked by score
    int id = 0;
    for (auto& e : vocab->arr) {
      if (e.is_array() && e.arr.size() == 2) {
        t->add_piece(e.arr[0].s, id, false);
        if ((size_t)id >= t->scores.size()) t->scores.resize(id + 1, -1e30f);
        t->scores[id] = (float)e.arr[1].as_double();
      }
      ++id;
    }
  }
  if (const Json* added = j.find("added_tokens"))
    for (auto& a : added->arr) {
      const Json* id = a.find("id");
      if (id) t->add_piece(a.get_string("content"), (int)id->as_int(), true);
    }
  t->finish();
  if (const Json* merges = model->find("merges")) {
    int rank = 0;
    for (auto& m : merges->arr) {
      if (m.is_string()) {
        size_t sp = m.s.find(' ');
        if (sp != std::string::npos) t->add_merge(m.s.substr(0, sp), m.s.substr(sp + 1), rank);
      } else if (m.is_array() && m.arr.size() == 2) {
        t->add_merge(m.arr[0].s, m.arr[1].s, rank);
      }
      ++rank;
    }
  }
  return t;
}

static Tokenizer* load_vocab_merges(const std::string& vocab_path, const std::string& merges_path, int mode) {
  auto* t = new Tokenizer();
  t->mode = mode;
  Json v = json_parse(read_file(vocab_path));
  for (auto& kv : v.obj) t->add_piece(kv.first, (int)kv.second.as_int(), false);
  t->finish();
  std::ifstream f(merges_path);
  std::string line;
  int rank = 0;
  while (std::getline(f, line)) {
    if (line.empty() || line[0] == '#') continue;
    size_t sp = line.find(' ');
    if (sp == std::string::npos) continue;
    t->add_merge(line.substr(0, sp), line.substr(sp + 1), rank++);
  }
  return t;
}

}  // namespace vh

using namespace vh;

extern "C" {

void* vh_tok_load_json(const char* path, int mode) {
  try { return load_tokenizer_json(path, mode); } catch (...) { return nullptr; }
}
void* vh_tok_load_vocab_merges(const char* vocab, const char* merges, int mode) {
  try { return load_vocab_merges(vocab, merges, mode); } catch (...) { return nullptr; }
}
void vh_tok_free(void* h) { delete (Tokenizer*)h; }
int vh_tok_add_special(void* h, const char* piece, int id) {
  auto* t = (Tokenizer*)h;
  t->add_piece(piece, id, true);
  t->finish();
  return 0;
}
int vh_tok_vocab_size(void* h) { return (int)((Tokenizer*)h)->id_to_bytes.size(); }
int vh_tok_piece_id(void* h, const char* piece) {
  auto* t = (Tokenizer*)h;
  for (auto& sp : t->specials) if (sp.first == piece) return sp.second;
  auto it = t->piece_to_id.find(piece);
  return it == t->piece_to_id.end() ? -1 : it->second;
}
// Returns the number of ids (may exceed cap: call again with a larger buffer).
int vh_tok_encode(void* h, const char* text, int len, int allow_special, int* out, int cap) {
  std::vector<int> ids;
  ((Tokenizer*)h)->encode(std::string(text, (size_t)len), allow_special != 0, ids);
  for (int k = 0; k < (int)ids.size() && k < cap; ++k) out[k] = ids[k];
  return (int)ids.size();
}
// Concatenated raw bytes of the ids; returns the byte count (may exceed cap).
int vh_tok_decode(void* h, const int* ids, int n, int skip_special, char* out, int cap) {
  auto* t = (Tokenizer*)h;
  int w = 0;
  for (int k = 0; k < n; ++k) {
    if (ids[k] < 0 || (size_t)ids[k] >= t->id_to_bytes.size()) continue;
    if (skip_special && t->is_special[ids[k]]) continue;
    const std::string& b = t->id_to_bytes[ids[k]];
    for (char c : b) {
      if (w < cap) out[w] = c;
      ++w;
    }
  }
  return w;
}
int vh_tok_is_special(void* h, int id) {
  auto* t = (Tokenizer*)h;
  return id >= 0 && (size_t)id < t->is_special.size() ? t->is_special[id] : 0;
}

}  // extern "C"
