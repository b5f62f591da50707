// WordPiece tokenizer with the behaviour the UIE and ERNIE models need from the reference's
// external fast_tokenizer library (fastdeploy/text/uie/model.cc:177-184, 557-622): BERT-style
// basic tokenisation (clean-up, lower-casing, accent stripping for Latin-1, one token per CJK
// character, punctuation split), greedy longest-match WordPiece with "##" continuations, pair
// encoding [CLS] a [SEP] b [SEP] with type ids 0/1, longest-first truncation from the right, and
// per-token character offsets relative to each segment (special tokens carry (0, 0)).
//
// The character classes are spelled out as ranges here and mirrored one to one by the Python
// implementation in fastdeploy_b200/text/tokenizer.py, which the tests use as the oracle.
#include <algorithm>
#include <cstring>
#include <fstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "fdb_cpu.h"

namespace fdbcpu {

struct Piece {
  int id;
  int start, end;   // code-point offsets into the segment's original text
};

static bool is_whitespace(uint32_t c) {
  return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
         c == 0x202F || c == 0x205F || c == 0x3000;
}
static bool is_control(uint32_t c) {
  if (c == '\t' || c == '\n' || c == '\r') return false;
  return c < 0x20 || (c >= 0x7F && c < 0xA0) || c == 0xAD || (c >= 0x200B && c <= 0x200F) || (c >= 0x202A && c <= 0x202E) ||
         (c >= 0x2060 && c <= 0x2064) || c == 0xFEFF;
}
static bool is_cjk(uint32_t c) {
  return (c >= 0x4E00 && c <= 0x9FFF) || (c >= 0x3400 && c <= 0x4DBF) || (c >= 0x20000 && c <= 0x2A6DF) ||
         (c >= 0x2A700 && c <= 0x2B73F) || (c >= 0x2B740 && c <= 0x2B81F) || (c >= 0x2B820 && c <= 0x2CEAF) ||
         (c >= 0xF900 && c <= 0xFAFF) || (c >= 0x2F800 && c <= 0x2FA1F);
}
static bool is_punct(uint32_t c) {
  if ((c >= 33 && c <= 47) || (c >= 58 && c <= 64) || (c >= 91 && c <= 96) || (c >= 123 && c <= 126)) return true;
  if (c == 0xA1 || c == 0xA7 || c == 0xAB || c == 0xB6 || c == 0xB7 || c == 0xBB || c == 0xBF) return true;
  return (c >= 0x2010 && c <= 0x2027) || (c >= 0x2030 && c <= 0x205E) || (c >= 0x3001 && c <= 0x303F) ||
         (c >= 0xFF01 && c <= 0xFF0F) || (c >= 0xFF1A && c <= 0xFF20) || (c >= 0xFF3B && c <= 0xFF40) ||
         (c >= 0xFF5B && c <= 0xFF65);
}
// lower-casing and accent stripping, one code point in, one out
static uint32_t fold(uint32_t c) {
  if (c >= 'A' && c <= 'Z') return c + 32;
  if (c >= 0xC0 && c <= 0xDE && c != 0xD7) c += 0x20;          // Latin-1 capitals
  if (c >= 0x391 && c <= 0x3A9 && c != 0x3A2) return c + 0x20;   // Greek
  if (c >= 0x410 && c <= 0x42F) return c + 0x20;                 // Cyrillic
  if (c >= 0x400 && c <= 0x40F) return c + 0x50;
  if (c >= 0xE0 && c <= 0xFF) {
    static const char* base = "aaaaaa\0ceeeeiiii\0nooooo\0\0uuuuy\0y";   // 0xE0..0xFF, \0 = keep
    const char b = base[c - 0xE0];
    if (b != 0) return static_cast<uint32_t>(b);
  }
  return c;
}

static void utf8_decode(const char* s, std::vector<uint32_t>* out) {
  const unsigned char* p = reinterpret_cast<const unsigned char*>(s);
  while (*p) {
    uint32_t c;
    int n;
    if (*p < 0x80) { c = *p; n = 1; }
    else if ((*p >> 5) == 0x6) { c = *p & 0x1F; n = 2; }
    else if ((*p >> 4) == 0xE) { c = *p & 0x0F; n = 3; }
    else if ((*p >> 3) == 0x1E) { c = *p & 0x07; n = 4; }
    else { c = 0xFFFD; n = 1; }
    for (int i = 1; i < n; ++i) {
      if ((p[i] & 0xC0) != 0x80) { c = 0xFFFD; n = i; break; }
      c = (c << 6) | (p[i] & 0x3F);
    }
    out->push_back(c);
    p += n;
  }
}
static void utf8_append(uint32_t c, std::string* s) {
  if (c < 0x80) s->push_back(static_cast<char>(c));
  else if (c < 0x800) { s->push_back(static_cast<char>(0xC0 | (c >> 6))); s->push_back(static_cast<char>(0x80 | (c & 0x3F))); }
  else if (c < 0x10000) {
    s->push_back(static_cast<char>(0xE0 | (c >> 12))); s->push_back(static_cast<char>(0x80 | ((c >> 6) & 0x3F)));
    s->push_back(static_cast<char>(0x80 | (c & 0x3F)));
  } else {
    s->push_back(static_cast<char>(0xF0 | (c >> 18))); s->push_back(static_cast<char>(0x80 | ((c >> 12) & 0x3F)));
    s->push_back(static_cast<char>(0x80 | ((c >> 6) & 0x3F))); s->push_back(static_cast<char>(0x80 | (c & 0x3F)));
  }
}

class Tokenizer {
 public:
  bool load(const char* path, bool lower) {
    std::ifstream f(path);
    if (!f) return false;
    std::string line;
    int id = 0;
    while (std::getline(f, line)) {
      while (!line.empty() && (line.back() == '\r' || line.back() == '\n')) line.pop_back();
      vocab_.emplace(line, id++);
    }
    lower_ = lower;
    pad_ = find("[PAD]", 0); unk_ = find("[UNK]", 0); cls_ = find("[CLS]", 0); sep_ = find("[SEP]", 0);
    return id > 0;
  }
  int size() const { return static_cast<int>(vocab_.size()); }
  int token_id(const char* t) const { return find(t, -1); }
  int pad() const { return pad_; }

  void encode_segment(const char* text, std::vector<Piece>* out) const {
    std::vector<uint32_t> cps;
    utf8_decode(text, &cps);
    std::vector<uint32_t> word;
    std::vector<int> word_pos;
    auto flush = [&]() {
      if (!word.empty()) wordpiece(word, word_pos, out);
      word.clear(); word_pos.clear();
    };
    for (int i = 0; i < static_cast<int>(cps.size()); ++i) {
      const uint32_t c = cps[i];
      if (c == 0 || c == 0xFFFD || is_control(c)) continue;
      if (is_whitespace(c)) { flush(); continue; }
      if (is_cjk(c) || is_punct(c)) {
        flush();
        word.push_back(lower_ ? fold(c) : c); word_pos.push_back(i);
        flush();
        continue;
      }
      word.push_back(lower_ ? fold(c) : c);
      word_pos.push_back(i);
    }
    flush();
  }

  // [CLS] a [SEP] (b [SEP]); returns the token count, fills the arrays up to cap
  int encode_pair(const char* a, const char* b, int max_length, int* ids, int* types, int* os, int* oe, int cap) const {
    std::vector<Piece> pa, pb;
    encode_segment(a, &pa);
    const bool pair = b != nullptr;
    if (pair) encode_segment(b, &pb);
    const int specials = pair ? 3 : 2;
    if (max_length > 0) {
      long over = static_cast<long>(pa.size() + pb.size()) + specials - max_length;
      while (over > 0 && (pa.size() + pb.size()) > 0) {     // longest first, from the right
        if (pa.size() > pb.size()) pa.pop_back(); else if (!pb.empty()) pb.pop_back(); else pa.pop_back();
        --over;
      }
    }
    int n = 0;
    auto put = [&](int id, int ty, int s, int e) {
      if (n < cap) { ids[n] = id; types[n] = ty; os[n] = s; oe[n] = e; }
      ++n;
    };
    put(cls_, 0, 0, 0);
    for (const Piece& p : pa) put(p.id, 0, p.start, p.end);
    put(sep_, 0, 0, 0);
    if (pair) {
      for (const Piece& p : pb) put(p.id, 1, p.start, p.end);
      put(sep_, 1, 0, 0);
    }
    return n;
  }

 private:
  int find(const std::string& t, int dflt) const {
    auto it = vocab_.find(t);
    return it == vocab_.end() ? dflt : it->second;
  }
  void wordpiece(const std::vector<uint32_t>& w, const std::vector<int>& pos, std::vector<Piece>* out) const {
    const int n = static_cast<int>(w.size());
    if (n > 100) { out->push_back({unk_, pos.front(), pos.back() + 1}); return; }
    std::vector<Piece> pieces;
    int start = 0;
    while (start < n) {
      int end = n, found = -1;
      while (start < end) {
        std::string s = start > 0 ? "##" : "";
        for (int i = start; i < end; ++i) utf8_append(w[i], &s);
        auto it = vocab_.find(s);
        if (it != vocab_.end()) { found = it->second; break; }
        --end;
      }
      if (found < 0) { out->push_back({unk_, pos.front(), pos.back() + 1}); return; }
      pieces.push_back({found, pos[start], pos[end - 1] + 1});
      start = end;
    }
    out->insert(out->end(), pieces.begin(), pieces.end());
  }
  std::unordered_map<std::string, int> vocab_;
  bool lower_ = true;
  int pad_ = 0, unk_ = 0, cls_ = 0, sep_ = 0;
};

}  // namespace fdbcpu

using fdbcpu::Tokenizer;

FDB_CPU_API void* fdb_tok_create(const char* vocab_path, int do_lower) {
  auto* t = new Tokenizer();
  if (!t->load(vocab_path, do_lower != 0)) {
    fdbcpu::set_error("tokenizer: cannot read the vocabulary file");
    delete t;
    return nullptr;
  }
  return t;
}
FDB_CPU_API void fdb_tok_destroy(void* h) { delete static_cast<Tokenizer*>(h); }
FDB_CPU_API int fdb_tok_vocab_size(void* h) { return static_cast<Tokenizer*>(h)->size(); }
FDB_CPU_API int fdb_tok_token_to_id(void* h, const char* token) { return static_cast<Tokenizer*>(h)->token_id(token); }
FDB_CPU_API int fdb_tok_pad_id(void* h) { return static_cast<Tokenizer*>(h)->pad(); }
// Returns the number of tokens the encoding has (may exceed cap; then only cap entries were written).
FDB_CPU_API int fdb_tok_encode_pair(void* h, const char* a, const char* b, int max_length, int* ids, int* type_ids,
                                    int* off_start, int* off_end, int cap) {
  return static_cast<Tokenizer*>(h)->encode_pair(a, b, max_length, ids, type_ids, off_start, off_end, cap);
}
