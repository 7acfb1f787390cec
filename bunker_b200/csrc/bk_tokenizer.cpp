// bk_tokenizer.cpp -- the tokenizer boundary of bunker's decode driver as a plain C++ library (libbunker_tok.so).
//
// bunker tokenizes through a Rust cdylib around the `gigatoken` BPE crate: gt_init / gt_encode / gt_encode_mt / gt_free
// (shim/gigatoken_wrapper/src/lib.rs:19-93), loaded from TypeScript (prototypes/decode.ts:76-87).  The crate is not
// vendored and there is no Rust toolchain here, so the same four entry points are provided by this file over a
// byte-level BPE built from a Hugging Face tokenizer.json (model.vocab, model.merges, added_tokens), plus the one the
// reference lacks and its driver asks for (prototypes/decode.ts:1071-1078): gt_decode, ids -> text.
//
// Algorithm (the published byte-level BPE scheme): text is cut at added (special) tokens, each piece is pre-tokenized
// with the Qwen pattern -- contractions | optional non-letter + letters | single digit | optional space + punctuation
// run + newlines | whitespace + newlines | trailing whitespace | whitespace -- every pre-token's bytes are mapped to
// the printable code points of the GPT-2 byte table, and adjacent symbols are merged in order of merge rank until no
// listed pair is left.  Letter / digit / space classes are exact for ASCII; code points >= 0x80 count as letters except
// the Unicode space and punctuation blocks listed in classify() -- an approximation of \p{L} / \p{N} that is exact for
// Latin, Cyrillic, Greek and CJK text without exotic symbols.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <string>
#include <thread>
#include <unordered_map>
#include <utility>
#include <vector>

#define GT_API extern "C" __attribute__((visibility("default")))

namespace {

// ---- minimal JSON reader (objects, arrays, strings with escapes, numbers, literals) ---------------------------
struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  double num = 0;
  bool b = false;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  const Json* get(const char* key) const {
    for (auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JsonParser {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
  static void put_utf8(std::string& s, uint32_t cp) {
    if (cp < 0x80) s.push_back((char)cp);
    else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 63))); }
    else if (cp < 0x10000) { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 63))); s.push_back((char)(0x80 | (cp & 63))); }
    else { s.push_back((char)(0xF0 | (cp >> 18))); s.push_back((char)(0x80 | ((cp >> 12) & 63))); s.push_back((char)(0x80 | ((cp >> 6) & 63))); s.push_back((char)(0x80 | (cp & 63))); }
  }
  bool hex4(uint32_t& v) {
    if (end - p < 4) return false;
    v = 0;
    for (int i = 0; i < 4; i++) {
      char c = *p++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else return false;
    }
    return true;
  }
  bool string(std::string& out) {
    if (p >= end || *p != '"') return false;
    p++;
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return false;
        char c = *p++;
        switch (c) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            uint32_t cp;
            if (!hex4(cp)) return false;
            if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
              p += 2;
              uint32_t lo;
              if (!hex4(lo)) return false;
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            put_utf8(out, cp);
            break;
          }
          default: out.push_back(c);
        }
      } else {
        out.push_back(*p++);
      }
    }
    if (p >= end) return false;
    p++;
    return true;
  }
  Json value() {
    Json j;
    ws();
    if (p >= end) { ok = false; return j; }
    if (*p == '{') {
      j.kind = Json::Obj;
      p++;
      ws();
      if (p < end && *p == '}') { p++; return j; }
      while (ok) {
        ws();
        std::string k;
        if (!string(k)) { ok = false; break; }
        ws();
        if (p >= end || *p != ':') { ok = false; break; }
        p++;
        j.obj.emplace_back(std::move(k), value());
        ws();
        if (p < end && *p == ',') { p++; continue; }
        if (p < end && *p == '}') { p++; break; }
        ok = false;
      }
    } else if (*p == '[') {
      j.kind = Json::Arr;
      p++;
      ws();
      if (p < end && *p == ']') { p++; return j; }
      while (ok) {
        j.arr.push_back(value());
        ws();
        if (p < end && *p == ',') { p++; continue; }
        if (p < end && *p == ']') { p++; break; }
        ok = false;
      }
    } else if (*p == '"') {
      j.kind = Json::Str;
      if (!string(j.str)) ok = false;
    } else if (!strncmp(p, "true", 4) && end - p >= 4) { j.kind = Json::Bool; j.b = true; p += 4; }
    else if (!strncmp(p, "false", 5) && end - p >= 5) { j.kind = Json::Bool; p += 5; }
    else if (!strncmp(p, "null", 4) && end - p >= 4) { p += 4; }
    else {
      char* e = nullptr;
      j.kind = Json::Num;
      j.num = strtod(p, &e);
      if (e == p) ok = false;
      p = e;
    }
    return j;
  }
};

// ---- UTF-8 helpers ---------------------------------------------------------------------------------------------
inline uint32_t decode_utf8(const uint8_t* s, size_t n, size_t& len) {
  uint8_t c = s[0];
  if (c < 0x80) { len = 1; return c; }
  if ((c >> 5) == 6 && n >= 2) { len = 2; return ((c & 31u) << 6) | (s[1] & 63u); }
  if ((c >> 4) == 14 && n >= 3) { len = 3; return ((c & 15u) << 12) | ((s[1] & 63u) << 6) | (s[2] & 63u); }
  if ((c >> 3) == 30 && n >= 4) { len = 4; return ((c & 7u) << 18) | ((s[1] & 63u) << 12) | ((s[2] & 63u) << 6) | (s[3] & 63u); }
  len = 1;   // stray byte: its own (letter-class) unit
  return 0xFFFD;
}

enum Cls { LETTER, DIGIT, SPACE, NEWLINE, OTHER };
inline Cls classify(uint32_t cp) {
  if (cp == '\n' || cp == '\r') return NEWLINE;
  if (cp == ' ' || cp == '\t' || cp == 0x0B || cp == 0x0C || cp == 0x85 || cp == 0xA0 || cp == 0x1680 || (cp >= 0x2000 && cp <= 0x200A) ||
      cp == 0x2028 || cp == 0x2029 || cp == 0x202F || cp == 0x205F || cp == 0x3000)
    return SPACE;
  if (cp >= '0' && cp <= '9') return DIGIT;
  if ((cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z')) return LETTER;
  if (cp < 0x80) return OTHER;
  if (cp < 0xC0 && cp != 0xAA && cp != 0xB5 && cp != 0xBA) return OTHER;        // Latin-1 signs
  if (cp == 0xD7 || cp == 0xF7) return OTHER;
  if ((cp >= 0x2010 && cp <= 0x206F) || (cp >= 0x20A0 && cp <= 0x20CF) || (cp >= 0x2190 && cp <= 0x2BFF) || (cp >= 0x3001 && cp <= 0x303F) ||
      (cp >= 0xFF01 && cp <= 0xFF0F) || (cp >= 0xFF1A && cp <= 0xFF20) || (cp >= 0xFF3B && cp <= 0xFF40) || (cp >= 0xFF5B && cp <= 0xFF65) ||
      (cp >= 0x1F000 && cp <= 0x1FAFF) || cp == 0xFFFD)
    return OTHER;
  return LETTER;
}

struct Tok {
  std::unordered_map<std::string, uint32_t> vocab;                 // symbol (byte-table code points, UTF-8) -> id
  std::vector<std::string> id_to_sym;
  std::unordered_map<std::string, uint32_t> merge_rank;            // "left\x01right" -> rank
  std::vector<std::pair<std::string, uint32_t>> added;             // content -> id, longest first
  std::unordered_map<uint32_t, std::string> added_by_id;
  std::string byte_sym[256];                                       // byte -> its symbol
  std::unordered_map<uint32_t, uint8_t> cp_to_byte;
  int n_threads = 1;

  void build_byte_table() {
    // the GPT-2 table: printable Latin-1 bytes map to themselves, the rest to 256, 257, ... in byte order
    int extra = 0;
    for (int b = 0; b < 256; b++) {
      bool keep = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
      uint32_t cp = keep ? (uint32_t)b : (uint32_t)(256 + extra++);
      std::string s;
      JsonParser::put_utf8(s, cp);
      byte_sym[b] = s;
      cp_to_byte[cp] = (uint8_t)b;
    }
  }

  // one pre-token (raw bytes) -> ids
  void bpe(const uint8_t* s, size_t n, std::vector<uint32_t>& out) const {
    if (n == 0) return;
    std::vector<std::string> sym;
    sym.reserve(n);
    for (size_t i = 0; i < n; i++) sym.push_back(byte_sym[s[i]]);
    if (sym.size() > 1) {
      std::string whole;
      for (auto& x : sym) whole += x;
      auto it = vocab.find(whole);
      if (it != vocab.end() && merge_rank.empty()) { out.push_back(it->second); return; }
    }
    while (sym.size() > 1) {
      uint32_t best = 0xffffffffu;
      size_t at = 0;
      for (size_t i = 0; i + 1 < sym.size(); i++) {
        std::string key = sym[i];
        key.push_back('\x01');
        key += sym[i + 1];
        auto it = merge_rank.find(key);
        if (it != merge_rank.end() && it->second < best) { best = it->second; at = i; }
      }
      if (best == 0xffffffffu) break;
      sym[at] += sym[at + 1];
      sym.erase(sym.begin() + at + 1);
    }
    for (auto& x : sym) {
      auto it = vocab.find(x);
      if (it != vocab.end()) { out.push_back(it->second); continue; }
      // a symbol the vocabulary lacks: fall back to its single-byte symbols
      size_t i = 0;
      while (i < x.size()) {
        size_t len;
        decode_utf8((const uint8_t*)x.data() + i, x.size() - i, len);
        auto b = vocab.find(x.substr(i, len));
        if (b != vocab.end()) out.push_back(b->second);
        i += len;
      }
    }
  }

  // the pre-tokenizer pattern, as a scanner over code points
  void pretokenize(const uint8_t* s, size_t n, std::vector<uint32_t>& out) const {
    std::vector<uint32_t> cps;
    std::vector<size_t> off;
    for (size_t i = 0; i < n;) {
      size_t len;
      cps.push_back(decode_utf8(s + i, n - i, len));
      off.push_back(i);
      i += len;
    }
    off.push_back(n);
    const size_t m = cps.size();
    auto cls = [&](size_t i) { return classify(cps[i]); };
    auto lower = [&](size_t i) { uint32_t c = cps[i]; return (c >= 'A' && c <= 'Z') ? c + 32 : c; };
    size_t i = 0;
    while (i < m) {
      size_t j = i;
      bool done = false;
      if (cps[i] == '\'' && i + 1 < m) {   // 's 't 'm 'd | 're 've 'll
        uint32_t a = lower(i + 1), b = i + 2 < m ? lower(i + 2) : 0;
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) { j = i + 3; done = true; }
        else if (a == 's' || a == 't' || a == 'm' || a == 'd') { j = i + 2; done = true; }
      }
      if (!done) {
        Cls c0 = cls(i);
        size_t k = i;
        // [^\r\n\p{L}\p{N}]?\p{L}+
        if (c0 == LETTER || ((c0 == SPACE || c0 == OTHER) && i + 1 < m && cls(i + 1) == LETTER)) {
          k = (c0 == LETTER) ? i : i + 1;
          while (k < m && cls(k) == LETTER) k++;
          j = k;
        } else if (c0 == DIGIT) {
          j = i + 1;   // \p{N}: one digit at a time
        } else if (c0 == OTHER || (cps[i] == ' ' && i + 1 < m && cls(i + 1) == OTHER)) {
          //  ?[^\s\p{L}\p{N}]+[\r\n]*
          k = (c0 == OTHER) ? i : i + 1;
          while (k < m && cls(k) == OTHER) k++;
          while (k < m && cls(k) == NEWLINE) k++;
          j = k;
        } else {
          // whitespace run [i, k)
          k = i;
          while (k < m && (cls(k) == SPACE || cls(k) == NEWLINE)) k++;
          size_t last_nl = (size_t)-1;
          for (size_t q = i; q < k; q++)
            if (cls(q) == NEWLINE) last_nl = q;
          if (last_nl != (size_t)-1) j = last_nl + 1;            // \s*[\r\n]+
          else if (k == m) j = k;                                // \s+(?!\S) at the end of the text
          else if (k - i > 1) j = k - 1;                         // \s+(?!\S): leave the last space for the next token
          else j = k;                                            // \s+ : a single space before a digit / at a boundary
        }
      }
      if (j <= i) j = i + 1;
      bpe(s + off[i], off[j] - off[i], out);
      i = j;
    }
  }

  void encode(const uint8_t* s, size_t n, std::vector<uint32_t>& out) const {
    size_t start = 0, i = 0;
    while (i < n && !added.empty()) {
      bool hit = false;
      for (auto& a : added) {
        const std::string& c = a.first;
        if (!c.empty() && c.size() <= n - i && (uint8_t)c[0] == s[i] && !memcmp(c.data(), s + i, c.size())) {
          pretokenize(s + start, i - start, out);
          out.push_back(a.second);
          i += c.size();
          start = i;
          hit = true;
          break;
        }
      }
      if (!hit) i++;
    }
    pretokenize(s + start, n - start, out);
  }

  void decode(const uint32_t* ids, size_t n, std::string& out) const {
    for (size_t k = 0; k < n; k++) {
      auto a = added_by_id.find(ids[k]);
      if (a != added_by_id.end()) { out += a->second; continue; }
      if (ids[k] >= id_to_sym.size()) continue;
      const std::string& sym = id_to_sym[ids[k]];
      for (size_t i = 0; i < sym.size();) {
        size_t len;
        uint32_t cp = decode_utf8((const uint8_t*)sym.data() + i, sym.size() - i, len);
        auto b = cp_to_byte.find(cp);
        if (b != cp_to_byte.end()) out.push_back((char)b->second);
        else out.append(sym, i, len);
        i += len;
      }
    }
  }
};

}  // namespace

GT_API void* gt_init(const char* path) {
  if (!path) return nullptr;
  FILE* f = fopen(path, "rb");
  if (!f) return nullptr;
  std::string text;
  char buf[1 << 16];
  size_t r;
  while ((r = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, r);
  fclose(f);
  JsonParser jp{text.data(), text.data() + text.size()};
  Json root = jp.value();
  if (!jp.ok || root.kind != Json::Obj) return nullptr;
  const Json* model = root.get("model");
  const Json* vocab = model ? model->get("vocab") : nullptr;
  const Json* merges = model ? model->get("merges") : nullptr;
  if (!vocab || vocab->kind != Json::Obj) return nullptr;
  Tok* t = new Tok();
  t->build_byte_table();
  uint32_t max_id = 0;
  for (auto& kv : vocab->obj) {
    uint32_t id = (uint32_t)kv.second.num;
    t->vocab[kv.first] = id;
    max_id = std::max(max_id, id);
  }
  if (merges && merges->kind == Json::Arr) {
    uint32_t rank = 0;
    for (auto& m : merges->arr) {
      std::string l, rgt;
      if (m.kind == Json::Str) {
        size_t sp = m.str.find(' ');
        if (sp == std::string::npos) continue;
        l = m.str.substr(0, sp);
        rgt = m.str.substr(sp + 1);
      } else if (m.kind == Json::Arr && m.arr.size() == 2) {
        l = m.arr[0].str;
        rgt = m.arr[1].str;
      } else {
        continue;
      }
      t->merge_rank[l + '\x01' + rgt] = rank++;
    }
  }
  if (const Json* added = root.get("added_tokens"))
    for (auto& a : added->arr) {
      const Json* c = a.get("content");
      const Json* id = a.get("id");
      if (!c || !id) continue;
      t->added.emplace_back(c->str, (uint32_t)id->num);
      t->added_by_id[(uint32_t)id->num] = c->str;
      max_id = std::max(max_id, (uint32_t)id->num);
    }
  std::sort(t->added.begin(), t->added.end(), [](auto& a, auto& b) { return a.first.size() > b.first.size(); });
  t->id_to_sym.assign((size_t)max_id + 1, std::string());
  for (auto& kv : t->vocab) t->id_to_sym[kv.second] = kv.first;
  unsigned hc = std::thread::hardware_concurrency();
  t->n_threads = hc ? (int)hc : 8;
  return t;
}

GT_API int gt_encode(void* tok, const uint8_t* text, size_t text_len, uint32_t* out_buf, size_t out_max) {
  if (!tok || !text || !out_buf) return -1;
  std::vector<uint32_t> out;
  out.reserve(text_len / 3 + 8);
  static_cast<Tok*>(tok)->encode(text, text_len, out);
  size_t n = std::min(out.size(), out_max);
  memcpy(out_buf, out.data(), n * sizeof(uint32_t));
  return (int)n;
}

// Chunks cut at spaces, encoded in parallel, results concatenated in text order (the reference writes its chunks at
// an atomic cursor, i.e. in completion order, shim/gigatoken_wrapper/src/lib.rs:76-88; text order is kept here).
GT_API int gt_encode_mt(void* tok, const uint8_t* text, size_t text_len, uint32_t* out_buf, size_t out_max) {
  if (!tok || !text || !out_buf) return -1;
  Tok* t = static_cast<Tok*>(tok);
  int nt = std::max(1, t->n_threads);
  size_t chunk = (text_len + nt - 1) / nt;
  if (chunk < 4096) return gt_encode(tok, text, text_len, out_buf, out_max);
  std::vector<std::pair<size_t, size_t>> parts;
  size_t s = 0;
  while (s < text_len) {
    size_t e = std::min(s + chunk, text_len);
    while (e < text_len && text[e] != ' ') e++;   // a pre-token never starts in the middle of a word
    parts.emplace_back(s, e);
    s = e;
  }
  std::vector<std::vector<uint32_t>> outs(parts.size());
  std::atomic<size_t> next{0};
  std::vector<std::thread> th;
  for (int i = 0; i < nt; i++)
    th.emplace_back([&] {
      for (size_t k; (k = next.fetch_add(1)) < parts.size();) t->encode(text + parts[k].first, parts[k].second - parts[k].first, outs[k]);
    });
  for (auto& x : th) x.join();
  size_t total = 0;
  for (auto& o : outs) {
    size_t n = total < out_max ? std::min(o.size(), out_max - total) : 0;
    if (n) memcpy(out_buf + total, o.data(), n * sizeof(uint32_t));
    total += o.size();
  }
  return (int)total;
}

GT_API int gt_decode(void* tok, const uint32_t* ids, size_t n_ids, uint8_t* out_buf, size_t out_max) {
  if (!tok || (!ids && n_ids) || (!out_buf && out_max)) return -1;
  std::string s;
  static_cast<Tok*>(tok)->decode(ids, n_ids, s);
  size_t n = std::min(s.size(), out_max);
  if (n) memcpy(out_buf, s.data(), n);
  return (int)s.size();   // bytes the text has; more than out_max means the buffer was too small
}

GT_API int gt_vocab_size(void* tok) { return tok ? (int)static_cast<Tok*>(tok)->id_to_sym.size() : -1; }

GT_API void gt_free(void* tok) { delete static_cast<Tok*>(tok); }
