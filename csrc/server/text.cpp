// Text layer of the server.  What each part keeps from the reference (crates/agens-server/src):
//   tokenizer.rs   byte-level BPE over tokenizer.json with the Qwen2 pre-tokenizer pattern (:21-22), added/special
//                  tokens matched before pre-tokenisation, skip_special_tokens on decode, and an incremental
//                  detokenizer that never emits a split UTF-8 sequence.  The pattern is implemented as a hand-written
//                  scanner (it needs a negative look-ahead); Unicode letter/number classes are approximated by block
//                  ranges (all scripts above U+00BF count as letters except the listed digit/punctuation/space blocks).
//   template.rs    here a built-in ChatML renderer instead of a Jinja engine (same observable prompts for the
//                  ChatML family: roles, tool preamble, think block handling, continue_final_message).
//   reasoning.rs   think-block splitter, streaming with partial-tag hold-back.
//   toolcall.rs    tool-call parsing, non-stream and stream, JSON-body and <function=..><parameter=..> wire formats,
//                  parameter values typed through the tool's JSON schema.
#include "text.hpp"

#include <algorithm>
#include <climits>
#include <cstring>
#include <queue>

namespace b2 {

// ------------------------------------------------------------------------------------------------ UTF-8 helpers
static unsigned decode_cp(const std::string& s, size_t& i) {
  const unsigned char c = (unsigned char)s[i];
  unsigned cp; int n;
  if (c < 0x80) { cp = c; n = 0; }
  else if ((c & 0xE0) == 0xC0) { cp = c & 0x1F; n = 1; }
  else if ((c & 0xF0) == 0xE0) { cp = c & 0x0F; n = 2; }
  else if ((c & 0xF8) == 0xF0) { cp = c & 0x07; n = 3; }
  else { ++i; return 0xFFFD; }
  ++i;
  for (int k = 0; k < n; ++k) {
    if (i >= s.size() || ((unsigned char)s[i] & 0xC0) != 0x80) return 0xFFFD;
    cp = (cp << 6) | ((unsigned char)s[i++] & 0x3F);
  }
  return cp;
}
static void append_cp(std::string& out, unsigned cp) {
  if (cp < 0x80) out.push_back((char)cp);
  else if (cp < 0x800) { out.push_back((char)(0xC0 | (cp >> 6))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) { out.push_back((char)(0xE0 | (cp >> 12))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
  else { out.push_back((char)(0xF0 | (cp >> 18))); out.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); out.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out.push_back((char)(0x80 | (cp & 0x3F))); }
}
static bool is_space_cp(unsigned c) {
  return c == ' ' || (c >= 9 && c <= 13) || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) || c == 0x2028 ||
         c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
static bool is_number_cp(unsigned c) {
  if (c < 0x80) return c >= '0' && c <= '9';
  return c == 0xB2 || c == 0xB3 || c == 0xB9 || (c >= 0xBC && c <= 0xBE) || (c >= 0x660 && c <= 0x669) || (c >= 0x6F0 && c <= 0x6F9) ||
         (c >= 0x966 && c <= 0x96F) || (c >= 0x9E6 && c <= 0x9EF) || (c >= 0xE50 && c <= 0xE59) || (c >= 0x2070 && c <= 0x2079) ||
         (c >= 0x2080 && c <= 0x2089) || (c >= 0x2150 && c <= 0x218B) || (c >= 0x2460 && c <= 0x249B) || (c >= 0x3021 && c <= 0x3029) ||
         (c >= 0xFF10 && c <= 0xFF19);
}
static bool is_letter_cp(unsigned c) {
  if (c < 0x80) return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z');
  if (c == 0xAA || c == 0xB5 || c == 0xBA) return true;
  if (c < 0xC0) return false;
  if (c == 0xD7 || c == 0xF7) return false;
  if (is_space_cp(c) || is_number_cp(c)) return false;
  if ((c >= 0x2000 && c <= 0x206F) || (c >= 0x20A0 && c <= 0x20CF) || (c >= 0x2190 && c <= 0x23FF) || (c >= 0x2500 && c <= 0x27BF) ||
      (c >= 0x2900 && c <= 0x2BFF) || (c >= 0x3000 && c <= 0x303F) || (c >= 0xFE30 && c <= 0xFE4F) || (c >= 0xFF00 && c <= 0xFF0F) ||
      (c >= 0xFF1A && c <= 0xFF20) || (c >= 0xFF3B && c <= 0xFF40) || (c >= 0xFF5B && c <= 0xFF65) || (c >= 0x1F000 && c <= 0x1FAFF) ||
      (c >= 0xE000 && c <= 0xF8FF) || (c >= 0x300 && c <= 0x36F))
    return false;
  return true;
}

// GPT-2 byte <-> printable code point tables
// Both tables are built once by the initialiser of a function-local static (thread safe: requests reach them from
// many connection threads at once).
struct ByteTables {
  unsigned to_cp[256];
  int to_byte[512];                                       // code points used by the mapping are below 256 + 68
  ByteTables() {
    int n = 0;
    for (int& v : to_byte) v = -1;
    for (int b = 0; b < 256; ++b) {
      const bool keep = (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
      to_cp[b] = keep ? (unsigned)b : 256u + (unsigned)(n++);
      to_byte[to_cp[b]] = b;
    }
  }
};
static const ByteTables& byte_tables() {
  static const ByteTables t;
  return t;
}
static const unsigned* byte_to_cp() { return byte_tables().to_cp; }
static int cp_to_byte(unsigned cp) { return cp < 512 ? byte_tables().to_byte[cp] : -1; }

// ------------------------------------------------------------------------------------------------ tokenizer
Tokenizer Tokenizer::from_json(const std::string& text) {
  Tokenizer t;
  Json j = Json::parse(text);
  const Json& model = j.at("model");
  int max_id = -1;
  for (auto& kv : model.at("vocab").members()) { t.vocab_[kv.first] = (int)kv.second.as_int(); max_id = std::max(max_id, (int)kv.second.as_int()); }
  if (auto a = j.find("added_tokens"); a && a->is_array())
    for (auto& e : a->items()) max_id = std::max(max_id, (int)e.at("id").as_int());
  t.id_to_tok_.assign(max_id + 1, std::string());
  for (auto& kv : t.vocab_) t.id_to_tok_[kv.second] = kv.first;
  int rank = 0;
  for (auto& m : model.at("merges").items()) {
    std::string key = m.is_string() ? m.as_string() : m[0].as_string() + " " + m[1].as_string();
    t.merge_rank_[key] = rank++;
  }
  if (auto a = j.find("added_tokens"); a && a->is_array()) {
    for (auto& e : a->items()) {
      const int id = (int)e.at("id").as_int();
      const std::string content = e.at("content").as_string();
      t.added_.emplace_back(content, id);
      t.id_to_tok_[id] = content;
      t.is_added_[id] = true;
      if (e.get_bool("special", false)) t.special_[id] = true;
    }
    std::sort(t.added_.begin(), t.added_.end(), [](auto& a, auto& b) { return a.first.size() > b.first.size(); });
    for (auto& a : t.added_) if (!a.first.empty()) t.added_first_[(unsigned char)a.first[0]] = true;
  }
  return t;
}

int Tokenizer::token_to_id(const std::string& s) const {
  for (auto& a : added_) if (a.first == s) return a.second;
  auto it = vocab_.find(s);
  return it == vocab_.end() ? -1 : it->second;
}

std::vector<std::string> Tokenizer::pretokenize(const std::string& text) const {
  std::vector<unsigned> cp;
  std::vector<size_t> off;          // byte offset of each code point, plus the end
  for (size_t i = 0; i < text.size();) { off.push_back(i); cp.push_back(decode_cp(text, i)); }
  off.push_back(text.size());
  std::vector<std::string> out;
  const size_t n = cp.size();
  auto lower = [](unsigned c) { return c >= 'A' && c <= 'Z' ? c + 32 : c; };
  size_t i = 0;
  auto emit = [&](size_t j) { out.push_back(text.substr(off[i], off[j] - off[i])); i = j; };
  while (i < n) {
    // 1. contractions
    if (cp[i] == '\'' && i + 1 < n) {
      const unsigned a = lower(cp[i + 1]), b = i + 2 < n ? lower(cp[i + 2]) : 0;
      if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) { emit(i + 3); continue; }
      if (a == 's' || a == 't' || a == 'm' || a == 'd') { emit(i + 2); continue; }
    }
    // 2. [^\r\n\p{L}\p{N}]?\p{L}+
    {
      size_t j = i;
      if (!(cp[j] == '\r' || cp[j] == '\n' || is_letter_cp(cp[j]) || is_number_cp(cp[j])) && j + 1 < n && is_letter_cp(cp[j + 1])) ++j;
      if (is_letter_cp(cp[j])) { while (j < n && is_letter_cp(cp[j])) ++j; emit(j); continue; }
    }
    // 3. \p{N}
    if (is_number_cp(cp[i])) { emit(i + 1); continue; }
    // 4.  ?[^\s\p{L}\p{N}]+[\r\n]*
    {
      size_t j = i;
      if (cp[j] == ' ' && j + 1 < n) ++j;
      auto other = [&](unsigned c) { return !is_space_cp(c) && !is_letter_cp(c) && !is_number_cp(c); };
      if (j < n && other(cp[j])) {
        while (j < n && other(cp[j])) ++j;
        while (j < n && (cp[j] == '\r' || cp[j] == '\n')) ++j;
        emit(j);
        continue;
      }
    }
    // whitespace alternatives
    size_t j = i;
    while (j < n && is_space_cp(cp[j])) ++j;
    if (j == i) { emit(i + 1); continue; }        // unreachable for valid classes; keeps progress
    // 5. \s*[\r\n]+ : up to the last newline of the run
    size_t last_nl = n;
    for (size_t k = i; k < j; ++k) if (cp[k] == '\r' || cp[k] == '\n') last_nl = k;
    if (last_nl != n) { emit(last_nl + 1); continue; }
    // 6. \s+(?!\S) : leave the last space to the following word
    if (j < n && j - i > 1) { emit(j - 1); continue; }
    if (j == n) { emit(j); continue; }
    // 7. \s+
    emit(j);
  }
  return out;
}

void Tokenizer::bpe(const std::string& piece, std::vector<int>& out) const {
  constexpr size_t kCacheWordBytes = 48, kCacheWords = 1u << 18;
  const bool cacheable = piece.size() <= kCacheWordBytes;
  if (cacheable) {
    std::shared_lock<std::shared_mutex> l(cache_->mu);
    auto it = cache_->ids.find(piece);
    if (it != cache_->ids.end()) { out.insert(out.end(), it->second.begin(), it->second.end()); return; }
  }
  const size_t out_start = out.size();
  // byte-level symbols
  std::vector<std::string> sym;
  const unsigned* b2c = byte_to_cp();
  for (unsigned char c : piece) { std::string s; append_cp(s, b2c[c]); sym.push_back(s); }
  // Lowest-ranked pair first, the leftmost one among equals: a heap of candidate pairs over a linked list of symbols
  // (n log n; a scan per merge took minutes on a hundred thousand spaces).  A popped candidate is stale when either
  // symbol has been merged since it was pushed, which its recorded lengths show.
  const int n = (int)sym.size();
  if (n > 1) {
    std::vector<int> prev(n), next(n);
    std::vector<char> alive(n, 1);
    for (int k = 0; k < n; ++k) { prev[k] = k - 1; next[k] = k + 1 < n ? k + 1 : -1; }
    struct Cand { int rank, left, right; size_t ll, rl; };
    auto later = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.left > b.left; };
    std::priority_queue<Cand, std::vector<Cand>, decltype(later)> heap(later);
    std::string key;
    auto push = [&](int l, int r) {
      if (l < 0 || r < 0) return;
      key.assign(sym[l]); key.push_back(' '); key.append(sym[r]);
      auto it = merge_rank_.find(key);
      if (it != merge_rank_.end()) heap.push(Cand{it->second, l, r, sym[l].size(), sym[r].size()});
    };
    for (int k = 0; k + 1 < n; ++k) push(k, k + 1);
    while (!heap.empty()) {
      const Cand c = heap.top();
      heap.pop();
      if (!alive[c.left] || !alive[c.right] || next[c.left] != c.right || sym[c.left].size() != c.ll || sym[c.right].size() != c.rl) continue;
      sym[c.left] += sym[c.right];
      alive[c.right] = 0;
      next[c.left] = next[c.right];
      if (next[c.right] >= 0) prev[next[c.right]] = c.left;
      push(prev[c.left], c.left);
      push(c.left, next[c.left]);
    }
    std::vector<std::string> merged;
    for (int k = 0; k >= 0; k = next[k]) merged.push_back(std::move(sym[k]));
    sym.swap(merged);
  }
  for (auto& s : sym) {
    auto it = vocab_.find(s);
    if (it != vocab_.end()) { out.push_back(it->second); continue; }
    // unknown merged symbol: fall back to its single byte-level characters
    for (size_t i = 0; i < s.size();) { size_t j = i; decode_cp(s, j); auto b = vocab_.find(s.substr(i, j - i)); if (b != vocab_.end()) out.push_back(b->second); i = j; }
  }
  if (cacheable) {
    std::unique_lock<std::shared_mutex> l(cache_->mu);
    if (cache_->ids.size() < kCacheWords) cache_->ids.emplace(piece, std::vector<int>(out.begin() + (long)out_start, out.end()));
  }
}

std::vector<int> Tokenizer::encode(const std::string& text) const {
  std::vector<int> out;
  size_t pos = 0, seg = 0;
  auto flush = [&](size_t end) {
    if (end > seg) for (auto& p : pretokenize(text.substr(seg, end - seg))) bpe(p, out);
  };
  while (pos < text.size()) {
    bool hit = false;
    if (added_first_[(unsigned char)text[pos]]) {          // only where an added token can start
      for (auto& a : added_) {
        if (!a.first.empty() && text.compare(pos, a.first.size(), a.first) == 0) {
          flush(pos);
          out.push_back(a.second);
          pos += a.first.size();
          seg = pos;
          hit = true;
          break;
        }
      }
    }
    if (!hit) ++pos;
  }
  flush(text.size());
  return out;
}

std::string Tokenizer::token_bytes(int id) const {
  if (id < 0 || id >= (int)id_to_tok_.size()) return std::string();
  const std::string& s = id_to_tok_[id];
  if (is_added_.count(id)) return s;
  std::string out;
  for (size_t i = 0; i < s.size();) { const unsigned cp = decode_cp(s, i); const int b = cp_to_byte(cp); if (b >= 0) out.push_back((char)b); else append_cp(out, cp); }
  return out;
}

std::string Tokenizer::decode(const std::vector<int>& ids, bool skip_special) const {
  std::string out;
  for (int id : ids) { if (skip_special && is_special(id)) continue; out += token_bytes(id); }
  return out;
}

// ------------------------------------------------------------------------------------------------ detokenizer
static size_t complete_utf8_prefix(const std::string& s) {
  // length of the longest prefix that does not end inside a multi-byte sequence
  size_t n = s.size();
  size_t back = 0;
  while (back < 4 && back < n && ((unsigned char)s[n - 1 - back] & 0xC0) == 0x80) ++back;
  if (back < n) {
    const unsigned char lead = (unsigned char)s[n - 1 - back];
    int need = lead < 0x80 ? 0 : ((lead & 0xE0) == 0xC0 ? 1 : ((lead & 0xF0) == 0xE0 ? 2 : ((lead & 0xF8) == 0xF0 ? 3 : 0)));
    if ((int)back < need) return n - 1 - back;
  }
  return n;
}
// Replaces every byte that is not part of a well-formed UTF-8 sequence by U+FFFD (what a lossy decode does), so that
// the text can always travel inside JSON.  A model may emit byte tokens in any order.
static std::string sanitize_utf8(const std::string& s) {
  std::string out;
  out.reserve(s.size());
  size_t i = 0;
  while (i < s.size()) {
    const unsigned char c = (unsigned char)s[i];
    int need = c < 0x80 ? 0 : ((c & 0xE0) == 0xC0 && c >= 0xC2 ? 1 : ((c & 0xF0) == 0xE0 ? 2 : ((c & 0xF8) == 0xF0 && c <= 0xF4 ? 3 : -1)));
    bool ok = need >= 0 && i + (size_t)need < s.size();
    if (ok)
      for (int j = 1; j <= need; ++j)
        if (((unsigned char)s[i + j] & 0xC0) != 0x80) { ok = false; break; }
    if (ok && need == 2) {
      const unsigned char c1 = (unsigned char)s[i + 1];
      if ((c == 0xE0 && c1 < 0xA0) || (c == 0xED && c1 >= 0xA0)) ok = false;      // overlong, surrogates
    }
    if (ok && need == 3) {
      const unsigned char c1 = (unsigned char)s[i + 1];
      if ((c == 0xF0 && c1 < 0x90) || (c == 0xF4 && c1 >= 0x90)) ok = false;
    }
    if (ok) { out.append(s, i, (size_t)need + 1); i += (size_t)need + 1; }
    else { out += "\xEF\xBF\xBD"; ++i; }
  }
  return out;
}
std::string Detokenizer::push(const std::vector<int>& ids) {
  for (int id : ids) { if (skip_special_ && tk_->is_special(id)) continue; pending_ += tk_->token_bytes(id); }
  const size_t k = complete_utf8_prefix(pending_);
  std::string out = sanitize_utf8(pending_.substr(0, k));
  pending_.erase(0, k);
  return out;
}
std::string Detokenizer::finish() {
  std::string out;
  if (!pending_.empty()) out = "\xEF\xBF\xBD";
  pending_.clear();
  return out;
}

// ------------------------------------------------------------------------------------------------ chat template
std::string render_chatml(const std::vector<ChatMessage>& msgs, const Json& tools, bool add_generation_prompt,
                          bool enable_thinking, bool continue_final) {
  std::string out;
  size_t first = 0;
  const bool has_tools = tools.is_array() && tools.size() > 0;
  if (has_tools) {
    out += "<|im_start|>system\n";
    if (!msgs.empty() && msgs[0].role == "system") { out += msgs[0].content + "\n\n"; first = 1; }
    out += "# Tools\n\nYou may call one or more functions to assist with the user query.\n\nYou are provided with function "
           "signatures within <tools></tools> XML tags:\n<tools>";
    for (auto& t : tools.items()) out += "\n" + t.dump_python();
    out += "\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
           "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n"
           "</tool_call><|im_end|>\n";
  } else if (!msgs.empty() && msgs[0].role == "system") {
    out += "<|im_start|>system\n" + msgs[0].content + "<|im_end|>\n";
    first = 1;
  }
  for (size_t i = first; i < msgs.size(); ++i) {
    const ChatMessage& m = msgs[i];
    const bool last = i + 1 == msgs.size();
    if (m.role == "tool") {
      const bool prev_tool = i > first && msgs[i - 1].role == "tool";
      const bool next_tool = !last && msgs[i + 1].role == "tool";
      if (!prev_tool) out += "<|im_start|>user";
      out += "\n<tool_response>\n" + m.content + "\n</tool_response>";
      if (!next_tool) out += "<|im_end|>\n";
      continue;
    }
    out += "<|im_start|>" + m.role + "\n";
    if (m.role == "assistant") {
      if (!m.reasoning.empty()) out += "<think>\n" + m.reasoning + "\n</think>\n\n";
      out += m.content;
      if (m.tool_calls.is_array())
        for (auto& tc : m.tool_calls.items()) {
          const Json* fn = tc.find("function");
          const Json& f = fn ? *fn : tc;
          Json args = Json::object();
          if (auto a = f.find("arguments")) { if (a->is_string()) { try { args = Json::parse(a->as_string()); } catch (...) { args = *a; } } else args = *a; }
          if (!m.content.empty() || &tc != &m.tool_calls.items()[0]) out += "\n";
          out += "<tool_call>\n{\"name\": \"" + f.get_string("name", "") + "\", \"arguments\": " + args.dump_python() + "}\n</tool_call>";
        }
    } else out += m.content;
    if (last && continue_final && m.role == "assistant") return out;
    out += "<|im_end|>\n";
  }
  if (add_generation_prompt) {
    out += "<|im_start|>assistant\n";
    if (!enable_thinking) out += "<think>\n\n</think>\n\n";
  }
  return out;
}

// ------------------------------------------------------------------------------------------------ reasoning parser
static size_t partial_suffix(const std::string& s, const std::string& tag) {
  // longest proper prefix of tag that is a suffix of s
  const size_t m = std::min(s.size(), tag.size() - 1);
  for (size_t k = m; k > 0; --k) if (s.compare(s.size() - k, k, tag, 0, k) == 0) return k;
  return 0;
}
ReasoningParser::Out ReasoningParser::parse_all(const std::string& text) const {
  Out o;
  std::string t = text;
  bool in = in_;
  const size_t op = t.find(open_);
  if (op != std::string::npos && (in || t.find_first_not_of(" \n\t") == op)) { t.erase(0, op + open_.size()); in = true; }
  if (!in) { o.content = text; return o; }
  const size_t cl = t.find(close_);
  if (cl == std::string::npos) { o.reasoning = t; return o; }
  o.reasoning = t.substr(0, cl);
  o.content = t.substr(cl + close_.size());
  auto trim = [](std::string& s) { size_t a = s.find_first_not_of("\n"); if (a == std::string::npos) { s.clear(); return; } s.erase(0, a); };
  trim(o.content);
  while (!o.reasoning.empty() && (o.reasoning.back() == '\n')) o.reasoning.pop_back();
  while (!o.reasoning.empty() && (o.reasoning.front() == '\n')) o.reasoning.erase(0, 1);
  return o;
}
ReasoningParser::Out ReasoningParser::push(const std::string& delta) {
  Out o;
  buf_ += delta;
  while (true) {
    if (!in_) {
      if (!stripped_open_) {
        const size_t op = buf_.find(open_);
        if (op != std::string::npos && buf_.find_first_not_of(" \n\t") == op) { buf_.erase(0, op + open_.size()); in_ = true; stripped_open_ = true; continue; }
        if (partial_suffix(buf_, open_) && buf_.find_first_not_of(" \n\t") != std::string::npos &&
            buf_.find_first_not_of(" \n\t") + partial_suffix(buf_, open_) == buf_.size()) return o;   // may still become the tag
      }
      if (stripped_open_ && !buf_.empty() && buf_.size() < open_.size() && open_.compare(0, buf_.size(), buf_) == 0) return o;   // may become an opening tag
      if (stripped_open_ && !open_.empty() && buf_.compare(0, open_.size(), open_) == 0) {
        // a later opening tag at the start of a piece of output begins another think block
        buf_.erase(0, open_.size()); in_ = true; continue;
      }
      if (strip_nl_) {       // newlines right after the closing tag belong to the block, whichever chunk brings them
        size_t a = buf_.find_first_not_of('\n');
        if (a == std::string::npos) { buf_.clear(); return o; }
        buf_.erase(0, a);
        strip_nl_ = false;
      }
      o.content += buf_;
      buf_.clear();
      return o;
    }
    if (!stripped_open_) {   // started inside the block: a leading open tag in the output is dropped
      const size_t op = buf_.find(open_);
      if (op == 0) { buf_.erase(0, open_.size()); stripped_open_ = true; continue; }
      if (!buf_.empty() && partial_suffix(buf_, open_) == buf_.size()) return o;
      stripped_open_ = true;
    }
    const size_t cl = buf_.find(close_);
    // a tool call that starts inside an unclosed thinking block ends the block: the call is content
    const size_t brk = interrupt_.empty() ? std::string::npos : buf_.find(interrupt_);
    if (brk != std::string::npos && (cl == std::string::npos || brk < cl)) {
      std::string r = buf_.substr(0, brk);
      buf_.erase(0, brk);
      in_ = false;
      if (stream_) o.reasoning += r; else { held_reasoning_ += r; o.reasoning += held_reasoning_; held_reasoning_.clear(); }
      stripped_open_ = true;
      continue;
    }
    if (cl != std::string::npos) {
      std::string r = buf_.substr(0, cl);
      buf_.erase(0, cl + close_.size());
      in_ = false;
      if (stream_) o.reasoning += r; else { held_reasoning_ += r; o.reasoning += held_reasoning_; held_reasoning_.clear(); }
      strip_nl_ = !keep_nl_;
      stripped_open_ = true;
      continue;
    }
    const size_t keep = std::max(partial_suffix(buf_, close_), interrupt_.empty() ? (size_t)0 : partial_suffix(buf_, interrupt_));
    std::string r = buf_.substr(0, buf_.size() - keep);
    buf_.erase(0, buf_.size() - keep);
    if (stream_) o.reasoning += r; else held_reasoning_ += r;
    return o;
  }
}
ReasoningParser::Out ReasoningParser::finish() {
  Out o;
  if (in_) { o.reasoning = held_reasoning_ + buf_; } else o.content = buf_;
  buf_.clear(); held_reasoning_.clear();
  return o;
}

// ------------------------------------------------------------------------------------------------ tool calls
static const Json* tool_schema(const Json& tools, const std::string& name) {
  if (!tools.is_array()) return nullptr;
  for (auto& t : tools.items()) {
    const Json* f = t.find("function");
    const Json& fn = f ? *f : t;
    if (fn.get_string("name", "") == name) return fn.find("parameters");
  }
  return nullptr;
}
// ---- typing of a parameter's text through the tool's JSON schema
// The contract (observed on the reference's parser corpus, crates/agens-server/tests/fixtures/parser_corpus.json):
//   * the text "null" in any letter case is JSON null, whatever the declared type;
//   * the declared types are the property's "type" (a string or a list) plus the types inside anyOf / oneOf / allOf;
//   * if "string" is among them the text stays a string; a property without any type information stays a string too;
//   * an enum without a type yields the enum member whose JSON text equals the value (so "2" becomes 2 for [1, 2]);
//   * integers follow Python's int(): sign, leading zeros, single underscores between digits;
//   * numbers follow Python's float(): inf / infinity / nan, exponents, underscores;
//   * booleans: "true" in any letter case is true, everything else false;
//   * objects and arrays: JSON first, then a Python literal (single quotes, True / False / None, tuples become lists);
//   * whatever does not convert stays the text.
static std::string lower_trim(const std::string& v) {
  size_t a = 0, b = v.size();
  while (a < b && std::isspace((unsigned char)v[a])) ++a;
  while (b > a && std::isspace((unsigned char)v[b - 1])) --b;
  std::string o = v.substr(a, b - a);
  for (auto& c : o) c = (char)std::tolower((unsigned char)c);
  return o;
}
static bool strip_underscores(const std::string& v, std::string& out) {       // Python's rule: single, between digits
  out.clear();
  for (size_t i = 0; i < v.size(); ++i) {
    if (v[i] == '_') {
      if (i == 0 || i + 1 >= v.size() || !std::isdigit((unsigned char)v[i - 1]) || !std::isdigit((unsigned char)v[i + 1])) return false;
      continue;
    }
    out.push_back(v[i]);
  }
  return true;
}
static bool python_int(const std::string& raw, long long& out) {
  std::string t, v = lower_trim(raw);
  if (!strip_underscores(v, t) || t.empty()) return false;
  size_t i = (t[0] == '+' || t[0] == '-') ? 1 : 0;
  if (i >= t.size() || t.size() - i > 18) return false;
  for (size_t j = i; j < t.size(); ++j) if (!std::isdigit((unsigned char)t[j])) return false;
  out = std::strtoll(t.c_str(), nullptr, 10);
  return true;
}
static bool python_float(const std::string& raw, double& out) {
  std::string t, v = lower_trim(raw);
  if (!strip_underscores(v, t) || t.empty()) return false;
  std::string u = t;
  const bool neg = u[0] == '-';
  if (u[0] == '+' || u[0] == '-') u.erase(0, 1);
  if (u == "inf" || u == "infinity") { out = neg ? -INFINITY : INFINITY; return true; }
  if (u == "nan") { out = NAN; return true; }
  bool digit = false;
  for (char c : u) {
    if (std::isdigit((unsigned char)c)) digit = true;
    else if (c != '.' && c != 'e' && c != '+' && c != '-') return false;
  }
  if (!digit) return false;
  char* end = nullptr;
  out = std::strtod(t.c_str(), &end);
  return end && *end == 0;
}
// Python literal (dict / list / tuple / str / numbers / True / False / None) -> Json; throws on anything else.
struct PyLit {
  const std::string& s;
  size_t i = 0;
  explicit PyLit(const std::string& t) : s(t) {}
  void ws() { while (i < s.size() && std::isspace((unsigned char)s[i])) ++i; }
  [[noreturn]] void bad() { throw std::runtime_error("not a Python literal"); }
  int depth = 0;                                          // as deep as the JSON parser goes; model output decides the text
  struct Level { int& d; explicit Level(int& x) : d(x) { if (++d > 200) { --d; throw std::runtime_error("literal nested too deeply"); } } ~Level() { --d; } };
  Json value() {
    Level lv(depth);
    ws();
    if (i >= s.size()) bad();
    const char c = s[i];
    if (c == '{') {
      ++i;
      Json o = Json::object();
      ws();
      if (i < s.size() && s[i] == '}') { ++i; return o; }
      while (true) {
        Json k = value();
        if (!k.is_string()) bad();
        ws();
        if (i >= s.size() || s[i] != ':') bad();
        ++i;
        o.set(k.as_string(), value());
        ws();
        if (i < s.size() && s[i] == ',') { ++i; ws(); if (i < s.size() && s[i] == '}') { ++i; return o; } continue; }
        if (i < s.size() && s[i] == '}') { ++i; return o; }
        bad();
      }
    }
    if (c == '[' || c == '(') {
      const char close = c == '[' ? ']' : ')';
      ++i;
      Json a = Json::array();
      ws();
      if (i < s.size() && s[i] == close) { ++i; return a; }
      while (true) {
        a.push_back(value());
        ws();
        if (i < s.size() && s[i] == ',') { ++i; ws(); if (i < s.size() && s[i] == close) { ++i; return a; } continue; }
        if (i < s.size() && s[i] == close) { ++i; return a; }
        bad();
      }
    }
    if (c == '\'' || c == '"') {
      ++i;
      std::string o;
      while (i < s.size() && s[i] != c) {
        if (s[i] == '\\' && i + 1 < s.size()) {
          const char e = s[i + 1];
          i += 2;
          if (e == 'n') o.push_back('\n'); else if (e == 't') o.push_back('\t'); else if (e == 'r') o.push_back('\r');
          else if (e == '\\' || e == '\'' || e == '"') o.push_back(e); else { o.push_back('\\'); o.push_back(e); }
          continue;
        }
        o.push_back(s[i++]);
      }
      if (i >= s.size()) bad();
      ++i;
      return Json(o);
    }
    size_t j = i;
    while (j < s.size() && (std::isalnum((unsigned char)s[j]) || s[j] == '_' || s[j] == '.' || s[j] == '+' || s[j] == '-')) ++j;
    const std::string tok = s.substr(i, j - i);
    if (tok.empty()) bad();
    i = j;
    if (tok == "True") return Json(true);
    if (tok == "False") return Json(false);
    if (tok == "None") return Json();
    long long iv;
    if (python_int(tok, iv)) return Json((int64_t)iv);
    double dv;
    if (python_float(tok, dv)) return Json(dv);
    bad();
  }
  Json parse() { Json v = value(); ws(); if (i != s.size()) bad(); return v; }
};
static void collect_types(const Json& p, std::vector<std::string>& types) {
  if (auto t = p.find("type")) {
    if (t->is_string()) types.push_back(t->as_string());
    else if (t->is_array()) for (auto& x : t->items()) if (x.is_string()) types.push_back(x.as_string());
  }
  for (const char* key : {"anyOf", "oneOf", "allOf"})
    if (auto a = p.find(key)) if (a->is_array()) for (auto& m : a->items()) if (m.is_object()) collect_types(m, types);
  if (types.empty() && p.contains("properties")) types.push_back("object");
}
static Json typed_value(const std::string& raw, const Json* schema, const std::string& key) {
  if (lower_trim(raw) == "null") return Json();
  const Json* prop = nullptr;
  if (schema) if (auto props = schema->find("properties")) prop = props->find(key);
  if (!prop || !prop->is_object()) return Json(raw);
  std::vector<std::string> types;
  collect_types(*prop, types);
  auto has = [&](const char* t) { for (auto& x : types) if (x == t) return true; return false; };
  auto has_prefix = [&](const char* t) { for (auto& x : types) if (x.rfind(t, 0) == 0) return true; return false; };
  if (types.empty()) {
    if (auto en = prop->find("enum")) if (en->is_array()) {
      const std::string v = lower_trim(raw) == raw ? raw : raw;      // members are compared with the text as written
      for (auto& m : en->items()) {
        if (m.is_string() && m.as_string() == v) return m;
        if (!m.is_string() && m.dump() == lower_trim(raw)) return m;
      }
    }
    return Json(raw);
  }
  if (has("string")) return Json(raw);
  long long iv;
  if ((has_prefix("int") || has_prefix("uint")) && python_int(raw, iv)) return Json((int64_t)iv);
  double dv;
  if ((has("number") || has("float") || has("double")) && python_float(raw, dv)) {
    // text that reads as an integer stays one: exactly when it fits 64 bits, else with the digits of the nearest double
    const std::string lt = lower_trim(raw);
    if (std::isfinite(dv) && lt.find_first_of(".en") == std::string::npos) {
      if (python_int(raw, iv)) return Json((int64_t)iv);
      return Json::big_integer(dv);
    }
    return Json(dv);
  }
  if (has("boolean")) return Json(lower_trim(raw) == "true");
  if (has("object") || has("array") || has("dict") || has("list") || has("tuple")) {
    try { return Json::parse(raw); } catch (...) {}
    try { return PyLit(raw).parse(); } catch (...) {}
  }
  return Json(raw);
}
static std::string strip_nl(std::string v) {
  if (!v.empty() && v[0] == '\n') v.erase(0, 1);
  if (!v.empty() && v.back() == '\n') v.pop_back();
  return v;
}
static bool parse_function_block(const std::string& body, const Json& tools, ToolCall& out) {
  // body = NAME>...<parameter=K>V</parameter>...
  const size_t gt = body.find('>');
  if (gt == std::string::npos) return false;
  out.name = body.substr(0, gt);
  const Json* schema = tool_schema(tools, out.name);
  Json args = Json::object();
  size_t pos = gt + 1;
  while (true) {
    const size_t p = body.find("<parameter=", pos);
    if (p == std::string::npos) break;
    const size_t kend = body.find('>', p);
    if (kend == std::string::npos) break;
    const std::string key = body.substr(p + 11, kend - p - 11);
    size_t vend = body.find("</parameter>", kend);
    const size_t next = body.find("<parameter=", kend);
    size_t stop = std::min(vend, next);
    if (stop == std::string::npos) stop = body.size();
    args.set(key, typed_value(strip_nl(body.substr(kend + 1, stop - kend - 1)), schema, key));
    pos = (vend != std::string::npos && vend == stop) ? vend + 12 : stop;
  }
  out.arguments_json = args.dump(Json::Style{true, false});
  return true;
}
ToolParse parse_tool_calls(const std::string& text, const Json& tools) { return parse_tool_calls(text, tools, "<tool_call>", "</tool_call>"); }

ToolParse parse_tool_calls(const std::string& text, const Json& tools, const std::string& call_open, const std::string& call_close) {
  ToolParse r;
  size_t pos = 0;
  const size_t lo = call_open.size(), lc = call_close.size();
  while (pos < text.size()) {
    const size_t a = text.find(call_open, pos), b = text.find("<function=", pos);
    const size_t s = std::min(a, b);
    if (s == std::string::npos) { r.content += text.substr(pos); break; }
    r.content += text.substr(pos, s - pos);
    if (s == a) {
      size_t e = text.find(call_close, s);
      const std::string body = text.substr(s + lo, (e == std::string::npos ? text.size() : e) - s - lo);
      const size_t fb = body.find("<function=");
      ToolCall tc;
      bool ok = false;
      if (e == std::string::npos && !r.calls.empty()) {
        // the output ended inside a further call: after a complete call the fragment is neither a call nor content
        r.unfinished = true;
        break;
      }
      if (fb != std::string::npos) {
        // a block closed by the call tag counts even without its </function>; a lone call that the output cut short is
        // salvaged with what it has (the value runs to the end of the text)
        size_t fe = body.find("</function>", fb);
        ok = parse_function_block(body.substr(fb + 10, (fe == std::string::npos ? body.size() : fe) - fb - 10), tools, tc);
      } else {
        try {
          Json j = Json::parse(body);
          tc.name = j.get_string("name", "");
          const Json* ar = j.find("arguments");
          if (!ar) ar = j.find("parameters");
          tc.arguments_json = ar ? (ar->is_string() ? ar->as_string() : ar->dump(Json::Style{true, false})) : "{}";
          ok = !tc.name.empty();
        } catch (...) { ok = false; }
      }
      if (ok) r.calls.push_back(tc); else r.content += text.substr(s, (e == std::string::npos ? text.size() : e + lc) - s);
      pos = e == std::string::npos ? text.size() : e + lc;
    } else {
      size_t e = text.find("</function>", s);
      if (e == std::string::npos && !r.calls.empty()) { r.unfinished = true; break; }
      ToolCall tc;
      if (parse_function_block(text.substr(s + 10, (e == std::string::npos ? text.size() : e) - s - 10), tools, tc)) r.calls.push_back(tc);
      pos = e == std::string::npos ? text.size() : e + 11;
    }
  }
  while (!r.content.empty() && (r.content.back() == '\n' || r.content.back() == ' ')) r.content.pop_back();
  return r;
}

ToolParse ToolStreamParser::push(const std::string& delta) {
  ToolParse out;
  if (content_before_calls_only_ && saw_call_ && buf_.empty()) {
    // in this mode text after a finished call is not content, but a further call still is a call
    tail_ += delta;
    buf_.swap(tail_);
  } else {
    buf_ += delta;
  }
  while (true) {
    const size_t a = buf_.find(call_open_), b = buf_.find("<function=");
    const size_t s = std::min(a, b);
    const bool drop = content_before_calls_only_ && saw_call_;
    if (s == std::string::npos) {
      // emit everything except a tail that may still grow into a tag
      const size_t keep = std::max(partial_suffix(buf_, call_open_), partial_suffix(buf_, "<function="));
      if (!drop) out.content += buf_.substr(0, buf_.size() - keep);
      buf_.erase(0, buf_.size() - keep);
      return out;
    }
    if (!drop) out.content += buf_.substr(0, s);
    buf_.erase(0, s);
    const std::string close = (s == a) ? call_close_ : "</function>";
    const size_t e = buf_.find(close);
    if (e == std::string::npos) return out;   // the call is still being generated
    ToolParse one = parse_tool_calls(buf_.substr(0, e + close.size()), tools_, call_open_, call_close_);
    for (auto& c : one.calls) out.calls.push_back(c);
    if (!one.calls.empty()) saw_call_ = true;
    out.content += one.content;
    buf_.erase(0, e + close.size());
  }
}
ToolParse ToolStreamParser::finish() {
  if (saw_call_) {
    // after a complete call a fragment of a further call at the end of the output is neither a call nor content
    const size_t a0 = buf_.find(call_open_), b0 = buf_.find("<function=");
    const size_t st0 = std::min(a0, b0);
    if (st0 != std::string::npos) {
      ToolParse cut;
      if (!content_before_calls_only_) cut.content = buf_.substr(0, st0);
      cut.unfinished = true;
      buf_.clear();
      return cut;
    }
  }
  ToolParse out = parse_tool_calls(buf_, tools_, call_open_, call_close_);
  if (content_before_calls_only_) {
    // an unfinished call at the end of the output is neither a call nor content
    const size_t a = buf_.find(call_open_), b = buf_.find("<function=");
    const size_t st = std::min(a, b);
    if (st != std::string::npos && out.calls.empty()) out.content = buf_.substr(0, st);
  }
  buf_.clear();
  return out;
}

// ---- incremental tool calls ----------------------------------------------------------------------------------------
static bool is_prefix_of(const std::string& s, const std::string& full) { return s.size() <= full.size() && full.compare(0, s.size(), s) == 0; }
static bool starts_with(const std::string& s, const std::string& p) { return s.size() >= p.size() && s.compare(0, p.size(), p) == 0; }

std::vector<ToolDelta> ToolDeltaParser::push(const std::string& delta) {
  std::vector<ToolDelta> out;
  auto content = [&](const std::string& t) {
    if (t.empty()) return;
    if (!out.empty() && out.back().kind == ToolDelta::Content) out.back().text += t; else out.push_back({ToolDelta::Content, -1, t});
  };
  auto args = [&](const std::string& t) { out.push_back({ToolDelta::Args, n_calls_ - 1, t}); };
  auto skip_ws = [&]() { size_t a = buf_.find_first_not_of(" \n\r\t"); buf_.erase(0, a == std::string::npos ? buf_.size() : a); };
  static const std::string kFn = "<function=", kFnEnd = "</function>", kPar = "<parameter=", kParEnd = "</parameter>";
  buf_ += delta;
  while (true) {
    if (st_ == Outside) {
      const size_t p = buf_.find(open_);
      if (p == std::string::npos) {
        const size_t keep = partial_suffix(buf_, open_);      // may still become the wrapper tag
        content(buf_.substr(0, buf_.size() - keep));
        buf_.erase(0, buf_.size() - keep);
        return out;
      }
      content(buf_.substr(0, p));
      buf_.erase(0, p + open_.size());
      st_ = WantFunction;
    } else if (st_ == WantFunction) {
      skip_ws();
      if (buf_.empty()) return out;
      if (starts_with(buf_, kFn)) {
        const size_t gt = buf_.find('>');
        if (gt == std::string::npos) return out;
        const std::string name = buf_.substr(kFn.size(), gt - kFn.size());
        buf_.erase(0, gt + 1);
        schema_ = tool_schema(tools_, name);
        out.push_back({ToolDelta::Start, n_calls_++, name});
        n_params_ = 0; opened_ = false;
        st_ = InBody;
      } else if (starts_with(buf_, close_)) { buf_.erase(0, close_.size()); st_ = Outside; }
      else if (is_prefix_of(buf_, kFn) || is_prefix_of(buf_, close_)) return out;
      else {
        // something else follows the wrapper tag: it is skipped up to a function header or the closing tag, whichever
        // comes (the reference's detector keeps waiting for a header the same way)
        const size_t f = buf_.find(kFn), c = buf_.find(close_);
        if (f == std::string::npos && c == std::string::npos) {
          const size_t keep = std::max(partial_suffix(buf_, kFn), partial_suffix(buf_, close_));
          buf_.erase(0, buf_.size() - keep);
          return out;
        }
        buf_.erase(0, std::min(f, c));
      }
    } else if (st_ == InBody) {
      skip_ws();
      if (buf_.empty()) return out;
      if (starts_with(buf_, kPar)) {
        const size_t gt = buf_.find('>');
        if (gt == std::string::npos) return out;
        key_ = buf_.substr(kPar.size(), gt - kPar.size());
        buf_.erase(0, gt + 1);
        st_ = InValue;
      } else if (starts_with(buf_, kFnEnd)) {
        if (!opened_) { args("{"); opened_ = true; }
        args("}");
        buf_.erase(0, kFnEnd.size());
        st_ = AfterFunction;
      } else if (starts_with(buf_, close_)) { buf_.erase(0, close_.size()); st_ = Outside; }   // no </function>: the object stays open
      else if (is_prefix_of(buf_, kPar) || is_prefix_of(buf_, kFnEnd) || is_prefix_of(buf_, close_)) return out;
      else {                                      // stray text inside a call: skipped up to the next tag
        const size_t lt = buf_.find('<', 1);
        if (lt == std::string::npos) { buf_.clear(); return out; }
        buf_.erase(0, lt);
      }
    } else if (st_ == InValue) {
      size_t end = std::string::npos;
      bool eat = false;
      const std::string* tags[4] = {&kParEnd, &kPar, &kFnEnd, &close_};
      for (const std::string* tag : tags) {
        const size_t p = buf_.find(*tag);
        if (p < end) { end = p; eat = tag == &kParEnd; }
      }
      if (end == std::string::npos) return out;   // the value is reported whole, when its parameter ends
      const Json v = typed_value(strip_nl(buf_.substr(0, end)), schema_, key_);
      if (!opened_) { args("{"); opened_ = true; }
      args(std::string(n_params_ ? ", " : "") + Json(key_).dump(Json::Style{true, false}) + ": " + v.dump(Json::Style{true, false}));
      ++n_params_;
      buf_.erase(0, end + (eat ? kParEnd.size() : 0));
      st_ = InBody;
    } else {                                      // AfterFunction
      skip_ws();
      if (buf_.empty()) return out;
      if (starts_with(buf_, close_)) { buf_.erase(0, close_.size()); st_ = Outside; }
      else if (is_prefix_of(buf_, close_)) return out;
      else st_ = Outside;
    }
  }
}

}  // namespace b2
