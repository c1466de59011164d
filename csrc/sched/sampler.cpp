// Host-side token sampler, reasoning budget and thinking-loop guard.
//
// Behavioural contract (reference: crates/agens-cli/src/sampler.rs:170-284, :19-149):
//   order   extra bias -> logit_bias -> suppressed ids (-inf) -> repetition (x > 0 ? x / r : x * r), frequency * count
//           + presence -> stop ids masked while fewer than min_new_tokens were produced -> greedy (first index of the
//           maximum) or temperature -> top-k (ties by index) -> top-p (smallest prefix whose mass reaches p) -> min-p
//           (p >= min_p * p_max) -> one draw from the renormalised prefix.
//   RNG     splitmix64(seed) seeds xorshift64*; one 53-bit uniform per sampled token.
// Implementation: the edits touch few ids, so they are collected as a sparse patch list and applied to a working copy
// of the row; candidates are ordered by ONE 64-bit key per id (order-preserving image of the logit in the high half, the
// inverted index in the low half), so "logit descending, index ascending" is a plain integer order and top-k is an
// nth_element over integers; probabilities are formed once, in that order, and one cumulative walk applies top-p,
// min-p and the draw.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
#include <functional>
#include <limits>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/json.hpp"

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace b2 {

struct SamplingParams {
  double temperature = 1.0, top_p = 1.0, min_p = 0.0;
  long long top_k = -1;           // -1 = off
  double repetition_penalty = 1.0, frequency_penalty = 0.0, presence_penalty = 0.0;
  long long min_new_tokens = 0;
  std::vector<std::pair<int, float>> logit_bias;
  std::vector<int> suppress, stop_ids;
  bool has_seed = false;
  uint64_t seed = 0;

  bool greedy() const { return top_k == 1 || temperature < 1e-6; }

  static SamplingParams from_json(const Json& j) {
    SamplingParams p;
    p.temperature = j.get_double("temperature", 1.0);
    p.top_p = j.get_double("top_p", 1.0);
    p.min_p = j.get_double("min_p", 0.0);
    p.top_k = j.get_int("top_k", -1);
    p.repetition_penalty = j.get_double("repetition_penalty", 1.0);
    p.frequency_penalty = j.get_double("frequency_penalty", 0.0);
    p.presence_penalty = j.get_double("presence_penalty", 0.0);
    p.min_new_tokens = j.get_int("min_new_tokens", 0);
    if (auto s = j.find("seed"); s && s->is_number()) { p.has_seed = true; p.seed = (uint64_t)s->as_int(); }
    if (auto b = j.find("logit_bias"); b && b->is_object())
      for (auto& kv : b->members()) p.logit_bias.emplace_back(std::atoi(kv.first.c_str()), (float)kv.second.as_double());
    if (auto b = j.find("suppress_tokens"); b && b->is_array()) for (auto& v : b->items()) p.suppress.push_back((int)v.as_int());
    if (auto b = j.find("stop_token_ids"); b && b->is_array()) for (auto& v : b->items()) p.stop_ids.push_back((int)v.as_int());
    return p;
  }
};

// Reasoning budget: a thinking block that runs for `limit` tokens without its closing tag gets the tag forced, and the
// block may not be reopened afterwards; from 80 % of the limit an optional bias nudges the model towards closing.
// The block is either not open, open since output index `since_`, or over (closed by the model or by force).
class ReasoningBudget {
 public:
  ReasoningBudget(int limit, double nudge, const int* prompt, int n_prompt, int open_tok, int close_tok)
      : open_tok_(open_tok), close_tok_(close_tok), limit_(limit), nudge_(nudge) {
    // a prompt that ends inside a thinking block (opening tag among its last 16 tokens, no closing tag after it)
    // starts the count at the first produced token
    int opened = -1;
    for (int i = n_prompt - 1; i >= 0 && i >= n_prompt - 16; --i)
      if (prompt[i] == open_tok) { opened = i; break; }
    if (opened >= 0 && std::find(prompt + opened + 1, prompt + n_prompt, close_tok) == prompt + n_prompt) {
      phase_ = Phase::Thinking;
      since_ = 0;
    }
  }

  void accept(long long out_index, int tok) {
    if (phase_ == Phase::Outside && tok == open_tok_) { phase_ = Phase::Thinking; since_ = out_index + 1; }
    else if (phase_ == Phase::Thinking && tok == close_tok_) phase_ = Phase::Over;
  }

  // 0: nothing; 1: force *tok; 2: add *delta to the logit of *tok (-inf masks it)
  int act(long long produced, int* tok, float* delta) {
    switch (phase_) {
      case Phase::Outside:
      case Phase::Over:
        return 0;
      case Phase::OverForced:                 // the block was cut short: the opening tag stays masked
        *tok = open_tok_;
        *delta = -std::numeric_limits<float>::infinity();
        return 2;
      case Phase::Thinking: {
        const long long spent = produced - since_;
        if (spent >= limit_) { phase_ = Phase::OverForced; *tok = close_tok_; return 1; }
        if (nudge_ != 0.0 && (double)spent >= 0.8 * (double)limit_) { *tok = close_tok_; *delta = (float)nudge_; return 2; }
        return 0;
      }
    }
    return 0;
  }

 private:
  enum class Phase { Outside, Thinking, Over, OverForced };
  int open_tok_, close_tok_;
  long long limit_;
  double nudge_;
  Phase phase_ = Phase::Outside;
  long long since_ = 0;
};

// Thinking-block repetition guard: an n-gram seen k times among the n-grams ending in the last w thinking tokens.
class ThinkGuard {
 public:
  ThinkGuard(int n, int k, int w, const int* prompt, int n_prompt, int start, int end)
      : n_(std::max(1, n)), k_(std::max(2, k)), w_(std::max(w, std::max(1, n))), start_(start), end_(end) {
    const int lo = std::max(0, n_prompt - 16);
    int last_start = -1;
    for (int i = lo; i < n_prompt; ++i) if (prompt[i] == start) last_start = i;
    if (last_start >= 0) {
      open_ = true;
      for (int i = last_start + 1; i < n_prompt; ++i) if (prompt[i] == end) open_ = false;
    }
  }
  // Token to emit for the model's choice t; `pending`: t may still be replaced (not yet fed back to the model).
  int filter(int t, bool pending) {
    if (pending && open_ && fired_ >= 0) t = end_;
    push(t);
    return t;
  }
  long long fired() const { return fired_; }
 private:
  void push(int t) {
    if (t == start_ && !open_ && !closed_) { open_ = true; return; }
    if (!open_) return;
    if (t == end_) { open_ = false; closed_ = true; return; }
    ++seen_;
    tail_.push_back(t);
    if ((int)tail_.size() > n_) tail_.pop_front();
    if ((int)tail_.size() < n_) return;
    uint64_t h = 1469598103934665603ull;                       // FNV-1a over the n-gram
    for (int v : tail_) { h ^= (uint32_t)v; h *= 1099511628211ull; }
    hashes_.push_back(h);
    if (++counts_[h] >= k_ && fired_ < 0) fired_ = seen_;
    if ((int)hashes_.size() > w_) {
      const uint64_t old = hashes_.front();
      hashes_.pop_front();
      auto it = counts_.find(old);
      if (it != counts_.end() && --it->second == 0) counts_.erase(it);
    }
  }
  int n_, k_, w_, start_, end_;
  bool open_ = false, closed_ = false;
  std::deque<int> tail_;
  std::deque<uint64_t> hashes_;
  std::unordered_map<uint64_t, int> counts_;
  long long seen_ = 0, fired_ = -1;
};

// splitmix64 finaliser: spreads small or correlated seeds over the whole 64-bit state space
static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

// xorshift64* generator; one 53-bit uniform in [0, 1) per call
struct Xorshift64Star {
  uint64_t state = 1;
  double next() {
    state ^= state >> 12; state ^= state << 25; state ^= state >> 27;
    return (double)((state * 0x2545f4914f6cdd1dull) >> 11) * (1.0 / 9007199254740992.0);
  }
};

// float -> uint32 such that the integer order equals the float order (finite values and infinities)
static inline uint32_t ordered_bits(float v) {
  v += 0.0f;                      // -0.0 and +0.0 compare equal as floats: give them one image
  uint32_t u;
  std::memcpy(&u, &v, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

class Sampler {
 public:
  Sampler(const SamplingParams& p, uint64_t request_id) : p_(p) {
    const uint64_t seed = p.has_seed ? p.seed : (0x1234567ull ^ (request_id * 0x9e3779b97f4a7c15ull));
    rng_.state = splitmix64(seed) | 1;
  }
  double uniform() { return rng_.next(); }
  void accept(int tok) { ++seen_[tok]; ++produced_; }
  long long produced() const { return produced_; }

  // Greedy requests whose logits would not be edited can take the device's argmax: no logits row is needed.
  bool needs_logits(int vocab_valid) const {
    const bool edits = !p_.logit_bias.empty() || p_.repetition_penalty != 1.0 || p_.frequency_penalty != 0.0 ||
                       p_.presence_penalty != 0.0 || (produced_ < p_.min_new_tokens && !p_.stop_ids.empty()) ||
                       std::any_of(p_.suppress.begin(), p_.suppress.end(), [&](int t) { return t < vocab_valid; });
    return edits || !p_.greedy();
  }

  int sample(const float* logits, int n, const std::pair<int, float>* extra, int n_extra) {
    row_.assign(logits, logits + n);
    apply_edits(n, extra, n_extra);
    if (p_.greedy()) return (int)(std::max_element(row_.begin(), row_.end()) - row_.begin());   // first index of the maximum

    // candidates in (logit descending, index ascending) order = descending order of one integer key per id
    keys_.clear();
    for (int i = 0; i < n; ++i)
      if (std::isfinite(row_[i])) keys_.push_back(((uint64_t)ordered_bits(row_[i]) << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i));
    if (keys_.empty()) return 0;
    size_t m = keys_.size();
    if (p_.top_k > 0 && (size_t)p_.top_k < m) {
      m = (size_t)p_.top_k;
      std::nth_element(keys_.begin(), keys_.begin() + (m - 1), keys_.end(), std::greater<uint64_t>());
      keys_.resize(m);
    }
    std::sort(keys_.begin(), keys_.end(), std::greater<uint64_t>());
    auto id_of = [](uint64_t key) { return (int)(0xFFFFFFFFu - (uint32_t)key); };

    // probabilities of the ordered candidates at the request's temperature
    const float temp = (float)p_.temperature;
    const float top = row_[id_of(keys_[0])] / temp;
    prob_.resize(m);
    double total = 0.0;
    for (size_t j = 0; j < m; ++j) { prob_[j] = std::exp((double)(row_[id_of(keys_[j])] / temp - top)); total += prob_[j]; }
    for (size_t j = 0; j < m; ++j) prob_[j] /= total;

    // nucleus: the shortest prefix whose mass reaches top_p; min-p: candidates at least min_p times as likely as the first
    size_t cut = m;
    if (p_.top_p < 1.0) {
      double mass = 0.0;
      for (size_t j = 0; j < m; ++j) { mass += prob_[j]; if (mass >= p_.top_p) { cut = j + 1; break; } }
    }
    if (p_.min_p > 0.0) {
      const double floor_p = prob_[0] * p_.min_p;
      size_t alive = 0;
      while (alive < m && prob_[alive] >= floor_p) ++alive;
      cut = std::min(cut, std::max<size_t>(alive, 1));
    }
    double kept = 0.0;
    for (size_t j = 0; j < cut; ++j) kept += prob_[j];
    double ticket = uniform() * kept;
    for (size_t j = 0; j < cut; ++j) { ticket -= prob_[j]; if (ticket <= 0.0) return id_of(keys_[j]); }
    return id_of(keys_[cut - 1]);
  }

 private:
  // extra bias -> logit_bias -> suppressed ids -> repetition / frequency / presence -> stop ids below min_new_tokens
  void apply_edits(int n, const std::pair<int, float>* extra, int n_extra) {
    auto valid = [n](int t) { return t >= 0 && t < n; };
    for (int i = 0; i < n_extra; ++i) if (valid(extra[i].first)) row_[extra[i].first] += extra[i].second;
    for (const auto& b : p_.logit_bias) if (valid(b.first)) row_[b.first] += b.second;
    for (int t : p_.suppress) if (valid(t)) row_[t] = -INFINITY;
    const float rep = (float)p_.repetition_penalty;
    for (const auto& sc : seen_) {
      if (!valid(sc.first)) continue;
      float v = row_[sc.first];
      if (p_.repetition_penalty != 1.0) v = v > 0.f ? v / rep : v * rep;
      v -= (float)p_.frequency_penalty * (float)sc.second + (sc.second > 0 ? (float)p_.presence_penalty : 0.f);
      row_[sc.first] = v;
    }
    if (produced_ < p_.min_new_tokens) for (int t : p_.stop_ids) if (valid(t)) row_[t] = -INFINITY;
  }

  SamplingParams p_;
  Xorshift64Star rng_;
  std::unordered_map<int, int> seen_;      // produced token -> count
  long long produced_ = 0;
  std::vector<float> row_;
  std::vector<uint64_t> keys_;
  std::vector<double> prob_;
};

}  // namespace b2

using namespace b2;

B2H_API void* b2h_sampler_new(const char* params_json, unsigned long long request_id) {
  try { return new Sampler(SamplingParams::from_json(Json::parse(params_json)), request_id); } catch (...) { return nullptr; }
}
B2H_API void b2h_sampler_free(void* s) { delete static_cast<Sampler*>(s); }
B2H_API int b2h_sampler_sample(void* s, const float* logits, int n, const int* extra_ids, const float* extra_delta, int n_extra) {
  std::vector<std::pair<int, float>> ex;
  for (int i = 0; i < n_extra; ++i) ex.emplace_back(extra_ids[i], extra_delta[i]);
  return static_cast<Sampler*>(s)->sample(logits, n, ex.data(), n_extra);
}
B2H_API void b2h_sampler_accept(void* s, int tok) { static_cast<Sampler*>(s)->accept(tok); }
B2H_API int b2h_sampler_needs_logits(void* s, int vocab_valid) { return static_cast<Sampler*>(s)->needs_logits(vocab_valid) ? 1 : 0; }
B2H_API double b2h_sampler_uniform(void* s) { return static_cast<Sampler*>(s)->uniform(); }

B2H_API void* b2h_budget_new(int n, double soft, const int* prompt, int n_prompt, int start, int end) {
  return new ReasoningBudget(n, soft, prompt, n_prompt, start, end);
}
B2H_API void b2h_budget_free(void* b) { delete static_cast<ReasoningBudget*>(b); }
B2H_API void b2h_budget_accept(void* b, long long out_index, int tok) { static_cast<ReasoningBudget*>(b)->accept(out_index, tok); }
B2H_API int b2h_budget_act(void* b, long long produced, int* tok, float* delta) { return static_cast<ReasoningBudget*>(b)->act(produced, tok, delta); }

B2H_API void* b2h_guard_new(int n, int k, int w, const int* prompt, int n_prompt, int start, int end) {
  return new ThinkGuard(n, k, w, prompt, n_prompt, start, end);
}
B2H_API void b2h_guard_free(void* g) { delete static_cast<ThinkGuard*>(g); }
B2H_API int b2h_guard_filter(void* g, int tok, int pending) { return static_cast<ThinkGuard*>(g)->filter(tok, pending != 0); }
B2H_API long long b2h_guard_fired(void* g) { return static_cast<ThinkGuard*>(g)->fired(); }
