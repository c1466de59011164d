// Host-side token sampler, reasoning budget and thinking-loop guard.
//
// Behavioural contract (reference: crates/agens-cli/src/sampler.rs:170-284, :19-149):
//   order   extra bias -> logit_bias -> suppressed ids (-inf) -> repetition (x > 0 ? x / r : x * r), frequency * count
//           + presence -> stop ids masked while fewer than min_new_tokens were produced -> greedy (first index of the
//           maximum) or temperature -> top-k (ties by index) -> top-p (smallest prefix whose mass reaches p) -> min-p
//           (p >= min_p * p_max) -> one draw from the renormalised prefix.
//   RNG     splitmix64(seed) seeds xorshift64*; one 53-bit uniform per sampled token.
// The implementation keeps a candidate list instead of a dense probability vector, so a draw costs O(vocab) once for
// the filter plus O(k log k) for the kept candidates.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <deque>
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

// Reasoning budget: after n thinking tokens without a closing tag, force the closing tag and forbid reopening.
class ReasoningBudget {
 public:
  ReasoningBudget(int n, double soft, const int* prompt, int n_prompt, int start, int end)
      : start_(start), end_(end), n_(n), soft_(soft) {
    const int lo = std::max(0, n_prompt - 16);
    int last_start = -1;
    for (int i = lo; i < n_prompt; ++i) if (prompt[i] == start) last_start = i;
    if (last_start >= 0) {
      bool ended = false;
      for (int i = last_start + 1; i < n_prompt; ++i) if (prompt[i] == end) ended = true;
      if (!ended) open_at_ = 0;
    }
  }
  void accept(long long out_index, int tok) {
    if (tok == start_) { if (open_at_ < 0 && !closed_) open_at_ = out_index + 1; }
    else if (tok == end_ && open_at_ >= 0) { open_at_ = -1; closed_ = true; }
  }
  // 0: nothing; 1: force *tok; 2: add *delta to logit of *tok (-inf masks)
  int act(long long produced, int* tok, float* delta) {
    if (closed_) {
      if (forced_) { *tok = start_; *delta = -std::numeric_limits<float>::infinity(); return 2; }
      return 0;
    }
    if (open_at_ < 0) return 0;
    const long long k = produced - open_at_;
    if (k >= n_) { forced_ = closed_ = true; open_at_ = -1; *tok = end_; return 1; }
    if (soft_ != 0.0 && (double)k >= 0.8 * n_) { *tok = end_; *delta = (float)soft_; return 2; }
    return 0;
  }
 private:
  int start_, end_;
  long long n_;
  double soft_;
  long long open_at_ = -1;
  bool closed_ = false, forced_ = false;
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

class Sampler {
 public:
  Sampler(const SamplingParams& p, uint64_t request_id) : p_(p) {
    uint64_t seed = p.has_seed ? p.seed : (0x1234567ull ^ (request_id * 0x9e3779b97f4a7c15ull));
    uint64_t z = seed + 0x9e3779b97f4a7c15ull;                 // splitmix64: small seeds must not correlate
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    rng_ = z | 1;
  }
  double uniform() {                                             // xorshift64*
    rng_ ^= rng_ >> 12; rng_ ^= rng_ << 25; rng_ ^= rng_ >> 27;
    return (double)((rng_ * 0x2545f4914f6cdd1dull) >> 11) / (double)(1ull << 53);
  }
  void accept(int tok) { ++counts_[tok]; ++produced_; }
  long long produced() const { return produced_; }
  bool needs_logits(int vocab_valid) const {
    if (!p_.greedy() || !p_.logit_bias.empty() || p_.repetition_penalty != 1.0 || p_.frequency_penalty != 0.0 ||
        p_.presence_penalty != 0.0) return true;
    if (produced_ < p_.min_new_tokens && !p_.stop_ids.empty()) return true;
    for (int t : p_.suppress) if (t < vocab_valid) return true;
    return false;
  }
  int sample(const float* logits, int n, const std::pair<int, float>* extra, int n_extra) {
    x_.assign(logits, logits + n);
    auto in = [&](int t) { return t >= 0 && t < n; };
    for (int i = 0; i < n_extra; ++i) if (in(extra[i].first)) x_[extra[i].first] += extra[i].second;
    for (auto& b : p_.logit_bias) if (in(b.first)) x_[b.first] += b.second;
    for (int t : p_.suppress) if (in(t)) x_[t] = -INFINITY;
    for (auto& kv : counts_) {
      if (!in(kv.first)) continue;
      float& v = x_[kv.first];
      if (p_.repetition_penalty != 1.0) { const float r = (float)p_.repetition_penalty; v = v > 0.f ? v / r : v * r; }
      v -= (float)p_.frequency_penalty * (float)kv.second + (kv.second > 0 ? (float)p_.presence_penalty : 0.f);
    }
    if (produced_ < p_.min_new_tokens) for (int t : p_.stop_ids) if (in(t)) x_[t] = -INFINITY;
    if (p_.greedy()) {
      int best = 0;
      for (int i = 1; i < n; ++i) if (x_[i] > x_[best]) best = i;
      return best;
    }
    idx_.clear();
    for (int i = 0; i < n; ++i) if (std::isfinite(x_[i])) idx_.push_back(i);
    if (idx_.empty()) return 0;
    auto by_logit = [&](int a, int b) { return x_[a] > x_[b] || (x_[a] == x_[b] && a < b); };
    size_t k = p_.top_k > 0 ? std::min<size_t>((size_t)p_.top_k, idx_.size()) : idx_.size();
    if (k < idx_.size()) { std::nth_element(idx_.begin(), idx_.begin() + (k - 1), idx_.end(), by_logit); idx_.resize(k); }
    std::sort(idx_.begin(), idx_.end(), by_logit);
    const float t = (float)p_.temperature;
    const float mx = x_[idx_[0]] / t;
    pr_.resize(idx_.size());
    double z = 0;
    for (size_t j = 0; j < idx_.size(); ++j) { pr_[j] = std::exp((double)(x_[idx_[j]] / t - mx)); z += pr_[j]; }
    for (auto& v : pr_) v /= z;
    size_t keep = pr_.size();
    if (p_.top_p < 1.0) {
      double c = 0;
      for (size_t j = 0; j < pr_.size(); ++j) { c += pr_[j]; if (c >= p_.top_p) { keep = j + 1; break; } }
    }
    if (p_.min_p > 0.0) {
      const double thr = pr_[0] * p_.min_p;
      size_t cnt = 0;
      while (cnt < pr_.size() && pr_[cnt] >= thr) ++cnt;
      keep = std::min(keep, std::max<size_t>(cnt, 1));
    }
    double zz = 0;
    for (size_t j = 0; j < keep; ++j) zz += pr_[j];
    double u = uniform() * zz;
    for (size_t j = 0; j < keep; ++j) { u -= pr_[j]; if (u <= 0.0) return idx_[j]; }
    return idx_[keep - 1];
  }
 private:
  SamplingParams p_;
  uint64_t rng_;
  std::unordered_map<int, int> counts_;
  long long produced_ = 0;
  std::vector<float> x_;
  std::vector<int> idx_;
  std::vector<double> pr_;
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
