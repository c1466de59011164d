// Per-GPU memory-budget planner and deployment profiles.
//
// The contract follows the reference (crates/agens-cli/src/plan.rs:14-241, m1.rs:502-541, 905-974, profile.rs:10-88):
// a hard per-GPU budget is split into measured weights + context, an itemised scratch estimate and a runtime-growth
// reserve; what is left becomes the paged KV pool; if the pool cannot hold the wanted context, KV pages are tiered to
// pinned host memory (capped by the pinnable host RAM) and the context is clamped rather than the load failing; ranks
// take the minimum.  Differences: pages of 16 tokens instead of rows, every layer is dense attention, and the cap is
// enforced on the host by the loader's budget ledger (serve/budget.py: every device allocation of a deployment is
// booked against the budget and refused past it) instead of a ballast allocation: the GPUs are shared.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>

#include "../core/json.hpp"

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace b2 {

static const double GiB = 1024.0 * 1024.0 * 1024.0;

struct PlanIn {
  double budget_gib = 0;            // 0 = no budget: use gpu_free_gib minus headroom
  double gpu_free_gib = 170;
  double headroom_gib = 8;          // kept free when no budget is given (reference auto_pool: 8 GiB)
  long long weights_bytes = 0;      // measured after upload (weights + CUDA context)
  long long kv_bytes_per_token = 0; // this rank's share
  int page_size = 16;
  int max_batch = 8, sessions = 8;
  int prefill_chunk = 8192;
  int d_model = 5120, ffn = 25600, q_dim = 8192, kv_dim = 1024, vocab = 151936, n_heads = 64, head_dim = 128;
  int tp = 1;
  long long wctx = 262148;          // wanted context per conversation
  double host_avail_gib = -1;       // < 0: read /proc/meminfo
  double host_headroom_gib = 8;
  bool allow_host_tier = true;
  int resident_window_pages = 0;    // pages of a tiered conversation that always stay on the GPU (0 = auto)
  int split_keys = 64;              // keys per attention split: the partial buffers hold wctx / split_keys splits per (row, head)
};

static PlanIn parse_in(const Json& j) {
  PlanIn p;
  p.budget_gib = j.get_double("budget_gib", 0);
  p.gpu_free_gib = j.get_double("gpu_free_gib", 170);
  p.headroom_gib = j.get_double("headroom_gib", 8);
  p.weights_bytes = j.get_int("weights_bytes", 0);
  p.kv_bytes_per_token = j.get_int("kv_bytes_per_token", 0);
  p.page_size = (int)j.get_int("page_size", 16);
  p.max_batch = (int)j.get_int("max_batch", 8);
  p.sessions = (int)j.get_int("sessions", 8);
  p.prefill_chunk = (int)j.get_int("prefill_chunk", 8192);
  p.d_model = (int)j.get_int("d_model", 5120);
  p.ffn = (int)j.get_int("ffn", 25600);
  p.q_dim = (int)j.get_int("q_dim", 8192);
  p.kv_dim = (int)j.get_int("kv_dim", 1024);
  p.vocab = (int)j.get_int("vocab", 151936);
  p.n_heads = (int)j.get_int("n_heads", 64);
  p.head_dim = (int)j.get_int("head_dim", 128);
  p.tp = (int)j.get_int("tp", 1);
  p.wctx = j.get_int("wctx", 262148);
  p.host_avail_gib = j.get_double("host_avail_gib", -1);
  p.host_headroom_gib = j.get_double("host_headroom_gib", 8);
  p.allow_host_tier = j.get_bool("allow_host_tier", true);
  p.resident_window_pages = (int)j.get_int("resident_window_pages", 0);
  p.split_keys = std::max(16, (int)j.get_int("split_keys", 64));
  // sizes the arithmetic below divides by or multiplies together
  auto in_range = [](long long v, long long lo, long long hi, const char* name) {
    if (v < lo || v > hi) throw std::runtime_error(std::string("plan: ") + name + " out of range");
  };
  in_range(p.tp, 1, 64, "tp");
  in_range(p.page_size, 1, 1 << 16, "page_size");
  in_range(p.max_batch, 1, 1 << 16, "max_batch");
  in_range(p.sessions, 0, 1 << 20, "sessions");
  in_range(p.prefill_chunk, 1, 1 << 22, "prefill_chunk");
  in_range(p.d_model, 1, 1 << 20, "d_model");
  in_range(p.ffn, 1, 1 << 24, "ffn");
  in_range(p.q_dim, 1, 1 << 24, "q_dim");
  in_range(p.kv_dim, 1, 1 << 24, "kv_dim");
  in_range(p.vocab, 1, 1 << 26, "vocab");
  in_range(p.n_heads, 1, 1 << 16, "n_heads");
  in_range(p.head_dim, 1, 1 << 16, "head_dim");
  in_range(p.wctx, 1, 1ll << 32, "wctx");
  in_range(p.weights_bytes, 0, 1ll << 50, "weights_bytes");
  in_range(p.kv_bytes_per_token, 0, 1ll << 32, "kv_bytes_per_token");
  in_range(p.resident_window_pages, 0, 1 << 30, "resident_window_pages");
  for (double g : {p.budget_gib, p.gpu_free_gib, p.headroom_gib, p.host_headroom_gib})
    if (!(g == g) || g < -1e6 || g > 1e6) throw std::runtime_error("plan: a GiB figure is out of range");
  if (!(p.host_avail_gib == p.host_avail_gib) || p.host_avail_gib > 1e6) throw std::runtime_error("plan: host_avail_gib out of range");
  return p;
}

// MemAvailable of the machine (or the cgroup limit when that is lower), in bytes; -1 when unknown.
static long long host_mem_available() {
  long long avail = -1;
  std::ifstream f("/proc/meminfo");
  std::string k;
  long long v;
  std::string unit;
  while (f >> k >> v) {
    std::getline(f, unit);
    if (k == "MemAvailable:") { avail = v * 1024; break; }
  }
  std::ifstream c("/sys/fs/cgroup/memory.max");
  std::string s;
  if (c >> s && s != "max") {
    const long long lim = std::atoll(s.c_str());
    std::ifstream u("/sys/fs/cgroup/memory.current");
    long long cur = 0;
    u >> cur;
    if (lim > 0 && (avail < 0 || lim - cur < avail)) avail = std::max(0ll, lim - cur);
  }
  return avail;
}

// Runtime growth that is not under the planner's control (lazily loaded modules, graphs): base + per batch row.
static long long runtime_reserve(int max_batch) {
  return (long long)(850e6) + (long long)std::min(max_batch, 64) * 6000000ll;
}

static Json scratch_items(const PlanIn& p) {
  const long long T = p.prefill_chunk;
  Json it = Json::object();
  const long long shard_ffn = p.ffn / p.tp, shard_q = p.q_dim / p.tp, shard_kv = p.kv_dim / p.tp;
  it.set("prefill_activations", (long long)(T * (2ll * p.d_model + shard_q + 2 * shard_kv + shard_q + 3ll * shard_ffn) * 2));
  it.set("dequant_tile", (long long)std::max<long long>((long long)p.d_model * 2 * shard_ffn * 2, 64ll << 20));
  // split partials of the decode / verify attention: [rows][heads][splits][head_dim + (max, sum)] fp32, rows = eight per
  // sequence slot between 32 and 128, splits = wanted context / keys per split
  const long long rows = std::min(128, std::max(32, 8 * p.max_batch));
  const long long splits = (p.wctx + p.split_keys - 1) / p.split_keys;
  it.set("attention_partials", (long long)(rows * (p.n_heads / p.tp) * splits * (p.head_dim + 2) * 4));
  it.set("gemv_scratch", (long long)(64ll << 20));
  it.set("logits", (long long)32 * (p.vocab / p.tp) * 4);
  // per-step inboxes of the fused decode all-reduce, plus the inbox of the fused GEMM + reduce-scatter of prefill chunks:
  // six slots of (chunk + 32) rows x d_model fp32 over all source ranks together
  it.set("tp_inboxes", (long long)(p.tp > 1 ? 129ll * p.tp * 32 * p.d_model * 4 + 6ll * (T + 32 + p.tp) * p.d_model * 4 : 0));
  it.set("runtime_reserve", runtime_reserve(p.max_batch));
  return it;
}

static Json plan(const PlanIn& p) {
  Json out = Json::object();
  Json lines = Json::array();
  char buf[256];
  const double budget = p.budget_gib > 0 ? p.budget_gib : std::max(0.0, p.gpu_free_gib - p.headroom_gib);
  const long long budget_b = (long long)(budget * GiB);
  Json scratch = scratch_items(p);
  long long scratch_b = 0;
  for (auto& kv : scratch.members()) scratch_b += kv.second.as_int();
  const long long fixed = p.weights_bytes + scratch_b;
  const long long page_b = p.kv_bytes_per_token * p.page_size;
  long long pool_pages = page_b > 0 ? std::max(0ll, budget_b - fixed) / page_b : 0;
  const long long want_pages = (p.wctx + p.page_size - 1) / p.page_size;
  snprintf(buf, sizeof buf, "plan: budget %.2f GiB, weights+context %.2f GiB, scratch %.2f GiB", budget, p.weights_bytes / GiB, scratch_b / GiB);
  lines.push_back(std::string(buf));
  std::string tier = "gpu";
  long long host_pages = 0;
  long long context = p.wctx;
  if (pool_pages < want_pages) {
    if (p.allow_host_tier) {
      tier = "host";
      const double avail = p.host_avail_gib >= 0 ? p.host_avail_gib : (host_mem_available() >= 0 ? host_mem_available() / GiB : 0);
      const long long pinnable = (long long)(std::max(0.0, avail - p.host_headroom_gib) * GiB);
      host_pages = page_b > 0 ? std::min(want_pages * std::max(1, p.sessions), pinnable / page_b) : 0;
      // one full context at most per conversation on the host; the GPU keeps the working set
      const long long total_pages = pool_pages + host_pages;
      if (total_pages < want_pages) {
        context = total_pages * p.page_size;
        snprintf(buf, sizeof buf, "plan: context clamped from %lld to %lld tokens (GPU pool %lld + host %lld pages)", p.wctx, context, pool_pages, host_pages);
        lines.push_back(std::string(buf));
      }
      snprintf(buf, sizeof buf, "plan: KV tiered to pinned host memory: %lld pages (%.2f GiB of %.2f GiB pinnable)", host_pages, host_pages * (double)page_b / GiB, pinnable / GiB);
      lines.push_back(std::string(buf));
    } else {
      context = pool_pages * p.page_size;
      snprintf(buf, sizeof buf, "plan: context clamped from %lld to %lld tokens (no host tier)", p.wctx, context);
      lines.push_back(std::string(buf));
    }
  }
  snprintf(buf, sizeof buf, "plan: KV pool %lld pages of %d tokens (%.2f GiB, %lld tokens) on the GPU", pool_pages, p.page_size, pool_pages * (double)page_b / GiB, pool_pages * p.page_size);
  lines.push_back(std::string(buf));
  const int window = p.resident_window_pages > 0 ? p.resident_window_pages : (int)std::min<long long>(pool_pages / std::max(1, p.sessions), want_pages);
  out.set("budget_bytes", budget_b);
  out.set("fixed_bytes", fixed);
  out.set("scratch", scratch);
  out.set("page_bytes", page_b);
  out.set("pool_pages", pool_pages);
  out.set("pool_tokens", pool_pages * p.page_size);
  out.set("tier", tier);
  out.set("host_pages", host_pages);
  out.set("resident_window_pages", window);
  out.set("context", context);
  out.set("fits", fixed <= budget_b);
  out.set("lines", lines);
  return out;
}

// Deployment profiles: name -> flags and environment defaults (reference profile.rs:41-76), plus a B200 profile.
static Json profile(const std::string& name, int tp) {
  Json o = Json::object();
  Json flags = Json::object(), env = Json::object();
  if (tp != 1 && tp != 2 && tp != 4 && tp != 8) throw std::runtime_error("--tp must be 1, 2, 4 or 8");
  if (name == "12gb") {
    flags.set("budget_gib", 12); flags.set("wctx", 65540); flags.set("mode", "personal"); flags.set("no_fork", 1); flags.set("spec_copy", 1);
    env.set("B200E_KV_TIER", "host");
  } else if (name == "16gb") {
    flags.set("budget_gib", 16); flags.set("wctx", 262148); flags.set("mode", "personal"); flags.set("no_fork", 1);
    env.set("B200E_KV_TIER", "host");
  } else if (name == "24gb") {
    flags.set("budget_gib", 23); flags.set("wctx", 262148); flags.set("mode", "server"); flags.set("max_batch", 4); flags.set("max_convs", 4); flags.set("sessions", 4);
  } else if (name == "48gb") {
    flags.set("budget_gib", 46); flags.set("wctx", 262148); flags.set("mode", "server"); flags.set("max_batch", 16); flags.set("max_convs", 16); flags.set("sessions", 16);
  } else if (name == "b200") {
    flags.set("budget_gib", 168); flags.set("wctx", 262148); flags.set("mode", "server"); flags.set("max_batch", 64); flags.set("max_convs", 64); flags.set("sessions", 64);
  } else {
    throw std::runtime_error("unknown profile: " + name + " (12gb, 16gb, 24gb, 48gb, b200)");
  }
  flags.set("tp", tp);
  o.set("flags", flags);
  o.set("env", env);
  return o;
}

}  // namespace b2

using namespace b2;

static char* dup_out(const std::string& s) {
  char* p = (char*)std::malloc(s.size() + 1);
  std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}

B2H_API void b2h_free_str(char* p) { std::free(p); }

// JSON in, JSON out; on error returns {"error": "..."}; free the result with b2h_free_str.
B2H_API char* b2h_plan(const char* in_json) {
  try { return dup_out(plan(parse_in(Json::parse(in_json))).dump()); }
  catch (const std::exception& e) { Json o = Json::object(); o.set("error", std::string(e.what())); return dup_out(o.dump()); }
}
B2H_API char* b2h_profile(const char* name, int tp) {
  try { return dup_out(profile(name, tp).dump()); }
  catch (const std::exception& e) { Json o = Json::object(); o.set("error", std::string(e.what())); return dup_out(o.dump()); }
}
B2H_API long long b2h_host_mem_available() { return host_mem_available(); }
