// Host model of the push collectives' inbox protocol (collectives.cu), run on CPU threads: one thread per rank, inboxes
// in ordinary memory as relaxed atomics.  It restates what the kernels do to the inboxes and nothing else:
//
//   * a slot holds one contribution per source rank; a 16-byte unit of four words is "not written yet" while any word
//     is the sentinel (the bit pattern of -0.0f), and data never contains the sentinel (-0.0 is stored as +0.0);
//   * the four words of a unit may land in any order (a peer store is not assumed to be atomic as a whole);
//   * the rotating calls (all-reduce, all-gather, reduce-scatter, barrier) take slots first + call % 3 and re-arm, at the
//     end of call k, the slot of call k - 1 over the extent that call used;
//   * the fused row-parallel linear takes slot pairs 2 * (call % 3), its readers re-arm every unit right after reading;
//   * every wait is bounded; a wait that runs out sets the rank's status word and the call completes with zeros;
//   * a thread pushes its unit before it waits for it and takes its units in ascending order on every rank (ranks that
//     took units in different orders could wait for each other's pushes for ever).
//
// The model checks the claim the kernels rely on: with these rules no rank can overwrite or re-arm a unit that another
// rank still has to read, however far the ranks drift apart (a rank cannot finish call k before every rank has
// started it, so ranks are at most one call apart).  Ranks are delayed at random points; results are compared with the
// exact sums.  A lost message (a rank that skips its pushes in one call) must show as a time-out status on every rank
// that waited for it, and the deployment's recovery (all ranks idle, every inbox re-armed) must make the following
// calls exact again.  Built into the host library; tests run it with 2 to 8 ranks, development also under
// ThreadSanitizer.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint32_t kSentinel = 0x80000000u;
constexpr int kMaxRanks = 8;

struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x1234567ull) {}
  uint64_t next() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; }
  int below(int n) { return (int)(next() % (uint64_t)n); }
};

uint32_t bits_of(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
float float_of(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

struct World {
  int size = 0, n_slots = 0;
  long slot_stride = 0;                                   // words per source rank inside a slot
  long slot_words = 0;                                    // words per slot (all sources)
  std::vector<std::unique_ptr<std::atomic<uint32_t>[]>> inbox;   // one region per rank
  std::atomic<int> status[kMaxRanks];
  std::atomic<int> arrived_at_barrier{0};
  std::atomic<int> barrier_gen{0};
  long timeout_us = 0;
  std::atomic<uint32_t>* unit(int rank, int slot, int src, long e) { return inbox[rank].get() + (long)slot * slot_words + (long)src * slot_stride + e; }
};

void host_barrier(World& w) {                              // the deployment's own (host side) barrier, used by recovery only
  const int gen = w.barrier_gen.load();
  if (w.arrived_at_barrier.fetch_add(1) + 1 == w.size) { w.arrived_at_barrier.store(0); w.barrier_gen.fetch_add(1); }
  else while (w.barrier_gen.load() == gen) std::this_thread::yield();
}

// A peer store of one unit: four relaxed word stores in a random order, -0.0 turned into +0.0.
void push_unit(std::atomic<uint32_t>* p, const float v[4], Rng& r) {
  const int first = r.below(4);
  for (int k = 0; k < 4; ++k) {
    const int j = (first + k) & 3;
    p[j].store(bits_of(v[j] + 0.f), std::memory_order_relaxed);
    if (r.below(16) == 0) std::this_thread::yield();
  }
}
using Clock = std::chrono::steady_clock;
// The deadline counts from the start of the call (the kernel's t_start), not from the start of this wait.
bool wait_unit(World& w, std::atomic<uint32_t>* p, float v[4], Clock::time_point t0) {
  unsigned spins = 0;
  for (;;) {
    uint32_t u[4];
    bool ok = true;
    for (int j = 0; j < 4; ++j) { u[j] = p[j].load(std::memory_order_relaxed); ok = ok && u[j] != kSentinel; }
    if (ok) { for (int j = 0; j < 4; ++j) v[j] = float_of(u[j]); return true; }
    if ((++spins & 63u) == 0u) {
      if (std::chrono::duration_cast<std::chrono::microseconds>(Clock::now() - t0).count() > w.timeout_us) break;
      std::this_thread::yield();
    }
  }
  for (int j = 0; j < 4; ++j) v[j] = 0.f;
  return false;
}
void clear_unit(std::atomic<uint32_t>* p) { for (int j = 0; j < 4; ++j) p[j].store(kSentinel, std::memory_order_relaxed); }

// The value rank `src` contributes to element e of call c for destination chunk d (small integers: sums are exact).
float contribution(int src, int call, long e, int d) { return (float)(((src + 1) * 7 + call * 3 + e * 5 + d * 11) % 61 - 30); }

struct Outcome { long wrong = 0, timeouts = 0; };

enum Kind { kAllReduce = 0, kAllGather = 1, kReduceScatter = 2, kBarrier = 3 };

// One rotating call of rank `me` (push_collective_kernel): slot `cur`, re-arm `prev` over prev_units afterwards.
void rotating_call(World& w, int me, int call, Kind kind, long units, int cur, int prev, long prev_units, bool skip_push, Rng& r, Outcome& o) {
  const auto t0 = Clock::now();
  // A kernel's threads each push their unit and then wait for it, and a thread takes its units in ascending order, the
  // same on every rank.  The model runs `window` such threads: units up to i + window - 1 are pushed before unit i is
  // waited for (a different window on every rank and call).
  const long window = 1 + r.below(8);
  long pushed = 0;
  for (long i = 0; i < units; ++i) {
    const long e = i * 4;
    for (; pushed < units && pushed < i + window; ++pushed) {
      if (skip_push) continue;
      for (int dst = 0; dst < w.size; ++dst) {
        float v[4];
        for (int j = 0; j < 4; ++j) v[j] = kind == kBarrier ? 1.f : contribution(me, call, pushed * 4 + j, kind == kReduceScatter ? dst : 0);
        push_unit(w.unit(dst, cur, me, pushed * 4), v, r);
      }
    }
    float s[4] = {0, 0, 0, 0};
    for (int src = 0; src < w.size; ++src) {
      float v[4];
      if (!wait_unit(w, w.unit(me, cur, src, e), v, t0)) { ++o.timeouts; w.status[me].store(1); continue; }
      for (int j = 0; j < 4; ++j) {
        if (kind == kAllGather || kind == kBarrier) {
          const float want = kind == kBarrier ? 1.f : contribution(src, call, e + j, 0);
          if (v[j] != want) ++o.wrong;
        }
        s[j] += v[j];
      }
    }
    if (kind == kAllReduce || kind == kReduceScatter) {
      for (int j = 0; j < 4; ++j) {
        float want = 0;
        for (int src = 0; src < w.size; ++src) want += contribution(src, call, e + j, kind == kReduceScatter ? me : 0);
        if (s[j] != want && w.status[me].load() == 0) ++o.wrong;
      }
    }
    if (r.below(8) == 0) std::this_thread::yield();
  }
  if (prev >= 0)
    for (long i = 0; i < prev_units; ++i)
      for (int src = 0; src < w.size; ++src) clear_unit(w.unit(me, prev, src, i * 4));
}

// One fused row-parallel linear of rank `me`: the GEMM epilogue's stores into the owners' slot A, then
// collect_gather_kernel: combine my rows, hand the sums on through slot B, take the peers' rows; readers re-arm.
void fused_call(World& w, int me, int call, long units_per_rank, int slot_a, Rng& r, Outcome& o) {
  const int slot_b = slot_a + 1;
  const auto t0 = Clock::now();
  for (int owner = 0; owner < w.size; ++owner)            // epilogue: my partial of every owner's rows
    for (long i = 0; i < units_per_rank; ++i) {
      float v[4];
      for (int j = 0; j < 4; ++j) v[j] = contribution(me, call, i * 4 + j, owner);
      push_unit(w.unit(owner, slot_a, me, i * 4), v, r);
    }
  for (long i = 0; i < units_per_rank; ++i) {             // my rows
    const long e = i * 4;
    float s[4] = {0, 0, 0, 0};
    for (int src = 0; src < w.size; ++src) {
      float v[4];
      std::atomic<uint32_t>* p = w.unit(me, slot_a, src, e);
      if (!wait_unit(w, p, v, t0)) { ++o.timeouts; w.status[me].store(1); }
      clear_unit(p);
      for (int j = 0; j < 4; ++j) s[j] += v[j];
    }
    for (int j = 0; j < 4; ++j) {
      float want = 0;
      for (int src = 0; src < w.size; ++src) want += contribution(src, call, e + j, me);
      if (s[j] != want && w.status[me].load() == 0) ++o.wrong;
    }
    for (int dst = 0; dst < w.size; ++dst)
      if (dst != me) push_unit(w.unit(dst, slot_b, me, e), s, r);
  }
  for (int k = 1; k < w.size; ++k) {                      // the peers' rows
    const int src = (me + k) % w.size;
    for (long i = 0; i < units_per_rank; ++i) {
      float v[4];
      std::atomic<uint32_t>* p = w.unit(me, slot_b, src, i * 4);
      if (!wait_unit(w, p, v, t0)) { ++o.timeouts; w.status[me].store(1); }
      clear_unit(p);
      for (int j = 0; j < 4; ++j) {
        float want = 0;
        for (int q = 0; q < w.size; ++q) want += contribution(q, call, i * 4 + j, src);
        if (v[j] != want && w.status[me].load() == 0) ++o.wrong;
      }
    }
  }
}

}  // namespace

// Runs `calls` collective calls on `ranks` threads.  mode 0: the rotating calls (kinds and sizes drawn from the seed,
// the same on every rank); mode 1: the fused row-parallel linear; mode 2: the rotating calls over two slots instead of
// three, a broken variant that the checks must catch (the slot a call re-arms is the one a faster peer already writes
// for the next call).  lose_rank >= 0: that rank skips its pushes in call
// lose_call (rotating mode); every rank that timed out must say so, then all ranks re-arm their inboxes behind a host
// barrier and the rest of the calls must be exact.  Returns 0 when every check held; report gets one line of counts.
B2H_API int b2h_comm_model_run(int ranks, int calls, int max_units, unsigned seed, int mode, int lose_rank, int lose_call,
                               int timeout_ms, char* report, int cap) {
  if (ranks < 1 || ranks > kMaxRanks || calls < 1 || max_units < 1 || max_units > 4096) return -1;
  World w;
  w.size = ranks;
  w.n_slots = mode == 1 ? 6 : 3;
  w.slot_stride = (long)max_units * 4;
  w.slot_words = w.slot_stride * ranks;
  w.timeout_us = (long)timeout_ms * 1000;
  for (int r = 0; r < ranks; ++r) {
    w.inbox.emplace_back(new std::atomic<uint32_t>[(size_t)w.slot_words * w.n_slots]);
    for (long i = 0; i < w.slot_words * w.n_slots; ++i) w.inbox[r][i].store(kSentinel, std::memory_order_relaxed);
    w.status[r].store(0);
  }
  std::vector<Outcome> out(ranks);
  std::vector<long> lost_seen(ranks, 0), late_timeouts(ranks, 0);
  std::vector<std::thread> th;
  for (int me = 0; me < ranks; ++me)
    th.emplace_back([&, me]() {
      Rng plan(seed);                                       // the same call sequence on every rank
      Rng jitter(seed * 977u + (unsigned)me * 131u + 7u);   // a different schedule on every rank
      long prev_units = 0;
      int rotation = 0;                                     // calls since the last recovery
      for (int c = 0; c < calls; ++c) {
        const Kind kind = (Kind)plan.below(4);
        const long units = kind == kBarrier ? 1 : 1 + plan.below(max_units);
        if (jitter.below(3) == 0) std::this_thread::sleep_for(std::chrono::microseconds(jitter.below(300)));
        if (mode == 1) {
          fused_call(w, me, c, units, 2 * (c % 3), jitter, out[me]);
          continue;
        }
        const int nrot = mode == 2 ? 2 : 3;                  // mode 2: a rotation over two slots, which is not enough
        const int cur = rotation % nrot, prev = rotation == 0 ? -1 : (rotation - 1) % nrot;
        const long before = out[me].timeouts;
        rotating_call(w, me, c, kind, units, cur, prev, prev_units, me == lose_rank && c == lose_call, jitter, out[me]);
        prev_units = units;
        ++rotation;
        if (lose_rank >= 0 && c == lose_call) {
          // what the deployment does after a status word reports a time-out: every rank goes idle, re-arms its whole
          // inbox and starts the rotation again
          lost_seen[me] = out[me].timeouts - before;
          host_barrier(w);
          for (long i = 0; i < w.slot_words * w.n_slots; ++i) w.inbox[me][i].store(kSentinel, std::memory_order_relaxed);
          w.status[me].store(0);
          host_barrier(w);
          rotation = 0;
          prev_units = 0;
        } else if (out[me].timeouts != before) {
          late_timeouts[me] += out[me].timeouts - before;
        }
      }
    });
  for (auto& t : th) t.join();
  long wrong = 0, late = 0, seen = 0;
  for (int r = 0; r < ranks; ++r) { wrong += out[r].wrong; late += late_timeouts[r]; seen += lost_seen[r] > 0; }
  const bool lost_ok = lose_rank < 0 || ranks == 1 || seen == ranks;     // every rank waited for the lost message
  if (report && cap > 0) snprintf(report, (size_t)cap, "ranks %d calls %d wrong %ld unexpected_timeouts %ld ranks_that_saw_the_loss %ld", ranks, calls, wrong, late, seen);
  return (wrong == 0 && late == 0 && lost_ok) ? 0 : 1;
}
