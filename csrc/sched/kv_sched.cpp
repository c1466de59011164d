// Host-side KV bookkeeping and scheduling policy: refcounted page allocator with fork, banker's-algorithm admission,
// eviction order, SRPT chunk scheduling, copy-from-context drafter and the hash-chained prefix cache.
//
// Reference behaviour restated here: alloc_row / own_partial_page / fork (kernels/m1/m1_model.cu:1694-1716, 4526-4585,
// 4869), KvPolicy + kv_safe + victim + prefill order (crates/agens-cli/src/serve.rs:343-422, 616-639), Lookup
// (crates/agens-cli/src/lookup.rs:107-201) and PrefixCache (crates/agens-cli/src/prefix.rs).  Pages hold 16 tokens
// here (the reference allocates single rows), so fork shares whole pages and copies at most one partial page.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <list>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace b2 {

// ------------------------------------------------------------------------------------------------ page allocator
class PageAllocator {
 public:
  PageAllocator(int n_pages, int page_size) : page_size_(page_size), ref_(n_pages, 0) {
    for (int i = n_pages - 1; i >= 0; --i) free_.push_back(i);
  }
  int free_pages() const { return (int)free_.size(); }
  int n_pages() const { return (int)ref_.size(); }
  int new_seq() { int id = next_id_++; seqs_[id] = Seq(); return id; }
  bool has(int s) const { return seqs_.count(s) != 0; }
  int seq_len(int s) const { return seqs_.at(s).len; }
  // Grow `s` to hold n_tokens; returns number of pages newly taken, -1 if the pool cannot serve it (nothing changes).
  int reserve(int s, int n_tokens) {
    Seq& q = seqs_.at(s);
    const int need = (n_tokens + page_size_ - 1) / page_size_;
    const int extra = need - (int)q.pages.size();
    if (extra <= 0) return 0;
    if (extra > (int)free_.size()) return -1;
    for (int i = 0; i < extra; ++i) { int p = free_.back(); free_.pop_back(); ref_[p] = 1; q.pages.push_back(p); }
    return extra;
  }
  void set_len(int s, int n) { seqs_.at(s).len = n; }
  // Drop everything past n_tokens (rejected speculative rows); returns pages released.
  int truncate(int s, int n_tokens) {
    Seq& q = seqs_.at(s);
    q.len = std::min(q.len, n_tokens);
    const int keep = (n_tokens + page_size_ - 1) / page_size_;
    int rel = 0;
    while ((int)q.pages.size() > keep) { rel += unref(q.pages.back()); q.pages.pop_back(); }
    return rel;
  }
  // Host tier: the page at `index` of the sequence moved to host memory; its GPU page goes back to the pool and the
  // position is marked kHostPage.  Returns 1 if a page was freed.
  static constexpr int kHostPage = -2;
  int evict_page(int s, int index) {
    Seq& q = seqs_.at(s);
    if (index < 0 || index >= (int)q.pages.size() || q.pages[index] < 0) return 0;
    const int rel = unref(q.pages[index]);
    q.pages[index] = kHostPage;
    return rel;
  }
  // Fork: the child shares all full pages; a partial last page must be copied by the caller into the page returned in
  // *copy_dst (source page in *copy_src), -1 when no copy is needed.  Returns the child id, -1 when no page is free.
  int fork(int s, int* copy_src, int* copy_dst) {
    const Seq& q = seqs_.at(s);
    *copy_src = *copy_dst = -1;
    for (int p : q.pages) if (p < 0) return -1;          // sequences with pages in the host tier do not fork
    const bool partial = q.len % page_size_ != 0;
    if (partial && free_.empty()) return -1;
    const int id = next_id_++;
    Seq c;
    c.len = q.len;
    const int used = (q.len + page_size_ - 1) / page_size_;
    for (int i = 0; i < used; ++i) {
      if (i == used - 1 && partial) {
        int p = free_.back(); free_.pop_back(); ref_[p] = 1;
        *copy_src = q.pages[i]; *copy_dst = p;
        c.pages.push_back(p);
      } else { ++ref_[q.pages[i]]; c.pages.push_back(q.pages[i]); }
    }
    seqs_[id] = c;
    return id;
  }
  int free_seq(int s) {
    auto it = seqs_.find(s);
    if (it == seqs_.end()) return 0;
    int rel = 0;
    for (int p : it->second.pages) rel += unref(p);   // unref ignores host-tier markers
    seqs_.erase(it);
    return rel;
  }
  const std::vector<int>& pages(int s) const { return seqs_.at(s).pages; }
  int refcount(int page) const { return ref_[page]; }
  // Pages only this sequence holds (what freeing it would give back).
  int exclusive_pages(int s) const { int n = 0; for (int p : seqs_.at(s).pages) n += p >= 0 && ref_[p] == 1; return n; }
 private:
  struct Seq { std::vector<int> pages; int len = 0; };
  int unref(int p) { if (p < 0) return 0; if (--ref_[p] == 0) { free_.push_back(p); return 1; } return 0; }
  int page_size_;
  std::vector<int> ref_, free_;
  std::unordered_map<int, Seq> seqs_;
  int next_id_ = 0;
};

// ------------------------------------------------------------------------------------------------ banker's check
// `avail` rows are free or reclaimable; item i may still take need[i] rows and gives back hold[i] when it finishes.
// Safe iff some order lets every item finish: visit by need ascending (ties by hold), as with one resource class.
static bool kv_safe(long avail, std::vector<std::pair<long, long>> items) {
  std::sort(items.begin(), items.end());
  for (auto& it : items) { if (it.first > avail) return false; avail += it.second; }
  return true;
}

// Eviction classes in the order they are given up (serve.rs:616-639): unreferenced prefix snapshots (LRU), idle
// conversations past the hold window (LRU), recently idle (most recent first), conversations with a queued turn
// (most recent first).  Candidates: (kind 0 snapshot / 1 conversation, id, idle seconds, queued flag).
struct EvictCand { int kind; long long id; double idle_s; int queued; };
static int pick_victim(const EvictCand* c, int n, double hold_s, bool allow_protected) {
  int best = -1;
  auto cls = [&](const EvictCand& e) { return e.kind == 0 ? 0 : (e.queued ? 3 : (e.idle_s >= hold_s ? 1 : 2)); };
  for (int i = 0; i < n; ++i) {
    const int ci = cls(c[i]);
    if (ci >= 2 && !allow_protected) continue;
    if (best < 0) { best = i; continue; }
    const int cb = cls(c[best]);
    if (ci != cb) { if (ci < cb) best = i; continue; }
    // classes 0,1: least recently used first; classes 2,3: most recently used first
    if (ci <= 1 ? c[i].idle_s > c[best].idle_s : c[i].idle_s < c[best].idle_s) best = i;
  }
  return best;
}

// Which prefilling request gets the next chunk: shortest remaining prompt first, every `fair`-th chunk to the oldest.
static int pick_prefill(const long* remaining, const double* age_s, int n, long chunk_index, int fair, int srpt) {
  if (n <= 0) return -1;
  int best = 0;
  const bool oldest = !srpt || (fair > 0 && chunk_index % fair == fair - 1);
  for (int i = 1; i < n; ++i) {
    if (oldest ? age_s[i] > age_s[best] : (remaining[i] < remaining[best] || (remaining[i] == remaining[best] && age_s[i] > age_s[best]))) best = i;
  }
  return best;
}

// ------------------------------------------------------------------------------------------------ copy-from-context drafter
// Proposes the tokens that followed the longest earlier occurrence of the text's current ending (behavioural contract:
// crates/agens-cli/src/lookup.rs: suffixes of 2..64 tokens, the 24 most recent places that end in the same two tokens
// are examined, the most recent one wins among equally long matches, at most 7 tokens are proposed; a running mean of
// accepted drafts per match-length class decides between this source and the model drafter).
//
// Data structure: every position p >= 1 carries a link to the previous position that ends the same token pair, and a
// hash map holds the newest position per pair.  The candidates of a query are the chain behind the newest entry, in
// recency order; appending is O(1) per token and cutting the text back just unlinks the removed positions.
class CopyLookup {
 public:
  static constexpr int kMaxDraft = 7, kProbe = 24, kLongest = 64, kClasses = 6;

  CopyLookup() {
    static const double start_mean[kClasses] = {0.6, 1.0, 1.8, 2.6, 3.6, 4.6};
    for (int c = 0; c < kClasses; ++c) by_class_[c] = Ema{start_mean[c], 4.0};
    model_ = Ema{2.0, 4.0};
  }

  void extend(const int* toks, int n) {
    for (int i = 0; i < n; ++i) text_.push_back(toks[i]);
  }

  void truncate(int n) {
    if (n >= (int)text_.size()) return;
    while (linked_ > std::max(n, 1)) unlink_last();
    text_.resize(n);
  }

  int size() const { return (int)text_.size(); }

  int propose(int* out, int* match_len, bool copy_only) {
    awaiting_copy_ = false;
    const int n = (int)text_.size();
    // the pair that ends the text is the query: it must not be among the candidates, so linking stops one short
    while (linked_ < n - 1) link_next();
    if (n < 3) return 0;
    auto head = newest_.find(pair_key(text_[n - 2], text_[n - 1]));
    if (head == newest_.end()) return 0;
    int win_len = 0, win_at = -1;
    int at = head->second;
    for (int probes = 0; at > 0 && probes < kProbe; ++probes, at = back_[at]) {
      const int len = common_suffix(at, n - 1);
      if (len > win_len) { win_len = len; win_at = at; }
    }
    if (win_at < 0) return 0;
    const int cls = length_class(win_len);
    if (!copy_only && by_class_[cls].mean <= model_.mean) return 0;       // the model drafter is expected to do better
    int cnt = 0;
    for (int q = win_at + 1; q < n && cnt < kMaxDraft; ++q) out[cnt++] = text_[q];
    *match_len = win_len;
    awaiting_copy_ = cnt > 0;
    awaiting_class_ = cls;
    return cnt;
  }

  // Outcome of the verified step: `accepted` drafts were kept; the mean of the source that made the proposal moves.
  void record(int accepted) {
    Ema& e = awaiting_copy_ ? by_class_[awaiting_class_] : model_;
    e.count += 1.0;
    e.mean += std::max(1.0 / e.count, 0.03) * ((double)accepted - e.mean);
    awaiting_copy_ = false;
  }

  double mean_lookup(int c) const { return by_class_[c].mean; }
  double mean_drafter() const { return model_.mean; }

 private:
  struct Ema { double mean, count; };

  static uint64_t pair_key(int a, int b) { return ((uint64_t)(uint32_t)a << 32) | (uint32_t)b; }

  static int length_class(int len) {
    static const int at_least[kClasses] = {2, 3, 4, 6, 10, 16};
    int c = 0;
    while (c + 1 < kClasses && len >= at_least[c + 1]) ++c;
    return c;
  }

  // Tokens shared by the text ending at position a and the text ending at position b (a < b), at most kLongest.
  int common_suffix(int a, int b) const {
    int len = 0;
    while (len < kLongest && a - len >= 0 && text_[a - len] == text_[b - len]) ++len;
    return len;
  }

  void link_next() {                       // position p = linked_ (or 1 at the start) gets its link
    const int p = std::max(linked_, 1);
    if ((int)back_.size() <= p) back_.resize(p + 1, 0);
    int& slot = newest_[pair_key(text_[p - 1], text_[p])];          // 0 = no earlier place (position 0 ends no pair)
    back_[p] = slot;
    slot = p;
    linked_ = p + 1;
  }

  void unlink_last() {
    const int p = linked_ - 1;
    if (p >= 1) {
      auto it = newest_.find(pair_key(text_[p - 1], text_[p]));
      if (it != newest_.end() && it->second == p) {
        if (back_[p] > 0) it->second = back_[p]; else newest_.erase(it);
      }
    }
    linked_ = p;
  }

  std::vector<int> text_;
  std::vector<int> back_;                              // back_[p]: previous position ending the same pair, 0 = none
  std::unordered_map<uint64_t, int> newest_;
  int linked_ = 0;                                     // positions below this carry their link
  Ema by_class_[kClasses], model_;
  bool awaiting_copy_ = false;
  int awaiting_class_ = 0;
};

// ------------------------------------------------------------------------------------------------ prefix cache
// Snapshots at chunk boundaries keyed by a hash chain over token ids (and image keys); lookup returns the longest
// cached prefix; insertion evicts least recently used entries that nobody references to stay inside the byte budget.
class PrefixCache {
 public:
  explicit PrefixCache(long long budget_bytes, int chunk) : budget_(budget_bytes), chunk_(chunk) {}
  static uint64_t mix(uint64_t h, uint64_t v) {
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h *= 0xff51afd7ed558ccdull;
    return h ^ (h >> 33);
  }
  // Hash of the first n tokens, chained chunk by chunk so that equal prefixes give equal keys.
  uint64_t key_of(const int* toks, int n, uint64_t salt) const {
    uint64_t h = 0x243f6a8885a308d3ull ^ salt;
    for (int i = 0; i < n; ++i) h = mix(h, (uint32_t)toks[i]);
    return mix(h, (uint64_t)n);
  }
  // Longest cached prefix of toks that ends on a chunk boundary; returns its length (0 = none) and snapshot handle.
  int lookup(const int* toks, int n, uint64_t salt, long long* handle) {
    int best = 0;
    uint64_t h = 0x243f6a8885a308d3ull ^ salt;
    for (int i = 0; i < n; ++i) {
      h = mix(h, (uint32_t)toks[i]);
      if ((i + 1) % chunk_ == 0) {
        auto it = map_.find(mix(h, (uint64_t)(i + 1)));
        if (it != map_.end()) { best = i + 1; *handle = it->second->handle; touch(it->second); }
      }
    }
    return best;
  }
  // Registers a snapshot of `bytes` for the first n tokens (n a multiple of the chunk).  Evicted handles are written
  // to `evicted` (caller frees their device/host memory); returns their count, -1 if the snapshot cannot fit.
  int insert(const int* toks, int n, uint64_t salt, long long handle, long long bytes, long long* evicted, int max_evicted) {
    if (n % chunk_ != 0 || bytes > budget_) return -1;
    return insert_key(key_of(toks, n, salt), handle, bytes, evicted, max_evicted);
  }
  // One entry per chunk boundary of the first n tokens in a single pass over them (n rounded down to a boundary); the
  // bytes are booked on the longest entry.  Same result as insert() per boundary, without hashing every prefix from the
  // start (a 128K-token conversation has 2048 boundaries).  Returns the number of evicted handles, -1 if it cannot fit.
  int insert_chain(const int* toks, int n, uint64_t salt, long long handle, long long bytes, long long* evicted, int max_evicted) {
    const int top = n / chunk_ * chunk_;
    if (bytes > budget_) return -1;
    uint64_t h = 0x243f6a8885a308d3ull ^ salt;
    int ne = 0;
    for (int i = 0; i < top; ++i) {
      h = mix(h, (uint32_t)toks[i]);
      if ((i + 1) % chunk_ == 0) {
        const int r = insert_key(mix(h, (uint64_t)(i + 1)), handle, i + 1 == top ? bytes : 0, evicted + ne, max_evicted - ne);
        if (r < 0) return -1;
        ne += r;
      }
    }
    return ne;
  }
  int insert_key(uint64_t k, long long handle, long long bytes, long long* evicted, int max_evicted) {
    if (map_.count(k)) return 0;
    int ne = 0;
    while (used_ + bytes > budget_) {
      auto victim = lru_.end();
      for (auto it = lru_.begin(); it != lru_.end(); ++it) if (it->refs == 0) { victim = it; break; }
      if (victim == lru_.end() || ne >= max_evicted) return -1;
      evicted[ne++] = victim->handle;
      used_ -= victim->bytes;
      map_.erase(victim->key);
      lru_.erase(victim);
    }
    lru_.push_back(Entry{k, handle, bytes, 0});
    map_[k] = std::prev(lru_.end());
    used_ += bytes;
    return ne;
  }
  void ref(long long handle, int delta) { for (auto& e : lru_) if (e.handle == handle) e.refs += delta; }
  long long used() const { return used_; }
  int entries() const { return (int)lru_.size(); }
  // Oldest unreferenced entry (eviction candidate of class 0), -1 if none.
  long long evict_lru() {
    for (auto it = lru_.begin(); it != lru_.end(); ++it)
      if (it->refs == 0) { long long h = it->handle; used_ -= it->bytes; map_.erase(it->key); lru_.erase(it); return h; }
    return -1;
  }
 private:
  struct Entry { uint64_t key; long long handle, bytes; int refs; };
  void touch(std::list<Entry>::iterator it) { lru_.splice(lru_.end(), lru_, it); }
  long long budget_, used_ = 0;
  int chunk_;
  std::list<Entry> lru_;
  std::unordered_map<uint64_t, std::list<Entry>::iterator> map_;
};

}  // namespace b2

using namespace b2;

// ---- C ABI ----
B2H_API void* b2h_pages_new(int n_pages, int page_size) { return new PageAllocator(n_pages, page_size); }
B2H_API void b2h_pages_free(void* a) { delete static_cast<PageAllocator*>(a); }
// An unknown sequence id or page index is the caller's bug; it comes back as kBadId (-1000) instead of an exception
// crossing the C boundary (which would end the process).
static constexpr int kBadId = -1000;
#define B2H_GUARD(expr) try { return (expr); } catch (const std::exception&) { return kBadId; }
B2H_API int b2h_pages_free_count(void* a) { return static_cast<PageAllocator*>(a)->free_pages(); }
B2H_API int b2h_pages_new_seq(void* a) { return static_cast<PageAllocator*>(a)->new_seq(); }
B2H_API int b2h_pages_reserve(void* a, int s, int n_tokens) { B2H_GUARD(static_cast<PageAllocator*>(a)->reserve(s, n_tokens)) }
B2H_API void b2h_pages_set_len(void* a, int s, int n) { try { static_cast<PageAllocator*>(a)->set_len(s, n); } catch (const std::exception&) {} }
B2H_API int b2h_pages_len(void* a, int s) { B2H_GUARD(static_cast<PageAllocator*>(a)->seq_len(s)) }
B2H_API int b2h_pages_truncate(void* a, int s, int n) { B2H_GUARD(static_cast<PageAllocator*>(a)->truncate(s, n)) }
B2H_API int b2h_pages_evict_page(void* a, int s, int index) { B2H_GUARD(static_cast<PageAllocator*>(a)->evict_page(s, index)) }
B2H_API int b2h_pages_fork(void* a, int s, int* src, int* dst) { B2H_GUARD(static_cast<PageAllocator*>(a)->fork(s, src, dst)) }
B2H_API int b2h_pages_free_seq(void* a, int s) { return static_cast<PageAllocator*>(a)->free_seq(s); }
B2H_API int b2h_pages_exclusive(void* a, int s) { B2H_GUARD(static_cast<PageAllocator*>(a)->exclusive_pages(s)) }
B2H_API int b2h_pages_refcount(void* a, int page) {
  auto al = static_cast<PageAllocator*>(a);
  return page >= 0 && page < al->n_pages() ? al->refcount(page) : kBadId;
}
B2H_API int b2h_pages_list(void* a, int s, int* out, int cap) {
  try {
    const auto& p = static_cast<PageAllocator*>(a)->pages(s);
    const int n = std::min<int>((int)p.size(), cap);
    std::memcpy(out, p.data(), sizeof(int) * n);
    return (int)p.size();
  } catch (const std::exception&) { return kBadId; }
}

B2H_API int b2h_kv_safe(long avail, const long* need, const long* hold, int n) {
  std::vector<std::pair<long, long>> items;
  for (int i = 0; i < n; ++i) items.emplace_back(need[i], hold[i]);
  return kv_safe(avail, items) ? 1 : 0;
}
B2H_API int b2h_pick_victim(const int* kind, const long long* id, const double* idle_s, const int* queued, int n, double hold_s,
                            int allow_protected) {
  std::vector<EvictCand> c(n);
  for (int i = 0; i < n; ++i) c[i] = EvictCand{kind[i], id[i], idle_s[i], queued[i]};
  return pick_victim(c.data(), n, hold_s, allow_protected != 0);
}
B2H_API int b2h_pick_prefill(const long* remaining, const double* age_s, int n, long chunk_index, int fair, int srpt) {
  return pick_prefill(remaining, age_s, n, chunk_index, fair, srpt);
}

B2H_API void* b2h_lookup_new() { return new CopyLookup(); }
B2H_API void b2h_lookup_free(void* l) { delete static_cast<CopyLookup*>(l); }
B2H_API void b2h_lookup_extend(void* l, const int* toks, int n) { static_cast<CopyLookup*>(l)->extend(toks, n); }
B2H_API void b2h_lookup_truncate(void* l, int n) { static_cast<CopyLookup*>(l)->truncate(n); }
B2H_API int b2h_lookup_propose(void* l, int* out, int* match_len, int copy_only) { return static_cast<CopyLookup*>(l)->propose(out, match_len, copy_only != 0); }
B2H_API void b2h_lookup_record(void* l, int accepted) { static_cast<CopyLookup*>(l)->record(accepted); }
B2H_API double b2h_lookup_mean(void* l, int bucket) { return bucket < 0 ? static_cast<CopyLookup*>(l)->mean_drafter() : static_cast<CopyLookup*>(l)->mean_lookup(bucket); }

B2H_API void* b2h_prefix_new(long long budget_bytes, int chunk) { return new PrefixCache(budget_bytes, chunk); }
B2H_API void b2h_prefix_free(void* p) { delete static_cast<PrefixCache*>(p); }
B2H_API int b2h_prefix_lookup(void* p, const int* toks, int n, unsigned long long salt, long long* handle) { return static_cast<PrefixCache*>(p)->lookup(toks, n, salt, handle); }
B2H_API int b2h_prefix_insert(void* p, const int* toks, int n, unsigned long long salt, long long handle, long long bytes, long long* evicted, int max_evicted) {
  return static_cast<PrefixCache*>(p)->insert(toks, n, salt, handle, bytes, evicted, max_evicted);
}
B2H_API int b2h_prefix_insert_chain(void* p, const int* toks, int n, unsigned long long salt, long long handle, long long bytes, long long* evicted, int max_evicted) {
  return static_cast<PrefixCache*>(p)->insert_chain(toks, n, salt, handle, bytes, evicted, max_evicted);
}
B2H_API void b2h_prefix_ref(void* p, long long handle, int delta) { static_cast<PrefixCache*>(p)->ref(handle, delta); }
B2H_API long long b2h_prefix_used(void* p) { return static_cast<PrefixCache*>(p)->used(); }
B2H_API long long b2h_prefix_evict_lru(void* p) { return static_cast<PrefixCache*>(p)->evict_lru(); }
