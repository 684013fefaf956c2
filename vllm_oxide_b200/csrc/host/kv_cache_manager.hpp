// The cache manager: one block table per request and per cache group, plus state slots.
//
// A cache group is a set of layers with the same needs: all keys (window 0) or the last
// `window` keys.  Each group has pages of its own (its own BlockPool); a request has one
// block table per group, indexed by position / block_size, with -1 where no page is held.
// Pages are given back when a request ends, when it is preempted, and, in a window group,
// as soon as the window has passed them.  Beside the pages the manager owns the slots for
// per-request state of fixed size (one slot per live request; a model whose layers keep no
// such state still gets a slot id, of zero bytes).
//
// The reference has one group and no state slots (vllm-oxide,
// crates/vllm-oxide/src/engine/kv_cache_manager.rs:54-146, block_pool.rs:198-358); its rules
// are kept where it has them: the last page of a prompt is never taken from the prefix
// cache, so at least one token is always computed (block_pool.rs:198-227); pages are freed
// in reverse table order (block_pool.rs:293-309); slot = page * block_size + offset, -1
// without a page (kv_cache_manager.rs:115-135).
#pragma once
#include <algorithm>
#include <map>
#include <sstream>

#include "block_pool.hpp"

namespace vob {

struct GroupSpec {
  int block_size = 16;
  int num_blocks = 1;
  int window = 0;  // 0: every key is kept; W > 0: only positions > query - W are read
};

class KvCacheManager {
 public:
  KvCacheManager(const std::vector<GroupSpec>& groups, int num_state_slots, bool prefix_caching)
      : specs_(groups) {
    if (groups.empty()) throw PoolError("KvCacheManager: at least one cache group is needed");
    if (num_state_slots <= 0) throw PoolError("KvCacheManager: at least one state slot is needed");
    bool same = true;
    for (const auto& g : groups) {
      if (g.window < 0) throw PoolError("KvCacheManager: negative window");
      pools_.emplace_back(g.num_blocks, g.block_size);
      same = same && g.block_size == groups[0].block_size;
    }
    // A prefix hit must hold in every group at once, page for page; with unequal page sizes it is off.
    prefix_caching_ = prefix_caching && same;
    for (int s = num_state_slots - 1; s >= 0; --s) free_slots_.push_back(s);
    num_state_slots_ = num_state_slots;
  }

  int num_groups() const { return static_cast<int>(specs_.size()); }
  const GroupSpec& group(int g) const { return specs_.at(g); }
  int num_free_blocks(int g) const { return pools_.at(g).num_free(); }
  int num_free_state_slots() const { return static_cast<int>(free_slots_.size()); }
  bool prefix_caching() const { return prefix_caching_; }
  bool has_request(int64_t id) const { return reqs_.count(id) != 0; }
  int num_requests() const { return static_cast<int>(reqs_.size()); }
  const BlockPool& pool(int g) const { return pools_.at(g); }

  // Registers a request and gives it a state slot. False when no slot is free.
  bool add_request(int64_t id) {
    if (reqs_.count(id)) throw PoolError("KvCacheManager: request " + std::to_string(id) + " is already live");
    if (free_slots_.empty()) return false;
    Req r;
    r.tables.resize(specs_.size());
    r.state_slot = free_slots_.back();
    free_slots_.pop_back();
    r.state_fresh = true;
    reqs_.emplace(id, std::move(r));
    return true;
  }

  // Takes the pages of the longest cached prefix of `tokens` into the (empty) block tables
  // and returns how many tokens they cover. The page that holds the last token is never taken.
  // A group that keeps all keys takes every page of the prefix; a window group only those that a
  // query after the prefix can still read (the earlier entries of its table stay empty, as if
  // the window had passed them).
  int lookup_prefix(int64_t id, const int32_t* tokens, int n) {
    Req& r = req(id);
    if (!prefix_caching_) return 0;
    for (auto& t : r.tables)
      if (!t.empty()) throw PoolError("KvCacheManager: lookup_prefix on a request that already holds pages");
    std::vector<int64_t> hashes;
    std::vector<std::vector<int>> found;
    const int hits = cached_prefix_pages(tokens, n, &hashes, &found);
    for (size_t g = 0; g < specs_.size(); ++g) {
      const int lo = first_page_needed(g, hits);
      r.tables[g].assign(hits, -1);
      for (int i = lo; i < hits; ++i) {
        pools_[g].retain(found[g][i]);
        r.tables[g][i] = found[g][i];
      }
      if (specs_[g].window > 0) r.released_upto[g] = lo;
    }
    r.page_hashes.assign(hashes.begin(), hashes.begin() + hits);
    return hits * specs_[0].block_size;
  }

  // "Restorable at which position?": how many leading tokens of `tokens` a new request could take from cached pages
  // right now, in every group at once (what lookup_prefix would return), without taking anything.  0 when prefix
  // caching is off, which it is when the groups' pages are of different sizes, and which the engine asks for when a
  // part keeps per-request state (nothing of a state survives outside its slot, so such a request can only be
  // computed from its first token).  A scheduler can price an admission with it.
  int restorable_tokens(const int32_t* tokens, int n) const {
    if (!prefix_caching_) return 0;
    return cached_prefix_pages(tokens, n, nullptr, nullptr) * specs_[0].block_size;
  }

  // New pages that positions [start, start+n) need, per group.
  std::vector<int> pages_needed(int64_t id, int start, int n) const {
    const Req& r = req(id);
    std::vector<int> need(specs_.size(), 0);
    if (n <= 0) return need;
    for (size_t g = 0; g < specs_.size(); ++g) {
      const int bs = specs_[g].block_size;
      for (int p = start / bs; p <= (start + n - 1) / bs; ++p)
        if (p >= static_cast<int>(r.tables[g].size()) || r.tables[g][p] < 0) ++need[g];
    }
    return need;
  }

  bool can_ensure(int64_t id, int start, int n) const {
    auto need = pages_needed(id, start, n);
    for (size_t g = 0; g < specs_.size(); ++g)
      if (need[g] > pools_[g].num_free()) return false;
    return true;
  }

  // Makes sure every group holds pages for positions [start, start+n): all of them or none.
  bool ensure(int64_t id, int start, int n) {
    if (n <= 0) return true;
    if (!can_ensure(id, start, n)) return false;
    Req& r = req(id);
    for (size_t g = 0; g < specs_.size(); ++g) {
      const int bs = specs_[g].block_size;
      auto& t = r.tables[g];
      const int last = (start + n - 1) / bs;
      if (static_cast<int>(t.size()) <= last) t.resize(last + 1, -1);
      for (int p = start / bs; p <= last; ++p)
        if (t[p] < 0) t[p] = pools_[g].allocate();
    }
    return true;
  }

  // After `num_computed` tokens are in the cache: a window group gives back every page that
  // no later query can read (the next query is at position >= num_computed and reads
  // positions > query - window).
  void advance(int64_t id, int num_computed) {
    Req& r = req(id);
    for (size_t g = 0; g < specs_.size(); ++g) {
      const int w = specs_[g].window;
      if (w <= 0) continue;
      const int bs = specs_[g].block_size;
      const int first_needed = num_computed - w + 1;  // lowest position still readable
      auto& t = r.tables[g];
      for (int p = r.released_upto[g]; p < static_cast<int>(t.size()) && (p + 1) * bs <= first_needed; ++p) {
        if (t[p] >= 0) { pools_[g].release(t[p]); t[p] = -1; }
        r.released_upto[g] = p + 1;
      }
    }
  }

  // Publishes the hashes of the pages that became full, so later requests can share them.
  void commit(int64_t id, const int32_t* tokens, int num_computed) {
    if (!prefix_caching_) return;
    Req& r = req(id);
    const int bs = specs_[0].block_size;
    const int full = num_computed / bs;
    for (int i = static_cast<int>(r.page_hashes.size()); i < full; ++i) {
      int64_t prev = i == 0 ? -1 : r.page_hashes[i - 1];
      int64_t h = chain_hash(prev, tokens + i * bs, bs);
      r.page_hashes.push_back(h);
      for (size_t g = 0; g < specs_.size(); ++g)
        if (i < static_cast<int>(r.tables[g].size()) && r.tables[g][i] >= 0)
          pools_[g].publish(r.tables[g][i], h, tokens + i * bs, bs);
    }
  }

  // Gives back every page (last page first) but keeps the request and its state slot:
  // what a preempted request does before it waits again.
  void release_pages(int64_t id) {
    Req& r = req(id);
    for (size_t g = 0; g < specs_.size(); ++g) {
      auto& t = r.tables[g];
      for (int p = static_cast<int>(t.size()) - 1; p >= 0; --p)
        if (t[p] >= 0) pools_[g].release(t[p]);
      t.clear();
      r.released_upto[g] = 0;
    }
    r.page_hashes.clear();
    r.state_fresh = true;
  }

  // The request ends: pages and state slot go back.
  void free_request(int64_t id) {
    release_pages(id);
    free_slots_.push_back(req(id).state_slot);
    reqs_.erase(id);
  }

  const std::vector<int>& block_table(int64_t id, int g) const { return req(id).tables.at(g); }
  int state_slot(int64_t id) const { return req(id).state_slot; }

  // True once after the slot was assigned or the request lost its pages: the state must be zeroed.
  bool take_state_fresh(int64_t id) {
    Req& r = req(id);
    bool f = r.state_fresh;
    r.state_fresh = false;
    return f;
  }

  void slot_mapping(int64_t id, int g, int start, int n, int32_t* out) const {
    const auto& t = req(id).tables.at(g);
    const int bs = specs_[g].block_size;
    for (int i = 0; i < n; ++i) {
      const int pos = start + i, p = pos / bs;
      out[i] = (p < static_cast<int>(t.size()) && t[p] >= 0) ? t[p] * bs + pos % bs : -1;
    }
  }

  // Empty when every page is either free or held exactly as often as block tables name it.
  std::string check_invariants() const {
    std::ostringstream err;
    for (size_t g = 0; g < specs_.size(); ++g) {
      const BlockPool& pool = pools_[g];
      std::vector<int> holders(pool.num_blocks(), 0);
      for (const auto& kv : reqs_)
        for (int b : kv.second.tables[g])
          if (b >= 0) {
            if (b >= pool.num_blocks()) { err << "group " << g << ": table names page " << b << "; "; continue; }
            ++holders[b];
          }
      int free_count = 0;
      for (int b = 0; b < pool.num_blocks(); ++b) {
        if (pool.ref_count(b) != holders[b])
          err << "group " << g << " page " << b << ": count " << pool.ref_count(b) << " but " << holders[b] << " holders; ";
        if (pool.is_free(b) != (holders[b] == 0))
          err << "group " << g << " page " << b << ": free flag wrong; ";
        free_count += pool.is_free(b);
      }
      if (free_count != pool.num_free()) err << "group " << g << ": free count " << pool.num_free() << " vs " << free_count << "; ";
      if (static_cast<int>(pool.free_order().size()) != pool.num_free()) err << "group " << g << ": free list broken; ";
    }
    std::vector<char> seen(num_state_slots_, 0);
    for (int s : free_slots_) { if (seen[s]) err << "state slot " << s << " free twice; "; seen[s] = 1; }
    for (const auto& kv : reqs_) {
      int s = kv.second.state_slot;
      if (seen[s]) err << "state slot " << s << " held twice or free and held; ";
      seen[s] = 1;
    }
    for (int s = 0; s < num_state_slots_; ++s) if (!seen[s]) err << "state slot " << s << " lost; ";
    return err.str();
  }

 private:
  // The first page of group g that a query at a position >= pages * block_size can read (0 for a group that keeps
  // all keys): the same rule by which advance() gives pages back.
  int first_page_needed(size_t g, int pages) const {
    const int w = specs_[g].window;
    if (w <= 0) return 0;
    const int first_needed = pages * specs_[g].block_size - w + 1;
    return first_needed <= 0 ? 0 : std::min(pages, first_needed / specs_[g].block_size);
  }

  // The most leading pages of `tokens` (never the one of the last token) that every group can supply: all of them in
  // a group that keeps all keys, the ones a later query can still read in a window group.  `found[g][i]` is group g's
  // page for page i of the prefix or -1, `hashes[i]` the chained hash of page i.
  int cached_prefix_pages(const int32_t* tokens, int n, std::vector<int64_t>* hashes,
                          std::vector<std::vector<int>>* found) const {
    const int bs = specs_[0].block_size;
    std::vector<int64_t> hs;
    std::vector<std::vector<int>> ids(specs_.size());
    int64_t prev = -1;
    int limit = 0;
    for (int i = 0; (i + 1) * bs < n; ++i) {
      const int64_t h = chain_hash(prev, tokens + i * bs, bs);
      bool all = true;
      for (size_t g = 0; g < specs_.size(); ++g) {
        const int page = pools_[g].lookup(h, tokens + i * bs, bs);
        ids[g].push_back(page);
        all = all && (page >= 0 || specs_[g].window > 0);
      }
      if (!all) break;
      hs.push_back(h);
      prev = h;
      limit = i + 1;
    }
    int hits = limit;
    for (; hits > 0; --hits) {
      bool ok = true;
      for (size_t g = 0; g < specs_.size() && ok; ++g)
        for (int i = first_page_needed(g, hits); i < hits && ok; ++i) ok = ids[g][i] >= 0;
      if (ok) break;
    }
    if (hashes) *hashes = std::move(hs);
    if (found) *found = std::move(ids);
    return hits;
  }

  struct Req {
    std::vector<std::vector<int>> tables;
    std::map<size_t, int> released_upto;  // per window group: first table index not yet released
    std::vector<int64_t> page_hashes;
    int state_slot = -1;
    bool state_fresh = true;
  };
  Req& req(int64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) throw PoolError("KvCacheManager: no live request " + std::to_string(id));
    return it->second;
  }
  const Req& req(int64_t id) const { return const_cast<KvCacheManager*>(this)->req(id); }

  std::vector<GroupSpec> specs_;
  std::vector<BlockPool> pools_;
  std::map<int64_t, Req> reqs_;
  std::vector<int> free_slots_;
  int num_state_slots_ = 0;
  bool prefix_caching_ = false;
};

}  // namespace vob
