// Pages of one cache group: reference counts, a free list and the prefix table.
//
// The behaviour follows the reference's BlockPool (vllm-oxide,
// crates/vllm-oxide/src/engine/block_pool.rs:45-369): pages leave the FRONT of the free list
// and come back at its BACK, a freed page keeps its hash so that it can be found again until
// it is handed out for other tokens, and a page is reusable exactly when its count is zero.
// The free list here is an intrusive doubly linked list, so taking a cached page back out of
// the middle is O(1) (the reference searches its deque, block_pool.rs:266-271).
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace vob {

struct PoolError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// XXH64, written from the public specification of the algorithm.
inline uint64_t xxh64(const uint8_t* p, size_t len, uint64_t seed) {
  constexpr uint64_t P1 = 0x9E3779B185EBCA87ULL, P2 = 0xC2B2AE3D27D4EB4FULL, P3 = 0x165667B19E3779F9ULL,
                     P4 = 0x85EBCA77C2B2AE63ULL, P5 = 0x27D4EB2F165667C5ULL;
  auto rotl = [](uint64_t x, int r) { return (x << r) | (x >> (64 - r)); };
  auto rd64 = [](const uint8_t* q) { uint64_t v; std::memcpy(&v, q, 8); return v; };
  auto rd32 = [](const uint8_t* q) { uint32_t v; std::memcpy(&v, q, 4); return v; };
  auto round = [&](uint64_t acc, uint64_t in) { acc += in * P2; acc = rotl(acc, 31); return acc * P1; };
  auto merge = [&](uint64_t acc, uint64_t v) { acc ^= round(0, v); return acc * P1 + P4; };
  const uint8_t* end = p + len;
  uint64_t h;
  if (len >= 32) {
    uint64_t v1 = seed + P1 + P2, v2 = seed + P2, v3 = seed, v4 = seed - P1;
    const uint8_t* limit = end - 32;
    do {
      v1 = round(v1, rd64(p)); v2 = round(v2, rd64(p + 8));
      v3 = round(v3, rd64(p + 16)); v4 = round(v4, rd64(p + 24));
      p += 32;
    } while (p <= limit);
    h = rotl(v1, 1) + rotl(v2, 7) + rotl(v3, 12) + rotl(v4, 18);
    h = merge(h, v1); h = merge(h, v2); h = merge(h, v3); h = merge(h, v4);
  } else {
    h = seed + P5;
  }
  h += static_cast<uint64_t>(len);
  while (p + 8 <= end) { h ^= round(0, rd64(p)); h = rotl(h, 27) * P1 + P4; p += 8; }
  if (p + 4 <= end) { h ^= static_cast<uint64_t>(rd32(p)) * P1; h = rotl(h, 23) * P2 + P3; p += 4; }
  while (p < end) { h ^= (*p) * P5; h = rotl(h, 11) * P1; ++p; }
  h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
  return h;
}

// Hash of one full page, chained to the page before it (block_pool.rs:133-142):
// XXH64(seed 0) over [previous hash as 8 LE bytes, left out for the first page] ++ tokens as u32 LE.
inline int64_t chain_hash(int64_t prev, const int32_t* tokens, int n) {
  std::vector<uint8_t> buf;
  buf.reserve(8 + 4 * static_cast<size_t>(n));
  if (prev != -1) {
    uint64_t u = static_cast<uint64_t>(prev);
    for (int i = 0; i < 8; ++i) buf.push_back(static_cast<uint8_t>(u >> (8 * i)));
  }
  for (int i = 0; i < n; ++i) {
    uint32_t t = static_cast<uint32_t>(tokens[i]);
    for (int b = 0; b < 4; ++b) buf.push_back(static_cast<uint8_t>(t >> (8 * b)));
  }
  int64_t h = static_cast<int64_t>(xxh64(buf.data(), buf.size(), 0));
  return h == -1 ? -2 : h;  // -1 is the "no hash" mark
}

class BlockPool {
 public:
  BlockPool(int num_blocks, int block_size) : block_size_(block_size), blocks_(num_blocks) {
    if (num_blocks <= 0 || block_size <= 0) throw PoolError("BlockPool: sizes must be positive");
    for (int i = 0; i < num_blocks; ++i) push_back_free(i);
  }

  int num_blocks() const { return static_cast<int>(blocks_.size()); }
  int block_size() const { return block_size_; }
  int num_free() const { return num_free_; }
  int ref_count(int id) const { return at(id).ref; }
  bool is_free(int id) const { return at(id).in_free; }
  int64_t hash_of(int id) const { return at(id).hash; }

  // A page for new tokens: the oldest free page. What it held is forgotten.
  int allocate() {
    if (head_ < 0) throw PoolError("BlockPool: out of pages");
    int id = head_;
    unlink_free(id);
    Block& b = blocks_[id];
    if (b.hash != -1) {
      auto it = table_.find(b.hash);
      if (it != table_.end() && it->second == id) table_.erase(it);
      b.hash = -1;
      b.tokens.clear();
    }
    b.ref = 1;
    return id;
  }

  // One more holder of a page found in the prefix table (it may be lying in the free list).
  void retain(int id) {
    Block& b = at_mut(id);
    if (b.in_free) { unlink_free(id); b.ref = 1; }
    else { if (b.ref <= 0) throw PoolError("BlockPool: retain of a page that nobody holds"); ++b.ref; }
  }

  // One holder fewer; the last one puts the page at the back of the free list.
  void release(int id) {
    Block& b = at_mut(id);
    if (b.in_free || b.ref <= 0) throw PoolError("BlockPool: page " + std::to_string(id) + " freed twice");
    if (--b.ref == 0) push_back_free(id);
  }

  // The page that holds exactly these tokens after this chain of pages, or -1.
  int lookup(int64_t hash, const int32_t* tokens, int n) const {
    auto it = table_.find(hash);
    if (it == table_.end()) return -1;
    const Block& b = blocks_[it->second];
    if (static_cast<int>(b.tokens.size()) != n || std::memcmp(b.tokens.data(), tokens, 4 * n) != 0) return -1;
    return it->second;
  }

  // Record a full page under its hash; an older page with the same hash keeps the entry.
  void publish(int id, int64_t hash, const int32_t* tokens, int n) {
    Block& b = at_mut(id);
    if (b.in_free) throw PoolError("BlockPool: publish of a free page");
    if (b.hash != -1) return;
    b.hash = hash;
    b.tokens.assign(tokens, tokens + n);
    table_.emplace(hash, id);
  }

  // Free list from oldest to newest (for tests).
  std::vector<int> free_order() const {
    std::vector<int> v;
    for (int i = head_; i >= 0; i = blocks_[i].next) v.push_back(i);
    return v;
  }

 private:
  struct Block {
    int ref = 0;
    int64_t hash = -1;
    std::vector<int32_t> tokens;
    int prev = -1, next = -1;
    bool in_free = false;
  };
  const Block& at(int id) const {
    if (id < 0 || id >= static_cast<int>(blocks_.size())) throw PoolError("BlockPool: no page " + std::to_string(id));
    return blocks_[id];
  }
  Block& at_mut(int id) { return const_cast<Block&>(at(id)); }
  void push_back_free(int id) {
    Block& b = blocks_[id];
    b.prev = tail_; b.next = -1; b.in_free = true; b.ref = 0;
    if (tail_ >= 0) blocks_[tail_].next = id; else head_ = id;
    tail_ = id;
    ++num_free_;
  }
  void unlink_free(int id) {
    Block& b = blocks_[id];
    if (b.prev >= 0) blocks_[b.prev].next = b.next; else head_ = b.next;
    if (b.next >= 0) blocks_[b.next].prev = b.prev; else tail_ = b.prev;
    b.prev = b.next = -1; b.in_free = false;
    --num_free_;
  }

  int block_size_;
  std::vector<Block> blocks_;
  std::unordered_map<int64_t, int> table_;
  int head_ = -1, tail_ = -1, num_free_ = 0;
};

}  // namespace vob
