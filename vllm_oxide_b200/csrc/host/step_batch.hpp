// The host side of a step's batch descriptor: every integer array of one step in ONE
// buffer, so that a step costs one host-to-device copy (the reference uploads two arrays per
// step and three more in every layer: vllm-oxide, crates/vllm-oxide/src/engine/mod.rs:200-201,
// crates/vllm-oxide/src/models/qwen3.rs:189-193, crates/vllm-oxide/src/attention/flash_attn.rs:23-24,48-50).
//
// Arrays (all int32), for capacities T tokens, B requests, R wanted rows, G groups, P table width:
//   token_ids[T] positions[T] token_req[T] | slot_mapping[G][T] | cu_q[B+1] context_lens[B]
//   state_slots[B] state_fresh[B] | logit_rows[R] | block_tables[G][B][P]
// Unused tails are padded so that kernels launched for the full capacity do nothing there:
// token_req -1, slots -1, context_lens 0, cu_q repeats its last value, block tables -1.
#pragma once
#include "kv_cache_manager.hpp"

namespace vob {

struct BatchLayout {
  int T = 0, B = 0, R = 0, G = 0, P = 0;
  long token_ids = 0, positions = 0, token_req = 0, slot_mapping = 0, cu_q = 0, context_lens = 0, state_slots = 0,
       state_fresh = 0, logit_rows = 0, block_tables = 0, total = 0;
  BatchLayout() = default;
  BatchLayout(int t, int b, int r, int g, int p) : T(t), B(b), R(r), G(g), P(p) {
    auto pad = [](long x) { return (x + 3) / 4 * 4; };  // every array starts on a 16-byte boundary
    long o = 0;
    token_ids = o; o = pad(o + T);
    positions = o; o = pad(o + T);
    token_req = o; o = pad(o + T);
    slot_mapping = o; o = pad(o + static_cast<long>(G) * T);
    cu_q = o; o = pad(o + B + 1);
    context_lens = o; o = pad(o + B);
    state_slots = o; o = pad(o + B);
    state_fresh = o; o = pad(o + B);
    logit_rows = o; o = pad(o + R);
    block_tables = o; o = pad(o + static_cast<long>(G) * B * P);
    total = o;
  }
};

struct BatchEntry {
  int64_t id;
  int start;                     // position of the first token of this portion
  std::vector<int32_t> tokens;   // the portion
  std::vector<int32_t> want;     // places among these tokens whose logits are wanted
};

struct BatchCounts {
  int num_tokens = 0, num_requests = 0, num_rows = 0, num_decode = 0, max_q = 0, max_context = 0;
};

// One request's part of a step, by reference: the tokens and wanted places live in the caller's entry or sequence.
struct EntryView {
  int64_t id;
  int start;
  const int32_t* tokens;
  int n;
  const int32_t* want;
  int n_want;
};

inline BatchCounts fill_step_views(KvCacheManager& mgr, const std::vector<EntryView>& entries, const BatchLayout& L,
                                   int32_t* out) {
  BatchCounts c;
  long T = 0, R = 0;
  for (const auto& e : entries) { T += e.n; R += e.n_want; }
  if (T > L.T || static_cast<int>(entries.size()) > L.B || R > L.R)
    throw PoolError("fill_step_batch: the step (" + std::to_string(T) + " tokens, " + std::to_string(entries.size()) +
                    " requests, " + std::to_string(R) + " rows) exceeds the buffer's capacity");
  if (L.G != mgr.num_groups()) throw PoolError("fill_step_batch: layout and manager disagree on the number of groups");
  std::fill(out, out + L.total, 0);
  std::fill(out + L.token_req, out + L.token_req + L.T, -1);
  std::fill(out + L.slot_mapping, out + L.slot_mapping + static_cast<long>(L.G) * L.T, -1);
  std::fill(out + L.block_tables, out + L.block_tables + static_cast<long>(L.G) * L.B * L.P, -1);
  int t = 0, r = 0, b = 0;
  for (const auto& e : entries) {
    const int n = e.n;
    if (n <= 0) throw PoolError("fill_step_batch: an entry without tokens");
    if (e.start < 0) throw PoolError("fill_step_batch: negative start");
    out[L.cu_q + b] = t;
    out[L.context_lens + b] = e.start + n;
    out[L.state_slots + b] = mgr.state_slot(e.id);
    out[L.state_fresh + b] = mgr.take_state_fresh(e.id) ? 1 : 0;
    for (int i = 0; i < n; ++i) {
      out[L.token_ids + t + i] = e.tokens[i];
      out[L.positions + t + i] = e.start + i;
      out[L.token_req + t + i] = b;
    }
    for (int g = 0; g < L.G; ++g) {
      mgr.slot_mapping(e.id, g, e.start, n, out + L.slot_mapping + static_cast<long>(g) * L.T + t);
      for (int i = 0; i < n; ++i)
        if (out[L.slot_mapping + static_cast<long>(g) * L.T + t + i] < 0)
          throw PoolError("fill_step_batch: request " + std::to_string(e.id) + " has no page for position " +
                          std::to_string(e.start + i) + " in group " + std::to_string(g));
      const auto& table = mgr.block_table(e.id, g);
      if (static_cast<int>(table.size()) > L.P)
        throw PoolError("fill_step_batch: a block table of " + std::to_string(table.size()) +
                        " pages exceeds the buffer's width " + std::to_string(L.P));
      std::copy(table.begin(), table.end(), out + L.block_tables + (static_cast<long>(g) * L.B + b) * L.P);
    }
    for (int j = 0; j < e.n_want; ++j) {
      const int w = e.want[j];
      if (w < 0 || w >= n) throw PoolError("fill_step_batch: wanted place " + std::to_string(w) + " outside the portion");
      out[L.logit_rows + r++] = t + w;
    }
    c.num_decode += n == 1;
    c.max_q = std::max(c.max_q, n);
    c.max_context = std::max(c.max_context, e.start + n);
    t += n;
    ++b;
  }
  for (int i = b; i <= L.B; ++i) out[L.cu_q + i] = t;
  c.num_tokens = t; c.num_requests = b; c.num_rows = r;
  return c;
}

inline BatchCounts fill_step_batch(KvCacheManager& mgr, const std::vector<BatchEntry>& entries,
                                   const BatchLayout& L, int32_t* out) {
  std::vector<EntryView> views;
  views.reserve(entries.size());
  for (const auto& e : entries)
    views.push_back({e.id, e.start, e.tokens.data(), static_cast<int>(e.tokens.size()), e.want.data(),
                     static_cast<int>(e.want.size())});
  return fill_step_views(mgr, views, L, out);
}

}  // namespace vob
