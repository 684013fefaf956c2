// The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
// finishes and frees.
//
// Names follow the reference's Scheduler (vllm-oxide, crates/vllm-oxide/src/engine/scheduler.rs:65-409):
// `waiting` and `running` queues, `schedule`, `postprocess`, preemption of the newest
// running request with recompute (scheduler.rs:241-263).  The algorithm differs where the
// reference's cannot serve a mixed batch:
//   * one token budget per step over ALL requests: running requests first (a decoding request
//     needs one token, a request still in its prompt, or recomputing after preemption, gets
//     min(remaining, budget left)), then new admissions (the reference limits only the first
//     request of a prefill step, scheduler.rs:360-369, and admits only into an empty engine,
//     scheduler.rs:144-148);
//   * a sampled token is appended only for a request whose last token was in the step (the
//     reference appends one for every running request, scheduler.rs:168-175);
//   * a preempted request is later recomputed over prompt AND generated tokens (the reference
//     recomputes the prompt only, scheduler.rs:251-255,352);
//   * a request that can never fit (prompt + max_tokens beyond max_model_len or beyond the
//     pool) is refused when it is added;
//   * the end-of-sequence id comes from the caller (the reference hard-codes 151645,
//     scheduler.rs:428).
// When pages run out: the newest running request gives back everything it holds, returns to
// the FRONT of `waiting` with num_computed = 0, and no request is admitted in that step.
#pragma once
#include <deque>
#include <memory>
#include <unordered_map>

#include "kv_cache_manager.hpp"
#include "step_batch.hpp"

namespace vob {

struct SamplingParams {
  float temperature = 0.0f;  // 0: greedy
  int top_k = 0;             // 0: off
  float top_p = 1.0f;        // >= 1 or <= 0: off
  int max_tokens = 16;
  bool ignore_eos = false;
  float presence_penalty = 0.0f, frequency_penalty = 0.0f, repetition_penalty = 0.0f;
  uint64_t seed = 0;
  bool own_seed = false;     // the request brought its seed: its random numbers then do not depend on its id
};

struct Sequence {
  int64_t id = -1;
  std::vector<int32_t> tokens;  // prompt, then generated tokens
  int num_prompt = 0;
  int num_computed = 0;         // tokens whose keys and values are in the cache
  int num_preemptions = 0;
  int num_cached = 0;           // tokens taken from the prefix cache at the last admission
  SamplingParams params;
  int num_generated() const { return static_cast<int>(tokens.size()) - num_prompt; }
};

struct ScheduledEntry {
  int64_t id;
  int start;
  int n;
  bool wants_logits;
};

struct RequestOutput {
  int64_t id;
  std::vector<int32_t> token_ids;  // generated tokens only
  bool finished;
  std::string finish_reason;       // "length", "stop"
};

struct SchedulerStats {
  int64_t steps = 0, prefill_tokens = 0, decode_tokens = 0, preemptions = 0, prefix_hit_tokens = 0, finished = 0;
  // sums over the steps booked so far: requests in a step, keys their queries could read (the context of every request
  // after its portion), rows that a token was sampled from.  They give a step's mean occupancy and its cache traffic.
  int64_t scheduled_requests = 0, context_tokens = 0, sampled_rows = 0;
};

// What the next step holds, for the engine to choose its buffers by: all single tokens -> a captured decode step.
struct StepSummary {
  int num_requests = 0, num_tokens = 0, num_rows = 0, max_pages = 0;
  bool all_single = true;
};

// The key of one sampled token's random numbers: a splitmix64 finaliser over (seed, request, index of the token in the
// request's output).  The same function as vllm_oxide_b200.sampling.sampler.row_key.
inline uint64_t sample_row_key(uint64_t seed, uint64_t request, uint64_t index) {
  uint64_t z = seed * 0x9E3779B97F4A7C15ull + request * 0xBF58476D1CE4E5B9ull + index * 0x94D049BB133111EBull +
               0x2545F4914F6CDD1Dull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

class Scheduler {
 public:
  Scheduler(std::shared_ptr<KvCacheManager> mgr, int max_num_batched_tokens, int max_num_seqs, int max_model_len,
            int eos_token_id)
      : mgr_(std::move(mgr)), budget_(max_num_batched_tokens), max_seqs_(max_num_seqs), max_len_(max_model_len),
        eos_(eos_token_id) {
    if (budget_ <= 0 || max_seqs_ <= 0 || max_len_ <= 0) throw PoolError("Scheduler: limits must be positive");
  }

  int64_t add_request(const std::vector<int32_t>& prompt, const SamplingParams& params) {
    if (prompt.empty()) throw PoolError("add_request: the prompt is empty");
    if (params.max_tokens <= 0) throw PoolError("add_request: max_tokens must be positive");
    const long total = static_cast<long>(prompt.size()) + params.max_tokens;
    if (total > max_len_)
      throw PoolError("add_request: prompt (" + std::to_string(prompt.size()) + ") + max_tokens (" +
                      std::to_string(params.max_tokens) + ") exceeds max_model_len " + std::to_string(max_len_));
    for (int g = 0; g < mgr_->num_groups(); ++g) {
      const auto& s = mgr_->group(g);
      long pages = (total + s.block_size - 1) / s.block_size;
      if (pages > s.num_blocks)
        throw PoolError("add_request: the request needs " + std::to_string(pages) + " pages of cache group " +
                        std::to_string(g) + " but the pool has " + std::to_string(s.num_blocks));
    }
    auto seq = std::make_unique<Sequence>();
    seq->id = next_id_++;
    seq->tokens = prompt;
    seq->num_prompt = static_cast<int>(prompt.size());
    seq->params = params;
    int64_t id = seq->id;
    by_id_[id] = seq.get();
    waiting_.push_back(std::move(seq));
    return id;
  }

  bool has_unfinished() const { return !waiting_.empty() || !running_.empty(); }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }
  const SchedulerStats& stats() const { return stats_; }

  const Sequence& sequence(int64_t id) const {
    auto it = by_id_.find(id);
    if (it == by_id_.end()) throw PoolError("Scheduler: no request " + std::to_string(id));
    return *it->second;
  }

  std::vector<int64_t> running_ids() const {
    std::vector<int64_t> v;
    for (const auto& s : running_) v.push_back(s->id);
    return v;
  }
  std::vector<int64_t> waiting_ids() const {
    std::vector<int64_t> v;
    for (const auto& s : waiting_) v.push_back(s->id);
    return v;
  }

  // The next step's batch: single tokens of decoding requests first, then portions.
  std::vector<ScheduledEntry> schedule() {
    std::vector<ScheduledEntry> entries;
    int budget = budget_;
    bool preempted = false;
    size_t i = 0;
    while (i < running_.size()) {
      Sequence* seq = running_[i].get();
      const int remaining = static_cast<int>(seq->tokens.size()) - seq->num_computed;
      const int n = std::min(remaining, budget);
      if (n <= 0) { ++i; continue; }
      bool gone = false;
      while (!mgr_->ensure(seq->id, seq->num_computed, n)) {
        Sequence* victim = running_.back().get();
        gone = victim == seq;
        preempt_last();
        preempted = true;
        if (gone) break;
      }
      if (gone) break;  // seq was the last running request
      entries.push_back({seq->id, seq->num_computed, n, seq->num_computed + n == static_cast<int>(seq->tokens.size())});
      budget -= n;
      ++i;
    }
    while (!preempted && budget > 0 && !waiting_.empty() && static_cast<int>(running_.size()) < max_seqs_) {
      Sequence* seq = waiting_.front().get();
      if (!mgr_->add_request(seq->id)) break;
      const int cached = mgr_->lookup_prefix(seq->id, seq->tokens.data(), static_cast<int>(seq->tokens.size()));
      const int remaining = static_cast<int>(seq->tokens.size()) - cached;
      const int n = std::min(remaining, budget);
      if (!mgr_->ensure(seq->id, cached, n)) {
        mgr_->free_request(seq->id);
        break;
      }
      seq->num_computed = cached;
      seq->num_cached = cached;
      stats_.prefix_hit_tokens += cached;
      entries.push_back({seq->id, cached, n, cached + n == static_cast<int>(seq->tokens.size())});
      budget -= n;
      running_.push_back(std::move(waiting_.front()));
      waiting_.pop_front();
    }
    std::stable_sort(entries.begin(), entries.end(),
                     [](const ScheduledEntry& a, const ScheduledEntry& b) { return (a.n > 1) < (b.n > 1); });
    last_ = entries;
    return entries;
  }

  // Books the step: `sampled` has one token for every entry that wanted logits, in entry order.
  std::vector<RequestOutput> postprocess(const std::vector<int32_t>& sampled) {
    std::vector<RequestOutput> outputs;
    size_t k = 0;
    ++stats_.steps;
    for (const auto& e : last_) {
      Sequence* seq = find_running(e.id);
      if (!seq) throw PoolError("postprocess: request " + std::to_string(e.id) + " is not running");
      seq->num_computed += e.n;
      (e.n == 1 && e.start >= seq->num_prompt ? stats_.decode_tokens : stats_.prefill_tokens) += e.n;
      ++stats_.scheduled_requests;
      stats_.context_tokens += e.start + e.n;
      stats_.sampled_rows += e.wants_logits;
      bool finished = false;
      std::string reason;
      if (e.wants_logits) {
        if (k >= sampled.size()) throw PoolError("postprocess: fewer sampled tokens than requests that wanted logits");
        const int32_t tok = sampled[k++];
        seq->tokens.push_back(tok);
        if (tok == eos_ && eos_ >= 0 && !seq->params.ignore_eos) { finished = true; reason = "stop"; }
        else if (seq->num_generated() >= seq->params.max_tokens || static_cast<int>(seq->tokens.size()) >= max_len_) {
          finished = true; reason = "length";
        }
      }
      mgr_->commit(seq->id, seq->tokens.data(), seq->num_computed);
      if (finished) {
        outputs.push_back({seq->id, std::vector<int32_t>(seq->tokens.begin() + seq->num_prompt, seq->tokens.end()),
                           true, reason});
        mgr_->free_request(seq->id);
        ++stats_.finished;
        by_id_.erase(seq->id);
        for (auto it = running_.begin(); it != running_.end(); ++it)
          if (it->get() == seq) { running_.erase(it); break; }
      } else {
        mgr_->advance(seq->id, seq->num_computed);
      }
    }
    if (k != sampled.size()) throw PoolError("postprocess: more sampled tokens than requests that wanted logits");
    last_.clear();
    return outputs;
  }

  const std::vector<ScheduledEntry>& last_entries() const { return last_; }

  // ---- the scheduled step without a detour through per-request objects of the caller's language
  StepSummary summary() const {
    StepSummary s;
    for (const auto& e : last_) {
      ++s.num_requests;
      s.num_tokens += e.n;
      s.num_rows += e.wants_logits;
      s.all_single = s.all_single && e.n == 1;
      for (int g = 0; g < mgr_->num_groups(); ++g)
        s.max_pages = std::max(s.max_pages, static_cast<int>(mgr_->block_table(e.id, g).size()));
    }
    return s;
  }

  // The step's arrays straight from the sequences (see fill_step_batch): a request that wants logits asks for its
  // last place.
  BatchCounts fill_batch(const BatchLayout& L, int32_t* out) {
    views_.clear();
    last_place_.resize(last_.size());
    for (size_t i = 0; i < last_.size(); ++i) {
      const auto& e = last_[i];
      const Sequence& q = sequence(e.id);
      last_place_[i] = e.n - 1;
      views_.push_back({e.id, e.start, q.tokens.data() + e.start, e.n, &last_place_[i], e.wants_logits ? 1 : 0});
    }
    return fill_step_views(*mgr_, views_, L, out);
  }

  // Sampling settings of the rows that a token is sampled from, in row order, into the caller's arrays (each of
  // `capacity` elements).  Returns the number of rows; *any_penalties says whether a row asks for penalties.
  int fill_sampling(float* temperature, float* top_p, int32_t* top_k, uint64_t* keys, int capacity, bool* any_penalties) const {
    int r = 0;
    *any_penalties = false;
    for (const auto& e : last_) {
      if (!e.wants_logits) continue;
      if (r >= capacity) throw PoolError("fill_sampling: more sampled rows than the arrays hold");
      const Sequence& q = sequence(e.id);
      const SamplingParams& p = q.params;
      temperature[r] = p.temperature;
      top_p[r] = p.top_p;
      top_k[r] = p.top_k;
      keys[r] = sample_row_key(p.seed, p.own_seed ? 0ull : static_cast<uint64_t>(q.id), static_cast<uint64_t>(q.num_generated()));
      *any_penalties = *any_penalties || p.presence_penalty != 0.f || p.frequency_penalty != 0.f || p.repetition_penalty != 0.f;
      ++r;
    }
    return r;
  }

 private:
  Sequence* find_running(int64_t id) {
    auto it = by_id_.find(id);
    return it == by_id_.end() ? nullptr : it->second;
  }
  void preempt_last() {
    std::unique_ptr<Sequence> v = std::move(running_.back());
    running_.pop_back();
    mgr_->free_request(v->id);
    v->num_computed = 0;
    ++v->num_preemptions;
    ++stats_.preemptions;
    waiting_.push_front(std::move(v));
  }

  std::shared_ptr<KvCacheManager> mgr_;
  int budget_, max_seqs_, max_len_, eos_;
  int64_t next_id_ = 0;
  std::deque<std::unique_ptr<Sequence>> waiting_, running_;
  std::unordered_map<int64_t, Sequence*> by_id_;   // every unfinished request, waiting or running
  std::vector<ScheduledEntry> last_;
  std::vector<EntryView> views_;
  std::vector<int32_t> last_place_;
  SchedulerStats stats_;
};

}  // namespace vob
