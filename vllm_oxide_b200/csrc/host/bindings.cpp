// Python bindings of the host runtime: block pool, cache manager, scheduler, batch builder.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "scheduler.hpp"
#include "step_batch.hpp"

namespace py = pybind11;
using namespace vob;

PYBIND11_MODULE(_host, m) {
  m.doc() = "host runtime of the engine: pages, block tables, state slots, scheduler";
  py::register_exception<PoolError>(m, "PoolError", PyExc_RuntimeError);

  m.def("xxh64", [](py::bytes data, uint64_t seed) {
    std::string s = data;
    return xxh64(reinterpret_cast<const uint8_t*>(s.data()), s.size(), seed);
  }, py::arg("data"), py::arg("seed") = 0);
  m.def("chain_hash", [](int64_t prev, const std::vector<int32_t>& tokens) {
    return chain_hash(prev, tokens.data(), static_cast<int>(tokens.size()));
  });

  py::class_<BlockPool>(m, "BlockPool")
      .def(py::init<int, int>(), py::arg("num_blocks"), py::arg("block_size"))
      .def_property_readonly("num_blocks", &BlockPool::num_blocks)
      .def_property_readonly("block_size", &BlockPool::block_size)
      .def_property_readonly("num_free", &BlockPool::num_free)
      .def("ref_count", &BlockPool::ref_count)
      .def("is_free", &BlockPool::is_free)
      .def("hash_of", &BlockPool::hash_of)
      .def("allocate", &BlockPool::allocate)
      .def("retain", &BlockPool::retain)
      .def("release", &BlockPool::release)
      .def("lookup", [](const BlockPool& p, int64_t h, const std::vector<int32_t>& t) {
        return p.lookup(h, t.data(), static_cast<int>(t.size()));
      })
      .def("publish", [](BlockPool& p, int id, int64_t h, const std::vector<int32_t>& t) {
        p.publish(id, h, t.data(), static_cast<int>(t.size()));
      })
      .def("free_order", &BlockPool::free_order);

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](int block_size, int num_blocks, int window) {
        GroupSpec g; g.block_size = block_size; g.num_blocks = num_blocks; g.window = window; return g;
      }), py::arg("block_size"), py::arg("num_blocks"), py::arg("window") = 0)
      .def_readwrite("block_size", &GroupSpec::block_size)
      .def_readwrite("num_blocks", &GroupSpec::num_blocks)
      .def_readwrite("window", &GroupSpec::window);

  py::class_<KvCacheManager, std::shared_ptr<KvCacheManager>>(m, "KvCacheManager")
      .def(py::init<const std::vector<GroupSpec>&, int, bool>(), py::arg("groups"), py::arg("num_state_slots"),
           py::arg("prefix_caching") = false)
      .def_property_readonly("num_groups", &KvCacheManager::num_groups)
      .def_property_readonly("prefix_caching", &KvCacheManager::prefix_caching)
      .def_property_readonly("num_requests", &KvCacheManager::num_requests)
      .def_property_readonly("num_free_state_slots", &KvCacheManager::num_free_state_slots)
      .def("group", &KvCacheManager::group)
      .def("num_free_blocks", &KvCacheManager::num_free_blocks, py::arg("group") = 0)
      .def("has_request", &KvCacheManager::has_request)
      .def("add_request", &KvCacheManager::add_request)
      .def("lookup_prefix", [](KvCacheManager& k, int64_t id, const std::vector<int32_t>& t) {
        return k.lookup_prefix(id, t.data(), static_cast<int>(t.size()));
      })
      .def("restorable_tokens", [](const KvCacheManager& k, const std::vector<int32_t>& t) {
        return k.restorable_tokens(t.data(), static_cast<int>(t.size()));
      })
      .def("pages_needed", &KvCacheManager::pages_needed)
      .def("can_ensure", &KvCacheManager::can_ensure)
      .def("ensure", &KvCacheManager::ensure)
      .def("advance", &KvCacheManager::advance)
      .def("commit", [](KvCacheManager& k, int64_t id, const std::vector<int32_t>& t, int n) {
        if (n > static_cast<int>(t.size())) throw PoolError("commit: more computed tokens than tokens");
        k.commit(id, t.data(), n);
      })
      .def("release_pages", &KvCacheManager::release_pages)
      .def("free_request", &KvCacheManager::free_request)
      .def("block_table", &KvCacheManager::block_table)
      .def("state_slot", &KvCacheManager::state_slot)
      .def("slot_mapping", [](const KvCacheManager& k, int64_t id, int g, int start, int n) {
        std::vector<int32_t> v(n);
        k.slot_mapping(id, g, start, n, v.data());
        return v;
      })
      .def("ref_count", [](const KvCacheManager& k, int g, int b) { return k.pool(g).ref_count(b); })
      .def("free_order", [](const KvCacheManager& k, int g) { return k.pool(g).free_order(); })
      .def("check_invariants", &KvCacheManager::check_invariants);

  py::class_<SamplingParams>(m, "SchedSamplingParams")
      .def(py::init<>())
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("max_tokens", &SamplingParams::max_tokens)
      .def_readwrite("ignore_eos", &SamplingParams::ignore_eos)
      .def_readwrite("presence_penalty", &SamplingParams::presence_penalty)
      .def_readwrite("frequency_penalty", &SamplingParams::frequency_penalty)
      .def_readwrite("repetition_penalty", &SamplingParams::repetition_penalty)
      .def_readwrite("seed", &SamplingParams::seed)
      .def_readwrite("own_seed", &SamplingParams::own_seed);

  py::class_<Sequence>(m, "Sequence")
      .def_readonly("id", &Sequence::id)
      .def_readonly("tokens", &Sequence::tokens)
      .def_readonly("num_prompt", &Sequence::num_prompt)
      .def_readonly("num_computed", &Sequence::num_computed)
      .def_readonly("num_preemptions", &Sequence::num_preemptions)
      .def_readonly("num_cached", &Sequence::num_cached)
      .def_readonly("params", &Sequence::params)
      .def_property_readonly("num_generated", &Sequence::num_generated);

  py::class_<ScheduledEntry>(m, "ScheduledEntry")
      .def_readonly("id", &ScheduledEntry::id)
      .def_readonly("start", &ScheduledEntry::start)
      .def_readonly("n", &ScheduledEntry::n)
      .def_readonly("wants_logits", &ScheduledEntry::wants_logits)
      .def("__repr__", [](const ScheduledEntry& e) {
        return "ScheduledEntry(id=" + std::to_string(e.id) + ", start=" + std::to_string(e.start) + ", n=" +
               std::to_string(e.n) + ", wants_logits=" + (e.wants_logits ? "True" : "False") + ")";
      });

  py::class_<RequestOutput>(m, "SchedRequestOutput")
      .def_readonly("id", &RequestOutput::id)
      .def_readonly("token_ids", &RequestOutput::token_ids)
      .def_readonly("finished", &RequestOutput::finished)
      .def_readonly("finish_reason", &RequestOutput::finish_reason);

  py::class_<SchedulerStats>(m, "SchedulerStats")
      .def_readonly("steps", &SchedulerStats::steps)
      .def_readonly("prefill_tokens", &SchedulerStats::prefill_tokens)
      .def_readonly("decode_tokens", &SchedulerStats::decode_tokens)
      .def_readonly("preemptions", &SchedulerStats::preemptions)
      .def_readonly("prefix_hit_tokens", &SchedulerStats::prefix_hit_tokens)
      .def_readonly("finished", &SchedulerStats::finished)
      .def_readonly("scheduled_requests", &SchedulerStats::scheduled_requests)
      .def_readonly("context_tokens", &SchedulerStats::context_tokens)
      .def_readonly("sampled_rows", &SchedulerStats::sampled_rows);

  py::class_<StepSummary>(m, "StepSummary")
      .def_readonly("num_requests", &StepSummary::num_requests)
      .def_readonly("num_tokens", &StepSummary::num_tokens)
      .def_readonly("num_rows", &StepSummary::num_rows)
      .def_readonly("max_pages", &StepSummary::max_pages)
      .def_readonly("all_single", &StepSummary::all_single);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<std::shared_ptr<KvCacheManager>, int, int, int, int>(), py::arg("manager"),
           py::arg("max_num_batched_tokens"), py::arg("max_num_seqs"), py::arg("max_model_len"),
           py::arg("eos_token_id") = -1)
      .def("add_request", &Scheduler::add_request)
      .def("has_unfinished", &Scheduler::has_unfinished)
      .def_property_readonly("num_waiting", &Scheduler::num_waiting)
      .def_property_readonly("num_running", &Scheduler::num_running)
      .def_property_readonly("stats", &Scheduler::stats)
      .def("sequence", &Scheduler::sequence, py::return_value_policy::copy)
      .def("running_ids", &Scheduler::running_ids)
      .def("waiting_ids", &Scheduler::waiting_ids)
      .def("schedule", &Scheduler::schedule)
      // schedule() for callers that go on with summary() / fill_batch(): returns the number of requests in the step
      .def("schedule_step", [](Scheduler& s) { return static_cast<int>(s.schedule().size()); })
      .def("row_key", [](const Scheduler&, uint64_t seed, uint64_t request, uint64_t index) {
        return sample_row_key(seed, request, index);
      })
      .def("postprocess", &Scheduler::postprocess)
      .def("last_entries", &Scheduler::last_entries)
      .def("summary", &Scheduler::summary)
      // The scheduled step's arrays into `out` (as fill_step_batch, without building entries).
      .def("fill_batch", [](Scheduler& s, const BatchLayout& L, py::array_t<int32_t, py::array::c_style> out) {
        if (out.size() < L.total) throw PoolError("fill_batch: the output buffer is smaller than the layout");
        return s.fill_batch(L, out.mutable_data());
      })
      // Sampling settings of the sampled rows into the caller's arrays; returns (rows, any row with penalties).
      .def("fill_sampling", [](const Scheduler& s, py::array_t<float, py::array::c_style> temperature,
                               py::array_t<float, py::array::c_style> top_p, py::array_t<int32_t, py::array::c_style> top_k,
                               py::array_t<uint64_t, py::array::c_style> keys) {
        const long cap = std::min(std::min(temperature.size(), top_p.size()), std::min(top_k.size(), keys.size()));
        bool any = false;
        int r = s.fill_sampling(temperature.mutable_data(), top_p.mutable_data(), top_k.mutable_data(), keys.mutable_data(),
                                static_cast<int>(cap), &any);
        return std::make_pair(r, any);
      })
      // For every scheduled request that wants logits, in entry order:
      // (id, generated so far, temperature, top_k, top_p, seed, has penalties).
      .def("sample_requests", [](const Scheduler& s) {
        std::vector<std::tuple<int64_t, int, float, int, float, uint64_t, bool, int64_t>> out;
        for (const auto& e : s.last_entries()) {
          if (!e.wants_logits) continue;
          const Sequence& q = s.sequence(e.id);
          const SamplingParams& p = q.params;
          out.emplace_back(q.id, q.num_generated(), p.temperature, p.top_k, p.top_p, p.seed,
                           p.presence_penalty != 0.f || p.frequency_penalty != 0.f || p.repetition_penalty != 0.f,
                           p.own_seed ? int64_t(0) : q.id);   // what the random numbers are keyed by, beside seed and index
        }
        return out;
      })
      // The scheduled portions as batch entries (tokens taken from the sequences; a request that
      // wants logits asks for its last place).
      .def("batch_entries", [](const Scheduler& s) {
        std::vector<BatchEntry> out;
        for (const auto& e : s.last_entries()) {
          const Sequence& q = s.sequence(e.id);
          BatchEntry b;
          b.id = e.id; b.start = e.start;
          b.tokens.assign(q.tokens.begin() + e.start, q.tokens.begin() + e.start + e.n);
          if (e.wants_logits) b.want.push_back(e.n - 1);
          out.push_back(std::move(b));
        }
        return out;
      });

  py::class_<BatchLayout>(m, "BatchLayout")
      .def(py::init<int, int, int, int, int>(), py::arg("T"), py::arg("B"), py::arg("R"), py::arg("G"), py::arg("P"))
      .def_readonly("T", &BatchLayout::T).def_readonly("B", &BatchLayout::B).def_readonly("R", &BatchLayout::R)
      .def_readonly("G", &BatchLayout::G).def_readonly("P", &BatchLayout::P)
      .def_readonly("token_ids", &BatchLayout::token_ids).def_readonly("positions", &BatchLayout::positions)
      .def_readonly("token_req", &BatchLayout::token_req).def_readonly("slot_mapping", &BatchLayout::slot_mapping)
      .def_readonly("cu_q", &BatchLayout::cu_q).def_readonly("context_lens", &BatchLayout::context_lens)
      .def_readonly("state_slots", &BatchLayout::state_slots).def_readonly("state_fresh", &BatchLayout::state_fresh)
      .def_readonly("logit_rows", &BatchLayout::logit_rows).def_readonly("block_tables", &BatchLayout::block_tables)
      .def_readonly("total", &BatchLayout::total);

  py::class_<BatchEntry>(m, "BatchEntry")
      .def(py::init([](int64_t id, int start, std::vector<int32_t> tokens, std::vector<int32_t> want) {
        BatchEntry e; e.id = id; e.start = start; e.tokens = std::move(tokens); e.want = std::move(want); return e;
      }), py::arg("id"), py::arg("start"), py::arg("tokens"), py::arg("want"))
      .def_readonly("id", &BatchEntry::id).def_readonly("start", &BatchEntry::start)
      .def_readonly("tokens", &BatchEntry::tokens).def_readonly("want", &BatchEntry::want);

  py::class_<BatchCounts>(m, "BatchCounts")
      .def_readonly("num_tokens", &BatchCounts::num_tokens).def_readonly("num_requests", &BatchCounts::num_requests)
      .def_readonly("num_rows", &BatchCounts::num_rows).def_readonly("num_decode", &BatchCounts::num_decode)
      .def_readonly("max_q", &BatchCounts::max_q).def_readonly("max_context", &BatchCounts::max_context);

  m.def("fill_step_batch", [](KvCacheManager& mgr, const std::vector<BatchEntry>& entries, const BatchLayout& L,
                              py::array_t<int32_t, py::array::c_style> out) {
    if (out.size() < L.total) throw PoolError("fill_step_batch: the output buffer is smaller than the layout");
    return fill_step_batch(mgr, entries, L, out.mutable_data());
  });
}
