// pybind11 face of the host runtime: cache manager, step batch builder, scheduler.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.hpp"
#include "scheduler.hpp"

namespace py = pybind11;
using namespace llmhost;

namespace {

// A step's entries, kept on the C++ side so that planning and batch building exchange no lists.
struct StepEntries {
  std::vector<StepEntry> v;
};

}  // namespace

PYBIND11_MODULE(_llmengine_host, m) {
  m.doc() = "llmengine host runtime: paged-cache bookkeeping, step batch builder, continuous-batching scheduler";

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](int num_pages, int window) { GroupSpec g; g.num_pages = num_pages; g.window = window; return g; }),
           py::arg("num_pages"), py::arg("window") = 0)
      .def_readonly("num_pages", &GroupSpec::num_pages)
      .def_readonly("window", &GroupSpec::window);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<int, std::vector<GroupSpec>, int>(), py::arg("page_size"), py::arg("groups"), py::arg("num_slots"))
      .def_property_readonly("page_size", &CacheManager::page_size)
      .def_property_readonly("num_groups", &CacheManager::num_groups)
      .def_property_readonly("num_slots", &CacheManager::num_slots)
      .def_property_readonly("free_slots", &CacheManager::free_slots)
      .def_property_readonly("num_requests", &CacheManager::num_requests)
      .def("num_pages", &CacheManager::num_pages, py::arg("group") = 0)
      .def("free_pages", &CacheManager::free_pages, py::arg("group") = 0)
      .def("window", &CacheManager::window, py::arg("group") = 0)
      .def("add_request", &CacheManager::add_request)
      .def("has_request", &CacheManager::has_request)
      .def("length", &CacheManager::length)
      .def("reserved", &CacheManager::reserved)
      .def("slot", &CacheManager::slot)
      .def("reserve", &CacheManager::reserve)
      .def("advance", &CacheManager::advance)
      .def("release", &CacheManager::release)
      .def("block_table", &CacheManager::block_table, py::arg("id"), py::arg("group") = 0)
      .def("request_ids", &CacheManager::request_ids)
      .def("check", &CacheManager::check);

  py::class_<StepEntries>(m, "StepEntries")
      .def(py::init<>())
      .def("add",
           [](StepEntries& s, std::int64_t id, std::vector<std::int32_t> tokens, std::vector<std::int32_t> want,
              float temperature, std::int32_t seed, std::int32_t draw) {
             StepEntry e;
             e.id = id; e.tokens = std::move(tokens); e.want = std::move(want);
             e.temperature = temperature; e.seed = seed; e.draw = draw;
             s.v.push_back(std::move(e));
           },
           py::arg("id"), py::arg("tokens"), py::arg("want"), py::arg("temperature") = 0.f, py::arg("seed") = 0,
           py::arg("draw") = 0)
      .def("__len__", [](const StepEntries& s) { return s.v.size(); })
      .def("ids", [](const StepEntries& s) { std::vector<std::int64_t> o; for (auto& e : s.v) o.push_back(e.id); return o; })
      .def("tokens", [](const StepEntries& s, int i) { return s.v.at(i).tokens; })
      .def("want", [](const StepEntries& s, int i) { return s.v.at(i).want; })
      .def("num_tokens", [](const StepEntries& s) { std::size_t n = 0; for (auto& e : s.v) n += e.tokens.size(); return n; })
      .def("num_rows", [](const StepEntries& s) { std::size_t n = 0; for (auto& e : s.v) n += e.want.size(); return n; })
      .def("max_tokens", [](const StepEntries& s) { std::size_t n = 0; for (auto& e : s.v) n = std::max(n, e.tokens.size()); return n; });

  py::class_<StepLayout>(m, "StepLayout")
      .def_static("make", &StepLayout::make, py::arg("cap_tokens"), py::arg("cap_seqs"), py::arg("cap_rows"),
                  py::arg("max_blocks"), py::arg("num_groups"))
      .def_readonly("cap_tokens", &StepLayout::cap_tokens)
      .def_readonly("cap_seqs", &StepLayout::cap_seqs)
      .def_readonly("cap_rows", &StepLayout::cap_rows)
      .def_readonly("max_blocks", &StepLayout::max_blocks)
      .def_readonly("num_groups", &StepLayout::num_groups)
      .def_readonly("token_ids", &StepLayout::token_ids)
      .def_readonly("positions", &StepLayout::positions)
      .def_readonly("token_seq", &StepLayout::token_seq)
      .def_readonly("logit_rows", &StepLayout::logit_rows)
      .def_readonly("row_temperature", &StepLayout::row_temperature)
      .def_readonly("row_seed", &StepLayout::row_seed)
      .def_readonly("row_draw", &StepLayout::row_draw)
      .def_readonly("seq_start", &StepLayout::seq_start)
      .def_readonly("seq_ntok", &StepLayout::seq_ntok)
      .def_readonly("seq_qoff", &StepLayout::seq_qoff)
      .def_readonly("seq_slot", &StepLayout::seq_slot)
      .def_readonly("seq_len", &StepLayout::seq_len)
      .def_readonly("block_tables", &StepLayout::block_tables)
      .def_readonly("total", &StepLayout::total);

  py::class_<StepCounts>(m, "StepCounts")
      .def_readonly("n_tokens", &StepCounts::n_tokens)
      .def_readonly("n_seqs", &StepCounts::n_seqs)
      .def_readonly("n_rows", &StepCounts::n_rows)
      .def_readonly("max_seq_len", &StepCounts::max_seq_len)
      .def_readonly("max_new_tokens", &StepCounts::max_new_tokens)
      .def_readonly("decode_only", &StepCounts::decode_only);

  m.def("fill_step",
        [](const CacheManager& cm, const StepEntries& entries, const StepLayout& layout, std::uintptr_t staging,
           bool pad, int vocab_size, int max_positions) {
          return fill_step(cm, entries.v, layout, reinterpret_cast<std::int32_t*>(staging), pad, vocab_size, max_positions);
        },
        py::arg("cache_manager"), py::arg("entries"), py::arg("layout"), py::arg("staging_ptr"), py::arg("pad"),
        py::arg("vocab_size"), py::arg("max_positions"),
        "Writes the step's flat int32 arrays at staging_ptr (host memory of layout.total int32s).");

  m.def("step_caps",
        [](const CacheManager& cm, const StepEntries& entries) {
          int tokens = 0, rows = 0, blocks = 1;
          for (const auto& e : entries.v) {
            tokens += static_cast<int>(e.tokens.size());
            rows += static_cast<int>(e.want.size());
            for (int g = 0; g < cm.num_groups(); ++g)
              blocks = std::max(blocks, static_cast<int>(cm.block_table(e.id, g).size()));
          }
          return py::make_tuple(tokens, static_cast<int>(entries.v.size()), rows, blocks);
        },
        "-> (tokens, requests, wanted rows, longest block table) of a step whose pages are reserved");

  py::class_<SequenceResult>(m, "SequenceResult")
      .def(py::init([](std::int64_t seq_id, int prompt_len, std::vector<std::int32_t> token_ids, std::string reason) {
             SequenceResult r; r.seq_id = seq_id; r.prompt_len = prompt_len; r.token_ids = std::move(token_ids);
             r.finish_reason = std::move(reason); return r;
           }),
           py::arg("seq_id") = 0, py::arg("prompt_len") = 0, py::arg("token_ids") = std::vector<std::int32_t>{},
           py::arg("finish_reason") = "")
      .def_readonly("seq_id", &SequenceResult::seq_id)
      .def_readonly("prompt_len", &SequenceResult::prompt_len)
      .def_readonly("token_ids", &SequenceResult::token_ids)
      .def_readonly("finish_reason", &SequenceResult::finish_reason)
      .def("__repr__", [](const SequenceResult& r) {
        return "SequenceResult(seq_id=" + std::to_string(r.seq_id) + ", prompt_len=" + std::to_string(r.prompt_len) +
               ", n_tokens=" + std::to_string(r.token_ids.size()) + ", finish_reason='" + r.finish_reason + "')";
      });

  py::class_<Scheduler>(m, "SchedulerCore")
      .def(py::init<CacheManager&, int, int, std::set<int>, int, int, std::int64_t, int>(), py::arg("cache_manager"),
           py::arg("vocab_size"), py::arg("max_positions"), py::arg("eos_token_ids"), py::arg("max_concurrent") = 64,
           py::arg("max_prefill_tokens_per_step") = 256, py::arg("id_base") = 0, py::arg("portion_multiple") = 1,
           py::keep_alive<1, 2>())
      .def_property_readonly("last_admitted", &Scheduler::last_admitted)
      .def("enqueue", &Scheduler::enqueue, py::arg("prompt"), py::arg("max_new_tokens"), py::arg("temperature") = 0.f,
           py::arg("seed") = 0)
      .def("plan", [](Scheduler& s) { StepEntries e; e.v = s.plan(); return e; })
      .def("commit", &Scheduler::commit)
      .def("fail_step", &Scheduler::fail_step, py::arg("reason") = "error")
      .def_property_readonly("portion_multiple", &Scheduler::portion_multiple)
      .def("finalize", &Scheduler::finalize)
      .def_property_readonly("idle", &Scheduler::idle)
      .def_property_readonly("has_unfinished", &Scheduler::has_unfinished)
      .def_property_readonly("plan_open", &Scheduler::plan_open)
      .def_property_readonly("results", &Scheduler::results)
      .def("clear_results", &Scheduler::clear_results)
      .def_property("budget", &Scheduler::budget, &Scheduler::set_budget)
      .def_property_readonly("max_concurrent", &Scheduler::max_concurrent)
      .def_property_readonly("num_waiting", &Scheduler::num_waiting)
      .def_property_readonly("num_prefilling", &Scheduler::num_prefilling)
      .def_property_readonly("num_running", &Scheduler::num_running);
}
