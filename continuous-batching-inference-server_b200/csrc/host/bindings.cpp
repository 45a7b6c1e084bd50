// pybind11 module of the host runtime: CacheManager and Scheduler.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "cache_manager.hpp"
#include "scheduler.hpp"
#include "step_packer.hpp"

namespace py = pybind11;
using namespace cbis;

PYBIND11_MODULE(_cbis_host, m) {
  m.doc() = "Host runtime: paged cache manager with groups and state slots, continuous-batching scheduler";

  py::class_<GroupSpec>(m, "GroupSpec")
      .def(py::init([](int page_size, int num_pages, int window) {
             GroupSpec g;
             g.page_size = page_size;
             g.num_pages = num_pages;
             g.window = window;
             return g;
           }),
           py::arg("page_size"), py::arg("num_pages"), py::arg("window") = 0)
      .def_readwrite("page_size", &GroupSpec::page_size)
      .def_readwrite("num_pages", &GroupSpec::num_pages)
      .def_readwrite("window", &GroupSpec::window);

  py::class_<CacheManager>(m, "CacheManager")
      .def(py::init<std::vector<GroupSpec>, int>(), py::arg("groups"), py::arg("max_requests"))
      .def("num_groups", &CacheManager::num_groups)
      .def("max_requests", &CacheManager::max_requests)
      .def("page_size", &CacheManager::page_size)
      .def("num_pages", &CacheManager::num_pages)
      .def("window", &CacheManager::window)
      .def("free_pages", &CacheManager::free_pages)
      .def("free_slots", &CacheManager::free_slots)
      .def("admit", &CacheManager::admit)
      .def("live", &CacheManager::live)
      .def("length", &CacheManager::length)
      .def("request_id", &CacheManager::request_id)
      .def("pages_needed", &CacheManager::pages_needed)
      .def("can_append", &CacheManager::can_append)
      .def("max_appendable", &CacheManager::max_appendable)
      .def("fits_fresh", &CacheManager::fits_fresh)
      .def("fits_at_all", &CacheManager::fits_at_all)
      .def("append", &CacheManager::append)
      .def("release_out_of_window", &CacheManager::release_out_of_window)
      .def("release", &CacheManager::release)
      .def("block_table", &CacheManager::block_table)
      .def("table_len", &CacheManager::table_len)
      .def("token_slot", &CacheManager::token_slot)
      .def("record_freed", &CacheManager::record_freed)
      .def("take_freed", &CacheManager::take_freed)
      .def("check", &CacheManager::check);

  py::class_<SchedulerLimits>(m, "SchedulerLimits")
      .def(py::init([](int max_num_seqs, int max_batched_tokens, int prefill_chunk, int max_positions) {
             SchedulerLimits l;
             l.max_num_seqs = max_num_seqs;
             l.max_batched_tokens = max_batched_tokens;
             l.prefill_chunk = prefill_chunk;
             l.max_positions = max_positions;
             return l;
           }),
           py::arg("max_num_seqs"), py::arg("max_batched_tokens"), py::arg("prefill_chunk"),
           py::arg("max_positions"));

  py::class_<PlannedEntry>(m, "PlannedEntry")
      .def_readonly("request_id", &PlannedEntry::request_id)
      .def_readonly("slot", &PlannedEntry::slot)
      .def_readonly("start", &PlannedEntry::start)
      .def_readonly("tokens", &PlannedEntry::tokens)
      .def_property_readonly("n_tokens", [](const PlannedEntry& e) { return (int)e.tokens.size(); })
      .def_readonly("sample", &PlannedEntry::sample)
      .def_readonly("output_index", &PlannedEntry::output_index)
      .def_readonly("ahead", &PlannedEntry::ahead)
      .def_readonly("source", &PlannedEntry::source);

  py::class_<Finished>(m, "Finished")
      .def_readonly("request_id", &Finished::request_id)
      .def_readonly("reason", &Finished::reason)
      .def_readonly("output", &Finished::output);

  py::class_<PackEntry>(m, "PackEntry")
      .def(py::init([](int slot, int start, std::vector<int> tokens, std::vector<int> want) {
             PackEntry e;
             e.slot = slot;
             e.start = start;
             e.tokens = std::move(tokens);
             e.want = std::move(want);
             return e;
           }),
           py::arg("slot"), py::arg("start"), py::arg("tokens"), py::arg("want"));

  py::class_<PackInfo>(m, "PackInfo")
      .def_readonly("n_rows", &PackInfo::n_rows)
      .def_readonly("n_tokens", &PackInfo::n_tokens)
      .def_readonly("n_wanting", &PackInfo::n_wanting)
      .def_readonly("n_wanted", &PackInfo::n_wanted)
      .def_readonly("n_segments", &PackInfo::n_segments)
      .def_readonly("n_logit_rows", &PackInfo::n_logit_rows)
      .def_readonly("n_decode", &PackInfo::n_decode)
      .def_readonly("max_seg_rows", &PackInfo::max_seg_rows)
      .def_readonly("max_ctx", &PackInfo::max_ctx)
      .def_readonly("seg_rows", &PackInfo::seg_rows)
      .def_readonly("seg_ctx", &PackInfo::seg_ctx);

  py::class_<StepPacker>(m, "StepPacker")
      .def(py::init<const CacheManager*, int, int, int, int, std::vector<int>, int>(), py::arg("cache"),
           py::arg("max_tokens"), py::arg("max_seqs"), py::arg("vocab"), py::arg("max_positions"),
           py::arg("max_blocks"), py::arg("n_groups"), py::keep_alive<1, 2>())
      .def("words", &StepPacker::words)
      .def("layout", &StepPacker::layout)
      .def("pack", &StepPacker::pack, py::arg("buffer"), py::arg("entries"), py::arg("pad_rows") = 0,
           py::arg("all_logits") = false, py::arg("reserved_ahead") = false, py::arg("pad_segments") = 0)
      .def("pack_plan", &StepPacker::pack_plan, py::arg("buffer"), py::arg("plan"), py::arg("pad_rows") = 0,
           py::arg("all_logits") = false, py::arg("pad_segments") = 0);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<CacheManager*, SchedulerLimits>(), py::arg("cache"), py::arg("limits"),
           py::keep_alive<1, 2>())
      .def("add", &Scheduler::add, py::arg("request_id"), py::arg("prompt"), py::arg("max_new_tokens"),
           py::arg("eos_token") = -1, py::arg("ignore_eos") = false)
      .def("abort", &Scheduler::abort)
      .def("num_waiting", &Scheduler::num_waiting)
      .def("num_running", &Scheduler::num_running)
      .def("idle", &Scheduler::idle)
      .def("preemptions", &Scheduler::preemptions)
      .def("running_ids", &Scheduler::running_ids)
      .def("waiting_ids", &Scheduler::waiting_ids)
      .def("schedule", &Scheduler::schedule)
      .def("schedule_ahead", &Scheduler::schedule_ahead)
      .def("ahead_sources", &Scheduler::ahead_sources)
      .def("take_new_slots", &Scheduler::take_new_slots)
      .def("update", &Scheduler::update)
      .def("update_plan", &Scheduler::update_plan);
}
