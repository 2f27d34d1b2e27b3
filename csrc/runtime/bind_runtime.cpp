// Python module `_runtime`: the C++ host runtime (planner, radix cache, pools, tiered state
// store, reshard planner) and, under `_runtime.golden`, the f32 CPU golden ops.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <pybind11/numpy.h>

#include "safetensors_file.h"
#include "slot_scheduler.h"
#include "tick_planner.h"

namespace py = pybind11;
using namespace fbrt;

void bind_golden(py::module_& m);

#ifndef FB_RUNTIME_BUILD_ID
#define FB_RUNTIME_BUILD_ID "unknown"
#endif

PYBIND11_MODULE(_runtime, m) {
    m.doc() = "ferrite_b200 host runtime";
    m.attr("build_id") = FB_RUNTIME_BUILD_ID;
    py::module_ g = m.def_submodule("golden", "f32 CPU golden ops");
    bind_golden(g);

    py::class_<SafetensorsFile>(m, "SafetensorsFile")
        .def(py::init<const std::string&>())
        .def("header", [](const SafetensorsFile& f) { return py::bytes(f.header()); })
        .def_property_readonly("data_offset", &SafetensorsFile::data_offset)
        .def_property_readonly("data_size", &SafetensorsFile::data_size)
        .def("view", [](py::object self, size_t begin, size_t end) {
            // zero-copy uint8 view of data bytes [begin, end); keeps the file alive
            auto& f = self.cast<SafetensorsFile&>();
            if (end > f.data_size() || begin > end) throw std::out_of_range("view range");
            return py::array_t<uint8_t>({(py::ssize_t)(end - begin)}, {1}, f.data() + begin, self);
        })
        .def("copy_rows", [](const SafetensorsFile& f, size_t begin, size_t row_bytes, size_t r0, size_t r1, size_t c0,
                             size_t c1, py::array_t<uint8_t, py::array::c_style> dst) {
            if ((size_t)dst.size() < (r1 - r0) * (c1 - c0)) throw std::out_of_range("dst too small");
            f.copy_rows(begin, row_bytes, r0, r1, c0, c1, dst.mutable_data());
        })
        .def("dequant_e4m3_block", [](const SafetensorsFile& f, size_t begin, size_t scale_begin, size_t rows, size_t cols,
                                      size_t blk, size_t r0, size_t r1) {
            py::array_t<float> out({(py::ssize_t)(r1 - r0), (py::ssize_t)cols});
            f.dequant_e4m3_block(begin, scale_begin, rows, cols, blk, r0, r1, out.mutable_data());
            return out;
        });
    m.def("e4m3_to_f32", &e4m3_to_f32);

    m.def("cp_layer_range", &cp_layer_range);
    m.def("bucket_for", &bucket_for);

    py::class_<PagePool>(m, "PagePool")
        .def(py::init<int>())
        .def("alloc", &PagePool::alloc).def("retain", &PagePool::retain).def("release", &PagePool::release)
        .def("refcount", &PagePool::refcount).def("can_alloc", &PagePool::can_alloc)
        .def_property_readonly("free_pages", &PagePool::free_pages)
        .def_property_readonly("pages_in_use", &PagePool::pages_in_use)
        .def_property_readonly("num_pages", &PagePool::num_pages);
    py::class_<SlotPool>(m, "SlotPool")
        .def(py::init<int>())
        .def("alloc", &SlotPool::alloc).def("free", &SlotPool::free).def("is_used", &SlotPool::is_used)
        .def_property_readonly("in_use", &SlotPool::in_use).def_property_readonly("capacity", &SlotPool::capacity);

    py::class_<PageMove>(m, "PageMove")
        .def_readonly("page", &PageMove::page).def_readonly("dst_rank", &PageMove::dst_rank)
        .def_readonly("dst_index", &PageMove::dst_index);
    py::class_<ReshardPlan>(m, "ReshardPlan")
        .def_static("compile", &ReshardPlan::compile)
        .def("filter_pages", &ReshardPlan::filter_pages)
        .def_readonly("state_layers", &ReshardPlan::state_layers).def_readonly("paged_layers", &ReshardPlan::paged_layers)
        .def_readonly("layer_owner", &ReshardPlan::layer_owner).def_readonly("moves", &ReshardPlan::moves)
        .def_readonly("n_cp", &ReshardPlan::n_cp).def_readonly("n_dcp", &ReshardPlan::n_dcp);

    py::class_<RadixStats>(m, "RadixStats")
        .def_readonly("tree_nodes", &RadixStats::tree_nodes).def_readonly("tree_blocks", &RadixStats::tree_blocks)
        .def_readonly("evictable_tokens", &RadixStats::evictable_tokens)
        .def_readonly("protected_tokens", &RadixStats::protected_tokens)
        .def_readonly("hits", &RadixStats::hits).def_readonly("misses", &RadixStats::misses);
    py::class_<RadixMatch>(m, "RadixMatch")
        .def_readonly("node", &RadixMatch::node).def_readonly("tokens", &RadixMatch::tokens)
        .def_readonly("pages", &RadixMatch::pages).def_readonly("snapshot", &RadixMatch::snapshot);
    py::class_<Evicted>(m, "Evicted")
        .def_readonly("pages", &Evicted::pages).def_readonly("snapshots", &Evicted::snapshots);
    py::class_<RadixCache>(m, "RadixCache")
        .def(py::init<int>())
        .def("match", &RadixCache::match)
        .def("insert", [](RadixCache& c, const std::vector<int32_t>& t, const std::vector<int>& p, const std::vector<int>& s) {
            std::vector<int> dp, ds;
            int node = c.insert(t, p, s, &dp, &ds);
            return py::make_tuple(node, dp, ds);
        })
        .def("lock", &RadixCache::lock).def("unlock", &RadixCache::unlock).def("evict", &RadixCache::evict)
        .def("clear_snapshot", &RadixCache::clear_snapshot).def("stats", &RadixCache::stats);

    py::class_<StateMove>(m, "StateMove")
        .def_readonly("snapshot", &StateMove::snapshot).def_readonly("from_tier", &StateMove::from_tier)
        .def_readonly("from_slot", &StateMove::from_slot).def_readonly("to_tier", &StateMove::to_tier)
        .def_readonly("to_slot", &StateMove::to_slot);
    py::class_<TieredStore>(m, "TieredStore")
        .def(py::init<int, int, int>())
        .def("capture", [](TieredStore& s, int row) {
            std::vector<StateMove> mv; std::vector<int> dr;
            int id = s.capture(row, &mv, &dr);
            return py::make_tuple(id, mv, dr);
        })
        .def("promote", [](TieredStore& s, int id) {
            std::vector<StateMove> mv; std::vector<int> dr;
            int slot = s.promote(id, &mv, &dr);
            return py::make_tuple(slot, mv, dr);
        })
        .def("release", &TieredStore::release).def("touch", &TieredStore::touch)
        .def("tier_of", &TieredStore::tier_of).def("slot_of", &TieredStore::slot_of).def("census", &TieredStore::census);

    py::class_<SchedConfig>(m, "SchedConfig")
        .def(py::init<>())
        .def_readwrite("max_rows", &SchedConfig::max_rows).def_readwrite("prefill_budget", &SchedConfig::prefill_budget)
        .def_readwrite("page_size", &SchedConfig::page_size).def_readwrite("num_pages", &SchedConfig::num_pages)
        .def_readwrite("device_slots", &SchedConfig::device_slots).def_readwrite("host_slots", &SchedConfig::host_slots)
        .def_readwrite("disk_slots", &SchedConfig::disk_slots).def_readwrite("buckets", &SchedConfig::buckets)
        .def_readwrite("max_ctx", &SchedConfig::max_ctx)
        .def_readwrite("spec_rows", &SchedConfig::spec_rows)
        .def("ctx_headroom", &SchedConfig::ctx_headroom);
    py::class_<PrefillChunk>(m, "PrefillChunk")
        .def_readonly("req", &PrefillChunk::req).def_readonly("row", &PrefillChunk::row)
        .def_readonly("start", &PrefillChunk::start).def_readonly("len", &PrefillChunk::len)
        .def_readonly("last", &PrefillChunk::last).def_readonly("snapshot_after", &PrefillChunk::snapshot_after);
    py::class_<RowRestore>(m, "RowRestore")
        .def_readonly("row", &RowRestore::row).def_readonly("snapshot", &RowRestore::snapshot)
        .def_readonly("device_slot", &RowRestore::device_slot);
    py::class_<RowMove>(m, "RowMove")
        .def_readonly("from_row", &RowMove::from_row).def_readonly("to_row", &RowMove::to_row).def_readonly("req", &RowMove::req);
    py::class_<DecodeWork>(m, "DecodeWork")
        .def_readonly("rows", &DecodeWork::rows).def_readonly("n_live", &DecodeWork::n_live)
        .def_readonly("bucket", &DecodeWork::bucket);
    py::class_<TickPlan>(m, "TickPlan")
        .def_readonly("admitted", &TickPlan::admitted).def_readonly("row_moves", &TickPlan::row_moves)
        .def_readonly("restores", &TickPlan::restores).def_readonly("state_moves", &TickPlan::state_moves)
        .def_readonly("prefill", &TickPlan::prefill).def_readonly("decode", &TickPlan::decode)
        .def("empty", &TickPlan::empty);
    py::class_<Event>(m, "Event")
        .def_readonly("req", &Event::req).def_readonly("kind", &Event::kind).def_readonly("tokens", &Event::tokens)
        .def_readonly("reason", &Event::reason).def_readonly("prompt_tokens", &Event::prompt_tokens)
        .def_readonly("completion_tokens", &Event::completion_tokens)
        .def_readonly("cached_tokens", &Event::cached_tokens).def_readonly("prefix_hit", &Event::prefix_hit);
    py::class_<SchedStats>(m, "SchedStats")
        .def_readonly("ticks", &SchedStats::ticks).def_readonly("tokens_committed", &SchedStats::tokens_committed)
        .def_readonly("live_rows", &SchedStats::live_rows).def_readonly("queued", &SchedStats::queued)
        .def_readonly("pages_in_use", &SchedStats::pages_in_use).def_readonly("pages_free", &SchedStats::pages_free)
        .def_readonly("tiers", &SchedStats::tiers).def_readonly("radix", &SchedStats::radix);
    py::class_<Request>(m, "Request")
        .def_readonly("id", &Request::id).def_readonly("prompt", &Request::prompt).def_readonly("state", &Request::state)
        .def_readonly("row", &Request::row).def_readonly("prefilled", &Request::prefilled)
        .def_readonly("cached_tokens", &Request::cached_tokens).def_readonly("generated", &Request::generated)
        .def_readonly("pages", &Request::pages).def_readonly("finish_reason", &Request::finish_reason)
        .def_readonly("max_new", &Request::max_new);
    py::class_<SlotSchedConfig>(m, "SlotSchedConfig")
        .def(py::init<>())
        .def_readwrite("max_seqs", &SlotSchedConfig::max_seqs)
        .def_readwrite("prefill_rows", &SlotSchedConfig::prefill_rows)
        .def_readwrite("prefill_budget", &SlotSchedConfig::prefill_budget)
        .def_readwrite("max_ctx", &SlotSchedConfig::max_ctx)
        .def_readwrite("buckets", &SlotSchedConfig::buckets);
    py::class_<SlotEvent>(m, "SlotEvent")
        .def_readonly("req", &SlotEvent::req)
        .def_readonly("kind", &SlotEvent::kind)
        .def_readonly("token", &SlotEvent::token)
        .def_readonly("reason", &SlotEvent::reason)
        .def_readonly("prompt_tokens", &SlotEvent::prompt_tokens)
        .def_readonly("completion_tokens", &SlotEvent::completion_tokens);
    m.attr("SLOT_EV_ADMITTED") = (int)SlotEvent::ADMITTED;
    m.attr("SLOT_EV_TOKEN") = (int)SlotEvent::TOKEN;
    m.attr("SLOT_EV_FINISHED") = (int)SlotEvent::FINISHED;
    py::class_<SlotChunk>(m, "SlotChunk")
        .def_readonly("req", &SlotChunk::req)
        .def_readonly("slot", &SlotChunk::slot)
        .def_readonly("start", &SlotChunk::start)
        .def_readonly("len", &SlotChunk::len)
        .def_readonly("last", &SlotChunk::last);
    py::class_<SlotDecodePlan>(m, "SlotDecodePlan")
        .def_readonly("slots", &SlotDecodePlan::slots)
        .def_readonly("reqs", &SlotDecodePlan::reqs)
        .def_readonly("bucket", &SlotDecodePlan::bucket);
    py::class_<SlotPrefillPlan>(m, "SlotPrefillPlan")
        .def_readonly("events", &SlotPrefillPlan::events)
        .def_readonly("reset_slots", &SlotPrefillPlan::reset_slots)
        .def_readonly("chunks", &SlotPrefillPlan::chunks);
    py::class_<SlotStats>(m, "SlotStats")
        .def_readonly("ticks", &SlotStats::ticks)
        .def_readonly("tokens_committed", &SlotStats::tokens_committed)
        .def_readonly("live", &SlotStats::live)
        .def_readonly("queued", &SlotStats::queued)
        .def_readonly("free_slots", &SlotStats::free_slots);
    // the three ingest / begin calls return (events, released slots)
    py::class_<SlotScheduler>(m, "SlotScheduler")
        .def(py::init<const SlotSchedConfig&>())
        .def("buckets", &SlotScheduler::buckets)
        .def("max_prompt", &SlotScheduler::max_prompt)
        .def("submit", &SlotScheduler::submit, py::arg("prompt"), py::arg("max_new"), py::arg("stop_ids") = std::vector<int32_t>())
        .def("cancel", &SlotScheduler::cancel)
        .def("idle", &SlotScheduler::idle)
        .def("free_slots", &SlotScheduler::free_slots)
        .def("begin_tick", [](SlotScheduler& s) { std::vector<int> rel; auto ev = s.begin_tick(&rel); return py::make_tuple(ev, rel); })
        .def("plan_decode", &SlotScheduler::plan_decode)
        .def("ingest_decode", [](SlotScheduler& s, const std::vector<int32_t>& toks) {
            std::vector<int> rel; auto ev = s.ingest_decode(toks, &rel); return py::make_tuple(ev, rel); })
        .def("plan_prefill", &SlotScheduler::plan_prefill)
        .def("ingest_first", [](SlotScheduler& s, int64_t rid, int32_t tok) {
            std::vector<int> rel; auto ev = s.ingest_first(rid, tok, &rel); return py::make_tuple(ev, rel); })
        .def("stats", &SlotScheduler::stats);

    py::class_<BatchScheduler>(m, "BatchScheduler")
        .def(py::init<const SchedConfig&>())
        .def("max_prompt", &BatchScheduler::max_prompt)
        .def("submit", &BatchScheduler::submit, py::arg("prompt"), py::arg("max_new"), py::arg("stop_ids") = std::vector<int32_t>())
        .def("cancel", &BatchScheduler::cancel)
        .def("plan", &BatchScheduler::plan)
        .def("ingest_prefill", [](BatchScheduler& s, int64_t id, int len, int first_token, bool snap) {
            std::vector<StateMove> mv;
            auto ev = s.ingest_prefill(id, len, first_token, snap, &mv);
            return py::make_tuple(ev, mv);
        }, py::arg("req"), py::arg("len"), py::arg("first_token") = -1, py::arg("snapshot_captured") = false)
        .def("ingest_decode", &BatchScheduler::ingest_decode)
        .def("get", &BatchScheduler::get, py::return_value_policy::reference_internal)
        .def("reserve_pages", [](BatchScheduler& s, int n) { return s.pages().alloc(n); })
        .def("forget", &BatchScheduler::forget).def("idle", &BatchScheduler::idle).def("stats", &BatchScheduler::stats);

    m.attr("EV_ADMITTED") = (int)EV_ADMITTED; m.attr("EV_TOKENS") = (int)EV_TOKENS; m.attr("EV_FINISHED") = (int)EV_FINISHED;
    m.attr("RS_QUEUED") = (int)RS_QUEUED; m.attr("RS_PREFILL") = (int)RS_PREFILL; m.attr("RS_DECODE") = (int)RS_DECODE;
    m.attr("RS_FINISHED") = (int)RS_FINISHED;
    m.attr("TIER_DEVICE") = (int)TIER_DEVICE; m.attr("TIER_HOST") = (int)TIER_HOST; m.attr("TIER_DISK") = (int)TIER_DISK;
    m.attr("TIER_NONE") = (int)TIER_NONE;
}
