// Python bindings of the host runtime (cache manager, scheduler).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>

#include "cache_manager.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace aien;

namespace {

// offsets: {"positions", "seq_of_token", "q_start", "ctx_len"} -> int offset into `buf`;
// group_offsets[g] = (block_table_offset, slot_map_offset, max_blocks); -1 offsets are skipped.
int fill_meta_py(const CacheManager& cm, const std::vector<int64_t>& ids, const std::vector<int>& counts,
                  py::array_t<int32_t, py::array::c_style> buf, int off_positions, int off_seq, int off_qstart,
                  int off_ctx, const std::vector<std::tuple<int, int, int>>& group_offsets) {
    auto info = buf.request(true);
    int32_t* base = static_cast<int32_t*>(info.ptr);
    const long long size = info.size;
    long long T = 0;
    for (int c : counts) T += c;
    const long long S = static_cast<long long>(ids.size());
    auto need = [&](long long off, long long n) {
        if (off < 0 || off + n > size) throw std::out_of_range("fill_meta: section does not fit the buffer");
    };
    need(off_positions, T); need(off_seq, T); need(off_qstart, S + 1); need(off_ctx, S);
    CacheManager::MetaLayout lay;
    lay.positions = base + off_positions;
    lay.seq_of_token = base + off_seq;
    lay.q_start = base + off_qstart;
    lay.ctx_len = base + off_ctx;
    if (static_cast<int>(group_offsets.size()) != cm.num_groups())
        throw std::invalid_argument("fill_meta: one offset triple per group is needed");
    for (int g = 0; g < cm.num_groups(); ++g) {
        const auto [bt, sm, mb] = group_offsets[g];
        const bool state = cm.group(g).kind == GroupKind::State;
        if (!state) { need(bt, S * mb); need(sm, T); } else if (sm >= 0) need(sm, S);
        lay.block_table.push_back(state || bt < 0 ? nullptr : base + bt);
        lay.slot_map.push_back(sm < 0 ? nullptr : base + sm);
        lay.max_blocks.push_back(mb);
    }
    cm.fill_meta(ids, counts, lay);
    int max_ctx = 0;
    for (long long i = 0; i < S; ++i) max_ctx = std::max(max_ctx, static_cast<int>(lay.ctx_len[i]));
    return max_ctx;   // longest context in the step
}

std::vector<std::tuple<int, int, int>> copies_py(const std::vector<PageCopy>& c) {
    std::vector<std::tuple<int, int, int>> out;
    out.reserve(c.size());
    for (const auto& x : c) out.emplace_back(x.group, x.src, x.dst);
    return out;
}

}  // namespace

PYBIND11_MODULE(_aien_host, m) {
    m.doc() = "Host runtime of the engine: paged cache manager and continuous-batching scheduler";
    m.attr("EXHAUSTED_PREFIX") = kExhaustedPrefix;

    py::register_exception<CacheExhausted>(m, "CacheExhausted", PyExc_RuntimeError);

    py::enum_<GroupKind>(m, "GroupKind")
        .value("Full", GroupKind::Full)
        .value("Window", GroupKind::Window)
        .value("State", GroupKind::State);

    py::class_<GroupSpec>(m, "GroupSpec")
        .def(py::init([](GroupKind kind, int window, int capacity) {
                 GroupSpec s; s.kind = kind; s.window = window; s.capacity = capacity; return s;
             }), py::arg("kind"), py::arg("window") = 0, py::arg("capacity") = 0)
        .def_readwrite("kind", &GroupSpec::kind)
        .def_readwrite("window", &GroupSpec::window)
        .def_readwrite("capacity", &GroupSpec::capacity);

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init<int, std::vector<GroupSpec>, int>(), py::arg("page_size"), py::arg("groups"), py::arg("max_requests"))
        .def_property_readonly("page_size", &CacheManager::page_size)
        .def_property_readonly("num_groups", &CacheManager::num_groups)
        .def_property_readonly("max_requests", &CacheManager::max_requests)
        .def_property_readonly("num_requests", &CacheManager::num_requests)
        .def("group", &CacheManager::group)
        .def("has", &CacheManager::has)
        .def("num_tokens", &CacheManager::num_tokens)
        .def("row_of", &CacheManager::row_of)
        .def("free_count", &CacheManager::free_count)
        .def("refcount", &CacheManager::refcount)
        .def("request_ids", &CacheManager::request_ids)
        .def("add_request", &CacheManager::add_request)
        .def("pages_needed", &CacheManager::pages_needed)
        .def("can_append", [](const CacheManager& cm, const std::vector<std::pair<int64_t, int>>& b) { return cm.can_append(b); })
        .def("append", [](CacheManager& cm, const std::vector<std::pair<int64_t, int>>& b) { return copies_py(cm.append(b)); })
        .def("fork", [](CacheManager& cm, int64_t p, int64_t c, int at) { return copies_py(cm.fork(p, c, at)); },
             py::arg("parent"), py::arg("child"), py::arg("at_token") = -1)
        .def("truncate", &CacheManager::truncate)
        .def("free_request", &CacheManager::free_request)
        .def("slot_of", &CacheManager::slot_of)
        .def("state_slot", &CacheManager::state_slot)
        .def("table", &CacheManager::table)
        .def("fill_meta", &fill_meta_py)
        .def("check", &CacheManager::check)
        .def("metrics", [](const CacheManager& cm) {
            const CacheMetrics& x = cm.metrics();
            py::dict d;
            d["cow_copies"] = x.cow_copies;
            d["pages_allocated"] = x.pages_allocated;
            d["pages_released"] = x.pages_released;
            d["window_releases"] = x.window_releases;
            return d;
        });

    bind_scheduler(m);
}
