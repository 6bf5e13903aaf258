// Python bindings of the host runtime (no CUDA dependency): tokenizer, token-shard loader, safetensors I/O, CPU AdamW,
// expert-parallel LPT planner, crash handler, NVML telemetry.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "bpe_tokenizer.h"
#include "host_api.h"
#include "safetensors_io.h"
#include "token_loader.h"

namespace py = pybind11;
using namespace sg;

static void* ptr(uintptr_t p) { return reinterpret_cast<void*>(p); }

// AsyncAdamW plus the Python objects whose memory its job in flight touches.  The worker needs no GIL, so the destructor can wait
// for it while holding the GIL; only then are the references dropped.
struct OwnedAsyncAdamW {
    AsyncAdamW w;
    py::object keep = py::none();
    explicit OwnedAsyncAdamW(bool overlap) : w(overlap) {}
    ~OwnedAsyncAdamW() {
        try {
            py::gil_scoped_release rel;
            w.drain();
        } catch (...) {   // a failed update is reported by submit() / drain(); a destructor has nobody to tell
        }
    }
};

PYBIND11_MODULE(sg_b200_host, m) {
    m.doc() = "surogate_b200 native host runtime";

    py::class_<BpeTokenizer, std::shared_ptr<BpeTokenizer>>(m, "BpeTokenizer")
        .def_static("from_file", &BpeTokenizer::from_file)
        .def_static("from_json", &BpeTokenizer::from_json)
        .def("encode", [](const BpeTokenizer& t, const std::string& s, bool added) {
                 py::gil_scoped_release rel;
                 return t.encode(s, added);
             }, py::arg("text"), py::arg("allow_added_tokens") = true)
        .def("encode_batch", [](const BpeTokenizer& t, const std::vector<std::string>& v, bool added, int threads) {
                 py::gil_scoped_release rel;
                 return t.encode_batch(v, added, threads);
             }, py::arg("texts"), py::arg("allow_added_tokens") = true, py::arg("threads") = 0)
        .def("decode", [](const BpeTokenizer& t, const std::vector<int32_t>& ids, bool skip) { return py::bytes(t.decode(ids, skip)); },
             py::arg("ids"), py::arg("skip_special") = false)
        .def("pre_tokenize", [](const BpeTokenizer& t, const std::string& s) {
                 std::vector<py::bytes> out;
                 for (auto& w : t.pre_tokenize(s)) out.emplace_back(w);
                 return out;
             })
        .def("vocab_size", &BpeTokenizer::vocab_size)
        .def("token_to_id", [](const BpeTokenizer& t, const py::bytes& b) { return t.token_to_id(std::string(b)); })
        .def("id_to_token", [](const BpeTokenizer& t, int32_t id) { return py::bytes(t.id_to_token(id)); })
        .def("is_special", &BpeTokenizer::is_special)
        .def("added_tokens", &BpeTokenizer::added_tokens)
        .def("style", [](const BpeTokenizer& t) {
            auto s = t.style();
            return py::dict(py::arg("legacy_gpt2") = s.legacy_gpt2, py::arg("contractions_ignore_case") = s.contractions_ignore_case,
                            py::arg("max_digits") = s.max_digits);
        });
    m.def("unicode_class", [](uint32_t cp) { return unicode_is_letter(cp) ? "L" : unicode_is_number(cp) ? "N" : unicode_is_space(cp) ? "S" : "O"; });

    py::class_<TokenLoader>(m, "TokenLoader")
        .def(py::init<const std::vector<std::string>&, int, int, int64_t, int, int, bool, int>(), py::arg("files"), py::arg("batch"), py::arg("seq_len"),
             py::arg("seed") = 0, py::arg("rank") = 0, py::arg("world") = 1, py::arg("shuffle") = true, py::arg("prefetch") = 2)
        .def("next_into", [](TokenLoader& l, uintptr_t x, uintptr_t y, uintptr_t p) {
                 py::gil_scoped_release rel;
                 l.next(static_cast<int32_t*>(ptr(x)), static_cast<int32_t*>(ptr(y)), static_cast<int32_t*>(ptr(p)));
             })
        .def("state", [](const TokenLoader& l) {
                 auto s = l.state();
                 return py::dict(py::arg("seed") = s.seed, py::arg("epoch") = s.epoch, py::arg("file_index") = s.file_index, py::arg("chunk_index") = s.chunk_index);
             })
        .def("set_state", [](TokenLoader& l, int64_t seed, int64_t epoch, int64_t fi, int64_t ci) { l.set_state(LoaderState{seed, epoch, fi, ci}); })
        .def("steps_per_epoch", &TokenLoader::steps_per_epoch)
        .def("total_chunks", &TokenLoader::total_chunks)
        .def("vocab", &TokenLoader::vocab);
    m.def("shuffled_order", &shuffled_order);

    py::class_<SafetensorsFile>(m, "SafetensorsFile")
        .def(py::init<const std::string&>())
        .def("entries", [](const SafetensorsFile& f) {
                 py::dict d;
                 for (auto& e : f.entries()) d[py::str(e.name)] = py::make_tuple(e.dtype, e.shape, e.begin, e.end);
                 return d;
             })
        .def("metadata", &SafetensorsFile::metadata)
        .def("data_start", &SafetensorsFile::data_start)
        .def("read_into", [](const SafetensorsFile& f, const std::string& name, uintptr_t dst, uint64_t nbytes, uint64_t off, int threads) {
                 py::gil_scoped_release rel;
                 f.read_into(name, ptr(dst), nbytes, off, threads);
             }, py::arg("name"), py::arg("dst"), py::arg("nbytes"), py::arg("offset") = 0, py::arg("threads") = 8)
        .def("read_rows", [](const SafetensorsFile& f, const std::string& name, uintptr_t dst, int64_t r0, int64_t r1, int threads) {
                 py::gil_scoped_release rel;
                 f.read_rows(name, ptr(dst), r0, r1, threads);
             }, py::arg("name"), py::arg("dst"), py::arg("row_begin"), py::arg("row_end"), py::arg("threads") = 8);
    m.def("write_safetensors", [](const std::string& path, const std::vector<std::tuple<std::string, std::string, std::vector<int64_t>, uintptr_t, uint64_t>>& items,
                                  const std::map<std::string, std::string>& meta, int threads) {
              std::vector<StWriteItem> v;
              for (auto& it : items) v.push_back({std::get<0>(it), std::get<1>(it), std::get<2>(it), ptr(std::get<3>(it)), std::get<4>(it)});
              py::gil_scoped_release rel;
              return write_safetensors(path, v, meta, threads);
          }, py::arg("path"), py::arg("items"), py::arg("metadata") = std::map<std::string, std::string>{}, py::arg("threads") = 8);
    m.def("dtype_size", &dtype_size);

    m.def("cpu_adamw_step", [](uintptr_t param, uintptr_t mm, uintptr_t vv, uintptr_t grad, bool grad_bf16, uintptr_t work, int64_t n, float lr, float b1,
                               float b2, float eps, float wd, float grad_scale, int64_t step, uintptr_t mask) {
              py::gil_scoped_release rel;
              cpu_adamw_step(static_cast<float*>(ptr(param)), static_cast<float*>(ptr(mm)), static_cast<float*>(ptr(vv)), ptr(grad), grad_bf16,
                             static_cast<uint16_t*>(ptr(work)), n, lr, b1, b2, eps, wd, grad_scale, step, static_cast<const uint8_t*>(ptr(mask)));
          }, py::arg("param"), py::arg("m"), py::arg("v"), py::arg("grad"), py::arg("grad_is_bf16"), py::arg("work_bf16"), py::arg("n"), py::arg("lr"),
          py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"), py::arg("grad_scale"), py::arg("step"), py::arg("decay_mask") = 0);
    py::class_<OwnedAsyncAdamW>(m, "AsyncAdamW")
        .def(py::init<bool>(), py::arg("overlap") = true)
        .def("submit", [](OwnedAsyncAdamW& o, const std::vector<std::tuple<uintptr_t, uintptr_t, uintptr_t, uintptr_t, bool, uintptr_t, bool, int64_t, uintptr_t>>& jobs,
                          float lr, float b1, float b2, float eps, float wd, float grad_scale, int64_t step, py::object keepalive) {
                 // job = (param, m, v, grad, grad_is_bf16, work, work_is_bf16, n, decay_mask).  ``keepalive`` (any Python object, normally the
                 // list of tensors behind the addresses) is owned by the worker until this update has completed, so dropping the
                 // optimizer or the trainer with an update in flight cannot free memory the worker thread still writes.
                 std::vector<AdamJob> v;
                 for (auto& j : jobs) {
                     void* work = ptr(std::get<5>(j));
                     const bool wb = std::get<6>(j);
                     v.push_back({static_cast<float*>(ptr(std::get<0>(j))), static_cast<float*>(ptr(std::get<1>(j))), static_cast<float*>(ptr(std::get<2>(j))),
                                  ptr(std::get<3>(j)), std::get<4>(j), wb ? static_cast<uint16_t*>(work) : nullptr, wb ? nullptr : static_cast<float*>(work),
                                  std::get<7>(j), static_cast<const uint8_t*>(ptr(std::get<8>(j)))});
                 }
                 {
                     py::gil_scoped_release rel;
                     o.w.drain();   // the previous update is complete: its buffers may go
                 }
                 o.keep = std::move(keepalive);
                 py::gil_scoped_release rel;
                 o.w.submit(std::move(v), AdamHyper{lr, b1, b2, eps, wd, grad_scale, step});
             }, py::arg("jobs"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"), py::arg("grad_scale"), py::arg("step"),
             py::arg("keepalive") = py::none())
        .def("drain", [](OwnedAsyncAdamW& o) {
            {
                py::gil_scoped_release rel;
                o.w.drain();
            }
            o.keep = py::none();
        })
        .def("completed", [](const OwnedAsyncAdamW& o) { return o.w.completed(); })
        .def_property_readonly("holds_buffers", [](const OwnedAsyncAdamW& o) { return !o.keep.is_none(); })
        .def_property_readonly("overlap", [](const OwnedAsyncAdamW& o) { return o.w.overlap(); });
    py::class_<MemoryStack>(m, "MemoryStack")
        .def(py::init<uint64_t, uint64_t, uint64_t>(), py::arg("base"), py::arg("capacity"), py::arg("align") = 4096)
        .def("allocate", &MemoryStack::allocate, py::arg("bytes"), py::arg("name") = "")
        .def("checkpoint", &MemoryStack::checkpoint)
        .def("restore", &MemoryStack::restore)
        .def("free_last", &MemoryStack::free_last)
        .def("live", &MemoryStack::live)
        .def("peak_by_name", &MemoryStack::peak_by_name)
        .def_property_readonly("used", &MemoryStack::used)
        .def_property_readonly("capacity", &MemoryStack::capacity)
        .def_property_readonly("high_water", &MemoryStack::high_water)
        .def_property_readonly("allocations", &MemoryStack::allocations);
    py::class_<AllocationRegistry>(m, "AllocationRegistry")
        .def(py::init<>())
        .def("record", &AllocationRegistry::record, py::arg("name"), py::arg("category"), py::arg("kind"), py::arg("bytes"))
        .def("release", &AllocationRegistry::release)
        .def("by_category", &AllocationRegistry::by_category, py::arg("kind") = "")
        .def("by_kind", &AllocationRegistry::by_kind, py::arg("peak") = false)
        .def("largest", &AllocationRegistry::largest, py::arg("n") = 10)
        .def("__len__", &AllocationRegistry::size);
    m.def("cpu_sum_squares", [](uintptr_t x, bool bf16, int64_t n) {
        py::gil_scoped_release rel;
        return cpu_sum_squares(ptr(x), bf16, n);
    });

    m.def("imbalance_ratio", [](const std::vector<int64_t>& counts, int ep) { return imbalance_ratio(counts.data(), static_cast<int>(counts.size()), ep); });
    m.def("compute_lpt_plan", [](const std::vector<int64_t>& counts, int ep, float threshold, float cap, int min_chunk) {
              LptPlan p = compute_lpt_plan(counts.data(), static_cast<int>(counts.size()), ep, threshold, cap, min_chunk);
              py::list assign;
              for (auto& chunks : p.assignments) {
                  py::list l;
                  for (auto& c : chunks) l.append(py::make_tuple(c.gpu, c.token_start, c.token_end));
                  assign.append(l);
              }
              py::list moves;
              for (auto& mv : p.moves) moves.append(py::make_tuple(mv.expert, mv.src_rank, mv.dst_rank));
              return py::dict(py::arg("assignments") = assign, py::arg("moves") = moves, py::arg("gpu_loads") = p.gpu_loads,
                              py::arg("expert_to_gpu") = p.expert_to_gpu, py::arg("uses_lpt") = p.uses_lpt, py::arg("imbalance") = p.imbalance);
          }, py::arg("counts"), py::arg("ep_size"), py::arg("threshold") = 1.3f, py::arg("capacity_factor") = 1.1f, py::arg("min_tokens_per_gemm") = 1024);

    m.def("balanced_placement", [](const std::vector<int64_t>& counts, int ep, const std::vector<int>& current, float tol) {
              int moved = 0;
              auto p = balanced_placement(counts.data(), static_cast<int>(counts.size()), ep, current.data(), tol, &moved);
              return py::make_tuple(p, moved);
          }, py::arg("counts"), py::arg("ep_size"), py::arg("current"), py::arg("tolerance") = 0.05f);

    m.def("plan_buffer_offsets", [](const std::vector<int64_t>& nbytes, const std::vector<int64_t>& first, const std::vector<int64_t>& last) {
        if (first.size() != nbytes.size() || last.size() != nbytes.size()) throw std::invalid_argument("plan_buffer_offsets: the three lists must have one entry per tensor");
        BufferPlanResult r = plan_buffer_offsets(nbytes, first, last);
        return py::make_tuple(r.offsets, r.total);
    });
    m.def("validate_buffer_plan", [](const std::vector<int64_t>& nbytes, const std::vector<int64_t>& first, const std::vector<int64_t>& last,
                                      const std::vector<int64_t>& offsets, int64_t total) {
        if (first.size() != nbytes.size() || last.size() != nbytes.size() || offsets.size() != nbytes.size())
            throw std::invalid_argument("validate_buffer_plan: the lists must have one entry per tensor");
        return validate_buffer_plan(nbytes, first, last, offsets, total);
    });
    m.def("install_crash_handler", &install_crash_handler, py::arg("tag") = "surogate_b200");
    m.def("query_gpu", [](int index) {
        GpuTelemetry t = query_gpu(index);
        py::dict d;
        d["ok"] = t.ok;
        d["error"] = t.error;
        d["name"] = t.name;
        d["sm_clock_mhz"] = t.sm_clock_mhz;
        d["sm_clock_max_mhz"] = t.sm_clock_max_mhz;
        d["mem_clock_mhz"] = t.mem_clock_mhz;
        d["power_w"] = t.power_mw / 1000.0;
        d["power_limit_w"] = t.power_limit_mw / 1000.0;
        d["temperature_c"] = t.temperature_c;
        d["gpu_util"] = t.gpu_util;
        d["mem_util"] = t.mem_util;
        d["mem_used"] = t.mem_used;
        d["mem_total"] = t.mem_total;
        d["throttle_reasons"] = t.throttle_reasons;
        d["pcie_rx_kbs"] = t.pcie_rx_kbs;
        d["pcie_tx_kbs"] = t.pcie_tx_kbs;
        return d;
    });
}
