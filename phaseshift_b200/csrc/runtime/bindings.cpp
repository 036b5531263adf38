// pybind11 module `ps_runtime`: the host runtime exposed to Python.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "ps_io.h"
#include "ps_runtime.h"
#include "ps_sampling.h"

namespace py = pybind11;
using namespace psrt;

static py::dict plan_to_dict(const StepPlan& p) {
    py::list seqs;
    for (const auto& s : p.seqs)
        seqs.append(py::make_tuple(s.request_id, s.slot, s.pos_start, s.token_offset, s.n_tokens, s.sample, s.is_decode,
                                   s.sample_index));
    py::list ups;
    for (const auto& u : p.block_updates) ups.append(py::make_tuple(u.slot, u.block, u.page));
    py::dict d;
    d["seqs"] = seqs; d["tokens"] = p.tokens; d["block_updates"] = ups; d["n_sampled"] = p.n_sampled;
    return d;
}

PYBIND11_MODULE(ps_runtime, m) {
    m.doc() = "phaseshift_b200 host runtime (C++)";
    py::register_exception<Error>(m, "RuntimeCoreError");

    m.def("checked_add", &checked_add); m.def("checked_mul", &checked_mul); m.def("align_up", &align_up);
    m.def("pages_for", &pages_for); m.def("additional_pages", &additional_pages);
    m.def("crc32", [](py::bytes b, uint32_t seed) { std::string s = b; return crc32((const uint8_t*)s.data(), s.size(), seed); },
          py::arg("data"), py::arg("seed") = 0);
    m.def("crc32_ptr", [](uintptr_t p, size_t n, uint32_t seed) { return crc32((const uint8_t*)p, n, seed); });

    py::class_<Handle>(m, "Handle").def_readonly("slot", &Handle::slot).def_readonly("generation", &Handle::generation);
    py::class_<SlotPool>(m, "SlotPool").def(py::init<uint32_t>()).def("acquire", &SlotPool::acquire)
        .def("release", &SlotPool::release).def("valid", &SlotPool::valid).def("free_count", &SlotPool::free_count);
    py::class_<PagePool>(m, "PagePool").def(py::init<uint32_t>()).def("acquire", &PagePool::acquire)
        .def("release", &PagePool::release).def("free_count", &PagePool::free_count).def("capacity", &PagePool::capacity);

    py::class_<BankerProcess>(m, "BankerProcess").def(py::init<>())
        .def_readwrite("allocated", &BankerProcess::allocated).def_readwrite("max_claim", &BankerProcess::max_claim);
    py::class_<KvBanker>(m, "KvBanker").def(py::init<>()).def_readwrite("available", &KvBanker::available)
        .def("add", [](KvBanker& b, uint32_t alloc, uint32_t claim) { b.processes.push_back({alloc, claim}); })
        .def("process", [](const KvBanker& b, size_t i) { return py::make_tuple(b.processes.at(i).allocated, b.processes.at(i).max_claim); })
        .def("num_processes", [](const KvBanker& b) { return b.processes.size(); })
        .def("grant", [](KvBanker& b, size_t i, uint32_t g) { b.available -= g; b.processes.at(i).allocated += g; })
        .def("is_safe", &KvBanker::is_safe).def("can_admit", &KvBanker::can_admit).def("max_safe_grant", &KvBanker::max_safe_grant);

    py::class_<Sampling>(m, "Sampling").def(py::init<>())
        .def(py::init([](float t, float p, uint32_t k, uint64_t seed) { Sampling s; s.temperature = t; s.top_p = p; s.top_k = k; s.seed = seed; return s; }),
             py::arg("temperature") = 0.f, py::arg("top_p") = 1.f, py::arg("top_k") = 0, py::arg("seed") = 0)
        .def_readwrite("temperature", &Sampling::temperature).def_readwrite("top_p", &Sampling::top_p)
        .def_readwrite("top_k", &Sampling::top_k).def_readwrite("seed", &Sampling::seed);

    py::class_<BatcherConfig>(m, "BatcherConfig").def(py::init<>())
        .def_readwrite("max_slots", &BatcherConfig::max_slots).def_readwrite("num_pages", &BatcherConfig::num_pages)
        .def_readwrite("page_tokens", &BatcherConfig::page_tokens).def_readwrite("max_seq_len", &BatcherConfig::max_seq_len)
        .def_readwrite("max_step_tokens", &BatcherConfig::max_step_tokens)
        .def_readwrite("max_step_requests", &BatcherConfig::max_step_requests)
        .def_readwrite("full_claim", &BatcherConfig::full_claim);

    py::class_<StepPlan>(m, "StepPlan").def("empty", &StepPlan::empty).def("to_dict", &plan_to_dict)
        .def_readonly("n_sampled", &StepPlan::n_sampled)
        .def("num_tokens", [](const StepPlan& p) { return p.tokens.size(); })
        .def("num_seqs", [](const StepPlan& p) { return p.seqs.size(); });

    py::class_<Batcher>(m, "Batcher").def(py::init<const BatcherConfig&>())
        .def("submit", &Batcher::submit, py::arg("prompt"), py::arg("max_new_tokens"), py::arg("sampling") = Sampling(),
             py::arg("stop_tokens") = std::vector<int32_t>(), py::arg("checkpoint_position") = 0)
        .def("cancel", &Batcher::cancel).def("cancel_all", &Batcher::cancel_all).def("admit", &Batcher::admit)
        .def("restore_prefix", [](Batcher& b, uint64_t id, uint32_t n) {
            std::vector<BlockUpdate> ups; b.restore_prefix(id, n, ups);
            py::list l; for (auto& u : ups) l.append(py::make_tuple(u.slot, u.block, u.page)); return l; })
        .def("plan", &Batcher::plan)
        .def("commit", [](Batcher& b, const StepPlan& p, const std::vector<int32_t>& sampled) {
            py::list l; for (auto& e : b.commit(p, sampled)) l.append(py::make_tuple(e.kind, e.request_id, e.token)); return l; })
        .def("fail", [](Batcher& b, const StepPlan& p, const std::string& why) {
            py::list l; for (auto& e : b.fail(p, why)) l.append(py::make_tuple(e.kind, e.request_id, e.token)); return l; })
        .def("request", [](const Batcher& b, uint64_t id) -> py::object {
            const Request* r = b.find(id);
            if (!r) return py::none();
            py::dict d;
            d["id"] = r->id; d["state"] = (int)r->state; d["finish_reason"] = finish_name(r->finish);
            d["generated"] = r->generated; d["prompt_tokens"] = r->prompt.size(); d["position"] = r->seq.position;
            d["slot"] = r->seq.handle.slot; d["generation"] = r->seq.handle.generation; d["pages"] = r->seq.pages;
            d["restored_tokens"] = r->restored_tokens; d["prefill_tokens"] = r->prefill_tokens;
            d["checkpoint_position"] = r->checkpoint_position; d["checkpoint_saved"] = r->checkpoint_saved;
            d["error"] = r->error; d["prompt"] = r->prompt; d["poisoned"] = r->seq.poisoned;
            d["temperature"] = r->sampling.temperature; d["top_p"] = r->sampling.top_p; d["top_k"] = r->sampling.top_k;
            d["seed"] = r->sampling.seed; d["max_new_tokens"] = r->max_new_tokens;
            return d; })
        .def("retire", &Batcher::retire).def("active_count", &Batcher::active_count).def("queued_count", &Batcher::queued_count)
        .def("free_pages", &Batcher::free_pages).def("idle", &Batcher::idle)
        .def("take_release_updates", [](Batcher& b) {
            py::list l; for (auto& u : b.take_release_updates()) l.append(py::make_tuple(u.slot, u.block, u.page)); return l; })
        .def("banker_snapshot", &Batcher::banker_snapshot);

    py::class_<PrefixHit>(m, "PrefixHit").def_readonly("entry", &PrefixHit::entry).def_readonly("tokens", &PrefixHit::tokens);
    py::class_<PrefixIndex>(m, "PrefixIndex").def(py::init<uint32_t, uint32_t, uint32_t>(), py::arg("max_entries"),
                                                  py::arg("capacity_tokens"), py::arg("min_tokens") = 64)
        .def("lookup", &PrefixIndex::lookup)
        .def("insert", [](PrefixIndex& p, const std::vector<int32_t>& t) { std::vector<int64_t> ev; int64_t id = p.insert(t, ev); return py::make_tuple(id, ev); })
        .def("erase", &PrefixIndex::erase).def("used_tokens", &PrefixIndex::used_tokens).def("entries", &PrefixIndex::entries)
        .def_readonly("hits", &PrefixIndex::hits).def_readonly("misses", &PrefixIndex::misses)
        .def_readonly("inserts", &PrefixIndex::inserts).def_readonly("evictions", &PrefixIndex::evictions)
        .def_readonly("skipped", &PrefixIndex::skipped);

    m.def("spec_greedy_accept", [](const std::vector<int32_t>& d, const std::vector<int32_t>& t) {
        auto r = spec_greedy_accept(d, t); return py::make_tuple(r.accepted, r.next_token, r.full); });
    py::class_<SpecTransaction>(m, "SpecTransaction").def(py::init<>()).def("begin", &SpecTransaction::begin)
        .def("verified", &SpecTransaction::verified).def("commit", &SpecTransaction::commit)
        .def("rollback", &SpecTransaction::rollback).def("reset", &SpecTransaction::reset)
        .def_property_readonly("state", [](const SpecTransaction& s) { return (int)s.state; })
        .def_readonly("accepted", &SpecTransaction::accepted).def_readonly("rows", &SpecTransaction::rows);
    m.def("ngram_tail", &ngram_tail);

    // ---- IO
    py::class_<SafetensorsReader>(m, "SafetensorsReader").def(py::init<const std::string&>())
        .def("names", &SafetensorsReader::names).def("has", &SafetensorsReader::has)
        .def("spec", [](const SafetensorsReader& r, const std::string& n) { const auto& s = r.spec(n); return py::make_tuple(s.dtype, s.shape, s.end - s.begin); })
        .def("metadata", &SafetensorsReader::metadata)
        .def("data", [](py::object self, const std::string& n) {
            auto& r = self.cast<SafetensorsReader&>();
            const auto& s = r.spec(n);
            // zero-copy uint8 view into the mapping; the array's base is the reader, so the mapping outlives
            // every tensor derived from it (do not call close() while such tensors are alive)
            return py::array_t<uint8_t>({(py::ssize_t)(s.end - s.begin)}, {(py::ssize_t)1}, r.data(n), self); })
        .def("crc32", [](const SafetensorsReader& r, const std::string& n) { const auto& s = r.spec(n); return crc32(r.data(n), s.end - s.begin); })
        .def("close", &SafetensorsReader::close);
    py::class_<SafetensorsWriter>(m, "SafetensorsWriter").def(py::init<const std::string&>())
        .def("set_metadata", &SafetensorsWriter::set_metadata).def("plan_tensor", &SafetensorsWriter::plan_tensor)
        .def("write_header", &SafetensorsWriter::write_header)
        .def("write_chunk", [](SafetensorsWriter& w, const std::string& n, py::buffer b) {
            py::buffer_info info = b.request(); w.write_chunk(n, (const uint8_t*)info.ptr, (size_t)(info.size * info.itemsize)); })
        .def("write_chunk_ptr", [](SafetensorsWriter& w, const std::string& n, uintptr_t p, size_t nbytes) { w.write_chunk(n, (const uint8_t*)p, nbytes); })
        .def("tensor_crc", &SafetensorsWriter::tensor_crc).def("finish", &SafetensorsWriter::finish);

    // ---- codecs / CPU reference quantisers
    m.def("e4m3_decode", &e4m3_decode); m.def("e4m3_encode", &e4m3_encode);
    m.def("e2m1_decode", &e2m1_decode); m.def("e2m1_encode", &e2m1_encode); m.def("ue8m0_decode", &ue8m0_decode);
    m.def("quantize_rows_nvfp4", [](uintptr_t w, int n, int k, int k_padded, float tensor_scale, int search, uintptr_t importance,
                                    uintptr_t codes, uintptr_t scales) {
        py::gil_scoped_release rel;
        for (int r = 0; r < n; ++r)
            quantize_row_nvfp4((const float*)w + (size_t)r * k, k, k_padded, tensor_scale, search, (const float*)importance,
                               (uint8_t*)codes + (size_t)r * (k_padded / 2), (uint8_t*)scales + (size_t)r * (k_padded / 16));
    });
    m.def("quantize_rows_mxfp8", [](uintptr_t w, int n, int k, int k_padded, int search, uintptr_t importance, uintptr_t codes,
                                    uintptr_t scales) {
        py::gil_scoped_release rel;
        for (int r = 0; r < n; ++r)
            quantize_row_mxfp8((const float*)w + (size_t)r * k, k, k_padded, search, (const float*)importance,
                               (uint8_t*)codes + (size_t)r * k_padded, (uint8_t*)scales + (size_t)r * (k_padded / 32));
    });

    m.def("kv_nvfp4_row_bytes", &kv_nvfp4_row_bytes);
    m.def("kv_nvfp4_encode_rows", [](uintptr_t x, int n, int d, uintptr_t rows, uintptr_t scales) {
        py::gil_scoped_release rel;
        const int rb = kv_nvfp4_row_bytes(d);
        for (int r = 0; r < n; ++r)
            kv_nvfp4_encode_row((const float*)x + (size_t)r * d, d, (uint8_t*)rows + (size_t)r * rb, (float*)scales + r);
    });
    m.def("kv_nvfp4_decode_rows", [](uintptr_t rows, uintptr_t scales, int n, int d, uintptr_t out) {
        py::gil_scoped_release rel;
        const int rb = kv_nvfp4_row_bytes(d);
        for (int r = 0; r < n; ++r)
            kv_nvfp4_decode_row((const uint8_t*)rows + (size_t)r * rb, ((const float*)scales)[r], d, (float*)out + (size_t)r * d);
    });

    // ---- sampling contract (host side of ps_sampling.h)
    m.def("sampling_bits", [](uint64_t seed, uint64_t idx, uint64_t attempt, uint64_t tok) { return ps::sampling_bits(seed, idx, attempt, tok); });
    m.def("sampling_uniform", [](uint64_t seed, uint64_t idx, uint64_t attempt, uint64_t tok) { return ps::sampling_uniform(seed, idx, attempt, tok); });
}
