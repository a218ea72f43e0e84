// pybind11 bindings of the C++ host runtime.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "devmem.h"
#include "kv_pool.h"
#include "memguard.h"
#include "oplog.h"
#include "pcache.h"
#include "safetensors.h"
#include "scheduler.h"
#include "sha256.h"

namespace py = pybind11;
using namespace spark_rt;

PYBIND11_MODULE(_runtime, m) {
  m.doc() = "spark_engine_b200 C++ host runtime: KV pool, prefix cache, scheduler core, op log, loaders";

  py::class_<Lease>(m, "Lease").def_readonly("id", &Lease::id).def_readonly("base", &Lease::base)
      .def_readonly("cap", &Lease::cap).def_readonly("used", &Lease::used).def_readonly("pinned", &Lease::pinned);
  py::class_<ArrayLayout>(m, "ArrayLayout").def(py::init<>()).def_readwrite("name", &ArrayLayout::name)
      .def_readwrite("div", &ArrayLayout::div).def_readwrite("width", &ArrayLayout::width).def_readwrite("kind", &ArrayLayout::kind);
  py::class_<KvPool>(m, "KvPool").def(py::init<int64_t, int64_t>())
      .def("acquire", &KvPool::acquire).def("grow", &KvPool::grow).def("shrink", &KvPool::shrink)
      .def("release", &KvPool::release).def("touch", &KvPool::touch).def("pin", &KvPool::pin)
      .def("set_used", &KvPool::set_used).def("get", &KvPool::get, py::return_value_policy::copy)
      .def("lru_victim", &KvPool::lru_victim).def("free_tokens", &KvPool::free_tokens)
      .def("largest_free_run", &KvPool::largest_free_run).def("allocated_tokens", &KvPool::allocated_tokens)
      .def("active_tokens", &KvPool::active_tokens).def("total", &KvPool::total).def("granule", &KvPool::granule)
      .def("bytes_per_token", &KvPool::bytes_per_token);

  py::class_<PcacheEntry>(m, "PcacheEntry").def_readonly("key", &PcacheEntry::key).def_readonly("tokens", &PcacheEntry::tokens)
      .def_readonly("bytes", &PcacheEntry::bytes);
  py::class_<Pcache>(m, "Pcache").def(py::init<const std::string&, const std::string&, int64_t, bool>(), py::arg("root"), py::arg("identity"), py::arg("byte_budget"), py::arg("direct_io") = true)
      .def_static("identity_dir", &Pcache::identity_dir)
      .def_static("prefix_key", [](const std::vector<int32_t>& ids) { return Pcache::prefix_key(ids.data(), ids.size()); })
      .def("save", [](Pcache& p, const std::string& key, int64_t tokens, py::buffer b) {
        py::buffer_info i = b.request();
        py::gil_scoped_release rel;
        return p.save(key, tokens, i.ptr, i.size * i.itemsize); })
      .def("save_ptr", [](Pcache& p, const std::string& key, int64_t tokens, uintptr_t ptr, int64_t bytes) {
        py::gil_scoped_release rel;
        return p.save(key, tokens, reinterpret_cast<const void*>(ptr), bytes); })
      .def("save_async_ptr", [](Pcache& p, const std::string& key, int64_t tokens, uintptr_t ptr, int64_t bytes) {
        p.save_async(key, tokens, reinterpret_cast<const void*>(ptr), bytes, nullptr); })
      .def("load_ptr", [](Pcache& p, const std::string& key, uintptr_t ptr, int64_t cap) {
        py::gil_scoped_release rel;
        return p.load(key, reinterpret_cast<void*>(ptr), cap); })
      .def("load", [](Pcache& p, const std::string& key, py::buffer b) {
        py::buffer_info i = b.request(true);
        py::gil_scoped_release rel;
        return p.load(key, i.ptr, i.size * i.itemsize); })
      .def("drain", &Pcache::drain, py::call_guard<py::gil_scoped_release>())
      .def("longest_prefix", [](Pcache& p, const std::vector<int32_t>& ids, int64_t granule) {
        std::string k; int64_t t = p.longest_prefix(ids.data(), ids.size(), granule, &k); return py::make_tuple(t, k); })
      .def("contains", &Pcache::contains).def("remove", &Pcache::remove).def("entries", &Pcache::entries)
      .def("keep_only", &Pcache::keep_only).def("bytes_used", &Pcache::bytes_used).def("reconcile", &Pcache::reconcile)
      .def("dir", &Pcache::dir)
      .def("stats", [](Pcache& p) { auto s = p.stats(); return py::dict(py::arg("saves") = s.saves, py::arg("loads") = s.loads, py::arg("hits") = s.hits, py::arg("misses") = s.misses, py::arg("evictions") = s.evictions, py::arg("corrupt") = s.corrupt); });

  py::class_<Request>(m, "Request").def(py::init<>()).def_readwrite("id", &Request::id).def_readwrite("prompt", &Request::prompt)
      .def_readwrite("max_new", &Request::max_new).def_readwrite("stop", &Request::stop).def_readwrite("temperature", &Request::temperature)
      .def_readwrite("seed", &Request::seed).def_readwrite("t_arrive", &Request::t_arrive);
  py::enum_<ReuseKind>(m, "ReuseKind").value("Cold", ReuseKind::Cold).value("ContinueStore", ReuseKind::ContinueStore)
      .value("Checkpoint", ReuseKind::Checkpoint).value("CloneStore", ReuseKind::CloneStore).value("Library", ReuseKind::Library)
      .value("Disk", ReuseKind::Disk);
  py::class_<AdmitPlan>(m, "AdmitPlan").def_readonly("request_id", &AdmitPlan::request_id).def_readonly("slot", &AdmitPlan::slot)
      .def_readonly("kind", &AdmitPlan::kind).def_readonly("source", &AdmitPlan::source).def_readonly("reuse_tokens", &AdmitPlan::reuse_tokens)
      .def_readonly("evict_slot", &AdmitPlan::evict_slot);
  py::class_<SlotState>(m, "SlotState").def_readonly("busy", &SlotState::busy).def_readonly("request_id", &SlotState::request_id)
      .def_readonly("tokens", &SlotState::tokens).def_readonly("prefilled", &SlotState::prefilled).def_readonly("prompt_len", &SlotState::prompt_len)
      .def_readonly("generated", &SlotState::generated).def_readonly("max_new", &SlotState::max_new).def_readonly("cancelled", &SlotState::cancelled);
  py::class_<PrefillPart>(m, "PrefillPart").def_readonly("slot", &PrefillPart::slot).def_readonly("begin", &PrefillPart::begin)
      .def_readonly("end", &PrefillPart::end);
  py::class_<Step> step(m, "Step");
  py::enum_<Step::Kind>(step, "Kind").value("Idle", Step::Idle).value("Admit", Step::Admit).value("Prefill", Step::Prefill)
      .value("Decode", Step::Decode).value("Cancel", Step::Cancel);
  step.def_readonly("kind", &Step::kind).def_readonly("admit", &Step::admit).def_readonly("slot", &Step::slot)
      .def_readonly("chunk_begin", &Step::chunk_begin).def_readonly("chunk_end", &Step::chunk_end).def_readonly("decode_slots", &Step::decode_slots)
      .def_readonly("parts", &Step::parts);
  py::class_<Scheduler>(m, "Scheduler").def(py::init<int, int64_t, int64_t, int, int>())
      .def("submit", &Scheduler::submit).def("cancel", &Scheduler::cancel).def("set_checkpoint", &Scheduler::set_checkpoint)
      .def("drop_checkpoint", &Scheduler::drop_checkpoint).def("next", &Scheduler::next, py::arg("disk_prefix_tokens") = 0)
      .def("on_admitted", &Scheduler::on_admitted).def("on_prefilled", &Scheduler::on_prefilled).def("on_tokens", &Scheduler::on_tokens)
      .def("on_finished", &Scheduler::on_finished).def("slot", &Scheduler::slot, py::return_value_policy::copy)
      .def("request", &Scheduler::request, py::return_value_policy::copy)
      .def("has_work", &Scheduler::has_work)
      .def("stats", [](Scheduler& s) { auto t = s.stats(); return py::dict(py::arg("waiting") = t.waiting, py::arg("running") = t.running, py::arg("decoding") = t.decoding, py::arg("prefilling") = t.prefilling, py::arg("admitted") = t.admitted, py::arg("finished") = t.finished, py::arg("cancelled") = t.cancelled, py::arg("prefix_hit_tokens") = t.prefix_hit_tokens, py::arg("kv_budget") = t.kv_budget, py::arg("kv_active") = t.kv_active); })
      .def_static("common_prefix", &Scheduler::common_prefix);

  py::class_<OpLog>(m, "OpLog").def(py::init<const std::string&, bool, int, int>(), py::arg("name"), py::arg("create"), py::arg("n_followers") = 0, py::arg("follower_index") = -1)
      .def("append", &OpLog::append, py::arg("kind"), py::arg("payload"), py::arg("timeout_ms") = 5000, py::call_guard<py::gil_scoped_release>()).def("head", &OpLog::head)
      .def("wait_acked", &OpLog::wait_acked, py::arg("seq"), py::arg("timeout_ms") = 2000, py::call_guard<py::gil_scoped_release>())
      .def("next", [](OpLog& o, uint64_t last, int timeout_ms) { int kind = 0; std::vector<int32_t> pl; bool ok; { py::gil_scoped_release rel; ok = o.next(last, timeout_ms, &kind, &pl); } return py::make_tuple(ok, kind, pl); })
      .def_static("unlink", &OpLog::unlink_name);

  py::class_<TensorInfo>(m, "TensorInfo").def_readonly("dtype", &TensorInfo::dtype).def_readonly("shape", &TensorInfo::shape)
      .def_readonly("begin", &TensorInfo::begin).def_readonly("end", &TensorInfo::end);
  py::class_<SafeTensors>(m, "SafeTensors").def(py::init<const std::string&>())
      .def("names", &SafeTensors::names).def("info", &SafeTensors::info, py::return_value_policy::copy).def("has", &SafeTensors::has)
      .def("read_into", [](SafeTensors& s, const std::string& n, uintptr_t dst, int64_t cap) { py::gil_scoped_release rel; return s.read_into(n, reinterpret_cast<void*>(dst), cap); })
      .def("bytes", [](SafeTensors& s, const std::string& n) { auto& ti = s.info(n); return py::bytes(reinterpret_cast<const char*>(s.data(n)), ti.end - ti.begin); })
      .def("prefetch", &SafeTensors::prefetch)
      .def("data_offset", &SafeTensors::data_offset)
      .def("path", &SafeTensors::path);

  m.def("mem_available_bytes", [](const std::string& p) { return mem_available_bytes(p.empty() ? nullptr : p.c_str()); }, py::arg("meminfo") = "");
  m.def("allocator_cap", [](int64_t r, int64_t mg, const std::string& p) { return allocator_cap(r, mg, p.empty() ? nullptr : p.c_str()); }, py::arg("reserved"), py::arg("margin"), py::arg("meminfo") = "");
  m.def("trim_host_memory", &trim_host_memory);
  m.def("drop_file_cache", &drop_file_cache);
  py::class_<MemWatch>(m, "MemWatch").def(py::init<int64_t, int, std::function<void(int64_t)>, const std::string&>(), py::arg("threshold"), py::arg("period_ms"), py::arg("on_low"), py::arg("meminfo") = "")
      .def("fired", &MemWatch::fired);
  // device-memory plumbing (driver API resolved at run time; `fake=True` runs against host memory)
  auto pick = [](bool fake) { return fake ? fake_driver_api() : cuda_driver_api(); };
  m.def("cuda_driver_available", []() { return cuda_driver_api() != nullptr; });
  m.def("fake_driver_mapped_bytes", &fake_driver_mapped_bytes);
  py::class_<VmmRegion>(m, "VmmRegion")
      .def(py::init([pick](int device, size_t max_bytes, bool fake) { return new VmmRegion(pick(fake), device, max_bytes); }),
           py::arg("device"), py::arg("max_bytes"), py::arg("fake") = false)
      .def_property_readonly("ptr", &VmmRegion::ptr).def_property_readonly("size", &VmmRegion::size)
      .def_property_readonly("capacity", &VmmRegion::capacity).def_property_readonly("granularity", &VmmRegion::granularity)
      .def("resize", &VmmRegion::resize);
  py::class_<PinnedBuffer>(m, "PinnedBuffer", py::buffer_protocol())
      .def(py::init([pick](size_t bytes, bool huge, bool fake) { return new PinnedBuffer(pick(fake), bytes, huge); }),
           py::arg("bytes"), py::arg("huge_pages") = false, py::arg("fake") = false)
      .def_property_readonly("registered", &PinnedBuffer::registered).def_property_readonly("size", &PinnedBuffer::size)
      .def_property_readonly("ptr", [](const PinnedBuffer& b) { return reinterpret_cast<uint64_t>(b.data()); })
      .def_buffer([](PinnedBuffer& b) { return py::buffer_info(b.data(), 1, py::format_descriptor<uint8_t>::format(), 1, {b.size()}, {1}); });
  py::class_<LoadStats>(m, "LoadStats").def_readonly("bytes", &LoadStats::bytes).def_readonly("reads", &LoadStats::reads)
      .def_readonly("copies", &LoadStats::copies).def_readonly("read_s", &LoadStats::read_s).def_readonly("total_s", &LoadStats::total_s).def_readonly("direct", &LoadStats::direct);
  m.def("fast_load", [pick](const std::string& path, int64_t offset, int64_t size, uint64_t dst, uint64_t stream, size_t chunk,
                            int n_buffers, int n_threads, bool fake, bool direct) {
          py::gil_scoped_release rel;
          return fast_load(pick(fake), path, offset, size, dst, stream, chunk, n_buffers, n_threads, direct);
        }, py::arg("path"), py::arg("offset"), py::arg("size"), py::arg("dst"), py::arg("stream") = 0,
        py::arg("chunk") = 64 << 20, py::arg("n_buffers") = 3, py::arg("n_threads") = 2, py::arg("fake") = false,
        py::arg("direct") = false);
  m.def("sha256_hex", [](py::bytes b) { std::string s = b; Sha256 h; h.update(s.data(), s.size()); return h.hex(); });
}
