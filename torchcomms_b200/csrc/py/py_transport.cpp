// Bindings of the one-sided point-to-point transport (`_comms.transport`).
//
// Parity: comms/torchcomms/transport/RdmaTransportPy.cpp and _transport.pyi
// (RdmaTransport, RdmaMemory, its views, RdmaRemoteBuffer).
#include "py_common.hpp"

#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAFunctions.h>

#include "../transport/p2p_transport.hpp"

namespace b200c {

namespace {

// A registration together with the tensor whose storage it covers.
struct PyTransportMemory {
  at::Tensor tensor;
  std::shared_ptr<TransportMemory> mem;
};

struct PyView {
  TransportView view;
  bool mutable_view;
};

std::shared_ptr<PyTransportMemory> register_tensor(const at::Tensor& t) {
  TORCH_CHECK(t.defined() && t.is_contiguous(), "TransportMemory needs a contiguous tensor");
  TORCH_CHECK(t.nbytes() > 0, "TransportMemory needs a non-empty tensor");
  TORCH_CHECK(t.is_cpu() || t.is_cuda(), "TransportMemory supports cpu and cuda tensors");
  auto out = std::make_shared<PyTransportMemory>();
  out->tensor = t;
  uint64_t alloc_base = 0;
  int device = -1;
  if (t.is_cuda()) {
    device = t.get_device();
    size_t alloc_size = 0;
    try {
      alloc_base = reinterpret_cast<uint64_t>(c10::cuda::CUDACachingAllocator::getBaseAllocation(t.data_ptr(), &alloc_size));
    } catch (const std::exception&) {
      alloc_base = 0;  // memory the caching allocator does not own: export from the pointer itself
    }
  }
  out->mem = TransportMemory::create(t.data_ptr(), t.nbytes(), device, alloc_base);
  return out;
}

PyView make_view(const PyTransportMemory& m, std::optional<size_t> offset, std::optional<size_t> length, bool mut) {
  const size_t off = offset.value_or(0);
  TORCH_CHECK(off <= m.mem->size(), "view offset outside the memory");
  const size_t len = length.value_or(m.mem->size() - off);
  TORCH_CHECK(len <= m.mem->size() - off, "view outside the memory");
  return PyView{TransportView{m.mem, off, len}, mut};
}

}  // namespace

void bind_transport(py::module_& m) {
  py::module_ t = m.def_submodule("transport", "one-sided point-to-point transport");

  t.def("strerror", [](int s) { return std::string(transport_strerror(s)); });
  t.def("register_segment", [](uint64_t ptr, uint64_t len, int device) {
    TransportMemory::register_segment(reinterpret_cast<void*>(ptr), len, device);
  }, py::arg("ptr"), py::arg("len"), py::arg("device"));
  t.def("unregister_segment", [](uint64_t ptr) { TransportMemory::unregister_segment(reinterpret_cast<void*>(ptr)); }, py::arg("ptr"));
  t.def("segment_count", &TransportMemory::segment_count);
  t.def("init_caching_allocator_hook", [] {
    // Every segment the CUDA caching allocator holds, now and from now on, becomes a long-lived
    // registration; tensors registered later reuse it. The callback runs under the allocator's
    // lock, so it only records the range (the export happens when a range is first used).
    TORCH_CHECK(c10::cuda::device_count() > 0, "init_caching_allocator_hook needs a CUDA device");
    static bool attached = false;
    if (attached) return;
    attached = true;
    namespace cca = c10::cuda::CUDACachingAllocator;
    cca::attachAllocatorTraceTracker([](const cca::TraceEntry& e) {
      if (e.action_ == cca::TraceEntry::SEGMENT_ALLOC) {
        TransportMemory::register_segment(reinterpret_cast<void*>(e.addr_), e.size_, static_cast<int>(e.device_));
      } else if (e.action_ == cca::TraceEntry::SEGMENT_FREE) {
        TransportMemory::unregister_segment(reinterpret_cast<void*>(e.addr_));
      }
    });
    for (const auto& seg : cca::snapshot({0, 0}, false).segments) {
      if (!seg.is_expandable) {
        TransportMemory::register_segment(reinterpret_cast<void*>(seg.address), seg.total_size, static_cast<int>(seg.device));
      }
    }
  });
  t.attr("OK") = static_cast<int>(kTransportOk);
  t.attr("BAD_KEY") = static_cast<int>(kTransportBadKey);
  t.attr("OUT_OF_RANGE") = static_cast<int>(kTransportOutOfRange);
  t.attr("NOT_CONNECTED") = static_cast<int>(kTransportNotConnected);
  t.attr("IO_ERROR") = static_cast<int>(kTransportIo);
  t.attr("CUDA_ERROR") = static_cast<int>(kTransportCuda);
  t.attr("TIMEOUT") = static_cast<int>(kTransportTimeout);
  t.attr("CLOSED") = static_cast<int>(kTransportClosed);
  t.attr("SIZE_MISMATCH") = static_cast<int>(kTransportSizeMismatch);

  py::class_<RemoteBuffer>(t, "RemoteBuffer")
      .def(py::init([](uint64_t ptr, uint64_t len, std::string key) { return RemoteBuffer{ptr, len, std::move(key)}; }),
           py::arg("ptr"), py::arg("len"), py::arg("access_key"))
      .def_readonly("ptr", &RemoteBuffer::ptr)
      .def_readonly("len", &RemoteBuffer::len)
      .def_readonly("access_key", &RemoteBuffer::access_key)
      .def("slice",
           [](const RemoteBuffer& b, uint64_t offset, uint64_t length) {
             TORCH_CHECK(offset <= b.len && length <= b.len - offset, "slice outside the buffer");
             return RemoteBuffer{b.ptr + offset, length, b.access_key};
           },
           py::arg("offset"), py::arg("length"))
      .def(py::pickle([](const RemoteBuffer& b) { return py::make_tuple(b.ptr, b.len, b.access_key); },
                      [](py::tuple s) {
                        TORCH_CHECK(s.size() == 3, "bad RemoteBuffer state");
                        return RemoteBuffer{s[0].cast<uint64_t>(), s[1].cast<uint64_t>(), s[2].cast<std::string>()};
                      }))
      .def("__repr__", [](const RemoteBuffer& b) {
        return "RemoteBuffer(ptr=" + std::to_string(b.ptr) + ", len=" + std::to_string(b.len) + ")";
      });

  py::class_<PyView>(t, "MemoryView")
      .def("size", [](const PyView& v) { return v.view.length; })
      .def_property_readonly("mutable", [](const PyView& v) { return v.mutable_view; });

  py::class_<PyTransportMemory, std::shared_ptr<PyTransportMemory>>(t, "TransportMemory")
      .def(py::init(&register_tensor), py::arg("tensor"))
      .def("to_view", [](const PyTransportMemory& m, std::optional<size_t> o, std::optional<size_t> l) { return make_view(m, o, l, false); },
           py::arg("offset") = py::none(), py::arg("length") = py::none())
      .def("to_mutable_view", [](const PyTransportMemory& m, std::optional<size_t> o, std::optional<size_t> l) { return make_view(m, o, l, true); },
           py::arg("offset") = py::none(), py::arg("length") = py::none())
      .def("to_remote_buffer", [](const PyTransportMemory& m) { return m.mem->remote_buffer(); })
      .def("reused_registration", [](const PyTransportMemory& m) { return m.mem->reused_registration(); })
      .def("size", [](const PyTransportMemory& m) { return m.mem->size(); })
      .def_property_readonly("tensor", [](const PyTransportMemory& m) { return m.tensor; })
      .def_property_readonly("access_key", [](const PyTransportMemory& m) { return m.mem->access_key(); });

  py::class_<TransportFuture, std::shared_ptr<TransportFuture>>(t, "TransportFuture")
      .def("done", &TransportFuture::done)
      .def("wait", &TransportFuture::wait, py::arg("timeout_ms") = -1, py::call_guard<py::gil_scoped_release>());

  py::class_<P2pTransport, std::shared_ptr<P2pTransport>>(t, "P2pTransport")
      .def(py::init([](const py::object& device) {
             if (device.is_none()) return std::make_shared<P2pTransport>(-1);
             if (py::isinstance<py::int_>(device)) return std::make_shared<P2pTransport>(device.cast<int>());
             const auto d = device.cast<c10::Device>();
             return std::make_shared<P2pTransport>(d.is_cuda() ? static_cast<int>(d.has_index() ? d.index() : 0) : -1);
           }),
           py::arg("device") = py::none())
      .def_static("supported", &P2pTransport::supported)
      .def("bind", [](P2pTransport& tr) { return py::bytes(tr.bind()); })
      .def("connect", [](P2pTransport& tr, const std::string& url) { return tr.connect(url); }, py::arg("peer_url"),
           py::call_guard<py::gil_scoped_release>())
      .def("connected", &P2pTransport::connected)
      .def("write_async", [](P2pTransport& tr, const PyView& v, const RemoteBuffer& r) { return tr.write(v.view, r); },
           py::arg("local_buffer"), py::arg("remote_buffer"))
      .def("read_async",
           [](P2pTransport& tr, const PyView& v, const RemoteBuffer& r) {
             TORCH_CHECK(v.mutable_view, "read needs a mutable view (to_mutable_view)");
             return tr.read(v.view, r);
           },
           py::arg("local_buffer"), py::arg("remote_buffer"))
      .def("write",
           [](P2pTransport& tr, const PyView& v, const RemoteBuffer& r) {
             auto f = tr.write(v.view, r);
             py::gil_scoped_release g;
             return f->wait(-1);
           },
           py::arg("local_buffer"), py::arg("remote_buffer"))
      .def("read",
           [](P2pTransport& tr, const PyView& v, const RemoteBuffer& r) {
             TORCH_CHECK(v.mutable_view, "read needs a mutable view (to_mutable_view)");
             auto f = tr.read(v.view, r);
             py::gil_scoped_release g;
             return f->wait(-1);
           },
           py::arg("local_buffer"), py::arg("remote_buffer"))
      .def("counters",
           [](const P2pTransport& tr) {
             const TransportCounters c = tr.counters();
             py::dict d;
             d["peer_copy_ops"] = c.peer_copy_ops;
             d["peer_copy_bytes"] = c.peer_copy_bytes;
             d["socket_ops"] = c.socket_ops;
             d["socket_bytes"] = c.socket_bytes;
             d["served_ops"] = c.served_ops;
             d["served_bytes"] = c.served_bytes;
             d["rejected"] = c.rejected;
             return d;
           })
      .def("close", &P2pTransport::close, py::call_guard<py::gil_scoped_release>());
}

}  // namespace b200c
