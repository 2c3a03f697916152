// Python module `torchcomms_b200._comms`: enums, options, work, window,
// communicator, factory.
//
// Parity: comms/torchcomms/TorchCommPy.cpp:55 (module), :577-1039 (window),
// :1116-1200 (new_comm), :1226-1244 (copy/deepcopy identity), :2393-2660 (hook
// registration); signatures follow comms/torchcomms/_comms.pyi:607-844.
#include "py_common.hpp"

#include "../backends/cpu_backends.hpp"
#include "../core/logging.hpp"

namespace b200c {

namespace {

py::object& pre_converter() {
  static py::object* fn = new py::object(py::none());
  return *fn;
}
py::object& post_converter() {
  static py::object* fn = new py::object(py::none());
  return *fn;
}

using OptHints = std::optional<Hints>;
using OptMillis = std::optional<Millis>;
using Release = py::call_guard<py::gil_scoped_release>;

} // namespace

py::object to_python_pre_args(const OpRecord& rec) {
  if (pre_converter().is_none()) {
    return py::cast(rec);
  }
  return pre_converter()(py::cast(rec));
}

py::object to_python_post_args(const OpRecord& rec) {
  if (post_converter().is_none()) {
    return py::cast(rec);
  }
  return post_converter()(py::cast(rec));
}

// The last reference to a communicator usually dies inside Python (object
// deallocation, GIL held). Tearing a backend down can join transport threads
// that themselves need the GIL for a moment (hook callables, work callbacks),
// so the C++ object is released with the GIL dropped.
static std::shared_ptr<Comm> gil_free_on_release(std::shared_ptr<Comm> inner) {
  if (!inner) return inner;
  Comm* raw = inner.get();
  return std::shared_ptr<Comm>(raw, [inner](Comm*) mutable {
    if (interpreter_dying()) {
      inner.reset();
    } else if (PyGILState_Check()) {
      py::gil_scoped_release nogil;
      inner.reset();
    } else {
      inner.reset();
    }
  });
}

void bind_core(py::module_& m) {
  m.attr("BACKEND_ABI_VERSION") = kBackendAbiVersion;

  py::enum_<RedOpType>(m, "RedOpType")
      .value("SUM", RedOpType::SUM)
      .value("PRODUCT", RedOpType::PRODUCT)
      .value("MIN", RedOpType::MIN)
      .value("MAX", RedOpType::MAX)
      .value("BAND", RedOpType::BAND)
      .value("BOR", RedOpType::BOR)
      .value("BXOR", RedOpType::BXOR)
      .value("PREMUL_SUM", RedOpType::PREMUL_SUM)
      .value("AVG", RedOpType::AVG);

  py::class_<ReduceOp> red(m, "ReduceOp");
  red.def(py::init<RedOpType>())
      .def_property_readonly("type", &ReduceOp::type)
      .def_property_readonly("factor", [](const ReduceOp& op) -> py::object {
        if (!op.factor()) {
          return py::none();
        }
        if (std::holds_alternative<double>(*op.factor())) {
          return py::cast(std::get<double>(*op.factor()));
        }
        return py::cast(std::get<at::Tensor>(*op.factor()));
      })
      .def_static("PREMUL_SUM", [](py::object factor) {
        if (THPVariable_Check(factor.ptr())) {
          return ReduceOp::premul_sum(factor.cast<at::Tensor>());
        }
        return ReduceOp::premul_sum(factor.cast<double>());
      }, py::arg("factor"))
      .def("__eq__", [](const ReduceOp& a, const ReduceOp& b) { return a.type() == b.type(); })
      .def("__hash__", [](const ReduceOp& a) { return static_cast<int>(a.type()); })
      .def("__repr__", [](const ReduceOp& a) { return std::string("ReduceOp.") + red_op_name(a.type()); });
  red.attr("SUM") = ReduceOp(RedOpType::SUM);
  red.attr("PRODUCT") = ReduceOp(RedOpType::PRODUCT);
  red.attr("MIN") = ReduceOp(RedOpType::MIN);
  red.attr("MAX") = ReduceOp(RedOpType::MAX);
  red.attr("BAND") = ReduceOp(RedOpType::BAND);
  red.attr("BOR") = ReduceOp(RedOpType::BOR);
  red.attr("BXOR") = ReduceOp(RedOpType::BXOR);
  red.attr("AVG") = ReduceOp(RedOpType::AVG);

  py::enum_<WorkStatus>(m, "WorkStatus")
      .value("NOT_STARTED", WorkStatus::NOT_STARTED)
      .value("INPROGRESS", WorkStatus::INPROGRESS)
      .value("COMPLETED", WorkStatus::COMPLETED)
      .value("TIMEDOUT", WorkStatus::TIMEDOUT)
      .value("ERROR", WorkStatus::ERROR);

  auto opname = py::enum_<OpName>(m, "OpName");
  for (int i = 0; i < static_cast<int>(OpName::kCount); ++i) {
    opname.value(std::string(op_name(static_cast<OpName>(i))).c_str(), static_cast<OpName>(i));
  }

  py::enum_<P2PKind>(m, "P2POpType").value("SEND", P2PKind::SEND).value("RECV", P2PKind::RECV);

  py::enum_<WinAccessType>(m, "TorchCommWinAccessType")
      .value("WIN_ACCESS_TYPE_UNIFIED", WinAccessType::UNIFIED)
      .value("WIN_ACCESS_TYPE_SEPARATE", WinAccessType::SEPARATE);

  py::class_<WindowAttr>(m, "TorchCommWindowAttr")
      .def(py::init<>())
      .def_readwrite("access_type", &WindowAttr::access_type);

  py::class_<RemovableHandle>(m, "RemovableHandle").def("remove", &RemovableHandle::remove);

  // Per-operation options. Python subclasses give the per-op names
  // (AllReduceOptions, ...) of the reference API.
  py::class_<OpOptions>(m, "OpOptions")
      .def(py::init<>())
      .def_readwrite("hints", &OpOptions::hints)
      .def_property("timeout", [](const OpOptions& o) { return o.timeout; },
                    [](OpOptions& o, Millis t) {
                      o.timeout = t;
                      o.timeout_set = true;
                    });

  py::class_<CommOptions>(m, "CommOptions")
      .def(py::init<>())
      .def_readwrite("abort_process_on_timeout_or_error", &CommOptions::abort_process_on_timeout_or_error)
      .def_readwrite("timeout", &CommOptions::timeout)
      .def_readwrite("is_high_priority_stream", &CommOptions::is_high_priority_stream)
      .def_readwrite("store", &CommOptions::store)
      .def_readwrite("enable_reconfigure", &CommOptions::enable_reconfigure)
      .def_readwrite("hints", &CommOptions::hints)
      .def_readwrite("name", &CommOptions::name);

  py::class_<ReconfigureOptions>(m, "ReconfigureOptions")
      .def(py::init([](int64_t uuid, py::object handles, OptMillis timeout, OptHints hints) {
        ReconfigureOptions o;
        o.uuid = uuid;
        o.handles_ordered = !py::isinstance<py::set>(handles) && !py::isinstance<py::frozenset>(handles);
        for (auto h : handles) {
          o.handles.push_back(h.cast<std::string>());
        }
        o.timeout = timeout;
        if (hints) {
          o.hints = *hints;
        }
        return o;
      }), py::arg("uuid"), py::arg("init_handles"), py::arg("timeout") = py::none(), py::arg("hints") = py::none())
      .def_readwrite("uuid", &ReconfigureOptions::uuid)
      .def_readwrite("handles", &ReconfigureOptions::handles)
      // The reference's name for the member list; assigning a set sorts the handles, a list fixes the rank order.
      .def_property("init_handles",
                    [](const ReconfigureOptions& o) { return o.handles; },
                    [](ReconfigureOptions& o, py::object handles) {
                      o.handles_ordered = !py::isinstance<py::set>(handles) && !py::isinstance<py::frozenset>(handles);
                      o.handles.clear();
                      for (auto h : handles) {
                        o.handles.push_back(h.cast<std::string>());
                      }
                    })
      .def_readwrite("timeout", &ReconfigureOptions::timeout)
      .def_readwrite("hints", &ReconfigureOptions::hints);

  py::class_<Work, c10::intrusive_ptr<Work>>(m, "TorchWork")
      .def("is_completed", &Work::is_completed)
      .def("status", &Work::status)
      .def("wait", &Work::wait, Release())
      .def("wait_blocking", &Work::wait_blocking, Release())
      .def("get_timeout", &Work::timeout)
      .def("error", &Work::error)
      .def("_set_status", &Work::set_status)
      .def("register_start_hook", [](Work& w, py::function f) { auto h = hold_callable(std::move(f)); w.on_start([h]() { py::gil_scoped_acquire g; (*h)(); }); })
      .def("register_end_hook", [](Work& w, py::function f) { auto h = hold_callable(std::move(f)); w.on_end([h]() { py::gil_scoped_acquire g; (*h)(); }); })
      .def("register_wait_pre_hook", [](Work& w, py::function f) { auto h = hold_callable(std::move(f)); w.on_wait_pre([h]() { py::gil_scoped_acquire g; (*h)(); }); })
      .def("register_wait_post_hook", [](Work& w, py::function f) { auto h = hold_callable(std::move(f)); w.on_wait_post([h]() { py::gil_scoped_acquire g; (*h)(); }); });

  m.def("_completed_work", []() -> WorkPtr { return c10::make_intrusive<CompletedWork>(); });

  py::class_<OpRecord>(m, "OpRecord")
      .def_property_readonly("op", [](const OpRecord& r) { return r.op; })
      .def_property_readonly("inputs", [](const OpRecord& r) { return r.inputs; })
      .def_property_readonly("outputs", [](const OpRecord& r) { return r.outputs; })
      .def_property_readonly("in_place", [](const OpRecord& r) { return r.in_place; })
      .def_property_readonly("root", [](const OpRecord& r) { return r.root; })
      .def_property_readonly("async_op", [](const OpRecord& r) { return r.async_op; })
      .def_property_readonly("red_op", [](const OpRecord& r) -> py::object {
        return r.red_op ? py::cast(*r.red_op) : py::none();
      })
      .def_property_readonly("in_splits", [](const OpRecord& r) { return r.in_splits; })
      .def_property_readonly("out_splits", [](const OpRecord& r) { return r.out_splits; })
      .def_property_readonly("p2p_ops", [](const OpRecord& r) { return r.p2p_ops; })
      .def_property_readonly("ranks", [](const OpRecord& r) { return r.ranks; })
      .def_property_readonly("name", [](const OpRecord& r) { return r.name; })
      .def_property_readonly("work", [](const OpRecord& r) -> py::object {
        auto w = r.work.lock();
        return w ? py::cast(w) : py::none();
      });

  m.def("_set_hook_arg_converters", [](py::object pre, py::object post) {
    pre_converter() = std::move(pre);
    post_converter() = std::move(post);
  });

  py::class_<P2POp>(m, "P2POp")
      .def(py::init([](P2PKind kind, at::Tensor t, int peer) { return P2POp{kind, std::move(t), peer}; }),
           py::arg("type"), py::arg("tensor"), py::arg("peer"))
      .def_readwrite("type", &P2POp::kind)
      .def_readwrite("tensor", &P2POp::tensor)
      .def_readwrite("peer", &P2POp::peer);

  py::class_<BatchSendRecv, std::shared_ptr<BatchSendRecv>>(m, "BatchSendRecv")
      .def_readwrite("ops", &BatchSendRecv::ops)
      .def("send", &BatchSendRecv::send, py::arg("tensor"), py::arg("dst"))
      .def("recv", [](BatchSendRecv& b, at::Tensor t, int src) { b.recv(t, src); }, py::arg("tensor"), py::arg("src"))
      .def("issue", [](BatchSendRecv& b, bool async_op, const OpOptions& o) { return b.issue(async_op, o); },
           py::arg("async_op"), py::arg("options") = OpOptions{}, Release());

  py::class_<AllGatherPHandle, std::shared_ptr<AllGatherPHandle>>(m, "AllGatherPHandle")
      .def_readonly("id", &AllGatherPHandle::id);

  py::class_<Window, std::shared_ptr<Window>>(m, "TorchCommWindow")
      .def_property_readonly("dtype", [](const Window& w) {
        return py::reinterpret_borrow<py::object>(reinterpret_cast<PyObject*>(torch::getTHPDtype(w.dtype())));
      })
      .def_property_readonly("shape", [](const Window& w) { return w.shape(); })
      .def_property_readonly("device", [](const Window& w) { return w.device(); })
      .def("get_size", &Window::get_size)
      .def("get_tensor", [](const Window& w) -> py::object {
        auto t = w.get_tensor();
        return t ? py::cast(*t) : py::none();
      })
      .def("tensor_register", &Window::tensor_register, py::arg("tensor"), py::arg("owning") = true, Release())
      .def("tensor_deregister", &Window::tensor_deregister, Release())
      .def("put", [](Window& w, const at::Tensor& t, int dst, int64_t off, bool async_op, OptHints h, OptMillis to) {
        return w.put(t, dst, off, async_op, make_op_options(h, to));
      }, py::arg("tensor"), py::arg("dst_rank"), py::arg("target_offset_nelems"), py::arg("async_op"),
         py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("signal", [](Window& w, int dst, bool async_op, OptHints h, OptMillis to) {
        return w.signal(dst, async_op, make_op_options(h, to));
      }, py::arg("dst_rank"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("wait_signal", [](Window& w, int peer, bool async_op, OptHints h, OptMillis to) {
        return w.wait_signal(peer, async_op, make_op_options(h, to));
      }, py::arg("peer_rank"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("map_remote_tensor", &Window::map_remote_tensor, py::arg("rank"))
      .def("get_attr", &Window::get_attr, py::arg("peer_rank"))
      .def("get_device_window", &Window::get_device_window, py::arg("signal_count") = -1,
           py::arg("counter_count") = -1, py::arg("barrier_count") = 1)
      .def("register_local_buffer", &Window::register_local_buffer, py::arg("tensor"))
      .def("deregister_local_buffer", &Window::deregister_local_buffer, py::arg("handle"))
      .def("__copy__", [](std::shared_ptr<Window> w) { return w; })
      .def("__deepcopy__", [](std::shared_ptr<Window> w, py::dict memo) {
        auto c = w->clone();
        auto src = w->get_tensor();
        auto dst = c->get_tensor();
        if (src && dst) {
          memo[py::int_(reinterpret_cast<uintptr_t>(py::cast(*src).ptr()))] = py::cast(*dst);
        }
        return c;
      }, py::arg("memo"));

  py::class_<Backend, std::shared_ptr<Backend>>(m, "_NativeBackend")
      .def("get_backend_name", &Backend::backend_name)
      .def("get_comm_name", &Backend::comm_name)
      .def("get_rank", &Backend::rank)
      .def("get_size", &Backend::size);

  py::class_<FakeBackend, Backend, std::shared_ptr<FakeBackend>>(m, "FakeBackend")
      .def_readonly("calls", &FakeBackend::calls);
  py::class_<GlooBackend, Backend, std::shared_ptr<GlooBackend>>(m, "GlooBackend");

  py::class_<Comm, std::shared_ptr<Comm>> comm(m, "TorchComm");
  comm.def("finalize", &Comm::finalize, Release())
      .def("get_rank", &Comm::get_rank)
      .def("get_size", &Comm::get_size)
      .def("get_name", &Comm::get_name)
      .def("get_options", &Comm::get_options)
      .def("get_device", &Comm::get_device)
      .def("get_backend", &Comm::get_backend)
      .def("get_backend_version", &Comm::get_backend_version)
      .def("comm_dump", [](Comm& c) { return c.get_backend_impl()->comm_dump(); })
      .def("get_backend_impl", &Comm::get_backend_impl)
      .def("unsafe_get_backend", &Comm::get_backend_impl)
      .def("get_ranks", &Comm::get_ranks)
      .def("get_init_handle", &Comm::get_init_handle)
      .def("reconfigure", [](Comm& c, int64_t uuid, py::object handles, OptMillis timeout, OptHints hints) {
        ReconfigureOptions o;
        o.uuid = uuid;
        o.handles_ordered = !py::isinstance<py::set>(handles) && !py::isinstance<py::frozenset>(handles);
        for (auto h : handles) {
          o.handles.push_back(h.cast<std::string>());
        }
        o.timeout = timeout;
        if (hints) {
          o.hints = *hints;
        }
        py::gil_scoped_release nogil;
        return c.reconfigure(o);
      }, py::arg("uuid"), py::arg("init_handles"), py::arg("timeout") = py::none(), py::arg("hints") = py::none())
      .def("abort", &Comm::abort, Release())
      .def("is_abort_supported", &Comm::is_abort_supported)
      .def("is_aborted", &Comm::is_aborted)
      .def("set_timeout", &Comm::set_timeout, py::arg("timeout"))
      .def("set_hints", &Comm::set_hints, py::arg("hints"))
      .def("send", [](Comm& c, const at::Tensor& t, int dst, bool a, OptHints h, OptMillis to) {
        return c.send(t, dst, a, make_op_options(h, to));
      }, py::arg("tensor"), py::arg("dst"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("recv", [](Comm& c, at::Tensor t, int src, bool a, OptHints h, OptMillis to) {
        return c.recv(t, src, a, make_op_options(h, to));
      }, py::arg("tensor"), py::arg("src"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("broadcast", [](Comm& c, at::Tensor t, int root, bool a, OptHints h, OptMillis to) {
        return c.broadcast(t, root, a, make_op_options(h, to));
      }, py::arg("tensor"), py::arg("root"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_reduce", [](Comm& c, at::Tensor t, const ReduceOp& op, bool a, OptHints h, OptMillis to) {
        return c.all_reduce(t, op, a, make_op_options(h, to));
      }, py::arg("tensor"), py::arg("op"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("reduce", [](Comm& c, const at::Tensor& t, int root, const ReduceOp& op, bool a, OptHints h, OptMillis to) {
        return c.reduce(t, root, op, a, make_op_options(h, to));
      }, py::arg("tensor"), py::arg("root"), py::arg("op"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_gather", [](Comm& c, const std::vector<at::Tensor>& outs, const at::Tensor& in, bool a, OptHints h, OptMillis to) {
        return c.all_gather(outs, in, a, make_op_options(h, to));
      }, py::arg("tensor_list"), py::arg("tensor"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_gather_v", [](Comm& c, const std::vector<at::Tensor>& outs, const at::Tensor& in, bool a, OptHints h, OptMillis to) {
        return c.all_gather_v(outs, in, a, make_op_options(h, to));
      }, py::arg("tensor_list"), py::arg("tensor"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_gather_single", [](Comm& c, at::Tensor out, const at::Tensor& in, bool a, OptHints h, OptMillis to) {
        return c.all_gather_single(out, in, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("reduce_scatter", [](Comm& c, at::Tensor out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool a, OptHints h, OptMillis to) {
        return c.reduce_scatter(out, ins, op, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input_list"), py::arg("op"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("reduce_scatter_v", [](Comm& c, at::Tensor out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool a, OptHints h, OptMillis to) {
        return c.reduce_scatter_v(out, ins, op, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input_list"), py::arg("op"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("reduce_scatter_single", [](Comm& c, at::Tensor out, const at::Tensor& in, const ReduceOp& op, bool a, OptHints h, OptMillis to) {
        return c.reduce_scatter_single(out, in, op, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("op"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_to_all_single", [](Comm& c, at::Tensor out, const at::Tensor& in, bool a, OptHints h, OptMillis to) {
        return c.all_to_all_single(out, in, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_to_all_v_single", [](Comm& c, at::Tensor out, const at::Tensor& in, const std::vector<int64_t>& os,
                                    const std::vector<int64_t>& is, bool a, OptHints h, OptMillis to) {
        return c.all_to_all_v_single(out, in, os, is, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("output_split_sizes"), py::arg("input_split_sizes"),
         py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_to_all", [](Comm& c, const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool a, OptHints h, OptMillis to) {
        return c.all_to_all(outs, ins, a, make_op_options(h, to));
      }, py::arg("output_tensor_list"), py::arg("input_tensor_list"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("barrier", [](Comm& c, bool a, OptHints h, OptMillis to) {
        return c.barrier(a, make_op_options(h, to));
      }, py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("scatter", [](Comm& c, at::Tensor out, const std::vector<at::Tensor>& ins, int root, bool a, OptHints h, OptMillis to) {
        return c.scatter(out, ins, root, a, make_op_options(h, to));
      }, py::arg("output_tensor"), py::arg("input_tensor_list"), py::arg("root"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("gather", [](Comm& c, const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool a, OptHints h, OptMillis to) {
        return c.gather(outs, in, root, a, make_op_options(h, to));
      }, py::arg("output_tensor_list"), py::arg("input_tensor"), py::arg("root"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("gather_single", [](Comm& c, at::Tensor out, const at::Tensor& in, int root, bool a, OptHints h, OptMillis to) {
        return c.gather_single(out, in, root, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("root"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("split", [](Comm& c, const std::vector<int>& ranks, const std::string& name, OptHints h, OptMillis to) {
        CommOptions o = c.get_options();
        if (h) {
          o.hints = *h;
        }
        if (to) {
          o.timeout = *to;
        }
        return gil_free_on_release(c.split(ranks, name, o));
      }, py::arg("ranks"), py::arg("name"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("batch_op_create", &Comm::batch_op_create)
      .def("new_window", [](Comm& c, std::optional<at::Tensor> t) { return c.new_window(t); },
           py::arg("tensor") = py::none(), Release())
      .def("all_gather_p_init", [](Comm& c, at::Tensor out, OptHints h, OptMillis to) {
        return c.all_gather_p_init(out, make_op_options(h, to));
      }, py::arg("output"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_gather_p_exec", [](Comm& c, std::shared_ptr<AllGatherPHandle> hd, const at::Tensor& in, bool a, OptHints h, OptMillis to) {
        return c.all_gather_p_exec(hd, in, a, make_op_options(h, to));
      }, py::arg("handle"), py::arg("input"), py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(), Release())
      .def("all_gather_p_free", &Comm::all_gather_p_free, py::arg("handle"), Release())
      .def("tensor_register", &Comm::tensor_register, py::arg("tensor"), Release())
      .def("tensor_deregister", &Comm::tensor_deregister, py::arg("tensor"), Release())
      .def("register_pre_hook", [](Comm& c, py::function cb) {
        auto h = hold_callable(std::move(cb));
        return c.register_pre_hook([h](OpName op, size_t id, const OpRecord& rec) {
          py::gil_scoped_acquire g;
          (*h)(op, id, to_python_pre_args(rec));
        });
      }, py::arg("callback"))
      .def("register_post_hook", [](Comm& c, py::function cb) {
        auto h = hold_callable(std::move(cb));
        return c.register_post_hook([h](size_t id, const OpRecord& rec) {
          py::gil_scoped_acquire g;
          (*h)(id, to_python_post_args(rec));
        });
      }, py::arg("callback"))
      .def("register_abort_hook", [](Comm& c, py::function cb) {
        auto h = hold_callable(std::move(cb));
        return c.register_abort_hook([h]() {
          py::gil_scoped_acquire g;
          (*h)();
        });
      }, py::arg("callback"))
      .def("register_graph_replay_hook", [](Comm& c, py::function cb) {
        auto h = hold_callable(std::move(cb));
        return c.register_graph_replay_hook([h](uint64_t gid, uint64_t rid, uintptr_t stream, size_t idx, char ev) {
          py::gil_scoped_acquire g;
          (*h)(gid, rid, stream, idx, std::string(1, ev));
        });
      }, py::arg("callback"))
      // A communicator is a process-level resource: copies are the object itself.
      .def("__copy__", [](std::shared_ptr<Comm> c) { return c; })
      .def("__deepcopy__", [](std::shared_ptr<Comm> c, py::dict) { return c; }, py::arg("memo"));

  m.def("_new_comm", [](const std::string& backend, at::Device device, const std::string& name, const CommOptions& opts) {
    return gil_free_on_release(new_comm(backend, device, name, opts));
  }, py::arg("backend"), py::arg("device"), py::arg("name"), py::arg("options"), Release());

  m.def("_is_backend_registered", [](const std::string& n) { return Factory::get().is_registered(n); });
  m.def("_registered_backends", []() { return Factory::get().registered(); });
  m.def("_next_op_id", &Comm::next_op_id);
  m.def("_query_ranksize", &query_ranksize);
  m.def("_create_prefix_store", [](const std::string& prefix, Millis timeout) {
    auto [rank, size] = query_ranksize();
    return create_prefix_store(prefix, rank, size, timeout);
  }, py::arg("prefix"), py::arg("timeout") = kDefaultTimeout, py::call_guard<py::gil_scoped_release>());
  m.def("_dup_prefix_store", &dup_prefix_store, py::arg("prefix"), py::arg("bootstrap_store"),
        py::arg("timeout") = kDefaultTimeout, py::call_guard<py::gil_scoped_release>());
  m.def("_knobs", [] {
    std::vector<std::tuple<std::string, std::string, std::string>> out;
    for (auto& k : knob_report()) {
      out.emplace_back(k[0], k[1], k[2]);
    }
    return out;
  });
  m.def("_reload_config", &reload_config_file);
  m.def("set_trainer_iteration", &set_trainer_iteration, py::arg("iteration"));
  m.def("trainer_iteration", &trainer_iteration);
  m.def("comm_dump_all", [](const std::optional<Hints>&) { return comm_dump_all(); }, py::arg("hints") = py::none(),
        "State of every live communicator of this process: {comm name: {key: value}}.");
  m.def("_recent_log_lines", []() { return Logger::get().recent(); });

  m.def("_health_is_healthy", &HealthCheck::healthy);
  m.def("_health_reason", &HealthCheck::reason);
  m.def("_health_mark_unhealthy", &HealthCheck::mark_unhealthy);
  m.def("_health_reset", &HealthCheck::reset);

  m.def("_install_gloo_maker", [](py::function maker) {
    // `maker(store, rank, size, timeout) -> torch.distributed.ProcessGroupGloo`
    auto held = hold_callable(std::move(maker));
    set_gloo_pg_maker([held](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, Millis timeout) {
      py::gil_scoped_acquire g;
      py::object pg = (*held)(store, rank, size, timeout);
      return pg.cast<c10::intrusive_ptr<c10d::Backend>>();
    });
  });

  Factory::get().register_backend("fake", [] { return std::make_shared<FakeBackend>(); });
  Factory::get().register_backend("gloo", [] { return std::make_shared<GlooBackend>(); });
}

} // namespace b200c

PYBIND11_MODULE(_comms, m) {
  m.doc() = "torchcomms_b200 native core";
  b200c::bind_core(m);
  b200c::bind_python_backend(m);
  b200c::bind_hooks(m);
  b200c::bind_c10d_wrapper(m);
  b200c::bind_cuda_backend(m);
  b200c::bind_ops(m);
  b200c::bind_ep(m);
  b200c::bind_ep_ll(m);
  b200c::bind_p2p(m);
  b200c::bind_tp(m);
  b200c::bind_transport(m);
  b200c::bind_arnorm(m);
  b200c::bind_fakes(m);
}
