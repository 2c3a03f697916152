// Backends written in Python.
//
// `register_backend(name, cls)` makes `new_comm(name, ...)` instantiate `cls`
// (a subclass of TorchCommBackend) and drive it through an adapter. A method
// may return None (finished), a TorchWork, or any object with `.wait()`.
//
// Parity: comms/torchcomms/PyTorchCommBackend.hpp:15-199 and
// comms/torchcomms/TorchCommBackendPy.cpp:15-347.
#include "py_common.hpp"

namespace b200c {

namespace {

struct PyBackendBase {}; // the Python-visible base class `TorchCommBackend`

// Wraps whatever a Python backend returned from a collective.
class PyObjWork final : public Work {
 public:
  explicit PyObjWork(py::object obj) : obj_(std::move(obj)) { set_status(WorkStatus::INPROGRESS); }
  ~PyObjWork() override { drop_object(obj_); }

 protected:
  void do_wait() override {
    py::gil_scoped_acquire g;
    if (py::hasattr(obj_, "wait")) {
      obj_.attr("wait")();
    }
    set_status(WorkStatus::COMPLETED);
  }

 private:
  py::object obj_;
};

WorkPtr to_work(py::object ret) {
  if (ret.is_none()) {
    return c10::make_intrusive<CompletedWork>();
  }
  if (py::isinstance<Work>(ret)) {
    return ret.cast<WorkPtr>();
  }
  return c10::make_intrusive<PyObjWork>(std::move(ret));
}

class PyBackendAdapter final : public Backend {
 public:
  explicit PyBackendAdapter(py::object self) : self_(std::move(self)) {}
  ~PyBackendAdapter() override { drop_object(self_); }

  template <typename... A>
  py::object call(const char* method, A&&... a) const {
    py::gil_scoped_acquire g;
    TORCH_CHECK(py::hasattr(self_, method), "Python backend does not implement '", method, "'");
    return self_.attr(method)(std::forward<A>(a)...);
  }
  template <typename... A>
  WorkPtr op(const char* method, A&&... a) const {
    py::gil_scoped_acquire g;
    return to_work(call(method, std::forward<A>(a)...));
  }

  void init(at::Device device, const std::string& name, const CommOptions& opts) override {
    opts_ = opts;
    device_ = device;
    py::gil_scoped_acquire g; // the returned object must die under the GIL
    call("init", device, name, opts);
  }
  void finalize() override {
    py::gil_scoped_acquire g;
    call("finalize");
  }
  int rank() const override {
    py::gil_scoped_acquire g;
    return call("get_rank").cast<int>();
  }
  int size() const override {
    py::gil_scoped_acquire g;
    return call("get_size").cast<int>();
  }
  std::string backend_name() const override {
    py::gil_scoped_acquire g;
    return call("get_backend_name").cast<std::string>();
  }
  std::string comm_name() const override {
    py::gil_scoped_acquire g;
    return call("get_comm_name").cast<std::string>();
  }
  at::Device device() const override { return device_; }
  const CommOptions& options() const override { return opts_; }

  WorkPtr send(const at::Tensor& t, int dst, bool a, const OpOptions&) override { return op("send", t, dst, a); }
  WorkPtr recv(at::Tensor& t, int src, bool a, const OpOptions&) override { return op("recv", t, src, a); }
  WorkPtr batch_op_issue(const std::vector<P2POp>& ops, bool a, const OpOptions&) override { return op("batch_op_issue", ops, a); }
  WorkPtr broadcast(at::Tensor& t, int root, bool a, const OpOptions&) override { return op("broadcast", t, root, a); }
  WorkPtr all_reduce(at::Tensor& t, const ReduceOp& r, bool a, const OpOptions&) override { return op("all_reduce", t, r, a); }
  WorkPtr reduce(const at::Tensor& t, int root, const ReduceOp& r, bool a, const OpOptions&) override { return op("reduce", t, root, r, a); }
  WorkPtr all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool a, const OpOptions&) override { return op("all_gather", outs, in, a); }
  WorkPtr all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool a, const OpOptions&) override { return op("all_gather_v", outs, in, a); }
  WorkPtr all_gather_single(at::Tensor& out, const at::Tensor& in, bool a, const OpOptions&) override { return op("all_gather_single", out, in, a); }
  WorkPtr reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& r, bool a, const OpOptions&) override { return op("reduce_scatter", out, ins, r, a); }
  WorkPtr reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& r, bool a, const OpOptions&) override { return op("reduce_scatter_v", out, ins, r, a); }
  WorkPtr reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& r, bool a, const OpOptions&) override { return op("reduce_scatter_single", out, in, r, a); }
  WorkPtr all_to_all_single(at::Tensor& out, const at::Tensor& in, bool a, const OpOptions&) override { return op("all_to_all_single", out, in, a); }
  WorkPtr all_to_all_v_single(at::Tensor& out, const at::Tensor& in, const std::vector<int64_t>& os, const std::vector<int64_t>& is, bool a, const OpOptions&) override {
    return op("all_to_all_v_single", out, in, os, is, a);
  }
  WorkPtr all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool a, const OpOptions&) override { return op("all_to_all", outs, ins, a); }
  WorkPtr barrier(bool a, const OpOptions&) override { return op("barrier", a); }
  WorkPtr scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool a, const OpOptions&) override { return op("scatter", out, ins, root, a); }
  WorkPtr gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool a, const OpOptions&) override { return op("gather", outs, in, root, a); }

  std::shared_ptr<Backend> split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) override {
    py::gil_scoped_acquire g;
    py::object child = call("split", ranks, name, opts);
    if (child.is_none()) {
      return nullptr;
    }
    auto b = std::make_shared<PyBackendAdapter>(std::move(child));
    b->opts_ = opts;
    b->device_ = device_;
    return b;
  }

  void set_timeout(Millis t) override {
    opts_.timeout = t;
    py::gil_scoped_acquire g;
    if (py::hasattr(self_, "set_timeout")) {
      self_.attr("set_timeout")(t);
    }
  }
  void set_hints(const Hints& h) override {
    py::gil_scoped_acquire g;
    if (py::hasattr(self_, "set_hints")) {
      self_.attr("set_hints")(h);
    }
  }
  void abort() override {
    py::gil_scoped_acquire g;
    if (py::hasattr(self_, "abort")) {
      self_.attr("abort")();
    }
    run_abort_hooks();
  }
  bool is_aborted() const override {
    py::gil_scoped_acquire g;
    return py::hasattr(self_, "is_aborted") && self_.attr("is_aborted")().cast<bool>();
  }
  bool is_abort_supported() const override {
    py::gil_scoped_acquire g;
    return py::hasattr(self_, "abort");
  }

  py::object python_object() const { return self_; }

 private:
  py::object self_;
  CommOptions opts_;
  at::Device device_{at::kCPU};
};

} // namespace

void bind_python_backend(py::module_& m) {
  py::class_<PyBackendBase>(m, "TorchCommBackend", py::dynamic_attr()).def(py::init<>());

  py::class_<PyBackendAdapter, Backend, std::shared_ptr<PyBackendAdapter>>(m, "_PythonBackendAdapter")
      .def("python_object", &PyBackendAdapter::python_object);

  m.def("register_backend", [](const std::string& name, py::object cls) {
    TORCH_CHECK(PyType_Check(cls.ptr()), "register_backend expects a class");
    auto held = std::make_shared<py::object>(std::move(cls));
    Factory::get().register_backend(name, [held]() -> std::shared_ptr<Backend> {
      py::gil_scoped_acquire g;
      py::object inst = (*held)();
      return std::make_shared<PyBackendAdapter>(std::move(inst));
    });
  }, py::arg("name"), py::arg("backend_class"));
}

} // namespace b200c
