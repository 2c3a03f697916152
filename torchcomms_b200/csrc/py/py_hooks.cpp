// Python bindings for the flight recorder and the collective log
// (submodules `_comms.hooks.fr` and `_comms.hooks.clog`).
//
// Parity: comms/torchcomms/hooks/fr/FlightRecorderPy.cpp and the clog binding
// registered from comms/torchcomms/TorchCommPy.cpp:2727-2754.
#include "py_common.hpp"

#include "../hooks/recorders.hpp"

namespace b200c {

void bind_hooks(py::module_& m) {
  auto hooks = m.def_submodule("hooks", "hook-based observers");
  auto fr = hooks.def_submodule("fr", "flight recorder");
  py::class_<FlightRecorder, std::shared_ptr<FlightRecorder>>(fr, "FlightRecorderHook")
      // Every hook object owns its recorder, so `isolated` (the reference's switch between a process-wide recorder
      // and one of the hook's own) is accepted and has nothing to choose between.
      .def(py::init([](size_t cap, bool /*isolated*/) { return std::make_shared<FlightRecorder>(cap); }),
           py::arg("max_entries") = 0, py::arg("isolated") = false)
      .def("is_enabled", [](const FlightRecorder& f) { return f.capacity() > 0; })
      .def("register_with_comm", &FlightRecorder::attach, py::arg("comm"))
      .def("unregister", &FlightRecorder::detach)
      .def("dump_json", &FlightRecorder::dump_json, py::arg("include_completed") = true)
      .def("dump_file", &FlightRecorder::dump_file, py::arg("rank"), py::arg("include_completed") = true)
      .def("size", &FlightRecorder::size)
      .def("capacity", &FlightRecorder::capacity)
      .def("reset", &FlightRecorder::reset)
      .def("entries", [](const FlightRecorder& f) {
        py::list out;
        for (auto& e : f.entries()) {
          py::dict d;
          d["record_id"] = e.record_id;
          d["op_id"] = e.op_id;
          d["comm_name"] = e.comm_name;
          d["op"] = e.op;
          d["state"] = e.state;
          d["collective_seq_id"] = e.collective_seq;
          d["p2p_seq_id"] = e.p2p_seq;
          d["is_p2p"] = e.is_p2p;
          d["input_sizes"] = e.in_sizes;
          d["output_sizes"] = e.out_sizes;
          d["input_dtypes"] = e.in_dtypes;
          d["output_dtypes"] = e.out_dtypes;
          d["retired"] = e.retired;
          d["iteration"] = e.iteration;
          out.append(d);
        }
        return out;
      });

  auto clog = hooks.def_submodule("clog", "pipe-delimited collective log");
  py::class_<CollectiveLog, std::shared_ptr<CollectiveLog>>(clog, "ClogHook")
      .def(py::init([](const std::string& path) { return std::make_shared<CollectiveLog>(path); }), py::arg("path") = "")
      .def("register_with_comm", &CollectiveLog::attach, py::arg("comm"))
      .def("unregister", &CollectiveLog::detach)
      .def("lines", &CollectiveLog::lines);
}

} // namespace b200c
