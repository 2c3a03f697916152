// Shared declarations for the Python binding translation units.
#pragma once

#include <pybind11/chrono.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include "../core/comm.hpp"

namespace py = pybind11;

namespace b200c {

inline OpOptions make_op_options(const std::optional<Hints>& hints, const std::optional<Millis>& timeout) {
  OpOptions o;
  if (hints) {
    o.hints = *hints;
  }
  if (timeout) {
    o.timeout = *timeout;
    o.timeout_set = true;
  }
  return o;
}

inline bool interpreter_dying() {
#if PY_VERSION_HEX >= 0x030D0000
  return !Py_IsInitialized() || Py_IsFinalizing();
#else
  return !Py_IsInitialized() || _Py_IsFinalizing();
#endif
}

// Drops a Python reference from a destructor that may run without the GIL or
// during interpreter shutdown.
inline void drop_object(py::object& o) {
  if (interpreter_dying()) {
    o.release();
    return;
  }
  py::gil_scoped_acquire g;
  o = py::object();
}

// Keeps a Python callable alive inside C++ callbacks that get copied and
// destroyed on threads that do not hold the GIL.
inline std::shared_ptr<py::function> hold_callable(py::function f) {
  return std::shared_ptr<py::function>(new py::function(std::move(f)), [](py::function* p) {
    if (interpreter_dying()) {
      p->release(); // the interpreter is going away: leak the reference
      delete p;
      return;
    }
    py::gil_scoped_acquire g;
    delete p;
  });
}

// Binding groups, one per translation unit.
void bind_core(py::module_& m);
void bind_python_backend(py::module_& m);
void bind_hooks(py::module_& m);
void bind_c10d_wrapper(py::module_& m);
void bind_cuda_backend(py::module_& m);
void bind_ops(py::module_& m);
void bind_ep(py::module_& m);
void bind_ep_ll(py::module_& m);
void bind_p2p(py::module_& m);
void bind_tp(py::module_& m);
void bind_transport(py::module_& m);
void bind_arnorm(py::module_& m);
void bind_fakes(py::module_& m);

// Converts a C++ hook record into the typed Python view; installed from
// Python (`_set_hook_arg_converters`).
py::object to_python_pre_args(const OpRecord& rec);
py::object to_python_post_args(const OpRecord& rec);

} // namespace b200c
