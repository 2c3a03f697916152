// placeholder until the CUDA backend lands
#include "py_common.hpp"
namespace b200c {
void bind_cuda_backend(py::module_&) {}
}
