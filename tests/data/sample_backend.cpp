// Out-of-tree backend used by the factory test: built into its own shared
// library at test time, found through TORCHCOMMS_BACKEND_LIB_PATH_SAMPLE and
// loaded with dlopen. It derives from the in-tree no-transport backend and
// only changes its name and one operation, which is enough to prove that the
// ABI string, the loader table and the virtual interface line up.
#include "backends/cpu_backends.hpp"

namespace {

class SampleBackend final : public b200c::FakeBackend {
 public:
  std::string backend_name() const override { return "sample"; }
  b200c::WorkPtr all_reduce(at::Tensor& t, const b200c::ReduceOp& op, bool async_op, const b200c::OpOptions& o) override {
    t.add_(1);  // visible side effect so the test can tell this class ran
    return b200c::FakeBackend::all_reduce(t, op, async_op, o);
  }
};

const char* abi() { return b200c::kBackendAbiVersion; }
b200c::Backend* create() { return new SampleBackend(); }
void destroy(b200c::Backend* b) { delete b; }

b200c::DynamicBackendLoader g_loader{&abi, &create, &destroy};

} // namespace

extern "C" __attribute__((visibility("default"))) b200c::DynamicBackendLoader* b200c_create_backend_sample() {
  return &g_loader;
}
