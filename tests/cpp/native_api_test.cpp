// Unit tests of the native (C++) API, compiled into a small shared library by
// tests/test_native_cpp.py and run through one C entry point. They exercise what a
// C++ user links against: the transport classes, the configuration tiers, the work
// state machine, the factory with the fake backend, hook ordering.
//
// Modelled on comms/torchcomms/tests/unit/cpp (TorchCommFactoryTest,
// TorchCommOptionsTest, TorchCommHooksTest, TorchWorkTest), which use GoogleTest;
// here a failed check records its text and the test reports the first one.
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "core/comm.hpp"
#include "core/options.hpp"
#include "transport/p2p_transport.hpp"

using namespace b200c;

namespace {

std::vector<std::string> g_failures;

#define CHECK_THAT(cond)                                                                         \
  do {                                                                                           \
    if (!(cond)) {                                                                               \
      std::ostringstream o;                                                                      \
      o << __FILE__ << ":" << __LINE__ << ": " #cond;                                            \
      g_failures.push_back(o.str());                                                             \
    }                                                                                            \
  } while (0)

void test_transport_roundtrip() {
  P2pTransport a(-1), b(-1);
  const std::string ua = a.bind(), ub = b.bind();
  CHECK_THAT(ua.rfind("b200p2p://", 0) == 0);
  CHECK_THAT(a.connect(ub) == kTransportOk && b.connect(ua) == kTransportOk);
  std::vector<int> src(4096), dst(4096, 0);
  for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<int>(i * 7);
  auto msrc = TransportMemory::create(src.data(), src.size() * sizeof(int), -1);
  auto mdst = TransportMemory::create(dst.data(), dst.size() * sizeof(int), -1);
  CHECK_THAT(msrc->contains(src.data() + 10, 16) && !msrc->contains(dst.data(), 4));
  auto fut = a.write(TransportView{msrc, 0, msrc->size()}, mdst->remote_buffer());
  CHECK_THAT(fut->wait(10000) == kTransportOk && fut->done());
  CHECK_THAT(src == dst);
  // partial read back through the other side, into the middle of a buffer
  std::vector<int> back(4096, -1);
  auto mback = TransportMemory::create(back.data(), back.size() * sizeof(int), -1);
  CHECK_THAT(b.read(TransportView{mback, 1024 * sizeof(int), 512 * sizeof(int)}, msrc->remote_buffer(2048 * sizeof(int), 512 * sizeof(int)))
                 ->wait(10000) == kTransportOk);
  CHECK_THAT(back[1023] == -1 && back[1024] == src[2048] && back[1535] == src[2559] && back[1536] == -1);
  // refused: range outside the registration, unknown key
  RemoteBuffer bad = mdst->remote_buffer();
  bad.ptr += 64;
  CHECK_THAT(a.write(TransportView{msrc, 0, msrc->size()}, bad)->wait(10000) == kTransportOutOfRange);
  RemoteBuffer forged = mdst->remote_buffer();
  forged.access_key = "b2k1:1:1:1:-1:0:0:0:-:x";
  CHECK_THAT(a.write(TransportView{msrc, 0, 16}, forged)->wait(10000) == kTransportBadKey);
  CHECK_THAT(b.counters().rejected == 2 && a.counters().socket_ops == 1);
  AccessKey k;
  CHECK_THAT(AccessKey::parse(mdst->access_key(), &k) && k.device == -1 && k.len == dst.size() * sizeof(int) && k.str() == mdst->access_key());
  a.close();
  CHECK_THAT(a.write(TransportView{msrc, 0, 16}, mdst->remote_buffer())->wait(1000) == kTransportClosed);
  b.close();
  CHECK_THAT(std::string(transport_strerror(kTransportTimeout)) == "timed out");
}

void test_config_tiers(const char* tmp_dir) {
  const std::string path = std::string(tmp_dir) + "/native.conf";
  {
    std::ofstream f(path);
    f << "B200C_TEST_INT = 41\nB200C_TEST_FLAG=yes # trailing comment\n";
  }
  setenv("B200COMMS_CONF_FILE", path.c_str(), 1);
  unsetenv("B200C_TEST_INT");
  reload_config_file();
  CHECK_THAT(env_to_value<int>("B200C_TEST_INT", 7) == 41);
  CHECK_THAT(env_to_value<bool>("B200C_TEST_FLAG", false));
  CHECK_THAT(env_to_value<std::string>("B200C_TEST_ABSENT", "dflt") == "dflt");
  setenv("B200C_TEST_INT", "43", 1);
  CHECK_THAT(env_to_value<int>("B200C_TEST_INT", 7) == 43);
  setenv("B200C_TEST_INT", "4x", 1);
  bool threw = false;
  try {
    env_to_value<int>("B200C_TEST_INT", 7);
  } catch (const std::runtime_error&) {
    threw = true;
  }
  CHECK_THAT(threw);
  unsetenv("B200C_TEST_INT");
  bool seen = false;
  for (auto& k : knob_report()) seen = seen || (k[0] == "B200C_TEST_FLAG" && k[1] == "yes" && k[2] == "file");
  CHECK_THAT(seen);
  unsetenv("B200COMMS_CONF_FILE");
  reload_config_file();
  Hints h{{"n", "12"}, {"on", "true"}};
  CHECK_THAT(hint_or<int>(h, "n", 1) == 12 && hint_or<bool>(h, "on", false) && hint_or<int>(h, "missing", 5) == 5);
}

void test_factory_hooks_and_work() {
  CommOptions opts;
  opts.timeout = Millis(5000);
  auto comm = new_comm("fake", at::Device(at::kCPU), "native_cpp", opts);
  CHECK_THAT(comm->get_rank() == 0 && comm->get_size() == 1 && comm->get_backend() == "fake");
  std::vector<std::string> order;
  size_t pre_id = 0, post_id = 0;
  auto h1 = comm->register_pre_hook([&](OpName op, size_t id, const OpRecord&) {
    order.push_back("pre");
    pre_id = id;
    CHECK_THAT(op == OpName::all_reduce);
  });
  RemovableHandle h2 = comm->register_post_hook([&](size_t id, const OpRecord&) {
    order.push_back("post");
    post_id = id;
  });
  at::Tensor t = at::ones({8});
  WorkPtr w = comm->all_reduce(t, ReduceOp(RedOpType::SUM), true, OpOptions{});
  CHECK_THAT(order.size() == 2 && order[0] == "pre" && order[1] == "post" && pre_id == post_id);
  int ends = 0;
  w->on_end([&] { ++ends; });
  w->wait();
  CHECK_THAT(w->status() == WorkStatus::COMPLETED && ends == 1);
  const size_t first = pre_id;
  h1.remove();
  h1.remove();  // removing twice is harmless
  comm->all_reduce(t, ReduceOp(RedOpType::SUM), false, OpOptions{});
  CHECK_THAT(order.size() == 3 && order.back() == "post" && post_id > first);
  bool threw = false;
  try {
    comm->send(t, 3, false, OpOptions{});
  } catch (const std::exception&) {
    threw = true;
  }
  CHECK_THAT(threw);  // rank out of range
  auto dumps = comm_dump_all();
  CHECK_THAT(dumps.count("native_cpp") == 1 && dumps["native_cpp"]["backend"] == "fake");
  comm->finalize();
  threw = false;
  try {
    new_comm("no_such_backend", at::Device(at::kCPU), "x", opts);
  } catch (const std::exception&) {
    threw = true;
  }
  CHECK_THAT(threw);
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int b200c_run_native_tests(const char* tmp_dir, char* message, int capacity) {
  g_failures.clear();
  try {
    test_transport_roundtrip();
    test_config_tiers(tmp_dir);
    test_factory_hooks_and_work();
  } catch (const std::exception& e) {
    g_failures.push_back(std::string("exception: ") + e.what());
  }
  std::string all;
  for (auto& f : g_failures) all += f + "\n";
  std::strncpy(message, all.c_str(), static_cast<size_t>(capacity) - 1);
  message[capacity - 1] = '\0';
  return static_cast<int>(g_failures.size());
}
