// Implementation of the value types, option parsing, logging and Work.
#include <torch/csrc/distributed/c10d/PrefixStore.hpp>
#include <torch/csrc/distributed/c10d/TCPStore.hpp>

#include <algorithm>
#include <cctype>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <thread>
#include <unordered_map>

#include "logging.hpp"
#include "options.hpp"
#include "work.hpp"

namespace b200c {

// ---------------------------------------------------------------- types ----

const char* red_op_name(RedOpType t) {
  switch (t) {
    case RedOpType::SUM: return "SUM";
    case RedOpType::PRODUCT: return "PRODUCT";
    case RedOpType::MIN: return "MIN";
    case RedOpType::MAX: return "MAX";
    case RedOpType::BAND: return "BAND";
    case RedOpType::BOR: return "BOR";
    case RedOpType::BXOR: return "BXOR";
    case RedOpType::PREMUL_SUM: return "PREMUL_SUM";
    case RedOpType::AVG: return "AVG";
  }
  return "?";
}

double ReduceOp::factor_as_double() const {
  if (!factor_) {
    return 1.0;
  }
  if (std::holds_alternative<double>(*factor_)) {
    return std::get<double>(*factor_);
  }
  return std::get<at::Tensor>(*factor_).to(at::kCPU, at::kDouble).item<double>();
}

const char* work_status_name(WorkStatus s) {
  switch (s) {
    case WorkStatus::NOT_STARTED: return "NOT_STARTED";
    case WorkStatus::INPROGRESS: return "INPROGRESS";
    case WorkStatus::COMPLETED: return "COMPLETED";
    case WorkStatus::TIMEDOUT: return "TIMEDOUT";
    case WorkStatus::ERROR: return "ERROR";
  }
  return "?";
}

std::string_view op_name(OpName op) {
  static constexpr std::string_view names[] = {
      "send", "recv", "broadcast", "all_reduce", "reduce", "all_gather",
      "all_gather_v", "all_gather_single", "reduce_scatter", "reduce_scatter_v",
      "reduce_scatter_single", "all_to_all_single", "all_to_all_v_single",
      "all_to_all", "barrier", "scatter", "gather", "gather_single", "split",
      "new_window", "batch_op_issue", "finalize"};
  const auto i = static_cast<size_t>(op);
  return i < sizeof(names) / sizeof(names[0]) ? names[i] : std::string_view("unknown");
}

// -------------------------------------------------------------- options ----

bool parse_bool(std::string_view text) {
  std::string s(text);
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
  if (s == "1" || s == "true" || s == "yes" || s == "on" || s == "y" || s == "t") {
    return true;
  }
  if (s == "0" || s == "false" || s == "no" || s == "off" || s == "n" || s == "f") {
    return false;
  }
  throw std::runtime_error("cannot parse '" + s + "' as a boolean");
}

namespace {

struct ConfigFile {
  std::mutex mu;
  bool loaded = false;
  std::unordered_map<std::string, std::string> values;
  std::map<std::string, std::pair<std::string, std::string>> knobs;  // key -> (value, source)
};

ConfigFile& config_file() {
  static ConfigFile* c = new ConfigFile();
  return *c;
}

std::string trimmed(const std::string& s) {
  const size_t a = s.find_first_not_of(" \t\r\n");
  if (a == std::string::npos) {
    return "";
  }
  const size_t b = s.find_last_not_of(" \t\r\n");
  return s.substr(a, b - a + 1);
}

}  // namespace

const char* config_raw(const char* key, const char** source) {
  const char* env = std::getenv(key);
  if (env != nullptr && *env != '\0') {
    if (source) *source = "env";
    return env;
  }
  ConfigFile& c = config_file();
  std::lock_guard<std::mutex> g(c.mu);
  if (!c.loaded) {
    c.loaded = true;
    c.values.clear();
    const char* path = std::getenv("B200COMMS_CONF_FILE");
    std::ifstream f(path && *path ? path : "/etc/b200comms.conf");
    std::string line;
    while (f && std::getline(f, line)) {
      const size_t hash = line.find('#');
      if (hash != std::string::npos) line.erase(hash);
      const size_t eq = line.find('=');
      if (eq == std::string::npos) continue;
      const std::string k = trimmed(line.substr(0, eq)), v = trimmed(line.substr(eq + 1));
      if (!k.empty()) c.values[k] = v;
    }
  }
  auto it = c.values.find(key);
  if (it == c.values.end() || it->second.empty()) {
    return nullptr;
  }
  if (source) *source = "file";
  return it->second.c_str();  // stable until reload_config_file()
}

void reload_config_file() {
  ConfigFile& c = config_file();
  std::lock_guard<std::mutex> g(c.mu);
  c.loaded = false;
}

void note_knob(const char* key, const std::string& value, const char* source) {
  ConfigFile& c = config_file();
  std::lock_guard<std::mutex> g(c.mu);
  c.knobs[key] = {value, source};
}

std::vector<std::array<std::string, 3>> knob_report() {
  ConfigFile& c = config_file();
  std::lock_guard<std::mutex> g(c.mu);
  std::vector<std::array<std::string, 3>> out;
  for (auto& kv : c.knobs) {
    out.push_back({kv.first, kv.second.first, kv.second.second});
  }
  return out;
}

CommOptions::CommOptions()
    : abort_process_on_timeout_or_error(env_to_value<bool>("TORCHCOMM_ABORT_ON_ERROR", true)),
      timeout(Millis(static_cast<int64_t>(
          env_to_value<double>("TORCHCOMM_TIMEOUT_SECONDS", kDefaultTimeout.count() / 1000.0) * 1000.0))) {}

namespace {

bool probe_pair(const char* rank_key, const char* size_key, int& rank, int& size) {
  const int r = env_to_value<int>(rank_key, -1);
  const int s = env_to_value<int>(size_key, -1);
  if (r >= 0 && s > 0) {
    rank = r;
    size = s;
    return true;
  }
  return false;
}

} // namespace

std::pair<int, int> query_ranksize() {
  std::string method = env_to_value<std::string>("TORCHCOMM_BOOTSTRAP_RANKSIZE_QUERY_METHOD", "auto");
  std::transform(method.begin(), method.end(), method.begin(), [](unsigned char c) { return std::tolower(c); });
  struct Source {
    const char* tag;
    const char* rank_key;
    const char* size_key;
  };
  static const Source sources[] = {
      {"torchcomm", "TORCHCOMM_RANK", "TORCHCOMM_SIZE"},
      {"ompi", "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE"},
      {"pmi", "PMI_RANK", "PMI_SIZE"},
      {"pals", "PALS_RANKID", "PALS_SIZE"},
      {"torchrun", "RANK", "WORLD_SIZE"},
  };
  int rank = -1, size = -1;
  for (const auto& src : sources) {
    if (method != "auto" && method != src.tag) {
      continue;
    }
    if (probe_pair(src.rank_key, src.size_key, rank, size)) {
      return {rank, size};
    }
  }
  throw std::runtime_error(
      "cannot determine rank and world size (method '" + method +
      "'): set TORCHCOMM_RANK and TORCHCOMM_SIZE, or launch with torchrun / mpirun");
}

c10::intrusive_ptr<c10d::Store> create_prefix_store(
    const std::string& prefix, int rank, int world_size, Millis timeout) {
  const std::string host = env_to_value<std::string>("MASTER_ADDR", "");
  const int port = env_to_value<int>("MASTER_PORT", -1);
  if (host.empty() || port < 0) {
    throw std::runtime_error(
        "no store was passed to new_comm and MASTER_ADDR / MASTER_PORT are not set");
  }
  c10d::TCPStoreOptions o;
  o.port = static_cast<uint16_t>(port);
  o.isServer = (rank == 0);
  o.numWorkers = world_size;
  o.waitWorkers = false;
  o.timeout = timeout;
  o.multiTenant = true; // several communicators of a process share one listening socket
  o.useLibUV = true;
  auto tcp = c10::make_intrusive<c10d::TCPStore>(host, o);
  return c10::make_intrusive<c10d::PrefixStore>(prefix, tcp);
}

c10::intrusive_ptr<c10d::Store> dup_prefix_store(
    const std::string& prefix, const c10::intrusive_ptr<c10d::Store>& bootstrap, Millis timeout) {
  const std::string host = env_to_value<std::string>("MASTER_ADDR", "");
  if (host.empty()) {
    throw std::runtime_error("dup_prefix_store: MASTER_ADDR is not set");
  }
  const int rank = query_ranksize().first;
  const std::string key = prefix + "/dup_store_port";
  c10d::TCPStoreOptions o;
  o.waitWorkers = false;
  o.useLibUV = true;
  o.timeout = timeout;
  c10::intrusive_ptr<c10d::TCPStore> tcp;
  if (rank == 0) {
    o.port = 0;  // the system picks a free port
    o.isServer = true;
    tcp = c10::make_intrusive<c10d::TCPStore>(host, o);
    store_set_string(*bootstrap, key, std::to_string(tcp->getPort()));
  } else {
    bootstrap->wait({key}, timeout);
    o.port = static_cast<uint16_t>(std::stoi(store_get_string(*bootstrap, key)));
    o.isServer = false;
    tcp = c10::make_intrusive<c10d::TCPStore>(host, o);
  }
  return c10::make_intrusive<c10d::PrefixStore>(prefix, tcp);
}

c10::intrusive_ptr<c10d::Store> scoped_store(
    const c10::intrusive_ptr<c10d::Store>& base, const std::string& prefix) {
  return c10::make_intrusive<c10d::PrefixStore>(prefix, base);
}

void store_set_string(c10d::Store& s, const std::string& key, const std::string& v) {
  s.set(key, std::vector<uint8_t>(v.begin(), v.end()));
}

std::string store_get_string(c10d::Store& s, const std::string& key) {
  auto raw = s.get(key);
  return std::string(raw.begin(), raw.end());
}

void store_barrier(c10d::Store& s, const std::string& key, int rank, int world, Millis timeout) {
  (void)rank;
  const int64_t arrived = s.add(key + "/count", 1);
  if (arrived == world) {
    store_set_string(s, key + "/done", "1");
  }
  s.wait({key + "/done"}, timeout);
}

// -------------------------------------------------------------- logging ----

Logger::Logger() {
  std::string lvl = env_to_value<std::string>("B200COMMS_LOG_LEVEL", "warn");
  std::transform(lvl.begin(), lvl.end(), lvl.begin(), [](unsigned char c) { return std::tolower(c); });
  if (lvl == "error") level_ = 0;
  else if (lvl == "info") level_ = 2;
  else if (lvl == "debug") level_ = 3;
  else level_ = 1;
}

Logger& Logger::get() {
  static Logger* inst = new Logger(); // leaked on purpose: usable during static destruction
  return *inst;
}

void Logger::write(LogLevel lvl, const std::string& who, const std::string& msg) {
  static const char* tags[] = {"E", "W", "I", "D"};
  const auto now = std::chrono::duration_cast<std::chrono::milliseconds>(
                       std::chrono::system_clock::now().time_since_epoch())
                       .count();
  std::ostringstream line;
  line << "[b200c " << tags[static_cast<int>(lvl)] << " " << now << "][" << who << "] " << msg;
  const std::string text = line.str();
  {
    std::lock_guard<std::mutex> g(mu_);
    ring_.push_back(text);
    if (ring_.size() > kRingCap) {
      ring_.pop_front();
    }
  }
  std::fprintf(stderr, "%s\n", text.c_str());
}

std::vector<std::string> Logger::recent() const {
  std::lock_guard<std::mutex> g(mu_);
  return {ring_.begin(), ring_.end()};
}

// ----------------------------------------------------------------- work ----

void Work::fire(std::vector<Hook>& hooks) {
  // Called with mu_ held by the caller having moved the list out.
  for (auto& h : hooks) {
    if (h) {
      h();
    }
  }
}

void Work::set_status(WorkStatus s) {
  std::vector<Hook> to_start, to_end;
  {
    std::lock_guard<std::mutex> g(mu_);
    const WorkStatus prev = status_.load(std::memory_order_relaxed);
    const bool prev_terminal = prev == WorkStatus::COMPLETED || prev == WorkStatus::TIMEDOUT ||
        prev == WorkStatus::ERROR;
    if (prev_terminal && s != prev && s != WorkStatus::ERROR && s != WorkStatus::TIMEDOUT) {
      return; // terminal states only escalate to failures
    }
    status_.store(s, std::memory_order_release);
    if (s != WorkStatus::NOT_STARTED && !started_) {
      started_ = true;
      to_start.swap(start_hooks_);
    }
    const bool terminal = s == WorkStatus::COMPLETED || s == WorkStatus::TIMEDOUT || s == WorkStatus::ERROR;
    if (terminal && !ended_) {
      ended_ = true;
      to_end.swap(end_hooks_);
    }
  }
  fire(to_start);
  fire(to_end);
}

void Work::on_start(Hook h) {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!started_) {
      start_hooks_.push_back(std::move(h));
      return;
    }
  }
  h();
}

void Work::on_end(Hook h) {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!ended_) {
      end_hooks_.push_back(std::move(h));
      return;
    }
  }
  h();
}

void Work::on_wait_pre(Hook h) {
  std::lock_guard<std::mutex> g(mu_);
  wait_pre_hooks_.push_back(std::move(h));
}

void Work::on_wait_post(Hook h) {
  std::lock_guard<std::mutex> g(mu_);
  wait_post_hooks_.push_back(std::move(h));
}

void Work::wait() {
  std::vector<Hook> pre, post;
  {
    std::lock_guard<std::mutex> g(mu_);
    pre = wait_pre_hooks_;
    post = wait_post_hooks_;
  }
  fire(pre);
  do_wait();
  fire(post);
  const WorkStatus s = status();
  if (s == WorkStatus::TIMEDOUT) {
    throw std::runtime_error("operation timed out" + (error().empty() ? "" : ": " + error()));
  }
  if (s == WorkStatus::ERROR) {
    throw std::runtime_error("operation failed" + (error().empty() ? "" : ": " + error()));
  }
}

void Work::wait_blocking() {
  std::vector<Hook> pre, post;
  {
    std::lock_guard<std::mutex> g(mu_);
    pre = wait_pre_hooks_;
    post = wait_post_hooks_;
  }
  fire(pre);
  do_wait_blocking();
  fire(post);
  const WorkStatus s = status();
  if (s == WorkStatus::TIMEDOUT) {
    throw std::runtime_error("operation timed out" + (error().empty() ? "" : ": " + error()));
  }
  if (s == WorkStatus::ERROR) {
    throw std::runtime_error("operation failed" + (error().empty() ? "" : ": " + error()));
  }
}

std::string Work::error() const {
  std::lock_guard<std::mutex> g(mu_);
  return error_;
}

void Work::set_error(std::string msg) {
  std::lock_guard<std::mutex> g(mu_);
  error_ = std::move(msg);
}

ThreadWork::ThreadWork(std::function<void()> fn, Millis timeout) {
  set_timeout(timeout);
  set_status(WorkStatus::INPROGRESS);
  fut_ = std::async(std::launch::async, [this, fn = std::move(fn)]() {
    try {
      fn();
      set_status(WorkStatus::COMPLETED);
    } catch (const std::exception& e) {
      set_error(e.what());
      set_status(WorkStatus::ERROR);
    }
  });
}

ThreadWork::~ThreadWork() {
  if (fut_.valid()) {
    fut_.wait();
  }
}

void ThreadWork::do_wait() {
  if (!fut_.valid()) {
    return;
  }
  const Millis t = timeout();
  if (t == kNoTimeout) {
    fut_.wait();
    return;
  }
  if (fut_.wait_for(t) == std::future_status::timeout) {
    set_error("host thread did not finish within " + std::to_string(t.count()) + " ms");
    set_status(WorkStatus::TIMEDOUT);
  }
}

} // namespace b200c
