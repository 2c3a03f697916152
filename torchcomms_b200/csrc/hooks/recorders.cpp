// Flight recorder and collective log.
#include "recorders.hpp"

#include <chrono>
#include <sstream>

namespace b200c {

namespace {

int64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::system_clock::now().time_since_epoch())
      .count();
}

std::string json_escape(const std::string& s) {
  std::string out;
  out.reserve(s.size() + 2);
  for (char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\t': out += "\\t"; break;
      default: out += c;
    }
  }
  return out;
}

void json_sizes(std::ostringstream& os, const std::vector<std::vector<int64_t>>& v) {
  os << "[";
  for (size_t i = 0; i < v.size(); ++i) {
    os << (i ? "," : "") << "[";
    for (size_t j = 0; j < v[i].size(); ++j) {
      os << (j ? "," : "") << v[i][j];
    }
    os << "]";
  }
  os << "]";
}

void json_strings(std::ostringstream& os, const std::vector<std::string>& v) {
  os << "[";
  for (size_t i = 0; i < v.size(); ++i) {
    os << (i ? "," : "") << "\"" << json_escape(v[i]) << "\"";
  }
  os << "]";
}

void describe(const std::vector<at::Tensor>& ts, std::vector<std::vector<int64_t>>& sizes,
              std::vector<std::string>& dtypes) {
  for (auto& t : ts) {
    if (t.defined()) {
      sizes.push_back(t.sizes().vec());
      dtypes.emplace_back(c10::toString(t.scalar_type()));
    }
  }
}

bool is_p2p_op(OpName op) {
  return op == OpName::send || op == OpName::recv || op == OpName::batch_op_issue;
}

} // namespace

// ------------------------------------------------------- FlightRecorder ----

FlightRecorder::FlightRecorder(size_t capacity) {
  cap_ = capacity ? capacity : env_to_value<size_t>("TORCHCOMM_FR_BUFFER_SIZE", 2000);
  if (cap_ == 0) {
    cap_ = 1;
  }
  ring_.reserve(std::min<size_t>(cap_, 4096));
}

void FlightRecorder::attach(const std::shared_ptr<Comm>& comm) {
  std::weak_ptr<FlightRecorder> weak = shared_from_this();
  std::weak_ptr<Comm> wcomm = comm;
  last_rank_ = comm->get_rank();
  handles_.push_back(comm->register_pre_hook([weak, wcomm](OpName op, size_t id, const OpRecord& rec) {
    auto self = weak.lock();
    auto c = wcomm.lock();
    if (self && c) {
      self->on_pre(c, op, id, rec);
    }
  }));
  handles_.push_back(comm->register_post_hook([weak](size_t id, const OpRecord& rec) {
    if (auto self = weak.lock()) {
      self->on_post(id, rec);
    }
  }));
  const int rank = comm->get_rank();
  handles_.push_back(comm->register_abort_hook([weak, rank]() {
    if (auto self = weak.lock()) {
      self->dump_file(rank);
    }
  }));
}

void FlightRecorder::detach() {
  for (auto& h : handles_) {
    h.remove();
  }
  handles_.clear();
}

void FlightRecorder::on_pre(const std::shared_ptr<Comm>& comm, OpName op, size_t op_id, const OpRecord& rec) {
  Entry e;
  e.op_id = op_id;
  e.comm_name = comm->get_name();
  e.rank = comm->get_rank();
  e.world = comm->get_size();
  e.op = std::string(op_name(op));
  e.is_p2p = is_p2p_op(op);
  describe(rec.inputs, e.in_sizes, e.in_dtypes);
  describe(rec.outputs, e.out_sizes, e.out_dtypes);
  for (auto& p : rec.p2p_ops) {
    std::vector<at::Tensor> one{p.tensor};
    if (p.kind == P2PKind::SEND) {
      describe(one, e.in_sizes, e.in_dtypes);
    } else {
      describe(one, e.out_sizes, e.out_dtypes);
    }
  }
  e.created_ns = now_ns();
  e.iteration = trainer_iteration();
  e.timeout_ms = comm->get_options().timeout.count();
  std::lock_guard<std::mutex> g(mu_);
  auto& seq = seq_[e.comm_name];
  if (e.is_p2p) {
    e.p2p_seq = ++seq.second;
    e.collective_seq = seq.first;
  } else {
    e.collective_seq = ++seq.first;
    e.p2p_seq = seq.second;
  }
  e.record_id = next_id_++;
  if (ring_.size() < cap_) {
    ring_.push_back(std::move(e));
  } else {
    Entry& slot = ring_[e.record_id % cap_];
    op_to_record_.erase(slot.op_id);
    slot = std::move(e);
  }
  op_to_record_[op_id] = next_id_ - 1;
}

void FlightRecorder::mark(uint64_t record_id, const char* state) {
  std::lock_guard<std::mutex> g(mu_);
  if (ring_.empty()) {
    return;
  }
  Entry& e = ring_[record_id % cap_ < ring_.size() ? record_id % cap_ : 0];
  if (e.record_id != record_id) {
    return; // overwritten meanwhile
  }
  const std::string s(state);
  if (s == "started") {
    if (e.state == "scheduled") {
      e.state = s;
      e.started_ns = now_ns();
    }
  } else {
    e.state = s;
    e.completed_ns = now_ns();
    if (e.started_ns == 0) {
      e.started_ns = e.completed_ns;
    }
    e.retired = true;
  }
}

void FlightRecorder::on_post(size_t op_id, const OpRecord& rec) {
  uint64_t record_id;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = op_to_record_.find(op_id);
    if (it == op_to_record_.end()) {
      return;
    }
    record_id = it->second;
    op_to_record_.erase(it);
  }
  auto work = rec.work.lock();
  if (!work) {
    mark(record_id, "completed");
    return;
  }
  std::weak_ptr<FlightRecorder> weak = shared_from_this();
  work->on_start([weak, record_id]() {
    if (auto self = weak.lock()) {
      self->mark(record_id, "started");
    }
  });
  c10::weak_intrusive_ptr<Work> wwork(work);
  work->on_end([weak, record_id, wwork]() {
    if (auto self = weak.lock()) {
      auto w = wwork.lock();
      const char* st = "completed";
      if (w && w->status() == WorkStatus::TIMEDOUT) {
        st = "timed_out";
      } else if (w && w->status() == WorkStatus::ERROR) {
        st = "failed";
      }
      self->mark(record_id, st);
    }
  });
}

size_t FlightRecorder::size() const {
  std::lock_guard<std::mutex> g(mu_);
  return ring_.size();
}

std::vector<FlightRecorder::Entry> FlightRecorder::entries() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<Entry> out = ring_;
  std::sort(out.begin(), out.end(), [](const Entry& a, const Entry& b) { return a.record_id < b.record_id; });
  return out;
}

void FlightRecorder::reset() {
  std::lock_guard<std::mutex> g(mu_);
  ring_.clear();
  op_to_record_.clear();
  seq_.clear();
  next_id_ = 0;
}

std::string FlightRecorder::dump_json(bool include_completed) const {
  const auto all = entries();
  std::ostringstream os;
  os << "{\"version\":\"2.10\",\"comm_lib_version\":\"" << kBackendAbiVersion << "\",\"rank\":" << last_rank_;
  // Per-communicator configuration and progress, as fr_trace expects.
  std::unordered_map<std::string, const Entry*> last;
  for (auto& e : all) {
    last[e.comm_name] = &e;
  }
  os << ",\"pg_config\":{";
  bool first = true;
  for (auto& kv : last) {
    os << (first ? "" : ",") << "\"" << json_escape(kv.first) << "\":{\"name\":\"" << json_escape(kv.first)
       << "\",\"desc\":\"torchcomms_b200\",\"ranks\":\"[0.." << (kv.second->world - 1) << "]\"}";
    first = false;
  }
  os << "},\"pg_status\":{";
  first = true;
  for (auto& kv : last) {
    uint64_t enq = 0, started = 0, done = 0;
    for (auto& e : all) {
      if (e.comm_name != kv.first) continue;
      enq = std::max(enq, e.collective_seq);
      if (e.state != "scheduled") started = std::max(started, e.collective_seq);
      if (e.retired) done = std::max(done, e.collective_seq);
    }
    os << (first ? "" : ",") << "\"" << json_escape(kv.first) << "\":{\"last_enqueued_collective\":" << enq
       << ",\"last_started_collective\":" << started << ",\"last_completed_collective\":" << done << "}";
    first = false;
  }
  os << "},\"entries\":[";
  first = true;
  for (auto& e : all) {
    if (!include_completed && e.retired) {
      continue;
    }
    os << (first ? "" : ",") << "{\"record_id\":" << e.record_id << ",\"pg_id\":0,\"process_group\":[\""
       << json_escape(e.comm_name) << "\",\"torchcomms_b200\"],\"collective_seq_id\":" << e.collective_seq
       << ",\"p2p_seq_id\":" << e.p2p_seq << ",\"op_id\":" << e.op_id << ",\"profiling_name\":\"b200c:"
       << e.op << "\",\"time_created_ns\":" << e.created_ns << ",\"input_sizes\":";
    json_sizes(os, e.in_sizes);
    os << ",\"input_dtypes\":";
    json_strings(os, e.in_dtypes);
    os << ",\"output_sizes\":";
    json_sizes(os, e.out_sizes);
    os << ",\"output_dtypes\":";
    json_strings(os, e.out_dtypes);
    os << ",\"state\":\"" << e.state << "\",\"time_discovered_started_ns\":";
    if (e.started_ns) os << e.started_ns; else os << "null";
    os << ",\"time_discovered_completed_ns\":";
    if (e.completed_ns) os << e.completed_ns; else os << "null";
    os << ",\"retired\":" << (e.retired ? "true" : "false") << ",\"timeout_ms\":" << e.timeout_ms
       << ",\"is_p2p\":" << (e.is_p2p ? "true" : "false") << ",\"iteration\":" << e.iteration << ",\"frames\":[]}";
    first = false;
  }
  os << "]}";
  return os.str();
}

std::string FlightRecorder::dump_file(int rank, bool include_completed) const {
  std::string prefix = env_to_value<std::string>("TORCHCOMM_FR_DUMP_TEMP_FILE", "");
  if (prefix.empty()) {
    prefix = env_to_value<std::string>("TORCH_FR_DUMP_TEMP_FILE", "/tmp/b200c_fr_trace_");
  }
  const std::string path = prefix + std::to_string(rank);
  std::ofstream f(path, std::ios::trunc);
  f << dump_json(include_completed);
  return path;
}

// -------------------------------------------------------- CollectiveLog ----

CollectiveLog::CollectiveLog(const std::string& path) {
  if (!path.empty()) {
    file_.open(path, std::ios::app);
  }
  emit("V|1|b200c-clog");
}

void CollectiveLog::emit(const std::string& line) {
  std::lock_guard<std::mutex> g(mu_);
  lines_.push_back(line);
  if (file_.is_open()) {
    file_ << line << '\n';
    file_.flush();
  }
}

std::vector<std::string> CollectiveLog::lines() const {
  std::lock_guard<std::mutex> g(mu_);
  return lines_;
}

std::string CollectiveLog::signature(const OpRecord& rec) {
  std::ostringstream os;
  os << op_name(rec.op);
  auto add = [&os](const char* tag, const std::vector<at::Tensor>& ts) {
    os << ";" << tag << "=";
    for (size_t i = 0; i < ts.size(); ++i) {
      if (!ts[i].defined()) continue;
      os << (i ? "," : "") << c10::toString(ts[i].scalar_type()) << "[";
      for (int64_t d = 0; d < ts[i].dim(); ++d) {
        os << (d ? "x" : "") << ts[i].size(d);
      }
      os << "]";
    }
  };
  add("in", rec.inputs);
  add("out", rec.outputs);
  if (rec.root >= 0) os << ";root=" << rec.root;
  if (rec.red_op) os << ";red=" << red_op_name(*rec.red_op);
  os << ";async=" << (rec.async_op ? 1 : 0);
  return os.str();
}

uint64_t CollectiveLog::correlation_id(const std::string& comm, const std::string& sig) {
  const std::string key = comm + "#" + sig;
  bool fresh = false;
  uint64_t id;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = sig_ids_.find(key);
    if (it == sig_ids_.end()) {
      id = sig_ids_.size();
      sig_ids_.emplace(key, id);
      fresh = true;
    } else {
      id = it->second;
    }
  }
  if (fresh) {
    emit("SIG|" + std::to_string(id) + "|" + comm + "|" + sig);
  }
  return id;
}

void CollectiveLog::attach(const std::shared_ptr<Comm>& comm) {
  std::weak_ptr<CollectiveLog> weak = shared_from_this();
  const std::string name = comm->get_name();
  const int rank = comm->get_rank();
  auto line = [name, rank](char ev, size_t op_id, uint64_t corr) {
    std::ostringstream os;
    os << ev << "|" << now_ns() << "|" << name << "|" << rank << "|" << op_id << "|" << corr;
    return os.str();
  };
  // Pre hook: Q (queued). The correlation id travels to the post hook by op id.
  auto pending = std::make_shared<std::unordered_map<size_t, uint64_t>>();
  auto pending_mu = std::make_shared<std::mutex>();
  handles_.push_back(comm->register_pre_hook([weak, name, line, pending, pending_mu](OpName, size_t id, const OpRecord& rec) {
    auto self = weak.lock();
    if (!self) return;
    const uint64_t corr = self->correlation_id(name, signature(rec));
    {
      std::lock_guard<std::mutex> g(*pending_mu);
      (*pending)[id] = corr;
    }
    self->emit(line('Q', id, corr));
  }));
  handles_.push_back(comm->register_post_hook([weak, line, pending, pending_mu](size_t id, const OpRecord& rec) {
    auto self = weak.lock();
    if (!self) return;
    uint64_t corr = 0;
    {
      std::lock_guard<std::mutex> g(*pending_mu);
      auto it = pending->find(id);
      if (it != pending->end()) {
        corr = it->second;
        pending->erase(it);
      }
    }
    auto work = rec.work.lock();
    if (!work) {
      return;
    }
    work->on_start([weak, line, id, corr]() {
      if (auto s = weak.lock()) s->emit(line('S', id, corr));
    });
    work->on_end([weak, line, id, corr]() {
      if (auto s = weak.lock()) s->emit(line('E', id, corr));
    });
    work->on_wait_post([weak, line, id, corr]() {
      if (auto s = weak.lock()) s->emit(line('W', id, corr));
    });
  }));
  handles_.push_back(comm->register_graph_replay_hook(
      [weak, name](uint64_t gid, uint64_t rid, uintptr_t, size_t idx, char ev) {
        if (auto s = weak.lock()) {
          std::ostringstream os;
          os << "G|" << gid << "|R|" << rid << "|C|" << idx << "|" << ev << "|" << name;
          s->emit(os.str());
        }
      }));
}

void CollectiveLog::detach() {
  for (auto& h : handles_) {
    h.remove();
  }
  handles_.clear();
}

} // namespace b200c
