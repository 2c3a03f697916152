// Hook-based observers: a flight recorder (bounded ring of per-collective
// entries, dumped as JSON in the layout PyTorch's fr_trace tooling reads) and
// a compact pipe-delimited collective log.
//
// Parity: comms/torchcomms/hooks/fr/FlightRecorder.hpp:59-200 (ring of 2000
// entries by default, TORCHCOMM_FR_BUFFER_SIZE, states scheduled / started /
// completed, dump_json / dump_file, registered as pre / post / abort hooks) and
// comms/torchcomms/hooks/clog/ClogHook.hpp:118-279 (signature de-duplication
// into correlation ids, events Q/S/E/W, graph replay lines).
#pragma once

#include <fstream>
#include <unordered_map>

#include "../core/comm.hpp"

namespace b200c {

class FlightRecorder : public std::enable_shared_from_this<FlightRecorder> {
 public:
  struct Entry {
    uint64_t record_id = 0;
    size_t op_id = 0;
    std::string comm_name;
    int rank = 0, world = 1;
    std::string op;
    uint64_t collective_seq = 0, p2p_seq = 0;
    bool is_p2p = false;
    std::vector<std::vector<int64_t>> in_sizes, out_sizes;
    std::vector<std::string> in_dtypes, out_dtypes;
    int64_t created_ns = 0, started_ns = 0, completed_ns = 0;
    std::string state = "scheduled";
    int64_t timeout_ms = 0;
    int64_t iteration = -1;  // trainer iteration at record time
    bool retired = false;
  };

  explicit FlightRecorder(size_t capacity = 0); // 0: TORCHCOMM_FR_BUFFER_SIZE or 2000
  // Registers pre, post and abort hooks on `comm`; the handles live as long
  // as the recorder or until detach().
  void attach(const std::shared_ptr<Comm>& comm);
  void detach();
  std::string dump_json(bool include_completed = true) const;
  // Writes dump_json() to `<prefix><rank>`; prefix from TORCHCOMM_FR_DUMP_TEMP_FILE,
  // then TORCH_FR_DUMP_TEMP_FILE, default /tmp/b200c_fr_trace_ . Returns the path.
  std::string dump_file(int rank, bool include_completed = true) const;
  size_t size() const;
  size_t capacity() const { return cap_; }
  std::vector<Entry> entries() const;
  void reset();

 private:
  void on_pre(const std::shared_ptr<Comm>& comm, OpName op, size_t op_id, const OpRecord& rec);
  void on_post(size_t op_id, const OpRecord& rec);
  void mark(uint64_t record_id, const char* state);

  size_t cap_;
  mutable std::mutex mu_;
  std::vector<Entry> ring_;
  uint64_t next_id_ = 0;
  std::unordered_map<size_t, uint64_t> op_to_record_;
  std::unordered_map<std::string, std::pair<uint64_t, uint64_t>> seq_; // comm -> (collective, p2p)
  std::vector<RemovableHandle> handles_;
  int last_rank_ = 0;
};

class CollectiveLog : public std::enable_shared_from_this<CollectiveLog> {
 public:
  // Lines go to `path`; an empty path keeps them in memory only.
  explicit CollectiveLog(const std::string& path = "");
  void attach(const std::shared_ptr<Comm>& comm);
  void detach();
  std::vector<std::string> lines() const;
  static std::string signature(const OpRecord& rec);

 private:
  void emit(const std::string& line);
  uint64_t correlation_id(const std::string& comm, const std::string& sig);

  mutable std::mutex mu_;
  std::ofstream file_;
  std::vector<std::string> lines_;
  std::unordered_map<std::string, uint64_t> sig_ids_;
  std::vector<RemovableHandle> handles_;
};

} // namespace b200c
