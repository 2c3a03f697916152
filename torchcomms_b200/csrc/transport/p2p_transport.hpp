// One-sided point-to-point transport between processes of one NVSwitch box.
//
// A process registers memory (`TransportMemory`), hands the resulting
// `RemoteBuffer` (address, length, access key) to a peer by any channel, and the
// peer writes into or reads from it without the owner making a call:
//
//   * device memory on both sides, same host: the initiator maps the owner's
//     allocation through a CUDA IPC handle carried in the access key and issues
//     one peer copy on its own stream (NVLink, no host in the data path);
//   * everything else (host memory, allocations that cannot be exported, or
//     `B200COMMS_TRANSPORT_STAGED=1`): the bytes travel over the connection's
//     TCP socket and the owner's service thread places them, staging device
//     memory through a pinned bounce buffer in 4 MB pieces.
//
// Every request is checked by the owner against its registration table
// (unknown key, wrong nonce, range outside the registration -> error status, no
// bytes moved). Operations are asynchronous: they run on the transport's
// worker thread and complete a future.
//
// Parity: comms/torchcomms/transport/RdmaTransport.h (bind / connect / write /
// read, RdmaMemory and its views, RdmaRemoteBuffer) and
// StagedRdmaTransport.h (copy-through-staging variant). The reference moves
// the bytes with InfiniBand verbs between hosts; on one box the same API rides
// on NVLink peer copies, with the socket path as the staged variant.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../core/types.hpp"

namespace b200c {

enum TransportStatus : int {
  kTransportOk = 0,
  kTransportBadKey = 1,        // the owner does not know the key (or the nonce differs)
  kTransportOutOfRange = 2,    // [ptr, ptr + len) leaves the registration
  kTransportNotConnected = 3,
  kTransportIo = 4,            // socket error or peer went away
  kTransportCuda = 5,
  kTransportTimeout = 6,
  kTransportClosed = 7,        // the transport was closed with the operation queued
  kTransportSizeMismatch = 8,  // local view and remote buffer differ in length
};

B200C_API const char* transport_strerror(int status);

// What a peer needs to address registered memory. Plain data; picklable in Python.
struct RemoteBuffer {
  uint64_t ptr = 0;
  uint64_t len = 0;
  std::string access_key;
};

// Fields of an access key ("b2k1:<pid>:<id>:<nonce>:<device>:<base>:<len>:<ipc_off>:<ipc hex|->:<boot>").
struct B200C_API AccessKey {
  int64_t pid = 0;
  uint64_t id = 0;
  uint64_t nonce = 0;
  int device = -1;  // -1: host memory
  uint64_t base = 0;
  uint64_t len = 0;
  uint64_t ipc_offset = 0;  // base - start of the exported allocation
  std::string ipc_hex;      // empty: not exportable
  std::string boot_id;      // same value on two processes <=> same host
  static bool parse(const std::string& s, AccessKey* out);
  std::string str() const;
};

class B200C_API TransportMemory {
 public:
  // `alloc_base` is the start of the device allocation that contains `ptr`
  // (what a CUDA IPC handle exports); 0 means `ptr` itself.
  static std::shared_ptr<TransportMemory> create(void* ptr, size_t len, int device, uint64_t alloc_base = 0);
  ~TransportMemory();
  // Long-lived registration of a whole allocator segment. Registrations of ranges inside it share
  // its key (one export per segment instead of one per tensor); `unregister_segment` ends it.
  static void register_segment(void* base, size_t len, int device);
  static void unregister_segment(void* base);
  static size_t segment_count();
  TransportMemory(const TransportMemory&) = delete;
  TransportMemory& operator=(const TransportMemory&) = delete;

  void* data() const { return ptr_; }
  size_t size() const { return len_; }
  int device() const { return device_; }
  const std::string& access_key() const { return key_; }
  bool reused_registration() const { return reused_; }
  bool contains(const void* p, size_t n) const;
  RemoteBuffer remote_buffer() const { return RemoteBuffer{reinterpret_cast<uint64_t>(ptr_), len_, key_}; }
  RemoteBuffer remote_buffer(size_t offset, size_t length) const;

 private:
  TransportMemory() = default;
  void* ptr_ = nullptr;
  size_t len_ = 0;
  int device_ = -1;
  uint64_t id_ = 0;
  bool reused_ = false;
  std::string key_;
};

// A byte range of a registration; keeps the registration alive.
struct TransportView {
  std::shared_ptr<TransportMemory> mem;
  size_t offset = 0;
  size_t length = 0;
  void* data() const { return static_cast<char*>(mem->data()) + offset; }
  size_t size() const { return length; }
};

class B200C_API TransportFuture {
 public:
  bool done() const;
  // Blocks until completion or `timeout_ms` (< 0: forever); kTransportTimeout if it ran out.
  int wait(int64_t timeout_ms = -1) const;

 private:
  friend class P2pTransport;
  void complete(int status);
  mutable std::mutex mu_;
  mutable std::condition_variable cv_;
  bool done_ = false;
  int status_ = kTransportOk;
};

struct TransportCounters {
  uint64_t peer_copy_ops = 0, peer_copy_bytes = 0;  // CUDA IPC mapping + one device copy
  uint64_t socket_ops = 0, socket_bytes = 0;        // through the owner's service thread
  uint64_t served_ops = 0, served_bytes = 0;        // requests this side's service thread placed
  uint64_t rejected = 0;                            // requests this side refused
};

class B200C_API P2pTransport {
 public:
  explicit P2pTransport(int device);  // -1: host-only transport
  ~P2pTransport();
  P2pTransport(const P2pTransport&) = delete;
  P2pTransport& operator=(const P2pTransport&) = delete;

  static bool supported();
  // Opens the listening socket (once) and returns this side's address.
  std::string bind();
  // Connects to a peer's address; returns a TransportStatus.
  int connect(const std::string& peer_url);
  bool connected() const;
  std::shared_ptr<TransportFuture> write(const TransportView& local, const RemoteBuffer& remote);
  std::shared_ptr<TransportFuture> read(const TransportView& local, const RemoteBuffer& remote);
  TransportCounters counters() const;
  void close();
  int device() const { return device_; }

 private:
  struct Op {
    bool is_write;
    TransportView local;
    RemoteBuffer remote;
    std::shared_ptr<TransportFuture> fut;
  };
  struct Mapped {
    void* alloc_base = nullptr;
  };

  std::shared_ptr<TransportFuture> enqueue(bool is_write, const TransportView& local, const RemoteBuffer& remote);
  void worker_loop();
  void accept_loop();
  void serve(int fd);
  int run_op(const Op& op);
  int run_peer_copy(const Op& op, const AccessKey& key);
  int run_socket(const Op& op);
  int validate_remote(const RemoteBuffer& remote);

  const int device_;
  const bool force_staged_;
  const int io_timeout_s_;
  int listen_fd_ = -1;
  int client_fd_ = -1;
  std::string url_;
  std::string peer_boot_id_;
  int64_t peer_pid_ = 0;
  std::atomic<bool> closing_{false};
  std::atomic<bool> connected_{false};
  std::thread accept_thread_;
  std::thread worker_;
  std::vector<std::thread> servers_;
  std::vector<int> server_fds_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Op> queue_;
  std::unordered_map<std::string, Mapped> mapped_;  // access key -> opened IPC mapping
  std::unordered_map<std::string, bool> validated_; // access key + range already approved by the owner
  void* stream_ = nullptr;                          // cudaStream_t of the peer copies
  void* bounce_ = nullptr;                          // pinned staging of the socket path
  TransportCounters counters_;
};

} // namespace b200c
