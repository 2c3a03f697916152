// See p2p_transport.hpp.
#include "p2p_transport.hpp"

#include <arpa/inet.h>
#include <cuda_runtime.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <random>
#include <sstream>
#include <stdexcept>

namespace b200c {

namespace {

constexpr uint32_t kMagic = 0x62327031;  // "b2p1"
constexpr size_t kBounceBytes = 4u << 20;
enum WireOp : uint32_t { kOpHello = 1, kOpWrite = 2, kOpRead = 3, kOpValidate = 4 };

struct WireHeader {
  uint32_t magic;
  uint32_t op;
  uint64_t ptr;
  uint64_t len;
  uint32_t key_len;
  uint32_t reserved;
};

struct Registration {
  uint64_t id = 0;
  uint64_t nonce = 0;
  uint64_t base = 0;
  uint64_t len = 0;
  int device = -1;
  int refs = 0;
  bool segment = false;  // a whole allocator segment; ranges inside it share its key
  std::string key;       // empty until first use (segments)
};

// Process-wide table of registered ranges; any transport's service thread answers for all of them.
struct Registry {
  std::mutex mu;
  std::unordered_map<uint64_t, Registration> by_id;
  uint64_t next_id = 1;
  static Registry& get() {
    static Registry* r = new Registry();  // never destroyed: service threads may outlive static teardown
    return *r;
  }
};

std::string env_str(const char* name, const char* dflt) {
  const char* v = std::getenv(name);
  return v && *v ? std::string(v) : std::string(dflt);
}

const std::string& boot_id() {
  static const std::string id = [] {
    std::ifstream f("/proc/sys/kernel/random/boot_id");
    std::string s;
    if (f && std::getline(f, s) && !s.empty()) {
      return s;
    }
    char host[256] = {0};
    gethostname(host, sizeof(host) - 1);
    return std::string(host);
  }();
  return id;
}

std::string to_hex(const void* p, size_t n) {
  static const char* d = "0123456789abcdef";
  const unsigned char* b = static_cast<const unsigned char*>(p);
  std::string s(n * 2, '0');
  for (size_t i = 0; i < n; ++i) {
    s[2 * i] = d[b[i] >> 4];
    s[2 * i + 1] = d[b[i] & 15];
  }
  return s;
}

bool from_hex(const std::string& s, void* out, size_t n) {
  if (s.size() != 2 * n) {
    return false;
  }
  auto val = [](char c) -> int {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'f') return c - 'a' + 10;
    return -1;
  };
  unsigned char* b = static_cast<unsigned char*>(out);
  for (size_t i = 0; i < n; ++i) {
    const int hi = val(s[2 * i]), lo = val(s[2 * i + 1]);
    if (hi < 0 || lo < 0) {
      return false;
    }
    b[i] = static_cast<unsigned char>(hi << 4 | lo);
  }
  return true;
}

// Full-length send / receive; false on error, close or timeout (errno kept).
bool send_all(int fd, const void* p, size_t n) {
  const char* c = static_cast<const char*>(p);
  while (n > 0) {
    const ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
    if (k <= 0) {
      if (k < 0 && errno == EINTR) continue;
      return false;
    }
    c += k;
    n -= static_cast<size_t>(k);
  }
  return true;
}

bool recv_all(int fd, void* p, size_t n) {
  char* c = static_cast<char*>(p);
  while (n > 0) {
    const ssize_t k = ::recv(fd, c, n, 0);
    if (k <= 0) {
      if (k < 0 && errno == EINTR) continue;
      return false;
    }
    c += k;
    n -= static_cast<size_t>(k);
  }
  return true;
}

int io_error_status() { return (errno == EAGAIN || errno == EWOULDBLOCK) ? kTransportTimeout : kTransportIo; }

void set_socket_options(int fd, int timeout_s) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  timeval tv{};
  tv.tv_sec = timeout_s;
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  int buf = 8 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

// Looks the request up in the registration table. On success `*device` is the memory's device.
int check_request(const std::string& key_str, uint64_t ptr, uint64_t len, int* device) {
  AccessKey key;
  if (!AccessKey::parse(key_str, &key) || key.pid != static_cast<int64_t>(getpid())) {
    return kTransportBadKey;
  }
  Registry& reg = Registry::get();
  std::lock_guard<std::mutex> g(reg.mu);
  auto it = reg.by_id.find(key.id);
  if (it == reg.by_id.end() || it->second.nonce != key.nonce) {
    return kTransportBadKey;
  }
  const Registration& r = it->second;
  if (ptr < r.base || len > r.len || ptr - r.base > r.len - len) {
    return kTransportOutOfRange;
  }
  *device = r.device;
  return kTransportOk;
}

}  // namespace

const char* transport_strerror(int status) {
  switch (status) {
    case kTransportOk: return "ok";
    case kTransportBadKey: return "access key not known to the owner";
    case kTransportOutOfRange: return "range outside the registered memory";
    case kTransportNotConnected: return "transport is not connected";
    case kTransportIo: return "connection error";
    case kTransportCuda: return "CUDA error";
    case kTransportTimeout: return "timed out";
    case kTransportClosed: return "transport closed";
    case kTransportSizeMismatch: return "local view and remote buffer differ in length";
    default: return "unknown transport status";
  }
}

// ------------------------------------------------------------------ access keys

std::string AccessKey::str() const {
  std::ostringstream o;
  o << "b2k1:" << pid << ':' << id << ':' << std::hex << nonce << std::dec << ':' << device << ':' << base << ':' << len << ':'
    << ipc_offset << ':' << (ipc_hex.empty() ? std::string("-") : ipc_hex) << ':' << boot_id;
  return o.str();
}

bool AccessKey::parse(const std::string& s, AccessKey* out) {
  std::vector<std::string> f;
  size_t start = 0;
  while (f.size() < 9) {
    const size_t c = s.find(':', start);
    if (c == std::string::npos) break;
    f.push_back(s.substr(start, c - start));
    start = c + 1;
  }
  f.push_back(s.substr(start));  // the boot id may itself contain no ':' but keep the rest whole
  if (f.size() != 10 || f[0] != "b2k1") {
    return false;
  }
  try {
    out->pid = std::stoll(f[1]);
    out->id = std::stoull(f[2]);
    out->nonce = std::stoull(f[3], nullptr, 16);
    out->device = std::stoi(f[4]);
    out->base = std::stoull(f[5]);
    out->len = std::stoull(f[6]);
    out->ipc_offset = std::stoull(f[7]);
    out->ipc_hex = f[8] == "-" ? std::string() : f[8];
    out->boot_id = f[9];
  } catch (const std::exception&) {
    return false;
  }
  return true;
}

// ------------------------------------------------------------------ registered memory

namespace {

// Fills in the access key of a registration (nonce, CUDA IPC export of the allocation that holds it).
void build_key(Registration& r, uint64_t alloc_base) {
  AccessKey key;
  key.pid = static_cast<int64_t>(getpid());
  key.id = r.id;
  key.device = r.device;
  key.base = r.base;
  key.len = r.len;
  key.boot_id = boot_id();
  std::random_device rd;
  key.nonce = (static_cast<uint64_t>(rd()) << 32) ^ rd();
  if (r.device >= 0 && env_str("B200COMMS_TRANSPORT_STAGED", "0") != "1") {
    const uint64_t start = alloc_base ? alloc_base : r.base;
    cudaIpcMemHandle_t h;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(r.device);
    const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(start));
    if (prev >= 0) cudaSetDevice(prev);
    if (e == cudaSuccess) {
      key.ipc_hex = to_hex(&h, sizeof(h));
      key.ipc_offset = r.base - start;
    } else {
      cudaGetLastError();  // not exportable (for example a virtual-memory allocation): staged path only
    }
  }
  r.nonce = key.nonce;
  r.key = key.str();
}

}  // namespace

std::shared_ptr<TransportMemory> TransportMemory::create(void* ptr, size_t len, int device, uint64_t alloc_base) {
  if (ptr == nullptr || len == 0) {
    throw std::invalid_argument("TransportMemory: empty range");
  }
  std::shared_ptr<TransportMemory> m(new TransportMemory());
  m->ptr_ = ptr;
  m->len_ = len;
  m->device_ = device;
  const uint64_t base = reinterpret_cast<uint64_t>(ptr);
  Registry& reg = Registry::get();
  std::lock_guard<std::mutex> g(reg.mu);
  // An identical range first, then an allocator segment that contains the range.
  Registration* hit = nullptr;
  for (auto& kv : reg.by_id) {
    Registration& r = kv.second;
    if (r.device != device) continue;
    if (r.base == base && r.len == len && !r.segment) {
      hit = &r;
      break;
    }
    if (r.segment && base >= r.base && len <= r.len && base - r.base <= r.len - len) {
      hit = &r;
    }
  }
  if (hit != nullptr) {
    if (hit->key.empty()) {
      build_key(*hit, hit->base);  // a segment is exported when a range inside it is first used
    }
    ++hit->refs;
    m->id_ = hit->id;
    m->key_ = hit->key;
    m->reused_ = true;
    return m;
  }
  Registration r;
  r.id = reg.next_id++;
  r.base = base;
  r.len = len;
  r.device = device;
  r.refs = 1;
  build_key(r, alloc_base);
  m->id_ = r.id;
  m->key_ = r.key;
  reg.by_id.emplace(r.id, std::move(r));
  return m;
}

void TransportMemory::register_segment(void* base_ptr, size_t len, int device) {
  if (base_ptr == nullptr || len == 0) return;
  const uint64_t base = reinterpret_cast<uint64_t>(base_ptr);
  Registry& reg = Registry::get();
  std::lock_guard<std::mutex> g(reg.mu);
  for (auto& kv : reg.by_id) {
    if (kv.second.segment && kv.second.base == base && kv.second.device == device) {
      kv.second.len = len;
      return;
    }
  }
  Registration r;
  r.id = reg.next_id++;
  r.base = base;
  r.len = len;
  r.device = device;
  r.refs = 1;  // held by the table until unregister_segment
  r.segment = true;
  reg.by_id.emplace(r.id, std::move(r));
}

void TransportMemory::unregister_segment(void* base_ptr) {
  const uint64_t base = reinterpret_cast<uint64_t>(base_ptr);
  Registry& reg = Registry::get();
  std::lock_guard<std::mutex> g(reg.mu);
  for (auto it = reg.by_id.begin(); it != reg.by_id.end(); ++it) {
    if (it->second.segment && it->second.base == base) {
      reg.by_id.erase(it);  // the memory is gone: keys that point into it stop validating
      return;
    }
  }
}

size_t TransportMemory::segment_count() {
  Registry& reg = Registry::get();
  std::lock_guard<std::mutex> g(reg.mu);
  size_t n = 0;
  for (auto& kv : reg.by_id) n += kv.second.segment ? 1 : 0;
  return n;
}

TransportMemory::~TransportMemory() {
  Registry& reg = Registry::get();
  std::lock_guard<std::mutex> g(reg.mu);
  auto it = reg.by_id.find(id_);
  if (it != reg.by_id.end() && --it->second.refs <= 0 && !it->second.segment) {
    reg.by_id.erase(it);
  }
}

bool TransportMemory::contains(const void* p, size_t n) const {
  const uint64_t a = reinterpret_cast<uint64_t>(p), b = reinterpret_cast<uint64_t>(ptr_);
  return a >= b && n <= len_ && a - b <= len_ - n;
}

RemoteBuffer TransportMemory::remote_buffer(size_t offset, size_t length) const {
  if (offset > len_ || length > len_ - offset) {
    throw std::out_of_range("TransportMemory::remote_buffer: range outside the registration");
  }
  return RemoteBuffer{reinterpret_cast<uint64_t>(ptr_) + offset, length, key_};
}

// ------------------------------------------------------------------ futures

bool TransportFuture::done() const {
  std::lock_guard<std::mutex> g(mu_);
  return done_;
}

int TransportFuture::wait(int64_t timeout_ms) const {
  std::unique_lock<std::mutex> g(mu_);
  if (timeout_ms < 0) {
    cv_.wait(g, [&] { return done_; });
  } else if (!cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return done_; })) {
    return kTransportTimeout;
  }
  return status_;
}

void TransportFuture::complete(int status) {
  {
    std::lock_guard<std::mutex> g(mu_);
    done_ = true;
    status_ = status;
  }
  cv_.notify_all();
}

// ------------------------------------------------------------------ transport

P2pTransport::P2pTransport(int device)
    : device_(device),
      force_staged_(env_str("B200COMMS_TRANSPORT_STAGED", "0") == "1"),
      io_timeout_s_(std::max(1, std::atoi(env_str("B200COMMS_TRANSPORT_TIMEOUT_SECONDS", "60").c_str()))) {}

P2pTransport::~P2pTransport() { close(); }

bool P2pTransport::supported() { return true; }

std::string P2pTransport::bind() {
  std::lock_guard<std::mutex> g(mu_);
  if (!url_.empty()) {
    return url_;
  }
  const std::string host = env_str("B200COMMS_TRANSPORT_HOST", "127.0.0.1");
  const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) {
    throw std::runtime_error(std::string("P2pTransport::bind: socket: ") + std::strerror(errno));
  }
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = 0;
  if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) {
    ::close(fd);
    throw std::runtime_error("P2pTransport::bind: B200COMMS_TRANSPORT_HOST must be an IPv4 address, got " + host);
  }
  socklen_t alen = sizeof(addr);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd, 16) != 0 ||
      getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &alen) != 0) {
    const std::string why = std::strerror(errno);
    ::close(fd);
    throw std::runtime_error("P2pTransport::bind: " + why);
  }
  listen_fd_ = fd;
  std::ostringstream o;
  o << "b200p2p://" << host << ':' << ntohs(addr.sin_port) << '/' << getpid() << '/' << device_ << '/' << boot_id();
  url_ = o.str();
  accept_thread_ = std::thread([this] { accept_loop(); });
  return url_;
}

void P2pTransport::accept_loop() {
  while (!closing_.load()) {
    pollfd p{listen_fd_, POLLIN, 0};
    const int r = ::poll(&p, 1, 200);
    if (r <= 0 || !(p.revents & POLLIN)) {
      continue;
    }
    const int fd = ::accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) {
      continue;
    }
    set_socket_options(fd, io_timeout_s_);
    std::lock_guard<std::mutex> g(mu_);
    if (closing_.load()) {
      ::close(fd);
      break;
    }
    server_fds_.push_back(fd);
    servers_.emplace_back([this, fd] { serve(fd); });
  }
}

// One connection's requests, answered against the process-wide registration table.
void P2pTransport::serve(int fd) {
  void* bounce = nullptr;      // pinned, allocated at the first request that touches device memory
  int bounce_device = -1;
  std::vector<char> sink;      // where the payload of a refused write goes
  auto reply = [&](uint32_t status) { return send_all(fd, &status, sizeof(status)); };
  auto ensure_bounce = [&](int device) {
    if (bounce == nullptr || bounce_device != device) {
      cudaSetDevice(device);
      if (bounce == nullptr && cudaMallocHost(&bounce, kBounceBytes) != cudaSuccess) {
        bounce = nullptr;
        return false;
      }
      bounce_device = device;
    }
    return true;
  };
  while (!closing_.load()) {
    pollfd p{fd, POLLIN, 0};
    const int r = ::poll(&p, 1, 200);
    if (r < 0 && errno != EINTR) break;
    if (r <= 0) continue;
    if (p.revents & (POLLERR | POLLNVAL)) break;
    WireHeader h{};
    if (!recv_all(fd, &h, sizeof(h)) || h.magic != kMagic || h.key_len > 4096) break;
    std::string key(h.key_len, '\0');
    if (h.key_len && !recv_all(fd, &key[0], h.key_len)) break;
    if (h.op == kOpHello) {
      if (!reply(kTransportOk)) break;
      continue;
    }
    int device = -1;
    int status = check_request(key, h.ptr, h.len, &device);
    if (status == kTransportOk && device >= 0 && h.op != kOpValidate && !ensure_bounce(device)) {
      status = kTransportCuda;
    }
    bool ok = true;
    if (h.op == kOpValidate) {
      ok = reply(static_cast<uint32_t>(status));
    } else if (h.op == kOpWrite) {
      char* dst = reinterpret_cast<char*>(h.ptr);
      if (status != kTransportOk) {
        sink.resize(std::min<uint64_t>(h.len, kBounceBytes));
        for (uint64_t off = 0; ok && off < h.len; off += sink.size()) {
          ok = recv_all(fd, sink.data(), std::min<uint64_t>(sink.size(), h.len - off));
        }
      } else if (device < 0) {
        ok = recv_all(fd, dst, h.len);
      } else {
        for (uint64_t off = 0; ok && off < h.len; off += kBounceBytes) {
          const size_t n = std::min<uint64_t>(kBounceBytes, h.len - off);
          ok = recv_all(fd, bounce, n);
          if (ok && status == kTransportOk && cudaMemcpy(dst + off, bounce, n, cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaGetLastError();
            status = kTransportCuda;  // keep draining so the stream stays framed
          }
        }
      }
      ok = ok && reply(static_cast<uint32_t>(status));
    } else if (h.op == kOpRead) {
      const char* src = reinterpret_cast<const char*>(h.ptr);
      ok = reply(static_cast<uint32_t>(status));
      if (ok && status == kTransportOk) {
        if (device < 0) {
          ok = send_all(fd, src, h.len);
        } else {
          // A failed device copy cannot be reported once the status went out: end the connection instead.
          for (uint64_t off = 0; ok && off < h.len; off += kBounceBytes) {
            const size_t n = std::min<uint64_t>(kBounceBytes, h.len - off);
            ok = cudaMemcpy(bounce, src + off, n, cudaMemcpyDeviceToHost) == cudaSuccess && send_all(fd, bounce, n);
          }
        }
      }
    } else {
      break;
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      if (status == kTransportOk) {
        if (h.op != kOpValidate) {
          ++counters_.served_ops;
          counters_.served_bytes += h.len;
        }
      } else {
        ++counters_.rejected;
      }
    }
    if (!ok) break;
  }
  if (bounce) {
    cudaFreeHost(bounce);
  }
  ::shutdown(fd, SHUT_RDWR);
}

int P2pTransport::connect(const std::string& peer_url) {
  // b200p2p://<host>:<port>/<pid>/<device>/<boot id>
  const std::string scheme = "b200p2p://";
  if (peer_url.compare(0, scheme.size(), scheme) != 0) {
    return kTransportNotConnected;
  }
  const size_t colon = peer_url.find(':', scheme.size());
  const size_t s1 = peer_url.find('/', scheme.size());
  if (colon == std::string::npos || s1 == std::string::npos || colon > s1) {
    return kTransportNotConnected;
  }
  const size_t s2 = peer_url.find('/', s1 + 1);
  const size_t s3 = s2 == std::string::npos ? s2 : peer_url.find('/', s2 + 1);
  if (s3 == std::string::npos) {
    return kTransportNotConnected;
  }
  const std::string host = peer_url.substr(scheme.size(), colon - scheme.size());
  int port = 0;
  int64_t pid = 0;
  try {
    port = std::stoi(peer_url.substr(colon + 1, s1 - colon - 1));
    pid = std::stoll(peer_url.substr(s1 + 1, s2 - s1 - 1));
  } catch (const std::exception&) {
    return kTransportNotConnected;
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    if (connected_.load()) {
      return kTransportOk;  // one peer per transport; a second connect is a no-op
    }
  }
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1) {
    return kTransportNotConnected;
  }
  const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) {
    return kTransportIo;
  }
  set_socket_options(fd, io_timeout_s_);
  WireHeader hello{kMagic, kOpHello, 0, 0, 0, 0};
  uint32_t status = 0;
  if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || !send_all(fd, &hello, sizeof(hello)) ||
      !recv_all(fd, &status, sizeof(status)) || status != kTransportOk) {
    const int st = io_error_status();
    ::close(fd);
    return st;
  }
  std::lock_guard<std::mutex> g(mu_);
  client_fd_ = fd;
  peer_pid_ = pid;
  peer_boot_id_ = peer_url.substr(s3 + 1);
  connected_.store(true);
  if (!worker_.joinable()) {
    worker_ = std::thread([this] { worker_loop(); });
  }
  return kTransportOk;
}

bool P2pTransport::connected() const { return connected_.load(); }

TransportCounters P2pTransport::counters() const {
  std::lock_guard<std::mutex> g(mu_);
  return counters_;
}

std::shared_ptr<TransportFuture> P2pTransport::enqueue(bool is_write, const TransportView& local, const RemoteBuffer& remote) {
  auto fut = std::make_shared<TransportFuture>();
  if (!local.mem || local.offset > local.mem->size() || local.length > local.mem->size() - local.offset) {
    throw std::out_of_range("P2pTransport: local view outside its registration");
  }
  std::unique_lock<std::mutex> g(mu_);
  if (closing_.load()) {
    g.unlock();
    fut->complete(kTransportClosed);
    return fut;
  }
  if (!connected_.load()) {
    g.unlock();
    fut->complete(kTransportNotConnected);
    return fut;
  }
  queue_.push_back(Op{is_write, local, remote, fut});
  g.unlock();
  cv_.notify_one();
  return fut;
}

std::shared_ptr<TransportFuture> P2pTransport::write(const TransportView& local, const RemoteBuffer& remote) {
  return enqueue(true, local, remote);
}

std::shared_ptr<TransportFuture> P2pTransport::read(const TransportView& local, const RemoteBuffer& remote) {
  return enqueue(false, local, remote);
}

void P2pTransport::worker_loop() {
  if (device_ >= 0) {
    cudaSetDevice(device_);
  }
  for (;;) {
    Op op;
    {
      std::unique_lock<std::mutex> g(mu_);
      cv_.wait(g, [&] { return closing_.load() || !queue_.empty(); });
      if (closing_.load()) {
        return;  // close() completes what is still queued
      }
      op = std::move(queue_.front());
      queue_.pop_front();
    }
    int status = kTransportIo;
    try {
      status = run_op(op);
    } catch (const std::exception&) {
      status = kTransportIo;
    }
    if (status == kTransportIo || status == kTransportTimeout) {
      connected_.store(false);  // the byte stream may be out of frame: no further requests on it
    }
    op.fut->complete(status);
  }
}

int P2pTransport::run_op(const Op& op) {
  if (op.local.length > op.remote.len) {
    return kTransportSizeMismatch;
  }
  if (!connected_.load()) {
    return kTransportNotConnected;
  }
  AccessKey key;
  if (!AccessKey::parse(op.remote.access_key, &key)) {
    return kTransportBadKey;
  }
  const bool same_process = key.pid == static_cast<int64_t>(getpid());
  const bool peer_copy = !force_staged_ && device_ >= 0 && op.local.mem->device() >= 0 && key.device >= 0 &&
      key.boot_id == boot_id() && (same_process || !key.ipc_hex.empty());
  return peer_copy ? run_peer_copy(op, key) : run_socket(op);
}

// Asks the owner (once per key and range) whether the request is allowed.
int P2pTransport::validate_remote(const RemoteBuffer& remote) {
  const std::string tag = remote.access_key + '@' + std::to_string(remote.ptr) + '+' + std::to_string(remote.len);
  if (validated_.count(tag)) {
    return kTransportOk;
  }
  WireHeader h{kMagic, kOpValidate, remote.ptr, remote.len, static_cast<uint32_t>(remote.access_key.size()), 0};
  uint32_t status = 0;
  if (!send_all(client_fd_, &h, sizeof(h)) || !send_all(client_fd_, remote.access_key.data(), remote.access_key.size()) ||
      !recv_all(client_fd_, &status, sizeof(status))) {
    return io_error_status();
  }
  if (status == kTransportOk) {
    validated_[tag] = true;
  }
  return static_cast<int>(status);
}

int P2pTransport::run_peer_copy(const Op& op, const AccessKey& key) {
  const int st = validate_remote(op.remote);
  if (st != kTransportOk) {
    return st;
  }
  char* remote_ptr = nullptr;
  if (key.pid == static_cast<int64_t>(getpid())) {
    remote_ptr = reinterpret_cast<char*>(op.remote.ptr);
  } else {
    auto it = mapped_.find(op.remote.access_key);
    if (it == mapped_.end()) {
      cudaIpcMemHandle_t h;
      void* p = nullptr;
      if (!from_hex(key.ipc_hex, &h, sizeof(h)) || cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return run_socket(op);  // cannot be mapped here (no peer access): staged path
      }
      it = mapped_.emplace(op.remote.access_key, Mapped{p}).first;
    }
    remote_ptr = static_cast<char*>(it->second.alloc_base) + key.ipc_offset + (op.remote.ptr - key.base);
  }
  if (stream_ == nullptr) {
    cudaStream_t s;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
      cudaGetLastError();
      return kTransportCuda;
    }
    stream_ = s;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  void* dst = op.is_write ? static_cast<void*>(remote_ptr) : op.local.data();
  const void* src = op.is_write ? op.local.data() : static_cast<const void*>(remote_ptr);
  if (cudaMemcpyAsync(dst, src, op.local.length, cudaMemcpyDefault, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return kTransportCuda;
  }
  std::lock_guard<std::mutex> g(mu_);
  ++counters_.peer_copy_ops;
  counters_.peer_copy_bytes += op.local.length;
  return kTransportOk;
}

int P2pTransport::run_socket(const Op& op) {
  const bool local_dev = op.local.mem->device() >= 0;
  const uint64_t n = op.local.length;
  if (local_dev) {
    cudaSetDevice(op.local.mem->device());
    if (bounce_ == nullptr && cudaMallocHost(&bounce_, kBounceBytes) != cudaSuccess) {
      cudaGetLastError();
      bounce_ = nullptr;
      return kTransportCuda;
    }
  }
  const int fd = client_fd_;
  WireHeader h{kMagic, op.is_write ? kOpWrite : kOpRead, op.remote.ptr, n, static_cast<uint32_t>(op.remote.access_key.size()), 0};
  if (!send_all(fd, &h, sizeof(h)) || !send_all(fd, op.remote.access_key.data(), op.remote.access_key.size())) {
    return io_error_status();
  }
  char* local = static_cast<char*>(op.local.data());
  uint32_t status = 0;
  if (op.is_write) {
    if (!local_dev) {
      if (!send_all(fd, local, n)) return io_error_status();
    } else {
      for (uint64_t off = 0; off < n; off += kBounceBytes) {
        const size_t k = std::min<uint64_t>(kBounceBytes, n - off);
        if (cudaMemcpy(bounce_, local + off, k, cudaMemcpyDeviceToHost) != cudaSuccess) {
          cudaGetLastError();
          return kTransportIo;  // the frame is incomplete: the connection is not reusable
        }
        if (!send_all(fd, bounce_, k)) return io_error_status();
      }
    }
    if (!recv_all(fd, &status, sizeof(status))) return io_error_status();
  } else {
    if (!recv_all(fd, &status, sizeof(status))) return io_error_status();
    if (status == kTransportOk) {
      if (!local_dev) {
        if (!recv_all(fd, local, n)) return io_error_status();
      } else {
        for (uint64_t off = 0; off < n; off += kBounceBytes) {
          const size_t k = std::min<uint64_t>(kBounceBytes, n - off);
          if (!recv_all(fd, bounce_, k)) return io_error_status();
          if (cudaMemcpy(local + off, bounce_, k, cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaGetLastError();
            return kTransportIo;
          }
        }
      }
    }
  }
  if (status == kTransportOk) {
    std::lock_guard<std::mutex> g(mu_);
    ++counters_.socket_ops;
    counters_.socket_bytes += n;
  }
  return static_cast<int>(status);
}

void P2pTransport::close() {
  std::deque<Op> pending;
  std::vector<std::thread> servers;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (closing_.exchange(true)) {
      return;
    }
    pending.swap(queue_);
    if (client_fd_ >= 0) ::shutdown(client_fd_, SHUT_RDWR);
    for (int fd : server_fds_) ::shutdown(fd, SHUT_RDWR);
    servers.swap(servers_);
  }
  cv_.notify_all();
  connected_.store(false);
  if (worker_.joinable()) worker_.join();
  if (accept_thread_.joinable()) accept_thread_.join();
  for (auto& t : servers) {
    if (t.joinable()) t.join();
  }
  for (auto& op : pending) {
    op.fut->complete(kTransportClosed);
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& op : queue_) op.fut->complete(kTransportClosed);
    queue_.clear();
    for (int fd : server_fds_) ::close(fd);
    server_fds_.clear();
    if (client_fd_ >= 0) ::close(client_fd_);
    client_fd_ = -1;
    if (listen_fd_ >= 0) ::close(listen_fd_);
    listen_fd_ = -1;
  }
  for (auto& kv : mapped_) {
    cudaIpcCloseMemHandle(kv.second.alloc_base);
  }
  mapped_.clear();
  if (bounce_) {
    cudaFreeHost(bounce_);
    bounce_ = nullptr;
  }
  if (stream_) {
    cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
    stream_ = nullptr;
  }
}

}  // namespace b200c
