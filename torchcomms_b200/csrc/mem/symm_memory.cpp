// Symmetric memory: allocation, handle exchange, peer mapping, multicast.
#include "symm_memory.hpp"

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstring>
#include <random>
#include <stdexcept>

#include "../core/logging.hpp"
#include "../core/options.hpp"

namespace b200c {

namespace {

size_t round_up(size_t v, size_t to) {
  return (v + to - 1) / to * to;
}

struct FdMsg {
  int32_t src;
  uint64_t tag;
};

} // namespace

// ------------------------------------------------------------ FdChannel ----

FdChannel::FdChannel(const std::string& token, int rank, int nranks)
    : token_(token), rank_(rank), nranks_(nranks) {
  sock_ = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (sock_ < 0) {
    throw std::runtime_error(std::string("fd channel: socket() failed: ") + strerror(errno));
  }
  sockaddr_un addr{};
  addr.sun_family = AF_UNIX;
  const std::string name = address_of(rank);
  // Abstract namespace: first byte of sun_path is NUL, no file is created.
  std::memcpy(addr.sun_path + 1, name.data(), name.size());
  const socklen_t len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  if (::bind(sock_, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
    const std::string err = strerror(errno);
    ::close(sock_);
    sock_ = -1;
    throw std::runtime_error("fd channel: bind(" + name + ") failed: " + err);
  }
}

FdChannel::~FdChannel() {
  for (auto& kv : stash_) {
    ::close(kv.second);
  }
  if (sock_ >= 0) {
    ::close(sock_);
  }
}

std::string FdChannel::address_of(int rank) const {
  std::string s = "b200c." + token_ + "." + std::to_string(rank);
  if (s.size() > 100) {
    s.resize(100);
  }
  return s;
}

void FdChannel::send_fd(int peer, int fd, uint64_t tag) {
  sockaddr_un addr{};
  addr.sun_family = AF_UNIX;
  const std::string name = address_of(peer);
  std::memcpy(addr.sun_path + 1, name.data(), name.size());
  const socklen_t alen = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());

  FdMsg payload{rank_, tag};
  iovec iov{&payload, sizeof(payload)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msghdr msg{};
  msg.msg_name = &addr;
  msg.msg_namelen = alen;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  // The peer's socket exists (ranks barrier after binding); retry briefly on
  // a full queue.
  for (int attempt = 0; attempt < 2000; ++attempt) {
    if (::sendmsg(sock_, &msg, 0) >= 0) {
      return;
    }
    if (errno != EAGAIN && errno != ENOBUFS && errno != ECONNREFUSED && errno != ENOENT) {
      break;
    }
    ::usleep(1000);
  }
  throw std::runtime_error("fd channel: sendmsg to rank " + std::to_string(peer) + " failed: " + strerror(errno));
}

int FdChannel::recv_fd(int src, uint64_t tag, int timeout_ms) {
  const auto key = std::make_pair(src, tag);
  int waited = 0;
  while (true) {
    auto it = stash_.find(key);
    if (it != stash_.end()) {
      const int fd = it->second;
      stash_.erase(it);
      return fd;
    }
    pollfd p{sock_, POLLIN, 0};
    const int rc = ::poll(&p, 1, 100);
    if (rc == 0) {
      waited += 100;
      if (waited >= timeout_ms) {
        throw std::runtime_error("fd channel: timed out waiting for a descriptor from rank " + std::to_string(src));
      }
      continue;
    }
    if (rc < 0) {
      if (errno == EINTR) continue;
      throw std::runtime_error(std::string("fd channel: poll failed: ") + strerror(errno));
    }
    FdMsg payload{};
    iovec iov{&payload, sizeof(payload)};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    const ssize_t n = ::recvmsg(sock_, &msg, MSG_CMSG_CLOEXEC);
    if (n < static_cast<ssize_t>(sizeof(payload))) {
      continue;
    }
    cmsghdr* cm = CMSG_FIRSTHDR(&msg);
    if (cm == nullptr || cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != SCM_RIGHTS) {
      continue;
    }
    int fd = -1;
    std::memcpy(&fd, CMSG_DATA(cm), sizeof(int));
    stash_[std::make_pair(static_cast<int>(payload.src), payload.tag)] = fd;
  }
}

// ----------------------------------------------------------- SymmMemory ----

SymmMemory::SymmMemory(c10::intrusive_ptr<c10d::Store> store, int rank, int nranks, int device_index,
                       std::shared_ptr<DriverApi> driver, std::chrono::milliseconds timeout, bool allow_multicast,
                       std::shared_ptr<CudaApi> cuda)
    : store_(std::move(store)), rank_(rank), nranks_(nranks), device_(device_index), drv_(std::move(driver)),
      cuda_(cuda ? std::move(cuda) : CudaApi::real()), timeout_(timeout), allow_mc_(allow_multicast) {
  decide_mode();
}

SymmMemory::~SymmMemory() = default;

std::vector<std::string> SymmMemory::all_gather_bytes(const std::string& key, const std::string& mine) {
  store_set_string(*store_, key + "/" + std::to_string(rank_), mine);
  std::vector<std::string> out(nranks_);
  for (int p = 0; p < nranks_; ++p) {
    out[p] = p == rank_ ? mine : store_get_string(*store_, key + "/" + std::to_string(p));
  }
  return out;
}

void SymmMemory::barrier(const std::string& what) {
  if (nranks_ > 1) {
    store_barrier(*store_, "symm/bar/" + what, rank_, nranks_, timeout_);
  }
}

void SymmMemory::decide_mode() {
  if (nranks_ <= 1) {
    mode_ = SymmMode::LOCAL;
    return;
  }
  const std::string forced = env_to_value<std::string>("B200COMMS_SYMM_MODE", "auto");
  bool vmm = false, mc = false;
  size_t gran = 2u << 20;
  if (drv_->available() && forced != "ipc") {
    try {
      B200C_CU_CHECK(drv_, drv_->deviceGet(&cu_dev_, device_));
      int vmm_ok = 0, fd_ok = 0, mc_ok = 0;
      drv_->deviceGetAttribute(&vmm_ok, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cu_dev_);
      drv_->deviceGetAttribute(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cu_dev_);
      drv_->deviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cu_dev_);
      vmm = vmm_ok && fd_ok;
      const bool nvls_env = env_to_value<bool>("B200COMMS_NVLS", true) && env_to_value<bool>("NCCL_NVLS_ENABLE", true);
      mc = vmm && mc_ok && allow_mc_ && nvls_env && nranks_ >= 2;
      if (vmm) {
        CUmemAllocationProp prop{};
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = device_;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t g = 0;
        B200C_CU_CHECK(drv_, drv_->memGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
        gran = std::max(gran, g);
      }
      if (mc) {
        CUmulticastObjectProp mp{};
        mp.numDevices = static_cast<unsigned>(nranks_);
        mp.size = gran;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t g = 0;
        if (drv_->multicastGetGranularity(&g, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && g > 0) {
          gran = round_up(gran, g);
        } else {
          mc = false;
        }
      }
    } catch (const std::exception& e) {
      B200C_LOG(WARN, "symm", "VMM probing failed, falling back to CUDA IPC: " << e.what());
      vmm = false;
      mc = false;
    }
  }
  // All ranks must take the same path.
  auto caps = all_gather_bytes("symm/caps", std::string(vmm ? "1" : "0") + (mc ? "1" : "0") + std::to_string(gran));
  bool all_vmm = true, all_mc = true;
  size_t max_gran = gran;
  for (auto& c : caps) {
    all_vmm = all_vmm && c[0] == '1';
    all_mc = all_mc && c[1] == '1';
    max_gran = std::max<size_t>(max_gran, std::strtoull(c.c_str() + 2, nullptr, 10));
  }
  mode_ = all_vmm ? SymmMode::VMM_FD : SymmMode::CUDA_IPC;
  mc_ok_ = all_vmm && all_mc;
  gran_ = max_gran;
  if (mode_ == SymmMode::VMM_FD) {
    std::string token;
    if (rank_ == 0) {
      std::random_device rd;
      token = std::to_string(getpid()) + "-" + std::to_string(rd()) + std::to_string(rd());
      store_set_string(*store_, "symm/fdtoken", token);
    } else {
      token = store_get_string(*store_, "symm/fdtoken");
    }
    fds_ = std::make_unique<FdChannel>(token, rank_, nranks_);
    barrier("fdchannel");  // every socket is bound before anybody sends
  }
  B200C_LOG(INFO, "symm", "mode=" << (mode_ == SymmMode::VMM_FD ? "vmm+fd" : "cuda-ipc") << " multicast=" << mc_ok_
                                   << " granularity=" << gran_);
}

void SymmMemory::map_vmm(SymmSegment& seg, CUmemGenericAllocationHandle local_handle, uint64_t seq) {
  const size_t size = seg.bytes;
  int my_fd = -1;
  B200C_CU_CHECK(drv_, drv_->memExportToShareableHandle(&my_fd, local_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  for (int p = 0; p < nranks_; ++p) {
    if (p != rank_) {
      fds_->send_fd(p, my_fd, seq * 4);
    }
  }
  seg.handles.assign(nranks_, 0);
  seg.handles[rank_] = local_handle;
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    const int fd = fds_->recv_fd(p, seq * 4, static_cast<int>(timeout_.count()));
    CUresult r = drv_->memImportFromShareableHandle(&seg.handles[p], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    if (r != CUDA_SUCCESS) {
      throw std::runtime_error("importing rank " + std::to_string(p) + "'s memory failed: " + drv_->errorString(r));
    }
  }
  ::close(my_fd);
  seg.va_bytes = size * nranks_;
  B200C_CU_CHECK(drv_, drv_->memAddressReserve(&seg.va_base, seg.va_bytes, gran_));
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device_;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  seg.peer_ptrs.assign(nranks_, nullptr);
  for (int p = 0; p < nranks_; ++p) {
    const CUdeviceptr at = seg.va_base + static_cast<CUdeviceptr>(p) * size;
    B200C_CU_CHECK(drv_, drv_->memMap(at, size, 0, seg.handles[p]));
    B200C_CU_CHECK(drv_, drv_->memSetAccess(at, size, &acc, 1));
    seg.peer_ptrs[p] = reinterpret_cast<char*>(at);
  }
}

void SymmMemory::try_multicast(SymmSegment& seg, uint64_t seq) {
  const size_t size = seg.bytes;
  const std::string key = "symm/mc/" + std::to_string(seq);
  bool ok = true;
  CUmemGenericAllocationHandle mc = 0;
  CUmulticastObjectProp prop{};
  prop.numDevices = static_cast<unsigned>(nranks_);
  prop.size = size;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  try {
    if (rank_ == 0) {
      int fd = -1;
      CUresult r = drv_->multicastCreate(&mc, &prop);
      if (r == CUDA_SUCCESS) {
        r = drv_->memExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      }
      store_set_string(*store_, key + "/root", r == CUDA_SUCCESS ? "1" : "0");
      if (r != CUDA_SUCCESS) {
        throw std::runtime_error("cuMulticastCreate/export failed: " + drv_->errorString(r));
      }
      for (int p = 1; p < nranks_; ++p) {
        fds_->send_fd(p, fd, seq * 4 + 1);
      }
      ::close(fd);
    } else {
      if (store_get_string(*store_, key + "/root") != "1") {
        throw std::runtime_error("the root could not create the multicast object");
      }
      const int fd = fds_->recv_fd(0, seq * 4 + 1, static_cast<int>(timeout_.count()));
      CUresult r = drv_->memImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fd);
      if (r != CUDA_SUCCESS) {
        throw std::runtime_error("importing the multicast object failed: " + drv_->errorString(r));
      }
    }
    B200C_CU_CHECK(drv_, drv_->multicastAddDevice(mc, cu_dev_));
  } catch (const std::exception& e) {
    B200C_LOG(WARN, "symm", "multicast setup failed on rank " << rank_ << ": " << e.what());
    ok = false;
  }
  // Every device must be added before any rank binds memory; the agreement
  // round doubles as that barrier.
  auto votes = all_gather_bytes(key + "/added", ok ? "1" : "0");
  bool all = true;
  for (auto& v : votes) all = all && v == "1";
  if (!all) {
    if (mc) drv_->memRelease(mc);
    mc_ok_ = false;
    return;
  }
  CUdeviceptr va = 0;
  bool bound = false, mapped = false;
  try {
    B200C_CU_CHECK(drv_, drv_->multicastBindMem(mc, 0, seg.handles[rank_], 0, size));
    bound = true;
    B200C_CU_CHECK(drv_, drv_->memAddressReserve(&va, size, gran_));
    B200C_CU_CHECK(drv_, drv_->memMap(va, size, 0, mc));
    mapped = true;
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    B200C_CU_CHECK(drv_, drv_->memSetAccess(va, size, &acc, 1));
  } catch (const std::exception& e) {
    B200C_LOG(WARN, "symm", "multicast bind/map failed on rank " << rank_ << ": " << e.what());
    ok = false;
  }
  votes = all_gather_bytes(key + "/bound", ok ? "1" : "0");
  all = true;
  for (auto& v : votes) all = all && v == "1";
  if (!all) {
    if (mapped) drv_->memUnmap(va, size);
    if (va) drv_->memAddressFree(va, size);
    if (bound) drv_->multicastUnbind(mc, cu_dev_, 0, size);
    drv_->memRelease(mc);
    mc_ok_ = false;
    return;
  }
  seg.mc_handle = mc;
  seg.mc_va = va;
  seg.mc_ptr = reinterpret_cast<char*>(va);
}

void SymmMemory::exchange_ipc(SymmSegment& seg, void* local_base, size_t offset, uint64_t seq) {
  cudaIpcMemHandle_t mine{};
  B200C_CUDA_CHECK(cudaIpcGetMemHandle(&mine, local_base));
  std::string blob(reinterpret_cast<const char*>(&mine), sizeof(mine));
  blob += std::to_string(offset);
  auto all = all_gather_bytes("symm/ipc/" + std::to_string(seq), blob);
  seg.peer_ptrs.assign(nranks_, nullptr);
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) {
      seg.peer_ptrs[p] = static_cast<char*>(local_base) + offset;
      continue;
    }
    cudaIpcMemHandle_t h{};
    std::memcpy(&h, all[p].data(), sizeof(h));
    const size_t off = std::strtoull(all[p].c_str() + sizeof(h), nullptr, 10);
    void* opened = nullptr;
    B200C_CUDA_CHECK(cudaIpcOpenMemHandle(&opened, h, cudaIpcMemLazyEnablePeerAccess));
    seg.ipc_opened.push_back(opened);
    seg.peer_ptrs[p] = static_cast<char*>(opened) + off;
  }
}

std::shared_ptr<SymmSegment> SymmMemory::allocate(size_t bytes, bool want_multicast) {
  const uint64_t seq = seq_++;
  auto seg = std::make_shared<SymmSegment>();
  seg->rank = rank_;
  seg->nranks = nranks_;
  seg->mode = mode_;
  seg->bytes = round_up(std::max<size_t>(bytes, 1), gran_);
  seg->cu_device = cu_dev_;
  B200C_CUDA_CHECK(cuda_->setDevice(device_));
  if (mode_ == SymmMode::LOCAL) {
    void* p = nullptr;
    B200C_CUDA_CHECK(cuda_->mallocDevice(&p, seg->bytes));
    B200C_CUDA_CHECK(cuda_->memsetDevice(p, 0, seg->bytes));
    seg->peer_ptrs = {static_cast<char*>(p)};
  } else if (mode_ == SymmMode::VMM_FD) {
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device_;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle h = 0;
    B200C_CU_CHECK(drv_, drv_->memCreate(&h, seg->bytes, &prop));
    map_vmm(*seg, h, seq);
    B200C_CUDA_CHECK(cuda_->memsetDevice(seg->local(), 0, seg->bytes));
  } else {
    void* p = nullptr;
    B200C_CUDA_CHECK(cudaMalloc(&p, seg->bytes));
    B200C_CUDA_CHECK(cudaMemset(p, 0, seg->bytes));
    exchange_ipc(*seg, p, 0, seq);
  }
  B200C_CUDA_CHECK(cuda_->deviceSynchronize());
  barrier("alloc/" + std::to_string(seq));  // zero-fill is complete everywhere
  if (want_multicast && mc_ok_ && mode_ == SymmMode::VMM_FD) {
    try_multicast(*seg, seq);
  }
  return seg;
}

std::shared_ptr<SymmSegment> SymmMemory::attach_user_buffer(void* local, size_t bytes, bool want_multicast) {
  const uint64_t seq = seq_++;
  auto seg = std::make_shared<SymmSegment>();
  seg->rank = rank_;
  seg->nranks = nranks_;
  seg->bytes = bytes;
  seg->owns_local = false;
  seg->cu_device = cu_dev_;
  if (mode_ == SymmMode::LOCAL) {
    seg->mode = SymmMode::LOCAL;
    seg->peer_ptrs = {static_cast<char*>(local)};
    return seg;
  }
  ExportableAlloc a;
  const bool exportable = mode_ == SymmMode::VMM_FD && ExportableRegistry::get().find(local, bytes, &a);
  auto votes = all_gather_bytes("symm/attach/" + std::to_string(seq), exportable ? "1" : "0");
  bool all = true, none = true;
  for (auto& v : votes) {
    all = all && v == "1";
    none = none && v == "0";
  }
  if (!all && !none) {
    throw std::runtime_error(
        "window registration: some ranks passed memory from the symmetric allocator and others did not");
  }
  if (all) {
    // Map every rank's whole allocation, then point at the tensor inside it.
    seg->mode = SymmMode::VMM_FD;
    const size_t my_off = reinterpret_cast<CUdeviceptr>(local) - a.base;
    auto metas = all_gather_bytes("symm/attachmeta/" + std::to_string(seq),
                                  std::to_string(a.bytes) + ":" + std::to_string(my_off));
    int my_fd = -1;
    B200C_CU_CHECK(drv_, drv_->memExportToShareableHandle(&my_fd, a.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    for (int p = 0; p < nranks_; ++p) {
      if (p != rank_) fds_->send_fd(p, my_fd, seq * 4);
    }
    seg->handles.assign(nranks_, 0);
    seg->peer_ptrs.assign(nranks_, nullptr);
    seg->peer_ptrs[rank_] = static_cast<char*>(local);
    bool whole_everywhere = my_off == 0 && bytes == a.bytes && bytes % gran_ == 0;
    for (int p = 0; p < nranks_; ++p) {
      whole_everywhere = whole_everywhere && metas[p] == std::to_string(bytes) + ":0";
    }
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (int p = 0; p < nranks_; ++p) {
      if (p == rank_) continue;
      const size_t colon = metas[p].find(':');
      const size_t psize = std::strtoull(metas[p].c_str(), nullptr, 10);
      const size_t poff = std::strtoull(metas[p].c_str() + colon + 1, nullptr, 10);
      const int fd = fds_->recv_fd(p, seq * 4, static_cast<int>(timeout_.count()));
      CUresult r = drv_->memImportFromShareableHandle(&seg->handles[p], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fd);
      if (r != CUDA_SUCCESS) {
        throw std::runtime_error("window registration: import failed: " + drv_->errorString(r));
      }
      CUdeviceptr va = 0;
      B200C_CU_CHECK(drv_, drv_->memAddressReserve(&va, psize, gran_));
      B200C_CU_CHECK(drv_, drv_->memMap(va, psize, 0, seg->handles[p]));
      B200C_CU_CHECK(drv_, drv_->memSetAccess(va, psize, &acc, 1));
      seg->ipc_opened.push_back(reinterpret_cast<void*>(va));        // reused as (va) list for teardown
      seg->ipc_opened.push_back(reinterpret_cast<void*>(psize));     // followed by its size
      seg->peer_ptrs[p] = reinterpret_cast<char*>(va) + poff;
    }
    ::close(my_fd);
    if (want_multicast && whole_everywhere && mc_ok_) {
      // try_multicast() binds handles[rank]; release() never frees the own
      // handle of memory it does not own.
      seg->handles[rank_] = a.handle;
      barrier("attachmc/" + std::to_string(seq));
      try_multicast(*seg, seq);
    }
  } else {
    seg->mode = SymmMode::CUDA_IPC;
    // cudaIpcGetMemHandle describes the whole allocation that contains `local`.
    CUdeviceptr base = 0;
    size_t range = 0;
    auto fn = drv_->available();
    (void)fn;
    cudaPointerAttributes attr{};
    B200C_CUDA_CHECK(cudaPointerGetAttributes(&attr, local));
    // The runtime has no address-range query; ask the driver through the
    // generic entry point.
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess || sym == nullptr) {
      throw std::runtime_error("window registration: cuMemGetAddressRange is not available");
    }
    auto get_range = reinterpret_cast<CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr)>(sym);
    B200C_CU_CHECK(drv_, get_range(&base, &range, reinterpret_cast<CUdeviceptr>(local)));
    exchange_ipc(*seg, reinterpret_cast<void*>(base), reinterpret_cast<CUdeviceptr>(local) - base, seq);
  }
  barrier("attach/" + std::to_string(seq));
  return seg;
}

void SymmMemory::release(const std::shared_ptr<SymmSegment>& seg) {
  if (!seg) return;
  if (seg->mc_ptr) {
    drv_->memUnmap(seg->mc_va, seg->bytes);
    drv_->memAddressFree(seg->mc_va, seg->bytes);
    drv_->multicastUnbind(seg->mc_handle, seg->cu_device, 0, seg->bytes);
    drv_->memRelease(seg->mc_handle);
    seg->mc_ptr = nullptr;
  }
  if (seg->mode == SymmMode::VMM_FD && seg->owns_local) {
    for (int p = 0; p < seg->nranks; ++p) {
      drv_->memUnmap(seg->va_base + static_cast<CUdeviceptr>(p) * seg->bytes, seg->bytes);
    }
    drv_->memAddressFree(seg->va_base, seg->va_bytes);
    for (auto h : seg->handles) {
      if (h) drv_->memRelease(h);
    }
  } else if (seg->mode == SymmMode::VMM_FD) {
    for (size_t i = 0; i + 1 < seg->ipc_opened.size(); i += 2) {
      const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(seg->ipc_opened[i]);
      const size_t sz = reinterpret_cast<size_t>(seg->ipc_opened[i + 1]);
      drv_->memUnmap(va, sz);
      drv_->memAddressFree(va, sz);
    }
    for (int p = 0; p < seg->nranks; ++p) {
      if (p != seg->rank && seg->handles[p]) drv_->memRelease(seg->handles[p]);
    }
  } else if (seg->mode == SymmMode::CUDA_IPC) {
    for (void* p : seg->ipc_opened) {
      cudaIpcCloseMemHandle(p);
    }
    if (seg->owns_local) cudaFree(seg->local());
  } else if (seg->owns_local && !seg->peer_ptrs.empty()) {
    cuda_->freeDevice(seg->peer_ptrs[0]);
  }
  seg->peer_ptrs.clear();
  seg->handles.clear();
  seg->ipc_opened.clear();
}

// ---------------------------------------------------- ExportableRegistry ----

ExportableRegistry& ExportableRegistry::get() {
  static ExportableRegistry* inst = new ExportableRegistry();
  return *inst;
}

void ExportableRegistry::add(const ExportableAlloc& a) {
  std::lock_guard<std::mutex> g(mu_);
  allocs_[a.base] = a;
}

bool ExportableRegistry::remove(CUdeviceptr base, ExportableAlloc* out) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = allocs_.find(base);
  if (it == allocs_.end()) return false;
  if (out) *out = it->second;
  allocs_.erase(it);
  return true;
}

bool ExportableRegistry::find(const void* ptr, size_t bytes, ExportableAlloc* out) const {
  std::lock_guard<std::mutex> g(mu_);
  const CUdeviceptr p = reinterpret_cast<CUdeviceptr>(ptr);
  auto it = allocs_.upper_bound(p);
  if (it == allocs_.begin()) return false;
  --it;
  if (p >= it->second.base && p + bytes <= it->second.base + it->second.bytes) {
    if (out) *out = it->second;
    return true;
  }
  return false;
}

size_t ExportableRegistry::live() const {
  std::lock_guard<std::mutex> g(mu_);
  return allocs_.size();
}

} // namespace b200c

// Allocator entry points for torch.cuda.memory.CUDAPluggableAllocator: memory
// that a later window registration can export to the peers.
extern "C" __attribute__((visibility("default"))) void* b200c_symm_alloc(size_t size, int device, void* /*stream*/) {
  using namespace b200c;
  auto drv = DriverApi::real();
  if (size == 0) size = 1;
  if (cudaSetDevice(device) != cudaSuccess || !drv->available()) return nullptr;
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  if (drv->memGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) {
    return nullptr;
  }
  const size_t bytes = (size + gran - 1) / gran * gran;
  ExportableAlloc a;
  a.bytes = bytes;
  a.device = device;
  if (drv->memCreate(&a.handle, bytes, &prop) != CUDA_SUCCESS) return nullptr;
  if (drv->memAddressReserve(&a.base, bytes, gran) != CUDA_SUCCESS) {
    drv->memRelease(a.handle);
    return nullptr;
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (drv->memMap(a.base, bytes, 0, a.handle) != CUDA_SUCCESS ||
      drv->memSetAccess(a.base, bytes, &acc, 1) != CUDA_SUCCESS) {
    drv->memAddressFree(a.base, bytes);
    drv->memRelease(a.handle);
    return nullptr;
  }
  ExportableRegistry::get().add(a);
  return reinterpret_cast<void*>(a.base);
}

extern "C" __attribute__((visibility("default"))) void b200c_symm_free(void* ptr, size_t /*size*/, int /*device*/, void* /*stream*/) {
  using namespace b200c;
  ExportableAlloc a;
  if (!ExportableRegistry::get().remove(reinterpret_cast<CUdeviceptr>(ptr), &a)) return;
  auto drv = DriverApi::real();
  drv->memUnmap(a.base, a.bytes);
  drv->memAddressFree(a.base, a.bytes);
  drv->memRelease(a.handle);
}
