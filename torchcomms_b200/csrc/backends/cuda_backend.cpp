// CUDA backend: bootstrap, stream/event protocol, watchdog, algorithm choice.
#include "cuda_backend.hpp"

#include <unistd.h>

#include <cstdio>
#include <fstream>
#include <limits>
#include <sstream>
#include <random>
#include <tuple>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstring>

#include "../core/logging.hpp"
#include "../kernels/fused_ops.h"
#include "../kernels/window.h"

namespace b200c {

namespace {

// Makes `device` current for the calling thread while in scope; a no-op when
// the runtime behind `api` is a test fake (no CUDA context exists then).
class DeviceScope {
 public:
  DeviceScope(const std::shared_ptr<CudaApi>& api, int device) {
    if (api->is_real()) guard_.emplace(static_cast<c10::DeviceIndex>(device));
  }

 private:
  std::optional<c10::cuda::CUDAGuard> guard_;
};

size_t round_up(size_t v, size_t to) {
  return (v + to - 1) / to * to;
}

constexpr size_t kMetaBytes = static_cast<size_t>(kMaxBlocks) * kMaxRanks * kMaxRanks * sizeof(uint64_t);
constexpr size_t kSmallBytes = 2 * static_cast<size_t>(kSmallBlocks) * kSmallPiece + kMetaBytes;
constexpr size_t kFlagBytes = static_cast<size_t>(kFlagSets) * kMaxBlocks * kMaxRanks * sizeof(uint32_t);

bool to_dtype(at::ScalarType t, DType* out) {
  switch (t) {
    case at::kFloat: *out = DType::F32; return true;
    case at::kHalf: *out = DType::F16; return true;
    case at::kBFloat16: *out = DType::BF16; return true;
    default: return false;
  }
}

bool to_nccl_dtype(at::ScalarType t, NcclDataType* out) {
  switch (t) {
    case at::kChar: *out = kNcclInt8; return true;
    case at::kByte: *out = kNcclUint8; return true;
    case at::kBool: *out = kNcclUint8; return true;
    case at::kInt: *out = kNcclInt32; return true;
    case at::kLong: *out = kNcclInt64; return true;
    case at::kHalf: *out = kNcclFloat16; return true;
    case at::kFloat: *out = kNcclFloat32; return true;
    case at::kDouble: *out = kNcclFloat64; return true;
    case at::kBFloat16: *out = kNcclBfloat16; return true;
    case at::kFloat8_e4m3fn: *out = kNcclFloat8e4m3; return true;
    case at::kFloat8_e5m2: *out = kNcclFloat8e5m2; return true;
    case at::kUInt32: *out = kNcclUint32; return true;
    case at::kUInt64: *out = kNcclUint64; return true;
    default: return false;
  }
}

// `real` is false under a test fake of the runtime, where tensors live on the host.
void check_tensor(const at::Tensor& t, const at::Device& dev, const char* what, bool real = true) {
  TORCH_CHECK(t.defined(), what, ": undefined tensor");
  TORCH_CHECK(t.is_contiguous(), "Tensor must be contiguous for ", what);
  TORCH_CHECK(!real || t.device() == dev, what, ": tensor is on ", t.device(), " but the communicator lives on ", dev);
}

Algo parse_algo(std::string s) {
  for (auto& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  if (s == "oneshot" || s == "one_shot") return Algo::ONESHOT;
  if (s == "twoshot" || s == "two_shot") return Algo::TWOSHOT;
  if (s == "staged") return Algo::STAGED;
  if (s == "kernel" || s == "kernels" || s == "own") return Algo::KERNEL;
  if (s == "nccl" || s == "orig") return Algo::NCCL;
  return Algo::AUTO;
}

} // namespace

// ------------------------------------------------------------- CudaWork ----

CudaWork::CudaWork(std::shared_ptr<CudaApi> api, cudaEvent_t start, cudaEvent_t end, bool pooled, int device,
                   Millis timeout, std::vector<at::Tensor> keep_alive, std::weak_ptr<CudaBackend> owner,
                   bool in_capture, cudaStream_t stream)
    : api_(std::move(api)), start_(start), end_(end), pooled_(pooled), device_(device),
      keep_alive_(std::move(keep_alive)), owner_(std::move(owner)), in_capture_(in_capture), stream_(stream) {
  set_timeout(timeout);
}

CudaWork::~CudaWork() {
  if ((start_ == nullptr && end_ == nullptr) || in_capture_) {
    return;  // nothing recorded, or events owned by the graph's bookkeeping
  }
  auto o = owner_.lock();
  if (pooled_ && o) {
    o->recycle_events(start_, end_);
  } else {
    if (start_) api_->eventDestroy(start_);
    if (end_) api_->eventDestroy(end_);
  }
}

void CudaWork::release_events(cudaEvent_t* start, cudaEvent_t* end) {
  *start = start_;
  *end = end_;
  start_ = nullptr;
  end_ = nullptr;
}

bool CudaWork::poll(std::chrono::steady_clock::time_point now) {
  std::lock_guard<std::mutex> g(poll_mu_);
  const WorkStatus s = status();
  if (s == WorkStatus::COMPLETED || s == WorkStatus::TIMEDOUT || s == WorkStatus::ERROR) {
    return true;
  }
  if (start_ == nullptr || end_ == nullptr) {
    return true;  // event-less work: nothing to follow
  }
  if (!started_seen_) {
    const cudaError_t q = api_->eventQuery(start_);
    if (q == cudaSuccess) {
      started_seen_ = true;
      started_at_ = now;
      set_status(WorkStatus::INPROGRESS);
    } else if (q != cudaErrorNotReady) {
      set_error(std::string("start event: ") + api_->errorString(q));
      set_status(WorkStatus::ERROR);
      return true;
    }
  }
  if (started_seen_) {
    const cudaError_t q = api_->eventQuery(end_);
    if (q == cudaSuccess) {
      set_status(WorkStatus::COMPLETED);
      return true;
    }
    if (q != cudaErrorNotReady) {
      set_error(std::string("end event: ") + api_->errorString(q));
      set_status(WorkStatus::ERROR);
      return true;
    }
    const Millis t = timeout();
    if (t != kNoTimeout && now - started_at_ > t) {
      set_error("no completion " + std::to_string(t.count()) + " ms after the operation started on the device");
      set_status(WorkStatus::TIMEDOUT);
      return true;
    }
  }
  return false;
}

void CudaWork::do_wait() {
  // Stream-ordered: the caller's current stream waits for the end event.
  DeviceScope guard(api_, device_);
  cudaStream_t cur = api_->currentStream(device_);
  if (end_ != nullptr) {
    const cudaError_t e = api_->streamWaitEvent(cur, end_);
    if (e != cudaSuccess) {
      set_error(std::string("cudaStreamWaitEvent: ") + api_->errorString(e));
      set_status(WorkStatus::ERROR);
    }
  } else if (!in_capture_) {
    // Event-less synchronous operation: the caller's stream is already behind it.
    set_status(WorkStatus::COMPLETED);
  }
  keep_alive_.clear();
}

void CudaWork::do_wait_blocking() {
  do_wait();
  if (in_capture_) {
    return;
  }
  if (end_ == nullptr) {
    // Event-less synchronous operation: everything up to now on its stream.
    if (stream_ != nullptr || device_ >= 0) {
      DeviceScope guard(api_, device_);
      const cudaError_t e = api_->streamSynchronize(stream_);
      if (e != cudaSuccess) {
        set_error(std::string("cudaStreamSynchronize: ") + api_->errorString(e));
        set_status(WorkStatus::ERROR);
        return;
      }
    }
    set_status(WorkStatus::COMPLETED);
    return;
  }
  // Host-blocking with the work's own deadline.
  const auto t0 = std::chrono::steady_clock::now();
  while (true) {
    const cudaError_t q = api_->eventQuery(end_);
    if (q == cudaSuccess) {
      set_status(WorkStatus::COMPLETED);
      return;
    }
    if (q != cudaErrorNotReady) {
      set_error(std::string("end event: ") + api_->errorString(q));
      set_status(WorkStatus::ERROR);
      return;
    }
    const WorkStatus s = status();
    if (s == WorkStatus::TIMEDOUT || s == WorkStatus::ERROR) {
      return;
    }
    const Millis t = timeout();
    if (t != kNoTimeout && std::chrono::steady_clock::now() - t0 > t + Millis(1000)) {
      set_error("host wait exceeded the operation timeout");
      set_status(WorkStatus::TIMEDOUT);
      return;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

// ---------------------------------------------------------- CudaBackend ----

CudaBackend::CudaBackend(std::string registered_as) : registered_as_(std::move(registered_as)) {
  drv_ = DriverApi::current();
  cuda_ = CudaApi::current();
  nccl_ = NcclApi::current();
}

CudaBackend::~CudaBackend() {
  if (initialized_ && !finalized_) {
    B200C_LOG(WARN, name_, "CUDA communicator destroyed without finalize(); tearing down");
    try {
      finalize();
    } catch (const std::exception& e) {
      B200C_LOG(ERROR, name_, "teardown failed: " << e.what());
    }
  }
}

std::string CudaBackend::backend_version() const {
  return std::string(kBackendAbiVersion) + "+nccl" + (nccl_ && nccl_->available() ? nccl_->version() : "-none");
}

void CudaBackend::parse_tuning(const Hints& h) {
  Tuning t = tune_;
  t.staging_bytes = static_cast<size_t>(hint_or<double>(h, "staging_mb", env_to_value<double>("B200COMMS_STAGING_MB", t.staging_bytes / 1048576.0)) * 1048576.0);
  t.oneshot_max_bytes = hint_or<size_t>(h, "oneshot_max_bytes", env_to_value<size_t>("B200COMMS_ONESHOT_MAX_BYTES", t.oneshot_max_bytes));
  t.max_blocks = hint_or<int>(h, "max_blocks", env_to_value<int>("B200COMMS_MAX_BLOCKS", t.max_blocks));
  t.threads = hint_or<int>(h, "threads", env_to_value<int>("B200COMMS_THREADS", t.threads));
  t.max_chunk_bytes = hint_or<size_t>(h, "max_chunk_bytes", env_to_value<size_t>("B200COMMS_MAX_CHUNK_BYTES", t.max_chunk_bytes));
  t.use_multicast = hint_or<bool>(h, "use_multicast", env_to_value<bool>("B200COMMS_NVLS", t.use_multicast));
  t.use_nccl = hint_or<bool>(h, "use_nccl", env_to_value<bool>("B200COMMS_USE_NCCL", t.use_nccl));
  t.force = parse_algo(hint_or<std::string>(h, "algo", env_to_value<std::string>("B200COMMS_ALGO", "auto")));
  t.device_wait_ns = static_cast<unsigned long long>(
      hint_or<double>(h, "device_wait_ms", env_to_value<double>("B200COMMS_DEVICE_WAIT_MS", t.device_wait_ns / 1.0e6)) * 1.0e6);
  t.watchdog_interval_ms = hint_or<int>(h, "garbage_collect_interval_ms", t.watchdog_interval_ms);
  t.max_event_pool = hint_or<size_t>(h, "max_event_pool_size", t.max_event_pool);
  // The reference's variable name is honoured as well (TorchCommNCCLX graph monitoring switch).
  t.graph_timeout_monitoring = hint_or<bool>(
      h, "graph_timeout_monitoring",
      env_to_value<bool>("B200COMMS_GRAPH_TIMEOUT_MONITORING",
                         env_to_value<bool>("TORCHCOMM_NCCLX_GRAPH_TIMEOUT_MONITORING", t.graph_timeout_monitoring)));
  t.max_blocks = std::max(1, std::min(t.max_blocks, kMaxBlocks));
  t.threads = std::max(32, std::min(t.threads, 256));
  t.ag_oneshot_max_bytes = hint_or<size_t>(h, "ag_oneshot_max_bytes", env_to_value<size_t>("B200COMMS_AG_ONESHOT_MAX_BYTES", t.ag_oneshot_max_bytes));
  t.rs_oneshot_max_bytes = hint_or<size_t>(h, "rs_oneshot_max_bytes", env_to_value<size_t>("B200COMMS_RS_ONESHOT_MAX_BYTES", t.rs_oneshot_max_bytes));
  t.ag_push_min_ranks = hint_or<int>(h, "ag_push_min_ranks", env_to_value<int>("B200COMMS_AG_PUSH_MIN_RANKS", t.ag_push_min_ranks));
  t.a2av_blocks = hint_or<int>(h, "a2av_blocks", env_to_value<int>("B200COMMS_A2AV_BLOCKS", t.a2av_blocks));
  t.auto_nccl = hint_or<bool>(h, "auto_nccl", env_to_value<bool>("B200COMMS_AUTO_NCCL", t.auto_nccl));
  t.tuner_file = hint_or<std::string>(h, "tuner_file", env_to_value<std::string>("B200COMMS_TUNER_FILE", t.tuner_file));
  t.steps_per_block = hint_or<int>(h, "steps_per_block", env_to_value<int>("B200COMMS_STEPS_PER_BLOCK", t.steps_per_block));
  t.symm_blocks = hint_or<int>(h, "symm_blocks", env_to_value<int>("B200COMMS_SYMM_BLOCKS", t.symm_blocks));
  t.symm_blocks_nomc = hint_or<int>(h, "symm_blocks_nomc", env_to_value<int>("B200COMMS_SYMM_BLOCKS_NOMC", t.symm_blocks_nomc));
  t.symm_ag_mc = hint_or<int>(h, "symm_ag_mc", env_to_value<int>("B200COMMS_SYMM_AG_MC", t.symm_ag_mc));
  t.symm_rs_mc = hint_or<int>(h, "symm_rs_mc", env_to_value<int>("B200COMMS_SYMM_RS_MC", t.symm_rs_mc));
  t.symm_ar_mc = hint_or<int>(h, "symm_ar_mc", env_to_value<int>("B200COMMS_SYMM_AR_MC", t.symm_ar_mc));
  t.symm_blocks = std::max(1, std::min(t.symm_blocks, 128));
  t.symm_blocks_nomc = std::max(1, std::min(t.symm_blocks_nomc, 128));
  t.symm_blocks_ld = hint_or<int>(h, "symm_blocks_ld", env_to_value<int>("B200COMMS_SYMM_BLOCKS_LD", t.symm_blocks_ld));
  t.symm_blocks_ld = std::max(1, std::min(t.symm_blocks_ld, 132));
  t.lamport_max_bytes = hint_or<size_t>(h, "lamport_max_bytes", env_to_value<size_t>("B200COMMS_LAMPORT_MAX_BYTES", t.lamport_max_bytes));
  t.lamport_max_bytes = std::min(t.lamport_max_bytes, static_cast<size_t>(kLamportBlocks) * kLamportPiece);
  t.channel_streams = hint_or<bool>(h, "channel_streams", env_to_value<bool>("B200COMMS_CHANNEL_STREAMS", t.channel_streams));
  t.fast_sync = hint_or<bool>(h, "fast_sync", env_to_value<bool>("B200COMMS_FAST_SYNC", t.fast_sync));
  t.colltrace = std::max(0, std::min(1 << 16, hint_or<int>(h, "colltrace", env_to_value<int>("B200COMMS_COLLTRACE", t.colltrace))));
  t.staging_bytes = std::max<size_t>(t.staging_bytes, 1u << 20);
  const bool reload = t.tuner_file != tune_.tuner_file;
  tune_ = t;
  if (reload) {
    for (auto& rules : tuner_rules_) rules.clear();
    if (!tune_.tuner_file.empty()) load_tuner_file(tune_.tuner_file);
  }
}

void CudaBackend::set_hints(const Hints& h) {
  // Only knobs that do not change memory layout may move after init.
  Tuning before = tune_;
  parse_tuning(h);
  tune_.staging_bytes = before.staging_bytes;
  tune_.use_nccl = before.use_nccl;
  tune_.channel_streams = before.channel_streams;
  for (auto& kv : h) {
    opts_.hints[kv.first] = kv.second;
  }
}

void CudaBackend::init(at::Device device, const std::string& name, const CommOptions& opts) {
  TORCH_CHECK(device.is_cuda(), "the '", registered_as_, "' backend needs a CUDA device, got ", device);
  int rank = 0, size = 1;
  if (opts.enable_reconfigure) {
    try {
      std::tie(rank, size) = query_ranksize();
    } catch (const std::exception&) {
      rank = 0;  // candidates need not come from one launcher
    }
  } else {
    std::tie(rank, size) = query_ranksize();
  }
  int ndev = 0;
  B200C_CUDA_CHECK(cuda_->getDeviceCount(&ndev));
  TORCH_CHECK(ndev > 0, "no CUDA device is visible");
  const int index = device.has_index() && device.index() >= 0 ? device.index() : rank % ndev;
  device_ = at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(index));
  name_ = name;
  opts_ = opts;
  parse_tuning(opts.hints);
  {
    // "<launcher rank>:<unique id>.<name>:<host>:<pid>", shown behind the backend name by get_init_handle().
    std::random_device rd;
    char host[256] = {0};
    gethostname(host, sizeof(host) - 1);
    char uid[32];
    std::snprintf(uid, sizeof(uid), "%08x%08x", static_cast<unsigned>(rd()), static_cast<unsigned>(rd()));
    handle_token_ = std::to_string(rank) + ":" + uid + "." + name + ":" + std::string(host) + ":" + std::to_string(getpid());
  }
  if (opts.enable_reconfigure) {
    // Membership arrives with reconfigure(); until then the communicator owns no device resources.
    TORCH_CHECK(opts.store, "enable_reconfigure needs a store shared by all candidate ranks");
    rank_ = -1;
    size_ = 0;
    return;
  }
  auto store = opts.store ? scoped_store(opts.store, "b200c/cuda/" + name)
                          : create_prefix_store("b200c/cuda/" + name, rank, size, opts.timeout);
  bootstrap(store, rank, size);
}

void CudaBackend::bootstrap(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size) {
  TORCH_CHECK(size >= 1 && size <= kMaxRanks, "the CUDA backend supports 1..", kMaxRanks, " ranks per communicator, got ", size);
  rank_ = rank;
  size_ = size;
  store_ = store;
  DeviceScope guard(cuda_, device_.index());
  B200C_CUDA_CHECK(cuda_->setDevice(device_.index()));

  symm_ = std::make_unique<SymmMemory>(store_, rank_, size_, device_.index(), drv_, opts_.timeout, tune_.use_multicast, cuda_);
  layout_.bulk_off = 0;
  layout_.bulk_bytes = round_up(tune_.staging_bytes, 4096);
  layout_.small_off = layout_.bulk_off + layout_.bulk_bytes;
  layout_.small_bytes = round_up(kSmallBytes, 4096);
  layout_.symm_meta_off = layout_.small_off + layout_.small_bytes;
  layout_.symm_meta_bytes = round_up(kSymmMetaBytes, 4096);
  layout_.lamport_off = layout_.symm_meta_off + layout_.symm_meta_bytes;
  layout_.lamport_bytes = round_up(kLamportBytes, 4096);
  const size_t flags_off = layout_.lamport_off + layout_.lamport_bytes;
  const size_t total = flags_off + round_up(kFlagBytes, 4096);
  heap_ = symm_->allocate(total, tune_.use_multicast);

  std::memset(&dev_, 0, sizeof(dev_));
  dev_.rank = rank_;
  dev_.nranks = size_;
  for (int p = 0; p < size_; ++p) {
    dev_.heap[p] = heap_->peer_ptrs[p];
    dev_.flags[p] = reinterpret_cast<uint32_t*>(heap_->peer_ptrs[p] + flags_off);
  }
  dev_.mc_heap = heap_->mc_ptr;
  dev_.mc_flags = heap_->mc_ptr ? reinterpret_cast<uint32_t*>(heap_->mc_ptr + flags_off) : nullptr;
  dev_.heap_bytes = total;
  dev_.timeout_ns = tune_.device_wait_ns;

  const size_t epoch_bytes = static_cast<size_t>(kFlagSets) * kMaxBlocks * sizeof(uint32_t);
  B200C_CUDA_CHECK(cuda_->mallocDevice(reinterpret_cast<void**>(&epochs_dev_), epoch_bytes));
  B200C_CUDA_CHECK(cuda_->memsetDevice(epochs_dev_, 0, epoch_bytes));
  dev_.epochs = epochs_dev_;
  B200C_CUDA_CHECK(cuda_->hostAllocMapped(reinterpret_cast<void**>(&status_host_), reinterpret_cast<void**>(&status_dev_), 64));
  std::memset(status_host_, 0, 64);
  dev_.status = status_dev_;
  B200C_CUDA_CHECK(cuda_->hostAllocMapped(reinterpret_cast<void**>(&replay_pool_host_),
                                          reinterpret_cast<void**>(&replay_pool_dev_),
                                          2 * kMaxGraphEntries * sizeof(unsigned long long)));
  std::memset(replay_pool_host_, 0, 2 * kMaxGraphEntries * sizeof(unsigned long long));
  if (tune_.colltrace > 0) {
    const size_t bytes = 2 * static_cast<size_t>(tune_.colltrace) * sizeof(unsigned long long);
    B200C_CUDA_CHECK(cuda_->hostAllocMapped(reinterpret_cast<void**>(&trace_ring_host_), reinterpret_cast<void**>(&trace_ring_dev_), bytes));
    std::memset(trace_ring_host_, 0, bytes);
    trace_meta_.assign(tune_.colltrace, {0, std::string()});
    trace_next_ = 0;
  }

  int lo = 0, hi = 0;
  B200C_CUDA_CHECK(cuda_->streamPriorityRange(&lo, &hi));
  for (int ch = 0; ch < kChanCount; ++ch) {
    ChanState& cs = chans_[ch];
    cs = ChanState{};
    if (ch == kChanMain || tune_.channel_streams) {
      B200C_CUDA_CHECK(cuda_->streamCreateWithPriority(&cs.stream, cudaStreamNonBlocking,
                                                       opts_.is_high_priority_stream ? hi : lo));
      cs.owns_stream = true;
    } else {
      cs.stream = chans_[kChanMain].stream;
    }
    B200C_CUDA_CHECK(cuda_->eventCreate(&cs.order_event, cudaEventDisableTiming));
  }
  internal_stream_ = chans_[kChanMain].stream;
  B200C_CUDA_CHECK(cuda_->eventCreate(&dep_event_, cudaEventDisableTiming));
  // The flag-less all-reduce starts from buffers full of its "nothing here yet" word.
  if (cuda_->is_real()) {
    B200C_CUDA_CHECK(launch_lamport_init(heap_->local() + layout_.lamport_off, internal_stream_));
  } else {
    cuda_->noteLaunch("lamport_init", internal_stream_);
  }
  B200C_CUDA_CHECK(cuda_->deviceSynchronize());
  if (size_ > 1) {
    // Nobody sends before every rank's buffers are prepared.
    store_barrier(*store_, "lamport_ready", rank_, size_, opts_.timeout);
  }

  if (size_ > 1 && tune_.use_nccl) {
    init_nccl();
  }
  initialized_ = true;
  start_watchdog();
  B200C_LOG(INFO, name_, "rank " << rank_ << "/" << size_ << " on " << device_ << ": staging "
                                 << (layout_.bulk_bytes >> 20) << " MiB, multicast " << (dev_.mc_heap != nullptr)
                                 << ", nccl " << (nccl_comm_ != nullptr));
}

void CudaBackend::nccl_check(NcclResult r, const char* what) const {
  if (r != kNcclSuccess && r != kNcclInProgress) {
    throw std::runtime_error(std::string(what) + " failed: " + nccl_->errorString(r));
  }
}

void CudaBackend::init_nccl() {
  if (!nccl_->available()) {
    B200C_LOG(WARN, name_, "libnccl is not loadable: point-to-point operations will be unavailable");
    return;
  }
  NcclUniqueId id{};
  if (rank_ == 0) {
    nccl_check(nccl_->getUniqueId(&id), "ncclGetUniqueId");
    store_set_string(*store_, "nccl_uid", std::string(id.internal, sizeof(id.internal)));
  } else {
    const std::string raw = store_get_string(*store_, "nccl_uid");
    TORCH_CHECK(raw.size() == sizeof(id.internal), "malformed NCCL unique id in the store");
    std::memcpy(id.internal, raw.data(), sizeof(id.internal));
  }
  const NcclConfig cfg = nccl_config_from_hints(opts_.hints, name_);
  nccl_check(nccl_->commInitRankConfig(&nccl_comm_, size_, id, rank_, cfg), "ncclCommInitRankConfig");
}

// Hints that name a field of ncclConfig_t go to NCCL when the communicator is
// created (camelCase as in nccl.h, or snake_case). Parity:
// comms/torchcomms/ncclx/TorchCommNCCLXBootstrap.cpp:218-321.
NcclConfig CudaBackend::nccl_config_from_hints(const Hints& h, const std::string& comm_name) {
  NcclConfig c;
  auto num = [&h](std::initializer_list<const char*> keys, int* out) {
    for (const char* k : keys) {
      auto it = h.find(k);
      if (it == h.end()) continue;
      const std::string& v = it->second;
      if (v == "true" || v == "True") {
        *out = 1;
      } else if (v == "false" || v == "False") {
        *out = 0;
      } else {
        size_t used = 0;
        int parsed = 0;
        try {
          parsed = std::stoi(v, &used);
        } catch (const std::exception&) {
          used = 0;
        }
        TORCH_CHECK(used == v.size() && !v.empty(), "hint '", k, "' must be an integer, got '", v, "'");
        *out = parsed;
      }
    }
  };
  num({"blocking"}, &c.blocking);
  num({"cgaClusterSize", "cga_cluster_size"}, &c.cgaClusterSize);
  num({"minCTAs", "min_ctas"}, &c.minCTAs);
  num({"maxCTAs", "max_ctas"}, &c.maxCTAs);
  num({"splitShare", "split_share"}, &c.splitShare);
  num({"trafficClass", "traffic_class"}, &c.trafficClass);
  num({"collnetEnable", "collnet_enable"}, &c.collnetEnable);
  num({"CTAPolicy", "cta_policy"}, &c.CTAPolicy);
  num({"shrinkShare", "shrink_share"}, &c.shrinkShare);
  num({"nvlsCTAs", "nvls_ctas"}, &c.nvlsCTAs);
  num({"nChannelsPerNetPeer", "n_channels_per_net_peer"}, &c.nChannelsPerNetPeer);
  num({"nvlinkCentricSched", "nvlink_centric_sched"}, &c.nvlinkCentricSched);
  auto it = h.find("netName");
  if (it != h.end()) c.netName = it->second;
  it = h.find("commName");
  if (it != h.end()) {
    c.commName = it->second;
  } else if (c.any()) {
    c.commName = comm_name;  // NCCL's own logs then carry the communicator's name
  }
  return c;
}

void CudaBackend::check_usable() const {
  TORCH_CHECK(initialized_, "communicator '", name_, "' is not initialised");
  TORCH_CHECK(!finalized_, "communicator '", name_, "' was finalized");
  if (failed_.load()) {
    throw std::runtime_error("communicator '" + name_ + "' is unusable after a failure: " + failure_text_);
  }
  TORCH_CHECK(!aborted_.load(), "communicator '", name_, "' was aborted");
}

void CudaBackend::on_failure(const std::string& what, bool timed_out) {
  bool expected = false;
  if (!failed_.compare_exchange_strong(expected, true)) {
    return;
  }
  failure_text_ = (timed_out ? "operation timed out: " : "operation failed: ") + what;
  HealthCheck::mark_unhealthy(name_ + ": " + failure_text_);
  B200C_LOG(ERROR, name_, failure_text_);
  if (status_host_ != nullptr) {
    // Kernels that are still waiting see this and fall through to their exit.
    reinterpret_cast<volatile uint32_t*>(status_host_)[0] |= kStatusAbort;
  }
  run_abort_hooks();
  if (opts_.abort_process_on_timeout_or_error) {
    B200C_LOG(ERROR, name_, "aborting the process (abort_process_on_timeout_or_error is set)");
    std::abort();
  }
  aborted_ = true;
}

void CudaBackend::abort() {
  aborted_ = true;
  if (status_host_ != nullptr) {
    reinterpret_cast<volatile uint32_t*>(status_host_)[0] |= kStatusAbort;
  }
  if (nccl_comm_ != nullptr) {
    nccl_->commAbort(nccl_comm_);
    nccl_comm_ = nullptr;
  }
  run_abort_hooks();
}

std::pair<cudaEvent_t, cudaEvent_t> CudaBackend::take_events() {
  cudaEvent_t a = nullptr, b = nullptr;
  {
    std::lock_guard<std::mutex> g(pool_mu_);
    if (event_pool_.size() >= 2) {
      a = event_pool_.back();
      event_pool_.pop_back();
      b = event_pool_.back();
      event_pool_.pop_back();
    }
  }
  if (a == nullptr) {
    B200C_CUDA_CHECK(cuda_->eventCreate(&a, cudaEventDisableTiming));
    B200C_CUDA_CHECK(cuda_->eventCreate(&b, cudaEventDisableTiming));
  }
  return {a, b};
}

void CudaBackend::give_events(cudaEvent_t a, cudaEvent_t b) {
  std::lock_guard<std::mutex> g(pool_mu_);
  for (cudaEvent_t e : {a, b}) {
    if (e == nullptr) continue;
    if (event_pool_.size() < tune_.max_event_pool && !finalized_) {
      event_pool_.push_back(e);
    } else {
      cuda_->eventDestroy(e);
    }
  }
}

namespace {
// Handed to the CUDA user object that rides on a captured graph; freed by the callback.
struct GraphReleaseNote {
  std::weak_ptr<CudaBackend> owner;
  unsigned long long graph_id;
};
void CUDART_CB on_graph_destroyed(void* arg) {
  // Runs on a driver thread once the graph and all its executables are gone.
  // No CUDA calls here: only leave a note for the watchdog.
  auto* note = static_cast<GraphReleaseNote*>(arg);
  if (auto owner = note->owner.lock()) {
    owner->note_graph_released(note->graph_id);
  }
  delete note;
}
} // namespace

void CudaBackend::note_graph_released(unsigned long long graph_id) {
  std::lock_guard<std::mutex> g(released_mu_);
  released_ids_.push_back(graph_id);
}

WorkPtr CudaBackend::run(const char* what, bool async_op, const OpOptions& o, std::vector<at::Tensor> keep_alive,
                         const std::function<void(cudaStream_t)>& launch, int chan, bool own_kernel, int sm_blocks) {
  check_usable();
  DeviceScope guard(cuda_, device_.index());
  cudaStream_t current = cuda_->currentStream(device_.index());
  ChanState& cs = chans_[chan];
  cudaStream_t stream = async_op ? cs.stream : current;
  bool capturing = false;
  unsigned long long graph_id = 0;
  cuda_->streamIsCapturing(current, &capturing, &graph_id);

  if (async_op) {
    B200C_CUDA_CHECK(cuda_->eventRecord(dep_event_, current));
    B200C_CUDA_CHECK(cuda_->streamWaitEvent(cs.stream, dep_event_));
  }
  if (capturing) {
    // Inside a capture every operation of the communicator follows the one
    // captured before it, whatever their channels and streams. Unordered
    // branches of one graph may be started in a different order on different
    // ranks; two kernels that each wait for their peers (an NCCL kernel and a
    // peer-memory kernel, say) could then wait for each other for good.
    std::lock_guard<std::mutex> g(wd_mu_);
    auto it = capture_tail_.find(graph_id);
    if (it != capture_tail_.end() && it->second.stream != stream) {
      B200C_CUDA_CHECK(cuda_->streamWaitEvent(stream, it->second.end));
    }
  } else if (cs.last_stream != nullptr && cs.last_stream != stream) {
    // Operations of one channel share staging slots and flags: keep them in
    // issue order across streams.
    if (cs.last_work) {
      B200C_CUDA_CHECK(cuda_->streamWaitEvent(stream, cs.last_work->end_event()));
    } else {
      // The previous operation recorded no event: mark its stream now.
      B200C_CUDA_CHECK(cuda_->eventRecord(cs.order_event, cs.last_stream));
      B200C_CUDA_CHECK(cuda_->streamWaitEvent(stream, cs.order_event));
    }
  }
  if (sm_blocks > 0 && !capturing) {
    // Blocks of the one-pass kernels hold an SM each while they wait for the same block of every peer. Kernels
    // of different channels run side by side, and each GPU starts their blocks in an order of its own: if
    // together they could hold more SMs than there are, one rank may fill up with blocks of kernel A and another
    // with blocks of kernel B, each waiting for peer blocks that find no SM. So a kernel that would push the sum
    // over the budget first waits for the other channels' latest kernels. The rule looks only at the order of
    // issue and at grid sizes, which are the same on every rank.
    constexpr int kSmBudget = 140;
    int others = 0;
    for (int ch = 0; ch < kChanCount; ++ch) {
      if (ch != chan) others += chans_[ch].sm_blocks;
    }
    if (others + sm_blocks > kSmBudget) {
      for (int ch = 0; ch < kChanCount; ++ch) {
        ChanState& other = chans_[ch];
        if (ch == chan || other.sm_blocks == 0 || other.last_stream == nullptr || other.last_stream == stream) continue;
        if (other.last_work) {
          B200C_CUDA_CHECK(cuda_->streamWaitEvent(stream, other.last_work->end_event()));
        } else {
          B200C_CUDA_CHECK(cuda_->eventRecord(other.order_event, other.last_stream));
          B200C_CUDA_CHECK(cuda_->streamWaitEvent(stream, other.order_event));
        }
      }
    }
    cs.sm_blocks = sm_blocks;
  }

  auto self = std::static_pointer_cast<CudaBackend>(shared_from_this());
  if (own_kernel && !async_op && !capturing && tune_.fast_sync && !observed()) {
    // Nobody follows this operation through work hooks, stream order gives
    // wait() its meaning, and a failed device wait shows in the status word
    // the watchdog reads: no events, nothing queued.
    const int64_t tslot = colltrace_begin(what, stream);
    if (cuda_->is_real()) {
      launch(stream);
    } else {
      cuda_->noteLaunch(what, stream);
    }
    colltrace_end(tslot, stream);
    cs.last_stream = stream;
    cs.last_work.reset();
    ops_issued_++;
    {
      std::lock_guard<std::mutex> g(wd_mu_);
      algo_counts_[what]++;
    }
    return c10::make_intrusive<CudaWork>(cuda_, nullptr, nullptr, false, device_.index(), effective_timeout(o),
                                         std::vector<at::Tensor>{}, self, false, stream);
  }

  cudaEvent_t ev_start = nullptr, ev_end = nullptr;
  unsigned long long* replay_counters = nullptr;  // device alias of this collective's replay counters
  if (capturing) {
    // Resource creation is not a capturable operation: step out of the strict
    // capture mode for these calls.
    cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
    cuda_->exchangeCaptureMode(&mode);
    const cudaError_t e1 = cuda_->eventCreate(&ev_start, cudaEventDisableTiming);
    const cudaError_t e2 = cuda_->eventCreate(&ev_end, cudaEventDisableTiming);
    cudaError_t e3 = cudaSuccess;
    bool need_retain = false;
    {
      std::lock_guard<std::mutex> g(wd_mu_);
      need_retain = !graphs_[graph_id].retained;
      graphs_[graph_id].retained = true;
    }
    if (need_retain) {
      // When the graph (and every executable made from it) is destroyed, its
      // entries are released: see the watchdog.
      cudaGraph_t graph = nullptr;
      e3 = cuda_->streamCaptureGraph(current, &graph);
      if (e3 == cudaSuccess && graph != nullptr) {
        auto* note = new GraphReleaseNote{self, graph_id};
        e3 = cuda_->graphRetainCallback(graph, on_graph_destroyed, note);
        if (e3 != cudaSuccess) delete note;
      }
    }
    cuda_->exchangeCaptureMode(&mode);
    B200C_CUDA_CHECK(e1);
    B200C_CUDA_CHECK(e2);
    B200C_CUDA_CHECK(e3);

    GraphEntry e{};
    e.graph_id = graph_id;
    e.stream = reinterpret_cast<uintptr_t>(stream);
    e.timeout = effective_timeout(o);
    std::lock_guard<std::mutex> g(wd_mu_);
    GraphState& gs = graphs_[graph_id];
    gs.events.push_back(ev_start);
    gs.events.push_back(ev_end);
    e.index = gs.next_index++;
    if (free_slots_.empty()) {
      TORCH_CHECK(next_slot_ < kMaxGraphEntries,
                  "too many collectives are captured in live CUDA graphs on this communicator (", kMaxGraphEntries,
                  "); destroy graphs that are no longer replayed");
      e.slot = next_slot_++;
    } else {
      e.slot = free_slots_.back();
      free_slots_.pop_back();
    }
    // Counter pairs come from a page pinned at start-up: nothing is allocated
    // while a capture is open.
    e.counters_host = replay_pool_host_ + 2 * e.slot;
    e.counters_dev = replay_pool_dev_ + 2 * e.slot;
    e.counters_host[0] = e.counters_host[1] = 0;
    replay_counters = e.counters_dev;
    graph_entries_.push_back(e);
  } else {
    std::tie(ev_start, ev_end) = take_events();
  }

  B200C_CUDA_CHECK(cuda_->eventRecord(ev_start, stream));
  const int64_t tslot = capturing ? -1 : colltrace_begin(what, stream);
  if (!cuda_->is_real()) {
    // Under a test fake of the runtime nothing can be launched. Operations that
    // only call NCCL ("<op>/nccl") still run, against the NCCL fake.
    cuda_->noteLaunch(what, stream);
    if (std::strstr(what, "/nccl") != nullptr) launch(stream);
  } else {
    if (replay_counters != nullptr) {
      B200C_CUDA_CHECK(launch_counter_increment(replay_counters, stream));
    }
    launch(stream);
    if (replay_counters != nullptr) {
      B200C_CUDA_CHECK(launch_counter_increment(replay_counters + 1, stream));
    }
  }
  colltrace_end(tslot, stream);
  B200C_CUDA_CHECK(cuda_->eventRecord(ev_end, stream));
  if (!async_op) {
    keep_alive.clear();  // stream order already protects the tensors
  }
  // Events made during a capture belong to the graph's bookkeeping (the next
  // captured operation may have to wait on them after this work is gone).
  auto work = c10::make_intrusive<CudaWork>(cuda_, ev_start, ev_end, !capturing, device_.index(), effective_timeout(o),
                                            std::move(keep_alive), self, capturing, stream);
  ops_issued_++;
  if (!capturing) {
    // The end event of the latest operation doubles as the cross-stream
    // ordering point for the next one (the work keeps the event alive).
    cs.last_work = work;
    cs.last_stream = stream;
  }
  {
    std::lock_guard<std::mutex> g(wd_mu_);
    algo_counts_[what]++;
    if (capturing) {
      capture_tail_[graph_id] = CaptureTail{ev_end, stream};
    } else {
      inflight_.push_back(work);
    }
  }
  return work;
}

int64_t CudaBackend::colltrace_begin(const char* what, cudaStream_t stream) {
  if (trace_ring_host_ == nullptr) return -1;
  int64_t slot;
  {
    std::lock_guard<std::mutex> g(wd_mu_);
    slot = static_cast<int64_t>(trace_next_ % trace_meta_.size());
    trace_meta_[slot] = {trace_next_++, what};
    trace_ring_host_[2 * slot] = trace_ring_host_[2 * slot + 1] = 0;
  }
  if (cuda_->is_real()) launch_timestamp(trace_ring_dev_ + 2 * slot, stream);
  return slot;
}

void CudaBackend::colltrace_end(int64_t slot, cudaStream_t stream) {
  if (slot >= 0 && cuda_->is_real()) launch_timestamp(trace_ring_dev_ + 2 * slot + 1, stream);
}

std::vector<CudaBackend::CollTraceEntry> CudaBackend::colltrace_dump() const {
  std::vector<CollTraceEntry> out;
  if (trace_ring_host_ == nullptr) return out;
  std::lock_guard<std::mutex> g(const_cast<std::mutex&>(wd_mu_));
  const uint64_t n = trace_meta_.size();
  const uint64_t first = trace_next_ > n ? trace_next_ - n : 0;
  for (uint64_t seq = first; seq < trace_next_; ++seq) {
    const uint64_t slot = seq % n;
    const volatile unsigned long long* w = trace_ring_host_ + 2 * slot;
    out.push_back({trace_meta_[slot].first, trace_meta_[slot].second, w[0], w[1]});
  }
  return out;
}

void CudaBackend::sync_own_streams() {
  for (int ch = 0; ch < kChanCount; ++ch) {
    if (chans_[ch].stream != nullptr && (ch == kChanMain || chans_[ch].owns_stream)) {
      cuda_->streamSynchronize(chans_[ch].stream);
    }
  }
  cuda_->streamSynchronize(cuda_->currentStream(device_.index()));
}

void CudaBackend::start_watchdog() {
  wd_stop_ = false;
  watchdog_ = std::thread([this]() { watchdog_loop(); });
}

void CudaBackend::stop_watchdog() {
  {
    std::lock_guard<std::mutex> g(wd_mu_);
    wd_stop_ = true;
  }
  wd_cv_.notify_all();
  if (watchdog_.joinable()) {
    watchdog_.join();
  }
}

void CudaBackend::watchdog_loop() {
  cuda_->setDevice(device_.index());
  std::unique_lock<std::mutex> lk(wd_mu_);
  while (!wd_stop_) {
    wd_cv_.wait_for(lk, std::chrono::milliseconds(tune_.watchdog_interval_ms));
    if (wd_stop_) break;
    const auto now = std::chrono::steady_clock::now();
    std::string failure;
    bool timed_out = false;
    // Works complete in issue order per stream; scan the whole queue anyway
    // (two streams interleave) and drop the terminal ones.
    for (auto it = inflight_.begin(); it != inflight_.end();) {
      auto& w = *it;
      if (w->poll(now)) {
        const WorkStatus s = w->status();
        if (s == WorkStatus::TIMEDOUT || s == WorkStatus::ERROR) {
          failure = w->error();
          timed_out = s == WorkStatus::TIMEDOUT;
        }
        it = inflight_.erase(it);
      } else {
        ++it;
      }
    }
    // Device-side bounded waits report through the status word.
    if (failure.empty() && status_host_ != nullptr) {
      const volatile uint32_t* s = reinterpret_cast<volatile uint32_t*>(status_host_);
      if (s[0] & kStatusTimeout) {
        std::ostringstream os;
        os << "a device-side wait ran out (rank " << s[1] << ", block " << s[2] << ", waiting for rank "
           << static_cast<int>(s[3]) << ", phase 0x" << std::hex << s[4] << ")";
        failure = os.str();
        timed_out = true;
      } else if (s[0] & kStatusBadArg) {
        failure = "a kernel rejected its arguments (bounds check)";
      }
    }
    if (failure.empty() && nccl_comm_ != nullptr) {
      NcclResult async = kNcclSuccess;
      if (nccl_->commGetAsyncError(nccl_comm_, &async) == kNcclSuccess && async != kNcclSuccess && async != kNcclInProgress) {
        failure = "NCCL asynchronous error: " + nccl_->errorString(async);
      }
    }
    drop_released_graphs();
    // Graph replays: counters tell how many times each captured collective
    // started and ended.
    std::vector<std::tuple<unsigned long long, unsigned long long, uintptr_t, size_t, char>> replay_events;
    for (auto& e : graph_entries_) {
      const unsigned long long st = reinterpret_cast<volatile unsigned long long*>(e.counters_host)[0];
      const unsigned long long en = reinterpret_cast<volatile unsigned long long*>(e.counters_host)[1];
      while (e.seen_start < st) {
        replay_events.emplace_back(e.graph_id, e.seen_start, e.stream, e.index, 'S');
        e.seen_start++;
        e.open_since = now;
      }
      while (e.seen_end < en) {
        replay_events.emplace_back(e.graph_id, e.seen_end, e.stream, e.index, 'E');
        e.seen_end++;
      }
      if (tune_.graph_timeout_monitoring && failure.empty() && e.seen_start > e.seen_end && e.timeout != kNoTimeout &&
          now - e.open_since > e.timeout) {
        failure = "a captured collective (graph " + std::to_string(e.graph_id) + ", index " + std::to_string(e.index) +
            ") did not finish within its timeout during replay";
        timed_out = true;
      }
    }
    lk.unlock();
    if (!replay_events.empty() && replay_hooks_) {
      for (auto& h : replay_hooks_->snapshot()) {
        for (auto& ev : replay_events) {
          h(std::get<0>(ev), std::get<1>(ev), std::get<2>(ev), std::get<3>(ev), std::get<4>(ev));
        }
      }
    }
    if (!failure.empty()) {
      on_failure(failure, timed_out);
    }
    lk.lock();
  }
}

void CudaBackend::drop_released_graphs() {
  std::vector<unsigned long long> gone;
  {
    std::lock_guard<std::mutex> g(released_mu_);
    gone.swap(released_ids_);
  }
  for (unsigned long long id : gone) {
    for (auto it = graph_entries_.begin(); it != graph_entries_.end();) {
      if (it->graph_id == id) {
        free_slots_.push_back(it->slot);
        it = graph_entries_.erase(it);
      } else {
        ++it;
      }
    }
    auto gs = graphs_.find(id);
    if (gs != graphs_.end()) {
      for (cudaEvent_t e : gs->second.events) cuda_->eventDestroy(e);
      graphs_.erase(gs);
    }
    capture_tail_.erase(id);
  }
}

void CudaBackend::suspend() {
  TORCH_CHECK(!finalized_, "communicator '", name_, "' was finalized");
  TORCH_CHECK(initialized_, "suspend: communicator '", name_, "' is not initialised");
  DeviceScope guard(cuda_, device_.index());
  resume_store_ = store_;
  drain_and_release(failed_.load() || aborted_.load(), "suspend");
  suspended_ = true;
}

void CudaBackend::resume() {
  TORCH_CHECK(!finalized_, "communicator '", name_, "' was finalized");
  TORCH_CHECK(suspended_, "resume: communicator '", name_, "' is not suspended");
  DeviceScope guard(cuda_, device_.index());
  ++suspend_gen_;
  failed_.store(false);
  aborted_.store(false);
  failure_text_.clear();
  bootstrap(scoped_store(resume_store_, "resume/" + std::to_string(suspend_gen_)), rank_, size_);
  suspended_ = false;
  resume_store_.reset();
}

void CudaBackend::finalize() {
  TORCH_CHECK(!finalized_, "communicator '", name_, "' was already finalized");
  TORCH_CHECK(initialized_ || suspended_ || opts_.enable_reconfigure, "communicator '", name_, "' is not initialised");
  if (!initialized_) {
    finalized_ = true;  // suspended, or a reconfigurable communicator that never got a membership: nothing is held
    return;
  }
  DeviceScope guard(cuda_, device_.index());
  const bool broken = failed_.load() || aborted_.load();
  drain_and_release(broken, "finalize");
  finalized_ = true;
  if (failed_.load()) {
    throw std::runtime_error("communicator '" + name_ + "' finalized after a failure: " + failure_text_);
  }
}

// Waits for this rank's work, meets the other members (unless the communicator is broken), and
// gives back everything bootstrap() created. The communicator can be bootstrapped again afterwards.
void CudaBackend::drain_and_release(bool broken, const char* why) {
  if (broken) {
    // Kernels of this rank may still be running. Tell them to stop waiting,
    // end NCCL's work, and only then wait for the streams: every device wait
    // is bounded and looks at the abort bit, so this returns, and nothing is
    // unmapped under a live kernel.
    if (status_host_ != nullptr) {
      reinterpret_cast<volatile uint32_t*>(status_host_)[0] |= kStatusAbort;
    }
    if (nccl_comm_ != nullptr) {
      nccl_->commAbort(nccl_comm_);
      nccl_comm_ = nullptr;
    }
    sync_own_streams();
  } else {
    // Drain: every rank's kernels are done before any mapping disappears.
    sync_own_streams();
    if (size_ > 1) {
      try {
        store_barrier(*store_, why, rank_, size_, std::min<Millis>(opts_.timeout, Millis(30000)));
      } catch (const std::exception& e) {
        // A peer that failed never arrives; its mappings are gone either way.
        B200C_LOG(WARN, name_, why << ": not every rank arrived at the closing barrier: " << e.what());
      }
    }
  }
  stop_watchdog();
  for (auto& cs : chans_) cs.last_work.reset();
  initialized_ = false;
  {
    std::lock_guard<std::mutex> g(wd_mu_);
    inflight_.clear();
    graph_entries_.clear();
    for (auto& kv : graphs_) {
      for (cudaEvent_t e : kv.second.events) cuda_->eventDestroy(e);
    }
    graphs_.clear();
    capture_tail_.clear();
    free_slots_.clear();
    next_slot_ = 0;
  }
  {
    // Tensors handed out by symm_empty() dangle from here on; registrations go with the mappings.
    std::lock_guard<std::mutex> g(symm_mu_);
    for (auto& kv : symm_regs_) {
      if (symm_) symm_->release(kv.second.seg);
    }
    symm_regs_.clear();
  }
  if (replay_pool_host_) cuda_->freeHost(replay_pool_host_);
  replay_pool_host_ = nullptr;
  if (trace_ring_host_) cuda_->freeHost(trace_ring_host_);
  trace_ring_host_ = nullptr;
  if (nccl_comm_ != nullptr) {
    if (broken) {
      nccl_->commAbort(nccl_comm_);
    } else {
      nccl_->commDestroy(nccl_comm_);
    }
    nccl_comm_ = nullptr;
  }
  if (heap_) {
    symm_->release(heap_);
    heap_.reset();
  }
  symm_.reset();
  if (epochs_dev_) cuda_->freeDevice(epochs_dev_);
  if (status_host_) cuda_->freeHost(status_host_);
  epochs_dev_ = nullptr;
  status_host_ = nullptr;
  {
    std::lock_guard<std::mutex> g(pool_mu_);
    for (cudaEvent_t e : event_pool_) cuda_->eventDestroy(e);
    event_pool_.clear();
  }
  if (dep_event_) cuda_->eventDestroy(dep_event_);
  dep_event_ = nullptr;
  for (auto& cs : chans_) {
    if (cs.order_event) cuda_->eventDestroy(cs.order_event);
    if (cs.stream && cs.owns_stream) cuda_->streamDestroy(cs.stream);
    cs = ChanState{};
  }
  internal_stream_ = nullptr;
}

InitHandle CudaBackend::get_init_handle() const {
  return registered_as_ + ":" + handle_token_;
}

// Elastic membership on one box: the members named by `handles` (rank = position in the list; a set
// is sorted) tear down what they hold - peer mappings, multicast bindings, the NCCL communicator -
// and run the bootstrap again among themselves under a store prefix derived from `uuid`. A first
// call creates the communicator; later calls shrink, grow or re-form it. A rank that is not in the
// list must not call. Parity: comms/torchcomms/ncclx/TorchCommNCCLXReconfigure.cpp:206-429.
WorkPtr CudaBackend::reconfigure(const ReconfigureOptions& o) {
  TORCH_CHECK(!finalized_, "communicator '", name_, "' was finalized");
  TORCH_CHECK(opts_.enable_reconfigure, "reconfigure() needs a communicator created with enable_reconfigure=True");
  std::vector<InitHandle> members = o.handles;
  if (!o.handles_ordered) {
    std::sort(members.begin(), members.end());
  }
  const InitHandle me = get_init_handle();
  int idx = -1;
  for (size_t i = 0; i < members.size(); ++i) {
    if (members[i] == me) idx = static_cast<int>(i);
  }
  TORCH_CHECK(idx >= 0, "reconfigure: this rank's init handle is not in the member list");
  if (o.timeout) {
    opts_.timeout = *o.timeout;
  }
  DeviceScope guard(cuda_, device_.index());
  auto scoped = scoped_store(opts_.store, "b200c/cuda/" + name_ + "/reconf/" + std::to_string(o.uuid));
  if (initialized_) {
    // Nothing of this rank is in flight any more; once every member of the NEW list says the same,
    // nobody can still be reading memory this rank is about to unmap. Members that left do not come
    // to any barrier, so the old membership's closing barrier is skipped (released as "broken").
    sync_own_streams();
    if (members.size() > 1) {
      store_barrier(*scoped, "quiesced", idx, static_cast<int>(members.size()), opts_.timeout);
    }
    drain_and_release(true, "reconfigure");
  }
  failed_.store(false);
  aborted_.store(false);
  failure_text_.clear();
  parse_tuning(o.hints);
  bootstrap(scoped, idx, static_cast<int>(members.size()));
  return c10::make_intrusive<CompletedWork>();
}

Algo CudaBackend::algo_override(const OpOptions& o) const {
  auto it = o.hints.find("algo");
  if (it != o.hints.end()) {
    return parse_algo(it->second);
  }
  return tune_.force;
}

// Cross-over sizes measured on 8 B200 over NVSwitch (bf16 sweep, 1 KB - 1 GB,
// device-timed, kernels against NCCL 2.28 on the same buffers): the
// peer-memory kernels win the latency-bound sizes (one barrier, one-shot:
// all-reduce up to 512 KB, all-gather up to 256 KB, reduce-scatter up to
// 8 KB) and the all-reduce between 4 and 64 MB (NVLS two-shot with 64 KB
// chunks); NCCL's protocols win the rest, all-to-all, and everything below
// 4 ranks. algo=kernel forces the kernels.
// Tuner file: lines of `<operation> <largest bytes | inf> <kernel | nccl>`, '#' starts a comment. For every
// operation the rules apply in ascending order of size; a size above the last rule keeps the built-in choice.
// Every rank must load the same file (the route has to be the same everywhere).
void CudaBackend::load_tuner_file(const std::string& path) {
  std::ifstream f(path);
  TORCH_CHECK(f.good(), "tuner file '", path, "' cannot be read");
  static const std::unordered_map<std::string, Coll> ops = {
      {"all_reduce", Coll::ALL_REDUCE}, {"all_gather", Coll::ALL_GATHER},
      {"reduce_scatter", Coll::REDUCE_SCATTER}, {"all_to_all", Coll::ALL_TO_ALL}, {"all_to_all_v", Coll::ALL_TO_ALL}};
  std::string line;
  int lineno = 0;
  while (std::getline(f, line)) {
    ++lineno;
    const size_t hash = line.find('#');
    if (hash != std::string::npos) line.resize(hash);
    std::istringstream is(line);
    std::string op, limit, algo;
    if (!(is >> op)) continue;
    TORCH_CHECK(static_cast<bool>(is >> limit >> algo), "tuner file ", path, ":", lineno, ": expected '<op> <bytes|inf> <kernel|nccl>'");
    auto it = ops.find(op);
    TORCH_CHECK(it != ops.end(), "tuner file ", path, ":", lineno, ": unknown operation '", op, "'");
    TORCH_CHECK(algo == "kernel" || algo == "nccl", "tuner file ", path, ":", lineno, ": algorithm must be kernel or nccl");
    size_t up_to = std::numeric_limits<size_t>::max();
    if (limit != "inf") {
      char* end = nullptr;
      up_to = std::strtoull(limit.c_str(), &end, 10);
      TORCH_CHECK(end != nullptr && *end == 0, "tuner file ", path, ":", lineno, ": bad size '", limit, "'");
    }
    tuner_rules_[static_cast<int>(it->second)].push_back({up_to, algo == "nccl" ? Algo::NCCL : Algo::KERNEL});
  }
  for (auto& rules : tuner_rules_) {
    std::stable_sort(rules.begin(), rules.end(), [](const TunerRule& a, const TunerRule& b) { return a.up_to < b.up_to; });
  }
}

Algo CudaBackend::route(Coll c, size_t bytes, const OpOptions& o) const {
  const Algo a = algo_override(o);
  if (a == Algo::KERNEL) return Algo::AUTO;
  if (a != Algo::AUTO) return a;
  if (nccl_comm_ != nullptr && size_ > 1) {
    for (const TunerRule& r : tuner_rules_[static_cast<int>(c)]) {
      if (bytes <= r.up_to) return r.algo == Algo::NCCL ? Algo::NCCL : Algo::AUTO;
    }
  }
  if (nccl_comm_ == nullptr || !tune_.auto_nccl || size_ == 1) return Algo::AUTO;
  if (size_ < 4) return Algo::NCCL;
  constexpr size_t KB = 1024, MB = 1024 * 1024;
  switch (c) {
    case Coll::ALL_REDUCE:
      return (bytes <= 512 * KB || (bytes >= 4 * MB && bytes <= 64 * MB)) ? Algo::AUTO : Algo::NCCL;
    case Coll::ALL_GATHER:   // bytes = gathered size
      return (bytes <= 256 * KB || (bytes >= 4 * MB && bytes < 8 * MB)) ? Algo::AUTO : Algo::NCCL;
    case Coll::REDUCE_SCATTER:   // bytes = input size
      return bytes <= 8 * KB ? Algo::AUTO : Algo::NCCL;
    case Coll::ALL_TO_ALL:
      return Algo::NCCL;
  }
  return Algo::AUTO;
}

bool CudaBackend::kernels_can_reduce(at::ScalarType t, const ReduceOp& op) const {
  DType d;
  if (!to_dtype(t, &d)) return false;
  switch (op.type()) {
    case RedOpType::BAND:
    case RedOpType::BOR:
    case RedOpType::BXOR:
      return false;
    default:
      return true;
  }
}

// Blocks and per-block chunk for `bytes` of payload when one slot holds
// `slot_multiplier` chunks (nranks for reduce-scatter / all-to-all, else 1).
LaunchShape CudaBackend::shape_for(size_t bytes, size_t slot_multiplier, int block_cap) const {
  LaunchShape s;
  s.threads = tune_.threads;
  const int max_blocks = block_cap > 0 ? std::min(block_cap, tune_.max_blocks) : tune_.max_blocks;
  const size_t max_chunk = std::max<size_t>(
      256, std::min(tune_.max_chunk_bytes, layout_.bulk_bytes / (static_cast<size_t>(max_blocks) * slot_multiplier * kPipeSlots)));
  // Aim for every block to run several steps on large payloads so that copy
  // and link phases of different blocks overlap; small payloads use few blocks.
  size_t chunk = round_up(std::max<size_t>(bytes / (static_cast<size_t>(max_blocks) * std::max(1, tune_.steps_per_block)) + 1, tune_.min_chunk_bytes), 256);
  chunk = std::min(chunk, max_chunk / 256 * 256);
  chunk = std::max<size_t>(chunk, 256);
  const size_t steps = (bytes + chunk - 1) / chunk;
  s.chunk_bytes = chunk;
  s.blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(max_blocks, steps)));
  return s;
}

// Grid of a one-pass kernel on symmetric buffers: the configured block count
// (hint "symm_blocks" for one call), fewer when the payload gives each block
// less than a few iterations. Depends only on sizes, hints and on whether the
// buffer has a multicast alias, so every rank computes the same number.
int CudaBackend::symm_blocks_for(bool mc, size_t vectors, const OpOptions& o, bool peer_loads) const {
  int cap = mc ? tune_.symm_blocks : peer_loads ? tune_.symm_blocks_ld : tune_.symm_blocks_nomc;
  cap = std::max(1, std::min(132, hint_or<int>(o.hints, "symm_blocks", cap)));  // never every SM: see kSmBudget in run()
  const size_t per_block = 512 * 4;  // threads x unroll
  const size_t want = (vectors + per_block - 1) / per_block;
  return static_cast<int>(std::max<size_t>(1, std::min<size_t>(cap, want)));
}

bool CudaBackend::symm_use_mc(int knob, bool mc_by_default, const SymmView& v, const OpOptions& o) const {
  if (!tune_.use_multicast || v.mc == nullptr) return false;
  const int want = hint_or<int>(o.hints, "symm_mc", knob);
  return want < 0 ? mc_by_default : want != 0;
}

// Payloads the flag-less kernels may carry: a word equal to their "nothing here
// yet" marker is delivered as +0.0, which is only harmless for these types.
static bool lamport_dtype(at::ScalarType t) {
  return t == at::kFloat || t == at::kHalf || t == at::kBFloat16;
}

static RedKind red_kind(const ReduceOp& op) {
  switch (op.type()) {
    case RedOpType::PRODUCT: return RedKind::PROD;
    case RedOpType::MIN: return RedKind::MIN;
    case RedOpType::MAX: return RedKind::MAX;
    default: return RedKind::SUM;
  }
}

static float red_scale(const ReduceOp& op, int nranks) {
  if (op.type() == RedOpType::AVG) return 1.0f / static_cast<float>(nranks);
  if (op.type() == RedOpType::PREMUL_SUM) return static_cast<float>(op.factor_as_double());
  return 1.0f;
}

WorkPtr CudaBackend::all_reduce(at::Tensor& t, const ReduceOp& op, bool async_op, const OpOptions& o) {
  check_tensor(t, device_, "all_reduce", cuda_->is_real());
  const size_t bytes = t.nbytes();
  if (bytes == 0) return c10::make_intrusive<CompletedWork>();
  Algo algo = route(Coll::ALL_REDUCE, bytes, o);
  const bool kernels_ok = kernels_can_reduce(t.scalar_type(), op);
  if (!kernels_ok) {
    TORCH_CHECK(op.type() != RedOpType::BAND && op.type() != RedOpType::BOR && op.type() != RedOpType::BXOR,
                "bitwise reductions are not supported on the CUDA backend");
    algo = Algo::NCCL;
  }
  if (algo == Algo::NCCL && (nccl_comm_ == nullptr || size_ == 1)) {
    if (size_ == 1) {
      // A lone rank: only PREMUL_SUM changes the data.
      if (op.type() == RedOpType::PREMUL_SUM) t.mul_(op.factor_as_double());
      return c10::make_intrusive<CompletedWork>();
    }
    TORCH_CHECK(kernels_ok, "all_reduce of ", t.scalar_type(), " needs NCCL, which is not available");
    algo = Algo::AUTO;
  }
  if (algo == Algo::NCCL) {
    NcclDataType dt;
    TORCH_CHECK(to_nccl_dtype(t.scalar_type(), &dt), "all_reduce: unsupported dtype ", t.scalar_type());
    const ReduceOp opc = op;
    at::Tensor tt = t;
    return run("all_reduce/nccl", async_op, o, {t}, [this, tt, dt, opc](cudaStream_t s) {
      NcclRedOp rop = kNcclSum;
      bool custom = false;
      switch (opc.type()) {
        case RedOpType::PRODUCT: rop = kNcclProd; break;
        case RedOpType::MIN: rop = kNcclMin; break;
        case RedOpType::MAX: rop = kNcclMax; break;
        case RedOpType::AVG: rop = kNcclAvg; break;
        case RedOpType::PREMUL_SUM: {
          // Host-immediate scalar in the tensor's own dtype.
          at::Tensor f = at::scalar_tensor(opc.factor_as_double(), at::TensorOptions().dtype(tt.scalar_type()));
          nccl_check(nccl_->redOpCreatePreMulSum(&rop, f.data_ptr(), dt, nccl_comm_), "ncclRedOpCreatePreMulSum");
          custom = true;
          break;
        }
        default: break;
      }
      nccl_check(nccl_->allReduce(tt.data_ptr(), tt.data_ptr(), tt.numel(), dt, rop, nccl_comm_, s), "ncclAllReduce");
      if (custom) nccl_->redOpDestroy(rop, nccl_comm_);
    });
  }
  DType dt;
  to_dtype(t.scalar_type(), &dt);
  const bool sum_like = red_kind(op) == RedKind::SUM;
  if (algo == Algo::AUTO && sum_like && size_ > 1) {
    const float scale = red_scale(op, size_);
    const bool mc = tune_.use_multicast && dev_.mc_heap != nullptr;
    at::Tensor tt = t;
    if (bytes <= tune_.lamport_max_bytes) {
      // Latency class: the flag-less kernel (one one-way trip, no barrier, no staging).
      bytes_issued_ += bytes;
      return run("all_reduce/lamport", async_op, o, {t}, [this, tt, dt, scale, mc](cudaStream_t s) {
        const void* in = tt.data_ptr();
        void* out = tt.data_ptr();
        B200C_CUDA_CHECK(launch_all_reduce_lamport(&dev_, layout_, 0, &in, &out, tt.numel(), dt, scale, mc, s));
      }, kChanSymAr, true);
    }
    SymmView sv;
    const size_t pack = 16 / dtype_size(dt);
    if (t.numel() % pack == 0 && lookup_symm(t.data_ptr(), bytes, &sv) &&
        reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0) {
      // The tensor lives in symmetric memory: reduce it in place, one pass over NVLink.
      const bool smc = symm_use_mc(tune_.symm_ar_mc, size_ >= 4, sv, o);
      const int blocks = symm_blocks_for(smc, t.numel() / pack / size_, o, true);
      bytes_issued_ += bytes;
      return run("all_reduce/symm", async_op, o, {t}, [this, tt, sv, dt, scale, smc, blocks](cudaStream_t s) {
        B200C_CUDA_CHECK(launch_symm_all_reduce(&dev_, 0, &sv, tt.numel(), dt, scale, smc, blocks, s));
      }, kChanSymAr, true, blocks);
    }
  }
  int kalgo;
  if (algo == Algo::ONESHOT) kalgo = 0;
  else if (algo == Algo::TWOSHOT || algo == Algo::STAGED) kalgo = 1;
  else kalgo = bytes <= tune_.oneshot_max_bytes ? 0 : 1;
  if (bytes > static_cast<size_t>(kSmallBlocks) * kSmallPiece) kalgo = 1;
  const float scale = red_scale(op, size_);
  const RedKind rk = red_kind(op);
  const bool mc = tune_.use_multicast && sum_like && dev_.mc_heap != nullptr;
  const LaunchShape shape = shape_for(bytes, 1);
  at::Tensor tt = t;
  bytes_issued_ += bytes;
  return run(kalgo == 0 ? "all_reduce/oneshot" : "all_reduce/twoshot", async_op, o, {t},
             [this, tt, dt, rk, scale, kalgo, mc, shape](cudaStream_t s) {
               const void* in = tt.data_ptr();
               void* out = tt.data_ptr();
               B200C_CUDA_CHECK(launch_all_reduce(&dev_, layout_, 0, &in, &out, tt.numel(), dt, rk, scale, kalgo, mc, shape, s));
             }, kChanMain, true);
}

static WorkPtr exchange(CudaBackend* self, const char* what, at::Tensor in, at::Tensor out,
                        std::vector<std::pair<size_t, size_t>> send, std::vector<std::pair<size_t, size_t>> recv,
                        bool async_op, const OpOptions& o, std::vector<at::Tensor> keep,
                        std::function<void(cudaStream_t)> after = nullptr, size_t known_max = 0);

WorkPtr CudaBackend::reduce(const at::Tensor& t, int root, const ReduceOp& op, bool async_op, const OpOptions& o) {
  check_tensor(t, device_, "reduce", cuda_->is_real());
  if (t.numel() == 0) return c10::make_intrusive<CompletedWork>();
  NcclDataType ndt;
  if (nccl_comm_ != nullptr && algo_override(o) == Algo::NCCL && to_nccl_dtype(t.scalar_type(), &ndt) &&
      op.type() != RedOpType::PREMUL_SUM) {
    NcclRedOp rop = kNcclSum;
    switch (op.type()) {
      case RedOpType::PRODUCT: rop = kNcclProd; break;
      case RedOpType::MIN: rop = kNcclMin; break;
      case RedOpType::MAX: rop = kNcclMax; break;
      case RedOpType::AVG: rop = kNcclAvg; break;
      default: break;
    }
    at::Tensor tt = t;
    return run("reduce/nccl", async_op, o, {t}, [this, tt, ndt, rop, root](cudaStream_t s) {
      nccl_check(nccl_->reduce(tt.data_ptr(), tt.data_ptr(), tt.numel(), ndt, rop, root, nccl_comm_, s), "ncclReduce");
    });
  }
  TORCH_CHECK(kernels_can_reduce(t.scalar_type(), op), "reduce: unsupported dtype / reduction for the CUDA backend");
  {
    // Bandwidth class: reduce-scatter (every rank reduces 1/size of the data),
    // then the root collects the slices. Half the traffic of an all-reduce,
    // and nobody but the root receives the result.
    const int64_t pack = std::max<int64_t>(1, 16 / static_cast<int64_t>(t.element_size()));
    if (size_ > 1 && t.nbytes() >= (1u << 20) && t.numel() % (static_cast<int64_t>(size_) * pack) == 0) {
      const int64_t slice = t.numel() / size_;
      const size_t slice_bytes = static_cast<size_t>(slice) * t.element_size();
      at::Tensor part = at::empty({slice}, t.options());
      at::Tensor flat = t.reshape({-1});
      WorkPtr first = reduce_scatter_single(part, flat, op, async_op, o);
      // The two steps may run on different channels (streams): order the
      // caller's stream behind the first; the second then follows it.
      if (async_op) first->wait();
      std::vector<std::pair<size_t, size_t>> send(size_, {0, 0}), recv(size_, {0, 0});
      send[root] = {0, slice_bytes};
      at::Tensor out = rank_ == root ? flat : at::empty({16}, t.options().dtype(at::kByte));
      if (rank_ == root) {
        for (int p = 0; p < size_; ++p) recv[p] = {static_cast<size_t>(p) * slice_bytes, slice_bytes};
      }
      return exchange(this, "reduce/scatter+gather", part, out, send, recv, async_op, o, {part, out});
    }
  }
  // All-reduce into the tensor on the root and into scratch elsewhere, so that
  // non-root inputs stay untouched.
  DType dt;
  to_dtype(t.scalar_type(), &dt);
  at::Tensor in = t;
  at::Tensor out = rank_ == root ? t : at::empty_like(t);
  const float scale = red_scale(op, size_);
  const RedKind rk = red_kind(op);
  const size_t bytes = t.nbytes();
  const int kalgo = bytes <= std::min(tune_.oneshot_max_bytes, static_cast<size_t>(kSmallBlocks) * kSmallPiece) ? 0 : 1;
  const bool mc = tune_.use_multicast && rk == RedKind::SUM && dev_.mc_heap != nullptr;
  const LaunchShape shape = shape_for(bytes, 1);
  return run("reduce/kernel", async_op, o, {in, out}, [this, in, out, dt, rk, scale, kalgo, mc, shape](cudaStream_t s) {
    const void* ip = in.data_ptr();
    void* op_ = out.data_ptr();
    B200C_CUDA_CHECK(launch_all_reduce(&dev_, layout_, 0, &ip, &op_, in.numel(), dt, rk, scale, kalgo, mc, shape, s));
  });
}

// A lone rank: gather / scatter / reduce over one member is a cast (and a
// scale) of the input into the output. One pass of a plain kernel instead of
// the staged pipeline. False = shape or alignment not covered, use the general path.
static bool single_rank_kind(at::ScalarType t, int* kind) {
  if (t == at::kFloat) { *kind = 0; return true; }
  if (t == at::kBFloat16) { *kind = 1; return true; }
  return false;
}

WorkPtr CudaBackend::all_gather_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) {
  check_tensor(out, device_, "all_gather_single", cuda_->is_real());
  check_tensor(in, device_, "all_gather_single", cuda_->is_real());
  TORCH_CHECK(out.numel() == in.numel() * size_, "all_gather_single: output numel must be input numel * size");
  const bool cast = in.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16;
  TORCH_CHECK(cast || in.scalar_type() == out.scalar_type(),
              "all_gather_single: dtypes must match (or float32 input with bfloat16 output for the fused cast)");
  if (in.numel() == 0) return c10::make_intrusive<CompletedWork>();
  {
    int ik = 0, ok = 0;
    if (size_ == 1 && single_rank_kind(in.scalar_type(), &ik) && single_rank_kind(out.scalar_type(), &ok) &&
        reinterpret_cast<uintptr_t>(in.data_ptr()) % 32 == 0 && reinterpret_cast<uintptr_t>(out.data_ptr()) % 32 == 0) {
      at::Tensor i = in, ot = out;
      bytes_issued_ += in.nbytes();
      return run("all_gather/single_rank", async_op, o, {in}, [i, ot, ik, ok](cudaStream_t s) {
        B200C_CUDA_CHECK(launch_cast_scale(i.data_ptr(), ik, ot.data_ptr(), ok, static_cast<size_t>(i.numel()), 1.0f, s));
      }, kChanSymAg, true);
    }
  }
  if (!cast && nccl_comm_ != nullptr && route(Coll::ALL_GATHER, out.nbytes(), o) == Algo::NCCL) {
    NcclDataType dt;
    if (to_nccl_dtype(in.scalar_type(), &dt)) {
      at::Tensor i = in, ot = out;
      return run("all_gather/nccl", async_op, o, {in}, [this, i, ot, dt](cudaStream_t s) {
        nccl_check(nccl_->allGather(i.data_ptr(), ot.data_ptr(), i.numel(), dt, nccl_comm_, s), "ncclAllGather");
      });
    }
  }
  const size_t bytes = in.nbytes();
  const Algo algo = algo_override(o);
  if ((algo == Algo::AUTO || algo == Algo::KERNEL) && !cast && size_ > 1 && lamport_dtype(in.scalar_type()) &&
      bytes % 16 == 0 && bytes <= tune_.lamport_max_bytes) {
    // Latency class: flag-less exchange (no barrier, nothing staged), whatever memory the tensors live in.
    const bool mc = tune_.use_multicast && dev_.mc_heap != nullptr;
    at::Tensor i = in, ot = out;
    bytes_issued_ += bytes;
    return run("all_gather/lamport", async_op, o, {in}, [this, i, ot, bytes, mc](cudaStream_t s) {
      const void* ip = i.data_ptr();
      void* op_ = ot.data_ptr();
      B200C_CUDA_CHECK(launch_exchange_lamport(&dev_, layout_, 0, 0, &ip, &op_, bytes, DType::F32, 1.0f, mc, s));
    }, kChanSymAr, true);
  }
  if (algo == Algo::AUTO || algo == Algo::KERNEL) {
    SymmView sv;
    const size_t wire = cast ? bytes / 2 : bytes;
    if (wire % 16 == 0 && lookup_symm(out.data_ptr(), out.nbytes(), &sv) &&
        reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0) {
      // The output lives in symmetric memory: every rank stores its shard
      // straight into every copy (through the switch's multicast when bound).
      const bool smc = symm_use_mc(tune_.symm_ag_mc, false, sv, o);
      const int blocks = symm_blocks_for(smc, wire / 16, o);
      at::Tensor i = in, ot = out;
      bytes_issued_ += bytes;
      return run(cast ? "all_gather/symm+cast" : "all_gather/symm", async_op, o, {in},
                 [this, i, ot, sv, bytes, cast, smc, blocks](cudaStream_t s) {
                   const void* ip = i.data_ptr();
                   B200C_CUDA_CHECK(launch_symm_all_gather(&dev_, 0, &ip, &sv, bytes, cast, smc, blocks, s));
                 }, kChanSymAg, true, blocks);
    }
  }
  // Multicast push pays while the message is latency / launch bound; big gathers pull.
  const bool mc = tune_.use_multicast && dev_.mc_heap != nullptr && size_ >= tune_.ag_push_min_ranks && bytes <= (8u << 20);
  const bool oneshot = !cast && algo != Algo::TWOSHOT && algo != Algo::STAGED &&
      bytes <= std::min(tune_.ag_oneshot_max_bytes, static_cast<size_t>(kSmallBlocks) * kSmallPiece);
  const int cap = out.nbytes() < (64u << 20) ? 148 : 0;  // one block per SM is enough below 64 MB
  LaunchShape shape = shape_for(cast ? bytes / 2 : bytes, mc ? static_cast<size_t>(size_) : 1, cap);
  if (oneshot) {
    shape.chunk_bytes = 0;
    shape.threads = 256;
  }
  at::Tensor i = in, ot = out;
  bytes_issued_ += bytes;
  return run(oneshot ? "all_gather/oneshot" : cast ? "all_gather/kernel+cast" : "all_gather/kernel", async_op, o, {in},
             [this, i, ot, bytes, cast, shape, mc](cudaStream_t s) {
               const void* ip = i.data_ptr();
               void* op_ = ot.data_ptr();
               B200C_CUDA_CHECK(launch_all_gather(&dev_, layout_, 0, &ip, &op_, bytes, cast, mc, shape, s));
             }, kChanMain, true);
}

WorkPtr CudaBackend::all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) {
  TORCH_CHECK(static_cast<int>(outs.size()) == size_, "all_gather: need size() output tensors");
  check_tensor(in, device_, "all_gather", cuda_->is_real());
  for (auto& t : outs) {
    check_tensor(t, device_, "all_gather", cuda_->is_real());
    TORCH_CHECK(t.numel() == in.numel() && t.scalar_type() == in.scalar_type(),
                "all_gather: every output must match the input's numel and dtype");
  }
  // Gather into one buffer, then fan out with device copies on the same stream.
  at::Tensor flat = at::empty({static_cast<int64_t>(size_) * in.numel()}, in.options());
  at::Tensor i = in;
  auto dsts = outs;
  const size_t bytes = in.nbytes();
  const LaunchShape shape = shape_for(bytes, 1);
  if (bytes == 0) return c10::make_intrusive<CompletedWork>();
  return run("all_gather_list/kernel", async_op, o, {in, flat}, [this, i, flat, dsts, bytes, shape](cudaStream_t s) {
    const void* ip = i.data_ptr();
    void* op_ = flat.data_ptr();
    B200C_CUDA_CHECK(launch_all_gather(&dev_, layout_, 0, &ip, &op_, bytes, false, false, shape, s));
    for (int r = 0; r < size_; ++r) {
      B200C_CUDA_CHECK(cudaMemcpyAsync(dsts[r].data_ptr(), static_cast<char*>(flat.data_ptr()) + r * bytes, bytes,
                                       cudaMemcpyDeviceToDevice, s));
    }
  });
}

// Generic exchange through the all-to-all kernel. `send` / `recv` list, per
// peer, (byte offset, byte length) into `in` / `out`.
static WorkPtr exchange(CudaBackend* self, const char* what, at::Tensor in, at::Tensor out,
                        std::vector<std::pair<size_t, size_t>> send, std::vector<std::pair<size_t, size_t>> recv,
                        bool async_op, const OpOptions& o, std::vector<at::Tensor> keep,
                        std::function<void(cudaStream_t)> after, size_t known_max) {
  const int n = self->size();
  LaunchShape shape;
  if (known_max != 0) {
    // Equal splits: every rank derives the same grid from the block size.
    shape = self->shape_for(known_max, static_cast<size_t>(n));
    shape.known_max = known_max;
  } else {
    // The grid must not depend on rank-local sizes (see launch_all_to_all).
    shape.threads = self->tuning().threads;
    shape.blocks = std::min(self->tuning().a2av_blocks, self->tuning().max_blocks);
    shape.chunk_bytes = std::min<size_t>(self->tuning().max_chunk_bytes,
                                         self->layout().bulk_bytes / (static_cast<size_t>(shape.blocks) * n * kPipeSlots)) / 256 * 256;
  }
  return self->run(what, async_op, o, std::move(keep), [self, in, out, send, recv, shape, n, after](cudaStream_t s) {
    std::vector<size_t> so(n), sl(n), ro(n), rl(n);
    size_t mx = 0;
    for (int p = 0; p < n; ++p) {
      so[p] = send[p].first;
      sl[p] = send[p].second;
      ro[p] = recv[p].first;
      rl[p] = recv[p].second;
      mx = std::max(mx, std::max(sl[p], rl[p]));
    }
    const void* ip = in.defined() ? in.data_ptr() : nullptr;
    void* op_ = out.defined() ? out.data_ptr() : nullptr;
    B200C_CUDA_CHECK(launch_all_to_all(&self->comm_dev(), self->layout(), 0, &ip, &op_, so.data(), sl.data(), ro.data(),
                                       rl.data(), mx, shape, s));
    if (after) after(s);
  });
}

// All-to-all(v) straight into a symmetric output: every rank stores its block
// for rank p into p's copy of `out`. `send` / `recv` as in exchange().
static WorkPtr exchange_symm(CudaBackend* self, const char* what, at::Tensor in, at::Tensor out, const SymmView& sv,
                             std::vector<std::pair<size_t, size_t>> send, std::vector<std::pair<size_t, size_t>> recv,
                             bool equal_splits, at::Tensor dev_counts, size_t elem_bytes, bool async_op,
                             const OpOptions& o) {
  const int n = self->size();
  int blocks = std::max(1, std::min(128, hint_or<int>(o.hints, "symm_blocks", self->tuning().symm_blocks_nomc)));
  if (equal_splits) {
    // Every rank sends the same amount: small exchanges need few blocks (fewer barriers to cross).
    const size_t want = (in.nbytes() / 16 + 512 * 4 - 1) / (512 * 4);
    blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(blocks, want)));
  }
  blocks = std::max(n, blocks / n * n);
  std::vector<at::Tensor> keep = {in};
  if (dev_counts.defined()) keep.push_back(dev_counts);
  return self->run(what, async_op, o, std::move(keep),
                   [self, in, out, sv, send, recv, equal_splits, dev_counts, elem_bytes, blocks, n](cudaStream_t s) {
                     std::vector<size_t> so(n), sl(n), ro(n), rl(n);
                     for (int p = 0; p < n; ++p) {
                       so[p] = send[p].first;
                       sl[p] = send[p].second;
                       ro[p] = recv[p].first;
                       rl[p] = recv[p].second;
                     }
                     const void* ip = in.data_ptr();
                     const long long* counts =
                         dev_counts.defined() ? reinterpret_cast<const long long*>(dev_counts.data_ptr<int64_t>()) : nullptr;
                     const size_t in_cap = in.nbytes(), out_cap = out.nbytes();
                     B200C_CUDA_CHECK(launch_symm_all_to_all(&self->comm_dev(), self->layout(), 0, &ip, &sv, &in_cap,
                                                             &out_cap, so.data(), sl.data(), ro.data(), rl.data(),
                                                             counts != nullptr ? &counts : nullptr, elem_bytes,
                                                             !equal_splits, blocks, s));
                   },
                   kChanSymAr, true, blocks);
}

WorkPtr CudaBackend::all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) {
  TORCH_CHECK(static_cast<int>(outs.size()) == size_, "all_gather_v: need size() output tensors");
  check_tensor(in, device_, "all_gather_v", cuda_->is_real());
  TORCH_CHECK(outs[rank_].numel() == in.numel(), "all_gather_v: own output slot must match the input");
  std::vector<std::pair<size_t, size_t>> send(size_), recv(size_);
  size_t total = 0;
  for (int r = 0; r < size_; ++r) {
    check_tensor(outs[r], device_, "all_gather_v", cuda_->is_real());
    TORCH_CHECK(outs[r].scalar_type() == in.scalar_type(), "all_gather_v: dtype mismatch");
    send[r] = {0, in.nbytes()};
    recv[r] = {total, outs[r].nbytes()};
    total += round_up(outs[r].nbytes(), 16);
    recv[r].first = total - round_up(outs[r].nbytes(), 16);
  }
  at::Tensor flat = at::empty({static_cast<int64_t>(std::max<size_t>(total, 16))}, in.options().dtype(at::kByte));
  auto dsts = outs;
  auto offs = recv;
  return exchange(this, "all_gather_v/kernel", in, flat, send, recv, async_op, o, {in, flat},
                  [dsts, flat, offs](cudaStream_t s) {
                    for (size_t r = 0; r < dsts.size(); ++r) {
                      if (offs[r].second == 0) continue;
                      B200C_CUDA_CHECK(cudaMemcpyAsync(dsts[r].data_ptr(), static_cast<char*>(flat.data_ptr()) + offs[r].first,
                                                       offs[r].second, cudaMemcpyDeviceToDevice, s));
                    }
                  });
}

WorkPtr CudaBackend::reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool async_op, const OpOptions& o) {
  check_tensor(out, device_, "reduce_scatter_single", cuda_->is_real());
  check_tensor(in, device_, "reduce_scatter_single", cuda_->is_real());
  TORCH_CHECK(in.numel() == out.numel() * size_, "reduce_scatter_single: input numel must be output numel * size");
  if (out.numel() == 0) return c10::make_intrusive<CompletedWork>();
  {
    int ik = 0, ok = 0;
    const bool sum_like = op.type() == RedOpType::SUM || op.type() == RedOpType::AVG || op.type() == RedOpType::PREMUL_SUM ||
        op.type() == RedOpType::MIN || op.type() == RedOpType::MAX || op.type() == RedOpType::PRODUCT;
    if (size_ == 1 && sum_like && single_rank_kind(in.scalar_type(), &ik) && single_rank_kind(out.scalar_type(), &ok) &&
        reinterpret_cast<uintptr_t>(in.data_ptr()) % 32 == 0 && reinterpret_cast<uintptr_t>(out.data_ptr()) % 32 == 0) {
      at::Tensor i = in, ot = out;
      const float scale = op.type() == RedOpType::PREMUL_SUM ? static_cast<float>(op.factor_as_double()) : 1.0f;
      bytes_issued_ += in.nbytes();
      return run("reduce_scatter/single_rank", async_op, o, {in}, [i, ot, ik, ok, scale](cudaStream_t s) {
        B200C_CUDA_CHECK(launch_cast_scale(i.data_ptr(), ik, ot.data_ptr(), ok, static_cast<size_t>(ot.numel()), scale, s));
      }, kChanSymRs, true);
    }
  }
  const bool same = in.scalar_type() == out.scalar_type();
  const bool plain = same && o.hints.find("wire_dtype") == o.hints.end();
  Algo algo = plain ? route(Coll::REDUCE_SCATTER, in.nbytes(), o) : algo_override(o);
  if (algo == Algo::KERNEL) algo = Algo::AUTO;
  if (!kernels_can_reduce(in.scalar_type(), op) || !kernels_can_reduce(out.scalar_type(), op)) {
    algo = Algo::NCCL;
  }
  if (algo == Algo::NCCL && nccl_comm_ != nullptr && same) {
    NcclDataType dt;
    TORCH_CHECK(to_nccl_dtype(in.scalar_type(), &dt), "reduce_scatter_single: unsupported dtype ", in.scalar_type());
    TORCH_CHECK(op.type() != RedOpType::PREMUL_SUM && op.type() != RedOpType::BAND && op.type() != RedOpType::BOR &&
                    op.type() != RedOpType::BXOR,
                "reduce_scatter_single: this reduction is not available on the NCCL path");
    NcclRedOp rop = kNcclSum;
    switch (op.type()) {
      case RedOpType::PRODUCT: rop = kNcclProd; break;
      case RedOpType::MIN: rop = kNcclMin; break;
      case RedOpType::MAX: rop = kNcclMax; break;
      case RedOpType::AVG: rop = kNcclAvg; break;
      default: break;
    }
    at::Tensor i = in, ot = out;
    return run("reduce_scatter/nccl", async_op, o, {in}, [this, i, ot, dt, rop](cudaStream_t s) {
      nccl_check(nccl_->reduceScatter(i.data_ptr(), ot.data_ptr(), ot.numel(), dt, rop, nccl_comm_, s), "ncclReduceScatter");
    });
  }
  TORCH_CHECK(kernels_can_reduce(in.scalar_type(), op) && kernels_can_reduce(out.scalar_type(), op),
              "reduce_scatter_single: unsupported dtype / reduction (", in.scalar_type(), " -> ", out.scalar_type(), ")");
  DType din, dout;
  to_dtype(in.scalar_type(), &din);
  to_dtype(out.scalar_type(), &dout);
  // Wire dtype: the input's, unless the caller asks for bf16 on the wire
  // (hint "wire_dtype") or mixes fp32 with bf16.
  DType dwire = din;
  auto it = o.hints.find("wire_dtype");
  if (it != o.hints.end() && (it->second == "bf16" || it->second == "bfloat16")) dwire = DType::BF16;
  if (!same) dwire = DType::BF16;
  if (dwire != din || !same) {
    TORCH_CHECK(red_kind(op) == RedKind::SUM, "mixed-precision reduce_scatter supports SUM / AVG / PREMUL_SUM only");
    TORCH_CHECK((din == DType::F32 || din == DType::BF16) && (dout == DType::F32 || dout == DType::BF16),
                "mixed-precision reduce_scatter supports float32 / bfloat16 only");
  }
  const float scale = red_scale(op, size_);
  const RedKind rk = red_kind(op);
  if (algo == Algo::AUTO && rk == RedKind::SUM && size_ > 1 && din == dout && dwire == din && out.nbytes() % 16 == 0 &&
      out.nbytes() <= tune_.lamport_max_bytes && hint_or<unsigned long long>(o.hints, "sr_seed", 0ull) == 0) {
    at::Tensor i = in, ot = out;
    bytes_issued_ += in.nbytes();
    return run("reduce_scatter/lamport", async_op, o, {in}, [this, i, ot, din, scale](cudaStream_t s) {
      const void* ip = i.data_ptr();
      void* op_ = ot.data_ptr();
      B200C_CUDA_CHECK(launch_exchange_lamport(&dev_, layout_, 0, 2, &ip, &op_, ot.nbytes(), din, scale, false, s));
    }, kChanSymAr, true);
  }
  if (algo == Algo::AUTO && rk == RedKind::SUM && dwire == din && hint_or<unsigned long long>(o.hints, "sr_seed", 0ull) == 0) {
    SymmView sv;
    const size_t pack = 16 / dtype_size(din);
    const bool types_ok = din == dout || (din == DType::BF16 && dout == DType::F32);
    if (types_ok && out.numel() % pack == 0 && lookup_symm(in.data_ptr(), in.nbytes(), &sv) &&
        reinterpret_cast<uintptr_t>(in.data_ptr()) % 16 == 0) {
      // The input lives in symmetric memory: every rank reads its slice of
      // every copy (summed by the switch when bound to the multicast object)
      // straight into the output; scale and cast happen in registers.
      const bool smc = symm_use_mc(tune_.symm_rs_mc, false, sv, o);
      const int blocks = symm_blocks_for(smc, out.numel() / pack, o, true);
      at::Tensor i = in, ot = out;
      bytes_issued_ += in.nbytes();
      return run("reduce_scatter/symm", async_op, o, {in}, [this, i, ot, sv, din, dout, scale, smc, blocks](cudaStream_t s) {
        void* op_ = ot.data_ptr();
        B200C_CUDA_CHECK(launch_symm_reduce_scatter(&dev_, 0, &sv, &op_, ot.numel(), din, dout, scale, smc, blocks, s));
      }, kChanSymRs, true, blocks);
    }
  }
  const bool mc = tune_.use_multicast && rk == RedKind::SUM && dev_.mc_heap != nullptr;
  const size_t wire_bytes = out.numel() * dtype_size(dwire);
  LaunchShape shape = shape_for(wire_bytes, size_, in.nbytes() < (64u << 20) ? 148 : 0);
  const size_t oneshot_cap = static_cast<size_t>(kSmallBlocks) * ((kSmallPiece / size_) / 16 * 16);
  const bool oneshot = din == dwire && dwire == dout && algo != Algo::TWOSHOT && algo != Algo::STAGED &&
      out.nbytes() <= std::min(tune_.rs_oneshot_max_bytes, oneshot_cap);
  if (oneshot) {
    shape.chunk_bytes = 0;
    shape.threads = 256;
  }
  at::Tensor i = in, ot = out;
  bytes_issued_ += in.nbytes();
  const unsigned long long sr_seed = hint_or<unsigned long long>(o.hints, "sr_seed", 0ull);
  return run(oneshot ? "reduce_scatter/oneshot" : "reduce_scatter/kernel", async_op, o, {in},
             [this, i, ot, din, dwire, dout, rk, scale, mc, shape, sr_seed](cudaStream_t s) {
               const void* ip = i.data_ptr();
               void* op_ = ot.data_ptr();
               B200C_CUDA_CHECK(launch_reduce_scatter(&dev_, layout_, 0, &ip, &op_, ot.numel(), din, dwire, dout, rk, scale, mc, shape, s, sr_seed));
             }, kChanMain, true);
}

WorkPtr CudaBackend::reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) {
  TORCH_CHECK(static_cast<int>(ins.size()) == size_, "reduce_scatter: need size() input tensors");
  for (auto& t : ins) {
    check_tensor(t, device_, "reduce_scatter", cuda_->is_real());
    TORCH_CHECK(t.numel() == out.numel() && t.scalar_type() == out.scalar_type(),
                "reduce_scatter: every input must match the output's numel and dtype");
  }
  std::vector<at::Tensor> flat_ins;
  for (auto& t : ins) flat_ins.push_back(t.reshape({-1}));
  at::Tensor flat = at::cat(flat_ins);
  return reduce_scatter_single(out, flat, op, async_op, o);
}

WorkPtr CudaBackend::reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) {
  TORCH_CHECK(static_cast<int>(ins.size()) == size_, "reduce_scatter_v: need size() input tensors");
  check_tensor(out, device_, "reduce_scatter_v", cuda_->is_real());
  TORCH_CHECK(ins[rank_].numel() == out.numel(), "reduce_scatter_v: own input slot must match the output");
  // Uneven shares. When they are not too uneven, pad every share to the
  // largest one and reduce-scatter the padded layout: each element then crosses
  // NVLink once, as in the even case. Otherwise (one share dominates) all-reduce
  // the concatenation and keep the own share.
  int64_t total = 0, max_share = 0;
  for (int r = 0; r < size_; ++r) {
    check_tensor(ins[r], device_, "reduce_scatter_v", cuda_->is_real());
    TORCH_CHECK(ins[r].scalar_type() == out.scalar_type(), "reduce_scatter_v: dtype mismatch");
    total += ins[r].numel();
    max_share = std::max<int64_t>(max_share, ins[r].numel());
  }
  if (total == 0) return c10::make_intrusive<CompletedWork>();
  const int64_t pack = std::max<int64_t>(1, 16 / static_cast<int64_t>(out.element_size()));
  const int64_t padded = (max_share + pack - 1) / pack * pack;
  if (padded * size_ <= 2 * total) {
    at::Tensor flat = at::zeros({padded * size_}, out.options());
    for (int r = 0; r < size_; ++r) {
      if (ins[r].numel() > 0) flat.narrow(0, r * padded, ins[r].numel()).copy_(ins[r].reshape({-1}));
    }
    at::Tensor mine = at::empty({padded}, out.options());
    WorkPtr w = reduce_scatter_single(mine, flat, op, async_op, o);
    at::Tensor dst = out;
    const int64_t len = out.numel();
    if (len == 0) return w;
    if (async_op) w->wait();  // the copy below may run on another channel's stream: order it behind the reduction
    // The copy-out is stream-ordered behind the reduce-scatter (same channel).
    return run("reduce_scatter_v/copy", async_op, o, {flat, mine}, [mine, dst, len](cudaStream_t s) {
      B200C_CUDA_CHECK(cudaMemcpyAsync(dst.data_ptr(), mine.data_ptr(), len * mine.element_size(), cudaMemcpyDeviceToDevice, s));
    });
  }
  std::vector<at::Tensor> flat_ins;
  int64_t my_off = 0, off = 0;
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) my_off = off;
    off += ins[r].numel();
    flat_ins.push_back(ins[r].reshape({-1}));
  }
  at::Tensor flat = at::cat(flat_ins);
  WorkPtr reduced = all_reduce(flat, op, async_op, o);
  if (async_op) reduced->wait();  // the copy below may run on another channel's stream
  at::Tensor dst = out;
  const int64_t len = out.numel();
  // The copy-out is stream-ordered behind the all-reduce.
  return run("reduce_scatter_v/copy", async_op, o, {flat}, [flat, dst, my_off, len](cudaStream_t s) {
    B200C_CUDA_CHECK(cudaMemcpyAsync(dst.data_ptr(), static_cast<char*>(flat.data_ptr()) + my_off * flat.element_size(),
                                     len * flat.element_size(), cudaMemcpyDeviceToDevice, s));
  });
}

// Baseline route: the exchange as grouped NCCL send/recv pairs (how NCCL
// backends implement all-to-all-v). Byte offsets and counts.
WorkPtr CudaBackend::exchange_nccl(const char* what, const at::Tensor& in, at::Tensor& out,
                                   const std::vector<std::pair<size_t, size_t>>& send,
                                   const std::vector<std::pair<size_t, size_t>>& recv, bool async_op, const OpOptions& o) {
  at::Tensor i = in, ot = out;
  return run(what, async_op, o, {in}, [this, i, ot, send, recv](cudaStream_t s) {
    nccl_check(nccl_->groupStart(), "ncclGroupStart");
    for (int p = 0; p < size_; ++p) {
      if (send[p].second > 0) {
        nccl_check(nccl_->send(static_cast<const char*>(i.data_ptr()) + send[p].first, send[p].second, kNcclUint8, p, nccl_comm_, s),
                   "ncclSend");
      }
      if (recv[p].second > 0) {
        nccl_check(nccl_->recv(static_cast<char*>(ot.data_ptr()) + recv[p].first, recv[p].second, kNcclUint8, p, nccl_comm_, s),
                   "ncclRecv");
      }
    }
    nccl_check(nccl_->groupEnd(), "ncclGroupEnd");
  });
}

WorkPtr CudaBackend::all_to_all_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) {
  check_tensor(out, device_, "all_to_all_single", cuda_->is_real());
  check_tensor(in, device_, "all_to_all_single", cuda_->is_real());
  TORCH_CHECK(out.numel() == in.numel() && out.scalar_type() == in.scalar_type(),
              "all_to_all_single: input and output must have the same numel and dtype");
  TORCH_CHECK(in.numel() % size_ == 0, "all_to_all_single: numel must divide by size()");
  if (in.numel() == 0) return c10::make_intrusive<CompletedWork>();
  const size_t blk = in.nbytes() / size_;
  std::vector<std::pair<size_t, size_t>> send(size_), recv(size_);
  for (int p = 0; p < size_; ++p) {
    send[p] = {p * blk, blk};
    recv[p] = {p * blk, blk};
  }
  bytes_issued_ += in.nbytes();
  {
    const Algo forced = algo_override(o);
    if ((forced == Algo::AUTO || forced == Algo::KERNEL) && size_ > 1 && lamport_dtype(in.scalar_type()) && blk % 16 == 0 &&
        blk <= tune_.lamport_max_bytes) {
      at::Tensor i = in, ot = out;
      return run("all_to_all_single/lamport", async_op, o, {in}, [this, i, ot, blk](cudaStream_t s) {
        const void* ip = i.data_ptr();
        void* op_ = ot.data_ptr();
        B200C_CUDA_CHECK(launch_exchange_lamport(&dev_, layout_, 0, 1, &ip, &op_, blk, DType::F32, 1.0f, false, s));
      }, kChanSymAr, true);
    }
    SymmView sv;
    if ((forced == Algo::AUTO || forced == Algo::KERNEL) && size_ > 1 && lookup_symm(out.data_ptr(), out.nbytes(), &sv)) {
      return exchange_symm(this, "all_to_all_single/symm", in, out, sv, send, recv, true, at::Tensor(), 1, async_op, o);
    }
  }
  if (nccl_comm_ != nullptr && route(Coll::ALL_TO_ALL, in.nbytes(), o) == Algo::NCCL) {
    return exchange_nccl("all_to_all_single/nccl", in, out, send, recv, async_op, o);
  }
  return exchange(this, "all_to_all_single/kernel", in, out, send, recv, async_op, o, {in}, nullptr, blk);
}

WorkPtr CudaBackend::all_to_all_v_single(at::Tensor& out, const at::Tensor& in, const std::vector<int64_t>& out_splits,
                                         const std::vector<int64_t>& in_splits, bool async_op, const OpOptions& o) {
  check_tensor(out, device_, "all_to_all_v_single", cuda_->is_real());
  check_tensor(in, device_, "all_to_all_v_single", cuda_->is_real());
  TORCH_CHECK(out.scalar_type() == in.scalar_type(), "all_to_all_v_single: dtype mismatch");
  TORCH_CHECK(static_cast<int>(out_splits.size()) == size_ && static_cast<int>(in_splits.size()) == size_,
              "all_to_all_v_single: need size() split sizes on both sides");
  // Split sizes count dim-0 slices.
  const size_t in_row = in.dim() > 0 && in.size(0) > 0 ? in.nbytes() / in.size(0) : in.element_size();
  const size_t out_row = out.dim() > 0 && out.size(0) > 0 ? out.nbytes() / out.size(0) : out.element_size();
  std::vector<std::pair<size_t, size_t>> send(size_), recv(size_);
  size_t so = 0, ro = 0;
  for (int p = 0; p < size_; ++p) {
    TORCH_CHECK(in_splits[p] >= 0 && out_splits[p] >= 0, "all_to_all_v_single: negative split size");
    send[p] = {so, in_splits[p] * in_row};
    recv[p] = {ro, out_splits[p] * out_row};
    so += send[p].second;
    ro += recv[p].second;
  }
  TORCH_CHECK(so <= in.nbytes(), "all_to_all_v_single: input splits exceed the input tensor");
  TORCH_CHECK(ro <= out.nbytes(), "all_to_all_v_single: output splits exceed the output tensor");
  bytes_issued_ += so;
  {
    const Algo forced = algo_override(o);
    // The flag-less exchange needs a bound on every part that all ranks share. The caller may give one
    // (hint `max_part_bytes`, the same on every rank; then the tensors may live anywhere) ...
    const size_t hinted = hint_or<size_t>(o.hints, "max_part_bytes", 0);
    if ((forced == Algo::AUTO || forced == Algo::KERNEL) && size_ > 1 && hinted > 0 && hinted <= tune_.lamport_max_bytes &&
        lamport_dtype(out.scalar_type())) {
      for (int p = 0; p < size_; ++p) {
        TORCH_CHECK(send[p].second <= hinted && recv[p].second <= hinted,
                    "all_to_all_v_single: a part exceeds the max_part_bytes hint (", hinted, ")");
      }
      at::Tensor i = in, ot = out;
      return run("all_to_all_v_single/lamport", async_op, o, {in}, [this, i, ot, send, recv, hinted](cudaStream_t s) {
        size_t so[kMaxRanks] = {}, sl[kMaxRanks] = {}, ro[kMaxRanks] = {}, rl[kMaxRanks] = {};
        for (int p = 0; p < size_; ++p) {
          so[p] = send[p].first;
          sl[p] = send[p].second;
          ro[p] = recv[p].first;
          rl[p] = recv[p].second;
        }
        const void* ip = i.data_ptr();
        void* op = ot.data_ptr();
        B200C_CUDA_CHECK(launch_exchangev_lamport(&dev_, layout_, 0, &ip, &op, so, sl, ro, rl, hinted, s));
      }, kChanSymAr, true);
    }
    // ... or it follows from the size of a symmetric receive buffer.
    SymmView sv;
    size_t region = 0;
    if ((forced == Algo::AUTO || forced == Algo::KERNEL) && size_ > 1 && lookup_symm(out.data_ptr(), out.nbytes(), &sv, &region)) {
      // A small symmetric receive buffer bounds every part on every rank by the same number (no part can be larger
      // than the buffer it lands in, and the buffer has the same size everywhere): the flag-less exchange, no
      // barrier. Floating types only (a payload word equal to the poison value travels as +0.0).
      if (region <= tune_.lamport_max_bytes && lamport_dtype(out.scalar_type())) {
        at::Tensor i = in, ot = out;
        return run("all_to_all_v_single/lamport", async_op, o, {in}, [this, i, ot, send, recv, region](cudaStream_t s) {
          size_t so[kMaxRanks] = {}, sl[kMaxRanks] = {}, ro[kMaxRanks] = {}, rl[kMaxRanks] = {};
          for (int p = 0; p < size_; ++p) {
            so[p] = send[p].first;
            sl[p] = send[p].second;
            ro[p] = recv[p].first;
            rl[p] = recv[p].second;
          }
          const void* ip = i.data_ptr();
          void* op = ot.data_ptr();
          B200C_CUDA_CHECK(launch_exchangev_lamport(&dev_, layout_, 0, &ip, &op, so, sl, ro, rl, region, s));
        }, kChanSymAr, true);
      }
      return exchange_symm(this, "all_to_all_v_single/symm", in, out, sv, send, recv, false, at::Tensor(), 1, async_op, o);
    }
  }
  if (nccl_comm_ != nullptr && route(Coll::ALL_TO_ALL, so, o) == Algo::NCCL) {
    return exchange_nccl("all_to_all_v_single/nccl", in, out, send, recv, async_op, o);
  }
  return exchange(this, "all_to_all_v_single/kernel", in, out, send, recv, async_op, o, {in});
}

WorkPtr CudaBackend::all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool async_op, const OpOptions& o) {
  TORCH_CHECK(static_cast<int>(outs.size()) == size_ && static_cast<int>(ins.size()) == size_,
              "all_to_all: need size() input and output tensors");
  std::vector<std::pair<size_t, size_t>> send(size_), recv(size_);
  std::vector<at::Tensor> flat_ins;
  size_t so = 0, ro = 0;
  for (int p = 0; p < size_; ++p) {
    check_tensor(ins[p], device_, "all_to_all", cuda_->is_real());
    check_tensor(outs[p], device_, "all_to_all", cuda_->is_real());
    TORCH_CHECK(ins[p].scalar_type() == ins[0].scalar_type() && outs[p].scalar_type() == ins[0].scalar_type(),
                "all_to_all: every tensor must have the same dtype");
    send[p] = {so, ins[p].nbytes()};
    recv[p] = {ro, outs[p].nbytes()};
    so += ins[p].nbytes();
    ro += round_up(outs[p].nbytes(), 16);
    flat_ins.push_back(ins[p].reshape({-1}));
  }
  at::Tensor in = at::cat(flat_ins);
  at::Tensor out = at::empty({static_cast<int64_t>(std::max<size_t>(ro, 16))}, in.options().dtype(at::kByte));
  auto dsts = outs;
  auto offs = recv;
  return exchange(this, "all_to_all_list/kernel", in, out, send, recv, async_op, o, {in, out},
                  [dsts, out, offs](cudaStream_t s) {
                    for (size_t r = 0; r < dsts.size(); ++r) {
                      if (offs[r].second == 0) continue;
                      B200C_CUDA_CHECK(cudaMemcpyAsync(dsts[r].data_ptr(), static_cast<char*>(out.data_ptr()) + offs[r].first,
                                                       offs[r].second, cudaMemcpyDeviceToDevice, s));
                    }
                  });
}

WorkPtr CudaBackend::device_alltoallv_single(at::Tensor& out, const at::Tensor& in, const at::Tensor& out_splits,
                                             const at::Tensor& in_splits, bool async_op, const OpOptions& o) {
  check_tensor(out, device_, "device_alltoallv_single", cuda_->is_real());
  check_tensor(in, device_, "device_alltoallv_single", cuda_->is_real());
  check_tensor(in_splits, device_, "device_alltoallv_single", cuda_->is_real());
  TORCH_CHECK(in_splits.scalar_type() == at::kLong && in_splits.numel() == size_,
              "device_alltoallv_single: input_split_sizes must be an int64 device tensor of size() entries");
  TORCH_CHECK(out.scalar_type() == in.scalar_type(), "device_alltoallv_single: dtype mismatch");
  const size_t row = in.dim() > 0 && in.size(0) > 0 ? in.nbytes() / in.size(0) : in.element_size();
  {
    const size_t out_row = out.dim() > 0 && out.size(0) > 0 ? out.nbytes() / out.size(0) : out.element_size();
    TORCH_CHECK(out_row == row, "device_alltoallv_single: input and output must have the same dim-0 slice size (",
                row, " vs ", out_row, " bytes)");
  }
  // Receive sizes are learnt from the senders on the device; `out_splits` is
  // the caller's own view of them and is only checked for shape.
  if (out_splits.defined() && out_splits.numel() != 0) {
    TORCH_CHECK(out_splits.scalar_type() == at::kLong && out_splits.numel() == size_,
                "device_alltoallv_single: output_split_sizes must be an int64 tensor of size() entries");
  }
  {
    SymmView sv;
    const Algo forced = algo_override(o);
    if ((forced == Algo::AUTO || forced == Algo::KERNEL) && size_ > 1 && lookup_symm(out.data_ptr(), out.nbytes(), &sv)) {
      std::vector<std::pair<size_t, size_t>> none(size_, {0, 0});
      return exchange_symm(this, "device_alltoallv/symm", in, out, sv, none, none, false, in_splits, row, async_op, o);
    }
  }
  LaunchShape shape;
  shape.threads = tune_.threads;
  shape.blocks = std::min(32, tune_.max_blocks);
  shape.chunk_bytes = std::min<size_t>(tune_.max_chunk_bytes, layout_.bulk_bytes / (static_cast<size_t>(shape.blocks) * size_ * kPipeSlots)) / 256 * 256;
  at::Tensor i = in, ot = out, sp = in_splits;
  return run("device_alltoallv/kernel", async_op, o, {in, in_splits}, [this, i, ot, sp, row, shape](cudaStream_t s) {
    const void* ip = i.data_ptr();
    void* op_ = ot.data_ptr();
    const long long* counts = reinterpret_cast<const long long*>(sp.data_ptr<int64_t>());
    const size_t in_cap = i.nbytes(), out_cap = ot.nbytes();
    B200C_CUDA_CHECK(launch_all_to_all_device_splits(&dev_, layout_, 0, &ip, &op_, &counts, row, shape, s, &in_cap, &out_cap));
  }, kChanMain, true);
}

WorkPtr CudaBackend::reduce_scatter_quantized(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, int64_t seed,
                                              bool async_op, const OpOptions& o) {
  TORCH_CHECK(in.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat,
              "reduce_scatter_quantized: float32 input and output");
  OpOptions oo = o;
  oo.hints["wire_dtype"] = "bf16";
  // seed 0 = round to nearest; anything else seeds the stochastic rounding of the wire values
  oo.hints["sr_seed"] = std::to_string(static_cast<unsigned long long>(seed));
  return reduce_scatter_single(out, in, op, async_op, oo);
}

WorkPtr CudaBackend::seq_heads_exchange(at::Tensor& out, const at::Tensor& in, bool to_heads, bool async_op,
                                        const OpOptions& o) {
  check_tensor(in, device_, "seq_heads_exchange", cuda_->is_real());
  check_tensor(out, device_, "seq_heads_exchange", cuda_->is_real());
  TORCH_CHECK(in.dim() == 4 && out.dim() == 4 && in.is_contiguous() && out.is_contiguous(),
              "seq_heads_exchange: contiguous [batch, heads, seq, dim] tensors");
  TORCH_CHECK(in.scalar_type() == out.scalar_type(), "seq_heads_exchange: dtype mismatch");
  const at::Tensor& full = to_heads ? in : out;       // [b, h, s, d]
  const at::Tensor& grouped = to_heads ? out : in;    // [b, h / n, n * s, d]
  const int64_t b = full.size(0), h = full.size(1), s_local = full.size(2), d = full.size(3);
  TORCH_CHECK(h % size_ == 0, "seq_heads_exchange: heads (", h, ") must divide by the number of ranks (", size_, ")");
  TORCH_CHECK(grouped.size(0) == b && grouped.size(1) == h / size_ && grouped.size(2) == s_local * size_ && grouped.size(3) == d,
              "seq_heads_exchange: expected [", b, ", ", h / size_, ", ", s_local * size_, ", ", d, "] on the head-sharded side");
  if (in.numel() == 0) return c10::make_intrusive<CompletedWork>();
  if (size_ == 1) {
    at::Tensor dst = out, src = in;
    return run("seq_heads_exchange/copy", async_op, o, {in, out}, [dst, src](cudaStream_t st) {
      B200C_CUDA_CHECK(cudaMemcpyAsync(dst.data_ptr(), src.data_ptr(), src.nbytes(), cudaMemcpyDeviceToDevice, st));
    });
  }
  SymmView sv;
  TORCH_CHECK(lookup_symm(out.data_ptr(), out.nbytes(), &sv),
              "seq_heads_exchange: the output must be a symmetric tensor (symm_empty or a registered allocation)");
  const size_t slab = static_cast<size_t>(s_local) * d * in.element_size();
  const size_t want = (in.nbytes() / 16 + 512 * 4 - 1) / (512 * 4);
  const int blocks = static_cast<int>(std::max<size_t>(
      1, std::min<size_t>(std::min(128, hint_or<int>(o.hints, "symm_blocks", tune_.symm_blocks_nomc)), want)));
  bytes_issued_ += in.nbytes();
  at::Tensor src = in;
  return run("seq_heads_exchange/symm", async_op, o, {in, out},
             [this, src, sv, b, h, slab, to_heads, blocks](cudaStream_t st) {
               const void* ip = src.data_ptr();
               B200C_CUDA_CHECK(launch_symm_seq_heads(&dev_, 0, &ip, &sv, static_cast<int>(b), static_cast<int>(h), slab,
                                                      to_heads, blocks, st));
             },
             kChanSymAr, true, blocks);
}

WorkPtr CudaBackend::broadcast(at::Tensor& t, int root, bool async_op, const OpOptions& o) {
  check_tensor(t, device_, "broadcast", cuda_->is_real());
  if (t.numel() == 0 || size_ == 1) return c10::make_intrusive<CompletedWork>();
  NcclDataType ndt;
  if (algo_override(o) == Algo::NCCL && nccl_comm_ != nullptr && to_nccl_dtype(t.scalar_type(), &ndt)) {
    at::Tensor tt = t;
    return run("broadcast/nccl", async_op, o, {t}, [this, tt, ndt, root](cudaStream_t s) {
      nccl_check(nccl_->broadcast(tt.data_ptr(), tt.data_ptr(), tt.numel(), ndt, root, nccl_comm_, s), "ncclBroadcast");
    });
  }
  const size_t bytes = t.nbytes();
  const LaunchShape shape = shape_for(bytes, 1);
  at::Tensor tt = t;
  bytes_issued_ += bytes;
  return run("broadcast/kernel", async_op, o, {t}, [this, tt, bytes, root, shape](cudaStream_t s) {
    void* p = tt.data_ptr();
    B200C_CUDA_CHECK(launch_broadcast(&dev_, layout_, 0, &p, bytes, root, dev_.mc_heap != nullptr, shape, s));
  });
}

WorkPtr CudaBackend::barrier(bool async_op, const OpOptions& o) {
  return run("barrier/kernel", async_op, o, {}, [this](cudaStream_t s) {
    B200C_CUDA_CHECK(launch_barrier(&dev_, 0, s));
  });
}

WorkPtr CudaBackend::scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool async_op, const OpOptions& o) {
  check_tensor(out, device_, "scatter", cuda_->is_real());
  std::vector<std::pair<size_t, size_t>> send(size_, {0, 0}), recv(size_, {0, 0});
  at::Tensor in;
  if (rank_ == root) {
    TORCH_CHECK(static_cast<int>(ins.size()) == size_, "scatter: the root needs size() input tensors");
    std::vector<at::Tensor> flat_ins;
    size_t off = 0;
    for (int p = 0; p < size_; ++p) {
      check_tensor(ins[p], device_, "scatter", cuda_->is_real());
      TORCH_CHECK(ins[p].numel() == out.numel() && ins[p].scalar_type() == out.scalar_type(),
                  "scatter: every input must match the output's numel and dtype");
      send[p] = {off, ins[p].nbytes()};
      off += ins[p].nbytes();
      flat_ins.push_back(ins[p].reshape({-1}));
    }
    in = at::cat(flat_ins);
  } else {
    in = at::empty({0}, out.options());
  }
  recv[root] = {0, out.nbytes()};
  return exchange(this, "scatter/kernel", in, out, send, recv, async_op, o, {in});
}

WorkPtr CudaBackend::gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool async_op, const OpOptions& o) {
  check_tensor(in, device_, "gather", cuda_->is_real());
  std::vector<std::pair<size_t, size_t>> send(size_, {0, 0}), recv(size_, {0, 0});
  send[root] = {0, in.nbytes()};
  at::Tensor out;
  std::function<void(cudaStream_t)> after;
  if (rank_ == root) {
    TORCH_CHECK(static_cast<int>(outs.size()) == size_, "gather: the root needs size() output tensors");
    const size_t blk = round_up(in.nbytes(), 16);
    for (int p = 0; p < size_; ++p) {
      check_tensor(outs[p], device_, "gather", cuda_->is_real());
      TORCH_CHECK(outs[p].numel() == in.numel() && outs[p].scalar_type() == in.scalar_type(),
                  "gather: every output must match the input's numel and dtype");
      recv[p] = {p * blk, in.nbytes()};
    }
    out = at::empty({static_cast<int64_t>(std::max<size_t>(blk * size_, 16))}, in.options().dtype(at::kByte));
    auto dsts = outs;
    auto offs = recv;
    at::Tensor flat = out;
    after = [dsts, flat, offs](cudaStream_t s) {
      for (size_t r = 0; r < dsts.size(); ++r) {
        if (offs[r].second == 0) continue;
        B200C_CUDA_CHECK(cudaMemcpyAsync(dsts[r].data_ptr(), static_cast<char*>(flat.data_ptr()) + offs[r].first,
                                         offs[r].second, cudaMemcpyDeviceToDevice, s));
      }
    };
  } else {
    out = at::empty({16}, in.options().dtype(at::kByte));
  }
  return exchange(this, "gather/kernel", in, out, send, recv, async_op, o, {in, out}, after);
}

WorkPtr CudaBackend::send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o) {
  check_tensor(t, device_, "send", cuda_->is_real());
  TORCH_CHECK(nccl_comm_ != nullptr, "send needs NCCL (communicator created with use_nccl=0, or libnccl missing)");
  NcclDataType dt;
  TORCH_CHECK(to_nccl_dtype(t.scalar_type(), &dt), "send: unsupported dtype ", t.scalar_type());
  at::Tensor tt = t;
  return run("send/nccl", async_op, o, {t}, [this, tt, dt, dst](cudaStream_t s) {
    nccl_check(nccl_->send(tt.data_ptr(), tt.numel(), dt, dst, nccl_comm_, s), "ncclSend");
  });
}

WorkPtr CudaBackend::recv(at::Tensor& t, int src, bool async_op, const OpOptions& o) {
  check_tensor(t, device_, "recv", cuda_->is_real());
  TORCH_CHECK(nccl_comm_ != nullptr, "recv needs NCCL (communicator created with use_nccl=0, or libnccl missing)");
  NcclDataType dt;
  TORCH_CHECK(to_nccl_dtype(t.scalar_type(), &dt), "recv: unsupported dtype ", t.scalar_type());
  at::Tensor tt = t;
  return run("recv/nccl", async_op, o, {t}, [this, tt, dt, src](cudaStream_t s) {
    nccl_check(nccl_->recv(tt.data_ptr(), tt.numel(), dt, src, nccl_comm_, s), "ncclRecv");
  });
}

WorkPtr CudaBackend::batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o) {
  if (ops.empty()) return c10::make_intrusive<CompletedWork>();
  TORCH_CHECK(nccl_comm_ != nullptr, "batched send/recv needs NCCL");
  std::vector<at::Tensor> keep;
  for (auto& op : ops) {
    check_tensor(op.tensor, device_, "batch_op_issue", cuda_->is_real());
    keep.push_back(op.tensor);
  }
  auto copy = ops;
  return run("batch_p2p/nccl", async_op, o, keep, [this, copy](cudaStream_t s) {
    nccl_check(nccl_->groupStart(), "ncclGroupStart");
    for (auto& op : copy) {
      NcclDataType dt;
      TORCH_CHECK(to_nccl_dtype(op.tensor.scalar_type(), &dt), "batch_op_issue: unsupported dtype");
      if (op.kind == P2PKind::SEND) {
        nccl_check(nccl_->send(op.tensor.data_ptr(), op.tensor.numel(), dt, op.peer, nccl_comm_, s), "ncclSend");
      } else {
        nccl_check(nccl_->recv(op.tensor.data_ptr(), op.tensor.numel(), dt, op.peer, nccl_comm_, s), "ncclRecv");
      }
    }
    nccl_check(nccl_->groupEnd(), "ncclGroupEnd");
  });
}

std::shared_ptr<Backend> CudaBackend::split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) {
  check_usable();
  const uint64_t gen = split_counter_++;
  if (ranks.empty()) {
    return nullptr;
  }
  int color = ranks[0], idx = -1;
  for (size_t i = 0; i < ranks.size(); ++i) {
    color = std::min(color, ranks[i]);
    if (ranks[i] == rank_) idx = static_cast<int>(i);
  }
  TORCH_CHECK(idx >= 0, "split: calling rank is not a member of the new group");
  auto child = std::make_shared<CudaBackend>(registered_as_);
  child->device_ = device_;
  child->name_ = name_ + "::split::" + std::to_string(color) + "_" + name + "_" + std::to_string(gen);
  child->opts_ = opts;
  child->opts_.store = nullptr;
  child->drv_ = drv_;
  child->cuda_ = cuda_;
  child->nccl_ = nccl_;
  child->tune_ = tune_;
  for (int i = 0; i < 4; ++i) child->tuner_rules_[i] = tuner_rules_[i];
  child->parse_tuning(opts.hints);
  auto sub = scoped_store(store_, "split/" + std::to_string(gen) + "/" + std::to_string(color));
  child->bootstrap(sub, idx, static_cast<int>(ranks.size()));
  return child;
}

std::shared_ptr<Backend> CudaBackend::create_pair_comm(int peer, const std::string& name) {
  check_usable();
  TORCH_CHECK(peer >= 0 && peer < size_ && peer != rank_, "create_pair_comm: bad peer ", peer);
  auto child = std::make_shared<CudaBackend>(registered_as_);
  child->device_ = device_;
  child->name_ = name_ + "::" + name;
  child->opts_ = opts_;
  child->opts_.store = nullptr;
  child->drv_ = drv_;
  child->cuda_ = cuda_;
  child->nccl_ = nccl_;
  child->tune_ = tune_;
  for (int i = 0; i < 4; ++i) child->tuner_rules_[i] = tuner_rules_[i];
  // Point-to-point only: a small staging heap and no multicast object per pair.
  child->tune_.staging_bytes = std::min<size_t>(tune_.staging_bytes, 4u << 20);
  child->tune_.use_multicast = false;
  auto sub = scoped_store(store_, "pair/" + name);
  child->bootstrap(sub, rank_ < peer ? 0 : 1, 2);
  return child;
}

std::unordered_map<std::string, std::string> CudaBackend::comm_dump() const {
  std::unordered_map<std::string, std::string> d;
  d["name"] = name_;
  d["backend"] = registered_as_;
  d["rank"] = std::to_string(rank_);
  d["size"] = std::to_string(size_);
  d["device"] = std::to_string(device_.index());
  d["symm_mode"] = symm_ ? (symm_->mode() == SymmMode::VMM_FD ? "vmm+fd" : symm_->mode() == SymmMode::CUDA_IPC ? "cuda-ipc" : "local") : "none";
  d["multicast"] = dev_.mc_heap != nullptr ? "1" : "0";
  d["nccl"] = nccl_comm_ != nullptr ? "1" : "0";
  d["staging_bytes"] = std::to_string(layout_.bulk_bytes);
  d["ops_issued"] = std::to_string(ops_issued_.load());
  d["bytes_issued"] = std::to_string(bytes_issued_.load());
  d["failed"] = failed_.load() ? failure_text_ : "";
  d["tuning/staging_bytes"] = std::to_string(tune_.staging_bytes);
  d["tuning/oneshot_max_bytes"] = std::to_string(tune_.oneshot_max_bytes);
  d["tuning/lamport_max_bytes"] = std::to_string(tune_.lamport_max_bytes);
  d["tuning/symm_blocks"] = std::to_string(tune_.symm_blocks);
  d["tuning/symm_blocks_nomc"] = std::to_string(tune_.symm_blocks_nomc);
  d["tuning/max_blocks"] = std::to_string(tune_.max_blocks);
  d["tuning/threads"] = std::to_string(tune_.threads);
  d["tuning/auto_nccl"] = tune_.auto_nccl ? "1" : "0";
  d["tuning/tuner_file"] = tune_.tuner_file;
  d["tuning/tuner_rules"] = std::to_string(tuner_rules_[0].size() + tuner_rules_[1].size() + tuner_rules_[2].size() + tuner_rules_[3].size());
  d["tuning/use_multicast"] = tune_.use_multicast ? "1" : "0";
  d["tuning/channel_streams"] = tune_.channel_streams ? "1" : "0";
  d["tuning/fast_sync"] = tune_.fast_sync ? "1" : "0";
  d["tuning/device_wait_ms"] = std::to_string(tune_.device_wait_ns / 1000000ull);
  d["tuning/max_event_pool"] = std::to_string(tune_.max_event_pool);
  d["tuning/watchdog_interval_ms"] = std::to_string(tune_.watchdog_interval_ms);
  {
    std::lock_guard<std::mutex> g(const_cast<std::mutex&>(pool_mu_));
    d["event_pool"] = std::to_string(event_pool_.size());
  }
  {
    std::lock_guard<std::mutex> g(symm_mu_);
    d["symm_regions"] = std::to_string(symm_regs_.size());
  }
  {
    std::lock_guard<std::mutex> g(const_cast<std::mutex&>(wd_mu_));
    d["inflight"] = std::to_string(inflight_.size());
    d["colltrace/entries"] = std::to_string(trace_meta_.size());
    d["colltrace/issued"] = std::to_string(trace_next_);
    d["graph_entries"] = std::to_string(graph_entries_.size());
    d["graphs"] = std::to_string(graphs_.size());
    for (auto& kv : algo_counts_) {
      d["count/" + kv.first] = std::to_string(kv.second);
    }
  }
  return d;
}

// ------------------------------------------------------ symmetric tensors ----

at::Tensor CudaBackend::symm_empty(const std::vector<int64_t>& sizes, at::ScalarType dtype) {
  check_usable();
  DeviceScope guard(cuda_, device_.index());
  int64_t numel = 1;
  for (int64_t d : sizes) {
    TORCH_CHECK(d >= 0, "symm_empty: negative dimension");
    numel *= d;
  }
  const size_t bytes = static_cast<size_t>(numel) * c10::elementSize(dtype);
  auto seg = symm_->allocate(std::max<size_t>(bytes, 16), tune_.use_multicast);
  {
    std::lock_guard<std::mutex> g(symm_mu_);
    symm_regs_[reinterpret_cast<uintptr_t>(seg->local())] = SymmReg{seg->bytes, seg, false, std::max<size_t>(bytes, 16)};
  }
  // The segment, not the tensor, owns the memory (unmapping is a collective matter).
  // (Under a test fake of the runtime the "device" memory is host memory.)
  const at::Device where = cuda_->is_real() ? device_ : at::Device(at::kCPU);
  return at::from_blob(seg->local(), sizes, [](void*) {}, at::TensorOptions().dtype(dtype).device(where));
}

void CudaBackend::symm_free(const at::Tensor& t) {
  check_usable();
  DeviceScope guard(cuda_, device_.index());
  std::shared_ptr<SymmSegment> seg;
  {
    std::lock_guard<std::mutex> g(symm_mu_);
    auto it = symm_regs_.find(reinterpret_cast<uintptr_t>(t.data_ptr()));
    TORCH_CHECK(it != symm_regs_.end() && !it->second.user_memory, "symm_free: not a tensor made by symm_empty()");
    seg = it->second.seg;
    symm_regs_.erase(it);
  }
  // Nobody may still be reading or writing this rank's copy.
  sync_own_streams();
  if (size_ > 1) {
    store_barrier(*store_, "symm_free/" + std::to_string(symm_free_seq_++), rank_, size_, opts_.timeout);
  }
  symm_->release(seg);
}

void CudaBackend::tensor_register(const at::Tensor& t) {
  check_usable();
  check_tensor(t, device_, "tensor_register", cuda_->is_real());
  DeviceScope guard(cuda_, device_.index());
  // Memory from the communicator's allocator is registered as the whole
  // allocation (every tensor inside it is then covered, and it can be bound to
  // the multicast object); anything else as the tensor's own range over CUDA IPC.
  void* base = t.data_ptr();
  size_t bytes = t.nbytes();
  ExportableAlloc a;
  if (ExportableRegistry::get().find(base, bytes, &a)) {
    base = reinterpret_cast<void*>(a.base);
    bytes = a.bytes;
  }
  {
    std::lock_guard<std::mutex> g(symm_mu_);
    if (symm_regs_.count(reinterpret_cast<uintptr_t>(base)) != 0) return;  // same decision on every rank
  }
  auto seg = symm_->attach_user_buffer(base, bytes, tune_.use_multicast);
  std::lock_guard<std::mutex> g(symm_mu_);
  symm_regs_[reinterpret_cast<uintptr_t>(base)] = SymmReg{bytes, seg, true, bytes};
}

void CudaBackend::tensor_deregister(const at::Tensor& t) {
  check_usable();
  DeviceScope guard(cuda_, device_.index());
  std::shared_ptr<SymmSegment> seg;
  {
    std::lock_guard<std::mutex> g(symm_mu_);
    const uintptr_t p = reinterpret_cast<uintptr_t>(t.data_ptr());
    auto it = symm_regs_.upper_bound(p);
    TORCH_CHECK(it != symm_regs_.begin(), "tensor_deregister: tensor is not registered");
    --it;
    TORCH_CHECK(p < it->first + it->second.bytes && it->second.user_memory, "tensor_deregister: tensor is not registered");
    seg = it->second.seg;
    symm_regs_.erase(it);
  }
  sync_own_streams();
  if (size_ > 1) {
    store_barrier(*store_, "symm_free/" + std::to_string(symm_free_seq_++), rank_, size_, opts_.timeout);
  }
  symm_->release(seg);
}

bool CudaBackend::lookup_symm(const void* p, size_t bytes, SymmView* view, size_t* region_bytes) const {
  std::lock_guard<std::mutex> g(symm_mu_);
  if (symm_regs_.empty()) return false;
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  auto it = symm_regs_.upper_bound(a);
  if (it == symm_regs_.begin()) return false;
  --it;
  if (a + bytes > it->first + it->second.bytes) return false;
  const size_t off = a - it->first;
  const SymmSegment& seg = *it->second.seg;
  for (int r = 0; r < kMaxRanks; ++r) {
    view->ptr[r] = r < size_ ? seg.peer_ptrs[r] + off : nullptr;
  }
  view->mc = seg.mc_ptr != nullptr ? seg.mc_ptr + off : nullptr;
  if (region_bytes != nullptr) *region_bytes = it->second.user_bytes;
  return true;
}

std::shared_ptr<Window> CudaBackend::new_window(const std::optional<at::Tensor>& tensor) {
  check_usable();
  auto self = std::static_pointer_cast<CudaBackend>(shared_from_this());
  auto w = std::make_shared<CudaWindow>(self);
  if (tensor) {
    w->tensor_register(*tensor, true);
  }
  return w;
}

// ----------------------------------------------------------- CudaWindow ----

namespace {
constexpr int kHostSignalId = 0;  // signal slot used by the host-side signal()/wait_signal()
}

CudaWindow::~CudaWindow() {
  if (registered_) {
    B200C_LOG(WARN, "window", "window destroyed while a tensor is still registered");
  }
}

void CudaWindow::tensor_register(const at::Tensor& t, bool owning) {
  TORCH_CHECK(!registered_, "window: a tensor is already registered");
  check_tensor(t, owner_->device(), "window.tensor_register");
  (void)owning;
  tensor_ = t;  // keeps the storage alive for the lifetime of the registration
  cache_meta(t);
  data_seg_ = owner_->symm().attach_user_buffer(t.data_ptr(), t.nbytes());
  registered_ = true;
  // Registration is the collective moment: the signal / barrier segment and the
  // device-side descriptor are made here, with the default counts, so that the
  // one-sided calls (put, signal, wait_signal) never have to allocate - a rank
  // that takes no part in an exchange is not needed for it.
  build_device_window(-1, -1, 1);
}

void CudaWindow::tensor_deregister() {
  TORCH_CHECK(registered_, "window: no tensor is registered");
  c10::cuda::CUDAGuard guard(owner_->device());
  bool capturing = false;
  unsigned long long gid = 0;
  owner_->cuda_api()->streamIsCapturing(at::cuda::getCurrentCUDAStream(owner_->device().index()).stream(), &capturing, &gid);
  if (capturing) {
    return;  // a captured region cannot change mappings
  }
  // Nobody may still be storing into this rank's buffer.
  owner_->barrier(false, {})->wait_blocking();
  cudaDeviceSynchronize();
  if (dev_window_) {
    cudaFree(dev_window_);
    dev_window_ = nullptr;
  }
  if (local_state_) {
    cudaFree(local_state_);
    local_state_ = nullptr;
  }
  if (ctrl_seg_) {
    owner_->symm().release(ctrl_seg_);
    ctrl_seg_.reset();
  }
  owner_->symm().release(data_seg_);
  data_seg_.reset();
  for (auto& lb : local_buffers_) cudaFree(lb.first);
  local_buffers_.clear();
  tensor_.reset();
  registered_ = false;
  custom_counts_ = false;
  owner_->barrier(false, {})->wait_blocking();
}

std::shared_ptr<Window> CudaWindow::clone() {
  auto w = std::make_shared<CudaWindow>(owner_);
  if (registered_ && tensor_) {
    // Memory from the same allocator class as the original where possible.
    at::Tensor copy = tensor_->clone();
    w->tensor_register(copy, true);
  }
  return w;
}

void CudaWindow::build_device_window(int signal_count, int counter_count, int barrier_count) {
  TORCH_CHECK(registered_, "window: register a tensor first");
  const int n = owner_->size();
  if (signal_count < 0) signal_count = n;
  if (counter_count < 0) counter_count = n;
  if (barrier_count < 1) barrier_count = 1;
  signal_count += 1;  // slot 0 belongs to the host API
  c10::cuda::CUDAGuard guard(owner_->device());
  const size_t sig_bytes = static_cast<size_t>(signal_count) * n * sizeof(uint64_t);
  const size_t bar_bytes = static_cast<size_t>(barrier_count) * n * sizeof(uint64_t);
  ctrl_seg_ = owner_->symm().allocate(sig_bytes + bar_bytes, false);
  const size_t local_words = static_cast<size_t>(counter_count) + barrier_count + n;
  B200C_CUDA_CHECK(cudaMalloc(&local_state_, local_words * sizeof(uint64_t)));
  B200C_CUDA_CHECK(cudaMemset(local_state_, 0, local_words * sizeof(uint64_t)));
  DeviceWindow w{};
  w.rank = owner_->rank();
  w.nranks = n;
  w.bytes = data_seg_->bytes;
  for (int p = 0; p < n; ++p) {
    w.data[p] = data_seg_->peer_ptrs[p];
    w.signals[p] = reinterpret_cast<uint64_t*>(ctrl_seg_->peer_ptrs[p]);
    w.barrier_flags[p] = reinterpret_cast<uint64_t*>(ctrl_seg_->peer_ptrs[p] + sig_bytes);
  }
  w.mc_data = data_seg_->mc_ptr;
  w.signal_count = signal_count;
  w.counter_count = counter_count;
  w.barrier_count = barrier_count;
  w.counters = local_state_;
  w.barrier_epochs = local_state_ + counter_count;
  w.status = owner_->comm_dev().status;
  w.timeout_ns = owner_->comm_dev().timeout_ns;
  host_copy_ = w;
  B200C_CUDA_CHECK(cudaMalloc(&dev_window_, sizeof(DeviceWindow)));
  B200C_CUDA_CHECK(cudaMemcpy(dev_window_, &w, sizeof(DeviceWindow), cudaMemcpyHostToDevice));
}

// With the default counts this returns the descriptor made at registration
// and is not collective. Asking for other counts rebuilds the control segment:
// that IS collective (every rank must make the same call), and is only
// possible while nothing is in flight on the window.
uintptr_t CudaWindow::get_device_window(int signal_count, int counter_count, int barrier_count) {
  TORCH_CHECK(registered_ && dev_window_ != nullptr, "window: register a tensor first");
  const int n = owner_->size();
  const int want_sig = (signal_count < 0 ? n : signal_count) + 1;
  const int want_cnt = counter_count < 0 ? n : counter_count;
  const int want_bar = barrier_count < 1 ? 1 : barrier_count;
  if (want_sig == host_copy_.signal_count && want_cnt == host_copy_.counter_count && want_bar == host_copy_.barrier_count) {
    return reinterpret_cast<uintptr_t>(dev_window_);
  }
  TORCH_CHECK(!custom_counts_, "window: the device window was already built with signal_count=",
              host_copy_.signal_count - 1, ", counter_count=", host_copy_.counter_count, ", barrier_count=",
              host_copy_.barrier_count, "; different counts need a new registration");
  c10::cuda::CUDAGuard guard(owner_->device());
  owner_->barrier(false, {})->wait_blocking();
  cudaDeviceSynchronize();
  cudaFree(dev_window_);
  cudaFree(local_state_);
  dev_window_ = nullptr;
  local_state_ = nullptr;
  owner_->symm().release(ctrl_seg_);
  ctrl_seg_.reset();
  build_device_window(signal_count, counter_count, barrier_count);
  custom_counts_ = true;
  return reinterpret_cast<uintptr_t>(dev_window_);
}

WorkPtr CudaWindow::put(const at::Tensor& src, int dst_rank, int64_t target_offset_nelems, bool async_op, const OpOptions& o) {
  TORCH_CHECK(registered_, "window.put: no tensor is registered");
  check_tensor(src, owner_->device(), "window.put");
  TORCH_CHECK(dst_rank >= 0 && dst_rank < owner_->size(), "window.put: bad destination rank ", dst_rank);
  TORCH_CHECK(target_offset_nelems >= 0, "window.put: negative offset");
  const size_t esz = c10::elementSize(dtype_);
  TORCH_CHECK((static_cast<size_t>(target_offset_nelems) + src.numel()) * esz <= static_cast<size_t>(get_size()),
              "window.put: ", src.numel(), " elements at offset ", target_offset_nelems, " do not fit the window");
  at::Tensor s = src;
  const size_t off = static_cast<size_t>(target_offset_nelems) * esz;
  DeviceWindow* dw = dev_window_;
  return owner_->run("window_put/kernel", async_op, o, {src}, [dw, s, dst_rank, off](cudaStream_t st) {
    B200C_CUDA_CHECK(launch_window_put(dw, s.data_ptr(), s.nbytes(), dst_rank, off, st));
  });
}

WorkPtr CudaWindow::signal(int dst_rank, bool async_op, const OpOptions& o) {
  TORCH_CHECK(registered_, "window.signal: no tensor is registered");
  TORCH_CHECK(dst_rank >= 0 && dst_rank < owner_->size(), "window.signal: bad rank ", dst_rank);
  DeviceWindow* dw = dev_window_;
  return owner_->run("window_signal/kernel", async_op, o, {}, [dw, dst_rank](cudaStream_t st) {
    B200C_CUDA_CHECK(launch_window_signal(dw, dst_rank, kHostSignalId, st));
  });
}

WorkPtr CudaWindow::wait_signal(int peer_rank, bool async_op, const OpOptions& o) {
  TORCH_CHECK(registered_, "window.wait_signal: no tensor is registered");
  TORCH_CHECK(peer_rank >= 0 && peer_rank < owner_->size(), "window.wait_signal: bad rank ", peer_rank);
  DeviceWindow* dw = dev_window_;
  uint64_t* expected = local_state_ + host_copy_.counter_count + host_copy_.barrier_count;
  return owner_->run("window_wait/kernel", async_op, o, {}, [dw, peer_rank, expected](cudaStream_t st) {
    B200C_CUDA_CHECK(launch_window_wait_signal(dw, peer_rank, kHostSignalId, expected, st));
  });
}

at::Tensor CudaWindow::map_remote_tensor(int rank) {
  TORCH_CHECK(registered_, "window.map_remote_tensor: no tensor is registered");
  TORCH_CHECK(rank >= 0 && rank < owner_->size(), "window.map_remote_tensor: bad rank ", rank);
  if (rank == owner_->rank()) {
    return *tensor_;
  }
  auto keep = data_seg_;
  // The memory physically lives on the peer's GPU but is addressable from
  // this device: name this device as the tensor's, without the ownership check.
  return at::for_blob(data_seg_->peer_ptrs[rank], shape_)
      .options(at::TensorOptions().dtype(dtype_).device(device_))
      .target_device(device_)
      .deleter([keep](void*) {})
      .make_tensor();
}

WindowAttr CudaWindow::get_attr(int peer_rank) {
  TORCH_CHECK(peer_rank >= 0 && peer_rank < owner_->size(), "window.get_attr: bad rank ", peer_rank);
  WindowAttr a;
  a.access_type = WinAccessType::UNIFIED;  // every peer is reachable with loads and stores
  return a;
}

uintptr_t CudaWindow::register_local_buffer(const at::Tensor& t) {
  TORCH_CHECK(dev_window_ != nullptr, "register_local_buffer: call get_device_window() first");
  check_tensor(t, owner_->device(), "register_local_buffer");
  RegisteredBuffer host{static_cast<char*>(t.data_ptr()), static_cast<size_t>(t.nbytes())};
  RegisteredBuffer* dev = nullptr;
  B200C_CUDA_CHECK(cudaMalloc(&dev, sizeof(RegisteredBuffer)));
  B200C_CUDA_CHECK(cudaMemcpy(dev, &host, sizeof(host), cudaMemcpyHostToDevice));
  local_buffers_.emplace_back(dev, t);
  return reinterpret_cast<uintptr_t>(dev);
}

void CudaWindow::deregister_local_buffer(uintptr_t handle) {
  for (auto it = local_buffers_.begin(); it != local_buffers_.end(); ++it) {
    if (reinterpret_cast<uintptr_t>(it->first) == handle) {
      cudaFree(it->first);
      local_buffers_.erase(it);
      return;
    }
  }
  TORCH_CHECK(false, "deregister_local_buffer: unknown handle");
}

void register_cuda_backends() {
  for (const char* name : {"b200", "nccl", "ncclx"}) {
    const std::string n = name;
    Factory::get().register_backend(n, [n] { return std::make_shared<CudaBackend>(n); });
  }
}

} // namespace b200c
