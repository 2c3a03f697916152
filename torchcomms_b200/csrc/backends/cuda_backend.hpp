// The CUDA backend ("b200"; also answers to "nccl" and "ncclx").
//
// One process per GPU inside one NVLink/NVSwitch domain. Collectives run as
// peer-memory kernels over a symmetric heap (see kernels/collectives.cu); NCCL
// carries point-to-point traffic and whatever the kernels do not cover.
//
// Stream rules: a synchronous operation is enqueued on the caller's current
// stream; an asynchronous one on the communicator's internal stream after an
// event dependency on the current stream. `work.wait()` never blocks the
// host: it makes the current stream wait for the operation's end event.
// Operations are grouped into channels. A channel owns flag sets and staging
// that its kernels share, so operations of one channel are kept in issue order
// even across streams; operations of different channels (for instance a
// parameter all-gather and a gradient reduce-scatter on symmetric buffers) have
// nothing in common, run on streams of their own when asynchronous, and may
// overlap.
//
// A watchdog thread polls the end events (cudaEventQuery only), the device
// status word written by bounded waits, and NCCL's asynchronous error state.
// A failure marks the process unhealthy, runs abort hooks, and either aborts
// the process or makes the next call raise, as configured.
//
// Parity: comms/torchcomms/ncclx/TorchCommNCCLX.hpp:86-561 (backend),
// TorchCommNCCLXUtils.cpp:202-343 (watchdog), :456-478 (stream choice),
// TorchWorkNCCLX.cpp:160-308 (events, wait), TorchCommNCCLXBootstrap.cpp:42-390
// (bootstrap over a c10d store), GraphEventTracker.hpp:26-195 (graph replay
// monitoring), TorchCommWindowNCCLX.hpp:59-246 (window).
#pragma once

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <thread>

#include "../core/comm.hpp"
#include "../cuda/driver_api.hpp"
#include "../cuda/nccl_api.hpp"
#include "../kernels/collectives.h"
#include "../kernels/window.h"
#include "../mem/symm_memory.hpp"

namespace b200c {

class CudaBackend;

// Asynchronous handle of a stream-ordered operation.
class CudaWork final : public Work {
 public:
  // `start` / `end` may be null for a synchronous operation of the library's
  // own kernels that nobody observes: stream order already gives wait() its
  // meaning, and `stream` is what wait_blocking() synchronises with.
  CudaWork(std::shared_ptr<CudaApi> api, cudaEvent_t start, cudaEvent_t end, bool pooled, int device,
           Millis timeout, std::vector<at::Tensor> keep_alive, std::weak_ptr<CudaBackend> owner, bool in_capture,
           cudaStream_t stream = nullptr);
  ~CudaWork() override;

  // Called by the watchdog: advances NOT_STARTED -> INPROGRESS -> COMPLETED /
  // TIMEDOUT from event queries. Returns true once the work is terminal.
  bool poll(std::chrono::steady_clock::time_point now);
  cudaEvent_t end_event() const { return end_; }
  cudaEvent_t start_event() const { return start_; }
  bool pooled() const { return pooled_; }
  void release_events(cudaEvent_t* start, cudaEvent_t* end);

 protected:
  void do_wait() override;
  void do_wait_blocking() override;

 private:
  std::shared_ptr<CudaApi> api_;
  cudaEvent_t start_, end_;
  bool pooled_;
  int device_;
  std::vector<at::Tensor> keep_alive_;
  std::weak_ptr<CudaBackend> owner_;
  bool in_capture_;
  cudaStream_t stream_ = nullptr;
  std::mutex poll_mu_;
  bool started_seen_ = false;
  std::chrono::steady_clock::time_point started_at_{};
};

// Which kernel family serves an operation.
enum class Algo : int { AUTO = 0, ONESHOT = 1, TWOSHOT = 2, STAGED = 3, NCCL = 4, KERNEL = 5 };

// Collective families that have both a peer-memory kernel and an NCCL route.
enum class Coll : int { ALL_REDUCE, ALL_GATHER, REDUCE_SCATTER, ALL_TO_ALL };

// Operations that share flags and staging. kChanMain: the staged kernels, NCCL
// and everything else; the others: one-pass kernels on symmetric buffers.
enum Chan : int { kChanMain = 0, kChanSymAg = 1, kChanSymRs = 2, kChanSymAr = 3, kChanCount = 4 };

struct Tuning {
  size_t staging_bytes = 128ull << 20;     // bulk staging per rank
  size_t oneshot_max_bytes = 512 * 1024;   // all-reduce: one-shot up to here
  size_t ag_oneshot_max_bytes = 512 * 1024;  // all-gather: one-shot up to this many bytes per rank
  size_t rs_oneshot_max_bytes = 64 * 1024;   // reduce-scatter: one-shot up to this many output bytes per rank
  int ag_push_min_ranks = 4;               // all-gather: multicast push from this many ranks on
  int a2av_blocks = 96;                    // grid of all-to-all-v (must not depend on rank-local sizes)
  int max_blocks = 444;                    // bulk kernels: 148 SMs x 3 resident blocks
  int threads = 256;
  size_t max_chunk_bytes = 256u << 10;     // bytes staged per block per step
  int steps_per_block = 8;                 // large payloads: steps each block should run
  size_t min_chunk_bytes = 64 * 1024;
  bool auto_nccl = false;                  // opt-in: algo=auto may pick NCCL where it measured faster
  std::string tuner_file;                  // opt-in: per-operation size ranges -> kernel / nccl, written by utils/tuning.py
  int symm_blocks = 32;                    // grid of the one-pass kernels on symmetric buffers (same on every rank)
  int symm_blocks_nomc = 64;               // same, when the data path is plain peer stores
  int symm_blocks_ld = 128;                // same, for plain peer loads: an SM keeps only so many remote reads in flight,
                                           // so read bandwidth grows with the number of SMs that read
  // Data path of the one-pass kernels: 1 = through the switch's multicast
  // object (multimem.st / multimem.ld_reduce), 0 = plain peer stores / loads,
  // -1 = by rank count. Multicast needs 1/nranks of the store or load
  // instructions, but the switch also delivers a rank's own copy back to it:
  // nranks/(nranks-1) times the bytes of the peer path for all-gather and
  // reduce-scatter, while for all-reduce it moves (1 + 1/nranks) S against
  // 2 (nranks-1)/nranks S and wins from 4 ranks on. By rank count: all-gather
  // uses peer stores (they stream at link rate from few SMs); reduce-scatter
  // uses peer loads (fastest, but they need most of the SMs to reach link
  // rate: callers that overlap it with compute ask for the switch path and a
  // small grid by hint); all-reduce uses the switch from 4 ranks on.
  int symm_ag_mc = -1;
  int symm_rs_mc = -1;
  int symm_ar_mc = -1;
  size_t lamport_max_bytes = 1024 * 1024;  // flag-less kernels up to this many bytes per message / per-rank part (0 = off)
  bool channel_streams = true;             // asynchronous operations of different channels get streams of their own
  bool fast_sync = true;                   // unobserved synchronous kernel operations skip the event pair
  int colltrace = 0;                       // > 0: GPU-written start / end timestamps of the last N operations
  bool use_multicast = true;
  bool use_nccl = true;                    // create the NCCL communicator at init
  Algo force = Algo::AUTO;                 // B200COMMS_ALGO / hint "algo"
  unsigned long long device_wait_ns = 10ull * 1000 * 1000 * 1000;  // budget of one device-side wait
  int watchdog_interval_ms = 100;
  bool graph_timeout_monitoring = true;   // watchdog fails a captured collective that stays open past its timeout during replay
  size_t max_event_pool = 1000;
};

class CudaWindow;

class CudaBackend final : public Backend {
 public:
  CudaBackend(std::string registered_as = "b200");
  ~CudaBackend() override;

  void init(at::Device device, const std::string& name, const CommOptions& opts) override;
  void finalize() override;
  int rank() const override { return rank_; }
  int size() const override { return size_; }
  std::string backend_name() const override { return registered_as_; }
  std::string backend_version() const override;
  std::string comm_name() const override { return name_; }
  at::Device device() const override { return device_; }
  const CommOptions& options() const override { return opts_; }

  WorkPtr send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o) override;
  WorkPtr recv(at::Tensor& t, int src, bool async_op, const OpOptions& o) override;
  WorkPtr batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o) override;
  WorkPtr broadcast(at::Tensor& t, int root, bool async_op, const OpOptions& o) override;
  WorkPtr all_reduce(at::Tensor& t, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr reduce(const at::Tensor& t, int root, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr all_gather_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr all_to_all_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr all_to_all_v_single(at::Tensor& out, const at::Tensor& in, const std::vector<int64_t>& out_splits,
                              const std::vector<int64_t>& in_splits, bool async_op, const OpOptions& o) override;
  WorkPtr all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool async_op, const OpOptions& o) override;
  WorkPtr barrier(bool async_op, const OpOptions& o) override;
  WorkPtr scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool async_op, const OpOptions& o) override;
  WorkPtr gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool async_op, const OpOptions& o) override;
  std::shared_ptr<Backend> split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) override;
  std::shared_ptr<Window> new_window(const std::optional<at::Tensor>& tensor) override;

  void set_timeout(Millis t) override { opts_.timeout = t; }
  void set_hints(const Hints& h) override;
  void abort() override;
  bool supports_reconfigure() const override { return true; }
  InitHandle get_init_handle() const override;
  WorkPtr reconfigure(const ReconfigureOptions& o) override;
  bool is_aborted() const override { return aborted_.load(); }
  bool is_abort_supported() const override { return true; }

  // Symmetric tensors: memory every rank has mapped (and, where the box
  // allows, bound to an NVLS multicast object). Collectives whose tensors live
  // there run as one-pass kernels without staging. Both calls are collective:
  // every rank calls them in the same order with the same sizes. The memory
  // stays mapped until symm_free() or finalize(); a tensor must not be used
  // after that.
  at::Tensor symm_empty(const std::vector<int64_t>& sizes, at::ScalarType dtype);
  void symm_free(const at::Tensor& t);
  // Collective: makes the allocation behind `t` (memory from this
  // communicator's allocator, see mem_allocator) reachable by every rank, so
  // that collectives on tensors inside it take the one-pass kernels.
  void tensor_register(const at::Tensor& t) override;
  void tensor_deregister(const at::Tensor& t) override;
  // Peer views of [p, p + bytes) if it lies inside a symmetric tensor or a
  // registered allocation.
  // `region_bytes` (optional): size the registration was made with, the same on every rank.
  bool lookup_symm(const void* p, size_t bytes, SymmView* view, size_t* region_bytes = nullptr) const;

  // Backend-specific operations (reached through get_backend_impl()).
  // Split sizes live on the device (int64 counts of dim-0 slices).
  WorkPtr device_alltoallv_single(at::Tensor& out, const at::Tensor& in, const at::Tensor& out_splits,
                                  const at::Tensor& in_splits, bool async_op, const OpOptions& o);
  // fp32 in / fp32 out, bf16 on the wire; optional stochastic rounding seed.
  WorkPtr reduce_scatter_quantized(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, int64_t seed,
                                   bool async_op, const OpOptions& o);
  // Checkpoint support. suspend(): collective; waits for this rank's work, meets the other members and gives back
  // everything the bootstrap created (peer mappings, multicast bindings, the NCCL communicator, streams, events,
  // the watchdog), so that the process holds no cross-process GPU state and can be checkpointed (CUDA checkpoint,
  // CRIU) or moved. Rank, size, name, options and hooks are kept. resume(): collective; bootstraps again among the
  // same members under a fresh store prefix. Objects that hold symmetric memory of the communicator (symm_empty
  // tensors, windows, fused layers) must be recreated after resume(), as after reconfigure().
  void suspend();
  void resume();
  bool is_suspended() const { return suspended_; }
  // Sequence <-> heads exchange of sequence-parallel attention with both layout changes folded in.
  // to_heads: in [b, h, s, d] -> out [b, h / size, size * s, d]; otherwise the inverse. Both contiguous;
  // `out` must be a symmetric tensor (symm_empty) of the same shape on every rank.
  WorkPtr seq_heads_exchange(at::Tensor& out, const at::Tensor& in, bool to_heads, bool async_op, const OpOptions& o);
  std::unordered_map<std::string, std::string> comm_dump() const override;
  // The timestamp ring (hint / variable `colltrace` = number of entries): for each of the last N operations that
  // were issued outside a graph capture, its sequence number, route name, and the device's nanosecond timer when
  // the stream reached the operation and when it left it (0 = not reached yet). Written by the GPU into mapped
  // host memory, read here without touching the GPU.
  struct CollTraceEntry {
    uint64_t seq;
    std::string op;
    unsigned long long start_ns, end_ns;
  };
  std::vector<CollTraceEntry> colltrace_dump() const;
  void set_config(const Hints& h) { set_hints(h); }
  uintptr_t get_nccl_comm_ptr() const { return reinterpret_cast<uintptr_t>(nccl_comm_); }
  // Kernel phase trace (performance work): kMaxBlocks x kTraceSlots int64
  // cycle stamps, rewritten by every traced kernel. An undefined tensor
  // switches tracing off.
  void set_trace_buffer(const at::Tensor& t) {
    trace_ = t;
    dev_.trace = t.defined() ? reinterpret_cast<long long*>(t.data_ptr<int64_t>()) : nullptr;
  }

  // Shared with windows and fused ops.
  WorkPtr exchange_nccl(const char* what, const at::Tensor& in, at::Tensor& out,
                        const std::vector<std::pair<size_t, size_t>>& send,
                        const std::vector<std::pair<size_t, size_t>>& recv, bool async_op, const OpOptions& o);
  LaunchShape shape_for(size_t bytes, size_t slot_multiplier, int block_cap = 0) const;
  // Multicast or peer path for one call of a one-pass kernel (`knob`: the Tuning field of its kind).
  bool symm_use_mc(int knob, bool mc_by_default, const SymmView& v, const OpOptions& o) const;
  int symm_blocks_for(bool mc, size_t vectors, const OpOptions& o, bool peer_loads = false) const;
  // Resolves algo=auto for one call: own kernels (AUTO) or NCCL, from measured cross-over sizes.
  Algo route(Coll c, size_t bytes, const OpOptions& o) const;
  std::shared_ptr<Backend> create_pair_comm(int peer, const std::string& name) override;
  const CommDev& comm_dev() const { return dev_; }
  const HeapLayout& layout() const { return layout_; }
  const Tuning& tuning() const { return tune_; }
  SymmMemory& symm() { return *symm_; }
  bool symm_alive() const { return symm_ != nullptr && !finalized_; }
  std::shared_ptr<CudaApi> cuda_api() const { return cuda_; }
  cudaStream_t internal_stream() const { return internal_stream_; }
  cudaStream_t channel_stream(int chan) const { return chans_[chan].stream; }

  // Runs `launch(stream)` with the backend's stream / event / watchdog
  // protocol and returns the work. `keep_alive` tensors are held until wait()
  // for asynchronous operations. `chan` names the channel whose order the
  // operation joins; `own_kernel` says that everything launched is one of the
  // library's kernels with bounded waits (failures then show in the status
  // word, and an unobserved synchronous call needs no events).
  // `sm_blocks` > 0: the operation is a kernel of that many one-block-per-SM blocks whose blocks wait for their
  // peers' blocks. Kernels of different channels that could hold more SMs together than the GPU has are chained
  // (see kSmBudget in run()), so that they can never starve each other's peers of SMs.
  WorkPtr run(const char* what, bool async_op, const OpOptions& o, std::vector<at::Tensor> keep_alive,
              const std::function<void(cudaStream_t)>& launch, int chan = kChanMain, bool own_kernel = false,
              int sm_blocks = 0);

  // Fields of ncclConfig_t named by hints (what ncclCommInitRankConfig is given).
  static NcclConfig nccl_config_from_hints(const Hints& h, const std::string& comm_name);

  // Test seams.
  void set_cuda_api(std::shared_ptr<CudaApi> api) { cuda_ = std::move(api); }
  void set_nccl_api(std::shared_ptr<NcclApi> api) { nccl_ = std::move(api); }

  // Called from the CUDA user-object callback of a destroyed graph.
  void note_graph_released(unsigned long long graph_id);
  // Called by works / watchdog on failures.
  void on_failure(const std::string& what, bool timed_out);
  // Returns a finished work's events to the pool.
  void recycle_events(cudaEvent_t a, cudaEvent_t b) { give_events(a, b); }

 private:
  friend class CudaWindow;
  void check_usable() const;
  void parse_tuning(const Hints& h);
  void bootstrap(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size);
  void init_nccl();
  void start_watchdog();
  void stop_watchdog();
  void watchdog_loop();
  Millis effective_timeout(const OpOptions& o) const { return o.timeout_set ? o.timeout : opts_.timeout; }
  Algo algo_override(const OpOptions& o) const;
  bool kernels_can_reduce(at::ScalarType t, const ReduceOp& op) const;
  std::pair<cudaEvent_t, cudaEvent_t> take_events();
  void give_events(cudaEvent_t a, cudaEvent_t b);
  void nccl_check(NcclResult r, const char* what) const;

  std::string registered_as_;
  int rank_ = -1, size_ = -1;
  std::string name_;
  at::Device device_{at::kCUDA, 0};
  CommOptions opts_;
  Tuning tune_;
  c10::intrusive_ptr<c10d::Store> store_;
  std::shared_ptr<DriverApi> drv_;
  std::shared_ptr<CudaApi> cuda_;
  std::shared_ptr<NcclApi> nccl_;
  NcclComm* nccl_comm_ = nullptr;
  std::unique_ptr<SymmMemory> symm_;
  std::shared_ptr<SymmSegment> heap_;
  HeapLayout layout_;
  CommDev dev_{};
  uint32_t* epochs_dev_ = nullptr;
  uint32_t* status_host_ = nullptr;   // mapped pinned
  uint32_t* status_dev_ = nullptr;    // device alias of status_host_
  cudaStream_t internal_stream_ = nullptr;   // == chans_[kChanMain].stream
  cudaEvent_t dep_event_ = nullptr;
  // Per channel: the stream asynchronous operations run on, and the latest
  // operation (its end event, or just its stream when it recorded none) that
  // the next operation of the channel must follow.
  struct ChanState {
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    cudaStream_t last_stream = nullptr;
    c10::intrusive_ptr<CudaWork> last_work;   // null when the last operation recorded no events
    cudaEvent_t order_event = nullptr;        // recorded on last_stream when an event-less operation must be followed
    int sm_blocks = 0;                        // SMs the channel's latest peer-waiting kernel may hold
  };
  ChanState chans_[kChanCount];
  // Inside a stream capture: last captured operation per graph, so that
  // captured operations stay chained across streams too.
  struct CaptureTail {
    cudaEvent_t end = nullptr;
    cudaStream_t stream = nullptr;
  };
  std::unordered_map<unsigned long long, CaptureTail> capture_tail_;
  void sync_own_streams();

  // Symmetric tensors and registered allocations, keyed by local base address.
  struct SymmReg {
    size_t bytes = 0;
    std::shared_ptr<SymmSegment> seg;
    bool user_memory = false;   // registered allocation (not freed by symm_free)
    size_t user_bytes = 0;      // size the caller asked for / registered: the same on every rank
  };
  mutable std::mutex symm_mu_;
  std::map<uintptr_t, SymmReg> symm_regs_;
  uint64_t symm_free_seq_ = 0;

  std::mutex pool_mu_;
  std::vector<cudaEvent_t> event_pool_;

  std::thread watchdog_;
  std::mutex wd_mu_;
  std::condition_variable wd_cv_;
  std::deque<c10::intrusive_ptr<CudaWork>> inflight_;
  bool wd_stop_ = false;

  // Graph replay monitoring: two counters in mapped pinned memory per
  // captured collective (started / ended), bumped by one-thread kernels.
  struct GraphEntry {
    unsigned long long graph_id;
    size_t index;
    size_t slot;                        // counter pair of the pinned pool
    unsigned long long* counters_host;  // [2]
    unsigned long long* counters_dev;
    unsigned long long seen_start = 0, seen_end = 0;
    std::chrono::steady_clock::time_point open_since{};
    uintptr_t stream;
    Millis timeout;
  };
  // Timestamp ring: two mapped words per entry, and what each entry describes.
  unsigned long long* trace_ring_host_ = nullptr;
  unsigned long long* trace_ring_dev_ = nullptr;
  std::vector<std::pair<uint64_t, std::string>> trace_meta_;
  uint64_t trace_next_ = 0;
  // Stamps the ring before (`end` = false) or after the launch; returns the slot, or -1 when tracing is off.
  int64_t colltrace_begin(const char* what, cudaStream_t stream);
  void colltrace_end(int64_t slot, cudaStream_t stream);
  // Route table of the tuner file: for each operation, (largest message size, algorithm) in ascending order.
  struct TunerRule {
    size_t up_to;
    Algo algo;
  };
  std::vector<TunerRule> tuner_rules_[4];
  void load_tuner_file(const std::string& path);
  static constexpr size_t kMaxGraphEntries = 2048;
  unsigned long long* replay_pool_host_ = nullptr;  // 2 x kMaxGraphEntries counters, mapped pinned
  unsigned long long* replay_pool_dev_ = nullptr;
  std::vector<GraphEntry> graph_entries_;
  // Per captured graph: the events its operations recorded (destroyed with the
  // bookkeeping), the next collective index, and whether the destroy callback
  // rides on the graph. A CUDA user object retained by the graph calls back
  // when the graph and all its executables are gone; the watchdog then drops
  // the graph's entries and returns their counter slots.
  // Parity: comms/torchcomms/ncclx/GraphEventTracker.cpp:99-121,237.
  struct GraphState {
    std::vector<cudaEvent_t> events;
    size_t next_index = 0;
    bool retained = false;
  };
  std::unordered_map<unsigned long long, GraphState> graphs_;
  std::vector<size_t> free_slots_;
  size_t next_slot_ = 0;
  std::mutex released_mu_;
  std::vector<unsigned long long> released_ids_;
  void drop_released_graphs();   // watchdog thread, wd_mu_ held

  at::Tensor trace_;
  std::atomic<bool> aborted_{false};
  std::atomic<bool> failed_{false};
  std::string failure_text_;
  bool finalized_ = false;
  bool initialized_ = false;
  bool suspended_ = false;
  int suspend_gen_ = 0;
  c10::intrusive_ptr<c10d::Store> resume_store_;   // the store of the bootstrap that suspend() took down
  uint64_t split_counter_ = 0;
  std::atomic<uint64_t> ops_issued_{0}, bytes_issued_{0};
  std::unordered_map<std::string, uint64_t> algo_counts_;
  std::string handle_token_;
  void drain_and_release(bool broken, const char* why);
};

class CudaWindow final : public Window {
 public:
  explicit CudaWindow(std::shared_ptr<CudaBackend> owner) : owner_(std::move(owner)) {}
  ~CudaWindow() override;
  void tensor_register(const at::Tensor& t, bool owning) override;
  void tensor_deregister() override;
  std::shared_ptr<Window> clone() override;
  WorkPtr put(const at::Tensor& src, int dst_rank, int64_t target_offset_nelems, bool async_op, const OpOptions& o) override;
  WorkPtr signal(int dst_rank, bool async_op, const OpOptions& o) override;
  WorkPtr wait_signal(int peer_rank, bool async_op, const OpOptions& o) override;
  at::Tensor map_remote_tensor(int rank) override;
  WindowAttr get_attr(int peer_rank) override;
  uintptr_t get_device_window(int signal_count, int counter_count, int barrier_count) override;
  uintptr_t register_local_buffer(const at::Tensor& t) override;
  void deregister_local_buffer(uintptr_t handle) override;

 private:
  void build_device_window(int signal_count, int counter_count, int barrier_count);
  std::shared_ptr<CudaBackend> owner_;
  std::shared_ptr<SymmSegment> data_seg_;
  std::shared_ptr<SymmSegment> ctrl_seg_;   // signals + barrier flags
  DeviceWindow host_copy_{};
  DeviceWindow* dev_window_ = nullptr;
  uint64_t* local_state_ = nullptr;         // counters, barrier epochs, wait expectations
  std::vector<std::pair<RegisteredBuffer*, at::Tensor>> local_buffers_;
  bool registered_ = false;
  bool custom_counts_ = false;   // the device window was rebuilt with explicit counts
};

void register_cuda_backends();
void register_lazy_backends();
int lazy_pair_count(const std::shared_ptr<Backend>& b);
std::shared_ptr<Backend> lazy_primary(const std::shared_ptr<Backend>& b);

} // namespace b200c
