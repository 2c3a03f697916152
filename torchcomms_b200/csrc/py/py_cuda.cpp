// Python bindings of the CUDA backend's extra operations and of a
// single-GPU emulation world used by kernel tests.
//
// Parity: comms/torchcomms/ncclx/TorchCommNCCLXPy.cpp:22-204 (device_alltoallv_single,
// reduce_scatter_quantized, comm_dump, set_config, get_nccl_comm_ptr).
#include "py_common.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "../backends/cuda_backend.hpp"

namespace b200c {

namespace {

using OptHints = std::optional<Hints>;
using OptMillis = std::optional<Millis>;

// N virtual ranks on one GPU: N private "heaps", one CommDev per rank whose
// peer table points at all of them. Kernels run through the emulation launch
// path (one cooperative launch, blockIdx.y = rank), which executes the same
// device code as a real multi-GPU launch.
class EmuWorld {
 public:
  EmuWorld(int nranks, size_t staging_bytes, double wait_ms) : n_(nranks) {
    TORCH_CHECK(nranks >= 1 && nranks <= kMaxRanks, "emulation supports 1..", kMaxRanks, " ranks");
    lay_.bulk_off = 0;
    lay_.bulk_bytes = (staging_bytes + 4095) / 4096 * 4096;
    lay_.small_off = lay_.bulk_bytes;
    const size_t meta = static_cast<size_t>(kMaxBlocks) * kMaxRanks * kMaxRanks * sizeof(uint64_t);
    lay_.small_bytes = (2 * static_cast<size_t>(kSmallBlocks) * kSmallPiece + meta + 4095) / 4096 * 4096;
    lay_.symm_meta_off = lay_.small_off + lay_.small_bytes;
    lay_.symm_meta_bytes = (kSymmMetaBytes + 4095) / 4096 * 4096;
    lay_.lamport_off = lay_.symm_meta_off + lay_.symm_meta_bytes;
    lay_.lamport_bytes = (kLamportBytes + 4095) / 4096 * 4096;
    flags_off_ = lay_.lamport_off + lay_.lamport_bytes;
    const size_t flag_bytes = static_cast<size_t>(kFlagSets) * kMaxBlocks * kMaxRanks * sizeof(uint32_t);
    total_ = flags_off_ + (flag_bytes + 4095) / 4096 * 4096;
    heaps_.resize(n_);
    epochs_.resize(n_);
    for (int r = 0; r < n_; ++r) {
      B200C_CUDA_CHECK(cudaMalloc(&heaps_[r], total_));
      B200C_CUDA_CHECK(cudaMemset(heaps_[r], 0, total_));
      B200C_CUDA_CHECK(launch_lamport_init(static_cast<char*>(heaps_[r]) + lay_.lamport_off, nullptr));
      B200C_CUDA_CHECK(cudaMalloc(&epochs_[r], kFlagSets * kMaxBlocks * sizeof(uint32_t)));
      B200C_CUDA_CHECK(cudaMemset(epochs_[r], 0, kFlagSets * kMaxBlocks * sizeof(uint32_t)));
    }
    B200C_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped));
    std::memset(status_host_, 0, 64);
    B200C_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev_), status_host_, 0));
    comms_.resize(n_);
    for (int r = 0; r < n_; ++r) {
      CommDev& c = comms_[r];
      std::memset(&c, 0, sizeof(c));
      c.rank = r;
      c.nranks = n_;
      for (int p = 0; p < n_; ++p) {
        c.heap[p] = static_cast<char*>(heaps_[p]);
        c.flags[p] = reinterpret_cast<uint32_t*>(static_cast<char*>(heaps_[p]) + flags_off_);
      }
      c.epochs = static_cast<uint32_t*>(epochs_[r]);
      c.status = status_dev_;
      c.timeout_ns = static_cast<unsigned long long>(wait_ms * 1.0e6);
      c.heap_bytes = total_;
    }
    B200C_CUDA_CHECK(cudaDeviceSynchronize());
  }
  ~EmuWorld() {
    for (void* p : heaps_) cudaFree(p);
    for (void* p : arn_stage_) cudaFree(p);
    for (void* p : epochs_) cudaFree(p);
    if (status_host_) cudaFreeHost(status_host_);
  }

  std::vector<uint32_t> status() const {
    return std::vector<uint32_t>(status_host_, status_host_ + 5);
  }
  void clear_status() { std::memset(status_host_, 0, 64); }

  static DType dtype_of(const at::Tensor& t) {
    switch (t.scalar_type()) {
      case at::kFloat: return DType::F32;
      case at::kHalf: return DType::F16;
      case at::kBFloat16: return DType::BF16;
      default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
    }
  }
  void check(const std::vector<at::Tensor>& v) const {
    TORCH_CHECK(static_cast<int>(v.size()) == n_, "need one tensor per virtual rank");
    for (auto& t : v) TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "tensors must be contiguous CUDA tensors");
  }
  static std::vector<size_t> nbytes_of(const std::vector<at::Tensor>& ts) {
    std::vector<size_t> out;
    for (auto& t : ts) out.push_back(t.nbytes());
    return out;
  }
  LaunchShape shape(int blocks, size_t chunk) const {
    LaunchShape s;
    s.blocks = blocks;
    s.threads = 256;
    s.chunk_bytes = chunk;
    return s;
  }
  cudaStream_t stream() const { return at::cuda::getCurrentCUDAStream().stream(); }

  void all_reduce(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, int red, double scale, int algo,
                  int blocks, size_t chunk) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
    }
    B200C_CUDA_CHECK(launch_all_reduce(comms_.data(), lay_, n_, ip.data(), op.data(), ins[0].numel(), dtype_of(ins[0]),
                                       static_cast<RedKind>(red), static_cast<float>(scale), algo, false,
                                       shape(blocks, chunk), stream()));
  }
  // Fused all-reduce + residual add + RMSNorm over the virtual ranks; `residuals` is empty or one per rank.
  void all_reduce_rmsnorm(std::vector<at::Tensor> ins, std::vector<at::Tensor> residuals, at::Tensor weight,
                          std::vector<at::Tensor> outs, double eps) {
    check(ins);
    check(outs);
    TORCH_CHECK(residuals.empty() || static_cast<int>(residuals.size()) == n_, "residuals: none or one per rank");
    TORCH_CHECK(ins[0].dim() == 2 && ins[0].scalar_type() == at::kBFloat16, "bf16 [rows, hidden] expected");
    const int hidden = static_cast<int>(ins[0].size(1));
    if (arn_stage_.empty()) {
      arn_stage_.resize(n_);
      for (int r = 0; r < n_; ++r) {
        B200C_CUDA_CHECK(cudaMalloc(&arn_stage_[r], ar_norm_stage_bytes(kArNormMaxHidden)));
      }
    }
    std::vector<ArNormArgs> args(n_);
    for (int r = 0; r < n_; ++r) {
      ArNormArgs& a = args[r];
      std::memset(&a, 0, sizeof(a));
      a.in = static_cast<const __nv_bfloat16*>(ins[r].data_ptr());
      a.residual = residuals.empty() ? nullptr : static_cast<__nv_bfloat16*>(residuals[r].data_ptr());
      a.weight = static_cast<const __nv_bfloat16*>(weight.data_ptr());
      a.out = static_cast<__nv_bfloat16*>(outs[r].data_ptr());
      for (int p = 0; p < n_; ++p) a.stage[p] = static_cast<char*>(arn_stage_[p]);
      a.rows = static_cast<int>(ins[r].size(0));
      a.hidden = hidden;
      a.eps = static_cast<float>(eps);
    }
    B200C_CUDA_CHECK(launch_all_reduce_rmsnorm(comms_.data(), n_, args.data(), stream()));
  }
  void reduce_scatter(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, const std::string& wire, int red,
                      double scale, int blocks, size_t chunk) {
    reduce_scatter_sr(std::move(ins), std::move(outs), wire, red, scale, blocks, chunk, 0);
  }
  void reduce_scatter_sr(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, const std::string& wire, int red,
                         double scale, int blocks, size_t chunk, uint64_t seed) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
    }
    const DType din = dtype_of(ins[0]), dout = dtype_of(outs[0]);
    const DType dwire = wire == "bf16" ? DType::BF16 : wire == "f16" ? DType::F16 : wire == "f32" ? DType::F32 : din;
    B200C_CUDA_CHECK(launch_reduce_scatter(comms_.data(), lay_, n_, ip.data(), op.data(), outs[0].numel(), din, dwire, dout,
                                           static_cast<RedKind>(red), static_cast<float>(scale), false,
                                           shape(blocks, chunk), stream(), seed));
  }
  void all_gather(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, bool cast, int blocks, size_t chunk) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
    }
    B200C_CUDA_CHECK(launch_all_gather(comms_.data(), lay_, n_, ip.data(), op.data(), ins[0].nbytes(), cast, false,
                                       shape(blocks, chunk), stream()));
  }
  // splits[r][p]: bytes rank r sends to rank p (blocks packed back to back on both sides).
  void all_to_all(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, std::vector<std::vector<int64_t>> splits,
                  int blocks, size_t chunk) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    std::vector<size_t> so(n_ * n_), sl(n_ * n_), ro(n_ * n_), rl(n_ * n_);
    size_t mx = 0;
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
      size_t s = 0, d = 0;
      for (int p = 0; p < n_; ++p) {
        so[r * n_ + p] = s;
        sl[r * n_ + p] = static_cast<size_t>(splits[r][p]);
        s += sl[r * n_ + p];
        ro[r * n_ + p] = d;
        rl[r * n_ + p] = static_cast<size_t>(splits[p][r]);
        d += rl[r * n_ + p];
        mx = std::max(mx, sl[r * n_ + p]);
      }
    }
    B200C_CUDA_CHECK(launch_all_to_all(comms_.data(), lay_, n_, ip.data(), op.data(), so.data(), sl.data(), ro.data(),
                                       rl.data(), mx, shape(blocks, chunk), stream()));
  }
  void all_to_all_device_splits(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs,
                                std::vector<at::Tensor> counts, size_t elem_bytes, int blocks, size_t chunk) {
    check(ins);
    check(outs);
    check(counts);
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    std::vector<const long long*> cp(n_);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
      TORCH_CHECK(counts[r].scalar_type() == at::kLong && counts[r].numel() == n_, "counts: int64[nranks] per rank");
      cp[r] = reinterpret_cast<const long long*>(counts[r].data_ptr<int64_t>());
    }
    B200C_CUDA_CHECK(launch_all_to_all_device_splits(comms_.data(), lay_, n_, ip.data(), op.data(), cp.data(), elem_bytes,
                                                     shape(blocks, chunk), stream(), nbytes_of(ins).data(), nbytes_of(outs).data()));
  }
  void broadcast(std::vector<at::Tensor> bufs, int root, int blocks, size_t chunk) {
    check(bufs);
    std::vector<void*> bp(n_);
    for (int r = 0; r < n_; ++r) bp[r] = bufs[r].data_ptr();
    B200C_CUDA_CHECK(launch_broadcast(comms_.data(), lay_, n_, bp.data(), bufs[0].nbytes(), root, false,
                                      shape(blocks, chunk), stream()));
  }
  // One-pass kernels on "symmetric" buffers: here simply every rank's tensor, all on this GPU.
  std::vector<SymmView> views(const std::vector<at::Tensor>& ts) const {
    SymmView v{};
    for (int p = 0; p < n_; ++p) v.ptr[p] = static_cast<char*>(ts[p].data_ptr());
    v.mc = nullptr;
    return std::vector<SymmView>(n_, v);
  }
  void symm_all_gather(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, bool cast, int blocks) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    for (int r = 0; r < n_; ++r) ip[r] = ins[r].data_ptr();
    auto v = views(outs);
    B200C_CUDA_CHECK(launch_symm_all_gather(comms_.data(), n_, ip.data(), v.data(), ins[0].nbytes(), cast, false, blocks, stream()));
  }
  void symm_reduce_scatter(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, double scale, int blocks) {
    check(ins);
    check(outs);
    std::vector<void*> op(n_);
    for (int r = 0; r < n_; ++r) op[r] = outs[r].data_ptr();
    auto v = views(ins);
    B200C_CUDA_CHECK(launch_symm_reduce_scatter(comms_.data(), n_, v.data(), op.data(), outs[0].numel(), dtype_of(ins[0]),
                                                dtype_of(outs[0]), static_cast<float>(scale), false, blocks, stream()));
  }
  void symm_all_reduce(std::vector<at::Tensor> bufs, double scale, int blocks) {
    check(bufs);
    auto v = views(bufs);
    B200C_CUDA_CHECK(launch_symm_all_reduce(comms_.data(), n_, v.data(), bufs[0].numel(), dtype_of(bufs[0]),
                                            static_cast<float>(scale), false, blocks, stream()));
  }
  // splits[r][p]: bytes rank r sends to rank p, blocks packed back to back on
  // both sides. mode 0: equal splits known to all; 1: host splits, offsets
  // exchanged in the kernel; 2: `counts` (int64 per rank, in units of
  // elem_bytes) are read from device memory.
  void symm_all_to_all(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, std::vector<std::vector<int64_t>> splits,
                       int mode, std::vector<at::Tensor> counts, size_t elem_bytes, int blocks) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    std::vector<const long long*> cp(n_);
    std::vector<size_t> so(n_ * n_, 0), sl(n_ * n_, 0), ro(n_ * n_, 0), rl(n_ * n_, 0);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      if (mode == 2) {
        TORCH_CHECK(counts[r].scalar_type() == at::kLong && counts[r].numel() == n_, "counts: int64[nranks] per rank");
        cp[r] = reinterpret_cast<const long long*>(counts[r].data_ptr<int64_t>());
        continue;
      }
      size_t s = 0, d = 0;
      for (int p = 0; p < n_; ++p) {
        so[r * n_ + p] = s;
        sl[r * n_ + p] = static_cast<size_t>(splits[r][p]);
        s += sl[r * n_ + p];
        ro[r * n_ + p] = d;
        rl[r * n_ + p] = static_cast<size_t>(splits[p][r]);
        d += rl[r * n_ + p];
      }
    }
    auto v = views(outs);
    B200C_CUDA_CHECK(launch_symm_all_to_all(comms_.data(), lay_, n_, ip.data(), v.data(), nbytes_of(ins).data(), nbytes_of(outs).data(),
                                            so.data(), sl.data(), ro.data(), rl.data(), mode == 2 ? cp.data() : nullptr,
                                            elem_bytes, mode != 0, blocks, stream()));
  }
  // ins[r]: [b, h, s, d] (to_heads) or [b, h/n, n*s, d]; outs[r]: the other layout.
  void symm_seq_heads(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, bool to_heads, int blocks) {
    check(ins);
    check(outs);
    const at::Tensor& full = to_heads ? ins[0] : outs[0];   // [b, h, s, d]
    TORCH_CHECK(full.dim() == 4, "symm_seq_heads: [batch, heads, seq, dim] tensors");
    std::vector<const void*> ip(n_);
    for (int r = 0; r < n_; ++r) ip[r] = ins[r].data_ptr();
    auto v = views(outs);
    const size_t slab = static_cast<size_t>(full.size(2)) * full.size(3) * full.element_size();
    B200C_CUDA_CHECK(launch_symm_seq_heads(comms_.data(), n_, ip.data(), v.data(), static_cast<int>(full.size(0)),
                                           static_cast<int>(full.size(1)), slab, to_heads, blocks, stream()));
  }
  void all_reduce_lamport(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, double scale) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
    }
    B200C_CUDA_CHECK(launch_all_reduce_lamport(comms_.data(), lay_, n_, ip.data(), op.data(), ins[0].numel(), dtype_of(ins[0]),
                                               static_cast<float>(scale), false, stream()));
  }
  // mode 0: all-gather, 1: all-to-all with equal parts, 2: reduce-scatter (scaled sum)
  void exchange_lamport(int mode, std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, double scale) {
    check(ins);
    check(outs);
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
    }
    const size_t part = mode == 0 ? ins[0].nbytes() : ins[0].nbytes() / n_;
    B200C_CUDA_CHECK(launch_exchange_lamport(comms_.data(), lay_, n_, mode, ip.data(), op.data(), part, dtype_of(ins[0]),
                                             static_cast<float>(scale), false, stream()));
  }
  // All-to-all with unequal parts: send_bytes[r][p] = bytes rank r sends to rank p (parts packed back to back on
  // both sides, in rank order). `cap_bytes` bounds every part.
  void exchangev_lamport(std::vector<at::Tensor> ins, std::vector<at::Tensor> outs,
                         std::vector<std::vector<int64_t>> send_bytes, int64_t cap_bytes) {
    check(ins);
    check(outs);
    TORCH_CHECK(static_cast<int>(send_bytes.size()) == n_, "one list of part sizes per rank");
    std::vector<const void*> ip(n_);
    std::vector<void*> op(n_);
    std::vector<size_t> so(n_ * kMaxRanks, 0), sl(n_ * kMaxRanks, 0), ro(n_ * kMaxRanks, 0), rl(n_ * kMaxRanks, 0);
    for (int r = 0; r < n_; ++r) {
      ip[r] = ins[r].data_ptr();
      op[r] = outs[r].data_ptr();
      TORCH_CHECK(static_cast<int>(send_bytes[r].size()) == n_, "one part size per peer");
      size_t s_at = 0, r_at = 0;
      for (int p = 0; p < n_; ++p) {
        so[r * kMaxRanks + p] = s_at;
        sl[r * kMaxRanks + p] = static_cast<size_t>(send_bytes[r][p]);
        s_at += sl[r * kMaxRanks + p];
        ro[r * kMaxRanks + p] = r_at;
        rl[r * kMaxRanks + p] = static_cast<size_t>(send_bytes[p][r]);
        r_at += rl[r * kMaxRanks + p];
      }
      TORCH_CHECK(s_at <= ins[r].nbytes() && r_at <= outs[r].nbytes(), "parts exceed the buffers");
    }
    B200C_CUDA_CHECK(launch_exchangev_lamport(comms_.data(), lay_, n_, ip.data(), op.data(), so.data(), sl.data(), ro.data(),
                                              rl.data(), static_cast<size_t>(cap_bytes), stream()));
  }
  void barrier() { B200C_CUDA_CHECK(launch_barrier(comms_.data(), n_, stream())); }
  // Runs the kernel whose wait can never be satisfied; returns the status words.
  std::vector<uint32_t> wait_unset_flag() {
    B200C_CUDA_CHECK(launch_wait_unset_flag(comms_.data(), n_, stream()));
    B200C_CUDA_CHECK(cudaStreamSynchronize(stream()));
    return status();
  }

  // DeviceWindow self-test: ring put + signal + barrier through the device API.
  std::vector<at::Tensor> window_ring(std::vector<at::Tensor> srcs, std::vector<at::Tensor> dsts) {
    check(srcs);
    check(dsts);
    const size_t bytes = srcs[0].nbytes();
    const int sigs = 2;
    std::vector<void*> ctrl(n_), local(n_);
    const size_t sig_bytes = static_cast<size_t>(sigs) * n_ * 8, bar_bytes = static_cast<size_t>(n_) * 8;
    for (int r = 0; r < n_; ++r) {
      B200C_CUDA_CHECK(cudaMalloc(&ctrl[r], sig_bytes + bar_bytes));
      B200C_CUDA_CHECK(cudaMemset(ctrl[r], 0, sig_bytes + bar_bytes));
      B200C_CUDA_CHECK(cudaMalloc(&local[r], 64 * 8));
      B200C_CUDA_CHECK(cudaMemset(local[r], 0, 64 * 8));
    }
    std::vector<DeviceWindow> wins(n_);
    std::vector<RegisteredBuffer> regs(n_);
    for (int r = 0; r < n_; ++r) {
      DeviceWindow& w = wins[r];
      std::memset(&w, 0, sizeof(w));
      w.rank = r;
      w.nranks = n_;
      w.bytes = dsts[r].nbytes();
      for (int p = 0; p < n_; ++p) {
        w.data[p] = static_cast<char*>(dsts[p].data_ptr());
        w.signals[p] = static_cast<uint64_t*>(ctrl[p]);
        w.barrier_flags[p] = reinterpret_cast<uint64_t*>(static_cast<char*>(ctrl[p]) + sig_bytes);
      }
      w.signal_count = sigs;
      w.counter_count = 1;
      w.barrier_count = 1;
      w.counters = static_cast<uint64_t*>(local[r]);
      w.barrier_epochs = static_cast<uint64_t*>(local[r]) + 8;
      w.status = status_dev_;
      w.timeout_ns = comms_[0].timeout_ns;
      regs[r] = RegisteredBuffer{static_cast<char*>(srcs[r].data_ptr()), static_cast<size_t>(srcs[r].nbytes())};
    }
    DeviceWindow* dwins = nullptr;
    RegisteredBuffer* dregs = nullptr;
    B200C_CUDA_CHECK(cudaMalloc(&dwins, sizeof(DeviceWindow) * n_));
    B200C_CUDA_CHECK(cudaMalloc(&dregs, sizeof(RegisteredBuffer) * n_));
    B200C_CUDA_CHECK(cudaMemcpy(dwins, wins.data(), sizeof(DeviceWindow) * n_, cudaMemcpyHostToDevice));
    B200C_CUDA_CHECK(cudaMemcpy(dregs, regs.data(), sizeof(RegisteredBuffer) * n_, cudaMemcpyHostToDevice));
    B200C_CUDA_CHECK(launch_window_selftest(dwins, n_, dregs, bytes, stream()));
    B200C_CUDA_CHECK(cudaStreamSynchronize(stream()));
    // Report each rank's put counter so the test can check it was bumped.
    std::vector<at::Tensor> counters;
    for (int r = 0; r < n_; ++r) {
      at::Tensor c = at::empty({1}, at::TensorOptions().dtype(at::kLong).device(at::kCUDA));
      B200C_CUDA_CHECK(cudaMemcpy(c.data_ptr(), local[r], 8, cudaMemcpyDeviceToDevice));
      counters.push_back(c);
    }
    cudaFree(dwins);
    cudaFree(dregs);
    for (int r = 0; r < n_; ++r) {
      cudaFree(ctrl[r]);
      cudaFree(local[r]);
    }
    return counters;
  }

 private:
  int n_;
  HeapLayout lay_;
  size_t flags_off_ = 0, total_ = 0;
  std::vector<void*> heaps_, epochs_, arn_stage_;
  uint32_t* status_host_ = nullptr;
  uint32_t* status_dev_ = nullptr;
  std::vector<CommDev> comms_;
};

} // namespace

namespace {

// Runtime seam with scripted event queries, for exercising the work state
// machine and the watchdog's timeout rule on a machine without a GPU.
class ScriptedCudaApi final : public CudaApi {
 public:
  ScriptedCudaApi(std::vector<int> start_script, std::vector<int> end_script)
      : start_(std::move(start_script)), end_(std::move(end_script)) {}
  cudaError_t eventCreate(cudaEvent_t* e, unsigned) override {
    *e = reinterpret_cast<cudaEvent_t>(++next_handle_);
    return cudaSuccess;
  }
  cudaError_t eventDestroy(cudaEvent_t) override {
    ++destroyed;
    return cudaSuccess;
  }
  cudaError_t eventRecord(cudaEvent_t, cudaStream_t) override { return cudaSuccess; }
  cudaError_t eventQuery(cudaEvent_t e) override {
    // handle 1 = start event, handle 2 = end event
    auto& script = reinterpret_cast<uintptr_t>(e) == 1 ? start_ : end_;
    size_t& pos = reinterpret_cast<uintptr_t>(e) == 1 ? start_pos_ : end_pos_;
    if (script.empty()) return cudaErrorNotReady;
    const int code = script[std::min(pos, script.size() - 1)];
    ++pos;
    return static_cast<cudaError_t>(code);
  }
  cudaError_t eventSynchronize(cudaEvent_t) override { return cudaSuccess; }
  cudaError_t streamWaitEvent(cudaStream_t, cudaEvent_t) override { return cudaSuccess; }
  cudaError_t streamIsCapturing(cudaStream_t, bool* capturing, unsigned long long* id) override {
    *capturing = false;
    *id = 0;
    return cudaSuccess;
  }
  const char* errorString(cudaError_t e) override { return e == cudaSuccess ? "ok" : "scripted failure"; }
  int destroyed = 0;

 private:
  std::vector<int> start_, end_;
  size_t start_pos_ = 0, end_pos_ = 0;
  uintptr_t next_handle_ = 0;
};

} // namespace

void bind_cuda_backend(py::module_& m) {
  // Test hook: drives one CudaWork through `polls` watchdog polls `step_ms` apart with scripted
  // cudaEventQuery results (0 = success, 600 = not ready, anything else = an error) and returns the
  // status after each poll, the error text and the number of events destroyed with the work.
  m.def("_scripted_work_polls", [](std::vector<int> start_script, std::vector<int> end_script, int timeout_ms, int step_ms,
                                   int polls) {
    auto api = std::make_shared<ScriptedCudaApi>(std::move(start_script), std::move(end_script));
    cudaEvent_t a = nullptr, b = nullptr;
    api->eventCreate(&a, 0);
    api->eventCreate(&b, 0);
    std::vector<std::string> seen;
    std::string err;
    {
      auto w = c10::make_intrusive<CudaWork>(api, a, b, false, 0, Millis(timeout_ms), std::vector<at::Tensor>{},
                                            std::weak_ptr<CudaBackend>(), false);
      auto now = std::chrono::steady_clock::now();
      for (int i = 0; i < polls; ++i) {
        w->poll(now);
        switch (w->status()) {
          case WorkStatus::NOT_STARTED: seen.emplace_back("NOT_STARTED"); break;
          case WorkStatus::INPROGRESS: seen.emplace_back("INPROGRESS"); break;
          case WorkStatus::COMPLETED: seen.emplace_back("COMPLETED"); break;
          case WorkStatus::TIMEDOUT: seen.emplace_back("TIMEDOUT"); break;
          case WorkStatus::ERROR: seen.emplace_back("ERROR"); break;
        }
        now += std::chrono::milliseconds(step_ms);
      }
      err = w->error();
    }
    return py::make_tuple(seen, err, api->destroyed);
  });

  register_cuda_backends();
  register_lazy_backends();
  m.def("_lazy_pair_count", [](const std::shared_ptr<Backend>& b) { return lazy_pair_count(b); });
  m.def("_lazy_primary", [](const std::shared_ptr<Backend>& b) { return lazy_primary(b); });

  py::class_<CudaBackend, Backend, std::shared_ptr<CudaBackend>>(m, "CudaBackend")
      .def("device_alltoallv_single", [](CudaBackend& b, at::Tensor out, const at::Tensor& in, const at::Tensor& os,
                                         const at::Tensor& is, bool a, OptHints h, OptMillis to) {
        return b.device_alltoallv_single(out, in, os, is, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("output_split_sizes"), py::arg("input_split_sizes"),
         py::arg("async_op"), py::arg("hints") = py::none(), py::arg("timeout") = py::none(),
         py::call_guard<py::gil_scoped_release>())
      .def("reduce_scatter_quantized", [](CudaBackend& b, at::Tensor out, const at::Tensor& in, const ReduceOp& op,
                                          int64_t seed, bool a, OptHints h, OptMillis to) {
        return b.reduce_scatter_quantized(out, in, op, seed, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("op"), py::arg("seed") = 0, py::arg("async_op") = false,
         py::arg("hints") = py::none(), py::arg("timeout") = py::none(), py::call_guard<py::gil_scoped_release>())
      .def("suspend", &CudaBackend::suspend, py::call_guard<py::gil_scoped_release>())
      .def("resume", &CudaBackend::resume, py::call_guard<py::gil_scoped_release>())
      .def("is_suspended", &CudaBackend::is_suspended)
      .def("seq_heads_exchange", [](CudaBackend& b, at::Tensor out, const at::Tensor& in, bool to_heads, bool a, OptHints h,
                                    OptMillis to) {
        return b.seq_heads_exchange(out, in, to_heads, a, make_op_options(h, to));
      }, py::arg("output"), py::arg("input"), py::arg("to_heads"), py::arg("async_op") = false,
         py::arg("hints") = py::none(), py::arg("timeout") = py::none(), py::call_guard<py::gil_scoped_release>())
      .def("symm_empty", [](CudaBackend& b, std::vector<int64_t> sizes, py::object dtype) {
        const at::ScalarType st = torch::python::detail::py_object_to_dtype(dtype);
        py::gil_scoped_release nogil;
        return b.symm_empty(sizes, st);
      }, py::arg("sizes"), py::arg("dtype"))
      .def("symm_free", &CudaBackend::symm_free, py::arg("tensor"), py::call_guard<py::gil_scoped_release>())
      .def("tensor_register", &CudaBackend::tensor_register, py::arg("tensor"), py::call_guard<py::gil_scoped_release>())
      .def("tensor_deregister", &CudaBackend::tensor_deregister, py::arg("tensor"), py::call_guard<py::gil_scoped_release>())
      .def("is_symmetric", [](CudaBackend& b, const at::Tensor& t) {
        SymmView v;
        return b.lookup_symm(t.data_ptr(), t.nbytes(), &v);
      })
      .def("has_multicast_alias", [](CudaBackend& b, const at::Tensor& t) {
        SymmView v;
        return b.lookup_symm(t.data_ptr(), t.nbytes(), &v) && v.mc != nullptr;
      })
      .def("channel_stream", [](CudaBackend& b, int chan) { return reinterpret_cast<uintptr_t>(b.channel_stream(chan)); })
      .def("comm_dump", &CudaBackend::comm_dump)
      .def("colltrace_dump", [](CudaBackend& b) {
        py::list out;
        for (const auto& e : b.colltrace_dump()) {
          py::dict d;
          d["seq"] = e.seq;
          d["op"] = e.op;
          d["start_ns"] = e.start_ns;
          d["end_ns"] = e.end_ns;
          out.append(d);
        }
        return out;
      })
      .def("set_config", &CudaBackend::set_config)
      .def("get_nccl_comm_ptr", &CudaBackend::get_nccl_comm_ptr)
      .def("enable_trace", [](CudaBackend& b) {
        at::Tensor t = at::zeros({kMaxBlocks, kTraceSlots}, at::TensorOptions().dtype(at::kLong).device(b.device()));
        b.set_trace_buffer(t);
        return t;
      })
      .def("disable_trace", [](CudaBackend& b) { b.set_trace_buffer(at::Tensor()); })
      .def("internal_stream", [](CudaBackend& b) { return reinterpret_cast<uintptr_t>(b.internal_stream()); })
      .def("has_multicast", [](CudaBackend& b) { return b.comm_dev().mc_heap != nullptr; });

  py::class_<EmuWorld>(m, "_EmuWorld")
      .def(py::init<int, size_t, double>(), py::arg("nranks"), py::arg("staging_bytes") = 8u << 20,
           py::arg("wait_ms") = 2000.0)
      .def("all_reduce", &EmuWorld::all_reduce)
      .def("all_reduce_rmsnorm", &EmuWorld::all_reduce_rmsnorm)
      .def("reduce_scatter", &EmuWorld::reduce_scatter)
      .def("reduce_scatter_sr", &EmuWorld::reduce_scatter_sr)
      .def("all_gather", &EmuWorld::all_gather)
      .def("all_to_all", &EmuWorld::all_to_all)
      .def("all_to_all_device_splits", &EmuWorld::all_to_all_device_splits)
      .def("symm_all_gather", &EmuWorld::symm_all_gather)
      .def("symm_reduce_scatter", &EmuWorld::symm_reduce_scatter)
      .def("symm_all_reduce", &EmuWorld::symm_all_reduce)
      .def("symm_all_to_all", &EmuWorld::symm_all_to_all)
      .def("symm_seq_heads", &EmuWorld::symm_seq_heads)
      .def("all_reduce_lamport", &EmuWorld::all_reduce_lamport)
      .def("exchange_lamport", &EmuWorld::exchange_lamport)
      .def("exchangev_lamport", &EmuWorld::exchangev_lamport)
      .def("broadcast", &EmuWorld::broadcast)
      .def("barrier", &EmuWorld::barrier)
      .def("wait_unset_flag", &EmuWorld::wait_unset_flag)
      .def("window_ring", &EmuWorld::window_ring)
      .def("status", &EmuWorld::status)
      .def("clear_status", &EmuWorld::clear_status);

  // What ncclCommInitRankConfig would be given for these hints: {field: value} of the fields that are set.
  m.def("_nccl_config_from_hints", [](const Hints& h, const std::string& comm_name) {
    const NcclConfig c = CudaBackend::nccl_config_from_hints(h, comm_name);
    std::map<std::string, std::string> out;
    auto put = [&out](const char* k, int v) {
      if (v != NcclConfig::kUnset) out[k] = std::to_string(v);
    };
    put("blocking", c.blocking);
    put("cgaClusterSize", c.cgaClusterSize);
    put("minCTAs", c.minCTAs);
    put("maxCTAs", c.maxCTAs);
    put("splitShare", c.splitShare);
    put("trafficClass", c.trafficClass);
    put("collnetEnable", c.collnetEnable);
    put("CTAPolicy", c.CTAPolicy);
    put("shrinkShare", c.shrinkShare);
    put("nvlsCTAs", c.nvlsCTAs);
    put("nChannelsPerNetPeer", c.nChannelsPerNetPeer);
    put("nvlinkCentricSched", c.nvlinkCentricSched);
    if (!c.netName.empty()) out["netName"] = c.netName;
    if (!c.commName.empty()) out["commName"] = c.commName;
    return out;
  });

  m.def("_symm_allocator_symbols", []() { return std::make_pair(std::string("b200c_symm_alloc"), std::string("b200c_symm_free")); });
  m.def("_exportable_allocations", []() { return ExportableRegistry::get().live(); });
}

} // namespace b200c
