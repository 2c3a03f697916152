// All-to-all (host- or device-resident split sizes), broadcast, barrier and
// the bounded-wait self test, over the symmetric heap (sm_100a).
//
// Replaces, in the reference: comms/prims/collectives/AllToAllv.cuh:113-263,
// comms/ctran/algos/AllToAll/DeviceAllToAllvPipes.cu (split sizes on the
// device, prefix sums in the kernel), comms/ctran/algos/Broadcast/Broadcast.cu:19,
// and the barrier-as-all-reduce of comms/torchcomms/ncclx/TorchCommNCCLX.cpp:1907-1944.
#include "coll_pipe2.cuh"

namespace b200c {
namespace coll {

struct A2aOp {
  struct Args {
    const char* in;
    char* out;
    // Per-peer byte ranges. With dev_send_len != nullptr the send lengths are
    // read from device memory (int64 element counts scaled by elem_bytes,
    // blocks packed back to back) and the receive side is learnt from the
    // senders.
    size_t send_off[kMaxRanks], send_len[kMaxRanks], recv_off[kMaxRanks], recv_len[kMaxRanks];
    // Non-zero: every rank already knows all block lengths (equal splits) and
    // this is the largest; the count exchange and its two barriers are skipped.
    size_t known_max;
    const long long* dev_send_len;
    size_t elem_bytes;
    // Capacities of `in` and `out` (0 = not checked). Lengths that do not fit
    // are clamped and reported through the status word: split sizes that come
    // from device memory are data, not arguments the host could have checked.
    size_t in_bytes, out_bytes;
    size_t bulk_off;
    size_t meta_off;      // kMaxBlocks x kMaxRanks x kMaxRanks uint64 per rank
    size_t chunk_bytes;   // per-peer bytes staged per step; multiple of 16
  };

  // Per-block view of the exchange, filled by prologue().
  struct Plan {
    size_t send_off[kMaxRanks], send_len[kMaxRanks], recv_off[kMaxRanks], recv_len[kMaxRanks];
    size_t max_len;
  };
  static __device__ Plan& plan() {
    __shared__ Plan p;
    return p;
  }

  // Tells every peer how much it will get from this rank and learns the
  // global maximum block length, so that all ranks agree on the step count.
  static __device__ size_t prologue(const CommDev& c, const Args& a) {
    Plan& pl = plan();
    if (a.known_max != 0 && a.dev_send_len == nullptr) {
      if (threadIdx.x < c.nranks) {
        const int p = threadIdx.x;
        pl.send_off[p] = a.send_off[p];
        pl.send_len[p] = a.send_len[p];
        pl.recv_off[p] = a.recv_off[p];
        pl.recv_len[p] = a.recv_len[p];
      }
      if (threadIdx.x == 0) pl.max_len = a.known_max;
      __syncthreads();
      return (a.known_max + a.chunk_bytes - 1) / a.chunk_bytes;
    }
    BlockEpoch ep;
    ep.load(c, kFlagSetMeta);
    unsigned long long* meta_mine = reinterpret_cast<unsigned long long*>(c.heap[c.rank] + a.meta_off) +
        static_cast<size_t>(blockIdx.x) * kMaxRanks * kMaxRanks;
    if (threadIdx.x < c.nranks) {
      const int p = threadIdx.x;
      // Row `rank` of peer p's table: what this rank sends to each destination.
      unsigned long long* meta_p = reinterpret_cast<unsigned long long*>(c.heap[p] + a.meta_off) +
          static_cast<size_t>(blockIdx.x) * kMaxRanks * kMaxRanks + static_cast<size_t>(c.rank) * kMaxRanks;
      size_t acc = 0;
      bool bad = false;
      for (int d = 0; d < c.nranks; ++d) {
        size_t soff, len;
        if (a.dev_send_len != nullptr) {
          long long cnt = a.dev_send_len[d];
          if (cnt < 0) {
            bad = true;
            cnt = 0;
          }
          soff = acc;
          len = static_cast<size_t>(cnt) * a.elem_bytes;
        } else {
          soff = a.send_off[d];
          len = a.send_len[d];
        }
        if (a.in_bytes != 0 && soff + len > a.in_bytes) {
          bad = true;
          len = soff < a.in_bytes ? a.in_bytes - soff : 0;
        }
        acc = soff + len;
        meta_p[d] = len;
        if (d == p) {
          pl.send_off[p] = soff;
          pl.send_len[p] = len;
        }
      }
      if (bad) c.status[0] = c.status[0] | kStatusBadArg;
    }
    block_barrier(c, kFlagSetMeta, ep, 0x51);
    if (threadIdx.x == 0) {
      size_t mx = 0, roff = 0;
      for (int q = 0; q < c.nranks; ++q) {
        for (int d = 0; d < c.nranks; ++d) {
          const size_t l = meta_mine[q * kMaxRanks + d];
          mx = l > mx ? l : mx;
        }
        size_t rl = meta_mine[q * kMaxRanks + c.rank];
        const size_t at = a.dev_send_len != nullptr ? roff : a.recv_off[q];
        if (a.out_bytes != 0) {
          // What the sender announces must fit where the receiver puts it.
          size_t cap = at < a.out_bytes ? a.out_bytes - at : 0;
          if (a.dev_send_len == nullptr && a.recv_len[q] < cap) cap = a.recv_len[q];
          if (rl > cap) {
            c.status[0] = c.status[0] | kStatusBadArg;
            rl = cap;
          }
        }
        pl.recv_len[q] = rl;
        pl.recv_off[q] = at;
        roff += rl;
      }
      pl.max_len = mx;
    }
    // Second barrier: nobody rewrites a count table (next call) while a peer
    // still reads it.
    block_barrier(c, kFlagSetMeta, ep, 0x52);
    ep.store(c, kFlagSetMeta);
    return (pl.max_len + a.chunk_bytes - 1) / a.chunk_bytes;
  }
  static __device__ size_t slot_bytes(const CommDev& c, const Args& a) { return a.chunk_bytes * c.nranks; }
  static __device__ void stage(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    const Plan& pl = plan();
    const size_t b0 = chunk * a.chunk_bytes;
    for (int p = 0; p < c.nranks; ++p) {
      if (pl.send_len[p] > b0) {
        block_copy(c.heap[c.rank] + off + p * a.chunk_bytes, a.in + pl.send_off[p] + b0,
                   min_sz(a.chunk_bytes, pl.send_len[p] - b0));
      }
    }
  }
  static __device__ void consume(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    const Plan& pl = plan();
    const size_t b0 = chunk * a.chunk_bytes;
    for (int i = 0; i < c.nranks; ++i) {
      int q = c.rank + i;
      if (q >= c.nranks) q -= c.nranks;
      if (pl.recv_len[q] > b0) {
        block_copy(a.out + pl.recv_off[q] + b0, c.heap[q] + off + static_cast<size_t>(c.rank) * a.chunk_bytes,
                   min_sz(a.chunk_bytes, pl.recv_len[q] - b0));
      }
    }
  }
};

struct BcastOp {
  struct Args {
    char* buf;
    size_t bytes;
    int root;
    int use_mc;
    size_t bulk_off;
    size_t chunk_bytes;
  };
  static __device__ size_t prologue(const CommDev&, const Args& a) {
    return (a.bytes + a.chunk_bytes - 1) / a.chunk_bytes;
  }
  static __device__ size_t slot_bytes(const CommDev&, const Args& a) { return a.chunk_bytes; }
  static __device__ void stage(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    if (c.rank != a.root) return;
    const size_t b0 = chunk * a.chunk_bytes;
    block_copy(c.heap[c.rank] + off, a.buf + b0, min_sz(a.chunk_bytes, a.bytes - b0));
  }
  static __device__ void consume(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    if (c.rank == a.root) return;
    const size_t b0 = chunk * a.chunk_bytes;
    block_copy(a.buf + b0, c.heap[a.root] + off, min_sz(a.chunk_bytes, a.bytes - b0));
  }
};

struct BarrierOp {
  struct Args {
    int unused;
  };
  static __device__ void run(const CommDev& c, const Args&) {
    BlockEpoch ep;
    ep.load(c, kFlagSetBarrier);
    block_barrier(c, kFlagSetBarrier, ep, 0x71);
    ep.store(c, kFlagSetBarrier);
  }
};

// Waits for a flag value nobody will ever write; exists to exercise the
// bounded-wait path (the wait gives up after c.timeout_ns and reports).
struct WaitUnsetOp {
  struct Args {
    int unused;
  };
  static __device__ void run(const CommDev& c, const Args&) {
    if (threadIdx.x == 0) {
      const uint32_t* slot = flag_slot(c, c.rank, kFlagSetBarrier, kMaxBlocks - 1, 0);
      const uint32_t want = ld_relaxed_sys(slot) + 0x40000000u;
      wait_flag_reached(c, slot, want, 0, 0x7f);
    }
  }
};

static cudaError_t a2a_launch(const CommDev* comms, const HeapLayout& lay, int emu_ranks, std::vector<A2aOp::Args>& args,
                              LaunchShape shape, cudaStream_t stream) {
  const int nranks = comms[0].nranks;
  const size_t chunk = (shape.chunk_bytes / 16) * 16;
  if (chunk == 0 || static_cast<size_t>(shape.blocks) * kPipeSlots * chunk * nranks > lay.bulk_bytes) return cudaErrorInvalidValue;
  for (auto& a : args) {
    a.bulk_off = lay.bulk_off;
    a.meta_off = lay.small_off + 2 * static_cast<size_t>(kSmallBlocks) * kSmallPiece;
    a.chunk_bytes = chunk;
  }
  // The grid must be identical on every rank, and ranks see different split
  // sizes: the caller picks `shape.blocks` from rank-independent facts only.
  return launch_op<Pipe2<A2aOp>>(comms, emu_ranks, args.data(), shape.blocks, shape.threads, stream);
}

} // namespace coll

cudaError_t launch_all_to_all(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                              void* const* out, const size_t* send_off, const size_t* send_len,
                              const size_t* recv_off, const size_t* recv_len, size_t max_len, LaunchShape shape,
                              cudaStream_t stream) {
  using namespace coll;
  (void)max_len;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const int nranks = comms[0].nranks;
  std::vector<A2aOp::Args> args(n);
  for (int i = 0; i < n; ++i) {
    A2aOp::Args& a = args[i];
    a = {};
    a.in = static_cast<const char*>(in[i]);
    a.out = static_cast<char*>(out[i]);
    for (int p = 0; p < nranks; ++p) {
      a.send_off[p] = send_off[i * nranks + p];
      a.send_len[p] = send_len[i * nranks + p];
      a.recv_off[p] = recv_off[i * nranks + p];
      a.recv_len[p] = recv_len[i * nranks + p];  // used only with known_max; otherwise learnt from the senders
    }
    a.known_max = shape.known_max;
    a.dev_send_len = nullptr;
    a.elem_bytes = 1;
  }
  return a2a_launch(comms, lay, emu_ranks, args, shape, stream);
}

cudaError_t launch_all_to_all_device_splits(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                                            const void* const* in, void* const* out,
                                            const long long* const* dev_send_counts, size_t elem_bytes,
                                            LaunchShape shape, cudaStream_t stream, const size_t* in_bytes, const size_t* out_bytes) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<A2aOp::Args> args(n);
  for (int i = 0; i < n; ++i) {
    A2aOp::Args& a = args[i];
    a = {};
    a.in = static_cast<const char*>(in[i]);
    a.out = static_cast<char*>(out[i]);
    a.dev_send_len = dev_send_counts[i];
    a.elem_bytes = elem_bytes;
    a.in_bytes = in_bytes != nullptr ? in_bytes[i] : 0;
    a.out_bytes = out_bytes != nullptr ? out_bytes[i] : 0;
  }
  return a2a_launch(comms, lay, emu_ranks, args, shape, stream);
}

cudaError_t launch_broadcast(const CommDev* comms, const HeapLayout& lay, int emu_ranks, void* const* buf,
                             size_t bytes, int root, bool use_mc, LaunchShape shape, cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const size_t chunk = (shape.chunk_bytes / 16) * 16;
  if (chunk == 0) return cudaErrorInvalidValue;
  const size_t nchunks = (bytes + chunk - 1) / chunk;
  const int blocks = static_cast<int>(std::min<size_t>(shape.blocks, std::max<size_t>(nchunks, 1)));
  if (static_cast<size_t>(blocks) * kPipeSlots * chunk > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<BcastOp::Args> args(n);
  for (int i = 0; i < n; ++i) args[i] = {static_cast<char*>(buf[i]), bytes, root, use_mc ? 1 : 0, lay.bulk_off, chunk};
  return launch_op<Pipe2<BcastOp>>(comms, emu_ranks, args.data(), blocks, shape.threads, stream);
}

cudaError_t launch_barrier(const CommDev* comms, int emu_ranks, cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<BarrierOp::Args> args(n);
  return launch_op<BarrierOp>(comms, emu_ranks, args.data(), 1, 32, stream);
}

cudaError_t launch_wait_unset_flag(const CommDev* comms, int emu_ranks, cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<WaitUnsetOp::Args> args(n);
  return launch_op<WaitUnsetOp>(comms, emu_ranks, args.data(), 1, 32, stream);
}

} // namespace b200c
