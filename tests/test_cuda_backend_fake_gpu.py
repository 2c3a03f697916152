"""The CUDA backend's host logic on a machine without a GPU.

Fakes of the CUDA runtime, the CUDA driver and NCCL are installed
(``_comms._install_fake_gpu``) before the communicator is created; the backend
then bootstraps, routes, records events, tracks captured graphs and runs its
watchdog exactly as on a GPU, except that kernels are noted in a log instead of
launched.  Multi-rank cases run as separate CPU processes that share a store,
with file descriptors of the fake memory handles travelling between them like
the real ones.

Covers what the reference's mock-driven suites cover
(comms/torchcomms/ncclx/tests/unit/cpp: TorchCommNCCLXTest,
TorchWorkNCCLXQueueTest, GraphEventTrackerTest, HintParsingTest).
"""
import os
import time
from datetime import timedelta

import pytest
import torch

from tests.mp_util import free_port, run_ranks


def _reset_health():
    from torchcomms_b200 import _comms

    _comms._health_reset()


def _new_comm(name, world_hints=None, **kw):
    import torchcomms_b200 as tc

    hints = {"staging_mb": "1"}
    hints.update(world_hints or {})
    return tc.new_comm("b200", torch.device("cuda", 0), name=name, hints=hints,
                       abort_process_on_timeout_or_error=False, **kw)


@pytest.fixture()
def single_rank_env(monkeypatch):
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(free_port()))
    from torchcomms_b200 import _comms

    fake = _comms._install_fake_gpu()
    yield fake
    _comms._uninstall_fake_gpu()


def test_bootstrap_streams_and_dump(single_rank_env):
    fake = single_rank_env
    comm = _new_comm("fake1", is_high_priority_stream=True)
    impl = comm.get_backend_impl()
    d = impl.comm_dump()
    assert d["rank"] == "0" and d["size"] == "1" and d["symm_mode"] == "local"
    # one stream per channel, created with the high priority of the fake range (-5)
    created = [l for l in fake.log() if l.startswith("stream_create")]
    assert len(created) == 4 and all(l.endswith("priority -5") for l in created)
    assert len({impl.channel_stream(c) for c in range(4)}) == 4
    assert any(l.startswith("launch lamport_init") for l in fake.log())
    comm.finalize()


def test_sync_operation_takes_the_event_less_path_until_somebody_observes(single_rank_env):
    fake = single_rank_env
    import torchcomms_b200 as tc

    comm = _new_comm("fake2")
    t = torch.ones(1024)
    fake.clear_log()
    w = comm.all_reduce(t, tc.ReduceOp.SUM, False)
    log = fake.log()
    assert [l.split()[0] for l in log] == ["launch"], log  # no events, nothing but the kernel
    assert log[0].split()[1].startswith("all_reduce/")
    w.wait()
    assert w.is_completed()
    # a post-hook makes every operation report start and end through events
    seen = []
    handle = comm.register_post_hook(lambda op_id, args: seen.append(op_id))
    fake.clear_log()
    comm.all_reduce(t, tc.ReduceOp.SUM, False).wait()
    kinds = [l.split()[0] for l in fake.log()]
    assert kinds[:3] == ["record", "launch", "record"], kinds
    assert seen
    handle.remove()
    comm.finalize()


def test_timestamp_ring_keeps_the_last_operations(single_rank_env):
    """`colltrace=N`: one ring entry per operation issued outside a capture, oldest entries overwritten."""
    import torchcomms_b200 as tc

    comm = _new_comm("fake_trace", world_hints={"colltrace": "4"})
    impl = comm.get_backend_impl()
    assert impl.colltrace_dump() == []
    t = torch.ones(256)
    for _ in range(3):
        comm.all_reduce(t, tc.ReduceOp.SUM, False)
    comm.barrier(True).wait()
    comm.all_reduce(t, tc.ReduceOp.SUM, True).wait()
    out = torch.empty(256)
    comm.all_gather_single(out, t, False)
    entries = impl.colltrace_dump()
    assert [e["seq"] for e in entries] == [2, 3, 4, 5], entries   # six operations, the ring holds four
    assert entries[0]["op"].startswith("all_reduce/") and entries[1]["op"].startswith("barrier")
    assert entries[3]["op"].startswith("all_gather")
    assert all(e["start_ns"] == 0 and e["end_ns"] == 0 for e in entries)   # nothing runs under the fake runtime
    d = impl.comm_dump()
    assert d["colltrace/entries"] == "4" and d["colltrace/issued"] == "6"
    comm.finalize()


def test_async_operation_protocol_and_cross_stream_order(single_rank_env):
    fake = single_rank_env
    import torchcomms_b200 as tc

    comm = _new_comm("fake3")
    impl = comm.get_backend_impl()
    main = f"s{impl.channel_stream(0)}"
    t = torch.ones(300_000)  # beyond the one-shot size: the staged two-shot kernel of the main channel
    fake.clear_log()
    w = comm.all_reduce(t, tc.ReduceOp.SUM, True, hints={"algo": "twoshot"})
    log = fake.log()
    # dependency on the caller's stream, then start event, kernel, end event on the channel's stream
    assert log[0].startswith("record") and log[0].endswith("s16")          # dep event on the current stream (0x10)
    assert log[1] == f"wait {main} {log[0].split()[1]}"
    assert log[2].startswith("record") and log[2].endswith(main)
    assert log[3] == f"launch all_reduce/twoshot {main}"
    assert log[4].startswith("record") and log[4].endswith(main)
    end_event = log[4].split()[1]
    # wait() is a stream dependency on the end event, not a host block
    fake.clear_log()
    w.wait()
    assert fake.log() == [f"wait s16 {end_event}"]
    # the next synchronous operation of the SAME channel on another stream follows that end event ...
    w2 = comm.all_reduce(t, tc.ReduceOp.SUM, True, hints={"algo": "twoshot"})
    end2 = [l for l in fake.log() if l.startswith("record")][-1].split()[1]
    fake.clear_log()
    comm.all_reduce(t, tc.ReduceOp.SUM, False, hints={"algo": "twoshot"})
    assert fake.log()[0] == f"wait s16 {end2}"
    w2.wait()
    # ... while an operation of another channel does not wait for it
    src = torch.ones(8)
    out = torch.empty(8)
    fake.clear_log()
    comm.all_gather_single(out, src, False)  # single rank: cast kernel on the all-gather channel
    assert not any(l.startswith("wait") for l in fake.log()), fake.log()
    comm.finalize()


def test_event_pool_is_reused(single_rank_env):
    fake = single_rank_env
    import torchcomms_b200 as tc

    comm = _new_comm("fake4", {"garbage_collect_interval_ms": "10"})
    t = torch.ones(64)
    for _ in range(50):
        comm.all_reduce(t, tc.ReduceOp.SUM, True).wait()
        time.sleep(0.002)
    time.sleep(0.1)
    # 50 asynchronous operations, but the watchdog recycles finished works' events
    assert fake.events_created() < 60
    d = comm.get_backend_impl().comm_dump()
    assert int(d["inflight"]) == 0
    comm.finalize()
    assert fake.live_events() == 0


def test_captured_operations_are_chained_counted_and_released(single_rank_env):
    fake = single_rank_env
    import torchcomms_b200 as tc

    comm = _new_comm("fake5", {"garbage_collect_interval_ms": "10"})
    impl = comm.get_backend_impl()
    t = torch.ones(1024)
    fake.set_capturing(True, 7)
    fake.clear_log()
    comm.all_reduce(t, tc.ReduceOp.SUM, False)           # on the capturing stream
    w = comm.all_reduce(t, tc.ReduceOp.SUM, True)        # forks to the channel's stream inside the capture
    w.wait()
    log = fake.log()
    assert sum(l.startswith("graph_retain") for l in log) == 1  # one destroy callback per graph
    records = [l for l in log if l.startswith("record")]
    first_end = records[1].split()[1]
    # the asynchronous operation follows the first one although it runs on another stream
    assert any(l.startswith("wait") and l.endswith(first_end) for l in log), log
    assert impl.comm_dump()["graph_entries"] == "2" and impl.comm_dump()["graphs"] == "1"
    fake.set_capturing(False, 0)
    # replay monitoring keeps the entries while the graph lives ...
    time.sleep(0.1)
    assert impl.comm_dump()["graph_entries"] == "2"
    # ... and drops them, with their events, when the graph is destroyed
    events_before = fake.live_events()
    assert fake.destroy_graph(7) == 1
    deadline = time.time() + 5
    while impl.comm_dump()["graph_entries"] != "0" and time.time() < deadline:
        time.sleep(0.02)
    assert impl.comm_dump()["graph_entries"] == "0" and impl.comm_dump()["graphs"] == "0"
    assert fake.live_events() == events_before - 4
    comm.finalize()


def test_watchdog_times_out_a_stuck_operation_and_runs_abort_hooks(single_rank_env):
    fake = single_rank_env
    import torchcomms_b200 as tc

    comm = _new_comm("fake6", {"garbage_collect_interval_ms": "10"}, timeout=timedelta(milliseconds=150))
    fired = []
    comm.register_abort_hook(lambda: fired.append(True))
    t = torch.ones(64)
    fake.set_stuck(True)                      # end events never complete from here on
    w = comm.all_reduce(t, tc.ReduceOp.SUM, True)
    deadline = time.time() + 5
    while (tc.healthy() or not fired or not comm.is_aborted()) and time.time() < deadline:
        time.sleep(0.02)                      # the watchdog marks the failure, then runs the hooks, then aborts
    assert not tc.healthy()
    assert fired
    assert comm.is_aborted()
    with pytest.raises(RuntimeError, match="unusable after a failure"):
        comm.all_reduce(t, tc.ReduceOp.SUM, False)
    fake.set_stuck(False)
    fake.clear_log()
    with pytest.raises(RuntimeError):
        comm.finalize()                       # reports the failure ...
    # ... after stopping the streams: the broken path synchronises before it unmaps anything
    assert any(l.startswith("sync") for l in fake.log())
    del w
    _reset_health()


def _nccl_error_body(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import _comms

    fake = _comms._install_fake_gpu()
    comm = _new_comm("fake7", {"garbage_collect_interval_ms": "10"})
    assert comm.get_backend_impl().comm_dump()["nccl"] == "1"
    fake.set_nccl_async_error(6)          # ncclRemoteError
    deadline = time.time() + 5
    while tc.healthy() and time.time() < deadline:
        time.sleep(0.02)
    assert not tc.healthy()
    with pytest.raises(RuntimeError, match="NCCL asynchronous error"):
        comm.all_reduce(torch.ones(4), tc.ReduceOp.SUM, False)
    try:
        comm.finalize()
    except RuntimeError:
        pass


def test_nccl_async_error_fails_the_communicator():
    run_ranks(_nccl_error_body, 2, timeout=120)


def test_backend_specific_operations_are_reachable_from_the_communicator(single_rank_env):
    comm = _new_comm("fwd_ops")
    assert comm.get_nccl_comm_ptr() == comm.get_backend_impl().get_nccl_comm_ptr()
    comm.set_config({"symm_blocks": "24"})
    assert comm.get_backend_impl().comm_dump()["tuning/symm_blocks"] == "24"
    comm.finalize()


def test_hints_become_nccl_config(single_rank_env):
    from torchcomms_b200 import _comms

    cfg = _comms._nccl_config_from_hints(
        {"blocking": "0", "cga_cluster_size": "2", "minCTAs": "4", "max_ctas": "16", "netName": "IB", "splitShare": "1",
         "trafficClass": "3", "CTAPolicy": "1", "nvlsCTAs": "8", "algo": "nccl"}, "job")
    assert cfg == {"blocking": "0", "cgaClusterSize": "2", "minCTAs": "4", "maxCTAs": "16", "netName": "IB",
                   "splitShare": "1", "trafficClass": "3", "CTAPolicy": "1", "nvlsCTAs": "8", "commName": "job"}
    assert _comms._nccl_config_from_hints({"algo": "kernel"}, "job") == {}  # nothing for NCCL: plain ncclCommInitRank
    assert _comms._nccl_config_from_hints({"commName": "mine", "blocking": "true"}, "job") == {"blocking": "1", "commName": "mine"}
    with pytest.raises(RuntimeError, match="must be an integer"):
        _comms._nccl_config_from_hints({"minCTAs": "many"}, "job")


def _multi_rank_body(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import _comms

    fake = _comms._install_fake_gpu()
    comm = tc.new_comm("b200", torch.device("cuda", rank), name="fakeN", abort_process_on_timeout_or_error=False,
                       hints={"staging_mb": "1", "minCTAs": "2", "max_ctas": "8", "auto_nccl": "1"})
    impl = comm.get_backend_impl()
    d = impl.comm_dump()
    assert d["symm_mode"] == "vmm+fd" and d["multicast"] == "1" and d["nccl"] == "1"
    # hints that name NCCL configuration fields reached ncclCommInitRankConfig
    assert fake.nccl_config() == {"minCTAs": "2", "maxCTAs": "8", "commName": "fakeN"}
    assert any(l.startswith("ncclCommInitRankConfig") for l in fake.nccl_log())

    def counts():
        return {k[6:]: int(v) for k, v in impl.comm_dump().items() if k.startswith("count/")}

    # ---- routing table with mixed routing on (world of 4)
    small = torch.ones(1024)                      # 4 KB
    mid = torch.ones(64 * 1024)                   # 256 KB
    big = torch.ones(2 * 1024 * 1024)             # 8 MB
    huge = torch.ones(32 * 1024 * 1024)           # 128 MB
    comm.all_reduce(small, tc.ReduceOp.SUM, False)
    comm.all_reduce(mid, tc.ReduceOp.SUM, False)
    comm.all_reduce(big, tc.ReduceOp.SUM, False)
    comm.all_reduce(huge, tc.ReduceOp.SUM, False)
    comm.all_reduce(torch.ones(8, dtype=torch.int64), tc.ReduceOp.SUM, False)     # dtype the kernels do not cover
    c = counts()
    assert c["all_reduce/lamport"] == 2           # latency class (up to 512 KB): flag-less kernel
    assert c["all_reduce/twoshot"] == 1           # 4 - 64 MB: NVLS two-shot
    assert c["all_reduce/nccl"] == 2              # beyond, and integers
    # symmetric tensors take the one-pass kernels whatever the size
    sym = comm.symm_empty((4 * 1024 * 1024,), torch.float32)
    comm.all_reduce(sym, tc.ReduceOp.SUM, False)
    out = comm.symm_empty((world * 4096,), torch.bfloat16)
    comm.all_gather_single(out, torch.ones(4096), False)                         # fused fp32 -> bf16
    comm.reduce_scatter_single(torch.empty(4096), out, tc.ReduceOp.AVG, False)   # bf16 in, fp32 out
    comm.all_to_all_single(out, torch.ones(world * 4096, dtype=torch.bfloat16), False)     # 8 KB blocks: flag-less
    wide = comm.symm_empty((world * 1024 * 1024,), torch.float32)
    comm.all_to_all_single(wide, torch.ones(world * 1024 * 1024), False)                   # 4 MB blocks: one-pass push
    comm.all_gather_single(torch.empty(world * 64), torch.ones(64), False)                 # plain small tensors: flag-less too
    c = counts()
    assert c["all_reduce/symm"] == 1 and c["all_gather/symm+cast"] == 1 and c["all_gather/lamport"] == 1
    assert c["reduce_scatter/symm"] == 1 and c["all_to_all_single/symm"] == 1 and c["all_to_all_single/lamport"] == 1
    comm.symm_free(wide)
    # forcing NCCL by hint
    comm.all_gather_single(torch.empty(world * 16), torch.ones(16), False, hints={"algo": "nccl"})
    assert counts()["all_gather/nccl"] == 1
    assert any(l.startswith("ncclAllGather sendcount=16") for l in fake.nccl_log())
    # point to point rides on NCCL, grouped
    batch = comm.batch_op_create()
    batch.send(torch.ones(4), (rank + 1) % world)
    batch.recv(torch.empty(4), (rank - 1) % world)
    batch.issue(False)
    tail = fake.nccl_log()[-4:]
    assert tail[0] == "ncclGroupStart" and tail[3] == "ncclGroupEnd"
    # asynchronous operations of different channels run on different streams
    fake.clear_log()
    w1 = comm.all_gather_single(out, torch.ones(4096), True)
    w2 = comm.reduce_scatter_single(torch.empty(4096), out, tc.ReduceOp.SUM, True)
    launches = [l for l in fake.log() if l.startswith("launch")]
    assert launches[0].split()[2] != launches[1].split()[2]
    w1.wait()
    w2.wait()
    # ... but kernels that could hold more SMs together than the GPU has are chained: a 64 MB all-gather (64 blocks)
    # and a 64 MB reduce-scatter (128 blocks) of different channels, the second waits for the first
    big_out = comm.symm_empty((world * 8 * 1024 * 1024,), torch.bfloat16)
    piece = torch.ones(8 * 1024 * 1024, dtype=torch.bfloat16)
    fake.clear_log()
    own = {"algo": "kernel"}     # this communicator has mixed routing on, which would hand both to NCCL
    w1 = comm.all_gather_single(big_out, piece, True, hints=own)
    w2 = comm.reduce_scatter_single(torch.empty(8 * 1024 * 1024, dtype=torch.bfloat16), big_out, tc.ReduceOp.SUM, True, hints=own)
    log = fake.log()
    launches = [i for i, l in enumerate(log) if l.startswith("launch")]
    ag_stream, rs_stream = log[launches[0]].split()[2], log[launches[1]].split()[2]
    ag_end = next(l.split()[1] for l in log[launches[0]:] if l.startswith("record") and l.split()[2] == ag_stream)
    assert f"wait {rs_stream} {ag_end}" in log[launches[0]:launches[1]], log
    w1.wait()
    w2.wait()
    comm.symm_free(big_out)
    # split: members bootstrap a communicator of their own
    members = [r for r in range(world) if r % 2 == rank % 2]
    sub = comm.split(members, "half")
    assert sub.get_size() == len(members)
    sub.finalize()
    comm.symm_free(out)
    comm.symm_free(sym)
    comm.finalize()
    assert "ncclCommDestroy" in fake.nccl_log()


def test_four_fake_ranks_bootstrap_route_and_split():
    run_ranks(_multi_rank_body, 4, timeout=180)


def _tuner_file_body(rank, world, path):
    import torchcomms_b200 as tc
    from torchcomms_b200 import _comms

    _comms._install_fake_gpu()
    comm = tc.new_comm("b200", torch.device("cuda", rank), name="tuned", abort_process_on_timeout_or_error=False,
                       hints={"staging_mb": "1", "tuner_file": path, "lamport_max_bytes": "0"})
    impl = comm.get_backend_impl()
    assert impl.comm_dump()["tuning/tuner_rules"] == "4"

    def counts():
        return {k[6:]: int(v) for k, v in impl.comm_dump().items() if k.startswith("count/")}

    comm.all_reduce(torch.ones(256), tc.ReduceOp.SUM, False)              # 1 KB   -> nccl (first rule)
    comm.all_reduce(torch.ones(64 * 1024), tc.ReduceOp.SUM, False)        # 256 KB -> kernel (second rule)
    comm.all_reduce(torch.ones(4 * 1024 * 1024), tc.ReduceOp.SUM, False)  # 16 MB  -> nccl (last rule: inf)
    comm.all_gather_single(torch.empty(world * 1024), torch.ones(1024), False)   # rule for all_gather: kernel everywhere
    c = counts()
    assert c["all_reduce/nccl"] == 2 and c.get("all_gather/nccl", 0) == 0, c
    assert sum(v for k, v in c.items() if k.startswith("all_reduce/") and k != "all_reduce/nccl") == 1, c
    # a call may still force its route
    comm.all_reduce(torch.ones(256), tc.ReduceOp.SUM, False, hints={"algo": "kernel"})
    assert counts()["all_reduce/nccl"] == 2
    comm.finalize()
    _comms._uninstall_fake_gpu()


def test_tuner_file_routes_by_operation_and_size(tmp_path):
    """A tuner file written from a sweep (utils/tuning.py --emit) decides kernel / NCCL per operation and size."""
    from torchcomms_b200.utils.tuning import tuner_file_lines

    rows = []
    for b, k, n in [(1024, 9.0, 7.0), (262144, 9.0, 14.0), (16 << 20, 70.0, 55.0)]:
        rows += [{"op": "all_reduce", "dtype": "bf16", "bytes": b, "algo": "kernel", "us": k},
                 {"op": "all_reduce", "dtype": "bf16", "bytes": b, "algo": "nccl", "us": n}]
    rows += [{"op": "all_gather", "dtype": "bf16", "bytes": 4096, "algo": "kernel", "us": 7.0},
             {"op": "all_gather", "dtype": "bf16", "bytes": 4096, "algo": "nccl", "us": 11.0}]
    lines = tuner_file_lines(rows)
    assert lines[1:] == ["all_gather inf kernel", "all_reduce 1024 nccl", "all_reduce 262144 kernel", "all_reduce inf nccl"]
    path = tmp_path / "tuner.txt"
    path.write_text("\n".join(lines) + "\n")
    run_ranks(_tuner_file_body, 2, args=(str(path),), timeout=120)


def _suspend_resume_body(rank, world):
    """suspend() gives back every cross-process resource (NCCL communicator destroyed, streams gone, operations
    refused), resume() builds them again among the same members; twice in a row; finalize of a suspended communicator."""
    import torchcomms_b200 as tc
    from torchcomms_b200 import _comms

    fake = _comms._install_fake_gpu()
    comm = tc.new_comm("b200", torch.device("cuda", rank), name="ckpt", abort_process_on_timeout_or_error=False,
                       hints={"staging_mb": "1"})
    impl = comm.get_backend_impl()
    t = torch.ones(1024)
    for cycle in range(2):
        comm.all_reduce(t, tc.ReduceOp.SUM, False)
        sym = comm.symm_empty((4096,), torch.float32)
        assert impl.is_symmetric(sym) and not impl.is_suspended()
        destroyed_before = sum(1 for l in fake.nccl_log() if l.startswith("ncclCommDestroy"))
        impl.suspend()
        assert impl.is_suspended()
        assert sum(1 for l in fake.nccl_log() if l.startswith("ncclCommDestroy")) == destroyed_before + 1
        with pytest.raises(RuntimeError, match="not initialised"):
            comm.all_reduce(t, tc.ReduceOp.SUM, False)
        with pytest.raises(RuntimeError, match="not initialised"):
            impl.suspend()
        inits_before = sum(1 for l in fake.nccl_log() if l.startswith("ncclCommInitRankConfig"))
        impl.resume()
        assert not impl.is_suspended() and comm.get_rank() == rank and comm.get_size() == world
        assert sum(1 for l in fake.nccl_log() if l.startswith("ncclCommInitRankConfig")) == inits_before + 1
        assert not impl.is_symmetric(sym)            # registrations went with the old mappings
        d = impl.comm_dump()
        assert d["size"] == str(world) and d["nccl"] == "1"
        with pytest.raises(RuntimeError, match="not suspended"):
            impl.resume()
    # the helpers act on the communicators that hold cross-process GPU state and skip the others
    from torchcomms_b200.checkpoint import checkpoint_prepare, checkpoint_restore

    other = tc.new_comm("fake", torch.device("cpu"), name="ckpt_cpu")
    assert checkpoint_prepare([other, comm]) == [comm] and impl.is_suspended()
    assert checkpoint_prepare([comm]) == []          # already suspended
    assert checkpoint_restore([comm, other]) == [comm] and not impl.is_suspended()
    other.finalize()
    # a communicator made by split() suspends and resumes on its own store scope, in any order with its parent
    members = [r for r in range(world) if r % 2 == rank % 2]
    sub = comm.split(members, "ckpt_half")
    assert checkpoint_prepare([comm, sub]) == [comm, sub]
    assert checkpoint_restore([sub, comm]) == [sub, comm]
    assert sub.get_size() == len(members) and sub.get_rank() == members.index(rank)
    sub.all_reduce(t, tc.ReduceOp.SUM, False)
    sub.finalize()
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    impl.suspend()
    comm.finalize()                                  # nothing is held: no barrier, no error
    with pytest.raises(RuntimeError, match="finalized"):
        impl.resume()


def test_suspend_and_resume_for_checkpoints():
    run_ranks(_suspend_resume_body, 4, timeout=180)


def test_shipped_tuner_file_loads(single_rank_env):
    """The tuner file that ships with the benchmarks is accepted by the backend's loader (comments, `inf`, both
    spellings of the all-to-all)."""
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "tuner_8xb200.txt")
    comm = _new_comm("shipped_tuner", world_hints={"tuner_file": path})
    rules = sum(1 for ln in open(path) if ln.split("#")[0].strip())
    assert comm.get_backend_impl().comm_dump()["tuning/tuner_rules"] == str(rules)
    comm.finalize()


def _seq_heads_route_body(rank, world):
    """The sequence <-> heads exchange on fake ranks: argument checks, the symmetric-output requirement, the route
    counter, the channel it shares with the all-to-all, the exchange object's ring of output buffers."""
    import torchcomms_b200 as tc
    from torchcomms_b200 import _comms
    from torchcomms_b200.parallel.context import SeqHeadsExchange

    fake = _comms._install_fake_gpu()
    comm = tc.new_comm("b200", torch.device("cuda", rank), name="fsh", abort_process_on_timeout_or_error=False,
                       hints={"staging_mb": "1"})
    impl = comm.get_backend_impl()
    b, h, s, d = 2, 2 * world, 8, 16
    x = torch.ones(b, h, s, d)
    out = comm.symm_empty((b, h // world, s * world, d), torch.float32)
    fake.clear_log()
    impl.seq_heads_exchange(out, x, True, False)
    impl.seq_heads_exchange(comm.symm_empty((b, h, s, d), torch.float32), out, False, True).wait()
    launches = [l for l in fake.log() if l.startswith("launch")]
    assert [l.split()[1] for l in launches] == ["seq_heads_exchange/symm"] * 2
    a2a_out = comm.symm_empty((world * 1024 * 1024,), torch.float32)
    fake.clear_log()
    comm.all_to_all_single(a2a_out, torch.ones(world * 1024 * 1024), True).wait()
    a2a_stream = next(l for l in fake.log() if l.startswith("launch")).split()[2]
    assert launches[1].split()[2] == a2a_stream           # asynchronous calls of both run on the same channel stream
    assert impl.comm_dump()["count/seq_heads_exchange/symm"] == "2"
    with pytest.raises(RuntimeError, match="symmetric"):
        impl.seq_heads_exchange(torch.empty(b, h // world, s * world, d), x, True, False)
    with pytest.raises(RuntimeError, match="expected"):
        impl.seq_heads_exchange(comm.symm_empty((b, h // world, s * world + 1, d), torch.float32), x, True, False)
    with pytest.raises(RuntimeError, match="divide"):
        impl.seq_heads_exchange(out, torch.ones(b, h + 1, s, d), True, False)
    ex = SeqHeadsExchange(comm, slots=2)
    assert ex.fused
    y1, y2, y3 = ex.to_heads(x), ex.to_heads(x), ex.to_heads(x)
    assert y1.data_ptr() == y3.data_ptr() != y2.data_ptr() and y1.shape == (b, h // world, s * world, d)
    assert ex.to_seq(y1, keep=True).shape == x.shape
    ex.close()
    comm.finalize()


def test_sequence_heads_exchange_route_on_fake_ranks():
    run_ranks(_seq_heads_route_body, 2, timeout=120)
