"""Single-process checks of the facade, factory, options, hooks and work
state machine on the ``fake`` backend and on Python-implemented backends.

Modelled on the reference's unit suites (comms/torchcomms/tests/unit/py:
test_factory, test_hooks, test_python_backend, test_copy).
"""
import copy
import os
from datetime import timedelta

import pytest
import torch

import torchcomms_b200 as tc
from torchcomms_b200 import _comms


def _fake(name, **kw):
    return tc.new_comm("fake", torch.device("cpu"), name=name, **kw)


def test_registered_backends():
    assert tc.is_backend_built("fake")
    assert tc.is_backend_built("gloo")
    assert "fake" in tc.built_backends()
    assert not tc.is_backend_built("nonexistent")


def test_unknown_backend_raises():
    with pytest.raises(ModuleNotFoundError, match="failed to find backend.*unknown communication backend"):
        tc.new_comm("nonexistent", torch.device("cpu"), name="x")


def test_basic_accessors_and_finalize():
    c = _fake("acc", timeout=timedelta(seconds=7), hints={"fake_rank": "2", "fake_size": "4"})
    assert (c.get_rank(), c.get_size()) == (2, 4)
    assert c.get_name() == "acc"
    assert c.get_backend() == "fake"
    assert c.get_device() == torch.device("cpu")
    assert c.get_options().timeout == timedelta(seconds=7)
    assert c.get_ranks() == [0, 1, 2, 3]
    c.finalize()
    with pytest.raises(RuntimeError, match="finalized"):
        c.barrier(False)
    with pytest.raises(RuntimeError, match="already finalized"):
        c.finalize()


def test_rank_validation():
    c = _fake("rv", hints={"fake_size": "2"})
    t = torch.zeros(2)
    with pytest.raises(RuntimeError, match="outside"):
        c.send(t, 5, False)
    with pytest.raises(RuntimeError, match="outside"):
        c.broadcast(t, -1, False)
    c.finalize()


def test_env_defaults(monkeypatch):
    monkeypatch.setenv("TORCHCOMM_ABORT_ON_ERROR", "0")
    monkeypatch.setenv("TORCHCOMM_TIMEOUT_SECONDS", "12.5")
    o = tc.CommOptions()
    assert o.abort_process_on_timeout_or_error is False
    assert o.timeout == timedelta(seconds=12.5)
    monkeypatch.setenv("TORCHCOMM_ABORT_ON_ERROR", "maybe")
    with pytest.raises(RuntimeError):
        tc.CommOptions()


def test_query_ranksize_order(monkeypatch):
    for k in ("TORCHCOMM_RANK", "TORCHCOMM_SIZE", "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE",
              "PMI_RANK", "PMI_SIZE", "RANK", "WORLD_SIZE", "TORCHCOMM_BOOTSTRAP_RANKSIZE_QUERY_METHOD"):
        monkeypatch.delenv(k, raising=False)
    with pytest.raises(RuntimeError, match="cannot determine rank"):
        _comms._query_ranksize()
    monkeypatch.setenv("RANK", "3")
    monkeypatch.setenv("WORLD_SIZE", "8")
    assert _comms._query_ranksize() == (3, 8)
    monkeypatch.setenv("TORCHCOMM_RANK", "1")
    monkeypatch.setenv("TORCHCOMM_SIZE", "2")
    assert _comms._query_ranksize() == (1, 2)
    monkeypatch.setenv("TORCHCOMM_BOOTSTRAP_RANKSIZE_QUERY_METHOD", "torchrun")
    assert _comms._query_ranksize() == (3, 8)


def test_op_ids_are_global_and_increasing():
    a, b = _fake("ida"), _fake("idb")
    ids = []
    a.register_pre_hook(lambda op, i, args: ids.append(i))
    b.register_pre_hook(lambda op, i, args: ids.append(i))
    t = torch.ones(3)
    a.all_reduce(t, tc.ReduceOp.SUM, False)
    b.all_reduce(t, tc.ReduceOp.SUM, False)
    a.barrier(False)
    assert ids == sorted(ids) and len(set(ids)) == 3
    a.finalize()
    b.finalize()


def test_hooks_typed_args_and_removal():
    c = _fake("hooks", hints={"fake_size": "2"})
    pre, post = [], []
    h1 = c.register_pre_hook(lambda op, i, a: pre.append((op, a)))
    h2 = c.register_post_hook(lambda i, a: post.append(a))
    t = torch.arange(4.0)
    out = torch.zeros(8)
    c.all_reduce(t, tc.ReduceOp.MAX, True)
    c.all_gather_single(out, t, False)
    c.send(t, 1, False)
    c.all_to_all_v_single(torch.zeros(4), t, [2, 2], [1, 3], False)
    ops = [p[0] for p in pre]
    assert ops == [tc.OpName.all_reduce, tc.OpName.all_gather_single, tc.OpName.send, tc.OpName.all_to_all_v_single]
    ar = pre[0][1]
    assert type(ar).__name__ == "AllReducePreHookArgs"
    assert ar.tensor is t and ar.async_op is True and ar.op == tc.RedOpType.MAX
    ag = pre[1][1]
    assert ag.input is t and ag.output is out and ag.async_op is False
    assert pre[2][1].peer == 1
    assert pre[3][1].input_split_sizes == [1, 3] and pre[3][1].output_split_sizes == [2, 2]
    assert type(post[0]).__name__ == "AllReducePostHookArgs"
    assert isinstance(post[0], tc.CollectivePostHookArgs)
    h1.remove()
    h1.remove()  # idempotent
    c.barrier(False)
    assert len(pre) == 4 and len(post) == 5
    h2.remove()
    fin = []
    c.register_pre_hook(lambda op, i, a: fin.append((op, i)))
    c.finalize()
    assert fin == [(tc.OpName.finalize, 2**64 - 1)]


def test_split_semantics():
    c = _fake("parent", hints={"fake_rank": "1", "fake_size": "4"})
    assert c.split([], "none") is None
    with pytest.raises(RuntimeError, match="not in the non-empty"):
        c.split([0, 2], "bad")
    with pytest.raises(RuntimeError, match="twice"):
        c.split([1, 1], "dup")
    with pytest.raises(RuntimeError, match="outside"):
        c.split([1, 9], "oob")
    child = c.split([3, 1], "kid")
    assert child.get_size() == 2 and child.get_rank() == 1
    assert child.get_ranks() == [3, 1]  # global ranks of the members
    child.finalize()
    c.finalize()


def test_deepcopy_is_identity():
    c = _fake("copy")
    assert copy.copy(c) is c
    assert copy.deepcopy(c) is c
    holder = {"comm": c, "x": torch.ones(2)}
    dup = copy.deepcopy(holder)
    assert dup["comm"] is c and dup["x"] is not holder["x"]
    c.finalize()


def test_reduce_op_api():
    assert tc.ReduceOp.SUM.type == tc.RedOpType.SUM
    assert tc.ReduceOp.AVG == tc.ReduceOp(tc.RedOpType.AVG)
    p = tc.ReduceOp.PREMUL_SUM(0.5)
    assert p.type == tc.RedOpType.PREMUL_SUM and p.factor == 0.5
    pt = tc.ReduceOp.PREMUL_SUM(torch.tensor([2.0]))
    assert torch.equal(pt.factor, torch.tensor([2.0]))


def test_work_state_machine_and_hooks():
    w = _comms._completed_work()
    assert w.is_completed() and w.status() == tc.WorkStatus.COMPLETED
    fired = []
    w.register_start_hook(lambda: fired.append("start"))  # already started: fires now
    w.register_end_hook(lambda: fired.append("end"))
    assert fired == ["start", "end"]
    w.register_wait_pre_hook(lambda: fired.append("pre"))
    w.register_wait_post_hook(lambda: fired.append("post"))
    w.wait()
    assert fired[-2:] == ["pre", "post"]
    w._set_status(tc.WorkStatus.TIMEDOUT)
    with pytest.raises(RuntimeError, match="timed out"):
        w.wait()


def test_batch_send_recv_records_ops():
    c = _fake("batch", hints={"fake_size": "2"})
    b = c.batch_op_create()
    t1, t2 = torch.ones(2), torch.zeros(2)
    b.send(t1, 1)
    b.recv(t2, 1)
    assert [op.type for op in b.ops] == [tc.P2POpType.SEND, tc.P2POpType.RECV]
    seen = []
    h = c.register_pre_hook(lambda op, i, a: seen.append((op, len(a.ops))))
    b.issue(True).wait()
    h.remove()
    assert seen == [(tc.OpName.batch_op_issue, 2)]
    assert "batch_op_issue" in c.get_backend_impl().calls
    c.finalize()


def test_per_op_option_classes():
    o = tc.AllReduceOptions()
    o.hints = {"k": "v"}
    o.timeout = timedelta(seconds=3)
    assert o.hints == {"k": "v"} and o.timeout == timedelta(seconds=3)
    assert issubclass(tc.BarrierOptions, tc.OpOptions)


class _Work:
    def __init__(self):
        self.waited = False

    def wait(self):
        self.waited = True


class _PyBackend(tc.TorchCommBackend):
    last_work = None

    def __init__(self):
        super().__init__()
        self._rank, self._size, self._name = 0, 1, ""

    def init(self, device, name, options):
        self._name = name

    def finalize(self):
        pass

    def get_rank(self):
        return self._rank

    def get_size(self):
        return self._size

    def get_backend_name(self):
        return "pyb"

    def get_comm_name(self):
        return self._name

    def all_reduce(self, tensor, op, async_op):
        if op.type == tc.RedOpType.SUM:
            tensor.mul_(3)
        if async_op:
            _PyBackend.last_work = _Work()
            return _PyBackend.last_work
        return None

    def split(self, ranks, name, options):
        b = _PyBackend()
        b._size, b._name = len(ranks), name
        return b

    def set_timeout(self, timeout):
        self.timeout = timeout


def test_python_backend():
    tc.register_backend("pyb", _PyBackend)
    assert tc.is_backend_built("pyb")
    c = tc.new_comm("pyb", torch.device("cpu"), name="py1")
    assert c.get_backend() == "pyb" and c.get_name() == "py1"
    t = torch.ones(2)
    w = c.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((2,), 3.0)) and w.is_completed()
    w = c.all_reduce(t, tc.ReduceOp.SUM, True)
    assert not _PyBackend.last_work.waited
    w.wait()
    assert _PyBackend.last_work.waited and w.is_completed()
    with pytest.raises(RuntimeError, match="does not implement"):
        c.barrier(False)
    kid = c.split([0], "kid")
    assert kid.get_size() == 1 and kid.get_name() == "kid"
    c.set_timeout(timedelta(seconds=2))
    assert c.get_backend_impl().timeout == timedelta(seconds=2)
    kid.finalize()
    c.finalize()


def test_dynamic_backend_env_missing_symbol(tmp_path, monkeypatch):
    bogus = tmp_path / "libnothing.so"
    bogus.write_bytes(b"not an elf")
    monkeypatch.setenv("TORCHCOMMS_BACKEND_LIB_PATH_DYNX", str(bogus))
    with pytest.raises(RuntimeError, match="cannot load backend library"):
        tc.new_comm("dynx", torch.device("cpu"), name="d")


def test_health_flag():
    _comms._health_reset()
    assert tc.healthy()
    _comms._health_mark_unhealthy("watchdog saw a timeout")
    assert not tc.healthy() and "timeout" in _comms._health_reason()
    _comms._health_reset()


def test_reconfigure_rejected_without_support():
    tc.register_backend("pyb2", _PyBackend)
    with pytest.raises(RuntimeError, match="does not support enable_reconfigure"):
        tc.new_comm("pyb2", torch.device("cpu"), name="r", enable_reconfigure=True)


def test_cuda_work_state_machine_with_scripted_runtime():
    """The watchdog's view of a stream-ordered work object, driven through a fake CUDA runtime (no GPU):
    start event seen -> INPROGRESS, end event -> COMPLETED, no end event within the timeout -> TIMEDOUT,
    a failing query -> ERROR; the work destroys its two events."""
    from torchcomms_b200 import _comms

    ok, not_ready, launch_failure = 0, 600, 719
    seen, err, destroyed = _comms._scripted_work_polls([not_ready, ok], [not_ready, not_ready, ok], 1000, 10, 5)
    assert seen == ["NOT_STARTED", "INPROGRESS", "INPROGRESS", "COMPLETED", "COMPLETED"] and err == "" and destroyed == 2
    seen, err, _ = _comms._scripted_work_polls([ok], [not_ready], 50, 20, 6)
    assert seen[0] == "INPROGRESS" and seen[-1] == "TIMEDOUT" and "50 ms" in err
    assert seen.index("TIMEDOUT") == 3  # 60 ms after the start was seen
    seen, err, _ = _comms._scripted_work_polls([ok], [not_ready, launch_failure], 1000, 10, 3)
    assert seen == ["INPROGRESS", "ERROR", "ERROR"] and "end event" in err
    seen, err, _ = _comms._scripted_work_polls([launch_failure], [not_ready], 1000, 10, 2)
    assert seen == ["ERROR", "ERROR"] and "start event" in err
    # a work that never starts (queued behind other work) does not time out
    seen, _, _ = _comms._scripted_work_polls([not_ready], [not_ready], 10, 50, 4)
    assert seen == ["NOT_STARTED"] * 4


def test_dynamic_backend_loaded_from_shared_library(tmp_path, monkeypatch):
    """An out-of-tree backend: compiled here into its own .so, found through the environment, loaded with
    dlopen, checked against the ABI string, and driven through the ordinary communicator API."""
    import os
    import subprocess
    import sysconfig

    from torch.utils.cpp_extension import include_paths

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "torchcomms_b200")
    lib = tmp_path / "libsample_backend.so"
    cmd = ["/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++", "-shared", "-fPIC", "-std=c++17", "-O1",
           "-D_GLIBCXX_USE_CXX11_ABI=1", "-I", os.path.join(pkg, "csrc")]
    for inc in include_paths(device_type="cuda") + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]:
        cmd += ["-isystem", inc]
    cmd += [os.path.join(root, "tests", "data", "sample_backend.cpp"), "-o", str(lib), "-L", pkg, "-l:_comms.so",
            f"-Wl,-rpath,{pkg}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-2000:]
    monkeypatch.setenv("TORCHCOMMS_BACKEND_LIB_PATH_SAMPLE", str(lib))
    c = tc.new_comm("sample", torch.device("cpu"), name="dyn")
    assert c.get_backend() == "sample" and c.get_size() == 1
    t = torch.zeros(3)
    c.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.ones(3))  # the library's override ran
    c.barrier(False)
    c.finalize()


def test_configuration_tiers_env_over_file_over_default(tmp_path, monkeypatch):
    """Environment > configuration file > built-in default (comms/utils/cvars/README.md:10-19)."""
    import torchcomms_b200 as tc

    conf = tmp_path / "b200comms.conf"
    conf.write_text("# site defaults\nTORCHCOMM_TIMEOUT_SECONDS = 7   # seconds\nTORCHCOMM_ABORT_ON_ERROR=0\nnot a setting\n")
    monkeypatch.setenv("B200COMMS_CONF_FILE", str(conf))
    monkeypatch.delenv("TORCHCOMM_TIMEOUT_SECONDS", raising=False)
    monkeypatch.delenv("TORCHCOMM_ABORT_ON_ERROR", raising=False)
    tc.reload_config()
    try:
        o = tc.CommOptions()
        assert o.timeout.total_seconds() == 7 and o.abort_process_on_timeout_or_error is False
        k = tc.knobs()
        assert k["TORCHCOMM_TIMEOUT_SECONDS"] == ("7", "file") and k["TORCHCOMM_ABORT_ON_ERROR"] == ("0", "file")
        monkeypatch.setenv("TORCHCOMM_TIMEOUT_SECONDS", "11")
        assert tc.CommOptions().timeout.total_seconds() == 11
        assert tc.knobs()["TORCHCOMM_TIMEOUT_SECONDS"] == ("11", "env")
        conf.write_text("")
        monkeypatch.delenv("TORCHCOMM_TIMEOUT_SECONDS")
        tc.reload_config()
        assert tc.CommOptions().timeout.total_seconds() == 600
        assert tc.knobs()["TORCHCOMM_TIMEOUT_SECONDS"][1] == "default"
    finally:
        monkeypatch.delenv("B200COMMS_CONF_FILE")
        tc.reload_config()


def test_comm_stats_hook_counts_calls_bytes_and_completions():
    import time

    import torchcomms_b200 as tc
    from torchcomms_b200.hooks import CommStatsHook

    comm = tc.new_comm("fake", torch.device("cpu"), name="stats")
    stats = CommStatsHook()
    stats.register_with_comm(comm)
    assert stats.is_enabled()
    t = torch.ones(1024)
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    comm.all_reduce(t, tc.ReduceOp.SUM, True).wait()
    out = torch.empty(3000)
    comm.all_gather_single(out, torch.ones(3000), False)
    deadline = time.time() + 5
    while time.time() < deadline and sum(s["completed"] for s in stats.snapshot().values()) < 3:
        time.sleep(0.01)
    snap = stats.snapshot()
    ar, ag = snap["all_reduce"], snap["all_gather_single"]
    assert (ar["calls"], ar["bytes"], ar["async_calls"], ar["completed"]) == (2, 8192, 1, 2)
    assert ar["size_histogram"] == {"4KiB": 2} and ag["size_histogram"] == {"16KiB": 1} and ag["bytes"] == 12000
    assert ar["busy_ms"] >= 0 and "all_reduce" in stats.report()
    stats.unregister()
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    assert stats.snapshot()["all_reduce"]["calls"] == 2 and not stats.is_enabled()
    stats.reset()
    assert stats.snapshot() == {}
    comm.finalize()


def test_comm_dump_and_comm_dump_all():
    import gc

    import torchcomms_b200 as tc

    a = tc.new_comm("fake", torch.device("cpu"), name="dump_a")
    b = tc.new_comm("fake", torch.device("cpu"), name="dump_b")
    one = a.comm_dump()
    assert one["name"] == "dump_a" and one["backend"] == "fake" and one["rank"] == "0" and one["size"] == "1"
    everything = tc.comm_dump_all()
    assert {"dump_a", "dump_b"} <= set(everything) and everything["dump_b"]["finalized"] == "0"
    a.finalize()
    assert tc.comm_dump_all()["dump_a"]["finalized"] == "1"
    del a
    gc.collect()
    assert "dump_a" not in tc.comm_dump_all() and "dump_b" in tc.comm_dump_all()
    b.finalize()


def test_flight_recorder_dumps_on_abort(tmp_path, monkeypatch):
    """The recorder's abort hook writes the ring to ``<prefix><rank>`` (hooks/fr/tests/py/FlightRecorderAbortTest.py)."""
    import json

    import torchcomms_b200 as tc
    from torchcomms_b200.hooks import fr

    monkeypatch.setenv("TORCHCOMM_FR_DUMP_TEMP_FILE", str(tmp_path / "fr_trace_"))
    comm = tc.new_comm("fake", torch.device("cpu"), name="fr_abort", abort_process_on_timeout_or_error=False)
    rec = fr.FlightRecorderHook(8)
    rec.register_with_comm(comm)
    for _ in range(3):
        comm.all_reduce(torch.ones(4), tc.ReduceOp.SUM, False)
    comm.barrier(False)
    assert rec.size() == 4 and rec.capacity() == 8
    comm.abort()
    dump = tmp_path / "fr_trace_0"
    assert dump.exists()
    data = json.loads(dump.read_text())
    entries = data["entries"] if isinstance(data, dict) else data
    names = [e.get("profiling_name", e.get("op", "")) for e in entries]
    assert len(entries) == 4 and any("all_reduce" in n for n in names) and any("barrier" in n for n in names)
    # the ring keeps the newest entries
    rec.reset()
    assert rec.size() == 0


def test_trainer_iteration_tags_recorder_entries_and_dumps():
    import json

    import torchcomms_b200 as tc
    from torchcomms_b200.hooks import fr

    comm = tc.new_comm("fake", torch.device("cpu"), name="iter_tag")
    rec = fr.FlightRecorderHook(8)
    rec.register_with_comm(comm)
    tc.set_trainer_iteration(41)
    comm.all_reduce(torch.ones(2), tc.ReduceOp.SUM, False)
    tc.set_trainer_iteration(42)
    comm.barrier(False)
    assert tc.trainer_iteration() == 42
    assert [e["iteration"] for e in rec.entries()] == [41, 42]
    dumped = json.loads(rec.dump_json())
    entries = dumped["entries"] if isinstance(dumped, dict) else dumped
    assert [e["iteration"] for e in entries] == [41, 42]
    assert tc.comm_dump_all()["iter_tag"]["iteration"] == "42"
    tc.set_trainer_iteration(-1)
    comm.finalize()


class _FullPyBackend(_PyBackend):
    """A single-rank Python backend that implements every overridable operation and logs the calls."""

    def __init__(self):
        super().__init__()
        self.calls = []

    def get_backend_name(self):
        return "pyfull"

    def _done(self, name, async_op):
        self.calls.append(name)
        return _Work() if async_op else None

    def send(self, tensor, dst, async_op):
        return self._done("send", async_op)

    def recv(self, tensor, src, async_op):
        tensor.fill_(7)
        return self._done("recv", async_op)

    def broadcast(self, tensor, root, async_op):
        return self._done("broadcast", async_op)

    def reduce(self, tensor, root, op, async_op):
        return self._done("reduce", async_op)

    def all_gather(self, tensor_list, tensor, async_op):
        tensor_list[0].copy_(tensor)
        return self._done("all_gather", async_op)

    def all_gather_single(self, output, input, async_op):
        output.copy_(input)
        return self._done("all_gather_single", async_op)

    def reduce_scatter_single(self, output, input, op, async_op):
        output.copy_(input)
        return self._done("reduce_scatter_single", async_op)

    def all_to_all_single(self, output, input, async_op):
        output.copy_(input)
        return self._done("all_to_all_single", async_op)

    def barrier(self, async_op):
        return self._done("barrier", async_op)

    def scatter(self, output, input_list, root, async_op):
        output.copy_(input_list[0])
        return self._done("scatter", async_op)

    def gather(self, output_list, input, root, async_op):
        output_list[0].copy_(input)
        return self._done("gather", async_op)


def test_python_backend_every_operation_reaches_the_override():
    """test_python_backend.py of the reference: each collective lands in the Python method, hooks included."""
    tc.register_backend("pyfull", _FullPyBackend)
    c = tc.new_comm("pyfull", torch.device("cpu"), name="pyfull1")
    impl = c.get_backend_impl()
    seen = []
    handle = c.register_pre_hook(lambda op, op_id, args: seen.append(op.name))
    t, out = torch.arange(4.0), torch.zeros(4)
    c.send(t, 0, False)
    c.recv(out, 0, False)
    assert torch.equal(out, torch.full((4,), 7.0))
    c.broadcast(t, 0, False)
    c.reduce(t, 0, tc.ReduceOp.SUM, False)
    lst = [torch.zeros(4)]
    c.all_gather(lst, t, False)
    assert torch.equal(lst[0], t)
    c.all_gather_single(out, t, False)
    c.reduce_scatter_single(out, t, tc.ReduceOp.SUM, False)
    c.all_to_all_single(out, t, False)
    c.barrier(False)
    c.scatter(out, [t], 0, False)
    c.gather([out], t, 0, False)
    w = c.barrier(True)
    w.wait()
    expected = ["send", "recv", "broadcast", "reduce", "all_gather", "all_gather_single", "reduce_scatter_single",
                "all_to_all_single", "barrier", "scatter", "gather", "barrier"]
    assert impl.calls == expected and seen == expected
    handle.remove()
    # two communicators of the same Python backend are independent objects
    c2 = tc.new_comm("pyfull", torch.device("cpu"), name="pyfull2")
    c2.barrier(False)
    assert c2.get_backend_impl().calls == ["barrier"] and len(impl.calls) == len(expected)
    c2.finalize()
    c.finalize()


def test_window_api_rules_on_the_fake_backend():
    """Window rules without a GPU (WindowRmaTest.py, RegisterTensorTest.py, test_copy.py of the reference):
    one registration at a time, bounds and dtype of put, signal / wait pairing, deepcopy clones the tensor."""
    import copy

    c = tc.new_comm("fake", torch.device("cpu"), name="win")
    w = c.new_window()
    assert w.get_tensor() is None and w.get_size() == 0
    t = torch.zeros(16)
    w.tensor_register(t)
    assert w.get_size() == 64 and w.shape == [16] and w.dtype == torch.float32
    with pytest.raises(RuntimeError, match="already"):
        w.tensor_register(torch.zeros(4))
    with pytest.raises(RuntimeError, match="contiguous"):
        c.new_window().tensor_register(torch.zeros(4, 4).t())
    w.put(torch.arange(4.0), 0, 8, False)
    assert torch.equal(t[8:12], torch.arange(4.0)) and float(t[:8].sum()) == 0
    w.put(torch.ones(4), 0, 12, True).wait()
    with pytest.raises(RuntimeError, match="outside the window"):
        w.put(torch.ones(4), 0, 13, False)
    with pytest.raises(RuntimeError, match="dtype"):
        w.put(torch.ones(4, dtype=torch.int32), 0, 0, False)
    with pytest.raises(RuntimeError, match="outside"):
        w.put(torch.ones(1), 1, 0, False)                      # no such rank
    w.signal(0, False)
    w.wait_signal(0, False)
    with pytest.raises(RuntimeError, match="wait forever"):
        w.wait_signal(0, False)
    assert w.map_remote_tensor(0).data_ptr() == t.data_ptr()
    assert w.get_attr(0).access_type == tc.TorchCommWinAccessType.WIN_ACCESS_TYPE_UNIFIED
    # copy is the same window; deepcopy clones window and tensor and records the tensor in the memo
    assert copy.copy(w) is w
    memo = {}
    w2 = copy.deepcopy(w, memo)
    assert w2 is not w and torch.equal(w2.get_tensor(), t) and w2.get_tensor().data_ptr() != t.data_ptr()
    w2.put(torch.full((2,), 9.0), 0, 0, False)
    assert float(t[0]) == 0.0 and float(w2.get_tensor()[0]) == 9.0
    w.tensor_deregister()
    with pytest.raises(RuntimeError):
        w.tensor_deregister()
    w.tensor_register(torch.zeros(4))                          # a window can be registered again after deregistration
    pre_made = c.new_window(torch.ones(3))
    assert pre_made.get_size() == 12
    with pytest.raises(RuntimeError, match="CUDA backend"):
        w.get_device_window()
    c.finalize()


def test_type_stubs_match_the_bindings():
    """torchcomms_b200/_comms.pyi is what the generator writes from the module as built (rerun
    ``python -m torchcomms_b200.utils.stubgen`` after changing a binding)."""
    import ast
    import os

    from torchcomms_b200.utils import stubgen

    if os.environ.get("TORCHCOMMS_PATCH_FOR_COMPILE") == "1":
        pytest.skip("communicator methods are wrapped for tracing in this process: their bound signatures are hidden")
    text = stubgen.generate()
    ast.parse(text)
    assert open(stubgen.stub_path()).read() == text
    for name in ("class TorchComm:", "class CudaBackend:", "def register_backend(", "class transport:", "def seq_heads_exchange("):
        assert name in text, name


def test_hooks_namespace_accepts_the_reference_spellings(tmp_path):
    """``hooks.FlightRecorderHook`` and ``hooks.clog(output=..., events=[...])`` as in the reference's hooks package,
    next to ``hooks.fr.FlightRecorderHook`` / ``hooks.clog.ClogHook``."""
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")
    import torchcomms_b200 as tc
    from torchcomms_b200 import hooks

    assert hooks.FlightRecorderHook is hooks.fr.FlightRecorderHook and hooks.clog.ClogHook is hooks.ClogHook
    path = tmp_path / "clog.log"
    logger = hooks.clog(output=str(path), events=["ALL"])
    comm = tc.new_comm("fake", torch.device("cpu"), name="hooks_ns")
    logger.register_with_comm(comm)
    comm.all_reduce(torch.ones(2), tc.ReduceOp.SUM, False)
    comm.finalize()
    logger.unregister()
    lines = path.read_text().splitlines()
    assert lines[0].startswith("V|") and any(ln.startswith("SIG|") and "all_reduce" in ln for ln in lines)
    with pytest.raises(ValueError):
        hooks.clog(output="", events=["sometimes"])
    # the recorder's constructor and dump take the reference's arguments
    os.environ["TORCHCOMM_FR_DUMP_TEMP_FILE"] = str(tmp_path / "fr_")
    rec = hooks.FlightRecorderHook(max_entries=16, isolated=True)
    assert rec.is_enabled() and rec.capacity() == 16
    comm2 = tc.new_comm("fake", torch.device("cpu"), name="hooks_fr")
    rec.register_with_comm(comm2)
    comm2.all_reduce(torch.ones(2), tc.ReduceOp.SUM, False)
    path2 = rec.dump_file(0, include_completed=True)
    assert path2 == str(tmp_path / "fr_0") and "all_reduce" in open(path2).read()
    assert "all_reduce" not in open(rec.dump_file(0, include_completed=False)).read()
    rec.unregister()
    comm2.finalize()
    del os.environ["TORCHCOMM_FR_DUMP_TEMP_FILE"]


def test_window_nvlink_address_on_a_cpu_window():
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")
    comm = tc.new_comm("fake", torch.device("cpu"), name="win_addr")
    win = comm.new_window()
    buf = torch.zeros(8)
    win.tensor_register(buf)
    assert win.get_nvlink_address(0) == buf.data_ptr() and win.get_nvlink_address(0, 16) == buf.data_ptr() + 16
    with pytest.raises(ValueError):
        win.get_nvlink_address(0, 1000)
    win.tensor_deregister()
    comm.finalize()


def test_reference_spellings_of_options_and_wrapper():
    """``ReconfigureOptions.init_handles`` (list keeps the order, set sorts at use) and ``_BackendWrapper.get_mem_allocator``."""
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")
    o = tc.ReconfigureOptions(1, ["b", "a"])
    assert o.init_handles == ["b", "a"] == o.handles
    o.init_handles = {"z", "y"}
    assert sorted(o.init_handles) == ["y", "z"]
    comm = tc.new_comm("fake", torch.device("cpu"), name="bw_alloc")
    wrapper = tc._BackendWrapper(comm)
    assert wrapper.get_comm() is comm or wrapper.get_comm().get_name() == "bw_alloc"
    with pytest.raises(RuntimeError, match="no device memory allocator"):
        wrapper.get_mem_allocator()
    comm.set_timeout(timeout=timedelta(seconds=5))
    comm.set_hints(hints={"k": "v"})
    # the options a backend is given carry the communicator's name, for the child of a split its own
    sub = comm.split([0], "bw_alloc_child")
    assert comm.get_options().name == "bw_alloc" and sub.get_options().name == "bw_alloc_child"
    assert tc.CommOptions().name == ""
    sub.finalize()
    comm.finalize()


def test_subpackages_resolve_as_attributes():
    """``import torchcomms_b200`` is enough for ``tc.hooks`` / ``tc.objcol`` / ... (the reference imports them eagerly)."""
    import subprocess
    import sys
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import torchcomms_b200 as tc\n"
            "assert tc.hooks.NanCheckHook and tc.objcol.all_gather_object and tc.checkpoint.checkpoint_prepare\n"
            "try:\n    tc.no_such_thing\nexcept AttributeError:\n    print('ok')\n")
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, PYTHONPATH=root, RANK="0", WORLD_SIZE="1"),
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stderr[-2000:]


def test_new_comm_accepts_the_name_in_third_position():
    """``new_comm(backend, device, "name")`` as the reference's binding takes it."""
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")
    comm = tc.new_comm("fake", torch.device("cpu"), "third_positional")
    assert comm.get_name() == "third_positional" and comm.get_options().name == "third_positional"
    comm.finalize()
    with pytest.raises(TypeError):
        tc.new_comm("fake", torch.device("cpu"), "a", name="b")
    with pytest.raises(ModuleNotFoundError, match="failed to find backend"):
        tc.new_comm("invalid", torch.device("cpu"), "my_comm")


def test_python_backend_instance_is_what_get_backend_impl_returns():
    """A backend class registered from Python: ``get_backend_impl()`` gives its instance, ``set_timeout`` reaches it,
    and ``init`` sees the communicator's name in the options."""
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")

    class Minimal(tc.TorchCommBackend):
        def __init__(self):
            super().__init__()
            self.timeout = None

        def init(self, device, name, options):
            self.name, self.options_name = name, options.name

        def finalize(self):
            pass

        def get_rank(self):
            return 0

        def get_size(self):
            return 1

        def get_backend_name(self):
            return "minimal_py"

        def get_comm_name(self):
            return self.name

        def set_timeout(self, timeout):
            self.timeout = timeout

        def all_reduce(self, tensor, op, async_op):
            tensor.mul_(2)
            return None

    tc.register_backend("minimal_py", Minimal)
    comm = tc.new_comm("minimal_py", torch.device("cpu"), name="py_impl")
    impl = comm.get_backend_impl()
    assert isinstance(impl, Minimal) and impl is comm.unsafe_get_backend() and impl.options_name == "py_impl"
    comm.set_timeout(timedelta(milliseconds=1234))
    assert impl.timeout == timedelta(milliseconds=1234)
    t = torch.ones(2)
    work = comm.all_reduce(t, tc.ReduceOp.SUM, async_op=False)
    work.wait()
    assert work.is_completed() and torch.equal(t, torch.full((2,), 2.0))
    comm.finalize()
