"""Multi-process CPU integration tests on the ``gloo`` backend.

Covers the CPU configuration of the benchmark set: world_size=2, fp32 tensors
of 1,048,576 elements ~N(0,1) seeded by rank; all_reduce SUM, all_gather,
reduce_scatter, all_to_all_single (equal splits), broadcast from rank 0 and a
send/recv ring, each checked against a torch reference.  A second battery on
4 ranks covers the remaining operations, reduce-op variants, split, object
collectives and the c10d wrapper.

Test matrix modelled on comms/torchcomms/tests/integration/py/*Test.py.
"""
from datetime import timedelta

import os

import pytest
import torch

from tests.mp_util import run_ranks

N_ELEMS = 1_048_576


def _rank_tensor(rank: int, n: int = N_ELEMS) -> torch.Tensor:
    g = torch.Generator().manual_seed(1234 + rank)
    return torch.randn(n, generator=g, dtype=torch.float32)


def _baseline_config_worker(rank, world):
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="baseline_cfg", timeout=timedelta(seconds=60))
    assert comm.get_rank() == rank and comm.get_size() == world
    everyone = [_rank_tensor(r) for r in range(world)]
    mine = everyone[rank]

    # all_reduce SUM, sync and async
    for async_op in (False, True):
        t = mine.clone()
        w = comm.all_reduce(t, tc.ReduceOp.SUM, async_op)
        w.wait()
        torch.testing.assert_close(t, sum(everyone), rtol=1e-5, atol=1e-5)

    # all_gather (list) and all_gather_single
    outs = [torch.empty(N_ELEMS) for _ in range(world)]
    comm.all_gather(outs, mine, False)
    for r in range(world):
        assert torch.equal(outs[r], everyone[r])
    flat = torch.empty(world * N_ELEMS)
    comm.all_gather_single(flat, mine, True).wait()
    assert torch.equal(flat, torch.cat(everyone))

    # reduce_scatter (list) and reduce_scatter_single
    chunk = N_ELEMS // world
    out = torch.empty(chunk)
    comm.reduce_scatter(out, list(mine.view(world, chunk).unbind(0)), tc.ReduceOp.SUM, False)
    expect = sum(e.view(world, chunk)[rank] for e in everyone)
    torch.testing.assert_close(out, expect, rtol=1e-5, atol=1e-5)
    out2 = torch.empty(chunk)
    comm.reduce_scatter_single(out2, mine, tc.ReduceOp.SUM, True).wait()
    torch.testing.assert_close(out2, expect, rtol=1e-5, atol=1e-5)

    # all_to_all_single with equal splits
    recv = torch.empty(N_ELEMS)
    comm.all_to_all_single(recv, mine, False)
    expect = torch.cat([e.view(world, chunk)[rank] for e in everyone])
    assert torch.equal(recv, expect)

    # broadcast from rank 0
    b = mine.clone()
    comm.broadcast(b, 0, False)
    assert torch.equal(b, everyone[0])

    # send/recv ring
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    got = torch.empty(N_ELEMS)
    if rank % 2 == 0:
        comm.send(mine, nxt, False)
        comm.recv(got, prv, False)
    else:
        comm.recv(got, prv, False)
        comm.send(mine, nxt, False)
    assert torch.equal(got, everyone[prv])

    comm.barrier(False)
    comm.finalize()


def test_baseline_cpu_config_world2():
    run_ranks(_baseline_config_worker, 2)


def _wide_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import objcol

    comm = tc.new_comm("gloo", torch.device("cpu"), name="wide", timeout=timedelta(seconds=60))
    ones = torch.ones(8) * (rank + 1)
    tri = world * (world + 1) // 2

    # reduce ops
    t = ones.clone(); comm.all_reduce(t, tc.ReduceOp.AVG, False)
    torch.testing.assert_close(t, torch.full((8,), tri / world))
    t = ones.clone(); comm.all_reduce(t, tc.ReduceOp.MAX, False)
    assert torch.equal(t, torch.full((8,), float(world)))
    t = ones.clone(); comm.all_reduce(t, tc.ReduceOp.MIN, False)
    assert torch.equal(t, torch.ones(8))
    t = ones.clone(); comm.all_reduce(t, tc.ReduceOp.PRODUCT, False)
    import math
    assert torch.equal(t, torch.full((8,), float(math.factorial(world))))
    t = ones.clone(); comm.all_reduce(t, tc.ReduceOp.PREMUL_SUM(0.5), False)
    torch.testing.assert_close(t, torch.full((8,), tri * 0.5))
    t = ones.clone(); comm.all_reduce(t, tc.ReduceOp.PREMUL_SUM(torch.tensor([2.0])), False)
    torch.testing.assert_close(t, torch.full((8,), tri * 2.0))
    ti = torch.full((4,), 1 << rank, dtype=torch.int32); comm.all_reduce(ti, tc.ReduceOp.BOR, False)
    assert torch.equal(ti, torch.full((4,), (1 << world) - 1, dtype=torch.int32))
    ti = torch.full((4,), 7, dtype=torch.int64); comm.all_reduce(ti, tc.ReduceOp.BAND, False)
    assert torch.equal(ti, torch.full((4,), 7, dtype=torch.int64))
    ti = torch.full((4,), rank + 1, dtype=torch.int32); comm.all_reduce(ti, tc.ReduceOp.AVG, False)
    assert torch.equal(ti, torch.full((4,), tri // world, dtype=torch.int32))
    try:
        comm.all_reduce(ones.clone(), tc.ReduceOp.BXOR, False)
        raise AssertionError("bitwise op on floats must raise")
    except RuntimeError as e:
        assert "integral" in str(e)

    # reduce to a root
    t = ones.clone(); comm.reduce(t, 1, tc.ReduceOp.SUM, False)
    if rank == 1:
        assert torch.equal(t, torch.full((8,), float(tri)))

    # all_gather_v / reduce_scatter_v with per-rank sizes
    sizes = [r + 1 for r in range(world)]
    outs = [torch.empty(s) for s in sizes]
    comm.all_gather_v(outs, torch.full((sizes[rank],), float(rank)), False)
    for r in range(world):
        assert torch.equal(outs[r], torch.full((sizes[r],), float(r)))
    ins = [torch.full((s,), float(rank + 1)) for s in sizes]
    out = torch.empty(sizes[rank])
    comm.reduce_scatter_v(out, ins, tc.ReduceOp.SUM, True).wait()
    assert torch.equal(out, torch.full((sizes[rank],), float(tri)))

    # all_to_all_v_single: rank r sends (d + 1) rows to destination d
    in_splits = [d + 1 for d in range(world)]
    out_splits = [rank + 1] * world
    src = torch.cat([torch.full((d + 1, 2), float(rank * 10 + d)) for d in range(world)])
    dst = torch.empty(sum(out_splits), 2)
    comm.all_to_all_v_single(dst, src, out_splits, in_splits, False)
    expect = torch.cat([torch.full((rank + 1, 2), float(s * 10 + rank)) for s in range(world)])
    assert torch.equal(dst, expect)

    # all_to_all (lists), scatter, gather, gather_single
    outs = [torch.empty(3) for _ in range(world)]
    comm.all_to_all(outs, [torch.full((3,), float(rank * world + d)) for d in range(world)], False)
    for s in range(world):
        assert torch.equal(outs[s], torch.full((3,), float(s * world + rank)))
    got = torch.empty(2)
    comm.scatter(got, [torch.full((2,), float(r)) for r in range(world)] if rank == 2 else [], 2, False)
    assert torch.equal(got, torch.full((2,), float(rank)))
    outs = [torch.empty(2) for _ in range(world)] if rank == 0 else []
    comm.gather(outs, torch.full((2,), float(rank)), 0, False)
    if rank == 0:
        for r in range(world):
            assert torch.equal(outs[r], torch.full((2,), float(r)))
    flat = torch.empty(world * 2) if rank == 3 else torch.empty(0)
    comm.gather_single(flat, torch.full((2,), float(rank)), 3, False)
    if rank == 3:
        assert torch.equal(flat, torch.arange(world).repeat_interleave(2).float())

    # batched p2p ring
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    got = torch.empty(5)
    batch = comm.batch_op_create()
    batch.send(torch.full((5,), float(rank)), nxt)
    batch.recv(got, prv)
    batch.issue(True).wait()
    assert torch.equal(got, torch.full((5,), float(prv)))

    # split into even / odd halves; child ranks are positions in the list
    members = [r for r in range(world) if r % 2 == rank % 2]
    sub = comm.split(members, "parity")
    assert sub.get_size() == len(members) and sub.get_rank() == members.index(rank)
    assert sub.get_ranks() == members
    t = torch.ones(4) * (rank + 1)
    sub.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((4,), float(sum(m + 1 for m in members))))
    sub.finalize()
    none = comm.split([] if rank != 0 else [0], "solo")
    assert (none is None) == (rank != 0)
    if none is not None:
        none.finalize()

    # hooks + flight recorder + collective log on a live backend
    fr = tc._comms.hooks.fr.FlightRecorderHook(16)
    fr.register_with_comm(comm)
    clog = tc._comms.hooks.clog.ClogHook()
    clog.register_with_comm(comm)
    w = comm.all_reduce(torch.ones(4), tc.ReduceOp.SUM, True)
    w.wait()
    comm.barrier(False)
    entries = fr.entries()
    assert [e["op"] for e in entries] == ["all_reduce", "barrier"]
    assert entries[0]["state"] == "completed" and entries[0]["input_sizes"] == [[4]]
    import json
    dumped = json.loads(fr.dump_json())
    assert dumped["version"] == "2.10" and len(dumped["entries"]) == 2
    assert dumped["entries"][0]["profiling_name"] == "b200c:all_reduce"
    lines = clog.lines()
    assert any(l.startswith("SIG|") and "all_reduce" in l for l in lines)
    assert sum(l.startswith("Q|") for l in lines) == 2
    assert sum(l.startswith("E|") for l in lines) == 2
    assert sum(l.startswith("W|") for l in lines) == 1
    fr.unregister(); clog.unregister()

    # object collectives
    objs = [None] * world
    objcol.all_gather_object(comm, objs, {"rank": rank, "pad": "x" * rank})
    assert [o["rank"] for o in objs] == list(range(world))
    lst = [("payload", 7)] if rank == 1 else [None]
    objcol.broadcast_object_list(comm, lst, root=1)
    assert lst == [("payload", 7)]
    g = objcol.gather_object(comm, rank * 3, root=2)
    assert (g == [0, 3, 6, 9][:world]) if rank == 2 else (g is None)
    out = [None]
    objcol.scatter_object_list(comm, 0, out, [f"to{r}" for r in range(world)] if rank == 0 else None)
    assert out == [f"to{rank}"]
    if rank == 0:
        objcol.send_object_list(comm, [{"a": 1}, [2, 3]], dst=1)
    elif rank == 1:
        got = [None, None]
        objcol.recv_object_list(comm, got, src=0)
        assert got == [{"a": 1}, [2, 3]]

    comm.barrier(False)
    comm.finalize()


def test_wide_battery_world4():
    run_ranks(_wide_worker, 4, timeout=240)


def _c10d_worker(rank, world):
    import torch.distributed as dist

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="mesh_dp", timeout=timedelta(seconds=60))
    mesh = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("dp",))
    pg = mesh.get_group("dp")
    assert dist.get_rank(pg) == rank and dist.get_world_size(pg) == world
    t = torch.ones(6) * (rank + 1)
    dist.all_reduce(t, group=pg)
    assert torch.equal(t, torch.full((6,), float(world * (world + 1) // 2)))
    out = torch.empty(world * 3)
    dist.all_gather_into_tensor(out, torch.full((3,), float(rank)), group=pg)
    assert torch.equal(out, torch.arange(world).repeat_interleave(3).float())
    rs = torch.empty(2)
    w = dist.reduce_scatter_tensor(rs, torch.arange(world * 2.0), group=pg, async_op=True)
    w.wait()
    assert torch.equal(rs, torch.arange(world * 2.0).view(world, 2)[rank] * world)
    objs = [None] * world
    dist.all_gather_object(objs, {"r": rank}, group=pg)
    assert [o["r"] for o in objs] == list(range(world))
    dist.barrier(group=pg)
    # batched isend/irecv goes through the wrapper's coalescing path
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    got = torch.empty(4)
    ops = [dist.P2POp(dist.isend, torch.full((4,), float(rank)), nxt, group=pg),
           dist.P2POp(dist.irecv, got, prv, group=pg)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    assert torch.equal(got, torch.full((4,), float(prv)))
    # torch.distributed.monitored_barrier() only admits its own gloo backend;
    # the group-level entry point reaches the adapter's implementation.
    pg.monitored_barrier(timedelta(seconds=30))
    comm.finalize()


def test_device_mesh_and_c10d_wrapper_world2():
    run_ranks(_c10d_worker, 2)


def _iface_worker(rank, world):
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="iface")
    t = torch.full((8,), float(rank + 1))
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((8,), 3.0))
    comm.finalize()


@pytest.mark.parametrize("env", [{"TORCHCOMM_GLOO_INTERFACE": "lo"}, {"TORCHCOMM_GLOO_HOSTNAME": "127.0.0.1"}])
def test_gloo_device_selection_by_environment(env):
    run_ranks(_iface_worker, 2, timeout=120, extra_env=env)


def _store_worker(rank, world):
    from torchcomms_b200.utils.store import create_prefix_store, dup_prefix_store

    boot = create_prefix_store("boot", timedelta(seconds=60))
    boot.set(f"hello/{rank}", str(rank))
    assert boot.get(f"hello/{1 - rank}").decode() == str(1 - rank)
    second = dup_prefix_store("second", boot, timedelta(seconds=60))
    second.set(f"k/{rank}", f"v{rank}")
    assert second.get(f"k/{1 - rank}").decode() == f"v{1 - rank}"
    # the two stores are different servers: a key of one is not a key of the other
    assert second.check([f"k/{rank}"]) and not boot.check([f"k/{rank}"])
    assert boot.get("second/dup_store_port").decode().isdigit()
    boot.set(f"bye/{rank}", "1")
    boot.wait([f"bye/{1 - rank}"])


def test_prefix_store_and_duplicate_store():
    run_ranks(_store_worker, 2, timeout=120)


def _objcol_pickle_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import objcol

    comm = tc.new_comm("gloo", torch.device("cpu"), name="objpickle", timeout=timedelta(seconds=60))
    objs = [None] * world
    objcol.all_gather_object(comm, objs, {"rank": rank, "t": torch.arange(rank + 1)})
    assert [o["rank"] for o in objs] == list(range(world)) and torch.equal(objs[1]["t"], torch.arange(2))
    # weights_only refuses arbitrary classes on the torch.save route and accepts plain containers
    lst = [{"a": [1, 2, 3], "w": torch.ones(2)}] if rank == 0 else [None]
    objcol.broadcast_object_list(comm, lst, 0, weights_only=True)
    assert lst[0]["a"] == [1, 2, 3] and torch.equal(lst[0]["w"], torch.ones(2))
    comm.finalize()


@pytest.mark.parametrize("serialization", ["pickle", "torch"])
def test_object_collectives_serialization_modes(serialization):
    run_ranks(_objcol_pickle_worker, 2, timeout=120, extra_env={"TORCHCOMMS_SERIALIZATION": serialization})


def _fr_analyze_worker(rank, world, out_dir):
    """Rank 1 issues a differently-shaped all-gather at step 3 and then stops: the analyzer names both."""
    import json

    import torchcomms_b200 as tc
    from torchcomms_b200.hooks import fr

    os.environ["TORCHCOMM_FR_DUMP_TEMP_FILE"] = os.path.join(out_dir, "trace_")
    comm = tc.new_comm("gloo", torch.device("cpu"), name="fra", timeout=timedelta(seconds=60))
    rec = fr.FlightRecorderHook(32)
    rec.register_with_comm(comm)
    for _ in range(2):
        comm.all_reduce(torch.ones(4), tc.ReduceOp.SUM, False)
    comm.barrier(False)
    # From here on only the recorder sees the operations (fake ones on a second communicator would not
    # share sequence numbers), so the divergence is written into the dumps by hand below.
    path = rec.dump_file(rank)
    data = json.load(open(path))
    last = data["entries"][-1]
    extra = dict(last, collective_seq_id=last["collective_seq_id"] + 1, profiling_name="b200c:all_gather_single",
                 input_sizes=[[8]] if rank == 0 else [[16]], state="started" if rank == 0 else "completed")
    data["entries"].append(extra)
    if rank == 0:                                              # rank 0 went on to one more collective, rank 1 never did
        data["entries"].append(dict(last, collective_seq_id=last["collective_seq_id"] + 2, state="scheduled"))
    json.dump(data, open(path, "w"))
    comm.finalize()


def test_flight_recorder_dumps_are_analyzed_across_ranks(tmp_path):
    import json

    from torchcomms_b200.hooks.fr_analyze import analyze, format_report, main

    run_ranks(_fr_analyze_worker, 2, args=(str(tmp_path),), timeout=120)
    paths = sorted(str(p) for p in tmp_path.glob("trace_*"))
    assert len(paths) == 2
    report = analyze([json.load(open(p)) for p in paths])["fra"]
    assert report["ranks"] == [0, 1]
    assert report["first_mismatch"]["seq"] == 4
    assert report["first_mismatch"]["by_rank"][0]["input_sizes"] == [[8]] and report["first_mismatch"]["by_rank"][1]["input_sizes"] == [[16]]
    assert report["never_issued"] == [{"seq": 5, "op": "b200c:barrier", "ranks_without": [1]}]
    assert report["not_completed"][0]["seq"] == 4 and report["not_completed"][0]["states"] == {0: "started"}
    assert report["progress"][0]["last_completed_collective"] == 3
    text = format_report({"fra": report})
    assert "ranks disagree at collective 4" in text and "never issued by ranks [1]" in text
    assert main(paths) == 0
    # healthy traces say so
    clean = [json.load(open(p)) for p in paths]
    for d in clean:
        d["entries"] = [e for e in d["entries"] if e["collective_seq_id"] <= 3]
    assert "all ranks issued and completed the same collectives" in format_report(analyze(clean))
