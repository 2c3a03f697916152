"""Numerics of the peer-memory kernels on ONE GPU.

Several virtual ranks run side by side in a single cooperative launch
(``_EmuWorld``; blockIdx.y is the rank), which executes exactly the device code
a multi-GPU launch runs - staging, per-block cross-rank barriers, peer reads -
with every "peer" heap living on the same device.  Each result is compared
against a plain PyTorch fp32 reference of the same operation.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

RED = {"sum": 0, "prod": 1, "min": 2, "max": 3}


def _world(n, staging=8 << 20, wait_ms=2000.0):
    from torchcomms_b200 import _comms

    return _comms._EmuWorld(n, staging, wait_ms)


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=1e-5, atol=1e-5)


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)


@pytest.mark.parametrize("nranks", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("algo,count", [(0, 1000), (0, 40_000), (1, 1000), (1, 300_001)])
def test_all_reduce_sum(nranks, dtype, algo, count):
    w = _world(nranks)
    ins = [_rand(count, dtype, 7 + r) for r in range(nranks)]
    outs = [torch.empty_like(t) for t in ins]
    w.all_reduce(ins, outs, RED["sum"], 1.0, algo, 4, 64 * 1024)
    torch.cuda.synchronize()
    ref = torch.stack([t.float() for t in ins]).sum(0)
    for o in outs:
        torch.testing.assert_close(o.float(), ref, **_tol(dtype))
    assert w.status()[0] == 0


@pytest.mark.parametrize("red", ["prod", "min", "max"])
@pytest.mark.parametrize("algo", [0, 1])
def test_all_reduce_other_ops(red, algo):
    n, count = 4, 5000
    w = _world(n)
    ins = [_rand(count, torch.float32, 3 + r) + (1.5 if red == "prod" else 0.0) for r in range(n)]
    outs = [torch.empty_like(t) for t in ins]
    w.all_reduce(ins, outs, RED[red], 1.0, algo, 3, 16 * 1024)
    torch.cuda.synchronize()
    st = torch.stack(ins)
    ref = {"prod": st.prod(0), "min": st.min(0).values, "max": st.max(0).values}[red]
    for o in outs:
        torch.testing.assert_close(o, ref, rtol=1e-5, atol=1e-5)


def test_all_reduce_in_place_scaled_and_repeated():
    # AVG = sum * 1/n, in place, several calls in a row on the same world
    # (exercises epoch counters, parity halves and slot reuse).
    n, count = 4, 70_000
    w = _world(n)
    for it in range(5):
        bufs = [_rand(count, torch.bfloat16, 100 * it + r) for r in range(n)]
        ref = torch.stack([t.float() for t in bufs]).mean(0)
        w.all_reduce(bufs, bufs, RED["sum"], 1.0 / n, it % 2, 4, 32 * 1024)
        torch.cuda.synchronize()
        for b in bufs:
            torch.testing.assert_close(b.float(), ref, rtol=2e-2, atol=2e-2)
    assert w.status()[0] == 0


def test_all_reduce_unaligned_views():
    n, count = 2, 4099
    w = _world(n)
    bases = [_rand(count + 3, torch.float32, r) for r in range(n)]
    ins = [b[1 : 1 + count] for b in bases]  # 4-byte aligned only
    outs = [torch.zeros(count + 3, device="cuda")[3:] for _ in range(n)]
    outs = [o[:count] for o in outs]
    w.all_reduce([i.contiguous() for i in ins], outs, RED["sum"], 1.0, 1, 2, 8 * 1024)
    torch.cuda.synchronize()
    ref = ins[0] + ins[1]
    for o in outs:
        torch.testing.assert_close(o, ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize(
    "din,wire,dout",
    [
        (torch.float32, "", torch.float32),
        (torch.bfloat16, "", torch.bfloat16),
        (torch.float16, "", torch.float16),
        (torch.float32, "bf16", torch.float32),
        (torch.float32, "bf16", torch.bfloat16),
        (torch.bfloat16, "bf16", torch.float32),
    ],
)
def test_reduce_scatter(nranks, din, wire, dout):
    count = 12_345
    w = _world(nranks)
    ins = [_rand(nranks * count, din, 11 + r) for r in range(nranks)]
    outs = [torch.empty(count, dtype=dout, device="cuda") for _ in range(nranks)]
    w.reduce_scatter(ins, outs, wire, RED["sum"], 0.5, 3, 8 * 1024)
    torch.cuda.synchronize()
    total = torch.stack([t.float() for t in ins]).sum(0).view(nranks, count) * 0.5
    loose = wire == "bf16" or din != torch.float32 or dout != torch.float32
    for r in range(nranks):
        torch.testing.assert_close(outs[r].float(), total[r], **(_tol(torch.bfloat16) if loose else _tol(torch.float32)))
    assert w.status()[0] == 0


def test_reduce_scatter_stochastic_rounding():
    """fp32 -> bf16 wire with stochastic rounding: unbiased, reproducible per seed, different across seeds."""
    nranks, count = 4, 64 * 1024
    w = _world(nranks)
    value = 1.0 + 2.0 ** -10          # between the bf16 neighbours 1 and 1 + 2^-7: rounds up with probability 1/8
    ins = [torch.full((nranks * count,), value, dtype=torch.float32, device="cuda") for _ in range(nranks)]

    def run(seed):
        outs = [torch.empty(count, dtype=torch.float32, device="cuda") for _ in range(nranks)]
        w.reduce_scatter_sr(ins, outs, "bf16", RED["sum"], 1.0, 4, 16 * 1024, seed)
        torch.cuda.synchronize()
        return outs

    nearest = run(0)
    # round to nearest loses the 2^-10 on every remote contribution (the own part stays fp32)
    assert torch.equal(nearest[0], torch.full((count,), (nranks - 1) * 1.0 + value, device="cuda"))
    a, b, c = run(1234), run(1234), run(99)
    for r in range(nranks):
        assert torch.equal(a[r], b[r])
    assert not torch.equal(a[0], c[0])
    # every remote term is 1 or 1 + 2^-7; the mean recovers the true value
    mean = torch.stack(a).mean().item()
    expect = nranks * value
    assert abs(mean - expect) < 2e-4, (mean, expect)
    frac_up = ((torch.stack(a) - ((nranks - 1) + value)) / 2.0 ** -7).mean().item() / (nranks - 1)
    assert 0.10 < frac_up < 0.15, frac_up
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks", [1, 2, 8])
@pytest.mark.parametrize("nbytes", [48, 4096, 1_000_003])
def test_all_gather_bytes(nranks, nbytes):
    w = _world(nranks)
    ins = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    outs = [torch.empty(nranks * nbytes, dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    w.all_gather(ins, outs, False, 4, 64 * 1024)
    torch.cuda.synchronize()
    ref = torch.cat(ins)
    for o in outs:
        assert torch.equal(o, ref)


@pytest.mark.parametrize("nranks", [2, 3, 8])
@pytest.mark.parametrize("nbytes", [48, 4096, 100_003, 512 * 1024])
def test_all_gather_one_shot(nranks, nbytes):
    """chunk 0 selects the latency kernel: one staged copy, one barrier, pull from every peer."""
    if nranks * ((nbytes + 4095) // 4096) > 400:
        pytest.skip("emulation runs all virtual ranks' blocks in one cooperative grid")
    w = _world(nranks)
    for it in range(3):  # consecutive calls alternate the parity buffer
        ins = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(nranks)]
        outs = [torch.empty(nranks * nbytes, dtype=torch.uint8, device="cuda") for _ in range(nranks)]
        w.all_gather(ins, outs, False, 1, 0)
        torch.cuda.synchronize()
        ref = torch.cat(ins)
        for o in outs:
            assert torch.equal(o, ref)
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("count", [7, 1000, 16_000])
def test_reduce_scatter_one_shot(nranks, dtype, count):
    if count * torch.empty(0, dtype=dtype).element_size() > 128 * ((4096 // nranks) // 16 * 16):
        pytest.skip("beyond the one-shot capacity for this rank count")
    sub = (4096 // nranks) // 16 * 16
    if nranks * -(-count * torch.empty(0, dtype=dtype).element_size() // sub) > 400:
        pytest.skip("emulation runs all virtual ranks' blocks in one cooperative grid")
    w = _world(nranks)
    for it in range(3):
        ins = [_rand(nranks * count, dtype, 100 * it + r) for r in range(nranks)]
        outs = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(nranks)]
        w.reduce_scatter(ins, outs, "same", RED["sum"], 1.0, 1, 0)
        torch.cuda.synchronize()
        total = torch.stack([t.float() for t in ins]).sum(0).view(nranks, count)
        for r in range(nranks):
            torch.testing.assert_close(outs[r].float(), total[r], **_tol(dtype))
    assert w.status()[0] == 0


def test_all_gather_fused_cast():
    n, count = 4, 33_333
    w = _world(n)
    ins = [_rand(count, torch.float32, 5 + r) for r in range(n)]
    outs = [torch.empty(n * count, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    w.all_gather(ins, outs, True, 4, 16 * 1024)
    torch.cuda.synchronize()
    ref = torch.cat(ins).to(torch.bfloat16)
    for o in outs:
        assert torch.equal(o, ref)


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_all_to_all_variable_splits(nranks):
    w = _world(nranks)
    g = torch.Generator().manual_seed(0)
    splits = torch.randint(0, 40_000, (nranks, nranks), generator=g)
    splits[0, 1 % nranks] = 0  # an empty block
    splits = (splits // 4 * 4).tolist()
    ins = [torch.randint(0, 255, (sum(splits[r]),), dtype=torch.uint8, device="cuda") for r in range(nranks)]
    outs = [torch.zeros(sum(splits[p][r] for p in range(nranks)), dtype=torch.uint8, device="cuda") for r in range(nranks)]
    w.all_to_all(ins, outs, splits, 4, 16 * 1024)
    torch.cuda.synchronize()
    for r in range(nranks):
        parts = []
        for p in range(nranks):
            off = sum(splits[p][:r])
            parts.append(ins[p][off : off + splits[p][r]])
        assert torch.equal(outs[r], torch.cat(parts))
    assert w.status()[0] == 0


def test_all_to_all_device_resident_splits():
    n, row = 4, 64  # 64-byte rows
    w = _world(n)
    counts = [[(r + p) % 5 for p in range(n)] for r in range(n)]
    ins = [torch.randint(0, 255, (sum(counts[r]) * row,), dtype=torch.uint8, device="cuda") for r in range(n)]
    outs = [torch.zeros(sum(counts[p][r] for p in range(n)) * row, dtype=torch.uint8, device="cuda") for r in range(n)]
    dev_counts = [torch.tensor(c, dtype=torch.int64, device="cuda") for c in counts]
    w.all_to_all_device_splits(ins, outs, dev_counts, row, 2, 4096)
    torch.cuda.synchronize()
    for r in range(n):
        parts = []
        for p in range(n):
            off = sum(counts[p][:r]) * row
            parts.append(ins[p][off : off + counts[p][r] * row])
        assert torch.equal(outs[r], torch.cat(parts))


@pytest.mark.parametrize("root", [0, 2])
def test_broadcast(root):
    n, nbytes = 4, 70_001
    w = _world(n)
    bufs = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(n)]
    ref = bufs[root].clone()
    w.broadcast(bufs, root, 3, 8 * 1024)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b, ref)


def test_barrier_repeats():
    w = _world(8)
    for _ in range(10):
        w.barrier()
    torch.cuda.synchronize()
    assert w.status()[0] == 0


def test_bounded_wait_reports_instead_of_hanging():
    # A wait on a flag nobody sets gives up after its budget (50 ms here),
    # records who waited for what, and the kernel returns normally.
    w = _world(2, wait_ms=50.0)
    status = w.wait_unset_flag()
    assert status[0] & 1, "timeout bit must be set"
    assert status[4] == 0x7F
    # The context stays usable, and a dead communicator makes later waits
    # return at once instead of burning their budget again.
    w.barrier()
    torch.cuda.synchronize()
    x = torch.ones(4, device="cuda")
    assert float(x.sum()) == 4.0
    w.clear_status()
    w2 = _world(2)
    w2.barrier()
    torch.cuda.synchronize()
    assert w2.status()[0] == 0


def test_device_window_ring_put_signal_barrier():
    n, count = 4, 10_000
    w = _world(n)
    srcs = [torch.full((count,), float(r + 1), device="cuda") for r in range(n)]
    dsts = [torch.zeros(count, device="cuda") for _ in range(n)]
    counters = w.window_ring(srcs, dsts)
    torch.cuda.synchronize()
    for r in range(n):
        left = (r - 1) % n
        assert torch.equal(dsts[r], srcs[left])
        assert int(counters[r].item()) == 1
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks,nbytes,nslots,slot", [(2, 4096, 2, 1024), (4, 1 << 20, 2, 16384), (8, 300_000, 3, 65536), (3, 48, 1, 16)])
def test_device_send_forward_recv_ring_broadcast(nranks, nbytes, nslots, slot):
    """Device-side send / forward / recv through slot FIFOs: a pipelined broadcast along the ring, messages far
    larger than the FIFO (the sender must wait for slots to come back), repeated calls, every root."""
    from torchcomms_b200 import _comms

    emu = _comms.P2pEmu(nranks, nslots, slot, 5000.0)
    for it in range(3):
        root = it % nranks
        bufs = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(nranks)]
        want = bufs[root].clone()
        emu.ring_broadcast(bufs, root)
        assert emu.status()[0] == 0, emu.status()
        for r in range(nranks):
            assert torch.equal(bufs[r], want), (it, r)


@pytest.mark.parametrize("nranks", [2, 8])
def test_ll_packets_carry_their_own_flag(nranks):
    from torchcomms_b200 import _comms

    words = 1000
    emu = _comms.P2pEmu(nranks, 1, 16, 5000.0)
    tables = [torch.zeros(words, dtype=torch.int64, device="cuda") for _ in range(nranks)]
    for epoch in (1, 2, 7):
        outs = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(nranks)]
        emu.ll_exchange(tables, outs, epoch)
        assert emu.status()[0] == 0
        for r in range(nranks):
            prev = (r - 1) % nranks
            assert torch.equal(outs[r], (torch.arange(words, device="cuda") + prev * 100000 + epoch).int())
