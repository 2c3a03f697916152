"""Numerics of the one-pass kernels on symmetric buffers and of the flag-less
small all-reduce, on ONE GPU.

Virtual ranks run side by side in one cooperative launch (``_EmuWorld``); every
rank's "symmetric" tensor is simply that rank's tensor on the same device, so
the kernels execute their plain peer load / store data path (the multicast path
needs a switch and is covered by the multi-process tests).  Every result is
compared with a PyTorch fp32 restatement of the operation.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _world(n, wait_ms=2000.0):
    from torchcomms_b200 import _comms

    return _comms._EmuWorld(n, 8 << 20, wait_ms)


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype != torch.float32 else dict(rtol=1e-5, atol=1e-5)


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)


@pytest.mark.parametrize("nranks", [1, 2, 4, 8])
@pytest.mark.parametrize("blocks", [1, 5])
@pytest.mark.parametrize("count", [8, 4096, 100_000])
def test_symm_all_gather(nranks, blocks, count):
    w = _world(nranks)
    ins = [_rand(count, torch.bfloat16, 3 + r) for r in range(nranks)]
    outs = [torch.zeros(nranks * count, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
    w.symm_all_gather(ins, outs, False, blocks)
    torch.cuda.synchronize()
    ref = torch.cat(ins)
    for o in outs:
        assert torch.equal(o, ref)
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks", [2, 8])
def test_symm_all_gather_fused_cast_and_unaligned_input(nranks):
    count = 24_576 + 8
    w = _world(nranks)
    bases = [_rand(count + 1, torch.float32, 5 + r) for r in range(nranks)]
    # rank 1's shard starts 4 bytes off a 16-byte boundary: the kernel's scalar load path
    ins = [b[1:] if r == 1 else b[:count] for r, b in enumerate(bases)]
    outs = [torch.zeros(nranks * count, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
    w.symm_all_gather(ins, outs, True, 4)
    torch.cuda.synchronize()
    ref = torch.cat([i.to(torch.bfloat16) for i in ins])
    for o in outs:
        assert torch.equal(o, ref)


@pytest.mark.parametrize("nranks", [1, 2, 4, 8])
@pytest.mark.parametrize(
    "din,dout",
    [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32), (torch.float32, torch.float32), (torch.float16, torch.float16)],
)
def test_symm_reduce_scatter(nranks, din, dout):
    count = 16 * 1531
    w = _world(nranks)
    ins = [_rand(nranks * count, din, 17 + r) for r in range(nranks)]
    outs = [torch.empty(count, dtype=dout, device="cuda") for _ in range(nranks)]
    w.symm_reduce_scatter(ins, outs, 1.0 / nranks, 3)
    torch.cuda.synchronize()
    ref = torch.stack([t.float() for t in ins]).sum(0).view(nranks, count) / nranks
    for r in range(nranks):
        torch.testing.assert_close(outs[r].float(), ref[r], **_tol(torch.bfloat16 if din != torch.float32 else torch.float32))
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_symm_all_reduce_in_place_repeated(nranks, dtype):
    count = 8 * 5001
    w = _world(nranks)
    for it in range(3):  # epochs advance, buffers are reused
        bufs = [_rand(count, dtype, 100 * it + r) for r in range(nranks)]
        ref = torch.stack([t.float() for t in bufs]).sum(0) * 0.5
        w.symm_all_reduce(bufs, 0.5, 1 + 3 * it)
        torch.cuda.synchronize()
        for b in bufs:
            torch.testing.assert_close(b.float(), ref, **_tol(dtype))
    assert w.status()[0] == 0


def _a2a_reference(ins, splits, nranks):
    """Concatenation, per receiver, of the blocks each sender addressed to it."""
    outs = []
    for r in range(nranks):
        parts = []
        for q in range(nranks):
            off = sum(splits[q][:r])
            parts.append(ins[q][off : off + splits[q][r]])
        outs.append(torch.cat(parts))
    return outs


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("blocks", [2, 16])
def test_symm_all_to_all_equal_splits(nranks, blocks):
    blk = 48 * 1024
    w = _world(nranks)
    ins = [torch.randint(0, 255, (nranks * blk,), dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    outs = [torch.zeros(nranks * blk, dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    splits = [[blk] * nranks for _ in range(nranks)]
    w.symm_all_to_all(ins, outs, splits, 0, [], 1, blocks)
    torch.cuda.synchronize()
    for o, ref in zip(outs, _a2a_reference(ins, splits, nranks)):
        assert torch.equal(o, ref)
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("mode", [1, 2])
def test_symm_all_to_all_variable_splits(nranks, mode):
    """Host splits (offsets exchanged in the kernel) and device-resident counts; odd sizes take the byte path."""
    g = torch.Generator().manual_seed(5 + nranks)
    elem = 6 if mode == 2 else 1
    splits = [[int(torch.randint(0, 9000, (1,), generator=g)) * elem for _ in range(nranks)] for _ in range(nranks)]
    splits[0][nranks - 1] = 0  # an empty block
    w = _world(nranks)
    in_cap = max(sum(s) for s in splits) + 64
    out_cap = max(sum(splits[q][r] for q in range(nranks)) for r in range(nranks)) + 64
    ins = [torch.randint(0, 255, (in_cap,), dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    outs = [torch.full((out_cap,), 7, dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    counts = [torch.tensor([x // elem for x in s], dtype=torch.int64, device="cuda") for s in splits] if mode == 2 else []
    w.symm_all_to_all(ins, outs, splits, mode, counts, elem, 8)
    torch.cuda.synchronize()
    for o, ref in zip(outs, _a2a_reference(ins, splits, nranks)):
        assert torch.equal(o[: ref.numel()], ref)
        assert bool((o[ref.numel() :] == 7).all())  # nothing written past the received data
    assert w.status()[0] == 0


def _to_heads_reference(xs, n):
    """xs[r]: [b, h, s, d] on rank r -> per rank p [b, h/n, n*s, d]: heads p*h/n.., sequence blocks in rank order."""
    hn = xs[0].shape[1] // n
    return [torch.cat([xs[r][:, p * hn:(p + 1) * hn] for r in range(n)], dim=2) for p in range(n)]


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("dtype,shape,blocks", [
    (torch.bfloat16, (2, 16, 24, 64), 8),     # 3 KB slabs
    (torch.bfloat16, (1, 8, 80, 64), 5),      # 10 KB slabs walked slab by slab, block ranges that straddle slabs
    (torch.float32, (1, 8, 5, 12), 3),        # 240-byte slabs, more vectors than a block's share
    (torch.bfloat16, (3, 8, 7, 9), 4),        # 126-byte slabs: not a multiple of 16, byte path
])
def test_symm_seq_heads_exchange_both_directions(nranks, dtype, shape, blocks):
    """Sequence shards -> head shards and back, layout changes inside the kernel, against cat / split."""
    b, h, s, d = shape
    w = _world(nranks)
    xs = [torch.randn(b, h, s, d, device="cuda").to(dtype) for _ in range(nranks)]
    heads = [torch.zeros(b, h // nranks, nranks * s, d, dtype=dtype, device="cuda") for _ in range(nranks)]
    w.symm_seq_heads(xs, heads, True, blocks)
    torch.cuda.synchronize()
    for got, ref in zip(heads, _to_heads_reference(xs, nranks)):
        assert torch.equal(got, ref)
    back = [torch.zeros(b, h, s, d, dtype=dtype, device="cuda") for _ in range(nranks)]
    w.symm_seq_heads(heads, back, False, blocks)
    torch.cuda.synchronize()
    for got, ref in zip(back, xs):
        assert torch.equal(got, ref)
    assert w.status()[0] == 0


def test_symm_all_to_all_counts_beyond_capacity_are_clamped():
    """A sender's device count exceeds what the receiver's output can hold: nothing lands out of bounds,
    and the status word reports the bad argument."""
    nranks, elem = 2, 16
    w = _world(nranks)
    guard = 4096
    out_rows = 100
    # outputs sit inside larger buffers whose margins must stay untouched
    backing = [torch.full((guard + out_rows * elem + guard,), 9, dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    outs = [b[guard : guard + out_rows * elem] for b in backing]
    ins = [torch.randint(0, 255, (400 * elem,), dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    # rank 0 sends 150 rows to rank 1 (capacity 100 rows in total); rank 1 sends a negative count
    counts = [torch.tensor([10, 150], dtype=torch.int64, device="cuda"), torch.tensor([-5, 20], dtype=torch.int64, device="cuda")]
    w.symm_all_to_all(ins, outs, [[0, 0], [0, 0]], 2, counts, elem, 4)
    torch.cuda.synchronize()
    for b in backing:
        assert bool((b[:guard] == 9).all()) and bool((b[-guard:] == 9).all())
    assert w.status()[0] & 4  # kStatusBadArg
    # rank 0 received its own 10 rows intact
    assert torch.equal(outs[0][: 10 * elem], ins[0][: 10 * elem])


def test_staged_all_to_all_device_counts_beyond_capacity_are_clamped():
    nranks, elem = 2, 16
    w = _world(nranks)
    guard = 4096
    out_rows = 100
    backing = [torch.full((guard + out_rows * elem + guard,), 9, dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    outs = [b[guard : guard + out_rows * elem] for b in backing]
    ins = [torch.randint(0, 255, (400 * elem,), dtype=torch.uint8, device="cuda") for _ in range(nranks)]
    counts = [torch.tensor([10, 150], dtype=torch.int64, device="cuda"), torch.tensor([-5, 20], dtype=torch.int64, device="cuda")]
    w.all_to_all_device_splits(ins, outs, counts, elem, 2, 8 * 1024)
    torch.cuda.synchronize()
    for b in backing:
        assert bool((b[:guard] == 9).all()) and bool((b[-guard:] == 9).all())
    assert w.status()[0] & 4
    assert torch.equal(outs[0][: 10 * elem], ins[0][: 10 * elem])


# ----------------------------------------------------- flag-less all-reduce ----


@pytest.mark.parametrize("nranks", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("count", [1, 500, 2048, 16_000])
def test_lamport_all_reduce(nranks, dtype, count):
    w = _world(nranks)
    ins = [_rand(count, dtype, 31 + r) for r in range(nranks)]
    outs = [torch.empty_like(t) for t in ins]
    w.all_reduce_lamport(ins, outs, 1.0)
    torch.cuda.synchronize()
    ref = torch.stack([t.float() for t in ins]).sum(0)
    for o in outs:
        torch.testing.assert_close(o.float(), ref, **_tol(dtype))
    assert w.status()[0] == 0


def test_lamport_all_reduce_many_calls_of_changing_size():
    """Buffers rotate per block; calls of different lengths in a row (in place, scaled) must not see stale data."""
    n = 4
    w = _world(n)
    sizes = [16_000, 64, 9_000, 1, 32_768, 2_048, 2_048, 2_048, 31_999, 5]
    for it, count in enumerate(sizes):
        bufs = [_rand(count, torch.bfloat16, 1000 * it + r) for r in range(n)]
        ref = torch.stack([t.float() for t in bufs]).sum(0) / n
        w.all_reduce_lamport(bufs, bufs, 1.0 / n)
        torch.cuda.synchronize()
        for b in bufs:
            torch.testing.assert_close(b.float(), ref, rtol=2e-2, atol=2e-2)
    assert w.status()[0] == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lamport_all_reduce_payload_that_looks_like_the_empty_marker(dtype):
    """-0.0 is the 'nothing arrived' word: payloads full of -0.0, NaN and infinities must still reduce correctly."""
    n, count = 4, 4096
    w = _world(n)
    ins = []
    for r in range(n):
        t = _rand(count, dtype, 77 + r)
        t[::3] = -0.0
        t[1::7] = 0.0
        ins.append(t)
    ins[1][5] = float("nan")
    ins[2][6] = float("inf")
    if dtype == torch.bfloat16:
        # a pair whose 32-bit word is exactly 0x80000000: low half +0.0, high half -0.0
        ins[0][10], ins[0][11] = 0.0, -0.0
    outs = [torch.empty_like(t) for t in ins]
    w.all_reduce_lamport(ins, outs, 1.0)
    torch.cuda.synchronize()
    ref = torch.stack([t.float() for t in ins]).sum(0)
    for o in outs:
        torch.testing.assert_close(o.float(), ref, equal_nan=True, **_tol(dtype))
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks", [1, 2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("part", [8, 1000, 20_000])
def test_lamport_all_gather_all_to_all_reduce_scatter(nranks, dtype, part):
    """The flag-less exchange in its three roles, several calls in a row on one world (buffers rotate)."""
    part = part // 8 * 8 if part >= 8 else 8          # whole 16-byte vectors in both dtypes
    w = _world(nranks)
    for it in range(3):
        # all-gather
        ins = [_rand(part, dtype, 10 * it + r) for r in range(nranks)]
        outs = [torch.zeros(nranks * part, dtype=dtype, device="cuda") for _ in range(nranks)]
        w.exchange_lamport(0, ins, outs, 1.0)
        torch.cuda.synchronize()
        for o in outs:
            assert torch.equal(o, torch.cat(ins))
        # all-to-all, equal parts
        ins = [_rand(nranks * part, dtype, 50 + 10 * it + r) for r in range(nranks)]
        outs = [torch.zeros(nranks * part, dtype=dtype, device="cuda") for _ in range(nranks)]
        w.exchange_lamport(1, ins, outs, 1.0)
        torch.cuda.synchronize()
        for r in range(nranks):
            assert torch.equal(outs[r], torch.cat([ins[q][r * part:(r + 1) * part] for q in range(nranks)]))
        # reduce-scatter with a scale
        outs = [torch.zeros(part, dtype=dtype, device="cuda") for _ in range(nranks)]
        w.exchange_lamport(2, ins, outs, 0.5)
        torch.cuda.synchronize()
        ref = torch.stack([t.float() for t in ins]).sum(0).view(nranks, part) * 0.5
        for r in range(nranks):
            torch.testing.assert_close(outs[r].float(), ref[r], **_tol(dtype))
    assert w.status()[0] == 0


def test_lamport_exchange_unaligned_views_and_marker_payload():
    n, part = 4, 512
    w = _world(n)
    bases = [_rand(part + 1, torch.float32, r) for r in range(n)]
    ins = [b[1:] for b in bases]                       # 4 bytes off a 16-byte boundary
    for t in ins:
        t[::5] = -0.0                                  # the "nothing here yet" word as payload
    out_bases = [torch.zeros(n * part + 1, device="cuda") for _ in range(n)]
    outs = [b[1:] for b in out_bases]
    w.exchange_lamport(0, ins, outs, 1.0)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o, torch.cat(ins))          # -0.0 == +0.0 numerically
    assert w.status()[0] == 0


@pytest.mark.parametrize("nranks,dtype", [(2, torch.float32), (4, torch.bfloat16), (8, torch.float32)])
def test_lamport_all_to_all_with_unequal_parts(nranks, dtype):
    """Flag-less all-to-all-v: parts of any byte length (odd element counts, empty parts, -0.0 payloads), interleaved
    with equal-split exchanges on the same world so that the rotating buffers are shared between the two kernels."""
    w = _world(nranks)
    esz = torch.empty(0, dtype=dtype).element_size()
    g = torch.Generator().manual_seed(99 + nranks)
    for it in range(4):
        counts = torch.randint(0, 700, (nranks, nranks), generator=g)      # elements rank r sends to rank p
        counts[0, nranks - 1] = 0
        counts[nranks - 1, 0] = 1 if it % 2 else 333
        ins, outs, want = [], [], []
        for r in range(nranks):
            parts = [_rand(int(counts[r, p]), dtype, 1000 * it + 10 * r + p) for p in range(nranks)]
            if parts[0].numel() > 2:
                parts[0][1] = -0.0                     # the marker value as payload
            ins.append(torch.cat(parts) if sum(p.numel() for p in parts) else torch.empty(0, dtype=dtype, device="cuda"))
        for r in range(nranks):
            total = int(counts[:, r].sum())
            outs.append(torch.full((total + 3,), 7.0, dtype=dtype, device="cuda"))   # three guard elements behind
        cap = int(counts.max()) * esz + 64
        w.exchangev_lamport([t if t.numel() else torch.zeros(4, dtype=dtype, device="cuda") for t in ins], outs,
                            (counts * esz).tolist(), cap)
        torch.cuda.synchronize()
        assert w.status()[0] == 0
        for r in range(nranks):
            at = 0
            for s in range(nranks):
                n = int(counts[s, r])
                off = int(counts[s, :r].sum())
                got, ref = outs[r][at : at + n], ins[s][off : off + n]
                assert torch.equal(got.float(), ref.float()), (it, r, s, n)    # -0.0 == +0.0
                at += n
            assert torch.equal(outs[r][at:].float(), torch.full((3,), 7.0, device="cuda")), "wrote past its parts"
        # an equal-split exchange in between uses the same buffers and call counters
        part = 256
        eins = [_rand(part * nranks, torch.float32, 5 * it + r) for r in range(nranks)]
        eouts = [torch.empty_like(t) for t in eins]
        w.exchange_lamport(1, eins, eouts, 1.0)
        torch.cuda.synchronize()
        for r in range(nranks):
            for s in range(nranks):
                assert torch.equal(eouts[r][s * part : (s + 1) * part], eins[s][r * part : (r + 1) * part])
