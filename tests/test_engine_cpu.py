"""The sharded training engine on CPU ranks (gloo): sharding, gather /
reduce-scatter plumbing, optimizer, and equivalence between 1 and 2 ranks."""
from datetime import timedelta

import torch

from tests.mp_util import run_ranks


def _train(rank, world, out_path):
    import torchcomms_b200 as tc
    from torchcomms_b200.models.llama import LlamaConfig
    from torchcomms_b200.parallel.engine import TrainEngine

    torch.manual_seed(0)
    comm = tc.new_comm("gloo", torch.device("cpu"), name="engine", timeout=timedelta(seconds=120))
    cfg = LlamaConfig(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=128, vocab_size=97, max_seq_len=32)
    engine = TrainEngine(cfg, comm, lr=1e-2, weight_decay=0.0, seed=3, recompute_blocks=1)
    g = torch.Generator().manual_seed(11)
    tokens = torch.randint(0, cfg.vocab_size, (2, 17), generator=g)  # same batch on every rank
    losses = []
    for _ in range(4):
        loss = engine.step(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous())
        losses.append(float(loss))
    assert all(l == l for l in losses)
    assert losses[-1] < losses[0], losses
    # every unit's transient buffers are gone after the step
    for u in engine.units:
        assert u.flat_grad is None and u.grad_shard is None
        assert u.flat_param.untyped_storage().nbytes() == 0 or u is engine.units[-1]
    state = engine.state_dict()
    assert state["step"] == 4
    if rank == 0:
        torch.save({"losses": losses, "world": world}, out_path)
    comm.finalize()


def test_engine_trains_and_matches_across_world_sizes(tmp_path):
    p1, p2 = str(tmp_path / "w1.pt"), str(tmp_path / "w2.pt")
    run_ranks(_train, 1, args=(p1,), timeout=240)
    run_ranks(_train, 2, args=(p2,), timeout=240)
    a, b = torch.load(p1), torch.load(p2)
    # identical data on every rank: the averaged gradient equals the single-rank gradient
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 5e-2, (a["losses"], b["losses"])
