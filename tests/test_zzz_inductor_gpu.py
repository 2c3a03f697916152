"""Inductor backend on a CUDA communicator (one GPU): communicator methods traced through ``functional.dynamo``,
lowered through ``functional.inductor`` and compiled with the generated Triton kernels around them, against the eager
run of the same function.  Kept in a file of its own that sorts last: it compiles code at run time, which takes
longer than the other GPU tests and depends on the compiler toolchain of the box.

Parity: comms/torchcomms/tests/integration/py/FullgraphCompileTest.py (inductor backend).
"""
import pytest
import torch


@pytest.mark.gpu
def test_inductor_compiles_communicator_methods_on_gpu():
    """Inductor backend on a CUDA communicator: the in-place all-reduce lowering, a started all-gather with its
    wait, the default handling of the other operators, against the eager run of the same function."""
    import os

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29631")
    os.environ["RANK"], os.environ["WORLD_SIZE"] = "0", "1"
    import torchcomms_b200 as tc
    from torch._inductor.utils import run_and_get_code
    from torchcomms_b200 import ReduceOp
    from torchcomms_b200.functional import dynamo as D
    from torchcomms_b200.functional import inductor as I

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    D.register_with_dynamo()
    assert I.register_with_inductor()
    comm = tc.new_comm("b200", dev, name="ind_gpu", abort_process_on_timeout_or_error=False)
    try:
        def step(x, out_g):
            y = x * 2 + 1
            comm.all_reduce(y, ReduceOp.SUM, False)
            w = comm.all_gather_single(out_g, y, True)
            z = torch.relu(y - 3) * comm.get_size()
            s = torch.empty_like(z)
            comm.reduce_scatter_single(s, z, ReduceOp.SUM, False)
            w.wait()
            return s + out_g.view_as(s)

        x = torch.randn(1024, 64, device=dev)
        ref_g = torch.zeros(1024 * 64, device=dev)
        ref = step(x, ref_g)
        out_g = torch.zeros(1024 * 64, device=dev)
        got, codes = run_and_get_code(torch.compile(step, fullgraph=True, backend="inductor"), x, out_g)
        torch.cuda.synchronize()
        assert torch.allclose(got, ref) and torch.equal(out_g, ref_g)
        code = "\n".join(codes)
        assert "torchcomms_b200.all_reduce_inplace" in code     # lowered to the in-place kernel
        assert "all_gather_single_start" in code and "wait_tensor" in code and "reduce_scatter_single" in code
    finally:
        comm.finalize()
        D.unregister_from_dynamo()
