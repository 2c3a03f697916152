"""The collective functions of ``distwrap`` under the module path the reference gives them
(``torchcomms.distwrap.collectives``); they are defined in the package's ``__init__``."""
from . import (  # noqa: F401
    all_gather, all_gather_into_tensor, all_gather_object, all_reduce, all_to_all, all_to_all_single, barrier,
    batch_isend_irecv, broadcast, broadcast_object_list, gather, gather_object, irecv, isend, recv, reduce,
    reduce_scatter, reduce_scatter_tensor, scatter, scatter_object_list, send,
)
from . import _make_nccl_premul_sum, get_mem_allocator, register_mem_pool  # noqa: F401
