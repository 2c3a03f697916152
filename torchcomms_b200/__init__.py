"""torchcomms_b200 — a Blackwell-native communications framework for PyTorch.

The public surface mirrors meta-pytorch/torchcomms (``comms/torchcomms/__init__.py:40-106``
and ``comms/torchcomms/_comms.pyi:607-844``): ``new_comm(backend, device, name=...)``
returns a ``TorchComm`` whose collectives return ``TorchWork`` handles.

Backends registered in-tree:

* ``"b200"`` (aliases ``"nccl"``, ``"ncclx"``): CUDA backend for NVLink/NVSwitch
  machines — peer-memory kernels on a symmetric heap, NCCL for point-to-point
  and as a selectable fallback.
* ``"gloo"``: CPU backend over TCP (also accepts CUDA tensors, staged through
  the host).
* ``"fake"``: moves no data; for unit tests.

Python-implemented backends are added with ``register_backend(name, cls)``.
"""
from __future__ import annotations

import importlib
import importlib.metadata
import os
import sys
from datetime import timedelta
from typing import Any, Dict, Optional

import torch  # noqa: F401  (must be loaded before the extension)


def _load_extension():
    here = os.path.dirname(os.path.abspath(__file__))
    so = os.path.join(here, "_comms.so")
    if not os.path.exists(so):
        if os.environ.get("B200COMMS_NO_AUTOBUILD", "0") == "1":
            raise ImportError(
                f"{so} is missing; run `python -m torchcomms_b200._build` first"
            )
        from . import _build

        _build.build()
    spec = importlib.util.spec_from_file_location("torchcomms_b200._comms", so)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["torchcomms_b200._comms"] = mod
    spec.loader.exec_module(mod)
    return mod


import importlib.util  # noqa: E402

_comms = _load_extension()

from ._comms import (  # noqa: E402,F401
    AllGatherPHandle,
    BatchSendRecv,
    CommOptions,
    OpName,
    OpOptions,
    P2POp,
    P2POpType,
    ReconfigureOptions,
    RedOpType,
    ReduceOp,
    RemovableHandle,
    TorchComm,
    TorchCommBackend,
    TorchCommWinAccessType,
    TorchCommWindow,
    TorchCommWindowAttr,
    TorchWork,
    WorkStatus,
    _BackendWrapper,
    _is_backend_registered,
    register_backend,
)
from ._hook_args import *  # noqa: E402,F401,F403
from ._hook_args import _to_post_args, _to_pre_args  # noqa: E402

_comms._set_hook_arg_converters(_to_pre_args, _to_post_args)

InitHandle = str
Timeout = timedelta


def _make_gloo_pg(store, rank, size, timeout):
    """The gloo process group under the ``gloo`` backend.  ``TORCHCOMM_GLOO_INTERFACE`` /
    ``TORCHCOMM_GLOO_HOSTNAME`` pick the TCP device, as in the reference
    (comms/torchcomms/gloo/TorchCommGloo.cpp:85-190)."""
    import os

    import torch.distributed as dist

    iface = os.environ.get("TORCHCOMM_GLOO_INTERFACE", "")
    host = os.environ.get("TORCHCOMM_GLOO_HOSTNAME", "")
    if not iface and not host:
        return dist.ProcessGroupGloo(store, rank, size, timeout)
    opts = dist.ProcessGroupGloo._Options()
    opts._timeout = timeout
    device = (dist.ProcessGroupGloo.create_device(interface=iface) if iface
              else dist.ProcessGroupGloo.create_device(hostname=host))
    opts._devices = [device]
    return dist.ProcessGroupGloo(store, rank, size, opts)


_comms._install_gloo_maker(_make_gloo_pg)


# Per-operation option classes: all carry ``hints`` and ``timeout``.
def _opt_class(name: str):
    return type(name, (OpOptions,), {"__doc__": f"Options for {name[:-7]} (hints, timeout)."})


for _n in (
    "SendOptions RecvOptions BatchP2POptions BroadcastOptions AllReduceOptions ReduceOptions "
    "AllGatherOptions AllGatherSingleOptions ReduceScatterOptions ReduceScatterSingleOptions "
    "AllToAllOptions AllToAllSingleOptions AllToAllvSingleOptions BarrierOptions ScatterOptions "
    "GatherOptions AllGatherPInitOptions AllGatherPExecOptions"
).split():
    globals()[_n] = _opt_class(_n)
del _n

_BUILTIN_BACKENDS = ("b200", "nccl", "ncclx", "gloo", "fake")


def _load_backend(backend: str) -> None:
    """Imports the module that registers ``backend`` if it is not known yet.

    Out-of-tree backends announce themselves through the entry-point groups
    ``torchcomms_b200.backends`` or ``torchcomms.backends``.
    """
    if _is_backend_registered(backend):
        return
    for group in ("torchcomms_b200.backends", "torchcomms.backends"):
        try:
            eps = importlib.metadata.entry_points(group=group)
        except Exception:  # pragma: no cover - metadata backends differ
            continue
        for ep in eps:
            if ep.name == backend:
                ep.load()
                return


def is_backend_built(backend: str) -> bool:
    return _is_backend_registered(backend)


def built_backends() -> list[str]:
    return list(_comms._registered_backends())


_comm_counter = 0


def new_comm(
    backend: str,
    device: Any,
    abort_process_on_timeout_or_error: Optional[bool] = None,
    timeout: Optional[timedelta] = None,
    store: Any = None,
    name: Optional[str] = None,
    enable_reconfigure: bool = False,
    hints: Optional[Dict[str, str]] = None,
    is_high_priority_stream: Optional[bool] = None,
) -> TorchComm:
    """Creates a communicator.

    Rank and world size come from the launcher environment (TORCHCOMM_RANK/SIZE,
    Open MPI, PMI, PALS or torchrun's RANK/WORLD_SIZE).  Without ``store`` a
    TCPStore on MASTER_ADDR:MASTER_PORT bootstraps the ranks.  ``name`` must be
    unique per process and identical across ranks.

    The reference's binding takes the name as its third positional argument (``new_comm("gloo", device, "dp")``)
    while its stubs list the keyword order used above; a string in the third position is therefore read as the name.
    """
    global _comm_counter
    if isinstance(abort_process_on_timeout_or_error, str):
        if name is not None:
            raise TypeError("new_comm: the name was given twice (third positional argument and name=)")
        name, abort_process_on_timeout_or_error = abort_process_on_timeout_or_error, None
    _load_backend(backend)
    if not _is_backend_registered(backend) and not os.environ.get(f"TORCHCOMMS_BACKEND_LIB_PATH_{backend.upper()}"):
        # The reference's loader fails with this type and wording when no module provides the backend.
        raise ModuleNotFoundError(
            f"failed to find backend '{backend}': unknown communication backend (not registered, no entry point "
            f"provides it and no TORCHCOMMS_BACKEND_LIB_PATH_{backend.upper()} library is set); known: {built_backends()}")
    opts = CommOptions()
    if abort_process_on_timeout_or_error is not None:
        opts.abort_process_on_timeout_or_error = abort_process_on_timeout_or_error
    if timeout is not None:
        opts.timeout = timeout
    if is_high_priority_stream is not None:
        opts.is_high_priority_stream = is_high_priority_stream
    if store is not None:
        opts.store = store
    opts.enable_reconfigure = enable_reconfigure
    if hints:
        opts.hints = dict(hints)
    if name is None:
        name = f"comm_{_comm_counter}"
    _comm_counter += 1
    if not isinstance(device, torch.device):
        device = torch.device(device)
    return _comms._new_comm(backend, device, name, opts)


def get_mem_allocator(backend: str):
    """Allocator whose memory is exportable to peers (symmetric heap)."""
    from .mem import get_mem_allocator as _g

    return _g(backend)


def _comm_mem_allocator(self):
    return get_mem_allocator(self.get_backend())


TorchComm.get_mem_allocator = _comm_mem_allocator
TorchComm.mem_allocator = property(_comm_mem_allocator)


def _comm_symm_empty(self, shape, dtype):
    """Collective: a tensor in memory every rank has mapped (see ``torchcomms_b200.mem.symm_empty``)."""
    from .mem import symm_empty as _s

    return _s(self, shape, dtype)


def _comm_symm_free(self, tensor):
    from .mem import symm_free as _f

    _f(self, tensor)


TorchComm.symm_empty = _comm_symm_empty
TorchComm.symm_free = _comm_symm_free


def _window_nvlink_address(self, peer: int, offset: int = 0) -> int:
    """Address at which this process reaches byte ``offset`` of rank ``peer``'s registered tensor (an NVLink peer
    mapping on the CUDA backend; the tensor's own address for ``peer`` = own rank), for kernels that take raw
    pointers.  The multicast alias of a window is available to device code through the device window
    (``get_device_window()``; ``DeviceWindow::get_multimem_address``).
    Parity: ``TorchCommWindowNCCLXGin.get_nvlink_address`` (comms/torchcomms/_comms_ncclx.pyi)."""
    t = self.map_remote_tensor(peer)
    if offset < 0 or offset > t.numel() * t.element_size():
        raise ValueError(f"offset {offset} outside the window ({t.numel() * t.element_size()} bytes)")
    return t.data_ptr() + offset


TorchCommWindow.get_nvlink_address = _window_nvlink_address


_native_get_backend_impl = TorchComm.get_backend_impl


def _comm_get_backend_impl(self):
    """The backend object behind the communicator: the native backend, or for a backend written in Python
    (``register_backend(name, cls)``) the instance of that class itself, as in the reference."""
    impl = _native_get_backend_impl(self)
    if isinstance(impl, _comms._PythonBackendAdapter):
        return impl.python_object()
    return impl


TorchComm.get_backend_impl = _comm_get_backend_impl
TorchComm.unsafe_get_backend = _comm_get_backend_impl


def _forward_to_backend(method: str):
    def call(self, *args, **kwargs):
        impl = self.get_backend_impl()
        fn = getattr(impl, method, None)
        if fn is None:
            raise RuntimeError(f"backend '{self.get_backend()}' has no {method}()")
        return fn(*args, **kwargs)

    call.__name__ = method
    call.__doc__ = (f"``get_backend_impl().{method}(...)``: a backend-specific operation of the CUDA backend "
                    "(comms/torchcomms/_comms_ncclx.pyi lists the same set), reachable from the communicator.")
    return call


for _m in ("get_nccl_comm_ptr", "device_alltoallv_single", "reduce_scatter_quantized", "set_config"):
    if not hasattr(TorchComm, _m):
        setattr(TorchComm, _m, _forward_to_backend(_m))
del _m


def _wrapper_mem_allocator(self):
    """The allocator of the wrapped communicator's backend (``_BackendWrapper.get_mem_allocator`` of the reference)."""
    return get_mem_allocator(self.get_comm().get_backend())


_BackendWrapper.get_mem_allocator = _wrapper_mem_allocator


def init_caching_allocator_hook() -> None:
    """Registers the caching allocator's segments (present and future) with the point-to-point transport, so that
    tensors from the ordinary allocator can be named in one-sided transfers without a registration per tensor.
    Parity: ``init_caching_allocator_hook`` of the reference's NCCLX module (comms/torchcomms/_comms_ncclx.pyi)."""
    from .transport import init_caching_allocator_hook as _hook

    _hook()


def healthy() -> bool:
    """False once any watchdog of this process saw a timeout or an async error."""
    return _comms._health_is_healthy()


def comm_dump_all(hints=None) -> dict:
    """State of every communicator alive in this process: ``{comm name: {key: value}}``
    (comms/torchcomms/ncclx/TorchCommNCCLXPy.cpp:137-184)."""
    return _comms.comm_dump_all(hints)


def set_trainer_iteration(iteration: int) -> None:
    """Tags what the process records from now on (flight-recorder entries, ``comm_dump_all``) with the
    training iteration, so a trace can be lined up with the step that produced it."""
    _comms.set_trainer_iteration(iteration)


def trainer_iteration() -> int:
    return _comms.trainer_iteration()


def knobs() -> dict:
    """Configuration keys read so far: ``{key: (value in force, "env" | "file" | "default")}``.

    A key is resolved from the environment, then from the configuration file
    (``B200COMMS_CONF_FILE``, default ``/etc/b200comms.conf``; ``KEY=VALUE`` lines),
    then from the built-in default -- the order the reference uses for its knobs
    (comms/utils/cvars/README.md:10-19).  Keys appear once something looked them up
    (creating a communicator reads the backend's tuning keys).
    """
    return {k: (v, src) for k, v, src in _comms._knobs()}


def reload_config() -> None:
    """Re-reads the configuration file at the next lookup."""
    _comms._reload_config()


__all__ = [n for n in dir() if not n.startswith("_")] + ["_BackendWrapper"]


def install_alias(name: str = "torchcomms") -> None:
    """Makes ``import torchcomms`` (and its sub-modules) resolve to this package in the current process.

    Code written against the reference package (``torchcomms.new_comm``, ``torchcomms.device_mesh``,
    ``torchcomms.distwrap``, ``torchcomms.objcol``, ``torchcomms.hooks``, ``torchcomms.functional``) then runs
    unchanged; backend names "nccl" and "ncclx" select this framework's CUDA backend.  Opt-in and at run time
    on purpose: a real top-level ``torchcomms`` directory would also be picked up by PyTorch's own start-up
    probing for that package, in the middle of ``import torch``.
    """
    import importlib
    import sys

    import types

    me = sys.modules[__name__]
    sys.modules[name] = me
    # `<name>._comms`: in the reference everything public lives in the native module (hook argument classes,
    # new_comm, get_mem_allocator, ...); here part of it is Python. Code that imports from `<name>._comms` gets a
    # module with the native names overlaid by this package's public ones.
    shim = types.ModuleType(f"{name}._comms")
    shim.__dict__.update({k: getattr(_comms, k) for k in dir(_comms) if not k.startswith("__")})
    shim.__dict__.update({k: v for k, v in vars(me).items() if not k.startswith("_") or k == "_BackendWrapper"})
    for sub in ("device_mesh", "distwrap", "functional", "objcol", "hooks", "mem", "ops", "parallel", "transport", "utils",
                "checkpoint"):
        sys.modules[f"{name}.{sub}"] = importlib.import_module(f"{__name__}.{sub}")
    sys.modules[f"{name}._comms"] = shim
    # The reference's per-backend modules name the backend classes that get_backend_impl() returns.
    per_backend = {
        "_comms_gloo": {"TorchCommGloo": _comms.GlooBackend},
        "_comms_nccl": {"TorchCommNCCL": _comms.CudaBackend},
        "_comms_ncclx": {"TorchCommNCCLX": _comms.CudaBackend, "comm_dump_all": comm_dump_all,
                         "init_caching_allocator_hook": init_caching_allocator_hook},
        "_comms_fake": {"TorchCommFake": _comms.FakeBackend},
    }
    for mod_name, members in per_backend.items():
        mod = types.ModuleType(f"{name}.{mod_name}")
        mod.__dict__.update(members)
        sys.modules[f"{name}.{mod_name}"] = mod


_LAZY_SUBMODULES = ("hooks", "objcol", "functional", "distwrap", "device_mesh", "mem", "ops", "parallel", "transport",
                    "checkpoint", "utils", "models")


def __getattr__(name):
    """``torchcomms_b200.hooks``, ``.objcol`` and the other sub-packages resolve on first use, as they do after a
    plain ``import torchcomms`` of the reference (which imports ``hooks`` and ``objcol`` eagerly)."""
    if name in _LAZY_SUBMODULES:
        import importlib

        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module '{__name__}' has no attribute '{name}'")


if os.environ.get("TORCHCOMMS_PATCH_FOR_COMPILE") == "1":
    # As in the reference (comms/torchcomms/__init__.py): with this variable set, importing the package is enough for
    # communicator methods to be traceable under torch.compile (functional/__init__.py does the registration).
    from . import functional as _functional  # noqa: E402,F401
