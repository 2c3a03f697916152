"""Import-path parity with the reference's ``torchcomms._transport`` extension module
(comms/torchcomms/transport/_transport.pyi): the same names, served by ``transport``."""
from .transport import *  # noqa: F401,F403
from .transport import RdmaMemory, RdmaMemoryMutableView, RdmaMemoryView, RdmaRemoteBuffer, RdmaTransport  # noqa: F401
