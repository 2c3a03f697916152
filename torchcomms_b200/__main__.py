"""``python -m torchcomms_b200``: what is installed and what this machine looks like.

Prints the package's backends, the extension it loaded, PyTorch / CUDA versions, the configuration
keys read so far, and - where NVML answers - the GPU topology.  Read-only."""
from __future__ import annotations

import os
import sys


def main() -> int:
    import torch

    import torchcomms_b200 as tc
    from torchcomms_b200 import _comms

    print(f"torchcomms_b200 at {os.path.dirname(tc.__file__)}")
    print(f"  extension      {_comms.__file__}")
    print(f"  backends       {', '.join(sorted(tc.built_backends()))}")
    print(f"  torch          {torch.__version__} (CUDA {torch.version.cuda}, {torch.cuda.device_count()} visible GPU(s))")
    print(f"  healthy        {tc.healthy()}")
    knobs = tc.knobs()
    if knobs:
        print("  configuration keys read so far:")
        for key, (value, source) in sorted(knobs.items()):
            print(f"    {key} = {value}  [{source}]")
    try:
        from torchcomms_b200.utils.topology import discover

        print(discover().summary())
    except Exception as e:  # noqa: BLE001 - NVML missing or no driver: not an error for this report
        print(f"  topology       unavailable ({type(e).__name__}: {e})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
