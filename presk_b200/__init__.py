"""presk_b200: a B200 (sm_100a) executor for Presk's realized kernels.

The product is the C ABI of include/presk_cuda.h, implemented by
presk_b200/_lib/libpresk_cuda.so (CUDA kernels in presk_b200/csrc). This
package is the thin Python face of that ABI: `Executor` is the reference's
`KernelExec` seam (presk-kernel/src/host.rs:28-95), `Host` its `Backend`
(presk-rt/src/lib.rs:1274-1303). Every computation happens in the library on
the GPU; when the library or a GPU is missing, construction raises.
"""
from . import abi, build
from .api import Comm, DataFile, Executor, Host, PreskError, describe, launch_desc

__all__ = ["abi", "build", "Comm", "DataFile", "Executor", "Host", "PreskError", "describe", "launch_desc"]
