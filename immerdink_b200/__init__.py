"""B200-native FP64 tensor contractions by Ozaki scheme II (drop-in for immerdink).

- `immerdink_b200.host`: host queries (workspace sizes, lowering, error estimates); no GPU.
- device API: `Plan`, `contract`, `PlanCache`, `Pack`, `PackedBuffer`, `DeviceArray`,
  `workspace_size` on caller-owned
  float64 CUDA arrays (`__cuda_array_interface__`, DLPack, raw pointers) over the C ABI of
  libimmerdink.so. Importing loads no library; libimmerdink.so is loaded on first use and the
  call fails loudly when it is missing (there is no CPU fallback).
- `immerdink_b200.hostpipe.HostContraction`: operands in pinned host memory, copies overlapped
  with the contraction slab by slab (imported on demand: needs torch and cuda-python).
"""
from .device import (AliasingError, AllocFailedError, CudaError, DeviceArray, Handle,  # noqa: F401
                     ImmerdinkError, InsufficientWorkspaceError, InvalidValueError, Layout,
                     MisalignedError, NotSupportedError, Pack, PackedBuffer, PackMismatchError,
                     PackRecord, Plan, PlanCache, pack_spec,
                     contract, default_handle, default_plan_cache, get_cai_stream_policy,
                     load_library, set_cai_stream_policy, workspace_size)
