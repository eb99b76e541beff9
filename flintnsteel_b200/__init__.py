"""B200-native (sm_100a) token sampler behind the FlintNSteel sampler interface.

The package holds the CUDA kernels and C ABI (``csrc/``, built into ``lib/libfns_b200.so``), a ctypes binding
(``sampler``), the multi-GPU dispatcher (``dispatch``) and seeded synthetic workloads (``workloads``).
"""

__all__ = ["build", "sampler", "workloads"]
