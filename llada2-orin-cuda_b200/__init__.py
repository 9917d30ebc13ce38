"""B200-native block-diffusion attention over the int4 "4c/4" KV cache, and its block-commit quantiser.

The package holds the CUDA sources (csrc/), the build step for the C-ABI shared library, the ctypes binding that
mirrors the reference's `attn` operator interface, the seeded workload generator and the request-sharding
helper. There is no CPU or PyTorch fallback: every compute entry point needs the built CUDA library and a GPU.
"""
from . import sharding, workload  # noqa: F401
