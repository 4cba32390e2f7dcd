"""cudapp_b200: the quantized MoE expert path of CUDA++ rebuilt for B200 (sm_100a).

The product is the C-ABI shared library cudapp_b200/lib/libb200moe.so (sources in csrc/, interface in the
repository's include/*.h). This package only loads it (api.py, ctypes) for tests, benchmarks and the
expert-parallel driver. Importing fails loudly when the library has not been built.
"""
from . import api  # noqa: F401
