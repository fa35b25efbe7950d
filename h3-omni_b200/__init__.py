"""h3-omni_b200: B200-native attention engine behind the H3-omni GPU primitive ABI.

The product is the CUDA library ``libh3b200_attn.so`` (sources in ``csrc/``, C ABI in
``include/h3b200_attn.h``). This package builds it and binds it through ctypes; there is no
CPU or framework fallback - importing ``native`` without the built library raises.
"""
from .build import build, LIB  # noqa: F401
