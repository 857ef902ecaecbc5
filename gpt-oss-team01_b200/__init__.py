"""B200-native GPT-OSS MoE FFN block (router, top-4 gating, expert grouping, grouped GEMMs with fused
SwiGLU / gate-weighted combine, cross-GPU combine) behind a C ABI.

The directory name carries a hyphen, so the package is imported under the alias ``gptoss_b200``
(see ``__graft_entry__.load_package``).  Submodules:

* ``synth``   seeded synthetic tensors (same bits on CPU and GPU)
* ``binfmt``  the reference's flat ``model.bin`` checkpoint format
* ``capi``    ctypes binding of ``include/gptoss_b200.h`` (loads the CUDA shared library)
* ``moe``     host-side operator interface mirroring the reference's per-layer launchers
"""
from . import binfmt, synth  # noqa: F401

__all__ = ["binfmt", "synth"]
