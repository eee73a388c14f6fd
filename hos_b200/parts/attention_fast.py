"""Python face of the tensor-core attention kernels (csrc/attention_decode.cu,
csrc/attention_prefill.cu), compiled per head size."""
from __future__ import annotations

ENABLED = False     # switched on once the kernels are built and checked


def attend(mixer, qkv, att, step, cache, packed: bool) -> bool:
    """Runs the tensor-core kernel if it takes the case; False hands it to the plain kernel."""
    return False
