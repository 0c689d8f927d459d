"""anode_b200: anode's train-mode batch-norm + ReLU hot path, rebuilt for B200 (sm_100a).

`anode_b200.ops` mirrors the reference's operator surface over the C ABI of
`libanode_routines_gpu.so` (declared in include/anode_routines_gpu.h).  Build the library
with `python -m anode_b200.build`; nothing here falls back to a CPU or PyTorch path.
"""
from . import _lib  # noqa: F401

__all__ = ["ops", "build", "_lib"]
