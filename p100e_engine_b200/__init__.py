"""B200 (sm_100a) paged-KV full-attention path, drop-in for the reference engine's p100e::fast attention entry points.

csrc/        hand-written CUDA kernels and the extern "C" boundary (include/b200attn.h)
lib.py       ctypes binding of the C ABI
fast.py      host-side mirror of the reference's p100e::fast attention interface over torch tensors
pool.py      paged KV pool / block tables / step descriptors the kernels index
dist.py      multi-GPU wrapper: KV-head shards, 2-way sequence split with an NCCL (O, m, l) merge
"""
from . import lib  # noqa: F401
