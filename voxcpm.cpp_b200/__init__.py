"""B200 attention engine for VoxCPM.cpp — Python access to the C ABI.

The product is ``libvoxattn.so`` (hand-written CUDA for sm_100a behind ``include/vox_attn.h``).
This package only loads it with ``ctypes`` and wraps the entry points so that tests and the
benchmark can pass torch tensors (used purely as device memory).  There is no CPU path: if
the library is missing or cannot be loaded, importing ``lib()`` raises.
"""
from __future__ import annotations

from .binding import (  # noqa: F401
    F16, F32, LINEAR_PLAIN, LINEAR_RESIDUAL, LINEAR_SWIGLU, Q8_0, AttnArgs, DecodeArgs, Engine, Group, GroupConfig, KVCache, KVConfig,
    LinearArgs, LocditArgs, StepBuffers,
    Tensor, VoxError, declared_symbols, lib, library_path, partition_streams,
)
