"""B200-native (sm_100a) implementation of rocWMMA's matrix-multiply-accumulate path.

    include/rocwmma/        the header-only device API (drop-in for <rocwmma/rocwmma.hpp>)
    include/rocwmma_b200.h  C ABI of the kernels built on it
    rocwmma_b200/csrc/      CUDA sources
    rocwmma_b200/api.py     host drivers over the C ABI (torch tensors for device memory)
    rocwmma_b200/synth.py   seeded synthetic inputs
"""
from ._lib import (BF16, COL_MAJOR, E4M3, E5M2, F16, F32, F64, I8, I32, ROW_MAJOR, XF32,  # noqa: F401
                   B200WmmaError, lib)

__all__ = ["F16", "BF16", "E4M3", "E5M2", "I8", "F32", "XF32", "F64", "I32", "ROW_MAJOR", "COL_MAJOR",
           "B200WmmaError", "lib"]
