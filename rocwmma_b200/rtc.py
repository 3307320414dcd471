"""Run-time compilation of kernels written on the fragment API (NVRTC).

The analogue of the reference's hipRTC sample (rocWMMA samples/hipRTC_gemm.cpp:26-400):
a kernel given as a source string is compiled for sm_100a at run time against the
headers under include/rocwmma, loaded through the driver API and launched.  This also
proves that the device headers are self-contained: under NVRTC no host header exists.

    mod = RtcModule(source, "gemm_rocwmma_d")
    mod.launch(grid, block, args...)          # args: ints / floats / device pointers
"""
from __future__ import annotations

import ctypes as C
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INCLUDE = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")

def _nvrtc():
    try:
        from cuda.bindings import nvrtc
    except ImportError:  # older cuda-python layout
        from cuda import nvrtc
    return nvrtc


def compile_to_ptx(source: str, name: str = "kernel.cu", extra_options=()) -> bytes:
    """Compiles `source` for sm_100a; raises RuntimeError with the compiler log on failure.
    Needs no GPU."""
    nvrtc = _nvrtc()
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), name.encode(), 0, [], [])
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        raise RuntimeError(f"nvrtcCreateProgram: {err}")
    opts = [b"--gpu-architecture=sm_100a", b"-std=c++17", b"-lineinfo",
            f"-I{os.path.join(ROOT, 'include')}".encode(), f"-I{CUDA_INCLUDE}".encode(),
            *[o.encode() for o in extra_options]]
    err, = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    _, n = nvrtc.nvrtcGetProgramLogSize(prog)
    log = b" " * n
    nvrtc.nvrtcGetProgramLog(prog, log)
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        raise RuntimeError("NVRTC compilation failed:\n" + log.decode(errors="replace"))
    _, n = nvrtc.nvrtcGetPTXSize(prog)
    ptx = b" " * n
    nvrtc.nvrtcGetPTX(prog, ptx)
    nvrtc.nvrtcDestroyProgram(prog)
    return ptx


class RtcModule:
    """A run-time compiled kernel loaded into the current CUDA context (driver API)."""

    def __init__(self, source: str, entry: str, extra_options=()):
        from cuda.bindings import driver
        self._drv = driver
        ptx = compile_to_ptx(source, entry + ".cu", extra_options)
        err, self.module = driver.cuModuleLoadData(ptx)
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"cuModuleLoadData: {err}")
        err, self.function = driver.cuModuleGetFunction(self.module, entry.encode())
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"cuModuleGetFunction: {err}")

    def launch(self, grid, block, args, stream=0, shared_bytes=0):
        """args: sequence of ctypes scalars (c_uint32, c_float, c_void_p ...)."""
        drv = self._drv
        holders = list(args)
        ptrs = (C.c_void_p * len(holders))(*[C.addressof(h) for h in holders])
        err, = drv.cuLaunchKernel(self.function, grid[0], grid[1], grid[2], block[0], block[1],
                                  block[2], shared_bytes, stream, C.addressof(ptrs), 0)
        if err != drv.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"cuLaunchKernel: {err}")

    def unload(self):
        self._drv.cuModuleUnload(self.module)
