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

# The kernel of the reference's run-time compilation sample, unchanged in its body
# (samples/hipRTC_gemm.cpp:106-165): bf16 inputs, fp32 accumulate and C/D, one 16x16x16
# tile per warp.
BF16_SIMPLE_GEMM_SOURCE = r"""
#include <rocwmma/rocwmma.hpp>

using rocwmma::accumulator;
using rocwmma::bfloat16_t;
using rocwmma::col_major;
using rocwmma::float32_t;
using rocwmma::matrix_a;
using rocwmma::matrix_b;
using rocwmma::row_major;

constexpr int ROCWMMA_M = 16;
constexpr int ROCWMMA_N = 16;
constexpr int ROCWMMA_K = 16;

extern "C" __global__ void gemm_rocwmma_d(uint32_t          m,
                                          uint32_t          n,
                                          uint32_t          k,
                                          bfloat16_t const* a,
                                          bfloat16_t const* b,
                                          float32_t const*  c,
                                          float32_t*        d,
                                          uint32_t          lda,
                                          uint32_t          ldb,
                                          uint32_t          ldc,
                                          uint32_t          ldd,
                                          float32_t         alpha,
                                          float32_t         beta)
{
    auto fragA = rocwmma::fragment<matrix_a, ROCWMMA_M, ROCWMMA_N, ROCWMMA_K, bfloat16_t, row_major>();
    auto fragB = rocwmma::fragment<matrix_b, ROCWMMA_M, ROCWMMA_N, ROCWMMA_K, bfloat16_t, col_major>();
    auto fragC   = rocwmma::fragment<accumulator, ROCWMMA_M, ROCWMMA_N, ROCWMMA_K, float32_t>();
    auto fragAcc = rocwmma::fragment<accumulator, ROCWMMA_M, ROCWMMA_N, ROCWMMA_K, float32_t>();

    rocwmma::fill_fragment(fragAcc, 0.0f);

    auto majorWarp = (blockIdx.x * blockDim.x + threadIdx.x) / rocwmma::Constants::AMDGCN_WAVE_SIZE;
    auto minorWarp = (blockIdx.y * blockDim.y + threadIdx.y);

    auto cRow = majorWarp * ROCWMMA_M;
    auto cCol = minorWarp * ROCWMMA_N;

    if(cRow < m && cCol < n)
    {
        for(uint32_t i = 0; i < k; i += ROCWMMA_K)
        {
            rocwmma::load_matrix_sync(fragA, a + (cRow * lda + i), lda);
            rocwmma::load_matrix_sync(fragB, b + (i + cCol * ldb), ldb);
            rocwmma::mma_sync(fragAcc, fragA, fragB, fragAcc);
        }
        rocwmma::load_matrix_sync(fragC, c + (cRow * ldc + cCol), ldc, rocwmma::mem_row_major);
        for(int i = 0; i < fragC.num_elements; ++i)
        {
            fragC.x[i] = alpha * fragAcc.x[i] + beta * fragC.x[i];
        }
        rocwmma::store_matrix_sync(d + (cRow * ldd + cCol), fragC, ldd, rocwmma::mem_row_major);
    }
}
"""


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
