"""Run-time compilation of a kernel on the fragment API (the reference's hipRTC sample,
samples/hipRTC_gemm.cpp).  Compilation needs no GPU and proves the device headers are
self-contained; running it is a GPU test."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle as O
from rocwmma_b200 import rtc
from tests.rtc_kernels import TILE32_BF16_GEMM

REF_RTC_SAMPLE = os.path.join(O.reference_dir(), "samples", "hipRTC_gemm.cpp")


def test_headers_compile_under_nvrtc():
    ptx = rtc.compile_to_ptx(TILE32_BF16_GEMM, "tile32_gemm.cu")
    text = ptx.decode(errors="replace")
    assert ".target sm_100a" in text
    assert "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32" in text
    assert "tile32_gemm" in text


def test_all_api_headers_compile_under_nvrtc():
    src = """
    #include <rocwmma/rocwmma.hpp>
    #include <rocwmma/rocwmma_coop.hpp>
    #include <rocwmma/rocwmma_transforms.hpp>
    #include <rocwmma/rocwmma_block.hpp>
    using namespace rocwmma;
    extern "C" __global__ void k(float16_t const* a, float16_t* o, uint32_t ld)
    {
        fragment<matrix_a, 32, 32, 16, float16_t, row_major> f;
        load_matrix_coop_sync(f, a, ld, threadIdx.x / 32, blockDim.x / 32);
        auto t = applyTranspose(f);
        store_matrix_sync(o, t, ld);
        synchronize_workgroup();
    }
    """
    assert b"sm_100a" in rtc.compile_to_ptx(src)


@pytest.mark.skipif(not os.path.isfile(REF_RTC_SAMPLE), reason="reference tree not mounted")
def test_reference_rtc_kernel_source_compiles_unmodified():
    """The kernel source string of the reference's own run-time compilation sample
    (samples/hipRTC_gemm.cpp:73-173, a raw string literal handed to hipRTC) goes through NVRTC
    against these headers as it is: read from the mounted tree, never stored here."""
    text = open(REF_RTC_SAMPLE).read()
    start = text.index('R"(') + 3
    source = text[start:text.index(')";', start)]
    assert "#include <rocwmma/rocwmma.hpp>" in source and "gemm_rocwmma_d" in source
    ptx = rtc.compile_to_ptx(source, "reference_hiprtc_kernel.cu").decode(errors="replace")
    assert ".target sm_100a" in ptx and "gemm_rocwmma_d" in ptx
    assert "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32" in ptx


def test_compile_errors_are_reported():
    with pytest.raises(RuntimeError, match="NVRTC compilation failed"):
        rtc.compile_to_ptx("#include <rocwmma/rocwmma.hpp>\n__global__ void k(){ nonsense; }")


@pytest.mark.gpu
def test_runtime_compiled_gemm_matches_the_oracle():
    import torch

    from rocwmma_b200 import synth
    torch.cuda.init()
    torch.zeros(1, device="cuda")          # make the primary context current
    m = n = k = 256
    a = synth.matrix(21, 1, synth.BF16, m, k)
    bt = synth.matrix(21, 2, synth.BF16, n, k)
    c = synth.matrix(21, 3, synth.F32, m, n)
    want = O.gemm(O.BF16, O.F32, m, n, k, a, bt, c, 2.1, 2.1)
    ta = torch.from_numpy(a.view(np.int16)).cuda()
    tb = torch.from_numpy(bt.view(np.int16)).cuda()
    tc = torch.from_numpy(c).cuda()
    td = torch.full((m * n,), float("nan"), device="cuda")
    mod = rtc.RtcModule(TILE32_BF16_GEMM, "tile32_gemm")
    u32, f32, ptr = C.c_uint32, C.c_float, C.c_void_p
    args = [u32(m), u32(n), u32(k), ptr(ta.data_ptr()), ptr(tb.data_ptr()), ptr(tc.data_ptr()),
            ptr(td.data_ptr()), f32(2.1), f32(2.1)]
    # 2 x 2 warps per block: 64 x 64 outputs per block
    mod.launch((m // 64, n // 64, 1), (64, 2, 1), args,
               stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    err = O.max_rel_err(O.F32, td.cpu().numpy(), want)
    assert 0 <= err <= 2e-3, err
    mod.unload()
