"""The scratch-free FP8 entry point (rwkvq_tc_gemm_fp8_static) against the regular one.

Some hosts of this library may not allocate device memory where they call it -- an inference server that has handed
all memory to its own pool, or a serving loop that must stay allocation-free -- so they cannot pass the workspace
rwkvq_tc_gemm_fp8 wants.  The static variant keeps that scratch in an array inside the library.  This test calls it
twice in a row through the C ABI (the array keeps the previous call's contents) and compares each result with the
regular entry point on the same inputs.  Both run the same kernel with the same deterministic order of additions, so
the bar is equality of every bit -- tighter than the 1e-2 relative bound the other FP8 tests use, which would let a
missed re-clear that only disturbs low bits slip through.  The file sorts last so that a failing run has already
executed every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu



def test_static_scratch_entry_point_matches_regular_one():
    import rwkvq_abi as abi
    abi.require_device()
    dev = "cuda"
    g = torch.Generator().manual_seed(11)
    import ctypes
    for m, n, k in ((1, 4096, 4096), (24, 1024, 2560), (16, 512, 16384), (128, 16384, 1024)):
        codes = torch.randint(0, 120, (m, k), generator=g, dtype=torch.uint8).to(dev)          # finite e4m3 codes
        w = torch.randint(0, 120, (n, k), generator=g, dtype=torch.uint8).to(dev)
        amax = torch.tensor([3.5], device=dev)
        wscale = torch.tensor([0.01], device=dev)
        ws = torch.zeros(int(abi.lib().rwkvq_workspace_bytes(m, n, k, 1)), dtype=torch.uint8, device=dev)
        ref = torch.empty((m, n), dtype=torch.float16, device=dev)
        abi.call("rwkvq_tc_gemm_fp8", codes.data_ptr(), k, amax.data_ptr(), 1, w.data_ptr(), k, wscale.data_ptr(),
                 ref.data_ptr(), n, m, n, k, abi.DIV_FULL, 0, ws.data_ptr(), ws.numel(), abi.stream_ptr())
        for _ in range(2):                                   # two calls in a row on the shared built-in scratch
            out = torch.zeros((m, n), dtype=torch.float16, device=dev)
            abi.call("rwkvq_tc_gemm_fp8_static", codes.data_ptr(), k, amax.data_ptr(), 1, w.data_ptr(), k, wscale.data_ptr(),
                     out.data_ptr(), n, m, n, k, abi.DIV_FULL, 0, abi.stream_ptr())
            torch.cuda.synchronize()
            assert torch.equal(out.view(torch.int16), ref.view(torch.int16)), (m, n, k)
            st = ctypes.c_int32(-1)
            abi.call("rwkvq_tc_static_status", ctypes.addressof(st))
            assert st.value == 0


def test_static_scratch_refuses_oversized_shapes():
    import rwkvq_abi as abi
    abi.require_device()
    x = torch.zeros(16, dtype=torch.uint8, device="cuda")
    f = torch.ones(1, device="cuda")
    L = abi.lib()
    # 16 tokens against 65536 weight rows stream the weights with split-K partial sums of 8.4 MB: more than the 8 MiB
    assert L.rwkvq_tc_gemm_fp8_static(x.data_ptr(), 4096, f.data_ptr(), 1, x.data_ptr(), 4096, f.data_ptr(), x.data_ptr(), 65536,
                                      16, 65536, 4096, 1, 0, abi.stream_ptr()) == -7
    assert b"built-in" in L.rwkvq_last_error_string()
