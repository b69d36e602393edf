"""The allocation-free projection entry point (q_linear_f32_static).

It exists for hosts that cannot allocate device memory themselves (everything is
owned by their pool, or an allocator call would stall the device at that point):
the split-K partials sit in a static array inside the library. This file is
collected last on purpose; the test passes alone in a fresh process and after the
rest of the suite. It calls the C ABI directly, twice in a row (the array keeps the
first call's contents), and compares with the existing entry points
(q_gemm_splitk into a caller buffer + q_reduce_partials): same kernels, so the
results must be bit-identical; the oracle bound (rtol = atol = 2e-3 on the fp32
product) is checked too."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_static_scratch_projection_matches_caller_buffer_path():
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    from oracle import qwen3_oracle as O
    from starter_b200 import _lib
    from starter_b200.weights import TiledWeight
    lib, check = _lib.lib, _lib.check
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    limit = lib.q_static_scratch_floats()
    assert limit == 2 * 8 * 20480
    gen = torch.Generator().manual_seed(77)
    # two different shapes back to back: the second call meets the first call's leftovers
    for M, N, K in ((4, 6144, 2560), (1, 2560, 4096)):
        w = (torch.randn((N, K), generator=gen) * 0.02).to(torch.bfloat16)
        x = torch.randn((M, K), generator=gen).to(torch.bfloat16)
        wt = TiledWeight.pack(w.cuda())
        xd = x.cuda()
        plan = _lib.plan(M, N, K)
        assert plan.slots * M * N <= limit
        # existing path: caller-allocated partials
        part = torch.empty((plan.slots, M, N), dtype=torch.float32, device="cuda")
        expect = torch.empty((M, N), dtype=torch.float32, device="cuda")
        check(lib.q_gemm_splitk(_ptr(xd), _ptr(wt.data), _ptr(part), M, N, K, stream))
        check(lib.q_reduce_partials(_ptr(part), C.byref(plan), _ptr(expect), stream))
        for _ in range(2):
            got = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
            check(lib.q_linear_f32_static(_ptr(xd), _ptr(wt.data), _ptr(got), M, N, K, stream))
            torch.cuda.synchronize()
            assert torch.equal(got, expect)
        torch.testing.assert_close(got.cpu(), O.linear_fp32(x, w), rtol=2e-3, atol=2e-3)
    # beyond the static array: a clear argument error, nothing launched
    with pytest.raises(ValueError, match="static array"):
        check(lib.q_linear_f32_static(_ptr(xd), _ptr(wt.data), _ptr(got), 8, 151936, 2560, stream))
