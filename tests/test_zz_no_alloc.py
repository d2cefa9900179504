"""The allocation-free contraction entry point against the ordinary executable path.

Some users of the library cannot allocate device memory at the point of the call (their own arena owns all of HBM,
they run under another allocator's lock, or their serving loop bans allocator traffic). For them
`pjrtx_b200_dot_static_scratch` runs the streaming contraction with its split-K scratch in a fixed array inside the
library. This file is collected last on purpose: a failure here cannot hide a failure anywhere else.
"""
import numpy as np
import pytest

from pjrtx_b200 import PlanBuilder
from pjrtx_b200 import backend as be_mod
from pjrtx_b200 import plan as P
from tests.util import assert_close, run_backend

pytestmark = pytest.mark.gpu


def _reference_through_executable(be, lhs, rhs, dtype):
    b = PlanBuilder()
    pl, pr = b.parameter(dtype, lhs.shape), b.parameter(dtype, rhs.shape)
    b.set_outputs([b.dot_general(pl, pr, [1], [0])])
    return run_backend(be, b, [lhs, rhs])[0]


@pytest.mark.parametrize("dtype,m,k,n", [(P.BF16_CODE, 1, 4096, 4096), (P.BF16_CODE, 4, 1000, 2048), (P.F32, 2, 512, 1024),
                                         (P.F16, 8, 4096, 6144)])
def test_static_scratch_matches_executable_twice_in_a_row(gpu_backend, dtype, m, k, n):
    import torch

    be = gpu_backend
    rng = np.random.default_rng(17)
    dt = P.np_dtype(dtype)
    lhs = rng.standard_normal((m, k), dtype=np.float32).astype(dt)
    rhs = rng.standard_normal((k, n), dtype=np.float32).astype(dt)
    want = _reference_through_executable(be, lhs, rhs, dtype)
    exact = lhs.astype(np.float64) @ rhs.astype(np.float64)
    # Device memory for the raw-pointer call comes from torch: the entry point itself must not allocate.
    as_bytes = lambda a: torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).cuda()
    dl, dr = as_bytes(lhs), as_bytes(rhs)
    out = torch.full((m * n * dt.itemsize,), 0xAB, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    for call in range(2):  # the second call finds the array as the first one left it
        out.fill_(0xAB)
        torch.cuda.synchronize()
        # What the driver reports as free counts every allocation on the GPU, whoever made it (the first call has
        # already loaded the kernel and resolved the array); the library's own accounting must not move either.
        free_before = torch.cuda.mem_get_info()[0] if call else None
        live_before = be.memory_stats(0)
        torch_before = torch.cuda.memory_allocated()
        be.dot_static_scratch(dtype, dl.data_ptr(), dr.data_ptr(), out.data_ptr(), m, k, n)
        be.dot_static_scratch_status(0)  # waits for the stream; raises if a bounded device-side wait gave up
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == torch_before
        assert be.memory_stats(0) == live_before
        if call:
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.current_device() == 0
        got = out.cpu().numpy().view(dt).reshape(m, n)
        assert_close(got, want, 1e-5 if dtype == P.F32 else 2e-2, what=f"call {call} vs the executable path")
        assert_close(got, exact, 1e-5 if dtype == P.F32 else 2e-2, what=f"call {call} vs the float64 product")


def test_static_scratch_rejects_what_does_not_fit(gpu_backend):
    import torch

    be = gpu_backend
    x = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    with pytest.raises(be_mod.BackendError, match="static scratch holds"):
        # 8 rows against 64 x 2,000,000 needs far more than 8 MiB of partial sums; refused before any pointer is used
        be.dot_static_scratch(P.BF16_CODE, x.data_ptr(), x.data_ptr(), x.data_ptr(), 8, 64, 2_000_000)
    with pytest.raises(be_mod.BackendError, match="1 <= m <= 8"):
        be.dot_static_scratch(P.BF16_CODE, x.data_ptr(), x.data_ptr(), x.data_ptr(), 9, 64, 256)
