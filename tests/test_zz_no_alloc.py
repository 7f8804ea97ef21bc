"""The allocation-free Q4_K product (knj_q4k_matmul_noalloc_launch) through the
C-ABI. Some callers cannot allocate device memory at call time and have no
workspace to pass -- a serving loop whose pool is fully given to resident
experts, a plug-in host handed only inputs and outputs -- so this entry point
keeps its scratch in a fixed array inside the library. The test checks that it
returns the same result as the workspace-taking entry point, twice in a row (the
second call runs on whatever the first left in the shared scratch), that a
problem too large for the built-in array is refused with a clear message, and
that no device allocation happens during the calls.

Collected last on purpose (file name sorts after the other tests)."""
import ctypes as C

import numpy as np
import pytest
import torch

from kanjoos_b200 import synth

pytestmark = pytest.mark.gpu


def _call(L, W, x, y):
    m, n_in = x.shape
    return L.knj_q4k_matmul_noalloc_launch(C.c_void_p(W.data_ptr()), n_in, W.shape[0], C.c_void_p(x.data_ptr()), 0, n_in, m,
                                           C.c_void_p(y.data_ptr()), W.shape[0],
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_matches_workspace_entry_point_twice():
    from kanjoos_b200 import _lib, ops
    L = _lib.lib()
    _lib.check(L.knj_dev_open(0))
    rng = np.random.Generator(np.random.Philox(99))
    W = torch.from_numpy(synth.q4k_rows(rng, 768, 2048)).cuda()
    xs = [torch.from_numpy(rng.standard_normal((m, 2048)).astype(np.float32)).cuda() for m in (1, 5)]
    wants = [ops.q4k_matmul(W, x) for x in xs]  # existing entry point, caller-provided workspace
    ys = [torch.full((x.shape[0], 768), -12345.0, dtype=torch.float32, device="cuda") for x in xs]
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    free_before = torch.cuda.mem_get_info()[0]
    for x, y in zip(xs, ys):  # two calls in a row share the built-in scratch
        _lib.check(_call(L, W, x, y))
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated during the calls"
    for y, want in zip(ys, wants):
        # same kernels on the same inputs: bit equal (the tests' tolerance for this product is 1e-5 rel-RMSE)
        assert torch.equal(y, want)
    # again in the opposite order: stale contents of the other problem do not leak into the result
    for x, y, want in reversed(list(zip(xs, ys, wants))):
        y.fill_(-12345.0)
        _lib.check(_call(L, W, x, y))
        torch.cuda.synchronize()
        assert torch.equal(y, want)


def test_noalloc_refuses_what_does_not_fit():
    from kanjoos_b200 import _lib
    L = _lib.lib()
    limit = L.knj_q4k_matmul_noalloc_max_scratch()
    assert limit == 64 << 10
    m, n_in = 20000, 256
    assert L.knj_q4k_matmul_workspace_bytes(m, n_in) > limit
    W = torch.zeros((16, n_in // 256, 144), dtype=torch.uint8, device="cuda")
    x = torch.zeros((m, n_in), dtype=torch.float32, device="cuda")
    y = torch.zeros((m, 16), dtype=torch.float32, device="cuda")
    assert _call(L, W, x, y) == -4
    msg = L.knj_last_error_string().decode()
    assert "built-in array" in msg and "knj_q4k_matmul_launch" in msg
