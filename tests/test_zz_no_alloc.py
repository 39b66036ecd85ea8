"""GPU: the allocation-free route sort agrees bit for bit with the workspace-taking entry point.

Collected last on purpose, so that a run stopping at the first failure has already run every
other test. The entry point serves callers that cannot allocate device memory when they route
(a frozen pool, a plugin with a fixed buffer set, a loop that must not stall in cudaMalloc); its
scratch is a built-in device array shared by all calls, so the test makes two calls in a row with
different inputs and checks that the second does not see leftovers of the first.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sort(lib, name, ids, experts, dev, workspace=None):
    from hyper_multicore_b200 import _lib

    entries = ids.numel()
    i32 = dict(dtype=torch.int32, device=dev)
    out = dict(mapping=torch.full((entries,), -7, **i32), sources=torch.full((entries,), -7, **i32),
               row_experts=torch.full((entries,), -7, **i32), counts=torch.full((experts,), -7, **i32),
               cumulative=torch.full((experts,), -7, dtype=torch.int64, device=dev))
    status = _lib.new_status(dev)
    head = [ids.data_ptr(), int(ids.dtype == torch.int64), entries, experts]
    tail = [out["mapping"].data_ptr(), out["sources"].data_ptr(), out["row_experts"].data_ptr(),
            out["counts"].data_ptr(), out["cumulative"].data_ptr(), status.data_ptr(),
            torch.cuda.current_stream(dev).cuda_stream]
    if workspace is not None:
        head += [workspace.data_ptr(), workspace.numel()]
    _lib.check(getattr(lib, name)(*head, *tail))
    torch.cuda.synchronize(dev)
    assert status.tolist()[0] == 0
    return out


def test_static_scratch_sort_matches_workspace_sort_on_two_calls_in_a_row(cuda_device):
    from hyper_multicore_b200 import _lib

    lib = _lib.load()
    dev = cuda_device
    rng = np.random.default_rng(5)
    # second call is smaller and uses fewer experts: stale chunk counts of the first would show
    for tokens, top_k, experts, dtype in ((8192, 8, 256, torch.int64), (777, 3, 40, torch.int32)):
        ids = torch.from_numpy(rng.integers(0, experts, size=(tokens, top_k))).to(dtype).to(dev).reshape(-1)
        workspace = torch.empty(lib.hmc_moe_sort_workspace_bytes(ids.numel(), experts), dtype=torch.uint8, device=dev)
        expected = _sort(lib, "hmc_moe_sort_routes", ids, experts, dev, workspace)
        got = _sort(lib, "hmc_moe_sort_routes_static", ids, experts, dev)
        for name, value in expected.items():
            assert torch.equal(got[name], value), name


def test_static_scratch_sort_rejects_sizes_beyond_its_array(cuda_device):
    from hyper_multicore_b200 import _lib

    lib = _lib.load()
    # 2048 chunks x 4096 experts x 4 bytes = 32 MiB of scratch, the array holds 4 MiB: refused before any launch
    code = lib.hmc_moe_sort_routes_static(None, 1, 2048 * 1024, 4096, None, None, None, None, None, None, None)
    assert code == -3
    assert b"built-in" in lib.hmc_last_error()
