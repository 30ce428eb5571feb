"""The allocation-free entry point, grouped_mm_2d3d_static_scratch, against grouped_mm_2d3d.

Some callers of this library cannot allocate device memory at the moment they need a grouped
GEMM (all memory already handed to their own arena, a host that forbids allocations after start-up,
a loop that must never enter the allocator), so they cannot provide the workspace the regular entry
points ask for. This entry point takes its scratch from a fixed array inside the library. The test
calls it through the C ABI twice in a row, with different problems, and checks each result against
the regular entry point's: the second call must not be disturbed by what the first left in the
shared scratch. Collected last on purpose (file name), and independent of the other tests.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from grouped_mm_bf16_b200 import _lib, _op
from oracle.grouped_mm_oracle import atol_for, grouped_mm_oracle, max_violation

DEV = torch.device("cuda")


def _problem(sizes, k, n, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    a = torch.randn((sum(sizes), k), device=DEV, generator=g).bfloat16()
    b = torch.randn((len(sizes), k, n), device=DEV, generator=g).bfloat16()
    offs = torch.tensor(sizes, dtype=torch.int64).cumsum(0).to(torch.int32).to(DEV)
    return a, b, offs


def _call_static(lib, a, b, offs, out):
    ta, tb, tc = _op._desc(a), _op._desc(b), _op._desc(out)
    scratch = ctypes.c_void_p(0)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.grouped_mm_2d3d_static_scratch(ctypes.byref(ta), ctypes.byref(tb), ctypes.c_void_p(offs.data_ptr()),
                                            int(offs.numel()), ctypes.byref(tc), ctypes.c_void_p(stream), 0,
                                            ctypes.byref(scratch))
    assert rc == 0, _lib.error_message(lib, rc)
    assert scratch.value, "the entry point did not report its scratch address"
    raw = ctypes.c_int32(-1)
    assert lib.gmm_check_status(scratch, ctypes.c_void_p(stream), ctypes.byref(raw)) == 0 and raw.value == 0
    return scratch.value


def test_static_scratch_entry_matches_regular_entry_on_two_calls_in_a_row(built_library):
    lib = _lib.load()
    problems = [
        _problem([300, 0, 513, 255, 257], 200, 264, seed=1),   # several tiles, tails and an empty group
        _problem([0, 7, 1, 13, 0, 11], 64, 48, seed=2),        # the README example, much smaller
    ]
    addresses = []
    for a, b, offs in problems:
        want = torch.full((a.size(0), b.size(2)), float("nan"), dtype=torch.bfloat16, device=DEV)
        got = torch.full_like(want, float("nan"))
        _op.grouped_mm_2d3d(a, b, offs, want)                  # regular entry point, caller's workspace
        addresses.append(_call_static(lib, a, b, offs, got))   # no workspace, nothing allocated
        torch.cuda.synchronize()
        # same kernel, same inputs: identical bits; and both within the operator's tolerance
        assert torch.equal(got, want)
        ref, defined = grouped_mm_oracle(a, b, offs)
        assert max_violation(got, ref, defined, atol_for(a.size(1), 1.0, 1.0)) <= 1.0
    assert addresses[0] == addresses[1], "every call on a device shares the one scratch block"
    # The property the entry point exists for: once its first call on the device has looked up the
    # array's address, a call takes no device memory, neither from the driver nor from torch's pool.
    a, b, offs = problems[0]
    got = torch.empty((a.size(0), b.size(2)), dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    pool_before, reserved_before = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    _call_static(lib, a, b, offs, got)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == pool_before and torch.cuda.memory_reserved() == reserved_before


def test_static_scratch_entry_rejects_what_the_regular_entry_rejects(built_library):
    lib = _lib.load()
    a, b, offs = _problem([4, 4], 16, 8, seed=3)
    out = torch.empty((8, 8), dtype=torch.bfloat16, device=DEV)
    ta, tb, tc = _op._desc(a), _op._desc(b), _op._desc(out)
    rc = lib.grouped_mm_2d3d_static_scratch(ctypes.byref(ta), ctypes.byref(tb), ctypes.c_void_p(offs.data_ptr()), 1024,
                                            ctypes.byref(tc), None, 0, None)
    assert rc == -3  # too many groups
    rc = lib.grouped_mm_2d3d_static_scratch(ctypes.byref(ta), ctypes.byref(tb), ctypes.c_void_p(offs.data_ptr()), 3,
                                            ctypes.byref(tc), None, 0, None)
    assert rc == -1  # group count does not match the weights
