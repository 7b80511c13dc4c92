"""me_sample_static, the sampling entry point that allocates nothing, through its exported C symbol.

It serves hosts that cannot call cudaMalloc when they need a token (a fixed memory plan, a path that
must not synchronise the device, no allocator at hand): the work buffer that ``me_sample`` takes from
its caller lives inside the library here.  This file is collected last (see conftest.py) so that a run
that stops at the first failure has already run every other test; it passes alone and after the others.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mini_engine_b200 import ops
    lib = ops.require_extension()
    fn = lib.me_sample_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return ops, lib, fn


def _inputs(S, V, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(S, V, generator=g) * 2).cuda()
    temps = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.0, 0.4, 2.0][:S] + [0.9] * max(0, S - 7)).cuda()
    seeds = torch.arange(11, 11 + S, dtype=torch.int32).cuda()
    pos = torch.arange(100 * seed, 100 * seed + S, dtype=torch.int32).cuda()
    return logits, temps, seeds, pos


def test_static_entry_point_matches_the_allocating_one_twice_in_a_row():
    ops, lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # One call beforehand: the first call on a device looks the built-in buffer's address up, and the first launch
    # of a kernel makes the driver load it; neither is what the memory check below is about.
    logits, temps, seeds, pos = _inputs(2, 300, seed=9)
    first = torch.empty(2, dtype=torch.int32, device="cuda")
    assert fn(logits.data_ptr(), logits.stride(0), temps.data_ptr(), seeds.data_ptr(), pos.data_ptr(), first.data_ptr(),
              2, 300, stream) == 0, lib.me_last_error().decode()
    torch.cuda.synchronize()
    for call, (S, V) in enumerate(((7, 5003), (3, 151936))):          # two calls in a row share the built-in buffer
        logits, temps, seeds, pos = _inputs(S, V, seed=call + 1)
        want = torch.empty(S, dtype=torch.int32, device="cuda")
        ops.sample(logits, temps, seeds, pos, want)                       # existing entry point, caller's buffer
        got = torch.full((S,), -1, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()                            # torch's own allocator ...
        free_before, _ = torch.cuda.mem_get_info()                        # ... and the driver's count of free bytes, which
        rc = fn(logits.data_ptr(), logits.stride(0), temps.data_ptr(), seeds.data_ptr(), pos.data_ptr(), got.data_ptr(),
                S, V, stream)                                             # a cudaMalloc inside the library would lower
        assert rc == 0, lib.me_last_error().decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before
        assert free_after >= free_before, f"{free_before - free_after} bytes of device memory were taken during the call"
        assert got.tolist() == want.tolist()                              # same kernels, same arithmetic: same tokens


def test_static_entry_point_refuses_sizes_beyond_its_buffer():
    ops, lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    logits, temps, seeds, pos = _inputs(2, 1000, seed=3)
    out = torch.empty(2, dtype=torch.int32, device="cuda")
    args = (logits.data_ptr(), logits.stride(0), temps.data_ptr(), seeds.data_ptr(), pos.data_ptr(), out.data_ptr())
    assert fn(*args, 65, 1000, stream) != 0 and b"rows" in lib.me_last_error()
    assert fn(*args, 2, 262145, stream) != 0 and b"vocabulary" in lib.me_last_error()
    assert fn(*args, 0, 1000, stream) == 0
    # a call that succeeds leaves no message of an earlier failure's kind behind
    assert fn(*args, 2, 1000, stream) == 0
    torch.cuda.synchronize()
    assert b"no usable CUDA device" not in lib.me_last_error()
