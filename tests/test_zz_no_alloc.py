"""The sampler's entry point for callers that cannot allocate (`llmk_sample_static`).

Some users of the kernel library sample from a place where device memory must not be
allocated: they run inside another program's runtime that owns the GPU's memory, or on a path
where cudaMalloc is forbidden.  For them the library keeps the first-stage scratch in a fixed
device array and exports one C symbol that takes only inputs and outputs.  This test calls that
symbol directly through ctypes, twice in a row with different logits (the second call finds the
first call's leftovers in the shared array), and checks that the ids are exactly those of the
ordinary entry point, which gets its scratch from the caller.  It also checks that more rows than
the array holds are refused.

The file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It passes alone in a fresh process as well as after the others.
"""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from llmgen_b200.kernels import build
    lib = build.load("sampling")
    lib.llmk_sample_static.restype = c_int
    lib.llmk_sample_static_max_rows.restype = c_int
    return lib


def _call_static(lib, out, logits, temps, seed):
    n, V = logits.shape
    return lib.llmk_sample_static(c_void_p(out.data_ptr()), c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)),
                                  c_void_p(temps.data_ptr()), c_void_p(seed.data_ptr()), c_int(n), c_int(V),
                                  c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_sampler_equals_the_ordinary_one_on_two_calls_in_a_row():
    from llmgen_b200.kernels import ops
    lib = _lib()
    torch.manual_seed(31)
    for call, (S, V) in enumerate([(7, 1013), (5, 389)]):
        logits = (torch.randn(S, V) * 3).cuda()
        temps = torch.tensor([0.0, 0.8, 1.3, 0.0, 0.5, 2.0, 0.0][:S]).cuda()
        seed = torch.tensor([977 + call], dtype=torch.int64, device="cuda")
        want = torch.zeros(S, dtype=torch.int32, device="cuda")
        scratch = ops.sample_scratch(S, "cuda")
        ops.sample(want, logits, temps, seed, scratch)
        got = torch.full((S,), -1, dtype=torch.int32, device="cuda")
        rc = _call_static(lib, got, logits, temps, seed)
        assert rc == 0, lib.llmk_last_error().decode()
        torch.cuda.synchronize()
        assert got.cpu().tolist() == want.cpu().tolist()
        greedy = [r for r in range(S) if float(temps[r]) <= 0]
        assert [got[r].item() for r in greedy] == [int(logits[r].argmax()) for r in greedy]


def test_static_scratch_sampler_refuses_more_rows_than_it_holds():
    lib = _lib()
    limit = lib.llmk_sample_static_max_rows()
    assert limit > 0
    S, V = limit + 1, 16
    logits = torch.zeros(S, V, device="cuda")
    temps = torch.zeros(S, device="cuda")
    seed = torch.tensor([1], dtype=torch.int64, device="cuda")
    out = torch.full((S,), -7, dtype=torch.int32, device="cuda")
    rc = _call_static(lib, out, logits, temps, seed)
    assert rc != 0
    assert str(limit) in lib.llmk_last_error().decode()
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [-7] * S        # nothing ran
