"""tllm_sample_noalloc, the sampling entry point for callers that cannot allocate device memory.

It is called here the way such a caller would call it: through the exported C symbol of the shared
object, with raw device pointers, and with no scratch buffer.  Its tokens must equal those of the
regular entry point (tllm_sample, which gets scratch from the caller) for the same inputs, on two
calls in a row with different inputs, since both calls share the library's built-in scratch array
and the second one finds the first one's leftovers in it.  A request larger than the built-in array
must be refused without launching anything.

This file sorts last on purpose, so that a run that stops at the first failure has already run
every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_FLOATS = 1 << 20


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def make_inputs(n, v, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(n, v, generator=g) * 3).to(DEV)
    temps = torch.tensor([0.7, 1.0, 1.3, 0.0][:n] + [0.9] * max(0, n - 4))[:n].to(DEV)
    top_k = torch.tensor(([50, 0, 5, 50] + [20] * n)[:n], dtype=torch.int32).to(DEV)
    top_p = torch.tensor(([0.95, 1.0, 0.5, 0.95] + [0.8] * n)[:n]).to(DEV)
    seeds = (torch.arange(n, dtype=torch.int64) * 104729 + seed).to(DEV)
    counters = (torch.arange(n, dtype=torch.int64) % 7).to(DEV)
    return logits, temps, top_k, top_p, seeds, counters


def test_noalloc_entry_point_matches_the_regular_one_twice_in_a_row():
    from tiny_llm_b200.ops import build
    torch.cuda.set_device(0)
    lib = ctypes.CDLL(build.compile_library("sampling"))      # the exported C symbols, nothing else
    lib.tllm_last_error.restype = ctypes.c_char_p
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (n, v) in enumerate([(6, 32000), (8, 4099)]):
        logits, temps, top_k, top_p, seeds, counters = make_inputs(n, v, seed=17 + call)
        want = torch.full((n,), -1, dtype=torch.int32, device=DEV)
        work = torch.empty(n * v, device=DEV)
        rc = lib.tllm_sample(ptr(logits), ptr(work), n, v, ptr(temps), ptr(top_k), ptr(top_p), ptr(seeds),
                             ptr(counters), ptr(want), ctypes.c_void_p(0), stream)
        assert rc == 0, lib.tllm_last_error().decode()
        got = torch.full((n,), -2, dtype=torch.int32, device=DEV)
        before = torch.cuda.memory_allocated()
        rc = lib.tllm_sample_noalloc(ptr(logits), n, v, ptr(temps), ptr(top_k), ptr(top_p), ptr(seeds), ptr(counters),
                                     ptr(got), stream)
        assert rc == 0, lib.tllm_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert got.tolist() == want.tolist(), (call, got.tolist(), want.tolist())
        assert all(0 <= t < v for t in got.tolist())


def test_noalloc_entry_point_refuses_what_its_array_cannot_hold():
    from tiny_llm_b200.ops import build
    torch.cuda.set_device(0)
    lib = ctypes.CDLL(build.compile_library("sampling"))
    lib.tllm_last_error.restype = ctypes.c_char_p
    n, v = 9, MAX_FLOATS // 8          # one row too many
    out = torch.full((n,), -3, dtype=torch.int32, device=DEV)
    tiny = torch.zeros(16, device=DEV)  # never read: the call must be refused before any launch
    rc = lib.tllm_sample_noalloc(ptr(tiny), n, v, ptr(tiny), ptr(tiny), ptr(tiny), ptr(tiny), ptr(tiny), ptr(out),
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -1
    msg = lib.tllm_last_error().decode()
    assert "scratch" in msg and str(MAX_FLOATS) in msg
    torch.cuda.synchronize()
    assert out.tolist() == [-3] * n
