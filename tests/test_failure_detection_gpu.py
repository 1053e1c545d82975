"""A bounded wait that runs out is seen by the host on the product path.

The engine's tcgen05 kernels wait on mbarriers with a time limit; when it passes they record a code in
the device's status word and return.  Here a test-only kernel (tests/wait_probe.cu) runs that very
wait on a barrier at which nothing arrives, built with a limit of five milliseconds.  Nothing faults
or hangs: the kernel ends by itself, and the tests check that the word reaches the host with the
sampled ids (the generation path) and through `check_status` (replay and bench), that it is cleared,
and that the device goes on computing right results."""
import ctypes
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HERE = os.path.dirname(os.path.abspath(__file__))
LIMIT_NS = 5_000_000


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    from tiny_llm_b200.ops import build
    out = str(tmp_path_factory.mktemp("wait_probe") / "wait_probe.so")
    cmd = [build.nvcc_path()] + build.ARCH_FLAGS + build.BASE_FLAGS + [
        f"-DTLLM_WAIT_LIMIT_NS={LIMIT_NS}ull", "-I", build.CSRC, "-o", out, os.path.join(HERE, "wait_probe.cu"), "-lcuda"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    lib = ctypes.CDLL(out)
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)

    def run(code):
        from tiny_llm_b200 import ops
        status = ops.status_word(DEV)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert lib.tllm_wait_probe(ctypes.c_void_p(status.data_ptr()), code, ctypes.c_void_p(waited.data_ptr()), stream) == 0
        return waited
    return run


def linear_is_right():
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(0)
    a = torch.randn(200, 256, generator=g).bfloat16().to(DEV)
    w = torch.randn(384, 256, generator=g).bfloat16().to(DEV)
    out = torch.empty(200, 384, dtype=torch.bfloat16, device=DEV)
    ops.linear(a, w, out)
    ref = a.float().cpu() @ w.float().cpu().T
    assert float((out.float().cpu() - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max())


def test_check_status_raises_clears_and_the_device_goes_on(probe):
    from tiny_llm_b200 import ops
    torch.cuda.set_device(0)
    ops.check_status()   # clean before
    waited = probe(2)
    torch.cuda.synchronize()
    ns = int(waited.item())
    assert LIMIT_NS <= ns < 1_000_000_000, ns          # the wait gave up at its limit, not later
    with pytest.raises(ops.KernelError, match="gave up waiting"):
        ops.check_status()
    ops.check_status()   # cleared by the raise
    linear_is_right()
    ops.check_status()


def test_the_status_word_travels_with_the_sampled_ids(probe):
    from tiny_llm_b200 import ops
    from tiny_llm_b200.sampling import Sampler, SamplingParams
    torch.cuda.set_device(0)
    sampler = Sampler(DEV, 300, max_rows=4)
    logits = torch.randn(3, 300, generator=torch.Generator().manual_seed(1)).to(DEV)
    greedy = [SamplingParams(do_sample=False)] * 3
    drawn = [SamplingParams(do_sample=True, temperature=0.9, top_k=20, top_p=0.9, seed=i) for i in range(3)]
    want = logits.argmax(dim=1).tolist()
    assert sampler.sample(logits, greedy, [0, 0, 0]) == want
    for params in (greedy, drawn):
        probe(3)                                        # "a kernel of this step gave up"
        ticket = sampler.launch(logits, params, [0, 0, 0])
        with pytest.raises(ops.KernelError, match="code 3"):
            sampler.collect(ticket)                     # the ids are not handed out
        assert int(ops.status_word(DEV).item()) == 0    # cleared: the next step starts clean
        assert sampler.sample(logits, greedy, [0, 0, 0]) == want
    linear_is_right()


def test_generation_raises_when_a_step_gave_up(probe, model_dirs):
    from tiny_llm_b200 import Pipeline, ops
    pipe = Pipeline(model_dirs["A"], dtype="bfloat16", max_tokens=256, max_requests=2)
    good = pipe.apply([[9, 8, 7]], max_new_tokens=6, do_sample=False, ignore_eos=True)[0]
    probe(1)
    with pytest.raises(ops.KernelError):
        pipe.apply([[9, 8, 7]], max_new_tokens=6, do_sample=False, ignore_eos=True)
    pipe2 = Pipeline(model_dirs["A"], dtype="bfloat16", max_tokens=256, max_requests=2)
    assert pipe2.apply([[9, 8, 7]], max_new_tokens=6, do_sample=False, ignore_eos=True)[0] == good
