"""A bounded wait that runs out, in the one form that is safe on a shared GPU: a self-test
kernel of the library waits, with a limit of a few thousand polls, on an mbarrier nobody
arrives on, while nothing is in flight.  The wait gives up, the kernel returns, status bit 8
reaches the host as a StepError, and the next step runs as if nothing had happened.  The
waits inside the TMA/tcgen05 kernels are the same function with a larger limit."""

from ctypes import c_int, c_void_p

import pytest
import torch

from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.step import Runner, StepEntry, StepError

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_a_wait_that_runs_out_is_reported_and_the_next_step_runs(tiny_models):
    tiny = tiny_models["tiny_a"]
    model, _ = load_model(tiny.dir, "bfloat16", DEV)
    rn = Runner(model, num_pages=8, page_size=16, max_requests=2, dtype=torch.bfloat16,
                device=DEV)
    toks = tiny.tokens(20, 3)
    before = rn.step([StepEntry("a", toks, want=[19])]).logits.clone()
    rn.close("a")
    wait = rn.ops.register_kernel("hs_selftest_wait_timeout", [c_void_p, c_void_p, c_int, c_void_p])
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    wait(rn.status.data_ptr(), gave_up.data_ptr(), 4000, rn.ops.stream())
    torch.cuda.synchronize()
    assert gave_up.item() == 1
    with pytest.raises(StepError, match="timed out"):
        rn.check_status()
    assert rn.status.item() == 0                       # reported once, then cleared
    after = rn.step([StepEntry("b", toks, want=[19])]).logits
    assert torch.equal(before, after)                  # the context is as usable as before
    from hetero_serve_b200.kernels import KernelError
    with pytest.raises(KernelError, match="unsupported"):
        wait(rn.status.data_ptr(), gave_up.data_ptr(), 0, rn.ops.stream())
