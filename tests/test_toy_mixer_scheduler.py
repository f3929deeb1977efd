"""The toy mixer with state of its own (tests/test_toy_mixer_gpu.py) under the scheduler,
without a GPU: requests are admitted by the scheduler, not by the step function, so the
state slot has to be cleared at admission — for the second of two requests that use the
only slot one after the other, and for a request that is preempted and prefilled again
over its own old state.  Kernels are the plain PyTorch twins; the cache manager, the
runner, the scheduler and the model assembly are the product's own."""

import torch

import plain_ops
from hetero_serve_b200.engine.scheduler import Request, Scheduler
from hetero_serve_b200.engine.step import Runner
from hetero_serve_b200.parts import Model, register_mixer
from test_toy_mixer_gpu import RunningMeanMixer, _plain, _spec


def _engine(live_requests, num_pages, max_batch):
    register_mixer("toy_running_mean", RunningMeanMixer, replace=True)
    spec = _spec(width=32, vocab=50, positions=64, mixed=True)
    model = Model(spec)
    g = torch.Generator().manual_seed(3)
    stored = {n: torch.randn(r.shape, generator=g) * (0.2 if len(r.shape) == 2 else 0.1)
              + (1.0 if n.endswith("w") and len(r.shape) == 1 else 0.0)
              for n, r in model.tensor_requests().items()}
    model.bind(stored, torch.float32, "cpu")
    rn = Runner(model, num_pages=num_pages, page_size=16, max_requests=live_requests,
                dtype=torch.float32, device="cpu", ops=plain_ops.PlainOps())
    sched = Scheduler(rn.manager, lambda entries: rn.step(entries, sample=True),
                      max_batch=max_batch, max_prefill_tokens=12, max_ctx=64, eos_token_id=None,
                      vocab_size=50)
    return rn, sched, stored, spec


def _greedy_plain(stored, spec, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(_plain(stored, spec, ids)[-1])))
    return ids[len(prompt):]


def _run(sched):
    while sched.has_work():
        sched.step()


def test_a_slot_is_cleared_for_the_next_request_the_scheduler_admits():
    rn, sched, stored, spec = _engine(live_requests=1, num_pages=8, max_batch=1)
    a = [(3 * i + 1) % 50 for i in range(30)]
    b = [(7 * i + 2) % 50 for i in range(21)]
    sa = sched.add(Request(a, max_new_tokens=6, stop_at_eos=False))
    sb = sched.add(Request(b, max_new_tokens=6, stop_at_eos=False))
    _run(sched)
    assert sa.output_ids == _greedy_plain(stored, spec, a, 6)
    assert sb.output_ids == _greedy_plain(stored, spec, b, 6)     # same slot, after a
    rn.manager.check()


def test_a_preempted_request_is_prefilled_again_on_cleared_state():
    # 5 pages: two requests of 30 and 28 tokens fit (2 + 2), and run out while decoding
    rn, sched, stored, spec = _engine(live_requests=2, num_pages=5, max_batch=2)
    a = [(3 * i + 1) % 50 for i in range(30)]
    b = [(11 * i + 5) % 50 for i in range(28)]
    sa = sched.add(Request(a, max_new_tokens=20, stop_at_eos=False))
    sb = sched.add(Request(b, max_new_tokens=20, stop_at_eos=False))
    _run(sched)
    assert sched.stats.preemptions >= 1
    assert sa.output_ids == _greedy_plain(stored, spec, a, 20)
    assert sb.output_ids == _greedy_plain(stored, spec, b, 20)
    rn.manager.check()
