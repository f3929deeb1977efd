"""Command line: generate from token ids with a model folder or random weights.

Option names and meanings follow the reference where it has them — the worker's
``--model --weights --device --block-size --num-blocks --max-batch
--max-prefill-tokens --max-ctx --seed`` (heteroserve/worker/worker.py:845-867) and the
demo's ``--model --num-blocks`` (run_demo.py:206-213).  The engine works on token ids;
there is no tokenizer here.

Without prompts it runs the demo of the reference's ``run_demo.py`` that applies to one
device: a cold request, then a warm request sharing its prefix (prefill skipped for the
cached pages), then a batch.
"""

from __future__ import annotations

import argparse
import json
import sys
import time

from .config import EngineConfig, preset_names
from .engine import LLMEngine, Request


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="hetero_serve_b200", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="gpt2",
                    help=f"named configuration for random weights: {', '.join(preset_names())}")
    ap.add_argument("--weights", default="",
                    help="model folder (config.json + model.safetensors); overrides --model")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--block-size", dest="block_size", type=int, default=16)
    ap.add_argument("--num-blocks", dest="num_blocks", type=int, default=512)
    ap.add_argument("--max-batch", dest="max_batch", type=int, default=8)
    ap.add_argument("--max-prefill-tokens", dest="max_prefill_tokens", type=int, default=256)
    ap.add_argument("--max-ctx", dest="max_ctx", type=int, default=512)
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights and sampling")
    ap.add_argument("--policy", default="prefill_first", choices=["prefill_first", "mixed"])
    ap.add_argument("--no-prefix-cache", dest="prefix_cache", action="store_false")
    ap.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false")
    ap.add_argument("--no-pipeline", dest="pipeline", action="store_false",
                    help="read every step's tokens before the next step is launched")
    ap.add_argument("--fused-decode", dest="fused_decode", action="store_true",
                    help="run pure decode steps of up to 16 tokens as one persistent kernel "
                         "(where the model has the shape it serves)")
    ap.add_argument("--prompt-ids", dest="prompt_ids", action="append", default=[],
                    help="comma-separated token ids; may be given several times")
    ap.add_argument("--prompt-file", dest="prompt_file", default="",
                    help="a file with one prompt per line: token ids separated by commas or blanks")
    ap.add_argument("--random-prompts", dest="random_prompts", default="",
                    help="N:LEN — N random prompts of LEN tokens")
    ap.add_argument("--max-new-tokens", dest="max_new_tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", dest="top_k", type=int, default=0)
    ap.add_argument("--sample-seed", dest="sample_seed", type=int, default=None,
                    help="seed of the sampling draws (request i uses seed + i); default: --seed")
    ap.add_argument("--no-eos-stop", dest="stop_at_eos", action="store_false")
    ap.add_argument("--json", action="store_true", help="one JSON object per request")
    return ap


def make_engine(args) -> LLMEngine:
    cfg = EngineConfig(dtype=args.dtype, block_size=args.block_size, num_blocks=args.num_blocks,
                       max_batch=args.max_batch, max_prefill_tokens=args.max_prefill_tokens,
                       max_ctx=args.max_ctx, policy=args.policy, prefix_cache=args.prefix_cache,
                       cuda_graphs=args.cuda_graphs, pipeline=args.pipeline,
                       fused_decode=args.fused_decode, seed=args.seed, device=args.device)
    if args.weights:
        return LLMEngine(args.weights, cfg)
    return LLMEngine.random(args.model, seed=args.seed, config=cfg)


def _report(rec, as_json: bool) -> None:
    if as_json:
        print(json.dumps(rec.as_dict()))
    else:
        print(f"{rec.req_id}: prompt {rec.prompt_tokens} tok (cached {rec.cached_prefix_tokens}, "
              f"computed {rec.prefill_tokens_computed}), generated {rec.generated_tokens} "
              f"[{rec.finish_reason}]  TTFT {rec.ttft * 1e3:.2f} ms  TPOT {rec.tpot * 1e3:.3f} ms  "
              f"E2E {rec.e2e * 1e3:.2f} ms\n    output_ids: {rec.output_ids}")


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    engine = make_engine(args)
    vocab = engine.model.spec.vocab_size
    prompts = [[int(t) for t in p.replace(" ", "").split(",") if t] for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as fh:
            for line in fh:
                ids = [int(t) for t in line.replace(",", " ").split()]
                if ids:
                    prompts.append(ids)
    if args.random_prompts:
        import torch
        n, length = (int(x) for x in args.random_prompts.split(":"))
        g = torch.Generator().manual_seed(args.seed)
        prompts += torch.randint(0, vocab, (n, length), generator=g).tolist()

    sample_seed = args.seed if args.sample_seed is None else args.sample_seed

    def req(p, i=0):
        return Request(p, args.max_new_tokens, args.temperature, args.top_k, sample_seed + i,
                       args.stop_at_eos)

    t0 = time.perf_counter()
    if prompts:
        seqs = [engine.submit_nowait(req(p, i)) for i, p in enumerate(prompts)]
        records = engine.run_until_done()
        order = {s.req_id: i for i, s in enumerate(seqs)}
        records.sort(key=lambda r: order[r.req_id])
        for r in records:
            _report(r, args.json)
    else:
        import torch
        g = torch.Generator().manual_seed(args.seed)
        limit = engine.scheduler.max_ctx - args.max_new_tokens - 1
        shared = torch.randint(0, vocab, (max(1, min(192, limit - 8)),), generator=g).tolist()
        tail = lambda: torch.randint(0, vocab, (8,), generator=g).tolist()  # noqa: E731
        print("1. cold request: nothing cached", file=sys.stderr)
        records = [engine.submit(req(shared + tail()))]
        _report(records[-1], args.json)
        print("2. warm request: same prefix, its pages are reused", file=sys.stderr)
        records.append(engine.submit(req(shared + tail(), 1)))
        _report(records[-1], args.json)
        print("3. a batch sharing the prefix", file=sys.stderr)
        for i in range(min(4, args.max_batch)):
            engine.submit_nowait(req(shared + tail(), 2 + i))
        batch = engine.run_until_done()
        for r in batch:
            _report(r, args.json)
        records += batch
    wall = time.perf_counter() - t0
    summary = engine.summarise(records, wall)
    summary["state"] = engine.state_message()
    print(json.dumps(summary) if args.json else
          f"{summary['n_requests']} requests, {summary['throughput_tok_s']} generated tok/s, "
          f"cache hit rate {summary['cache_hit_rate']}, preemptions {summary['preemptions']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
