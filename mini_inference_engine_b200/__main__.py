"""Command line, in the manner of the reference's scripts (it has no console entry point of its
own): the options of benchmarks/bench_throughput.py (``--batch --workload --num-requests
--overrides --batches``), benchmarks/bench_latency.py (``--batches --prompt --steps``) and
benchmarks/profile_decode.py (``--graphs --batch --prompt --steps``) keep their names and meanings.

    python -m mini_inference_engine_b200 generate   --model DIR --prompt-ids 1,2,3 --max-tokens 16
    python -m mini_inference_engine_b200 latency    --preset tinyllama-1.1b --batches 1 8 64 --prompt 512 --steps 100
    python -m mini_inference_engine_b200 throughput --preset tinyllama-1.1b --batch 32 --workload mixed
    python -m mini_inference_engine_b200 throughput --preset llama-3-8b --workload long
    python -m mini_inference_engine_b200 profile-decode --preset tinyllama-1.1b --graphs 1 --batch 32 --steps 50
    python -m mini_inference_engine_b200 make-model --preset tiny-llama-a --seed 0 --out DIR

A model is a folder (``--model``) or a preset with random weights (``--preset`` + ``--seed``), which
is first written as a model folder and then loaded like any other.
"""
from __future__ import annotations

import argparse
import json
import random
import statistics
import sys
import shutil
import tempfile
import time


def _model_args(p):
    p.add_argument("--model", help="model folder (config.json + *.safetensors)")
    p.add_argument("--preset", help="named configuration for the random-weights mode")
    p.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--overrides", default=None, help="JSON EngineConfig overrides")


def _engine(args, **forced):
    import torch

    from . import EngineConfig, LLMEngine
    from .config import load_preset
    from .weights import write_model_folder
    folder, made = args.model, None
    if folder is None:
        if not args.preset:
            raise SystemExit("give --model DIR or --preset NAME")
        folder = made = tempfile.mkdtemp(prefix="mie_b200_model_")
    ov = json.loads(args.overrides) if args.overrides else {}
    ov.update(forced)
    ov.setdefault("seed", args.seed)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    try:
        if made:
            write_model_folder(folder, load_preset(args.preset), args.seed)
        return LLMEngine(folder, EngineConfig.from_overrides(ov), dtype=dtype, load_tokenizer=False, verbose=True)
    finally:
        if made:                # gigabytes of random weights: the engine holds its copy on the device, the folder goes now
            shutil.rmtree(made, ignore_errors=True)


def cmd_generate(args):
    from . import SamplingParams
    eng = _engine(args)
    if args.prompt_ids:
        prompts = [[int(t) for t in p.split(",")] for p in args.prompt_ids]
    else:
        rng = random.Random(args.seed)
        prompts = [[rng.randrange(eng.vocab_size) for _ in range(args.prompt_len)] for _ in range(args.num_prompts)]
    sp = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, ignore_eos=args.ignore_eos)
    for o in eng.generate(prompts, sp):
        print(json.dumps({"seq_id": o.seq_id, "prompt_len": o.prompt_len, "output_ids": o.output_ids,
                          "ttft": o.ttft, "latency": o.latency}))


def decode_latency(eng, batch: int, prompt: int, steps: int) -> float:
    """Median milliseconds of a pure-decode ``step()`` at a batch size, contexts of ``prompt`` tokens
    (the measurement of benchmarks/bench_latency.py:33-49)."""
    import torch

    from . import SamplingParams
    ids = [[1] + [1000 % eng.vocab_size + (i * 7 + j) % max(1, eng.vocab_size - 1000) for j in range(prompt - 1)]
           for i in range(batch)]
    ids = [[t % eng.vocab_size for t in p] for p in ids]
    for p in ids:
        eng.add_request(p, SamplingParams(max_tokens=steps + 40, ignore_eos=True))
    while any(s.num_new_tokens > 1 for s in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(10):
        eng.step()
    times = []
    for _ in range(steps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.step()
        eng.drain()                      # read this step's tokens: the measurement is of one whole step
        times.append(time.perf_counter() - t0)
    while eng.has_work():
        eng.step()
    return statistics.median(times) * 1e3


def cmd_latency(args):
    eng = _engine(args, use_cuda_graphs=bool(args.graphs))
    for b in args.batches:
        ms = decode_latency(eng, b, args.prompt, args.steps)
        print(f"bs={b:3d}  {ms:7.3f} ms/token-step  ({b / ms * 1e3:9.1f} tok/s)", flush=True)


LONG_WORKLOAD = dict(num_requests=64, batch=64, max_model_len=8192, max_num_batched_tokens=2048)


def make_workload(kind: str, n: int, seed: int, vocab: int):
    """benchmarks/bench_throughput.py:34-44: mixed = prompt U[128,512], output U[64,512]; fixed = 256/256.
    ``long`` is not the reference's: prompts U[512,4096] with 256 generated tokens each, so that prompts go
    in several portions of the token budget beside the decoding requests."""
    rng = random.Random(seed)
    reqs = []
    for _ in range(n):
        if kind == "long":
            p, o = rng.randint(512, 4096), 256
        else:
            p, o = (rng.randint(128, 512), rng.randint(64, 512)) if kind == "mixed" else (256, 256)
        reqs.append(([1 % vocab] + [rng.randint(min(100, vocab - 1), vocab - 1) for _ in range(p - 1)], o))
    return reqs


def cmd_throughput(args):
    import gc

    import torch

    long = args.workload == "long"
    if args.batch is None:
        args.batch = LONG_WORKLOAD["batch"] if long else 32
    if args.num_requests is None:
        args.num_requests = LONG_WORKLOAD["num_requests"] if long else 256
    if args.batches:                       # several concurrency caps, one engine after the other
        for bs in args.batches:
            one = argparse.Namespace(**{**vars(args), "batch": bs, "batches": None})
            cmd_throughput(one)
            gc.collect()
            torch.cuda.empty_cache()
        return
    from . import SamplingParams
    forced = dict(max_num_seqs=args.batch)
    if args.workload == "long":            # contexts of up to 4,352 positions: the model's limit permitting
        ov = json.loads(args.overrides) if args.overrides else {}
        forced.update({k: LONG_WORKLOAD[k] for k in ("max_model_len", "max_num_batched_tokens") if k not in ov})
    eng = _engine(args, **forced)
    reqs = make_workload(args.workload, args.num_requests, 0, eng.vocab_size)
    too_long = [len(i) + o for i, o in reqs if len(i) + o > eng.cfg.max_model_len]
    if too_long:
        raise SystemExit(f"the workload needs {max(too_long)} positions; this model and these overrides allow "
                         f"{eng.cfg.max_model_len}")
    eng.generate([ids for ids, _ in reqs[:4]], SamplingParams(max_tokens=16, ignore_eos=True))
    eng.num_steps = eng.num_graph_steps = eng.num_portion_graph_steps = 0
    eng.scheduler.num_preemptions = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate([ids for ids, _ in reqs], [SamplingParams(max_tokens=o, ignore_eos=True) for _, o in reqs])
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    assert all(len(o.output_ids) == n for o, (_, n) in zip(outs, reqs))
    out_tokens, in_tokens = sum(o for _, o in reqs), sum(len(i) for i, _ in reqs)
    print("RESULT " + json.dumps({
        "system": "engine", "batch": args.batch, "workload": args.workload, "num_requests": len(reqs),
        "seconds": secs, "steps": eng.num_steps, "graph_steps": eng.num_graph_steps,
        "portion_graph_steps": eng.num_portion_graph_steps,
        "eager_steps": eng.num_steps - eng.num_graph_steps - eng.num_portion_graph_steps,
        "preemptions": eng.scheduler.num_preemptions,
        "kv_cache_tokens": eng.cache.pools[0].num_pages * eng.cfg.block_size,
        "output_tokens": out_tokens, "prompt_tokens": in_tokens, "output_tok_per_s": out_tokens / secs,
        "total_tok_per_s": (out_tokens + in_tokens) / secs}))


def cmd_profile_decode(args):
    """Steady-state decode at one batch size, for a profiler (the workload of
    benchmarks/profile_decode.py:29-42): every engine step is wrapped in NVTX ranges (schedule /
    prepare / forward / sample), the measured steps in a range "decode_steps".  Without a profiler it
    still says what a step costs: wall and device time, kernels of this package and launch calls."""
    import torch

    from . import SamplingParams
    from .kernels import ops
    from . import EngineConfig
    forced = {"max_num_seqs": args.batch} if args.batch > EngineConfig().max_num_seqs else {}
    eng = _engine(args, use_cuda_graphs=bool(args.graphs), **forced)
    for i in range(args.batch):
        ids = [1 % eng.vocab_size] + [(1000 + (i * 7 + j) % 30000) % eng.vocab_size for j in range(args.prompt - 1)]
        eng.add_request(ids, SamplingParams(max_tokens=args.steps + 30, ignore_eos=True))
    while any(s.num_new_tokens > 1 for s in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(20):
        eng.step()
    eng.drain()
    torch.cuda.synchronize()
    launches0, graph0 = ops.launches, eng.num_graph_steps
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.nvtx.range_push("decode_steps")
    t0 = time.perf_counter()
    start.record()
    for _ in range(args.steps):
        eng.step()
    eng.drain()
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    torch.cuda.nvtx.range_pop()
    graph_steps = eng.num_graph_steps - graph0
    nodes = eng.decode_graph(args.batch, args.prompt + args.steps).kernels if graph_steps else 0   # of the graph the batch ran in
    print("RESULT " + json.dumps({
        "batch": args.batch, "prompt_len": args.prompt, "steps": args.steps, "graphs": bool(args.graphs),
        "wall_ms_per_step": wall / args.steps * 1e3, "device_ms_per_step": start.elapsed_time(end) / args.steps,
        "graph_steps": graph_steps,
        "kernels_per_step": nodes if graph_steps else (ops.launches - launches0) / args.steps,
        "launch_calls_per_step": 1 if graph_steps else (ops.launches - launches0) / args.steps}))


def cmd_make_model(args):
    import torch

    from .config import load_preset
    from .weights import write_model_folder
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    print(write_model_folder(args.out, load_preset(args.preset), args.seed, dt))


def main(argv=None):
    ap = argparse.ArgumentParser(prog="mini_inference_engine_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    _model_args(g)
    g.add_argument("--prompt-ids", action="append", help="comma-separated token ids; may be given several times")
    g.add_argument("--prompt-len", type=int, default=16, help="length of random prompts when no ids are given")
    g.add_argument("--num-prompts", type=int, default=1)
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--ignore-eos", action="store_true")
    g.set_defaults(fn=cmd_generate)

    l = sub.add_parser("latency", help="median ms per pure-decode step at several batch sizes")
    _model_args(l)
    l.add_argument("--batches", type=int, nargs="+", default=[1, 8, 32, 64])
    l.add_argument("--prompt", type=int, default=512)
    l.add_argument("--steps", type=int, default=100)
    l.add_argument("--graphs", type=int, default=1)
    l.set_defaults(fn=cmd_latency)

    t = sub.add_parser("throughput", help="offline throughput on the reference's synthetic workloads")
    _model_args(t)
    t.add_argument("--batch", type=int, default=None, help="most requests running at once (32; 64 for --workload long)")
    t.add_argument("--workload", choices=["mixed", "fixed", "long"], default="mixed")
    t.add_argument("--num-requests", type=int, default=None, help="256; 64 for --workload long")
    t.add_argument("--batches", type=int, nargs="+", default=None, help="several values of --batch, one run each")
    t.set_defaults(fn=cmd_throughput)

    pd = sub.add_parser("profile-decode", help="steady-state decode at one batch size under NVTX ranges, for a profiler")
    _model_args(pd)
    pd.add_argument("--graphs", type=int, default=1)
    pd.add_argument("--batch", type=int, default=32)
    pd.add_argument("--prompt", type=int, default=512)
    pd.add_argument("--steps", type=int, default=50)
    pd.set_defaults(fn=cmd_profile_decode)

    m = sub.add_parser("make-model", help="write a model folder with random weights")
    m.add_argument("--preset", required=True)
    m.add_argument("--seed", type=int, default=0)
    m.add_argument("--out", required=True)
    m.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    m.set_defaults(fn=cmd_make_model)

    args = ap.parse_args(argv)
    args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
