#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, random weights, synthetic tokens.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 512] [--layers L]
    python bench.py --impl reference

Prints ONE JSON line.  ``value`` is decoded tokens per second at the given batch and context, timed
on the device with CUDA events around K back-to-back launches of the captured decode step (model +
sampling) on the live batch; ``e2e`` is the same batch driven through ``LLMEngine.step()``: every
step packs the batch on the host, copies it from pinned memory, launches, and reads the sampled
tokens back.  ``prefill`` is one 2,048-token prompt through the entry point's step, ``points`` are
decode at batch 1 and 64, ``roofline`` relates the decode step to the bytes it must read.
Between timed iterations nothing is flushed: one step reads all weights (over 2 GB), far more than
the 126 MB L2 holds.  The K-step measurement is repeated until about half a second has been timed;
``value`` is the median repeat, ``spread`` gives the fastest and slowest.

``--impl reference`` measures the unmodified reference (the ``inference_engine`` package installed
under ``baseline/_ref``) the same way on the same model folder: its ``LLMEngine`` with stock options,
its captured decode step for ``value`` and its ``step()`` for ``e2e``
(benchmarks/bench_latency.py:33-49 of the reference).  Nothing of this package runs on that path
except the writer of the random-weights folder.
"""
import argparse
import json
import os
import shutil
import statistics
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_DECODE_TOK_S = {1: 104.0, 8: 798.0, 32: 2680.0, 64: 3646.0}   # the reference's README, RTX 5070 Laptop


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            m = json.load(f)
        return dict(hbm_gbs=float(m["hbm_gbs"]), tflops=float(m.get("bf16_tflops_sustained") or m["bf16_tflops"]),
                    tflops_burst=float(m["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_burst=1590.0, source="fallback")


class ClockSampler:
    """SM clocks and throttle reasons while the timed region runs, read by ``nvidia-smi`` in a process of
    its own (a sampling thread in this process would take the interpreter away from the step loop that is
    being timed).  Reads only; NVML in this process is the fallback where nvidia-smi is missing."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._proc = self._log = self._thread = None
        self._stop = threading.Event()

    def __enter__(self):
        import subprocess
        exe = shutil.which("nvidia-smi")
        if exe:
            try:
                self._log = tempfile.NamedTemporaryFile("w+", prefix="mie_b200_clocks_", suffix=".csv", delete=False)
                self._proc = subprocess.Popen([exe, "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                               "-lms", "100"], stdout=self._log, stderr=subprocess.DEVNULL)
                return self
            except OSError:
                self._proc = None
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)

            def run():
                while not self._stop.is_set():
                    try:
                        self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    except Exception:      # noqa: BLE001 - sampling must never end the run
                        pass
                    time.sleep(0.25)

            self._thread = threading.Thread(target=run, daemon=True)
            self._thread.start()
        except Exception:                  # noqa: BLE001
            pass
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        if self._proc is not None:
            time.sleep(0.12)               # let a last sample land
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:              # noqa: BLE001
                self._proc.kill()
            self._log.flush()
            self._log.seek(0)
            for line in self._log.read().splitlines():
                f = [x.strip() for x in line.split(",")]
                if len(f) != 2 + len(self.REASONS) or not f[0].isdigit():
                    continue
                self.samples.append(int(f[0]))
                if f[1].isdigit():
                    self.max_mhz = int(f[1])
                self.reasons.update(n for n, v in zip(self.REASONS, f[2:]) if v == "Active")
            self._log.close()
            try:
                os.unlink(self._log.name)
            except OSError:
                pass

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples), "reasons": sorted(self.reasons)}


def prompts_for(batch, length, vocab):
    return [[1] + [(1000 + i * 7 + j) % vocab for j in range(length - 1)] for i in range(batch)]


TIMED_REGION_S = 0.5        # the K-step measurement is repeated until about this much has been timed
MAX_REPEATS = 200
E2E_STEPS_MOST = 128        # end-to-end steps lengthen the contexts: keep them near the stated length


def timed_replays(graph, steps):
    """K back-to-back launches of a captured step between two events, repeated; ms per step of every repeat."""
    import torch
    per_step = []
    spent = 0.0
    while len(per_step) < 3 or (spent < TIMED_REGION_S and len(per_step) < MAX_REPEATS):
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        per_step.append(ms / steps)
        spent += ms * 1e-3
    return per_step


def timed_steps(eng, steps, after=lambda: None):
    """Wall time of K calls of ``eng.step()`` (host work, copies in, launch, tokens out), repeated."""
    import torch
    per_step = []
    for _ in range(max(1, min(3, E2E_STEPS_MOST // steps))):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.step()
        after()
        torch.cuda.synchronize()
        per_step.append((time.perf_counter() - t0) * 1e3 / steps)
    return per_step


def spread(per_step):
    return {"repeats": len(per_step), "ms_min": round(min(per_step), 4), "ms_max": round(max(per_step), 4)}


def decode_point(eng, batch, context, steps, warmup, e2e=False):
    """Device time per decode step at (batch, context) and, if asked, the end-to-end step time."""
    from mini_inference_engine_b200 import SamplingParams
    for p in prompts_for(batch, context, eng.vocab_size):
        eng.add_request(p, SamplingParams(max_tokens=4 * steps + warmup + E2E_STEPS_MOST, ignore_eos=True))
    while any(s.num_new_tokens > 1 for s in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(warmup):
        eng.step()
    eng.drain()
    g = eng.decode_graph(batch, max(s.cache.num_computed + 1 for s in eng.scheduler.running))
    out = {}
    per_step = timed_replays(g.graph, steps)            # the captured step on the live batch: model + sampling
    out["device_ms"] = statistics.median(per_step)
    out["spread"] = spread(per_step)
    out["launches_per_step"] = g.kernels
    if e2e:
        h0, d0, n0 = eng.h2d_bytes, eng.d2h_bytes, eng.num_steps
        per_step = timed_steps(eng, steps, after=eng.drain)
        out["e2e_ms"] = statistics.median(per_step)
        out["e2e_spread"] = spread(per_step)
        out["h2d"] = (eng.h2d_bytes - h0) // (eng.num_steps - n0)
        out["d2h"] = (eng.d2h_bytes - d0) // (eng.num_steps - n0)
    eng.drain()
    for s in list(eng.scheduler.running):
        eng.scheduler.finish(s)
    return out


def prefill_point(eng, tokens, steps, warmup):
    import torch

    from mini_inference_engine_b200 import SamplingParams
    times = []
    for i in range(warmup + steps):
        eng.add_request(prompts_for(1, tokens, eng.vocab_size)[0], SamplingParams(max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        eng.step()
        eng.drain()
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        assert not eng.has_work()
    return statistics.median(times)


def model_numbers(cfg, batch, context, prefill_tokens):
    """Bytes a decode step has to read and flops a prompt step has to do, from the configuration."""
    L, h, I, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    layer_params = (H + 2 * Hkv) * D * h + h * H * D + 3 * I * h
    weight_bytes = 2 * (L * (layer_params + 2 * h) + h + V * h)                 # every matrix once, norms, head
    kv_bytes = batch * context * 2 * L * Hkv * D * 2                            # the live requests' cache
    T = prefill_tokens
    flops = 2 * T * L * layer_params + 2 * V * h + L * 4 * H * D * T * (T + 1) // 2
    return {"step_bytes": weight_bytes + kv_bytes + batch * h * 2, "prefill_flops": flops}


def result_line(args, cfg, full_layers, steps, warmup, pk, main_pt, points, pre_ms, clocks, impl, extra_config):
    nums = model_numbers(cfg, args.batch, args.context + warmup, args.prefill_tokens)
    achieved = nums["step_bytes"] / (main_pt["device_ms"] * 1e-3) / 1e9
    T = args.prefill_tokens
    value = args.batch / main_pt["device_ms"] * 1e3
    base = BASELINE_DECODE_TOK_S.get(args.batch)
    config = {"model": args.preset, "layers": cfg.num_hidden_layers, "layers_full": full_layers, "hidden": cfg.hidden_size,
              "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
              "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
              "seq_len": args.context, "prefill_tokens": T, "page_size": 16, "weights": "random N(0,0.02) seed 0",
              "parallelism": "single_gpu", "l2": "inputs larger than L2 (weights 2 GB per step), no flush",
              "peaks": pk["source"]}
    config.update(extra_config)
    return {
        "metric": "decode tok/s", "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(main_pt["device_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / base, 2) if base else None, "dtype": "bf16", "data": "synthetic",
        "config": config,
        "spread": main_pt["spread"],
        "e2e": {"value": round(args.batch / main_pt["e2e_ms"] * 1e3, 1), "unit": "tok/s",
                "h2d_bytes_per_step": main_pt["h2d"], "d2h_bytes_per_step": main_pt["d2h"],
                "ms_per_step": round(main_pt["e2e_ms"], 4), **main_pt["e2e_spread"]},
        "gpu_launches": main_pt["launches_per_step"] * steps * main_pt["spread"]["repeats"],
        "prefill": {"value": round(T / pre_ms * 1e3, 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(nums["prefill_flops"] / (pre_ms * 1e-3) / (pk["tflops_burst"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(),
        "impl": impl,
    }


# ---------------------------------------------------------------------------------- the reference arm
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def reference_decode_point(eng, SamplingParams, batch, context, steps, warmup, vocab, e2e=False):
    """The reference's own latency loop (benchmarks/bench_latency.py:33-49): requests are prefilled,
    then pure decode steps are timed; device time is its captured step replayed on the live batch."""
    for p in prompts_for(batch, context, vocab):
        eng.add_request(p, SamplingParams(max_tokens=4 * steps + warmup + E2E_STEPS_MOST, ignore_eos=True))
    while any(s.num_new_tokens > 1 for s in eng.scheduler.running) or eng.scheduler.waiting:
        eng.step()
    for _ in range(warmup):
        eng.step()
    bucket = next(s for s in eng.graph_sizes if s >= batch)
    out = {}
    per_step = timed_replays(eng.graphs[bucket].graph, steps)
    out["device_ms"] = statistics.median(per_step)
    out["spread"] = spread(per_step)
    if e2e:
        per_step = timed_steps(eng, steps)              # its step() ends with .tolist() on the sampled tokens
        out["e2e_ms"] = statistics.median(per_step)
        out["e2e_spread"] = spread(per_step)
        # what its step copies (inference_engine/engine.py:106-120,159-168,205-207): ids, positions and slots
        # as int64, the block tables and context lengths as int32, temperatures as float32; tokens back as int64
        width = -(-(context + warmup + 4 * steps) // eng.cfg.block_size)
        out["h2d"] = batch * (3 * 8 + 4 * width + 4 + 4)
        out["d2h"] = batch * 8
    for s in list(eng.scheduler.running):
        eng.scheduler.finish(s)
    return out


def reference_prefill_point(eng, SamplingParams, tokens, vocab, steps, warmup):
    import torch
    times = []
    for i in range(warmup + steps):
        eng.add_request(prompts_for(1, tokens, vocab)[0], SamplingParams(max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        while eng.scheduler.has_work():
            eng.step()
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def count_kernels(fn):
    """Kernel launches inside ``fn()``, counted by the profiler of torch (the reference's kernels are
    Triton's, torch's and the vendor library's); None if the profiler is not usable."""
    try:
        import torch
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        return sum(e.count for e in prof.key_averages() if e.device_type.name == "CUDA")
    except Exception:          # noqa: BLE001
        return None


def run_reference(args, steps, warmup):
    if not os.path.isdir(os.path.join(REF_DIR, "inference_engine")):
        return {"impl": "reference", "unavailable": "baseline/_ref holds no inference_engine package (see baseline/"
                "install_reference.py: pip install --target baseline/_ref from a copy with a minimal pyproject.toml)"}
    try:
        import dataclasses

        import torch
        sys.path.insert(0, REF_DIR)
        from inference_engine import LLMEngine as RefEngine
        from inference_engine import SamplingParams as RefParams
        from inference_engine.config import EngineConfig as RefConfig

        from mini_inference_engine_b200.config import load_preset
        from mini_inference_engine_b200.weights import write_model_folder     # only writes the folder both arms load
        if not torch.cuda.is_available():
            return {"impl": "reference", "unavailable": "no CUDA device: the reference's LLMEngine needs one"}
        cfg = load_preset(args.preset)
        full_layers = cfg.num_hidden_layers
        if args.layers:
            cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers)
        point_batches = [int(b) for b in args.points.split(",") if b]
        max_seqs = max([args.batch] + point_batches)
        folder = tempfile.mkdtemp(prefix="mie_b200_bench_ref_")
        try:
            write_model_folder(folder, cfg, seed=0)
            # stock options but for the cache's share of memory: its pool is (free - 768 MiB) x fraction, and the
            # default 0.85 would zero 150 GB for a workload that uses 0.1 GB
            eng = RefEngine(folder, RefConfig(max_num_seqs=max_seqs, max_num_batched_tokens=max(2048, args.prefill_tokens),
                                              max_model_len=cfg.max_position_embeddings, kv_cache_memory_fraction=0.1),
                            dtype=torch.bfloat16, load_tokenizer=False, verbose=False)
        finally:
            shutil.rmtree(folder, ignore_errors=True)
        pk = peaks()
        V = cfg.vocab_size
        with ClockSampler() as clocks:
            main_pt = reference_decode_point(eng, RefParams, args.batch, args.context, steps, warmup, V, e2e=True)
        bucket = next(s for s in eng.graph_sizes if s >= args.batch)
        main_pt["launches_per_step"] = count_kernels(eng.graphs[bucket].graph.replay) or 0
        points = {}
        for b in point_batches:
            pt = reference_decode_point(eng, RefParams, b, args.context, max(10, steps // 2), warmup, V)
            points[f"decode_b{b}"] = round(b / pt["device_ms"] * 1e3, 1)
        pre_ms = reference_prefill_point(eng, RefParams, args.prefill_tokens, V, max(3, min(10, steps // 10)), 3)
        line = result_line(args, cfg, full_layers, steps, warmup, pk, main_pt, points, pre_ms, clocks, "reference",
                           {"reference": "inference_engine (unmodified) from baseline/_ref, stock options, "
                                         "kv_cache_memory_fraction 0.1", "same_config": True})
        line["vs_baseline"] = None
        return line
    except Exception as e:      # noqa: BLE001 - whatever stops the reference on this box is the reason it is unavailable
        import traceback
        last = traceback.extract_tb(e.__traceback__)[-1]
        return {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]} "
                f"(at {os.path.basename(last.filename)}:{last.lineno})".replace("\n", " ")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--preset", default="tinyllama-1.1b")
    ap.add_argument("--points", default="1,64", help="further decode batch sizes, comma separated ('' for none)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    if args.impl == "reference":
        print(json.dumps(run_reference(args, steps, warmup)))
        return 0

    import dataclasses

    import torch

    from mini_inference_engine_b200 import EngineConfig, LLMEngine
    from mini_inference_engine_b200.config import load_preset
    from mini_inference_engine_b200.weights import write_model_folder

    cfg = load_preset(args.preset)
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers)
    folder = tempfile.mkdtemp(prefix="mie_b200_bench_")
    try:
        write_model_folder(folder, cfg, seed=0)
        point_batches = [int(b) for b in args.points.split(",") if b]
        max_seqs = max([args.batch] + point_batches)
        eng = LLMEngine(folder, EngineConfig(max_num_seqs=max_seqs, max_num_batched_tokens=max(2048, args.prefill_tokens),
                                             max_model_len=cfg.max_position_embeddings,
                                             cuda_graph_batch_sizes=tuple(sorted({args.batch, *point_batches}))),
                        dtype=torch.bfloat16, load_tokenizer=False, verbose=False)
    finally:
        shutil.rmtree(folder, ignore_errors=True)

    pk = peaks()
    with ClockSampler() as clocks:
        main_pt = decode_point(eng, args.batch, args.context, steps, warmup, e2e=True)
    points = {}
    for b in point_batches:
        pt = decode_point(eng, b, args.context, max(10, steps // 2), warmup)
        points[f"decode_b{b}"] = round(b / pt["device_ms"] * 1e3, 1)
    pre_ms = prefill_point(eng, args.prefill_tokens, max(3, min(10, steps // 10)), 3)
    print(json.dumps(result_line(args, cfg, full_layers, steps, warmup, pk, main_pt, points, pre_ms, clocks, "ours",
                                 {"page_size": eng.cfg.block_size})))
    return 0


if __name__ == "__main__":
    sys.exit(main())
