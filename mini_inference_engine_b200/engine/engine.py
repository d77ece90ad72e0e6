"""``LLMEngine``: the Python entry point, with the surface of inference_engine/engine.py:35-244 --
``LLMEngine(model, engine_config, dtype, load_tokenizer, verbose)``, ``add_request``, ``step``,
``generate`` returning ``RequestOutput(seq_id, prompt_len, output_ids, text, ttft, latency)``.

One step: schedule -> pack the batch (one host->device transfer) -> the model's step function
(a captured CUDA graph for pure-decode steps, eager otherwise) -> sample on the device -> one small
device->host read of the new tokens -> bookkeeping.  Sampling is inside the captured graph, so a
decode step is one transfer in, one graph launch, one transfer out.
"""
from __future__ import annotations

import contextlib
import os
import time
from dataclasses import dataclass

import numpy as np
import torch

from ..config import EngineConfig, load_config
from ..kernels import gemm_tc, ops
from ..models.decoder import DecoderModel
from ..parts.base import Runtime
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights import read_model_folder
from .runner import ModelRunner
from .scheduler import Scheduler
from .sequence import Sequence

ACTIVATION_RESERVE = 768 * 2 ** 20      # kept free for activations when sizing the cache (inference_engine/engine.py:51)


@dataclass
class RequestOutput:
    seq_id: int
    prompt_len: int
    output_ids: list
    text: str | None
    ttft: float | None          # seconds from arrival to the first generated token
    latency: float | None       # seconds from arrival to the end


PENDING = -1          # in token_ids: a token that the step in flight is sampling


class _InFlight:
    """A launched step whose sampled tokens the host has not read yet.  ``sources``: (pinned row, count)
    in the order of ``seqs`` -- one entry, or two when the step ran as two graphs."""

    def __init__(self, seqs, places, ending, sources, event):
        self.seqs, self.places, self.ending, self.sources, self.event = seqs, places, ending, sources, event

    def tokens(self) -> list:
        out = []
        for row, n in self.sources:
            out += row[:n].tolist()
        return out


class _DecodeGraph:
    def __init__(self, graph, layout, buffer, tokens, kernels):
        self.graph, self.layout, self.buffer, self.tokens = graph, layout, buffer, tokens
        self.kernels = kernels        # kernels of this package inside the captured step


def _nvtx_range(name):
    return torch.cuda.nvtx.range(name)


class LLMEngine:
    def __init__(self, model: str, engine_config: EngineConfig | None = None, dtype=torch.bfloat16,
                 load_tokenizer: bool = True, verbose: bool = True, device: str = "cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("LLMEngine needs a CUDA device: every operator is a CUDA kernel of this package")
        self.cfg = engine_config or EngineConfig()
        self.verbose = verbose
        if not os.path.isdir(model):
            raise FileNotFoundError(f"{model!r} is not a model folder (config.json + *.safetensors); "
                                    "downloading by name is not supported")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.model_cfg = load_config(model)
        spec = self.model_cfg.model_spec()
        self.cfg.max_model_len = min(self.cfg.max_model_len, spec.max_position)      # inference_engine/engine.py:42
        self.eos_token_id = spec.eos_token_id
        self.vocab_size = spec.vocab_size
        rt = Runtime(self.device, dtype)
        self.model = DecoderModel(spec, read_model_folder(model), rt, where=model)
        torch.cuda.empty_cache()

        layout = self.model.cache_layout
        per_page = sum(layout.bytes_per_page(g, self.cfg.block_size, dtype) for g in range(len(layout.groups)))
        if self.cfg.num_blocks is not None:
            num_blocks = int(self.cfg.num_blocks)
        else:                                      # size the pool from the memory left after the weights
            free, _ = torch.cuda.mem_get_info(self.device)
            state = layout.bytes_per_state_slot() * (self.cfg.max_num_seqs + 1)
            kv_bytes = int((free - ACTIVATION_RESERVE - state) * self.cfg.kv_cache_memory_fraction)
            num_blocks = kv_bytes // max(per_page, 1)
            # no request can use more than max_model_len positions: cap what max_num_seqs can ever hold
            ceiling = self.cfg.max_num_seqs * (-(-self.cfg.max_model_len // self.cfg.block_size)) + 1
            num_blocks = min(num_blocks, ceiling + max(1, ceiling // 100) + 1)
        if num_blocks < 2:
            raise RuntimeError(f"not enough memory for the cache: {num_blocks} pages of {per_page} bytes")
        self.runner = ModelRunner(self.model, num_blocks, self.cfg.block_size, self.cfg.max_num_seqs)
        self.cache = self.runner.cache
        self.scheduler = Scheduler(self.cfg, self.cache)
        self.max_blocks_per_seq = -(-self.cfg.max_model_len // self.cfg.block_size)
        self.sampler = Sampler(self.device, self.cfg.seed)
        if verbose:
            print(f"[mini_inference_engine_b200] cache: {num_blocks} pages x {self.cfg.block_size} tokens = "
                  f"{num_blocks * self.cfg.block_size} tokens ({num_blocks * per_page / 2 ** 30:.2f} GiB)")

        self.tokenizer = None
        if load_tokenizer and any(os.path.isfile(os.path.join(model, f))
                                  for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
            from transformers import AutoTokenizer          # text in/out only; never on the token path
            self.tokenizer = AutoTokenizer.from_pretrained(model)

        most = max(self.cfg.max_num_batched_tokens, self.cfg.max_num_seqs, 256, *self.cfg.cuda_graph_batch_sizes)
        # the sampled tokens as the host sees them: two rows, taken in turns (step N's are read while step
        # N+1 runs); the sampling kernel writes them itself (pinned memory is addressable from the device)
        self._pinned_tokens = torch.zeros(2, most, dtype=torch.int32, pin_memory=True)
        # a prompt portion that runs as a graph of its own beside the decode graph leaves its token apart
        self._pinned_portion = torch.zeros(2, 8, dtype=torch.int32, pin_memory=True)
        self._portion_slot = most
        self._sampled = torch.zeros(most + 8, dtype=torch.int32, device=self.device)   # the last step's tokens, on the device
        self._turn = 0
        self._in_flight = None
        self.graphs: dict = {}                   # (bucket, context bound) -> captured decode step
        self.graph_sizes: list = []
        self.graph_bounds: list = []             # the context bounds the buckets were captured for, ascending
        self.num_steps = 0
        self.num_graph_steps = 0
        self.num_portion_graph_steps = 0
        self._portion_graphs: dict = {}          # (tokens, wanted logits) -> captured step of one prompt portion
        self._portion_seen: dict = {}
        self._graph_pool = None
        self._capture_stream = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        if self.cfg.use_cuda_graphs:
            self._capture_cuda_graphs()
        if self.cfg.warm_up_prompt_step:
            self._warm_up_prompt_step()

    @torch.inference_mode()
    def _warm_up_prompt_step(self):
        """One prompt step of the whole token budget on scratch rows (tokens 0 at positions 0.. of page 0, as the
        padding of a portion graph; no logits wanted), and one that wants a token: what a first real step would
        otherwise pay for -- kernel modules loaded at first use, the library's choice of a product for that many rows,
        blocks of the allocator -- is paid here.  Nothing but the scratch page is written."""
        from .batch import BatchRow
        n = min(self.cfg.max_num_batched_tokens, self.cfg.max_model_len)
        if n < 2:
            return
        b = self.runner.builder
        pages = -(-n // self.cfg.block_size)
        zeros = [np.zeros(pages, dtype=np.int32) for _ in range(b.num_groups)]
        for want in ((), (n - 1,)):
            row = BatchRow(np.zeros(n, dtype=np.int32), 0, zeros, 0, want)
            buf, layout = b.pack([row], extras=self.sampler.inputs(len(want)))
            ctx = b.to_device(buf, layout)
            ctx.token_feedback = self._sampled
            self._forward_and_sample(ctx, self._sampled[self._portion_slot:self._portion_slot + len(want)],
                                     host_out=self._pinned_portion)
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ CUDA graphs of decode steps
    def _forward_and_sample(self, ctx, tokens_out=None, host_out=None, seed=None):
        logits = self.model.step(ctx)
        if logits.shape[0] == 0:
            return None
        return self.sampler.sample(logits, ctx.extras["temperature"], ctx.extras["request"],
                                   ctx.extras["out_position"], out=tokens_out, seed=seed,
                                   host_out=self._pinned_tokens if host_out is None else host_out,
                                   host_turn=ctx.extras["host_turn"])

    @torch.inference_mode()
    def _capture_cuda_graphs(self):
        """One graph per batch-size bucket, largest first so the smaller ones share its memory
        pool (inference_engine/engine.py:76-104), and per context bound (``graph_context_bounds`` and
        ``max_model_len``): a step replays the graph of the smallest bound that covers its longest
        request.  A graph covers the whole step including the sampling kernel; its inputs live in one
        static device buffer that a step overwrites with one copy.  Rows that pad a batch up to its
        bucket are scratch rows: one token at position 0 of page 0, context length 1."""
        t0 = time.perf_counter()
        sizes = sorted(b for b in self.cfg.cuda_graph_batch_sizes if b <= self.cfg.max_num_seqs)
        if not sizes:
            return
        b = self.runner.builder
        pool = None
        bounds = sorted({c for c in self.cfg.graph_context_bounds if c < self.cfg.max_model_len} | {self.cfg.max_model_len})
        for bs in reversed(sizes):
            static = None
            for bound in reversed(bounds):
                buf, layout = b.pack([], pad_rows=bs, table_width=self.max_blocks_per_seq,
                                     extras=self.sampler.inputs(bs))
                layout["max_ctx_len"] = bound                       # static bound for kernels that plan by it
                if static is None:                                  # the bounds of a bucket share its input buffer
                    static = torch.zeros(layout["size"], dtype=torch.int32, device=self.device)
                ctx = b.to_device(buf, layout, into=static)
                ctx.token_feedback = self._sampled
                tokens = self._sampled[:bs]
                self._forward_and_sample(ctx, tokens)               # warm-up: builds kernels, sizes buffers
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                before = ops.launches
                with torch.cuda.graph(g, pool=pool):
                    self._forward_and_sample(ctx, tokens)
                pool = g.pool()
                self.graphs[bs, bound] = _DecodeGraph(g, layout, static, tokens, ops.launches - before)
        torch.cuda.synchronize()
        self._graph_pool = pool
        self.graph_sizes = sizes
        self.graph_bounds = bounds
        if self.verbose:
            print(f"[mini_inference_engine_b200] captured {len(self.graphs)} decode graphs (batch <= {sizes[-1]}, "
                  f"contexts <= {' / '.join(str(c) for c in bounds)}) in {time.perf_counter() - t0:.1f} s")

    def decode_graph(self, rows: int, context: int):
        """The captured step that serves ``rows`` decoding requests whose longest context (the new token
        included) is ``context``."""
        bs = next(s for s in self.graph_sizes if s >= rows)
        return self.graphs[bs, next(c for c in self.graph_bounds if c >= context)]

    # ------------------------------------------------------------------ CUDA graphs of prompt portions
    PORTION_GRAPH_MIN_TOKENS = 2

    @contextlib.contextmanager
    def _capturing(self, graph):
        """Captures what the body launches into ``graph`` (memory from the graphs' shared pool) in the middle of
        serving: on a side stream that waits for the serving stream, without the device-wide synchronisation and the
        emptying of the device and pinned-memory caches that ``torch.cuda.graph`` begins with -- those cost a capture
        10 to 60 ms, stall the step in flight, and leave the next eager steps to allocate their buffers anew."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
        side, main = self._capture_stream, torch.cuda.current_stream()
        side.wait_stream(main)
        with torch.cuda.stream(side):
            graph.capture_begin(self._graph_pool) if self._graph_pool is not None else graph.capture_begin()
            try:
                yield
            finally:
                graph.capture_end()
        main.wait_stream(side)

    @staticmethod
    def _padded_length(n: int) -> int:
        """The token count of the graph that serves a portion of ``n`` tokens: the next multiple of 32 up to
        256 tokens, of 64 up to 1,024, of 128 beyond (at most an eighth more tokens than the portion has)."""
        step = 32 if n <= 256 else (64 if n <= 1024 else 128)
        return -(-n // step) * step

    def _portion_rows(self, row, padded: int):
        """The portion's row and, behind it, a scratch row that brings the batch to ``padded`` tokens: its
        tokens sit at positions 0.. of page 0 (every block-table entry 0, state slot 0), nobody wants their
        logits, and what they write lands in the scratch page."""
        from .batch import BatchRow
        extra = padded - len(row.tokens)
        if extra == 0:
            return [row]
        pages = -(-extra // self.cfg.block_size)
        zeros = [np.zeros(pages, dtype=np.int32) for _ in row.tables]
        return [row, BatchRow(np.zeros(extra, dtype=np.int32), 0, zeros, 0, ())]

    @torch.inference_mode()
    def _portion_graph(self, row, extras, wanted: int):
        """The captured step for ONE prompt portion, if a step of the same padded shape (tokens, wanted
        logits) has run before; else None, and the shape is remembered.  Launching some 160 kernels one by
        one costs the host about 3 ms a step, more than a short portion takes on the device; portions are
        cut by what is left of the token budget, so their lengths are rounded up (``_padded_length``) for
        shapes to repeat.  What differs between replays -- tokens, positions, block table, the split between
        the portion and its padding, sampling inputs -- lives in the graph's static input buffer; the context
        bound that kernels plan by is the model's longest.  At most ``graph_prompt_portions`` graphs are kept
        (the least recently used one goes).  The reference launches such steps eagerly."""
        n = len(row.tokens)
        padded = self._padded_length(n)
        key = (padded, padded == n, wanted)
        g = self._portion_graphs.get(key)
        if g is not None:
            self._portion_graphs[key] = self._portion_graphs.pop(key)        # most recently used last
            return g
        if not self._portion_seen.get(key):
            if len(self._portion_seen) > 256:
                self._portion_seen.clear()
            self._portion_seen[key] = 1
            return None
        b = self.runner.builder
        buf, layout = b.pack(self._portion_rows(row, padded), table_width=self.max_blocks_per_seq, extras=extras)
        layout["max_ctx_len"] = self.cfg.max_model_len
        layout["q_len"] = None              # the split between portion and padding changes from replay to replay
        layout["few_single_rows"] = True    # (a padding of one token is a row like a decoding one: the kernel for portions serves it)
        static = torch.zeros(layout["size"], dtype=torch.int32, device=self.device)
        ctx = b.to_device(buf, layout, into=static)
        ctx.token_feedback = self._sampled
        tokens = self._sampled[self._portion_slot:self._portion_slot + wanted]
        # no warm-up run: a step of this shape has run before (kernels built, buffers sized), and running
        # this one twice would write the request's cache twice -- harmless, but not free
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        with self._capturing(graph):
            self._forward_and_sample(ctx, tokens, host_out=self._pinned_portion)
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        g = _DecodeGraph(graph, layout, static, tokens, ops.launches - before)
        while len(self._portion_graphs) >= max(1, self.cfg.graph_prompt_portions):
            self._portion_graphs.pop(next(iter(self._portion_graphs)))
        self._portion_graphs[key] = g
        return g

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt, params: SamplingParams | None = None) -> Sequence:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer in the model folder; pass token ids instead")
            ids = self.tokenizer.encode(prompt)
        else:
            ids = [int(t) for t in prompt]
        params = params or SamplingParams()
        if not ids:
            raise ValueError("empty prompt")
        bad = [t for t in ids if not 0 <= t < self.vocab_size]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary [0, {self.vocab_size})")
        if len(ids) > self.cfg.max_model_len:
            raise ValueError(f"prompt of {len(ids)} tokens exceeds max_model_len {self.cfg.max_model_len}")
        if len(ids) + params.max_tokens > self.cfg.max_model_len:     # inference_engine/engine.py:126-127
            params = SamplingParams(**{**params.__dict__, "max_tokens": max(1, self.cfg.max_model_len - len(ids))})
        most = min(len(ids) + params.max_tokens, self.cfg.max_model_len)
        if not self.scheduler.can_ever_fit(most):
            raise ValueError(f"a request of {most} positions can never fit the cache "
                             f"({self.cache.pools[0].num_usable} usable pages of {self.cfg.block_size})")
        seq = Sequence(ids, params)
        self.scheduler.add(seq)
        return seq

    # ------------------------------------------------------------------ one engine step
    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._in_flight is not None

    @torch.inference_mode()
    def step(self) -> list:
        """One scheduling + model step; returns the requests whose end became known in it.

        With ``overlap_steps`` the host runs one step ahead of the device: step N+1 is scheduled,
        packed and launched while step N still runs, and only then are step N's tokens read.  The
        tokens a step samples stay on the device and are fed to the next step there (a token id
        -(k+1) in the batch means "entry k of the previous step's samples"), so nothing but the stop
        rules waits for the host: a request that ends by count is known beforehand, one that ends by
        EOS runs one step too many, whose token is dropped."""
        launched = self._launch()
        finished = self._complete(self._in_flight) if self._in_flight is not None else []
        self._in_flight = launched
        # nothing to run ahead of: read the step's tokens now (also keeps the reference's loop
        # `while engine.scheduler.has_work(): engine.step()` complete)
        if launched is not None and (not self.cfg.overlap_steps or not self.scheduler.has_work()):
            finished += self.drain()
        return finished

    def drain(self) -> list:
        """Reads the tokens of the step in flight, if any; returns the requests that ended with it."""
        fl, self._in_flight = self._in_flight, None
        return self._complete(fl) if fl is not None else []

    def _launch(self):
        with _nvtx_range("schedule"):
            batch = self.scheduler.schedule()
        if not batch:
            return None
        with _nvtx_range("prepare"):
            rows, sample_seqs, decoding, others = [], [], [], []
            make_row = self.runner.make_row
            for i, (seq, n) in enumerate(batch):
                nc = seq.cache.num_computed
                last = nc + n == len(seq.token_ids)
                if nc + n <= seq.prompt_len:
                    tokens = seq.prompt_array[nc:nc + n]       # a view: a prompt portion
                else:
                    tokens = seq.token_ids[nc:nc + n]
                    if tokens[-1] == PENDING:              # sampled by the step in flight: read on the device
                        tokens[-1] = -(seq.pending_index + 1)
                rows.append(make_row(seq.cache, tokens, (n - 1,) if last else ()))
                if last:
                    sample_seqs.append(seq)
                (decoding if n == 1 and last else others).append(i)
            turn = self._turn ^ 1                              # the row of the pinned token buffers that this step fills
            row_seeds, seeds = self.sampler.seeds_of(sample_seqs)
            graphs_ok = bool(self.graph_sizes) and len(decoding) <= self.graph_sizes[-1] and seeds <= {self.cfg.seed}
            use_graph = graphs_ok and not others
            # One prompt portion, alone or beside requests that decode, runs as a graph of its padded length
            # -- beside the decode bucket's graph if there is one: two replays instead of some 200 launches
            # that cost the host more than the step costs the device.  The rows of the two replays do not
            # depend on one another, so the split changes nothing in what each computes.
            portion_graph = (graphs_ok and self.cfg.use_cuda_graphs and self.cfg.graph_prompt_portions > 0
                             and len(others) == 1 and len(rows[others[0]].tokens) >= self.PORTION_GRAPH_MIN_TOKENS
                             and (not decoding or len(rows[others[0]].tokens) <= self.cfg.split_step_max_tokens))

        def extras_for(seqs, pad_to):
            return self.sampler.inputs(pad_to or len(seqs), seqs, turn)

        with _nvtx_range("forward"):
            b = self.runner.builder
            sources = []
            if use_graph or (portion_graph and decoding):      # ---- the requests that decode, from their bucket's graph
                drows = [rows[i] for i in decoding]
                dseqs = [batch[i][0] for i in decoding]
                bs = next(s for s in self.graph_sizes if s >= len(drows))
                g = self.decode_graph(bs, max(seq.cache.num_computed + 1 for seq in dseqs))
                buf, layout = b.pack(drows, pad_rows=bs, table_width=self.max_blocks_per_seq, extras=extras_for(dseqs, bs))
                assert layout["size"] == g.layout["size"]
                b.to_device(buf, g.layout, into=g.buffer)
                g.graph.replay()
                self.h2d_bytes += buf.nbytes
                sources.append((self._pinned_tokens[turn], len(dseqs)))
                for k, seq in enumerate(dseqs):
                    seq.pending_index = k
                if use_graph:
                    self.num_graph_steps += 1
            if use_graph:
                pass
            elif portion_graph:                                # ---- the one prompt portion, from a graph of its padded length
                row = rows[others[0]]
                pseq = batch[others[0]][0]
                pseqs = [pseq] if row.want else []
                extras = extras_for(pseqs, 0)
                pg = self._portion_graph(row, extras, len(pseqs))
                tokens = self._sampled[self._portion_slot:self._portion_slot + len(pseqs)]
                if pg is not None:
                    buf, layout = b.pack(self._portion_rows(row, self._padded_length(len(row.tokens))),
                                         table_width=self.max_blocks_per_seq, extras=extras)
                    assert layout["size"] == pg.layout["size"]
                    b.to_device(buf, pg.layout, into=pg.buffer)
                    pg.graph.replay()
                    self.num_portion_graph_steps += 1
                else:                                          # the first time a shape occurs: launched kernel by kernel
                    buf, layout = b.pack([row], extras=extras)
                    ctx = b.to_device(buf, layout)
                    ctx.token_feedback = self._sampled
                    self._forward_and_sample(ctx, tokens, host_out=self._pinned_portion)
                self.h2d_bytes += buf.nbytes
                if pseqs:
                    sources.append((self._pinned_portion[turn], 1))
                    pseq.pending_index = self._portion_slot
            else:                                              # ---- any other mix: one batch, launched kernel by kernel
                k = len(sample_seqs)
                extras = extras_for(sample_seqs, 0)
                buf, layout = b.pack(rows, extras=extras)
                ctx = b.to_device(buf, layout)
                ctx.token_feedback = self._sampled
                self.h2d_bytes += buf.nbytes
                logits = self.model.step(ctx)
                if sample_seqs and not self.sampler.sample_step(logits, ctx.extras, self._sampled[:k], row_seeds, seeds,
                                                                host_out=self._pinned_tokens):
                    self._pinned_tokens[turn, :k].copy_(self._sampled[:k], non_blocking=True)   # this rare way copies
                sources.append((self._pinned_tokens[turn], k))
                for k2, seq in enumerate(sample_seqs):
                    seq.pending_index = k2
            self._turn = turn
            self.d2h_bytes += 4 * len(sample_seqs)             # written by the sampling kernel into pinned host memory
            done_event = torch.cuda.Event()
            done_event.record()

        # bookkeeping that does not need the tokens: progress, the place each token will take, and the
        # requests that end by count with this step
        self.num_steps += 1
        for seq, n in batch:
            self.cache.advance(seq.cache, n)
        ending = []
        max_len = self.cfg.max_model_len
        for seq in sample_seqs:
            seq.token_ids.append(PENDING)
            total = len(seq.token_ids)
            if total - seq.prompt_len >= seq.params.max_tokens or total >= max_len:
                self.scheduler.finish(seq)                 # its pages may go to the next step: that one runs after this one
                ending.append(seq)
        return _InFlight(sample_seqs, [s.num_tokens - 1 for s in sample_seqs], ending, sources, done_event)

    def _complete(self, fl) -> list:
        with _nvtx_range("sample"):
            fl.event.synchronize()
            new_tokens = fl.tokens()
        ops.check_range_errors()           # an integer out of range that a kernel refused to follow
        ops.check_tc_errors()
        gemm_tc.check_error()              # a bounded wait that ran out in a tensor-core product is an error, not a result
        now = time.perf_counter()
        finished = []
        for seq, place, tok in zip(fl.seqs, fl.places, new_tokens):
            if seq.ended_by_eos:
                del seq.token_ids[place:]                  # it ended by EOS a step ago: this token is one too many
                continue
            seq.token_ids[place] = tok
            if seq.first_token_time is None:
                seq.first_token_time = now
            if seq in fl.ending:
                seq.finish_time = now
                finished.append(seq)
            elif tok == self.eos_token_id and not seq.params.ignore_eos:      # inference_engine/engine.py:222-224
                del seq.token_ids[place + 1:]              # a token pending from the step already in flight
                seq.ended_by_eos = True
                seq.finish_time = now
                self.scheduler.finish(seq)
                finished.append(seq)
        return finished

    # ------------------------------------------------------------------ offline API
    def generate(self, prompts, params=None, decode_text: bool = True) -> list:
        if not isinstance(params, list):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt")
        seqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_work():
            self.step()
        outs = []
        for s in seqs:
            text = None
            if decode_text and self.tokenizer is not None:
                text = self.tokenizer.decode(s.output_ids, skip_special_tokens=True)
            outs.append(RequestOutput(s.seq_id, s.prompt_len, s.output_ids, text,
                                      s.first_token_time - s.arrival_time, s.finish_time - s.arrival_time))
        return outs
