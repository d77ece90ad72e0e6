"""Engine options.  Names and meanings follow ``EngineConfig`` of
inference_engine/config.py:45-56; the two Triton switches have no counterpart here
(every GPU op is this package's own CUDA), and ``num_blocks`` and ``seed`` are added:
tests need tiny page pools (the reference can only shrink its pool through the memory
fraction, tests/test_correctness.py:46), and seeded sampling needs a seed; ``overlap_steps`` and
``graph_prompt_portions`` (with ``split_step_max_tokens``) switch two things that the reference does not have."""
from __future__ import annotations

from dataclasses import dataclass, fields


@dataclass
class EngineConfig:
    block_size: int = 16                    # tokens per cache page
    max_num_seqs: int = 256                 # most requests running at once
    max_num_batched_tokens: int = 2048      # token budget of one step (caps a prompt portion)
    kv_cache_memory_fraction: float = 0.85  # of the memory free after the weights are loaded
    max_model_len: int = 2048
    enable_chunked_prefill: bool = True
    use_cuda_graphs: bool = True
    cuda_graph_batch_sizes: tuple = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 160, 192, 224, 256)
    graph_context_bounds: tuple = (960,)    # decode graphs are captured once per bucket for each of these context bounds
                                            # below max_model_len, and once for max_model_len: kernels that plan by the
                                            # longest context a launch may meet (decode attention cuts long contexts into
                                            # parts) then get a plan that fits the requests a step really holds
    num_blocks: int | None = None           # explicit pool size in pages (page 0 included); None = from memory
    seed: int = 0                           # sampling seed
    overlap_steps: bool = True              # launch step N+1 before reading step N's tokens (they are fed back on the device)
    graph_prompt_portions: int = 16         # graphs kept for prompt portions, by padded length (0 = none: such steps launch kernel by kernel)
    warm_up_prompt_step: bool = True        # run one prompt step of the whole token budget on the scratch page at construction:
                                            # kernels for portions, the library's choices for that many rows and the
                                            # allocator's blocks are then in place before the first request's first step
    split_step_max_tokens: int = 512        # a portion of up to this many tokens beside decoding requests runs as a graph of
                                            # its own after the decode graph (the weights are read twice, the host launches
                                            # twice instead of 200 times); a longer one keeps the device busy longer than the
                                            # host needs for its launches, and the step stays one batch

    def __post_init__(self):
        if self.block_size < 16 or self.block_size & (self.block_size - 1) or self.block_size > 128:
            raise ValueError(f"block_size must be a power of two in 16..128, got {self.block_size}")
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1 or self.max_model_len < 1:
            raise ValueError("max_num_seqs, max_num_batched_tokens and max_model_len must be positive")
        self.cuda_graph_batch_sizes = tuple(sorted(set(int(b) for b in self.cuda_graph_batch_sizes)))
        self.graph_context_bounds = tuple(sorted(set(int(b) for b in self.graph_context_bounds if int(b) > 0)))

    @classmethod
    def from_overrides(cls, overrides: dict | None) -> "EngineConfig":
        """``--overrides '<json>'`` of benchmarks/bench_throughput.py:100,147."""
        overrides = dict(overrides or {})
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(overrides) - known)
        if unknown:
            raise ValueError(f"unknown EngineConfig option(s): {', '.join(unknown)}")
        return cls(**overrides)
