"""The benchmark language model of the reference's training configurations, as a harness.

A pre-norm causal decoder (LayerNorm, bias-free projections, SwiGLU MLP, learned position
embedding) whose residual stream is replaced by AttnRes reads, with the two source schedules
of the reference's benchmark model (benchmarks/model.py:293-338 of the reference):

* **Full**: the first attention consumes the embedding; every later sublayer and the LM head
  read ALL earlier sublayer outputs plus the embedding (S = 2 .. 2L+1), and
* **Block**: sublayer outputs are summed inside blocks of ``block_layers`` layers; a read sees
  the embedding, the sums of the completed blocks and the running partial sum of the current
  block (S <= blocks + 1).

Both are one schedule here: a block boundary after every event gives Full.  Every read has its
own learned ``[rank]`` query (rank < width reads the last ``rank`` coordinates as the key, the
reference's "sliced" variant) and goes through an injected ``operator(values, query)``, so
this library, the reference's Triton package and the oracle all drive the same network.
Parameter names follow the reference model so state dicts are interchangeable.

This file is benchmark and test scaffolding (used by bench.py's model workloads,
baseline/train_step_ab.py and tests/test_lm_schedule.py), not part of the operator package.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class LMConfig:
    layers: int = 2
    width: int = 128
    heads: int = 4
    ffn: int = 512
    vocab: int = 512
    sequence: int = 64
    rank: int | None = None          # None: full rank (= width)
    mode: str = "full"               # "full" or "block"
    block_layers: int = 4            # layers per block in Block mode
    layout: str = "list"             # "list": a tuple of sources; "packed": torch.stack first

    def __post_init__(self):
        if self.rank is None:
            self.rank = self.width
        if self.mode not in ("full", "block") or self.layout not in ("list", "packed"):
            raise ValueError("mode is 'full' or 'block', layout 'list' or 'packed'")
        if self.width % self.heads or not 1 <= self.rank <= self.width:
            raise ValueError("width must be divisible by heads and 1 <= rank <= width")

    @property
    def events(self) -> int:          # sublayers: attention and MLP of every layer
        return 2 * self.layers

    @property
    def block_count(self) -> int:
        return self.events if self.mode == "full" else math.ceil(self.layers / self.block_layers)


def block_ends(events: int, block_count: int) -> tuple[int, ...]:
    """One-based event indices after which a block is complete: evenly sized blocks
    (benchmarks/model.py:117-121 of the reference)."""
    count = min(events, block_count)
    return tuple(math.ceil(events * i / count) for i in range(1, count + 1))


class SourceSchedule:
    """Which tensors a read sees.  ``completed`` holds the embedding and the finished block
    sums, ``partial`` the running sum of the current block."""

    def __init__(self, embedding, events: int, block_count: int):
        self.completed = [embedding]
        self.partial = None
        self.ends = set(block_ends(events, block_count))
        self.done = 0

    def sources(self) -> list:
        return self.completed + ([self.partial] if self.partial is not None else [])

    def emit(self, value, add=lambda a, b: a + b) -> None:
        self.partial = value if self.partial is None else add(self.partial, value)
        self.done += 1
        if self.done in self.ends:
            self.completed.append(self.partial)
            self.partial = None


def read_source_counts(config: LMConfig) -> tuple[int, ...]:
    """S of every read, in order (the last one feeds the LM head).  Matches the reference's
    own count (benchmarks/run.py:687-739): Full gives 2 .. 2L+1."""
    schedule = SourceSchedule(0, config.events, config.block_count)
    counts = []
    for event in range(config.events):
        if event:
            counts.append(len(schedule.sources()))
        schedule.emit(1, add=lambda a, b: a)
    counts.append(len(schedule.sources()))
    return tuple(counts)


def attnres_algorithmic_bytes(config: LMConfig, rows: int) -> int:
    """Forward + backward bytes of all reads of one step: 6 S D + 4 D per position and read."""
    return rows * sum(6 * s * config.width + 4 * config.width for s in read_source_counts(config))


class _Layer(nn.Module):
    def __init__(self, config: LMConfig):
        super().__init__()
        width = config.width
        self.heads, self.width = config.heads, width
        self.norm_attention = nn.LayerNorm(width)
        self.q_proj = nn.Linear(width, width, bias=False)
        self.k_proj = nn.Linear(width, width, bias=False)
        self.v_proj = nn.Linear(width, width, bias=False)
        self.attention_output = nn.Linear(width, width, bias=False)
        self.norm_mlp = nn.LayerNorm(width)
        self.gate_proj = nn.Linear(width, config.ffn, bias=False)
        self.up_proj = nn.Linear(width, config.ffn, bias=False)
        self.down_proj = nn.Linear(config.ffn, width, bias=False)

    def attention_from_normed(self, h):
        b, t, _ = h.shape
        split = lambda y: y.view(b, t, self.heads, self.width // self.heads).transpose(1, 2)
        a = F.scaled_dot_product_attention(split(self.q_proj(h)), split(self.k_proj(h)),
                                           split(self.v_proj(h)), is_causal=True)
        return self.attention_output(a.transpose(1, 2).reshape(b, t, self.width))

    def mlp_from_normed(self, h):
        return self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))

    def attention(self, x):
        return self.attention_from_normed(self.norm_attention(x))

    def mlp(self, x):
        return self.mlp_from_normed(self.norm_mlp(x))


class CausalLM(nn.Module):
    """``operator(values, query)`` is any implementation of the read; ``normed_operator``,
    when given, is ``(values, query, weight, bias, norm_eps) -> LayerNorm(read)`` and replaces
    the read + LayerNorm pair in front of every sublayer (the fused epilogue)."""

    def __init__(self, config: LMConfig, operator, normed_operator=None):
        super().__init__()
        self.config, self.operator, self.normed_operator = config, operator, normed_operator
        self.token_embedding = nn.Embedding(config.vocab, config.width)
        self.position_embedding = nn.Parameter(torch.empty(config.sequence, config.width))
        self.layers = nn.ModuleList(_Layer(config) for _ in range(config.layers))
        self.lm_head = nn.Linear(config.width, config.vocab, bias=False)
        self.queries = nn.ParameterList(nn.Parameter(torch.empty(config.rank))
                                        for _ in range(config.events))
        for module in self.modules():
            if isinstance(module, (nn.Linear, nn.Embedding)):
                nn.init.normal_(module.weight, mean=0.0, std=0.02)
        nn.init.normal_(self.position_embedding, mean=0.0, std=0.02)
        for query in self.queries:
            nn.init.normal_(query, mean=0.0, std=0.02)

    def embed(self, tokens):
        """The first source, in the working dtype of the residual stream: the autocast dtype
        when autocast is on, else the parameters' (benchmarks/model.py:239-245 of the reference).
        Reads always see BF16 and return the working dtype."""
        embedded = self.token_embedding(tokens) + self.position_embedding[: tokens.shape[-1]]
        device_type = embedded.device.type
        if torch.is_autocast_enabled(device_type):
            embedded = embedded.to(torch.get_autocast_dtype(device_type))
        return embedded

    def _values(self, sources):
        sources = tuple(s.to(torch.bfloat16) for s in sources)
        return torch.stack(sources) if self.config.layout == "packed" else sources

    def read(self, sources, index):
        out = self.operator(self._values(sources), self.queries[index].to(torch.bfloat16))
        return out.to(sources[0].dtype)

    def sublayer(self, event, sources):
        """Output of sublayer `event` (even: attention, odd: MLP) given what it may read."""
        layer = self.layers[event // 2]
        norm = layer.norm_attention if event % 2 == 0 else layer.norm_mlp
        body = layer.attention_from_normed if event % 2 == 0 else layer.mlp_from_normed
        if event == 0:
            return body(norm(sources[0]))
        if self.normed_operator is not None:
            normed = self.normed_operator(self._values(sources),
                                          self.queries[event - 1].to(torch.bfloat16),
                                          norm.weight, norm.bias, norm.eps)
            return body(normed.to(norm.weight.dtype)
                        if not torch.is_autocast_enabled(normed.device.type) else normed)
        return body(norm(self.read(sources, event - 1)))

    def forward(self, tokens):
        config = self.config
        schedule = SourceSchedule(self.embed(tokens), config.events, config.block_count)
        for event in range(config.events):
            schedule.emit(self.sublayer(event, schedule.sources()))
        return self.lm_head(self.read(schedule.sources(), config.events - 1))


def make_optimizer(model, *, capturable: bool, lr: float = 3e-4):
    """The reference's optimiser settings (benchmarks/run.py:2369-2375 of the reference)."""
    return torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.1,
                             fused=True, capturable=capturable)


def training_step(model, optimizer, tokens, targets, *, accumulation: int = 1, sync_context=None):
    """zero_grad, BF16-autocast forward, cross entropy, backward over `accumulation`
    microbatches, optimiser step (benchmarks/training_graph.py:24-58 of the reference).
    ``sync_context(last)`` may return a context manager per microbatch (DDP's ``no_sync``)."""
    import contextlib
    optimizer.zero_grad(set_to_none=False)
    loss = None
    for index, (micro_tokens, micro_targets) in enumerate(zip(tokens.chunk(accumulation),
                                                              targets.chunk(accumulation))):
        context = (sync_context(index == accumulation - 1) if sync_context is not None
                   else contextlib.nullcontext())
        with context:
            with torch.autocast("cuda" if tokens.is_cuda else "cpu", dtype=torch.bfloat16):
                logits = model(micro_tokens)
                loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]),
                                       micro_targets.reshape(-1))
            (loss / accumulation).backward()
    optimizer.step()
    return loss.detach()


class CapturedStep:
    """One training step captured in ONE CUDA graph after eager warm-up on a side stream, with
    model and optimiser state restored to their values from before the warm-up so that every
    arm of a comparison starts its timed replays from the same state
    (benchmarks/training_graph.py:126-255 of the reference)."""

    def __init__(self, step, model, optimizer, *, warmup: int = 3):
        self.loss = torch.zeros((), device=next(model.parameters()).device)
        model_state = {k: v.detach().clone() for k, v in model.state_dict().items()}
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.loss.copy_(step())
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.loss_after_warmup = float(self.loss)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss.copy_(step())
        # restore: parameters in place, optimiser moments and step counters to zero
        with torch.no_grad():
            current = model.state_dict()
            for name, value in model_state.items():
                current[name].copy_(value)
            for state in optimizer.state.values():
                for value in state.values():
                    if isinstance(value, torch.Tensor):
                        value.zero_()
        torch.cuda.synchronize()

    def replay(self):
        self.graph.replay()

    def time_replays(self, steps: int, discard: int = 2) -> list[float]:
        times = []
        for _ in range(steps + discard):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            self.graph.replay()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        return times[discard:]
