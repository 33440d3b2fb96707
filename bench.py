"""Benchmark of the AttnRes read (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the reference's "standard full-rank operator sweep", its second benchmark
configuration): packed BF16
values [S, 16384, D] ~ N(0,1) for S in {2,5,9,17,25,49} x D in {1024,2048,4096},
query [D] ~ N(0,0.02), R = D, upstream gradient ~ N(0,1).  One STEP is one
forward and one backward of every one of the 18 cells: all forwards first, then
all backwards in reverse order, as a network would run them; more than 25 GB of
other traffic separates a cell's forward from its backward, so nothing is served
from L2 between timed passes.

With N > 1 (torchrun) every rank owns its own 16 384 positions of every cell
(position sharding, no data-path collective; weak scaling) and the FP32 query
gradients of all cells are summed over NCCL (one bucketed all-reduce per step) before the
BF16 cast.  The same line then carries a `strong` record (the 16 384 positions of every
cell split over the ranks), every rank's own kernel time and the collective's own time.

`--workload config4|config5` times a training step of the benchmark language model instead
(baseline/lm.py: the reference's 24-layer Full-schedule and 8-GPU Block-schedule
configurations), data-parallel over the ranks with the gradient all-reduce overlapping the
backward.

Printed JSON (rank 0, one line): whole-job tokens/s (`value`), the HBM roofline
of the dominant (backward) kernel, the same metric end to end from pinned host
buffers through the public `attnres()` API (`e2e`), the CPU oracle timed on the
host cores (`cpu_baseline`) and the SM clocks sampled during the timed region.

`--impl reference` times the reference's CPU definition of the path (the PyTorch
oracle port, all host threads) on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for entry in (ROOT, ROOT / "fast-attnres_b200"):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))

import torch  # noqa: E402

ROWS = 16384
SOURCE_COUNTS = (2, 5, 9, 17, 25, 49)
WIDTHS = (1024, 2048, 4096)
CELLS = [(s, d) for d in WIDTHS for s in SOURCE_COUNTS]
CPU_SAMPLE_ROWS = 512
E2E_BLOCK_ROWS = 4096   # rows per host-to-device block of the end-to-end leg
SEED = 20260827
METRIC = "attnres_fwd_bwd_tokens_per_s"
WORKLOAD = "config2_operator_sweep_packed_S{2,5,9,17,25,49}xD{1024,2048,4096}_N16384_R=D"


def algorithmic_bytes(sources: int, rows: int, width: int) -> tuple[int, int]:
    """(forward, backward) bytes per call: values read + output written; values and
    upstream read + value gradients written.  Statistics, the dquery workspace and
    the query itself are overhead and are not counted."""
    forward = rows * (2 * sources * width + 2 * width)
    backward = rows * (2 * sources * width + 2 * width + 2 * sources * width)
    return forward, backward


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def traffic_ratios() -> dict:
    """DRAM bytes / algorithmic bytes per backward kernel family ("stream", "stash", "ring")
    from the committed ncu captures (profiles/dram_traffic.json); empty when none is recorded."""
    path = ROOT / "profiles" / "dram_traffic.json"
    if path.exists():
        try:
            table = json.loads(path.read_text())["backward"]
            return {name: float(entry["dram_over_algorithmic"]) for name, entry in table.items()
                    if isinstance(entry, dict) and "dram_over_algorithmic" in entry}
        except Exception:
            return {}
    return {}


def backward_family(sources: int, saves_output: bool) -> str:
    """Which backward kernel the library runs for a cell of the sweep (aligned layout)."""
    if saves_output:
        return "stream"
    return "ring" if sources <= 4 else "stash"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = index
            if visible:
                entries = [e.strip() for e in visible.split(",") if e.strip()]
                if index < len(entries) and entries[index].isdigit():
                    physical = int(entries[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None

    def _loop(self):
        nv = self.nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"]}
        ordered = sorted(self.samples)
        return {"sm_mhz": ordered[len(ordered) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(ordered)}


# ----------------------------------------------------------------------------- CPU arm

def cpu_oracle_tokens_per_s(rows: int, repeats: int = 1) -> tuple[float, float, int]:
    """Forward+backward of the PyTorch oracle port on the host, every cell at `rows`
    rows; returns (tokens/s, seconds of CPU work, threads)."""
    from oracle import attnres_oracle as ao
    generator = torch.Generator().manual_seed(SEED)
    cases = []
    for sources, width in CELLS:
        values = torch.randn(sources, rows, width, generator=generator).to(torch.bfloat16)
        query = (torch.randn(width, generator=generator) * 0.02).to(torch.bfloat16)
        upstream = torch.randn(rows, width, generator=generator).to(torch.bfloat16)
        cases.append((values, query, upstream))
    ao.oracle_with_grads(*cases[0])  # warm the thread pool
    start = time.perf_counter()
    for _ in range(repeats):
        for values, query, upstream in cases:
            ao.oracle_with_grads(values, query, upstream)
    seconds = time.perf_counter() - start
    return repeats * len(CELLS) * rows / seconds, seconds, torch.get_num_threads()


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1 to every rank; the CPU arm runs on rank 0 alone and
    takes every host core, as it does when launched without torchrun."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    return torch.get_num_threads()


def run_reference_arm(args, rank: int) -> None:
    if rank != 0:
        return
    use_all_host_threads()
    rates, elapsed = [], 0.0
    for _ in range(max(1, min(args.warmup, 2))):  # untimed passes
        cpu_oracle_tokens_per_s(CPU_SAMPLE_ROWS)
    for _ in range(args.steps):
        rate, seconds, threads = cpu_oracle_tokens_per_s(CPU_SAMPLE_ROWS)
        rates.append(rate)
        elapsed += seconds
    value = sum(rates) / len(rates)
    sample = f"all 18 cells at {CPU_SAMPLE_ROWS} rows each per step (same S, D, R; rows reduced)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * elapsed / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 storage / fp32 arithmetic", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_step": CPU_SAMPLE_ROWS * len(CELLS)},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm

class Cell:
    """Device buffers and captured graphs of one (S, D) cell."""

    def __init__(self, sources, width, device, generator, grad_buffer, out_buffer, upstream):
        from attnres import _native
        self.S, self.D, self.N = sources, width, ROWS
        self.values = torch.randn(sources, ROWS, width, device=device, dtype=torch.bfloat16,
                                  generator=generator)
        self.query = (torch.randn(width, device=device, generator=generator) * 0.02).to(torch.bfloat16)
        self.upstream = upstream
        # Where the library's one-pass backward wants the forward's output and its 16-bit
        # residual, both must survive until the cell's backward: such a cell owns them.
        self.saves_output = _native.wants_output_residual(sources, width, width)
        if self.saves_output:
            self.out = torch.empty(ROWS, width, device=device, dtype=torch.bfloat16)
            self.residual = torch.empty(ROWS, width, device=device, dtype=torch.int16)
        else:
            self.out = out_buffer[:ROWS * width].view(ROWS, width)
            self.residual = None
        self.family = backward_family(sources, self.saves_output)
        self.grad = grad_buffer[:sources * ROWS * width].view(sources, ROWS, width)
        self.logits = torch.empty(sources, ROWS, device=device, dtype=torch.float32)
        self.stats = torch.empty(2, ROWS, device=device, dtype=torch.float32)
        self.partial_rows = _native.dq_workspace_rows(ROWS, sources, width, width, device.index)
        self.partials = torch.empty(self.partial_rows, width, device=device, dtype=torch.float32)
        self.dq32 = torch.empty(width, device=device, dtype=torch.float32)
        self.dq = torch.empty(width, device=device, dtype=torch.bfloat16)
        step = ROWS * width * 2
        self.src_ptrs = [self.values.data_ptr() + s * step for s in range(sources)]
        self.grad_ptrs = [self.grad.data_ptr() + s * step for s in range(sources)]
        self.fwd_bytes, self.bwd_bytes = algorithmic_bytes(sources, ROWS, width)
        self.graphs = {}   # rows -> (forward graph, backward graph)

    def forward(self, stream, rows):
        """The first `rows` positions of the cell (all of them in the weak-scaling step; a
        1/world share in the strong-scaling one: the row stride of the sources is unchanged,
        the logits and statistics are laid out for `rows` positions)."""
        from attnres import _native
        _native.forward(self.src_ptrs, [self.D] * self.S, [1] * self.S, self.S, rows, self.D,
                        self.D, self.query.data_ptr(), 1, 2**-23, 1.0, self.out.data_ptr(), self.D,
                        self.logits.data_ptr(), self.stats.data_ptr(), 0, stream,
                        residual_ptr=self.residual.data_ptr() if self.saves_output else None)

    def backward(self, stream, rows, distributed):
        from attnres import _native
        _native.backward(self.src_ptrs, [self.D] * self.S, [1] * self.S, self.S, rows, self.D,
                         self.D, self.query.data_ptr(), 1, 2**-23, 1.0,
                         self.upstream.data_ptr(), self.D, 1,
                         self.logits.data_ptr(), self.stats.data_ptr(),
                         self.grad_ptrs, [self.D] * self.S,
                         self.partials.data_ptr(), self.partial_rows,
                         None if distributed else self.dq.data_ptr(),
                         self.dq32.data_ptr() if distributed else None, 0, stream,
                         out_ptr=self.out.data_ptr() if self.saves_output else None,
                         residual_ptr=self.residual.data_ptr() if self.saves_output else None)

    def capture(self, rows, distributed):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.forward(side.cuda_stream, rows)
            self.backward(side.cuda_stream, rows, distributed)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        fwd_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fwd_graph):
            self.forward(torch.cuda.current_stream().cuda_stream, rows)
        bwd_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(bwd_graph):
            self.backward(torch.cuda.current_stream().cuda_stream, rows, distributed)
        self.graphs[rows] = (fwd_graph, bwd_graph)


def time_sweep(cells, rows, steps, warmup, flat32, flat16, distributed, device, sampler=None):
    """`warmup` untimed and `steps` timed steps of the sweep at `rows` positions per cell and
    rank.  Returns (ms per step, max over ranks; per-cell forward ms; per-cell backward ms;
    this rank's own kernel ms per step; ms per step of the collective and the cast)."""
    import contextlib
    import torch.distributed as dist

    def pairs(count):
        return [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                for _ in range(count)]

    def step(fwd_events=None, bwd_events=None, tail_events=None):
        for index, cell in enumerate(cells):
            if fwd_events:
                fwd_events[index][0].record()
            cell.graphs[rows][0].replay()
            if fwd_events:
                fwd_events[index][1].record()
        for index in reversed(range(len(cells))):
            if bwd_events:
                bwd_events[index][0].record()
            cells[index].graphs[rows][1].replay()
            if bwd_events:
                bwd_events[index][1].record()
        if distributed:
            # The host is many launches ahead of the GPU here, so the collective is already
            # queued when the last backward ends; what it costs is its own kernels and the wait
            # for the slowest rank.
            if tail_events:
                tail_events[0].record()
            dist.all_reduce(flat32)
            flat16.copy_(flat32)
            if tail_events:
                tail_events[1].record()

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    records = []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with (sampler if sampler is not None else contextlib.nullcontext()):
        start.record()
        for _ in range(steps):
            fe, be, te = pairs(len(cells)), pairs(len(cells)), pairs(1)[0]
            step(fe, be, te)
            records.append((fe, be, te))
        stop.record()
        barrier()
    total_ms = start.elapsed_time(stop)
    fwd_ms, bwd_ms, tail_ms = [0.0] * len(cells), [0.0] * len(cells), 0.0
    for fe, be, te in records:
        for index in range(len(cells)):
            fwd_ms[index] += fe[index][0].elapsed_time(fe[index][1]) / steps
            bwd_ms[index] += be[index][0].elapsed_time(be[index][1]) / steps
        if distributed:
            tail_ms += te[0].elapsed_time(te[1]) / steps
    own_ms = sum(fwd_ms) + sum(bwd_ms)
    if distributed:
        worst = torch.tensor([total_ms], device=device, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        total_ms = float(worst.item())
    return total_ms / steps, fwd_ms, bwd_ms, own_ms, tail_ms


COPY_PIECE_ELEMS = 128 * 1024 * 1024      # BF16 elements per memcpy of the calibration copies


def time_same_size_copies(cells, grad_buffer, steps, warmup):
    """A plain device-to-device copy that moves as many bytes as each cell's forward and each
    cell's backward (half read, half written), replayed and timed exactly like the sweep: one
    CUDA graph per copy, the forward-sized copies in cell order, the backward-sized ones in
    reverse, CUDA events around every replay.  The copy bandwidth a short launch reaches is
    well below the large-copy peak (launch, ramp-up and tail are a fixed cost), so this is what
    the small cells' rates are to be read against.  A copy is issued in pieces of 256 MiB: one
    device-to-device memcpy of more than about 500 MB ran at 2.9 TB/s on B200 (0.45 of what the
    smaller ones reach), which would be no yardstick.  Returns per cell (forward-sized copy
    GB/s, backward-sized copy GB/s)."""
    plans = []
    for cell in cells:
        source = cell.values.view(-1)
        graphs = []
        for total in (cell.fwd_bytes, cell.bwd_bytes):
            elems = min(total // 4, source.numel())       # 2 B read + 2 B written per element
            src, dst = source[:elems], grad_buffer[:elems]

            def copy_in_pieces():
                for begin in range(0, elems, COPY_PIECE_ELEMS):
                    dst[begin:begin + COPY_PIECE_ELEMS].copy_(src[begin:begin + COPY_PIECE_ELEMS])

            copy_in_pieces()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                copy_in_pieces()
            graphs.append((graph, elems * 4))
        plans.append(graphs)
    totals = [[0.0, 0.0] for _ in cells]
    for iteration in range(warmup + steps):
        events = [[None, None] for _ in cells]
        for which, order in ((0, range(len(cells))), (1, reversed(range(len(cells))))):
            for index in order:
                first, last = (torch.cuda.Event(enable_timing=True) for _ in range(2))
                first.record()
                plans[index][which][0].replay()
                last.record()
                events[index][which] = (first, last)
        torch.cuda.synchronize()
        if iteration >= warmup:
            for index in range(len(cells)):
                for which in (0, 1):
                    first, last = events[index][which]
                    totals[index][which] += first.elapsed_time(last) / steps
    return [(plans[i][0][1] / (totals[i][0] * 1e-3) / 1e9, plans[i][1][1] / (totals[i][1] * 1e-3) / 1e9)
            for i in range(len(cells))]


def gather_floats(value: float, device, world: int) -> list[float]:
    import torch.distributed as dist
    if world == 1:
        return [value]
    mine = torch.tensor([value], device=device, dtype=torch.float64)
    every = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    return [float(t.item()) for t in every]


def run_gpu_arm(args, rank: int, world: int, local_rank: int) -> None:
    from attnres import _native
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    distributed = world > 1
    _native.load()
    generator = torch.Generator(device=device).manual_seed(SEED + rank)

    max_elems = max(s * ROWS * d for s, d in CELLS)
    grad_buffer = torch.empty(max_elems, device=device, dtype=torch.bfloat16)
    out_buffer = torch.empty(ROWS * max(WIDTHS), device=device, dtype=torch.bfloat16)
    upstreams = {d: torch.randn(ROWS, d, device=device, dtype=torch.bfloat16, generator=generator)
                 for d in WIDTHS}
    cells = [Cell(s, d, device, generator, grad_buffer, out_buffer, upstreams[d]) for s, d in CELLS]
    # The query gradients of all cells live in one flat FP32 bucket (and one BF16 bucket), so
    # the cross-rank sum of a step is ONE all-reduce, as a data-parallel framework buckets them.
    flat32 = torch.empty(sum(c.D for c in cells), device=device, dtype=torch.float32)
    flat16 = torch.empty_like(flat32, dtype=torch.bfloat16)
    offset = 0
    for cell in cells:
        cell.dq32, cell.dq = flat32[offset:offset + cell.D], flat16[offset:offset + cell.D]
        offset += cell.D
    # Weak scaling (the headline): every rank owns ROWS positions of every cell.  Strong
    # scaling (a sub-record): the ROWS positions of every cell are split over the ranks.
    strong_rows = ROWS // world
    for cell in cells:
        cell.capture(ROWS, distributed)
        if distributed:
            cell.capture(strong_rows, distributed)
    torch.cuda.synchronize()

    clocks = ClockSampler(local_rank)
    ms_per_step, fwd_ms, bwd_ms, own_ms, tail_ms = time_sweep(
        cells, ROWS, args.steps, args.warmup, flat32, flat16, distributed, device, clocks)
    tokens_per_step = world * len(cells) * ROWS
    value = tokens_per_step / (ms_per_step * 1e-3)
    rank_kernel_ms = gather_floats(own_ms, device, world)
    rank_tail_ms = gather_floats(tail_ms, device, world)

    copies = None if distributed else time_same_size_copies(cells, grad_buffer, args.steps, args.warmup)

    strong = None
    if distributed:
        s_ms, s_fwd, s_bwd, s_own, s_tail = time_sweep(
            cells, strong_rows, args.steps, args.warmup, flat32, flat16, distributed, device)
        strong_rank_ms = gather_floats(s_own, device, world)
        # A cell is called launch-bound when its two passes take more than twice what its
        # bytes need at the measured copy bandwidth (fixed launch, ramp-up and tail costs
        # dominate a 1/world share of a small cell).
        peak_now, _ = measured_peak_gbs()
        slow = []
        for cell, f, b in zip(cells, s_fwd, s_bwd):
            ideal_ms = (cell.fwd_bytes + cell.bwd_bytes) / world / (peak_now * 1e9) * 1e3
            if f + b > 2.0 * ideal_ms:
                slow.append({"S": cell.S, "D": cell.D, "ms": round(f + b, 4),
                             "ms_at_peak": round(ideal_ms, 4)})
        strong = {"scaling": "strong", "rows_per_gpu": strong_rows, "ms_per_step": s_ms,
                  "value": len(cells) * ROWS / (s_ms * 1e-3), "unit": "tokens/s",
                  "rank_kernel_ms": {"min": min(strong_rank_ms), "max": max(strong_rank_ms)},
                  "collective_ms": max(gather_floats(s_tail, device, world)),
                  "launch_bound_cells": slow,
                  "note": "the same 18 x 16 384 positions split over the ranks; compare "
                          "ms_per_step with the N = 1 line's"}

    # ---- end to end: pinned host buffers -> public API -> host results
    e2e = (run_e2e(args, cells, device, distributed, world) if not args.skip_e2e
           else {"ms_per_step": float("inf"), "h2d": 0, "d2h": 0, "steps": 0, "pcie": None})
    if distributed:
        import torch.distributed as dist
        worst = torch.tensor([e2e["ms_per_step"]], device=device, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        e2e["ms_per_step"] = float(worst.item())
    e2e_value = tokens_per_step / (e2e["ms_per_step"] * 1e-3)
    torch.cuda.synchronize()
    gave_up = _native.error_flag()   # the sticky "a bounded wait ran out" flag of this device

    if rank != 0:
        return
    peak, peak_kind = measured_peak_gbs()
    bwd_bytes = sum(c.bwd_bytes for c in cells)
    fwd_bytes = sum(c.fwd_bytes for c in cells)
    bwd_gbs = bwd_bytes / (sum(bwd_ms) * 1e-3) / 1e9
    fwd_gbs = fwd_bytes / (sum(fwd_ms) * 1e-3) / 1e9
    both_gbs = (bwd_bytes + fwd_bytes) / ((sum(bwd_ms) + sum(fwd_ms)) * 1e-3) / 1e9
    ratios = traffic_ratios()
    # DRAM traffic of the average backward launch: every cell weighted by the ratio measured
    # for the kernel family that serves it (None when a family has no capture on record).
    traffic = None
    if ratios and all(c.family in ratios for c in cells):
        traffic = sum(ratios[c.family] * c.bwd_bytes for c in cells) / len(cells)
    per_cell = []
    for cell, f, b in zip(cells, fwd_ms, bwd_ms):
        per_cell.append({
            "S": cell.S, "D": cell.D, "fwd_ms": round(f, 4), "bwd_ms": round(b, 4),
            "tokens_per_s": round(ROWS / ((f + b) * 1e-3)),
            "fwd_gbs": round(cell.fwd_bytes / (f * 1e-3) / 1e9, 1),
            "bwd_gbs": round(cell.bwd_bytes / (b * 1e-3) / 1e9, 1),
            "gbs": round((cell.fwd_bytes + cell.bwd_bytes) / ((f + b) * 1e-3) / 1e9, 1),
            "frac_of_peak": round((cell.fwd_bytes + cell.bwd_bytes) / ((f + b) * 1e-3) / 1e9 / peak, 4),
            "backward_kernel": cell.family,
        })
    same_size = None
    if copies is not None:
        copy_ms = 0.0
        for entry, cell, f, b, (copy_f, copy_b) in zip(per_cell, cells, fwd_ms, bwd_ms, copies):
            entry["copy_gbs_fwd_size"], entry["copy_gbs_bwd_size"] = round(copy_f, 1), round(copy_b, 1)
            entry["fwd_vs_copy"] = round(cell.fwd_bytes / (f * 1e-3) / 1e9 / copy_f, 4)
            entry["bwd_vs_copy"] = round(cell.bwd_bytes / (b * 1e-3) / 1e9 / copy_b, 4)
            copy_ms += cell.fwd_bytes / (copy_f * 1e9) * 1e3 + cell.bwd_bytes / (copy_b * 1e9) * 1e3
        same_size = {"ms_per_step_of_copies": copy_ms,
                     "kernels_vs_copies": copy_ms / (sum(fwd_ms) + sum(bwd_ms)),
                     "note": "plain device-to-device copies moving each launch's algorithmic "
                             "bytes, replayed and timed like the sweep; per cell in `cells`"}
    # The CPU oracle is timed at N = 1 only (the reference arm reports it at every N).
    run_cpu = not args.skip_cpu and world == 1
    if run_cpu:
        use_all_host_threads()
    cpu_rate, cpu_seconds, threads = (cpu_oracle_tokens_per_s(CPU_SAMPLE_ROWS) if run_cpu
                                      else (None, 0.0, 0))
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 storage / fp32 arithmetic", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": ROWS, "cells": len(cells),
                   "layout": "packed", "parallelism": f"position-sharded x{world}",
                   "cache": "25 GB of other cells' traffic between a cell's passes (>> 126 MB L2)",
                   "timing": "CUDA events around per-cell CUDA-graph replays"},
        "gbs_fwd_bwd": both_gbs * world, "frac_of_peak_fwd_bwd": both_gbs / peak,
        "frac_of_nominal_8TBs": both_gbs / 8000.0,
        "roofline": {"bound": "hbm", "kernel": "backward (dominant: 2/3 of the bytes)",
                     "achieved": bwd_gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": bwd_gbs / peak,
                     "traffic": traffic,
                     "traffic_over_algorithmic_by_kernel": ratios or None,
                     "algorithmic_bytes_per_launch": bwd_bytes / len(cells),
                     "forward": {"achieved": fwd_gbs, "frac": fwd_gbs / peak}},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": e2e["ms_per_step"],
                "steps": e2e["steps"], "pcie_measured_gbs": e2e["pcie"]},
        "cpu_baseline": ({"value": cpu_rate, "unit": "tokens/s", "cores": threads, "kind": "port",
                          "sample": f"PyTorch oracle port, all 18 cells at {CPU_SAMPLE_ROWS} rows "
                                    f"each ({cpu_seconds:.1f} s of CPU work)"} if run_cpu else None),
        "gpu_launches": args.steps * len(cells) * 3,
        "clocks": clocks.summary(),
        "ranks": {"kernel_ms_per_step": {"min": min(rank_kernel_ms), "max": max(rank_kernel_ms)},
                  "collective_ms_per_step": max(rank_tail_ms) if distributed else 0.0,
                  "note": "kernel_ms: a rank's own forward+backward launches; collective_ms: the "
                          "FP32 all-reduce of the 43 008 query-gradient floats plus the BF16 "
                          "cast, including the wait for the slowest rank"},
        "strong": strong,
        "same_size_copy": same_size,
        "wait_gave_up_flag": gave_up,
        "cells": per_cell,
    }
    print(json.dumps(line), flush=True)


def pinned_copy_probe(device, distributed, world) -> dict:
    """Plain pinned-memory copies, all ranks at once, both directions at once: the ceiling of
    the end-to-end leg on this host.  256 MiB each way per repetition, three repetitions,
    GB/s per direction: this rank's own figure is gathered so the line shows the slowest
    rank, the fastest and the aggregate."""
    import torch.distributed as dist
    size = 256 * 1024 * 1024
    host_in = torch.empty(size, dtype=torch.uint8).pin_memory()
    host_out = torch.empty(size, dtype=torch.uint8).pin_memory()
    dev_in = torch.empty(size, device=device, dtype=torch.uint8)
    dev_out = torch.zeros(size, device=device, dtype=torch.uint8)
    up, down = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def both_ways(repeats):
        events = []
        for stream, dst, src in ((up, dev_in, host_in), (down, host_out, dev_out)):
            with torch.cuda.stream(stream):
                first = stream.record_event(torch.cuda.Event(enable_timing=True))
                for _ in range(repeats):
                    dst.copy_(src, non_blocking=True)
                last = stream.record_event(torch.cuda.Event(enable_timing=True))
            events.append((first, last))
        torch.cuda.synchronize()
        return [repeats * size / (first.elapsed_time(last) * 1e-3) / 1e9 for first, last in events]

    both_ways(1)
    if distributed:
        dist.barrier()
    h2d, d2h = both_ways(3)
    every_h2d = gather_floats(h2d, device, world)
    every_d2h = gather_floats(d2h, device, world)
    return {"ranks_copying_at_once": world, "duplex": True,
            "h2d_per_rank": {"min": min(every_h2d), "max": max(every_h2d)},
            "d2h_per_rank": {"min": min(every_d2h), "max": max(every_d2h)},
            "h2d_aggregate": sum(every_h2d), "d2h_aggregate": sum(every_d2h)}


def run_e2e(args, cells, device, distributed, world=1) -> dict:
    """The same sweep through `attnres()` + autograd with every input starting in pinned
    host memory and every result (out, value gradients, query gradient) copied back.

    Three streams form a pipeline, as a training loop that feeds from host memory would.
    Positions are independent, so every cell is fed in blocks of E2E_BLOCK_ROWS rows: while
    block i runs its forward and backward, the inputs of block i+1 cross PCIe host-to-device
    and the results of block i-1 cross it device-to-host (the link is full duplex).  The
    query gradient of a cell is the FP32 sum of its blocks' BF16 gradients, rounded once (what
    gradient accumulation into an FP32 master gives).  Every byte still moves inside the
    timed region, every step."""
    import torch.distributed as dist
    from attnres import attnres
    steps = max(1, min(args.steps, 3))
    max_elems = max(c.S * ROWS * c.D for c in cells)
    max_row = ROWS * max(WIDTHS)
    block_rows = min(args.e2e_block_rows or E2E_BLOCK_ROWS, ROWS)
    block_elems = max(c.S * block_rows * c.D for c in cells)
    block_row = block_rows * max(WIDTHS)
    host_values = torch.empty(max_elems, dtype=torch.bfloat16).pin_memory()
    host_grads = torch.empty(max_elems, dtype=torch.bfloat16).pin_memory()
    host_up = torch.empty(max_row, dtype=torch.bfloat16).pin_memory()
    host_out = torch.empty(max_row, dtype=torch.bfloat16).pin_memory()
    host_query = torch.empty(max(WIDTHS), dtype=torch.bfloat16).pin_memory()
    host_dq = torch.empty(max(WIDTHS), dtype=torch.bfloat16).pin_memory()
    host_values.normal_()
    host_up.normal_()
    host_query.normal_(std=0.02)
    # Two sets of device input buffers: one being filled while the other is computed on.
    dev_values = [torch.empty(block_elems, device=device, dtype=torch.bfloat16) for _ in range(2)]
    dev_up = [torch.empty(block_row, device=device, dtype=torch.bfloat16) for _ in range(2)]
    dev_query = [torch.empty(max(WIDTHS), device=device, dtype=torch.bfloat16) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    compute = torch.cuda.current_stream(device)
    computed = [None, None]   # event: the cell that last used input set k has finished
    h2d = d2h = 0

    def one_step(count):
        nonlocal h2d, d2h
        turn = 0
        for cell in cells:
            host_v = host_values[:cell.S * ROWS * cell.D].view(cell.S, ROWS, cell.D)
            host_g = host_grads[:cell.S * ROWS * cell.D].view(cell.S, ROWS, cell.D)
            host_u = host_up[:ROWS * cell.D].view(ROWS, cell.D)
            host_o = host_out[:ROWS * cell.D].view(ROWS, cell.D)
            dq32 = torch.zeros(cell.D, device=device, dtype=torch.float32)
            for first in range(0, ROWS, block_rows):
                rows = min(block_rows, ROWS - first)
                k, turn = turn % 2, turn + 1
                values = dev_values[k][:cell.S * rows * cell.D].view(cell.S, rows, cell.D)
                upstream = dev_up[k][:rows * cell.D].view(rows, cell.D)
                query = dev_query[k][:cell.D]
                with torch.cuda.stream(copy_in):
                    if computed[k] is not None:
                        copy_in.wait_event(computed[k])
                    for source in range(cell.S):      # one contiguous copy per source
                        values[source].copy_(host_v[source, first:first + rows], non_blocking=True)
                    upstream.copy_(host_u[first:first + rows], non_blocking=True)
                    query.copy_(host_query[:cell.D], non_blocking=True)
                    arrived = copy_in.record_event()
                compute.wait_event(arrived)
                values.requires_grad_()
                query.requires_grad_()
                out = attnres(values, query)
                dv, dq = torch.autograd.grad(out, (values, query), upstream)
                dq32 += dq.float()
                computed[k] = compute.record_event()
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(computed[k])
                    host_o[first:first + rows].copy_(out, non_blocking=True)
                    for source in range(cell.S):
                        host_g[source, first:first + rows].copy_(dv[source], non_blocking=True)
                for tensor in (out, dv):
                    tensor.record_stream(copy_out)     # keep the blocks until the copy has run
                values.requires_grad_(False)
                query.requires_grad_(False)
                del out, dv, dq
            if distributed:
                dist.all_reduce(dq32)
            dq = dq32.to(torch.bfloat16)
            done = compute.record_event()
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                host_dq[:cell.D].copy_(dq, non_blocking=True)
            dq.record_stream(copy_out)
            if count:
                moved = 2 * (cell.S * ROWS * cell.D + ROWS * cell.D)
                h2d += moved + 2 * cell.D * ((ROWS + block_rows - 1) // block_rows)
                d2h += moved + 2 * cell.D
        compute.wait_stream(copy_out)

    one_step(False)
    if distributed:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for index in range(steps):
        one_step(index == 0)
    stop.record()
    if distributed:
        dist.barrier()
    torch.cuda.synchronize()
    ms_per_step = start.elapsed_time(stop) / steps
    pcie = pinned_copy_probe(device, distributed, world)
    # the leg's own copy rate per direction and rank, next to what plain copies reach here
    pcie["e2e_leg_per_rank_per_direction"] = h2d / (ms_per_step * 1e-3) / 1e9
    return {"ms_per_step": ms_per_step, "h2d": h2d, "d2h": d2h, "steps": steps, "pcie": pcie}


MODEL_WORKLOADS = {
    # the reference's 24-layer Full-schedule training step (its fourth benchmark configuration)
    "config4": dict(layers=24, width=1024, heads=16, ffn=4096, vocab=32000, sequence=2048,
                    rank=None, mode="full", block_layers=1, layout="list", batch_per_gpu=8,
                    global_batch=None, parameters="fp32 + bf16 autocast"),
    # its 8-GPU Block-schedule configuration: D = 4096, blocks of 4 layers (S <= 7), R = 1024
    "config5": dict(layers=24, width=4096, heads=32, ffn=16384, vocab=32000, sequence=4096,
                    rank=1024, mode="block", block_layers=4, layout="list", batch_per_gpu=4,
                    global_batch=32, parameters="bf16"),
}


def run_model_workload(args, rank: int, world: int, local_rank: int) -> None:
    """`--workload config4|config5`: one training step of the benchmark language model
    (baseline/lm.py) with this library's reads, data-parallel over the ranks.

    Every rank holds a replica and its own microbatches (positions are sharded by the batch
    split, so the reads need no communication); DistributedDataParallel all-reduces the weight
    gradients and the [R] query gradients over NCCL in buckets that overlap the backward.
    With a fixed global batch (config5: 32 sequences) a rank runs 32 / (4 world) microbatches
    per step and synchronises on the last one.  Timed: K whole steps (zero_grad, forward,
    cross entropy, backward, all-reduce, fused AdamW) between barriers, CUDA events, max over
    ranks.  The step is also timed with the all-reduce switched off (`no_sync`), which shows
    how much of it the overlap does not hide."""
    import contextlib
    import torch.distributed as dist
    from attnres import _native, attnres
    from baseline import lm
    spec = dict(MODEL_WORKLOADS[args.workload])
    if args.layers:
        spec["layers"] = args.layers
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    distributed = world > 1
    batch_per_gpu = spec.pop("batch_per_gpu")
    global_batch = spec.pop("global_batch")
    parameters = spec.pop("parameters")
    accumulation = 1
    if global_batch and not args.weak:
        accumulation = max(1, global_batch // (batch_per_gpu * world))
    config = lm.LMConfig(**spec)
    torch.manual_seed(SEED)            # the same initial weights on every rank
    with torch.device(device):
        model = lm.CausalLM(config, attnres)
    if parameters == "bf16":
        model = model.to(torch.bfloat16)
    wrapped = model
    if distributed:
        wrapped = torch.nn.parallel.DistributedDataParallel(
            model, device_ids=[local_rank], gradient_as_bucket_view=True, bucket_cap_mb=256)
    runner = torch.compile(wrapped, fullgraph=False) if args.compile else wrapped
    # The reference's learning rate (3e-4) is set for its 1024-wide models; Adam's first steps
    # move every weight by the learning rate, which at 4096 features per row sends the loss up,
    # so wider models take it scaled by 1024 / width.
    learning_rate = 3e-4 * min(1.0, 1024 / config.width)
    optimizer = lm.make_optimizer(model, capturable=False, lr=learning_rate)
    generator = torch.Generator(device=device).manual_seed(SEED + 1 + rank)
    shape = (batch_per_gpu * accumulation, config.sequence)
    tokens = torch.randint(config.vocab, shape, device=device, generator=generator)
    targets = torch.randint(config.vocab, shape, device=device, generator=generator)

    def sync_context(last):
        if distributed and not last:
            return wrapped.no_sync()
        return contextlib.nullcontext()

    def never_sync(last):
        return wrapped.no_sync() if distributed else contextlib.nullcontext()

    def timed(steps, context):
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        loss = None
        for _ in range(steps):
            loss = lm.training_step(runner, optimizer, tokens, targets, accumulation=accumulation,
                                    sync_context=context)
        stop.record()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        if distributed:
            worst = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            ms = float(worst.item())
        return ms, float(loss)

    warmup = max(args.warmup, 1)
    timed(warmup, sync_context)
    with ClockSampler(local_rank) as clocks:
        ms_per_step, loss = timed(args.steps, sync_context)
    quiet_ms = None
    if distributed:
        quiet_ms, _ = timed(max(1, min(args.steps, 2)), never_sync)
    torch.cuda.synchronize()
    gave_up = _native.error_flag()
    if rank != 0:
        return
    rows = batch_per_gpu * config.sequence            # positions per microbatch and rank
    tokens_per_step = rows * accumulation * world
    parameters_count = sum(p.numel() for p in model.parameters())
    grad_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    query_grad_bytes = sum(q.numel() * q.element_size() for q in model.queries)
    counts = lm.read_source_counts(config)
    line = {
        "metric": "train_step_tokens_per_s", "value": tokens_per_step / (ms_per_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak" if (args.weak or not global_batch) else "strong (fixed global batch)",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}_{config.mode}_schedule_L{config.layers}_D{config.width}"
                               f"_R{config.rank}_seq{config.sequence}",
                   "layers": config.layers, "full_layers": MODEL_WORKLOADS[args.workload]["layers"],
                   "sequences_per_gpu_microbatch": batch_per_gpu,
                   "microbatches_per_gpu_step": accumulation,
                   "global_batch_sequences": batch_per_gpu * accumulation * world,
                   "parameters": parameters, "parameter_count": parameters_count,
                   "optimizer": f"AdamW fused lr {learning_rate:g} betas 0.9/0.95 wd 0.1",
                   "compiled": bool(args.compile),
                   "parallelism": f"data parallel x{world} (DistributedDataParallel, NCCL, "
                                  "256 MB buckets overlapping the backward)",
                   "reads_per_microbatch": len(counts), "sources_per_read": sorted(set(counts)),
                   "attnres_algorithmic_gb_per_gpu_step":
                       lm.attnres_algorithmic_bytes(config, rows) * accumulation / 1e9},
        "collective": {"gradient_bytes_all_reduced_per_step": grad_bytes if distributed else 0,
                       "of_which_query_gradients": query_grad_bytes if distributed else 0,
                       "ms_per_step_without_all_reduce": quiet_ms,
                       "exposed_ms_per_step": None if quiet_ms is None else ms_per_step - quiet_ms},
        "loss": loss, "peak_memory_gb": torch.cuda.max_memory_allocated() / 1e9,
        "clocks": clocks.summary(), "wait_gave_up_flag": gave_up,
    }
    print(json.dumps(line), flush=True)


def run_single_cell(args) -> None:
    """`--cell S,D[,R]`: one shape, eager launches through the C ABI, per-call CUDA-event
    times.  This is the small case the ncu captures under profiles/ were taken on."""
    from attnres import _native
    parts = [int(x) for x in args.cell.split(",")]
    sources, width = parts[0], parts[1]
    rank = parts[2] if len(parts) > 2 else width
    rows = args.rows
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    generator = torch.Generator(device=device).manual_seed(SEED)
    values = torch.randn(sources, rows, width, device=device, dtype=torch.bfloat16, generator=generator)
    query = (torch.randn(rank, device=device, generator=generator) * 0.02).to(torch.bfloat16)
    upstream = torch.randn(rows, width, device=device, dtype=torch.bfloat16, generator=generator)
    out = torch.empty(rows, width, device=device, dtype=torch.bfloat16)
    grad = torch.empty_like(values)
    logits = torch.empty(sources, rows, device=device, dtype=torch.float32)
    stats = torch.empty(2, rows, device=device, dtype=torch.float32)
    partial_rows = _native.dq_workspace_rows(rows, sources, width, rank, 0)
    partials = torch.empty(partial_rows, rank, device=device, dtype=torch.float32)
    dq = torch.empty(rank, device=device, dtype=torch.bfloat16)
    flush = torch.empty(256 * 1024 * 1024, device=device, dtype=torch.uint8)
    step = rows * width * 2
    src = [values.data_ptr() + s * step for s in range(sources)]
    dst = [grad.data_ptr() + s * step for s in range(sources)]
    stream = torch.cuda.current_stream().cuda_stream
    scale = rank ** -0.5 if rank != width else 1.0
    flags = _native.FLAG_FORCE_GENERIC if args.generic else 0
    if args.one_pass:
        flags |= _native.FLAG_PREFER_STREAM
    saves = args.one_pass or (not args.two_pass and
                              _native.wants_output_residual(sources, width, rank))
    residual = torch.empty_like(out) if saves else None
    saved = dict(out_ptr=out.data_ptr(), residual_ptr=residual.data_ptr()) if saves else {}
    fwd_ms, bwd_ms = [], []
    for index in range(args.warmup + args.steps):
        flush.zero_()  # 256 MB write: evicts the 126 MB L2 between timed launches
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        _native.forward(src, [width] * sources, [1] * sources, sources, rows, width, rank,
                        query.data_ptr(), 1, 2**-23, scale, out.data_ptr(), width,
                        logits.data_ptr(), stats.data_ptr(), flags, stream,
                        residual_ptr=saved.get("residual_ptr"))
        e1.record()
        flush.zero_()
        e1b = torch.cuda.Event(enable_timing=True)
        e1b.record()
        _native.backward(src, [width] * sources, [1] * sources, sources, rows, width, rank,
                         query.data_ptr(), 1, 2**-23, scale, upstream.data_ptr(), width, 1,
                         logits.data_ptr(), stats.data_ptr(), dst, [width] * sources,
                         partials.data_ptr(), partial_rows, dq.data_ptr(), None, flags, stream,
                         **saved)
        e2.record()
        torch.cuda.synchronize()
        if index >= args.warmup:
            fwd_ms.append(e0.elapsed_time(e1))
            bwd_ms.append(e1b.elapsed_time(e2))
    fwd_bytes = rows * (2 * sources * width + 2 * width)
    bwd_bytes = rows * (4 * sources * width + 2 * width)
    peak, _ = measured_peak_gbs()
    f, b = sorted(fwd_ms)[len(fwd_ms) // 2], sorted(bwd_ms)[len(bwd_ms) // 2]
    extra = {}
    if args.accumulate:
        # Running gradient buffers: (a) this backward followed by the elementwise add autograd
        # would run, (b) the backward that adds in the kernel (needs the saved output).
        buffer = torch.zeros_like(values)
        if residual is None:
            residual = torch.empty_like(out)
            _native.forward(src, [width] * sources, [1] * sources, sources, rows, width, rank,
                            query.data_ptr(), 1, 2**-23, scale, out.data_ptr(), width,
                            logits.data_ptr(), stats.data_ptr(), flags, stream,
                            residual_ptr=residual.data_ptr())
        acc = [buffer.data_ptr() + s * step for s in range(sources)]
        add_ms, fused_ms = [], []
        for index in range(args.warmup + args.steps):
            flush.zero_()
            a0, a1 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            a0.record()
            _native.backward(src, [width] * sources, [1] * sources, sources, rows, width, rank,
                             query.data_ptr(), 1, 2**-23, scale, upstream.data_ptr(), width, 1,
                             logits.data_ptr(), stats.data_ptr(), dst, [width] * sources,
                             partials.data_ptr(), partial_rows, dq.data_ptr(), None, flags, stream,
                             **saved)
            buffer.add_(grad)
            a1.record()
            flush.zero_()
            b0, b1 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            b0.record()
            _native.backward(src, [width] * sources, [1] * sources, sources, rows, width, rank,
                             query.data_ptr(), 1, 2**-23, scale, upstream.data_ptr(), width, 1,
                             logits.data_ptr(), stats.data_ptr(), acc, [width] * sources,
                             partials.data_ptr(), partial_rows, dq.data_ptr(), None,
                             flags | _native.FLAG_ACCUMULATE_DV, stream,
                             out_ptr=out.data_ptr(), residual_ptr=residual.data_ptr())
            b1.record()
            torch.cuda.synchronize()
            if index >= args.warmup:
                add_ms.append(a0.elapsed_time(a1))
                fused_ms.append(b0.elapsed_time(b1))
        a, fu = sorted(add_ms)[len(add_ms) // 2], sorted(fused_ms)[len(fused_ms) // 2]
        acc_bytes = rows * (6 * sources * width + 2 * width)   # values, old sums, new sums, dO
        extra = {"bwd_then_add_ms": a, "bwd_accumulate_ms": fu, "accumulate_speedup": a / fu,
                 "bwd_accumulate_gbs": acc_bytes / fu / 1e6,
                 "bwd_accumulate_frac": acc_bytes / fu / 1e6 / peak}
    if args.fused_norm:
        # The read with the LayerNorm of the next sublayer in its epilogue (one more [N,D] BF16
        # row written), and the LayerNorm backward kernel that precedes the read's backward.
        weight = torch.ones(width, device=device, dtype=torch.float32)
        bias = torch.zeros(width, device=device, dtype=torch.float32)
        normed = torch.empty_like(out)
        norm_stats = torch.empty(2, rows, device=device, dtype=torch.float32)
        through = torch.empty_like(out)
        ln_rows = _native.layer_norm_workspace_rows(rows, width, 0)
        ln_partials = torch.empty(ln_rows, 2 * width, device=device, dtype=torch.float32)
        both = torch.empty(2 * width, device=device, dtype=torch.float32)
        norm_fwd_ms, norm_bwd_ms = [], []
        for index in range(args.warmup + args.steps):
            flush.zero_()
            n0, n1, n2, n3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
            n0.record()
            _native.forward_layer_norm(src, [width] * sources, [1] * sources, sources, rows, width,
                                       rank, query.data_ptr(), 1, 2**-23, scale, out.data_ptr(),
                                       width, logits.data_ptr(), stats.data_ptr(),
                                       weight.data_ptr(), bias.data_ptr(), 1e-5,
                                       normed.data_ptr(), norm_stats.data_ptr(), flags, stream,
                                       residual_ptr=saved.get("residual_ptr"))
            n1.record()
            flush.zero_()
            n2.record()
            _native.check(_native.layer_norm_backward(
                upstream.data_ptr(), width, out.data_ptr(), norm_stats.data_ptr(),
                weight.data_ptr(), rows, width, through.data_ptr(), ln_partials.data_ptr(),
                ln_rows, both.data_ptr(), stream), "attnres_b200_layer_norm_backward")
            n3.record()
            torch.cuda.synchronize()
            if index >= args.warmup:
                norm_fwd_ms.append(n0.elapsed_time(n1))
                norm_bwd_ms.append(n2.elapsed_time(n3))
        nf = sorted(norm_fwd_ms)[len(norm_fwd_ms) // 2]
        nb = sorted(norm_bwd_ms)[len(norm_bwd_ms) // 2]
        norm_fwd_bytes = fwd_bytes + rows * 2 * width        # + the normalised row
        norm_bwd_bytes = rows * 6 * width                    # gradient and read in, gradient out
        extra.update({"fwd_layer_norm_ms": nf, "fwd_layer_norm_gbs": norm_fwd_bytes / nf / 1e6,
                      "fwd_layer_norm_frac": norm_fwd_bytes / nf / 1e6 / peak,
                      "layer_norm_bwd_ms": nb, "layer_norm_bwd_gbs": norm_bwd_bytes / nb / 1e6,
                      "layer_norm_bwd_frac": norm_bwd_bytes / nb / 1e6 / peak})
    print(json.dumps({"cell": [sources, rows, width, rank], "fwd_ms": f, "bwd_ms": b, **extra,
                      "fwd_gbs": fwd_bytes / f / 1e6, "bwd_gbs": bwd_bytes / b / 1e6,
                      "fwd_frac": fwd_bytes / f / 1e6 / peak, "bwd_frac": bwd_bytes / b / 1e6 / peak,
                      "family_fwd": _native.kernel_family(sources, width, rank, True, False)
                      if not args.generic else "generic",
                      "family_bwd": _native.kernel_family(sources, width, rank, True, True)
                      if not args.generic else "generic",
                      "one_pass_backward": bool(saves)}), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--skip-e2e", action="store_true",
                        help="profiling runs: leave out the host-buffer end-to-end leg")
    parser.add_argument("--e2e-block-rows", type=int, default=0,
                        help="rows per host-to-device block of the end-to-end leg (default 4096)")
    parser.add_argument("--skip-cpu", action="store_true",
                        help="profiling runs: leave out the CPU-oracle leg")
    parser.add_argument("--workload", choices=("sweep", *MODEL_WORKLOADS), default="sweep",
                        help="sweep (default): the operator sweep; config4 / config5: a training "
                             "step of the benchmark language model, data-parallel over the ranks")
    parser.add_argument("--layers", type=int, default=0,
                        help="model workloads: fewer layers than the configuration names")
    parser.add_argument("--weak", action="store_true",
                        help="config5: one microbatch per GPU and step instead of the fixed "
                             "global batch of 32 sequences")
    parser.add_argument("--compile", action="store_true",
                        help="model workloads: run the model under torch.compile")
    parser.add_argument("--cell", default=None, help="S,D[,R]: time one shape instead of the sweep")
    parser.add_argument("--rows", type=int, default=ROWS, help="rows of the --cell run")
    parser.add_argument("--generic", action="store_true", help="--cell: force the generic kernels")
    parser.add_argument("--one-pass", action="store_true",
                        help="--cell: save the output residual and prefer the one-pass backward")
    parser.add_argument("--accumulate", action="store_true",
                        help="--cell: also time the backward that adds into running gradient buffers")
    parser.add_argument("--fused-norm", action="store_true",
                        help="--cell: also time the read with the LayerNorm epilogue and the "
                             "LayerNorm backward kernel")
    parser.add_argument("--two-pass", action="store_true",
                        help="--cell: never save the output residual (staged backward)")
    parser.add_argument("--strong", action="store_true",
                        help="kept for old command lines: the strong-scaling record (the 16 384 "
                             "rows of every cell split over the ranks) is part of every N > 1 line")
    args = parser.parse_args()
    if args.cell is not None:
        run_single_cell(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU fallback")
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload != "sweep":
            run_model_workload(args, rank, world, local_rank)
        else:
            run_gpu_arm(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
