"""24-layer Full-schedule training step (the reference's 24-layer model benchmark): this
library against the reference's Triton kernels on the same GPU.

    python baseline/train_step_ab.py --compile                 # every arm, ABBA order, table
    python baseline/train_step_ab.py --arm ours-list --compile # one arm: one JSON line

Model: baseline/lm.py (the shape of the reference's benchmark LM, benchmarks/model.py:137-311
of the reference): pre-norm decoder, D=1024, 16 heads, SwiGLU MLP 4x, vocab 32000, sequence
2048, batch 8, random-init weights N(0, 0.02), uniform random tokens.  Full schedule: 48 reads
per step with S = 2..49, one learned [D] query each.

Step (benchmarks/training_graph.py:24-58, 126-255 of the reference): zero_grad + BF16-autocast
forward + cross entropy + backward + fused capturable AdamW (lr 3e-4, betas 0.9/0.95, wd 0.1).
With ``--compile`` the model runs under ``torch.compile(fullgraph=True)``; either way the whole
step is captured in ONE CUDA graph after eager warm-up on a side stream, model and optimiser
state are put back to their pre-warm-up values, and the replays are timed with CUDA events.

Arms (every arm is its own process, because both packages are called ``attnres``):

* ``triton-list``    reference package, sources passed as a tuple: the layout the reference
                     headlines (its kernels specialise and autotune per source count);
* ``triton-packed``  reference package, ``torch.stack`` then the packed operator;
* ``ours-list``      this library, tuple of sources (pointer table, no packing copy);
* ``ours-packed``    this library, ``torch.stack`` then the packed operator;
* ``ours-fused``     this library, list layout, the LayerNorm in front of every sublayer
                     computed in the read's epilogue (``attnres.fused.attnres_layer_norm``);
* ``ours-accumulate`` this library, list layout, staged backward: every read takes detached
                     sources and its backward kernel adds the value gradients into one running
                     buffer per sublayer output (``attnres.accumulate.attnres_accumulate``);
                     the sublayer outputs are then back-propagated newest first.  Here
                     ``--compile`` compiles the sublayers one by one (the staging is Python).

With ``--arm all`` the arms run in the order A B .. B A (every arm twice, mirrored), the replay
times of an arm's two runs are pooled, and every arm is reported against ``triton-list`` as
the ratio of the medians with a 95 % bootstrap interval (2 000 resamples, fixed seed; the
protocol of benchmarks/statistics.py:87-211 of the reference, across processes here).
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
ARMS = ("triton-list", "triton-packed", "ours-list", "ours-packed", "ours-fused", "ours-accumulate")
# `--arm all` without `--arms` runs these; `ours-fused` is selectable by name (its set-up under
# torch.compile has taken minutes in this harness for a reason not found, while a stand-alone
# compile of the same model takes seconds).
DEFAULT_ARMS = ("triton-list", "triton-packed", "ours-list", "ours-packed", "ours-accumulate")


def staged_step_factory(torch, model, lm, accumulate, buffers, optimizer, tokens, targets,
                        compile_sublayers):
    """The step of the ``ours-accumulate`` arm.  The forward detaches every sublayer output
    before it becomes a source; the backward of every read adds into ``buffers``; afterwards
    the sublayer outputs are back-propagated newest first with their finished buffer."""
    import torch.nn.functional as F
    config = model.config
    bodies = []
    for event in range(config.events):
        layer = model.layers[event // 2]
        body = layer.attention if event % 2 == 0 else layer.mlp
        bodies.append(torch.compile(body, fullgraph=True) if compile_sublayers else body)
    last = config.events

    def step():
        optimizer.zero_grad(set_to_none=False)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            embedded = model.embed(tokens)
            attached, sources = [embedded], [embedded.detach()]
            first_input = embedded.detach().requires_grad_()

            def read(index):
                query = model.queries[index].to(torch.bfloat16)
                # the LAST read runs its backward first and touches every buffer: it overwrites
                return accumulate(tuple(sources), query, buffers[: len(sources)],
                                  overwrite=index == last - 1)

            for event in range(config.events):
                x = first_input if event == 0 else read(event - 1)
                attached.append(bodies[event](x).to(torch.bfloat16))
                sources.append(attached[-1].detach())
            logits = model.lm_head(read(last - 1))
            loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1))
        loss.backward()                       # LM head and the last read: fills every buffer
        for index in range(len(attached) - 1, 0, -1):
            attached[index].backward(buffers[index])   # its reads have all run by now
        buffers[0] += first_input.grad        # the first attention consumed the embedding directly
        attached[0].backward(buffers[0])
        optimizer.step()
        return loss.detach()

    return step


def run_arm(arm: str, steps: int, layers: int, batch: int, sequence: int, compiled: bool) -> dict:
    backend, layout = arm.split("-")
    package_dir = ROOT / "baseline" / "_ref" if backend == "triton" else ROOT / "fast-attnres_b200"
    sys.path[:] = [e for e in sys.path if "fast-attnres_b200" not in e and "baseline/_ref" not in e]
    sys.path.insert(0, str(package_dir))
    sys.path.insert(1, str(ROOT))
    began = time.perf_counter()
    import torch
    import attnres as package
    from baseline import lm
    assert str(package_dir) in str(Path(package.__file__).resolve()), package.__file__
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(20260827)
    config = lm.LMConfig(layers=layers, width=1024, heads=16, ffn=4096, vocab=32000,
                         sequence=sequence, mode="full",
                         layout="packed" if layout == "packed" else "list")
    normed = None
    if layout == "fused":
        from attnres.fused import attnres_layer_norm
        normed = attnres_layer_norm
    with torch.device(device):
        model = lm.CausalLM(config, package.attnres, normed_operator=normed)
    optimizer = lm.make_optimizer(model, capturable=True)
    tokens = torch.randint(config.vocab, (batch, sequence), device=device)
    targets = torch.randint(config.vocab, (batch, sequence), device=device)
    if layout == "accumulate":
        from attnres.accumulate import attnres_accumulate
        buffers = [torch.zeros(batch, sequence, config.width, device=device, dtype=torch.bfloat16)
                   for _ in range(config.events + 1)]
        step = staged_step_factory(torch, model, lm, attnres_accumulate, buffers, optimizer,
                                   tokens, targets, compiled)
    else:
        runner = torch.compile(model, fullgraph=True, dynamic=False) if compiled else model

        def step():
            return lm.training_step(runner, optimizer, tokens, targets)

    captured = lm.CapturedStep(step, model, optimizer, warmup=3)
    ready = time.perf_counter()
    times = captured.time_replays(steps)
    ordered = sorted(times)
    rows = batch * sequence
    return {"arm": arm, "compiled": compiled, "step_ms": ordered[len(ordered) // 2],
            "step_ms_min": ordered[0], "samples_ms": times,
            "tokens_per_s": rows / (ordered[len(ordered) // 2] * 1e-3),
            "loss_after_warmup": captured.loss_after_warmup, "loss_last": float(captured.loss),
            "layers": layers, "rows": rows, "reads": len(lm.read_source_counts(config)),
            "attnres_algorithmic_gb_per_step": lm.attnres_algorithmic_bytes(config, rows) / 1e9,
            "peak_memory_gb": torch.cuda.max_memory_allocated() / 1e9,
            "setup_seconds": round(ready - began, 1),
            "package": str(Path(package.__file__).resolve().parent)}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--arm", choices=(*ARMS, "all"), default="all")
    parser.add_argument("--arms", default=None,
                        help="comma-separated subset for --arm all (default: every arm)")
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--layers", type=int, default=24)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--sequence", type=int, default=2048)
    parser.add_argument("--compile", action="store_true",
                        help="run the model under torch.compile(fullgraph=True) before capture")
    parser.add_argument("--once", action="store_true",
                        help="--arm all: run every arm once instead of twice in mirrored order")
    parser.add_argument("--arm-timeout", type=int, default=1500, help="seconds per arm process")
    args = parser.parse_args()
    if args.arm != "all":
        print(json.dumps(run_arm(args.arm, args.steps, args.layers, args.batch, args.sequence,
                                 args.compile)), flush=True)
        return
    arms = [a for a in (args.arms.split(",") if args.arms else DEFAULT_ARMS)]
    order = arms if args.once else arms + arms[::-1]
    runs = []
    for arm in order:
        if arm.startswith("triton") and not (ROOT / "baseline" / "_ref" / "attnres").exists():
            print(json.dumps({"arm": arm, "unavailable": "baseline/_ref holds no reference install"}))
            continue
        command = [sys.executable, str(Path(__file__).resolve()), "--arm", arm,
                   "--steps", str(args.steps), "--layers", str(args.layers),
                   "--batch", str(args.batch), "--sequence", str(args.sequence)]
        if args.compile:
            command.append("--compile")
        try:
            done = subprocess.run(command, capture_output=True, text=True, timeout=args.arm_timeout)
        except subprocess.TimeoutExpired:
            print(json.dumps({"arm": arm, "failed": f"no result within {args.arm_timeout} s"}),
                  flush=True)
            continue
        if done.returncode != 0:
            print(json.dumps({"arm": arm, "failed": done.stderr[-1500:]}), flush=True)
            continue
        runs.append(json.loads(done.stdout.strip().splitlines()[-1]))
        print(json.dumps({k: v for k, v in runs[-1].items() if k != "samples_ms"}), flush=True)
    # pooled medians and ratios against the reference's headline arm
    import numpy as np
    pooled = {}
    for run in runs:
        pooled.setdefault(run["arm"], []).extend(run["samples_ms"])
    base = "triton-list" if "triton-list" in pooled else ("triton-packed" if "triton-packed" in pooled
                                                           else None)
    generator = np.random.default_rng(20260827)
    print("| arm | step ms (median of pooled replays) | tokens/s | vs " + str(base) + " | 95 % interval |")
    print("|---|---|---|---|---|")
    rows = args.batch * args.sequence
    for arm, samples in pooled.items():
        samples = np.array(samples)
        median = float(np.median(samples))
        ratio = interval = ""
        if base is not None and arm != base:
            reference = np.array(pooled[base])
            ratio = f"{np.median(reference) / median:.3f}x"
            draws = [np.median(generator.choice(reference, reference.size)) /
                     np.median(generator.choice(samples, samples.size)) for _ in range(2000)]
            low, high = np.percentile(draws, [2.5, 97.5])
            interval = f"{low:.3f}x – {high:.3f}x"
        print(f"| {arm} | {median:.2f} | {rows / (median * 1e-3):,.0f} | {ratio} | {interval} |")


if __name__ == "__main__":
    main()
