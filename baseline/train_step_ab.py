"""24-layer Full-schedule training step (the reference's 24-layer model benchmark): this library vs the reference's
Triton kernels on the same GPU.

    python baseline/train_step_ab.py                       # every arm, one after the other
    python baseline/train_step_ab.py --arm ours-list       # one arm: one JSON line

Model (the shape of the reference's benchmark LM, benchmarks/model.py:137-311, re-implemented
here): pre-norm decoder, D=1024, 16 heads, SwiGLU MLP 4x, vocab 32000, sequence 2048, batch 8,
random-init weights N(0, 0.02), uniform random tokens.  Full schedule: the first attention
reads the embedding; every later sublayer and the LM head read ALL earlier sublayer outputs
plus the embedding through ``attnres`` with their own learned [D] query (48 reads, S = 2..49).
One step = zero_grad + BF16-autocast forward + cross-entropy + backward + fused capturable
AdamW (lr 3e-4, betas 0.9/0.95, wd 0.1), captured in ONE CUDA graph after eager warm-up and
replayed; CUDA events around each replay, median reported.  The model itself runs eagerly
(no torch.compile) in every arm, so the arms differ only in the AttnRes operator and layout.

Arms: ``ours-list`` (sources passed as a tuple, no packing copy), ``ours-packed``
(``torch.stack`` then the packed operator, the reference model's default layout),
``triton-packed`` (reference package from ``baseline/_ref``), and ``ours-accumulate``: the list
layout with a staged backward that owns one running gradient buffer per sublayer output.  Every
read takes DETACHED sources and adds its value gradients to those buffers inside the backward
kernel (``attnres.accumulate.attnres_accumulate``); after the loss's backward has run the last
read, the sublayer outputs are back-propagated one by one, newest first, each with its finished
buffer as the incoming gradient.  Autograd then never materialises or sums the 1 224 per-read
source gradients.  The reference's list-layout
Triton path autotunes 48 configurations for each of 96 kernel specialisations of this model
and is not run here for GPU-time reasons.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
ARMS = ("triton-packed", "ours-packed", "ours-list", "ours-accumulate")


def build_model(torch, operator, layout, layers, width, heads, ffn, vocab, sequence):
    from torch import nn
    import torch.nn.functional as F

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm_attention = nn.LayerNorm(width)
            self.q_proj = nn.Linear(width, width, bias=False)
            self.k_proj = nn.Linear(width, width, bias=False)
            self.v_proj = nn.Linear(width, width, bias=False)
            self.attention_output = nn.Linear(width, width, bias=False)
            self.norm_mlp = nn.LayerNorm(width)
            self.gate_proj = nn.Linear(width, ffn, bias=False)
            self.up_proj = nn.Linear(width, ffn, bias=False)
            self.down_proj = nn.Linear(ffn, width, bias=False)

        def attention(self, x):
            h = self.norm_attention(x)
            b, t, _ = h.shape
            split = lambda y: y.view(b, t, heads, width // heads).transpose(1, 2)
            a = F.scaled_dot_product_attention(split(self.q_proj(h)), split(self.k_proj(h)),
                                               split(self.v_proj(h)), is_causal=True)
            return self.attention_output(a.transpose(1, 2).reshape(b, t, width))

        def mlp(self, x):
            h = self.norm_mlp(x)
            return self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.token_embedding = nn.Embedding(vocab, width)
            self.position_embedding = nn.Parameter(torch.empty(sequence, width))
            self.layers = nn.ModuleList([Layer() for _ in range(layers)])
            self.lm_head = nn.Linear(width, vocab, bias=False)
            self.queries = nn.ParameterList([nn.Parameter(torch.empty(width))
                                             for _ in range(2 * layers)])
            for module in self.modules():
                if isinstance(module, (nn.Linear, nn.Embedding)):
                    nn.init.normal_(module.weight, mean=0.0, std=0.02)
            nn.init.normal_(self.position_embedding, mean=0.0, std=0.02)
            for query in self.queries:
                nn.init.normal_(query, mean=0.0, std=0.02)

        def read(self, sources, index):
            query = self.queries[index].to(torch.bfloat16)
            if layout == "packed":
                return operator(torch.stack(sources), query)
            return operator(tuple(sources), query)

        def forward_staged(self, tokens, accumulate, buffers):
            """Forward for the staged backward: returns (logits, sublayer outputs still attached
            to their own graph segment, the detached embedding the first attention consumed)."""
            bf16 = lambda t: t.to(torch.bfloat16)
            embedded = bf16(self.token_embedding(tokens) + self.position_embedding[: tokens.shape[-1]])
            attached, sources = [embedded], [embedded.detach()]
            first_input = embedded.detach().requires_grad_()
            last = 2 * len(self.layers)

            def read(index):
                query = self.queries[index].to(torch.bfloat16)
                # the LAST read runs its backward first and touches every buffer: it overwrites
                return accumulate(tuple(sources), query, buffers[: len(sources)],
                                  overwrite=index == last)

            x, reads = first_input, 0
            for index, layer in enumerate(self.layers):
                if index > 0:
                    x = read(reads)
                    reads += 1
                attached.append(bf16(layer.attention(x)))
                sources.append(attached[-1].detach())
                x = read(reads)
                reads += 1
                attached.append(bf16(layer.mlp(x)))
                sources.append(attached[-1].detach())
            return self.lm_head(read(reads)), attached, first_input

        def forward(self, tokens):
            bf16 = lambda t: t.to(torch.bfloat16)
            x = bf16(self.token_embedding(tokens) + self.position_embedding[: tokens.shape[-1]])
            sources = [x]
            reads = 0
            for index, layer in enumerate(self.layers):
                if index > 0:
                    x = self.read(sources, reads)
                    reads += 1
                sources.append(bf16(layer.attention(x)))
                x = self.read(sources, reads)
                reads += 1
                sources.append(bf16(layer.mlp(x)))
            x = self.read(sources, reads)
            return self.lm_head(x)

    return Model()


def run_arm(arm: str, steps: int, layers: int, batch: int, sequence: int) -> dict:
    backend, layout = arm.split("-")
    package_dir = ROOT / "baseline" / "_ref" if backend == "triton" else ROOT / "fast-attnres_b200"
    sys.path[:] = [e for e in sys.path if "fast-attnres_b200" not in e and "baseline/_ref" not in e]
    sys.path.insert(0, str(package_dir))
    import torch
    import torch.nn.functional as F
    import attnres as package
    assert str(package_dir) in str(Path(package.__file__).resolve()), package.__file__
    width, heads, ffn, vocab = 1024, 16, 4096, 32000
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(20260827)
    model = build_model(torch, package.attnres, layout, layers, width, heads, ffn, vocab,
                        sequence).to(device)
    staged = layout == "accumulate"
    if staged:
        from attnres.accumulate import attnres_accumulate
        buffers = [torch.zeros(batch, sequence, width, device=device, dtype=torch.bfloat16)
                   for _ in range(2 * layers + 1)]
    optimizer = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95),
                                  weight_decay=0.1, fused=True, capturable=True)
    tokens = torch.randint(vocab, (batch, sequence), device=device)
    targets = torch.randint(vocab, (batch, sequence), device=device)
    loss_buffer = torch.zeros((), device=device)

    def step():
        optimizer.zero_grad(set_to_none=False)
        if not staged:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits = model(tokens)
            loss = F.cross_entropy(logits.float().view(-1, vocab), targets.view(-1))
            loss.backward()
        else:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits, attached, first_input = model.forward_staged(tokens, attnres_accumulate, buffers)
            loss = F.cross_entropy(logits.float().view(-1, vocab), targets.view(-1))
            loss.backward()                       # LM head and the last read: fills every buffer
            for index in range(len(attached) - 1, 0, -1):
                attached[index].backward(buffers[index])   # its reads have all run by now
            buffers[0] += first_input.grad        # the first attention consumed the embedding directly
            attached[0].backward(buffers[0])
        optimizer.step()
        loss_buffer.copy_(loss.detach())

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    first_loss = float(loss_buffer)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    times = []
    for _ in range(steps + 2):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    times = sorted(times[2:])
    rows = batch * sequence
    read_bytes = rows * sum(6 * s * width + 4 * width for s in range(2, 2 * layers + 2))
    return {"arm": arm, "step_ms": times[len(times) // 2], "step_ms_min": times[0],
            "tokens_per_s": rows / (times[len(times) // 2] * 1e-3), "loss_after_warmup": first_loss,
            "loss_last": float(loss_buffer), "layers": layers, "rows": rows,
            "attnres_algorithmic_gb_per_step": read_bytes / 1e9,
            "peak_memory_gb": torch.cuda.max_memory_allocated() / 1e9,
            "package": str(Path(package.__file__).resolve().parent)}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--arm", choices=(*ARMS, "all"), default="all")
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--layers", type=int, default=24)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--sequence", type=int, default=2048)
    args = parser.parse_args()
    if args.arm != "all":
        print(json.dumps(run_arm(args.arm, args.steps, args.layers, args.batch, args.sequence)),
              flush=True)
        return
    for arm in ARMS:
        if arm.startswith("triton") and not (ROOT / "baseline" / "_ref" / "attnres").exists():
            print(json.dumps({"arm": arm, "unavailable": "baseline/_ref holds no reference install"}))
            continue
        command = [sys.executable, str(Path(__file__).resolve()), "--arm", arm,
                   "--steps", str(args.steps), "--layers", str(args.layers),
                   "--batch", str(args.batch), "--sequence", str(args.sequence)]
        done = subprocess.run(command, capture_output=True, text=True)
        if done.returncode != 0:
            print(json.dumps({"arm": arm, "failed": done.stderr[-1500:]}), flush=True)
        else:
            print(done.stdout.strip().splitlines()[-1], flush=True)


if __name__ == "__main__":
    main()
