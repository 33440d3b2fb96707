"""Full and Block source schedules through the one operator, under torch.compile and replayed
from a CUDA graph.  Needs a CUDA device.

    python fast-attnres_b200/examples/schedules_compile_graph.py

(The scenarios of the reference's examples block_schedules.py and torch_compile.py.)
"""
from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

from attnres import attnres  # noqa: E402


def run(device: str = "cuda") -> dict:
    torch.manual_seed(2)
    writers, rows, width, block = 6, 64, 512, 2
    embedding = torch.randn(rows, width, device=device, dtype=torch.bfloat16)
    outputs = [torch.randn(rows, width, device=device, dtype=torch.bfloat16) for _ in range(writers)]
    query = torch.randn(width, device=device, dtype=torch.bfloat16) * 0.1

    # Full: the embedding and every earlier output are sources of their own
    full = attnres((embedding, *outputs), query)

    # Block: completed block sums plus the running partial sum of the current block
    completed, partial, reads = [embedding], None, []
    for index, output in enumerate(outputs):
        partial = output if partial is None else partial + output
        reads.append(attnres((*completed, partial), query))
        if (index + 1) % block == 0:
            completed.append(partial)
            partial = None
    assert len(completed) == 1 + writers // block

    # torch.compile(fullgraph=True): the read is one opaque operator in the graph
    @torch.compile(fullgraph=True, dynamic=False)
    def compiled(sources, q):
        return attnres(sources, q)

    again = compiled((embedding, *outputs), query)
    assert torch.equal(again, full)

    # CUDA graph: capture once, replay with new data in the same buffers
    static = [t.clone() for t in (embedding, *outputs)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        attnres(tuple(static), query)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = attnres(tuple(static), query)
    static[0].copy_(torch.randn_like(static[0]))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, attnres(tuple(static), query))
    return {"full": tuple(full.shape), "block_reads": len(reads), "completed": len(completed)}


if __name__ == "__main__":
    print(run())
