"""Child process of the programmatic-dependent-launch test: a chain of GEMMs and small kernels, each reading what the one before wrote,
eager and as a CUDA graph; prints a digest of every result.  The parent runs it with MARY_PDL=0 and MARY_PDL=1 and compares."""
import hashlib
import sys

import torch

from mary_b200 import ops
from mary_b200.ops import cuda as K


def chain(x, ws, norm_w):
    outs = []
    h = x
    for i, w in enumerate(ws):
        h = ops.linear(h, w)                              # constant weights: may be requested early under PDL
        h = ops.rmsnorm(h, norm_w[i], 1e-6)
        outs.append(h)
    # a GEMM whose "weights" were written by the previous kernel: no early request allowed
    g = K.gemm(outs[-1], outs[-2][: outs[-1].shape[1]].contiguous()) if outs[-2].shape[0] >= outs[-1].shape[1] else outs[-1]
    outs.append(g)
    lg = ops.linear_f32(outs[-2], ws[0])
    outs.append(lg)
    return outs


def main():
    torch.manual_seed(0)
    dev = "cuda"
    M = int(sys.argv[1]) if len(sys.argv) > 1 else 48
    dims = [1024, 2048, 512, 1024, 1536]
    x = (torch.randn(M, dims[0], device=dev) * 0.5).bfloat16()
    ws = [(torch.randn(dims[i + 1], dims[i], device=dev) * dims[i] ** -0.5).bfloat16() for i in range(len(dims) - 1)]
    ws.append((torch.randn(dims[0], dims[-1], device=dev) * dims[-1] ** -0.5).bfloat16())
    norm_w = [torch.ones(w.shape[0], device=dev, dtype=torch.bfloat16) for w in ws]
    dig = hashlib.sha256()
    for rep in range(3):
        for t in chain(x, ws, norm_w):
            dig.update(t.float().cpu().numpy().tobytes())
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain(x, ws, norm_w)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        outs = chain(x, ws, norm_w)
    for rep in range(3):
        x.mul_(-1.0)                                      # new inputs between replays: stale reads would show
        g.replay()
        torch.cuda.synchronize()
        for t in outs:
            dig.update(t.float().cpu().numpy().tobytes())
    assert K.last_status() == 0
    import os
    print("DIGEST", dig.hexdigest(), "PDL", os.environ.get("MARY_PDL", "0"))


if __name__ == "__main__":
    main()
