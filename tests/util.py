"""Shared helpers of the test-suite: seeded graphs, tolerances, oracle wrappers."""
import numpy as np
import torch

# Parity tolerances (relative to the largest reference magnitude of the compared tensor):
# float64 within 1e-10; float32 operators within 1e-5 on outputs and 1e-4 on gradients, the bounds
# the energy (1e-5) and force (1e-4) targets are stated with.
TOL = {torch.float64: dict(out=1e-10, grad=1e-10), torch.float32: dict(out=1e-5, grad=1e-4)}


def rel_err(a, b):
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    scale = b.abs().max().item()
    if scale == 0.0:
        return (a - b).abs().max().item() if a.numel() else 0.0
    return (a - b).abs().max().item() / scale


def random_graph(seed, n_nodes, mean_degree, n_senders=None, empty_every=0):
    """Receiver-sorted random edge list with Poisson degrees; `empty_every` > 0 strips the edges of
    every k-th receiver (isolated atoms).  Returns int32 (sender, receiver)."""
    g = torch.Generator().manual_seed(seed)
    deg = torch.poisson(torch.full((n_nodes,), float(mean_degree)), generator=g).long()
    if empty_every:
        deg[::empty_every] = 0
    recv = torch.repeat_interleave(torch.arange(n_nodes), deg)
    send = torch.randint(0, n_senders or n_nodes, (int(deg.sum()),), generator=g)
    return send.to(torch.int32), recv.to(torch.int32)


def unit_vectors(seed, n, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    v = torch.randn(n, 3, generator=g, dtype=torch.float64)
    return (v / v.norm(dim=-1, keepdim=True)).to(dtype)
