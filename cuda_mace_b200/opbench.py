"""Op-level timings of the CUDA operators on the isolated-operator configurations of the benchmark spec.

    python -m cuda_mace_b200.opbench [--op all|symcon|imp|fused|linear|radial|nlist] [--dtype f32|f64] [--iters 20]

symcon  SymmetricContraction, N = 4096 atoms, 128 channels, 10 species, forward and forward+backward
imp     InvariantMessagePassing, N = 8192 receivers, Poisson(30) edges each, 128 channels, forward and backward
fused   message passing with the last radial layer inside (float32), N receivers with Poisson(52) edges each
gradr   gradient of the last hidden radial layer from operands formed inside the tensor-core kernel (float32)
linear  Linear, N = 3000 and N = 64000 nodes, 128 channels; ElementalLinear, N = 64000, 4 elements
edge    spherical harmonics and the tabulated (cubic spline) radial weights, E = 157 000 and 3 331 524 edges
radial  the three hidden radial layers in one kernel (float32), E edges
nlist   neighbour list of the 64 000-atom slab system on the device (cell-list kernels) and on the host (numpy)

One JSON line per measurement: CUDA-event time per call (after warm-up, inputs larger than L2 or L2 flushed by
the other operands of the same call), algorithmic bytes and the bandwidth they imply.  Inputs are seeded
synthetic tensors with the shapes and distributions of the spec.
"""
import argparse
import json

import torch

from . import cg, ops


def _time(fn, iters, warmup=3):
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


RECORDS = []   # every measurement of this process, for callers that want them as data (bench.py)


def _emit(op, what, ms, nbytes, **extra):
    line = {"op": op, "case": what, "ms": round(ms, 4), "algorithmic_bytes": int(nbytes),
            "gb_per_s": round(nbytes / (ms * 1e-3) / 1e9, 1)}
    line.update(extra)
    RECORDS.append(line)
    print(json.dumps(line), flush=True)


def _graph(N, mean_degree, gen):
    deg = torch.poisson(torch.full((N,), float(mean_degree)), generator=gen).long()
    recv = torch.repeat_interleave(torch.arange(N), deg)
    send = torch.randint(0, N, (recv.numel(),), generator=gen)
    return send.int(), recv.int()


def bench_symcon(dtype, iters, dev):
    gen = torch.Generator().manual_seed(1)
    N, C, Z = 4096, 128, 10
    s = 4 if dtype == torch.float32 else 8
    U = cg.u_matrices()
    W = [torch.randn(Z, n, C, generator=gen, dtype=torch.float64).to(dtype) / n ** 0.5 for n in (23, 4, 1)]
    mod = ops.SymmetricContraction(*U, *W).to(dev)
    X = torch.randn(N, 16, C, generator=gen, dtype=torch.float64).to(dtype).to(dev).requires_grad_(True)
    at = torch.randint(0, Z, (N,), generator=gen, dtype=torch.int32).to(dev)

    def fwd_bwd():
        X.grad = None
        (mod(X, at) ** 2).sum().backward()

    with torch.no_grad():
        _emit("symcon", f"N={N} C={C} Z={Z} forward", _time(lambda: mod(X, at), iters), s * 17 * N * C)
    _emit("symcon", f"N={N} C={C} Z={Z} forward+backward", _time(fwd_bwd, iters), s * (17 + 33) * N * C)


def bench_imp(dtype, iters, dev, graph="poisson"):
    """graph = "poisson": the configuration of the spec (Poisson(30) receivers, uniform random senders);
    "symmetric": the symmetrised random graph of the same mean degree in which every node has an edge, the only kind
    of list the reference's kernels accept, so that both libraries can be timed on identical lists."""
    from . import systems

    gen = torch.Generator().manual_seed(2)
    N, C = 8192, 128
    s = 4 if dtype == torch.float32 else 8
    send, recv = systems.symmetric_graph(2, N, 30) if graph == "symmetric" else _graph(N, 30, gen)
    E = send.numel()
    X = torch.randn(N, C, generator=gen, dtype=torch.float64).to(dtype).to(dev).requires_grad_(True)
    Y = torch.randn(16, E, generator=gen, dtype=torch.float64).to(dtype).to(dev).requires_grad_(True)
    R = torch.randn(E, 4, C, generator=gen, dtype=torch.float64).to(dtype).to(dev).requires_grad_(True)
    topo = ops.EdgeTopology(send.to(dev), recv.to(dev), N, N)
    tp = ops.InvariantMessagePassingTP()
    G = torch.randn(N, 16, C, generator=gen, dtype=torch.float64).to(dtype).to(dev)
    out = tp.forward(X, Y, R, topo.sender, topo.receiver, N, topology=topo)
    with torch.no_grad():
        t_f = _time(lambda: tp.forward(X, Y, R, topo.sender, topo.receiver, N, topology=topo), iters)
    _emit("imp", f"N={N} E={E} C={C} forward", t_f, s * (4 * E * C + 16 * E + N * C + 16 * N * C) + 8 * E)
    t_b = _time(lambda: torch.autograd.grad(out, (X, Y, R), G, retain_graph=True), iters)
    _emit("imp", f"N={N} E={E} C={C} backward (edge + sender pass)", t_b,
          s * (8 * E * C + 32 * E + 2 * N * C + 16 * N * C) + 8 * E)


def bench_fused(dtype, iters, dev, nodes):
    if dtype != torch.float32:
        return
    gen = torch.Generator().manual_seed(0)
    N, C, K = nodes, 128, 64
    send, recv = _graph(N, 52, gen)
    E = send.numel()
    X = torch.randn(N, C, generator=gen).to(dev).requires_grad_(True)
    Y = torch.randn(16, E, generator=gen).to(dev)
    H = torch.randn(E, K, generator=gen).to(dev)
    W = (torch.randn(K, 4 * C, generator=gen) / 8).to(dev)
    WT = W.t().contiguous()
    topo = ops.EdgeTopology(send.to(dev), recv.to(dev), N, N)
    t = _time(lambda: ops.fused_radial_message_passing(X, Y, H, W, WT, topo), iters)
    ops.check_status()
    _emit("fused", f"N={N} E={E} C={C} K={K} forward, R written for the backward", t,
          4 * (E * K + 16 * E + N * C + 16 * N * C + 4 * E * C) + 8 * E)
    Xd = X.detach()   # no gradient requested: the kernel does not write R
    t = _time(lambda: ops.fused_radial_message_passing(Xd, Y, H, W, WT, topo), iters)
    _emit("fused", f"N={N} E={E} C={C} K={K} forward only", t, 4 * (E * K + 16 * E + N * C + 16 * N * C) + 8 * E)


def bench_gradr(dtype, iters, dev, nodes):
    """Backward of the last radial layer + message passing without a gradR array: the tensor-core product whose
    A operand is formed on the fly, and the edge pass that no longer writes gradR; Poisson(52) receivers."""
    if dtype != torch.float32:
        return
    gen = torch.Generator().manual_seed(5)
    N, C, K = nodes, 128, 64
    send, recv = _graph(N, 52, gen)
    E = send.numel()
    X = torch.randn(N, C, generator=gen).to(dev)
    Y = torch.randn(16, E, generator=gen).to(dev)
    G = torch.randn(N, 16, C, generator=gen).to(dev)
    W = (torch.randn(K, 4 * C, generator=gen) / 8).to(dev)
    topo = ops.EdgeTopology(send.to(dev), recv.to(dev), N, N)
    t = _time(lambda: ops.radial_gradient_product(X, G, Y, W, topo), iters)
    ops.check_status()
    _emit("gradr", f"N={N} E={E} C={C} K={K} grad H from operands formed on the fly", t,
          4 * (E * K + 16 * E + N * C + 16 * N * C + K * 4 * C) + 8 * E, gflops=round(3 * 2 * E * 4 * C * K / t / 1e6, 1))


def bench_linear(dtype, iters, dev):
    gen = torch.Generator().manual_seed(3)
    C = 128
    s = 4 if dtype == torch.float32 else 8
    W = (torch.randn(4, C, C, generator=gen, dtype=torch.float64)).to(dtype).to(dev)
    WT = W.transpose(-1, -2).contiguous()
    for N in (3000, 64000):
        X = torch.randn(N, 16, C, generator=gen, dtype=torch.float64).to(dtype).to(dev)
        with torch.no_grad():
            t = _time(lambda: ops.linear_forward(X, W, WT), iters)
        _emit("linear", f"N={N} K=Nout={C}", t, s * (32 * N * C + 4 * C * C), gflops=round(32 * N * C * C / t / 1e6, 1))
    N, Z = 64000, 4
    WE = torch.randn(Z, 4, C, C, generator=gen, dtype=torch.float64).to(dtype).to(dev)
    WET = WE.transpose(-1, -2).contiguous()
    oh = torch.zeros(N, Z, dtype=dtype, device=dev)
    oh[torch.arange(N), torch.randint(0, Z, (N,), generator=gen)] = 1.0
    with torch.no_grad():
        t = _time(lambda: ops.elemental_linear_forward(X, WE, WET, oh), iters)
    _emit("elinear", f"N={N} Z={Z} K=Nout={C}", t, s * (32 * N * C + 4 * Z * C * C))
    ops.check_status()


def bench_edge(dtype, iters, dev):
    """Spherical harmonics alone (the reference's operator) and the tabulated radial weights, at the edge counts of
    the 3 000-atom box and of one 64 000-atom slab."""
    import math

    s = 4 if dtype == torch.float32 else 8
    sh = ops.SphericalHarmonics()
    knots = torch.linspace(1e-12, 6.0, 256, dtype=torch.float64)
    vals = torch.sin(knots[:, None] * torch.arange(1, 513, dtype=torch.float64) / 100.0)
    h = float(knots[1] - knots[0])
    spl = ops.CubicSpline(knots.to(dtype).to(dev), vals.to(dtype).to(dev), h, 5.0)
    for E in (157000, 3331524):
        gen = torch.Generator().manual_seed(4)
        xyz = torch.randn(E, 3, generator=gen).to(dtype).to(dev).requires_grad_(True)
        GY = torch.randn(16, E, generator=gen).to(dtype).to(dev)
        Y = sh(xyz)
        _emit("sh", f"E={E} forward", _time(lambda: sh(xyz), iters), s * E * (3 + 16))
        _emit("sh", f"E={E} backward (derivatives recomputed)", _time(
            lambda: torch.autograd.grad(Y, xyz, GY, retain_graph=True), iters), s * E * (3 + 16 + 3))
        del Y, GY
        r = (0.3 + 4.7 * torch.rand(E, generator=gen)).to(dtype).to(dev).requires_grad_(True)
        R = spl(r)
        GR = torch.randn(E, 512, dtype=dtype, device=dev)
        _emit("spline", f"E={E} F=512 forward", _time(lambda: spl(r), iters), s * E * (1 + 512))
        _emit("spline", f"E={E} F=512 backward (derivatives recomputed)", _time(
            lambda: torch.autograd.grad(R, r, GR, retain_graph=True), iters), s * E * (1 + 512 + 1))
        del R, GR


def bench_radial(dtype, iters, dev, edges):
    if dtype != torch.float32:
        return
    gen = torch.Generator().manual_seed(4)
    E = edges
    Ws = [(torch.randn(a, b, generator=gen) / a ** 0.5).to(dev) for a, b in ((8, 64), (64, 64), (64, 64))]
    WTs = [w.t().contiguous() for w in Ws]
    basis = torch.randn(E, 8, generator=gen).to(dev).requires_grad_(True)
    g = torch.randn(E, 64, generator=gen).to(dev)
    out = ops.radial_hidden(basis, Ws, WTs)
    t_f = _time(lambda: ops.radial_hidden(basis, Ws, WTs), iters)
    _emit("radial", f"E={E} hidden layers forward (derivatives saved)", t_f, 4 * E * (8 + 64 + 192))
    t_b = _time(lambda: torch.autograd.grad(out, basis, g, retain_graph=True), iters)
    _emit("radial", f"E={E} hidden layers backward", t_b, 4 * E * (64 + 192 + 8))
    ops.check_status()


def bench_nlist(iters, dev, nodes):
    import time

    import numpy as np

    from . import systems

    s = systems.make_system("slab", n_atoms=nodes)
    pos = torch.from_numpy(s["positions"]).to(dev)
    box = np.asarray(s["box"], dtype=np.float64)
    ei, sh, si = ops.neighbor_list(pos, box, (True, True, True), 5.0)
    E = int(ei.shape[1])
    t = _time(lambda: ops.neighbor_list(pos, box, (True, True, True), 5.0), iters)
    _emit("nlist", f"N={nodes} E={E} periodic box, device cell list (includes the host read of the edge count)", t,
          nodes * 24 + E * (8 + 3 + 24))
    t0 = time.perf_counter()
    ei_h, sh_h = systems.neighbor_list(s["positions"], box, (True, True, True), 5.0)
    _emit("nlist", f"N={nodes} E={ei_h.shape[1]} periodic box, host cell list (numpy, 1 call)",
          (time.perf_counter() - t0) * 1e3, nodes * 24 + E * (8 + 3 + 24))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="all", choices=["all", "symcon", "imp", "fused", "gradr", "linear", "edge", "radial", "nlist"])
    ap.add_argument("--graph", default="poisson", choices=["poisson", "symmetric"], help="edge list of the imp case")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nodes", type=int, default=64000, help="receivers of the fused case")
    ap.add_argument("--edges", type=int, default=3331524, help="edges of the radial case")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("opbench needs a CUDA device (there is no CPU fallback for the kernels)")
    dev = torch.device("cuda")
    dtype = torch.float32 if args.dtype == "f32" else torch.float64
    if args.op in ("all", "symcon"):
        bench_symcon(dtype, args.iters, dev)
    if args.op in ("all", "imp"):
        bench_imp(dtype, args.iters, dev, args.graph)
    if args.op in ("all", "linear"):
        bench_linear(dtype, args.iters, dev)
    if args.op in ("all", "edge"):
        bench_edge(dtype, args.iters, dev)
    if args.op in ("all", "radial"):
        bench_radial(dtype, args.iters, dev, args.edges)
    if args.op in ("all", "gradr"):
        bench_gradr(dtype, args.iters, dev, args.nodes)
    if args.op in ("all", "fused"):
        bench_fused(dtype, args.iters, dev, args.nodes)
    if args.op in ("all", "nlist"):
        bench_nlist(args.iters, dev, args.nodes)


if __name__ == "__main__":
    main()
