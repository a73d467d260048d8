"""Runs the reference's own operator classes (oracle/_ref/libcuda_mace.so, see oracle/build_ref.py) on a CUDA device.
TEST AND BASELINE INFRASTRUCTURE ONLY.  Always a process of its own: the reference library and this project's
TorchScript library register the same class names and cannot share an interpreter.

    python -m oracle.ref_run parity --size fixture|live --out results.npz
        every operator, forward and input gradients with loss (out * G).sum(), on the seeded cases of
        oracle.ref_cases, float32 (and float64 where the reference's templates allow it)
    python -m oracle.ref_run model --atoms 375 --out results.npz
        energy + forces of the re-assembled reference step (oracle.ref_model) on a seeded periodic box
    python -m oracle.ref_run step --atoms 8000 --iters 20 --warmup 5 --out result.json
        the same step timed with CUDA events (atom-steps/s of the reference's kernels on this GPU)
    python -m oracle.ref_run bench --out results.json [--iters 100 --warmup 10]
        the timing protocol of the reference's own scripts (warm-up, then timed iterations bracketed by
        synchronisation: tests/symmetric_contraction.py:78-87, tools/model_surgery.py:198-233), with CUDA events

Every input passes the host-side guards of oracle.ref_cases before the first launch, because the reference's
kernels do not check their arguments.  The reference needs CUDA_HOME for NVRTC (set to /usr/local/cuda when unset).
"""
import argparse
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libcuda_mace.so")


def load_reference():
    if not os.path.isfile(LIB):
        raise SystemExit(f"{LIB} is missing: run `python -m oracle.build_ref` where the reference checkout is")
    os.environ.setdefault("CUDA_HOME", "/usr/local/cuda")
    torch.classes.load_library(LIB)
    return torch.classes


def _f(dtype):
    return "f32" if dtype == torch.float32 else "f64"


def _put(res, prefix, **tensors):
    for k, v in tensors.items():
        res[f"{prefix}.{k}"] = v.detach().cpu().numpy()


def run_parity(size, classes, dev):
    from . import cg, ref_cases

    U = cg.u_matrices()
    res = {}
    for dtype in (torch.float32, torch.float64):
        d = dict(dtype=dtype, device=dev)
        tag = _f(dtype)
        # spherical harmonics ---------------------------------------------------------------------------------
        c = ref_cases.case_sh(size)
        xyz = c["xyz"].to(**d).requires_grad_(True)
        Y = classes.spherical_harmonics.SphericalHarmonics().forward(xyz)
        (g,) = torch.autograd.grad((Y * c["G"].to(**d)).sum(), xyz)
        _put(res, f"sh.{tag}", out=Y, grad_xyz=g)
        # cubic spline ------------------------------------------------------------------------------------------
        c = ref_cases.case_spline(size)
        r = c["r"].to(**d).requires_grad_(True)
        R = classes.cubic_spline.CubicSpline().forward(r, c["knots"].to(**d), c["coeffs"].to(**d).contiguous(),
                                                       c["h"], c["r_max"])
        (g,) = torch.autograd.grad((R * c["G"].to(**d)).sum(), r)
        _put(res, f"spline.{tag}", out=R, grad_r=g)
        # message passing -----------------------------------------------------------------------------------------
        c = ref_cases.case_imp(size)
        X, Y, R = (c[k].to(**d).contiguous().requires_grad_(True) for k in ("X", "Y", "R"))
        out = classes.inv_message_passing.InvariantMessagePassingTP().forward(
            X, Y, R, c["sender"].to(dev), c["receiver"].to(dev), c["nnodes"])
        gX, gY, gR = torch.autograd.grad((out * c["G"].to(**d)).sum(), (X, Y, R))
        _put(res, f"imp.{tag}", out=out, grad_X=gX, grad_Y=gY, grad_R=gR)
        # symmetric contraction -------------------------------------------------------------------------------------
        c = ref_cases.case_symcon(size, U)
        X = c["X"].to(**d).requires_grad_(True)
        tb = c["tables"]
        out = classes.symm_contract.SymmetricContraction().forward(
            X, c["atom_types"].to(dev), tb[0], *[t.to(dev) for t in tb[1:]],
            c["W3"].to(**d)[None].contiguous(), c["W2"].to(**d)[None].contiguous(), c["W1"].to(**d)[None].contiguous(),
            c["W3"].shape[1], c["W2"].shape[1], c["W1"].shape[1])
        (g,) = torch.autograd.grad((out * c["G"].to(**d)).sum(), X)
        _put(res, f"symcon.{tag}", out=out, grad_X=g)
        # Linear / ElementalLinear: float32 only (data_ptr<float>, jit_wrappers/src/linear_wrapper.cpp:67-70) --------
        if dtype == torch.float32:
            c = ref_cases.case_linear(size)
            X = c["X"].to(**d).requires_grad_(True)
            W = c["W"].to(**d).contiguous()
            out = classes.linear_wmma.Linear().forward(X, W, W.transpose(-1, -2).contiguous())
            (g,) = torch.autograd.grad((out * c["G"].to(**d)).sum(), X)
            _put(res, "linear.f32", out=out, grad_X=g)
            X = c["X"].to(**d).requires_grad_(True)
            W = c["WE"].to(**d).contiguous()
            out = classes.linear_wmma.ElementalLinear().forward(X, W, W.transpose(-1, -2).contiguous(),
                                                                c["one_hot"].to(**d))
            (g,) = torch.autograd.grad((out * c["G"].to(**d)).sum(), X)
            _put(res, "elinear.f32", out=out, grad_X=g)
    torch.cuda.synchronize()
    return res


def model_system(atoms, channels, n_species, seed):
    """Seeded periodic box at 0.1 atoms per cubic angstrom; the box is at least 2 r_max wide so that the full
    neighbour list holds every pair once per direction, which the reference needs."""
    from cuda_mace_b200 import systems

    side = (atoms / 0.1) ** (1.0 / 3.0)
    if side < 10.5:
        raise ValueError("box narrower than twice the cutoff: the list would hold duplicate image pairs")
    pos = systems.random_box(atoms, np.full(3, side), 0.9, seed)
    species = np.random.default_rng(seed + 1).integers(0, n_species, atoms)
    if n_species == 4:          # H : C : N : O = 50 : 30 : 10 : 10, the mix of the slab configuration
        species = np.random.default_rng(seed + 1).choice(4, size=atoms, p=[0.5, 0.3, 0.1, 0.1])
    if n_species == 2:          # the 1 : 2 oxygen : hydrogen mix of the 3 000-atom configuration
        species = (np.arange(atoms) >= atoms // 3).astype(np.int64)
    ei, sh = systems.neighbor_list(pos, np.full(3, side), (True, True, True), 5.0)
    params = systems.init_params(channels, n_species, 1)
    return pos, species, ei, sh, params


def run_model(atoms, channels, n_species, classes, dev, iters=0, warmup=0):
    from cuda_mace_b200 import systems

    from . import cg, ref_model

    pos, species, ei, sh, params = model_system(atoms, channels, n_species, seed=1)
    step = ref_model.ReferenceStep(params, cg.u_matrices(), classes, dev)
    p, e, s = torch.from_numpy(pos), torch.from_numpy(ei), torch.from_numpy(sh)
    step.check_inputs(p, e, s)
    args = (p.to(dev), systems.one_hot(species, n_species).to(dev), e.to(dev), s.to(dev))
    energy, forces = step(*args)
    torch.cuda.synchronize()
    out = dict(energy=energy.cpu().numpy(), forces=forces.cpu().numpy(), atoms=np.int64(atoms),
               edges=np.int64(ei.shape[1]))
    ms = None
    if iters:
        ms = _time(lambda: step(*args), iters, warmup)
    return out, ms


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(iters):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / iters


def run_bench(classes, dev, iters, warmup):
    """Reference kernels at the isolated-operator configurations of the benchmark spec, float32 (the dtype the
    reference model runs them in), one JSON-able record per measurement."""
    from . import cg, ref_cases
    from . import ops as oops

    rec = []
    f32 = dict(dtype=torch.float32, device=dev)

    def emit(op, case, ms, nbytes):
        rec.append(dict(op=op, case=case, ms=round(ms, 4), algorithmic_bytes=int(nbytes),
                        gb_per_s=round(nbytes / (ms * 1e-3) / 1e9, 1)))
        print(json.dumps(rec[-1]), flush=True)

    # symmetric contraction N = 4096, C = 128, Z = 10 ---------------------------------------------------------------
    g = torch.Generator().manual_seed(1)
    N, C, Z = 4096, 128, 10
    U = cg.u_matrices()
    tb = oops.pack_sparse_u(*U)
    tbd = [t.to(dev) for t in tb[1:]]
    W = [(torch.randn(Z, n, C, generator=g, dtype=torch.float64) / n ** 0.5).to(**f32)[None].contiguous()
         for n in (23, 4, 1)]
    X = torch.randn(N, 16, C, generator=g, dtype=torch.float64).to(**f32)
    at = torch.randint(0, Z, (N,), generator=g, dtype=torch.int32).to(dev)
    sc = classes.symm_contract.SymmetricContraction()

    def sc_fwd(x):
        return sc.forward(x, at, tb[0], *tbd, W[0], W[1], W[2], 23, 4, 1)

    Xg = X.clone().requires_grad_(True)

    def sc_fwd_bwd():
        Xg.grad = None
        (sc_fwd(Xg) ** 2).sum().backward()

    emit("symcon", f"N={N} C={C} Z={Z} forward", _time(lambda: sc_fwd(X), iters, warmup), 4 * 17 * N * C)
    emit("symcon", f"N={N} C={C} Z={Z} forward+backward", _time(sc_fwd_bwd, iters, warmup), 4 * (17 + 33) * N * C)

    # message passing N = 8192, mean degree 30 (symmetrised random graph, every node has an edge) -------------------
    N, C = 8192, 128
    send, recv = ref_cases.symmetric_graph(2, N, 30)
    ref_cases.check_graph(send, recv, N, C)
    E = send.shape[0]
    g = torch.Generator().manual_seed(2)
    X = torch.randn(N, C, generator=g).to(**f32).requires_grad_(True)
    Y = torch.randn(16, E, generator=g).to(**f32).requires_grad_(True)
    R = torch.randn(E, 4, C, generator=g).to(**f32).requires_grad_(True)
    G = torch.randn(N, 16, C, generator=g).to(**f32)
    sd, rd = send.to(dev), recv.to(dev)
    tp = classes.inv_message_passing.InvariantMessagePassingTP()
    with torch.no_grad():
        t_f = _time(lambda: tp.forward(X, Y, R, sd, rd, N), iters, warmup)
    emit("imp", f"N={N} E={E} C={C} forward", t_f, 4 * (4 * E * C + 16 * E + N * C + 16 * N * C) + 8 * E)
    out = tp.forward(X, Y, R, sd, rd, N)
    t_b = _time(lambda: torch.autograd.grad(out, (X, Y, R), G, retain_graph=True), iters, warmup)
    emit("imp", f"N={N} E={E} C={C} backward", t_b, 4 * (8 * E * C + 32 * E + 2 * N * C + 16 * N * C) + 8 * E)
    del X, Y, R, G, out

    # Linear N = 3000 and N = 64000 -------------------------------------------------------------------------------------
    g = torch.Generator().manual_seed(3)
    C = 128
    W = torch.randn(4, C, C, generator=g).to(**f32)
    WT = W.transpose(-1, -2).contiguous()
    lin = classes.linear_wmma.Linear()
    for N in (3000, 64000):
        X = torch.randn(N, 16, C, generator=g).to(**f32)
        with torch.no_grad():
            t = _time(lambda: lin.forward(X, W, WT), iters, warmup)
        emit("linear", f"N={N} K=Nout={C}", t, 4 * (32 * N * C + 4 * C * C))
    # ElementalLinear N = 64000, Z = 4 (one host synchronisation and four launches per element in the reference)
    N, Z = 64000, 4
    WE = torch.randn(Z, 4, C, C, generator=g).to(**f32)
    WET = WE.transpose(-1, -2).contiguous()
    oh = torch.zeros(N, Z, **f32)
    oh[torch.arange(N), torch.randint(0, Z, (N,), generator=g)] = 1.0
    el = classes.linear_wmma.ElementalLinear()
    with torch.no_grad():
        t = _time(lambda: el.forward(X, WE, WET, oh), iters, warmup)
    emit("elinear", f"N={N} Z={Z} K=Nout={C}", t, 4 * (32 * N * C + 4 * Z * C * C))
    del X

    # spherical harmonics and spline at the edge count of the 3 000-atom system and of one 64 000-atom slab ---------
    shc = classes.spherical_harmonics.SphericalHarmonics()
    spl = classes.cubic_spline.CubicSpline()
    c = ref_cases.case_spline("live")
    knots, coeffs = c["knots"].to(**f32), c["coeffs"].to(**f32).contiguous()
    for E in (157000, 3331524):
        g = torch.Generator().manual_seed(4)
        xyz = torch.randn(E, 3, generator=g).to(**f32).requires_grad_(True)
        GY = torch.randn(16, E, generator=g).to(**f32)
        Yo = shc.forward(xyz)
        with torch.no_grad():
            t_f = _time(lambda: shc.forward(xyz.detach()), iters, warmup)
        emit("sh", f"E={E} forward (no derivatives)", t_f, 4 * E * (3 + 16))
        emit("sh", f"E={E} forward with derivatives", _time(lambda: shc.forward(xyz), iters, warmup), 4 * E * (3 + 16 + 48))
        t_b = _time(lambda: torch.autograd.grad(Yo, xyz, GY, retain_graph=True), iters, warmup)
        emit("sh", f"E={E} backward", t_b, 4 * E * (48 + 16 + 3))
        del Yo, GY
        r = (0.3 + 4.7 * torch.rand(E, generator=g)).to(**f32).requires_grad_(True)
        ref_cases.check_spline(r.detach().cpu(), knots.shape[0], coeffs.shape[0], c["h"], c["r_max"])
        if E * 512 >= 2**31:
            raise ValueError("32-bit offsets of the spline kernels would overflow")
        Ro = spl.forward(r, knots, coeffs, c["h"], c["r_max"])
        GR = torch.randn(E, 512, **f32)
        emit("spline", f"E={E} F=512 forward with derivatives", _time(lambda: spl.forward(r, knots, coeffs, c["h"], c["r_max"]),
                                                                      iters, warmup), 4 * E * (1 + 2 * 512))
        t_b = _time(lambda: torch.autograd.grad(Ro, r, GR, retain_graph=True), iters, warmup)
        emit("spline", f"E={E} F=512 backward", t_b, 4 * E * (2 * 512 + 1))
        del Ro, GR, r
    return rec


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("mode", choices=["parity", "model", "step", "bench"])
    ap.add_argument("--size", default="live", choices=["fixture", "live"])
    ap.add_argument("--atoms", type=int, default=375)
    ap.add_argument("--channels", type=int, default=128)
    ap.add_argument("--species", type=int, default=4)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the reference's kernels need a CUDA device")
    classes = load_reference()
    dev = torch.device("cuda")
    if a.mode == "parity":
        np.savez_compressed(a.out, **run_parity(a.size, classes, dev))
    elif a.mode == "model":
        out, _ = run_model(a.atoms, a.channels, a.species, classes, dev)
        np.savez_compressed(a.out, **out)
    elif a.mode == "step":
        out, ms = run_model(a.atoms, a.channels, a.species, classes, dev, iters=max(1, a.iters), warmup=a.warmup)
        rec = dict(atoms=int(out["atoms"]), edges=int(out["edges"]), channels=a.channels, species=a.species,
                   steps=max(1, a.iters), warmup=a.warmup, ms_per_step=ms, atom_steps_per_s=a.atoms / (ms * 1e-3),
                   energy=float(out["energy"]))
        print(json.dumps(rec), flush=True)
        with open(a.out, "w") as f:
            json.dump(rec, f)
    else:
        rec = run_bench(classes, dev, a.iters, a.warmup)
        out, ms = run_model(3000, 128, 2, classes, dev, iters=max(10, a.iters // 5), warmup=a.warmup)
        rec.append(dict(op="model", case=f"3000 atoms H/O, E={int(out['edges'])}, C=128, float32 + spline, energy+forces",
                        ms=round(ms, 4), atom_steps_per_s=round(3000 / (ms * 1e-3), 1)))
        print(json.dumps(rec[-1]), flush=True)
        with open(a.out, "w") as f:
            json.dump(rec, f, indent=1)
    print("reference run done:", a.mode, a.out)


if __name__ == "__main__":
    main()
    sys.exit(0)
