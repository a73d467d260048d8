"""Benchmark of the invariant-MACE energy+force step (metric: atom-steps/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype f32|f64] [--atoms-per-gpu A]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...        # the reference's own kernels (same GPU) on a bounded sample of the
                                                # workload; the CPU restatement on the host cores beside it

Workload: the weak-scaled slab configuration: 64 000 atoms per GPU (H:C:N:O = 50:30:10:10,
0.1 atoms/A^3, 0.9 A minimum distance, 80 x 80 A cross-section, periodic), 128-channel 2-layer
invariant MACE (l_max 3, correlation 3, 8 Bessel functions, r_max 5 A), seeded synthetic data and
random-init weights.  With N GPUs the box is N times longer and is cut into N slabs with 5 A ghost
halos; ghost node features are exchanged once per evaluation and ghost gradients are sent back.

One step = one energy+force evaluation of all atoms.  `value` is measured with every input
resident on the device and nothing but the step inside the timed region (the per-kernel timings of
the `kernels` table come from a separate pass that brackets every entry-point call with CUDA events); `e2e` goes through EnergyForceEvaluator.evaluate_host with pinned host
buffers, so host->device copies of positions / species / edge list / shifts and the device->host
copy of energy and forces are inside its timed region.  The working set of a step (several GB) is
far larger than the 126 MB L2, so no explicit L2 flush is needed between steps.

At one GPU the line also carries
  `secondary`          the other configurations of the spec on the same device: the 3 000-atom H/O box in
                       float32 (eager and replayed as a CUDA graph) and float64, and the slab in float64;
  `reference_kernels`  the reference library's own kernels (oracle/_ref, run in a child process because both
                       libraries register the same TorchScript class names) next to this library's on the
                       isolated-operator shapes, and its whole 3 000-atom step;
  `cpu_baseline`       the float64 CPU restatement on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

R_MAX = 5.0
METRIC = "energy+force atom-steps/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--atoms-per-gpu", type=int, default=64000)
    ap.add_argument("--workload", default="slab", choices=["slab", "water3000"],
                    help="slab: the weak-scaled 4-species configuration (default, the headline); water3000: the "
                         "single-GPU 3 000-atom H/O box of the spec (1 GPU only)")
    ap.add_argument("--cpu-sample-atoms", type=int, default=400)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the other configurations (profiling runs)")
    ap.add_argument("--no-reference-kernels", action="store_true", help="skip the reference library's kernels")
    ap.add_argument("--reference-sample-atoms", type=int, default=8000,
                    help="--impl reference: atoms of the sample the reference's kernels run on (they index an "
                         "N x N table with 32-bit offsets, so at most 8192)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--radial", default="exact", choices=["exact", "spline"],
                    help="exact: Bessel basis + multilayer perceptron per edge (the headline); spline: the reference's "
                         "tabulated radial weights (cubic spline, --spline-knots knots), a secondary figure")
    ap.add_argument("--spline-knots", type=int, default=256)
    ap.add_argument("--materialise-gradr", action="store_true",
                    help="float32: write the radial-weight gradient [E,4,C] and multiply it afterwards (the path "
                         "before radial_message_passing), for A/B timing")
    ap.add_argument("--graph", action="store_true",
                    help="1 GPU: replay the step as a CUDA graph in the device-resident leg (no per-kernel timings, "
                         "no roofline object); useful for small systems, which are launch-bound")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples every 50 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    smax.append(float(p[2]))
                except ValueError:
                    continue
                for n, v in zip(names, p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons),
                "samples": len(sm)}


def algorithmic_bytes(name, s, N, Ns, E, C, Z):
    """Bytes each kernel has to move when every tensor is read or written once (indices 4 B)."""
    if name.startswith("cmace_gemm3x_f32["):  # tagged with its shape: A [rows,K] in, [rows,N] out, weights
        dims = dict(x.split("=") for x in name[name.index("[") + 1:-1].split(","))
        rows, k, n = int(dims.get("M", E)), int(dims["K"]), int(dims["N"])   # no M: a product over the edges
        return 4 * (rows * k + rows * n + k * n)
    if name == "cmace_imp_bwd_edge_f32[no gradR]":   # the edge pass of radial_message_passing: R in, no gradR out
        return s * (4 * E * C + 2 * 16 * E + Ns * C + 16 * N * C) + 8 * E
    base = name[:-4]
    return {
        "cmace_imp_fwd": s * (4 * E * C + 16 * E + Ns * C + 16 * N * C) + 8 * E,
        "cmace_imp_bwd_edge": s * (2 * 4 * E * C + 2 * 16 * E + Ns * C + 16 * N * C) + 8 * E,
        "cmace_imp_bwd_node": s * (E * C + Ns * C) + 4 * E,
        "cmace_linear": s * (16 * N * C * 2 + 4 * Z * C * C),
        "cmace_linear_tc": s * (16 * N * C * 2 + 4 * Z * C * C),
        "cmace_symcon_fwd": s * (16 * N * C + N * C),
        "cmace_symcon_bwd": s * (16 * N * C * 2 + N * C),
        # hidden radial layers: basis in, h3 out, three saved derivative arrays (written forward, read backward)
        "cmace_radial_hidden_fwd": 4 * E * (8 + 64 + 3 * 64),
        "cmace_radial_hidden_bwd": 4 * E * (64 + 3 * 64 + 8),
        "cmace_imp_radial_fused_fwd": 4 * (E * 64 + 16 * E + Ns * C + 16 * N * C + 4 * E * C) + 8 * E,
        # grad h3 from operands formed on the fly: X, G, Y, the edge lists and the weights in, [E,64] out
        "cmace_gemm3x_gradr": 4 * (E * 64 + 16 * E + Ns * C + 16 * N * C + 64 * 4 * C) + 8 * E,
        # tabulated radial weights (secondary configuration): r in, R [E,4C] out / gradR in, grad r out; table in L2
        "cmace_spline_fwd": s * (E + 4 * E * C),
        "cmace_spline_bwd": s * (2 * E + 4 * E * C),
        "cmace_edge_vectors_fwd": 24 * Ns + 24 * E + 8 * E + s * 3 * E,
        "cmace_edge_vectors_bwd": 2 * s * 3 * E + 4 * E + 24 * Ns,
        "cmace_edge_basis_fwd": s * E * (3 + 16 + 8),
        "cmace_edge_basis_bwd": s * E * (3 + 16 + 8 + 3),
    }.get(base)


# DRAM traffic per edge (dram__bytes_read.sum + dram__bytes_write.sum of one launch / edges) from the ncu capture of
# the 8 000-atom case summarised in profiles/step_kernels_small_case_f32.txt (E = 417 248 there); the traffic of every
# edge kernel grows in proportion to E, so a full launch moves this many bytes times its own E.
_SRC = "profiles/step_kernels_small_case_f32.txt"
NCU_TRAFFIC_PER_EDGE = {
    "cmace_imp_bwd_edge_f32[no gradR]": (2622.0, _SRC),   # mean of a step's two launches (with / without the T array)
    "cmace_imp_fwd_f32": (2173.0, _SRC),
    "cmace_gemm3x_gradr_f32": (402.0, _SRC),
    "cmace_gemm3x_f32[K=64,N=512]": (2163.0, _SRC),
    "cmace_radial_hidden_fwd_f32": (920.0, _SRC),
    "cmace_radial_hidden_bwd_f32": (1060.0, _SRC),
}


def tensor_flops(name, E, C):
    """Tensor-core flops one launch executes, for the kernels whose binding roof is the tensor pipe: the product of
    the radial-weight gradient with the last radial layer runs three TF32 terms of 2 * E * 4C * 64 flops each."""
    if name == "cmace_gemm3x_gradr_f32":
        return 3 * 2 * E * 4 * C * 64
    return None


def tf32_peak():
    """Dense TF32 peak = half the measured dense bf16 rate (MEASURED_PEAKS.json bf16_tflops, the burst figure of a kernel
    timed alone); TF32 runs at half the bf16 rate on this tensor core."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]) / 2.0, "half of the measured bf16 burst rate (MEASURED_PEAKS.json bf16_tflops)"
    return 1590.0 / 2.0, "fallback (half of 1.59 PFLOP/s bf16)"


def cpu_reference_run(args, steps, warmup):
    """The float64 CPU restatement on a bounded sample of the same workload (same density,
    species mix and model; `--cpu-sample-atoms` atoms in a periodic cube)."""
    from cuda_mace_b200 import cg, systems
    from oracle import model as omodel

    torch.set_num_threads(os.cpu_count() or 1)
    n = args.cpu_sample_atoms
    side = (n / 0.1) ** (1.0 / 3.0)
    pos = systems.random_box(n, np.full(3, side), 0.9, 4)
    rng = np.random.default_rng(5)
    species = rng.choice(4, size=n, p=[0.5, 0.3, 0.1, 0.1])
    ei, sh = systems.neighbor_list(pos, np.full(3, side), (True, True, True), R_MAX)
    params = systems.init_params(128, 4, 1)
    U = cg.u_matrices()
    attrs = systems.one_hot(species, 4)
    tpos, tei, tsh = torch.from_numpy(pos), torch.from_numpy(ei), torch.from_numpy(sh)
    for _ in range(warmup):
        omodel.energy_and_forces(params, U, tpos, attrs, tei, tsh)
    t0 = time.perf_counter()
    for _ in range(steps):
        omodel.energy_and_forces(params, U, tpos, attrs, tei, tsh)
    dt = (time.perf_counter() - t0) / steps
    return {"value": n / dt, "unit": "atom-steps/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n} atoms ({ei.shape[1]} edges) of the same density, species mix and 128-channel model, "
                      f"float64 torch restatement (oracle/), {steps} timed call(s) of {dt:.2f} s"}, dt


def cpu_named_config(name, steps):
    """The CPU restatement on a named configuration of the spec at its full size: "cfg0" (192 atoms, 64 channels,
    4 species) or "water3000" (3 000 atoms, 128 channels).  Returns atoms, seconds per call, atom-steps/s."""
    from cuda_mace_b200 import cg, systems
    from oracle import model as omodel

    torch.set_num_threads(os.cpu_count() or 1)
    sysd = systems.make_system(name)
    pos, species = sysd["positions"], sysd["species"]
    ei, sh = systems.neighbor_list(pos, sysd["box"], (True, True, True), R_MAX)
    params = systems.init_params(sysd["channels"], sysd["n_species"], 0 if name == "cfg0" else 1)
    U = cg.u_matrices()
    attrs = systems.one_hot(species, sysd["n_species"])
    tpos, tei, tsh = torch.from_numpy(pos), torch.from_numpy(ei), torch.from_numpy(sh)
    t0 = time.perf_counter()
    for _ in range(steps):
        omodel.energy_and_forces(params, U, tpos, attrs, tei, tsh)
    dt = (time.perf_counter() - t0) / steps
    n = pos.shape[0]
    return {"config": name, "atoms": n, "edges": int(ei.shape[1]), "channels": sysd["channels"], "dtype": "f64",
            "calls": steps, "s_per_call": dt, "atom_steps_per_s": n / dt, "cores": torch.get_num_threads()}


REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcuda_mace.so")


def run_reference_child(mode_args, timeout=600):
    """python -m oracle.ref_run ... in a child process; returns the parsed JSON it wrote, or {"unavailable": why}."""
    if not os.path.isfile(REF_LIB):
        return {"unavailable": "oracle/_ref/libcuda_mace.so is not built (python -m oracle.build_ref needs the "
                               "reference's sources)"}
    fd, out = tempfile.mkstemp(suffix=".json")
    os.close(fd)
    try:
        r = subprocess.run([sys.executable, "-m", "oracle.ref_run"] + mode_args + ["--out", out], cwd=ROOT,
                           capture_output=True, text=True, timeout=timeout)
        if r.returncode != 0:
            return {"unavailable": "the reference run failed: " + (r.stderr.strip().splitlines() or ["?"])[-1][:300]}
        with open(out) as f:
            return json.load(f)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference run did not finish in {timeout} s"}
    finally:
        if os.path.exists(out):
            os.unlink(out)


def reference_kernels_block(iters):
    """The reference library's kernels and this library's on the same isolated-operator shapes, on this GPU."""
    from cuda_mace_b200 import opbench

    ref = run_reference_child(["bench", "--iters", str(iters), "--warmup", "10"])
    if isinstance(ref, dict):
        return ref
    dev = torch.device("cuda")
    opbench.RECORDS.clear()
    opbench.bench_symcon(torch.float32, iters, dev)
    opbench.bench_imp(torch.float32, iters, dev, graph="symmetric")
    opbench.bench_linear(torch.float32, iters, dev)
    opbench.bench_edge(torch.float32, iters, dev)
    def key(r):
        c = r["case"]
        stem = c.split(" forward")[0].split(" backward")[0]
        which = " forward+backward" if "forward+backward" in c else " forward" if " forward" in c else \
            " backward" if " backward" in c else ""
        return r["op"], stem + which

    ours = {key(r): r for r in opbench.RECORDS}
    rows = []
    for r in ref:
        row = {"op": r["op"], "case": r["case"], "reference_ms": r["ms"]}
        if "atom_steps_per_s" in r:
            row["reference_atom_steps_per_s"] = r["atom_steps_per_s"]
        # "with derivatives" (reference stores them in the forward) pairs with this library's plain forward
        if "no derivatives" in r["case"]:
            rows.append(row)
            continue
        mine = ours.get(key(r))
        if mine is not None:
            row["ours_ms"] = mine["ms"]
            row["reference_over_ours"] = round(r["ms"] / mine["ms"], 2)
        rows.append(row)
    return {"protocol": f"10 warm-up + {iters} timed calls, CUDA events, float32, identical shapes and edge lists "
                        "(symmetrised random graph: the only kind the reference accepts)",
            "reference_library": "oracle/_ref/libcuda_mace.so, built from the reference's sources by oracle/build_ref.py, "
                                 "kernels compiled by NVRTC for this GPU at first launch",
            "rows": rows}


def secondary_block(args, dev, sysd_slab, dom_slab, steps):
    """The other configurations of the spec on this GPU: device-resident ms per step and atom-steps/s."""
    from cuda_mace_b200 import cg, domain, evaluator, model, systems

    out = {}
    U = cg.u_matrices()

    def run(name, sysd, dom, dtype, graph):
        params = systems.init_params(128, sysd["n_species"], 1)
        net = model.InvariantMACE(params, U, dtype=dtype, device=dev)
        ev = evaluator.EnergyForceEvaluator(net, dom, dev)
        pos = ev.load_domain()
        if graph:
            ev.capture(pos)
        for _ in range(3):
            ev(pos)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            energy, forces = ev(pos)
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / steps
        n = dom.n_owned
        out[name] = {"atoms": n, "edges": int(dom.edge_index.shape[1]), "dtype": "f32" if dtype == torch.float32 else "f64",
                     "cuda_graph": bool(graph), "steps": steps, "ms_per_step": ms, "atom_steps_per_s": n / (ms * 1e-3),
                     "energy": float(energy)}
        del ev, net
        torch.cuda.empty_cache()

    w = systems.make_system("water3000")
    wdom = domain.partition_slabs(w["positions"], w["species"], w["box"], 1, R_MAX, 0)
    run("water3000_f32", w, wdom, torch.float32, False)
    run("water3000_f32_graph", w, wdom, torch.float32, True)
    run("water3000_f64", w, wdom, torch.float64, False)
    run("water3000_f64_graph", w, wdom, torch.float64, True)
    if args.dtype == "f32" and args.workload == "slab":
        run("slab_f64", sysd_slab, dom_slab, torch.float64, False)
    return out


def main():
    args = parse()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    workload = (f"slab: {args.atoms_per_gpu} atoms per GPU, H:C:N:O 50:30:10:10, 0.1 atoms/A^3, 128-channel "
                f"2-layer invariant MACE, r_max {R_MAX} A, energy+forces")
    if args.workload == "water3000":
        if world != 1:
            raise SystemExit("the water3000 workload is a single-GPU configuration")
        workload = (f"water3000: 3000 atoms (1000 O, 2000 H) in a periodic cube at 0.1 atoms/A^3, 128-channel "
                    f"2-layer invariant MACE, r_max {R_MAX} A, energy+forces")

    if args.impl == "reference":
        # Rank 0 alone.  The reference is a GPU library without a CPU path, so the arm times ITS OWN KERNELS on this
        # GPU: the energy+force step re-assembled from its operator classes (oracle/ref_model.py) on a sample of the
        # workload (same density, species mix and 128-channel model) that its N x N reverse-edge table and 32-bit
        # offsets can hold; `--steps` / `--warmup` are honoured.  The float64 CPU restatement is timed beside it
        # (`cpu_baseline`, bounded sample) together with two configurations of the spec at their full size.
        if rank != 0:
            return
        warmup = max(args.warmup, 3)
        n_ref = min(args.reference_sample_atoms, 8192)
        ref = run_reference_child(["step", "--atoms", str(n_ref), "--channels", "128", "--species", "4",
                                   "--iters", str(args.steps), "--warmup", str(warmup)])
        cpu_steps = max(1, min(args.steps, 3))
        base, dt = cpu_reference_run(args, cpu_steps, 1)
        cpu_configs = [cpu_named_config("cfg0", max(1, min(args.steps, 10))), cpu_named_config("water3000", 1)]
        if "unavailable" in ref:
            value, ms, dtype, kind = base["value"], dt * 1e3, "f64", "port"
            sample, steps, launches = base["sample"], cpu_steps, 0
        else:
            value, ms, dtype, kind = ref["atom_steps_per_s"], ref["ms_per_step"], "f32", "reference"
            sample = (f"{ref['atoms']} atoms ({ref['edges']} edges) of the same density, species mix and 128-channel "
                      "model in a periodic cube; the reference's own kernels on this GPU (float32, 256-knot spline, "
                      "its TorchScript classes from oracle/_ref/libcuda_mace.so driven by oracle/ref_model.py), "
                      "inputs resident on the device")
            steps, launches = ref["steps"], None
        line = {
            "impl": "reference", "metric": METRIC, "value": value, "unit": "atom-steps/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": workload, "sample": sample},
            "reference_kind": kind,
            "reference_gpu_step": ref,
            "cpu_baseline": base,
            "cpu_configs": cpu_configs,
            "e2e": {"value": value, "unit": "atom-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": launches,
        }
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the kernels)")
    # libraries (NCCL's version banner) write to stdout; keep stdout clean for the one JSON line
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    import torch.distributed as dist

    from cuda_mace_b200 import _abi, cg, domain, evaluator, model, ops, systems

    if args.materialise_gradr:
        ops.RADIAL_GRADIENT_ON_THE_FLY = False
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch.float32 if args.dtype == "f32" else torch.float64
    s_bytes = 4 if args.dtype == "f32" else 8

    # ---- workload ------------------------------------------------------------------------------
    if args.workload == "water3000":
        sysd = systems.make_system("water3000")
        n_total = sysd["positions"].shape[0]
    else:
        n_total = args.atoms_per_gpu * world
        sysd = systems.make_system("slab", n_atoms=n_total, seed=4)
    dom = domain.partition_slabs(sysd["positions"], sysd["species"], sysd["box"], world, R_MAX, rank)
    params = systems.init_params(128, sysd["n_species"], 1)
    if args.radial == "spline":
        model.add_spline_knots(params, args.spline_knots)
    net = model.InvariantMACE(params, cg.u_matrices(), dtype=dtype, device=dev, radial=args.radial)
    ev = evaluator.EnergyForceEvaluator(net, dom, dev)
    pos = ev.load_domain()
    E, N, Ns = dom.edge_index.shape[1], dom.n_owned, dom.n_local

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------------------------
    if args.graph:
        if world != 1:
            raise SystemExit("--graph needs a single GPU")
        ev.capture(pos)
    for _ in range(max(args.warmup, 3)):
        energy, forces = ev(pos)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _abi.launch_count
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        energy, forces = ev(pos)
    t1.record()
    barrier()
    launches = _abi.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms) / args.steps
    value = n_total / (ms_per_step * 1e-3)
    if args.graph:
        launches = None   # a replayed graph launches the recorded kernels without passing through the binding

    # ---- per-kernel pass: the same steps again with CUDA events around every entry-point call -------
    kernel_steps = 0 if args.graph else min(args.steps, 5)
    kernel_ms, bracketed_ms = {}, None
    if kernel_steps:
        _abi.start_timing()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(kernel_steps):
            ev(pos)
        k1.record()
        kernel_ms = _abi.stop_timing()
        bracketed_ms = k0.elapsed_time(k1) / kernel_steps
    barrier()

    # ---- end-to-end timing with host buffers -----------------------------------------------------
    e2e_value, h2d, d2h = None, 0, 0
    if not args.no_e2e:
        ev._graph = None    # the host-buffer leg rebuilds the topology every step and runs eagerly
        batch = ev.host_batch()
        out_forces = torch.empty(N, 3, dtype=torch.float64, pin_memory=True)
        # the device-resident leg above leaves the host link idle; a few more warm-up calls than the minimum let it
        # come back to full speed before the timed region (first-call-on-a-fresh-box runs measured 20 % low otherwise)
        for _ in range(max(args.warmup, 8)):
            ev.evaluate_host(batch, out_forces)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            e_host, _ = ev.evaluate_host(batch, out_forces)
        e1.record()
        barrier()
        ems = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
        e2e_value = n_total / (float(ems) / args.steps * 1e-3)
        h2d = evaluator.EnergyForceEvaluator.h2d_bytes(batch)
        d2h = out_forces.numel() * out_forces.element_size() + 8

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel --------------------------------------------------------
    peak, peak_src = peaks()
    per_kernel = {}
    top, top_ms = None, -1.0
    # products over the edges keep the short name [K=..,N=..]; the node products carry their row count
    kernel_ms = {(name.replace(f"M={E},", "") if name.startswith("cmace_gemm3x_f32[") else name): v
                 for name, v in kernel_ms.items()}
    for name, (calls, tot) in sorted(kernel_ms.items()):
        b = algorithmic_bytes(name, s_bytes, N, Ns, E, 128, sysd["n_species"])
        avg = tot / calls
        per_kernel[name] = {"calls_per_step": calls / kernel_steps, "avg_ms": avg,
                            "share_of_step": tot / (bracketed_ms * kernel_steps),
                            "achieved_gbs": (b / (avg * 1e-3) / 1e9) if b else None}
        if b and tot > top_ms:
            top, top_ms = name, tot
    roofline = None
    if top:
        per_edge = NCU_TRAFFIC_PER_EDGE.get(top)
        traffic = per_edge[0] * E if per_edge else None
        traffic_src = f"ncu capture of a smaller case scaled by edges, {per_edge[1]}" if per_edge else None
        flops = tensor_flops(top, E, 128)
        if flops:
            # not HBM-bound (its operands are formed on chip): the tensor pipe is the roof that binds it
            tpeak, tsrc = tf32_peak()
            ach = flops / (per_kernel[top]["avg_ms"] * 1e-3) / 1e12
            roofline = {"kernel": top, "bound": "tensor", "achieved": ach, "peak": tpeak, "unit": "TFLOP/s",
                        "frac": ach / tpeak, "traffic": traffic, "traffic_source": traffic_src, "peak_source": tsrc,
                        "algorithmic_flops_per_launch": flops, "avg_launch_ms": per_kernel[top]["avg_ms"],
                        "hbm_gbs_of_algorithmic_bytes": per_kernel[top]["achieved_gbs"],
                        "note": "of the two roofs this schema knows the tensor pipe is the nearer one; the unit that "
                                "binds the kernel is the SM's load/store data pipe (about 80 % busy in the ncu "
                                "capture named in traffic_source): the operand is formed from shared-memory reads"}
        else:
            ach = per_kernel[top]["achieved_gbs"]
            roofline = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s",
                        "frac": ach / peak, "traffic": traffic, "traffic_source": traffic_src, "peak_source": peak_src,
                        "algorithmic_bytes_per_launch": algorithmic_bytes(top, s_bytes, N, Ns, E, 128, sysd["n_species"]),
                        "avg_launch_ms": per_kernel[top]["avg_ms"]}
        # the largest HBM-bound kernel beside it, for the fraction of the copy peak the streaming kernels reach
        hbm = [(v["share_of_step"], k) for k, v in per_kernel.items() if v["achieved_gbs"] and not tensor_flops(k, E, 128)]
        if hbm:
            k = max(hbm)[1]
            roofline["largest_hbm_bound_kernel"] = {"kernel": k, "achieved": per_kernel[k]["achieved_gbs"], "peak": peak,
                                                    "unit": "GB/s", "frac": per_kernel[k]["achieved_gbs"] / peak}

    line = {
        "metric": METRIC, "value": value, "unit": "atom-steps/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": workload, "atoms_total": n_total, "edges_per_gpu": E, "owned_per_gpu": N,
                   "local_incl_ghosts": Ns, "parallelism": f"slab domain decomposition x{world}",
                   "l2_policy": "inputs larger than L2 (per-step working set of several GB)",
                   "energy": float(energy), "max_abs_force": float(forces.abs().max())},
        "roofline": roofline,
        "kernels": per_kernel,
        "kernels_pass": {"steps": kernel_steps, "ms_per_step_with_events": bracketed_ms},
        "e2e": {"value": e2e_value, "unit": "atom-steps/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if args.radial == "spline":
        line["config"]["radial"] = f"cubic spline table, {args.spline_knots} knots (not the headline configuration)"
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"], _ = cpu_reference_run(args, 2, 1)
    if world == 1 and not args.no_secondary:
        del ev, net, energy, forces
        torch.cuda.empty_cache()
        line["secondary"] = secondary_block(args, dev, sysd, dom, min(args.steps, 10))
    if world == 1 and not args.no_reference_kernels:
        torch.cuda.empty_cache()
        line["reference_kernels"] = reference_kernels_block(50)
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
