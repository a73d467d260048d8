"""Benchmark of the invariant-MACE energy+force step (metric: atom-steps/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype f32|f64] [--atoms-per-gpu A]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...        # CPU restatement of the path on the host cores

Workload: the weak-scaled slab configuration: 64 000 atoms per GPU (H:C:N:O = 50:30:10:10,
0.1 atoms/A^3, 0.9 A minimum distance, 80 x 80 A cross-section, periodic), 128-channel 2-layer
invariant MACE (l_max 3, correlation 3, 8 Bessel functions, r_max 5 A), seeded synthetic data and
random-init weights.  With N GPUs the box is N times longer and is cut into N slabs with 5 A ghost
halos; ghost node features are exchanged once per evaluation and ghost gradients are sent back.

One step = one energy+force evaluation of all atoms.  `value` is measured with every input
resident on the device; `e2e` goes through EnergyForceEvaluator.evaluate_host with pinned host
buffers, so host->device copies of positions / species / edge list / shifts and the device->host
copy of energy and forces are inside its timed region.  The working set of a step (several GB) is
far larger than the 126 MB L2, so no explicit L2 flush is needed between steps.
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
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--radial", default="exact", choices=["exact", "spline"],
                    help="exact: Bessel basis + multilayer perceptron per edge (the headline); spline: the reference's "
                         "tabulated radial weights (cubic spline, --spline-knots knots), a secondary figure")
    ap.add_argument("--spline-knots", type=int, default=256)
    ap.add_argument("--graph", action="store_true",
                    help="1 GPU: replay the step as a CUDA graph in the device-resident leg (no per-kernel timings, "
                         "no roofline object); useful for small systems, which are launch-bound")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


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
        # tabulated radial weights (secondary configuration): r in, R [E,4C] out / gradR in, grad r out; table in L2
        "cmace_spline_fwd": s * (E + 4 * E * C),
        "cmace_spline_bwd": s * (2 * E + 4 * E * C),
        "cmace_edge_vectors_fwd": 24 * Ns + 24 * E + 8 * E + s * 3 * E,
        "cmace_edge_vectors_bwd": 2 * s * 3 * E + 4 * E + 24 * Ns,
        "cmace_edge_basis_fwd": s * E * (3 + 16 + 8),
        "cmace_edge_basis_bwd": s * E * (3 + 16 + 8 + 3),
    }.get(base)


# DRAM traffic per edge (dram__bytes_read.sum + dram__bytes_write.sum of one launch / edges) from the ncu captures of
# the 8 000-atom case summarised under profiles/ (E = 417 248 there); the traffic of every edge kernel grows in
# proportion to E, so a full launch moves this many bytes times its own E.
NCU_TRAFFIC_PER_EDGE = {
    # staged kernel, mean of a step's two launches: 1016 + 1050 MB with the T array, 1008 + 840 MB without
    "cmace_imp_bwd_edge_f32": (4691.0, "profiles/imp_kernels_small_case_f32.txt"),
    "cmace_imp_fwd_f32": (2170.0, "profiles/imp_kernels_small_case_f32.txt"),
    "cmace_gemm3x_f32[K=512,N=64]": (2285.0, "profiles/gemm3x_tf32_small_case_f32.txt"),
    "cmace_gemm3x_f32[K=64,N=512]": (2176.0, "profiles/gemm3x_tf32_small_case_f32.txt"),
    "cmace_radial_hidden_fwd_f32": (925.0, "profiles/radial_hidden_small_case_f32.txt"),
    "cmace_radial_hidden_bwd_f32": (1057.0, "profiles/radial_hidden_small_case_f32.txt"),
}


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
        # the reference has no CPU implementation of its own; the float64 CPU restatement stands in
        if rank != 0:
            return
        steps = max(1, min(args.steps, 3))
        base, dt = cpu_reference_run(args, steps, 1 if args.warmup > 0 else 0)
        line = {
            "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "atom-steps/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": 1 if args.warmup > 0 else 0, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": workload, "sample": base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "atom-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
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

    from cuda_mace_b200 import _abi, cg, domain, evaluator, model, systems

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
    _abi.start_timing()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        energy, forces = ev(pos)
    t1.record()
    barrier()
    kernel_ms = _abi.stop_timing()
    launches = _abi.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms) / args.steps
    value = n_total / (ms_per_step * 1e-3)

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
        per_kernel[name] = {"calls_per_step": calls / args.steps, "avg_ms": avg,
                            "share_of_step": tot / (ms_per_step * args.steps),
                            "achieved_gbs": (b / (avg * 1e-3) / 1e9) if b else None}
        if b and tot > top_ms:
            top, top_ms = name, tot
    roofline = None
    if top:
        ach = per_kernel[top]["achieved_gbs"]
        per_edge = NCU_TRAFFIC_PER_EDGE.get(top)
        roofline = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s",
                    "frac": ach / peak, "traffic": per_edge[0] * E if per_edge else None,
                    "traffic_source": (f"ncu capture of a smaller case scaled by edges, {per_edge[1]}"
                                       if per_edge else None),
                    "peak_source": peak_src,
                    "algorithmic_bytes_per_launch": algorithmic_bytes(top, s_bytes, N, Ns, E, 128, sysd["n_species"]),
                    "avg_launch_ms": per_kernel[top]["avg_ms"]}

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
        "e2e": {"value": e2e_value, "unit": "atom-steps/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if args.radial == "spline":
        line["config"]["radial"] = f"cubic spline table, {args.spline_knots} knots (not the headline configuration)"
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"], _ = cpu_reference_run(args, 2, 1)
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
