"""Slab domain decomposition and halo exchange on CPU ranks (gloo), with the oracle's model math:
the energies and forces assembled from 2 or 3 slabs equal those of the undivided periodic system."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cuda_mace_b200 import cg, domain, systems
from oracle import model as omodel


def make_case():
    rng = np.random.default_rng(0)
    box = np.array([11.0, 12.0, 33.0])
    pos = systems.random_box(120, box, 1.2, seed=2)
    species = rng.integers(0, 3, pos.shape[0])
    params = systems.init_params(32, 3, 21, avg_num_neighbors=12.0)
    return pos, species, box, params


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        pos, species, box, params = make_case()
        U = cg.u_matrices()
        dom = domain.partition_slabs(pos, species, box, world, 5.0, rank)
        plan = domain.HaloPlan(dom, "cpu")
        attrs = systems.one_hot(dom.species, 3)
        ei, sh = torch.from_numpy(dom.edge_index), torch.from_numpy(dom.shifts)

        def node_energy(pos_local, exchange):
            return omodel.node_energies(params, U, pos_local, attrs, ei, sh, exchange=exchange, n_owned=dom.n_owned)

        e, f = domain.distributed_energy_forces(node_energy, dom, plan, torch.from_numpy(dom.positions[: dom.n_owned]))
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), e=e.numpy(), f=f.numpy(), ids=dom.owned_global,
                 n_local=dom.n_local)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_slabs_reproduce_the_periodic_system(world, tmp_path):
    pos, species, box, params = make_case()
    U = cg.u_matrices()
    ei, sh = systems.neighbor_list(pos, box, (True, True, True), 5.0)
    _, e_ref, f_ref = omodel.energy_and_forces(params, U, torch.from_numpy(pos), systems.one_hot(species, 3),
                                               torch.from_numpy(ei), torch.from_numpy(sh))
    mp.spawn(worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    forces = np.zeros_like(pos)
    seen = np.zeros(pos.shape[0], dtype=int)
    for r in range(world):
        z = np.load(tmp_path / f"rank{r}.npz")
        assert abs(float(z["e"]) - float(e_ref)) < 1e-10 * abs(float(e_ref))
        forces[z["ids"]] = z["f"]
        seen[z["ids"]] += 1
        assert int(z["n_local"]) > len(z["ids"])  # ghosts exist
    assert (seen == 1).all()  # every atom owned exactly once
    assert np.abs(forces - f_ref.numpy()).max() < 1e-10 * np.abs(f_ref.numpy()).max()


def test_partition_bookkeeping():
    pos, species, box, _ = make_case()
    doms = [domain.partition_slabs(pos, species, box, 3, 5.0, r) for r in range(3)]
    assert sum(d.n_owned for d in doms) == pos.shape[0]
    for d in doms:
        # receivers are owned atoms, sorted; what I send up is what the upper neighbour holds as lower ghosts
        assert d.edge_index[0].max() < d.n_owned and (np.diff(d.edge_index[0]) >= 0).all()
        up = doms[d.up]
        assert len(d.send_up) == up.recv_down[1] and len(d.send_down) == doms[d.down].recv_up[1]
        ghost = up.positions[up.recv_down[0]: up.recv_down[0] + up.recv_down[1]] - up.ghost_shift[up.recv_down[0]: up.recv_down[0] + up.recv_down[1]]
        assert np.allclose(ghost, d.positions[d.send_up])
    with pytest.raises(ValueError):
        domain.partition_slabs(pos, species, box, 8, 5.0, 0)  # slabs thinner than the cutoff


def test_single_rank_is_plain_periodic():
    pos, species, box, _ = make_case()
    d = domain.partition_slabs(pos, species, box, 1, 5.0, 0)
    assert d.n_local == d.n_owned == pos.shape[0] and len(d.send_up) == 0


# ---- failure detection on the host (no GPU involved, nothing is made to fault) -------------------------------------
def _failing_worker(rank, world, port, out_dir, mode):
    import datetime
    import time

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    pos, species, box, params = make_case()
    dom = domain.partition_slabs(pos, species, box, world, 5.0, rank)
    outcome = "ok"
    t0 = time.time()
    try:
        if mode == "wrong_halo" and rank == 1:
            dom.recv_up = (dom.recv_up[0], dom.recv_up[1] + 3)     # this rank expects three rows too many
        plan = domain.HaloPlan(dom, "cpu")
        if mode == "wrong_halo":
            plan.verify()
        if mode == "rank_dies" and rank == 1:
            os._exit(3)                                            # leaves between steps, nothing in flight
        x = torch.from_numpy(dom.positions[: dom.n_owned])
        domain.halo_exchange(x, plan)
    except Exception as exc:  # noqa: BLE001 - the test records whatever the survivor sees
        outcome = type(exc).__name__ + ": " + str(exc)[:200]
    with open(os.path.join(out_dir, f"outcome{rank}.txt"), "w") as f:
        f.write(f"{time.time() - t0:.1f}\n{outcome}")
    os._exit(0)


def _run_failing(world, mode, tmp_path):
    ctx = mp.get_context("spawn")
    port = free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, str(tmp_path), mode)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
        assert not p.is_alive(), "a rank hung instead of ending with an error"
    return procs


def test_mismatched_halo_sizes_are_caught_on_the_host(tmp_path):
    """One rank expects a different ghost count than its neighbour sends: HaloPlan.verify() (run once per
    decomposition by the evaluator) raises on every rank before any exchange is posted."""
    _run_failing(2, "wrong_halo", tmp_path)
    for r in range(2):
        seconds, outcome = open(tmp_path / f"outcome{r}.txt").read().split("\n", 1)
        assert outcome.startswith("ValueError: halo plan mismatch"), outcome


def test_a_rank_that_leaves_ends_the_neighbours_exchange_with_an_error(tmp_path):
    """Rank 1 exits between steps; rank 0's next halo exchange ends with an exception within the process-group
    timeout instead of waiting forever."""
    procs = _run_failing(2, "rank_dies", tmp_path)
    assert procs[1].exitcode == 3
    seconds, outcome = open(tmp_path / "outcome0.txt").read().split("\n", 1)
    assert outcome != "ok" and float(seconds) < 60.0, outcome
