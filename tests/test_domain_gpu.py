"""Two-rank slab decomposition on two GPUs (NCCL): energy and forces equal the single-GPU periodic
evaluation.  Skipped when fewer than two devices are visible.  Ranks are child processes that leave
only after the step has finished; NVLS is switched off for the children."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def case():
    from cuda_mace_b200 import systems

    box = np.array([22.0, 22.0, 40.0])
    pos = systems.random_box(1800, box, 0.9, seed=3)
    rng = np.random.default_rng(3)
    species = rng.integers(0, 4, pos.shape[0])
    params = systems.init_params(64, 4, 8)
    return pos, species, box, params


def worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from cuda_mace_b200 import cg, domain, evaluator, model, ops

        pos, species, box, params = case()
        dom = domain.partition_slabs(pos, species, box, world, 5.0, rank)
        net = model.InvariantMACE(params, cg.u_matrices(), dtype=torch.float64, device=f"cuda:{rank}")
        ev = evaluator.EnergyForceEvaluator(net, dom, f"cuda:{rank}")
        p = ev.load_domain()
        e, f = ev(p)
        ops.check_status()
        # second pass with the neighbour list of the slab (owned + ghost atoms, open z axis) rebuilt on the device
        n_edges = ev.edge_index.shape[1]
        ev.rebuild_neighbor_list(p)
        assert ev.edge_index.shape[1] == n_edges
        e2, f2 = ev(p)
        assert abs(float(e2) - float(e)) < 1e-11 * abs(float(e))
        assert float((f2 - f).abs().max()) < 1e-10 * float(f.abs().max())
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), e=e.cpu().numpy(), f=f.cpu().numpy(), ids=dom.owned_global)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_slabs_equal_single_gpu(tmp_path):
    from cuda_mace_b200 import cg, model, systems

    pos, species, box, params = case()
    ei, sh = systems.neighbor_list(pos, box, (True, True, True), 5.0)
    net = model.InvariantMACE(params, cg.u_matrices(), dtype=torch.float64, device="cuda:0")
    ref = net(dict(positions=torch.from_numpy(pos).cuda(), species=torch.from_numpy(species).to(torch.int32).cuda(),
                   edge_index=torch.from_numpy(ei).to(torch.int32).cuda(), shifts=torch.from_numpy(sh).cuda()))
    mp.spawn(worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    forces = np.zeros_like(pos)
    for r in range(2):
        z = np.load(tmp_path / f"rank{r}.npz")
        assert abs(float(z["e"]) - float(ref["interaction_energy"])) < 1e-10 * abs(float(ref["interaction_energy"]))
        forces[z["ids"]] = z["f"]
    fr = ref["forces"].cpu().numpy()
    assert np.abs(forces - fr).max() < 1e-10 * np.abs(fr).max()
