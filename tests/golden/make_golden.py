"""Generates tests/golden/*.npz from the float64 CPU restatement in oracle/.

    python tests/golden/make_golden.py

The reference project holds no golden vectors (its tests compare against live mace/e3nn installs),
so these fixtures freeze the restatement's outputs on small seeded inputs: any later change of the
oracle, of the U tensors or of the parameter generator shows up as a fixture mismatch.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from cuda_mace_b200 import cg, systems  # noqa: E402
from oracle import model as omodel  # noqa: E402
from oracle import ops as oops  # noqa: E402
from oracle.sh import real_sh_l3  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def small_graph(seed, n_nodes, mean_degree):
    g = torch.Generator().manual_seed(seed)
    deg = torch.poisson(torch.full((n_nodes,), float(mean_degree)), generator=g).long()
    recv = torch.repeat_interleave(torch.arange(n_nodes), deg)
    send = torch.randint(0, n_nodes, (int(deg.sum()),), generator=g)
    return send, recv


def main():
    U = cg.u_matrices()
    g = torch.Generator().manual_seed(1234)
    f8 = dict(generator=g, dtype=torch.float64)

    # operators on a 12-node graph, 32 channels
    N, C, Z = 12, 32, 3
    send, recv = small_graph(7, N, 4)
    E = send.numel()
    X = torch.randn(N, C, **f8)
    vec = torch.randn(E, 3, **f8)
    Y = real_sh_l3(vec)
    R = torch.randn(E, 4, C, **f8)
    imp = oops.invariant_message_passing(X, Y, R, send, recv, N)
    M = torch.randn(N, 16, C, **f8)
    W = torch.randn(4, C, C, **f8)
    WZ = torch.randn(Z, 4, C, C, **f8)
    at = torch.randint(0, Z, (N,), generator=g)
    W3, W2, W1 = torch.randn(Z, 23, C, **f8), torch.randn(Z, 4, C, **f8), torch.randn(Z, 1, C, **f8)
    con = oops.symmetric_contraction(M, at, *U, W3, W2, W1)
    np.savez_compressed(
        os.path.join(HERE, "ops_small.npz"),
        send=send.numpy(), recv=recv.numpy(), X=X.numpy(), vec=vec.numpy(), Y=Y.numpy(), R=R.numpy(),
        imp=imp.numpy(), M=M.numpy(), W=W.numpy(), WZ=WZ.numpy(), at=at.numpy(),
        lin=oops.linear(M, W).numpy(), elin=oops.elemental_linear(M, WZ, systems.one_hot(at, Z)).numpy(),
        W3=W3.numpy(), W2=W2.numpy(), W1=W1.numpy(), con=con.numpy(),
        bessel=omodel.radial_embedding(vec.norm(dim=-1), 5.0).numpy(),
    )

    # whole model: the 192-atom configuration (C=64, 4 species, seed 0), energy + forces
    s = systems.make_system("cfg0")
    ei, sh = systems.neighbor_list(s["positions"], s["box"], (True, True, True), 5.0)
    params = systems.init_params(s["channels"], s["n_species"], 0)
    e, e_inter, f = omodel.energy_and_forces(params, U, torch.from_numpy(s["positions"]),
                                             systems.one_hot(s["species"], 4), torch.from_numpy(ei),
                                             torch.from_numpy(sh))
    np.savez_compressed(os.path.join(HERE, "cfg0_energy_forces.npz"), energy=e.numpy(), interaction=e_inter.numpy(),
                        forces=f.numpy(), n_edges=np.array(ei.shape[1]))
    print("wrote fixtures:", E, "edges;", ei.shape[1], "edges in cfg0; E =", float(e))

    # whole model at full size: the 3 000-atom H/O box (C=128, seed 1), energy + forces (about a minute of CPU)
    s = systems.make_system("water3000")
    ei, sh = systems.neighbor_list(s["positions"], s["box"], (True, True, True), 5.0)
    params = systems.init_params(s["channels"], s["n_species"], 1)
    e, e_inter, f = omodel.energy_and_forces(params, U, torch.from_numpy(s["positions"]),
                                             systems.one_hot(s["species"], 2), torch.from_numpy(ei),
                                             torch.from_numpy(sh))
    np.savez_compressed(os.path.join(HERE, "water3000_energy_forces.npz"), energy=e.numpy(),
                        interaction=e_inter.numpy(), forces=f.numpy(), n_edges=np.array(ei.shape[1]))
    print("wrote water3000 fixture:", ei.shape[1], "edges; E_inter =", float(e_inter))


if __name__ == "__main__":
    main()
