"""Spatial domain decomposition of the energy+force evaluation: one process per GPU, slabs along z.

The reference is single-GPU (no distributed code anywhere in cuda-mace); this module is new design.
Each rank owns the atoms of one slab and keeps ghost copies of the atoms within the cutoff beyond
its two faces.  Receivers are owned atoms only; senders are owned or ghost.  Per evaluation:

  1. ghost positions are filled from their owners (halo exchange, + the periodic shift);
  2. layer 0 needs no communication (its node features depend on the species only);
  3. layer-0 outputs of the boundary atoms are exchanged into the neighbours' ghost rows;
  4. layer 1 + readouts give the rank's partial energy; one scalar all-reduce sums the energies;
  5. backward: the halo exchange is an autograd function whose backward sends ghost-row gradients
     back to the owners and adds them, so forces on owned atoms include the contributions of their
     ghost copies on other ranks (reverse communication) without extra code.

Messages are small (about n_boundary x C scalars per face), sent with torch.distributed
point-to-point operations (NCCL over NVLink on GPUs, gloo on CPU).
"""
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from .systems import neighbor_list


@dataclass
class SlabDomain:
    rank: int
    nranks: int
    n_owned: int
    n_local: int                 # owned + ghosts; owned atoms come first
    owned_global: np.ndarray     # [n_owned] global atom ids
    positions: np.ndarray        # [n_local, 3] owned positions, ghost rows already shifted
    species: np.ndarray          # [n_local]
    ghost_shift: np.ndarray      # [n_local, 3] zero for owned rows
    edge_index: np.ndarray       # [2, E] local ids, row 0 receivers (owned, sorted), row 1 senders
    shifts: np.ndarray           # [E, 3]
    send_down: np.ndarray        # owned local ids sent to the lower neighbour (its upper ghosts)
    send_up: np.ndarray          # owned local ids sent to the upper neighbour (its lower ghosts)
    recv_down: tuple             # (start, count) ghost rows filled by the lower neighbour
    recv_up: tuple               # (start, count) ghost rows filled by the upper neighbour
    down: int                    # rank of the lower neighbour
    up: int                      # rank of the upper neighbour
    box: np.ndarray = None       # (3,) edge lengths of the whole periodic system
    pbc: tuple = (True, True, True)  # periodic axes of the local list: z is open once slabs carry ghost atoms


def partition_slabs(positions, species, box, nranks, r_cut, rank, group_species=True):
    """Splits a periodic orthorhombic system into `nranks` slabs along z with equal atom counts and
    returns the local view of `rank`.  Every rank computes this from the same global arrays.

    group_species: the owned atoms of a slab are stored grouped by species (`owned_global` maps local rows back to
    the caller's numbering, as it does for the slab order anyway).  The element-dependent operators then work on
    contiguous row ranges instead of gather lists."""
    positions = np.asarray(positions, dtype=np.float64)
    species = np.asarray(species)
    N = positions.shape[0]
    if nranks == 1:
        mine = np.argsort(species, kind="stable") if group_species else np.arange(N)
        positions, species = positions[mine], species[mine]
        ei, sh = neighbor_list(positions, box, (True, True, True), r_cut)
        zero = np.zeros(0, dtype=np.int64)
        return SlabDomain(0, 1, N, N, mine, positions, species, np.zeros_like(positions), ei, sh,
                          zero, zero, (N, 0), (N, 0), 0, 0, np.asarray(box, dtype=np.float64), (True, True, True))
    order = np.argsort(positions[:, 2], kind="stable")
    bounds = [(N * p) // nranks for p in range(nranks + 1)]
    zs = positions[order, 2]
    # slab p covers [cut[p], cut[p+1]); cut[0] = 0 and cut[P] = Lz close the periodic ring
    cut = np.array([0.0] + [0.5 * (zs[bounds[p] - 1] + zs[bounds[p]]) for p in range(1, nranks)] + [box[2]])
    if np.min(np.diff(cut)) < r_cut:
        raise ValueError("a slab is thinner than the cutoff; use fewer ranks or a longer box")
    owned = [order[bounds[p]:bounds[p + 1]] for p in range(nranks)]
    if group_species:
        owned = [o[np.argsort(species[o], kind="stable")] for o in owned]
    down, up = (rank - 1) % nranks, (rank + 1) % nranks

    def boundary(p, side):
        """owned atoms of rank p within r_cut of its lower ('lo') or upper ('hi') face, in owned order"""
        z = positions[owned[p], 2]
        m = (z < cut[p] + r_cut) if side == "lo" else (z >= cut[p + 1] - r_cut)
        return np.flatnonzero(m)

    mine = owned[rank]
    send_down = boundary(rank, "lo")
    send_up = boundary(rank, "hi")
    from_down = owned[down][boundary(down, "hi")]   # becomes my lower ghosts
    from_up = owned[up][boundary(up, "lo")]         # becomes my upper ghosts
    shift_down = np.zeros((from_down.shape[0], 3))
    shift_up = np.zeros((from_up.shape[0], 3))
    if rank == 0:
        shift_down[:, 2] = -box[2]
    if rank == nranks - 1:
        shift_up[:, 2] = box[2]
    n_owned = mine.shape[0]
    pos_local = np.concatenate([positions[mine], positions[from_down] + shift_down, positions[from_up] + shift_up])
    spec_local = np.concatenate([species[mine], species[from_down], species[from_up]])
    ghost_shift = np.concatenate([np.zeros((n_owned, 3)), shift_down, shift_up])
    ei, sh = neighbor_list(pos_local, box, (True, True, False), r_cut, n_receivers=n_owned)
    return SlabDomain(rank, nranks, n_owned, pos_local.shape[0], mine, pos_local, spec_local, ghost_shift, ei, sh,
                      send_down, send_up, (n_owned, from_down.shape[0]),
                      (n_owned + from_down.shape[0], from_up.shape[0]), down, up,
                      np.asarray(box, dtype=np.float64), (True, True, False))


class HaloPlan:
    """Device-side index lists of one SlabDomain, plus the process group to talk over."""

    def __init__(self, dom: SlabDomain, device, group=None):
        self.dom = dom
        self.group = group
        self.send_down = torch.as_tensor(dom.send_down, dtype=torch.long, device=device)
        self.send_up = torch.as_tensor(dom.send_up, dtype=torch.long, device=device)
        self.n_owned, self.n_local = dom.n_owned, dom.n_local
        self.device = torch.device(device)
        self._ghost_shift = {}

    def ghost_shift(self, dtype):
        """Shift vectors of the ghost rows on the device (copied once per dtype, not per step)."""
        if dtype not in self._ghost_shift:
            self._ghost_shift[dtype] = torch.as_tensor(self.dom.ghost_shift, dtype=dtype).to(self.device)
        return self._ghost_shift[dtype]

    def verify(self):
        """Host-side check, once per decomposition: every rank's send counts must equal what its neighbours expect
        to receive (a wrong halo size would otherwise surface as a truncated or hanging receive).  Collective over
        the group; raises ValueError on every rank when any pair disagrees."""
        d = self.dom
        if d.nranks == 1:
            return self
        mine = torch.tensor([self.send_down.numel(), self.send_up.numel(), d.recv_down[1], d.recv_up[1]],
                            dtype=torch.int64, device=self.device)
        every = [torch.zeros_like(mine) for _ in range(d.nranks)]
        dist.all_gather(every, mine, group=self.group)
        counts = torch.stack(every).cpu().tolist()
        bad = []
        for r in range(d.nranks):
            down, up = (r - 1) % d.nranks, (r + 1) % d.nranks
            if counts[r][1] != counts[up][2]:
                bad.append(f"rank {r} sends {counts[r][1]} rows up, rank {up} expects {counts[up][2]}")
            if counts[r][0] != counts[down][3]:
                bad.append(f"rank {r} sends {counts[r][0]} rows down, rank {down} expects {counts[down][3]}")
        if bad:
            raise ValueError("halo plan mismatch: " + "; ".join(bad))
        return self

    def _exchange(self, out_down, out_up, in_from_down, in_from_up):
        """Sends out_down / out_up to the lower / upper neighbour and receives their counterparts.
        Both neighbours may be the same rank (two ranks): messages are matched by posting order, the
        upward message first, and by tag where the backend supports tags."""
        d = self.dom
        ops = [
            dist.P2POp(dist.isend, out_up, d.up, self.group, tag=1),
            dist.P2POp(dist.isend, out_down, d.down, self.group, tag=2),
            dist.P2POp(dist.irecv, in_from_down, d.down, self.group, tag=1),
            dist.P2POp(dist.irecv, in_from_up, d.up, self.group, tag=2),
        ]
        for req in dist.batch_isend_irecv(ops):
            req.wait()

    def forward_fill(self, x_owned):
        """[n_owned, F] -> [n_local, F] with ghost rows received from their owners."""
        d = self.dom
        F = x_owned.shape[1:]
        from_down = x_owned.new_empty((d.recv_down[1],) + tuple(F))
        from_up = x_owned.new_empty((d.recv_up[1],) + tuple(F))
        if d.nranks > 1:
            self._exchange(x_owned.index_select(0, self.send_down).contiguous(),
                           x_owned.index_select(0, self.send_up).contiguous(), from_down, from_up)
        return torch.cat([x_owned, from_down, from_up], dim=0)

    def backward_reduce(self, g_local):
        """[n_local, F] gradient -> [n_owned, F]: ghost-row gradients go back to the owners and are added."""
        d = self.dom
        g_owned = g_local[: d.n_owned].clone()
        if d.nranks > 1:
            g_down = g_local[d.recv_down[0]: d.recv_down[0] + d.recv_down[1]].contiguous()
            g_up = g_local[d.recv_up[0]: d.recv_up[0] + d.recv_up[1]].contiguous()
            back_down = g_local.new_empty((self.send_down.numel(),) + tuple(g_local.shape[1:]))
            back_up = g_local.new_empty((self.send_up.numel(),) + tuple(g_local.shape[1:]))
            # my lower ghosts belong to the lower neighbour: their gradients travel downward, and the
            # gradients of the rows I sent upward come back from the upper neighbour
            self._exchange(g_down, g_up, back_down, back_up)
            g_owned.index_add_(0, self.send_down, back_down)
            g_owned.index_add_(0, self.send_up, back_up)
        return g_owned


class _HaloFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_owned, plan):
        ctx.plan = plan
        return plan.forward_fill(x_owned)

    @staticmethod
    def backward(ctx, g):
        return ctx.plan.backward_reduce(g.contiguous()), None


def halo_exchange(x_owned, plan):
    """Differentiable owner -> ghost copy: forward fills ghost rows, backward adds ghost gradients
    into the owners' rows."""
    return _HaloFunction.apply(x_owned, plan)


def distributed_energy_forces(node_energy_fn, dom: SlabDomain, plan: HaloPlan, positions_owned, dtype_pos=None):
    """Energy and forces of the whole system from this rank's slab.

    node_energy_fn(positions_local, exchange) must return the per-node interaction energies of the
    owned atoms [n_owned], calling exchange(h_owned) -> h_local before the second interaction.
    Returns (total interaction energy summed over ranks, forces on owned atoms [n_owned, 3])."""
    pos = positions_owned.detach().requires_grad_(True)
    pos_local = halo_exchange(pos, plan) + plan.ghost_shift(pos.dtype)
    e_nodes = node_energy_fn(pos_local, lambda h: halo_exchange(h, plan))
    e_local = e_nodes.sum()
    (g,) = torch.autograd.grad(e_local, pos)
    e_total = e_local.detach().clone()
    if dom.nranks > 1:
        dist.all_reduce(e_total, group=plan.group)
    return e_total, -g
