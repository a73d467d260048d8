"""Energy+force evaluation of one slab (or of the whole periodic box on a single GPU): the call a
user of the package makes per step.

    ev = EnergyForceEvaluator(model, domain, device, group)
    energy, forces = ev(positions_owned)            # tensors already on the device
    energy, forces = ev.evaluate_host(host_batch)   # pinned host buffers in, host results out

`evaluate_host` moves the step's inputs (positions, species, edge list, shifts) to the device,
rebuilds the edge topology for the list it was given, runs the model and copies energy and forces
back, so it is the end-to-end path including every host<->device byte.  The shift vectors of a periodic
neighbour list take only a handful of distinct values (lattice translations), so the host batch carries
them as a small table plus one byte per edge instead of three float64 per edge.
"""
import torch

from . import domain as _domain
from . import ops


class EnergyForceEvaluator:
    def __init__(self, model, dom, device, group=None):
        self.model = model
        self.dom = dom
        self.device = torch.device(device)
        self.plan = _domain.HaloPlan(dom, self.device, group).verify()
        self.species = None
        self.edge_index = None
        self.shifts = None
        self.topology = None
        self._graph = None

    def set_neighbor_list(self, species, edge_index, shifts):
        """Device tensors: species [n_local] int32, edge_index [2,E] int32 (receivers sorted), shifts [E,3]."""
        self.species = species
        self.edge_index = edge_index
        self.shifts = shifts
        self.topology = ops.EdgeTopology(edge_index[1], edge_index[0], self.dom.n_owned, self.dom.n_local)
        self._graph = None   # a captured step belongs to the list it was captured with
        return self

    def rebuild_neighbor_list(self, positions_owned, r_cut=None):
        """Builds the neighbour list of the current positions on the device (cell-list kernels) instead of taking
        it from the host: ghost positions come from the neighbouring slabs, receivers are the owned atoms, the
        slab's z axis is open once it carries ghosts.  One host synchronisation (edge count)."""
        d = self.dom
        if d.box is None:
            raise RuntimeError("the domain does not carry its box")
        r_cut = float(self.model.r_max if r_cut is None else r_cut)
        with torch.no_grad():
            pos_local = _domain.halo_exchange(positions_owned.detach(), self.plan) + self.plan.ghost_shift(positions_owned.dtype)
        lo, ext = [0.0, 0.0, 0.0], [float(v) for v in d.box]
        for ax in range(3):
            if not d.pbc[ax]:
                zmin, zmax = float(pos_local[:, ax].min()), float(pos_local[:, ax].max())
                lo[ax], ext[ax] = zmin, max(zmax - zmin, 1e-6) * (1 + 1e-12) + 1e-9
        edge_index, shifts, _ = ops.neighbor_list(pos_local, ext, d.pbc, r_cut, d.n_owned, lo=lo)
        if self.species is None:
            self.species = torch.as_tensor(d.species, dtype=torch.int32, device=self.device)
        return self.set_neighbor_list(self.species, edge_index, shifts.to(positions_owned.dtype))

    def load_domain(self, pos_dtype=torch.float64):
        d = self.dom
        dev = self.device
        self.set_neighbor_list(torch.as_tensor(d.species, dtype=torch.int32, device=dev),
                               torch.as_tensor(d.edge_index, dtype=torch.int32, device=dev),
                               torch.as_tensor(d.shifts, dtype=pos_dtype, device=dev))
        return torch.as_tensor(d.positions[: d.n_owned], dtype=pos_dtype, device=dev)

    def capture(self, positions_owned):
        """Records the whole energy+force step for the current neighbour list as a CUDA graph; later calls copy
        the positions into the graph's input and replay it, which removes the per-launch cost that dominates
        small systems (about a hundred launches per step).  Single-rank domains only: the halo exchange of a
        multi-rank step is host-driven.  A new neighbour list drops the recording."""
        if self.dom.nranks != 1:
            raise RuntimeError("capture() needs a single-rank domain")
        self._graph = None
        static_pos = positions_owned.detach().clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):      # warm-up outside the recording: weight packing, caches, allocator pools
                self(static_pos)
        torch.cuda.current_stream(self.device).wait_stream(side)
        ops.check_status()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            energy, forces = self(static_pos)
        self._graph = (graph, static_pos, energy, forces)
        return self

    def __call__(self, positions_owned):
        if self._graph is not None and not torch.cuda.is_current_stream_capturing():
            graph, static_pos, energy, forces = self._graph
            static_pos.copy_(positions_owned)
            graph.replay()
            return energy.clone(), forces.clone()

        def node_energy(pos_local, exchange):
            return self.model.node_energies(pos_local, self.species, self.edge_index, self.shifts,
                                            topology=self.topology, exchange=exchange, n_owned=self.dom.n_owned)

        return _domain.distributed_energy_forces(node_energy, self.dom, self.plan, positions_owned)

    # ---- end-to-end path with host buffers ----------------------------------------------------
    def host_batch(self, pos_dtype=torch.float64):
        """Pinned host copies of one step's inputs, as a data loader would hand them over."""
        import numpy as np

        d = self.dom
        pin = lambda t: t.pin_memory() if torch.cuda.is_available() else t
        batch = {
            "positions": pin(torch.as_tensor(d.positions[: d.n_owned], dtype=pos_dtype)),
            "species": pin(torch.as_tensor(d.species, dtype=torch.int32)),
            "edge_index": pin(torch.as_tensor(d.edge_index, dtype=torch.int32)),
        }
        table, index = np.unique(np.asarray(d.shifts), axis=0, return_inverse=True)
        if table.shape[0] <= 256:
            batch["shift_table"] = pin(torch.as_tensor(table, dtype=pos_dtype))
            batch["shift_index"] = pin(torch.as_tensor(index.reshape(-1).astype(np.uint8)))
        else:  # not a lattice-translation list: ship the vectors themselves
            batch["shifts"] = pin(torch.as_tensor(d.shifts, dtype=pos_dtype))
        return batch

    @staticmethod
    def h2d_bytes(batch):
        return int(sum(t.numel() * t.element_size() for t in batch.values()))

    def evaluate_host(self, batch, out_forces=None):
        dev = self.device
        moved = {k: v.to(dev, non_blocking=True) for k, v in batch.items()}
        shifts = moved["shifts"] if "shifts" in moved else \
            moved["shift_table"].index_select(0, moved["shift_index"].to(torch.int64))
        self.set_neighbor_list(moved["species"], moved["edge_index"], shifts)
        energy, forces = self(moved["positions"])
        if out_forces is None:
            out_forces = torch.empty(forces.shape, dtype=forces.dtype, pin_memory=torch.cuda.is_available())
        out_forces.copy_(forces, non_blocking=True)
        e = float(energy.cpu())  # synchronises
        ops.check_status()
        return e, out_forces
