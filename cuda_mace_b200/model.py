"""Energy+force evaluation of an invariant MACE model on the CUDA operators.

Mirror of cuda_mace/models/InvariantMACE.py (``OptimizedInvariantMACE``): same data dictionary in,
same output dictionary out, same operator sequence (:246-379).  The reference transplants the
weights of an upstream ``mace`` model object; upstream is not a dependency here, so the model is
built from a plain parameter dictionary (see ``cuda_mace_b200.systems.init_params`` for the
layout), whose tensors play the roles of the upstream sub-modules the reference deep-copies
(node_embedding, radial_embedding, conv_tp_weights, linear_up, linear, skip_tp, products,
readouts, scale_shift: InvariantMACE.py:77-88, :124-134, :184-244).

Differences from the reference, all required by the float64 1e-10 target:
  * the radial weights are computed exactly (Bessel x cutoff in the edge kernel, then the radial
    multilayer perceptron) instead of through a 256-knot cubic spline; ``radial="spline"`` selects
    the reference's tabulated path;
  * the whole model runs in the dtype it is built with (float32 or float64); readouts, scale-shift
    and the energy sum are float64 in both cases, as in the reference (:196, :330-347).
"""
import math

import torch

from . import ops

SILU_2MOM = 1.676532470331092  # 1/sqrt(E[silu(x)^2]), x ~ N(0,1)


def _silu_n(x):
    return torch.nn.functional.silu(x) * SILU_2MOM


def add_spline_knots(params, nknots=256):
    """Adds the knot grid of the tabulated radial path to every layer's parameters: nknots equidistant knots on
    [1e-12, r_max + 1] (cuda_mace/models/InvariantMACE.py:226-240).  The table itself is computed by the model."""
    r_max = float(params["r_max"])
    r = torch.linspace(1e-12, r_max + 1.0, nknots, dtype=torch.float64)
    for P in params["layers"]:
        P["spline_knots"] = r
        P["spline_h"] = float(r[1] - r[0])
    return params


class _SelectElementBlock(torch.autograd.Function):
    """big [N, Z*C] -> out[n] = big[n, z_n*C:(z_n+1)*C].  With big = h @ [W_0 | W_1 | ...] this is the element-dependent
    product h[n] @ W[z_n] as ONE dense product plus a row-wise selection (instead of one masked product per
    element); the backward scatters the gradient into the selected block of an otherwise zero [N, Z*C] array."""

    @staticmethod
    def forward(ctx, big, z, C):
        N = z.shape[0]
        ctx.save_for_backward(z)
        ctx.width = big.shape[1]
        return big.view(N, ctx.width // C, C)[torch.arange(N, device=big.device), z]

    @staticmethod
    def backward(ctx, g):
        (z,) = ctx.saved_tensors
        N, C = g.shape
        out = torch.zeros(N, ctx.width // C, C, dtype=g.dtype, device=g.device)
        out[torch.arange(N, device=g.device), z] = g
        return out.view(N, ctx.width), None, None


class InvariantMACE(torch.nn.Module):
    def __init__(self, params, U, dtype=torch.float32, device="cuda", radial="exact"):
        super().__init__()
        if radial not in ("exact", "spline"):
            raise ValueError(radial)
        self.radial = radial
        self.dtype = dtype
        self.r_max = float(params["r_max"])
        W_embed = params["W_embed"]
        Z, C = W_embed.shape
        self.num_elements, self.channels = Z, C
        dd = dict(dtype=dtype, device=device)
        d64 = dict(dtype=torch.float64, device=device)
        self.register_buffer("atomic_energies", params["atomic_energies"].to(**d64))
        self.register_buffer("embedding", (W_embed / math.sqrt(Z)).to(**dd))
        self.edge_basis = ops.EdgeBasis(self.r_max, params["layers"][0]["W_radial"][0].shape[0], 5)
        self.spherical_harmonics = ops.SphericalHarmonics()
        self.tp = ops.InvariantMessagePassingTP()
        self.scale, self.shift = float(params["scale"]), float(params["shift"])
        U3, U2, U1 = U
        self.layers = torch.nn.ModuleList()
        for t, P in enumerate(params["layers"]):
            L = torch.nn.Module()
            L.register_buffer("W_up", (P["W_up"] / math.sqrt(C)).to(**dd))
            L.register_buffer("W_up_T", L.W_up.t().contiguous())
            for i, W in enumerate(P["W_radial"]):
                # 1/sqrt(fan_in) of e3nn's FullyConnectedNet; the second-moment constant of the activation
                # that feeds layers 1.. is folded in as well, so the activation itself is a plain SiLU
                Wn = (W / math.sqrt(W.shape[0]) * (SILU_2MOM if i > 0 else 1.0)).to(**dd)
                L.register_buffer(f"W_radial{i}", Wn)
                L.register_buffer(f"W_radial{i}_T", Wn.t().contiguous())
            L.n_radial = len(P["W_radial"])
            if t == 0:
                # linear followed by skip_tp is one element-dependent map per l: the constant weights are multiplied
                # once, in float64, instead of running two channel-mixing passes over [N,16,C] every step.  Each of
                # the two operators divides by sqrt(fan_in); the fused one does so once, hence the factor here.
                W_lin = P["W_lin"].double() / (float(P["avg_num_neighbors"]) * math.sqrt(P["W_lin"].shape[1]))
                W_skip = P["W_skip"].double() / math.sqrt(Z)
                L.linear = ops.ElementalLinear(torch.einsum("lab,zlbc->zlac", W_lin, W_skip).to(**dd))
                L.register_buffer("W_readout", (P["W_readout"] / math.sqrt(C)).to(**d64))
                L.register_buffer("W_readout_T", L.W_readout.t().contiguous())
            else:
                L.linear = ops.Linear(P["W_lin"].to(**dd), scale=1.0 / float(P["avg_num_neighbors"]))
                # W_sc [C, Z, C]: as one [C, Z*C] matrix, column block z is the matrix of element z
                L.register_buffer("W_sc", (P["W_sc"] / math.sqrt(C * Z)).reshape(C, Z * C).contiguous().to(**dd))
                L.register_buffer("W_sc_T", L.W_sc.t().contiguous())
                L.register_buffer("W_readout1", (P["W_readout1"] / math.sqrt(C)).to(**d64))
                L.register_buffer("W_readout2", (P["W_readout2"] / math.sqrt(P["W_readout2"].shape[0])).to(**d64))
                L.register_buffer("W_readout1_T", L.W_readout1.t().contiguous())
                L.register_buffer("W_readout2_T", L.W_readout2.t().contiguous())
            L.contraction = ops.SymmetricContraction(U3, U2, U1, P["W3"].to(dtype), P["W2"].to(dtype),
                                                     P["W1"].to(dtype)).to(device)
            L.register_buffer("W_prod", (P["W_prod"] / math.sqrt(C)).to(**dd))
            L.register_buffer("W_prod_T", L.W_prod.t().contiguous())
            if radial == "spline":
                L.spline = ops.CubicSpline(P["spline_knots"].to(**dd), self._tabulate(P).to(**dd),
                                           float(P["spline_h"]), self.r_max)
            self.layers.append(L)

    def _tabulate(self, P):
        """Radial weights at the spline knots, float64 on the host (InvariantMACE.py:226-240)."""
        r = P["spline_knots"].to(torch.float64).cpu()
        n = torch.arange(1, P["W_radial"][0].shape[0] + 1, dtype=torch.float64)
        x = r / self.r_max
        env = (1.0 - 21.0 * x**5 + 35.0 * x**6 - 15.0 * x**7) * (x < 1.0)
        h = math.sqrt(2.0 / self.r_max) * torch.sin(n * math.pi / self.r_max * r[:, None]) / r[:, None] * env[:, None]
        for i, W in enumerate(P["W_radial"]):
            h = h @ W.to(torch.float64) / math.sqrt(W.shape[0])
            if i + 1 < len(P["W_radial"]):
                h = _silu_n(h)
        return h

    def _radial_weights(self, L, bessel, lengths):
        if self.radial == "spline":
            return L.spline(lengths)
        Ws = [getattr(L, f"W_radial{i}") for i in range(L.n_radial)]
        on_tc = all(ops.tensor_core_ok(bessel.dtype, W.shape[0], W.shape[1]) for W in Ws)
        h = bessel
        if on_tc and ops.radial_hidden_ok(bessel.dtype, Ws[:-1]):
            # all hidden layers and their activations in one kernel, then the last, linear layer
            h = ops.radial_hidden(bessel, Ws[:-1], [getattr(L, f"W_radial{i}_T") for i in range(L.n_radial - 1)])
            return ops.matmul3x(h, Ws[-1], getattr(L, f"W_radial{L.n_radial - 1}_T"))
        for i, W in enumerate(Ws):
            h = self._mm(h, W, getattr(L, f"W_radial{i}_T"))
            if i + 1 < L.n_radial:
                h = torch.nn.functional.silu(h)
        return h

    def _messages(self, L, up, Y, bessel, lengths, send, recv, n_owned, topology):
        """Radial weights and message passing of one interaction; in float32 with the standard perceptron the
        hidden layers run in one kernel and the last layer inside the message-passing kernel."""
        C = self.channels
        Ws = [getattr(L, f"W_radial{i}") for i in range(L.n_radial)]
        if (self.radial == "exact" and ops.radial_hidden_ok(up.dtype, Ws[:-1])
                and ops.FUSED_RADIAL_MESSAGE_PASSING and ops.fused_radial_ok(up.dtype, C, Ws[-1].shape[0])
                and all(ops.tensor_core_ok(up.dtype, W.shape[0], W.shape[1]) for W in Ws)):
            hidden = ops.radial_hidden(bessel, Ws[:-1], [getattr(L, f"W_radial{i}_T") for i in range(L.n_radial - 1)])
            return ops.fused_radial_message_passing(up, Y, hidden, Ws[-1], getattr(L, f"W_radial{L.n_radial - 1}_T"),
                                                    topology)
        if (self.radial == "exact" and ops.RADIAL_GRADIENT_ON_THE_FLY and ops.radial_hidden_ok(up.dtype, Ws[:-1])
                and ops.radial_message_passing_ok(up.dtype, C, Ws[-1].shape[0])
                and all(ops.tensor_core_ok(up.dtype, W.shape[0], W.shape[1]) for W in Ws)):
            # float32 default: hidden layers in one kernel; last layer as a product whose gradient array is never
            # written (the backward forms the radial-weight gradient inside the tensor-core kernel that consumes it)
            hidden = ops.radial_hidden(bessel, Ws[:-1], [getattr(L, f"W_radial{i}_T") for i in range(L.n_radial - 1)])
            return ops.radial_message_passing(up, Y, hidden, Ws[-1], getattr(L, f"W_radial{L.n_radial - 1}_T"), topology)
        R = self._radial_weights(L, bessel, lengths).view(-1, 4, C)
        return self.tp(up, Y, R, send, recv, n_owned, topology=topology)

    def node_energies(self, positions, species, edge_index, shifts, topology=None, exchange=None, n_owned=None):
        """Interaction energy per receiving node [n_owned] (float64); differentiable with respect to
        positions.

        positions [N,3]; species [N] integer element index; edge_index [2,E] (row 0 receivers, sorted;
        row 1 senders); shifts [E,3].  With a domain decomposition only the first `n_owned` rows
        receive, the rest are ghost atoms that only send; `exchange(h_owned) -> h_local` then refreshes
        the ghost rows of the node features before the second interaction."""
        C = self.channels
        recv, send = edge_index[0], edge_index[1]
        N = positions.shape[0]
        n_owned = N if n_owned is None else int(n_owned)
        if topology is None:
            topology = ops.topology_for(send, recv, n_owned, N)
        if positions.is_cuda and positions.dtype == torch.float64 and shifts.dtype == torch.float64:
            # one kernel forward; one kernel for the whole position gradient in the backward (no atomics)
            vectors = ops.edge_vectors(positions, shifts, topology, self.dtype)
        else:
            vectors = positions.index_select(0, send.long()) - positions.index_select(0, recv.long()) + shifts
            vectors = vectors.to(self.dtype)
        if self.radial == "exact":
            Y, bessel = self.edge_basis(vectors)
            lengths = None
        else:
            Y = self.spherical_harmonics(vectors)
            bessel, lengths = None, vectors.norm(dim=-1)
        species = species.to(torch.int32)
        species_owned = species[:n_owned] if n_owned != N else species
        h = self.embedding.index_select(0, species.long())
        es = []
        for t, L in enumerate(self.layers):
            sc = None
            if t == 1:
                # FullyConnectedTensorProduct(h, one_hot): sc[n] = h[n] @ W_sc[z_n]
                sc = _SelectElementBlock.apply(self._mm(h, L.W_sc, L.W_sc_T), species_owned.long(), C)
                if exchange is not None:
                    h = exchange(h)
            up = self._mm(h, L.W_up, L.W_up_T)
            m = self._messages(L, up, Y, bessel, lengths, send, recv, n_owned, topology)
            m = L.linear(m, species_owned) if t == 0 else L.linear(m)
            b = L.contraction(m, species_owned)[:, 0, :]
            h = self._mm(b, L.W_prod, L.W_prod_T)
            if sc is not None:
                h = h + sc
            h64 = h.double()
            if t == 0:
                es.append(self._mm(h64, L.W_readout, L.W_readout_T)[:, 0])
            else:
                hid = _silu_n(self._mm(h64, L.W_readout1, L.W_readout1_T))
                es.append(self._mm(hid, L.W_readout2, L.W_readout2_T)[:, 0])
        return self.scale * (es[0] + es[1]) + self.shift

    @staticmethod
    def _mm(x, W, W_T):
        """x @ W for a constant weight on this library's kernels: tcgen05 with a 3-term TF32 split in float32, the
        FP64 tensor cores (DMMA) in float64; torch.matmul only for float32 shapes the tensor-core kernel does not
        take and for CPU tensors (the oracle-side domain tests)."""
        if ops.tensor_core_ok(x.dtype, W.shape[0], W.shape[1]):
            return ops.matmul3x(x, W, W_T)
        if x.is_cuda and x.dtype == torch.float64:
            return ops.matmul_f64(x, W, W_T)
        return x @ W

    def forward(self, data, training=False, compute_force=True, topology=None):
        """data: positions [N,3], node_attrs [N,Z] one-hot (or species [N]), edge_index [2,E], shifts [E,3].
        Returns energy (float64 scalar tensor), node_energy, interaction_energy, forces [N,3]."""
        positions = data["positions"]
        if compute_force:
            positions = positions.detach().requires_grad_(True)
        species = data["species"] if "species" in data else data["node_attrs"].argmax(dim=-1)
        node_inter = self.node_energies(positions, species, data["edge_index"], data["shifts"], topology=topology)
        inter_e = node_inter.sum()
        node_e0 = self.atomic_energies.index_select(0, species.long())
        forces = None
        if compute_force:
            (g,) = torch.autograd.grad(inter_e, positions, create_graph=training)
            forces = -g
        return {
            "energy": node_e0.sum() + inter_e.detach(),
            "node_energy": node_e0 + node_inter.detach(),
            "interaction_energy": inter_e.detach(),
            "forces": forces,
        }
