"""The reference's energy+force step re-assembled from the reference's OWN operator classes (loaded from
oracle/_ref/libcuda_mace.so) plus torch for the parts it borrows from upstream MACE.  BASELINE AND TEST
INFRASTRUCTURE ONLY; it needs a CUDA device and must run in a process that has not loaded this project's
TorchScript classes (both register the same class names).

cuda_mace/models/InvariantMACE.py itself cannot be imported here (it imports mace, e3nn and ase at module level),
so its forward (:246-379) and its two interaction blocks (:77-165) are followed operator by operator on a plain
parameter dictionary (`cuda_mace_b200.systems.init_params` layout):
  node_attrs.requires_grad_(True) (:257)          so that layer 0's X requires grad, which the reference's message
                                                   passing backward insists on (invariant_message_passing_wrapper.cpp:171-177)
  vectors.float() -> SphericalHarmonics (:303-306)
  per layer: spline(lengths.float()) (:320), linear_up as matmul / sqrt(C) (:41-53), message passing with
  receiver = edge_index[0], sender = edge_index[1] (:99-112), Linear / avg_num_neighbors (:114), ElementalLinear in
  layer 0 (:116) or the upstream skip product in layer 1 (:149), contraction on argmax(one-hot).int() (:35-38),
  product linear + sc (:223-224), float64 readouts (:330-337), scale-shift, sum, autograd forces (:341-364).
The spline tables are 256 knots on [1e-12, r_max + 1] (:226-240); float32 everywhere except the readouts.
"""
import math

import torch

from . import model as omodel
from . import ops as oops
from . import ref_cases


class ReferenceStep:
    def __init__(self, params, U, classes, device="cuda"):
        self.c = classes
        f32 = dict(dtype=torch.float32, device=device)
        f64 = dict(dtype=torch.float64, device=device)
        Z, C = params["W_embed"].shape
        ref_cases.check_channels(C)
        self.Z, self.C, self.r_max = Z, C, float(params["r_max"])
        self.embed = (params["W_embed"] / math.sqrt(Z)).to(**f64)
        self.scale, self.shift = float(params["scale"]), float(params["shift"])
        self.sh = classes.spherical_harmonics.SphericalHarmonics()
        tables = oops.pack_sparse_u(*U)
        self.u3_max = tables[0]
        self.tables = [t.to(device) for t in tables[1:]]
        omodel.add_spline_tables(params)
        self.layers = []
        for t, P in enumerate(params["layers"]):
            L = dict(
                W_up=(P["W_up"] / math.sqrt(C)).to(**f32),
                knots=P["spline_knots"].to(**f32), coeffs=P["spline_coeffs"].to(**f32).contiguous(),
                h=float(P["spline_h"]),
                W_lin=P["W_lin"].to(**f32).contiguous(),
                avg=float(P["avg_num_neighbors"]),
                W3=P["W3"].to(**f32)[None].contiguous(), W2=P["W2"].to(**f32)[None].contiguous(),
                W1=P["W1"].to(**f32)[None].contiguous(),
                W_prod=(P["W_prod"] / math.sqrt(C)).to(**f32),
                spline=classes.cubic_spline.CubicSpline(), tp=classes.inv_message_passing.InvariantMessagePassingTP(),
                linear=classes.linear_wmma.Linear(), contraction=classes.symm_contract.SymmetricContraction(),
            )
            L["W_lin_T"] = L["W_lin"].transpose(-1, -2).contiguous()
            ref_cases.check_spline(torch.tensor([0.0]), L["knots"].shape[0], L["coeffs"].shape[0], L["h"], self.r_max)
            if t == 0:
                L["W_skip"] = (P["W_skip"] / math.sqrt(Z)).to(**f32).contiguous()
                L["W_skip_T"] = L["W_skip"].transpose(-1, -2).contiguous()
                L["skip"] = classes.linear_wmma.ElementalLinear()
                L["W_readout"] = (P["W_readout"] / math.sqrt(C)).to(**f64)
            else:
                L["W_sc"] = (P["W_sc"] / math.sqrt(C * Z)).to(**f32)
                L["W_readout1"] = (P["W_readout1"] / math.sqrt(C)).to(**f64)
                L["W_readout2"] = (P["W_readout2"] / math.sqrt(P["W_readout2"].shape[0])).to(**f64)
            self.layers.append(L)

    def check_inputs(self, positions, edge_index, shifts):
        """Host-side guard: the same rules as oracle.ref_cases.check_graph, plus distances inside the table."""
        ref_cases.check_graph(edge_index[1].int(), edge_index[0].int(), positions.shape[0], self.C)
        vec = positions[edge_index[1].long()] - positions[edge_index[0].long()] + shifts
        length = vec.norm(dim=-1)
        if float(length.min()) < 1e-3:
            raise ValueError("coincident atoms")

    def __call__(self, positions, node_attrs, edge_index, shifts):
        """positions [N,3] float64, node_attrs [N,Z] float64 one-hot, edge_index [2,E] int64 (row 0 receivers,
        sorted), shifts [E,3] float64, all on the device and already checked.  Returns (energy, forces)."""
        positions = positions.detach().requires_grad_(True)
        node_attrs = node_attrs.detach().requires_grad_(True)
        N = positions.shape[0]
        recv, send = edge_index[0].int(), edge_index[1].int()
        h = node_attrs @ self.embed
        vectors = positions[edge_index[1]] - positions[edge_index[0]] + shifts
        lengths = vectors.norm(dim=-1)
        Y = self.sh.forward(vectors.float())
        attrs32 = node_attrs.float()
        types = node_attrs.argmax(dim=-1).int()
        es = []
        for t, L in enumerate(self.layers):
            R = L["spline"].forward(lengths.float(), L["knots"], L["coeffs"], L["h"], self.r_max)
            h32 = h.float()
            sc = None
            if t == 1:
                sc = torch.einsum("nc,nz,czo->no", h32, attrs32, L["W_sc"])
            up = h32 @ L["W_up"]
            m = L["tp"].forward(up, Y, R.view(R.shape[0], 4, self.C), send, recv, N)
            m = L["linear"].forward(m, L["W_lin"], L["W_lin_T"]) / L["avg"]
            if t == 0:
                m = L["skip"].forward(m, L["W_skip"], L["W_skip_T"], attrs32)
            b = L["contraction"].forward(m, types, self.u3_max, *self.tables, L["W3"], L["W2"], L["W1"], L["W3"].shape[2],
                                         L["W2"].shape[2], L["W1"].shape[2]).squeeze()
            h32 = b @ L["W_prod"]
            if sc is not None:
                h32 = h32 + sc
            h = h32.double()
            if t == 0:
                es.append((h @ L["W_readout"])[:, 0])
            else:
                es.append((omodel.silu_n(h @ L["W_readout1"]) @ L["W_readout2"])[:, 0])
        energy = (self.scale * (es[0] + es[1]) + self.shift).sum()
        (g,) = torch.autograd.grad(energy, positions)
        return energy.detach(), -g
