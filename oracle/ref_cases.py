"""Seeded inputs for running the reference's own operators next to this library and the float64 restatement
(TEST AND BASELINE INFRASTRUCTURE ONLY), and the host-side guards every input passes before a reference launch.

The reference's kernels trust their inputs.  From reading them, a launch is only safe when
  * receivers are sorted and EVERY node receives at least one edge: the offsets of an edgeless node are never
    written (jit_wrappers/src/invariant_message_passing_wrapper.cpp:26-29) and are then used as an index
    (cuda/src/invariant_message_passing_impl.cu:99-101);
  * no node has more than 512 neighbours (shared-memory sender cache, impl.cu:88, :106-108, :317-318);
  * the list is symmetric and free of duplicate pairs: the backward looks the reverse edge up in an N x N table that
    only the forward's reverse edges fill (impl.cu:112-116, :331-336);
  * N x N int32 fits (N <= 8192 here) and E*4*C < 2^31 (32-bit flat offsets, impl.cu:138, :242, :288);
  * channels are 32, 64, 96 or 128, Linear is float32, indices and atom types are int32 (wrappers);
  * spline arguments stay inside the table: floor(r / h) below the number of intervals for every r <= r_max
    (cuda/src/cubic_spline_impl.cu:35-41 clamps to nknots - 1, one past the 255 intervals the table holds).
`check_*` raise ValueError when a rule is broken; oracle.ref_run calls them on every case.
"""
import math

import numpy as np
import torch

from . import ops as oops
from .sh import real_sh_l3

SIZES = {
    # fixture: small enough to commit the reference's outputs;  live: the template instances the model uses
    "fixture": dict(imp_nodes=24, imp_degree=8, imp_channels=32, edges=200, nodes=20, channels=32, elements=3,
                    spline_outputs=128),
    "live": dict(imp_nodes=300, imp_degree=24, imp_channels=128, edges=5000, nodes=256, channels=128, elements=10,
                 spline_outputs=512),
}


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def symmetric_graph(seed, n_nodes, mean_degree):
    """See cuda_mace_b200.systems.symmetric_graph (host-side data generation, shared with the benchmarks)."""
    from cuda_mace_b200 import systems

    return systems.symmetric_graph(seed, n_nodes, mean_degree)


def check_graph(sender, receiver, n_nodes, channels):
    s = sender.cpu().numpy().astype(np.int64)
    r = receiver.cpu().numpy().astype(np.int64)
    E = s.shape[0]
    if sender.dtype != torch.int32 or receiver.dtype != torch.int32:
        raise ValueError("edge lists must be int32")
    if E == 0 or n_nodes < 1 or n_nodes > 8192:
        raise ValueError("needs 1..8192 nodes and at least one edge")
    if s.min() < 0 or s.max() >= n_nodes or r.min() < 0 or r.max() >= n_nodes:
        raise ValueError("node index out of range")
    if np.any(np.diff(r) < 0):
        raise ValueError("receivers must be sorted")
    deg = np.bincount(r, minlength=n_nodes)
    if deg.min() < 1:
        raise ValueError("every node must receive at least one edge")
    if deg.max() > 512:
        raise ValueError("more than 512 neighbours on one node")
    key = r * n_nodes + s
    if np.unique(key).shape[0] != E:
        raise ValueError("duplicate (receiver, sender) pair")
    if not np.array_equal(np.sort(key), np.sort(s * n_nodes + r)):
        raise ValueError("edge list is not symmetric")
    if channels not in (32, 64, 96, 128):
        raise ValueError("channels must be 32, 64, 96 or 128")
    if E * 4 * channels >= 2**31 or n_nodes * 16 * channels >= 2**31:
        raise ValueError("32-bit flat offsets would overflow")


def check_spline(r, n_knots, n_intervals, h, r_max):
    if n_intervals != n_knots - 1:
        raise ValueError("coefficient table must hold nknots - 1 intervals")
    if not (h > 0 and math.floor(r_max / h) < n_intervals - 1):
        raise ValueError("r_max reaches past the coefficient table")
    if float(r.min()) < 0.0 or not bool(torch.isfinite(r).all()):
        raise ValueError("distances must be finite and non-negative")


def check_channels(C, what="channels"):
    if C not in (32, 64, 96, 128):
        raise ValueError(f"{what} must be 32, 64, 96 or 128")


# ------------------------------------------------------------------------------------------------------------
# cases: every function returns float64 / int32 CPU tensors; the runner casts to the dtype under test
# ------------------------------------------------------------------------------------------------------------
def case_sh(size):
    g = _gen(101)
    E = SIZES[size]["edges"]
    v = torch.randn(E, 3, generator=g, dtype=torch.float64)
    v = v / v.norm(dim=-1, keepdim=True) * (0.7 + 4.0 * torch.rand(E, 1, generator=g, dtype=torch.float64))
    return dict(xyz=v, G=torch.randn(16, E, generator=g, dtype=torch.float64))


def case_spline(size, r_max=5.0, n_knots=256):
    """Knots like cuda_mace/models/InvariantMACE.py:226 (256 on [1e-12, r_max + 1]); smooth seeded table values;
    coefficients from the restatement of the reference's solve (pinned against it in tests/test_oracle.py)."""
    g = _gen(102)
    F, E = SIZES[size]["spline_outputs"], SIZES[size]["edges"]
    knots = torch.linspace(1e-12, r_max + 1.0, n_knots, dtype=torch.float64)
    h = float(knots[1] - knots[0])
    amp = torch.randn(4, F, generator=g, dtype=torch.float64)
    x = knots[:, None] / r_max
    values = sum(amp[k] * torch.sin((k + 1) * math.pi * x) for k in range(4)) * (1 - x.clamp(max=1.0) ** 2)
    coeffs = oops.cubic_spline_coefficients(knots, values, h)
    r = 0.3 + (r_max + 0.4 - 0.3) * torch.rand(E, generator=g, dtype=torch.float64)   # some beyond r_max
    check_spline(r, n_knots, coeffs.shape[0], h, r_max)
    return dict(r=r, knots=knots, coeffs=coeffs, h=h, r_max=r_max, G=torch.randn(E, F, generator=g, dtype=torch.float64))


def case_imp(size, channels=None):
    S = SIZES[size]
    C = channels or S["imp_channels"]
    N = S["imp_nodes"]
    send, recv = symmetric_graph(103, N, S["imp_degree"])
    check_graph(send, recv, N, C)
    g = _gen(104)
    E = send.shape[0]
    v = torch.randn(E, 3, generator=g, dtype=torch.float64)
    return dict(X=torch.randn(N, C, generator=g, dtype=torch.float64), Y=real_sh_l3(v).contiguous(),
                R=torch.randn(E, 4, C, generator=g, dtype=torch.float64), sender=send, receiver=recv, nnodes=N,
                G=torch.randn(N, 16, C, generator=g, dtype=torch.float64))


def case_symcon(size, U):
    S = SIZES[size]
    N, C, Z = S["nodes"], S["channels"], S["elements"]
    check_channels(C)
    g = _gen(105)
    U3, U2, U1 = U
    W = [torch.randn(Z, n, C, generator=g, dtype=torch.float64) / math.sqrt(n) for n in (U3.shape[-1], U2.shape[-1],
                                                                                          U1.shape[-1])]
    return dict(X=torch.randn(N, 16, C, generator=g, dtype=torch.float64),
                atom_types=torch.randint(0, Z, (N,), generator=g, dtype=torch.int32), W3=W[0], W2=W[1], W1=W[2],
                tables=oops.pack_sparse_u(U3, U2, U1), G=torch.randn(N, 1, C, generator=g, dtype=torch.float64))


def case_linear(size):
    S = SIZES[size]
    N, C, Z = S["nodes"], S["channels"], S["elements"]
    check_channels(C)
    g = _gen(106)
    z = torch.randint(0, Z, (N,), generator=g)
    one_hot = torch.zeros(N, Z, dtype=torch.float64)
    one_hot[torch.arange(N), z] = 1.0
    return dict(X=torch.randn(N, 16, C, generator=g, dtype=torch.float64),
                W=torch.randn(4, C, C, generator=g, dtype=torch.float64),
                WE=torch.randn(Z, 4, C, C, generator=g, dtype=torch.float64), one_hot=one_hot,
                G=torch.randn(N, 16, C, generator=g, dtype=torch.float64))


# ------------------------------------------------------------------------------------------------------------
# the float64 restatement on the same cases: outputs and input gradients with loss (out * G).sum()
# ------------------------------------------------------------------------------------------------------------
def _grads(out, G, inputs):
    return torch.autograd.grad((out * G).sum(), inputs)


def oracle_results(size, U):
    res = {}
    c = case_sh(size)
    xyz = c["xyz"].clone().requires_grad_(True)
    Y = real_sh_l3(xyz)
    res["sh.out"], (res["sh.grad_xyz"],) = Y.detach(), _grads(Y, c["G"], (xyz,))
    c = case_spline(size)
    r = c["r"].clone().requires_grad_(True)
    R = oops.cubic_spline_eval(r, c["knots"], c["coeffs"], c["h"], c["r_max"])
    res["spline.out"], (res["spline.grad_r"],) = R.detach(), _grads(R, c["G"], (r,))
    c = case_imp(size)
    X, Y, R = (c[k].clone().requires_grad_(True) for k in ("X", "Y", "R"))
    out = oops.invariant_message_passing(X, Y, R, c["sender"], c["receiver"], c["nnodes"])
    res["imp.out"] = out.detach()
    res["imp.grad_X"], res["imp.grad_Y"], res["imp.grad_R"] = _grads(out, c["G"], (X, Y, R))
    c = case_symcon(size, U)
    X = c["X"].clone().requires_grad_(True)
    out = oops.symmetric_contraction_chunked(X, c["atom_types"], *U, c["W3"], c["W2"], c["W1"], chunk=64)
    res["symcon.out"], (res["symcon.grad_X"],) = out.detach(), _grads(out, c["G"], (X,))
    c = case_linear(size)
    X = c["X"].clone().requires_grad_(True)
    out = oops.linear(X, c["W"])
    res["linear.out"], (res["linear.grad_X"],) = out.detach(), _grads(out, c["G"], (X,))
    X = c["X"].clone().requires_grad_(True)
    out = oops.elemental_linear(X, c["WE"], c["one_hot"])
    res["elinear.out"], (res["elinear.grad_X"],) = out.detach(), _grads(out, c["G"], (X,))
    return res
