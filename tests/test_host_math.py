"""The formulas the CUDA kernels execute, compiled for the host from the same headers
(csrc/edge_math.cuh, csrc/symcon_plan.hpp) and compared with the oracle on the CPU."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import model as omodel
from oracle import ops as oops
from oracle.sh import real_sh_l3


def P(a):
    return ctypes.c_void_p(a.ctypes.data)


@pytest.fixture(scope="module")
def hc(hostcheck_library):
    return ctypes.CDLL(hostcheck_library)


def edges(seed, n):
    rng = np.random.default_rng(seed)
    v = rng.normal(size=(n, 3))
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    return v * rng.uniform(0.6, 5.4, size=(n, 1))  # a few beyond the 5.0 cutoff


def test_edge_basis_forward_f64(hc):
    xyz = edges(0, 1500)
    E = xyz.shape[0]
    Y, B = np.zeros((16, E)), np.zeros((E, 8))
    hc.hc_edge_basis_fwd_f64(P(xyz), ctypes.c_int64(E), ctypes.c_double(5.0), 8, 5, P(Y), P(B))
    t = torch.from_numpy(xyz)
    assert np.abs(Y - real_sh_l3(t).numpy()).max() < 1e-13
    Bo = omodel.radial_embedding(t.norm(dim=-1), 5.0).numpy()
    assert np.abs(B - Bo).max() < 1e-13
    assert (B[np.linalg.norm(xyz, axis=1) >= 5.0] == 0).all()


def test_edge_basis_forward_f32_accuracy(hc):
    xyz = edges(1, 1500).astype(np.float32)
    E = xyz.shape[0]
    Y, B = np.zeros((16, E), np.float32), np.zeros((E, 8), np.float32)
    hc.hc_edge_basis_fwd_f32(P(xyz), ctypes.c_int64(E), ctypes.c_float(5.0), 8, 5, P(Y), P(B))
    t = torch.from_numpy(xyz).double()
    assert np.abs(Y - real_sh_l3(t).numpy()).max() < 2e-6 * 4.0
    Bo = omodel.radial_embedding(t.norm(dim=-1), 5.0).numpy()
    assert np.abs(B - Bo).max() < 1e-6 * np.abs(Bo).max()


def test_edge_basis_backward_f64(hc):
    xyz = edges(2, 1500)
    E = xyz.shape[0]
    rng = np.random.default_rng(3)
    gY, gB = rng.normal(size=(16, E)), rng.normal(size=(E, 8))
    t = torch.from_numpy(xyz).requires_grad_(True)
    loss = (real_sh_l3(t) * torch.from_numpy(gY)).sum() + (omodel.radial_embedding(t.norm(dim=-1), 5.0) * torch.from_numpy(gB)).sum()
    (ref,) = torch.autograd.grad(loss, t)
    out = np.zeros((E, 3))
    hc.hc_edge_basis_bwd_f64(P(xyz), P(gY), P(gB), ctypes.c_int64(E), ctypes.c_double(5.0), 8, 5, P(out))
    assert np.abs(out - ref.numpy()).max() < 1e-12 * np.abs(ref.numpy()).max()
    # harmonics only
    (ref_y,) = torch.autograd.grad((real_sh_l3(t) * torch.from_numpy(gY)).sum(), t)
    hc.hc_edge_basis_bwd_f64(P(xyz), P(gY), None, ctypes.c_int64(E), ctypes.c_double(5.0), 8, 5, P(out))
    assert np.abs(out - ref_y.numpy()).max() < 1e-12 * np.abs(ref_y.numpy()).max()


def tables_f64(U):
    U3, U2, U1 = U
    maxnz, n3, i3, v3, n2, i2, v2, n1, i1 = oops.pack_sparse_u(U3, U2, U1)
    v3d = torch.zeros(maxnz, 16, 16, dtype=torch.float64)
    v2d = torch.zeros(16, 16, dtype=torch.float64)
    for i in range(16):
        for j in range(16):
            k1, p1 = torch.where(U3[i, j] != 0)
            for t in range(k1.shape[0]):
                v3d[t, i, j] = U3[i, j, k1[t], p1[t]]
            (p,) = torch.where(U2[i, j] != 0)
            if p.shape[0]:
                v2d[i, j] = U2[i, j, p[0]]
    return maxnz, n3.numpy(), i3.numpy(), v3d.numpy(), n2.numpy(), i2.numpy(), v2d.numpy()


@pytest.mark.parametrize("canonical", [0, 1])
@pytest.mark.parametrize("rescale", [False, True])
def test_contraction_program_matches_dense_oracle(hc, U, canonical, rescale):
    """Table-driven program (canonical=0) and generated straight-line code (canonical=1) against the dense
    einsum; `rescale` multiplies every coupling path by its own factor, as a different upstream
    normalisation of the U tensors would: the plan must still recognise the canonical forms."""
    U3, U2, U1 = U
    if rescale:
        g0 = torch.Generator().manual_seed(9)
        U3 = U3 * (0.5 + torch.rand(23, generator=g0, dtype=torch.float64)) * torch.where(torch.arange(23) % 3 == 0, -1.0, 1.0)
        U2 = U2 * (0.5 + torch.rand(4, generator=g0, dtype=torch.float64))
    Uc = (U3, U2, U1)
    maxnz, n3, i3, v3, n2, i2, v2 = tables_f64(Uc)
    N, C, Z = 9, 32, 3
    g = torch.Generator().manual_seed(0)
    X = torch.randn(N, 16, C, generator=g, dtype=torch.float64, requires_grad=True)
    at = torch.randint(0, Z, (N,), generator=g, dtype=torch.int32)
    W3, W2, W1 = (torch.randn(Z, n, C, generator=g, dtype=torch.float64) for n in (23, 4, 1))
    ref = oops.symmetric_contraction(X, at, *Uc, W3, W2, W1)[:, 0]
    (gref,) = torch.autograd.grad(ref.sum(), X)
    out, grad, info = np.zeros((N, C)), np.zeros((N, 16, C)), np.zeros(5, np.int32)
    Xn, atn, a, b, c = X.detach().numpy(), at.numpy(), W3.numpy(), W2.numpy(), W1.numpy()
    rc = hc.hc_symcon_f64(maxnz, P(n3), P(i3), P(v3), P(n2), P(i2), P(v2), 23, 4, 1, P(Xn), P(atn), P(a), P(b), P(c),
                          ctypes.c_int64(N), C, P(out), P(grad), P(info), canonical)
    assert rc == 0
    # 23 coupling paths collapse to 8 distinct cubic invariants, 4 quadratic ones, all canonical
    assert info[0] == 8 and info[1] == 4 and info[4] == 1
    assert np.abs(out - ref.detach().numpy()).max() < 1e-12 * np.abs(ref.detach().numpy()).max()
    assert np.abs(grad - gref.numpy()).max() < 1e-12 * np.abs(gref.numpy()).max()


def test_non_canonical_tables_are_detected(hc, U):
    """A coupling tensor with one perturbed entry is no longer proportional to a canonical form."""
    U3, U2, U1 = (t.clone() for t in U)
    idx = (U3[..., 5] != 0).nonzero()[0]
    U3[idx[0], idx[1], idx[2], 5] *= 1.5
    maxnz, n3, i3, v3, n2, i2, v2 = tables_f64((U3, U2, U1))
    info = np.zeros(5, np.int32)
    z = np.zeros((1, 16, 32))
    w = np.zeros((1, 23, 32))
    at, out, grad = np.zeros(1, np.int32), np.zeros((1, 32)), np.zeros((1, 16, 32))  # kept alive across the call
    rc = hc.hc_symcon_f64(maxnz, P(n3), P(i3), P(v3), P(n2), P(i2), P(v2), 23, 4, 1, P(z), P(at),
                          P(w), P(w), P(w), ctypes.c_int64(1), 32, P(out), P(grad), P(info), 1)
    assert rc == 0 and info[4] == 0


def test_contraction_program_rejects_bad_tables(hc, U):
    maxnz, n3, i3, v3, n2, i2, v2 = tables_f64(U)
    bad = i3.copy()
    bad[0, 1, 1] |= 0xFF  # path index beyond w3
    z = np.zeros((1, 16, 32))
    info = np.zeros(5, np.int32)
    at = np.zeros(1, np.int32)
    w = np.zeros((1, 23, 32))
    out, grad = np.zeros((1, 32)), np.zeros((1, 16, 32))
    rc = hc.hc_symcon_f64(maxnz, P(n3), P(bad), P(v3), P(n2), P(i2), P(v2), 23, 4, 1, P(z), P(at), P(w), P(w), P(w),
                          ctypes.c_int64(1), 32, P(out), P(grad), P(info), 0)
    assert rc == 1
