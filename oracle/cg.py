"""Generalised Clebsch-Gordan ("U") tensors for the invariant (L=0) symmetric
contraction of correlation order 3 over 0e+1o+2e+3o features (test infrastructure).

The reference obtains these from upstream ``mace.tools.cg.U_matrix_real``
(cuda_mace/ops/symmetric_contraction.py:25-35), which is not available here.
They are restated from their defining property instead: for an L=0 output every
coupling path of three irreps (l1, l2, l3) is the unique rotation-invariant
three-index tensor of those irreps, i.e. (up to scale) the Gaunt integral

    U3[i, j, k, p] ~ integral over the sphere of Y_i Y_j Y_k ,

for (l_i, l_j, l_k) = path p, which is non-zero exactly when the triple obeys the
triangle rule and l1+l2+l3 is even.  The integral is evaluated exactly with a
Gauss-Legendre x uniform-phi quadrature of this directory's own harmonics, so
the tensors are consistent with the harmonics' sign and axis conventions by
construction.  Each path is scaled to unit Frobenius norm, with the sign that
makes its m1 = m2 = m3 = 0 entry positive (the Gaunt integral of three m = 0
harmonics is a square, so this is the integral's own sign).  That rule does not
depend on the order of (l1, l2, l3), which keeps the tensor symmetric under a
simultaneous permutation of its indices and of the path's l's:
U3[i,j,k,(l1,l2,l3)] = U3[j,i,k,(l2,l1,l3)] = U3[j,k,i,(l2,l3,l1)].  The
reference's contraction kernel RELIES on that symmetry for its gradient
(cuda_mace/cuda/src/symmetric_contraction_impl.cu:160-169 sums the weights of
the three permuted paths against one stored value), so tables without it give
the reference a wrong gradient; upstream's U_matrix_real must have it too.
Upstream's tensors may still differ from these by one scale factor (and sign)
per symmetric class of paths, which the learnable weights absorb: PARITY
UNPINNED against upstream for that scale.

Shapes follow cuda_mace/ops/symmetric_contraction.py:100-176:
U3 [16,16,16,P3], U2 [16,16,P2], U1 [16,P1] with P3=23, P2=4, P1=1.
"""
import itertools

import numpy as np
import torch

from .sh import L_OF_LM, real_sh_l3


def _sphere_quadrature(n_theta: int = 12, n_phi: int = 24):
    """Nodes/weights exact for polynomials of degree <= min(2*n_theta-1, n_phi-1)."""
    ct, wt = np.polynomial.legendre.leggauss(n_theta)
    phi = (np.arange(n_phi) + 0.5) * (2.0 * np.pi / n_phi)
    st = np.sqrt(1.0 - ct * ct)
    pts = np.stack(
        [
            (st[:, None] * np.cos(phi)[None, :]).ravel(),
            (st[:, None] * np.sin(phi)[None, :]).ravel(),
            (ct[:, None] * np.ones_like(phi)[None, :]).ravel(),
        ],
        axis=-1,
    )
    w = (wt[:, None] * np.full_like(phi, 2.0 * np.pi / n_phi)[None, :]).ravel()
    return pts, w / (4.0 * np.pi)


def paths_nu3():
    """Ordered (l1, l2, l3) triples coupling to L=0, lexicographic order."""
    out = []
    for l1, l2, l3 in itertools.product(range(4), repeat=3):
        if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0:
            out.append((l1, l2, l3))
    return out


def u_matrices(dtype=torch.float64):
    """Returns (U3, U2, U1) dense tensors as float64 (or `dtype`) CPU tensors."""
    pts, w = _sphere_quadrature()
    Y = real_sh_l3(torch.from_numpy(pts)).numpy()  # [16, Q]
    gaunt = np.einsum("iq,jq,kq,q->ijk", Y, Y, Y, w)
    gaunt[np.abs(gaunt) < 1e-12] = 0.0
    lof = np.asarray(L_OF_LM)
    paths = paths_nu3()
    U3 = np.zeros((16, 16, 16, len(paths)))
    for p, (l1, l2, l3) in enumerate(paths):
        mask = (
            (lof[:, None, None] == l1)
            & (lof[None, :, None] == l2)
            & (lof[None, None, :] == l3)
        )
        t = np.where(mask, gaunt, 0.0)
        t = t / np.sqrt((t * t).sum())
        U3[..., p] = t * np.sign(t[l1 * l1 + l1, l2 * l2 + l2, l3 * l3 + l3])  # m = 0 sits at index l^2 + l
    U2 = np.zeros((16, 16, 4))
    for l in range(4):
        idx = np.flatnonzero(lof == l)
        U2[idx, idx, l] = 1.0 / np.sqrt(2 * l + 1)
    U1 = np.zeros((16, 1))
    U1[0, 0] = 1.0
    return (
        torch.from_numpy(U3).to(dtype),
        torch.from_numpy(U2).to(dtype),
        torch.from_numpy(U1).to(dtype),
    )
