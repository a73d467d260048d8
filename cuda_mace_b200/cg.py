"""Generalised Clebsch-Gordan ("U") tensors for the L=0 symmetric contraction, correlation <= 3.

The reference gets these from upstream ``mace.tools.cg.U_matrix_real``
(cuda_mace/ops/symmetric_contraction.py:25-35).  That package is not a dependency
here; for an invariant output every coupling path (l1, l2, l3) is the real-basis
Wigner 3j symbol of the three irreps, which is what this module builds:
Racah's closed formula for the complex 3j symbol, then the unitary change of basis
from complex to real harmonics on each index.  Upstream's tensors can differ by one
scale and sign per path, which the per-path weights absorb.

U3 [16,16,16,23], U2 [16,16,4], U1 [16,1]; the 16 components are (l, m) with
l = 0..3, m = -l..l, and the paths of U3 are the ordered (l1, l2, l3) triples that
obey the triangle rule with l1+l2+l3 even, in lexicographic order.
"""
import itertools
from fractions import Fraction
from math import factorial, sqrt

import numpy as np
import torch

L_OF_LM = [0, 1, 1, 1, 2, 2, 2, 2, 2, 3, 3, 3, 3, 3, 3, 3]


def wigner_3j(j1, j2, j3, m1, m2, m3):
    """Complex-basis Wigner 3j symbol for integer arguments (Racah's formula)."""
    if m1 + m2 + m3 != 0 or not (abs(j1 - j2) <= j3 <= j1 + j2):
        return 0.0
    if abs(m1) > j1 or abs(m2) > j2 or abs(m3) > j3:
        return 0.0
    f = factorial
    tri = Fraction(f(j1 + j2 - j3) * f(j1 - j2 + j3) * f(-j1 + j2 + j3), f(j1 + j2 + j3 + 1))
    pre = tri * f(j1 + m1) * f(j1 - m1) * f(j2 + m2) * f(j2 - m2) * f(j3 + m3) * f(j3 - m3)
    s = Fraction(0)
    for t in range(0, j1 + j2 - j3 + 1):
        d = [t, j3 - j2 + t + m1, j3 - j1 + t - m2, j1 + j2 - j3 - t, j1 - t - m1, j2 - t + m2]
        if min(d) < 0:
            continue
        den = 1
        for x in d:
            den *= f(x)
        s += Fraction((-1) ** t, den)
    return (-1) ** (j1 - j2 - m3) * sqrt(pre) * float(s)


def complex_to_real(l):
    """Unitary Q [2l+1, 2l+1] with Y_real[m] = sum_mu Q[m, mu] Y_complex[mu] (Condon-Shortley)."""
    Q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    for m in range(-l, l + 1):
        r = m + l
        if m == 0:
            Q[r, l] = 1.0
        elif m > 0:
            # sqrt(2) (-1)^m Re Y_l^m = ((-1)^m Y_l^m + Y_l^-m) / sqrt(2)
            Q[r, l + m] = (-1) ** m / sqrt(2.0)
            Q[r, l - m] = 1.0 / sqrt(2.0)
        else:
            # sqrt(2) (-1)^m Im Y_l^|m| = -i ((-1)^m Y_l^|m| - Y_l^-|m|) / sqrt(2)
            a = -m
            Q[r, l + a] = -1j * (-1) ** a / sqrt(2.0)
            Q[r, l - a] = 1j / sqrt(2.0)
    return Q


def real_wigner_3j(l1, l2, l3):
    """Rotation-invariant tensor [2l1+1, 2l2+1, 2l3+1] in the real basis, Frobenius norm 1."""
    w = np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1))
    for a, b, c in itertools.product(range(-l1, l1 + 1), range(-l2, l2 + 1), range(-l3, l3 + 1)):
        w[a + l1, b + l2, c + l3] = wigner_3j(l1, l2, l3, a, b, c)
    # an invariant tensor transforms with the conjugate of the basis change on every index
    t = np.einsum("ia,jb,kc,abc->ijk", complex_to_real(l1).conj(), complex_to_real(l2).conj(),
                  complex_to_real(l3).conj(), w)
    # for even l1+l2+l3 the result is real, for odd it would be imaginary
    t = t.real if abs(t.real).max() >= abs(t.imag).max() else t.imag
    t[np.abs(t) < 1e-12] = 0.0
    return t / np.sqrt((t * t).sum())


def paths_nu3():
    return [
        (a, b, c)
        for a, b, c in itertools.product(range(4), repeat=3)
        if abs(a - b) <= c <= a + b and (a + b + c) % 2 == 0
    ]


def u_matrices(dtype=torch.float64):
    """(U3, U2, U1) dense CPU tensors; every path has unit Frobenius norm and a positive m1 = m2 = m3 = 0 entry.
    That sign rule does not depend on the order of (l1, l2, l3), so U3[i,j,k,(l1,l2,l3)] = U3[j,i,k,(l2,l1,l3)] =
    U3[j,k,i,(l2,l3,l1)]: the symmetry the reference's contraction kernel assumes when it forms its gradient
    from one stored value and the weights of the three permuted paths (symmetric_contraction_impl.cu:160-169)."""
    lof = np.asarray(L_OF_LM)
    paths = paths_nu3()
    U3 = np.zeros((16, 16, 16, len(paths)))
    for p, (l1, l2, l3) in enumerate(paths):
        t = real_wigner_3j(l1, l2, l3)
        t = t * np.sign(t[l1, l2, l3])  # the m = 0 entry of every index
        i0, j0, k0 = l1 * l1, l2 * l2, l3 * l3
        U3[i0 : i0 + 2 * l1 + 1, j0 : j0 + 2 * l2 + 1, k0 : k0 + 2 * l3 + 1, p] = t
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
