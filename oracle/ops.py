"""Float64 torch restatements of the five reference operators (test infrastructure).

Every function is differentiable through torch autograd, which supplies the
oracle for the backward kernels as well (the reference's tests do the same with
``(out**2).sum().backward()``, tests/invariant_message_passing.py:135-137).
"""
import math

import torch

from .sh import L_OF_LM


# --------------------------------------------------------------------------------------
# invariant message passing
# --------------------------------------------------------------------------------------
def invariant_message_passing(X, Y, radial, sender, receiver, nnodes):
    """out[i, lm, c] = sum_{e: receiver(e)=i} X[sender(e), c] * Y[lm, e] * radial[e, l(lm), c].

    Restates inv_tp_kernel_ptr (cuda_mace/cuda/src/invariant_message_passing_impl.cu:118-152);
    the e3nn ``uvu`` tensor product with unit path weights followed by scatter_sum that the
    reference tests against (tests/invariant_message_passing.py:86-118) is this plain product.
    X [N, C], Y [16, E], radial [E, 4, C], sender/receiver [E] -> [N, 16, C].
    Receivers without edges get zero rows.
    """
    # one [E, C] product per (l, m) instead of one [E, 16, C] array: the same sums, a sixteenth of the temporaries
    recv = receiver.long()
    xs = X[sender.long()]
    rows = []
    for lm, l in enumerate(L_OF_LM):
        if lm == l * l:
            xr = xs * radial[:, l, :]
        rows.append(torch.zeros(nnodes, X.shape[1], dtype=X.dtype).index_add(0, recv, xr * Y[lm][:, None]))
    return torch.stack(rows, dim=1)


# --------------------------------------------------------------------------------------
# Linear / ElementalLinear
# --------------------------------------------------------------------------------------
def linear(X, W):
    """out[n, l^2+m, :] = X[n, l^2+m, :] @ W[l] / sqrt(K).

    Restates linear_kernel_ptr (cuda_mace/cuda/src/linear_impl.cu:33, :65-66, :125-129);
    W [4, K, Nout] is the per-l split of the e3nn weight (cuda_mace/ops/linear.py:30-51).
    """
    lof = torch.as_tensor(L_OF_LM, dtype=torch.long)
    return torch.einsum("nmk,mko->nmo", X, W[lof]) / math.sqrt(W.shape[1])


def elemental_linear(X, W, one_hot):
    """out[n, l^2+m, :] = X[n, l^2+m, :] @ W[z_n, l] / sqrt(K) with z_n the node's element.

    Restates elemental_linear_kernel_ptr (cuda_mace/cuda/src/linear_impl.cu:157-158, :186) and the
    per-element row selection of jit_elemental_linear (jit_wrappers/src/linear_wrapper.cpp:137-143).
    W [Z, 4, K, Nout]; one_hot [N, Z].
    """
    lof = torch.as_tensor(L_OF_LM, dtype=torch.long)
    z = one_hot.argmax(dim=-1)
    Wn = W[z][:, lof]  # [N, 16, K, Nout]
    return torch.einsum("nmk,nmko->nmo", X, Wn) / math.sqrt(W.shape[2])


# --------------------------------------------------------------------------------------
# symmetric contraction (correlation 3, output L=0)
# --------------------------------------------------------------------------------------
def symmetric_contraction(X, atom_types, U3, U2, U1, W3, W2, W1):
    """out[n, c] = sum_ijk,p U3[i,j,k,p] W3[z_n,p,c] x_i x_j x_k
                 + sum_ij,p  U2[i,j,p]   W2[z_n,p,c] x_i x_j
                 + sum_i,p   U1[i,p]     W1[z_n,p,c] x_i          with x_i = X[n, i, c].

    Dense form of symmetric_contraction_kernel
    (cuda_mace/cuda/src/symmetric_contraction_impl.cu:108-175); U shapes as in
    cuda_mace/ops/symmetric_contraction.py:100-176, weight shapes [Z, P, C] as in :189-232.
    Returns [N, 1, C] like the reference wrapper (symmetric_contraction_wrapper.cpp:39-41).
    """
    z = atom_types.long()
    out = torch.zeros(X.shape[0], X.shape[2], dtype=X.dtype)
    for e in range(W3.shape[0]):
        (idx,) = torch.where(z == e)
        if idx.numel() == 0:
            continue
        x = X[idx]
        T3 = torch.einsum("ijkp,pc->ijkc", U3, W3[e])
        T2 = torch.einsum("ijp,pc->ijc", U2, W2[e])
        T1 = torch.einsum("ip,pc->ic", U1, W1[e])
        # nested like the kernel: innermost k, then j, then i
        t = torch.einsum("ijkc,nkc->nijc", T3, x) + T2[None]
        t = torch.einsum("nijc,njc->nic", t, x) + T1[None]
        out = out.index_add(0, idx, torch.einsum("nic,nic->nc", t, x))
    return out[:, None, :]


def symmetric_contraction_chunked(X, atom_types, U3, U2, U1, W3, W2, W1, chunk=256):
    """Same as symmetric_contraction but bounded in memory for thousands of nodes."""
    outs = []
    for s in range(0, X.shape[0], chunk):
        outs.append(
            symmetric_contraction(X[s : s + chunk], atom_types[s : s + chunk], U3, U2, U1, W3, W2, W1)
        )
    return torch.cat(outs, dim=0)


def symmetric_contraction_sparse_tables(X, atom_types, tables, W3, W2, W1):
    """The reference kernel's own loop over the SPARSE tables, value and gradient, restated statement by statement
    from symmetric_contraction_kernel<scalar_t, true> (cuda_mace/cuda/src/symmetric_contraction_impl.cu:108-180).

    `tables` = pack_sparse_u(...).  Returns (out [N, C], grad [N, 16, C]) where grad is what the kernel stores as
    d out / d x_i: per (i, j) and stored non-zero k it adds u3 * (W3[p1] + W3[p2] + W3[p3]) * x_k * x_j with the
    three path indices unpacked from one int32 (:147-169), i.e. it assumes that the value stored for
    U3[i, j, k, p1] is also the value of U3[j, i, k, p2] and of U3[j, k, i, p3].  That holds for tables that are
    symmetric under a simultaneous permutation of indices and path (see oracle/cg.py); for other tables the forward
    value is still right and this gradient is not the derivative.  Used to pin the restatement of that rule
    against the gradient the reference's kernel produced on the GPU."""
    maxnz, n3, idx3, val3, n2, idx2, val2, _, _ = tables
    z = atom_types.long()
    N, _, C = X.shape
    W3n, W2n, W1n = W3[z], W2[z], W1[z]  # [N, P, C]
    zero = torch.zeros(N, C, dtype=X.dtype)
    out = zero.clone()
    grad = torch.zeros_like(X)
    for i in range(16):
        uw1 = W1n[:, 0] if i == 0 else zero
        output_2 = zero.clone()
        deriv1 = uw1.clone()
        for j in range(16):
            uw2 = float(val2[i, j]) * W2n[:, int(idx2[i, j])] if int(n2[i, j]) > 0 else zero
            output_3 = zero.clone()
            deriv_1_j = uw2.clone()
            for k in range(int(n3[i, j])):
                packed = int(idx3[k, i, j])
                p1, kdx, p3, p2 = packed & 0xFF, (packed >> 8) & 0xFF, (packed >> 16) & 0xFF, (packed >> 24) & 0xFF
                u3 = float(val3[k, i, j])
                output_3 = output_3 + u3 * W3n[:, p1] * X[:, kdx]
                deriv_1_j = deriv_1_j + u3 * (W3n[:, p1] + W3n[:, p2] + W3n[:, p3]) * X[:, kdx]
            output_2 = output_2 + (output_3 + uw2) * X[:, j]
            deriv1 = deriv1 + (uw2 + deriv_1_j) * X[:, j]
        out = out + (output_2 + uw1) * X[:, i]
        grad[:, i] = deriv1
    return out, grad


def pack_sparse_u(U3, U2, U1):
    """Packs dense U tensors into the reference's sparse tables.

    Follows cuda_mace/ops/symmetric_contraction.py:91-187 (bit layout at :118-125):
    per (i, j) the k-th non-zero of U3[i, j] is stored as value + 4 packed bytes:
    bits 7:0 path of U3[i,j,k,:], 15:8 k, 23:16 the k-th non-zero path of U3[j,:,i,:],
    31:24 the k-th non-zero path of U3[j,i,:,:].
    """
    n3 = torch.zeros(16, 16, dtype=torch.int16)
    for i in range(16):
        for j in range(16):
            n3[i, j] = int((U3[i, j] != 0).sum())
    maxnz = int(n3.max())
    idx3 = torch.zeros(maxnz, 16, 16, dtype=torch.int32)
    val3 = torch.zeros(maxnz, 16, 16, dtype=torch.float32)
    for i in range(16):
        for j in range(16):
            k1, p1 = torch.where(U3[i, j] != 0)
            _, p2 = torch.where(U3[j, i] != 0)
            _, p3 = torch.where(U3[j, :, i, :] != 0)
            for t in range(k1.shape[0]):
                lo = (int(k1[t]) << 8) | int(p1[t])
                hi = (int(p2[t]) << 8) | int(p3[t])
                idx3[t, i, j] = (hi << 16) | lo
                val3[t, i, j] = U3[i, j, k1[t], p1[t]]
    n2 = torch.zeros(16, 16, dtype=torch.int16)
    idx2 = torch.zeros(16, 16, dtype=torch.int16)
    val2 = torch.zeros(16, 16, dtype=torch.float32)
    for i in range(16):
        for j in range(16):
            (p,) = torch.where(U2[i, j] != 0)
            n2[i, j] = p.shape[0]
            if p.shape[0] > 0:
                idx2[i, j] = int(p[0])
                val2[i, j] = U2[i, j, p[0]]
    n1 = torch.zeros(16, dtype=torch.int16)
    idx1 = torch.zeros(16, dtype=torch.int16)
    for i in range(16):
        (p,) = torch.where(U1[i] != 0)
        if p.shape[0] > 0:
            n1[i] = 1
            idx1[i] = int(p[0])
    return maxnz, n3, idx3, val3, n2, idx2, val2, n1, idx1


# --------------------------------------------------------------------------------------
# cubic spline (natural) of the radial weights
# --------------------------------------------------------------------------------------
def cubic_spline_coefficients(x, y, h):
    """Natural cubic spline coefficients [n, 4, F] of y [n+1, F] on equidistant knots x.

    Same tridiagonal solve as cuda_mace/ops/cubic_spline.py:41-84.
    """
    n = x.shape[0] - 1
    F = y.shape[1]
    alpha = torch.zeros(n, F, dtype=y.dtype)
    alpha[1:] = 3.0 / h * (y[2:] - y[1:-1]) - 3.0 / h * (y[1:-1] - y[:-2])
    l = torch.ones(n + 1, dtype=y.dtype)
    mu = torch.zeros(n, dtype=y.dtype)
    z = torch.zeros(n + 1, F, dtype=y.dtype)
    for i in range(1, n):
        l[i] = 2.0 * (x[i + 1] - x[i - 1]) - h * mu[i - 1]
        mu[i] = h / l[i]
        z[i] = (alpha[i] - h * z[i - 1]) / l[i]
    c = torch.zeros(n + 1, F, dtype=y.dtype)
    for j in range(n - 1, -1, -1):
        c[j] = z[j] - mu[j] * c[j + 1]
    b = (y[1:] - y[:-1]) / h - h * (c[1:] + 2.0 * c[:-1]) / 3.0
    d = (c[1:] - c[:-1]) / (3.0 * h)
    return torch.stack((y[:-1], b, c[:-1], d), dim=1)


def cubic_spline_eval(r, r_knots, coeffs, r_width, r_max):
    """R[e, j] = a + b x + c x^2 + d x^3 in the knot interval floor(r/h); zero for r > r_max.

    Restates evaluate_spline_kernel_ptr (cuda_mace/cuda/src/cubic_spline_impl.cu:19-64); the
    interval index is clamped to [0, nknots-1] like :35-41, where nknots is the number of
    intervals the coefficient table holds.  Differentiable with respect to r.
    """
    nint = coeffs.shape[0]
    idx = torch.clamp((r.detach() / r_width).floor().long(), 0, nint - 1)
    x = (r - r_knots[idx])[:, None]
    cf = coeffs[idx]
    out = cf[:, 0] + cf[:, 1] * x + cf[:, 2] * x * x + cf[:, 3] * x * x * x
    return torch.where((r > r_max)[:, None], torch.zeros_like(out), out)
