"""Parity of every CUDA operator (through the C-ABI) with the float64 CPU oracle: outputs and all
input gradients with loss (out**2).sum(), float32 and float64, edge cases included."""
import os

import numpy as np
import pytest
import torch

from tests.util import TOL, random_graph, rel_err, unit_vectors

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DTYPES = [torch.float64, torch.float32]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "the gpu tests need a CUDA device"
    return torch.device("cuda:0")


def imp_case(seed, N, deg, C, dtype, dev, nsend=None, empty_every=0):
    send, recv = random_graph(seed, N, deg, n_senders=nsend, empty_every=empty_every)
    E = send.numel()
    g = torch.Generator().manual_seed(seed + 100)
    X = torch.randn(nsend or N, C, generator=g, dtype=torch.float64)
    Y = torch.randn(16, E, generator=g, dtype=torch.float64)
    R = torch.randn(E, 4, C, generator=g, dtype=torch.float64)
    return send, recv, X, Y, R


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,deg,C,nsend,empty", [
    (97, 7, 128, None, 0),      # odd degrees, one f32 chunk / two f64 chunks
    (64, 30, 64, None, 5),      # isolated receivers
    (33, 3, 96, None, 0),       # three 32-channel chunks
    (50, 5, 32, 80, 3),         # more sender rows than receivers (ghost atoms), isolated receivers
    (5, 600, 128, None, 0),     # more than 512 neighbours per receiver
    (8192, 30, 128, None, 0),   # the isolated-operator configuration of the benchmark spec at its full size
])
def test_message_passing(dtype, N, deg, C, nsend, empty, dev):
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    send, recv, X, Y, R = imp_case(N + C, N, deg, C, dtype, dev, nsend, empty)
    Xo, Yo, Ro = (t.to(dtype).double().clone().requires_grad_(True) for t in (X, Y, R))
    ref = oops.invariant_message_passing(Xo, Yo, Ro, send, recv, N)
    (ref ** 2).sum().backward()

    Xg, Yg, Rg = (t.to(dtype).to(dev).clone().requires_grad_(True) for t in (X, Y, R))
    tp = ops.InvariantMessagePassingTP()
    out = tp(Xg, Yg, Rg, send.to(dev), recv.to(dev), N)
    assert out.shape == (N, 16, C)
    (out ** 2).sum().backward()
    tol = TOL[dtype]
    assert rel_err(out, ref) < tol["out"]
    assert rel_err(Xg.grad, Xo.grad) < tol["grad"]
    assert rel_err(Yg.grad, Yo.grad) < tol["grad"]
    assert rel_err(Rg.grad, Ro.grad) < tol["grad"]
    if empty:  # receivers without edges are written as zeros, not left as garbage
        assert out[::empty].abs().max().item() == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_message_passing_without_edges_and_determinism(dtype, dev):
    from cuda_mace_b200 import ops

    tp = ops.InvariantMessagePassingTP()
    e = torch.zeros(0, dtype=torch.int32, device=dev)
    out = tp(torch.randn(4, 32, dtype=dtype, device=dev), torch.zeros(16, 0, dtype=dtype, device=dev),
             torch.zeros(0, 4, 32, dtype=dtype, device=dev), e, e, 4)
    assert out.shape == (4, 16, 32) and out.abs().max().item() == 0.0
    send, recv, X, Y, R = imp_case(5, 300, 20, 128, dtype, dev)
    args = [t.to(dtype).to(dev) for t in (X, Y, R)] + [send.to(dev), recv.to(dev), 300]
    assert torch.equal(tp(*args), tp(*args))  # no atomics: bitwise reproducible


def test_topology(dev):
    from cuda_mace_b200 import ops

    send, recv = random_graph(3, 1000, 9, empty_every=7)
    topo = ops.EdgeTopology(send.to(dev), recv.to(dev), 1000)
    counts = torch.bincount(recv.long(), minlength=1000)
    ref_ptr = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)])
    assert torch.equal(topo.row_ptr.cpu().long(), ref_ptr)
    perm, send_ptr = topo.sender_order()
    perm = perm.cpu().long()[: send.numel()]
    assert torch.equal(send[perm].long(), torch.sort(send.long(), stable=True).values)
    assert torch.equal(perm, torch.sort(send.long(), stable=True).indices)
    sc = torch.bincount(send.long(), minlength=1000)
    assert torch.equal(send_ptr.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), sc.cumsum(0)]))
    # empty list
    e = torch.zeros(0, dtype=torch.int32, device=dev)
    assert ops.EdgeTopology(e, e, 5).row_ptr.cpu().tolist() == [0] * 6


@pytest.mark.parametrize("dtype", DTYPES)
# (77, 40, 136): K not a multiple of the K slice, two column tiles; (33, 15, 9): odd sizes take the FMA kernel in float64
@pytest.mark.parametrize("N,K,Nout", [(130, 128, 128), (9, 64, 64), (40, 96, 32), (1, 32, 96), (77, 40, 136),
                                      (33, 15, 9), (700, 128, 128)])
def test_linear(dtype, N, K, Nout, dev):
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    g = torch.Generator().manual_seed(N)
    X = torch.randn(N, 16, K, generator=g, dtype=torch.float64).to(dtype)
    W = torch.randn(4, K, Nout, generator=g, dtype=torch.float64).to(dtype)
    Xo = X.double().clone().requires_grad_(True)
    ref = oops.linear(Xo, W.double())
    (ref ** 2).sum().backward()
    Xg = X.to(dev).clone().requires_grad_(True)
    Wg = W.to(dev)
    out = ops.linear_forward(Xg, Wg, Wg.transpose(-1, -2).contiguous())
    (out ** 2).sum().backward()
    assert rel_err(out, ref) < TOL[dtype]["out"]
    assert rel_err(Xg.grad, Xo.grad) < TOL[dtype]["grad"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,Z,K", [(200, 4, 128), (37, 10, 64), (5, 3, 32)])
def test_elemental_linear(dtype, N, Z, K, dev):
    from cuda_mace_b200 import ops, systems
    from oracle import ops as oops

    g = torch.Generator().manual_seed(N + Z)
    X = torch.randn(N, 16, K, generator=g, dtype=torch.float64).to(dtype)
    W = torch.randn(Z, 4, K, K, generator=g, dtype=torch.float64).to(dtype)
    at = torch.randint(0, Z, (N,), generator=g)
    at[at == 1] = 0  # one element with no atoms at all
    onehot = systems.one_hot(at, Z)
    Xo = X.double().clone().requires_grad_(True)
    ref = oops.elemental_linear(Xo, W.double(), onehot)
    (ref ** 2).sum().backward()
    Xg = X.to(dev).clone().requires_grad_(True)
    Wg = W.to(dev)
    out = ops.elemental_linear_forward(Xg, Wg, Wg.transpose(-1, -2).contiguous(), onehot.to(dtype).to(dev))
    (out ** 2).sum().backward()
    assert rel_err(out, ref) < TOL[dtype]["out"]
    assert rel_err(Xg.grad, Xo.grad) < TOL[dtype]["grad"]
    # int32 element index instead of one-hot
    out2 = ops.elemental_linear_forward(X.to(dev), Wg, Wg.transpose(-1, -2).contiguous(), at.to(torch.int32).to(dev))
    assert torch.equal(out2, out.detach())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,Z,K", [(1000, 4, 128), (37, 10, 64), (333, 3, 32), (4, 2, 128)])
def test_elemental_linear_on_nodes_stored_grouped_by_element(dtype, N, Z, K, dev):
    """Nodes whose element index is already non-decreasing need no gather list: the operator passes none, and the
    float32 kernel moves whole-node boxes by TMA (the last, partial box of every element row by row).  Same oracle,
    same tolerances; elements without atoms and elements of fewer atoms than a box included."""
    from cuda_mace_b200 import ops, systems
    from oracle import ops as oops

    g = torch.Generator().manual_seed(7 * N + Z)
    X = torch.randn(N, 16, K, generator=g, dtype=torch.float64).to(dtype)
    W = torch.randn(Z, 4, K, K, generator=g, dtype=torch.float64).to(dtype)
    at = torch.randint(0, Z, (N,), generator=g)
    at[at == 1] = 0  # one element with no atoms at all
    at = torch.sort(at).values
    onehot = systems.one_hot(at, Z)
    Xo = X.double().clone().requires_grad_(True)
    ref = oops.elemental_linear(Xo, W.double(), onehot)
    (ref ** 2).sum().backward()
    Xg = X.to(dev).clone().requires_grad_(True)
    Wg = W.to(dev)
    elem = at.to(torch.int32).to(dev)
    order, start = ops.group_by_element(elem, Z)
    assert order is None and start.tolist()[-1] == N
    out = ops.elemental_linear_forward(Xg, Wg, Wg.transpose(-1, -2).contiguous(), elem)
    (out ** 2).sum().backward()
    ops.check_status()
    assert rel_err(out, ref) < TOL[dtype]["out"]
    assert rel_err(Xg.grad, Xo.grad) < TOL[dtype]["grad"]
    # rows of other elements' nodes are not touched by a neighbour's partial box: exact agreement with the gathered path
    shuffled = torch.randperm(N, generator=g)
    out_g = ops.elemental_linear_forward(X[shuffled].to(dev), Wg, Wg.transpose(-1, -2).contiguous(), elem[shuffled.to(dev)])
    assert rel_err(out_g, out.detach()[shuffled.to(dev)]) < (1e-6 if dtype == torch.float32 else 1e-13)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,C,Z", [(256, 128, 10), (19, 32, 1), (64, 64, 4),
                                   (4096, 128, 10)])   # last: the benchmark spec's configuration at full size
def test_symmetric_contraction(dtype, N, C, Z, dev, U):
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    g = torch.Generator().manual_seed(N + C)
    X = torch.randn(N, 16, C, generator=g, dtype=torch.float64).to(dtype)
    at = torch.randint(0, Z, (N,), generator=g, dtype=torch.int32)
    W3, W2, W1 = (torch.randn(Z, n, C, generator=g, dtype=torch.float64).to(dtype) / n for n in (23, 4, 1))
    Xo = X.double().clone().requires_grad_(True)
    ref = oops.symmetric_contraction_chunked(Xo, at, *U, W3.double(), W2.double(), W1.double())
    (ref ** 2).sum().backward()
    mod = ops.SymmetricContraction(*U, W3, W2, W1).to(dev)
    Xg = X.to(dev).clone().requires_grad_(True)
    out = mod(Xg, at.to(dev))
    assert out.shape == (N, 1, C)
    (out ** 2).sum().backward()
    assert rel_err(out, ref) < TOL[dtype]["out"]
    assert rel_err(Xg.grad, Xo.grad) < TOL[dtype]["grad"]


def test_symmetric_contraction_reference_argument_list(dev, U):
    """The reference's float32 sparse tables passed positionally, as torch.classes.symm_contract does."""
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    maxnz, n3, i3, v3, n2, i2, v2, n1, i1 = oops.pack_sparse_u(*U)  # float32 values like the reference
    g = torch.Generator().manual_seed(0)
    N, C, Z = 40, 64, 3
    X = torch.randn(N, 16, C, generator=g)
    at = torch.randint(0, Z, (N,), generator=g, dtype=torch.int32)
    W = [torch.randn(1, Z, n, C, generator=g) / n for n in (23, 4, 1)]
    ref = oops.symmetric_contraction(X.double(), at, *U, *[w[0].double() for w in W])
    d = lambda t: t.to(dev)
    out = ops.symmetric_contraction_forward(d(X), d(at), maxnz, d(n3), d(i3), d(v3), d(n2), d(i2), d(v2), d(n1), d(i1),
                                            d(W[0]), d(W[1]), d(W[2]), 23, 4, 1)
    assert rel_err(out, ref) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_spherical_harmonics_and_edge_basis(dtype, dev):
    from cuda_mace_b200 import ops
    from oracle import model as omodel
    from oracle.sh import real_sh_l3

    E = 5000
    g = torch.Generator().manual_seed(9)
    xyz = unit_vectors(9, E) * (0.7 + 4.6 * torch.rand(E, 1, generator=g, dtype=torch.float64))
    xyz = xyz.to(dtype)
    xo = xyz.double().clone().requires_grad_(True)
    Yo = real_sh_l3(xo)
    Bo = omodel.radial_embedding(xo.norm(dim=-1), 5.0)
    gy = torch.randn(16, E, generator=g, dtype=torch.float64)
    gb = torch.randn(E, 8, generator=g, dtype=torch.float64)
    (go_y,) = torch.autograd.grad((Yo * gy).sum(), xo, retain_graph=True)
    (go_all,) = torch.autograd.grad((Yo * gy).sum() + (Bo * gb).sum(), xo)
    tol = TOL[dtype]

    xg = xyz.to(dev).requires_grad_(True)
    Y = ops.SphericalHarmonics()(xg)
    assert Y.shape == (16, E) and rel_err(Y, Yo) < tol["out"]
    (gx,) = torch.autograd.grad((Y * gy.to(dtype).to(dev)).sum(), xg)
    assert rel_err(gx, go_y) < tol["grad"]

    xg = xyz.to(dev).requires_grad_(True)
    Y, B = ops.EdgeBasis(5.0, 8, 5)(xg)
    assert rel_err(Y, Yo) < tol["out"] and rel_err(B, Bo) < tol["out"]
    assert B[xyz.norm(dim=-1).to(dev) >= 5.0].abs().max().item() == 0.0
    (gx,) = torch.autograd.grad((Y * gy.to(dtype).to(dev)).sum() + (B * gb.to(dtype).to(dev)).sum(), xg)
    assert rel_err(gx, go_all) < tol["grad"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_cubic_spline(dtype, dev):
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    g = torch.Generator().manual_seed(4)
    nk, F, E = 256, 512, 3000
    knots = torch.linspace(1e-12, 6.0, nk, dtype=torch.float64)
    h = float(knots[1] - knots[0])
    table = torch.randn(nk, F, generator=g, dtype=torch.float64).cumsum(0) * 0.1
    coeffs = oops.cubic_spline_coefficients(knots, table, h)
    assert rel_err(ops.cubic_spline_coefficients(knots, table, h), coeffs) < 1e-13
    r = (0.5 + 5.2 * torch.rand(E, generator=g, dtype=torch.float64)).to(dtype)
    ro = r.double().clone().requires_grad_(True)
    ko, co = knots.to(dtype).double(), coeffs.to(dtype).double()
    ref = oops.cubic_spline_eval(ro, ko, co, float(torch.tensor(h, dtype=dtype)), 5.0)
    (ref ** 2).sum().backward()
    rg = r.to(dev).clone().requires_grad_(True)
    out = ops.cubic_spline_forward(rg, knots.to(dtype).to(dev), coeffs.to(dtype).to(dev), h, 5.0)
    (out ** 2).sum().backward()
    assert out.shape == (E, F)
    assert out[r.to(dev) > 5.0].abs().max().item() == 0.0
    # The table is a random walk, so within an interval the cubic's four terms are each about as large as the
    # largest table value while most results are much smaller: the evaluation keeps a few ulp of the largest TERM,
    # not of the result, and the gradient sums 512 such values per edge.  Hence ten times the operator tolerance
    # here; the smooth table of tests/test_reference_pin.py meets the plain tolerance.
    assert rel_err(out, ref) < TOL[dtype]["out"] * 10
    assert rel_err(rg.grad, ro.grad) < TOL[dtype]["grad"] * 10


def test_golden_fixture_through_the_kernels(dev, U):
    """The committed small fixture (generated by tests/golden/make_golden.py) through the CUDA path."""
    from cuda_mace_b200 import ops

    z = np.load(os.path.join(GOLD, "ops_small.npz"))
    t = {k: torch.from_numpy(z[k]) for k in z.files}
    d = lambda x: x.to(dev)
    N = t["X"].shape[0]
    Y = ops.SphericalHarmonics()(d(t["vec"]))
    assert rel_err(Y, t["Y"]) < 1e-12
    out = ops.InvariantMessagePassingTP()(d(t["X"]), Y, d(t["R"]), d(t["send"]).int(), d(t["recv"]).int(), N)
    assert rel_err(out, t["imp"]) < 1e-12
    W = d(t["W"])
    assert rel_err(ops.linear_forward(d(t["M"]), W, W.transpose(-1, -2).contiguous()), t["lin"]) < 1e-12
    WZ = d(t["WZ"])
    assert rel_err(ops.elemental_linear_forward(d(t["M"]), WZ, WZ.transpose(-1, -2).contiguous(), d(t["at"]).int()),
                   t["elin"]) < 1e-12
    mod = ops.SymmetricContraction(*U, t["W3"], t["W2"], t["W1"]).to(dev)
    assert rel_err(mod(d(t["M"]), d(t["at"]).int()), t["con"]) < 1e-11
    _, B = ops.EdgeBasis(5.0, 8, 5)(d(t["vec"]))
    assert rel_err(B, t["bessel"]) < 1e-12


def test_cpu_tensors_are_rejected():
    from cuda_mace_b200 import ops

    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.SphericalHarmonics()(torch.randn(4, 3))


@pytest.mark.parametrize("M,K,N", [(1000, 64, 512), (300, 8, 64), (129, 64, 64), (257, 512, 64), (64, 64, 8),
                                   (5000, 128, 128), (1, 32, 96),
                                   # column counts that are not a multiple of the 32-column store box, ragged row tails
                                   (513, 64, 40), (777, 96, 136), (40001, 64, 72), (95, 512, 104)])
def test_tensor_core_gemm_has_float32_accuracy(M, K, N, dev):
    """tcgen05 kind::tf32 with the hi/lo split against a float64 matmul: float32-grade, not TF32-grade."""
    from cuda_mace_b200 import ops

    g = torch.Generator().manual_seed(M + K + N)
    A = torch.randn(M, K, generator=g)
    W = torch.randn(K, N, generator=g)
    ref = A.double() @ W.double()
    Ag = A.to(dev).requires_grad_(True)
    out = ops.matmul3x(Ag, W.to(dev))
    ops.check_status()
    assert out.shape == (M, N)
    e_fwd = rel_err(out, ref)
    Gr = torch.randn(M, N, generator=g)
    out.backward(Gr.to(dev))
    ops.check_status()
    e_bwd = rel_err(Ag.grad, Gr.double() @ W.double().t())
    print(f"gemm3x M={M} K={K} N={N}: fwd {e_fwd:.2e} bwd {e_bwd:.2e}")
    # error relative to the largest output; the tensor core's float32 accumulation adds a term that
    # grows with the number of accumulated K steps (measured 5e-7 at K=64, 4e-6 at K=512)
    assert e_fwd < 6e-7 * (1 + K / 64) and e_bwd < 6e-7 * (1 + N / 64)


@pytest.mark.parametrize("M,K,N", [(1000, 8, 64), (517, 64, 512), (300, 512, 64), (129, 128, 1), (64, 3, 5),
                                   (128, 128, 128), (1, 16, 2)])
def test_float64_product_on_the_tensor_cores(M, K, N, dev):
    """cmace_gemm_f64 (DMMA tile loop for even K and N, FMA tiles otherwise) against a float64 host product, value
    and gradient with respect to A."""
    from cuda_mace_b200 import ops

    g = torch.Generator().manual_seed(M + K + N)
    A = torch.randn(M, K, generator=g, dtype=torch.float64)
    W = torch.randn(K, N, generator=g, dtype=torch.float64)
    G = torch.randn(M, N, generator=g, dtype=torch.float64)
    Ad = A.to(dev).requires_grad_(True)
    out = ops.matmul_f64(Ad, W.to(dev))
    (gA,) = torch.autograd.grad(out, Ad, G.to(dev))
    assert rel_err(out, A @ W) < 1e-13
    assert rel_err(gA, G @ W.t()) < 1e-13


def test_tensor_core_and_fma_linear_agree(dev):
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    g = torch.Generator().manual_seed(1)
    X = torch.randn(700, 16, 128, generator=g)
    W = torch.randn(3, 4, 128, 128, generator=g)
    at = torch.randint(0, 3, (700,), generator=g, dtype=torch.int32)
    ref = oops.elemental_linear(X.double(), W.double(), torch.nn.functional.one_hot(at.long(), 3).double())
    Wg = W.to(dev)
    Wt = Wg.transpose(-1, -2).contiguous()
    outs = []
    for flag in (True, False):
        ops.USE_TENSOR_CORES = flag
        try:
            outs.append(ops.elemental_linear_forward(X.to(dev), Wg, Wt, at.to(dev)))
        finally:
            ops.USE_TENSOR_CORES = True
    ops.check_status()
    assert rel_err(outs[0], ref) < 2e-6 and rel_err(outs[1], ref) < 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_contraction_generated_and_table_driven_kernels_agree(dtype, dev, U, monkeypatch):
    """The build-time generated register kernel (selected for the canonical couplings) and the
    table-driven kernel (any tables) give the same numbers; a rescaled U still takes the fast path."""
    from cuda_mace_b200 import _abi, ops
    from oracle import ops as oops

    g = torch.Generator().manual_seed(2)
    N, C, Z = 300, 128, 4
    U3, U2, U1 = U
    U3 = U3 * (0.5 + torch.rand(23, generator=g, dtype=torch.float64))
    X = torch.randn(N, 16, C, generator=g, dtype=torch.float64).to(dtype)
    at = torch.randint(0, Z, (N,), generator=g, dtype=torch.int32)
    W3, W2, W1 = (torch.randn(Z, n, C, generator=g, dtype=torch.float64).to(dtype) / n for n in (23, 4, 1))
    Xo = X.double().clone().requires_grad_(True)
    ref = oops.symmetric_contraction_chunked(Xo, at, U3, U2, U1, W3.double(), W2.double(), W1.double())
    (ref ** 2).sum().backward()
    results = []
    for generic in ("0", "1"):
        monkeypatch.setenv("CMACE_SYMCON_GENERIC", generic)
        mod = ops.SymmetricContraction(U3, U2, U1, W3, W2, W1).to(dev)
        Xg = X.to(dev).clone().requires_grad_(True)
        out = mod(Xg, at.to(dev))
        assert _abi.call("cmace_symcon_plan_is_canonical", mod._plan.handle) == 1
        (out ** 2).sum().backward()
        assert rel_err(out, ref) < TOL[dtype]["out"] and rel_err(Xg.grad, Xo.grad) < TOL[dtype]["grad"]
        results.append((out.detach(), Xg.grad))
    assert rel_err(results[0][0], results[1][0]) < TOL[dtype]["out"]


@pytest.mark.parametrize("E,nb", [(3000, 8), (128, 8), (517, 16), (1, 32), (70000, 8), (400000, 8), (150000, 24)])
def test_hidden_radial_layers_in_one_kernel(E, nb, dev):
    """Three hidden layers with their activations on chip against the oracle's perceptron without its last
    layer: value and gradient with respect to the basis, ragged last tile included."""
    import math

    from cuda_mace_b200 import ops
    from oracle import model as omodel

    g = torch.Generator().manual_seed(13 + E)
    dims = [nb, 64, 64, 64]
    Ws = [torch.randn(dims[i], dims[i + 1], generator=g, dtype=torch.float64).float().double() for i in range(3)]
    b = (torch.randn(E, nb, generator=g, dtype=torch.float64) * 0.7).float().double()
    bo = b.clone().requires_grad_(True)
    # oracle: layers with the activation after every one of them (the perceptron's hidden part)
    h = bo
    for W in Ws:
        h = omodel.silu_n(h @ W / math.sqrt(W.shape[0]))
    gr = torch.randn(E, 64, generator=g, dtype=torch.float64).float()
    (h * gr.double()).sum().backward()
    # kernel weights carry 1/sqrt(fan_in) and, from the second layer on, the activation's constant; the
    # kernel's output lacks the constant of the last activation
    Wn = [(W / math.sqrt(W.shape[0]) * (omodel.SILU_2MOM if i > 0 else 1.0)).float().to(dev) for i, W in enumerate(Ws)]
    bg = b.float().to(dev).requires_grad_(True)
    out = ops.radial_hidden(bg, Wn, [w.t().contiguous() for w in Wn])
    ops.check_status()
    assert out.shape == (E, 64)
    assert rel_err(out * omodel.SILU_2MOM, h) < 5e-6
    out.backward(gr.to(dev) * omodel.SILU_2MOM)
    ops.check_status()
    assert rel_err(bg.grad, bo.grad) < 2e-5


@pytest.mark.parametrize("N,deg,C,K,nsend", [(300, 30, 128, 64, None), (64, 5, 32, 32, None), (200, 52, 64, 64, 260),
                                             (50, 200, 96, 64, None), (3, 1, 128, 64, None)])
def test_message_passing_with_the_last_radial_layer_inside(N, deg, C, K, nsend, dev):
    """R = H @ W formed inside the scatter kernel against the oracle's message passing on the float64 product:
    output, the R it writes for the backward, and the gradients with respect to X, Y and H."""
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    g = torch.Generator().manual_seed(100 + N)
    Ns = N if nsend is None else nsend
    degs = torch.poisson(torch.full((N,), float(deg)), generator=g).long()
    degs[N // 2] = 0  # a receiver without edges
    recv = torch.repeat_interleave(torch.arange(N), degs)
    E = int(recv.numel())
    send = torch.randint(0, Ns, (E,), generator=g)
    X = torch.randn(Ns, C, generator=g, dtype=torch.float64).float().double()
    Y = torch.randn(16, E, generator=g, dtype=torch.float64).float().double()
    H = torch.randn(E, K, generator=g, dtype=torch.float64).float().double()
    W = (torch.randn(K, 4 * C, generator=g, dtype=torch.float64) / K ** 0.5).float().double()
    Xo, Yo, Ho = (t.clone().requires_grad_(True) for t in (X, Y, H))
    ref = oops.invariant_message_passing(Xo, Yo, (Ho @ W).view(E, 4, C), send, recv, N)
    Gr = torch.randn(N, 16, C, generator=g, dtype=torch.float64).float()
    (ref * Gr.double()).sum().backward()

    Xg, Yg, Hg = (t.float().to(dev).requires_grad_(True) for t in (X, Y, H))
    Wg = W.float().to(dev)
    topo = ops.EdgeTopology(send.int().to(dev), recv.int().to(dev), N, Ns)
    out = ops.fused_radial_message_passing(Xg, Yg, Hg, Wg, Wg.t().contiguous(), topo)
    ops.check_status()
    assert rel_err(out, ref) < 1e-5
    assert float(out.detach()[N // 2].abs().max()) == 0.0
    out.backward(Gr.to(dev))
    ops.check_status()
    assert rel_err(Xg.grad, Xo.grad) < 1e-4
    assert rel_err(Yg.grad, Yo.grad) < 1e-4
    assert rel_err(Hg.grad, Ho.grad) < 1e-4


@pytest.mark.parametrize("N,deg,C,K,nsend", [(300, 30, 128, 64, None), (64, 5, 32, 32, None), (200, 52, 64, 64, 260),
                                             (50, 200, 96, 64, None), (3, 1, 128, 64, None), (1000, 40, 128, 64, None)])
def test_message_passing_whose_backward_forms_the_radial_gradient_on_the_fly(N, deg, C, K, nsend, dev):
    """radial_message_passing: out = message passing on R = H @ W; its backward gives grad H without a gradR array
    (rows of gradR are formed inside the tensor-core kernel that multiplies them with W^T).  Against the oracle's
    message passing on the float64 product: output and the gradients with respect to X, Y and H; edge counts that
    are not a multiple of the 128-row tile, ghost senders, a receiver without edges."""
    from cuda_mace_b200 import ops
    from oracle import ops as oops

    g = torch.Generator().manual_seed(200 + N)
    Ns = N if nsend is None else nsend
    degs = torch.poisson(torch.full((N,), float(deg)), generator=g).long()
    degs[N // 2] = 0  # a receiver without edges
    recv = torch.repeat_interleave(torch.arange(N), degs)
    E = int(recv.numel())
    send = torch.randint(0, Ns, (E,), generator=g)
    X = torch.randn(Ns, C, generator=g, dtype=torch.float64).float().double()
    Y = torch.randn(16, E, generator=g, dtype=torch.float64).float().double()
    H = torch.randn(E, K, generator=g, dtype=torch.float64).float().double()
    W = (torch.randn(K, 4 * C, generator=g, dtype=torch.float64) / K ** 0.5).float().double()
    Xo, Yo, Ho = (t.clone().requires_grad_(True) for t in (X, Y, H))
    ref = oops.invariant_message_passing(Xo, Yo, (Ho @ W).view(E, 4, C), send, recv, N)
    Gr = torch.randn(N, 16, C, generator=g, dtype=torch.float64).float()
    (ref * Gr.double()).sum().backward()

    Xg, Yg, Hg = (t.float().to(dev).requires_grad_(True) for t in (X, Y, H))
    Wg = W.float().to(dev)
    topo = ops.EdgeTopology(send.int().to(dev), recv.int().to(dev), N, Ns)
    out = ops.radial_message_passing(Xg, Yg, Hg, Wg, Wg.t().contiguous(), topo)
    assert rel_err(out, ref) < 1e-5
    assert float(out.detach()[N // 2].abs().max()) == 0.0
    out.backward(Gr.to(dev))
    ops.check_status()
    assert rel_err(Xg.grad, Xo.grad) < 1e-4
    assert rel_err(Yg.grad, Yo.grad) < 1e-4
    assert rel_err(Hg.grad, Ho.grad) < 1e-4
    # and the same numbers as the path that writes gradR and multiplies it afterwards
    Xh, Yh, Hh = (t.float().to(dev).requires_grad_(True) for t in (X, Y, H))
    R = ops.matmul3x(Hh, Wg, Wg.t().contiguous()).view(E, 4, C)
    out2 = ops.InvariantMessagePassingTP()(Xh, Yh, R, topo.sender, topo.receiver, N, topology=topo)
    out2.backward(Gr.to(dev))
    assert rel_err(out2, out) < 1e-6
    assert rel_err(Hh.grad, Hg.grad) < 1e-5


def _edge_keys(edge_index, shift_index):
    """One sortable integer per edge: (receiver, sender, shift index triple)."""
    ei = edge_index.long().cpu()
    si = shift_index.long().cpu() + 2
    return torch.sort(((ei[0] * (2 ** 22) + ei[1]) * 125 + (si[:, 0] * 25 + si[:, 1] * 5 + si[:, 2])))[0]


@pytest.mark.parametrize("name,n_atoms,pbc", [("cfg0", None, (True, True, True)), ("water3000", 375, (True, True, True)),
                                              ("water3000", 3000, (True, True, True)), ("slab", 6000, (True, True, False)),
                                              ("cfg0", None, (False, False, False))])
def test_device_neighbor_list_equals_host_list(name, n_atoms, pbc, dev):
    """The cell-list kernels give exactly the host list: same edges, same shifts (bit-exact index work), sorted by
    receiver; also with a box of two cells per axis (cfg0), open boundaries, and receivers = a prefix of the atoms."""
    import numpy as np

    from cuda_mace_b200 import ops, systems

    s = systems.make_system(name, n_atoms=n_atoms)
    pos, box = s["positions"], np.asarray(s["box"], dtype=np.float64)
    lo = np.zeros(3)
    ext = box.copy()
    for d in range(3):
        if not pbc[d]:
            lo[d], ext[d] = pos[:, d].min(), max(pos[:, d].max() - pos[:, d].min(), 1e-6) * (1 + 1e-12) + 1e-9
    for n_recv in (None, pos.shape[0] // 3):
        ei_h, sh_h = systems.neighbor_list(pos, box, pbc, 5.0, n_recv)
        ei_d, sh_d, si_d = ops.neighbor_list(torch.from_numpy(pos).to(dev), ext, pbc, 5.0, n_recv, lo=lo)
        assert ei_d.dtype == torch.int32 and ei_d.shape == (2, ei_h.shape[1])
        assert bool((ei_d[0, 1:] >= ei_d[0, :-1]).all())          # sorted by receiver
        si_h = torch.from_numpy(np.rint(sh_h / box).astype(np.int64))
        assert torch.equal(_edge_keys(ei_d, si_d), _edge_keys(torch.from_numpy(ei_h), si_h))
        assert torch.equal(sh_d.cpu(), si_d.double().cpu() * torch.from_numpy(ext))
        # every vector is inside the cutoff
        p = torch.from_numpy(pos).to(dev)
        v = p[ei_d[1].long()] - p[ei_d[0].long()] + sh_d
        assert float(v.norm(dim=1).max()) < 5.0 if v.numel() else True


def test_device_neighbor_list_without_atoms_or_edges(dev):
    from cuda_mace_b200 import ops

    far = torch.tensor([[1.0, 1.0, 1.0], [20.0, 20.0, 20.0]], dtype=torch.float64, device=dev)
    ei, sh, si = ops.neighbor_list(far, (40.0, 40.0, 40.0), (True, True, True), 5.0)
    assert ei.shape == (2, 0) and sh.shape == (0, 3)
    with pytest.raises(RuntimeError):
        ops.neighbor_list(far, (3.0, 40.0, 40.0), (True, True, True), 5.0)  # periodic axis shorter than the cutoff


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_owned,n_ghost", [(50, 0), (40, 17)])
def test_edge_vectors_and_position_gradient(dtype, n_owned, n_ghost, dev):
    """Edge vectors and their adjoint against index_select / autograd in float64; ghost atoms only send."""
    from cuda_mace_b200 import ops

    g = torch.Generator().manual_seed(7 + n_ghost)
    N = n_owned + n_ghost
    deg = torch.randint(0, 9, (n_owned,), generator=g)
    recv = torch.repeat_interleave(torch.arange(n_owned), deg)
    send = torch.randint(0, N, (recv.numel(),), generator=g)
    E = recv.numel()
    pos = torch.randn(N, 3, generator=g, dtype=torch.float64) * 3
    shifts = torch.randn(E, 3, generator=g, dtype=torch.float64)
    w = torch.randn(E, 3, generator=g, dtype=torch.float64)
    po = pos.clone().requires_grad_(True)
    ref = (po[send] - po[recv] + shifts).to(dtype)
    (ref.double() * w).sum().backward()
    topo = ops.EdgeTopology(send.to(dev), recv.to(dev), n_owned, N)
    pg = pos.to(dev).requires_grad_(True)
    vec = ops.edge_vectors(pg, shifts.to(dev), topo, dtype)
    assert vec.dtype == dtype and torch.equal(vec.cpu(), ref.detach())
    (vec.double() * w.to(dev)).sum().backward()
    tol = 1e-13 if dtype == torch.float64 else 1e-6
    assert rel_err(pg.grad, po.grad) < tol
    # no shifts, no edges
    assert torch.equal(ops.edge_vectors(pg, None, topo, dtype).cpu(), (pos[send] - pos[recv]).to(dtype))
    e = torch.zeros(0, dtype=torch.int32, device=dev)
    assert ops.edge_vectors(pg, None, ops.EdgeTopology(e, e, n_owned, N), dtype).shape == (0, 3)


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(dev):
    """Failure detection without a fault: a kernel waits (bounded) on a barrier nothing completes, gives up after
    50 ms and records a code; check_status() raises with that code, clears it, and the device keeps working."""
    from cuda_mace_b200 import ops

    ops.check_status()
    ops.probe_bounded_wait(dev, code=77, limit_seconds=0.05)
    with pytest.raises(RuntimeError, match="77"):
        ops.check_status()
    ops.check_status()                                   # cleared
    x = torch.randn(8, 16, 32, device=dev)
    w = torch.randn(4, 32, 32, device=dev)
    out = ops.linear_forward(x, w, w.transpose(-1, -2).contiguous())
    assert torch.isfinite(out).all()
    ops.check_status()
