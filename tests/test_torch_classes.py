"""The TorchScript custom classes registered under the reference's names: registration and pickling on the CPU,
values and gradients against the oracle on the GPU with the reference's positional argument lists."""
import io

import pytest
import torch

from tests.util import random_graph, rel_err

CLASSES = [("inv_message_passing", "InvariantMessagePassingTP"), ("symm_contract", "SymmetricContraction"),
           ("linear_wmma", "Linear"), ("linear_wmma", "ElementalLinear"),
           ("spherical_harmonics", "SphericalHarmonics"), ("cubic_spline", "CubicSpline")]


@pytest.fixture(scope="module")
def classes():
    from cuda_mace_b200 import torch_classes

    torch_classes.load()
    return torch.classes


@pytest.mark.parametrize("ns,name", CLASSES)
def test_classes_register_and_pickle(classes, ns, name):
    """No-argument construction, a forward method, and pickling with an empty state, as the reference's classes
    (cuda_mace/src/*.cpp, def_pickle with an empty tensor list)."""
    obj = getattr(getattr(classes, ns), name)()
    assert hasattr(obj, "forward")
    buf = io.BytesIO()
    torch.save(obj, buf)
    buf.seek(0)
    again = torch.load(buf, weights_only=False)
    assert hasattr(again, "forward")


def test_cpu_tensors_are_rejected_by_the_classes(classes):
    with pytest.raises(RuntimeError):
        classes.spherical_harmonics.SphericalHarmonics().forward(torch.zeros(4, 3))
    with pytest.raises(RuntimeError):
        classes.linear_wmma.Linear().forward(torch.zeros(2, 16, 8), torch.zeros(4, 8, 8), torch.zeros(4, 8, 8))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_message_passing_class(classes, dtype):
    from oracle import ops as oops

    tol = 1e-10 if dtype == torch.float64 else 1e-4
    N, C = 150, 64
    send, recv = random_graph(3, N, 12, empty_every=17)
    E = send.numel()
    g = torch.Generator().manual_seed(5)
    X, Y, R = (torch.randn(*s, generator=g, dtype=torch.float64) for s in ((N, C), (16, E), (E, 4, C)))
    Xo, Yo, Ro = (t.to(dtype).double().clone().requires_grad_(True) for t in (X, Y, R))
    ref = oops.invariant_message_passing(Xo, Yo, Ro, send, recv, N)
    (ref ** 2).sum().backward()
    Xg, Yg, Rg = (t.detach().to(dtype).cuda().requires_grad_(True) for t in (X, Y, R))
    out = classes.inv_message_passing.InvariantMessagePassingTP().forward(Xg, Yg, Rg, send.int().cuda(),
                                                                         recv.int().cuda(), N)
    (out ** 2).sum().backward()
    assert rel_err(out, ref) < tol
    for a, b in ((Xg, Xo), (Yg, Yo), (Rg, Ro)):
        assert rel_err(a.grad, b.grad) < tol


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_linear_classes(classes, dtype):
    from oracle import ops as oops

    tol = 1e-10 if dtype == torch.float64 else 1e-4
    g = torch.Generator().manual_seed(6)
    N, K, Z = 70, 64, 3
    X = torch.randn(N, 16, K, generator=g, dtype=torch.float64).to(dtype)
    W = torch.randn(4, K, K, generator=g, dtype=torch.float64).to(dtype)
    Xo = X.double().clone().requires_grad_(True)
    ref = oops.linear(Xo, W.double())
    (ref ** 2).sum().backward()
    Xg = X.detach().cuda().requires_grad_(True)
    out = classes.linear_wmma.Linear().forward(Xg, W.cuda(), W.transpose(-1, -2).contiguous().cuda())
    (out ** 2).sum().backward()
    assert rel_err(out, ref) < tol and rel_err(Xg.grad, Xo.grad) < tol

    WZ = torch.randn(Z, 4, K, K, generator=g, dtype=torch.float64).to(dtype)
    elem = torch.randint(0, Z, (N,), generator=g)
    one_hot = torch.nn.functional.one_hot(elem, Z).to(dtype)
    Xo2 = X.double().clone().requires_grad_(True)
    ref2 = oops.elemental_linear(Xo2, WZ.double(), one_hot.double())
    (ref2 ** 2).sum().backward()
    Xg2 = X.detach().cuda().requires_grad_(True)
    out2 = classes.linear_wmma.ElementalLinear().forward(Xg2, WZ.cuda(), WZ.transpose(-1, -2).contiguous().cuda(),
                                                         one_hot.cuda())
    (out2 ** 2).sum().backward()
    assert rel_err(out2, ref2) < tol and rel_err(Xg2.grad, Xo2.grad) < tol


@pytest.mark.gpu
def test_contraction_harmonics_and_spline_classes(classes, U):
    from oracle import ops as oops
    from oracle import sh as osh

    d = lambda t: t.cuda()
    maxnz, n3, i3, v3, n2, i2, v2, n1, i1 = oops.pack_sparse_u(*U)
    g = torch.Generator().manual_seed(1)
    N, C, Z = 40, 64, 3
    X = torch.randn(N, 16, C, generator=g)
    at = torch.randint(0, Z, (N,), generator=g, dtype=torch.int32)
    W = [torch.randn(1, Z, n, C, generator=g) / n for n in (23, 4, 1)]
    Xo = X.double().requires_grad_(True)
    ref = oops.symmetric_contraction(Xo, at, *U, *[w[0].double() for w in W])
    (ref ** 2).sum().backward()
    Xg = d(X).requires_grad_(True)
    out = classes.symm_contract.SymmetricContraction().forward(
        Xg, d(at), maxnz, d(n3), d(i3), d(v3), d(n2), d(i2), d(v2), d(n1), d(i1), d(W[0]), d(W[1]), d(W[2]), 23, 4, 1)
    (out ** 2).sum().backward()
    assert out.shape == (N, 1, C)
    assert rel_err(out, ref) < 1e-5 and rel_err(Xg.grad, Xo.grad) < 1e-4

    xyz = torch.randn(500, 3, generator=g, dtype=torch.float64)
    xo = xyz.clone().requires_grad_(True)
    yref = osh.real_sh_l3(xo)
    gy = torch.randn(16, 500, generator=g, dtype=torch.float64)  # (Y**2).sum() is constant on the sphere
    (yref * gy).sum().backward()
    xg = d(xyz).requires_grad_(True)
    y = classes.spherical_harmonics.SphericalHarmonics().forward(xg)
    (y * d(gy)).sum().backward()
    assert y.shape == (16, 500)
    assert rel_err(y, yref) < 1e-10 and rel_err(xg.grad, xo.grad) < 1e-10

    knots = torch.linspace(1e-12, 6.0, 33, dtype=torch.float64)
    h = float(knots[1] - knots[0])
    vals = torch.randn(33, 12, generator=g, dtype=torch.float64)
    coeffs = oops.cubic_spline_coefficients(knots, vals, h)
    r = 0.5 + 5.2 * torch.rand(300, generator=g, dtype=torch.float64)
    ro = r.clone().requires_grad_(True)
    rref = oops.cubic_spline_eval(ro, knots, coeffs, h, 5.0)
    (rref ** 2).sum().backward()
    rg = d(r).requires_grad_(True)
    out = classes.cubic_spline.CubicSpline().forward(rg, d(knots), d(coeffs), h, 5.0)
    (out ** 2).sum().backward()
    assert rel_err(out, rref) < 1e-10 and rel_err(rg.grad, ro.grad) < 1e-10
