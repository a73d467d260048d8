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


def test_schemas_equal_the_reference_library(classes):
    """Argument names, types and order of forward / __getstate__ / __setstate__ are those the reference's own
    library registers (tests/golden/reference_schemas.json, written by tests/golden/make_reference_schemas.py from
    the library built out of the reference's sources), so positional AND keyword calls written against it work."""
    import json
    import os

    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_schemas.json")) as f:
        ref = json.load(f)
    assert sorted(ref) == sorted(f"{ns}.{name}" for ns, name in CLASSES)
    for ns, name in CLASSES:
        obj = getattr(getattr(classes, ns), name)()
        for method, schema in ref[f"{ns}.{name}"].items():
            assert str(obj._get_method(method).schema) == schema, (ns, name, method)


def _reference_root():
    from oracle import build_ref

    return build_ref.DEFAULT_REFERENCE


REFERENCE_ROOT = _reference_root()


def _load_reference_python(rel_path, name):
    """Loads one of the reference's Python operator modules by file path, with empty stand-ins for the mace / e3nn
    imports at its top (never called here), as tests/golden/make_reference_pins.py does."""
    import importlib.util
    import os
    import sys
    import types

    for mod in ("e3nn", "mace", "mace.tools", "mace.tools.cg", "mace.modules", "mace.modules.symmetric_contraction"):
        sys.modules.setdefault(mod, types.ModuleType(mod))
    sys.modules["e3nn"].o3 = types.SimpleNamespace(Linear=object)
    sys.modules["mace.tools.cg"].U_matrix_real = None
    sys.modules["mace.modules.symmetric_contraction"].SymmetricContraction = object
    spec = importlib.util.spec_from_file_location(name, os.path.join(REFERENCE_ROOT, rel_path))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_reference_python_layer_binds_to_this_library(classes):
    """The drop-in seen from the reference's side: its own Python operator modules (cuda_mace/ops/*.py), loaded by
    file path, find every handle they ask for in THIS library (ops/__init__.py:7-15 only loads a library; the
    modules then call torch.classes.<ns>.<Class>()), and the argument lists their forward methods pass
    (ops/invariant_message_passing.py:20-22, ops/linear.py:54,:108, ops/symmetric_contraction.py:68-86,
    ops/cubic_spline.py:35-37) bind to the registered schemas.  Runs where the reference checkout is (no GPU
    needed); the numerical side of the same classes is test_*_class above."""
    import inspect
    import os

    if not os.path.isdir(os.path.join(REFERENCE_ROOT, "cuda_mace", "ops")):
        pytest.skip("no reference checkout on this machine")
    imp = _load_reference_python("cuda_mace/ops/invariant_message_passing.py", "ref_ops_imp")
    mod = imp.InvariantMessagePassingTP()          # constructs torch.classes.inv_message_passing....()
    assert "inv_message_passing.InvariantMessagePassingTP" in str(mod.cuda_obj._type())
    lin = _load_reference_python("cuda_mace/ops/linear.py", "ref_ops_linear")
    spl = _load_reference_python("cuda_mace/ops/cubic_spline.py", "ref_ops_spline")
    sym = _load_reference_python("cuda_mace/ops/symmetric_contraction.py", "ref_ops_symcon")
    # number of arguments each reference forward hands to cuda_obj.forward == arguments of the registered schema
    expected = {(imp.InvariantMessagePassingTP, "inv_message_passing", "InvariantMessagePassingTP"): 6,
                (lin.Linear, "linear_wmma", "Linear"): 3, (lin.ElementalLinear, "linear_wmma", "ElementalLinear"): 4,
                (spl.CubicSpline, "cubic_spline", "CubicSpline"): 5,
                (sym.SymmetricContraction, "symm_contract", "SymmetricContraction"): 17}
    for (cls, ns, name), nargs in expected.items():
        src = inspect.getsource(cls.forward)
        assert "self.cuda_obj.forward(" in src
        schema = getattr(getattr(classes, ns), name)()._get_method("forward").schema
        assert len(schema.arguments) - 1 == nargs, (name, schema)
    # the spline module builds its coefficient table with plain torch: run it and check it is what this
    # project's packing produces (the table is an argument of the class's forward)
    from cuda_mace_b200 import ops

    knots = torch.linspace(1e-12, 6.0, 17, dtype=torch.float64)
    vals = torch.sin(knots)[:, None] * torch.arange(1, 5, dtype=torch.float64)
    h = float(knots[1] - knots[0])
    theirs = spl.CubicSpline.cubic_spline_coefficients(None, knots, vals, h)
    assert rel_err(ops.cubic_spline_coefficients(knots, vals, h), theirs) < 1e-12


@pytest.mark.gpu
def test_weight_caches_do_not_outlive_their_tensors(classes):
    """Temporary weights of the same shape, each freed before the next is made: the caching allocator may hand
    the next one the same address, and the packed-image cache must not answer with the previous image.  (A cache
    entry keeps its source tensor alive, so while the entry lives that address cannot come back at all.)"""
    from oracle import ops as oops

    g = torch.Generator().manual_seed(9)
    N, K = 64, 64
    X = torch.randn(N, 16, K, generator=g)
    lin = classes.linear_wmma.Linear()
    with torch.no_grad():
        for trial in range(4):
            W = torch.randn(4, K, K, generator=g)
            Wd = W.cuda()
            WTd = W.transpose(-1, -2).contiguous().cuda()
            out = lin.forward(X.cuda(), Wd, WTd)
            assert rel_err(out, oops.linear(X.double(), W.double())) < 1e-5, trial
            del Wd, WTd, out


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_elemental_linear_class_single_species(classes, dtype):
    """Z = 1 (the reference's own test cells are single-species diamond): every node uses W[0]."""
    from oracle import ops as oops

    tol = 1e-10 if dtype == torch.float64 else 1e-4
    g = torch.Generator().manual_seed(12)
    N, K = 50, 64
    X = torch.randn(N, 16, K, generator=g, dtype=torch.float64).to(dtype)
    WZ = torch.randn(1, 4, K, K, generator=g, dtype=torch.float64).to(dtype)
    one_hot = torch.ones(N, 1, dtype=dtype)
    Xo = X.double().clone().requires_grad_(True)
    ref = oops.elemental_linear(Xo, WZ.double(), one_hot.double())
    (ref ** 2).sum().backward()
    Xg = X.cuda().requires_grad_(True)
    out = classes.linear_wmma.ElementalLinear().forward(Xg, WZ.cuda(), WZ.transpose(-1, -2).contiguous().cuda(),
                                                        one_hot.cuda())
    (out ** 2).sum().backward()
    assert rel_err(out, ref) < tol and rel_err(Xg.grad, Xo.grad) < tol


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_elemental_linear_class_on_grouped_and_on_shuffled_nodes(classes, dtype):
    """The class caches the element grouping of a one-hot matrix and passes no gather list when the nodes are stored
    grouped by element (whole-node boxes by TMA in float32); the same nodes in random order take the gather list.
    Both against the oracle, twice in a row with the same one-hot tensor (second call: cached grouping), and once
    more after the tensor was edited in place (the cache must not serve the old grouping)."""
    from oracle import ops as oops
    from cuda_mace_b200 import systems

    tol = 1e-10 if dtype == torch.float64 else 1e-4
    g = torch.Generator().manual_seed(21)
    N, K, Z = 700, 128, 4
    X = torch.randn(N, 16, K, generator=g, dtype=torch.float64).to(dtype)
    WZ = torch.randn(Z, 4, K, K, generator=g, dtype=torch.float64).to(dtype)
    Wg, WTg = WZ.cuda(), WZ.transpose(-1, -2).contiguous().cuda()
    at_sorted = torch.sort(torch.randint(0, Z, (N,), generator=g)).values
    for at in (at_sorted, at_sorted[torch.randperm(N, generator=g)]):
        one_hot = systems.one_hot(at, Z).to(dtype)
        Xo = X.double().clone().requires_grad_(True)
        ref = oops.elemental_linear(Xo, WZ.double(), one_hot.double())
        (ref ** 2).sum().backward()
        oh = one_hot.cuda()
        for _ in range(2):
            Xg = X.cuda().requires_grad_(True)
            out = classes.linear_wmma.ElementalLinear().forward(Xg, Wg, WTg, oh)
            (out ** 2).sum().backward()
            assert rel_err(out, ref) < tol and rel_err(Xg.grad, Xo.grad) < tol
        # in-place edit: node 0 moves to the last element
        oh[0] = 0.0
        oh[0, Z - 1] = 1.0
        at2 = at.clone()
        at2[0] = Z - 1
        ref2 = oops.elemental_linear(X.double(), WZ.double(), systems.one_hot(at2, Z).double())
        out2 = classes.linear_wmma.ElementalLinear().forward(X.cuda(), Wg, WTg, oh)
        assert rel_err(out2, ref2) < tol
    assert int(torch.ops.cmace_b200_internal.check_status()) == 0


@pytest.mark.gpu
def test_keyword_call_and_status_op(classes):
    """A keyword call with the reference's argument names (including its spelling "raidal"), and the status
    operator that reports kernels whose bounded waits gave up (0 = none did)."""
    send, recv = random_graph(4, 30, 6)
    E = send.numel()
    g = torch.Generator().manual_seed(2)
    X, Y, R = torch.randn(30, 32, generator=g).cuda(), torch.randn(16, E, generator=g).cuda(), \
        torch.randn(E, 4, 32, generator=g).cuda()
    tp = classes.inv_message_passing.InvariantMessagePassingTP()
    a = tp.forward(X, Y, R, send.cuda(), recv.cuda(), 30)
    b = tp.forward(X=X, Y=Y, raidal=R, sender_list=send.cuda(), receiver_list=recv.cuda(), nnodes=30)
    assert torch.equal(a, b)
    assert torch.ops.cmace_b200_internal.check_status() == 0
