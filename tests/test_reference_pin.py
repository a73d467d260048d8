"""Operator parity pinned against the REFERENCE'S OWN kernels.

Three sources meet on the same seeded inputs (oracle/ref_cases.py):
  reference   the reference's TorchScript classes over its NVRTC-compiled kernels, run on a B200
              (oracle/ref_run.py over oracle/_ref/libcuda_mace.so, built by oracle/build_ref.py);
  oracle      the float64 CPU restatement (oracle/);
  product     this library's kernels through the C-ABI (cuda_mace_b200.ops).

* tests/golden/reference_ops_b200.npz holds the reference's outputs on the small "fixture" cases, produced on a
  B200 by `python -m oracle.ref_run parity --size fixture --out tests/golden/reference_ops_b200.npz`.  The CPU
  tests check the oracle against it; the GPU tests check the product against it.
* When the reference library is present (it travels with the repository, git-ignored), the GPU tests also run
  the reference live in a child process on the larger "live" cases (128 channels, the template instances the
  model uses) and on a whole energy+force step, and compare all three.

Tolerances: the reference computes in float32 for the model and its float64 templates exist for every operator but
Linear; against the float64 oracle a float32 result is held to 1e-5 (outputs) / 1e-4 (gradients) relative to the
largest magnitude of the tensor, a float64 one to 1e-10.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.util import TOL, rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FIXTURE = os.path.join(ROOT, "tests", "golden", "reference_ops_b200.npz")
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcuda_mace.so")

# which results are compared, and the tolerance class of each
KEYS = {
    "sh": (("out", "out"), ("grad_xyz", "grad")),
    "spline": (("out", "out"), ("grad_r", "grad")),
    "imp": (("out", "out"), ("grad_X", "grad"), ("grad_Y", "grad"), ("grad_R", "grad")),
    "symcon": (("out", "out"), ("grad_X", "grad")),
    "linear": (("out", "out"), ("grad_X", "grad")),
    "elinear": (("out", "out"), ("grad_X", "grad")),
}
DTYPES = {"f32": torch.float32, "f64": torch.float64}
# The reference keeps the U values in float32 tables whatever the dtype of X (const float *U3_values,
# symmetric_contraction_impl.cu:11,:14), so its float64 contraction carries float32 rounding of the couplings.
LOOSER = {("symcon", "f64"): 1e-6}


def _ops_with_dtype(ref):
    for op in KEYS:
        for tag in DTYPES:
            if f"{op}.{tag}.out" in ref:
                yield op, tag


def _compare(got, want, op, tag, what):
    """got, want: dicts name -> tensor/array for one operator."""
    for name, kind in KEYS[op]:
        a = torch.as_tensor(np.asarray(got[name])) if not torch.is_tensor(got[name]) else got[name]
        b = torch.as_tensor(np.asarray(want[name])) if not torch.is_tensor(want[name]) else want[name]
        err = rel_err(a, b)
        tol = LOOSER.get((op, tag), TOL[DTYPES[tag]][kind])
        assert err < tol, f"{what}: {op}.{tag}.{name} differs by {err:.3e}"


@pytest.fixture(scope="module")
def oracle_cache():
    from oracle import cg, ref_cases

    cache = {}

    def get(size):
        if size not in cache:
            cache[size] = ref_cases.oracle_results(size, cg.u_matrices())
        return cache[size]
    return get


def product_results(size, dtype):
    """This library's operators (cuda_mace_b200.ops -> C-ABI) on the cases of oracle.ref_cases."""
    from cuda_mace_b200 import cg, ops
    from oracle import ref_cases

    d = dict(dtype=dtype, device="cuda")
    res = {}

    def grads(out, G, inputs):
        return torch.autograd.grad((out * G.to(**d)).sum(), inputs)

    c = ref_cases.case_sh(size)
    xyz = c["xyz"].to(**d).requires_grad_(True)
    Y = ops.SphericalHarmonics()(xyz)
    res["sh"] = dict(out=Y, grad_xyz=grads(Y, c["G"], (xyz,))[0])
    c = ref_cases.case_spline(size)
    r = c["r"].to(**d).requires_grad_(True)
    R = ops.cubic_spline_forward(r, c["knots"].to(**d), c["coeffs"].to(**d), c["h"], c["r_max"])
    res["spline"] = dict(out=R, grad_r=grads(R, c["G"], (r,))[0])
    c = ref_cases.case_imp(size)
    X, Y, R = (c[k].to(**d).contiguous().requires_grad_(True) for k in ("X", "Y", "R"))
    out = ops.InvariantMessagePassingTP()(X, Y, R, c["sender"].cuda(), c["receiver"].cuda(), c["nnodes"])
    gX, gY, gR = grads(out, c["G"], (X, Y, R))
    res["imp"] = dict(out=out, grad_X=gX, grad_Y=gY, grad_R=gR)
    U = cg.u_matrices()
    c = ref_cases.case_symcon(size, U)
    X = c["X"].to(**d).requires_grad_(True)
    mod = ops.SymmetricContraction(*U, c["W3"].to(dtype), c["W2"].to(dtype), c["W1"].to(dtype)).cuda()
    out = mod(X, c["atom_types"].cuda())
    res["symcon"] = dict(out=out, grad_X=grads(out, c["G"], (X,))[0])
    c = ref_cases.case_linear(size)
    X = c["X"].to(**d).requires_grad_(True)
    W = c["W"].to(**d).contiguous()
    out = ops.linear_forward(X, W, W.transpose(-1, -2).contiguous())
    res["linear"] = dict(out=out, grad_X=grads(out, c["G"], (X,))[0])
    X = c["X"].to(**d).requires_grad_(True)
    W = c["WE"].to(**d).contiguous()
    out = ops.elemental_linear_forward(X, W, W.transpose(-1, -2).contiguous(), c["one_hot"].to(**d))
    res["elinear"] = dict(out=out, grad_X=grads(out, c["G"], (X,))[0])
    ops.check_status()
    return res


def _split(npz, op, tag):
    return {name: npz[f"{op}.{tag}.{name}"] for name, _ in KEYS[op]}


# ---------------------------------------------------------------------------------------------------------------
# committed outputs of the reference (CPU: oracle; GPU: product)
# ---------------------------------------------------------------------------------------------------------------
def test_oracle_matches_reference_outputs(oracle_cache):
    """The float64 restatement against what the reference's kernels produced on a B200, every operator, float32 and
    float64 templates: this is the pin of the oracle's operator numerics against the reference itself."""
    ref = np.load(FIXTURE)
    ora = oracle_cache("fixture")
    seen = 0
    for op, tag in _ops_with_dtype(ref):
        _compare(_split(ref, op, tag), {name: ora[f"{op}.{name}"] for name, _ in KEYS[op]}, op, tag,
                 "reference vs oracle")
        seen += 1
    assert seen == 10   # sh, spline, imp, symcon in two dtypes; linear, elinear in float32


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_product_matches_reference_outputs(tag):
    ref = np.load(FIXTURE)
    got = product_results("fixture", DTYPES[tag])
    for op in KEYS:
        if f"{op}.{tag}.out" in ref:
            _compare(got[op], _split(ref, op, tag), op, tag, "product vs reference")


# ---------------------------------------------------------------------------------------------------------------
# the reference run live, next to the product, on the same device
# ---------------------------------------------------------------------------------------------------------------
def _run_reference(args, out):
    """python -m oracle.ref_run ... in a child process (the two libraries register the same class names)."""
    if not os.path.isfile(REF_LIB):
        pytest.skip("oracle/_ref/libcuda_mace.so is not built (python -m oracle.build_ref needs the reference sources)")
    cmd = [sys.executable, "-m", "oracle.ref_run"] + args + ["--out", out]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, f"reference run failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    return np.load(out)


@pytest.fixture(scope="module")
def reference_live(tmp_path_factory):
    return _run_reference(["parity", "--size", "live"], str(tmp_path_factory.mktemp("ref") / "live.npz"))


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["f32", "f64"])
def test_live_reference_product_and_oracle_agree(reference_live, oracle_cache, tag):
    """128 channels, 300 receivers / 7 426 edges, 256 nodes x 10 elements: reference kernels, this library and the
    oracle on identical tensors."""
    ora = oracle_cache("live")
    got = product_results("live", DTYPES[tag])
    for op in KEYS:
        if f"{op}.{tag}.out" not in reference_live:
            continue
        want = _split(reference_live, op, tag)
        _compare(want, {name: ora[f"{op}.{name}"] for name, _ in KEYS[op]}, op, tag, "reference vs oracle")
        _compare(got[op], want, op, tag, "product vs reference")


@pytest.mark.gpu
def test_whole_step_against_the_reference_operators(tmp_path, U):
    """Energy and forces of 375 atoms (4 species, 128 channels): the reference's step re-assembled from its own
    classes (oracle/ref_model.py: float32, 256-knot spline, as models/InvariantMACE.py runs it), this library with
    the same tabulated radial path, and the float64 oracle.  float32 tolerances: 1e-5 energy, 1e-4 forces."""
    from cuda_mace_b200 import model
    from oracle import model as omodel
    from oracle import ref_run

    atoms, channels, species = 375, 128, 4
    ref = _run_reference(["model", "--atoms", str(atoms), "--channels", str(channels), "--species", str(species)],
                         str(tmp_path / "model.npz"))
    pos, z, ei, sh, params = ref_run.model_system(atoms, channels, species, seed=1)
    from cuda_mace_b200 import systems

    omodel.add_spline_tables(params)
    _, e_o, f_o = omodel.energy_and_forces(params, U, torch.from_numpy(pos), systems.one_hot(z, species),
                                           torch.from_numpy(ei), torch.from_numpy(sh), radial="spline")
    data = dict(positions=torch.from_numpy(pos).cuda(), species=torch.from_numpy(z).to(torch.int32).cuda(),
                edge_index=torch.from_numpy(ei).to(torch.int32).cuda(), shifts=torch.from_numpy(sh).cuda())
    out = model.InvariantMACE(params, U, dtype=torch.float32, device="cuda", radial="spline")(data)
    e_p, f_p = float(out["interaction_energy"]), out["forces"].cpu()
    e_r, f_r = float(ref["energy"]), torch.from_numpy(ref["forces"])
    scale_f = float(f_o.abs().max())
    for what, e, f in (("reference vs oracle", e_r, f_r), ("product vs oracle", e_p, f_p)):
        assert abs(e - float(e_o)) / abs(float(e_o)) < 1e-5, (what, e, float(e_o))
        assert float((f - f_o).abs().max()) / scale_f < 1e-4, what
    assert abs(e_p - e_r) / abs(e_r) < 1e-5
    assert float((f_p - f_r).abs().max()) / scale_f < 1e-4


def test_reference_gradient_rule_needs_symmetric_tables(U):
    """The reference's contraction kernel forms its gradient from one stored value and the weights of three
    permuted paths (symmetric_contraction_impl.cu:160-169).  oracle.ops.symmetric_contraction_sparse_tables restates
    that loop; here: (1) it reproduces the gradient the reference's kernel wrote on the B200 (committed outputs),
    (2) on this project's U tensors, which are symmetric under a simultaneous permutation of indices and path, it
    equals the exact derivative (what this library computes), (3) on tables without that symmetry (one path's sign
    flipped, which the forward absorbs into the weights) it does not -- the reason the sign rule of the U tensors
    is the permutation-invariant one."""
    from oracle import ops as oops
    from oracle import ref_cases

    c = ref_cases.case_symcon("fixture", U)
    ref = np.load(FIXTURE)
    out, grad = oops.symmetric_contraction_sparse_tables(c["X"], c["atom_types"], c["tables"], c["W3"], c["W2"], c["W1"])
    assert rel_err(out[:, None], torch.from_numpy(ref["symcon.f64.out"])) < 1e-12
    assert rel_err(grad * c["G"], torch.from_numpy(ref["symcon.f64.grad_X"])) < 1e-12
    X = c["X"].clone().requires_grad_(True)
    exact = oops.symmetric_contraction(X, c["atom_types"], *U, c["W3"], c["W2"], c["W1"])
    (gx,) = torch.autograd.grad(exact.sum(), X)
    assert rel_err(grad, gx) < 1e-7          # float32 table values
    flipped = U[0].clone()
    flipped[..., 1] = -flipped[..., 1]       # path (0,1,1) but not (1,0,1), (1,1,0)
    Uf = (flipped, U[1], U[2])
    X = c["X"].clone().requires_grad_(True)
    exact = oops.symmetric_contraction(X, c["atom_types"], *Uf, c["W3"], c["W2"], c["W1"])
    (gx,) = torch.autograd.grad(exact.sum(), X)
    out, grad = oops.symmetric_contraction_sparse_tables(c["X"], c["atom_types"], oops.pack_sparse_u(*Uf), c["W3"],
                                                         c["W2"], c["W1"])
    assert rel_err(out[:, None], exact) < 1e-7
    assert rel_err(grad, gx) > 1e-3
