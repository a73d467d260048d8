"""CPU restatement (float64, PyTorch on the host) of the invariant-MACE energy+force path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is the checker used by the tests, by the smoke entry and by the
CPU-baseline legs of the benchmark.  The product path runs CUDA kernels through
the C-ABI library and raises when that library is missing.

What it restates (paths are relative to the cuda-mace project):

* spherical harmonics            cuda_mace/cuda/src/spherical_harmonics_impl.cu:62-125
* cubic spline radial table      cuda_mace/ops/cubic_spline.py:41-84,
                                 cuda_mace/cuda/src/cubic_spline_impl.cu:5-107
* invariant message passing      cuda_mace/cuda/src/invariant_message_passing_impl.cu:74-399
* Linear / ElementalLinear       cuda_mace/cuda/src/linear_impl.cu:16-255,
                                 cuda_mace/ops/linear.py:9-108
* symmetric contraction          cuda_mace/cuda/src/symmetric_contraction_impl.cu:6-234,
                                 cuda_mace/ops/symmetric_contraction.py:91-232
* model wiring                   cuda_mace/models/InvariantMACE.py:77-165, :246-379

Parity status: the reference holds no golden vectors and its own tests compare
against live `mace` / `e3nn` installs (tests/*.py), neither of which exists in
this environment.  The Bessel basis, polynomial cutoff, radial MLP, readout and
generalised Clebsch-Gordan conventions are therefore restated from the published
MACE / e3nn definitions: PARITY UNPINNED against upstream MACE for those parts.
The operator semantics that live in the reference tree itself (the files listed
above) are followed line by line and the small committed fixtures under
tests/golden/ freeze this restatement's outputs.

PINNED against the reference's own code, run on seeded inputs
(tests/golden/make_reference_pins.py -> tests/golden/reference_pins.npz): the
sparse packing of the U tensors (cuda_mace/ops/symmetric_contraction.py:91-187,
bit for bit) and the natural-spline coefficient solve
(cuda_mace/ops/cubic_spline.py:41-84).  The reference's kernels themselves only
run on a GPU through its cmake / NVRTC build, which this project does not run.
"""
