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

Parity status.  PINNED against the reference's own kernels: oracle/build_ref.py builds the reference's library
from its sources, oracle/ref_run.py runs its six operator classes (and an energy+force step re-assembled from them,
oracle/ref_model.py) on a B200, and tests/test_reference_pin.py holds this restatement and the CUDA library to those
outputs, both through committed fixtures (tests/golden/reference_ops_b200.npz) and live where the built library is
present.  Also pinned, against the reference's Python run on the CPU (tests/golden/make_reference_pins.py): the
sparse packing of the U tensors (cuda_mace/ops/symmetric_contraction.py:91-187, bit for bit) and the natural-spline
coefficient solve (cuda_mace/ops/cubic_spline.py:41-84).

PARITY UNPINNED against upstream MACE / e3nn for what the reference borrows from them and this environment cannot
install: the Bessel basis, polynomial cutoff, radial perceptron, readout normalisations and the scale and sign of
each symmetric class of generalised Clebsch-Gordan paths are restated from the published definitions.
"""
