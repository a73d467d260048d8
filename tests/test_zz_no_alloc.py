"""The entry point for callers that cannot allocate device memory: cmace_imp_bwd_edge_f64_noalloc keeps
its scratch in an array inside the library, so it is called with inputs and outputs only.  Checked through
the C-ABI against cmace_imp_bwd_edge_f64 (caller-provided scratch) and against the oracle's gradients on two calls
in a row, the second with different data, so stale contents of the shared array would show.  Collected last on
purpose."""
import pytest
import torch

from tests.util import random_graph, rel_err

pytestmark = pytest.mark.gpu


def run_pair(seed, N, deg, C, dev):
    from cuda_mace_b200 import _abi, ops

    send, recv = random_graph(seed, N, deg, empty_every=6)
    E = send.numel()
    g = torch.Generator().manual_seed(seed)
    X, Y, R, G = (torch.randn(*shape, generator=g, dtype=torch.float64).to(dev)
                  for shape in ((N, C), (16, E), (E, 4, C), (N, 16, C)))
    topo = ops.EdgeTopology(send.to(dev), recv.to(dev), N)
    p = lambda t: t.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for variant in ("reference", "noalloc"):
        gradR, gradY, T = torch.full_like(R, float("nan")), torch.full_like(Y, float("nan")), torch.full((E, C), float("nan"), dtype=torch.float64, device=dev)
        if variant == "reference":
            n = _abi.call("cmace_imp_bwd_scratch_elems", E, C, 1)
            assert n > 0  # float64 at C = 128 needs the two-chunk scratch: this is the path under test
            scratch = torch.empty(n, dtype=torch.float64, device=dev)
            _abi.call("cmace_imp_bwd_edge_f64", p(X), p(Y), p(R), p(G), p(topo.sender), p(topo.row_ptr), N, E, C,
                      p(gradR), p(gradY), p(T), p(scratch), stream)
        else:
            _abi.call("cmace_imp_bwd_edge_f64_noalloc", p(X), p(Y), p(R), p(G), p(topo.sender), p(topo.row_ptr), N, E,
                      C, p(gradR), p(gradY), p(T), stream)
        torch.cuda.synchronize()
        outs.append((gradR, gradY, T))
    for a, b in zip(*outs):
        assert not torch.isnan(b).any()
        assert rel_err(b, a) < 1e-10  # the float64 tolerance of the other operator tests
    # and against the oracle's gradients of sum(out * G): dL/dR, dL/dY, and dL/dX = the T rows summed per sender
    from oracle import ops as oops

    Xo, Yo, Ro = (t.cpu().clone().requires_grad_(True) for t in (X, Y, R))
    out = oops.invariant_message_passing(Xo, Yo, Ro, send.long(), recv.long(), N)
    (out * G.cpu()).sum().backward()
    gradR, gradY, T = outs[1]
    assert rel_err(gradR.cpu(), Ro.grad) < 1e-10
    assert rel_err(gradY.cpu(), Yo.grad) < 1e-10
    gradX = torch.zeros(N, C, dtype=torch.float64).index_add_(0, send.long(), T.cpu())
    assert rel_err(gradX, Xo.grad) < 1e-10


def test_noalloc_entry_point_matches_on_two_calls_in_a_row():
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    run_pair(1, 400, 24, 128, dev)
    run_pair(2, 150, 9, 128, dev)   # smaller second call: leftovers of the first must not leak in


def test_noalloc_rejects_sizes_beyond_the_built_in_array():
    from cuda_mace_b200 import _abi

    lib = _abi.load()
    limit = _abi.call("cmace_imp_bwd_edge_f64_noalloc_max_elems")
    too_many_edges = limit // 32 + 1   # 2 chunks x 16 components per edge at C = 128
    rc = lib.cmace_imp_bwd_edge_f64_noalloc(None, None, None, None, None, None, 10, too_many_edges, 128, None, None,
                                            None, None)
    assert rc == 3 and b"built-in array" in lib.cmace_last_error()
