"""Host-side mirror of the reference's operator layer (cuda_mace/ops/*.py and the autograd
Functions of cuda_mace/src/*.cpp) on top of the C-ABI library.

Each class keeps the reference's ``forward`` signature and autograd contract:

* ``InvariantMessagePassingTP.forward(X, Y, radial, sender_list, receiver_list, nnodes)``
  (src/invariant_message_passing.cpp:73-90) -> [N,16,C]; grads for X, Y, radial.
* ``Linear.forward(X, W, W_T)``, ``ElementalLinear.forward(X, W, W_T, one_hot)``
  (src/linear.cpp:105-138); grad for X only, computed with the transposed weights.
* ``SymmetricContraction.forward(X, atom_types, <sparse U tables>, W3, W2, W1, sizes)``
  (src/symmetric_contraction.cpp:124-158) -> [N,1,C]; grad for X only.
* ``SphericalHarmonics.forward(xyz)`` (src/spherical_harmonics.cpp:52-69) -> [16,E].
* ``CubicSpline.forward(r, r_knots, coeffs, r_width, r_max)`` (src/cubic_spline.cpp:54-68) -> [E,F].

All tensors must live on a CUDA device; float32 and float64 are supported everywhere (the
reference's Linear is float32 only).  Kernels run on torch's current stream.  There is no
fallback: a CPU tensor raises.
"""
import math
from collections import OrderedDict

import torch

from . import _abi


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _suffix(t):
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    raise TypeError(f"float32 or float64 expected, got {t.dtype}")


def _check_cuda(*tensors):
    """Every operand on the GPU, and on the CURRENT device: the entry points launch on the current device's
    stream and allocate their outputs there (use torch.cuda.device(...) around calls for another GPU)."""
    cur = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("cuda_mace_b200 operators need CUDA tensors (there is no CPU path)")
        if cur is None:
            cur = torch.cuda.current_device()
        if t.device.index != cur:
            raise RuntimeError(f"operand on cuda:{t.device.index} while cuda:{cur} is the current device")


class _RefCache:
    """Small LRU keyed by the identity of live tensors.  The cached entry keeps a reference to its
    key tensors, so their storage cannot be recycled for other data while the entry lives, and
    in-place edits are caught by the version counter."""

    def __init__(self, size=8):
        self.size = size
        self.entries = OrderedDict()

    @staticmethod
    def key(*tensors):
        return tuple((t.data_ptr(), tuple(t.shape), t.dtype, t._version) for t in tensors)

    def get(self, key):
        hit = self.entries.get(key)
        if hit is not None:
            self.entries.move_to_end(key)
            return hit[1]
        return None

    def put(self, key, tensors, value):
        self.entries[key] = (tensors, value)
        while len(self.entries) > self.size:
            self.entries.popitem(last=False)
        return value


# --------------------------------------------------------------------------------------
# float32 tensor-core GEMM (tcgen05, 3-term TF32 split)
# --------------------------------------------------------------------------------------
_status = {}          # device index -> int32[1] written by kernels whose bounded waits time out
_packed_cache = _RefCache(32)
USE_TENSOR_CORES = True   # float32 Linear / ElementalLinear / matmul3x go through tcgen05 when shapes allow
# Last radial layer formed inside the message-passing forward (R is only written when a backward will follow).
# Measured at 64 000 atoms (E = 3.33 M, C = 128): 3.4 ms (3.7 ms with R written) against 1.6 + 1.25 ms for the product
# followed by the plain forward, so the model does not use it by default; fused_radial_message_passing() always does.
FUSED_RADIAL_MESSAGE_PASSING = False
# The backward of the last radial layer + message passing without a gradR [E,4,C] array (radial_message_passing):
# the model's float32 default.  False selects the separate product / message-passing operators.
RADIAL_GRADIENT_ON_THE_FLY = True


def _status_tensor(device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status():
    """Raises if any tensor-core kernel reported a timed-out wait since the last check (synchronises)."""
    if _abi.call("cmace_imp_staged_stalled") != 0:
        raise RuntimeError("cuda_mace_b200: the message-passing backward gave up waiting for a bulk copy")
    for idx, t in _status.items():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"cuda_mace_b200: a tensor-core kernel on cuda:{idx} gave up waiting (code {code})")


def probe_bounded_wait(device, code=77, limit_seconds=0.05):
    """Launches the library's wait-that-runs-out probe on `device`: after `limit_seconds` the kernel records `code`
    in the status word that check_status() reads.  Exercises the time-out reporting without hanging the GPU."""
    _abi.call("cmace_bounded_wait_probe", _ptr(_status_tensor(torch.device(device))), int(code), float(limit_seconds),
              _stream())


def _pack(Bt):
    """Packs Bt [nmat, N, K] (or [N, K]) float32, K contiguous, into the tensor-core weight image (cached)."""
    key = _RefCache.key(Bt)
    hit = _packed_cache.get(key)
    if hit is not None:
        return hit
    B3 = Bt.reshape(-1, Bt.shape[-2], Bt.shape[-1]).contiguous()
    nmat, N, K = B3.shape
    n = _abi.call("cmace_gemm_packed_floats", nmat, N, K)
    packed = torch.empty(int(n), dtype=torch.float32, device=Bt.device)
    _abi.call("cmace_gemm_pack_weights_f32", _ptr(B3), nmat, N, K, _ptr(packed), _stream())
    return _packed_cache.put(key, (Bt,), packed)


def _gemm3x(A, Bt, scale=1.0):
    """A [M,K] @ B with Bt = B^T [N,K]; float32 on the tensor cores (3-term TF32 split)."""
    A = A.contiguous()
    M, K = A.shape
    N = Bt.shape[0]
    out = torch.empty(M, N, dtype=torch.float32, device=A.device)
    _abi.call("cmace_gemm3x_f32", _ptr(A), _ptr(_pack(Bt)), M, K, N, float(scale), _ptr(out),
              _ptr(_status_tensor(A.device)), _stream(), tag=f"M={M},K={K},N={N}")
    return out


class _RadialHiddenFunction(torch.autograd.Function):
    """basis [E,nb] -> silu(silu(silu(basis W1) W2) W3) [E,64] in one kernel; the forward keeps the activation
    derivatives (tiled), the backward is the mirrored chain of three products."""

    @staticmethod
    def forward(ctx, basis, W1, W2, W3, W1T, W2T, W3T):
        basis = basis.contiguous()
        E, nb = basis.shape
        h3 = torch.empty(E, 64, dtype=torch.float32, device=basis.device)
        saved = None
        if basis.requires_grad:
            n = _abi.call("cmace_radial_hidden_saved_floats", E)
            saved = torch.empty(max(int(n), 4), dtype=torch.float32, device=basis.device)
        _abi.call("cmace_radial_hidden_fwd_f32", _ptr(basis), nb, _ptr(_pack(W1T)), _ptr(_pack(W2T)), _ptr(_pack(W3T)),
                  E, _ptr(h3), _ptr(saved), _ptr(_status_tensor(basis.device)), _stream())
        ctx.saved = saved
        ctx.weights = (W1, W2, W3)
        ctx.nb = nb
        return h3

    @staticmethod
    def backward(ctx, g):
        if ctx.saved is None:
            raise RuntimeError("radial_hidden: the forward ran without a gradient request")
        g = g.contiguous()
        E = g.shape[0]
        W1, W2, W3 = ctx.weights
        gb = torch.empty(E, ctx.nb, dtype=torch.float32, device=g.device)
        _abi.call("cmace_radial_hidden_bwd_f32", _ptr(g), _ptr(ctx.saved), _ptr(_pack(W3)), _ptr(_pack(W2)),
                  _ptr(_pack(W1)), ctx.nb, E, _ptr(gb), _ptr(_status_tensor(g.device)), _stream())
        return gb, None, None, None, None, None, None


def radial_hidden_ok(dtype, weights):
    """True when the one-kernel version of the perceptron's hidden layers applies: float32, three hidden layers
    of width 64 and a basis of 8, 16, 24 or 32 functions."""
    if not USE_TENSOR_CORES or dtype != torch.float32 or len(weights) != 3:
        return False
    nb = weights[0].shape[0]
    return (nb in (8, 16, 24, 32) and tuple(weights[0].shape) == (nb, 64)
            and tuple(weights[1].shape) == (64, 64) and tuple(weights[2].shape) == (64, 64))


def radial_hidden(basis, weights, weights_t):
    """Hidden layers of the radial perceptron: silu(... silu(basis @ W1) ...) for three constant float32 weight
    matrices [nb,64], [64,64], [64,64] (no weight gradients); weights_t are their contiguous transposes."""
    _check_cuda(basis)
    if not radial_hidden_ok(basis.dtype, weights):
        raise RuntimeError("radial_hidden needs float32, a basis of 8/16/24/32 functions and three layers of width 64")
    return _RadialHiddenFunction.apply(basis, *weights, *weights_t)


class _Matmul3xFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, W, W_T):
        ctx.save_for_backward(W)
        return _gemm3x(A, W_T)

    @staticmethod
    def backward(ctx, G):
        (W,) = ctx.saved_tensors
        return _gemm3x(G, W), None, None


def matmul3x(A, W, W_T=None):
    """A [M,K] @ W [K,N] for a constant float32 weight W (no weight gradient), on the tensor cores with
    float32-grade accuracy.  W_T = W^T contiguous may be passed to avoid re-creating it."""
    _check_cuda(A, W)
    if W_T is None:
        W_T = W.t().contiguous()
    return _Matmul3xFunction.apply(A, W, W_T)


class _MatmulF64Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A, W, W_T):
        ctx.save_for_backward(W_T)
        return _gemm_f64(A, W)

    @staticmethod
    def backward(ctx, G):
        (W_T,) = ctx.saved_tensors
        return _gemm_f64(G, W_T), None, None


def _gemm_f64(A, B):
    A = A.contiguous()
    M, K = A.shape
    N = B.shape[1]
    out = torch.empty(M, N, dtype=torch.float64, device=A.device)
    _abi.call("cmace_gemm_f64", _ptr(A), _ptr(B), M, K, N, 1.0, _ptr(out), _stream(), tag=f"M={M},K={K},N={N}")
    return out


def matmul_f64(A, W, W_T=None):
    """A [M,K] @ W [K,N] for a constant float64 weight W (no weight gradient) on the FP64 tensor cores."""
    _check_cuda(A, W)
    if A.dtype != torch.float64 or W.dtype != torch.float64:
        raise TypeError("matmul_f64 needs float64 operands")
    W = W.contiguous()
    if W_T is None:
        W_T = W.t().contiguous()
    return _MatmulF64Function.apply(A, W, W_T)


def tensor_core_ok(dtype, K, N):
    return USE_TENSOR_CORES and dtype == torch.float32 and K % 8 == 0 and N % 4 == 0


# --------------------------------------------------------------------------------------
# edge topology
# --------------------------------------------------------------------------------------
class EdgeTopology:
    """Receiver CSR and (lazily) the sender-grouped edge order of one neighbour list.

    Replaces the per-call first-occurrence kernel and the N x N reverse-edge table of the
    reference (jit_wrappers/src/invariant_message_passing_wrapper.cpp:19-70, :91-93).  Build it
    once per neighbour list and reuse it for every layer and step.
    """

    def __init__(self, sender, receiver, nnodes, nsenders=None):
        _check_cuda(sender, receiver)
        self.sender = sender.to(torch.int32).contiguous()
        self.receiver = receiver.to(torch.int32).contiguous()
        self.nnodes = int(nnodes)  # receiver rows
        # rows of the node-feature matrix the senders index; larger than nnodes when ghost atoms send
        self.nsenders = self.nnodes if nsenders is None else int(nsenders)
        self.nedges = int(self.sender.numel())
        self.row_ptr = torch.empty(self.nnodes + 1, dtype=torch.int32, device=sender.device)
        _abi.call("cmace_receiver_csr", _ptr(self.receiver), self.nedges, self.nnodes,
                  _ptr(self.row_ptr), _stream())
        self._perm = None
        self._send_ptr = None

    def sender_order(self):
        if self._perm is None:
            dev = self.sender.device
            nbytes = _abi.call("cmace_sender_order_workspace_bytes", self.nedges)
            ws = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=dev)
            perm = torch.empty(max(self.nedges, 1), dtype=torch.int32, device=dev)
            send_ptr = torch.empty(self.nsenders + 1, dtype=torch.int32, device=dev)
            _abi.call("cmace_sender_order", _ptr(self.sender), self.nedges, self.nsenders, _ptr(perm),
                      _ptr(send_ptr), _ptr(ws), int(nbytes), _stream())
            self._perm, self._send_ptr = perm, send_ptr
        return self._perm, self._send_ptr


_topology_cache = _RefCache(8)


def topology_for(sender, receiver, nnodes, nsenders=None):
    key = _RefCache.key(sender, receiver) + (int(nnodes), nsenders)
    topo = _topology_cache.get(key)
    if topo is None:
        topo = _topology_cache.put(key, (sender, receiver), EdgeTopology(sender, receiver, nnodes, nsenders))
    return topo


# --------------------------------------------------------------------------------------
# neighbour list on the device
# --------------------------------------------------------------------------------------
def neighbor_list(positions, box, pbc, r_cut, n_receivers=None, lo=(0.0, 0.0, 0.0)):
    """Full neighbour list of an orthorhombic cell, built on the device with a cell list.

    positions [N,3] CUDA tensor (converted to float64); box (3,) edge lengths (for a non-periodic axis the
    extent the atoms lie in, starting at `lo`); pbc (3,) bools; only the first `n_receivers` atoms receive.
    Returns edge_index [2,E] int32 (row 0 receivers, sorted; row 1 senders), shifts [E,3] float64 with
    vector = pos[sender] - pos[receiver] + shift, and shift_index [E,3] int8 (shift = shift_index * box):
    the same list as cuda_mace_b200.systems.neighbor_list builds on the host.  One host synchronisation (the
    edge count) to size the outputs."""
    _check_cuda(positions)
    pos = positions.detach().to(torch.float64).contiguous()
    dev = pos.device
    n = int(pos.shape[0])
    nrecv = n if n_receivers is None else int(n_receivers)
    geom = [float(v) for v in lo] + [float(v) for v in box]
    mask = sum(1 << d for d in range(3) if bool(pbc[d]))
    st = _stream()
    i32 = dict(dtype=torch.int32, device=dev)
    ncells = int(_abi.call("cmace_nl_num_cells", *geom[3:], float(r_cut)))
    if ncells < 1:
        raise RuntimeError("neighbor_list: bad box or cutoff")
    cell_id = torch.empty(max(n, 1), **i32)
    _abi.call("cmace_nl_cell_ids_f64", _ptr(pos), n, *geom, mask, float(r_cut), _ptr(cell_id), st)
    nbytes = int(_abi.call("cmace_sender_order_workspace_bytes", n))
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=dev)
    perm = torch.empty(max(n, 1), **i32)
    cell_ptr = torch.empty(ncells + 1, **i32)
    _abi.call("cmace_sender_order", _ptr(cell_id), n, ncells, _ptr(perm), _ptr(cell_ptr), _ptr(ws), nbytes, st)
    count = torch.zeros(nrecv + 1, **i32)
    _abi.call("cmace_nl_count_f64", _ptr(pos), n, nrecv, *geom, mask, float(r_cut), _ptr(perm), _ptr(cell_ptr),
              _ptr(count), st)
    row_ptr = torch.empty(nrecv + 1, **i32)
    sbytes = int(_abi.call("cmace_scan_workspace_bytes", nrecv + 1))
    sws = torch.empty(sbytes, dtype=torch.uint8, device=dev)
    _abi.call("cmace_exclusive_scan_i32", _ptr(count), nrecv + 1, _ptr(row_ptr), _ptr(sws), sbytes, st)
    E = int(row_ptr[nrecv].item())
    sender = torch.empty(E, **i32)
    receiver = torch.empty(E, **i32)
    shift_index = torch.empty(E, 3, dtype=torch.int8, device=dev)
    shifts = torch.empty(E, 3, dtype=torch.float64, device=dev)
    if E > 0:
        _abi.call("cmace_nl_fill_f64", _ptr(pos), n, nrecv, *geom, mask, float(r_cut), _ptr(perm), _ptr(cell_ptr),
                  _ptr(row_ptr), _ptr(sender), _ptr(receiver), _ptr(shift_index), _ptr(shifts), st)
    return torch.stack([receiver, sender]), shifts, shift_index


# --------------------------------------------------------------------------------------
# invariant message passing
# --------------------------------------------------------------------------------------
class _IMPFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, Y, radial, topo):
        X, Y, radial = X.contiguous(), Y.contiguous(), radial.contiguous()
        N, C = topo.nnodes, X.shape[1]
        E = topo.nedges
        if X.dim() != 2 or X.shape[0] != topo.nsenders or Y.shape != (16, E) or radial.shape != (E, 4, C):
            raise RuntimeError(f"shape mismatch: X {tuple(X.shape)}, Y {tuple(Y.shape)}, radial "
                               f"{tuple(radial.shape)} for {N} nodes and {E} edges")
        if Y.dtype != X.dtype or radial.dtype != X.dtype:
            raise TypeError("X, Y and radial must have the same dtype")
        out = torch.empty(N, 16, C, dtype=X.dtype, device=X.device)
        _abi.call("cmace_imp_fwd_" + _suffix(X), _ptr(X), _ptr(Y), _ptr(radial), _ptr(topo.sender),
                  _ptr(topo.row_ptr), N, E, C, _ptr(out), _stream())
        ctx.save_for_backward(X, Y, radial)
        ctx.topo = topo
        return out

    @staticmethod
    def backward(ctx, G):
        X, Y, radial = ctx.saved_tensors
        topo = ctx.topo
        G = G.contiguous()
        N, C, E = topo.nnodes, X.shape[1], topo.nedges
        need_x = ctx.needs_input_grad[0]
        gradR = torch.empty_like(radial)
        gradY = torch.empty_like(Y)
        T = torch.empty(E, C, dtype=X.dtype, device=X.device) if need_x else None
        nscratch = _abi.call("cmace_imp_bwd_scratch_elems", E, C, 1 if X.dtype == torch.float64 else 0)
        scratch = torch.empty(nscratch, dtype=X.dtype, device=X.device) if nscratch > 0 else None
        _abi.call("cmace_imp_bwd_edge_" + _suffix(X), _ptr(X), _ptr(Y), _ptr(radial), _ptr(G),
                  _ptr(topo.sender), _ptr(topo.row_ptr), N, E, C, _ptr(gradR), _ptr(gradY), _ptr(T),
                  _ptr(scratch), _stream())
        gradX = None
        if need_x:
            perm, send_ptr = topo.sender_order()
            gradX = torch.empty(topo.nsenders, C, dtype=X.dtype, device=X.device)
            _abi.call("cmace_imp_bwd_node_" + _suffix(X), _ptr(T), _ptr(perm), _ptr(send_ptr), topo.nsenders, C,
                      _ptr(gradX), _stream())
        return gradX, gradY, gradR, None


class _RadialIMPFunction(torch.autograd.Function):
    """Message passing on radial weights R = H @ W (H the last hidden activations of the radial perceptron, W its
    last layer) with a backward that never materialises gradR [E,4,C]: the edge pass is called without a gradR
    output (it still gives gradY and the sender contributions T), and grad H = gradR @ W^T comes from the
    tensor-core kernel whose producer warps form the rows of gradR on the fly (cmace_gemm3x_gradr_f32).  The forward
    is the plain product followed by cmace_imp_fwd_f32; R is kept for the backward's edge pass."""

    @staticmethod
    def forward(ctx, X, Y, H, W, W_T, topo):
        X, Y, H = X.contiguous(), Y.contiguous(), H.contiguous()
        N, C, E, K = topo.nnodes, X.shape[1], topo.nedges, H.shape[1]
        if X.shape[0] != topo.nsenders or Y.shape != (16, E) or H.shape[0] != E or W.shape != (K, 4 * C):
            raise RuntimeError(f"shape mismatch: X {tuple(X.shape)}, Y {tuple(Y.shape)}, H {tuple(H.shape)}, "
                               f"W {tuple(W.shape)} for {N} nodes and {E} edges")
        R = _gemm3x(H, W_T)
        out = torch.empty(N, 16, C, dtype=torch.float32, device=X.device)
        _abi.call("cmace_imp_fwd_f32", _ptr(X), _ptr(Y), _ptr(R), _ptr(topo.sender), _ptr(topo.row_ptr), N, E, C,
                  _ptr(out), _stream())
        ctx.save_for_backward(X, Y, R, W)
        ctx.topo = topo
        return out

    @staticmethod
    def backward(ctx, G):
        X, Y, R, W = ctx.saved_tensors
        topo = ctx.topo
        G = G.contiguous()
        N, C, E, K = topo.nnodes, X.shape[1], topo.nedges, W.shape[0]
        need_x = ctx.needs_input_grad[0]
        gradY = torch.empty_like(Y)
        T = torch.empty(E, C, dtype=X.dtype, device=X.device) if need_x else None
        nscratch = _abi.call("cmace_imp_bwd_scratch_elems", E, C, 0)
        scratch = torch.empty(nscratch, dtype=X.dtype, device=X.device) if nscratch > 0 else None
        _abi.call("cmace_imp_bwd_edge_f32", _ptr(X), _ptr(Y), _ptr(R), _ptr(G), _ptr(topo.sender), _ptr(topo.row_ptr),
                  N, E, C, 0, _ptr(gradY), _ptr(T), _ptr(scratch), _stream(), tag="no gradR")
        gradX = None
        if need_x:
            perm, send_ptr = topo.sender_order()
            gradX = torch.empty(topo.nsenders, C, dtype=X.dtype, device=X.device)
            _abi.call("cmace_imp_bwd_node_f32", _ptr(T), _ptr(perm), _ptr(send_ptr), topo.nsenders, C, _ptr(gradX),
                      _stream())
        gradH = radial_gradient_product(X, G, Y, W, topo) if ctx.needs_input_grad[2] else None
        return gradX, gradY, gradH, None, None, None


def radial_gradient_product(X, G, Y, W, topo):
    """grad H [E,K] = gradR @ W^T with gradR[e,l,c] = X[sender(e),c] * sum_{m in l} Y[m,e] * G[receiver(e),m,c] formed
    inside the tensor-core kernel (never written).  X [Ns,C], G [N,16,C], Y [16,E], W [K,4C], float32."""
    E, C, K = topo.nedges, X.shape[1], W.shape[0]
    gradH = torch.empty(E, K, dtype=torch.float32, device=X.device)
    _abi.call("cmace_gemm3x_gradr_f32", _ptr(X), _ptr(G), _ptr(Y), _ptr(topo.sender), _ptr(topo.receiver),
              _ptr(_pack(W)), E, C, K, _ptr(gradH), _ptr(_status_tensor(X.device)), _stream())
    return gradH


def radial_message_passing_ok(dtype, C, K):
    """True when radial_message_passing applies (float32, 32/64/96/128 channels, hidden width 32..128)."""
    return USE_TENSOR_CORES and dtype == torch.float32 and C in (32, 64, 96, 128) and 32 <= K <= 128 and K % 8 == 0


def radial_message_passing(X, Y, H, W, W_T, topology):
    """out[i,lm,c] = sum_e X[sender(e),c] Y[lm,e] (H @ W)[e, l(lm)*C + c], differentiable with respect to X, Y and H.
    X [Ns,C], Y [16,E], H [E,K], W [K,4C] constant float32 (no weight gradient), W_T its contiguous transpose.  Same
    values as InvariantMessagePassingTP applied to H @ W; the backward moves 2 x 4C floats per edge less through
    memory because the gradient of the radial weights is consumed where it is formed."""
    _check_cuda(X, Y, H, W, W_T)
    if not radial_message_passing_ok(X.dtype, X.shape[1], H.shape[1]):
        raise RuntimeError("radial_message_passing needs float32, 32/64/96/128 channels and a hidden width in 32..128")
    return _RadialIMPFunction.apply(X, Y, H, W, W_T, topology)


def _pack_fused_radial(W_T, C):
    """Weight image of the fused kernel: one 128-row block per group of 32 channels, rows ordered (l, channel),
    from W_T [4C, K] (the transpose of the last radial layer W [K, 4C])."""
    key = _RefCache.key(W_T) + ("fused", C)
    hit = _packed_cache.get(key)
    if hit is not None:
        return hit
    K = W_T.shape[1]
    nq = C // 32
    Bt = W_T.reshape(4, nq, 32, K).permute(1, 0, 2, 3).reshape(nq, 128, K).contiguous()
    return _packed_cache.put(key, (W_T,), _pack(Bt))


def fused_radial_ok(dtype, C, K):
    """True when the kernel with the last radial layer inside applies (shapes and dtype)."""
    return USE_TENSOR_CORES and dtype == torch.float32 and C in (32, 64, 96, 128) and K in (32, 64)


class _FusedRadialIMPFunction(torch.autograd.Function):
    """Message passing whose radial weights R = H @ W are formed on the tensor cores inside the scatter
    kernel.  The forward also writes R when a backward will follow; the backward is the unfused one
    (edge pass, sender pass, then grad H = grad R @ W^T)."""

    @staticmethod
    def forward(ctx, X, Y, H, W, W_T, topo):
        X, Y, H = X.contiguous(), Y.contiguous(), H.contiguous()
        N, C, E, K = topo.nnodes, X.shape[1], topo.nedges, H.shape[1]
        if X.shape[0] != topo.nsenders or Y.shape != (16, E) or H.shape[0] != E or W.shape != (K, 4 * C):
            raise RuntimeError(f"shape mismatch: X {tuple(X.shape)}, Y {tuple(Y.shape)}, H {tuple(H.shape)}, "
                               f"W {tuple(W.shape)} for {N} nodes and {E} edges")
        need_grad = any(ctx.needs_input_grad[:3])
        out = torch.empty(N, 16, C, dtype=torch.float32, device=X.device)
        R = torch.empty(E, 4, C, dtype=torch.float32, device=X.device) if need_grad else None
        _abi.call("cmace_imp_radial_fused_fwd_f32", _ptr(X), _ptr(Y), _ptr(H), _ptr(_pack_fused_radial(W_T, C)),
                  _ptr(topo.sender), _ptr(topo.receiver), N, E, C, K, _ptr(out), _ptr(R),
                  _ptr(_status_tensor(X.device)), _stream())
        ctx.save_for_backward(X, Y, W)
        ctx.R = R
        ctx.topo = topo
        return out

    @staticmethod
    def backward(ctx, G):
        X, Y, W = ctx.saved_tensors
        topo, R = ctx.topo, ctx.R
        G = G.contiguous()
        N, C, E = topo.nnodes, X.shape[1], topo.nedges
        need_x = ctx.needs_input_grad[0]
        gradR = torch.empty_like(R)
        gradY = torch.empty_like(Y)
        T = torch.empty(E, C, dtype=X.dtype, device=X.device) if need_x else None
        nscratch = _abi.call("cmace_imp_bwd_scratch_elems", E, C, 0)
        scratch = torch.empty(nscratch, dtype=X.dtype, device=X.device) if nscratch > 0 else None
        _abi.call("cmace_imp_bwd_edge_f32", _ptr(X), _ptr(Y), _ptr(R), _ptr(G), _ptr(topo.sender), _ptr(topo.row_ptr),
                  N, E, C, _ptr(gradR), _ptr(gradY), _ptr(T), _ptr(scratch), _stream())
        ctx.R = None
        gradX = None
        if need_x:
            perm, send_ptr = topo.sender_order()
            gradX = torch.empty(topo.nsenders, C, dtype=X.dtype, device=X.device)
            _abi.call("cmace_imp_bwd_node_f32", _ptr(T), _ptr(perm), _ptr(send_ptr), topo.nsenders, C, _ptr(gradX),
                      _stream())
        gradH = _gemm3x(gradR.view(E, 4 * C), W) if ctx.needs_input_grad[2] else None
        return gradX, gradY, gradH, None, None, None


def fused_radial_message_passing(X, Y, H, W, W_T, topology):
    """out[i,lm,c] = sum_e X[sender(e),c] Y[lm,e] (H @ W)[e, l(lm)*C + c]: InvariantMessagePassingTP applied to
    the radial weights H @ W without a separate pass for that product.  X [Ns,C], Y [16,E], H [E,K] (K = 32 or
    64), W [K,4C] constant float32 (no weight gradient), W_T its contiguous transpose."""
    _check_cuda(X, Y, H, W, W_T)
    if not fused_radial_ok(X.dtype, X.shape[1], H.shape[1]):
        raise RuntimeError("fused_radial_message_passing needs float32, 32/64/96/128 channels and K = 32 or 64")
    return _FusedRadialIMPFunction.apply(X, Y, H, W, W_T, topology)


class InvariantMessagePassingTP(torch.nn.Module):
    """out[i,lm,c] = sum_{e: receiver(e)=i} X[sender(e),c] * Y[lm,e] * radial[e,l(lm),c].

    Same call as cuda_mace/ops/invariant_message_passing.py:8-22: X [N,C], Y [16,E], radial [E,4,C],
    int32 sender/receiver lists sorted by receiver.  Unlike the reference, receivers without edges
    get zero rows, any neighbour count per receiver is allowed, and the list need not be symmetric.
    """

    def forward(self, node_feats, edge_attrs, tp_weights, sender_list, receiver_list, nnodes, topology=None):
        _check_cuda(node_feats, edge_attrs, tp_weights, sender_list, receiver_list)
        topo = topology if topology is not None else topology_for(sender_list, receiver_list, int(nnodes),
                                                                  int(node_feats.shape[0]))
        return _IMPFunction.apply(node_feats, edge_attrs, tp_weights, topo)


# --------------------------------------------------------------------------------------
# Linear / ElementalLinear
# --------------------------------------------------------------------------------------
def _linear_call(X, W, W_other, node_order, elem_start, nelements, scale):
    """out = scale * X @ W[z, l] per row; W_other is the transposed copy of W (the tensor-core path
    packs it, since it wants B^T with K contiguous)."""
    X = X.contiguous()
    N, K = X.shape[0], X.shape[2]
    Nout = W.shape[-1]
    if X.shape[1] != 16 or W.shape[-2] != K or W.numel() != nelements * 4 * K * Nout:
        raise RuntimeError(f"shape mismatch: X {tuple(X.shape)}, W {tuple(W.shape)}")
    if W.dtype != X.dtype:
        raise TypeError("X and W must have the same dtype")
    out = torch.empty(N, 16, Nout, dtype=X.dtype, device=X.device)
    if tensor_core_ok(X.dtype, K, Nout) and Nout <= 128 and nelements <= 128:   # the kernel's problem table holds 4 x 128
        _abi.call("cmace_linear_tc_f32", _ptr(X), _ptr(_pack(W_other)), _ptr(node_order), _ptr(elem_start),
                  nelements, N, K, Nout, float(scale), _ptr(out), _ptr(_status_tensor(X.device)), _stream())
        return out
    _abi.call("cmace_linear_" + _suffix(X), _ptr(X), _ptr(W.contiguous()), _ptr(node_order), _ptr(elem_start),
              nelements, N, K, Nout, float(scale), _ptr(out), _stream())
    return out


class _LinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, W, W_T, node_order, elem_start, nelements):
        ctx.save_for_backward(W, W_T)
        scale = 1.0 / math.sqrt(X.shape[2])  # the path weight of linear_impl.cu:33
        ctx.grouping = (node_order, elem_start, nelements, scale)
        return _linear_call(X, W, W_T, node_order, elem_start, nelements, scale)

    @staticmethod
    def backward(ctx, G):
        W, W_T = ctx.saved_tensors
        node_order, elem_start, nelements, scale = ctx.grouping
        return _linear_call(G, W_T, W, node_order, elem_start, nelements, scale), None, None, None, None, None


def linear_forward(X, W, W_T):
    """torch.classes.linear_wmma.Linear.forward equivalent: W [4,K,N], W_T [4,N,K]."""
    _check_cuda(X, W, W_T)
    return _LinearFunction.apply(X, W, W_T, None, None, 1)


_grouping_cache = _RefCache(8)


def group_by_element(elem, nelements):
    """(node_order, elem_start) of an int32 element index per node, on the device, no host sync."""
    key = _RefCache.key(elem) + (int(nelements),)
    hit = _grouping_cache.get(key)
    if hit is not None:
        return hit
    n = elem.numel()
    dev = elem.device
    nbytes = _abi.call("cmace_sender_order_workspace_bytes", n)
    ws = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=dev)
    order = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    start = torch.empty(nelements + 1, dtype=torch.int32, device=dev)
    _abi.call("cmace_group_by_element", _ptr(elem), n, int(nelements), _ptr(order), _ptr(start), _ptr(ws),
              int(nbytes), _stream())
    # Nodes already stored grouped by element need no gather list, and the float32 tensor-core kernel then moves
    # their rows by TMA.  The check reads one flag back, once per element tensor (not while a graph is captured).
    if n > 1 and not torch.cuda.is_current_stream_capturing():
        if bool((elem[1:] >= elem[:-1]).all().item()):
            order = None
    return _grouping_cache.put(key, (elem,), (order, start))


def elemental_linear_forward(X, W, W_T, one_hot_or_index):
    """torch.classes.linear_wmma.ElementalLinear.forward equivalent: W [Z,4,K,N]; the last argument
    is the one-hot node attribute matrix [N,Z] of the reference or an int32 element index [N]."""
    _check_cuda(X, W, W_T, one_hot_or_index)
    Z = W.shape[0]
    if one_hot_or_index.dim() == 2:
        hit = _onehot_cache.get(_RefCache.key(one_hot_or_index))
        if hit is None:
            hit = _onehot_cache.put(_RefCache.key(one_hot_or_index), (one_hot_or_index,),
                                    one_hot_or_index.argmax(dim=-1).to(torch.int32))
        elem = hit
    else:
        elem = one_hot_or_index.to(torch.int32)
    if Z == 1:
        return _LinearFunction.apply(X, W, W_T, None, None, 1)
    order, start = group_by_element(elem, Z)
    return _LinearFunction.apply(X, W, W_T, order, start, Z)


_onehot_cache = _RefCache(8)


class Linear(torch.nn.Module):
    """Per-l channel mixing of [N,16,K] features, weights [4,K,N] (one matrix per l).

    Mirrors cuda_mace/ops/linear.py:6-54; the e3nn weight split is done by the caller because e3nn
    is not a dependency: pass the four per-l matrices.  `scale` is folded into the weights (used
    for the 1/avg_num_neighbors of models/InvariantMACE.py:114)."""

    def __init__(self, weights, scale=1.0):
        super().__init__()
        w = (weights * scale).contiguous()
        self.register_buffer("weights", w)
        self.register_buffer("weights_transposed", w.transpose(-1, -2).contiguous())

    def forward(self, x):
        return linear_forward(x, self.weights, self.weights_transposed)


class ElementalLinear(torch.nn.Module):
    """Element-dependent per-l channel mixing, weights [Z,4,K,N] (cuda_mace/ops/linear.py:57-108)."""

    def __init__(self, weights):
        super().__init__()
        w = weights.contiguous()
        self.register_buffer("weights", w)
        self.register_buffer("weights_transposed", w.transpose(-1, -2).contiguous())

    def forward(self, x, y):
        return elemental_linear_forward(x, self.weights, self.weights_transposed, y)


# --------------------------------------------------------------------------------------
# symmetric contraction
# --------------------------------------------------------------------------------------
class _Plan:
    def __init__(self, handle):
        self.handle = handle

    def __del__(self):
        try:
            _abi.call("cmace_symcon_plan_destroy", self.handle)
        except Exception:
            pass


def make_plan(u3_max, U3_num_nonzero, U3_indices, U3_values, U2_num_nonzero, U2_indices, U2_values,
              w3, w2, w1):
    """Builds the device program from (host copies of) the reference's sparse tables."""
    import ctypes

    n3 = U3_num_nonzero.detach().to("cpu", torch.int16).contiguous()
    i3 = U3_indices.detach().to("cpu", torch.int32).contiguous()
    v3 = U3_values.detach().to("cpu", torch.float64).contiguous()
    n2 = U2_num_nonzero.detach().to("cpu", torch.int16).contiguous()
    i2 = U2_indices.detach().to("cpu", torch.int16).contiguous()
    v2 = U2_values.detach().to("cpu", torch.float64).contiguous()
    handle = ctypes.c_void_p()
    _abi.call("cmace_symcon_plan_create", int(u3_max), _ptr(n3), _ptr(i3), _ptr(v3), _ptr(n2), _ptr(i2),
              _ptr(v2), int(w3), int(w2), int(w1), ctypes.byref(handle))
    return _Plan(handle)


class _SymConFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, atom_types, W3, W2, W1, plan, nelements):
        X = X.contiguous()
        N, C = X.shape[0], X.shape[2]
        out = torch.empty(N, 1, C, dtype=X.dtype, device=X.device)
        _abi.call("cmace_symcon_fwd_" + _suffix(X), plan.handle, _ptr(X), _ptr(atom_types), _ptr(W3), _ptr(W2),
                  _ptr(W1), nelements, N, C, _ptr(out), _stream())
        ctx.save_for_backward(X, atom_types, W3, W2, W1)
        ctx.plan, ctx.nelements = plan, nelements
        return out

    @staticmethod
    def backward(ctx, G):
        X, atom_types, W3, W2, W1 = ctx.saved_tensors
        G = G.contiguous()
        N, C = X.shape[0], X.shape[2]
        gradX = torch.empty_like(X)
        _abi.call("cmace_symcon_bwd_" + _suffix(X), ctx.plan.handle, _ptr(X), _ptr(atom_types), _ptr(W3),
                  _ptr(W2), _ptr(W1), _ptr(G), ctx.nelements, N, C, _ptr(gradX), _stream())
        return gradX, None, None, None, None, None, None


_plan_cache = _RefCache(4)


def symmetric_contraction_forward(X, atom_types, U3_max_nonsparse, U3_num_nonzero, U3_indices, U3_values,
                                  U2_num_nonzero, U2_indices, U2_values, U1_num_nonzero, U1_index, W3, W2, W1,
                                  W3_size, W2_size, W1_size, plan=None):
    """torch.classes.symm_contract.SymmetricContraction.forward equivalent (same argument list).

    W3/W2/W1 may be the reference's [nlout, Z, w, C] buffers (output irrep 0 is used, as in
    symmetric_contraction_impl.cu:64-76) or plain [Z, w, C].  The device program is built from the
    tables on first use and cached per table set."""
    _check_cuda(X, atom_types, W3, W2, W1)
    if plan is None:
        key = _RefCache.key(U3_indices, U3_values, U2_indices, U2_values)
        plan = _plan_cache.get(key)
        if plan is None:
            plan = _plan_cache.put(
                key, (U3_indices, U3_values, U2_indices, U2_values),
                make_plan(U3_max_nonsparse, U3_num_nonzero, U3_indices, U3_values, U2_num_nonzero, U2_indices,
                          U2_values, W3_size, W2_size, W1_size))
    W3, W2, W1 = [w[0] if w.dim() == 4 else w for w in (W3, W2, W1)]
    if W3.dtype != X.dtype:
        raise TypeError("X and the weights must have the same dtype")
    if W3.shape[1] != W3_size or W2.shape[1] != W2_size or W1.shape[1] != W1_size:
        raise RuntimeError("weight buffers do not match W3_size/W2_size/W1_size")
    return _SymConFunction.apply(X, atom_types.to(torch.int32).contiguous(), W3.contiguous(), W2.contiguous(),
                                 W1.contiguous(), plan, W3.shape[0])


def pack_sparse_u(U3, U2, U1):
    """Sparse U tables in the reference's layout (cuda_mace/ops/symmetric_contraction.py:91-187) from
    dense tensors U3 [16,16,16,P3], U2 [16,16,P2], U1 [16,P1].  The values are returned in the dense
    tensors' dtype (the reference stores float32); the packed int32 carries, per (i,j) and per k-th
    non-zero, bits 7:0 the path, 15:8 k, 23:16 / 31:24 the partner paths the reference's gradient uses."""
    U3c, U2c, U1c = U3.cpu(), U2.cpu(), U1.cpu()
    nz3 = U3c != 0
    n3 = nz3.sum(dim=(2, 3)).to(torch.int16)
    maxnz = int(n3.max())
    idx3 = torch.zeros(maxnz, 16, 16, dtype=torch.int32)
    val3 = torch.zeros(maxnz, 16, 16, dtype=U3c.dtype)
    for i in range(16):
        for j in range(16):
            k1, p1 = torch.where(nz3[i, j])
            _, p2 = torch.where(nz3[j, i])
            _, p3 = torch.where(nz3[j, :, i, :])
            for t in range(k1.shape[0]):
                lo = (int(k1[t]) << 8) | int(p1[t])
                hi = ((int(p2[t]) << 8) | int(p3[t])) if t < p2.shape[0] and t < p3.shape[0] else 0
                idx3[t, i, j] = (hi << 16) | lo
                val3[t, i, j] = U3c[i, j, k1[t], p1[t]]
    nz2 = U2c != 0
    n2 = nz2.sum(dim=2).to(torch.int16)
    idx2 = torch.zeros(16, 16, dtype=torch.int16)
    val2 = torch.zeros(16, 16, dtype=U2c.dtype)
    for i in range(16):
        for j in range(16):
            (p,) = torch.where(nz2[i, j])
            if p.shape[0] > 0:
                idx2[i, j] = int(p[0])
                val2[i, j] = U2c[i, j, p[0]]
    n1 = (U1c != 0).any(dim=1).to(torch.int16)
    idx1 = (U1c != 0).to(torch.int16).argmax(dim=1).to(torch.int16)
    return maxnz, n3, idx3, val3, n2, idx2, val2, n1, idx1


class SymmetricContraction(torch.nn.Module):
    """Correlation-3, L=0 symmetric contraction with per-element weights.

    Mirrors cuda_mace/ops/symmetric_contraction.py:6-232: keeps the sparse U tables and the weight
    buffers [1, Z, w, C] as registered buffers and forwards them with the reference's argument list.
    Built from dense U tensors and weights [Z, P, C] because upstream's SymmetricContraction module
    and U_matrix_real are not dependencies here (see cuda_mace_b200.cg.u_matrices)."""

    def __init__(self, U3, U2, U1, W3, W2, W1):
        super().__init__()
        maxnz, n3, i3, v3, n2, i2, v2, n1, i1 = pack_sparse_u(U3, U2, U1)
        self.u3_max_nonsparse = maxnz
        for name, t in (("U3_num_nonsparse", n3), ("U3_indices", i3), ("U3_values", v3),
                        ("U2_num_nonsparse", n2), ("U2_indices", i2), ("U2_values", v2),
                        ("U1_num_values", n1), ("U1_index", i1)):
            self.register_buffer(name, t)
        self.register_buffer("weights_3", W3[None].contiguous())
        self.register_buffer("weights_2", W2[None].contiguous())
        self.register_buffer("weights_1", W1[None].contiguous())
        self.W3_L0_size, self.W2_L0_size, self.W1_L0_size = W3.shape[1], W2.shape[1], W1.shape[1]
        self._plan = None

    def forward(self, x, atom_types):
        assert x.shape[-1] % 32 == 0, "channel dimension of x ([-1]) must be a multiple of 32."
        assert x.shape[1] == 16, "l dimension of x ([1]) must be 16."
        if self._plan is None:
            self._plan = make_plan(self.u3_max_nonsparse, self.U3_num_nonsparse, self.U3_indices, self.U3_values,
                                   self.U2_num_nonsparse, self.U2_indices, self.U2_values, self.W3_L0_size,
                                   self.W2_L0_size, self.W1_L0_size)
        return symmetric_contraction_forward(
            x, atom_types, self.u3_max_nonsparse, self.U3_num_nonsparse, self.U3_indices, self.U3_values,
            self.U2_num_nonsparse, self.U2_indices, self.U2_values, self.U1_num_values, self.U1_index,
            self.weights_3, self.weights_2, self.weights_1, self.W3_L0_size, self.W2_L0_size, self.W1_L0_size,
            plan=self._plan)


# --------------------------------------------------------------------------------------
# spherical harmonics / edge basis
# --------------------------------------------------------------------------------------
class _EdgeBasisFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xyz, r_max, nbessel, p, with_radial):
        xyz = xyz.contiguous()
        E = xyz.shape[0]
        Y = torch.empty(16, E, dtype=xyz.dtype, device=xyz.device)
        B = torch.empty(E, nbessel, dtype=xyz.dtype, device=xyz.device) if with_radial else None
        _abi.call("cmace_edge_basis_fwd_" + _suffix(xyz), _ptr(xyz), E, float(r_max), int(nbessel), int(p),
                  _ptr(Y), _ptr(B), _stream())
        ctx.save_for_backward(xyz)
        ctx.cfg = (float(r_max), int(nbessel), int(p), with_radial)
        if with_radial:
            return Y, B
        return Y

    @staticmethod
    def backward(ctx, gY, gB=None):
        (xyz,) = ctx.saved_tensors
        r_max, nbessel, p, with_radial = ctx.cfg
        E = xyz.shape[0]
        gY = torch.zeros(16, E, dtype=xyz.dtype, device=xyz.device) if gY is None else gY.contiguous()
        if with_radial:
            gB = torch.zeros(E, nbessel, dtype=xyz.dtype, device=xyz.device) if gB is None else gB.contiguous()
        gxyz = torch.empty_like(xyz)
        _abi.call("cmace_edge_basis_bwd_" + _suffix(xyz), _ptr(xyz), _ptr(gY), _ptr(gB if with_radial else None),
                  E, r_max, nbessel, p, _ptr(gxyz), _stream())
        return gxyz, None, None, None, None


class _EdgeVectorsFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, positions, shifts, topo, dtype):
        E = topo.nedges
        vec = torch.empty(E, 3, dtype=dtype, device=positions.device)
        _abi.call("cmace_edge_vectors_fwd_" + _suffix(vec), _ptr(positions), _ptr(topo.sender), _ptr(topo.receiver),
                  _ptr(shifts), E, _ptr(vec), _stream())
        ctx.topo = topo
        return vec

    @staticmethod
    def backward(ctx, g):
        topo = ctx.topo
        g = g.contiguous()
        perm, send_ptr = topo.sender_order()
        grad = torch.empty(topo.nsenders, 3, dtype=torch.float64, device=g.device)
        _abi.call("cmace_edge_vectors_bwd_" + _suffix(g), _ptr(g), _ptr(topo.row_ptr), _ptr(perm), _ptr(send_ptr),
                  topo.nnodes, topo.nsenders, _ptr(grad), _stream())
        return grad, None, None, None


def edge_vectors(positions, shifts, topology, dtype):
    """vec[e] = positions[sender] - positions[receiver] + shifts[e] as [E,3] of `dtype`, from float64 positions
    [nsenders,3] and float64 shifts [E,3] (or None); the backward gives the position gradient in one kernel from the
    topology's two edge groupings (no atomics).  What the reference does with get_edge_vectors_and_lengths
    (models/InvariantMACE.py:297-304) and autograd."""
    _check_cuda(positions)
    if positions.dtype != torch.float64 or positions.shape != (topology.nsenders, 3):
        raise RuntimeError("edge_vectors: positions must be float64 [nsenders, 3]")
    if shifts is not None and (shifts.dtype != torch.float64 or shifts.shape != (topology.nedges, 3)):
        raise RuntimeError("edge_vectors: shifts must be float64 [E, 3]")
    return _EdgeVectorsFunction.apply(positions.contiguous(), None if shifts is None else shifts.contiguous(),
                                      topology, dtype)


class SphericalHarmonics(torch.nn.Module):
    """xyz [E,3] -> Y [16,E]: real harmonics to l=3 of the normalised vectors, e3nn component order and
    normalisation; same call as torch.classes.spherical_harmonics.SphericalHarmonics.forward
    (src/spherical_harmonics.cpp:52-69)."""

    def forward(self, xyz):
        _check_cuda(xyz)
        return _EdgeBasisFunction.apply(xyz, 1.0, 0, 1, False)


class EdgeBasis(torch.nn.Module):
    """xyz [E,3] -> (Y [16,E], B [E,nbessel]) in one pass: harmonics plus the Bessel basis with
    polynomial cutoff, i.e. upstream MACE's radial_embedding evaluated exactly rather than through the
    reference's spline table (models/InvariantMACE.py:226-240)."""

    def __init__(self, r_max, num_bessel=8, p=5):
        super().__init__()
        self.r_max, self.num_bessel, self.p = float(r_max), int(num_bessel), int(p)

    def forward(self, xyz):
        _check_cuda(xyz)
        return _EdgeBasisFunction.apply(xyz, self.r_max, self.num_bessel, self.p, True)


# --------------------------------------------------------------------------------------
# cubic spline
# --------------------------------------------------------------------------------------
class _SplineFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, r_knots, coeffs, r_width, r_max):
        r = r.contiguous()
        E, nint, nout = r.shape[0], coeffs.shape[0], coeffs.shape[2]
        R = torch.empty(E, nout, dtype=r.dtype, device=r.device)
        _abi.call("cmace_spline_fwd_" + _suffix(r), _ptr(r), _ptr(r_knots), _ptr(coeffs), E, nint, nout,
                  float(r_width), float(r_max), _ptr(R), _stream())
        ctx.save_for_backward(r, r_knots, coeffs)
        ctx.cfg = (float(r_width), float(r_max))
        return R

    @staticmethod
    def backward(ctx, gR):
        r, r_knots, coeffs = ctx.saved_tensors
        gR = gR.contiguous()
        E, nint, nout = r.shape[0], coeffs.shape[0], coeffs.shape[2]
        gr = torch.empty_like(r)
        _abi.call("cmace_spline_bwd_" + _suffix(r), _ptr(r), _ptr(r_knots), _ptr(coeffs), _ptr(gR), E, nint,
                  nout, ctx.cfg[0], ctx.cfg[1], _ptr(gr), _stream())
        return gr, None, None, None, None


def cubic_spline_forward(r, r_knots, coeffs, r_width, r_max):
    """torch.classes.cubic_spline.CubicSpline.forward equivalent: coeffs [nintervals,4,F] -> R [E,F]."""
    _check_cuda(r, r_knots, coeffs)
    if coeffs.dim() != 3 or coeffs.shape[1] != 4:
        raise RuntimeError("coeffs must be [nintervals, 4, noutputs]")
    return _SplineFunction.apply(r, r_knots.contiguous(), coeffs.contiguous(), r_width, r_max)


def cubic_spline_coefficients(x, y, h):
    """Natural-spline coefficients [n,4,F] of y [n+1,F] on equidistant knots (the solve of
    cuda_mace/ops/cubic_spline.py:41-84, vectorised over the channel axis)."""
    n, F = x.shape[0] - 1, y.shape[1]
    alpha = torch.zeros(n, F, dtype=y.dtype, device=y.device)
    alpha[1:] = 3.0 / h * (y[2:] - y[1:-1]) - 3.0 / h * (y[1:-1] - y[:-2])
    mu = [0.0] * n
    z = torch.zeros(n + 1, F, dtype=y.dtype, device=y.device)
    xs = x.tolist()
    for i in range(1, n):
        li = 2.0 * (xs[i + 1] - xs[i - 1]) - h * mu[i - 1]
        mu[i] = h / li
        z[i] = (alpha[i] - h * z[i - 1]) / li
    c = torch.zeros(n + 1, F, dtype=y.dtype, device=y.device)
    for j in range(n - 1, -1, -1):
        c[j] = z[j] - mu[j] * c[j + 1]
    b = (y[1:] - y[:-1]) / h - h * (c[1:] + 2.0 * c[:-1]) / 3.0
    d = (c[1:] - c[:-1]) / (3.0 * h)
    return torch.stack((y[:-1], b, c[:-1], d), dim=1).contiguous()


class CubicSpline(torch.nn.Module):
    """Tabulated radial weights: natural cubic spline through R_out [nknots,F] at r_knots, zero
    beyond rmax (cuda_mace/ops/cubic_spline.py:4-39)."""

    def __init__(self, r_knots, R_out, h, rmax):
        super().__init__()
        self.register_buffer("r_knots", r_knots.contiguous())
        self.register_buffer("coefficients", cubic_spline_coefficients(r_knots, R_out, float(h)))
        self.h, self.rmax = float(h), float(rmax)

    def forward(self, r_trial):
        return cubic_spline_forward(r_trial, self.r_knots, self.coefficients, self.h, self.rmax)
