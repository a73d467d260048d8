"""ctypes binding of the C-ABI library (include/cuda_mace_b200.h).

The library is the product: there is no fallback.  Importing this module without the built
library raises ImportError naming the build command.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libcuda_mace_b200.so")

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64
_D = ctypes.c_double

# name -> argument ctypes (every function returns int unless listed in _RESTYPES)
SIGNATURES = {
    "cmace_abi_version": [],
    "cmace_receiver_csr": [_P, _L, _L, _P, _P],
    "cmace_sender_order_workspace_bytes": [_L],
    "cmace_sender_order": [_P, _L, _L, _P, _P, _P, _L, _P],
    "cmace_group_by_element": [_P, _L, _I, _P, _P, _P, _L, _P],
    "cmace_sph_fwd_f32": [_P, _L, _P, _P],
    "cmace_sph_fwd_f64": [_P, _L, _P, _P],
    "cmace_sph_bwd_f32": [_P, _P, _L, _P, _P],
    "cmace_sph_bwd_f64": [_P, _P, _L, _P, _P],
    "cmace_edge_basis_fwd_f32": [_P, _L, _D, _I, _I, _P, _P, _P],
    "cmace_edge_basis_fwd_f64": [_P, _L, _D, _I, _I, _P, _P, _P],
    "cmace_edge_basis_bwd_f32": [_P, _P, _P, _L, _D, _I, _I, _P, _P],
    "cmace_edge_basis_bwd_f64": [_P, _P, _P, _L, _D, _I, _I, _P, _P],
    "cmace_edge_vectors_fwd_f32": [_P, _P, _P, _P, _L, _P, _P],
    "cmace_edge_vectors_fwd_f64": [_P, _P, _P, _P, _L, _P, _P],
    "cmace_edge_vectors_bwd_f32": [_P, _P, _P, _P, _L, _L, _P, _P],
    "cmace_edge_vectors_bwd_f64": [_P, _P, _P, _P, _L, _L, _P, _P],
    "cmace_spline_fwd_f32": [_P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_spline_fwd_f64": [_P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_spline_bwd_f32": [_P, _P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_spline_bwd_f64": [_P, _P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_imp_fwd_f32": [_P, _P, _P, _P, _P, _L, _L, _I, _P, _P],
    "cmace_imp_fwd_f64": [_P, _P, _P, _P, _P, _L, _L, _I, _P, _P],
    "cmace_imp_bwd_scratch_elems": [_L, _I, _I],
    "cmace_imp_bwd_edge_f32": [_P, _P, _P, _P, _P, _P, _L, _L, _I, _P, _P, _P, _P, _P],
    "cmace_imp_bwd_edge_f64": [_P, _P, _P, _P, _P, _P, _L, _L, _I, _P, _P, _P, _P, _P],
    "cmace_imp_bwd_edge_f64_noalloc_max_elems": [],
    "cmace_imp_bwd_edge_f64_noalloc": [_P, _P, _P, _P, _P, _P, _L, _L, _I, _P, _P, _P, _P],
    "cmace_imp_bwd_node_f32": [_P, _P, _P, _L, _I, _P, _P],
    "cmace_imp_bwd_node_f64": [_P, _P, _P, _L, _I, _P, _P],
    "cmace_linear_f32": [_P, _P, _P, _P, _I, _L, _I, _I, _D, _P, _P],
    "cmace_linear_f64": [_P, _P, _P, _P, _I, _L, _I, _I, _D, _P, _P],
    "cmace_gemm_f64": [_P, _P, _L, _I, _I, _D, _P, _P],
    "cmace_gemm_packed_floats": [_I, _I, _I],
    "cmace_gemm_pack_weights_f32": [_P, _I, _I, _I, _P, _P],
    "cmace_gemm3x_f32": [_P, _P, _L, _I, _I, _D, _P, _P, _P],
    "cmace_linear_tc_f32": [_P, _P, _P, _P, _I, _L, _I, _I, _D, _P, _P, _P],
    "cmace_bounded_wait_probe": [_P, _I, _D, _P],
    "cmace_gemm3x_gradr_f32": [_P, _P, _P, _P, _P, _P, _L, _I, _I, _P, _P, _P],
    "cmace_radial_hidden_saved_floats": [_L],
    "cmace_radial_hidden_fwd_f32": [_P, _I, _P, _P, _P, _L, _P, _P, _P, _P],
    "cmace_radial_hidden_bwd_f32": [_P, _P, _P, _P, _P, _I, _L, _P, _P, _P],
    "cmace_imp_radial_fused_fwd_f32": [_P, _P, _P, _P, _P, _P, _L, _L, _I, _I, _P, _P, _P, _P],
    "cmace_imp_staged_stalled": [],
    "cmace_nl_num_cells": [_D, _D, _D, _D],
    "cmace_nl_cell_ids_f64": [_P, _L, _D, _D, _D, _D, _D, _D, _I, _D, _P, _P],
    "cmace_nl_count_f64": [_P, _L, _L, _D, _D, _D, _D, _D, _D, _I, _D, _P, _P, _P, _P],
    "cmace_scan_workspace_bytes": [_L],
    "cmace_exclusive_scan_i32": [_P, _L, _P, _P, _L, _P],
    "cmace_nl_fill_f64": [_P, _L, _L, _D, _D, _D, _D, _D, _D, _I, _D, _P, _P, _P, _P, _P, _P, _P, _P],
    "cmace_symcon_plan_create": [_I, _P, _P, _P, _P, _P, _P, _I, _I, _I, ctypes.POINTER(_P)],
    "cmace_symcon_plan_destroy": [_P],
    "cmace_symcon_plan_nterms": [_P],
    "cmace_symcon_plan_nclasses": [_P],
    "cmace_symcon_plan_is_canonical": [_P],
    "cmace_symcon_fwd_f32": [_P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
    "cmace_symcon_fwd_f64": [_P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
    "cmace_symcon_bwd_f32": [_P, _P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
    "cmace_symcon_bwd_f64": [_P, _P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
}
_RESTYPES = {
    "cmace_sender_order_workspace_bytes": _L,
    "cmace_imp_bwd_scratch_elems": _L,
    "cmace_gemm_packed_floats": _L,
    "cmace_radial_hidden_saved_floats": _L,
    "cmace_nl_num_cells": _L,
    "cmace_scan_workspace_bytes": _L,
    "cmace_imp_bwd_edge_f64_noalloc_max_elems": _L,
    "cmace_symcon_plan_destroy": None,
}
# functions whose integer result is a value, not a status
_VALUE_FUNCS = {"cmace_abi_version", "cmace_sender_order_workspace_bytes", "cmace_imp_bwd_scratch_elems",
                "cmace_gemm_packed_floats", "cmace_imp_bwd_edge_f64_noalloc_max_elems",
                "cmace_radial_hidden_saved_floats", "cmace_nl_num_cells", "cmace_scan_workspace_bytes",
                "cmace_imp_staged_stalled",
                "cmace_symcon_plan_destroy", "cmace_symcon_plan_nterms", "cmace_symcon_plan_nclasses",
                "cmace_symcon_plan_is_canonical"}

_lib = None

# entry points that launch kernels, with the number of kernels of ours each call launches
# (cub's radix sort inside the two grouping calls is counted as one)
KERNEL_LAUNCHES = {
    "cmace_receiver_csr": 1, "cmace_sender_order": 3, "cmace_group_by_element": 3,
    "cmace_sph_fwd": 1, "cmace_sph_bwd": 1, "cmace_edge_basis_fwd": 1, "cmace_edge_basis_bwd": 1,
    "cmace_edge_vectors_fwd": 1, "cmace_edge_vectors_bwd": 1,
    "cmace_spline_fwd": 1, "cmace_spline_bwd": 1, "cmace_imp_fwd": 1, "cmace_imp_bwd_edge": 1, "cmace_imp_bwd_edge_f64_noalloc": 2,
    "cmace_imp_bwd_node": 1, "cmace_linear": 1, "cmace_symcon_fwd": 1, "cmace_symcon_bwd": 1,
    "cmace_gemm_pack_weights": 1, "cmace_gemm3x": 1, "cmace_gemm": 1, "cmace_gemm3x_gradr": 1, "cmace_bounded_wait_probe": 1, "cmace_linear_tc": 1,
    "cmace_radial_hidden_fwd": 1, "cmace_radial_hidden_bwd": 1, "cmace_imp_radial_fused_fwd": 1,
    "cmace_nl_cell_ids": 1, "cmace_nl_count": 1, "cmace_exclusive_scan_i32": 1, "cmace_nl_fill": 1,
}
launch_count = 0       # kernels launched through this binding since import
_timing = None         # list of (name, start_event, end_event) while timing is on


def load():
    """Loads the shared library once and declares every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.isfile(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m cuda_mace_b200.build` "
            "(there is no CPU or PyTorch fallback for the CUDA kernels)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.cmace_last_error.restype = ctypes.c_char_p
    lib.cmace_last_error.argtypes = []
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, _I)
    _lib = lib
    return lib


def call(name, *args, tag=None):
    """Calls a status-returning entry point; raises RuntimeError with the library's message.
    `tag` only labels the call in the optional kernel timing (e.g. the GEMM shape)."""
    global launch_count
    lib = load()
    if name in _VALUE_FUNCS:
        return getattr(lib, name)(*args)
    base = name[:-4] if name.endswith(("_f32", "_f64")) else name
    n_launch = KERNEL_LAUNCHES.get(base, 0)
    if _timing is not None and n_launch:
        import torch

        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        rc = getattr(lib, name)(*args)
        ev1.record()
        _timing.append((name if tag is None else f"{name}[{tag}]", ev0, ev1))
    else:
        rc = getattr(lib, name)(*args)
    launch_count += n_launch
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {lib.cmace_last_error().decode()}")
    return 0


def start_timing():
    """Brackets every kernel-launching call with CUDA events on torch's current stream."""
    global _timing
    _timing = []


def stop_timing():
    """Returns {entry point: (calls, total milliseconds)}; synchronises the device."""
    global _timing
    import torch

    torch.cuda.synchronize()
    out = {}
    for name, ev0, ev1 in _timing or []:
        calls, ms = out.get(name, (0, 0.0))
        out[name] = (calls + 1, ms + ev0.elapsed_time(ev1))
    _timing = None
    return out
