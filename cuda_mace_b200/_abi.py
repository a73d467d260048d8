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
    "cmace_spline_fwd_f32": [_P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_spline_fwd_f64": [_P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_spline_bwd_f32": [_P, _P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_spline_bwd_f64": [_P, _P, _P, _P, _L, _I, _I, _D, _D, _P, _P],
    "cmace_imp_fwd_f32": [_P, _P, _P, _P, _P, _L, _L, _I, _P, _P],
    "cmace_imp_fwd_f64": [_P, _P, _P, _P, _P, _L, _L, _I, _P, _P],
    "cmace_imp_bwd_scratch_elems": [_L, _I, _I],
    "cmace_imp_bwd_edge_f32": [_P, _P, _P, _P, _P, _P, _L, _L, _I, _P, _P, _P, _P, _P],
    "cmace_imp_bwd_edge_f64": [_P, _P, _P, _P, _P, _P, _L, _L, _I, _P, _P, _P, _P, _P],
    "cmace_imp_bwd_node_f32": [_P, _P, _P, _L, _I, _P, _P],
    "cmace_imp_bwd_node_f64": [_P, _P, _P, _L, _I, _P, _P],
    "cmace_linear_f32": [_P, _P, _P, _P, _I, _L, _I, _I, _P, _P],
    "cmace_linear_f64": [_P, _P, _P, _P, _I, _L, _I, _I, _P, _P],
    "cmace_symcon_plan_create": [_I, _P, _P, _P, _P, _P, _P, _I, _I, _I, ctypes.POINTER(_P)],
    "cmace_symcon_plan_destroy": [_P],
    "cmace_symcon_plan_nterms": [_P],
    "cmace_symcon_plan_nclasses": [_P],
    "cmace_symcon_fwd_f32": [_P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
    "cmace_symcon_fwd_f64": [_P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
    "cmace_symcon_bwd_f32": [_P, _P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
    "cmace_symcon_bwd_f64": [_P, _P, _P, _P, _P, _P, _P, _I, _L, _I, _P, _P],
}
_RESTYPES = {
    "cmace_sender_order_workspace_bytes": _L,
    "cmace_imp_bwd_scratch_elems": _L,
    "cmace_symcon_plan_destroy": None,
}
# functions whose integer result is a value, not a status
_VALUE_FUNCS = {"cmace_abi_version", "cmace_sender_order_workspace_bytes", "cmace_imp_bwd_scratch_elems",
                "cmace_symcon_plan_destroy", "cmace_symcon_plan_nterms", "cmace_symcon_plan_nclasses"}

_lib = None


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


def call(name, *args):
    """Calls a status-returning entry point; raises RuntimeError with the library's message."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if name in _VALUE_FUNCS:
        return rc
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {lib.cmace_last_error().decode()}")
    return 0
