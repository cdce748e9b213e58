"""ctypes binding of libyitu_b200.so (the C ABI declared in include/yitu_b200.h).

There is no fallback: if the CUDA library has not been built, importing an operator module raises.
Build it with `python -m yitu_b200.build`.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libyitu_b200.so")

OK, ERR_INVALID_ARG, ERR_CUDA, ERR_WORKSPACE, ERR_UNSUPPORTED, ERR_LIMIT = range(6)
W_NONE, W_NODE, W_EDGE, W_EDGE_HEAD = range(4)
ACT_NONE, ACT_RELU, ACT_ELU = range(3)

c_i64, c_i32, c_f32, c_vp = C.c_int64, C.c_int32, C.c_float, C.c_void_p


class Csr(C.Structure):
    _fields_ = [("n_rows", c_i64), ("n_cols", c_i64), ("nnz", c_i64), ("indptr", c_vp), ("indptr_is64", c_i32),
                ("index_mask", c_i32), ("indices", c_vp)]


class HubPlan(C.Structure):
    _fields_ = [("chunk_edges", c_i32), ("reserved", c_i32), ("n_chunks", c_i64), ("chunk_row", c_vp),
                ("chunk_begin", c_vp)]


class SpmmArgs(C.Structure):
    _fields_ = [("graph", Csr), ("n_heads", c_i64), ("n_feats", c_i64), ("weight_mode", c_i32), ("accumulate", c_i32),
                ("edge_values", c_vp), ("edge_perm", c_vp), ("norm_dst", c_vp), ("norm_src", c_vp),
                ("row_scale", c_vp), ("alpha", c_f32), ("activation", c_i32), ("x", c_vp), ("x_stride", c_i64),
                ("out", c_vp), ("out_stride", c_i64), ("plan", C.POINTER(HubPlan)), ("scratch", c_vp),
                ("scratch_bytes", c_i64), ("bias", c_vp), ("x_shared_heads", c_i32), ("reserved", c_i32)]


class SpmmBwdArgs(C.Structure):
    _fields_ = [("graph", Csr), ("n_heads", c_i64), ("n_feats", c_i64), ("edge_values", c_vp), ("x", c_vp),
                ("grad_out", c_vp), ("t_indptr", c_vp), ("t_rows", c_vp), ("t_perm", c_vp), ("grad_values", c_vp),
                ("grad_x", c_vp), ("t_plan", C.POINTER(HubPlan)), ("scratch", c_vp), ("scratch_bytes", c_i64)]


class GatArgs(C.Structure):
    _fields_ = [("graph", Csr), ("n_heads", c_i64), ("n_feats", c_i64), ("slope", c_f32), ("head_mean", c_i32),
                ("query", c_vp), ("key", c_vp), ("x", c_vp), ("out", c_vp), ("row_max", c_vp), ("row_sum", c_vp),
                ("activation", c_i32), ("reserved", c_i32), ("out_heads", c_vp), ("plan", C.POINTER(HubPlan)),
                ("scratch", c_vp), ("scratch_bytes", c_i64)]


class GatBwdArgs(C.Structure):
    _fields_ = [("fwd", GatArgs), ("grad_out", c_vp), ("t_indptr", c_vp), ("t_rows", c_vp), ("t_perm", c_vp),
                ("grad_query", c_vp), ("grad_key", c_vp), ("grad_x", c_vp), ("edge_attn", c_vp), ("edge_grad", c_vp),
                ("t_plan", C.POINTER(HubPlan)), ("scratch", c_vp), ("scratch_bytes", c_i64)]


# every symbol include/yitu_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "yitu_status_string": (C.c_char_p, [C.c_int]),
    "yitu_last_error": (C.c_char_p, []),
    "yitu_version": (C.c_int, []),
    "yitu_hub_plan_workspace_bytes": (c_i64, [c_i64]),
    "yitu_hub_plan_count": (C.c_int, [C.POINTER(Csr), c_i32, c_vp, c_i64, C.POINTER(c_i64), c_vp]),
    "yitu_hub_plan_fill": (C.c_int, [C.POINTER(Csr), c_i32, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "yitu_csr_transpose_workspace_bytes": (c_i64, [c_i64, c_i64, c_i64]),
    "yitu_csr_transpose": (C.c_int, [C.POINTER(Csr), c_vp, c_vp, c_vp, c_vp, c_i64, c_vp]),
    "yitu_partition_rows": (C.c_int, [C.POINTER(Csr), c_i32, c_vp, c_vp]),
    "yitu_partition_rows_host": (C.c_int, [c_i64, c_vp, c_i32, c_i32, c_vp]),
    "yitu_coo_to_csr_workspace_bytes": (c_i64, [c_i64, c_i64, c_i32]),
    "yitu_coo_to_csr": (C.c_int, [c_i64, c_i64, c_i64, c_vp, c_vp, c_i32, c_vp, c_i32, c_vp, C.POINTER(c_i64), c_vp, c_i64,
                                  c_vp]),
    "yitu_degree_norm_f32": (C.c_int, [c_i64, c_vp, c_i32, c_i32, c_vp, c_vp]),
    "yitu_stitch_csr": (C.c_int, [c_i32, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "yitu_build_part_count_host": (c_i64, [c_i32, c_vp, c_i64]),
    "yitu_build_part_host": (C.c_int, [c_i32, c_vp, c_i64, c_vp, c_vp]),
    "yitu_stitch_csr_host": (C.c_int, [c_i32, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "yitu_reorder_workspace_bytes": (c_i64, [c_i64, c_i64, c_i32]),
    "yitu_reorder_communities": (C.c_int, [c_i64, c_i64, c_vp, c_vp, c_i32, c_vp, C.POINTER(c_i32), C.POINTER(c_i64), c_vp,
                                           c_i64, c_vp]),
    "yitu_relabel_edges": (C.c_int, [c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "yitu_edge_span_sum": (C.c_int, [c_i64, c_vp, c_vp, c_vp, c_vp]),
    "yitu_spmm_csr_f32": (C.c_int, [C.POINTER(SpmmArgs), c_vp]),
    "yitu_spmm_bwd_f32": (C.c_int, [C.POINTER(SpmmBwdArgs), c_vp]),
    "yitu_static_scratch_bytes": (c_i64, []),
    "yitu_spmm_csr_f32_static": (C.c_int, [C.POINTER(SpmmArgs), c_vp]),
    "yitu_epilogue_grad_f32": (C.c_int, [c_i64, c_i64, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "yitu_segment_mean_weights_f32": (C.c_int, [C.POINTER(Csr), c_vp, c_vp]),
    "yitu_edge_dot_f32": (C.c_int, [C.POINTER(Csr), c_i64, c_i64, c_vp, c_vp, c_vp, C.POINTER(HubPlan), c_vp]),
    "yitu_edge_softmax_fwd_f32": (C.c_int, [C.POINTER(Csr), c_i32, c_i64, c_f32, c_vp, c_vp, c_vp, C.POINTER(HubPlan),
                                            c_vp]),
    "yitu_edge_softmax_bwd_f32": (C.c_int, [C.POINTER(Csr), c_i32, c_i64, c_f32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp,
                                            C.POINTER(HubPlan), c_vp]),
    "yitu_edge_gather_sum_f32": (C.c_int, [c_i64, c_vp, c_i32, c_vp, c_i64, c_vp, c_vp, C.POINTER(HubPlan), c_vp]),
    "yitu_gat_fwd_scratch_bytes": (c_i64, [c_i64, c_i64, c_i64]),
    "yitu_gat_bwd_scratch_bytes": (c_i64, [c_i64, c_i64, c_i64, c_i64, c_i64]),
    "yitu_gat_fwd_f32": (C.c_int, [C.POINTER(GatArgs), c_vp]),
    "yitu_gat_bwd_f32": (C.c_int, [C.POINTER(GatBwdArgs), c_vp]),
    "yitu_shared_alloc": (C.c_int, [c_i64, C.POINTER(c_vp), c_vp]),
    "yitu_shared_open": (C.c_int, [c_vp, C.POINTER(c_vp)]),
    "yitu_shared_close": (C.c_int, [c_vp]),
    "yitu_shared_free": (C.c_int, [c_vp]),
    "yitu_halo_gather_f32": (C.c_int, [c_i32, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp]),
    "yitu_halo_push_f32": (C.c_int, [c_i32, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_i32, c_vp]),
    "yitu_flags_signal": (C.c_int, [c_i32, c_vp, C.c_uint64, c_vp]),
    "yitu_flags_wait": (C.c_int, [c_vp, C.c_uint32, C.c_uint64, c_i64, c_vp, c_vp]),
}

_lib = None


class YituError(RuntimeError):
    """Failure reported by the C ABI (the reference raises c10::Error -> RuntimeError on a bad argument)."""

    def __init__(self, status, detail):
        RuntimeError.__init__(self, "yitu_b200: %s" % detail)
        self.status = status


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("yitu_b200: %s is missing — build it with `python -m yitu_b200.build`; "
                              "there is no CPU or PyTorch fallback for these operators" % LIB_PATH)
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status):
    if status != OK:
        L = lib()
        detail = L.yitu_last_error().decode() or L.yitu_status_string(status).decode()
        raise YituError(status, "%s (%s)" % (detail, L.yitu_status_string(status).decode()))
