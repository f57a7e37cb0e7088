"""ctypes binding of ``libscn_b200.so`` (``include/scn_b200.h``).

The library is the only compute path: if it is missing or does not export a symbol the
import fails loudly.  There is no CPU or PyTorch fallback.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libscn_b200.so")

_i64p = C.POINTER(C.c_int64)
_vp = C.c_void_p

# name -> (restype, argtypes); mirrors include/scn_b200.h one to one
SIGNATURES = {
    "scn_abi_version": (C.c_int, []),
    "scn_status_string": (C.c_char_p, [C.c_int]),
    "scn_last_error": (C.c_char_p, []),
    "scn_launch_count": (C.c_longlong, []),
    "scn_rulebook_build_count": (C.c_longlong, []),
    "scn_host_wait_count": (C.c_longlong, []),
    "scn_last_conv_kernel": (C.c_int, []),
    "scn_tc_probe_mma": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp,
                                   C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "scn_test_drop_barrier_arrival": (C.c_int, []),
    "scn_set_weight_token": (C.c_int, [C.c_uint64]),
    "scn_release_weight_token": (C.c_int, [C.c_uint64, _vp]),
    "scn_set_deferred_counts": (C.c_int, [C.c_int]),
    "scn_set_backward_precision": (C.c_int, [C.c_int]),
    "scn_md_take_count_ticket": (C.c_int, [_vp, C.POINTER(_vp)]),
    "scn_count_ticket_total": (C.c_int, [_vp, _i64p]),
    "scn_count_ticket_release": (C.c_int, [_vp]),
    "scn_md_create": (C.c_int, [C.c_int, C.POINTER(_vp)]),
    "scn_md_destroy": (C.c_int, [_vp]),
    "scn_md_destroy_on_stream": (C.c_int, [_vp, _vp]),
    "scn_trim_memory": (C.c_int, [C.c_uint64]),
    "scn_memory_usage": (C.c_int, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "scn_md_clear": (C.c_int, [_vp, _vp]),
    "scn_md_input_layer": (C.c_int, [_vp, _i64p, _vp, C.c_int, C.c_int64, C.c_int, C.c_int64,
                                     C.c_int, _vp, _i64p]),
    "scn_md_bl_input_layer": (C.c_int, [_vp, _i64p, _vp, C.c_int, C.c_int64, C.c_int64, C.c_int, _vp, _i64p]),
    "scn_input_layer_forward": (C.c_int, [_vp, _vp, C.c_int64, _vp, C.c_int64, C.c_int, _vp]),
    "scn_output_layer_forward": (C.c_int, [_vp, _vp, C.c_int64, _vp, C.c_int64, C.c_int, _vp]),
    "scn_md_poll_errors": (C.c_int, [_vp, _vp]),
    "scn_md_n_active": (C.c_int, [_vp, _i64p, _i64p]),
    "scn_md_batch_size": (C.c_int, [_vp, _i64p, _i64p]),
    "scn_md_spatial_locations": (C.c_int, [_vp, _i64p, _vp, _vp]),
    "scn_md_submanifold_rulebook": (C.c_int, [_vp, _i64p, _i64p, _vp, _i64p]),
    "scn_md_strided_rulebook": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _i64p, _i64p]),
    "scn_md_strided_chain": (C.c_int, [_vp, _i64p, _i64p, _i64p, C.c_int, _vp, C.POINTER(C.c_int)]),
    "scn_md_strided_chain_start": (C.c_int, [_vp, _i64p, _i64p, _i64p, C.c_int, _vp]),
    "scn_md_rulebook_export": (C.c_int, [_vp, C.c_int, _i64p, _i64p, _i64p, _i64p, _i64p, _vp, _vp]),
    "scn_submanifold_convolution_forward": (C.c_int, [_vp, _i64p, _i64p, _vp, _vp, _vp, _vp, C.c_int,
                                                      C.c_int, C.c_int, C.c_int, _vp,
                                                      C.POINTER(C.c_double)]),
    "scn_submanifold_convolution_forward_static": (C.c_int, [_vp, _i64p, _i64p, _vp, _vp, _vp, _vp, C.c_int,
                                                             C.c_int, C.c_int, _vp]),
    "scn_convolution_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp,
                                          C.c_int, C.c_int, C.c_int, C.c_int, _vp,
                                          C.POINTER(C.c_double)]),
    "scn_deconvolution_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp,
                                            C.c_int, C.c_int, C.c_int, C.c_int, _vp,
                                            C.POINTER(C.c_double)]),
    "scn_batchnorm_join_forward": (C.c_int, [_vp, C.c_int, _vp, C.c_int, _vp, C.c_int64, _vp, _vp, _vp, _vp, C.c_double,
                                             C.c_double, _vp]),
    "scn_rows_affine_forward": (C.c_int, [_vp, _vp, C.c_int64, C.c_int, C.c_int, _vp, _vp, _vp]),
    "scn_batchnorm_fold": (C.c_int, [_vp, _vp, _vp, _vp, C.c_double, C.c_int, _vp, _vp, _vp]),
    "scn_submanifold_convolution_bn_forward": (C.c_int, [_vp, _i64p, _i64p, _vp, _vp, _vp, _vp, _vp, _vp, C.c_double,
                                                         C.c_int, C.c_int, C.c_int, C.c_int, _vp,
                                                         C.POINTER(C.c_double)]),
    "scn_convolution_bn_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp, _vp, _vp,
                                             C.c_double, C.c_int, C.c_int, C.c_int, C.c_int, _vp,
                                             C.POINTER(C.c_double)]),
    "scn_submanifold_convolution_joined_forward": (C.c_int, [_vp, _i64p, _i64p, _vp, C.c_int, _vp, C.c_int, _vp, _vp, _vp,
                                                             _vp, _vp, C.c_double, _vp, _vp, C.c_double, C.c_int,
                                                             C.c_int, _vp, C.POINTER(C.c_double)]),
    "scn_convolution_bn_bn_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp, _vp, _vp,
                                                C.c_double, _vp, _vp, C.c_double, C.c_int, C.c_int, C.c_int, C.c_int,
                                                _vp, C.POINTER(C.c_double)]),
    "scn_deconvolution_bn_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp, _vp, _vp,
                                               C.c_double, C.c_int, C.c_int, C.c_int, C.c_int, _vp,
                                               C.POINTER(C.c_double)]),
    "scn_submanifold_convolution_backward": (C.c_int, [_vp, _i64p, _i64p, _vp, _vp, _vp, _vp, _vp, _vp,
                                                       C.c_int, C.c_int, C.c_int, _vp]),
    "scn_convolution_backward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp, _vp, _vp,
                                           C.c_int, C.c_int, C.c_int, _vp]),
    "scn_deconvolution_backward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp, _vp, _vp,
                                             C.c_int, C.c_int, C.c_int, _vp]),
    "scn_input_layer_backward": (C.c_int, [_vp, _vp, C.c_int64, _vp, C.c_int64, C.c_int, _vp]),
    "scn_output_layer_backward": (C.c_int, [_vp, _vp, C.c_int64, _vp, C.c_int64, C.c_int, _vp]),
    "scn_max_pooling_backward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, _vp, _vp, C.c_int, C.c_int,
                                           _vp]),
    "scn_average_pooling_backward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, C.c_int, C.c_int, _vp]),
    "scn_unpooling_backward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, C.c_int, C.c_int, _vp]),
    "scn_sparse_to_dense_backward": (C.c_int, [_vp, _i64p, _vp, _vp, C.c_int, _vp]),
    "scn_batchnorm_backward": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int64, C.c_int, C.c_int64, C.c_int64, _vp, _vp,
                                         _vp, _vp, _vp, C.c_double, _vp]),
    "scn_batchnorm_forward": (C.c_int, [_vp, _vp, C.c_int64, C.c_int, C.c_int64, C.c_int64, _vp, _vp,
                                        _vp, _vp, _vp, _vp, C.c_double, C.c_double, C.c_int,
                                        C.c_double, _vp]),
    "scn_batchnorm_moments": (C.c_int, [_vp, C.c_int64, C.c_int, C.c_int64, _vp, _vp]),
    "scn_batchnorm_forward_moments": (C.c_int, [_vp, _vp, C.c_int64, C.c_int64, C.c_int, C.c_int64, C.c_int64, _vp,
                                                _vp, _vp, _vp, _vp, _vp, _vp, C.c_double, C.c_double, C.c_double,
                                                _vp]),
    "scn_batchnorm_backward_sums": (C.c_int, [_vp, _vp, _vp, C.c_int64, C.c_int, C.c_int64, C.c_int64, _vp,
                                              C.c_double, _vp, _vp]),
    "scn_batchnorm_backward_sums_apply": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int64, C.c_int64, C.c_int, C.c_int64,
                                                    C.c_int64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_double, _vp]),
    "scn_max_pooling_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, C.c_int, C.c_int,
                                          _vp]),
    "scn_average_pooling_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, C.c_int, C.c_int,
                                          _vp]),
    "scn_unpooling_forward": (C.c_int, [_vp, _i64p, _i64p, _i64p, _i64p, _vp, _vp, C.c_int, C.c_int,
                                          _vp]),
    "scn_sparse_to_dense_forward": (C.c_int, [_vp, _i64p, _vp, _vp, C.c_int, _vp]),
}


class ScnError(RuntimeError):
    def __init__(self, status, message):
        RuntimeError.__init__(self, "scn_b200 status %d: %s" % (status, message))
        self.status = status


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "%s is missing: build it with `python sparseconvnet_b200/build.py` "
            "(there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.scn_abi_version() != 1:
        raise ImportError("libscn_b200.so has ABI version %d, expected 1" % lib.scn_abi_version())
    return lib


lib = _load()


def check(status):
    if status != 0:
        raise ScnError(status, lib.scn_last_error().decode() or lib.scn_status_string(status).decode())


_sizes_cache = {}


def sizes(seq):
    """Host int64 array for a spatial size / filter size / stride.  The arrays are only read by the
    library, so one array per distinct value is kept and shared (a network asks for the same handful of
    sizes hundreds of times per pass; iterating a tensor element by element costs microseconds each)."""
    vals = tuple(seq.tolist()) if hasattr(seq, "tolist") else tuple(int(v) for v in seq)
    arr = _sizes_cache.get(vals)
    if arr is None:
        if len(_sizes_cache) > 4096:
            _sizes_cache.clear()
        arr = _sizes_cache[vals] = (C.c_int64 * len(vals))(*[int(v) for v in vals])
    return arr
