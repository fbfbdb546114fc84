"""ctypes declarations for every symbol of include/tfb.h."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtfb.so")

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
EPI_NONE, EPI_BIAS_COL, EPI_BIAS_ROW, EPI_RELU = 0, 1, 2, 4
(TUNE_GEMM_TILE_N, TUNE_GEMM_PAIR, TUNE_GEMM_SPLIT_K, TUNE_GEMM_CHUNK_KB, TUNE_CONV_TMA, TUNE_CONV_DIRECT,
 TUNE_CONV_PAIR, TUNE_HOST_PANEL_ROWS, TUNE_PDL, TUNE_FUSE_PLANES, TUNE_GEMM_GROUP_M, TUNE_SMALL_GEMM,
 TUNE_RAW_HI, TUNE_CLUSTER_K) = range(14)


class TfbError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"libtfb error {code}: {message}")
        self.code = code


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `make -C tensors_b200/csrc` "
        "(or `python -c 'import __graft_entry__ as g; g.build()'`). There is no fallback path."
    )

lib = ctypes.CDLL(LIB_PATH)

_vp, _i64, _i32, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
_ip = ctypes.POINTER(ctypes.c_int)

# name -> (restype, argtypes); kept in the order of include/tfb.h
PROTOTYPES = {
    "tfb_init": (_i32, []),
    "tfb_last_error_string": (ctypes.c_char_p, []),
    "tfb_set_tuning": (_i32, [_i32, _i32]),
    "tfb_get_tuning": (_i32, [_i32, _ip]),
    "tfb_device_status": (_i32, [_ip]),
    "tfb_inject_device_status": (_i32, [_i32, _i32]),
    "tfb_gemm": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tfb_matmul": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tfb_matmul_batched": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tfb_gemm_trace": (_i32, [_vp]),
    "tfb_gemm_describe_plan": (_i32, [_i64, _i64, _i64, _i32, _i32, ctypes.POINTER(ctypes.c_int)]),
    "tfb_gemm_ex": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32,
                           _vp, _i32, _vp]),
    "tfb_split_tf32": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _vp]),
    "tfb_gemm_presplit": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _vp,
                                 _i32, _vp]),
    "tfb_matmul_host": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tfb_matmul_host_b_resident": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tfb_matmul_row_panels": (_i32, [_i32, _ip, ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_vp),
                                     ctypes.POINTER(_i64), _i64, _i64, _i32, _i32, ctypes.POINTER(_vp)]),
    "tfb_matmul_f32_static_limit": (_sz, []),
    "tfb_matmul_f32_static": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "tfb_matmul_backward": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tfb_linear_forward": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tfb_linear_backward": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp]),
    "tfb_linear_backward_presplit": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                            _i32, _vp]),
    "tfb_conv_out_dim": (_i64, [_i64, _i64, _i64, _i64, _i64]),
    "tfb_conv2d_forward": (_i32, [_vp, _vp, _vp, _vp] + [_i64] * 13 + [_i32, _i32, _vp]),
    "tfb_conv2d_backward": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp] + [_i64] * 13 + [_i32, _vp]),
    "tfb_im2col_index_map": (_i32, [_vp] + [_i64] * 13 + [_vp]),
    "tfb_log_softmax_nll": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "tfb_sgd_momentum": (_i32, [_vp, _vp, _vp, _i64, ctypes.c_float, ctypes.c_float, ctypes.c_float, _vp]),
    "tfb_mlp_create": (_i32, [_i32, ctypes.POINTER(_i64), _i64, ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_mlp_destroy": (_i32, [_vp]),
    "tfb_mlp_numel": (_i64, [_vp]),
    "tfb_mlp_segment": (_i32, [_vp, _i32, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "tfb_mlp_buffer": (_i32, [_vp, _i32, _i32, ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_mlp_forward_backward": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "tfb_mlp_update": (_i32, [_vp, ctypes.c_float, ctypes.c_float, _vp]),
    "tfb_mlp_exchange_update": (_i32, [_vp, ctypes.c_float, ctypes.c_float, _vp]),
    "tfb_mlp_step": (_i32, [_vp, _vp, _vp, _i64, _i64, ctypes.c_float, ctypes.c_float, _vp]),
    "tfb_mlp_capture_step": (_i32, [_vp, _vp, _vp, _i64, _i64, ctypes.c_float, ctypes.c_float, _i32, _vp]),
    "tfb_mlp_replay": (_i32, [_vp, _vp]),
    "tfb_mlp_set_option": (_i32, [_vp, _i32, _i64]),
    "tfb_mlp_ipc_handle_bytes": (_sz, []),
    "tfb_mlp_ipc_handle": (_i32, [_vp, _vp]),
    "tfb_mlp_connect_ipc": (_i32, [_vp, _i32, _i32, _vp]),
    "tfb_mlp_connect_ptrs": (_i32, [_vp, _i32, _i32, ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_mlp_connect_local": (_i32, [ctypes.POINTER(ctypes.c_void_p), _i32]),
    "tfb_mlp_exchange_update_one_device": (_i32, [ctypes.POINTER(ctypes.c_void_p), _i32, ctypes.c_float,
                                                   ctypes.c_float, _vp]),
    "tfb_peer_group_create": (_i32, [_i64, ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_peer_group_destroy": (_i32, [_vp]),
    "tfb_peer_group_buffers": (_i32, [_vp, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                      ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_peer_group_set_wait_limit": (_i32, [_vp, _i64]),
    "tfb_peer_group_ipc_handle": (_i32, [_vp, _vp]),
    "tfb_peer_group_connect_ipc": (_i32, [_vp, _i32, _i32, _vp]),
    "tfb_peer_group_connect_ptrs": (_i32, [_vp, _i32, _i32, ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_peer_allreduce_sum": (_i32, [_vp, _i64, _vp]),
    "tfb_peer_allreduce_sum_one_device": (_i32, [ctypes.POINTER(ctypes.c_void_p), _i32, _i64, _vp]),
    "tfb_conv2d_backward_sharded": (_i32, [_vp, _vp, _vp, _vp, _vp] + [_i64] * 13 + [_i32, _vp]),
    "tfb_fill": (_i32, [_vp, _i64, ctypes.c_float, _vp]),
    "tfb_relu_forward": (_i32, [_vp, _vp, _i64, _vp]),
    "tfb_relu_backward": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "tfb_accumulate": (_i32, [_vp, _vp, _i64, _vp]),
    "tfb_scale_by_device_scalar": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "tfb_device_count": (_i32, [_ip]),
    "tfb_alloc": (_i32, [_i32, _sz, _vp, ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_free": (_i32, [_vp, _i32, _vp]),
    "tfb_pool_set_release_threshold": (_i32, [_i32, ctypes.c_uint64]),
    "tfb_pool_trim": (_i32, [_i32, _sz]),
    "tfb_pool_stats": (_i32, [_i32] + [ctypes.POINTER(ctypes.c_uint64)] * 4),
    "tfb_pool_enable_peer": (_i32, [_i32, _i32]),
    "tfb_scratch_stats": (_i32, [_i32] + [ctypes.POINTER(ctypes.c_uint64)] * 2),
    "tfb_set_device": (_i32, [_i32]),
    "tfb_get_device": (_i32, [_ip]),
    "tfb_stream_create": (_i32, [_i32, ctypes.POINTER(ctypes.c_void_p)]),
    "tfb_stream_destroy": (_i32, [_vp]),
    "tfb_stream_synchronize": (_i32, [_vp]),
    "tfb_memcpy": (_i32, [_vp, _vp, _sz, _i32, _vp]),
}

for _name, (_res, _args) in PROTOTYPES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.tfb_last_error_string().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != 0:
        raise TfbError(rc, last_error())


def device_status() -> int:
    """Synchronises the current device and returns the first error a kernel recorded."""
    code = ctypes.c_int(0)
    rc = lib.tfb_device_status(ctypes.byref(code))
    if rc != 0 and code.value == 0:
        raise TfbError(rc, last_error())
    return code.value
