"""The C-ABI library loads without a GPU and exports every function include/*.h declares;
the Python prototype table covers the same set. No compute calls here."""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(tfb_[a-z0-9_]+)\s*\(", text))
    return names


def test_header_declares_something():
    assert len(declared_symbols()) >= 7


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(os.path.join(ROOT, "tensors_b200", "libtfb.so"))
    missing = [n for n in sorted(declared_symbols()) if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_python_prototypes_match_header():
    import tensors_b200.capi as capi
    assert set(capi.PROTOTYPES) == declared_symbols()


def header_defines(prefix):
    text = open(os.path.join(ROOT, "include", "tfb.h")).read()
    return {m.group(1): int(m.group(2)) for m in re.finditer(r"#define\s+(" + prefix + r"[A-Z0-9_]+)\s+(-?\d+)", text)}


def test_python_constants_match_header_defines():
    # the numbering of the tuning knobs and of the tfb_mlp options is part of the C-ABI: the Python side must
    # not drift from include/tfb.h
    import tensors_b200.capi as capi
    from tensors_b200.mlp import MLP
    knobs = header_defines("TFB_TUNE_")
    count = knobs.pop("TFB_TUNE_COUNT")
    assert sorted(knobs.values()) == list(range(count))
    for name, value in knobs.items():
        assert getattr(capi, name[len("TFB_"):]) == value, name
    opts = header_defines("TFB_MLP_OPT_")
    py = {"TFB_MLP_OPT_WAIT_LIMIT_NS": MLP.OPT_WAIT_NS, "TFB_MLP_OPT_EXCHANGE_CTAS": MLP.OPT_CTAS,
          "TFB_MLP_OPT_KEEP_REDUCED_GRADS": MLP.OPT_KEEP_REDUCED, "TFB_MLP_OPT_TRACE_EXCHANGE": MLP.OPT_TRACE,
          "TFB_MLP_OPT_EXCHANGE_BUCKETS": MLP.OPT_BUCKETS}
    assert opts == py


def test_dispatch_of_the_named_shapes_is_pinned():
    # tfb_gemm_describe_plan is a host function: which kernel and split a shape gets on a 148-SM device under
    # the default knobs. The choices below were each measured to be the fastest on a B200; a change of the cost
    # model that moves one of them has to be measured again.
    import tensors_b200.capi as capi
    lib = capi.lib

    def plan(M, N, K, dtype=capi.DTYPE_F32):
        out = (ctypes.c_int * 5)()
        assert lib.tfb_gemm_describe_plan(M, N, K, dtype, 148, out) == 0
        return dict(zip(("tile_n", "pair", "splits", "cluster", "cuda_core"), out))

    assert plan(8192, 8192, 8192) == dict(tile_n=256, pair=1, splits=1, cluster=0, cuda_core=0)       # the headline
    assert plan(8192, 1024, 784) == dict(tile_n=256, pair=1, splits=1, cluster=0, cuda_core=0)        # MLP forward, full batch
    assert plan(1024, 1024, 8192) == dict(tile_n=256, pair=1, splits=4, cluster=0, cuda_core=0)       # its weight gradients
    assert plan(1024, 1024, 1024) == dict(tile_n=128, pair=0, splits=2, cluster=1, cuda_core=0)       # a 1024-row shard
    assert plan(1024, 784, 1024) == dict(tile_n=128, pair=0, splits=2, cluster=1, cuda_core=0)
    assert plan(2048, 1024, 1024) == dict(tile_n=128, pair=0, splits=1, cluster=0, cuda_core=0)       # a 2048-row shard
    assert plan(64, 256, 784)["cuda_core"] == 1                                                       # config 2 forward
    assert plan(10, 1024, 1024)["cuda_core"] == 1 and plan(1024, 10, 1024)["cuda_core"] == 1          # the 10-class head
    assert plan(10, 1024, 8192)["cuda_core"] == 0 and plan(10, 1024, 8192)["splits"] > 1              # too long for it
    assert plan(1024, 1024, 1024, capi.DTYPE_BF16)["splits"] == 1                                     # 7.5 us unsplit, 12.9 split
    assert plan(512, 512, 4096, capi.DTYPE_BF16)["splits"] > 1                                        # 10.9 us split, 18.9 unsplit
    out = (ctypes.c_int * 5)()
    assert lib.tfb_gemm_describe_plan(0, 8, 8, 0, 148, out) == -1
    assert lib.tfb_gemm_describe_plan(8, 8, 8, 7, 148, out) == -2


def test_tuning_knobs_and_host_only_queries_work_without_gpu():
    # knobs are plain host state (defaults, or the environment read once); nothing here touches CUDA
    import ctypes
    import tensors_b200.capi as capi
    lib = capi.lib
    v = ctypes.c_int(-99)
    assert lib.tfb_get_tuning(capi.TUNE_PDL, ctypes.byref(v)) == 0 and v.value in (0, 1)
    old = v.value
    assert lib.tfb_set_tuning(capi.TUNE_PDL, 0) == 0
    assert lib.tfb_get_tuning(capi.TUNE_PDL, ctypes.byref(v)) == 0 and v.value == 0
    assert lib.tfb_set_tuning(capi.TUNE_PDL, old) == 0
    assert lib.tfb_set_tuning(999, 1) == -1 and "knob" in capi.last_error()
    assert lib.tfb_get_tuning(capi.TUNE_GEMM_TILE_N, None) == -1
    assert lib.tfb_conv_out_dim(32, 3, 1, 1, 1) == 32 and lib.tfb_conv_out_dim(13, 3, 2, 1, 2) == 6
    assert lib.tfb_mlp_numel(None) == 0
    assert lib.tfb_mlp_ipc_handle_bytes() == 64
    assert lib.tfb_matmul_f32_static_limit() == 16 << 20
    n, b = ctypes.c_uint64(7), ctypes.c_uint64(7)
    assert lib.tfb_scratch_stats(0, ctypes.byref(n), ctypes.byref(b)) == 0 and (n.value, b.value) == (0, 0)


def test_flat_parameter_layout_matches_the_documented_rule():
    # every weight and bias starts on a multiple of 4 floats (16 bytes): the layout tfb_mlp_segment reports
    from tensors_b200.mlp import flat_layout, shard_rows
    offsets, numel = flat_layout((784, 1024, 1024, 10))
    assert offsets == [0, 802816, 803840, 1852416, 1853440, 1863680] and numel == 1863692
    offsets, numel = flat_layout((5, 3, 2))
    assert offsets == [0, 16, 20, 28] and numel == 32
    assert all(o % 4 == 0 for o in offsets)
    assert [shard_rows(8192, r, 8) for r in (0, 7)] == [(0, 1024), (7168, 8192)]


def test_error_string_is_callable_without_gpu():
    import tensors_b200.capi as capi
    assert isinstance(capi.last_error(), str)
