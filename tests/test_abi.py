"""CPU tests of the boundary: the C-ABI library loads, exports every declared symbol, and fails loudly without a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from eddl_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_declares_the_expected_surface():
    names = [n for n, _, _ in capi.declared_functions()]
    assert len(names) == len(set(names)) and len(names) >= 60
    for must in ("eddlb200_conv2d_fwd", "eddlb200_conv2d_bwd_data", "eddlb200_conv2d_bwd_weight", "eddlb200_bn_fwd", "eddlb200_bn_bwd",
                 "eddlb200_maxpool2d_fwd", "eddlb200_avgpool2d_bwd", "eddlb200_softmax_fwd", "eddlb200_cce_value", "eddlb200_accuracy",
                 "eddlb200_mult2d", "eddlb200_sgd_momentum_multi", "eddlb200_adam", "eddlb200_allreduce_avg", "eddlb200_avg_grad_sgd"):
        assert must in names


def test_library_exports_every_declared_symbol():
    cdll = ctypes.CDLL(capi.LIBPATH)
    missing = [n for n, _, _ in capi.declared_functions() if not hasattr(cdll, n)]
    assert not missing, missing


def test_every_declaration_cites_the_reference():
    text = open(capi.HEADER).read()
    assert text.count("src/hardware/gpu/") >= 8 and text.count("src/hardware/cpu/") >= 6
    assert "src/optimizers/optim_sgd.cpp" in text and "src/net/net_func.cpp" in text


def test_no_cpu_fallback_without_a_gpu():
    L = capi.lib()
    if L.device_count() > 0:
        pytest.skip("a GPU is visible")
    a = np.zeros(4, np.float32)
    with pytest.raises(capi.Error):
        L.call("fill", 0, a.ctypes.data_as(ctypes.c_void_p), 4, 1.0)
    assert L.last_error()


def test_product_code_never_touches_the_oracle():
    bad = []
    for d, _, fs in os.walk(os.path.join(ROOT, "eddl_b200")):
        for f in fs:
            if f.endswith((".py", ".cpp", ".cu", ".cuh", ".h")):
                t = open(os.path.join(d, f), errors="ignore").read()
                # no import of the oracle package, none of its modules by name (also not through a sys.path entry), no path into it
                if re.search(r"^\s*(from|import)\s+oracle|oracle/_ref|eddl_oracle|build_ref|ref_capi|[\"']oracle[\"']|oracle/", t, flags=re.M):
                    bad.append(f)
    assert not bad, bad


def test_dropin_library_exports_harness_and_distributed_api():
    from eddl_b200 import harness
    if not os.path.exists(harness.DROPIN):
        pytest.skip("drop-in library not built (needs the EDDL source tree)")
    cdll = harness.load()
    for s in ("ebh_create", "ebh_train_batch", "ebh_train_resident", "ebh_init_distributed", "ebh_avg_weights", "ebh_broadcast_params"):
        assert hasattr(cdll, s)
    # mangled C++ names of the new entry points and of a few reference gpu_* functions defined by the shim
    for s in ("_ZN9eddl_b20016init_distributedEv", "_ZN9eddl_b20023avg_weights_distributedEP3Netii",
              "_ZN9eddl_b20028broadcast_params_distributedEP3Net", "_Z10gpu_conv2DP16ConvolDescriptor", "_Z8gpu_reluP6TensorS0_"):
        assert hasattr(cdll, s), s


def test_tuning_options_are_host_side_switches():
    """The kernel tuning switches are plain host state: they can be set without a GPU, and unknown names or values are refused."""
    cdll = ctypes.CDLL(capi.LIBPATH)
    cdll.eddlb200_set_option.argtypes = [ctypes.c_char_p, ctypes.c_int]
    cdll.eddlb200_set_option.restype = ctypes.c_int
    for name, value in ((b"conv_prefetch", 0), (b"conv_prefetch", 1), (b"bn_waves", 4), (b"bn_waves", 16),
                        (b"bn_min_items", 2048), (b"bn_min_items", 8192), (b"conv_path", 0), (b"conv_tma", 0), (b"conv_tma", 2), (b"conv_tma_wgrad", 0), (b"conv_tma_wgrad", 2),
                        (b"conv_tma_3x3", 0), (b"conv_tma_3x3", 1), (b"conv_tma_wgrad_3x3", 0), (b"conv_tma_wgrad_3x3", 1), (b"conv_dense_1x1", 0), (b"conv_dense_1x1", 1), (b"conv_pack_cache", 0), (b"conv_pack_cache", 1)):
        assert cdll.eddlb200_set_option(name, value) == 0, (name, value)
    for name, value in ((b"conv_prefetch", 2), (b"bn_waves", 0), (b"no_such_option", 1), (b"conv_path", 7), (b"conv_tma", 3), (b"conv_tma_3x3", 2),
                        (b"conv_dense_1x1", -1)):
        assert cdll.eddlb200_set_option(name, value) == -1, (name, value)      # EDDLB200_EINVAL
