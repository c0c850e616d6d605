"""The C-ABI library loads and exports every symbol include/seera_b200.h declares, and the Python
binding module exports every function name of the reference's binding.  No compute, no GPU."""
import ctypes
import os

import pytest

from ml_framework_b200 import capi

# the 60 m.def names of engine_cuda/src/cuda_bindings.cpp:23-532
REFERENCE_BINDING_NAMES = """
cuda_malloc cuda_malloc_f16 cuda_malloc_f32 cuda_malloc_i32 cuda_malloc_i16 cuda_free cuda_memcopy_devicetodevice cuda_memset
to_device_f16 to_host_f16 to_device_f32 to_host_f32 to_host_i32 to_host_i16 to_device_i16 to_device_i32
cuda_relu_fwd cuda_sigmoid_fwd cuda_tanh_fwd cuda_log_fwd cuda_exp_fwd cuda_abs_fwd cuda_sqrt_fwd cuda_pow_fwd cuda_clip_fwd
cuda_softmax_fwd cuda_softmax_vjp cuda_matmul cuda_matmul_bwd cuda_transpose_2d cuda_transpose_3d
cuda_conv2d_fwd cuda_conv2d_bwd cuda_conv2DTranpose_fwd cuda_conv2DTranspose_bwd
cuda_maxpool_fwd cuda_maxpool_bwd cuda_unpooling_fwd cuda_unpooling_bwd
cuda_sum_fwd cuda_mean_fwd cuda_max_fwd cuda_min_fwd cuda_argmax_fwd cuda_argmin_fwd
cuda_sum_bwd cuda_mean_bwd cuda_max_bwd cuda_min_bwd
cuda_scaler_multiply_f cuda_scaler_add_f cuda_ones_f cuda_zeros_f cuda_power_of
cuda_elemadd cuda_elemsub cuda_elemdiv cuda_elemmult broadcast_add_4d broadcast_mul_4d
""".split()


def test_reference_binding_has_sixty_names():
    assert len(REFERENCE_BINDING_NAMES) == 60 and len(set(REFERENCE_BINDING_NAMES)) == 60


def test_library_exports_every_declared_symbol():
    assert os.path.exists(capi.LIB_PATH), "build first: python -m ml_framework_b200.build"
    decl = capi.declared_functions()
    assert len(decl) >= 70
    lib = ctypes.CDLL(capi.LIB_PATH)
    missing = [n for n, _, _ in decl if not hasattr(lib, n)]
    assert not missing, missing
    capi.load()                                           # binds argtypes for every declaration


def test_binding_module_exports_the_reference_names():
    import ml_framework_b200.seera_cuda as sc
    missing = [n for n in REFERENCE_BINDING_NAMES if not hasattr(sc, n)]
    assert not missing, missing
    for extra in ("cuda_adam_step", "cuda_sgd_step", "bias_act_fwd", "act_bias_bwd", "softmax_cce_fwd_bwd",
                  "stream_synchronize", "last_status", "set_precision", "launch_count"):
        assert hasattr(sc, extra)


def test_no_device_gives_an_error_not_a_fallback():
    import ml_framework_b200.seera_cuda as sc
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        sc.cuda_malloc_f32(16)
