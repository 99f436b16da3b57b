"""The GPU kernel tests once more with IEEE half elements: the same test functions, run against the half-precision
build of the kernel library (``libfbam_kernels_fp16.so``).  The reference parametrises its operator tests over
{bf16, fp16} the same way (``tests/common/test_dtype_utils.h:47-62``); fp16 is its default model dtype
(``src/config.cpp:43-51``).  Every comparison is against the fp32 PyTorch definition of the op, as in the bf16 run."""
import pytest
import torch

import test_gpu_kernels as K
import test_gpu_embconv as E

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _half_elements(monkeypatch):
    monkeypatch.setattr(K, "BF", torch.float16)
    monkeypatch.setattr(E, "BF", torch.float16)
    yield


from test_gpu_kernels import (  # noqa: E402,F401  (collected here, with this module's fixture)
    test_gemm_k_major, test_gemm_split_k_with_slab_reduction, test_gemm_mn_major_operands, test_gemm_operands_without_16_byte_pitch, test_gemm_tall_tiles,
    test_gemm_epilogues, test_conv_fprop_and_dgrad, test_linear_autograd_matches_reference, test_rmsnorm_fwd_bwd,
    test_layernorm_gelu_geglu_pools, test_layernorm_fwd_bwd, test_cell_embed_fwd_bwd, test_lm_head_ce_fwd_bwd,
    test_persistent_lstm_fwd_bwd, test_conv_wgrad, test_conv_gelu_stack_pool_matches_unfused_reference,
    test_flash_attention_fwd_bwd, test_gemm_cta_pairs, test_conv_cta_pairs, test_linear_relu_fwd_bwd,
    test_strided_dgrad_with_fused_parity_classes,
    test_expected_backends_are_chosen_on_gpu)
from test_gpu_embconv import (  # noqa: E402,F401
    test_colour_features_kernel, test_forward_gather_kernel, test_backward_reduce_kernel,
    test_one_tap_weight_gradient_is_a_plain_product, test_cell_conv_gelu_matches_separate_ops,
    test_fused_cells_stack_matches_unfused_reference)


def test_half_library_is_the_one_that_ran():
    """The half-precision tensors above must have gone through the library built with half elements."""
    from fbamtrain_b200.ops import native as nv
    x = torch.randn(256, 256, device="cuda").half()
    from fbamtrain_b200.ops import native_ops as no
    before = nv.launches()
    y = no.gemm(x, x)
    assert nv.launches() == before + 1 and y.dtype == torch.float16
    assert nv.lib(torch.float16).fbam_elem_is_fp16() == 1 and nv.lib(torch.bfloat16).fbam_elem_is_fp16() == 0
    assert nv.lib(torch.float16) is not nv.lib(torch.bfloat16)
