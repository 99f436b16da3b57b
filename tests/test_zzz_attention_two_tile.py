"""The opt-in attention forward with two query tiles per CTA (``FBAMTRAIN_ATTENTION_FWD2=1``) against the fp32
PyTorch definition, forward and (through the unchanged backward kernel, which consumes its output and log-sum-exp)
backward.  Runs only when the variable is set: the variant is not the default path."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("FBAMTRAIN_ATTENTION_FWD2") != "1",
                                 reason="set FBAMTRAIN_ATTENTION_FWD2=1 to test the two-tile forward")]


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,t,h,d", [(2, 128, 2, 64), (1, 300, 3, 64), (2, 256, 2, 128), (1, 1024, 4, 64),
                                     (1, 480, 2, 128), (1, 129, 1, 128)])
def test_two_tile_forward_matches_reference(causal, b, t, h, d):
    from fbamtrain_b200.ops import native as nv
    from fbamtrain_b200.ops import reference as ref
    from fbamtrain_b200.ops.mha import flash_attention
    from fbamtrain_b200.utils.testing import assert_similar
    torch.manual_seed(14)
    qkv = torch.randn(b, t, 3, h, d, device="cuda").to(torch.bfloat16).requires_grad_(True)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    o = flash_attention(q, k, v, causal)
    nv.check_status(qkv.device)
    g = torch.randn_like(o)
    (gqkv,) = torch.autograd.grad(o, qkv, g)
    nv.check_status(qkv.device)
    f = qkv.detach().float().requires_grad_(True)
    of = ref.attention(f[:, :, 0], f[:, :, 1], f[:, :, 2], causal)
    (eqkv,) = torch.autograd.grad(of, f, g.float())
    assert_similar(of.to(torch.bfloat16), o, 3e-2)
    for i in range(3):
        err = float((gqkv[:, :, i].float() - eqkv[:, :, i]).norm() / eqkv[:, :, i].norm())
        assert err < 3e-2, (i, err)
