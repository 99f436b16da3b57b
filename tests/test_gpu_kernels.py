"""Numerics of the native sm_100a kernels against plain PyTorch fp32 definitions of the same ops."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from fbamtrain_b200.ops import reference as ref  # noqa: E402
from fbamtrain_b200.utils.testing import assert_similar  # noqa: E402

DEV = "cuda"
BF = torch.bfloat16


def _nops():
    from fbamtrain_b200.ops import native, native_ops
    return native, native_ops


def _rel_err(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 256, 512), (4096, 4096, 4096), (300, 200, 136),
                                   (1000, 72, 256), (64, 64, 64), (8192, 1024, 4096)])
def test_gemm_k_major(m, n, k):
    nv, no = _nops()
    torch.manual_seed(0)
    a = torch.randn(m, k, device=DEV).to(BF)
    b = torch.randn(n, k, device=DEV).to(BF)
    d = no.gemm(a, b)
    nv.check_status(a.device)
    expect = a.float() @ b.float().t()
    assert _rel_err(d, expect) < 5e-3
    assert_similar(expect.to(BF), d, 0.02 * math.sqrt(k))


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 512, 320), (1024, 4096, 8192), (200, 264, 136)])
def test_gemm_mn_major_operands(a_mn, b_mn, m, n, k):
    nv, no = _nops()
    torch.manual_seed(1)
    a = torch.randn(m, k, device=DEV).to(BF)
    b = torch.randn(n, k, device=DEV).to(BF)
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    d = no.gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn)
    nv.check_status(a.device)
    expect = a.float() @ b.float().t()
    assert _rel_err(d, expect) < 5e-3


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True), (False, True)])
@pytest.mark.parametrize("m,n,k", [(200, 100, 100), (128, 36, 52), (77, 130, 1001)])
def test_gemm_operands_without_16_byte_pitch(m, n, k, a_mn, b_mn):
    """Row pitches that are not multiples of 16 bytes (e.g. an embedding width of 100) and bases at odd offsets."""
    nv, no = _nops()
    torch.manual_seed(2)
    a = torch.randn((k, m) if a_mn else (m, k), device=DEV).to(BF)
    flat = torch.randn(n * k + 3, device=DEV).to(BF)
    b = flat[3:].view((k, n) if b_mn else (n, k))                    # base address 6 bytes past an aligned one
    out = no.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    af = a.float().t() if a_mn else a.float()
    bf_ = b.float() if b_mn else b.float().t()
    assert _rel_err(out, af @ bf_) < 1e-2
    nv.check_status(a.device)


@pytest.mark.parametrize("out_dtype", ["elem", "fp32"])
@pytest.mark.parametrize("m,n,k,splits", [(1024, 1024, 8192, 8), (3072, 1024, 8192, 3), (200, 136, 1000, 4)])
def test_gemm_split_k_with_slab_reduction(m, n, k, splits, out_dtype):
    """Split-K for small outputs with a long K (weight gradients of the linear layers): every split writes its fp32
    partial tile to its own slab, one reduction sums the slabs — against the fp32 product."""
    nv, no = _nops()
    torch.manual_seed(2)
    a = torch.randn(k, m, device=DEV).to(BF)          # dY (rows x out features), read as A^T
    b = torch.randn(k, n, device=DEV).to(BF)          # X  (rows x in features)
    dtype = BF if out_dtype == "elem" else torch.float32
    got = no.gemm(a, b, a_mn=True, b_mn=True, out_dtype=dtype, splits=splits)
    nv.check_status(a.device)
    expect = a.float().t() @ b.float()
    assert got.dtype == dtype and _rel_err(got, expect) < (5e-3 if out_dtype == "elem" else 1e-4)
    assert no.weight_grad_splits(1024, 1024, 8192) == 8 and no.weight_grad_splits(4096, 4096, 8192) == 0


@pytest.mark.parametrize("bm", [128, 256])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True)])
def test_gemm_tall_tiles(bm, a_mn, b_mn):
    nv, no = _nops()
    torch.manual_seed(13)
    m, n, k = 1000, 520, 328
    a = torch.randn(m, k, device=DEV).to(BF)
    b = torch.randn(n, k, device=DEV).to(BF)
    d = no.gemm(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, a_mn=a_mn, b_mn=b_mn, bm=bm)
    nv.check_status(a.device)
    assert _rel_err(d, a.float() @ b.float().t()) < 5e-3
    bias = torch.randn(n, device=DEV).to(BF)
    d = no.gemm(a, b, bias=bias, act="gelu", bm=bm, bn=128)
    assert_similar(torch.nn.functional.gelu(a.float() @ b.float().t() + bias.float()).to(BF), d, 0.25)


def test_gemm_epilogues():
    nv, no = _nops()
    torch.manual_seed(2)
    m, n, k = 512, 384, 256
    a = torch.randn(m, k, device=DEV).to(BF)
    b = (torch.randn(n, k, device=DEV) / math.sqrt(k)).to(BF)
    bias = torch.randn(n, device=DEV).to(BF)
    res = torch.randn(m, n, device=DEV).to(BF)
    pre = torch.empty(m, n, device=DEV, dtype=BF)
    z = a.float() @ b.float().t() + bias.float()
    d = no.gemm(a, b, bias=bias, act="gelu", residual=res, preact_out=pre)
    assert_similar((torch.nn.functional.gelu(z) + res.float()).to(BF), d, 3e-2)
    assert_similar(z.to(BF), pre, 3e-2)
    # gelu-gradient epilogue
    aux = torch.randn(m, n, device=DEV).to(BF)
    d2 = no.gemm(a, b, gelu_grad_in=aux)
    assert_similar(((a.float() @ b.float().t()) * ref.gelu_grad(aux)).to(BF), d2, 3e-2)
    # fp32 output, accumulate (read-modify-write and atomic), alpha, fp32 bias
    c0 = torch.randn(m, n, device=DEV)
    out = c0.clone()
    no.gemm(a, b, out=out, accumulate=nv.GEMM_ACC_RMW, alpha=0.5)
    assert_similar(c0 + 0.5 * (a.float() @ b.float().t()), out, 2e-3)
    out = c0.clone()
    no.gemm(a, b, out=out, accumulate=nv.GEMM_ACC_ATOMIC)
    assert_similar(c0 + a.float() @ b.float().t(), out, 2e-3)
    out = no.gemm(a, b, out_dtype=torch.float32, bias=bias.float())
    assert_similar(z, out, 2e-3)
    nv.check_status(a.device)


@pytest.mark.parametrize("stride,pad,dil", [(1, 1, 1), (2, 1, 1), (1, 2, 2)])
@pytest.mark.parametrize("shape", [(4, 24, 80, 64, 128), (3, 12, 40, 128, 64), (16, 48, 160, 128, 256)])
def test_conv_fprop_and_dgrad(stride, pad, dil, shape):
    nv, no = _nops()
    n, h, w, c, o = shape
    torch.manual_seed(3)
    x = torch.randn(n, h, w, c, device=DEV).to(BF)
    wt = (torch.randn(o, 3, 3, c, device=DEV) / math.sqrt(9 * c)).to(BF)
    y = no.conv2d_fprop(x, wt, stride, pad, dil)
    expect = ref.conv2d_nhwc(x.float(), wt.float(), stride, pad, dil)
    assert y.shape == expect.shape
    assert _rel_err(y, expect) < 5e-3
    if o >= 128:   # the same convolution with the other tile height
        oh, ow = no.conv_out_hw(h, w, stride, pad, dil)
        taps = [(r * dil - pad, s * dil - pad) for r in range(3) for s in range(3)]
        for rows in (128, 256):
            y2 = torch.empty_like(y)
            no.conv_pass(x, wt.reshape(o, 9 * c), o, y2, grid_hw=(oh, ow), in_mul=stride, taps=taps, tile_rows=rows)
            assert _rel_err(y2, expect) < 5e-3, rows
    dy = torch.randn_like(expect).to(BF)
    dx = no.conv2d_dgrad(dy, wt, (h, w), stride, pad, dil)
    xf = x.float().requires_grad_(True)
    ref.conv2d_nhwc(xf, wt.float(), stride, pad, dil).backward(dy.float())
    assert _rel_err(dx, xf.grad) < 5e-3
    nv.check_status(x.device)


def test_linear_autograd_matches_reference():
    nv, no = _nops()
    torch.manual_seed(4)
    x = torch.randn(6, 50, 256, device=DEV).to(BF).requires_grad_(True)
    w = (torch.randn(512, 256, device=DEV) / 16).to(BF).requires_grad_(True)
    b = torch.randn(512, device=DEV).to(BF).requires_grad_(True)
    for act in ("none", "gelu"):
        y = no.linear(x, w, b, act)
        g = torch.randn_like(y)
        gx, gw, gb = torch.autograd.grad(y, (x, w, b), g)
        xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
        yf = ref.linear(xf, wf, bf, act)
        ex, ew, eb = torch.autograd.grad(yf, (xf, wf, bf), g.float())
        assert_similar(yf.to(BF), y, 3e-2)
        assert _rel_err(gx, ex) < 1e-2 and _rel_err(gw, ew) < 1e-2 and _rel_err(gb, eb) < 1e-2
    nv.check_status(x.device)


@pytest.mark.parametrize("dim", [64, 256, 1024, 2048])
def test_rmsnorm_fwd_bwd(dim):
    nv, no = _nops()
    torch.manual_seed(5)
    x = torch.randn(777, dim, device=DEV).to(BF).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(dim, device=DEV)).to(BF).requires_grad_(True)
    y = no.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    gx, gw = torch.autograd.grad(y, (x, w), g)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yf = ref.rms_norm(xf, wf, 1e-5)
    ex, ew = torch.autograd.grad(yf, (xf, wf), g.float())
    assert_similar(yf.to(BF), y, 2e-2)
    assert_similar(ex.to(BF), gx, 3e-2)
    assert _rel_err(gw, ew) < 1e-2


def test_layernorm_gelu_geglu_pools():
    nv, no = _nops()
    torch.manual_seed(6)
    x = torch.randn(100, 320, device=DEV).to(BF)
    w, b = torch.randn(320, device=DEV).to(BF), torch.randn(320, device=DEV).to(BF)
    assert_similar(ref.layer_norm(x.float(), w.float(), b.float(), 1e-5).to(BF), no.layer_norm(x, w, b, 1e-5), 3e-2)
    xg = torch.randn(64, 512, device=DEV).to(BF).requires_grad_(True)
    for fn, rf in ((no.gelu, ref.gelu), (no.geglu, ref.geglu)):
        y = fn(xg)
        g = torch.randn_like(y)
        (gx,) = torch.autograd.grad(y, xg, g)
        xf = xg.detach().float().requires_grad_(True)
        yf = rf(xf)
        (ex,) = torch.autograd.grad(yf, xf, g.float())
        assert_similar(yf.to(BF), y, 2e-2)
        assert_similar(ex.to(BF), gx, 3e-2)
    xp = torch.randn(3, 8, 12, 64, device=DEV).to(BF).requires_grad_(True)
    for fn, rf in ((no.avg_pool2x2_nhwc, ref.avg_pool2x2_nhwc),
                   (no.global_avg_pool_nhwc, lambda t: t.float().mean(dim=(1, 2)))):
        y = fn(xp)
        g = torch.randn_like(y)
        (gx,) = torch.autograd.grad(y, xp, g)
        xf = xp.detach().float().requires_grad_(True)
        yf = rf(xf)
        (ex,) = torch.autograd.grad(yf, xf, g.float())
        assert_similar(yf.to(BF), y, 2e-2)
        assert_similar(ex.to(BF), gx, 2e-2)


@pytest.mark.parametrize("rows,dim,with_bias", [(100, 320, True), (700, 1024, True), (33, 2048, False), (9, 5000, True)])
def test_layernorm_fwd_bwd(rows, dim, with_bias):
    nv, no = _nops()
    torch.manual_seed(8)
    x = torch.randn(rows, dim, device=DEV).to(BF).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(dim, device=DEV)).to(BF).requires_grad_(True)
    b = torch.randn(dim, device=DEV).to(BF).requires_grad_(True) if with_bias else None
    params = (x, w, b) if with_bias else (x, w)
    y = no.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    got = torch.autograd.grad(y, params, g)
    fl = [t.detach().float().requires_grad_(True) for t in params]
    yf = ref.layer_norm(fl[0], fl[1], fl[2] if with_bias else None, 1e-5)
    want = torch.autograd.grad(yf, fl, g.float())
    assert_similar(yf.to(BF), y, 3e-2)
    for name, a, e in zip(("dx", "dw", "db"), got, want):
        assert _rel_err(a, e) < 2e-2, (name, _rel_err(a, e))
    nv.check_status(x.device)


def test_cell_embed_fwd_bwd():
    nv, no = _nops()
    torch.manual_seed(7)
    n, p, e, vocab = 20, 96, 128, 50
    cells = torch.stack([torch.randint(0, vocab + 5, (n, p)), torch.randint(0, 1 << 24, (n, p)),
                         torch.randint(0, 1 << 24, (n, p))], -1).to(torch.int32).to(DEV)
    cp = torch.randn(vocab, e, device=DEV, requires_grad=True)
    pos = torch.randn(p, e, device=DEV, requires_grad=True)
    col = torch.randn(6, e, device=DEV, requires_grad=True)
    y = no.cell_embed(cells, cp, pos, col, BF)
    g = torch.randn_like(y)
    got = torch.autograd.grad(y, (cp, pos, col), g)
    yf = ref.cell_embed(cells, cp, pos, col, torch.float32)
    exp = torch.autograd.grad(yf, (cp, pos, col), g.float())
    assert_similar(yf.to(BF), y, 3e-2)
    for a, b_ in zip(got, exp):
        assert _rel_err(a, b_) < 1e-2


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("rows,h,vocab,vpad", [(1000, 256, 250, 256), (700, 128, 1000, 1000), (513, 512, 4096, 4096)])
def test_lm_head_ce_fwd_bwd(rows, h, vocab, vpad, fused):
    """The LM head with the cross-entropy in the GEMM epilogue (no logits in HBM) and with a chunk of fp32 logits."""
    nv, no = _nops()
    torch.manual_seed(8)
    x = torch.randn(rows, h, device=DEV).to(BF).requires_grad_(True)
    w = (torch.randn(vpad, h, device=DEV) / 16).to(BF).requires_grad_(True)
    t = torch.randint(0, vocab, (rows,), device=DEV)
    old = no.LM_HEAD_CHUNK_ROWS, no.FUSED_LM_HEAD_CE
    no.LM_HEAD_CHUNK_ROWS = 384          # exercise several chunks and a ragged tail
    no.FUSED_LM_HEAD_CE = fused
    try:
        loss = no.lm_head_ce(x, w, t, vocab, 1.0 / rows)
        gx, gw = torch.autograd.grad(loss, (x, w))
    finally:
        no.LM_HEAD_CHUNK_ROWS, no.FUSED_LM_HEAD_CE = old
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lf = ref.lm_head_ce(xf, wf, t, vocab, 1.0 / rows)
    ex, ew = torch.autograd.grad(lf, (xf, wf))
    assert abs(float(loss) - float(lf)) < 2e-2
    assert _rel_err(gx, ex) < 3e-2 and _rel_err(gw, ew) < 3e-2
    if vpad > vocab:
        assert float(gw[vocab:].abs().max()) == 0.0
    nv.check_status(x.device)


def test_fused_adamw_matches_reference_rule():
    nv, no = _nops()
    torch.manual_seed(9)
    n = 10_000 + 3
    for dtype in (torch.float32, BF):
        master = torch.randn(n, device=DEV)
        p = master.to(dtype)
        g = torch.randn(n, device=DEV).to(dtype)
        m, v = torch.rand(n, device=DEV) * 0.1, torch.rand(n, device=DEV) * 0.01
        em, ev, ew = m.clone(), v.clone(), master.clone()
        lr, b1, b2, eps, wd, step = 1e-2, 0.9, 0.99, 1e-8, 0.1, 3
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        no.adamw_flat(p, g, m, v, master if dtype == BF else None, 0, n, lr, b1, b2, eps, wd, bc1, bc2)
        gf = g.float()
        ew.mul_(1 - lr * wd)
        em.mul_(b1).add_(gf, alpha=1 - b1)
        ev.mul_(b2).addcmul_(gf, gf, value=1 - b2)
        ew.addcdiv_(em / bc1, (ev / bc2).sqrt() + eps, value=-lr)
        assert_similar(em, m, 1e-6)
        assert_similar(ev, v, 1e-6)
        assert_similar(ew, master if dtype == BF else p, 2e-6)
        if dtype == BF:
            assert torch.equal(p, master.to(BF))


def test_model_step_native_vs_reference_path():
    """One training step of the tiny model in bf16: native kernels against the PyTorch op definitions."""
    from fbamtrain_b200 import RunConfiguration, Trainer, ops, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    d = presets.tiny("bf16")
    d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64], "n_embed": 64})
    cfg = RunConfiguration.from_json(d)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=0, pin=False)
    cells, tg = src.next_batch(2, 16)
    losses = {}
    for backend in ("auto", "torch"):
        ops.set_backend(backend)
        try:
            tr = Trainer(cfg, device=torch.device(DEV))
            losses[backend] = [float(tr.train_step(cells, tg)) for _ in range(3)]
            tr.close()
        finally:
            ops.set_backend("auto")
    assert losses["auto"] == pytest.approx(losses["torch"], abs=5e-2)


@pytest.mark.parametrize("t_len,b,i_dim,h", [(5, 2, 64, 64), (33, 8, 128, 256), (16, 3, 256, 1024),
                                             (9, 4, 128, 2048), (7, 8, 64, 1536)])
def test_persistent_lstm_fwd_bwd(t_len, b, i_dim, h):
    nv, no = _nops()
    from fbamtrain_b200.ops import lstm as L
    torch.manual_seed(10)
    x = torch.randn(t_len, b, i_dim, device=DEV).to(BF).requires_grad_(True)
    k = 1.0 / math.sqrt(h)
    w_ih = ((torch.rand(4 * h, i_dim, device=DEV) * 2 - 1) * k).requires_grad_(True)
    w_hh = ((torch.rand(4 * h, h, device=DEV) * 2 - 1) * k).requires_grad_(True)
    b_ih = ((torch.rand(4 * h, device=DEV) * 2 - 1) * k).requires_grad_(True)
    b_hh = ((torch.rand(4 * h, device=DEV) * 2 - 1) * k).requires_grad_(True)
    h0 = (0.1 * torch.randn(h, device=DEV)).requires_grad_(True)
    c0 = (0.1 * torch.randn(h, device=DEV)).requires_grad_(True)
    params = (x, w_ih, w_hh, b_ih, b_hh, h0, c0)
    assert L.persistent_ok(b, h)
    y, hT, cT = L.lstm_sequence(*params, BF)
    nv.check_status(x.device)
    g = torch.randn_like(y)
    got = torch.autograd.grad((y.float() * g.float()).sum() + cT.sum(), params)
    nv.check_status(x.device)
    fp = [p.detach().float().requires_grad_(True) for p in params]
    yf, hf, cf = ref.lstm_sequence(*fp, torch.float32)
    exp = torch.autograd.grad((yf * g.float()).sum() + cf.sum(), fp)
    assert_similar(yf.to(BF), y, 3e-2)
    assert_similar(cf, cT, 3e-2)
    names = ["dx", "dw_ih", "dw_hh", "db_ih", "db_hh", "dh0", "dc0"]
    for name, a, e in zip(names, got, exp):
        assert _rel_err(a, e) < 4e-2, (name, _rel_err(a, e))


@pytest.mark.parametrize("stride,pad,dil", [(1, 1, 1), (2, 1, 1), (1, 2, 2)])
@pytest.mark.parametrize("shape", [(4, 24, 80, 64, 128), (3, 12, 40, 128, 64), (16, 48, 160, 128, 256),
                                   (5, 10, 14, 256, 512)])
def test_conv_wgrad(stride, pad, dil, shape):
    nv, no = _nops()
    from fbamtrain_b200.ops.conv_wgrad import conv2d_wgrad
    n, h, w, c, o = shape
    torch.manual_seed(11)
    x = torch.randn(n, h, w, c, device=DEV).to(BF)
    wt = torch.zeros(o, 3, 3, c, device=DEV, requires_grad=True)
    yf = ref.conv2d_nhwc(x.float(), wt, stride, pad, dil)
    dy = torch.randn_like(yf).to(BF)
    (expect,) = torch.autograd.grad(yf, wt, dy.float())
    got = conv2d_wgrad(x, dy, wt.shape, stride, pad, dil, out_dtype=torch.float32)
    nv.check_status(x.device)
    assert _rel_err(got, expect) < 5e-3


def test_conv_gelu_stack_pool_matches_unfused_reference():
    nv, no = _nops()
    torch.manual_seed(12)
    x = torch.randn(6, 24, 40, 64, device=DEV).to(BF).requires_grad_(True)
    w1 = (torch.randn(128, 3, 3, 64, device=DEV) / 24).to(BF).requires_grad_(True)
    w2 = (torch.randn(256, 3, 3, 128, device=DEV) / 34).to(BF).requires_grad_(True)
    v = no.conv_gelu_stack_pool(x, [w1, w2], 2, [1, 1], [1, 1])
    g = torch.randn_like(v)
    got = torch.autograd.grad(v, (x, w1, w2), g)
    fx, f1, f2 = (t.detach().float().requires_grad_(True) for t in (x, w1, w2))
    y = ref.gelu(ref.conv2d_nhwc(fx, f1, 2, 1, 1))
    y = ref.gelu(ref.conv2d_nhwc(y, f2, 2, 1, 1))
    vf = y.mean(dim=(1, 2))
    exp = torch.autograd.grad(vf, (fx, f1, f2), g.float())
    assert_similar(vf.to(BF), v, 2e-2)
    for name, a, e in zip(("dx", "dw1", "dw2"), got, exp):
        assert _rel_err(a, e) < 2e-2, (name, _rel_err(a, e))
    nv.check_status(x.device)


@pytest.mark.parametrize("two_tile", ["1", "0"])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("b,t,h,d", [(2, 128, 2, 64), (1, 300, 3, 64), (2, 256, 2, 128), (1, 1024, 4, 64),
                                     (1, 480, 2, 128), (1, 129, 1, 128)])
def test_flash_attention_fwd_bwd(causal, b, t, h, d, two_tile, monkeypatch):
    """Both forward kernels (two query tiles per CTA, the default, and one) with the shared backward."""
    monkeypatch.setenv("FBAMTRAIN_ATTENTION_FWD2", two_tile)
    nv, no = _nops()
    from fbamtrain_b200.ops.mha import flash_attention
    torch.manual_seed(14)
    qkv = torch.randn(b, t, 3, h, d, device=DEV).to(BF).requires_grad_(True)     # fused projection layout
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    o = flash_attention(q, k, v, causal)
    nv.check_status(qkv.device)
    g = torch.randn_like(o)
    (gqkv,) = torch.autograd.grad(o, qkv, g)
    nv.check_status(qkv.device)
    f = qkv.detach().float().requires_grad_(True)
    of = ref.attention(f[:, :, 0], f[:, :, 1], f[:, :, 2], causal)
    (eqkv,) = torch.autograd.grad(of, f, g.float())
    assert_similar(of.to(BF), o, 3e-2)
    for i, name in enumerate(("dq", "dk", "dv")):
        assert _rel_err(gqkv[:, :, i], eqkv[:, :, i]) < 3e-2, (name, _rel_err(gqkv[:, :, i], eqkv[:, :, i]))


@pytest.mark.parametrize("shape", [(256, 512), (1024, 256), (64, 64)])
def test_newton_schulz_on_tensor_cores_matches_reference(shape):
    nv, no = _nops()
    from fbamtrain_b200.optim.muon import newton_schulz as ns_ref
    torch.manual_seed(15)
    g = torch.randn(*shape, device=DEV)
    got = no.newton_schulz(g, 5).float()
    exp = ns_ref(g, 5, torch.float32)
    nv.check_status(g.device)
    assert _rel_err(got, exp) < 5e-2
    s = torch.linalg.svdvals(got)
    assert float(s.min()) > 0.4 and float(s.max()) < 1.4


def test_muon_training_step_native():
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    d = presets.tiny("bf16")
    d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64], "n_embed": 64})
    d["optimizer"]["type"] = "muon"
    d["optimizer"]["learning_rate"] = 2e-3
    cfg = RunConfiguration.from_json(d)
    tr = Trainer(cfg, device=torch.device(DEV))
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=1, pin=False)
    cells, tg = src.next_batch(2, 16)
    losses = [float(tr.train_step(cells, tg)) for _ in range(8)]
    tr.close()
    assert losses[-1] < losses[0], losses


@pytest.mark.parametrize("offload", [False, True])
def test_streaming_lstm_head_ce_matches_resident_reference(offload):
    """Chunked streaming (state carry, per-chunk head/CE hook, recompute in backward, optional host residence)
    against the fp32 PyTorch LSTM + head + CE on the whole sequence."""
    nv, no = _nops()
    from fbamtrain_b200.ops.streaming import streaming_lstm_head_ce
    torch.manual_seed(16)
    t_len, b, i_dim, h, vocab = 37, 4, 64, 128, 50
    vpad = 56
    k = 1.0 / math.sqrt(h)
    x = torch.randn(t_len, b, i_dim).to(BF)
    x_in = (x.pin_memory() if offload else x.to(DEV)).requires_grad_(not offload)
    ps = [((torch.rand(4 * h, i_dim, device=DEV) * 2 - 1) * k), ((torch.rand(4 * h, h, device=DEV) * 2 - 1) * k),
          ((torch.rand(4 * h, device=DEV) * 2 - 1) * k), ((torch.rand(4 * h, device=DEV) * 2 - 1) * k),
          0.1 * torch.randn(h, device=DEV), 0.1 * torch.randn(h, device=DEV)]
    ps = [p.requires_grad_(True) for p in ps]
    w_head = (torch.randn(vpad, h, device=DEV) * k).to(BF).requires_grad_(True)
    tg = torch.randint(0, vocab, (t_len, b), device=DEV)
    scale = 1.0 / (t_len * b)
    loss = streaming_lstm_head_ce(x_in, *ps, w_head, tg, vocab, scale, 8, offload)
    got = torch.autograd.grad(loss, ps + [w_head])
    nv.check_status(torch.device(DEV))
    fp = [p.detach().float().requires_grad_(True) for p in ps]
    wf = w_head.detach().float().requires_grad_(True)
    yf, _, _ = ref.lstm_sequence(x.to(DEV).float(), *fp, torch.float32)
    lf = ref.lm_head_ce(yf.reshape(t_len * b, h), wf, tg.reshape(-1), vocab, scale)
    exp = torch.autograd.grad(lf, fp + [wf])
    assert abs(float(loss) - float(lf)) < 2e-2
    for name, a, e in zip(["dw_ih", "dw_hh", "db_ih", "db_hh", "dh0", "dc0", "dw_head"], got, exp):
        assert _rel_err(a, e) < 5e-2, (name, _rel_err(a, e))


def test_reference_structure_model_streams_on_gpu():
    """The reference's own model shape (1-layer LSTM → head) trains through the streaming path and agrees with the
    PyTorch definitions."""
    from fbamtrain_b200 import RunConfiguration, Trainer, ops, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    d = presets.tiny("bf16")
    d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64], "n_embed": 64, "lstm_layers": 1,
                              "action_blocks": 0, "streaming_chunk_size": 5})
    cfg = RunConfiguration.from_json(d)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=2, pin=False)
    cells, tg = src.next_batch(2, 16)
    losses = {}
    for backend in ("auto", "torch"):
        ops.set_backend(backend)
        try:
            tr = Trainer(cfg, device=torch.device(DEV))
            assert tr.model.action_model.streaming
            losses[backend] = [float(tr.train_step(cells, tg)) for _ in range(3)]
            tr.close()
        finally:
            ops.set_backend("auto")
    assert losses["auto"] == pytest.approx(losses["torch"], abs=5e-2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("m,n,k", [(512, 256, 128), (1000, 520, 328), (4096, 4096, 1024), (304, 128, 64)])
def test_gemm_cta_pairs(a_mn, b_mn, m, n, k):
    """cta_group::2 kernel: two SMs per 256-row tile."""
    nv, no = _nops()
    torch.manual_seed(17)
    a = torch.randn(m, k, device=DEV).to(BF)
    b = torch.randn(n, k, device=DEV).to(BF)
    d = no.gemm(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, a_mn=a_mn, b_mn=b_mn,
                two_cta=True)
    nv.check_status(a.device)
    assert _rel_err(d, a.float() @ b.float().t()) < 5e-3
    if not a_mn and not b_mn:
        bias = torch.randn(n, device=DEV).to(BF)
        d = no.gemm(a, b, bias=bias, act="gelu", two_cta=True)
        assert_similar(torch.nn.functional.gelu(a.float() @ b.float().t() + bias.float()).to(BF), d, 0.25)
        nv.check_status(a.device)


@pytest.mark.parametrize("stride,pad,dil", [(2, 1, 1), (1, 2, 2)])
def test_conv_cta_pairs(stride, pad, dil):
    nv, no = _nops()
    torch.manual_seed(18)
    n, h, w, c, o = 9, 24, 80, 128, 256
    x = torch.randn(n, h, w, c, device=DEV).to(BF)
    wt = (torch.randn(o, 3, 3, c, device=DEV) / math.sqrt(9 * c)).to(BF)
    expect = ref.conv2d_nhwc(x.float(), wt.float(), stride, pad, dil)
    oh, ow = no.conv_out_hw(h, w, stride, pad, dil)
    taps = [(r * dil - pad, s * dil - pad) for r in range(3) for s in range(3)]
    y = torch.empty(n, oh, ow, o, device=DEV, dtype=BF)
    no.conv_pass(x, wt.reshape(o, 9 * c), o, y, grid_hw=(oh, ow), in_mul=stride, taps=taps, two_cta=True)
    nv.check_status(x.device)
    assert _rel_err(y, expect) < 5e-3


@pytest.mark.parametrize("with_gelu_grad", [False, True])
@pytest.mark.parametrize("shape", [(160, 24, 40, 256, 64), (300, 16, 32, 320, 128), (40, 23, 41, 256, 64)])
def test_strided_dgrad_with_fused_parity_classes(shape, with_gelu_grad, monkeypatch):
    """Stride-2 data gradient with all four parity classes in one launch of the CTA-pair kernel (every tile computed
    once per class by the same pair), against the one-launch-per-class form and against fp32 autograd.  The last
    shape has odd sides: its classes have different grids, which keeps the per-class form."""
    nv, no = _nops()
    n, h, w, c, o = shape
    torch.manual_seed(5)
    wt = (torch.randn(o, 3, 3, c, device=DEV) / math.sqrt(9 * c)).to(BF)
    oh, ow = no.conv_out_hw(h, w, 2, 1, 1)
    dy = torch.randn(n, oh, ow, o, device=DEV).to(BF)
    z = torch.randn(n, h, w, c, device=DEV).to(BF) if with_gelu_grad else None
    launches = []
    real = no.conv_pass
    monkeypatch.setattr(no, "conv_pass", lambda *a, **k: (launches.append(k.get("classes")), real(*a, **k))[1])
    fused = no.conv2d_dgrad(dy, wt, (h, w), 2, 1, 1, gelu_grad_in=z)
    fused_launches = list(launches)
    monkeypatch.setattr(no, "FUSE_DGRAD_CLASSES", False)
    separate = no.conv2d_dgrad(dy, wt, (h, w), 2, 1, 1, gelu_grad_in=z)
    nv.check_status(dy.device)
    if h % 2 == 0 and w % 2 == 0:
        assert len(fused_launches) == 1 and len(fused_launches[0]) == 4
    else:
        assert len(fused_launches) == 4 and all(cl is None for cl in fused_launches)
    assert torch.equal(fused, separate)
    xf = torch.zeros(n, h, w, c, device=DEV, requires_grad=True)
    ref.conv2d_nhwc(xf, wt.float(), 2, 1, 1).backward(dy.float())
    expect = xf.grad
    if with_gelu_grad:
        zf = z.float().requires_grad_(True)
        torch.nn.functional.gelu(zf).sum().backward()
        expect = expect * zf.grad
    assert _rel_err(fused, expect) < 6e-3


def test_device_fingerprint_detects_single_bit_changes():
    _nops()
    from fbamtrain_b200.parallel.ftccl import tensor_hashes
    torch.manual_seed(21)
    a = torch.randn(1_000_003, device=DEV)
    b = a.clone()
    c = a.clone()
    c.view(torch.int32)[777_777] ^= 1
    odd = torch.arange(13, device=DEV, dtype=torch.uint8)
    odd2 = odd.clone()
    odd2[12] = 99
    ha, hb, hc, ho, ho2 = tensor_hashes([a, b, c, odd, odd2])
    assert ha == hb and ha != hc and ho != ho2 and len(ha) == 32
    swapped = a.clone()
    swapped[[0, 1]] = swapped[[1, 0]]
    assert tensor_hashes([swapped])[0] != ha          # position matters


@pytest.mark.parametrize("dtype", ["fp16", "fp32"])
def test_fp16_models_train_on_the_native_kernels_and_fp32_on_the_library_path(dtype):
    """fp16 (the reference's default dtype, ``src/config.cpp:43-51``) runs on the half-precision build of the sm_100a
    kernels; fp32 configurations run on a GPU through the PyTorch definitions."""
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    from fbamtrain_b200.ops import dispatch
    d = presets.tiny(dtype)
    d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64], "n_embed": 64})
    cfg = RunConfiguration.from_json(d)
    src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, 256, 32, seed=3, pin=False)
    cells, tg = src.next_batch(2, cfg.train_sequence_length)
    tr = Trainer(cfg, device=torch.device(DEV))
    losses = [float(tr.train_step(cells, tg)) for _ in range(4)]
    tr.close()
    assert all(math.isfinite(x) for x in losses) and losses[-1] < losses[0]
    expected = "native" if dtype == "fp16" else "torch"
    assert dispatch.last_backend("gemm") == expected and dispatch.last_backend("conv2d") == expected


def test_frame_head_recompute_gives_the_same_gradients():
    """``frame_head_recompute`` keeps only the cells and runs the frame head again in the backward (the reference
    replays frames and recomputes: ``src/main.cpp:3354-3483``): same loss, same gradients, less memory kept."""
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    results = {}
    for recompute in (False, True):
        d = presets.tiny("bf16")
        d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64, 128], "downsample_blocks": 2,
                                  "n_embed": 64, "frame_rows": 16, "frame_cols": 24, "frame_head_recompute": recompute})
        d["frame_rows"], d["frame_cols"] = 16, 24
        cfg = RunConfiguration.from_json(d)
        tr = Trainer(cfg, device=torch.device(DEV), frame_chunk=8)
        src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, tr.vocab, seed=3,
                                   pin=False)
        cells, tg = src.next_batch(cfg.micro_batch_size, cfg.train_sequence_length)
        tr.zero_grad()
        loss = tr._forward_backward(cells, tg)
        results[recompute] = (float(loss), {n: p.grad.detach().float().clone()
                                            for n, p in tr.model.frame_head.named_parameters()})
        tr.close()
    assert results[True][0] == pytest.approx(results[False][0], abs=1e-3)
    for name, g in results[False][1].items():
        assert _rel_err(results[True][1][name], g) < 2e-2, name


def test_frame_replay_matches_resident_frames_on_gpu():
    """``frame_replay``: the frames stay in pinned host memory, chunks are copied in for the forward and again for the
    backward on the copy stream (the reference re-decodes and recomputes: ``src/main.cpp:3354-3483``): same loss and
    gradients as with the whole micro-batch resident, twice the chunk uploads."""
    from fbamtrain_b200 import RunConfiguration, Trainer, presets
    from fbamtrain_b200.data import SyntheticBatchSource
    results = {}
    for replay in (False, True):
        d = presets.tiny("bf16")
        d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64, 128], "downsample_blocks": 2,
                                  "n_embed": 64, "frame_rows": 16, "frame_cols": 24, "frame_replay": replay})
        d["frame_rows"], d["frame_cols"] = 16, 24
        cfg = RunConfiguration.from_json(d)
        tr = Trainer(cfg, device=torch.device(DEV), frame_chunk=8)
        src = SyntheticBatchSource(cfg.frame_rows, cfg.frame_cols, cfg.model_config.max_code_point, tr.vocab, seed=3,
                                   pin=True)
        cells, tg = src.next_batch(cfg.micro_batch_size, cfg.train_sequence_length)
        tr.zero_grad()
        loss = tr._forward_backward(cells, tg)
        torch.cuda.synchronize()
        results[replay] = (float(loss), {n: p.grad.detach().float().clone()
                                         for n, p in tr.model.frame_head.named_parameters()})
        if replay:
            chunks = (cells.shape[0] * cells.shape[1] + 7) // 8
            # every chunk is copied in twice, except the last two, which are still in the two buffers when the
            # backward starts
            assert tr.last_replay.uploads == 2 * chunks - 2
        tr.close()
    assert results[True][0] == pytest.approx(results[False][0], abs=1e-3)
    for name, g in results[False][1].items():
        assert _rel_err(results[True][1][name], g) < 2e-2, name


def test_expected_backends_are_chosen_on_gpu():
    """16-bit CUDA tensors must reach the sm_100a kernels (no silent library fallback), fp32 the library."""
    _nops()
    from fbamtrain_b200 import ops
    from fbamtrain_b200.ops import dispatch
    x = torch.randn(256, 512, device=DEV).to(BF)
    w = torch.randn(256, 512, device=DEV).to(BF)
    ops.linear(x, w)
    assert dispatch.last_backend("gemm") == "native"
    q, k, v = (torch.randn(2, 128, 2, 64, device=DEV).to(BF) for _ in range(3))
    ops.attention(q, k, v, True)
    assert dispatch.last_backend("mha") == "native"
    img = torch.randn(3, 12, 40, 128, device=DEV).to(BF)
    wt = torch.randn(64, 3, 3, 128, device=DEV).to(BF)
    ops.conv2d_nhwc(img, wt, 1, 1, 1)
    assert dispatch.last_backend("conv2d") == "native"
    ops.linear(x.float(), w.float())
    assert dispatch.last_backend("gemm") == "torch"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("momentum,nesterov", [(0.0, False), (0.9, False), (0.9, True)])
def test_fused_sgd_step_matches_torch_path(dtype, momentum, nesterov):
    _nops()
    from fbamtrain_b200 import ops
    from fbamtrain_b200.optim import SgdOptimizer
    torch.manual_seed(22)
    results = {}
    for backend in ("auto", "torch"):
        p = torch.nn.Parameter(torch.linspace(-1, 1, 1000, device=DEV).to(dtype))
        opt = SgdOptimizer([("w", p)], "optim/t", lr=0.1, momentum=momentum, nesterov=nesterov, weight_decay=0.01)
        ops.set_backend(backend)
        try:
            for k in range(3):
                p.grad = torch.sin(torch.arange(1000, device=DEV) * 0.01 * (k + 1)).to(dtype)
                opt.step()
        finally:
            ops.set_backend("auto")
        results[backend] = (p.detach().float().clone(), {n: t.clone() for n, t in opt.state["w"].items()})
    assert torch.allclose(results["auto"][0], results["torch"][0], atol=1e-6 if dtype == torch.float32 else 1e-2)
    for n, t in results["torch"][1].items():
        assert torch.allclose(results["auto"][1][n], t, atol=1e-5), n


def test_linear_relu_fwd_bwd():
    """``relu(x·Wᵀ + b)``: the epilogue applies the activation, the backward masks by the output's sign."""
    _nops()
    from fbamtrain_b200 import ops
    from fbamtrain_b200.ops import reference as ref
    torch.manual_seed(31)
    x = torch.randn(256, 512, device=DEV).to(BF).requires_grad_(True)
    w = (torch.randn(256, 512, device=DEV) * 0.05).to(BF).requires_grad_(True)
    b = torch.randn(256, device=DEV).to(BF).requires_grad_(True)
    y = ops.linear(x, w, b, "relu")
    g = torch.randn_like(y)
    dx, dw, db = torch.autograd.grad(y, (x, w, b), g)
    xf, wf, bf_ = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yf = ref.linear(xf, wf, bf_, "relu")
    ex, ew, eb = torch.autograd.grad(yf, (xf, wf, bf_), g.float())
    assert_similar(yf.to(BF), y, 3e-2)
    # elements whose pre-activation rounds across zero in bf16 may be masked differently: compare in norm
    for got, exp in ((dx, ex), (dw, ew), (db, eb)):
        assert float((got.float() - exp).norm() / exp.norm()) < 3e-2
