"""The kernels of ``csrc/embconv.cu`` (cell embedding fused with the first convolution) on a GPU: each kernel against
its plain-PyTorch form, and the fused frame-head stack against fp32 autograd through the separate definitions."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
BF = torch.bfloat16


def _cells(n, rows, cols, vocab, seed, change=0.1):
    g = torch.Generator().manual_seed(seed)
    p = rows * cols

    def fresh():
        return torch.stack([torch.randint(-1, vocab + 2, (p,), generator=g),          # a few outside the table
                            torch.randint(0, 1 << 24, (p,), generator=g),
                            torch.randint(0, 1 << 24, (p,), generator=g)], -1).int()
    out = torch.zeros(n, p, 3, dtype=torch.int32)
    frame = fresh()
    for i in range(n):
        if i > 0:
            frame = torch.where((torch.rand(p, generator=g) < change).unsqueeze(-1), fresh(), frame)
        out[i] = frame
    return out.to(DEV)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


GEOMS = [(8, 16, 2, 1, 1), (9, 15, 2, 1, 1), (8, 12, 1, 1, 1), (12, 10, 2, 2, 2)]


@pytest.mark.parametrize("rows,cols,stride,pad,dil", GEOMS)
def test_colour_features_kernel(rows, cols, stride, pad, dil):
    from fbamtrain_b200.ops import embconv
    cells = _cells(37, rows, cols, 50, 1)
    taps = embconv.tap_cells(rows, cols, stride, pad, dil, DEV)
    got = embconv.features_native(cells, rows, cols, stride, pad, dil, BF)
    want = embconv.features_torch(cells, taps, BF)
    assert torch.equal(got, want)


@pytest.mark.parametrize("change", [0.05, 1.0])
@pytest.mark.parametrize("o", [64, 256, 320])
@pytest.mark.parametrize("rows,cols,stride,pad,dil", GEOMS)
def test_forward_gather_kernel(rows, cols, stride, pad, dil, o, change):
    from fbamtrain_b200.ops import embconv, native as nv
    torch.manual_seed(2)
    vocab, n = 50, 150                               # more frames than one segment, not a multiple of the prefetch depth
    cells = _cells(n, rows, cols, vocab, 3, change)
    taps = embconv.tap_cells(rows, cols, stride, pad, dil, DEV)
    table = torch.randn(vocab, 9, o, device=DEV).to(BF)
    oh, ow = embconv.out_hw(rows, cols, stride, pad, dil)
    pos = torch.randn(oh * ow, o, device=DEV)
    z0 = torch.randn(n, oh * ow, o, device=DEV).to(BF)
    z, y = z0.clone(), torch.empty_like(z0)
    embconv.forward_native(cells, table, pos, z, y, rows, cols, stride, pad, dil)
    nv.check_status(cells.device)
    want = embconv.gather_torch(cells, taps, table) + pos.unsqueeze(0) + z0.float()
    assert _rel(z, want) < 4e-3, _rel(z, want)
    assert float((z.float() - want).abs().max()) < 0.08          # bf16 rounding of values of size ~5, plus drift bound
    assert _rel(y, torch.nn.functional.gelu(want)) < 4e-3


@pytest.mark.parametrize("change", [0.05, 1.0])
@pytest.mark.parametrize("o", [64, 256, 320])
@pytest.mark.parametrize("rows,cols,stride,pad,dil", GEOMS)
def test_backward_reduce_kernel(rows, cols, stride, pad, dil, o, change):
    from fbamtrain_b200.ops import embconv, native as nv
    torch.manual_seed(4)
    vocab, n = 50, 150
    cells = _cells(n, rows, cols, vocab, 5, change)
    taps = embconv.tap_cells(rows, cols, stride, pad, dil, DEV)
    oh, ow = embconv.out_hw(rows, cols, stride, pad, dil)
    dz = torch.randn(n, oh * ow, o, device=DEV).to(BF)
    s = torch.zeros(vocab, 9, o, device=DEV)
    d = torch.zeros(oh * ow, o, device=DEV)
    embconv.reduce_native(cells, dz, s, d, rows, cols, stride, pad, dil)
    nv.check_status(cells.device)
    s_want, d_want = embconv.reduce_torch(cells, taps, dz, vocab)
    assert _rel(s, s_want) < 1e-5, _rel(s, s_want)
    assert _rel(d, d_want) < 1e-5, _rel(d, d_want)


def test_one_tap_weight_gradient_is_a_plain_product():
    """The colour-weighted sums are taken as a 1x1 weight gradient: ``dYᵀ · X`` over all pixels."""
    from fbamtrain_b200.ops.conv_wgrad import wgrad_pass
    torch.manual_seed(6)
    x = torch.randn(40, 6, 10, 64, device=DEV).to(BF)
    dy = torch.randn(40, 6, 10, 128, device=DEV).to(BF)
    got = wgrad_pass(x, dy, 128, 64, [(0, 0)], 1, out_dtype=torch.float32)
    want = dy.float().reshape(-1, 128).t() @ x.float().reshape(-1, 64)
    assert _rel(got, want) < 1e-3


@pytest.mark.parametrize("stride,pad,dil", [(2, 1, 1), (1, 1, 1)])
def test_cell_conv_gelu_matches_separate_ops(stride, pad, dil):
    from fbamtrain_b200.ops import embconv, native as nv, reference as ref
    torch.manual_seed(7)
    rows, cols, vocab, c, o, n = 12, 20, 96, 64, 128, 70
    cells = _cells(n, rows, cols, vocab, 8)
    cp = torch.randn(vocab, c, device=DEV, requires_grad=True)
    pos = torch.randn(rows * cols, c, device=DEV, requires_grad=True)
    col = torch.randn(6, c, device=DEV, requires_grad=True)
    w = (torch.randn(o, 3, 3, c, device=DEV) / 24).to(BF).requires_grad_(True)
    y = embconv.cell_conv_gelu(cells, cp, pos, col, w, rows, cols, stride, pad, dil)
    g = torch.randn_like(y)
    got = torch.autograd.grad(y, (cp, pos, col, w), g)
    nv.check_status(cells.device)
    wf = w.detach().float().requires_grad_(True)
    e = ref.cell_embed(cells, cp, pos, col, torch.float32).view(n, rows, cols, c)
    yf = ref.gelu(ref.conv2d_nhwc(e, wf, stride, pad, dil))
    want = torch.autograd.grad(yf, (cp, pos, col, wf), g.float())
    assert _rel(y, yf) < 1e-2, _rel(y, yf)
    for name, a, b in zip(("cp_embed", "pos_embed", "colour", "weight"), got, want):
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))


def test_fused_cells_stack_matches_unfused_reference():
    """cells → embedding → two stride-2 convolutions with GELU → mean, against fp32 autograd through the separate
    definitions: the frame vector and every parameter gradient."""
    from fbamtrain_b200.ops import native as nv, native_ops as no, reference as ref
    torch.manual_seed(9)
    rows, cols, vocab, c, n = 24, 40, 128, 64, 80
    cells = _cells(n, rows, cols, vocab, 10)
    cp = torch.randn(vocab, c, device=DEV, requires_grad=True)
    pos = torch.randn(rows * cols, c, device=DEV, requires_grad=True)
    col = torch.randn(6, c, device=DEV, requires_grad=True)
    w1 = (torch.randn(128, 3, 3, 64, device=DEV) / 24).to(BF).requires_grad_(True)
    w2 = (torch.randn(256, 3, 3, 128, device=DEV) / 34).to(BF).requires_grad_(True)
    v = no.cell_conv_gelu_stack_pool(cells, cp, pos, col, rows, cols, [w1, w2], 2, [1, 1], [1, 1])
    g = torch.randn_like(v)
    got = torch.autograd.grad(v, (cp, pos, col, w1, w2), g)
    nv.check_status(cells.device)
    f1, f2 = (t.detach().float().requires_grad_(True) for t in (w1, w2))
    e = ref.cell_embed(cells, cp, pos, col, torch.float32).view(n, rows, cols, c)
    y = ref.gelu(ref.conv2d_nhwc(e, f1, 2, 1, 1))
    y = ref.gelu(ref.conv2d_nhwc(y, f2, 2, 1, 1))
    vf = y.mean(dim=(1, 2))
    want = torch.autograd.grad(vf, (cp, pos, col, f1, f2), g.float())
    assert _rel(v, vf) < 1e-2, _rel(v, vf)
    for name, a, b in zip(("cp_embed", "pos_embed", "colour", "w1", "w2"), got, want):
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))


def test_frame_head_uses_the_fused_first_layer_and_matches_the_separate_kernels(monkeypatch):
    """The model-level switch: the same frame head with and without ``FBAMTRAIN_EMBCONV`` gives the same frame vectors
    and parameter gradients (bf16 tolerances), and the fused path launches no embedding kernel."""
    from fbamtrain_b200 import RunConfiguration, presets
    from fbamtrain_b200.models.fbam import FbamModel
    d = presets.tiny("bf16")
    d["model_config"].update({"cell_embed_dim": 64, "downsample_channels": [64, 128], "downsample_blocks": 2,
                              "n_embed": 64, "frame_rows": 16, "frame_cols": 24, "max_code_point": 64})
    d["frame_rows"], d["frame_cols"] = 16, 24
    cfg = RunConfiguration.from_json(d)
    torch.manual_seed(11)
    model = FbamModel(cfg.model_config, 32).to(DEV)
    cells = _cells(40, 16, 24, 64, 12)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("FBAMTRAIN_EMBCONV", flag)
        for p in model.parameters():
            p.grad = None
        v = model.frame_head(cells)
        v.float().square().sum().backward()
        outs.append((v.detach().float(), {n: p.grad.detach().float().clone() for n, p in model.frame_head.named_parameters()}))
    assert _rel(outs[0][0], outs[1][0]) < 2e-2
    for name in outs[0][1]:
        assert _rel(outs[0][1][name], outs[1][1][name]) < 3e-2, (name, _rel(outs[0][1][name], outs[1][1][name]))
