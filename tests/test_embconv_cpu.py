"""The table decomposition of "cell embedding → first convolution → GELU" (``ops/embconv.py``) against autograd through
the plain definitions (``ops/reference.py``): forward values and the gradients of the code-point table, the position
table, the colour vectors and the filter, over strides, dilations, paddings and code points outside the table."""
import pytest
import torch

from fbamtrain_b200.ops import embconv, reference as ref


def _random_cells(n, rows, cols, vocab, seed, coherent):
    g = torch.Generator().manual_seed(seed)
    p = rows * cols
    cells = torch.zeros(n, p, 3, dtype=torch.int32)
    frame = torch.stack([torch.randint(0, vocab + 3, (p,), generator=g),              # some code points past the table
                         torch.randint(0, 1 << 24, (p,), generator=g),
                         torch.randint(0, 1 << 24, (p,), generator=g)], -1).int()
    for i in range(n):
        if coherent and i > 0:
            change = torch.rand(p, generator=g) < 0.1
            fresh = torch.stack([torch.randint(0, vocab + 3, (p,), generator=g),
                                 torch.randint(0, 1 << 24, (p,), generator=g),
                                 torch.randint(0, 1 << 24, (p,), generator=g)], -1).int()
            frame = torch.where(change.unsqueeze(-1), fresh, frame)
        elif i > 0:
            frame = torch.stack([torch.randint(-1, vocab + 3, (p,), generator=g),
                                 torch.randint(0, 1 << 24, (p,), generator=g),
                                 torch.randint(0, 1 << 24, (p,), generator=g)], -1).int()
        cells[i] = frame
    return cells


@pytest.mark.parametrize("rows,cols,stride,pad,dil", [(6, 8, 2, 1, 1), (5, 7, 2, 1, 1), (6, 8, 1, 1, 1), (8, 9, 2, 2, 2),
                                                     (7, 6, 1, 2, 2), (6, 6, 2, 0, 1)])
@pytest.mark.parametrize("coherent", [True, False])
def test_decomposition_matches_autograd(rows, cols, stride, pad, dil, coherent):
    torch.manual_seed(3)
    n, vocab, c, o = 5, 11, 8, 16
    cells = _random_cells(n, rows, cols, vocab, 5, coherent)
    cp = torch.randn(vocab, c, requires_grad=True)
    pos = torch.randn(rows * cols, c, requires_grad=True)
    col = torch.randn(6, c, requires_grad=True)
    w = (torch.randn(o, 3, 3, c) / 8).requires_grad_(True)

    e = ref.cell_embed(cells, cp, pos, col, torch.float32).view(n, rows, cols, c)
    y_ref = ref.gelu(ref.conv2d_nhwc(e, w, stride, pad, dil))
    g = torch.randn_like(y_ref)
    grads_ref = torch.autograd.grad(y_ref, [cp, pos, col, w], g)

    y = embconv.cell_conv_gelu(cells, cp, pos, col, w, rows, cols, stride, pad, dil)
    grads = torch.autograd.grad(y, [cp, pos, col, w], g)
    assert y.shape == y_ref.shape
    assert torch.allclose(y, y_ref, atol=2e-4, rtol=1e-4)
    for got, want, name in zip(grads, grads_ref, ("cp_embed", "pos_embed", "colour", "weight")):
        assert got.shape == want.shape, name
        assert torch.allclose(got, want, atol=5e-4, rtol=1e-3), (name, float((got - want).abs().max()))


def test_tap_cells_geometry():
    taps = embconv.tap_cells(4, 6, 2, 1, 1, "cpu")
    oh, ow = embconv.out_hw(4, 6, 2, 1, 1)
    assert taps.shape == (oh * ow, 9)
    # pixel (0, 0): the first row and column of taps fall into the padding; the centre tap reads cell (0, 0)
    assert taps[0].tolist() == [-1, -1, -1, -1, 0, 1, -1, 6, 7]
    # last pixel (1, 2): centre tap reads cell (2, 4)
    assert taps[-1, 4].item() == 2 * 6 + 4


def test_features_layout():
    cells = torch.zeros(1, 4, 3, dtype=torch.int32)
    cells[0, :, 1] = torch.tensor([0xFF0000, 0x00FF00, 0x0000FF, 0x000000])
    cells[0, :, 2] = torch.tensor([0x000000, 0xFF0000, 0x00FF00, 0x0000FF])
    taps = embconv.tap_cells(2, 2, 2, 1, 1, "cpu")        # one output pixel; taps 4, 5, 7, 8 read cells 0..3
    f = embconv.features_torch(cells, taps, torch.float32)[0, 0]
    assert f[4 * 6:4 * 6 + 6].tolist() == [1, 0, 0, 0, 0, 0]
    assert f[5 * 6:5 * 6 + 6].tolist() == [0, 1, 0, 1, 0, 0]
    assert f[7 * 6:7 * 6 + 6].tolist() == [0, 0, 1, 0, 1, 0]
    assert f[8 * 6:8 * 6 + 6].tolist() == [0, 0, 0, 0, 0, 1]
    assert float(f[:24].abs().sum()) == 0 and float(f[54:].abs().sum()) == 0
