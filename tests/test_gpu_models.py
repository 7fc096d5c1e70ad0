"""Model-level GPU checks: converted torchvision ResNets run a training step (signed path, STE and LRE) and
an inference pass (unsigned path) through the kernels of this package, and the converted network's first
approximate layer agrees with the oracle chain on the activations it actually received."""

import numpy as np
import pytest
import torch

from oracle import lut_oracle as lo

pytestmark = pytest.mark.gpu


def _cifar_resnet18():
    import torchvision
    m = torchvision.models.resnet18(num_classes=10)
    m.conv1 = torch.nn.Conv2d(3, 64, 3, 1, 1, bias=False)
    m.maxpool = torch.nn.Identity()
    return m


@pytest.mark.parametrize("grad,bits", [("ste", 8), ("lre", 4)])
def test_resnet18_qat_step(dev, grad, bits):
    import approxtorch_b200 as at
    torch.manual_seed(0)
    lutn = lo.lut_signed_truncated(4)
    dx, dw = lo.lre_slopes(lutn)
    lut = torch.from_numpy(lutn.reshape(-1)).to(dev)
    model = _cifar_resnet18()
    at.convert_model(model, lut, qtype="int8", grad=grad, dx=torch.from_numpy(dx).to(dev), dw=torch.from_numpy(dw).to(dev),
                     weight_bits=bits, scale_momentum=0.1)
    convs = [m for m in model.modules() if isinstance(m, at.nn.Conv2d_int8)]
    assert len(convs) == 19 and isinstance(model.conv1, torch.nn.Conv2d)
    model = model.to(dev).train()
    x = torch.randn(16, 3, 32, 32, device=dev)
    y = torch.randint(0, 10, (16,), device=dev)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    for _ in range(3):
        opt.zero_grad(set_to_none=True)
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert all(np.isfinite(losses))
    assert all(c.weight.grad is not None and torch.isfinite(c.weight.grad).all() for c in convs)
    assert all(c.scale_x.item() != 1.0 for c in convs)           # EMA statistics moved off their initial value
    # the first approximate layer against the oracle chain on its real input
    layer = convs[0]
    feats = {}
    h = layer.register_forward_hook(lambda m, i, o: feats.update(x=i[0].detach(), y=o.detach()))
    model.eval()
    with torch.no_grad():
        model(x)
    h.remove()
    xin = feats["x"].cpu().numpy()
    sw = layer.scale_w.cpu().numpy()
    qm = 2 ** (bits - 1) - 1
    xq, _ = lo.fakequant_sym(xin, np.float32(layer.scale_x.item()), -127, 127)
    wq, _ = lo.fakequant_sym(layer.weight.detach().cpu().numpy(), sw.reshape(-1, 1, 1, 1), -qm, qm)
    cols = lo.im2col_index(lo.to_lut_index(xq, 128), 3, 3, 1, 1, 1, 1)
    yint = lo.bgemm_exact(cols, lo.to_lut_index(wq.reshape(64, -1), 128), lutn)
    ref = lo.dequant(yint.reshape(16, 64, 32, 32), layer.scale_x.item(), sw)
    np.testing.assert_allclose(feats["y"].cpu().numpy(), ref, rtol=1e-5, atol=1e-5 * np.abs(ref).max())


def test_resnet50_uint8_inference(dev):
    import torchvision
    import approxtorch_b200 as at
    torch.manual_seed(0)
    lut = torch.from_numpy(lo.lut_unsigned_truncated(6).reshape(-1)).to(dev)
    model = torchvision.models.resnet50()
    at.convert_model(model, lut, qtype="uint8", scale_momentum=1.0)
    layers = [m for m in model.modules() if isinstance(m, at.nn.Conv2d_uint8)]
    assert len(layers) == 52
    model = model.to(dev).train()
    x = torch.randn(4, 3, 64, 64, device=dev)
    with torch.no_grad():
        model(x)                                                   # calibration pass (momentum 1)
    model.eval()
    with torch.no_grad():
        a = model(x)
        b = model(x)
    assert a.shape == (4, 1000) and torch.isfinite(a).all() and torch.equal(a, b)
    assert all(torch.equal(m.zero_x, torch.round(m.zero_x)) for m in layers)
