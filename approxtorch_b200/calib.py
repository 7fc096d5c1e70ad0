"""Offline min-max calibration (same entry points and checkpoint keys as approxtorch/calib.py:7-335).

``calibrate_int8`` / ``calibrate_uint8`` run a *floating-point* model over calibration batches with forward
hooks on its ``nn.Conv2d`` layers and return the model's ``state_dict`` augmented with the quantisation state
the approximate layers load directly:

* int8:  ``{layer}.scale_x`` (scalar, absmax / 127) and ``{layer}.scale_w`` ([O], absmax / (2^(bits-1) - 1));
* uint8: ``{layer}.x_min / x_max / w_min / w_max`` (ranges forced to contain 0) and the qparams derived from
  them, ``scale_x / zero_x / scale_w / zero_w`` (zero points integer-valued, stored as float32).

The per-batch activation statistics of CUDA fp32 activations come from this package's single-pass
abs-max / min / max kernel (one read of the activation instead of ``abs().max()`` or ``amin()`` + ``amax()``);
the running extrema stay on the device, so the hooks never synchronise.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .nn.Conv2d_uint8 import uint8_qparams


def _select_convs(model, skip_first):
    picked, seen_first = {}, False
    for name, module in model.named_modules():
        if isinstance(module, nn.Conv2d):
            if skip_first and not seen_first:
                seen_first = True
                continue
            seen_first = True
            picked[name] = module
    return picked


def _model_device(model):
    p = next(model.parameters(), None)
    if p is not None:
        return p.device
    b = next(model.buffers(), None)
    return b.device if b is not None else torch.device("cpu")


def _batch_stats(x):
    """(absmax, min, max) of one activation tensor as fp32 device scalars."""
    x = x.detach()
    if x.is_cuda and x.dtype == torch.float32:
        from .backend import ops
        st = ops.absmax(x, want_minmax=True)
        return st[0], st[1], st[2]
    return x.abs().max().float(), x.amin().float(), x.amax().float()


def _observe(model, layers, data_loader, num_pictures, device, trim_last_batch):
    """Run the loader through the model; returns {layer: [absmax, min, max]} and the number of samples used.
    Train / eval flags of every module are restored afterwards."""
    record = {}
    hooks = []

    def make_hook(name):
        def hook(module, inputs, output):
            if not inputs or not isinstance(inputs[0], torch.Tensor):
                raise TypeError(f"input of Conv2d '{name}' must be a torch.Tensor")
            am, mn, mx = _batch_stats(inputs[0])
            if name in record:
                r = record[name]
                r[0], r[1], r[2] = torch.maximum(r[0], am), torch.minimum(r[1], mn), torch.maximum(r[2], mx)
            else:
                record[name] = [am, mn, mx]
        return hook

    for name, module in layers.items():
        hooks.append(module.register_forward_hook(make_hook(name)))
    flags = {m: m.training for m in model.modules()}
    seen = 0
    model.eval()
    try:
        with torch.no_grad():
            for batch in data_loader:
                images = batch[0] if isinstance(batch, (list, tuple)) else batch
                if not isinstance(images, torch.Tensor):
                    raise TypeError("calibration batch must be a Tensor or a list/tuple whose first element is a Tensor")
                if images.dim() == 0:
                    raise ValueError("calibration input must have a batch dimension")
                yield_all = num_pictures is None
                if not yield_all:
                    left = num_pictures - seen
                    if left <= 0:
                        break
                    if trim_last_batch:
                        images = images[:left]
                if images.shape[0] == 0:
                    continue
                model(images.to(device))
                seen += images.shape[0]
                if not yield_all and seen >= num_pictures:
                    break
    finally:
        for h in hooks:
            h.remove()
        for m, flag in flags.items():
            m.training = flag
    return record, seen


def _insert_after_layer(state, extra_by_layer):
    """Copy of ``state`` with each layer's extra entries placed right after that layer's last own entry."""
    last = {}
    for k in state:
        layer = k.rsplit(".", 1)[0]
        if layer in extra_by_layer:
            last[layer] = k
    out = {}
    for k, v in state.items():
        out[k] = v
        layer = k.rsplit(".", 1)[0]
        if last.get(layer) == k:
            for field, value in extra_by_layer[layer].items():
                out[f"{layer}.{field}"] = value
    return out


def calibrate_int8(model, data_loader, num_pictures, save_path, weight_bits=8):
    """Absmax calibration for the signed layers; the first ``nn.Conv2d`` is skipped.  Returns (and saves to
    ``save_path``) the state_dict with ``scale_x`` / ``scale_w`` inserted after each calibrated layer's
    parameters."""
    if not 3 <= weight_bits <= 8:
        raise ValueError(f"weight_bits must be between 3 and 8, got {weight_bits}")
    model.eval()
    device = next(model.parameters()).device
    layers = _select_convs(model, skip_first=True)
    record, _ = _observe(model, layers, data_loader, num_pictures, device, trim_last_batch=False)   # whole batches
    model.eval()
    qmax_w = 2 ** (weight_bits - 1) - 1
    extra = {}
    for name, module in layers.items():
        absmax = float(record[name][0].item()) if name in record else 0.0
        scale_x = torch.tensor(absmax / 127.0 if absmax > 0 else 1.0)
        w = module.weight.detach()
        scale_w = w.abs().amax(dim=tuple(range(1, w.dim()))) / qmax_w
        scale_w = torch.where(scale_w > 0, scale_w, torch.ones_like(scale_w))
        extra[name] = {"scale_x": scale_x, "scale_w": scale_w}
    new_state = _insert_after_layer(model.state_dict(), extra)
    torch.save(new_state, save_path)
    return new_state


def calibrate_uint8(model, data_loader, num_pictures, save_path=None, ignore_first_conv=True):
    """Min/max calibration for the unsigned layers.  ``num_pictures=None`` uses the whole loader; otherwise the
    last batch is trimmed so exactly that many samples are seen.  Returns the augmented state_dict (saved when
    ``save_path`` is given)."""
    if num_pictures is not None:
        if isinstance(num_pictures, bool) or not isinstance(num_pictures, int):
            raise TypeError("num_pictures must be a positive int or None")
        if num_pictures <= 0:
            raise ValueError("num_pictures must be positive")
    device = _model_device(model)
    layers = _select_convs(model, skip_first=ignore_first_conv)
    if not layers:
        raise ValueError("no Conv2d layers selected for uint8 calibration; if the model contains only one Conv2d, "
                         "pass ignore_first_conv=False")
    record, seen = _observe(model, layers, data_loader, num_pictures, device, trim_last_batch=True)
    if seen == 0:
        raise ValueError("data_loader yielded no calibration samples")
    new_state = model.state_dict()
    for name, module in layers.items():
        if name not in record:
            raise RuntimeError(f"Conv2d '{name}' did not run during calibration")
        _, mn, mx = record[name]
        if not (torch.isfinite(mn) and torch.isfinite(mx)):
            raise ValueError(f"non-finite activation observed at Conv2d '{name}'")
        wdev = module.weight.device
        x_min = torch.minimum(mn, torch.zeros_like(mn)).to(wdev)
        x_max = torch.maximum(mx, torch.zeros_like(mx)).to(wdev)
        w = module.weight.detach()
        if not torch.isfinite(w).all():
            raise ValueError(f"non-finite weight observed at Conv2d '{name}'")
        dims = tuple(range(1, w.dim()))
        w_min = torch.clamp(w.amin(dim=dims).float(), max=0.0)
        w_max = torch.clamp(w.amax(dim=dims).float(), min=0.0)
        scale_x, zero_x = uint8_qparams(x_min, x_max)
        scale_w, zero_w = uint8_qparams(w_min, w_max)
        fields = {"x_min": x_min, "x_max": x_max, "w_min": w_min, "w_max": w_max,
                  "scale_x": scale_x, "zero_x": zero_x.float(), "scale_w": scale_w, "zero_w": zero_w.float()}
        for field, value in fields.items():
            new_state[f"{name}.{field}" if name else field] = value.detach().clone()
    if save_path is not None:
        torch.save(new_state, save_path)
    return new_state
