"""Per-kernel timings of the hot path with their roofline fractions (CUDA events, device-resident operands).

    python -m approxtorch_b200.kernel_bench [--only stream,backward,custom,layers,lds,model] [--batch 16]

``bench.py`` calls :func:`run_all` and reports the result under ``extra``; each function here can also be run on
its own (the commands the profiler summaries under ``profiles/`` were captured with).

What is measured, and against what:

* ``lds``      - conflict-free 8-byte shared-memory loads (the instruction the LUT GEMM's lookups are made of):
                 measured bank words / clk / SM beside the architectural 32;
* ``stream``   - the HBM-bound kernels (abs-max / min-max statistics, fused fake-quant to a 1-byte image, the
                 operator-form fake-quant forward and backward) on a 256 MiB fp32 tensor: algorithmic bytes / time
                 against the measured copy bandwidth;
* ``backward`` - STE / LRE image-space backward (grad_x, grad_w) on the ResNet-18 layer set: 2*B*L*K*O flop / time;
* ``fp32``     - a table of the fp32 class on the headline GEMM shape: table on chip (cluster) vs global memory;
* ``custom``   - custom-pair backward and the depthwise forward on the single-layer configuration's shape: lookups/s;
* ``layers``   - the LUT conv forward per distinct ResNet-50 layer shape (with the unsigned zero-point epilogue):
                 plan chosen, time, lookups/s, fraction of the lookup roofline, and the multiplicity-weighted total.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os

import torch

from .backend import _C, ops

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# distinct approximate-conv shapes of torchvision's ResNet-50 (all but the stem): (C, H, O, k, stride, pad, count)
RESNET50_LAYERS = [
    (64, 56, 64, 1, 1, 0, 1), (64, 56, 64, 3, 1, 1, 3), (64, 56, 256, 1, 1, 0, 4), (256, 56, 64, 1, 1, 0, 2),
    (256, 56, 128, 1, 1, 0, 1), (128, 56, 128, 3, 2, 1, 1), (128, 28, 512, 1, 1, 0, 4), (256, 56, 512, 1, 2, 0, 1),
    (512, 28, 128, 1, 1, 0, 3), (128, 28, 128, 3, 1, 1, 3),
    (512, 28, 256, 1, 1, 0, 1), (256, 28, 256, 3, 2, 1, 1), (256, 14, 1024, 1, 1, 0, 6), (512, 28, 1024, 1, 2, 0, 1),
    (1024, 14, 256, 1, 1, 0, 5), (256, 14, 256, 3, 1, 1, 5),
    (1024, 14, 512, 1, 1, 0, 1), (512, 14, 512, 3, 2, 1, 1), (512, 7, 2048, 1, 1, 0, 3), (1024, 14, 2048, 1, 2, 0, 1),
    (2048, 7, 512, 1, 1, 0, 2), (512, 7, 512, 3, 1, 1, 2),
]
# approximate-conv shapes of the CIFAR-stem ResNet-18: (C, H, O, k, stride, pad, count)
RESNET18_CIFAR_LAYERS = [
    (64, 32, 64, 3, 1, 1, 4), (64, 32, 128, 3, 2, 1, 1), (128, 16, 128, 3, 1, 1, 3), (64, 32, 128, 1, 2, 0, 1),
    (128, 16, 256, 3, 2, 1, 1), (256, 8, 256, 3, 1, 1, 3), (128, 16, 256, 1, 2, 0, 1),
    (256, 8, 512, 3, 2, 1, 1), (512, 4, 512, 3, 1, 1, 3), (256, 8, 512, 1, 2, 0, 1),
]


def peaks(dev):
    """Roofline denominators: measured HBM copy bandwidth and max SM clock when the measurement file is present."""
    out = {"hbm_gbs": 6650.0, "sm_max_mhz": 1965.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(os.path.join(_REPO, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        out.update(hbm_gbs=float(m["hbm_gbs"]), sm_max_mhz=float(m["sm_max_mhz"]), bf16_tflops=float(m["bf16_tflops"]),
                   source="MEASURED_PEAKS.json")
    except Exception:
        pass
    out["sms"] = torch.cuda.get_device_properties(dev).multi_processor_count
    out["lookup_peak"] = out["sms"] * 32 * out["sm_max_mhz"] * 1e6
    return out


def _time_ms(fn, iters=10, warmup=3, flush=None, reps=1):
    """Mean device time of fn() in ms.  ``flush``: a buffer larger than L2 rewritten before every timed event pair
    (outside it) for kernels whose operands would otherwise stay in L2.  ``reps`` > 1 enqueues that many calls
    back to back inside one event pair, so that the host's launch latency hides behind the queued work (needed
    for kernels of a few hundred microseconds launched from Python)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / (iters * reps)


# ----------------------------------------------------------------------------------------------- shared-memory peak
def lds_peak(dev, pk=None):
    pk = pk or peaks(dev)
    blocks, iters = pk["sms"], 4096
    seed = torch.randint(0, 2 ** 31 - 1, (256,), dtype=torch.int32, device=dev)
    out = torch.empty(blocks * 1024, dtype=torch.int32, device=dev)
    st = ops._stream(out)

    def fn():
        _C.check(_C.lib.atb_probe_shared_load(ops._ptr(seed), ops._ptr(out), blocks, iters, st), "probe")
    ms = _time_ms(fn, iters=5)
    words = blocks * 1024 * iters * 8 * 2
    per_clk_sm = words / (ms * 1e-3) / (pk["sms"] * pk["sm_max_mhz"] * 1e6)
    return {"bank_words_per_clk_per_sm_measured": per_clk_sm, "architectural": 32,
            "measured_lookup_peak": per_clk_sm * pk["sms"] * pk["sm_max_mhz"] * 1e6,
            "note": "conflict-free 8-byte ld.shared, 32 warps/SM, 8 independent loads in flight per thread; "
                    "clock taken as the max SM clock"}


# ----------------------------------------------------------------------------------------------- HBM-bound kernels
def stream_kernels(dev, pk=None, mib=512):
    pk = pk or peaks(dev)
    n = mib * (1 << 20) // 4
    x = torch.randn(n, device=dev)
    scale = torch.tensor(0.03, device=dev)
    zero = torch.tensor(117.0, device=dev)
    q8, mask = ops.quantize_image(x, scale, None, -127, 127)
    go = torch.randn(n, device=dev)
    cases = {
        "stats_kernel(absmax)": (lambda: ops.absmax(x), 4),
        "stats_kernel(absmax+min+max)": (lambda: ops.absmax(x, want_minmax=True), 4),
        "quantize_image_kernel(int8+mask)": (lambda: ops.quantize_image(x, scale, None, -127, 127), 6),
        "quantize_image_kernel(uint8,no mask)": (lambda: ops.quantize_image(x, scale, zero, 0, 255, want_mask=False), 5),
        "fakequant_fwd_kernel": (lambda: ops._fakequant(x, scale, None, -127, 127), 9),
        "fakequant_bwd_kernel": (lambda: ops._fakequant_backward(go, mask, scale), 9),
    }
    out = {}
    for name, (fn, bytes_per_elem) in cases.items():
        ms = _time_ms(fn, reps=6)                       # operands four times the size of L2: no flush needed
        gbs = n * bytes_per_elem / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "bytes_per_elem": bytes_per_elem, "gbs": gbs, "frac_of_hbm_peak": gbs / pk["hbm_gbs"]}
    out["tensor_mib"] = mib
    out["peak_gbs"] = pk["hbm_gbs"]
    out["peak_source"] = pk["source"]
    return out


# ----------------------------------------------------------------------------------------------- dense backward
def backward_kernels(dev, batch=256, layers=None, mode="ste", tensor_cores=True, packed=True):
    """grad_x and grad_w of the image-space STE / LRE backward per layer shape; flop = 2 * B*OH*OW * C*k*k * O (the
    useful fp32-equivalent work, whatever number of bf16 products the tensor-core path spends on it)."""
    layers = layers or RESNET18_CIFAR_LAYERS
    pk = peaks(dev)
    rows, tot = [], {"gx_ms": 0.0, "gw_ms": 0.0, "flop": 0.0}
    table = ops.decode_table(dev, 128) if mode == "ste" else torch.randn(256, device=dev)
    exact = mode == "ste"
    saved, saved_packed = ops.TENSOR_CORE_BACKWARD, ops.PACKED_BACKWARD
    ops.TENSOR_CORE_BACKWARD, ops.PACKED_BACKWARD = tensor_cores, packed
    try:
        for (C, H, O, k, s, p, count) in layers:
            x8 = torch.randint(-127, 128, (batch, C, H, H), dtype=torch.int8, device=dev)
            widx = torch.randint(0, 256, (O, C * k * k), dtype=torch.uint8, device=dev)
            g4 = ((k, k), (s, s), (p, p), (1, 1))
            OH = (H + 2 * p - k) // s + 1
            go = torch.randn(batch, O, OH, OH, device=dev)
            gs = torch.rand(O, device=dev)
            gx_ms = _time_ms(lambda: ops.lre_conv_backward(go, x8, widx, table, table, g4, 128, go_scale=gs, need_w=False,
                                                           exact_tables=exact), iters=3, warmup=2, reps=4)
            gw_ms = _time_ms(lambda: ops.lre_conv_backward(go, x8, widx, table, table, g4, 128, go_scale=gs, need_x=False,
                                                           exact_tables=exact), iters=3, warmup=2, reps=4)
            flop = 2.0 * batch * OH * OH * C * k * k * O
            rows.append({"C": C, "H": H, "O": O, "k": k, "stride": s, "count": count, "grad_x_ms": gx_ms, "grad_w_ms": gw_ms,
                         "grad_x_tflops": flop / gx_ms / 1e9, "grad_w_tflops": flop / gw_ms / 1e9})
            tot["gx_ms"] += gx_ms * count
            tot["gw_ms"] += gw_ms * count
            tot["flop"] += flop * count
    finally:
        ops.TENSOR_CORE_BACKWARD, ops.PACKED_BACKWARD = saved, saved_packed
    return {"batch": batch, "mode": mode,
            "path": ("tcgen05 (bf16 x3 split, fp32 TMEM accumulator), " + ("operands packed ahead by one pass over the gradient (included in the times)"
                                                                        if packed else "operands built inside the kernel")) if tensor_cores else "fp32 SIMT",
            "layers": rows, "total_grad_x_ms": tot["gx_ms"], "total_grad_w_ms": tot["gw_ms"],
            "total_grad_x_tflops": tot["flop"] / tot["gx_ms"] / 1e9, "total_grad_w_tflops": tot["flop"] / tot["gw_ms"] / 1e9,
            "fp32_fma_peak_tflops": 74.4,
            # tensor-core roofline: every useful product costs 3 (exact table) or 6 bf16 products
            "bf16_products_per_product": (3 if exact else 6) if tensor_cores else None,
            "frac_of_measured_bf16_peak": ({"grad_x": (3 if exact else 6) * tot["flop"] / tot["gx_ms"] / 1e9 / pk["bf16_tflops"],
                                            "grad_w": (3 if exact else 6) * tot["flop"] / tot["gw_ms"] / 1e9 / pk["bf16_tflops"],
                                            "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}
                                           if tensor_cores else None)}


# ----------------------------------------------------------------------------------------------- custom pair / depthwise
def custom_kernels(dev, pk=None):
    """The single-layer configuration's GEMM shape (N=8, K=576, L=1024, O=64): custom-pair dX / dW as lookups/s
    (each touches every (x, w) pair once), and a depthwise 3x3 forward on [64,128,56,56]."""
    pk = pk or peaks(dev)
    N, K, L, O = 8, 576, 1024, 64
    x = torch.randint(0, 256, (N, K, L), dtype=torch.uint8, device=dev)
    w = torch.randint(0, 256, (O, K), dtype=torch.uint8, device=dev)
    dy = torch.randn(N, O, L, device=dev)
    tab = torch.randn(65536, device=dev)
    out = {}
    pairs = float(N) * K * L * O
    for name, fn in (("custom_dx", lambda: ops.bgemm_custom_grad_uint8_dx(x, w, dy, tab)),
                     ("custom_dw", lambda: ops.bgemm_custom_grad_uint8_dw(x, w, dy, tab))):
        ms = _time_ms(fn, iters=3, warmup=2, reps=4)
        out[name] = {"ms": ms, "lookups_per_s": pairs / (ms * 1e-3), "frac_of_lookup_peak": pairs / (ms * 1e-3) / pk["lookup_peak"]}
    B, C, H = 64, 128, 56
    lut = torch.round(torch.randn(65536, device=dev) * 100)
    x8 = torch.randint(-127, 128, (B, C, H, H), dtype=torch.int8, device=dev)
    wd = torch.randint(-127, 128, (C, 9), device=dev).float()
    ms = _time_ms(lambda: ops.dwconv_fake_int8_claude(x8, wd, lut, 3, 1, 1, 1), iters=3, warmup=2, reps=4)
    taps = float(B) * C * H * H * 9
    out["dwconv_3x3"] = {"ms": ms, "lookups_per_s": taps / (ms * 1e-3), "shape": [B, C, H, H],
                         "hbm_gbs": B * C * H * H * 5 / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": B * C * H * H * 5 / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
    return out


# ----------------------------------------------------------------------------------------------- LUT conv per layer
def _plan_name(R, K, O):
    plan = _C.GemmPlan()
    _C.check(_C.lib.atb_lut_gemm_plan(R, K, O, 0, -1, ctypes.byref(plan)), "plan")
    per_tile = plan.units_per_block / plan.chunks_per_tile
    kind = f"{plan.blocks} blocks x {per_tile:.2f} tiles" + (" (cut)" if plan.cut_tiles else "")
    return f"{plan.block_rows} rows, {kind}"


def lut_conv_layers(dev, batch, pk=None, layers=None):
    """Unsigned LUT conv forward (zero-point epilogue, scale) per distinct ResNet-50 layer shape at ``batch`` images."""
    pk = pk or peaks(dev)
    layers = layers or RESNET50_LAYERS
    lut = (torch.arange(256, device=dev).view(-1, 1) * torch.arange(256, device=dev).view(1, -1) // 64 * 64).float().reshape(-1)
    img = ops.lut_image(lut)
    rows, tot_ms, tot_macs = [], 0.0, 0.0
    for (C, H, O, k, s, p, count) in layers:
        x = torch.randint(0, 256, (batch, C, H, H), dtype=torch.uint8, device=dev)
        w = torch.randint(0, 256, (O, C * k * k), dtype=torch.uint8, device=dev)
        g4 = ((k, k), (s, s), (p, p), (1, 1))
        zx, zw = torch.tensor(117.0, device=dev), torch.full((O,), 120.0, device=dev)
        ws = w.sum(dim=1, dtype=torch.int32)
        al = torch.rand(O, device=dev)
        OH = (H + 2 * p - k) // s + 1
        R, K = batch * OH * OH, C * k * k
        ms = _time_ms(lambda: ops.lut_conv2d_launch(x, w, img, g4, -1, alpha=al, zero_x=zx, zero_w=zw, wsum=ws),
                      iters=3, warmup=2, reps=8)
        macs = float(R) * K * O
        by_channels = ops.ROWS_ORIENTATION and ops._rows_orientation_wins(R, K, O)
        rows.append({"C": C, "H": H, "O": O, "k": k, "stride": s, "count": count, "R": R, "K": K,
                     "tile_rows": "channels" if by_channels else "pixels",
                     "plan": _plan_name(O, K, R) if by_channels else _plan_name(R, K, O),
                     "ms": ms, "lookups_per_s": macs / (ms * 1e-3), "frac_of_lookup_peak": macs / (ms * 1e-3) / pk["lookup_peak"]})
        tot_ms += ms * count
        tot_macs += macs * count
    return {"batch": batch, "layers": rows, "total_ms": tot_ms, "total_lut_macs": tot_macs,
            "lookups_per_s": tot_macs / (tot_ms * 1e-3), "frac_of_lookup_peak": tot_macs / (tot_ms * 1e-3) / pk["lookup_peak"],
            "timing": "8 launches back to back per event pair (host launch latency hidden); operands L2-warm, as in "
                      "the model, where the previous layer has just written them"}


# ----------------------------------------------------------------------------------------------- fp32-class tables
def fp32_table(dev, pk=None):
    """A table that is not 16-bit exact (0.5 grid) on the headline GEMM shape (65536 x 576 x 256): the kernel that holds
    the fp32 table in a two-block cluster's shared memory, the same kernel staging from global memory, and the
    generic kernel's gather from global memory."""
    pk = pk or peaks(dev)
    R, K, O = 65536, 576, 256
    lut = (torch.randint(-4000, 4000, (65536,), device=dev).float() * 0.5)
    img = ops.lut_image(lut)
    x = torch.randint(0, 256, (R, K), dtype=torch.uint8, device=dev)
    w = torch.randint(0, 256, (O, K), dtype=torch.uint8, device=dev)
    y = torch.empty((R, O), dtype=torch.float32, device=dev)
    macs = float(R) * K * O
    out = {}
    saved = ops.FP32_TABLE_ON_CHIP
    try:
        for name, on_chip, cfg in (("cluster_shared_memory", True, -1), ("staged_from_global_memory", True, 1 << 25),
                                   ("gather_from_global_memory", False, -1)):
            ops.FP32_TABLE_ON_CHIP = on_chip
            ms = _time_ms(lambda: ops.lut_gemm_launch(x, w, img, y, R, K, 1, O, cfg=cfg), iters=3, warmup=2, reps=3)
            out[name] = {"ms": ms, "lookups_per_s": macs / (ms * 1e-3), "frac_of_lookup_peak": macs / (ms * 1e-3) / pk["lookup_peak"]}
    finally:
        ops.FP32_TABLE_ON_CHIP = saved
    out["shape"] = [R, K, O]
    return out


# ----------------------------------------------------------------------------------------------- whole model
def unsigned_truncated_table(dev, low_bits=6):
    """Exact unsigned product i*j with its low bits cleared (the ResNet-50 inference configuration's table)."""
    i = torch.arange(256, device=dev, dtype=torch.int64)
    prod = i.view(-1, 1) * i.view(1, -1)
    return ((prod >> low_bits) << low_bits).float().reshape(-1)


def build_resnet50_uint8(dev, calib_images=8):
    """torchvision ResNet-50, random init, every conv but the first swapped for the unsigned approximate layer,
    ranges frozen after one calibration pass (momentum 1: ranges := that batch's min / max)."""
    import torchvision
    from . import convert_model, nn as atnn
    torch.manual_seed(0)
    model = torchvision.models.resnet50()
    convert_model(model, unsigned_truncated_table(dev), qtype="uint8", update_scale=True, scale_momentum=1.0)
    model = model.to(dev).train()
    with torch.no_grad():
        model(torch.randn(calib_images, 3, 224, 224, device=dev))
    model.eval()
    for m in model.modules():
        if isinstance(m, atnn.Conv2d_uint8):
            m.freeze_scale()
    return model


def resnet50_forward(dev, batch, iters=3):
    """Eager eval forwards of the converted ResNet-50 (the command whose kernel list the profiler summary shows)."""
    model = build_resnet50_uint8(dev)
    x = torch.randn(batch, 3, 224, 224, device=dev)
    with torch.no_grad():
        ms = _time_ms(lambda: model(x), iters=iters, warmup=2)
    return {"batch": batch, "ms": ms, "img_s": batch / (ms * 1e-3), "launch": "eager (no CUDA graph)"}


# ----------------------------------------------------------------------------------------------- one launch of each kernel
def profile_once(dev):
    """Every hot kernel launched exactly once on a case sized for a profiler capture (operands of the streaming
    kernels larger than L2, a few hundred MB on the device in all): the command behind the summaries in profiles/."""
    pk = peaks(dev)
    n = 64 * (1 << 20)                                     # 256 MiB of fp32
    x = torch.randn(n, device=dev)
    scale, zero = torch.tensor(0.03, device=dev), torch.tensor(117.0, device=dev)
    ops.absmax(x, want_minmax=True)
    q8, mask = ops.quantize_image(x, scale, None, -127, 127)
    ops._fakequant_backward(x, mask, scale)
    del x, q8, mask
    # LUT conv forward: a ResNet-50 stage-3 1x1 layer at batch 128, and the headline GEMM shape's kernel on one batch item
    lut = unsigned_truncated_table(dev)
    img = ops.lut_image(lut)
    xi = torch.randint(0, 256, (128, 256, 14, 14), dtype=torch.uint8, device=dev)
    w = torch.randint(0, 256, (1024, 256), dtype=torch.uint8, device=dev)
    zw = torch.full((1024,), 120.0, device=dev)
    ops.lut_conv2d_launch(xi, w, img, ((1, 1), (1, 1), (0, 0), (1, 1)), -1, alpha=torch.rand(1024, device=dev), zero_x=zero,
                          zero_w=zw, wsum=w.sum(dim=1, dtype=torch.int32))
    # tensor-core backward: a ResNet-18 stage-2 3x3 layer at batch 256
    x8 = torch.randint(-127, 128, (256, 128, 16, 16), dtype=torch.int8, device=dev)
    wi = torch.randint(0, 256, (128, 128 * 9), dtype=torch.uint8, device=dev)
    go = torch.randn(256, 128, 16, 16, device=dev)
    dec = ops.decode_table(dev, 128)
    ops.lre_conv_backward(go, x8, wi, dec, dec, ((3, 3), (1, 1), (1, 1), (1, 1)), 128, exact_tables=True)
    saved = ops.PACKED_BACKWARD
    ops.PACKED_BACKWARD = False                            # the same layer with the operands built inside the kernel
    try:
        ops.lre_conv_backward(go, x8, wi, dec, dec, ((3, 3), (1, 1), (1, 1), (1, 1)), 128, exact_tables=True)
    finally:
        ops.PACKED_BACKWARD = saved
    # custom-pair backward and a table of the fp32 class on the single-layer configuration's GEMM shape
    N, K, L, O = 8, 576, 1024, 64
    xc = torch.randint(0, 256, (N, K, L), dtype=torch.uint8, device=dev)
    wc = torch.randint(0, 256, (O, K), dtype=torch.uint8, device=dev)
    dy = torch.randn(N, O, L, device=dev)
    tab = torch.randn(65536, device=dev)
    ops.bgemm_custom_grad_uint8_dx(xc, wc, dy, tab)
    ops.bgemm_custom_grad_uint8_dw(xc, wc, dy, tab)
    half = torch.randint(-4000, 4000, (65536,), device=dev).float() * 0.5
    y = torch.empty((N, O, L), dtype=torch.float32, device=dev)
    ops.lut_gemm_launch(xc, wc, ops.lut_image(half), y, N, K, L, O)
    torch.cuda.synchronize()
    return {"launched": "stats, quantize_image, fakequant_bwd, lut_gemm (1x1 conv), tc_pack_go, tc_pack_w, tc_packed (grad_x, grad_w), "
                        "tc_gemm (grad_x, grad_w), pair_grad (dx, dw), pair_fwd"}


def orientation(dev, pk=None, batch=16):
    """Two late ResNet-50 layers at a small batch with the pixels and with the output channels as tile rows (same
    results bit for bit): the case the channels-as-rows orientation exists for."""
    pk = pk or peaks(dev)
    lut = unsigned_truncated_table(dev)
    img = ops.lut_image(lut)
    out = {"batch": batch, "table_kept_alive": lut.numel()}
    real = ops._rows_orientation_wins
    try:
        for (C, H, O, k, s, p) in ((2048, 7, 512, 1, 1, 0), (512, 7, 512, 3, 1, 1)):
            x = torch.randint(0, 256, (batch, C, H, H), dtype=torch.uint8, device=dev)
            w = torch.randint(0, 256, (O, C * k * k), dtype=torch.uint8, device=dev)
            g4 = ((k, k), (s, s), (p, p), (1, 1))
            zx, zw = torch.tensor(117.0, device=dev), torch.full((O,), 120.0, device=dev)
            ws = w.sum(dim=1, dtype=torch.int32)
            al = torch.rand(O, device=dev)
            OH = (H + 2 * p - k) // s + 1
            macs = float(batch * OH * OH) * C * k * k * O
            row = {}
            ys = []
            for name, force in (("pixels_as_rows", False), ("channels_as_rows", True)):
                ops._rows_orientation_wins = (lambda R_, K_, O_, f=force: f)
                ms = _time_ms(lambda: ops.lut_conv2d_launch(x, w, img, g4, -1, alpha=al, zero_x=zx, zero_w=zw, wsum=ws),
                              iters=3, warmup=2, reps=8)
                ys.append(ops.lut_conv2d_launch(x, w, img, g4, -1, alpha=al, zero_x=zx, zero_w=zw, wsum=ws))
                row[name] = {"ms": ms, "lookups_per_s": macs / (ms * 1e-3), "frac_of_lookup_peak": macs / (ms * 1e-3) / pk["lookup_peak"]}
            row["bit_identical"] = bool(torch.equal(ys[0], ys[1]))
            out[f"C{C}_H{H}_O{O}_k{k}"] = row
    finally:
        ops._rows_orientation_wins = real
    return out


def run_all(dev, which=("lds", "stream", "backward", "custom", "fp32", "orientation", "layers"), batches=(128, 16)):
    pk = peaks(dev)
    out = {"peaks": pk}
    for name in which:
        try:
            if name == "lds":
                out["lds"] = lds_peak(dev, pk)
            elif name == "stream":
                out["stream"] = stream_kernels(dev, pk)
            elif name == "backward":
                out["backward_ste_resnet18_cifar_b256"] = backward_kernels(dev)
                out["backward_lre_resnet18_cifar_b256"] = backward_kernels(dev, mode="lre")
                out["backward_ste_resnet18_cifar_b256_operands_in_kernel"] = backward_kernels(dev, packed=False)
                out["backward_ste_resnet18_cifar_b256_simt"] = backward_kernels(dev, tensor_cores=False)
            elif name == "custom":
                out["custom"] = custom_kernels(dev, pk)
            elif name == "profile":
                out["profile"] = profile_once(dev)
            elif name == "orientation":
                out["orientation_b16"] = orientation(dev, pk)
            elif name == "fp32":
                out["fp32_class_table"] = fp32_table(dev, pk)
            elif name == "model":
                for b in batches:
                    out[f"resnet50_forward_b{b}"] = resnet50_forward(dev, b)
            elif name == "layers":
                for b in batches:
                    out[f"resnet50_lut_conv_layers_b{b}"] = lut_conv_layers(dev, b, pk)
        except Exception as exc:                       # a measurement aid must not take the headline line down
            out[name + "_error"] = f"{type(exc).__name__}: {exc}"[:300]
        torch.cuda.empty_cache()
    return out


def _print_table(res):
    for key, val in res.items():
        if isinstance(val, dict) and "layers" in val:
            print(f"== {key}")
            for r in val["layers"]:
                print("  " + "  ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in r.items()))
            print("  " + "  ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in val.items() if k != "layers"))
        else:
            print(f"== {key}: {json.dumps(val)}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="lds,stream,backward,custom,fp32,orientation,layers")
    ap.add_argument("--batch", default="128,16")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args()
    device = torch.device("cuda:0")
    result = run_all(device, tuple(a.only.split(",")), tuple(int(b) for b in a.batch.split(",")))
    if a.json:
        print(json.dumps(result))
    else:
        _print_table(result)
