"""world_size-2 gloo checks of the only collectives on the path: the activation-statistic exchange that
precedes quantisation in training (MAX for the signed layer, MIN + MAX for the unsigned one).  Ranks see
different data and must end with bit-identical scales equal to the statistics of the union."""

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import approxtorch_b200 as at
        lut = torch.zeros(65536)
        torch.manual_seed(0)                        # same weights on every rank, as under DDP
        a = at.nn.Conv2d_int8(3, 4, 3, lut, scale_momentum=0.1)
        b = at.nn.Conv2d_uint8(3, 4, 3, lut, scale_momentum=0.2)
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(2, 3, 5, 5, generator=g) * (1 + 3 * rank)
        a._update_scale(x)
        a._update_scale_w()
        b._update_scale(x)
        b._update_scale_w()
        torch.save({"x": x, "a_sx": a.scale_x, "a_sw": a.scale_w, "b": [b.x_min, b.x_max, b.scale_x, b.zero_x]},
                   os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_scale_exchange_world_size_2(tmp_path):
    from oracle import lut_oracle as lo
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "r0.pt")
    r1 = torch.load(tmp_path / "r1.pt")
    assert not torch.equal(r0["x"], r1["x"])
    for key in ("a_sx", "a_sw"):
        assert torch.equal(r0[key], r1[key])
    for u, v in zip(r0["b"], r1["b"]):
        assert torch.equal(u, v)
    both = torch.cat([r0["x"], r1["x"]]).numpy()
    assert r0["a_sx"].item() == lo.ema_scale_x(np.abs(both).max(), 1.0, 0.1)
    xmin = lo.ema(both.min(), 0.0, 0.2)
    xmax = lo.ema(both.max(), 1.0, 0.2)
    sx, zx = lo.uint8_qparams(xmin, xmax)
    assert r0["b"][0].item() == xmin and r0["b"][1].item() == xmax
    assert r0["b"][2].item() == sx and r0["b"][3].item() == zx
