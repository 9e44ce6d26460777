"""2+ GPU check of the halo-fused convolution against the convolution of the gathered image (run under torchrun)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from physicsnemo_b200 import ops
    from physicsnemo_b200.parallel.halo_conv import HaloConvRuntime, halo_conv2d_3x3

    rt = HaloConvRuntime()
    torch.manual_seed(0)
    n, cin, cout, h, w = 2, 64, 128, 16 * world, 40
    xg = torch.randn(n, cin, h, w, device="cuda")
    wt = torch.randn(cout, cin, 3, 3, device="cuda") / (9 * cin) ** 0.5
    b = torch.randn(cout, device="cuda")
    dyg = torch.randn(n, cout, h, w, device="cuda")
    hl = h // world
    sl = slice(rank * hl, (rank + 1) * hl)
    worst = 0.0
    for it in range(3):                                            # several calls: exercises the double-buffered mailboxes
        x = (xg[:, :, sl] * (1 + it)).clone().requires_grad_(True)
        wl, bl = wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
        y = halo_conv2d_3x3(x, wl, bl, rt)
        y.backward(dyg[:, :, sl].to(y.dtype))
        xr = (xg * (1 + it)).clone().requires_grad_(True)
        wr, br = wt.clone().requires_grad_(True), b.clone().requires_grad_(True)
        ref = torch.nn.functional.conv2d(xr, wr, br, padding=1)
        ref.backward(dyg)
        dw, db = wl.grad.clone(), bl.grad.clone()
        dist.all_reduce(dw)
        dist.all_reduce(db)
        scale = float(ref.abs().max())
        errs = [float((y.float() - ref[:, :, sl]).abs().max()) / scale,
                float((x.grad - xr.grad[:, :, sl]).abs().max()) / float(xr.grad.abs().max()),
                float((dw - wr.grad).abs().max()) / float(wr.grad.abs().max()),
                float((db - br.grad).abs().max()) / float(br.grad.abs().max())]
        worst = max(worst, *errs)
    rt.check()
    t = torch.tensor([worst], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # timing: fused halo conv vs. the unfused local conv of the same slab (no neighbour rows)
    x = xg[:, :, sl].contiguous(memory_format=torch.channels_last)
    big = torch.randn(4, 128, 512, 512, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    wb = (torch.randn(128, 128, 3, 3, device="cuda") / 34).to(torch.bfloat16)
    from physicsnemo_b200.ops import conv as C

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record(); torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / 10], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    with torch.no_grad():
        t_halo = timed(lambda: halo_conv2d_3x3(big, wb, None, rt))
        t_local = timed(lambda: C.conv2d_same(big, wb, None))
    rt.check()
    if rank == 0:
        print({"world": world, "worst_rel_err": float(t), "halo_conv_ms": t_halo, "local_conv_ms": t_local,
               "device_error": ops.device_error()})
        assert float(t) < 4e-2
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
