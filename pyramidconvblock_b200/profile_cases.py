"""Small, self-contained launches of one C-ABI entry point, sized for profiler captures.

    python -m pyramidconvblock_b200.profile_cases CASE [--k 17] [--dtype bf16] [--batch 32]
                                                   [--size 96] [--channels 256] [--iters 3]
                                                   [--tile TH TW]

CASE is one of dwconv_fwd, dwconv_bwd_input, dwconv_bwd_weight, pool_fwd, pool_bwd, upsample_fwd,
upsample_bwd, gate_fwd, gate_bwd.  The default tensors ([32,96,96,256] 16-bit = 151 MB each) are
larger than the 126 MB L2, so DRAM counters mean something, yet hold well under 1 GB on the
device.  ``--tile`` forces the thread-block tile of the convolution kernels (the planner's choice
depends on the batch size; this reproduces the tile of a larger batch on the small capture).
Prints the average launch time measured with CUDA events.
"""
import argparse

import torch

from . import _lib, ops

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--k", type=int, default=17)
    ap.add_argument("--dtype", default="bf16", choices=sorted(DTYPES))
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--size", type=int, default=96)
    ap.add_argument("--channels", type=int, default=256)
    ap.add_argument("--small", type=int, default=0, help="pooled / pre-upsample extent (default size/2)")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--tile", type=int, nargs=2, metavar=("TH", "TW"), help="force the convolution tile")
    a = ap.parse_args()
    if a.tile:
        for key, value in ((3, a.tile[0]), (4, a.tile[1]), (5, a.tile[0]), (6, a.tile[1])):
            _lib.lib().pdw_set_tuning(key, value)
    dt = DTYPES[a.dtype]
    dev = torch.device("cuda", 0)
    B, S, C, k = a.batch, a.size, a.channels, a.k
    s = a.small or S // 2
    gen = torch.Generator(device=dev).manual_seed(0)
    big = torch.randn((B, S, S, C), generator=gen, device=dev).to(dt)
    big2 = torch.randn((B, S, S, C), generator=gen, device=dev).to(dt)
    small = torch.randn((B, s, s, C), generator=gen, device=dev).to(dt)
    w = (torch.randn((k, k, C), generator=gen, device=dev) / k).to(dt)
    bias = torch.zeros(C, device=dev, dtype=dt)
    inv = 1.0 / (C / 2) ** -0.5
    cases = {
        "dwconv_fwd": lambda: ops.dwconv_forward(big, w, bias, 1, k // 2, 1),
        "dwconv_bwd_input": lambda: ops.dwconv_backward_input(big, w, (S, S), 1, k // 2, 1),
        "dwconv_bwd_weight": lambda: ops.dwconv_backward_weight(big, big2, k, 1, k // 2, 1, with_bias=True),
        "pool_fwd": lambda: ops.pool_forward(big, (s, s)),
        "pool_bwd": lambda: ops.pool_backward(small, (S, S)),
        "upsample_fwd": lambda: ops.upsample_forward(small, (S, S)),
        "upsample_bwd": lambda: ops.upsample_backward(big, (s, s)),
        "gate_fwd": lambda: ops.gate_forward(big, inv),
        "gate_bwd": lambda: ops.gate_backward(big, big2[..., : C // 2].contiguous(), inv),
    }
    fn = cases[a.case]
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    print("%s k=%d %s [%d,%d,%d,%d] small=%d: %.4f ms per call" % (a.case, k, a.dtype, B, S, S, C, s,
                                                                  e0.elapsed_time(e1) / a.iters))


if __name__ == "__main__":
    main()
