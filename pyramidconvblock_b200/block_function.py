"""ConvBlock as ONE autograd Function with a hand-ordered backward.

Same arithmetic as composing the per-op Functions (pyramid_dwconv/conv_block.py:36-49), but because
the whole block is visible at once:

* each branch writes straight into its channel slice of the concatenated buffer and reads its slice
  of the concatenated gradient in place (no ``torch.cat`` kernel, no strided copies);
* the broadcast ``+ x_pool`` and the gradient of the spatial mean are in-place row-broadcast adds
  instead of full-size broadcast kernels followed by an add;
* the pooled branch's input gradient is accumulated onto the full-resolution branch's inside the
  pool-backward kernel;
* the gradient w.r.t. the pooled row (needed by both output biases) is reduced once.

The three ``nn.Linear`` are dense GEMMs and stay on cuBLAS (``torch.mm`` / ``F.linear``).
"""
import torch
import torch.nn.functional as F

from . import ops


class ConvBlockFunction(torch.autograd.Function):
    """apply(x, scales, w_up, b_up, w_out, b_out, w_pool, b_pool, *dw_weights) -> y, all [B,H,W,*] NHWC."""

    @staticmethod
    def forward(ctx, x, scales, w_up, b_up, w_out, b_out, w_pool, b_pool, *dw_weights):
        x = x.contiguous()
        B, H, W, dim = x.shape
        inter = w_up.shape[0]
        half = inter // 2
        inv_scale = 1.0 / (inter / 2) ** -0.5
        t = F.linear(x, w_up, b_up)                                     # conv_up
        cat = torch.empty((B, H, W, half * len(scales)), device=x.device, dtype=x.dtype)
        saved = []
        for i, (s, w) in enumerate(zip(scales, dw_weights)):
            k = w.shape[0]
            out_slice = cat[..., i * half:(i + 1) * half]
            if s != 1.:
                pin = ops.pool_forward(t, (int(H * s), int(W * s)))
                c = ops.dwconv_forward(pin, w, None, 1, k // 2, 1)
                ops.upsample_forward_into(ops.gate_forward(c, inv_scale), out_slice)
                saved += [pin, c]
            else:
                c = ops.dwconv_forward(t, w, None, 1, k // 2, 1)
                ops.gate_forward_into(c, out_slice, inv_scale)
                saved += [c]
        y = F.linear(cat, w_out, b_out)                                  # conv_out
        mean = x.mean(dim=(1, 2))                                        # [B, dim]
        ops.add_pooled_(y, F.linear(mean, w_pool, b_pool))               # + conv_pool(mean), broadcast
        ctx.scales = tuple(scales)
        ctx.has_bias = (b_up is not None, b_out is not None, b_pool is not None)
        ctx.inv_scale = inv_scale
        ctx.save_for_backward(x, t, cat, mean, w_up, w_out, w_pool, *dw_weights, *saved)
        return y

    @staticmethod
    def backward(ctx, g):
        scales = ctx.scales
        n = len(scales)
        x, t, cat, mean, w_up, w_out, w_pool = ctx.saved_tensors[:7]
        dw_weights = ctx.saved_tensors[7:7 + n]
        saved = list(ctx.saved_tensors[7 + n:])
        B, H, W, dim = x.shape
        N = B * H * W
        half = w_up.shape[0] // 2
        dtype = x.dtype
        g = g.contiguous()
        g2 = g.view(N, dim)

        # conv_out / conv_pool: the pooled row's gradient (sum of g over the image) serves both biases
        dpooled32 = g.sum(dim=(1, 2), dtype=torch.float32)               # [B, dim]
        dpooled = dpooled32.to(dtype)
        dbias = dpooled32.sum(0).to(dtype)
        d_w_out = g2.t().mm(cat.view(N, -1))
        dcat = g2.mm(w_out).view(B, H, W, -1)
        d_w_pool = dpooled.t().mm(mean)
        dmean = dpooled.mm(w_pool)                                       # [B, dim]

        d_dw = [None] * n
        dt = None
        order = sorted(range(n), key=lambda i: scales[i] != 1.)          # a full-resolution branch first
        pos = {}
        off = 0
        for i, s in enumerate(scales):
            pos[i] = off
            off += 2 if s != 1. else 1
        for i in order:
            s, w = scales[i], dw_weights[i]
            k = w.shape[0]
            gslice = dcat[..., i * half:(i + 1) * half]
            if s != 1.:
                pin, c = saved[pos[i]], saved[pos[i] + 1]
                dgate = ops.upsample_backward_from(gslice, (c.shape[1], c.shape[2]))
                dc = ops.gate_backward(c, dgate, ctx.inv_scale)
            else:
                pin, c = t, saved[pos[i]]
                dc = ops.gate_backward_from(c, gslice, ctx.inv_scale)
            # parameter gradient first, then the input gradient (whoever reduces parameter gradients
            # across ranks can start earlier)
            d_dw[i], _ = ops.dwconv_backward_weight(pin, dc, k, 1, k // 2, 1)
            dpin = ops.dwconv_backward_input(dc, w, (pin.shape[1], pin.shape[2]), 1, k // 2, 1)
            if s != 1.:
                if dt is None:
                    dt = ops.pool_backward(dpin, (H, W))
                else:
                    ops.pool_backward_accumulate(dpin, dt)
            else:
                dt = dpin if dt is None else dt.add_(dpin)

        dt2 = dt.view(N, -1)
        d_w_up = dt2.t().mm(x.view(N, dim))
        d_b_up = dt2.sum(0, dtype=torch.float32).to(dtype) if ctx.has_bias[0] else None
        dx = None
        if ctx.needs_input_grad[0]:
            dx = dt2.mm(w_up).view(B, H, W, dim)
            ops.add_pooled_(dx, dmean, 1.0 / (H * W))                    # gradient of the spatial mean
        return (dx, None, d_w_up, d_b_up, d_w_out, dbias if ctx.has_bias[1] else None, d_w_pool,
                dbias if ctx.has_bias[2] else None, *d_dw)
