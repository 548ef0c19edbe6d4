/*
 * pdw_oracle.c - CPU restatement of the reference's hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA kernels are compared against; it is never the thing that is
 * shipped or measured as the product.  Only tests/, __graft_entry__.smoke() and the CPU-baseline
 * leg of bench.py may call it.
 *
 * Each function restates one kernel of IrisRainbowNeko/PyramidConvBlock (file:line cited per
 * function) as plain loops over dense NHWC float arrays.  The reference accumulates in fp32
 * (tl.float32 accumulators); here sums are carried in double so the oracle is a tighter truth than
 * either implementation, and inputs that model 16-bit tensors are rounded to that grid by the
 * caller before they get here.
 *
 * Parity pin: tests/test_oracle.py checks every function against tests/golden/ (outputs of the
 * unmodified reference run under TRITON_INTERPRET=1, see tests/golden/make_golden.py) and against
 * the torch CPU ops the reference names as its own comparator (dwconv_triton.py:457,494-516).
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define IDX4(b, h, w, c, H, W, C) ((((size_t)(b) * (H) + (h)) * (W) + (w)) * (C) + (c))

static int out_size(int in, int k, int s, int p, int d) { return (in + 2 * p - d * (k - 1) - 1) / s + 1; }

/* _depthwise_conv_kernel_optimized, pyramid_dwconv/dwconv_triton.py:55-104: for every tap the
 * input tile is read at (o*s - p + k*d), zero outside the image, times w[kh,kw,c]. */
void oracle_dwconv_fwd(const float* x, const float* w, const float* bias, float* y, int B, int H, int W, int C,
                       int KH, int KW, int sh, int sw, int ph, int pw, int dh, int dw) {
    const int OH = out_size(H, KH, sh, ph, dh), OW = out_size(W, KW, sw, pw, dw);
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow)
                for (int c = 0; c < C; ++c) {
                    double acc = bias ? (double)bias[c] : 0.0;
                    for (int kh = 0; kh < KH; ++kh) {
                        const int ih = oh * sh - ph + kh * dh;
                        if (ih < 0 || ih >= H) continue;
                        for (int kw = 0; kw < KW; ++kw) {
                            const int iw = ow * sw - pw + kw * dw;
                            if (iw < 0 || iw >= W) continue;
                            acc += (double)x[IDX4(b, ih, iw, c, H, W, C)] * (double)w[((size_t)kh * KW + kw) * C + c];
                        }
                    }
                    y[IDX4(b, oh, ow, c, OH, OW, C)] = (float)acc;
                }
}

/* _depthwise_conv_backward_input_kernel, pyramid_dwconv/dwconv_triton.py:154-203.  The reference
 * writes it as a correlation of grad_out with the filter mirrored on both axes, which is the
 * adjoint of the forward only for stride 1 and 2p == (k-1)d.  The oracle states the adjoint itself
 * (every forward product scattered back), which coincides with the reference wherever the
 * reference is right and defines the answer elsewhere. */
void oracle_dwconv_bwd_input(const float* gout, const float* w, float* dx, int B, int H, int W, int C, int KH,
                             int KW, int sh, int sw, int ph, int pw, int dh, int dw) {
    const int OH = out_size(H, KH, sh, ph, dh), OW = out_size(W, KW, sw, pw, dw);
    const size_t n = (size_t)B * H * W * C;
    double* acc = (double*)calloc(n, sizeof(double));
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow)
                for (int kh = 0; kh < KH; ++kh) {
                    const int ih = oh * sh - ph + kh * dh;
                    if (ih < 0 || ih >= H) continue;
                    for (int kw = 0; kw < KW; ++kw) {
                        const int iw = ow * sw - pw + kw * dw;
                        if (iw < 0 || iw >= W) continue;
                        const float* g = gout + IDX4(b, oh, ow, 0, OH, OW, C);
                        const float* wt = w + ((size_t)kh * KW + kw) * C;
                        double* a = acc + IDX4(b, ih, iw, 0, H, W, C);
                        for (int c = 0; c < C; ++c) a[c] += (double)g[c] * (double)wt[c];
                    }
                }
    for (size_t i = 0; i < n; ++i) dx[i] = (float)acc[i];
    free(acc);
}

/* _depthwise_conv_weight_grad_kernel, pyramid_dwconv/dwconv_triton.py:266-296:
 * dW[kh,kw,c] = sum_{b,oh,ow} gout[b,oh,ow,c] * x[b, oh*s-p+kh*d, ow*s-p+kw*d, c] (the reference
 * writes the same sum with mirrored indices and atomics).  dbias (not in the reference) is the plain
 * sum of gout over b,oh,ow. */
void oracle_dwconv_bwd_weight(const float* x, const float* gout, float* dwt, float* dbias, int B, int H, int W,
                              int C, int KH, int KW, int sh, int sw, int ph, int pw, int dh, int dw) {
    const int OH = out_size(H, KH, sh, ph, dh), OW = out_size(W, KW, sw, pw, dw);
    const size_t nw = (size_t)KH * KW * C;
    double* acc = (double*)calloc(nw + C, sizeof(double));
    double* accb = acc + nw;
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow) {
                const float* g = gout + IDX4(b, oh, ow, 0, OH, OW, C);
                for (int c = 0; c < C; ++c) accb[c] += (double)g[c];
                for (int kh = 0; kh < KH; ++kh) {
                    const int ih = oh * sh - ph + kh * dh;
                    if (ih < 0 || ih >= H) continue;
                    for (int kw = 0; kw < KW; ++kw) {
                        const int iw = ow * sw - pw + kw * dw;
                        if (iw < 0 || iw >= W) continue;
                        const float* xi = x + IDX4(b, ih, iw, 0, H, W, C);
                        double* a = acc + ((size_t)kh * KW + kw) * C;
                        for (int c = 0; c < C; ++c) a[c] += (double)g[c] * (double)xi[c];
                    }
                }
            }
    for (size_t i = 0; i < nw; ++i) dwt[i] = (float)acc[i];
    if (dbias)
        for (int c = 0; c < C; ++c) dbias[c] = (float)accb[c];
    free(acc);
}

static int win_start(int o, int in, int out) { return (int)(((long long)o * in) / out); }
static int win_end(int o, int in, int out) { return (int)((((long long)o + 1) * in + out - 1) / out); }

/* _adaptive_avg_pool_kernel, pyramid_dwconv/avgpool_triton.py:42-89: mean over the window
 * [floor(o*in/out), ceil((o+1)*in/out)).  The reference evaluates the bounds in float16, which is
 * wrong for many non-power-of-two sizes; the oracle uses exact integers (torch's definition), equal
 * to the reference wherever its float16 arithmetic is exact. */
void oracle_pool_fwd(const float* x, float* y, int B, int H, int W, int C, int OH, int OW) {
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow) {
                const int hs = win_start(oh, H, OH), he = win_end(oh, H, OH);
                const int ws = win_start(ow, W, OW), we = win_end(ow, W, OW);
                for (int c = 0; c < C; ++c) {
                    double acc = 0.0;
                    for (int ih = hs; ih < he; ++ih)
                        for (int iw = ws; iw < we; ++iw) acc += (double)x[IDX4(b, ih, iw, c, H, W, C)];
                    y[IDX4(b, oh, ow, c, OH, OW, C)] = (float)(acc / (double)((he - hs) * (we - ws)));
                }
            }
}

/* _adaptive_avg_pool_grad_kernel, pyramid_dwconv/avgpool_triton.py:150-203: every output's
 * gradient divided by its window area is added to each input of the window. */
void oracle_pool_bwd(const float* gout, float* dx, int B, int H, int W, int C, int OH, int OW) {
    const size_t n = (size_t)B * H * W * C;
    double* acc = (double*)calloc(n, sizeof(double));
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow) {
                const int hs = win_start(oh, H, OH), he = win_end(oh, H, OH);
                const int ws = win_start(ow, W, OW), we = win_end(ow, W, OW);
                const double inv = 1.0 / (double)((he - hs) * (we - ws));
                for (int ih = hs; ih < he; ++ih)
                    for (int iw = ws; iw < we; ++iw)
                        for (int c = 0; c < C; ++c)
                            acc[IDX4(b, ih, iw, c, H, W, C)] += (double)gout[IDX4(b, oh, ow, c, OH, OW, C)] * inv;
            }
    for (size_t i = 0; i < n; ++i) dx[i] = (float)acc[i];
    free(acc);
}

/* Source coordinates of _bilinear_interp_kernel, pyramid_dwconv/up_triton.py:42-59, in float32 as
 * the reference computes them: src = max((dst + 0.5) * in/out - 0.5, 0), lo = floor clamped,
 * hi = min(lo + 1, in - 1). */
static void taps(int dst, int in, int out, int* lo, int* hi, float* frac) {
    const float scale = (float)in / (float)out;
    float src = ((float)dst + 0.5f) * scale - 0.5f;
    if (src < 0.f) src = 0.f;
    int l = (int)floorf(src);
    if (l > in - 1) l = in - 1;
    *lo = l;
    *hi = l + 1 < in - 1 ? l + 1 : in - 1;
    *frac = src - (float)l;
}

/* _bilinear_interp_kernel, pyramid_dwconv/up_triton.py:62-125: four gathers times fp32 weights. */
void oracle_upsample_fwd(const float* x, float* y, int B, int H, int W, int C, int OH, int OW) {
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh) {
            int y0, y1; float fy;
            taps(oh, H, OH, &y0, &y1, &fy);
            for (int ow = 0; ow < OW; ++ow) {
                int x0, x1; float fx;
                taps(ow, W, OW, &x0, &x1, &fx);
                const double wlt = (double)(1.f - fx) * (double)(1.f - fy), wrt = (double)fx * (double)(1.f - fy);
                const double wlb = (double)(1.f - fx) * (double)fy, wrb = (double)fx * (double)fy;
                for (int c = 0; c < C; ++c)
                    y[IDX4(b, oh, ow, c, OH, OW, C)] =
                        (float)((double)x[IDX4(b, y0, x0, c, H, W, C)] * wlt + (double)x[IDX4(b, y0, x1, c, H, W, C)] * wrt +
                                (double)x[IDX4(b, y1, x0, c, H, W, C)] * wlb + (double)x[IDX4(b, y1, x1, c, H, W, C)] * wrb);
            }
        }
}

/* The reference has no upsample backward (up_triton.py:127-162 is a plain nn.Module); inside
 * ConvBlock the gradient of conv_block.py:21 is the adjoint of the forward above: every output
 * gradient scattered to its four sources with the forward weights. */
void oracle_upsample_bwd(const float* gout, float* dx, int B, int H, int W, int C, int OH, int OW) {
    const size_t n = (size_t)B * H * W * C;
    double* acc = (double*)calloc(n, sizeof(double));
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh) {
            int y0, y1; float fy;
            taps(oh, H, OH, &y0, &y1, &fy);
            for (int ow = 0; ow < OW; ++ow) {
                int x0, x1; float fx;
                taps(ow, W, OW, &x0, &x1, &fx);
                const double wlt = (double)(1.f - fx) * (double)(1.f - fy), wrt = (double)fx * (double)(1.f - fy);
                const double wlb = (double)(1.f - fx) * (double)fy, wrb = (double)fx * (double)fy;
                for (int c = 0; c < C; ++c) {
                    const double g = (double)gout[IDX4(b, oh, ow, c, OH, OW, C)];
                    acc[IDX4(b, y0, x0, c, H, W, C)] += g * wlt;
                    acc[IDX4(b, y0, x1, c, H, W, C)] += g * wrt;
                    acc[IDX4(b, y1, x0, c, H, W, C)] += g * wlb;
                    acc[IDX4(b, y1, x1, c, H, W, C)] += g * wrb;
                }
            }
        }
    for (size_t i = 0; i < n; ++i) dx[i] = (float)acc[i];
    free(acc);
}
