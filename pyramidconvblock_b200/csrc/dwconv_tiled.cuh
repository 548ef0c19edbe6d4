// Tiled depthwise-convolution kernels for stride 1 / dilation 1 (any zero padding).
//
// Data layout in shared memory: the input tile with its halo is brought in by ONE TMA copy
// (cp.async.bulk.tensor.4d) as a dense [rows][cols][CT channels] block, channel fastest, i.e.
// the NHWC order of global memory.  Parts of the box that fall outside the image are filled
// with zeros by the copy engine, which is the convolution's zero padding.  A warp's 32 lanes are
// CPL = CT/2 channel pairs x RL = 32/CPL consecutive rows; `cols` is kept odd so the RL row
// lanes hit different banks.  Each thread owns one channel pair and a strip of 16 output
// columns, keeps one filter row (K taps) in registers and slides it over the strip:
// every value read from shared memory feeds up to K packed FMAs.
//
// The same kernel computes the input gradient: it is run over grad_out with the filter taps
// mirrored while they are staged (pyramid_dwconv/dwconv_triton.py:177-182 does the same through
// its weight index) and padding K-1-p.
#pragma once

#include <type_traits>

#include "common.cuh"

namespace pdw {

constexpr int kStrip = 16;          // output columns per thread
constexpr int kFwdThreads = 256;    // 8 warps
constexpr int kSmemPerCta2 = 113 * 1024;  // lets two thread blocks share one SM
constexpr int kSmemMax = 227 * 1024;

struct TiledArgs {
    const void* in;
    const void* w;
    const void* bias;
    void* out;
    int B, H, W, C;      // input extents
    int OH, OW;          // output extents
    int KH, KW;
    int pad_h, pad_w;
    int flip;            // 1: mirror taps (input gradient)
    int dtype;
    int32_t* status;
    cudaStream_t stream;
};

struct TiledParams {
    const void* w;
    const void* bias;
    void* out;
    int OH, OW, C;
    int KH, pad_h, pad_w, flip;
    int TH, TWc;          // output tile of one thread block
    int rows, cols;       // shared-memory tile extents (with halo; cols odd)
    int tiles_w, tiles_h, nct;
    int n_items, n_strips;
    int32_t* status;
};

template <typename T, bool MIXED> struct WReg { using type = float2; };
template <typename T> struct WReg<T, true> { using type = uint32_t; };

template <typename T, int K, int CT, int MATH>
__global__ void __launch_bounds__(kFwdThreads, 2)
dwconv_tiled_kernel(const __grid_constant__ CUtensorMap tmap, const TiledParams p) {
    using E = Elem<T>;
    using pair_t = typename E::pair_t;
    constexpr bool MIXED = (MATH == 1) && (sizeof(T) == 2);
    using wreg_t = typename WReg<T, MIXED>::type;
    constexpr int CPL = CT / 2;
    constexpr int RL = 32 / CPL;
    constexpr int PIXB = CT * (int)sizeof(T);

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
    unsigned char* xs = smem + 128;
    const int x_bytes = p.rows * p.cols * PIXB;
    wreg_t* ws = reinterpret_cast<wreg_t*>(xs + round_up(x_bytes, 128));

    int t = blockIdx.x;
    const int ct = t % p.nct;  t /= p.nct;
    const int tw = t % p.tiles_w;  t /= p.tiles_w;
    const int th = t % p.tiles_h;
    const int b = t / p.tiles_h;

    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(bar, (uint32_t)x_bytes);
        tma_load_4d(xs, &tmap, bar, ct * CT, tw * p.TWc - p.pad_w, th * p.TH - p.pad_h, b);
    }

    // Stage this block's CT channels of the filter (converted once, mirrored for the input gradient)
    // while the copy engine fills the tile.
    {
        const T* wg = static_cast<const T*>(p.w);
        const int n = p.KH * K * CPL;
        for (int i = threadIdx.x; i < n; i += kFwdThreads) {
            const int cpi = i % CPL;
            const int kw = (i / CPL) % K;
            const int kh = i / (CPL * K);
            const int skh = p.flip ? (p.KH - 1 - kh) : kh;
            const int skw = p.flip ? (K - 1 - kw) : kw;
            const int c = ct * CT + 2 * cpi;
            pair_t v{};
            if (c < p.C) v = *reinterpret_cast<const pair_t*>(wg + ((size_t)(skh * K + skw) * p.C + c));
            if constexpr (MIXED) ws[i] = v; else ws[i] = E::unpack(v);
        }
    }
    __syncthreads();
    const bool arrived = mbar_wait_bounded(bar, 0, p.status);
    if (__syncthreads_or(!arrived)) return;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cp = lane % CPL, rl = lane / CPL;
    const int c = ct * CT + 2 * cp;
    float2 bias2 = make_float2(0.f, 0.f);
    if (p.bias != nullptr && c < p.C)
        bias2 = E::unpack(*reinterpret_cast<const pair_t*>(static_cast<const T*>(p.bias) + c));
    const int row_bytes = p.cols * PIXB;

    for (int item = warp; item < p.n_items; item += kFwdThreads / 32) {
        const int strip = item % p.n_strips;
        const int orow = (item / p.n_strips) * RL + rl;
        const int ocol = strip * kStrip;
        float2 acc[kStrip];
#pragma unroll
        for (int o = 0; o < kStrip; ++o) acc[o] = bias2;

        const unsigned char* xp = xs + (size_t)orow * row_bytes + ocol * PIXB + cp * (int)sizeof(pair_t);
        const wreg_t* wp = ws + cp;
        for (int kh = 0; kh < p.KH; ++kh) {
            wreg_t wr[K];
#pragma unroll
            for (int kw = 0; kw < K; ++kw) wr[kw] = wp[kw * CPL];
#pragma unroll
            for (int j = 0; j < kStrip + K - 1; ++j) {
                const pair_t xv = *reinterpret_cast<const pair_t*>(xp + j * PIXB);
                if constexpr (MIXED) {
#pragma unroll
                    for (int kw = 0; kw < K; ++kw) {
                        const int o = j - kw;
                        if (o >= 0 && o < kStrip) fma_mixed<T>(acc[o], xv, wr[kw]);
                    }
                } else {
                    const float2 xf = E::unpack(xv);
#pragma unroll
                    for (int kw = 0; kw < K; ++kw) {
                        const int o = j - kw;
                        if (o >= 0 && o < kStrip) ffma2(acc[o], xf, wr[kw]);
                    }
                }
            }
            xp += row_bytes;
            wp += K * CPL;
        }

        const int oh = th * p.TH + orow;
        if (oh < p.OH && c < p.C) {
            const int ow0 = tw * p.TWc + ocol;
            T* orow_ptr = static_cast<T*>(p.out) + (((size_t)b * p.OH + oh) * p.OW + ow0) * p.C + c;
#pragma unroll
            for (int o = 0; o < kStrip; ++o) {
                if (ow0 + o < p.OW) *reinterpret_cast<pair_t*>(orow_ptr + (size_t)o * p.C) = E::pack(acc[o]);
            }
        }
    }
}

// Picks the thread-block tile: as little padding waste at the image edges and as few idle warps
// as possible, then the larger tile (smaller halo share).  Returns false if nothing fits.
template <int CT>
inline bool plan_fwd_tile(int OH, int OW, int KH, int K, int esize, int wreg_bytes, int n_batch_ct, int sms,
                          TiledParams* p, int* smem_bytes) {
    constexpr int CPL = CT / 2, RL = 32 / CPL;
    const int pixb = CT * esize;
    double best = -1.0;
    for (int TH = RL; TH <= 64; TH += RL) {
        for (int TWc = kStrip; TWc <= 128; TWc += kStrip) {
            const int rows = TH + KH - 1;
            int cols = TWc + K - 1;
            if (RL > 1 && (cols % 2) == 0) cols++;
            if (rows > 256 || cols > 256) continue;
            const int smem = 128 + round_up(rows * cols * pixb, 128) + KH * K * CPL * wreg_bytes;
            if (smem > kSmemMax) continue;
            const int tiles_h = ceil_div(OH, TH), tiles_w = ceil_div(OW, TWc);
            const double eff_sp = (double)OH * OW / ((double)tiles_h * TH * tiles_w * TWc);
            const int items = (TH / RL) * (TWc / kStrip);
            const int warps = kFwdThreads / 32;
            const double eff_w = (double)items / (ceil_div(items, warps) * warps);
            const int per_sm = smem <= kSmemPerCta2 ? 2 : 1;
            const double waves = (double)tiles_h * tiles_w * n_batch_ct / ((double)per_sm * sms);
            const double eff_wave = waves / (double)(long long)(waves + 0.999999);
            const double halo = (double)TH * TWc / ((double)rows * cols);
            const double occ = per_sm == 2 ? 1.0 : 0.85;
            const double score = eff_sp * eff_w * eff_wave * occ * (0.9 + 0.1 * halo);
            if (score > best) {
                best = score;
                p->TH = TH; p->TWc = TWc; p->rows = rows; p->cols = cols;
                p->tiles_h = tiles_h; p->tiles_w = tiles_w;
                p->n_strips = TWc / kStrip; p->n_items = items;
                *smem_bytes = smem;
            }
        }
    }
    return best > 0.0;
}

template <typename T, int K, int CT, int MATH>
int launch_tiled(const TiledArgs& a) {
    constexpr bool MIXED = (MATH == 1) && (sizeof(T) == 2);
    using wreg_t = typename WReg<T, MIXED>::type;
    TiledParams p{};
    p.w = a.w; p.bias = a.bias; p.out = a.out;
    p.OH = a.OH; p.OW = a.OW; p.C = a.C;
    p.KH = a.KH; p.pad_h = a.pad_h; p.pad_w = a.pad_w; p.flip = a.flip;
    p.nct = ceil_div(a.C, CT);
    p.status = a.status;
    int smem = 0;
    if (!plan_fwd_tile<CT>(a.OH, a.OW, a.KH, K, (int)sizeof(T), (int)sizeof(wreg_t), a.B * p.nct, sm_count(), &p, &smem))
        return PDW_ERR_UNSUPPORTED;
    CUtensorMap tmap;
    int rc = make_nhwc_tensor_map(&tmap, a.in, a.dtype, a.B, a.H, a.W, a.C, CT, p.cols, p.rows);
    if (rc != PDW_OK) return rc;
    auto kern = dwconv_tiled_kernel<T, K, CT, MATH>;
    PDW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const long long blocks = (long long)p.tiles_h * p.tiles_w * a.B * p.nct;
    if (blocks > 0x7fffffffLL) return PDW_ERR_BAD_SHAPE;
    kern<<<(unsigned)blocks, kFwdThreads, smem, a.stream>>>(tmap, p);
    return check_launch();
}

// ---------------------------------------------------------------------------------------------
// Weight (+bias) gradient, first level.
//
// A persistent grid of S x nct thread blocks: block (s, ct) owns CT channels and walks over the
// spatial tiles s, s+S, ... of every image.  Per tile, TMA brings the grad_out tile and the x tile
// with its halo into one stage of a ring of NS shared-memory stages (the next tiles load while
// this one is consumed).  Warp kh owns filter row kh; a lane owns one channel pair and every RL-th
// row of the tile and keeps the K partial sums dW[kh, 0..K-1, pair] in registers for the whole
// kernel.  At the end the RL row lanes are folded with warp shuffles and the block writes its fp32
// partial sums once; wgrad_reduce_kernel adds the S partials per output in a fixed order.
// ---------------------------------------------------------------------------------------------
struct WgradArgs {
    const void* x;
    const void* gout;
    void* dw;
    void* dbias;       // may be null
    int B, H, W, C;    // x extents
    int OH, OW;        // grad_out extents
    int KH, KW;
    int pad_h, pad_w;
    int dtype;
    int out_fp32;
    void* workspace;
    size_t workspace_bytes;
    int32_t* status;
    cudaStream_t stream;
};

struct WgradParams {
    float* partial;      // [S][KH*K*C]
    float* partial_b;    // [S][C]
    int C, KH, pad_h, pad_w;
    int TH, TWc;
    int xrows, xcols, gcols;
    int tiles_w, tiles_h, n_tiles;   // n_tiles = B * tiles_h * tiles_w
    int nct, S, NS;
    int x_stage_bytes, g_stage_bytes;
    int want_bias;
    int32_t* status;
};

struct WgradPlan {
    WgradParams p;
    int smem_bytes;
    int threads;
    size_t workspace_bytes;
};

template <typename T, int K, int CT, int MATH>
__global__ void __launch_bounds__(K * 32, 1)
dwconv_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_g,
                    const WgradParams p) {
    using E = Elem<T>;
    using pair_t = typename E::pair_t;
    constexpr bool MIXED = (MATH == 1) && (sizeof(T) == 2);
    using greg_t = typename WReg<T, MIXED>::type;   // how a grad_out pair is held in registers
    constexpr int CPL = CT / 2;
    constexpr int RL = 32 / CPL;
    constexpr int PIXB = CT * (int)sizeof(T);
    constexpr int MAX_STAGES = 4;

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);   // MAX_STAGES barriers in the first 128 bytes
    unsigned char* stage0 = smem + 128;
    const int stage_bytes = p.x_stage_bytes + p.g_stage_bytes;

    const int ct = blockIdx.x % p.nct;
    const int s = blockIdx.x / p.nct;
    const int kh = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cp = lane % CPL, rl = lane / CPL;

    auto issue = [&](int tile, int st) {
        int t = tile;
        const int tw = t % p.tiles_w;  t /= p.tiles_w;
        const int th = t % p.tiles_h;
        const int b = t / p.tiles_h;
        unsigned char* xs = stage0 + (size_t)st * stage_bytes;
        unsigned char* gs = xs + p.x_stage_bytes;
        mbar_arrive_expect_tx(&full[st], (uint32_t)(p.xrows * p.xcols * PIXB + p.TH * p.gcols * PIXB));
        tma_load_4d(xs, &tmap_x, &full[st], ct * CT, tw * p.TWc - p.pad_w, th * p.TH - p.pad_h, b);
        tma_load_4d(gs, &tmap_g, &full[st], ct * CT, tw * p.TWc, th * p.TH, b);
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < MAX_STAGES; ++i) mbar_init(&full[i], 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 0; i < p.NS; ++i) {
            const int tile = s + i * p.S;
            if (tile < p.n_tiles) issue(tile, i);
        }
    }

    float2 acc[K];
#pragma unroll
    for (int kw = 0; kw < K; ++kw) acc[kw] = make_float2(0.f, 0.f);
    float2 bsum = make_float2(0.f, 0.f);
    const bool bias_warp = p.want_bias && (kh == (p.KH > 1 ? 1 : 0));
    const int xrow_bytes = p.xcols * PIXB, grow_bytes = p.gcols * PIXB;
    const int n_chunks = p.TWc / kStrip;

    int it = 0;
    for (int tile = s; tile < p.n_tiles; tile += p.S, ++it) {
        const int st = it % p.NS;
        const uint32_t phase = (uint32_t)(it / p.NS) & 1u;
        const bool arrived = mbar_wait_bounded(&full[st], phase, p.status);
        if (__syncthreads_or(!arrived)) return;

        const unsigned char* xs = stage0 + (size_t)st * stage_bytes;
        const unsigned char* gs = xs + p.x_stage_bytes;
        for (int r = rl; r < p.TH; r += RL) {
            const unsigned char* gp = gs + (size_t)r * grow_bytes + cp * (int)sizeof(pair_t);
            const unsigned char* xp = xs + (size_t)(r + kh) * xrow_bytes + cp * (int)sizeof(pair_t);
            for (int ch = 0; ch < n_chunks; ++ch) {
                greg_t g[kStrip];
#pragma unroll
                for (int o = 0; o < kStrip; ++o) {
                    const pair_t gv = *reinterpret_cast<const pair_t*>(gp + o * PIXB);
                    if constexpr (MIXED) g[o] = gv; else g[o] = E::unpack(gv);
                }
                if (bias_warp) {
#pragma unroll
                    for (int o = 0; o < kStrip; ++o) {
                        float2 gf;
                        if constexpr (MIXED) gf = E::unpack(g[o]); else gf = g[o];
                        bsum.x += gf.x; bsum.y += gf.y;
                    }
                }
#pragma unroll
                for (int j = 0; j < kStrip + K - 1; ++j) {
                    const pair_t xv = *reinterpret_cast<const pair_t*>(xp + j * PIXB);
                    if constexpr (MIXED) {
#pragma unroll
                        for (int kw = 0; kw < K; ++kw) {
                            const int o = j - kw;
                            if (o >= 0 && o < kStrip) fma_mixed<T>(acc[kw], g[o], xv);
                        }
                    } else {
                        const float2 xf = E::unpack(xv);
#pragma unroll
                        for (int kw = 0; kw < K; ++kw) {
                            const int o = j - kw;
                            if (o >= 0 && o < kStrip) ffma2(acc[kw], g[o], xf);
                        }
                    }
                }
                gp += kStrip * PIXB;
                xp += kStrip * PIXB;
            }
        }
        __syncthreads();   // every warp is done with this stage: refill it
        if (threadIdx.x == 0) {
            const int next = tile + p.NS * p.S;
            if (next < p.n_tiles) issue(next, st);
        }
    }

    // Fold the row lanes (warp shuffles), then one fp32 store per (block, tap, channel pair).
#pragma unroll
    for (int kw = 0; kw < K; ++kw) {
#pragma unroll
        for (int off = CPL; off < 32; off <<= 1) {
            acc[kw].x += __shfl_xor_sync(0xffffffffu, acc[kw].x, off);
            acc[kw].y += __shfl_xor_sync(0xffffffffu, acc[kw].y, off);
        }
    }
#pragma unroll
    for (int off = CPL; off < 32; off <<= 1) {
        bsum.x += __shfl_xor_sync(0xffffffffu, bsum.x, off);
        bsum.y += __shfl_xor_sync(0xffffffffu, bsum.y, off);
    }
    const int c = ct * CT + 2 * cp;
    if (rl == 0 && c < p.C) {
        float* dst = p.partial + (size_t)s * p.KH * K * p.C + (size_t)kh * K * p.C + c;
#pragma unroll
        for (int kw = 0; kw < K; ++kw) *reinterpret_cast<float2*>(dst + (size_t)kw * p.C) = acc[kw];
        if (bias_warp) *reinterpret_cast<float2*>(p.partial_b + (size_t)s * p.C + c) = bsum;
    }
}

// Second level: out[e] = sum_s partial[s][e], s ascending (fixed order => reproducible bits).
template <typename T>
__global__ void wgrad_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ partial_b,
                                    void* dw, void* dbias, int n_w, int n_b, int S, int out_fp32) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n_w) {
        float sum = 0.f;
        for (int s = 0; s < S; ++s) sum += partial[(size_t)s * n_w + e];
        if (out_fp32) static_cast<float*>(dw)[e] = sum; else static_cast<T*>(dw)[e] = Elem<T>::from_f(sum);
    } else if (e < n_w + n_b) {
        const int c = e - n_w;
        float sum = 0.f;
        for (int s = 0; s < S; ++s) sum += partial_b[(size_t)s * n_b + c];
        if (out_fp32) static_cast<float*>(dbias)[c] = sum; else static_cast<T*>(dbias)[c] = Elem<T>::from_f(sum);
    }
}

template <int CT>
inline bool plan_wgrad(int B, int OH, int OW, int C, int KH, int K, int esize, int sms, WgradPlan* plan) {
    constexpr int CPL = CT / 2, RL = 32 / CPL;
    const int pixb = CT * esize;
    WgradParams& p = plan->p;
    p.nct = ceil_div(C, CT);
    double best = -1.0;
    for (int TH = RL; TH <= 64; TH += RL) {
        for (int TWc = kStrip; TWc <= 128; TWc += kStrip) {
            const int xrows = TH + KH - 1;
            int xcols = TWc + K - 1, gcols = TWc;
            if (RL > 1 && (xcols % 2) == 0) xcols++;
            if (RL > 1 && (gcols % 2) == 0) gcols++;
            if (xrows > 256 || xcols > 256) continue;
            const int xb = round_up(xrows * xcols * pixb, 128), gb = round_up(TH * gcols * pixb, 128);
            int NS = (kSmemMax - 128) / (xb + gb);
            if (NS < 2) continue;
            if (NS > 3) NS = 3;
            const int tiles_h = ceil_div(OH, TH), tiles_w = ceil_div(OW, TWc);
            const long long n_tiles = (long long)B * tiles_h * tiles_w;
            if (n_tiles > 0x7fffffffLL) continue;
            int S = sms / p.nct;
            if (S < 1) S = 1;
            if (S > n_tiles) S = (int)n_tiles;
            const double eff_sp = (double)OH * OW / ((double)tiles_h * TH * tiles_w * TWc);
            const double per = (double)n_tiles / S;
            const double eff_bal = per / (double)(long long)(per + 0.999999);
            const double halo = (double)TH * TWc / ((double)xrows * xcols);
            const double score = eff_sp * eff_bal * (0.9 + 0.1 * halo) * (NS >= 3 ? 1.0 : 0.97);
            if (score > best) {
                best = score;
                p.TH = TH; p.TWc = TWc; p.xrows = xrows; p.xcols = xcols; p.gcols = gcols;
                p.tiles_h = tiles_h; p.tiles_w = tiles_w; p.n_tiles = (int)n_tiles;
                p.S = S; p.NS = NS; p.x_stage_bytes = xb; p.g_stage_bytes = gb;
                plan->smem_bytes = 128 + NS * (xb + gb);
            }
        }
    }
    if (best <= 0.0) return false;
    p.C = C; p.KH = KH;
    plan->threads = KH * 32;
    plan->workspace_bytes = (size_t)p.S * ((size_t)KH * K * C + C) * sizeof(float);
    return true;
}

template <typename T, int K, int CT, int MATH>
int launch_wgrad(const WgradArgs& a) {
    WgradPlan plan{};
    if (a.KH != K || !plan_wgrad<CT>(a.B, a.OH, a.OW, a.C, a.KH, K, (int)sizeof(T), sm_count(), &plan))
        return PDW_ERR_UNSUPPORTED;
    if (a.workspace == nullptr || a.workspace_bytes < plan.workspace_bytes) return PDW_ERR_WORKSPACE;
    WgradParams& p = plan.p;
    p.partial = static_cast<float*>(a.workspace);
    p.partial_b = p.partial + (size_t)p.S * a.KH * K * a.C;
    p.pad_h = a.pad_h; p.pad_w = a.pad_w;
    p.want_bias = a.dbias != nullptr;
    p.status = a.status;
    CUtensorMap tx, tg;
    int rc = make_nhwc_tensor_map(&tx, a.x, a.dtype, a.B, a.H, a.W, a.C, CT, p.xcols, p.xrows);
    if (rc != PDW_OK) return rc;
    rc = make_nhwc_tensor_map(&tg, a.gout, a.dtype, a.B, a.OH, a.OW, a.C, CT, p.gcols, p.TH);
    if (rc != PDW_OK) return rc;
    auto kern = dwconv_wgrad_kernel<T, K, CT, MATH>;
    PDW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem_bytes));
    kern<<<p.S * p.nct, plan.threads, plan.smem_bytes, a.stream>>>(tx, tg, p);
    rc = check_launch();
    if (rc != PDW_OK) return rc;
    const int n_w = a.KH * K * a.C, n_b = p.want_bias ? a.C : 0;
    wgrad_reduce_kernel<T><<<ceil_div(n_w + n_b, 256), 256, 0, a.stream>>>(p.partial, p.partial_b, a.dw, a.dbias, n_w,
                                                                            n_b, p.S, a.out_fp32);
    return check_launch();
}

// Per-K entry points, one translation unit each (dwconv_k.cu compiled with -DPDW_K=<K>).
typedef int (*tiled_launch_fn)(const TiledArgs&);
typedef int (*wgrad_launch_fn)(const WgradArgs&);
typedef size_t (*wgrad_ws_fn)(int B, int OH, int OW, int C, int KH, int dtype);
struct KernelSet {
    int k;
    tiled_launch_fn tiled;
    wgrad_launch_fn wgrad;
    wgrad_ws_fn wgrad_workspace;
};
const KernelSet* find_kernel_set(int kw);

}  // namespace pdw
