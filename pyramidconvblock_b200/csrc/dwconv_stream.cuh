// Streaming variant of the tiled depthwise convolution for 16-bit tensors (forward and input
// gradient): one persistent thread block per SM, 16 compute warps and one producer warp.
//
// The producer warp (one lane) keeps a ring of NS shared-memory stages full: for each tile of the
// block's tile list it waits until every compute warp has left the stage, then issues two TMA copies
// into it - the input tile with its halo and the tile's 16-channel slice of the filter ([KH][KW][16],
// exactly the layout the inner loop reads) - completing on the stage's "full" barrier.  Compute warps
// never meet at a block barrier: a warp waits for the tile, takes items (4 rows x 16 columns) from the
// stage's shared counter until none is left, tells the stage's "empty" barrier that it is gone and
// moves on to the next tile, so a fast warp runs ahead into the next tile while slow ones finish.
// For the input gradient the filter is read back to front instead of being mirrored while staged.
#pragma once

#include "dwconv_tiled.cuh"

namespace pdw {

constexpr int kStreamWarps = 16;                         // compute warps
constexpr int kStreamThreads = (kStreamWarps + 1) * 32;  // + producer warp
constexpr int kStreamStagesMax = 4;

struct StreamParams {
    const void* bias;
    void* out;
    int H, W;             // input extents
    int OH, OW, C;
    int KH, pad_h, pad_w;
    int TH, TWc, rows, cols;
    int x_bytes, w_bytes, stage_bytes, NS;
    int tiles_w, tiles_h, n_spatial, nct, n_tiles;
    int n_strips, n_row_groups;
    int32_t* status;
};

template <typename T, int K, bool FLIP>
__global__ void __launch_bounds__(kStreamThreads, 1)
dwconv_stream_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                     const StreamParams p) {
    using E = Elem<T>;
    constexpr int CT = 16, CPL = 8, RL = 4;
    constexpr int PIXB = CT * (int)sizeof(T);
    static_assert(sizeof(T) == 2, "streaming kernel is for 16-bit tensors");

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);              // [kStreamStagesMax]
    uint64_t* empty = full + kStreamStagesMax;                       // [kStreamStagesMax]
    int* next_item = reinterpret_cast<int*>(empty + kStreamStagesMax);   // [kStreamStagesMax]
    unsigned char* stage0 = smem + 128;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t_begin = (int)((long long)blockIdx.x * p.n_tiles / gridDim.x);
    const int t_end = (int)((long long)(blockIdx.x + 1) * p.n_tiles / gridDim.x);
    const int my_tiles = t_end - t_begin;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStreamStagesMax; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kStreamWarps);
            next_item[i] = 0;
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == kStreamWarps) {
        // ---- producer ----
        if (lane == 0) {
            for (int k = 0; k < my_tiles; ++k) {
                const int st = k % p.NS;
                if (k >= p.NS) {
                    if (!mbar_wait_bounded(&empty[st], (uint32_t)(k / p.NS - 1) & 1u, p.status)) break;
                    next_item[st] = 0;     // every compute warp has left the stage
                }
                const int tile = t_begin + k;
                const int ct = tile / p.n_spatial;
                int t = tile - ct * p.n_spatial;
                const int tw = t % p.tiles_w;  t /= p.tiles_w;
                const int th = t % p.tiles_h;
                const int b = t / p.tiles_h;
                unsigned char* xs = stage0 + (size_t)st * p.stage_bytes;
                mbar_arrive_expect_tx(&full[st], (uint32_t)(p.x_bytes + p.w_bytes));
                tma_load_4d(xs, &tmap_x, &full[st], ct * CT, tw * p.TWc - p.pad_w, th * p.TH - p.pad_h, b);
                tma_load_4d(xs + round_up(p.x_bytes, 128), &tmap_w, &full[st], ct * CT, 0, 0, 0);
            }
        }
        return;
    }

    // ---- compute warps ----
    const int cp = lane % CPL, rl = lane / CPL;
    const int row_bytes = p.cols * PIXB;
    for (int k = 0; k < my_tiles; ++k) {
        const int st = k % p.NS;
        if (!mbar_wait_bounded(&full[st], (uint32_t)(k / p.NS) & 1u, p.status)) return;
        const int tile = t_begin + k;
        const int ct = tile / p.n_spatial;
        int t = tile - ct * p.n_spatial;
        const int tw = t % p.tiles_w;  t /= p.tiles_w;
        const int th = t % p.tiles_h;
        const int b = t / p.tiles_h;
        const int c = ct * CT + 2 * cp;
        const unsigned char* xs = stage0 + (size_t)st * p.stage_bytes;
        const uint32_t* ws = reinterpret_cast<const uint32_t*>(xs + round_up(p.x_bytes, 128));

        const int oh_tile = th * p.TH, ow_tile = tw * p.TWc;
        const int groups = min(p.n_row_groups, (p.OH - oh_tile + RL - 1) / RL);
        const int strips = min(p.n_strips, (p.OW - ow_tile + kStrip - 1) / kStrip);
        const int n_items = groups * strips;
        float2 bias2 = make_float2(0.f, 0.f);
        if (p.bias != nullptr && c < p.C)
            bias2 = E::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(p.bias) + c));

        for (;;) {
            int item = 0;
            if (lane == 0) item = atomicAdd(&next_item[st], 1);
            item = __shfl_sync(0xffffffffu, item, 0);
            if (item >= n_items) break;
            const int strip = item % strips;
            const int grp = item / strips;
            const int orow = grp * RL + rl;
            const int ocol = strip * kStrip;
            float2 acc[kStrip];
#pragma unroll
            for (int o = 0; o < kStrip; ++o) acc[o] = bias2;

            const int oh_first = oh_tile + grp * RL;
            const int kh_lo = max(0, p.pad_h - (oh_first + RL - 1));
            const int kh_hi = min(p.KH, p.H + p.pad_h - oh_first);
            const unsigned char* xp = xs + (size_t)(orow + kh_lo) * row_bytes + ocol * PIXB + cp * 4;
            // filter row kh of the (possibly mirrored) filter
            const uint32_t* wp = ws + cp + (FLIP ? (p.KH - 1 - kh_lo) : kh_lo) * K * CPL;
            for (int kh = kh_lo; kh < kh_hi; ++kh) {
                uint32_t wr[K];
#pragma unroll
                for (int kw = 0; kw < K; ++kw) wr[kw] = wp[(FLIP ? (K - 1 - kw) : kw) * CPL];
#pragma unroll
                for (int j = 0; j < kStrip + K - 1; ++j) {
                    const uint32_t xv = *reinterpret_cast<const uint32_t*>(xp + j * PIXB);
#pragma unroll
                    for (int kw = 0; kw < K; ++kw) {
                        const int o = j - kw;
                        if (o >= 0 && o < kStrip) fma_mixed<T>(acc[o], xv, wr[kw]);
                    }
                }
                xp += row_bytes;
                wp += FLIP ? -K * CPL : K * CPL;
            }

            const int oh = oh_tile + orow;
            if (oh < p.OH && c < p.C) {
                const int ow0 = ow_tile + ocol;
                T* orow_ptr = static_cast<T*>(p.out) + (((size_t)b * p.OH + oh) * p.OW + ow0) * p.C + c;
#pragma unroll
                for (int o = 0; o < kStrip; ++o) {
                    if (ow0 + o < p.OW) *reinterpret_cast<uint32_t*>(orow_ptr + (size_t)o * p.C) = E::pack(acc[o]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);     // this warp has left the stage
    }
}

// Tile for the streaming kernel: 32x32 when two stages of it fit, else the first smaller shape of the
// preference list that does.
inline bool plan_stream(int B, int OH, int OW, int C, int KH, int K, int esize, int sms, StreamParams* p,
                        int* smem_bytes, int* grid) {
    constexpr int CT = 16, RL = 4;
    const int pixb = CT * esize;
    const int force_th = tuning(3), force_tw = tuning(4);
    for (const TileShape& ts : kTilePreference) {
        const int TH = (force_th && force_tw) ? force_th : ts.th, TWc = (force_th && force_tw) ? force_tw : ts.tw;
        if (TH % RL != 0 || TWc % kStrip != 0) continue;
        const int rows = TH + KH - 1;
        int cols = TWc + K - 1;
        if (cols % 2 == 0) cols++;
        if (rows > 256 || cols > 256) continue;
        const int x_bytes = rows * cols * pixb, w_bytes = KH * K * CT * esize;
        const int stage = round_up(x_bytes, 128) + round_up(w_bytes, 128);
        int NS = (kSmemMax - 128) / stage;
        if (NS < 2) continue;
        if (NS > 3) NS = 3;
        const int tiles_h = ceil_div(OH, TH), tiles_w = ceil_div(OW, TWc);
        const long long n_spatial = (long long)B * tiles_h * tiles_w;
        const int nct = ceil_div(C, CT);
        if (n_spatial * nct > 0x7fffffffLL) continue;
        p->TH = TH; p->TWc = TWc; p->rows = rows; p->cols = cols;
        p->x_bytes = x_bytes; p->w_bytes = w_bytes; p->stage_bytes = stage; p->NS = NS;
        p->tiles_h = tiles_h; p->tiles_w = tiles_w; p->n_spatial = (int)n_spatial; p->nct = nct;
        p->n_tiles = (int)(n_spatial * nct);
        p->n_strips = TWc / kStrip; p->n_row_groups = TH / RL;
        *smem_bytes = 128 + NS * stage;
        *grid = p->n_tiles < sms ? p->n_tiles : sms;
        return true;
    }
    return false;
}

template <typename T, int K>
int launch_stream(const TiledArgs& a) {
    StreamParams p{};
    int smem = 0, grid = 0;
    if (!plan_stream(a.B, a.OH, a.OW, a.C, a.KH, K, (int)sizeof(T), sm_count(), &p, &smem, &grid))
        return PDW_ERR_UNSUPPORTED;
    p.bias = a.bias; p.out = a.out;
    p.H = a.H; p.W = a.W; p.OH = a.OH; p.OW = a.OW; p.C = a.C;
    p.KH = a.KH; p.pad_h = a.pad_h; p.pad_w = a.pad_w;
    p.status = a.status;
    CUtensorMap tx, tw;
    int rc = make_nhwc_tensor_map(&tx, a.in, a.dtype, a.B, a.H, a.W, a.C, 16, p.cols, p.rows);
    if (rc != PDW_OK) return rc;
    rc = make_nhwc_tensor_map(&tw, a.w, a.dtype, 1, a.KH, K, a.C, 16, K, a.KH);   // filter as a [1,KH,KW,C] image
    if (rc != PDW_OK) return rc;
    if (a.flip) {
        auto kern = dwconv_stream_kernel<T, K, true>;
        PDW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kern<<<grid, kStreamThreads, smem, a.stream>>>(tx, tw, p);
    } else {
        auto kern = dwconv_stream_kernel<T, K, false>;
        PDW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kern<<<grid, kStreamThreads, smem, a.stream>>>(tx, tw, p);
    }
    return check_launch();
}

}  // namespace pdw
