// Host-only check of the tile planners of the convolution kernels: for a grid of image sizes, filter
// widths, element sizes and batch sizes the chosen tiles must satisfy what the kernels and the TMA
// descriptors need.  Compiled and run by tests/test_planner_host.py; no GPU is touched.
#include <cstdio>

#include "../pyramidconvblock_b200/csrc/dwconv_tiled.cuh"

namespace pdw {
thread_local int g_last_cuda_error = 0;
static int g_probe_tuning[10] = {1, 16, 0, 0, 0, 0, 0, 0, 0, 0};
int tuning(int key) { return g_probe_tuning[key]; }
int sm_count() { return 148; }
int make_nhwc_tensor_map(CUtensorMap*, const void*, int, int, int, int, int, int, int, int) { return 0; }
}  // namespace pdw

using namespace pdw;

static long long g_cases = 0, g_failures = 0;
#define EXPECT(cond, ...)                                  \
    do {                                                   \
        if (!(cond)) {                                     \
            if (g_failures < 20) { std::printf("FAIL %s: ", #cond); std::printf(__VA_ARGS__); std::printf("\n"); } \
            ++g_failures;                                  \
        }                                                  \
    } while (0)

template <int K>
static void check_one(int OH, int OW, int B, int C, int esize) {
    constexpr int CT = 16, RL = 4;
    const int nct = (C + CT - 1) / CT;
    const int wreg = esize == 2 ? 4 : 8;
    TiledParams p{};
    int smem = 0;
    const bool ok = plan_fwd_tile<CT>(OH, OW, K, K, esize, wreg, B * nct, 148, &p, &smem);
    ++g_cases;
    EXPECT(ok, "fwd OH=%d OW=%d K=%d B=%d C=%d es=%d", OH, OW, K, B, C, esize);
    if (ok) {
        EXPECT(p.TH > 0 && p.TH % RL == 0 && p.TWc > 0 && p.TWc % kStrip == 0, "tile %dx%d", p.TH, p.TWc);
        EXPECT(p.rows == p.TH + K - 1 && p.rows <= 256, "rows %d", p.rows);
        EXPECT(p.cols >= p.TWc + K - 1 && p.cols <= p.TWc + K && p.cols <= 256, "cols %d", p.cols);
        EXPECT(smem > 0 && smem <= kSmemMax, "smem %d", smem);
        EXPECT(smem >= 128 + p.rows * p.cols * CT * esize + K * K * (CT / 2) * wreg, "smem %d too small", smem);
        EXPECT(p.tiles_h * p.TH >= OH && (p.tiles_h - 1) * p.TH < OH, "tiles_h %d TH %d OH %d", p.tiles_h, p.TH, OH);
        EXPECT(p.tiles_w * p.TWc >= OW && (p.tiles_w - 1) * p.TWc < OW, "tiles_w %d TW %d OW %d", p.tiles_w, p.TWc, OW);
        EXPECT(p.n_strips == p.TWc / kStrip && p.n_items == (p.TH / RL) * p.n_strips, "items %d", p.n_items);
    }
    WgradPlan wp{};
    const bool okw = plan_wgrad<CT, K>(B, OH, OW, C, K, esize, 148, &wp);
    ++g_cases;
    if (okw) {   // the planner may decline (the entry point then uses the untiled kernel)
        const WgradParams& q = wp.p;
        EXPECT(q.TH % RL == 0 && q.TWc % kStrip == 0, "wgrad tile %dx%d", q.TH, q.TWc);
        EXPECT(q.xrows == q.TH + K - 1 && q.xrows <= 256 && q.xcols <= 256 && q.xcols >= q.TWc + K - 1, "x box %dx%d", q.xrows, q.xcols);
        EXPECT(q.gcols >= q.TWc && q.gcols <= 256, "g cols %d", q.gcols);
        EXPECT(q.NS >= 2 && q.NS <= 4, "stages %d", q.NS);
        EXPECT(wp.smem_bytes <= kSmemMax && wp.smem_bytes == 128 + q.NS * (q.x_stage_bytes + q.g_stage_bytes), "smem %d", wp.smem_bytes);
        EXPECT(q.x_stage_bytes >= q.xrows * q.xcols * CT * esize && q.g_stage_bytes >= q.TH * q.gcols * CT * esize, "stage bytes");
        EXPECT(q.x_stage_bytes % 128 == 0 && q.g_stage_bytes % 128 == 0, "stage alignment");
        EXPECT(q.S >= 1 && (long long)q.S <= (long long)q.n_tiles && q.S * q.nct <= 148 + q.nct, "S %d", q.S);
        EXPECT(q.n_tiles == B * q.tiles_h * q.tiles_w, "n_tiles %d", q.n_tiles);
        EXPECT(wp.workspace_bytes == (size_t)q.S * ((size_t)K * K * C + C) * sizeof(float), "workspace");
        // the block-level reduction of the shared filter row reuses the first stage
        EXPECT((size_t)(wp.threads / 32) * K * (CT / 2) * sizeof(float2) <= (size_t)q.x_stage_bytes + q.g_stage_bytes, "reduction scratch");
    }
}

template <int K>
static void sweep() {
    const int sizes[] = {1, 2, 3, 4, 7, 15, 16, 17, 31, 32, 33, 40, 47, 48, 49, 63, 64, 65, 95, 96, 97, 100, 127, 128, 129, 192, 224, 255, 256, 300, 512};
    const int batches[] = {1, 2, 16, 128};
    const int chans[] = {8, 16, 24, 256, 512};
    for (int generic = 0; generic < 2; ++generic) {
        g_probe_tuning[8] = generic;
        for (int oh : sizes) for (int ow : sizes) for (int b : batches) for (int c : chans) {
            check_one<K>(oh, ow, b, c, 2);
            if (c % 4 == 0 && b <= 16) check_one<K>(oh, ow, b, c, 4);
        }
    }
    g_probe_tuning[8] = 0;
}

int main() {
    sweep<3>(); sweep<5>(); sweep<7>(); sweep<9>(); sweep<11>(); sweep<13>(); sweep<15>(); sweep<17>();
    std::printf("%lld cases, %lld failures\n", g_cases, g_failures);
    return g_failures == 0 ? 0 : 1;
}
