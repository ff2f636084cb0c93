// Convolutions whose whole GEMM K extent (taps x padded input channels) fits one pipeline stage:
// the first layer of an image network (3 channels -> cp = 4, 3x3 -> K = 36).  Included by conv.cu.
//
// The general gather kernel spends most of such a layer on per-CTA fixed costs (barrier and TMEM
// setup, index divisions, an epilogue nothing overlaps) for two K slabs of work per tile.  Here a
// CTA is persistent: it keeps the weights in shared memory, walks over pixel tiles, and splits its
// nine warps by role so that the gather of tile i+1, the MMAs of tile i and the store of tile i-1
// run at the same time:
//   warps 0-3  producers: thread p owns tile row p (one output pixel) and copies its receptive
//              field, one 16-byte cell per (tap, 4 channels), into a K-major A stage
//   warps 4-7  epilogue: TMEM -> shared memory -> coalesced global stores (+bias, activation)
//   warp 8     allocates TMEM (two accumulators) and issues the MMAs
#pragma once

namespace {

constexpr int THIN_THREADS = 288;
constexpr int THIN_MAX_CELLS = 32;     // K <= 128
constexpr int THIN_MAX_STAGES = 4;

// Division by a run-time constant as multiply-high and shift (round-up method; exact for dividends
// below 2^31): the producers turn a pixel index into (image, row, column) once per tile.
struct FastDiv {
    uint32_t mul, shr, d;
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f = {0u, 0u, d};
    if (d > 1) {
        uint32_t lg = 0;
        while ((1ull << lg) < d) ++lg;
        const uint32_t p = 31 + lg;
        f.mul = (uint32_t)(((1ull << p) + d - 1) / d);
        f.shr = p - 32;
    }
    return f;
}
__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv &f) { return f.d == 1 ? n : __umulhi(n, f.mul) >> f.shr; }

struct ThinArgs {
    ConvGeom g;
    FastDiv div_ohw, div_ow;
    const float *x, *w, *bias;
    const float *stat_shift;   // batch-norm statistics of the output (see ConvArgs)
    float *stat_partial;
    float *y;
    int act, bn, n_rows, n_cols, out_ld;
    int cells;            // valid 16-byte K cells of a row (K / 4)
    int ksteps;           // MMAs per tile (K / 8 rounded up)
    int tiles, stages, tmem_cols;
    int *status;
    unsigned long long *span;   // profiling: first CTA entry / last CTA exit (null: off)
};

struct ThinCtl {
    unsigned long long full[THIN_MAX_STAGES], empty[THIN_MAX_STAGES];
    unsigned long long acc_full[2], acc_empty[2], weights, stat_bar;
    uint32_t tmem_base;
    int abort_flag;
    int4 ctab[THIN_MAX_CELLS];   // cell -> {row tap, column tap, element offset from the receptive field's corner, 0}
};

__global__ void __launch_bounds__(THIN_THREADS, 2) conv_fprop_thin_kernel(const ThinArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ ThinCtl ctl;
    span_begin(a.span);
    const ConvGeom &g = a.g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bn = a.bn;
    const int kcells = 2 * a.ksteps;                       // cells per row including the zero padding
    const uint32_t b_bytes = (uint32_t)kcells * bn * 16;
    const uint32_t a_bytes = (uint32_t)kcells * BM * 16;
    unsigned char *smem_b = smem;
    unsigned char *smem_a = smem + b_bytes;
    float *staging = reinterpret_cast<float *>(smem_a + (size_t)a.stages * a_bytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 128);
            mbar_init(smem_u32(&ctl.empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl.acc_full[b]), 1);
            mbar_init(smem_u32(&ctl.acc_empty[b]), 4);
        }
        mbar_init(smem_u32(&ctl.weights), 128);
        mbar_init(smem_u32(&ctl.stat_bar), 4);
        ctl.abort_flag = 0;
        fence_barrier_init();
    }
    if (threadIdx.x < THIN_MAX_CELLS) {
        const int k = threadIdx.x * 4, tap = k / g.cp;
        ctl.ctab[threadIdx.x] = make_int4(tap / g.S, tap % g.S, ((tap / g.S) * g.W + tap % g.S) * g.cp + k - tap * g.cp, 0);
    }
    // the padding cells (K rounded up to whole MMAs) of the weights and of every stage stay zero
    {
        const int pad_cells = kcells - a.cells;
        for (int i = threadIdx.x; i < pad_cells * (bn + a.stages * BM); i += THIN_THREADS) {
            const int kc = a.cells + i / (bn + a.stages * BM), r = i % (bn + a.stages * BM);
            unsigned char *dst = r < bn ? smem_b + (size_t)kc * (bn * 16) + r * 16
                                        : smem_a + (size_t)((r - bn) / BM) * a_bytes + (size_t)kc * (BM * 16) + ((r - bn) % BM) * 16;
            *reinterpret_cast<float4 *>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        fence_proxy_async_smem();
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(&ctl.tmem_base), a.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = ctl.tmem_base;
    pdl_enter();   // everything above touched only shared memory, TMEM and kernel parameters
    volatile int *abort_flag = &ctl.abort_flag;

    if (warp >= 4 && warp < 8) {
        // weights: K-major rows = filters, cell (row, kc) at kc * (bn * 16) + row * 16 (rows past the last
        // filter are zero).  The epilogue warps copy them while the producers already gather the first tile.
        for (int i = threadIdx.x - 128; i < bn * a.cells; i += 128) {
            const int row = i / a.cells, kc = i - row * a.cells;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < g.K) v = ldg4(a.w + (size_t)row * (a.cells * 4) + kc * 4);
            *reinterpret_cast<float4 *>(smem_b + (size_t)kc * (bn * 16) + row * 16) = v;
        }
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&ctl.weights));
    }

    if (warp < 4) {
        // ------------------------------------------------------------------ producers
        const int p = threadIdx.x;
        int it = 0;
        for (int tile = blockIdx.x; tile < a.tiles; tile += gridDim.x, ++it) {
            const int s = it % a.stages;
            const uint32_t phase = (it / a.stages) & 1;
            const uint32_t m = (uint32_t)(tile * BM + p);
            const bool valid = m < (uint32_t)a.n_rows;
            const uint32_t n = fast_div(m, a.div_ohw), rem = m - n * (uint32_t)(g.OH * g.OW);
            const uint32_t oh = fast_div(rem, a.div_ow), ow = rem - oh * (uint32_t)g.OW;
            const int iy0 = (int)oh * g.sy - g.pad, ix0 = (int)ow * g.sx - g.pad;
            // element offset of the receptive field's corner (may lie outside the image; int32: checked on the host)
            const float *corner = a.x + (((int)n * g.H + iy0) * g.W + ix0) * g.cp;
            unsigned char *dst = smem_a + (size_t)s * a_bytes + p * 16;
            bool ok = true;
            for (int c0 = 0; c0 < a.cells && ok; c0 += 16) {
                float4 v[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (c0 + u < a.cells) {
                        const int4 e = ctl.ctab[c0 + u];
                        if (valid && (unsigned)(iy0 + e.x) < (unsigned)g.H && (unsigned)(ix0 + e.y) < (unsigned)g.W) v[u] = ldg4(corner + e.z);
                    }
                }
                if (c0 == 0) ok = mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag);
                if (ok) {
#pragma unroll
                    for (int u = 0; u < 16; ++u)
                        if (c0 + u < a.cells) *reinterpret_cast<float4 *>(dst + (size_t)(c0 + u) * (BM * 16)) = v[u];
                }
            }
            if (!ok) break;
            fence_proxy_async_smem();
            mbar_arrive(smem_u32(&ctl.full[s]));
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ epilogue
        const int ew = warp - 4;   // TMEM lane quarter = warp id modulo 4
        StatAcc st;
        stat_init(st, a.stat_partial ? a.stat_shift : nullptr);
        bool all_ready = true;
        int it = 0;
        for (int tile = blockIdx.x; tile < a.tiles; tile += gridDim.x, ++it) {
            const int b = it & 1;
            bool ready = mbar_wait(smem_u32(&ctl.acc_full[b]), (uint32_t)(it >> 1) & 1, abort_flag);
            ready = __all_sync(0xffffffffu, ready);
            if (!ready) { all_ready = false; break; }
            tc_fence_after_sync();
            const int m0 = tile * BM;
            store_accumulator<true>(staging, tmem + (uint32_t)(b * bn), true, ew, lane, bn, a.y + (size_t)m0 * a.out_ld,
                                    (size_t)a.out_ld, a.n_rows - m0, 0, a.n_cols, a.bias, a.act, 1, 1, 0, &st);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl.acc_empty[b]));
        }
        if (st.shift && all_ready)
            stats_commit(staging, st, ew, lane, bn, a.stat_partial + (size_t)blockIdx.x * 2 * a.out_ld, a.out_ld, a.n_cols, &ctl.stat_bar,
                         abort_flag);
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const uint32_t idesc = make_idesc_tf32(BM, bn, 0, 0);
        const uint64_t da0 = make_desc(smem_u32(smem_a), BM * 16, 128, LAYOUT_NONE);
        const uint64_t db0 = make_desc(smem_u32(smem_b), bn * 16, 128, LAYOUT_NONE);
        const uint64_t a_step = (uint64_t)((2 * BM * 16) >> 4), b_step = (uint64_t)((2 * bn * 16) >> 4);
        int it = 0;
        bool have_weights = mbar_wait(smem_u32(&ctl.weights), 0, abort_flag);
        for (int tile = blockIdx.x; have_weights && tile < a.tiles; tile += gridDim.x, ++it) {
            const int s = it % a.stages;
            const int b = it & 1;
            if (!mbar_wait(smem_u32(&ctl.acc_empty[b]), ((uint32_t)(it >> 1) & 1) ^ 1, abort_flag)) break;
            if (!mbar_wait(smem_u32(&ctl.full[s]), (uint32_t)(it / a.stages) & 1, abort_flag)) break;
            tc_fence_after_sync();
            const uint64_t st16 = (uint64_t)(((uint32_t)s * a_bytes) >> 4);
            for (int j = 0; j < a.ksteps; ++j)
                mma_tf32(tmem + (uint32_t)(b * bn), da0 + st16 + j * a_step, db0 + j * b_step, idesc, (uint32_t)(j > 0));
            mma_commit(smem_u32(&ctl.empty[s]));
            mma_commit(smem_u32(&ctl.acc_full[b]));
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) {
        tmem_dealloc(tmem, a.tmem_cols);
        if (lane == 0 && ctl.abort_flag && a.status) atomicOr(a.status, AET_STATUS_TIMEOUT);
    }
    span_end(a.span);
}

// Forward pass through the persistent thin-K kernel; 1 = not eligible.
int thin_fprop(aet_layer *l, const ConvArgs &a, double flops) {
    aet_context *ctx = l->ctx;
    const ConvGeom &g = a.g;
    if (ctx->conv_path != 0 || ctx->math == AET_MATH_3XTF32 || !ctx->opt[OPT_THIN] || l->groups > 1 || l->dilation > 1) return 1;
    if (tma_common_ok(l)) return 1;                                         // wide channel counts belong to the TMA kernels
    if (a.k_total > THIN_MAX_CELLS * 4) return 1;
    const int bn = round_up(a.n_cols, 16);
    if (bn > 128) return 1;                    // two accumulators of two co-resident CTAs share the 512 TMEM columns
    ThinArgs t = {};
    t.g = g; t.x = a.src_a; t.w = a.src_b; t.bias = a.bias; t.y = a.out; t.act = a.act;
    t.stat_shift = a.stat_shift; t.stat_partial = a.stat_partial;
    t.bn = bn; t.n_rows = a.n_rows; t.n_cols = a.n_cols; t.out_ld = a.out_ld;
    if ((double)g.N * g.H * g.W * g.cp >= 2147483648.0 || (double)a.n_rows >= 2147483648.0) return 1;   // 32-bit element offsets
    t.div_ohw = make_fastdiv((uint32_t)(g.OH * g.OW)); t.div_ow = make_fastdiv((uint32_t)g.OW);
    t.cells = a.k_total / 4; t.ksteps = (a.k_total + 7) / 8;
    t.tiles = (a.n_rows + BM - 1) / BM;
    t.tmem_cols = pow2_cols(2 * bn);
    t.status = ctx->status_dev;
    const size_t kcells = 2 * (size_t)t.ksteps;
    const size_t b_bytes = kcells * bn * 16, a_bytes = kcells * BM * 16, staging = (size_t)BM * (bn + 4) * 4;
    int stages = (int)((110 * 1024 - 1024 - b_bytes - staging) / a_bytes);   // two CTAs per SM when it fits
    if (stages < 2) stages = (int)((220 * 1024 - 1024 - b_bytes - staging) / a_bytes);
    if (stages > THIN_MAX_STAGES) stages = THIN_MAX_STAGES;
    if (stages < 2) return 1;
    t.stages = stages;
    const size_t smem_bytes = b_bytes + stages * a_bytes + staging + 1024;
    AET_TRY(ctx_smem_attr(ctx, conv_fprop_thin_kernel));
    const int resident = smem_bytes <= 110 * 1024 ? 2 : 1;
    int grid = ctx->sm_count * resident;
    if (grid > t.tiles) grid = t.tiles;
    if (a.stat_rows_out) *a.stat_rows_out = grid;
    LaunchScope scope(ctx, "conv_fprop_thin", 0, flops);
    t.span = ctx->span_ptr;
    launch_k(ctx->stream, grid, THIN_THREADS, smem_bytes, conv_fprop_thin_kernel, t);
    return aet_check_launch("conv_fprop_thin");
}


// ------------------------------------------------------------------------------------ weight gradient
// dW[filter][(tap, c)] = sum over output pixels of delta[pixel][filter] * patch[pixel][(tap, c)]: M = filters,
// N = taps x padded channels (<= 128), K = pixels, split over the grid (a CTA owns a run of 64-pixel
// stages and one accumulator; the partial tiles are summed by wgrad_reduce_kernel in a fixed order).
// The delta tile arrives by TMA in the MN-major swizzle; the patches are gathered, thread = (pixel, cells).
constexpr int THINW_PX = 64;          // pixels per stage (two 32-pixel MN-major slabs)
constexpr int THINW_MAX_STAGES = 4;

struct ThinWArgs {
    ConvGeom g;
    FastDiv div_ohw, div_ow;
    const float *x;
    float *partial;
    int bn, n_rows, n_cols, out_ld, cells;
    int pixels, stages_total, stages_per_split;
    int m_blocks;          // 32-filter blocks the TMA box brings (the MMA reads four; the rest are never stored)
    long long split_stride;
    int stages, tmem_cols;
    int *status;
    unsigned long long *span;   // profiling: first CTA entry / last CTA exit (null: off)
};

struct ThinWCtl {
    unsigned long long full[THINW_MAX_STAGES], empty[THINW_MAX_STAGES], accum;
    uint32_t tmem_base;
    int abort_flag;
    int4 ctab[THIN_MAX_CELLS];
};

__global__ void __launch_bounds__(NTHREADS, 2) conv_wgrad_thin_kernel(const __grid_constant__ CUtensorMap map_a, const ThinWArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ ThinWCtl ctl;
    span_begin(a.span);
    const ConvGeom &g = a.g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bn = a.bn;
    const uint32_t a_slab = 4 * 4096;                                  // M = 128: four 32-filter blocks of [32 k][128 B]
    const uint32_t b_slab = (uint32_t)((bn + 31) / 32) * 4096;
    const uint32_t a_bytes = 2 * a_slab, stage_bytes = a_bytes + 2 * b_slab;
    const int st_begin = blockIdx.x * a.stages_per_split;
    int st_end = st_begin + a.stages_per_split;
    if (st_end > a.stages_total) st_end = a.stages_total;
    const int nst = st_end > st_begin ? st_end - st_begin : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 129);   // 128 gather arrivals + the TMA issuer's expect_tx
            mbar_init(smem_u32(&ctl.empty[s]), 1);
        }
        mbar_init(smem_u32(&ctl.accum), 1);
        ctl.abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_a);
    }
    if (threadIdx.x < THIN_MAX_CELLS) {
        const int k = threadIdx.x * 4, tap = k / g.cp;
        ctl.ctab[threadIdx.x] = make_int4(tap / g.S, tap % g.S, ((tap / g.S) * g.W + tap % g.S) * g.cp + k - tap * g.cp, 0);
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(&ctl.tmem_base), a.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = ctl.tmem_base;
    pdl_enter();   // everything above touched only shared memory, TMEM and kernel parameters
    volatile int *abort_flag = &ctl.abort_flag;

    if (warp < 4) {
        // ------------------------------------------------------------------ producers
        const int px = threadIdx.x & (THINW_PX - 1);       // pixel of the stage
        const int cg = threadIdx.x / THINW_PX;             // first cell; the thread takes every second cell
        const int slab = px >> 5, kq = px & 31, k3 = kq & 3;
        const uint32_t kbase = (uint32_t)(kq >> 2) * 512u + (uint32_t)k3 * 128u;
        for (int it = 0; it < nst; ++it) {
            const int s = it % a.stages;
            const uint32_t phase = (it / a.stages) & 1;
            const int p0 = (st_begin + it) * THINW_PX;
            unsigned char *stage = smem + (size_t)s * stage_bytes;
            if (threadIdx.x == 0) {
                if (!mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag)) break;
                const uint32_t bar = smem_u32(&ctl.full[s]);
                mbar_arrive_expect_tx(bar, 2u * (uint32_t)a.m_blocks * 4096u);
                tma_load_3d(smem_u32(stage), &map_a, bar, 0, p0, 0);
                tma_load_3d(smem_u32(stage) + a_slab, &map_a, bar, 0, p0 + 32, 0);
            }
            const uint32_t p = (uint32_t)(p0 + px);
            const bool valid = p < (uint32_t)a.pixels;
            const uint32_t n = fast_div(p, a.div_ohw), rem = p - n * (uint32_t)(g.OH * g.OW);
            const uint32_t oh = fast_div(rem, a.div_ow), ow = rem - oh * (uint32_t)g.OW;
            const int iy0 = (int)oh * g.sy - g.pad, ix0 = (int)ow * g.sx - g.pad;
            const float *corner = a.x + (((int)n * g.H + iy0) * g.W + ix0) * g.cp;
            unsigned char *dst = stage + a_bytes + (size_t)slab * b_slab + kbase;
            bool ok = true, waited = threadIdx.x == 0;
            // every thread passes the empty barrier before it arrives on the full one, also with no cell to copy
            for (int c0 = cg; (c0 < a.cells || !waited) && ok; c0 += 16) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int cell = c0 + 2 * u;
                    v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (cell < a.cells) {
                        const int4 e = ctl.ctab[cell];
                        if (valid && (unsigned)(iy0 + e.x) < (unsigned)g.H && (unsigned)(ix0 + e.y) < (unsigned)g.W) v[u] = ldg4(corner + e.z);
                    }
                }
                if (!waited) { ok = mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag); waited = true; }
                if (ok) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int cell = c0 + 2 * u;
                        // mn_cell_offset(cell, kq) with the pixel's share (kbase) hoisted out of the stage loop
                        if (cell < a.cells)
                            *reinterpret_cast<float4 *>(dst + (uint32_t)(cell >> 3) * 4096u + (uint32_t)((((cell & 7) >> 1) ^ k3) * 32) + (uint32_t)(cell & 1) * 16u) = v[u];
                    }
                }
            }
            if (!ok) break;
            fence_proxy_async_smem();
            mbar_arrive(smem_u32(&ctl.full[s]));
        }
        // ------------------------------------------------------------------ epilogue
        bool ready = nst == 0 ? true : mbar_wait(smem_u32(&ctl.accum), 0, abort_flag);
        ready = __all_sync(0xffffffffu, ready);
        tc_fence_after_sync();
        if (ready)
            store_accumulator<false>(reinterpret_cast<float *>(smem), tmem, nst > 0, warp, lane, bn,
                                     a.partial + (size_t)blockIdx.x * a.split_stride, (size_t)a.out_ld, a.n_rows, 0, a.n_cols,
                                     nullptr, (int)AET_LINEAR);
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const uint32_t idesc = make_idesc_tf32(BM, bn, 1, 1);
        const uint32_t s0 = smem_u32(smem);
        const uint64_t da0 = make_desc(s0, 4096, 512, LAYOUT_SW128_32B);
        const uint64_t db0 = make_desc(s0 + a_bytes, 4096, 512, LAYOUT_SW128_32B);
        uint32_t accumulate = 0;
        for (int it = 0; it < nst; ++it) {
            const int s = it % a.stages;
            if (!mbar_wait(smem_u32(&ctl.full[s]), (uint32_t)(it / a.stages) & 1, abort_flag)) break;
            tc_fence_after_sync();
            const uint64_t st16 = (uint64_t)(((uint32_t)s * stage_bytes) >> 4);
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
                const uint64_t da = da0 + st16 + (uint64_t)((sl * a_slab) >> 4), db = db0 + st16 + (uint64_t)((sl * b_slab) >> 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    mma_tf32(tmem, da + j * 64, db + j * 64, idesc, accumulate);
                    accumulate = 1;
                }
            }
            mma_commit(smem_u32(&ctl.empty[s]));
        }
        mma_commit(smem_u32(&ctl.accum));
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) {
        tmem_dealloc(tmem, a.tmem_cols);
        if (lane == 0 && ctl.abort_flag && a.status) atomicOr(a.status, AET_STATUS_TIMEOUT);
    }
    span_end(a.span);
}

// Weight gradient through the thin-K kernel: fills `partial` (ctx scratch) with `*splits` tiles; 1 = not eligible.
int thin_wgrad(aet_layer *l, const ConvArgs &a, double flops, int *splits_out, float **partial_out) {
    aet_context *ctx = l->ctx;
    const ConvGeom &g = a.g;
    if (ctx->conv_path != 0 || ctx->math == AET_MATH_3XTF32 || !ctx->opt[OPT_THIN] || l->groups > 1 || l->dilation > 1) return 1;
    if (tma_common_ok(l)) return 1;                                         // wide channel counts belong to the TMA kernels
    if (a.n_cols > THIN_MAX_CELLS * 4 || g.K > BM) return 1;
    if (!(g.kp % 32 == 0 || g.kp < 32)) return 1;          // whole 32-filter blocks for the TMA box
    const int bn = round_up(a.n_cols, 16);
    ThinWArgs t = {};
    t.g = g; t.x = a.src_b; t.bn = bn; t.n_rows = a.n_rows; t.n_cols = a.n_cols; t.out_ld = a.out_ld;
    if ((double)g.N * g.H * g.W * g.cp >= 2147483648.0 || (double)a.k_total >= 2147483648.0 - 2 * THINW_PX) return 1;   // 32-bit element offsets
    t.div_ohw = make_fastdiv((uint32_t)(g.OH * g.OW)); t.div_ow = make_fastdiv((uint32_t)g.OW);
    t.cells = a.n_cols / 4;
    t.pixels = a.k_total;
    t.stages_total = (t.pixels + THINW_PX - 1) / THINW_PX;
    t.m_blocks = (g.kp + 31) / 32;
    const size_t stage = 2 * (size_t)(4 * 4096) + 2 * (size_t)((bn + 31) / 32) * 4096;
    int stages = (int)((110 * 1024 - 1024) / stage);
    const int resident = stages >= 2 ? 2 : 1;
    if (stages < 2) stages = (int)((220 * 1024 - 1024) / stage);
    if (stages > THINW_MAX_STAGES) stages = THINW_MAX_STAGES;
    if (stages < 2 || (size_t)stages * stage < (size_t)BM * (bn + 4) * 4) return 1;
    t.stages = stages;
    // one CTA per resident slot, but at least four stages of work each (the partial tiles cost a reduction pass)
    int splits = ctx->sm_count * resident;
    if (splits > t.stages_total / 4) splits = t.stages_total / 4;
    if (splits < 1) splits = 1;
    t.stages_per_split = (t.stages_total + splits - 1) / splits;
    splits = (t.stages_total + t.stages_per_split - 1) / t.stages_per_split;
    const size_t out_floats = (size_t)g.K * a.n_cols;
    t.split_stride = (long long)out_floats;
    float *partial = nullptr;
    AET_TRY(ctx_scratch(ctx, out_floats * splits * sizeof(float), &partial));
    t.partial = partial;
    t.tmem_cols = pow2_cols(bn);
    t.status = ctx->status_dev;
    const CUtensorMap *ma;
    {
        cuuint64_t dims[3] = {(cuuint64_t)(g.kp < 32 ? g.kp : 32), (cuuint64_t)t.pixels, (cuuint64_t)t.m_blocks};
        cuuint64_t str[2] = {(cuuint64_t)g.kp * 4, 128};
        cuuint32_t box[3] = {32, 32, (cuuint32_t)t.m_blocks};
        if (get_map(l, 12, a.src_a, 3, dims, str, box, true, &ma) != AET_OK) return 1;
    }
    const size_t smem_bytes = stage * stages + 1024;
    AET_TRY(ctx_smem_attr(ctx, conv_wgrad_thin_kernel));
    LaunchScope scope(ctx, "conv_wgrad_thin", 0, flops);
    t.span = ctx->span_ptr;
    launch_k(ctx->stream, splits, NTHREADS, smem_bytes, conv_wgrad_thin_kernel, *ma, t);
    *splits_out = splits;
    *partial_out = partial;
    return aet_check_launch("conv_wgrad_thin");
}


// Data gradient of a layer with at most 4 input channels (cp = 4): N = 4 is far below what an MMA tile can use (the
// general kernel pads it to 16 columns of a 128-row tile and spends its time gathering), and the work is small:
//     dx[n][h][w][c] = sum over taps (r, s) and filters k of  dy[n][h + pad - r][w + pad - s][k] * W[k][r][s][c]
// in exact FP32 on the CUDA cores.  Sixteen lanes share four neighbouring input pixels of one row: lane g takes the
// filters 4g..4g+3 (and every 64 further on), so the sixteen 16-byte loads of one dy pixel are one contiguous 256-byte
// read; per filter row the lanes load the S + 3 dy columns the four pixels touch and the row's S taps of weights once
// (from shared memory, laid out so that the lanes' reads do not collide) and every value feeds all the pixels that
// use it; the lanes' partial sums meet in a shuffle tree at the end.
struct NarrowDgradArgs {
    const float *dy, *w;
    float *dx;
    int N, H, W, K, OH, OW, R, pad, ys, xs;
    long long quads;   // groups of four pixels (W is a multiple of 4)
};
constexpr int NARROW_THREADS = 256, NARROW_LANES = 16, NARROW_QUADS = 2;   // 16 lane groups per block, 2 quads each
template <int S>
__global__ void __launch_bounds__(NARROW_THREADS) conv_dgrad_narrow_kernel(const NarrowDgradArgs a) {
    extern __shared__ float4 narrow_w[];
    const int taps = a.R * S;
    pdl_enter();
    // filter k of a tap sits at [tap][k % 4][k / 4]: the lanes of a group (consecutive k / 4) read consecutive 16-byte cells
    const int kq_count = a.K / 4;
    for (int i = threadIdx.x; i < taps * a.K; i += NARROW_THREADS) {
        const int tap = i / a.K, k = i - tap * a.K;
        narrow_w[(size_t)(tap * 4 + (k & 3)) * kq_count + (k >> 2)] = *reinterpret_cast<const float4 *>(a.w + ((size_t)k * taps + tap) * 4);
    }
    __syncthreads();
    const int g = threadIdx.x & (NARROW_LANES - 1), grp = threadIdx.x / NARROW_LANES;
    const long long base = ((long long)blockIdx.x * (NARROW_THREADS / NARROW_LANES) + grp) * NARROW_QUADS;
    constexpr int COLS = S + 3;
    for (int j = 0; j < NARROW_QUADS; ++j) {
        const long long quad = base + j;
        const bool live = quad < a.quads;          // uniform over the 16 lanes of a group; all 32 lanes reach the shuffles
        const long long p = (live ? quad : 0) * 4;
        const int w0 = (int)(p % a.W), h = (int)((p / a.W) % a.H), n = (int)(p / ((long long)a.W * a.H));
        float4 acc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 4 * g; k < a.K; k += 4 * NARROW_LANES) {
            for (int r = 0; r < a.R; ++r) {
                const int oh = h + a.pad - r;
                if (!live || oh < 0 || oh >= a.OH) continue;
                // column c is output column w0 + pad - (S - 1) + c; pixel i meets it through tap s = i + S - 1 - c
                float4 d[COLS];
                const float *row = a.dy + (size_t)((size_t)n * a.OH + oh) * a.OW * a.ys + k;
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
                    const int ow = w0 + a.pad - (S - 1) + c;
                    d[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (ow >= 0 && ow < a.OW) d[c] = __ldg(reinterpret_cast<const float4 *>(row + (size_t)ow * a.ys));
                }
                float4 wv[S][4];
#pragma unroll
                for (int t = 0; t < S; ++t) {
                    const float4 *wt = narrow_w + (size_t)(r * S + t) * a.K + (k >> 2);
#pragma unroll
                    for (int q = 0; q < 4; ++q) wv[t][q] = wt[q * kq_count];
                }
#pragma unroll
                for (int c = 0; c < COLS; ++c) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int t = i + S - 1 - c;
                        if (t < 0 || t >= S) continue;
                        const float4 v = d[c];
                        acc[i].x = fmaf(v.x, wv[t][0].x, acc[i].x); acc[i].y = fmaf(v.x, wv[t][0].y, acc[i].y); acc[i].z = fmaf(v.x, wv[t][0].z, acc[i].z); acc[i].w = fmaf(v.x, wv[t][0].w, acc[i].w);
                        acc[i].x = fmaf(v.y, wv[t][1].x, acc[i].x); acc[i].y = fmaf(v.y, wv[t][1].y, acc[i].y); acc[i].z = fmaf(v.y, wv[t][1].z, acc[i].z); acc[i].w = fmaf(v.y, wv[t][1].w, acc[i].w);
                        acc[i].x = fmaf(v.z, wv[t][2].x, acc[i].x); acc[i].y = fmaf(v.z, wv[t][2].y, acc[i].y); acc[i].z = fmaf(v.z, wv[t][2].z, acc[i].z); acc[i].w = fmaf(v.z, wv[t][2].w, acc[i].w);
                        acc[i].x = fmaf(v.w, wv[t][3].x, acc[i].x); acc[i].y = fmaf(v.w, wv[t][3].y, acc[i].y); acc[i].z = fmaf(v.w, wv[t][3].z, acc[i].z); acc[i].w = fmaf(v.w, wv[t][3].w, acc[i].w);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int o = NARROW_LANES / 2; o > 0; o >>= 1) {
                acc[i].x += __shfl_xor_sync(0xffffffffu, acc[i].x, o); acc[i].y += __shfl_xor_sync(0xffffffffu, acc[i].y, o);
                acc[i].z += __shfl_xor_sync(0xffffffffu, acc[i].z, o); acc[i].w += __shfl_xor_sync(0xffffffffu, acc[i].w, o);
            }
        }
        // lane i of the group stores pixel i
        if (live && g < 4) {
            const float4 v = g == 0 ? acc[0] : (g == 1 ? acc[1] : (g == 2 ? acc[2] : acc[3]));
            *reinterpret_cast<float4 *>(a.dx + (size_t)(p + g) * a.xs) = v;
        }
    }
}

template <int S>
static int narrow_dgrad_launch(aet_context *ctx, const NarrowDgradArgs &t, size_t smem, double flops) {
    AET_TRY(ctx_smem_attr(ctx, conv_dgrad_narrow_kernel<S>, 96 * 1024));
    const long long per_block = (NARROW_THREADS / NARROW_LANES) * NARROW_QUADS;
    LaunchScope scope(ctx, "conv_dgrad_narrow", 0, flops);
    launch_k(ctx->stream, (unsigned)((t.quads + per_block - 1) / per_block), NARROW_THREADS, smem, conv_dgrad_narrow_kernel<S>, t);
    return aet_check_launch("conv_dgrad_narrow");
}

// Data gradient through the narrow-channel kernel; 1 = not eligible.
int narrow_dgrad(aet_layer *l, const ConvArgs &a, double flops) {
    aet_context *ctx = l->ctx;
    const ConvGeom &g = a.g;
    if (ctx->conv_path != 0 || !ctx->opt[OPT_THIN] || l->groups > 1 || g.dil > 1 || g.sx != 1 || g.sy != 1) return 1;
    if (g.cp != 4 || g.xs != 4 || g.kp % 4 || g.K != g.kp || g.W % 4) return 1;
    if (g.S != 3 && g.S != 5) return 1;
    const size_t smem = (size_t)g.R * g.S * g.kp * sizeof(float4);
    if (smem > 96 * 1024) return 1;
    NarrowDgradArgs t = {};
    t.dy = a.src_a; t.w = a.src_b; t.dx = a.out;
    t.N = g.N; t.H = g.H; t.W = g.W; t.K = g.kp; t.OH = g.OH; t.OW = g.OW; t.R = g.R; t.pad = g.pad; t.ys = g.ys; t.xs = g.xs;
    t.quads = (long long)g.N * g.H * g.W / 4;
    return g.S == 3 ? narrow_dgrad_launch<3>(ctx, t, smem, flops) : narrow_dgrad_launch<5>(ctx, t, smem, flops);
}

}  // namespace
