// Row-sharing TMA kernels (included by conv.cu after conv_tma.cuh).
//
// The plain TMA kernels fetch one operand tile per filter tap, so a 3x3 convolution pulls every
// activation through the L2 -> SM path nine times; measured, that path (about 25 bytes per clock and
// SM) and not the tensor pipe bounds them.  Taps that differ only in their ROW offset read the
// same pixels shifted by whole image rows, and whole image rows are whole swizzle periods of the
// shared-memory tile.  So one copy of `rows + R - 1` image rows serves all R row taps: the MMA
// descriptor of tap r simply starts r image rows further down.  Column taps still need their own
// copy (a one-pixel shift is not a multiple of the swizzle period).
//
// wgrad: CTA = (filter tile, column tap s, channel group, K split).  Per 32-pixel K slab it loads
// the delta tile once and one input super-tile, and issues R x 4 MMAs into R accumulators
// (R * channels-per-group <= 512 TMEM columns).

namespace {

struct RowsArgs {
    float *out;
    int bn, n_rows, n_cols, out_ld;
    long long split_stride;
    int R, S, pad, cp;
    int img_w, pix_per_img, rows;       // OW, OH*OW, image rows per 32-pixel slab
    int col_groups;                      // channel groups per tap
    int total_slabs, slabs_per_split;
    int stages, tmem_cols;
    uint32_t a_bytes, b_bytes, tx_bytes, b_lbo;
    int *status;
    unsigned long long *span;   // profiling: first CTA entry / last CTA exit (null: off)
};

__global__ void __launch_bounds__(NTHREADS, 1)
conv_wgrad_rows_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const RowsArgs a) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ SharedCtl ctl;
    span_begin(a.span);
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM;
    const int bn = a.bn;
    const int s_tap = blockIdx.y / a.col_groups;
    const int cg = blockIdx.y - s_tap * a.col_groups;
    const int slab_begin = blockIdx.z * a.slabs_per_split;
    int nslabs = a.total_slabs - slab_begin;
    if (nslabs > a.slabs_per_split) nslabs = a.slabs_per_split;
    if (nslabs < 0) nslabs = 0;
    const uint32_t stage_bytes = a.a_bytes + a.b_bytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 1);
            mbar_init(smem_u32(&ctl.empty[s]), 1);
        }
        mbar_init(smem_u32(&ctl.accum), 1);
        mbar_init(smem_u32(&ctl.stat_bar), 4);
        ctl.abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
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
        if (threadIdx.x == 0) {
            for (int it = 0; it < nslabs; ++it) {
                const int s = it % a.stages;
                const uint32_t phase = (it / a.stages) & 1;
                if (!mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag)) break;
                const uint32_t bar = smem_u32(&ctl.full[s]);
                const uint32_t sa = smem_base + (uint32_t)s * stage_bytes;
                const uint32_t sb = sa + a.a_bytes;
                mbar_arrive_expect_tx(bar, a.tx_bytes);
                const int p0 = (slab_begin + it) * BK;
                const int img = p0 / a.pix_per_img;
                const int oh0 = (p0 - img * a.pix_per_img) / a.img_w;
                tma_load_5d(sa, &map_a, bar, 0, 0, oh0, img, m0 / 32);
                tma_load_5d(sb, &map_b, bar, 0, s_tap - a.pad, oh0 - a.pad, img, cg * (bn / 32));
            }
        }
        __syncwarp();
        bool ready = nslabs == 0 ? true : mbar_wait(smem_u32(&ctl.accum), 0, abort_flag);
        ready = __all_sync(0xffffffffu, ready);
        tc_fence_after_sync();
        if (ready) {
            float *obase = a.out + (size_t)blockIdx.z * a.split_stride + (size_t)m0 * a.out_ld;
            float *tile = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw)));
            for (int r = 0; r < a.R; ++r)
                store_accumulator<false>(tile, tmem + (uint32_t)(r * bn), nslabs > 0, warp, lane, bn, obase, (size_t)a.out_ld,
                                         a.n_rows - m0, (r * a.S + s_tap) * a.cp + cg * bn, a.n_cols, nullptr, 0);
        }
    } else if (lane == 0) {
        const uint32_t idesc = make_idesc_tf32(BM, bn, 1, 1);
        const uint32_t row16 = ((uint32_t)a.img_w * 128u) >> 4;   // one image row of the super-tile, in 16-byte units
        // One thread issues every MMA, so its instruction count per MMA is on the critical path: the
        // descriptors are built once and only their start-address field (low bits, 16-byte units) moves.
        const uint64_t da0 = make_desc(smem_base, 4096, 512, LAYOUT_SW128_32B);
        const uint64_t db0 = make_desc(smem_base + a.a_bytes, a.b_lbo, 512, LAYOUT_SW128_32B);
        uint32_t accumulate = 0;
        for (int it = 0; it < nslabs; ++it) {
            const int s = it % a.stages;
            const uint32_t phase = (it / a.stages) & 1;
            if (!mbar_wait(smem_u32(&ctl.full[s]), phase, abort_flag)) break;
            tc_fence_after_sync();
            const uint32_t st16 = ((uint32_t)s * stage_bytes) >> 4;
            if (a.R == 3) {
                // The issuing thread sets the pace (an MMA leaves it about 77 clocks): everything unrolled, only the
                // descriptors' low words computed, consecutive MMAs to different accumulators.
                const uint32_t a_lo = (uint32_t)da0 + st16, b_lo = (uint32_t)db0 + st16;
                const uint64_t a_hi = da0 & 0xffffffff00000000ull, b_hi = db0 & 0xffffffff00000000ull;
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int r = 0; r < 3; ++r)
                        mma_tf32(tmem + (uint32_t)(r * bn), a_hi | (uint64_t)(a_lo + (uint32_t)(j * 64)),
                                 b_hi | (uint64_t)(b_lo + (uint32_t)r * row16 + (uint32_t)(j * 64)), idesc, j > 0 ? 1u : accumulate);
            } else
            for (int r = 0; r < a.R; ++r) {
                const uint64_t db_r = db0 + st16 + (uint64_t)(r * row16);
                const uint32_t d_r = tmem + (uint32_t)(r * bn);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    mma_tf32(d_r, da0 + st16 + (uint64_t)(j * 64), db_r + (uint64_t)(j * 64), idesc, (accumulate | (uint32_t)(j > 0)));
            }
            accumulate = 1;
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

// Returns AET_OK (launched; *splits_out and *partial_out set), 1 (not eligible), or an error.
int tma_wgrad_rows(aet_layer *l, const ConvArgs &a, double flops, int *splits_out, float **partial_out) {
    aet_context *ctx = l->ctx;
    const ConvGeom &g = a.g;
    if (!tma_common_ok(l) || !ctx->opt[OPT_ROWS]) return 1;
    if (g.R < 2 || g.OW > 32 || g.OW % 8 || 32 % g.OW) return 1;
    const int rows = 32 / g.OW;
    if (g.OH % rows || g.OW > g.W || g.OH > g.H) return 1;
    int bn = g.cp < 128 ? g.cp : 128;
    if (g.cp % bn || g.R * bn > 512) return 1;
    const int k_blocks = (g.kp + 31) / 32;
    const int m_blocks = k_blocks < 4 ? k_blocks : 4;
    const int super_rows = rows + g.R - 1;
    const uint32_t b_lbo = (uint32_t)super_rows * g.OW * 128u;
    if (b_lbo >= (1u << 18)) return 1;
    const CUtensorMap *ma, *mb;
    {
        cuuint64_t dims[5] = {(cuuint64_t)(g.kp < 32 ? g.kp : 32), (cuuint64_t)g.OW, (cuuint64_t)g.OH, (cuuint64_t)g.N,
                              (cuuint64_t)k_blocks};
        cuuint64_t str[4] = {(cuuint64_t)g.kp * 4, (cuuint64_t)g.OW * g.kp * 4, (cuuint64_t)g.OH * g.OW * g.kp * 4, 128};
        cuuint32_t box[5] = {32, (cuuint32_t)g.OW, (cuuint32_t)rows, 1, (cuuint32_t)m_blocks};
        if (get_map(l, 6, a.src_a, 5, dims, str, box, true, &ma) != AET_OK) return g.kp % 32 ? 1 : AET_E_CUDA;
    }
    {
        cuuint64_t dims[5] = {32, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N, (cuuint64_t)g.cp / 32};
        cuuint64_t str[4] = {(cuuint64_t)g.cp * 4, (cuuint64_t)g.W * g.cp * 4, (cuuint64_t)g.H * g.W * g.cp * 4, 128};
        cuuint32_t box[5] = {32, (cuuint32_t)g.OW, (cuuint32_t)super_rows, 1, (cuuint32_t)bn / 32};
        AET_TRY(get_map(l, 7, a.src_b, 5, dims, str, box, true, &mb));
    }
    RowsArgs t = {};
    t.bn = bn; t.n_rows = a.n_rows; t.n_cols = a.n_cols; t.out_ld = a.out_ld;
    t.R = g.R; t.S = g.S; t.pad = g.pad; t.cp = g.cp;
    t.img_w = g.OW; t.pix_per_img = g.OH * g.OW; t.rows = rows;
    t.col_groups = g.cp / bn;
    t.total_slabs = (a.k_total + BK - 1) / BK;
    t.a_bytes = BM * BK * 4;
    t.b_bytes = b_lbo * (uint32_t)(bn / 32);
    t.b_lbo = b_lbo;
    t.tx_bytes = (uint32_t)m_blocks * 4096 + t.b_bytes;
    t.tmem_cols = pow2_cols(g.R * bn);
    t.status = ctx->status_dev;
    const int m_tiles = (g.K + BM - 1) / BM;
    const int tiles = m_tiles * g.S * t.col_groups;
    // one CTA per SM (the stages fill most of its shared memory): a single wave, and no more K
    // splits than that needs, because every split costs a full partial-gradient write and read
    int want = ctx->sm_count / tiles;
    if (ctx->opt[OPT_WGRAD_SPLITS] > 0) want = ctx->opt[OPT_WGRAD_SPLITS];
    if (want < 1) want = 1;
    int max_splits = t.total_slabs / 4;
    if (max_splits < 1) max_splits = 1;
    if (want > max_splits) want = max_splits;
    t.slabs_per_split = (t.total_slabs + want - 1) / want;
    const int splits = (t.total_slabs + t.slabs_per_split - 1) / t.slabs_per_split;
    const size_t out_floats = (size_t)g.K * a.n_cols;
    t.split_stride = (long long)out_floats;
    float *partial = nullptr;
    AET_TRY(ctx_scratch(ctx, out_floats * splits * sizeof(float), &partial));
    t.out = partial;
    const size_t stage = (size_t)t.a_bytes + t.b_bytes;
    int stages = (int)((200 * 1024) / stage);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > 4) stages = 4;
    if (stages < 2) return 1;
    t.stages = stages;
    const size_t smem_bytes = stage * stages + 1024;
    AET_TRY(ctx_smem_attr(ctx, conv_wgrad_rows_kernel));
    dim3 grid(m_tiles, g.S * t.col_groups, splits);
    {
        char variant[40];
        snprintf(variant, sizeof(variant), "n%d_sp%d", bn, splits);
        LaunchScope scope(ctx, "conv_wgrad_tma_rows", 0, flops, variant);
        t.span = ctx->span_ptr;
        launch_k(ctx->stream, grid, NTHREADS, smem_bytes, conv_wgrad_rows_kernel, *ma, *mb, t);
        AET_TRY(aet_check_launch("conv_wgrad_tma_rows"));
    }
    *splits_out = splits;
    *partial_out = partial;
    return AET_OK;
}

}  // namespace

// ---------------------------------------------------------------------------- fprop / dgrad with row sharing
// CTA = (pixel tile, filter/channel tile).  A pipeline stage holds, for one column tap s and one
// 32-channel slab, ONE activation super-tile of (MT*bh + R - 1) image rows and the R weight tiles of
// taps (0..R-1, s); it is consumed by R x MT x 4 MMAs into MT accumulators (MT = 2 pixel tiles of
// the same image share every weight tile, halving the weight traffic too).
namespace {

struct FdRowsArgs {
    float *out;
    const float *bias;
    const float *stat_shift;   // fprop: batch-norm statistics of the output (see ConvArgs)
    float *stat_partial;
    int act, bn, n_rows, n_cols, out_ld;
    int R, S, pad, inner;          // inner = channels of the K dimension (cp for fprop, kp for dgrad)
    int slabs_per_s;               // ceil(inner / 32)
    int mt, bh, bi, w, pix_per_img, n_img;
    int ksplit;                    // 1, or 2: the two CTAs of a cluster (grid z) take half of the K slabs each
    int smerge_S;                  // data gradient of a narrow layer: the S column taps ride in one MMA of N = S * channels
                                   // (0 = off); the epilogue adds the S column blocks, each shifted by its tap
    int par_epi;                   // mt == 2 with nine warps: warps 5-8 store the second pixel tile while warps 0-3 store the first
    int dual_acc;                  // mt == 1: two accumulators per tile (even / odd K steps), added by the epilogue
    int rotate;                    // every CTA starts its K slabs at another offset (spreads the reads of the shared weight tiles)
    int pair;                      // the two CTAs of a cluster along grid x form a cta_group::2 pair: MMAs of M = 256 issued by the
                                   // even CTA, each CTA loading its own pixel tiles and half of every weight tile
    int stages, tmem_cols;
    uint32_t a_bytes, b_tile_bytes, tx_bytes;
    int *status;
    unsigned long long *span;   // profiling: first CTA entry / last CTA exit (null: off)
};

constexpr int FD_THREADS_WIDE = 288;   // five warps + a second epilogue group

// The MMAs of one pipeline stage, issued by one thread.  A lone thread issues an instruction every few clocks, and an
// MMA of 128 x N x 8 leaves the tensor pipe only about 77 clocks per instruction: with run-time loop bounds and
// 64-bit descriptor arithmetic the issuing thread, not the tensor pipe, sets the pace.  So the tap count R and the
// tiles per CTA MT are compile-time here (everything unrolls, offsets become immediates), only the low word of a
// descriptor -- the start-address field sits in its low 14 bits -- is computed per MMA, and consecutive MMAs go to
// different accumulators where there are two.
// DUAL (with MT = 1): even and odd K steps go to two accumulators of the one tile, which the epilogue adds.
template <int KIND, bool PAIR, int R, int MT, bool DUAL = false>
__device__ __forceinline__ void issue_stage_mmas(uint32_t tmem, int bn, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t img_row16, uint32_t tile_rows16, uint32_t btile16, uint32_t b_step,
                                                 uint32_t idesc, uint32_t accumulate) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int rr = KIND == KIND_FPROP ? r : R - 1 - r;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int t = 0; t < MT; ++t) {
                const uint64_t da = ((uint64_t)a_hi << 32) | (uint64_t)(a_lo + (uint32_t)t * tile_rows16 + (uint32_t)rr * img_row16 + (uint32_t)(j * 2));
                const uint64_t db = ((uint64_t)b_hi << 32) | (uint64_t)(b_lo + (uint32_t)r * btile16 + (uint32_t)j * b_step);
                const uint32_t acc = (r > 0 || j > (DUAL ? 1 : 0)) ? 1u : accumulate;
                const uint32_t d = tmem + (uint32_t)((DUAL ? (j & 1) : t) * bn);
                if (PAIR) mma_tf32_pair(d, da, db, idesc, acc);
                else mma_tf32(d, da, db, idesc, acc);
            }
        }
    }
}
// PAIR: the cta_group::2 form.  It is a separate instantiation because a kernel that contains cta_group::2
// instructions can only be launched as a cluster of CTA pairs.
template <int KIND, bool PAIR>
__global__ void __launch_bounds__(FD_THREADS_WIDE, 1)
conv_fd_rows_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const FdRowsArgs a) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ SharedCtl ctl;
    span_begin(a.span);
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bn = a.bn;
    const int n0 = blockIdx.y * bn;
    const int m0 = blockIdx.x * BM * a.mt;                  // first pixel (in (n,h,w) order) of this CTA
    const int img0 = m0 / a.pix_per_img;
    const int row0 = (m0 - img0 * a.pix_per_img) / a.w;      // 0 when the tile spans whole images
    const int total_slabs = a.S * a.slabs_per_s;
    // K split over a cluster of two CTAs: rank 1 adds nothing to global memory, rank 0 reads rank 1's
    // staged accumulator through distributed shared memory and stores the sum
    const int krank = a.ksplit > 1 ? (int)blockIdx.z : 0;
    const int slab_begin = a.ksplit > 1 ? krank * ((total_slabs + 1) / 2) : 0;
    const int slab_end = a.ksplit > 1 ? (krank == 0 ? (total_slabs + 1) / 2 : total_slabs) : total_slabs;
    const int nslabs = slab_end - slab_begin;
    const uint32_t stage_bytes = a.a_bytes + (uint32_t)a.R * a.b_tile_bytes;
    bool epilogue_ready = false;
    // Cluster shapes: (1,1,2) K split only, (2,1,1) a CTA pair, (2,1,2) two pairs that split K.  Ranks run x first,
    // so a pair is ranks {0,1} or {2,3} and the K-split partner of rank r is r ^ 2 (r ^ 1 without pairs).
    const uint32_t crank = (PAIR || a.ksplit > 1) ? cluster_ctarank() : 0u;
    const uint32_t prank = PAIR ? (crank & 1u) : 0u;        // rank inside the CTA pair; 0 = the CTA that issues the MMAs
    const uint32_t pair_base = crank & ~1u;                 // cluster rank of this pair's leader
    const bool leader = prank == 0u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 1);
            mbar_init(smem_u32(&ctl.empty[s]), 1);
        }
        mbar_init(smem_u32(&ctl.accum), 1);
        mbar_init(smem_u32(&ctl.stat_bar), 4);
        mbar_init(smem_u32(&ctl.stat_bar2), 4);
        ctl.abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
    }
    if (warp == 4) {
        if (PAIR) { tmem_alloc_pair(smem_u32(&ctl.tmem_base), a.tmem_cols); tmem_relinquish_pair(); }
        else { tmem_alloc(smem_u32(&ctl.tmem_base), a.tmem_cols); tmem_relinquish(); }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = ctl.tmem_base;
    // A pair's leader writes into its partner's TMEM and arrives on its partner's barriers: both CTAs must have
    // finished the set-up above before either goes on.
    if (PAIR) cooperative_groups::this_cluster().sync();
    pdl_enter();   // everything above touched only shared memory, TMEM and kernel parameters
    volatile int *abort_flag = &ctl.abort_flag;

    if (warp != 4) {
        const int q = warp & 3, grp = warp < 4 ? 0 : 1;   // TMEM lane quarter; which pixel tile this warp stores
        if (threadIdx.x == 0) {
            const int rot = (a.rotate && nslabs > 0) ? (int)(((blockIdx.x >> (PAIR ? 1 : 0)) * 5u + blockIdx.y * 3u) % (unsigned)nslabs) : 0;
            for (int it = 0; it < nslabs; ++it) {
                const int s = it % a.stages;
                const uint32_t phase = (it / a.stages) & 1;
                if (!mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag)) break;
                const uint32_t sa = smem_base + (uint32_t)s * stage_bytes;
                const uint32_t sb = sa + a.a_bytes;
                // CTAs walk their K slabs from different starting points: all of them read the same weight tiles, and in
                // lockstep every SM would ask the same L2 lines at the same moment.  The order depends on the CTA index
                // only, so results stay reproducible (a pair's two CTAs share their order).
                int itr = it + rot;
                if (itr >= nslabs) itr -= nslabs;
                const int slab = slab_begin + itr;
                const int st = slab / a.slabs_per_s, cb = slab - st * a.slabs_per_s;   // column tap, channel slab
                // fprop reads input pixel (h + r - pad, w + s - pad); dgrad reads delta pixel (h + pad - r, w + pad - s)
                const int wx = a.smerge_S ? 0 : (KIND == KIND_FPROP ? st - a.pad : a.pad - st);
                const int hy = KIND == KIND_FPROP ? row0 - a.pad : row0 + a.pad - (a.R - 1);
                if (PAIR) {
                    // Both CTAs' copies complete on the LEADER's barrier, which expects the bytes of both; this CTA
                    // brings its own pixel tiles and its half of the N rows of every weight tile.
                    const uint32_t bar = map_to_cta(smem_u32(&ctl.full[s]), pair_base);
                    if (leader) mbar_arrive_expect_tx(smem_u32(&ctl.full[s]), 2u * a.tx_bytes);
                    const int half = (int)prank * (bn / 2);
                    if (a.bi > 1) tma_load_4d_pair(sa, &map_a, bar, cb * 32, wx, img0, hy);
                    else          tma_load_4d_pair(sa, &map_a, bar, cb * 32, wx, hy, img0);
                    for (int r = 0; r < a.R; ++r) {
                        const int tap = r * a.S + st;
                        if (KIND == KIND_FPROP) tma_load_2d_pair(sb + r * a.b_tile_bytes, &map_b, bar, tap * a.inner + cb * 32, n0 + half);
                        else if (a.smerge_S)    tma_load_4d_pair(sb + r * a.b_tile_bytes, &map_b, bar, 0, cb * 32, half / 32, r);
                        else                    tma_load_4d_pair(sb + r * a.b_tile_bytes, &map_b, bar, 0, cb * 32, (n0 + half) / 32, tap);
                    }
                    continue;
                }
                const uint32_t bar = smem_u32(&ctl.full[s]);
                mbar_arrive_expect_tx(bar, a.tx_bytes);
                if (a.bi > 1) tma_load_4d(sa, &map_a, bar, cb * 32, wx, img0, hy);      // dims (c, w, n, h)
                else          tma_load_4d(sa, &map_a, bar, cb * 32, wx, hy, img0);      // dims (c, w, h, n)
                for (int r = 0; r < a.R; ++r) {
                    const int tap = r * a.S + st;
                    if (KIND == KIND_FPROP) tma_load_2d(sb + r * a.b_tile_bytes, &map_b, bar, tap * a.inner + cb * 32, n0);
                    else if (a.smerge_S)    tma_load_4d(sb + r * a.b_tile_bytes, &map_b, bar, 0, cb * 32, 0, r);   // dims (n%32, filter, n/32, r)
                    else                    tma_load_4d(sb + r * a.b_tile_bytes, &map_b, bar, 0, cb * 32, n0 / 32, tap);
                }
            }
        }
        __syncwarp();
        bool ready = mbar_wait(smem_u32(&ctl.accum), 0, abort_flag);
        ready = __all_sync(0xffffffffu, ready);
        tc_fence_after_sync();
        epilogue_ready = ready;
        if (ready && a.ksplit > 1) {
            // only stage the accumulator (mt == 1 here); the sum of the two halves is stored after the cluster barrier
            stage_accumulator(reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw))), tmem, true, q, lane, bn,
                              a.dual_acc ? tmem + (uint32_t)bn : 0u);
        } else if (ready && a.smerge_S && 32 % a.w == 0 && bn / a.smerge_S <= 128) {
            // Column taps merged into N: accumulator column block sx holds the partial result that belongs to the
            // output pixel (pad - sx) columns further on, i.e. to the TMEM lane (pad - sx) rows away.  A warp's 32
            // lanes are whole image rows here (the image width divides 32), so every neighbour a lane needs sits
            // in the same warp, and the lanes at an image row's ends are exactly those whose neighbour falls outside
            // the image: the column blocks are combined with warp shuffles straight out of the TMEM registers, and
            // only the finished cpn-wide tile goes through shared memory for the coalesced store.
            const int cpn = bn / a.smerge_S;                 // output channels
            const int pitch = cpn + 4;
            float *tile = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw))) + (size_t)grp * BM * pitch;
            float *mine = tile + (size_t)(q * 32 + lane) * pitch;
            const int wcol = lane % a.w;
            const uint32_t tbase = tmem + (uint32_t)(grp * bn) + ((uint32_t)(q * 32) << 16);
            for (int c0 = 0; c0 < cpn; c0 += 16) {
                float acc[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = 0.f;
                for (int sx0 = 0; sx0 < a.smerge_S; sx0 += 3) {          // three column blocks in flight per wait
                    uint32_t v[3][16];
#pragma unroll
                    for (int k = 0; k < 3; ++k)
                        if (sx0 + k < a.smerge_S) tmem_ld16_issue(tbase + (uint32_t)((sx0 + k) * cpn + c0), v[k]);
                    tmem_ld_wait();
#pragma unroll
                    for (int k = 0; k < 3; ++k) {
                        if (sx0 + k >= a.smerge_S) break;
                        const int d = a.pad - (sx0 + k);             // this block's values belong d lanes down
                        const bool ok = (unsigned)(wcol + d) < (unsigned)a.w;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float t = __shfl_sync(0xffffffffu, __uint_as_float(v[k][i]), (lane + d) & 31);
                            acc[i] += ok ? t : 0.f;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) *reinterpret_cast<float4 *>(mine + c0 + 4 * i) = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
            }
            __syncwarp();
            const int mt0 = m0 + grp * BM;
            flush_tile<false>(tile, nullptr, q, lane, cpn, a.out + (size_t)mt0 * a.out_ld, (size_t)a.out_ld, a.n_rows - mt0, 0, a.n_cols,
                              nullptr, (int)AET_LINEAR, 1, 1, 0, nullptr);
        } else if (ready && a.smerge_S) {
            // General form (image rows wider than a warp): accumulator column block s holds the partial result that belongs to
            // the output pixel pad - s columns further on.  The four warps of a group stage their tile, then every
            // row adds its (up to) S neighbours' blocks; a tile is whole image rows, so the neighbours are rows
            // +-1.. of the same tile.  With two pixel tiles the two warp groups work side by side.
            const int pitch = bn + 4;
            float *tile = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw))) + (size_t)grp * BM * pitch;
            const int cpn = bn / a.smerge_S;
            const int lpr = cpn >= 128 ? 32 : cpn / 4, rpi = 32 / lpr, sub = lane / lpr, lcol = (lane - sub * lpr) * 4;
            unsigned long long *bar = grp ? &ctl.stat_bar2 : &ctl.stat_bar;
            stage_accumulator(tile, tmem + (uint32_t)(grp * bn), true, q, lane, bn);
            if (lane == 0) mbar_arrive(smem_u32(bar));
            bool ok = mbar_wait(smem_u32(bar), 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                const int mt0 = m0 + grp * BM, rows_valid = a.n_rows - mt0;
                float *out = a.out + (size_t)mt0 * a.out_ld;
                for (int c0 = 0; c0 < cpn; c0 += 128) {
                    const int c = c0 + lcol;
                    const bool active = c < cpn && c < a.n_cols && sub < rpi;
                    for (int r0 = 0; r0 < 32; r0 += 4 * rpi) {
                        float4 v[4];
                        int rows[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int row = q * 32 + r0 + u * rpi + sub;
                            rows[u] = (active && r0 + u * rpi + sub < 32 && row < rows_valid) ? row : -1;
                            v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (rows[u] < 0) continue;
                            const int wcol = row % a.w;
                            for (int sx = 0; sx < a.smerge_S; ++sx) {
                                const int d = a.pad - sx;              // this block's contribution comes from column w + d
                                if ((unsigned)(wcol + d) >= (unsigned)a.w) continue;
                                const float4 q4 = *reinterpret_cast<const float4 *>(tile + (size_t)(row + d) * pitch + sx * cpn + c);
                                v[u].x += q4.x; v[u].y += q4.y; v[u].z += q4.z; v[u].w += q4.w;
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (rows[u] >= 0) *reinterpret_cast<float4 *>(out + (size_t)rows[u] * a.out_ld + c) = v[u];
                    }
                }
            }
        } else if (ready && a.par_epi) {
            // two epilogue groups, one pixel tile each, side by side in the (now idle) stage memory
            float *tile = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw))) + (size_t)grp * BM * (bn + 4);
            StatAcc st;
            stat_init(st, KIND == KIND_FPROP ? a.stat_partial ? a.stat_shift : nullptr : nullptr);
            const int mt0 = m0 + grp * BM;
            store_accumulator<KIND == KIND_FPROP>(tile, tmem + (uint32_t)(grp * bn), true, q, lane, bn, a.out + (size_t)mt0 * a.out_ld,
                                                  (size_t)a.out_ld, a.n_rows - mt0, n0, a.n_cols, a.bias, a.act, a.bi, a.w,
                                                  a.pix_per_img, &st);
            if (KIND == KIND_FPROP && st.shift)   // each group writes its own partial row
                stats_commit(tile, st, q, lane, bn, a.stat_partial + ((size_t)blockIdx.x * 2 + grp) * 2 * a.out_ld + n0, a.out_ld,
                             a.n_cols - n0, grp ? &ctl.stat_bar2 : &ctl.stat_bar, abort_flag);
        } else if (ready) {
            float *tile = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw)));
            StatAcc st;
            stat_init(st, KIND == KIND_FPROP ? a.stat_partial ? a.stat_shift : nullptr : nullptr);
            for (int t = 0; t < a.mt; ++t) {
                const int mt0 = m0 + t * BM;
                store_accumulator<KIND == KIND_FPROP>(tile, tmem + (uint32_t)(t * bn), true, warp, lane, bn,
                                                      a.out + (size_t)mt0 * a.out_ld, (size_t)a.out_ld, a.n_rows - mt0, n0, a.n_cols,
                                                      a.bias, a.act, a.bi, a.w, a.pix_per_img, &st, a.dual_acc ? tmem + (uint32_t)bn : 0u);
            }
            if (KIND == KIND_FPROP && st.shift)
                stats_commit(tile, st, warp, lane, bn, a.stat_partial + (size_t)blockIdx.x * 2 * a.out_ld + n0, a.out_ld, a.n_cols - n0,
                             &ctl.stat_bar, abort_flag);
        }
    } else if (lane == 0 && leader) {
        const int b_mn = KIND == KIND_FPROP ? 0 : 1;
        const uint32_t idesc = make_idesc_tf32(PAIR ? 2 * BM : BM, bn, 0, b_mn);
        const uint64_t da0 = make_desc(smem_base, 0, 1024, LAYOUT_SW128);
        const uint64_t db0 = b_mn ? make_desc(smem_base + a.a_bytes, 4096, 512, LAYOUT_SW128_32B)
                                  : make_desc(smem_base + a.a_bytes, 0, 1024, LAYOUT_SW128);
        const uint64_t b_step = b_mn ? 64 : 2;
        const uint32_t img_row16 = ((uint32_t)(a.bi * a.w) * 128u) >> 4;      // one image row (of every image in the tile)
        const uint32_t tile_rows16 = (uint32_t)a.bh * img_row16;               // one 128-pixel tile
        const uint32_t btile16 = a.b_tile_bytes >> 4;
        uint32_t accumulate = 0;
        for (int it = 0; it < nslabs; ++it) {
            const int s = it % a.stages;
            const uint32_t phase = (it / a.stages) & 1;
            if (!mbar_wait(smem_u32(&ctl.full[s]), phase, abort_flag)) break;
            tc_fence_after_sync();
            const uint32_t st16 = ((uint32_t)s * stage_bytes) >> 4;
            if (a.R == 3 && a.mt <= 2) {
                // the common 3x3 case: fully unrolled (the low words cannot carry into the descriptors' high words: start
                // addresses stay below 2^14 sixteen-byte units)
                const uint32_t a_lo = (uint32_t)da0 + st16, b_lo = (uint32_t)db0 + st16;
                if (a.mt == 2) issue_stage_mmas<KIND, PAIR, 3, 2>(tmem, bn, a_lo, (uint32_t)(da0 >> 32), b_lo, (uint32_t)(db0 >> 32), img_row16,
                                                                  tile_rows16, btile16, (uint32_t)b_step, idesc, accumulate);
                else if (a.dual_acc) issue_stage_mmas<KIND, PAIR, 3, 1, true>(tmem, bn, a_lo, (uint32_t)(da0 >> 32), b_lo, (uint32_t)(db0 >> 32),
                                                                             img_row16, tile_rows16, btile16, (uint32_t)b_step, idesc, accumulate);
                else issue_stage_mmas<KIND, PAIR, 3, 1>(tmem, bn, a_lo, (uint32_t)(da0 >> 32), b_lo, (uint32_t)(db0 >> 32), img_row16,
                                                        tile_rows16, btile16, (uint32_t)b_step, idesc, accumulate);
            } else
            for (int r = 0; r < a.R; ++r) {
                const int rr = KIND == KIND_FPROP ? r : a.R - 1 - r;
                const uint64_t db_r = db0 + st16 + (uint64_t)(r * btile16);
                for (int t = 0; t < a.mt; ++t) {
                    const uint64_t da_rt = da0 + st16 + (uint64_t)(t * tile_rows16 + rr * img_row16);
                    const uint32_t d_t = tmem + (uint32_t)(t * bn);
                    if (PAIR) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            mma_tf32_pair(d_t, da_rt + (uint64_t)(j * 2), db_r + j * b_step, idesc, (accumulate | (uint32_t)(r > 0 || j > 0)));
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            mma_tf32(d_t, da_rt + (uint64_t)(j * 2), db_r + j * b_step, idesc, (accumulate | (uint32_t)(r > 0 || j > 0)));
                    }
                }
            }
            accumulate = 1;
            if (PAIR) mma_commit_pair(smem_u32(&ctl.empty[s]), (uint16_t)(3u << pair_base));   // frees the stage in both CTAs
            else mma_commit(smem_u32(&ctl.empty[s]));
        }
        if (PAIR) mma_commit_pair(smem_u32(&ctl.accum), (uint16_t)(3u << pair_base));
        else mma_commit(smem_u32(&ctl.accum));
    }

    __syncwarp();   // the MMA warp's lanes rejoin their issuing lane before any warp-wide barrier
    if (a.ksplit > 1) {
        // Every thread of both CTAs reaches these two barriers whatever happened above (the role loops
        // leave by `break`, never by `return`), so a timed-out CTA cannot strand its partner.
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();                                   // both staging tiles are complete
        if (warp < 4 && epilogue_ready) {
            // Each CTA stores half of the tile's rows (its 16-row half of every warp's 32-row block) as the sum of its
            // own and its partner's staged accumulator, read through distributed shared memory: a + b on one side,
            // b + a on the other, the same bits.
            float *tile = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw)));
            const float *remote = cluster.map_shared_rank(tile, PAIR ? (crank ^ 2u) : (crank ^ 1u));
            StatAcc st;
            stat_init(st, KIND == KIND_FPROP ? a.stat_partial ? a.stat_shift : nullptr : nullptr);
            flush_tile<KIND == KIND_FPROP>(tile, remote, warp, lane, bn, a.out + (size_t)m0 * a.out_ld, (size_t)a.out_ld, a.n_rows - m0,
                                           n0, a.n_cols, a.bias, a.act, a.bi, a.w, a.pix_per_img, &st, krank * 16, krank * 16 + 16);
            cluster.sync();                               // the partner has read this CTA's staged tile: it may be reused
            if (KIND == KIND_FPROP && st.shift)           // one partial row per CTA of the pair
                stats_commit(tile, st, warp, lane, bn, a.stat_partial + ((size_t)blockIdx.x * 2 + krank) * 2 * a.out_ld + n0, a.out_ld,
                             a.n_cols - n0, &ctl.stat_bar, abort_flag);
        } else {
            cluster.sync();                               // (the warps that store nothing keep the barrier count whole)
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    // the pair's TMEM is released together, once both CTAs have read their accumulators (every thread of both
    // CTAs gets here whatever happened above)
    if (PAIR) cooperative_groups::this_cluster().sync();
    if (warp == 4) {
        if (PAIR) tmem_dealloc_pair(tmem, a.tmem_cols);
        else tmem_dealloc(tmem, a.tmem_cols);
        if (lane == 0 && ctl.abort_flag && a.status) atomicOr(a.status, AET_STATUS_TIMEOUT);
    }
    span_end(a.span);
}

// fprop (KIND_FPROP) or dgrad (KIND_DGRAD) through the row-sharing kernel; 1 = not eligible.
template <int KIND>
int tma_fd_rows(aet_layer *l, const ConvArgs &a, double flops) {
    aet_context *ctx = l->ctx;
    const ConvGeom &g = a.g;
    if (!tma_common_ok(l) || !ctx->opt[OPT_ROWS] || !ctx->opt[KIND == KIND_FPROP ? OPT_ROWS_FPROP : OPT_ROWS_DGRAD]) return 1;
    if (g.R < 2 || g.OH != g.H || g.OW != g.W) return 1;                 // same-size convolutions
    const int inner = KIND == KIND_FPROP ? g.cp : g.kp;
    if (KIND == KIND_DGRAD && !(g.kp % 32 == 0)) return 1;
    cuuint32_t bw, bh, bi;
    if (!pixel_box(BM, g.H, g.W, &bw, &bh, &bi) || (int)bw != g.W) return 1;
    if (((int)bi * g.W) % 8) return 1;                                    // image rows must be whole swizzle periods
    // The stages fill most of an SM's shared memory, so one CTA runs per SM: take the widest N tile
    // that still gives a CTA to most SMs (wider tiles re-read the activations less often).
    const int m_tiles = (a.n_rows + BM - 1) / BM;
    const int full = round_up(a.n_cols, 16);
    const int cands[4] = {full <= 256 ? full : 256, 128, 64, 32};
    int bn = 0, mt = 1, stages = 0, n_tiles = 0, ksplit = 1;
    uint32_t a_bytes = 0, b_tile = 0;
    size_t stage = 0;
    const int total_slabs = g.S * ((inner + 31) / 32);
    // Data gradient of a narrow layer (few input channels): an MMA of N = 64 costs as much as one of N = 128, so the S
    // column taps are merged into one MMA of N = S * channels; the activations then cross L2 once per channel slab
    // instead of once per column tap, and the epilogue adds the S column blocks with their column shifts.
    int smerge = 0;
    if (KIND == KIND_DGRAD && bi == 1 && g.S == g.R && g.pad == (g.S - 1) / 2 && g.cp % 32 == 0 && g.cp < 128 && g.S * g.cp <= 256 &&
        a.n_cols == g.cp && ctx->opt[OPT_SMERGE]) {
        const int c = g.S * g.cp;
        int m = (g.H % (2 * (int)bh) == 0 && 2 * c <= 512 && (m_tiles / 2) >= (ctx->sm_count * 3) / 4) ? 2 : 1;
        for (; m >= 1 && !smerge; --m) {
            const uint32_t ab = (uint32_t)(m * (int)bh + g.R - 1) * bi * g.W * 128u;
            const size_t st = (size_t)ab + (size_t)g.R * c * 128u;
            int ns = (int)((218 * 1024) / st);
            if (ns > 4) ns = 4;
            if (ns >= 2 && st * ns >= (size_t)m * BM * (c + 4) * 4 && (m_tiles + m - 1) / m <= ctx->sm_count) {   // one staging tile per pixel tile
                bn = c; mt = m; stages = ns; n_tiles = 1; a_bytes = ab; b_tile = (uint32_t)c * 128u; stage = st; smerge = g.S;
            }
        }
    }
    for (int i = 0; i < 4 && !bn; ++i) {
        const int c = cands[i];
        if (c > full || (KIND == KIND_DGRAD && (c % 32 || g.cp % c))) continue;
        const int nt = (a.n_cols + c - 1) / c;
        // too few tiles for the machine: keep the wide N tile (an MMA of N = 64 costs as much as one of
        // N = 128) and let the two CTAs of a cluster take half of the K range each
        const bool split = c >= 128 && m_tiles * nt * 2 <= ctx->sm_count && total_slabs >= 8 && ctx->opt[OPT_KSPLIT];
        if (!(m_tiles * nt >= (ctx->sm_count * 3) / 5 || c <= 64 || split)) continue;
        // two pixel tiles per CTA when they are rows of one image and there are still enough CTAs
        int m = 1;
        if (bi == 1 && g.H % (2 * (int)bh) == 0 && 2 * c <= 512 && (m_tiles / 2) * nt >= (ctx->sm_count * 3) / 4 &&
            ctx->opt[OPT_MT2])
            m = 2;
        for (; m >= 1; --m) {
            const uint32_t ab = (uint32_t)(m * (int)bh + g.R - 1) * bi * g.W * 128u;
            const size_t st = (size_t)ab + (size_t)g.R * c * 128u;
            int ns = (int)((218 * 1024) / st);
            if (ns > 4) ns = 4;
            if (ns >= 2 && st * ns >= (size_t)BM * (c + 4) * 4) {   // pipeline depth and room for the epilogue tile
                bn = c; mt = m; stages = ns; n_tiles = nt; a_bytes = ab; b_tile = (uint32_t)c * 128u; stage = st;
                ksplit = (split && m == 1) ? 2 : 1;
                break;
            }
        }
    }
    if (!bn) return 1;
    // CTA pairs (cta_group::2, option "pair"): the two CTAs of a cluster along grid x run MMAs of M = 256 together and each
    // loads only half of every weight tile, so the weights cross L2 -> SM once per pair.  Needs an even number of CTAs
    // along x and half tiles that are whole swizzle blocks.
    int pair = 0;
    {
        const int gx = (m_tiles + mt - 1) / mt;
        const bool halves_ok = KIND == KIND_FPROP ? bn % 16 == 0 : bn % 64 == 0;
        if (ctx->opt[OPT_PAIR] && gx % 2 == 0 && halves_ok && m_tiles % mt == 0) {
            const uint32_t bt = (uint32_t)(bn / 2) * 128u;
            const size_t st = (size_t)a_bytes + (size_t)g.R * bt;
            int ns = (int)((218 * 1024) / st);   // + 1 KB of alignment slack stays inside the 220 KB the kernel may use
            if (ns > MAX_STAGES) ns = MAX_STAGES;
            const size_t need = (size_t)(mt == 2 ? 2 : 1) * BM * (bn + 4) * 4;   // staging tile(s) of the epilogue
            if (ns >= 2 && st * ns >= need) { pair = 1; b_tile = bt; stage = st; stages = ns; }
        }
    }
    // The large stages allow one CTA per SM, so this kernel is for grids of at most one wave; a grid that needs a
    // second, partial wave goes to the plain TMA kernel, whose smaller stages let two CTAs share an SM.
    if (((m_tiles + mt - 1) / mt) * n_tiles * ksplit > ctx->sm_count && !ctx->opt[OPT_ROWS_MULTI]) return 1;
    const int super_rows = mt * (int)bh + g.R - 1;
    const CUtensorMap *ma, *mb;
    const float *act = a.src_a;
    const int ac = inner;   // channels of the A tensor
    if (bi > 1) {
        cuuint64_t dims[4] = {(cuuint64_t)ac, (cuuint64_t)g.W, (cuuint64_t)g.N, (cuuint64_t)g.H};
        cuuint64_t str[3] = {(cuuint64_t)ac * 4, (cuuint64_t)g.H * g.W * ac * 4, (cuuint64_t)g.W * ac * 4};
        cuuint32_t box[4] = {32, (cuuint32_t)g.W, bi, (cuuint32_t)super_rows};
        AET_TRY(get_map(l, KIND == KIND_FPROP ? 8 : 10, act, 4, dims, str, box, false, &ma));
    } else {
        cuuint64_t dims[4] = {(cuuint64_t)ac, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N};
        cuuint64_t str[3] = {(cuuint64_t)ac * 4, (cuuint64_t)g.W * ac * 4, (cuuint64_t)g.H * g.W * ac * 4};
        cuuint32_t box[4] = {32, (cuuint32_t)g.W, (cuuint32_t)super_rows, 1};
        AET_TRY(get_map(l, KIND == KIND_FPROP ? 8 : 10, act, 4, dims, str, box, false, &ma));
    }
    const int bnb = pair ? bn / 2 : bn;   // N rows of a weight tile one CTA brings
    if (smerge) {
        const int taps = g.R * g.S;
        cuuint64_t dims[4] = {32, (cuuint64_t)g.K, (cuuint64_t)(g.S * g.cp) / 32, (cuuint64_t)g.R};
        cuuint64_t str[3] = {(cuuint64_t)taps * g.cp * 4, 128, (cuuint64_t)g.S * g.cp * 4};
        cuuint32_t box[4] = {32, 32, (cuuint32_t)bnb / 32, 1};
        AET_TRY(get_map(l, 13, a.src_b, 4, dims, str, box, true, &mb));
    } else if (KIND == KIND_FPROP) {
        cuuint64_t dims[2] = {(cuuint64_t)a.k_total, (cuuint64_t)g.K};
        cuuint64_t str[1] = {(cuuint64_t)a.k_total * 4};
        cuuint32_t box[2] = {32, (cuuint32_t)bnb};
        AET_TRY(get_map(l, 9, a.src_b, 2, dims, str, box, false, &mb));
    } else {
        const int taps = g.R * g.S;
        cuuint64_t dims[4] = {32, (cuuint64_t)g.K, (cuuint64_t)g.cp / 32, (cuuint64_t)taps};
        cuuint64_t str[3] = {(cuuint64_t)taps * g.cp * 4, 128, (cuuint64_t)g.cp * 4};
        cuuint32_t box[4] = {32, 32, (cuuint32_t)bnb / 32, 1};
        AET_TRY(get_map(l, 11, a.src_b, 4, dims, str, box, true, &mb));
    }
    FdRowsArgs t = {};
    t.out = a.out; t.bias = KIND == KIND_FPROP ? a.bias : nullptr; t.act = KIND == KIND_FPROP ? a.act : (int)AET_LINEAR;
    t.stat_shift = KIND == KIND_FPROP ? a.stat_shift : nullptr; t.stat_partial = KIND == KIND_FPROP ? a.stat_partial : nullptr;
    t.bn = bn; t.n_rows = a.n_rows; t.n_cols = a.n_cols; t.out_ld = a.out_ld;
    t.R = g.R; t.S = smerge ? 1 : g.S; t.pad = g.pad; t.inner = inner; t.slabs_per_s = (inner + 31) / 32;
    t.smerge_S = smerge;
    t.mt = mt; t.bh = (int)bh; t.bi = (int)bi; t.w = g.W; t.pix_per_img = g.H * g.W; t.n_img = g.N;
    // one pixel tile per CTA: its K steps alternate between two accumulators (3x3 filters, whose issue path is unrolled)
    t.dual_acc = (mt == 1 && !smerge && g.R == 3 && 2 * bn <= 512 && ctx->opt[OPT_DUAL_ACC]) ? 1 : 0;
    t.stages = stages; t.tmem_cols = pow2_cols((t.dual_acc ? 2 : mt) * bn); t.ksplit = ksplit;
    t.par_epi = (mt == 2 && !smerge && stage * stages >= 2 * (size_t)BM * (bn + 4) * 4 && ctx->opt[OPT_PAR_EPILOGUE]) ? 1 : 0;
    t.pair = pair;
    t.rotate = ctx->opt[OPT_ROTATE];
    const int threads = (t.par_epi || (smerge && mt == 2)) ? FD_THREADS_WIDE : NTHREADS;
    t.a_bytes = a_bytes; t.b_tile_bytes = b_tile; t.tx_bytes = a_bytes + (uint32_t)g.R * b_tile;
    t.status = ctx->status_dev;
    const size_t smem_bytes = stage * stages + 1024;
    if (pair) AET_TRY(ctx_smem_attr(ctx, conv_fd_rows_kernel<KIND, true>));
    else AET_TRY(ctx_smem_attr(ctx, conv_fd_rows_kernel<KIND, false>));
    dim3 grid((m_tiles + mt - 1) / mt, n_tiles, ksplit);
    if (KIND == KIND_FPROP && a.stat_rows_out) *a.stat_rows_out = (int)grid.x * ((t.par_epi || ksplit > 1) ? 2 : 1);
    const char *name = KIND == KIND_FPROP ? "conv_fprop_tma_rows" : "conv_dgrad_tma_rows";
    char variant[40];   // e.g. "mt2e_n128x1_p2": two pixel tiles, second epilogue group, N tile 128, one N tile, CTA pairs
    snprintf(variant, sizeof(variant), "%smt%d%s%s_n%dx%d%s%s", smerge ? "sm_" : "", mt, t.par_epi ? "e" : "", t.dual_acc ? "d" : "", bn, n_tiles,
             ksplit > 1 ? "_ks2" : "", pair ? "_p2" : "");
    LaunchScope scope(ctx, name, 0, flops, variant);
    t.span = ctx->span_ptr;
    if (pair) launch_k_cluster(ctx->stream, grid, threads, smem_bytes, 2, ksplit, conv_fd_rows_kernel<KIND, true>, *ma, *mb, t);
    else if (ksplit > 1) launch_k_cluster(ctx->stream, grid, threads, smem_bytes, 1, ksplit, conv_fd_rows_kernel<KIND, false>, *ma, *mb, t);
    else launch_k(ctx->stream, grid, threads, smem_bytes, conv_fd_rows_kernel<KIND, false>, *ma, *mb, t);
    return aet_check_launch(name);
}

}  // namespace
