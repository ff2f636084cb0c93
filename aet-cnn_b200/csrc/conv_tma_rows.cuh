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
};

__global__ void __launch_bounds__(NTHREADS, 1)
conv_wgrad_rows_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const RowsArgs a) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ SharedCtl ctl;
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
            const uint64_t st16 = (uint64_t)(((uint32_t)s * stage_bytes) >> 4);
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
        if (lane == 0 && ctl.abort_flag && a.status) atomicExch(a.status, AET_STATUS_TIMEOUT);
    }
}

// Returns AET_OK (launched; *splits_out and *partial_out set), 1 (not eligible), or an error.
int tma_wgrad_rows(aet_layer *l, const ConvArgs &a, double flops, int *splits_out, float **partial_out) {
    aet_context *ctx = l->ctx;
    const ConvGeom &g = a.g;
    if (!tma_common_ok(l) || getenv("AET_NO_ROWS")) return 1;
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
    if (const char *e = getenv("AET_WGRAD_SPLITS")) want = atoi(e);
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
    static bool attr_set = false;
    if (!attr_set) {
        AET_CUDA(cudaFuncSetAttribute(conv_wgrad_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        attr_set = true;
    }
    dim3 grid(m_tiles, g.S * t.col_groups, splits);
    {
        LaunchScope scope(ctx, "conv_wgrad_tma_rows", 0, flops);
        conv_wgrad_rows_kernel<<<grid, NTHREADS, smem_bytes, ctx->stream>>>(*ma, *mb, t);
        AET_TRY(aet_check_launch("conv_wgrad_tma_rows"));
    }
    *splits_out = splits;
    *partial_out = partial;
    return AET_OK;
}

}  // namespace
