// TMA producer variant of the implicit-GEMM convolution kernels (included by conv.cu).
//
// Eligible shapes: stride 1, padded channel counts that are multiples of 32, and a 128-pixel M
// tile (fprop, dgrad) or 32-pixel K slab (wgrad) that is a whole number of image rows or whole
// images.  One thread issues tiled bulk-tensor copies whose coordinates are shifted by the filter
// tap; pixels outside the image are zero-filled by the copy engine, so there is no halo logic and
// no im2col buffer.  Tiles land in shared memory in the 128-byte swizzled layout that the
// tcgen05 descriptors name directly (16-byte-atom swizzle for K-major operands, 32-byte-atom
// swizzle for the MN-major operands of dgrad and wgrad).  Only plain per-CTA tensor copies are used.
//
// Return convention of tma_fprop / tma_dgrad / tma_wgrad: AET_OK launched, 1 not eligible (caller
// falls back to the gather producer), negative error.

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

struct TmaKey {
    const void *ptr;
    int tag;
    int box[5];
};
struct TmaEntry {
    TmaKey key;
    CUtensorMap map;
};
struct TmaCache {
    std::deque<TmaEntry> entries;   // a deque never moves its elements: the maps handed out stay valid as the cache grows
};

// dims/strides innermost first; strides[i] is the byte stride of dim i+1.
int get_map(aet_layer *l, int tag, const void *ptr, int rank, const cuuint64_t *dims, const cuuint64_t *strides,
            const cuuint32_t *box, bool mn_major, const CUtensorMap **out) {
    if (!l->tma_cache) l->tma_cache = new TmaCache();
    TmaCache *c = static_cast<TmaCache *>(l->tma_cache);
    TmaKey key = {ptr, tag, {0, 0, 0, 0, 0}};
    for (int i = 0; i < rank; ++i) key.box[i] = (int)box[i];
    for (auto &e : c->entries)
        if (e.key.ptr == key.ptr && e.key.tag == key.tag && memcmp(e.key.box, key.box, sizeof(key.box)) == 0) {
            *out = &e.map;
            return AET_OK;
        }
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        aet_set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
        return AET_E_CUDA;
    }
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    TmaEntry e;
    e.key = key;
    CUresult r = fn(&e.map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void *>(ptr), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        aet_set_error("cuTensorMapEncodeTiled failed with code %d (tag %d)", (int)r, tag);
        return AET_E_CUDA;
    }
    c->entries.push_back(e);
    *out = &c->entries.back().map;
    return AET_OK;
}

struct TmaArgs {
    float *out;
    const float *bias;
    const float *stat_shift;   // fprop: batch-norm statistics of the output (see ConvArgs)
    float *stat_partial;
    int act, bn, n_rows, n_cols, out_ld;
    long long split_stride;
    int slabs_per_tap;   // fprop/dgrad: inner channel count / 32
    int S, pad;
    int pix_per_img, tile_w, img_w;  // M-tile (fprop/dgrad) or K-slab (wgrad) decomposition
    // Maps whose rows do not divide the tile ("ragged": 13x13, 27x27): an M tile (fprop/dgrad) or K slab (wgrad) is
    // `rows_t` whole rows of ONE image, `tiles_per_img` of them per image; the tile's remaining rows stay unused
    // (M: never stored; K: zero in both operands).  0 = dense tiling.
    int tiles_per_img, rows_t, img_h;
    // wgrad on maps wider than a K slab whose width is no multiple of it (55, 56, 112 ...): a slab is 32 columns of ONE
    // row, `row_slabs` of them per row; the last one reaches past the row's end, where the copy engine fills zeros
    // into the delta operand, so the extra products vanish.  0 = off.
    int row_slabs;
    int total_slabs, slabs_per_split;
    int col_blocks;      // wgrad: N tiles per tap
    int m_blocks;        // wgrad: 32-filter blocks of the A operand per stage
    int stages, tmem_cols;
    uint32_t tx_bytes, a_bytes;
    int *status;
    unsigned long long *span;   // profiling: first CTA entry / last CTA exit (null: off)
};

template <int KIND>
__global__ void __launch_bounds__(NTHREADS, 1)
conv_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TmaArgs a) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ SharedCtl ctl;
    span_begin(a.span);
    // 128-byte swizzled tiles must start on a 1024-byte boundary
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int m0 = blockIdx.x * BM;
    int rows_here = a.n_rows - m0;          // rows of this M tile that exist
    int img0 = 0, row0 = 0;                 // fprop/dgrad tile origin
    if (KIND != KIND_WGRAD) {
        if (a.tiles_per_img) {
            img0 = blockIdx.x / a.tiles_per_img;
            row0 = (blockIdx.x - img0 * a.tiles_per_img) * a.rows_t;
            int rows = a.img_h - row0;
            if (rows > a.rows_t) rows = a.rows_t;
            m0 = img0 * a.pix_per_img + row0 * a.tile_w;
            rows_here = rows * a.tile_w;
        } else {
            img0 = m0 / a.pix_per_img;
            row0 = (m0 - img0 * a.pix_per_img) / a.tile_w;
        }
    }
    const int bn = a.bn;
    int n0 = blockIdx.y * bn;   // GEMM column of this tile
    int tap_w = 0, cblk_w = 0;  // wgrad: tap and channel block of this N tile
    if (KIND == KIND_WGRAD) {
        tap_w = blockIdx.y / a.col_blocks;
        cblk_w = blockIdx.y - tap_w * a.col_blocks;
        n0 = tap_w * (a.col_blocks * bn) + cblk_w * bn;
    }
    int slab_begin = 0, nslabs = a.total_slabs;
    const bool split_k = KIND == KIND_WGRAD || gridDim.z > 1;   // forward / data gradient of a layer with few tiles: see fd_splits
    if (split_k) {
        slab_begin = blockIdx.z * a.slabs_per_split;
        nslabs = a.total_slabs - slab_begin;
        if (nslabs > a.slabs_per_split) nslabs = a.slabs_per_split;
        if (nslabs < 0) nslabs = 0;
    }
    const uint32_t b_bytes = (uint32_t)bn * BK * 4;
    const uint32_t stage_bytes = a.a_bytes + b_bytes;

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
    if (KIND == KIND_WGRAD && a.tiles_per_img) {
        // ragged K slabs: the copies fill only the first rows_t * width pixel rows of every 32-row slab; the rest
        // must read as zero in both operands, so the stages start out cleared
        float4 *z = reinterpret_cast<float4 *>(smem_raw + (smem_base - smem_u32(smem_raw)));
        const uint32_t n16 = (uint32_t)a.stages * stage_bytes / 16;
        for (uint32_t i = threadIdx.x; i < n16; i += NTHREADS) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        fence_proxy_async_smem();
        __syncthreads();
    }
    pdl_enter();   // everything above touched only shared memory, TMEM and kernel parameters
    volatile int *abort_flag = &ctl.abort_flag;

    if (warp < 4) {
        if (KIND == KIND_WGRAD && a.tiles_per_img) {
            // ------------------------------------------------------------------ TMA producer, ragged K slabs
            // A slab is one copy per 32-element block of each operand (a block is 4 KB in the swizzled layout, a copy
            // of several blocks would pack them at the box's own, smaller, pitch): seven small copies for four MMAs.
            // Issued by one thread they set the pace of the loop, so the lanes of warp 0 issue one copy each.
            if (warp == 0) {
                const int ncopies = a.m_blocks + bn / 32;
                const int r = tap_w / a.S, sx = tap_w - r * a.S;
                for (int it = 0; it < nslabs; ++it) {
                    const int s = it % a.stages;
                    const uint32_t phase = (it / a.stages) & 1;
                    bool ok = mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const uint32_t bar = smem_u32(&ctl.full[s]);
                    const uint32_t sa = smem_base + (uint32_t)s * stage_bytes;
                    const uint32_t sb = sa + a.a_bytes;
                    if (lane == 0) mbar_arrive_expect_tx(bar, a.tx_bytes);
                    __syncwarp();   // the transaction count is announced before any copy can complete
                    const int sl = slab_begin + it;
                    const int img = sl / a.tiles_per_img;
                    const int oh0 = (sl - img * a.tiles_per_img) * a.rows_t;
                    if (lane < a.m_blocks) {
                        tma_load_5d(sa + lane * 4096u, &map_a, bar, 0, 0, oh0, img, m0 / 32 + lane);
                    } else if (lane < ncopies) {
                        const int q = lane - a.m_blocks;
                        tma_load_5d(sb + q * 4096u, &map_b, bar, 0, sx - a.pad, oh0 + r - a.pad, img, cblk_w * (bn / 32) + q);
                    }
                }
            }
        } else if (threadIdx.x == 0) {
            // ------------------------------------------------------------------ TMA producer
            // CTAs walk the K slabs from different starting points: all of them read the same weight
            // tiles, and marching in lockstep would send every SM to the same L2 lines at once.  The
            // order is a function of the CTA index only, so results stay reproducible.
            const int rot = (KIND == KIND_WGRAD || nslabs == 0) ? 0 : (int)((blockIdx.x * 7u + blockIdx.y * 3u) % (unsigned)nslabs);
            for (int it0 = 0; it0 < nslabs; ++it0) {
                int it = it0 + rot;
                if (it >= nslabs) it -= nslabs;
                const int s = it0 % a.stages;
                const uint32_t phase = (it0 / a.stages) & 1;
                if (!mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag)) break;
                const uint32_t bar = smem_u32(&ctl.full[s]);
                const uint32_t sa = smem_base + (uint32_t)s * stage_bytes;
                const uint32_t sb = sa + a.a_bytes;
                mbar_arrive_expect_tx(bar, a.tx_bytes);
                if (KIND == KIND_FPROP) {
                    const int ig = slab_begin + it;
                    const int tap = ig / a.slabs_per_tap, cb = ig - tap * a.slabs_per_tap;
                    const int r = tap / a.S, sx = tap - r * a.S;
                    tma_load_4d(sa, &map_a, bar, cb * 32, sx - a.pad, row0 + r - a.pad, img0);
                    tma_load_2d(sb, &map_b, bar, ig * 32, n0);
                } else if (KIND == KIND_DGRAD) {
                    const int ig = slab_begin + it;
                    const int tap = ig / a.slabs_per_tap, kb = ig - tap * a.slabs_per_tap;
                    const int r = tap / a.S, sx = tap - r * a.S;
                    tma_load_4d(sa, &map_a, bar, kb * 32, a.pad - sx, row0 + a.pad - r, img0);
                    tma_load_4d(sb, &map_b, bar, 0, kb * 32, n0 / 32, tap);
                } else {
                    int img, oh0, ow0;
                    if (a.row_slabs) {
                        const int sl = slab_begin + it, row = sl / a.row_slabs;
                        ow0 = (sl - row * a.row_slabs) * BK;
                        img = row / a.img_h;
                        oh0 = row - img * a.img_h;
                    } else {
                        const int p0 = (slab_begin + it) * BK;
                        img = p0 / a.pix_per_img;
                        const int rem = p0 - img * a.pix_per_img;
                        oh0 = rem / a.img_w;
                        ow0 = rem - oh0 * a.img_w;
                    }
                    const int r = tap_w / a.S, sx = tap_w - r * a.S;
                    tma_load_5d(sa, &map_a, bar, 0, ow0, oh0, img, m0 / 32);
                    tma_load_5d(sb, &map_b, bar, 0, ow0 + sx - a.pad, oh0 + r - a.pad, img, cblk_w * (bn / 32));
                }
            }
        }
        __syncwarp();
        // ------------------------------------------------------------------ epilogue
        bool ready = nslabs == 0 ? true : mbar_wait(smem_u32(&ctl.accum), 0, abort_flag);
        ready = __all_sync(0xffffffffu, ready);   // the TMEM loads below are warp-collective
        tc_fence_after_sync();
        if (ready) {
            float *obase = a.out + (split_k ? (size_t)blockIdx.z * a.split_stride : 0) + (size_t)m0 * a.out_ld;
            float *tile = reinterpret_cast<float *>(smem_raw + (smem_base - smem_u32(smem_raw)));
            StatAcc st;
            stat_init(st, KIND == KIND_FPROP ? a.stat_partial ? a.stat_shift : nullptr : nullptr);
            store_accumulator<KIND == KIND_FPROP>(tile, tmem, nslabs > 0, warp, lane, bn, obase, (size_t)a.out_ld, rows_here,
                                                  n0, a.n_cols, a.bias, a.act, 1, 1, 0, &st);
            if (KIND == KIND_FPROP && st.shift)
                stats_commit(tile, st, warp, lane, bn, a.stat_partial + (size_t)blockIdx.x * 2 * a.out_ld + n0, a.out_ld, a.n_cols - n0,
                             &ctl.stat_bar, abort_flag);
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const int a_mn = (KIND == KIND_WGRAD) ? 1 : 0;
        const int b_mn = (KIND == KIND_FPROP) ? 0 : 1;
        const uint32_t idesc = make_idesc_tf32(BM, bn, a_mn, b_mn);
        // descriptors are built once; per MMA only the start-address field (16-byte units) advances
        const uint64_t da0 = a_mn ? make_desc(smem_base, 4096, 512, LAYOUT_SW128_32B) : make_desc(smem_base, 0, 1024, LAYOUT_SW128);
        const uint64_t db0 = b_mn ? make_desc(smem_base + a.a_bytes, 4096, 512, LAYOUT_SW128_32B)
                                  : make_desc(smem_base + a.a_bytes, 0, 1024, LAYOUT_SW128);
        const uint64_t a_step = a_mn ? 64 : 2, b_step = b_mn ? 64 : 2;   // 1024 or 32 bytes per K step
        uint32_t accumulate = 0;
        for (int it = 0; it < nslabs; ++it) {
            const int s = it % a.stages;
            const uint32_t phase = (it / a.stages) & 1;
            if (!mbar_wait(smem_u32(&ctl.full[s]), phase, abort_flag)) break;
            tc_fence_after_sync();
            // K-major tiles: 128B swizzle, 16-byte atoms, K advances 32 bytes per MMA inside the row.
            // MN-major tiles: [32-element block][32 k-rows][128 B] in the 32-byte-atom swizzle.
            const uint64_t st16 = (uint64_t)(((uint32_t)s * stage_bytes) >> 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                mma_tf32(tmem, da0 + st16 + j * a_step, db0 + st16 + j * b_step, idesc, accumulate);
                accumulate = 1;
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

// A 128-pixel (or `tile`-pixel) run of consecutive (n,h,w) pixels is a box iff it is whole rows
// of one image or whole images.  Fills box = {w, rows, images}.
bool pixel_box(int tile, int h, int w, cuuint32_t *bw, cuuint32_t *bh, cuuint32_t *bi) {
    if (w <= 0 || h <= 0) return false;
    if (w >= tile) {
        if (w % tile) return false;
        *bw = tile; *bh = 1; *bi = 1;
        return true;
    }
    if (tile % w) return false;
    int rows = tile / w;
    if (h >= rows) {
        if (h % rows) return false;
        *bw = w; *bh = rows; *bi = 1;
        return true;
    }
    if (rows % h) return false;
    *bw = w; *bh = h; *bi = rows / h;
    return bw[0] <= 256 && bh[0] <= 256 && bi[0] <= 256;
}

// Ragged tiling of an h x w map: `tile` / w whole rows per tile (at least one), ceil(h / rows) tiles per image.
// Refused when the tiles would be less than half full (tiny maps): the dense gather kernel is the better choice
// there, and the forward statistics scratch is sized for at most two tiles per 128 pixels.
bool ragged_box(int tile, int h, int w, int *rows, int *per_img) {
    if (w <= 0 || h <= 0 || w > tile) return false;
    *rows = tile / w;
    if (*rows > h) *rows = h;
    *per_img = (h + *rows - 1) / *rows;
    return 2 * h * w >= *per_img * tile;
}

template <int KIND>
int launch_tma(aet_context *ctx, const CUtensorMap *ma, const CUtensorMap *mb, TmaArgs &t, dim3 grid, const char *name,
               double flops) {
    t.tmem_cols = pow2_cols(t.bn);
    t.status = ctx->status_dev;
    const size_t stage = (size_t)t.a_bytes + (size_t)t.bn * BK * 4;
    int stages = (int)((99 * 1024) / stage);
    if (stages < 3) stages = (int)((200 * 1024) / stage);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    t.stages = stages;
    const size_t smem_bytes = stage * stages + 1024;
    AET_TRY(ctx_smem_attr(ctx, conv_tma_kernel<KIND>));
    LaunchScope scope(ctx, name, 0, flops);
    t.span = ctx->span_ptr;
    launch_k(ctx->stream, grid, NTHREADS, smem_bytes, conv_tma_kernel<KIND>, *ma, *mb, t);
    return aet_check_launch(name);
}

// Input channels must fill whole 32-channel (128-byte) rows.  The filter side may be narrower than one
// row (ocp < 32: the copy engine zero-fills the rest of the box) or a whole number of rows.
// (The forward pass reads the filters as rows of a K-major tile, so any filter count works there: rows past the last
// filter are zero-filled by the copy.)
bool tma_common_ok(const aet_layer *l, bool filters_inner = true) {
    const ConvGeom g = layer_geom(l);   // the geometry the kernels see (a fully connected layer is a 1x1 convolution)
    return l->ctx->conv_path == 0 && l->ctx->math == AET_MATH_TF32 && l->groups == 1 && l->dilation == 1 && g.sx == 1 && g.sy == 1 &&
           g.cp % 32 == 0 && (!filters_inner || g.kp % 32 == 0 || g.kp < 32);
}

// A forward pass or data gradient with few output tiles and a long K loop (a fully connected layer at the training
// batch: one 128-row tile, thousands of K slabs) leaves most SMs idle and is bound by what the few CTAs can pull from
// L2.  Its K range is then split over blockIdx.z like the weight gradient's, the partial tiles go to scratch and a
// second kernel sums them (and adds bias and activation).  Returns the split count (1 = do not split).
int fd_splits(const aet_context *ctx, int ctas, int total_slabs) {
    if (!ctx->opt[OPT_FD_SPLIT] || ctas * 2 > ctx->sm_count || total_slabs < 32) return 1;
    int splits = ctx->sm_count / ctas;
    if (splits > 8) splits = 8;
    while (splits > 1 && total_slabs / splits < 16) --splits;
    return splits;
}

int tma_fprop(aet_layer *l, const ConvArgs &a, double flops) {
    const ConvGeom &g = a.g;
    if (!tma_common_ok(l, false)) return 1;
    cuuint32_t bw, bh, bi;
    int rows_t = 0, per_img = 0;
    if (!pixel_box(BM, g.OH, g.OW, &bw, &bh, &bi) || (int)bw != g.OW) {
        if (!l->ctx->opt[OPT_RAGGED] || !ragged_box(BM, g.OH, g.OW, &rows_t, &per_img)) return 1;
        bw = (cuuint32_t)g.OW; bh = (cuuint32_t)rows_t; bi = 1;
    }
    if (g.OW > g.W || g.OH > g.H) return 1;
    int bn = a.bn;                            // any multiple of 16: K-major rows in 8-row swizzle groups
    const int m_tiles_f = per_img ? g.N * per_img : (a.n_rows + BM - 1) / BM;
    int splits = 1;
    if (!a.stat_partial && !per_img) {
        // with the K range split, wide filter tiles are affordable again (the caller shrank them to get more CTAs)
        const int wide = a.n_cols >= 128 ? 128 : bn;
        splits = fd_splits(l->ctx, m_tiles_f * ((a.n_cols + wide - 1) / wide), a.k_total / 32);
        if (splits > 1) bn = wide;
    }
    const CUtensorMap *ma, *mb;
    {
        cuuint64_t dims[4] = {(cuuint64_t)g.cp, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N};
        cuuint64_t str[3] = {(cuuint64_t)g.cp * 4, (cuuint64_t)g.W * g.cp * 4, (cuuint64_t)g.H * g.W * g.cp * 4};
        cuuint32_t box[4] = {32, bw, bh, bi};
        AET_TRY(get_map(l, 0, a.src_a, 4, dims, str, box, false, &ma));
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)a.k_total, (cuuint64_t)g.K};
        cuuint64_t str[1] = {(cuuint64_t)a.k_total * 4};
        cuuint32_t box[2] = {32, (cuuint32_t)bn};
        AET_TRY(get_map(l, 1, a.src_b, 2, dims, str, box, false, &mb));
    }
    TmaArgs t = {};
    t.out = a.out; t.bias = a.bias; t.act = a.act; t.bn = bn;
    t.stat_shift = a.stat_shift; t.stat_partial = a.stat_partial;
    t.n_rows = a.n_rows; t.n_cols = a.n_cols; t.out_ld = a.out_ld;
    t.slabs_per_tap = g.cp / 32; t.S = g.S; t.pad = g.pad;
    t.pix_per_img = g.OH * g.OW; t.tile_w = g.OW; t.img_w = g.OW;
    t.total_slabs = a.k_total / 32; t.slabs_per_split = t.total_slabs;
    t.a_bytes = BM * BK * 4;
    t.tx_bytes = (uint32_t)(bw * bh * bi) * BK * 4 + bn * BK * 4;
    t.tiles_per_img = per_img; t.rows_t = rows_t; t.img_h = g.OH;
    dim3 grid(m_tiles_f, (a.n_cols + bn - 1) / bn, splits);
    if (a.stat_rows_out) *a.stat_rows_out = (int)grid.x;   // only the forward launcher is given one
    if (splits > 1) {
        const size_t out_floats = (size_t)a.n_rows * a.out_ld;
        float *partial = nullptr;
        AET_TRY(ctx_scratch(l->ctx, out_floats * splits * sizeof(float), &partial));
        t.out = partial; t.bias = nullptr; t.act = AET_LINEAR;
        t.split_stride = (long long)out_floats;
        t.slabs_per_split = (t.total_slabs + splits - 1) / splits;
        AET_TRY(launch_tma<KIND_FPROP>(l->ctx, ma, mb, t, grid, "conv_fprop_tma.ks", flops));
        return launch_fprop_reduce(l->ctx, partial, a.out, a.bias, out_floats, a.out_ld, splits, a.act);
    }
    return launch_tma<KIND_FPROP>(l->ctx, ma, mb, t, grid, per_img ? "conv_fprop_tma.ragged" : "conv_fprop_tma", flops);
}

int tma_dgrad(aet_layer *l, const ConvArgs &a, double flops) {
    const ConvGeom &g = a.g;
    // the filters are the K dimension here: a count that is no multiple of 32 ends in a slab whose tail the copy engine
    // zero-fills in both operands (the delta's channel dimension and the weight view's filter dimension end there)
    if (!tma_common_ok(l, false)) return 1;
    if (g.OH != g.H || g.OW != g.W) return 1;   // same-size convolutions only
    cuuint32_t bw, bh, bi;
    int rows_t = 0, per_img = 0;
    if (!pixel_box(BM, g.H, g.W, &bw, &bh, &bi) || (int)bw != g.W) {
        if (!l->ctx->opt[OPT_RAGGED] || !ragged_box(BM, g.H, g.W, &rows_t, &per_img)) return 1;
        bw = (cuuint32_t)g.W; bh = (cuuint32_t)rows_t; bi = 1;
    }
    // N tile: whole 32-channel blocks that divide the channel count; the caller's choice when it qualifies, otherwise
    // the widest divisor up to 256 (384 channels -> 192, 96 -> 96)
    int bn = (a.bn % 32 == 0 && g.cp % a.bn == 0) ? a.bn : 0;
    if (!bn)
        for (int c = 256; c >= 32; c -= 32)
            if (g.cp % c == 0) { bn = c; break; }
    if (!bn) return 1;
    if (!per_img && bn < 256) {
        // where the K range will be split anyway (few tiles, long K), wide channel tiles move fewer bytes per flop
        int wide = bn;
        for (int c = 256; c > bn; c -= 32)
            if (g.cp % c == 0) { wide = c; break; }
        const int m_tiles_d = (a.n_rows + BM - 1) / BM;
        if (wide > bn && fd_splits(l->ctx, m_tiles_d * (a.n_cols / wide), g.R * g.S * ((g.kp + 31) / 32)) > 1) bn = wide;
    }
    const CUtensorMap *ma, *mb;
    {
        cuuint64_t dims[4] = {(cuuint64_t)g.kp, (cuuint64_t)g.OW, (cuuint64_t)g.OH, (cuuint64_t)g.N};
        cuuint64_t str[3] = {(cuuint64_t)g.kp * 4, (cuuint64_t)g.OW * g.kp * 4, (cuuint64_t)g.OH * g.OW * g.kp * 4};
        cuuint32_t box[4] = {32, bw, bh, bi};
        if (get_map(l, 2, a.src_a, 4, dims, str, box, false, &ma) != AET_OK) return g.kp % 32 ? 1 : AET_E_CUDA;
    }
    {
        // weights [filter][tap][cp] viewed as (c%32, filter, c/32, tap)
        const int taps = g.R * g.S;
        cuuint64_t dims[4] = {32, (cuuint64_t)g.K, (cuuint64_t)g.cp / 32, (cuuint64_t)taps};
        cuuint64_t str[3] = {(cuuint64_t)taps * g.cp * 4, 128, (cuuint64_t)g.cp * 4};
        cuuint32_t box[4] = {32, 32, (cuuint32_t)bn / 32, 1};
        AET_TRY(get_map(l, 3, a.src_b, 4, dims, str, box, true, &mb));
    }
    TmaArgs t = {};
    t.out = a.out; t.bias = nullptr; t.act = AET_LINEAR; t.bn = bn;
    t.n_rows = a.n_rows; t.n_cols = a.n_cols; t.out_ld = a.out_ld;
    t.slabs_per_tap = (g.kp + 31) / 32; t.S = g.S; t.pad = g.pad;
    t.pix_per_img = g.H * g.W; t.tile_w = g.W; t.img_w = g.W;
    t.total_slabs = g.R * g.S * t.slabs_per_tap; t.slabs_per_split = t.total_slabs;
    t.a_bytes = BM * BK * 4;
    t.tx_bytes = (uint32_t)(bw * bh * bi) * BK * 4 + bn * BK * 4;
    t.tiles_per_img = per_img; t.rows_t = rows_t; t.img_h = g.H;
    dim3 grid(per_img ? g.N * per_img : (a.n_rows + BM - 1) / BM, (a.n_cols + bn - 1) / bn, 1);
    if (a.stat_rows_out) *a.stat_rows_out = (int)grid.x;   // only the forward launcher is given one
    const int splits = per_img ? 1 : fd_splits(l->ctx, (int)(grid.x * grid.y), t.total_slabs);
    if (splits > 1) {
        const size_t out_floats = (size_t)a.n_rows * a.out_ld;
        float *partial = nullptr;
        AET_TRY(ctx_scratch(l->ctx, out_floats * splits * sizeof(float), &partial));
        t.out = partial;
        t.split_stride = (long long)out_floats;
        t.slabs_per_split = (t.total_slabs + splits - 1) / splits;
        grid.z = splits;
        AET_TRY(launch_tma<KIND_DGRAD>(l->ctx, ma, mb, t, grid, "conv_dgrad_tma.ks", flops));
        return launch_wgrad_reduce(l->ctx, partial, a.out, out_floats, splits, 0);
    }
    return launch_tma<KIND_DGRAD>(l->ctx, ma, mb, t, grid, per_img ? "conv_dgrad_tma.ragged" : "conv_dgrad_tma", flops);
}

// `a.out` already points at the split-K partial buffer sized for `splits_hint` splits of the
// gather decomposition; the TMA variant keeps the same split count and partial layout.
int tma_wgrad(aet_layer *l, ConvArgs &a, int splits_hint, double flops) {
    const ConvGeom &g = a.g;
    if (!tma_common_ok(l)) return 1;
    if (g.OW > g.W || g.OH > g.H) return 1;
    cuuint32_t bw, bh, bi;
    int rows_t = 0, per_img = 0;
    int row_slabs = 0;
    if (!pixel_box(BK, g.OH, g.OW, &bw, &bh, &bi)) {
        if (!l->ctx->opt[OPT_RAGGED]) return 1;
        if (g.OW > BK) {
            row_slabs = (g.OW + BK - 1) / BK;   // 32-column slabs of one row, the last one zero-filled past the row's end
            bw = BK; bh = 1; bi = 1;
        } else {
            if (g.OW != g.W || g.OH != g.H || g.kp % 32 || !ragged_box(BK, g.OH, g.OW, &rows_t, &per_img)) return 1;
            bw = (cuuint32_t)g.OW; bh = (cuuint32_t)rows_t; bi = 1;
        }
    }
    const int bn = g.cp <= 256 ? g.cp : (g.cp % 256 == 0 ? 256 : (g.cp % 128 == 0 ? 128 : 0));
    if (!bn) return 1;
    const int k_blocks = (g.kp + 31) / 32;
    const int m_blocks = k_blocks < 4 ? k_blocks : 4;
    const CUtensorMap *ma, *mb;
    {
        cuuint64_t dims[5] = {(cuuint64_t)(g.kp < 32 ? g.kp : 32), (cuuint64_t)g.OW, (cuuint64_t)g.OH, (cuuint64_t)g.N,
                              (cuuint64_t)k_blocks};
        cuuint64_t str[4] = {(cuuint64_t)g.kp * 4, (cuuint64_t)g.OW * g.kp * 4, (cuuint64_t)g.OH * g.OW * g.kp * 4, 128};
        cuuint32_t box[5] = {32, bw, bh, bi, (cuuint32_t)(per_img ? 1 : m_blocks)};
        if (get_map(l, 4, a.src_a, 5, dims, str, box, true, &ma) != AET_OK) return g.kp % 32 ? 1 : AET_E_CUDA;
    }
    {
        cuuint64_t dims[5] = {32, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N, (cuuint64_t)g.cp / 32};
        cuuint64_t str[4] = {(cuuint64_t)g.cp * 4, (cuuint64_t)g.W * g.cp * 4, (cuuint64_t)g.H * g.W * g.cp * 4, 128};
        cuuint32_t box[5] = {32, bw, bh, bi, (cuuint32_t)(per_img ? 1 : bn / 32)};
        AET_TRY(get_map(l, 5, a.src_b, 5, dims, str, box, true, &mb));
    }
    TmaArgs t = {};
    t.out = a.out; t.bias = nullptr; t.act = AET_LINEAR; t.bn = bn;
    t.n_rows = a.n_rows; t.n_cols = a.n_cols; t.out_ld = a.out_ld;
    t.split_stride = a.split_stride;
    t.S = g.S; t.pad = g.pad;
    t.pix_per_img = g.OH * g.OW; t.tile_w = g.OW; t.img_w = g.OW;
    t.total_slabs = (a.k_total + BK - 1) / BK;
    t.slabs_per_split = a.k_per_split / BK;
    t.col_blocks = g.cp / bn;
    t.m_blocks = m_blocks;
    t.a_bytes = BM * BK * 4;                                   // stage slot; the copy fills m_blocks * 4 KB of it
    t.tx_bytes = (uint32_t)m_blocks * 4096 + (uint32_t)bn * BK * 4;
    if (per_img) {
        // slabs are rows_t rows of one image; the split count and the partial buffer stay the caller's
        t.tiles_per_img = per_img; t.rows_t = rows_t; t.img_h = g.OH;
        t.total_slabs = g.N * per_img;
        t.slabs_per_split = (t.total_slabs + splits_hint - 1) / splits_hint;
        t.tx_bytes = (uint32_t)(m_blocks + bn / 32) * (uint32_t)(bw * bh) * 128u;
    }
    if (row_slabs) {
        t.row_slabs = row_slabs; t.img_h = g.OH;
        t.total_slabs = g.N * g.OH * row_slabs;
        t.slabs_per_split = (t.total_slabs + splits_hint - 1) / splits_hint;
    }
    const int m_tiles = (g.K + BM - 1) / BM;
    dim3 grid(m_tiles, g.R * g.S * t.col_blocks, splits_hint);
    return launch_tma<KIND_WGRAD>(l->ctx, ma, mb, t, grid, per_img ? "conv_wgrad_tma.ragged" : (row_slabs ? "conv_wgrad_tma.wide" : "conv_wgrad_tma"), flops);
}

void tma_release(aet_layer *l) {
    if (l->tma_cache) {
        delete static_cast<TmaCache *>(l->tma_cache);
        l->tma_cache = nullptr;
    }
}

}  // namespace
