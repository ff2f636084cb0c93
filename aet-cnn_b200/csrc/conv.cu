// Convolution forward / backward-data / backward-weight as implicit GEMMs on the sm_100a
// tensor cores (tcgen05.mma kind::tf32, FP32 accumulators in TMEM).  No im2col buffer exists:
// operand tiles are assembled in shared memory straight from the NHWC activations.
//
// Replaces the per-image im2col + SGEMM (+ col2im) loops of the reference:
//   forward   mtcs/MtcsConvLayer.c:78-149   (dnn/ConvolutionalLayer.c:717-806)
//   backward  mtcs/MtcsConvLayer.c:332-409  (dnn/ConvolutionalLayer.c:909-947)
//
// GEMM views (M x N x K), all with a 128-row M tile:
//   fprop  M = output pixels (n,oh,ow)   N = filters           K = (tap, input channel)
//   dgrad  M = input pixels  (n,h,w)     N = input channels    K = (tap, filter)
//   wgrad  M = filters                   N = (tap, in channel) K = output pixels, split over CTAs
//
// Two producers feed the same MMA/epilogue skeleton:
//   * gather producer: 128 threads build the tiles with 16-byte loads into the un-swizzled
//     core-matrix layout (any size / stride / padding / ragged edge);
//   * TMA producer (conv_tma.cuh): one thread issues tiled bulk-tensor copies with out-of-bounds
//     zero fill into 128-byte-swizzled tiles (stride-1 convolutions whose 128-pixel tile is a
//     whole number of image rows, channel count a multiple of 32).
//
// CTA = 5 warps: warps 0-3 produce and later run the epilogue (TMEM lane quarter = warp id),
// warp 4 allocates TMEM and its lane 0 issues every MMA.
#include "common.h"
#include "umma.cuh"
#include "activation.cuh"
#include <cooperative_groups.h>
#include <deque>

using namespace umma;

namespace {

enum { KIND_FPROP = 0, KIND_DGRAD = 1, KIND_WGRAD = 2 };
constexpr int BM = 128;        // MMA M
constexpr int BK = 32;         // K elements per pipeline stage (4 MMAs of K=8)
constexpr int MAX_STAGES = 6;
constexpr int NTHREADS = 160;

struct ConvArgs {
    ConvGeom g;
    const float *src_a;   // fprop: x      dgrad: dy      wgrad: dy
    const float *src_b;   // fprop: w      dgrad: w       wgrad: x
    float *out;           // fprop: y      dgrad: dx      wgrad: split-K partials
    const float *bias;    // fprop epilogue, may be null
    const float *stat_shift;   // fprop: accumulate batch-norm statistics of the output around this per-channel shift
    float *stat_partial;       //        into one row [2][out_ld] per CTA along M (null: off)
    int *stat_rows_out;        // host side: the launcher stores the number of partial rows (its grid.x) here
    int act;              // fprop epilogue activation
    int bn;               // N tile (multiple of 16, <= 256)
    int n_rows, n_cols;   // valid GEMM M and N extents
    int k_total;          // GEMM K extent
    int k_per_split;      // K handled by one blockIdx.z (multiple of BK)
    int out_ld;
    long long split_stride;
    int stages, x3, tmem_cols;
    int *status;
};

struct SharedCtl {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long accum, stat_bar, stat_bar2;
    uint32_t tmem_base;
    int abort_flag;
    int4 jtab[64];  // wgrad: per 4-column chunk of the N tile -> {r, s, c, valid}
};

__device__ __forceinline__ float apply_act(float v, int act) { return act_forward(v, act); }

__device__ __forceinline__ float4 ldg4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }

__device__ __forceinline__ void st_cell(unsigned char *stage, uint32_t off, uint32_t lo_off, float4 v, int x3) {
    if (x3) {
        float4 hi, lo;
        hi.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
        hi.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
        hi.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
        hi.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
        lo.x = v.x - hi.x; lo.y = v.y - hi.y; lo.z = v.z - hi.z; lo.w = v.w - hi.w;
        *reinterpret_cast<float4 *>(stage + off) = hi;
        *reinterpret_cast<float4 *>(stage + lo_off + off) = lo;
    } else {
        *reinterpret_cast<float4 *>(stage + off) = v;
    }
}

// Epilogue of one accumulator: TMEM -> registers -> shared memory (the idle pipeline stages, row
// pitch bn+4 floats so that a quarter warp of consecutive rows hits eight distinct 16-byte bank
// groups) -> global memory with lanes along the COLUMNS of one row.  A thread owns a TMEM lane = an
// output row, so storing straight from registers would make every warp store touch 32 rows
// 512 or more bytes apart (measured: 10 us for a 128x128 tile, half the kernel); through shared
// memory every store instruction writes one contiguous row segment.
// Each warp only re-reads the 32 rows it wrote itself: __syncwarp is the only synchronisation.
// Per-lane running sums of the batch-norm statistics a forward epilogue gathers on the way out:
// sum (y - shift) and sum (y - shift)^2 of the lane's four columns of each 128-column chunk, over
// every valid row the warp stores.  shift == null switches them off.
struct StatAcc {
    const float *shift;
    float4 s1[2], s2[2];
};
__device__ __forceinline__ void stat_init(StatAcc &st, const float *shift) {
    st.shift = shift;
    st.s1[0] = st.s1[1] = st.s2[0] = st.s2[1] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// Phase one of the epilogue: TMEM -> this warp's 32 rows of the staging tile, 32 columns (two loads in
// flight) per wait.
// `tmem_acc2` (0 = none): a second accumulator of the same tile holding the other half of the K steps (the MMA issuer
// alternates between the two so that consecutive MMAs do not depend on each other); the two are added on the way.
__device__ __forceinline__ void stage_accumulator(float *tile, uint32_t tmem_acc, bool have_acc, int warp, int lane, int bn,
                                                  uint32_t tmem_acc2 = 0) {
    const int pitch = bn + 4;
    float *mine = tile + (size_t)(warp * 32 + lane) * pitch;
    for (int cc = 0; cc < bn; cc += 32) {
        uint32_t v[32];
        const bool second = cc + 16 < bn;
        if (have_acc) {
            tmem_ld16_issue(tmem_acc + ((uint32_t)(warp * 32) << 16) + (uint32_t)cc, v);
            if (second) tmem_ld16_issue(tmem_acc + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cc + 16), v + 16);
            if (tmem_acc2) {
                uint32_t w[32];
                tmem_ld16_issue(tmem_acc2 + ((uint32_t)(warp * 32) << 16) + (uint32_t)cc, w);
                if (second) tmem_ld16_issue(tmem_acc2 + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cc + 16), w + 16);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 32; ++q)
                    if (q < 16 || second) v[q] = __float_as_uint(__uint_as_float(v[q]) + __uint_as_float(w[q]));
            } else {
                tmem_ld_wait();
            }
        } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = 0u;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
            if (q < 4 || second)
                *reinterpret_cast<uint4 *>(mine + cc + q * 4) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    }
    __syncwarp();
}

// Phase two: staging tile -> global memory.  `remote` (may be null) is the staging tile of the cluster's
// other CTA, which accumulated the other half of the K range: its rows are added on the way out.
template <bool FPROP>
__device__ __forceinline__ void flush_tile(const float *tile, const float *remote, int warp, int lane, int bn,
                                           float *out, size_t out_ld, int rows_valid, int col_base, int n_cols,
                                           const float *bias, int act, int map_bi, int map_w, int map_pix, StatAcc *st,
                                           int row_lo = 0, int row_hi = 32) {
    // [row_lo, row_hi): the part of this warp's 32 rows to store (multiples of 16; the whole block by default)
    const int pitch = bn + 4;
    // tiles that span several small images order their rows (h, image, w): each lane maps one row to
    // its pixel index once (the divisions cost more than the stores) and the others fetch it by shuffle
    int my_grow = warp * 32 + lane;
    if (map_bi > 1) my_grow = ((my_grow / map_w) % map_bi) * map_pix + (my_grow / (map_bi * map_w)) * map_w + my_grow % map_w;
    // a store instruction covers whole rows, 32 / lpr of them when the tile is narrower than 128
    // columns; four rows are read before they are written so that the latencies overlap
    const int lpr = bn >= 128 ? 32 : bn / 4;          // lanes per row (bn is a multiple of 16)
    const int rpi = 32 / lpr;                         // rows per instruction
    const int sub = lane / lpr, lcol = (lane - sub * lpr) * 4;
    for (int c0 = 0; c0 < bn; c0 += 128) {
        const int c = c0 + lcol;
        const int col = col_base + c;
        const bool active = c < bn && col < n_cols && sub < rpi;
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (FPROP && bias && active) b = ldg4(bias + col);
        const bool stats = FPROP && st && st->shift;
        float4 sh = make_float4(0.f, 0.f, 0.f, 0.f);
        if (stats && active) sh = ldg4(st->shift + col);
        float4 t1 = make_float4(0.f, 0.f, 0.f, 0.f), t2 = t1;
        for (int r0 = row_lo; r0 < row_hi; r0 += 4 * rpi) {
            float4 o[4];
            int grow[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int r = (r0 + u * rpi + sub) & 31;
                grow[u] = __shfl_sync(0xffffffffu, my_grow, r);
                if (r0 + u * rpi + sub >= row_hi) grow[u] = rows_valid;   // past the rows to store (lpr not a divisor of 32)
                const size_t off = (size_t)(warp * 32 + r) * pitch + c * (active ? 1 : 0);
                o[u] = *reinterpret_cast<const float4 *>(tile + off);
                if (remote) {
                    const float4 q = *reinterpret_cast<const float4 *>(remote + off);
                    o[u].x += q.x; o[u].y += q.y; o[u].z += q.z; o[u].w += q.w;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (!active || grow[u] >= rows_valid) continue;
                float4 v = o[u];
                if (stats) {
                    const float dx = v.x - sh.x, dy = v.y - sh.y, dz = v.z - sh.z, dw = v.w - sh.w;
                    t1.x += dx; t1.y += dy; t1.z += dz; t1.w += dw;
                    t2.x += dx * dx; t2.y += dy * dy; t2.z += dz * dz; t2.w += dw * dw;
                }
                if (FPROP) {
                    v.x = apply_act(v.x + b.x, act); v.y = apply_act(v.y + b.y, act);
                    v.z = apply_act(v.z + b.z, act); v.w = apply_act(v.w + b.w, act);
                }
                *reinterpret_cast<float4 *>(out + (size_t)grow[u] * out_ld + col) = v;
            }
        }
        if (stats) {   // constant indices keep the sums in registers
            if (c0 == 0) {
                st->s1[0].x += t1.x; st->s1[0].y += t1.y; st->s1[0].z += t1.z; st->s1[0].w += t1.w;
                st->s2[0].x += t2.x; st->s2[0].y += t2.y; st->s2[0].z += t2.z; st->s2[0].w += t2.w;
            } else {
                st->s1[1].x += t1.x; st->s1[1].y += t1.y; st->s1[1].z += t1.z; st->s1[1].w += t1.w;
                st->s2[1].x += t2.x; st->s2[1].y += t2.y; st->s2[1].z += t2.z; st->s2[1].w += t2.w;
            }
        }
    }
    __syncwarp();
}

template <bool FPROP>
__device__ __forceinline__ void store_accumulator(float *tile, uint32_t tmem_acc, bool have_acc, int warp, int lane, int bn,
                                                  float *out, size_t out_ld, int rows_valid, int col_base, int n_cols,
                                                  const float *bias, int act, int map_bi = 1, int map_w = 1, int map_pix = 0,
                                                  StatAcc *st = nullptr, uint32_t tmem_acc2 = 0) {
    stage_accumulator(tile, tmem_acc, have_acc, warp, lane, bn, tmem_acc2);
    flush_tile<FPROP>(tile, nullptr, warp, lane, bn, out, out_ld, rows_valid, col_base, n_cols, bias, act, map_bi, map_w, map_pix, st);
}

// Ends a forward CTA's statistics: folds the lanes that hold the same columns, parks each epilogue
// warp's sums in its own rows of the staging tile, and lets epilogue warp 0 add the four warps in a
// fixed order into the CTA's partial row (row[c] = sum, row[ld + c] = sum of squares).  The wait is
// bounded like every other; after a timeout the row is simply not written.
__device__ __forceinline__ void stats_commit(float *tile, StatAcc &st, int warp, int lane, int bn, float *row, int ld, int cols_left,
                                             unsigned long long *bar, volatile int *abort_flag) {
    const int pitch = bn + 4;
    const int lpr = bn >= 128 ? 32 : bn / 4, rpi = 32 / lpr;
    const int sub = lane / lpr, lcol = (lane - sub * lpr) * 4;
    float *mine = tile + (size_t)(warp * 32) * pitch;
    for (int c0 = 0; c0 < bn; c0 += 128) {
        const float4 o1 = c0 == 0 ? st.s1[0] : st.s1[1], o2 = c0 == 0 ? st.s2[0] : st.s2[1];
        float4 a1 = o1, a2 = o2;
        for (int k = 1; k < rpi; ++k) {
            const int src = lane + k * lpr;   // lanes past the warp return their own value; only sub 0 keeps the result
            a1.x += __shfl_sync(0xffffffffu, o1.x, src); a1.y += __shfl_sync(0xffffffffu, o1.y, src);
            a1.z += __shfl_sync(0xffffffffu, o1.z, src); a1.w += __shfl_sync(0xffffffffu, o1.w, src);
            a2.x += __shfl_sync(0xffffffffu, o2.x, src); a2.y += __shfl_sync(0xffffffffu, o2.y, src);
            a2.z += __shfl_sync(0xffffffffu, o2.z, src); a2.w += __shfl_sync(0xffffffffu, o2.w, src);
        }
        const int c = c0 + lcol;
        if (sub == 0 && c < bn) {
            *reinterpret_cast<float4 *>(mine + c) = a1;
            *reinterpret_cast<float4 *>(mine + bn + c) = a2;
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(bar));
    if (warp != 0) return;
    if (!mbar_wait(smem_u32(bar), 0, abort_flag)) return;
    for (int c = lane; c < bn && c < cols_left; c += 32) {
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            s1 += tile[(size_t)(w * 32) * pitch + c];
            s2 += tile[(size_t)(w * 32) * pitch + bn + c];
        }
        row[c] = s1;
        row[ld + c] = s2;
    }
}

// Byte offset of the 16-byte cell holding M/N elements 4*mc..4*mc+3 at K index k (0..31) inside an
// MN-major tile stored as [32-element block][32 k-rows][128 B] in the 128B / 32-byte-atom swizzle.
__device__ __forceinline__ uint32_t mn_cell_offset(int mc, int k) {
    return (uint32_t)(mc >> 3) * 4096u + (uint32_t)(k >> 2) * 512u + (uint32_t)(k & 3) * 128u +
           (uint32_t)((((mc & 7) >> 1) ^ (k & 3)) * 32) + (uint32_t)(mc & 1) * 16u;
}

// NB = B-operand cells per producer thread and stage (N tile <= 16*NB).
template <int KIND, int NB>
__global__ void __launch_bounds__(NTHREADS, NB <= 4 ? 3 : 1) conv_gather_kernel(const ConvArgs a) {
    extern __shared__ unsigned char smem_raw[];
    // swizzled MN-major tiles need their 512-byte atoms aligned; align every stage to 1024 bytes
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ SharedCtl ctl;

    const ConvGeom &g = a.g;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM;
    const int n0 = blockIdx.y * a.bn;
    const int bn = a.bn;
    const int k_begin = (KIND == KIND_WGRAD) ? blockIdx.z * a.k_per_split : 0;
    int k_end = (KIND == KIND_WGRAD) ? k_begin + a.k_per_split : a.k_total;
    if (k_end > a.k_total) k_end = a.k_total;
    const int nslabs = (k_end > k_begin) ? (k_end - k_begin + BK - 1) / BK : 0;

    const uint32_t a_bytes = BM * BK * 4;
    const uint32_t b_bytes = ((bn + 31) / 32) * 32 * BK * 4;
    const uint32_t half_bytes = a_bytes + b_bytes;            // one precision half of a stage
    const uint32_t stage_bytes = half_bytes * (a.x3 ? 2 : 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 128);
            mbar_init(smem_u32(&ctl.empty[s]), 1);
        }
        mbar_init(smem_u32(&ctl.accum), 1);
        mbar_init(smem_u32(&ctl.stat_bar), 4);
        ctl.abort_flag = 0;
        fence_barrier_init();
    }
    if (KIND == KIND_WGRAD && threadIdx.x < 64) {
        int4 e = make_int4(0, 0, 0, 0);
        int j = n0 + threadIdx.x * 4;
        if ((int)threadIdx.x * 4 < bn && j < a.n_cols) {
            int tap = j / g.cp;
            e.z = j - tap * g.cp;
            e.x = tap / g.S;
            e.y = tap - e.x * g.S;
            e.w = 1;
        }
        ctl.jtab[threadIdx.x] = e;
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
        // ------------------------------------------------------------------ producer
        // K-major operands: a thread owns 4 rows x 2 sixteen-byte cells; a warp instruction
        // touches 8 rows x 4 cells (128 contiguous bytes of shared memory per quarter warp).
        int rinfo_base[4], rinfo_y[4], rinfo_x[4];
        if (KIND != KIND_WGRAD) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int m = m0 + (warp + 4 * i) * 8 + (lane & 7);
                if (m < a.n_rows) {
                    if (KIND == KIND_FPROP) {
                        int n = m / (g.OH * g.OW);
                        int rem = m - n * g.OH * g.OW;
                        int oh = rem / g.OW, ow = rem - oh * g.OW;
                        rinfo_base[i] = n * g.H * g.W;
                        rinfo_y[i] = oh * g.sy - g.pad * g.dil;
                        rinfo_x[i] = ow * g.sx - g.pad * g.dil;
                    } else {
                        int n = m / (g.H * g.W);
                        int rem = m - n * g.H * g.W;
                        int h = rem / g.W, w = rem - h * g.W;
                        rinfo_base[i] = n * g.OH * g.OW;
                        rinfo_y[i] = h + g.pad * g.dil;
                        rinfo_x[i] = w + g.pad * g.dil;
                    }
                } else {
                    rinfo_base[i] = 0;
                    rinfo_y[i] = -(1 << 28);
                    rinfo_x[i] = -(1 << 28);
                }
            }
        }
        const int kc_lo = lane >> 3;  // first of the thread's two K cells (second is +4)
        // MN-major operands: a warp instruction covers 8 k-rows x 4 cells; this lane split makes each
        // quarter warp hit eight distinct 16-byte slots of the swizzled rows (no bank conflicts)
        const int mn_k = (lane & 3) + 4 * ((lane >> 3) & 1);
        const int mn_c = ((lane >> 2) & 1) + 2 * ((lane >> 4) & 1);
        const int nb_groups = bn / 16;  // B groups handled per warp

        for (int it = 0; it < nslabs; ++it) {
            const int s = it % a.stages;
            const uint32_t phase = (it / a.stages) & 1;
            const int k0 = k_begin + it * BK;
            unsigned char *stage = smem + (size_t)s * stage_bytes;
            float4 va[8];
            uint32_t oa[8];

            if (KIND != KIND_WGRAD) {
                // ---- A: K-major gather
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int kc = kc_lo + 4 * h;
                    const int kk = k0 + kc * 4;
                    int tap = 0, ch = 0, r = 0, sx_ = 0;
                    const bool kvalid = kk < k_end;
                    const int inner = (KIND == KIND_FPROP) ? g.cp : g.kp;
                    if (kvalid) {
                        tap = kk / inner;
                        ch = kk - tap * inner;
                        r = tap / g.S;
                        sx_ = tap - r * g.S;
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (kvalid) {
                            if (KIND == KIND_FPROP) {
                                int ih = rinfo_y[i] + r * g.dil, iw = rinfo_x[i] + sx_ * g.dil;
                                if ((unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W)
                                    v = ldg4(a.src_a + ((size_t)(rinfo_base[i] + ih * g.W + iw) * g.xs + ch));
                            } else {
                                int th = rinfo_y[i] - r * g.dil, tw = rinfo_x[i] - sx_ * g.dil;
                                if (th >= 0 && tw >= 0) {
                                    int oh = th / g.sy, ow = tw / g.sx;
                                    if (oh * g.sy == th && ow * g.sx == tw && oh < g.OH && ow < g.OW)
                                        v = ldg4(a.src_a + ((size_t)(rinfo_base[i] + oh * g.OW + ow) * g.ys + ch));
                                }
                            }
                        }
                        const int row = (warp + 4 * i) * 8 + (lane & 7);
                        va[h * 4 + i] = v;
                        oa[h * 4 + i] = (uint32_t)kc * (BM * 16) + (uint32_t)row * 16;
                    }
                }
            } else {
                // ---- A: MN-major gather from dy: one pixel per thread, 8 channel cells
                const int kq = warp * 8 + mn_k;
                const int p = k0 + kq;
                const bool pvalid = p < k_end;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int mc = i * 4 + mn_c;
                    const int ko = m0 + mc * 4;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (pvalid && ko < g.kp) v = ldg4(a.src_a + ((size_t)p * g.ys + ko));
                    va[i] = v;
                    oa[i] = mn_cell_offset(mc, kq);
                }
            }

            // ---- B: all loads of the stage are issued before anything is stored, so that their
            // latencies overlap instead of adding up
            unsigned char *stage_b = stage + a_bytes;
            float4 vb[NB];
            uint32_t ob[NB];
            if (KIND == KIND_FPROP) {
                // K-major, rows = filters
#pragma unroll
                for (int i = 0; i < NB; ++i) {
                    if (i >= nb_groups) break;
                    const int gi = warp + 4 * i;
                    const int rb = gi % (bn / 8), half = gi / (bn / 8);
                    const int row = rb * 8 + (lane & 7);
                    const int kc = half * 4 + (lane >> 3);
                    const int kk = k0 + kc * 4;
                    const int j = n0 + row;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (j < g.K && kk < k_end) v = ldg4(a.src_b + ((size_t)j * a.k_total + kk));
                    vb[i] = v;
                    ob[i] = (uint32_t)kc * (bn * 16) + (uint32_t)row * 16;
                }
            } else if (KIND == KIND_DGRAD) {
                // MN-major, rows = input channels (contiguous in the weight tensor), K = (tap, filter)
                const int kq = warp * 8 + mn_k;
                const int kk = k0 + kq;
                int tap = 0, ko = 0;
                const bool kvalid = kk < k_end;
                if (kvalid) { tap = kk / g.kp; ko = kk - tap * g.kp; }
                const bool fvalid = kvalid && ko < g.K;
                const float *wrow = a.src_b + ((size_t)ko * (g.R * g.S) + tap) * g.cp;
#pragma unroll
                for (int i = 0; i < NB; ++i) {
                    if (i >= nb_groups) break;
                    const int mc = i * 4 + mn_c;
                    const int c = n0 + mc * 4;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (fvalid && c < g.cp) v = ldg4(wrow + c);
                    vb[i] = v;
                    ob[i] = mn_cell_offset(mc, kq);
                }
            } else {
                // MN-major gather from x, rows = (tap, channel), K = output pixel
                const int kq = warp * 8 + mn_k;
                const int p = k0 + kq;
                const bool pvalid = p < k_end;
                int nb = 0, ih0 = 0, iw0 = 0;
                if (pvalid) {
                    int n = p / (g.OH * g.OW);
                    int rem = p - n * g.OH * g.OW;
                    int oh = rem / g.OW, ow = rem - oh * g.OW;
                    nb = n * g.H * g.W;
                    ih0 = oh * g.sy - g.pad * g.dil;
                    iw0 = ow * g.sx - g.pad * g.dil;
                }
#pragma unroll
                for (int i = 0; i < NB; ++i) {
                    if (i >= nb_groups) break;
                    const int mc = i * 4 + mn_c;
                    const int4 e = ctl.jtab[mc];
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (pvalid && e.w) {
                        int ih = ih0 + e.x * g.dil, iw = iw0 + e.y * g.dil;
                        if ((unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W)
                            v = ldg4(a.src_b + ((size_t)(nb + ih * g.W + iw) * g.xs + e.z));
                    }
                    vb[i] = v;
                    ob[i] = mn_cell_offset(mc, kq);
                }
            }
            if (!mbar_wait(smem_u32(&ctl.empty[s]), phase ^ 1, abort_flag)) break;
#pragma unroll
            for (int i = 0; i < 8; ++i) st_cell(stage, oa[i], half_bytes, va[i], a.x3);
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                if (i >= nb_groups) break;
                st_cell(stage_b, ob[i], half_bytes, vb[i], a.x3);
            }
            fence_proxy_async_smem();
            mbar_arrive(smem_u32(&ctl.full[s]));
        }

        // ------------------------------------------------------------------ epilogue
        bool ready = nslabs == 0 ? true : mbar_wait(smem_u32(&ctl.accum), 0, abort_flag);
        ready = __all_sync(0xffffffffu, ready);   // the TMEM loads below are warp-collective
        tc_fence_after_sync();
        if (ready) {
            float *obase = a.out + (KIND == KIND_WGRAD ? (size_t)blockIdx.z * a.split_stride : 0) + (size_t)m0 * a.out_ld;
            StatAcc st;
            stat_init(st, KIND == KIND_FPROP ? a.stat_partial ? a.stat_shift : nullptr : nullptr);
            store_accumulator<KIND == KIND_FPROP>(reinterpret_cast<float *>(smem), tmem, nslabs > 0, warp, lane, bn, obase,
                                                  (size_t)a.out_ld, a.n_rows - m0, n0, a.n_cols, a.bias, a.act, 1, 1, 0, &st);
            if (KIND == KIND_FPROP && st.shift)
                stats_commit(reinterpret_cast<float *>(smem), st, warp, lane, bn, a.stat_partial + (size_t)blockIdx.x * 2 * a.out_ld + n0,
                             a.out_ld, a.n_cols - n0, &ctl.stat_bar, abort_flag);
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        const int a_mn = (KIND == KIND_WGRAD) ? 1 : 0;
        const int b_mn = (KIND == KIND_FPROP) ? 0 : 1;
        const uint32_t idesc = make_idesc_tf32(BM, bn, a_mn, b_mn);
        // Descriptors are built once; per MMA only the start-address field (16-byte units) advances.
        // K-major: un-swizzled core matrices, two 16-byte K chunks per MMA at LBO, 8-row groups at SBO.
        // MN-major: 128B / 32-byte-atom swizzle, 32-element blocks at LBO, 4-k atoms at SBO.
        const uint32_t s0 = smem_u32(smem);
        const uint64_t da0 = a_mn ? make_desc(s0, 4096, 512, LAYOUT_SW128_32B) : make_desc(s0, BM * 16, 128, LAYOUT_NONE);
        const uint64_t db0 = b_mn ? make_desc(s0 + a_bytes, 4096, 512, LAYOUT_SW128_32B) : make_desc(s0 + a_bytes, bn * 16, 128, LAYOUT_NONE);
        const uint64_t a_step = a_mn ? 64 : (2 * BM * 16) >> 4, b_step = b_mn ? 64 : (uint64_t)((2 * bn * 16) >> 4);
        const uint64_t lo16 = (uint64_t)(half_bytes >> 4);
        uint32_t accumulate = 0;
        for (int it = 0; it < nslabs; ++it) {
            const int s = it % a.stages;
            const uint32_t phase = (it / a.stages) & 1;
            if (!mbar_wait(smem_u32(&ctl.full[s]), phase, abort_flag)) break;
            tc_fence_after_sync();
            const uint64_t st16 = (uint64_t)(((uint32_t)s * stage_bytes) >> 4);
            const int k0 = k_begin + it * BK;
            int ksteps = (k_end - k0 + 7) / 8;
            if (ksteps > 4) ksteps = 4;
            for (int j = 0; j < ksteps; ++j) {
                const uint64_t da = da0 + st16 + j * a_step, db = db0 + st16 + j * b_step;
                if (a.x3) {
                    mma_tf32(tmem, da + lo16, db, idesc, accumulate);
                    mma_tf32(tmem, da, db + lo16, idesc, 1);
                    mma_tf32(tmem, da, db, idesc, 1);
                } else {
                    mma_tf32(tmem, da, db, idesc, accumulate);
                }
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
}

// Fixed-order second stage of the split-K weight gradient: dw (+)= sum over splits.  `lanes` (a power of two, at
// most 32) threads of a warp share one float4 of the output: lane p sums splits p, p + lanes, ... with eight loads in
// flight, then the lanes are folded by a fixed xor tree, so the result does not depend on scheduling.  Large outputs
// run with lanes = 1, small ones with many splits (a first layer's 9 x 4 taps) with up to 32.  The partials were
// written by the kernel just before and sit in L2.
constexpr int RED_THREADS = 256;
__global__ void __launch_bounds__(RED_THREADS)
wgrad_reduce_kernel(const float *__restrict__ partial, float *__restrict__ dw, size_t count4, int splits,
                    size_t split_stride, int accumulate, int lanes) {
    pdl_enter();
    const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t i = t / (size_t)lanes;
    const int p0 = (int)(t - i * (size_t)lanes);
    const bool live = i < count4;
    const float4 *p = reinterpret_cast<const float4 *>(partial) + (live ? i : 0);
    const size_t stride4 = split_stride / 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        int s = p0;
        for (; s + 7 * lanes < splits; s += 8 * lanes) {
            float4 v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __ldcg(p + (size_t)(s + k * lanes) * stride4);
#pragma unroll
            for (int k = 0; k < 8; ++k) { acc.x += v[k].x; acc.y += v[k].y; acc.z += v[k].z; acc.w += v[k].w; }
        }
        for (; s < splits; s += lanes) {
            const float4 v = __ldcg(p + (size_t)s * stride4);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    }
    for (int o = 1; o < lanes; o <<= 1) {   // whole warps reach this: lanes divides 32 and the grid is whole warps
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o); acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o); acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (!live || p0 != 0) return;
    float4 *o4 = reinterpret_cast<float4 *>(dw) + i;
    if (accumulate) {
        const float4 q = *o4;
        acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
    *o4 = acc;
}
int launch_wgrad_reduce(aet_context *ctx, const float *partial, float *dw, size_t out_floats, int splits, int accumulate) {
    const size_t count4 = out_floats / 4;
    int lanes = 1;
    while (lanes < 32 && count4 * (size_t)lanes < 65536 && lanes * 2 <= splits) lanes <<= 1;
    LaunchScope scope(ctx, "wgrad_reduce", (double)out_floats * 4.0 * (splits + 1 + (accumulate ? 1 : 0)), 0);
    const size_t threads = count4 * (size_t)lanes;
    launch_k(ctx->stream, (unsigned)((threads + RED_THREADS - 1) / RED_THREADS), RED_THREADS, 0, wgrad_reduce_kernel, partial, dw, count4,
             splits, out_floats, accumulate, lanes);
    return aet_check_launch("wgrad_reduce");
}

// Second stage of a split-K forward pass: y = activation(sum over splits + bias), four output columns per thread.
// `ld` floats per output row (a multiple of 4), bias indexed by column; fixed summation order.
__global__ void __launch_bounds__(RED_THREADS)
fprop_reduce_kernel(const float *__restrict__ partial, float *__restrict__ y, const float *__restrict__ bias, size_t count4, int ld4,
                    int splits, size_t split_stride, int act) {
    pdl_enter();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count4) return;
    const float4 *p = reinterpret_cast<const float4 *>(partial) + i;
    const size_t stride4 = split_stride / 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
        const float4 v = __ldcg(p + (size_t)s * stride4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias) {
        const float4 b = ldg4(bias + (i % (size_t)ld4) * 4);
        acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    acc.x = act_forward(acc.x, act); acc.y = act_forward(acc.y, act); acc.z = act_forward(acc.z, act); acc.w = act_forward(acc.w, act);
    reinterpret_cast<float4 *>(y)[i] = acc;
}

int launch_fprop_reduce(aet_context *ctx, const float *partial, float *y, const float *bias, size_t out_floats, int ld, int splits, int act) {
    const size_t count4 = out_floats / 4;
    LaunchScope scope(ctx, "fprop_reduce", (double)out_floats * 4.0 * (splits + 1), 0);
    launch_k(ctx->stream, (unsigned)((count4 + RED_THREADS - 1) / RED_THREADS), RED_THREADS, 0, fprop_reduce_kernel, partial, y, bias, count4,
             ld / 4, splits, out_floats, act);
    return aet_check_launch("fprop_reduce");
}

int pow2_cols(int n) {
    int c = 32;
    while (c < n) c <<= 1;
    return c;
}

ConvGeom layer_geom(const aet_layer *l) {
    ConvGeom g;
    g.N = l->batch; g.C = l->c; g.H = l->h; g.W = l->w; g.cp = l->cp;
    g.K = l->oc; g.OH = l->oh; g.OW = l->ow; g.kp = l->ocp;
    g.R = l->size; g.S = l->size; g.sy = l->stride_y; g.sx = l->stride_x; g.pad = l->pad;
    g.xs = l->cp; g.ys = l->ocp; g.dil = l->dilation;
    if (l->groups > 1) {   // one group's GEMM: its own channels and filters, pixels still a whole layer's channel count apart
        g.C = l->cg; g.cp = l->cgp;
        g.K = l->oc / l->groups; g.kp = g.K;
    }
    // A filter that covers the whole unpadded map is a fully connected layer (the reference has no other kind):
    // with NHWC activations and [filter][tap][channel] weights it IS a 1x1 convolution over H*W*cp channels of a
    // 1x1 map, byte for byte.  Seen that way the data gradient is a plain GEMM over the batch instead of a
    // convolution in which 35 of 36 taps of every input pixel fall outside the single output pixel.
    if (l->size == l->h && l->size == l->w && l->pad == 0 && l->size > 1 && l->groups == 1 && l->ctx->opt[OPT_FC_ALIAS]) {
        g.C = g.cp = g.xs = l->h * l->w * l->cp;
        g.H = g.W = g.OH = g.OW = 1;
        g.R = g.S = 1;
        g.sy = g.sx = 1;
    }
    return g;
}

int pick_bn(int n_cols, int m_tiles, int sm_count, int forced) {
    int full = round_up(n_cols, 16);
    if (forced) {   // tuning aid (option "bn_tile")
        int v = forced;
        if (v >= 16 && v % 16 == 0 && v <= 256) return v < full ? v : (full <= 256 ? full : v);
    }
    if (full <= 64) return full;
    const int cands[3] = {256, 128, 64};
    for (int i = 0; i < 3; ++i) {
        int bn = cands[i] < full ? cands[i] : full;
        int n_tiles = (n_cols + bn - 1) / bn;
        if (m_tiles * n_tiles >= sm_count) return bn;
    }
    return full < 64 ? full : 64;
}

template <int KIND, int NB>
int launch_gather_nb(aet_context *ctx, const ConvArgs &a, dim3 grid, size_t smem_bytes, const char *name, double flops) {
    AET_TRY(ctx_smem_attr(ctx, conv_gather_kernel<KIND, NB>));
    LaunchScope scope(ctx, name, 0, flops);
    launch_k(ctx->stream, grid, NTHREADS, smem_bytes, conv_gather_kernel<KIND, NB>, a);
    return aet_check_launch(name);
}

template <int KIND>
int launch_gather(aet_context *ctx, ConvArgs &a, dim3 grid, const char *name, double flops) {
    a.x3 = ctx->math == AET_MATH_3XTF32 ? 1 : 0;
    a.tmem_cols = pow2_cols(a.bn);
    a.status = ctx->status_dev;
    const size_t half = (size_t)BM * BK * 4 + (size_t)((a.bn + 31) / 32) * 32 * BK * 4;
    const size_t stage = half * (a.x3 ? 2 : 1);
    int stages = (int)((96 * 1024) / stage);
    if (a.bn <= 64 && stages > 3) stages = 3;   // small tiles: three CTAs share an SM
    if (stages < 3) stages = (int)((200 * 1024) / stage);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    a.stages = stages;
    const size_t smem_bytes = stage * stages + 1024;
    if (a.bn <= 64) return launch_gather_nb<KIND, 4>(ctx, a, grid, smem_bytes, name, flops);
    return launch_gather_nb<KIND, 16>(ctx, a, grid, smem_bytes, name, flops);
}

}  // namespace

#include "conv_tma.cuh"
#include "conv_tma_rows.cuh"
#include "conv_thin.cuh"

// Channel groups (dnn/ConvolutionalLayer.c:716-722, 913-946): group j convolves input channels [j*C/G, (j+1)*C/G) with
// filters [j*K/G, (j+1)*K/G).  With channels innermost a group is a column slice of every pixel row, so each group is
// one implicit GEMM over the same pixels with pointers moved by the slice and the pixel pitch left at the layer's.
static int conv_fprop_one(aet_layer *l, const float *x, float *y, const float *bias, int act_in_epilogue, ConvStats *stats, int gi) {
    aet_context *ctx = l->ctx;
    ConvArgs a = {};
    a.g = layer_geom(l);
    const ConvGeom &g = a.g;
    a.src_a = x + (size_t)gi * g.C; a.src_b = layer_W(l) + (size_t)gi * g.K * g.R * g.S * g.cp; a.out = y + (size_t)gi * g.K;
    a.bias = bias ? bias + (size_t)gi * g.K : nullptr;
    a.act = act_in_epilogue ? (int)l->act : (int)AET_LINEAR;
    a.n_rows = g.N * g.OH * g.OW;
    a.n_cols = g.kp;
    a.k_total = g.R * g.S * g.cp;
    a.k_per_split = a.k_total;
    a.out_ld = g.ys;
    const int m_tiles = (a.n_rows + BM - 1) / BM;
    if (stats) {
        stats->rows = 0;
        // the statistics describe the raw convolution result: no bias or activation in this epilogue
        if (!bias && a.act == (int)AET_LINEAR && ctx->math != AET_MATH_3XTF32 && ctx->opt[OPT_EPILOGUE_STATS]) {
            AET_TRY(ctx_scratch(ctx, (size_t)m_tiles * 4 * g.kp * sizeof(float), &stats->partial));   // at most two rows per pixel tile
            a.stat_shift = stats->shift;
            a.stat_partial = stats->partial;
            a.stat_rows_out = &stats->rows;
        }
    }
    a.bn = pick_bn(a.n_cols, m_tiles, ctx->sm_count, ctx->opt[OPT_BN_TILE]);
    const double flops = 2.0 * g.N * g.OH * g.OW * (double)g.K * g.C * g.R * g.S;
    int r = tma_fd_rows<KIND_FPROP>(l, a, flops);
    if (r != 1) return r;   // 1 = shape not eligible
    r = tma_fprop(l, a, flops);
    if (r != 1) return r;
    r = thin_fprop(l, a, flops);
    if (r != 1) return r;
    dim3 grid(m_tiles, (a.n_cols + a.bn - 1) / a.bn, 1);
    if (a.stat_rows_out) *a.stat_rows_out = (int)grid.x;
    return launch_gather<KIND_FPROP>(ctx, a, grid, "conv_fprop_gather", flops);
}

#include "conv_s2d.cuh"

int conv_fprop(aet_layer *l, const float *x, float *y, const float *bias, int act_in_epilogue, ConvStats *stats) {
    {
        const int r = s2d_fprop(l, x, y, bias, act_in_epilogue, stats);   // large strided first-layer filters: regrouped to stride 1
        if (r != 1) return r;
    }
    if (l->groups == 1) return conv_fprop_one(l, x, y, bias, act_in_epilogue, stats, 0);
    if (stats) stats->rows = 0;   // grouped layers take their batch statistics from the stand-alone reduction
    for (int gi = 0; gi < l->groups; ++gi) AET_TRY(conv_fprop_one(l, x, y, bias, act_in_epilogue, nullptr, gi));
    return AET_OK;
}

static int conv_dgrad_one(aet_layer *l, const float *dy, float *dx, int gi) {
    aet_context *ctx = l->ctx;
    ConvArgs a = {};
    a.g = layer_geom(l);
    const ConvGeom &g = a.g;
    a.src_a = dy + (size_t)gi * g.K; a.src_b = layer_W(l) + (size_t)gi * g.K * g.R * g.S * g.cp; a.out = dx + (size_t)gi * g.C;
    a.n_rows = g.N * g.H * g.W;
    a.n_cols = g.cp;
    a.k_total = g.R * g.S * g.kp;
    a.k_per_split = a.k_total;
    a.out_ld = g.xs;
    const int m_tiles = (a.n_rows + BM - 1) / BM;
    a.bn = pick_bn(a.n_cols, m_tiles, ctx->sm_count, ctx->opt[OPT_BN_TILE]);
    const double flops = 2.0 * g.N * g.OH * g.OW * (double)g.K * g.C * g.R * g.S;
    int r = tma_fd_rows<KIND_DGRAD>(l, a, flops);
    if (r != 1) return r;
    r = tma_dgrad(l, a, flops);
    if (r != 1) return r;
    r = narrow_dgrad(l, a, flops);
    if (r != 1) return r;
    dim3 grid(m_tiles, (a.n_cols + a.bn - 1) / a.bn, 1);
    return launch_gather<KIND_DGRAD>(ctx, a, grid, "conv_dgrad_gather", flops);
}

int conv_dgrad(aet_layer *l, const float *dy, float *dx) {
    for (int gi = 0; gi < l->groups; ++gi) AET_TRY(conv_dgrad_one(l, dy, dx, gi));
    return AET_OK;
}

static int conv_wgrad_one(aet_layer *l, const float *x, const float *dy, float *dw, int accumulate, int gi) {
    aet_context *ctx = l->ctx;
    ConvArgs a = {};
    a.g = layer_geom(l);
    const ConvGeom &g = a.g;
    a.src_a = dy + (size_t)gi * g.K; a.src_b = x + (size_t)gi * g.C;
    dw += (size_t)gi * g.K * g.R * g.S * g.cp;
    a.n_rows = g.K;
    a.n_cols = g.R * g.S * g.cp;
    a.k_total = g.N * g.OH * g.OW;
    a.out_ld = a.n_cols;
    const int m_tiles = (g.K + BM - 1) / BM;
    const double flops = 2.0 * g.N * g.OH * g.OW * (double)g.K * g.C * g.R * g.S;
    const size_t out_floats = (size_t)g.K * a.n_cols;
    {
        int rsplits = 0;
        float *rpartial = nullptr;
        int rr = tma_wgrad_rows(l, a, flops, &rsplits, &rpartial);
        if (rr < 0) return rr;
        if (rr == AET_OK) {
            return launch_wgrad_reduce(ctx, rpartial, dw, out_floats, rsplits, accumulate);
        }
    }
    {
        int tsplits = 0;
        float *tpartial = nullptr;
        int tr = thin_wgrad(l, a, flops, &tsplits, &tpartial);
        if (tr < 0) return tr;
        if (tr == AET_OK) {
            return launch_wgrad_reduce(ctx, tpartial, dw, out_floats, tsplits, accumulate);
        }
    }
    // N tile: the multiple of 16 (<= 256) that wastes the fewest padded columns, larger on ties
    int best_bn = 16, best_pad = 1 << 30;
    const int full = round_up(a.n_cols, 16);
    if (full <= 256) best_bn = full;
    else
        for (int bn = 256; bn >= 64; bn -= 16) {
            int padded = (a.n_cols + bn - 1) / bn * bn;
            if (padded < best_pad) { best_pad = padded; best_bn = bn; }
        }
    a.bn = best_bn;
    const int n_tiles = (a.n_cols + a.bn - 1) / a.bn;
    const int total_slabs = (a.k_total + BK - 1) / BK;
    int want = (2 * ctx->sm_count) / (m_tiles * n_tiles);
    if (want < 1) want = 1;
    int max_splits = total_slabs / 4;
    if (max_splits < 1) max_splits = 1;
    if (want > max_splits) want = max_splits;
    const int slabs_per_split = (total_slabs + want - 1) / want;
    const int splits = (total_slabs + slabs_per_split - 1) / slabs_per_split;
    a.k_per_split = slabs_per_split * BK;
    a.split_stride = (long long)out_floats;
    // One split that overwrites (a training step's first and only gradient of this layer): the tiles go straight to
    // their place, without the trip through scratch and the second kernel (a fully connected layer's gradient is as
    // large as its weights and has four K slabs).
    const bool direct = splits == 1 && !accumulate;
    float *partial = dw;
    if (!direct) AET_TRY(ctx_scratch(ctx, out_floats * splits * sizeof(float), &partial));
    a.out = partial;
    int r = tma_wgrad(l, a, splits, flops);
    if (r == 1) {
        dim3 grid(m_tiles, n_tiles, splits);
        r = launch_gather<KIND_WGRAD>(ctx, a, grid, "conv_wgrad_gather", flops);
    }
    if (r != AET_OK || direct) return r;
    return launch_wgrad_reduce(ctx, partial, dw, out_floats, splits, accumulate);
}

int conv_wgrad(aet_layer *l, const float *x, const float *dy, float *dw, int accumulate) {
    {
        const int r = s2d_wgrad(l, x, dy, dw, accumulate);
        if (r != 1) return r;
    }
    for (int gi = 0; gi < l->groups; ++gi) AET_TRY(conv_wgrad_one(l, x, dy, dw, accumulate, gi));
    return AET_OK;
}

void conv_release(aet_layer *l) {
    s2d_release(l);
    tma_release(l);
}

int conv_set_wait_limit(unsigned long long ns) {
    AET_CUDA(cudaMemcpyToSymbol(umma::g_wait_limit_ns, &ns, sizeof(ns)));
    return AET_OK;
}

namespace {
// Self-test of the bounded waits: one warp waits on an mbarrier that nothing ever arrives at, through the same
// mbar_wait every kernel uses.  The wait runs out after the context's limit, the kernel records the status word
// and returns normally; the context stays usable.
__global__ void wait_probe_kernel(int *status) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    pdl_enter();
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag);
    __syncthreads();
    if (threadIdx.x == 0 && !ok && status) atomicOr(status, AET_STATUS_TIMEOUT);
}
}  // namespace

int conv_wait_probe(aet_context *ctx) {
    LaunchScope scope(ctx, "wait_probe", 0, 0);
    launch_k(ctx->stream, 1, 32, 0, wait_probe_kernel, ctx->status_dev);
    return aet_check_launch("wait_probe");
}
