// Bandwidth-bound kernels around the convolution: batch-norm statistics / apply / backward fused
// with the activation and its gradient, bias gradient, max-pool and global average-pool in both
// directions, softmax + cross-entropy with an on-device loss reduction, dropout, and the fused
// SGD-momentum update.  All tensors are NHWC with `cp` (multiple of 4) floats per pixel, so every
// access is a 16-byte vector and consecutive threads touch consecutive addresses.  Reductions
// are two-stage with a fixed summation order (no floating-point atomics): results are bitwise
// reproducible from run to run and identical on every rank of a data-parallel job.
//
// Reference kernels replaced (one scalar thread per element / one block per channel each):
//   BN forward   mtcs/MtcsNormData.c:54-133,193-232,336-347   (CPU: dnn/NormData.c:141-282)
//   BN backward  mtcs/MtcsBiasData.c:27-45, mtcs/MtcsScaleData.c:53-71, mtcs/MtcsDeltaData.c:40-52,
//                89-114,158-185,229-236                        (CPU: dnn/DeltaData.c:23-80)
//   activation   mtcs/MtcsActivation.c:112-138,471-513
//   max-pool     mtcs/MtcsMaxPoolLayer.c:60-100,295-332        (CPU: dnn/MaxPoolLayer.c:237-272,318-331)
//   avg-pool     dnn/AvgPoolLayer.c:49-66,92-106
//   softmax-CE   dnn/SoftMaxLayer.c:122-139,172-199, mtcs/MtcsData.c:20-29
//   dropout      dnn/DropoutLayer.c:55-86
//   SGD          mtcs/MtcsConvLayer.c:618-631 -> mtcs/MtcsTool.c:33-52
#include <atomic>
#include <mutex>
#include <float.h>
#include <math.h>

#include "common.h"
#include "activation.cuh"

namespace {

constexpr int TB = 256;

// Thread -> (channel vector, pixel lane) map shared by the per-channel kernels: a block covers
// `lanes_c` channel vectors (4 channels each) times `pl_count` pixel lanes.
struct CMap {
    int cvec, lanes_c, pl_count, cslabs;
};
CMap make_cmap(int cp) {
    CMap m;
    m.cvec = cp / 4;
    m.lanes_c = m.cvec < TB ? m.cvec : TB;
    m.pl_count = TB / m.lanes_c;
    m.cslabs = (m.cvec + TB - 1) / TB;
    return m;
}
__device__ __forceinline__ bool cmap_thread(const CMap &m, int &cv, int &pl) {
    int t = threadIdx.x;
    int cl = t % m.lanes_c;
    pl = t / m.lanes_c;
    cv = blockIdx.y * TB + cl;
    return pl < m.pl_count && cv < m.cvec;
}

__device__ __forceinline__ float act_fwd(float v, int act) { return act_forward(v, act); }
// Gradient of the activation evaluated on its OUTPUT, as the reference does (dnn/Activation.h:99,104).
__device__ __forceinline__ float act_grad(float y, int act) { return act_gradient(y, act); }
__device__ __forceinline__ float bn_val(float x, float mean, float inv, float g, float b) {
    return __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(x, mean), inv), g), b);
}

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }

// ---------------------------------------------------------------------------- max-pool gather (fusion helper)
// When a max-pool follows a BN convolution inside a network, the pool's backward pass is not run as
// a kernel of its own: the BN backward kernels fetch "the delta the pool would have scattered here"
// on the fly from the pool's (4x smaller) delta and argmax tensors.  Same gather rule as
// maxpool_bwd_kernel (mtcs/MtcsMaxPoolLayer.c:295-332).
// windows [o * stride, o * stride + size) that contain coordinate v (already shifted by the pool's offset): first and last o
__device__ __forceinline__ int window_first(int v, int size, int stride) {
    const int t = v - size + 1;
    return t <= 0 ? 0 : (t + stride - 1) / stride;
}
__device__ __forceinline__ int window_last(int v, int stride) { return v < 0 ? -1 : v / stride; }
struct PoolGather {
    const float *delta;   // pool layer delta  [N][OH][OW][cp]
    const int *idx;       // pool argmax       [N][OH][OW][cp], reference numbering
    int C, H, W, OH, OW, size, sx, sy, off;
    int simple2;          // size 2, stride 2, no offset: every input belongs to exactly one window
};
__device__ __forceinline__ float4 pool_gather(const PoolGather &g, long long p, int c, int cp) {
    const unsigned pi = (unsigned)p;           // pixel counts stay far below 2^31
    const int j = (int)(pi % (unsigned)g.W);
    const unsigned q = pi / (unsigned)g.W;
    const int i = (int)(q % (unsigned)g.H);
    const int n = (int)(q / (unsigned)g.H);
    const int hw = g.H * g.W;
    const int my = j + g.W * (i + g.H * (c + n * g.C));
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
    if (g.simple2) {
        const int ow = j >> 1, oh = i >> 1;
        if (ow < g.OW && oh < g.OH) {
            const size_t o = ((size_t)(n * g.OH + oh) * g.OW + ow) * cp + c;
            const int4 id = __ldg(reinterpret_cast<const int4 *>(g.idx + o));
            const float4 dv = __ldg(reinterpret_cast<const float4 *>(g.delta + o));
            if (id.x == my) d.x = dv.x;
            if (id.y == my + hw) d.y = dv.y;
            if (id.z == my + 2 * hw) d.z = dv.z;
            if (id.w == my + 3 * hw) d.w = dv.w;
        }
        return d;
    }
    // The reference walks every window within (size - 1) / stride of the pixel's own; an argmax can only name a pixel
    // inside its window, so the windows that do not contain the pixel add nothing and are not read.
    const int oh_lo = window_first(i - g.off, g.size, g.sy), oh_hi = min(window_last(i - g.off, g.sy), g.OH - 1);
    const int ow_lo = window_first(j - g.off, g.size, g.sx), ow_hi = min(window_last(j - g.off, g.sx), g.OW - 1);
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
        for (int ow = ow_lo; ow <= ow_hi; ++ow) {
            const size_t o = ((size_t)(n * g.OH + oh) * g.OW + ow) * cp + c;
            const int4 id = __ldg(reinterpret_cast<const int4 *>(g.idx + o));
            const float4 dv = __ldg(reinterpret_cast<const float4 *>(g.delta + o));
            if (id.x == my) d.x += dv.x;
            if (id.y == my + hw) d.y += dv.y;
            if (id.z == my + 2 * hw) d.z += dv.z;
            if (id.w == my + 3 * hw) d.w += dv.w;
        }
    return d;
}

// ---------------------------------------------------------------------------- generic two-sum reduction
// MODE 0: BN statistics        s1 = sum(x - shift), s2 = sum((x - shift)^2)
// MODE 1: BN backward          d' = delta * act'(bn(x)); s1 = sum d', s2 = sum d' * (x - mean)
// MODE 2: bias/act backward    d' = delta * act'(y) written back in place; s1 = sum d'
struct ReduceArgs {
    const float *x;       // MODE 0/1: conv result before BN;  MODE 2: layer output y
    float *delta;         // MODE 1/2
    const float *mean, *inv, *gamma, *beta, *shift;
    float *partial;       // [blocks][2][cp]
    int act;
    long long pixels;
    int cp;
    long long pix_per_block;
    CMap m;
    PoolGather pool;      // MODE 1 with POOL: delta comes from the following max-pool layer
};

template <int MODE, bool POOL = false>
__global__ void __launch_bounds__(TB) reduce2_kernel(const ReduceArgs a) {
    pdl_enter();
    __shared__ float4 sh1[TB];
    __shared__ float4 sh2[TB];
    int cv, pl;
    const bool active = cmap_thread(a.m, cv, pl);
    float4 s1 = make_float4(0.f, 0.f, 0.f, 0.f), s2 = s1;
    if (active) {
        const int c = cv * 4;
        float4 mean = make_float4(0.f, 0.f, 0.f, 0.f), inv = mean, gam = mean, bet = mean, sft = mean;
        if (MODE == 0) sft = ld4(a.shift + c);
        if (MODE == 1) { mean = ld4(a.mean + c); inv = ld4(a.inv + c); gam = ld4(a.gamma + c); bet = ld4(a.beta + c); }
        long long p0 = (long long)blockIdx.x * a.pix_per_block;
        long long p1 = p0 + a.pix_per_block;
        if (p1 > a.pixels) p1 = a.pixels;
        // four pixels per trip: all loads of a trip are issued before any arithmetic, which is what
        // keeps enough bytes in flight per SM to approach HBM bandwidth
        constexpr int U = 4;
        const long long step = a.m.pl_count;
        for (long long pb = p0 + pl; pb < p1; pb += U * step) {
            float4 v[U], d[U];
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long p = pb + u * step;
                ok[u] = p < p1;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                d[u] = v[u];
                if (ok[u]) {
                    const size_t off = (size_t)p * a.cp + c;
                    v[u] = ld4(a.x + off);
                    if (MODE == 1) d[u] = POOL ? pool_gather(a.pool, p, c, a.cp) : ld4(a.delta + off);
                    if (MODE == 2) d[u] = ld4(a.delta + off);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!ok[u]) continue;
                if (MODE == 0) {
                    float4 t = v[u];
                    t.x -= sft.x; t.y -= sft.y; t.z -= sft.z; t.w -= sft.w;
                    s1.x += t.x; s1.y += t.y; s1.z += t.z; s1.w += t.w;
                    s2.x += t.x * t.x; s2.y += t.y * t.y; s2.z += t.z * t.z; s2.w += t.w * t.w;
                } else if (MODE == 1) {
                    const float4 t = v[u];
                    float4 q = d[u];
                    q.x *= act_gradient_pre(bn_val(t.x, mean.x, inv.x, gam.x, bet.x), a.act);
                    q.y *= act_gradient_pre(bn_val(t.y, mean.y, inv.y, gam.y, bet.y), a.act);
                    q.z *= act_gradient_pre(bn_val(t.z, mean.z, inv.z, gam.z, bet.z), a.act);
                    q.w *= act_gradient_pre(bn_val(t.w, mean.w, inv.w, gam.w, bet.w), a.act);
                    s1.x += q.x; s1.y += q.y; s1.z += q.z; s1.w += q.w;
                    s2.x += q.x * (t.x - mean.x); s2.y += q.y * (t.y - mean.y);
                    s2.z += q.z * (t.z - mean.z); s2.w += q.w * (t.w - mean.w);
                } else {
                    const float4 y = v[u];
                    float4 q = d[u];
                    q.x *= act_grad(y.x, a.act); q.y *= act_grad(y.y, a.act);
                    q.z *= act_grad(y.z, a.act); q.w *= act_grad(y.w, a.act);
                    if (a.act != AET_LINEAR) st4(a.delta + (size_t)(pb + u * step) * a.cp + c, q);
                    s1.x += q.x; s1.y += q.y; s1.z += q.z; s1.w += q.w;
                }
            }
        }
    }
    sh1[threadIdx.x] = s1;
    sh2[threadIdx.x] = s2;
    __syncthreads();
    if (active && pl == 0) {
        const int cl = threadIdx.x;  // pl == 0 => threadIdx.x is the channel lane
        for (int q = 1; q < a.m.pl_count; ++q) {
            float4 t1 = sh1[q * a.m.lanes_c + cl], t2 = sh2[q * a.m.lanes_c + cl];
            s1.x += t1.x; s1.y += t1.y; s1.z += t1.z; s1.w += t1.w;
            s2.x += t2.x; s2.y += t2.y; s2.z += t2.z; s2.w += t2.w;
        }
        float *dst = a.partial + (size_t)blockIdx.x * 2 * a.cp + cv * 4;
        st4(dst, s1);
        st4(dst + a.cp, s2);
    }
}

// Window-major BN backward for the common 2x2 / stride-2 pool over even-sized maps: one thread owns
// one pool output (4 channels) and the four inputs of its window, so the pool's delta and argmax are
// read once per window and no per-input index arithmetic is needed.  blockDim must be a multiple
// of cp/4 so that a thread keeps its channel vector over the grid-stride loop.
struct PoolWinArgs {
    const float *x;          // conv result [N][H][W][cp]
    float *dx;               // conv delta  [N][H][W][cp]   (apply pass)
    const float *pdelta;     // pool delta  [N][OH][OW][cp]
    const int *pidx;         // pool argmax
    const float *mean, *inv, *gamma, *beta, *coef;
    float *partial;          // [blocks][2][cp]              (reduce pass)
    int act, cp, C, H, W, OH, OW;
    unsigned total;          // N*OH*OW*cvec
};

template <bool APPLY>
__global__ void __launch_bounds__(TB) bn_bwd_poolwin_kernel(const PoolWinArgs a) {
    pdl_enter();
    __shared__ float4 sh1[TB];
    __shared__ float4 sh2[TB];
    const unsigned cvec = (unsigned)a.cp / 4;
    const int cv = (int)(threadIdx.x % cvec);
    const int c = cv * 4;
    const float4 mean = ld4(a.mean + c), inv = ld4(a.inv + c), gam = ld4(a.gamma + c), bet = ld4(a.beta + c);
    float4 ka, kb, kc;
    if (APPLY) { ka = ld4(a.coef + c); kb = ld4(a.coef + a.cp + c); kc = ld4(a.coef + 2 * a.cp + c); }
    float4 s1 = make_float4(0.f, 0.f, 0.f, 0.f), s2 = s1;
    const int hw = a.H * a.W;
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < a.total; e += gridDim.x * blockDim.x) {
        unsigned p = e / cvec;                      // e % cvec == cv because blockDim and the stride are multiples of cvec
        const int ow = (int)(p % (unsigned)a.OW); p /= (unsigned)a.OW;
        const int oh = (int)(p % (unsigned)a.OH);
        const int n = (int)(p / (unsigned)a.OH);
        const size_t o = ((size_t)(n * a.OH + oh) * a.OW + ow) * a.cp + c;
        const int4 id = __ldg(reinterpret_cast<const int4 *>(a.pidx + o));
        const float4 dv = __ldg(reinterpret_cast<const float4 *>(a.pdelta + o));
        const size_t i00 = ((size_t)(n * a.H + 2 * oh) * a.W + 2 * ow) * a.cp + c;
        const size_t offs[4] = {i00, i00 + a.cp, i00 + (size_t)a.W * a.cp, i00 + (size_t)a.W * a.cp + a.cp};
        float4 v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) v[t] = ld4(a.x + offs[t]);
        // reference numbering of the window's top-left input, channel c
        const int pos00 = 2 * ow + a.W * (2 * oh + a.H * (c + n * a.C));
        // Only a window's argmax input receives the pool's delta: per channel the tap t it sits at follows from the
        // stored index, and the activation gradient is evaluated for that one input instead of all four
        // (the other three contribute exact zeros to the sums, and only their (x - mean) term to the apply pass).
        int tsel[4];
        float qa[4];
        {
            const int ids[4] = {id.x, id.y, id.z, id.w};
            const float dvs[4] = {dv.x, dv.y, dv.z, dv.w};
            const float means[4] = {mean.x, mean.y, mean.z, mean.w}, invs[4] = {inv.x, inv.y, inv.z, inv.w};
            const float gams[4] = {gam.x, gam.y, gam.z, gam.w}, bets[4] = {bet.x, bet.y, bet.z, bet.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int d = ids[k] - (pos00 + k * hw);
                const int t = d == 0 ? 0 : (d == 1 ? 1 : (d == a.W ? 2 : (d == a.W + 1 ? 3 : -1)));
                const float x0 = k == 0 ? v[0].x : (k == 1 ? v[0].y : (k == 2 ? v[0].z : v[0].w));
                const float x1 = k == 0 ? v[1].x : (k == 1 ? v[1].y : (k == 2 ? v[1].z : v[1].w));
                const float x2 = k == 0 ? v[2].x : (k == 1 ? v[2].y : (k == 2 ? v[2].z : v[2].w));
                const float x3 = k == 0 ? v[3].x : (k == 1 ? v[3].y : (k == 2 ? v[3].z : v[3].w));
                const float xa = t == 0 ? x0 : (t == 1 ? x1 : (t == 2 ? x2 : x3));
                tsel[k] = t;
                qa[k] = t >= 0 ? dvs[k] * act_gradient_pre(bn_val(xa, means[k], invs[k], gams[k], bets[k]), a.act) : 0.f;
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            float4 q;
            q.x = tsel[0] == t ? qa[0] : 0.f;
            q.y = tsel[1] == t ? qa[1] : 0.f;
            q.z = tsel[2] == t ? qa[2] : 0.f;
            q.w = tsel[3] == t ? qa[3] : 0.f;
            if (APPLY) {
                q.x = q.x * ka.x + (v[t].x - mean.x) * kb.x + kc.x;
                q.y = q.y * ka.y + (v[t].y - mean.y) * kb.y + kc.y;
                q.z = q.z * ka.z + (v[t].z - mean.z) * kb.z + kc.z;
                q.w = q.w * ka.w + (v[t].w - mean.w) * kb.w + kc.w;
                st4(a.dx + offs[t], q);
            } else {
                s1.x += q.x; s1.y += q.y; s1.z += q.z; s1.w += q.w;
                s2.x += q.x * (v[t].x - mean.x); s2.y += q.y * (v[t].y - mean.y);
                s2.z += q.z * (v[t].z - mean.z); s2.w += q.w * (v[t].w - mean.w);
            }
        }
    }
    if (APPLY) return;
    sh1[threadIdx.x] = s1;
    sh2[threadIdx.x] = s2;
    __syncthreads();
    if (threadIdx.x < cvec) {
        for (unsigned q = threadIdx.x + cvec; q < blockDim.x; q += cvec) {
            float4 t1 = sh1[q], t2 = sh2[q];
            s1.x += t1.x; s1.y += t1.y; s1.z += t1.z; s1.w += t1.w;
            s2.x += t2.x; s2.y += t2.y; s2.z += t2.z; s2.w += t2.w;
        }
        float *dst = a.partial + (size_t)blockIdx.x * 2 * a.cp + c;
        st4(dst, s1);
        st4(dst + a.cp, s2);
    }
}

struct FinalizeArgs {
    const float *partial;
    int blocks, cp, c;
    long long m;          // elements per channel
    int parity, update_rolling;
    const float *shift;
    float *mean, *variance, *inv, *rolling_mean, *rolling_variance;
    // backward
    const float *gamma;
    float *g_gamma, *g_beta, *coef;   // coef: [3][cp]
};

// MODE 0: statistics -> mean, variance, 1/std, rolling update.  MODE 1: BN backward coefficients
// and the scale / shift gradients.  MODE 2: bias gradient.
constexpr int FIN_CH = 8;   // channels per finalize block
template <int MODE>
__global__ void __launch_bounds__(1024) finalize_kernel(const FinalizeArgs a) {
    pdl_enter();
    // A block owns 8 channels (one 32-byte sector of each partial row) and splits the rows over 128
    // thread groups, so that even 600 rows are one round of independent loads per thread.  The sums
    // are formed in double in a fixed order: within the thread, over the warp's four groups by
    // shuffle, then over the 32 warps.
    __shared__ double sh1[32][FIN_CH + 1], sh2[32][FIN_CH + 1];
    const int cl = threadIdx.x & (FIN_CH - 1), part = threadIdx.x / FIN_CH;
    const int warp = threadIdx.x >> 5;
    const int c = blockIdx.x * FIN_CH + cl;
    double s1 = 0.0, s2 = 0.0;
    if (c < a.cp) {
        for (int b0 = part; b0 < a.blocks; b0 += (1024 / FIN_CH) * 4) {
            float v1[4], v2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int b = b0 + (1024 / FIN_CH) * i;
                v1[i] = 0.f; v2[i] = 0.f;
                if (b < a.blocks) {
                    v1[i] = __ldg(a.partial + (size_t)b * 2 * a.cp + c);
                    if (MODE != 2) v2[i] = __ldg(a.partial + (size_t)b * 2 * a.cp + a.cp + c);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) { s1 += (double)v1[i]; s2 += (double)v2[i]; }
        }
    }
#pragma unroll
    for (int o = FIN_CH; o < 32; o <<= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if ((threadIdx.x & 31) < FIN_CH) { sh1[warp][cl] = s1; sh2[warp][cl] = s2; }
    // the finishing warp's per-channel operands are requested before the barrier, off the critical path
    float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
    const bool live = part == 0 && c < a.c;   // threads 0..7 finish their channel
    if (live) {
        if (MODE == 0) {
            p0 = a.shift[c];
            if (a.update_rolling) { p1 = a.rolling_mean[c]; p2 = a.rolling_variance[c]; }
        } else if (MODE == 1) {
            p0 = a.variance[c]; p1 = a.gamma[c]; p2 = a.inv[c]; p3 = a.g_gamma[c];
        } else {
            p0 = a.g_beta[c];
        }
    }
    __syncthreads();
    if (part != 0 || c >= a.cp) return;
    {   // fixed-order sum of the 32 warp sums in four independent chains
        double t1[4] = {0.0, 0.0, 0.0, 0.0}, t2[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
        for (int q = 0; q < 32; ++q) { t1[q & 3] += sh1[q][cl]; t2[q & 3] += sh2[q][cl]; }
        s1 = (t1[0] + t1[1]) + (t1[2] + t1[3]);
        s2 = (t2[0] + t2[1]) + (t2[2] + t2[3]);
    }
    const double m = (double)a.m;
    if (MODE == 0) {
        if (c >= a.c) { a.mean[c] = 0.f; a.variance[c] = 0.f; a.inv[c] = 0.f; return; }
        const double mean_sh = s1 / m;
        double ss = s2 - s1 * mean_sh;   // sum (x - mean)^2
        if (ss < 0.0) ss = 0.0;
        const float mean = (float)(mean_sh + (double)p0);
        float var, inv;
        if (a.parity == AET_PARITY_CPU) {
            var = (float)(ss / (m - 1.0));
            inv = (float)(1.0 / (sqrt((double)var) + (double).000001f));
        } else {
            var = (float)(ss / m);
            inv = 1.0f / sqrtf(var + .00001f);
        }
        a.mean[c] = mean; a.variance[c] = var; a.inv[c] = inv;
        if (a.update_rolling) {
            const float keep = a.parity == AET_PARITY_CPU ? .9f : .99f, add = a.parity == AET_PARITY_CPU ? .1f : .01f;
            float rm = p1 * keep; rm += add * mean;
            float rv = p2 * keep; rv += add * var;
            a.rolling_mean[c] = rm; a.rolling_variance[c] = rv;
        }
    } else if (MODE == 1) {
        if (c >= a.c) { a.coef[c] = 0.f; a.coef[a.cp + c] = 0.f; a.coef[2 * a.cp + c] = 0.f; return; }
        const float var = p0, gam = p1;
        const float S1 = (float)s1, S2 = (float)s2;
        a.g_gamma[c] = p3 + S2 * p2;
        float md, vd, k1;
        // v^(-3/2) is formed as 1 / (v * sqrt(v)) in double: it agrees with pow() to the last few bits of
        // the double, far below the float the product is rounded to, and costs a fraction of pow()
        if (a.parity == AET_PARITY_CPU) {
            const double v = (double)(var + .00001f), rs = sqrt(v);
            md = (float)((double)(gam * S1) * (-1. / rs));
            vd = (float)((double)(gam * S2) * (-.5 / (v * rs)));
            k1 = (float)(1. / rs);
        } else {
            a.g_beta[c] += S1;
            const float v = var + .000001f;
            md = (gam * S1) * (-1.f / sqrtf(v));
            vd = (float)((double)(gam * S2) * (-.5 * (double)(1.f / (v * sqrtf(v)))));
            k1 = 1.f / (sqrtf(var) + .000001f);
        }
        a.coef[c] = gam * k1;
        a.coef[a.cp + c] = (float)((double)vd * 2. / m);
        a.coef[2 * a.cp + c] = (float)((double)md / m);
    } else {
        if (c < a.c) a.g_beta[c] = p0 + (float)s1;
    }
}

// y = act(bn(x)) ; optionally with the rolling statistics (eval).
struct ApplyArgs {
    const float *x;
    float *y;
    const float *mean, *inv, *gamma, *beta;
    int act, cp;
    long long pixels, pix_per_block;
    CMap m;
};
__global__ void __launch_bounds__(TB) bn_apply_kernel(const ApplyArgs a) {
    pdl_enter();
    int cv, pl;
    if (!cmap_thread(a.m, cv, pl)) return;
    const int c = cv * 4;
    const float4 mean = ld4(a.mean + c), inv = ld4(a.inv + c), gam = ld4(a.gamma + c), bet = ld4(a.beta + c);
    long long p0 = (long long)blockIdx.x * a.pix_per_block, p1 = p0 + a.pix_per_block;
    if (p1 > a.pixels) p1 = a.pixels;
    constexpr int U = 4;
    const long long step = a.m.pl_count;
    for (long long pb = p0 + pl; pb < p1; pb += U * step) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long p = pb + u * step;
            if (p < p1) v[u] = ld4(a.x + (size_t)p * a.cp + c);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long p = pb + u * step;
            if (p >= p1) continue;
            float4 t = v[u];
            t.x = act_fwd(bn_val(t.x, mean.x, inv.x, gam.x, bet.x), a.act);
            t.y = act_fwd(bn_val(t.y, mean.y, inv.y, gam.y, bet.y), a.act);
            t.z = act_fwd(bn_val(t.z, mean.z, inv.z, gam.z, bet.z), a.act);
            t.w = act_fwd(bn_val(t.w, mean.w, inv.w, gam.w, bet.w), a.act);
            st4(a.y + (size_t)p * a.cp + c, t);
        }
    }
}

// delta <- d' * a[c] + (x - mean) * b[c] + c0[c], with d' = delta * act'(y) recomputed from x.
struct BwdApplyArgs {
    const float *x;
    float *delta;
    const float *mean, *inv, *gamma, *beta, *coef;
    int act, cp;
    long long pixels, pix_per_block;
    CMap m;
    PoolGather pool;
};
template <bool POOL>
__global__ void __launch_bounds__(TB) bn_bwd_apply_kernel(const BwdApplyArgs a) {
    pdl_enter();
    int cv, pl;
    if (!cmap_thread(a.m, cv, pl)) return;
    const int c = cv * 4;
    const float4 mean = ld4(a.mean + c), inv = ld4(a.inv + c), gam = ld4(a.gamma + c), bet = ld4(a.beta + c);
    const float4 ka = ld4(a.coef + c), kb = ld4(a.coef + a.cp + c), kc = ld4(a.coef + 2 * a.cp + c);
    long long p0 = (long long)blockIdx.x * a.pix_per_block, p1 = p0 + a.pix_per_block;
    if (p1 > a.pixels) p1 = a.pixels;
    constexpr int U = 4;
    const long long step = a.m.pl_count;
    for (long long pb = p0 + pl; pb < p1; pb += U * step) {
        float4 v[U], d[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long p = pb + u * step;
            if (p < p1) {
                const size_t off = (size_t)p * a.cp + c;
                v[u] = ld4(a.x + off);
                d[u] = POOL ? pool_gather(a.pool, p, c, a.cp) : ld4(a.delta + off);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long p = pb + u * step;
            if (p >= p1) continue;
            const float4 t = v[u];
            float4 q = d[u];
            q.x *= act_gradient_pre(bn_val(t.x, mean.x, inv.x, gam.x, bet.x), a.act);
            q.y *= act_gradient_pre(bn_val(t.y, mean.y, inv.y, gam.y, bet.y), a.act);
            q.z *= act_gradient_pre(bn_val(t.z, mean.z, inv.z, gam.z, bet.z), a.act);
            q.w *= act_gradient_pre(bn_val(t.w, mean.w, inv.w, gam.w, bet.w), a.act);
            q.x = q.x * ka.x + (t.x - mean.x) * kb.x + kc.x;
            q.y = q.y * ka.y + (t.y - mean.y) * kb.y + kc.y;
            q.z = q.z * ka.z + (t.z - mean.z) * kb.z + kc.z;
            q.w = q.w * ka.w + (t.w - mean.w) * kb.w + kc.w;
            st4(a.delta + (size_t)p * a.cp + c, q);
        }
    }
}

__global__ void eval_inv_kernel(const float *rolling_variance, float *inv, int c, int cp, int parity) {
    pdl_enter();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= cp) return;
    float v = 0.f;
    if (i < c)
        v = parity == AET_PARITY_CPU ? (float)(1.0 / (sqrt((double)rolling_variance[i]) + (double).000001f))
                                     : 1.0f / sqrtf(rolling_variance[i] + .00001f);
    inv[i] = v;
}

// ---------------------------------------------------------------------------- max pool
struct PoolArgs {
    const float *x;
    float *y;
    int *idx;
    int N, C, H, W, cp, OH, OW, size, sx, sy, off, parity;
    long long total;   // N*OH*OW*cvec
};
__global__ void __launch_bounds__(TB) maxpool_fwd_kernel(const PoolArgs a) {
    pdl_enter();
    const long long e64 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e64 >= a.total) return;
    const unsigned e = (unsigned)e64;          // element counts stay below 2^32
    const unsigned cvec = (unsigned)a.cp / 4;
    const int cv = (int)(e % cvec);
    unsigned p = e / cvec;
    const int ow = (int)(p % (unsigned)a.OW); p /= (unsigned)a.OW;
    const int oh = (int)(p % (unsigned)a.OH);
    const int n = (int)(p / (unsigned)a.OH);
    const float lowest = a.parity == AET_PARITY_CPU ? -FLT_MAX : -INFINITY;
    float4 mx = make_float4(lowest, lowest, lowest, lowest);
    int4 mi = make_int4(-1, -1, -1, -1);
    const int c = cv * 4;
    for (int l = 0; l < a.size; ++l)
        for (int m = 0; m < a.size; ++m) {
            const int ch = a.off + oh * a.sy + l, cw = a.off + ow * a.sx + m;
            const bool valid = ch >= 0 && ch < a.H && cw >= 0 && cw < a.W;
            float4 v = make_float4(lowest, lowest, lowest, lowest);
            if (valid) v = ld4(a.x + ((size_t)(n * a.H + ch) * a.W + cw) * a.cp + c);
            // index in the reference's NCHW numbering: cw + W*(ch + H*(k + n*C))
            const int base = cw + a.W * (ch + a.H * (c + n * a.C));
            const int hw = a.H * a.W;
            if (v.x > mx.x) { mx.x = v.x; mi.x = base; }
            if (v.y > mx.y) { mx.y = v.y; mi.y = base + hw; }
            if (v.z > mx.z) { mx.z = v.z; mi.z = base + 2 * hw; }
            if (v.w > mx.w) { mx.w = v.w; mi.w = base + 3 * hw; }
        }
    if (c + 1 >= a.C) { mx.y = 0.f; mi.y = -1; }   // pad channels stay zero
    if (c + 2 >= a.C) { mx.z = 0.f; mi.z = -1; }
    if (c + 3 >= a.C) { mx.w = 0.f; mi.w = -1; }
    const size_t o = ((size_t)(n * a.OH + oh) * a.OW + ow) * a.cp + c;
    st4(a.y + o, mx);
    if (a.idx) *reinterpret_cast<int4 *>(a.idx + o) = mi;
}

// Fused BN-apply + activation + max-pool: y = act(bn(x)) is formed in registers for each window tap
// and only the pooled values and argmax indices are written.  Comparison order and tie rule are those
// of maxpool_fwd_kernel, on bit-identical y values.
struct BnPoolArgs {
    PoolArgs p;
    const float *mean, *inv, *gamma, *beta;
    int act;
    float *ymax;           // optional: the convolution result (before BN) at each window's argmax, same layout as the pool output
    unsigned char *code;   // with ymax: the argmax's position inside the window (0..3 row-major; 4: none)
};
__global__ void __launch_bounds__(TB) bn_pool_fwd_kernel(const BnPoolArgs b) {
    pdl_enter();
    const PoolArgs &a = b.p;
    const long long e64 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e64 >= a.total) return;
    const unsigned e = (unsigned)e64;          // element counts stay below 2^32
    const unsigned cvec = (unsigned)a.cp / 4;
    const int cv = (int)(e % cvec);
    unsigned p = e / cvec;
    const int ow = (int)(p % (unsigned)a.OW); p /= (unsigned)a.OW;
    const int oh = (int)(p % (unsigned)a.OH);
    const int n = (int)(p / (unsigned)a.OH);
    const float lowest = a.parity == AET_PARITY_CPU ? -FLT_MAX : -INFINITY;
    float4 mx = make_float4(lowest, lowest, lowest, lowest);
    int4 mi = make_int4(-1, -1, -1, -1);
    const int c = cv * 4;
    const float4 mean = __ldg(reinterpret_cast<const float4 *>(b.mean + c)), inv = __ldg(reinterpret_cast<const float4 *>(b.inv + c));
    const float4 gam = __ldg(reinterpret_cast<const float4 *>(b.gamma + c)), bet = __ldg(reinterpret_cast<const float4 *>(b.beta + c));
    if (a.size == 2 && a.sx == 2 && a.sy == 2 && a.off == 0 && 2 * oh + 1 < a.H && 2 * ow + 1 < a.W) {
        // The usual 2x2 / stride-2 window, wholly inside the map: its four taps are requested before any of them is
        // used (four independent 16-byte loads per thread instead of a chain of dependent ones), then compared in the
        // same (row, column) order with the same strict '>' as the general loop below.
        const size_t i00 = ((size_t)(n * a.H + 2 * oh) * a.W + 2 * ow) * a.cp + c;
        float4 t[4] = {ld4(a.x + i00), ld4(a.x + i00 + a.cp), ld4(a.x + i00 + (size_t)a.W * a.cp), ld4(a.x + i00 + (size_t)a.W * a.cp + a.cp)};
        const int hw = a.H * a.W;
        const int base00 = 2 * ow + a.W * (2 * oh + a.H * (c + n * a.C));
        float4 raw = make_float4(0.f, 0.f, 0.f, 0.f);
        uchar4 cd = make_uchar4(4, 4, 4, 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float4 v = t[k];
            v.x = act_fwd(bn_val(v.x, mean.x, inv.x, gam.x, bet.x), b.act);
            v.y = act_fwd(bn_val(v.y, mean.y, inv.y, gam.y, bet.y), b.act);
            v.z = act_fwd(bn_val(v.z, mean.z, inv.z, gam.z, bet.z), b.act);
            v.w = act_fwd(bn_val(v.w, mean.w, inv.w, gam.w, bet.w), b.act);
            const int base = base00 + (k & 1) + (k >> 1) * a.W;
            if (v.x > mx.x) { mx.x = v.x; mi.x = base; raw.x = t[k].x; cd.x = (unsigned char)k; }
            if (v.y > mx.y) { mx.y = v.y; mi.y = base + hw; raw.y = t[k].y; cd.y = (unsigned char)k; }
            if (v.z > mx.z) { mx.z = v.z; mi.z = base + 2 * hw; raw.z = t[k].z; cd.z = (unsigned char)k; }
            if (v.w > mx.w) { mx.w = v.w; mi.w = base + 3 * hw; raw.w = t[k].w; cd.w = (unsigned char)k; }
        }
        if (b.ymax) {
            if (c + 1 >= a.C) cd.y = 4;   // pad channels
            if (c + 2 >= a.C) cd.z = 4;
            if (c + 3 >= a.C) cd.w = 4;
            const size_t o = ((size_t)(n * a.OH + oh) * a.OW + ow) * a.cp + c;
            st4(b.ymax + o, raw);
            *reinterpret_cast<uchar4 *>(b.code + o) = cd;
        }
    } else
    for (int l = 0; l < a.size; ++l)
        for (int m = 0; m < a.size; ++m) {
            const int ch = a.off + oh * a.sy + l, cw = a.off + ow * a.sx + m;
            const bool valid = ch >= 0 && ch < a.H && cw >= 0 && cw < a.W;
            float4 v = make_float4(lowest, lowest, lowest, lowest);
            if (valid) {
                v = ld4(a.x + ((size_t)(n * a.H + ch) * a.W + cw) * a.cp + c);
                v.x = act_fwd(bn_val(v.x, mean.x, inv.x, gam.x, bet.x), b.act);
                v.y = act_fwd(bn_val(v.y, mean.y, inv.y, gam.y, bet.y), b.act);
                v.z = act_fwd(bn_val(v.z, mean.z, inv.z, gam.z, bet.z), b.act);
                v.w = act_fwd(bn_val(v.w, mean.w, inv.w, gam.w, bet.w), b.act);
            }
            const int base = cw + a.W * (ch + a.H * (c + n * a.C));
            const int hw = a.H * a.W;
            if (v.x > mx.x) { mx.x = v.x; mi.x = base; }
            if (v.y > mx.y) { mx.y = v.y; mi.y = base + hw; }
            if (v.z > mx.z) { mx.z = v.z; mi.z = base + 2 * hw; }
            if (v.w > mx.w) { mx.w = v.w; mi.w = base + 3 * hw; }
        }
    if (c + 1 >= a.C) { mx.y = 0.f; mi.y = -1; }
    if (c + 2 >= a.C) { mx.z = 0.f; mi.z = -1; }
    if (c + 3 >= a.C) { mx.w = 0.f; mi.w = -1; }
    const size_t o = ((size_t)(n * a.OH + oh) * a.OW + ow) * a.cp + c;
    st4(a.y + o, mx);
    if (a.idx) *reinterpret_cast<int4 *>(a.idx + o) = mi;
}

struct PoolBwdArgs {
    const float *delta;
    const int *idx;
    float *prev;
    int N, C, H, W, cp, OH, OW, size, sx, sy, off, accumulate;
    long long total;   // N*H*W*cvec
};
// Gather form (mtcs/MtcsMaxPoolLayer.c:295-332): every input element adds the deltas of the
// windows whose argmax it is.
__global__ void __launch_bounds__(TB) maxpool_bwd_kernel(const PoolBwdArgs a) {
    pdl_enter();
    const long long e64 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e64 >= a.total) return;
    const unsigned e = (unsigned)e64;
    const unsigned cvec = (unsigned)a.cp / 4;
    const int cv = (int)(e % cvec);
    unsigned p = e / cvec;
    const int j = (int)(p % (unsigned)a.W); p /= (unsigned)a.W;
    const int i = (int)(p % (unsigned)a.H);
    const int n = (int)(p / (unsigned)a.H);
    const int c = cv * 4;
    const int hw = a.H * a.W;
    const int my = j + a.W * (i + a.H * (c + n * a.C));
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
    // only the windows that contain the pixel can name it (see pool_gather); same order as the reference's walk
    const int oh_lo = window_first(i - a.off, a.size, a.sy), oh_hi = min(window_last(i - a.off, a.sy), a.OH - 1);
    const int ow_lo = window_first(j - a.off, a.size, a.sx), ow_hi = min(window_last(j - a.off, a.sx), a.OW - 1);
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
        for (int ow = ow_lo; ow <= ow_hi; ++ow) {
            const size_t o = ((size_t)(n * a.OH + oh) * a.OW + ow) * a.cp + c;
            const int4 id = *reinterpret_cast<const int4 *>(a.idx + o);
            const float4 dv = ld4(a.delta + o);
            if (id.x == my) d.x += dv.x;
            if (id.y == my + hw) d.y += dv.y;
            if (id.z == my + 2 * hw) d.z += dv.z;
            if (id.w == my + 3 * hw) d.w += dv.w;
        }
    const size_t io = ((size_t)(n * a.H + i) * a.W + j) * a.cp + c;
    if (a.accumulate) {
        float4 q = ld4(a.prev + io);
        d.x += q.x; d.y += q.y; d.z += q.z; d.w += q.w;
    }
    st4(a.prev + io, d);
}

// ---------------------------------------------------------------------------- global average pool
__global__ void avgpool_fwd_kernel(const float *x, float *y, int N, int spatial, int cp) {
    pdl_enter();
    int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int cvec = cp / 4;
    if (e >= N * cvec) return;
    const int cv = e % cvec, n = e / cvec;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    const float *src = x + (size_t)n * spatial * cp + cv * 4;
    for (int i = 0; i < spatial; ++i) {
        float4 v = ld4(src + (size_t)i * cp);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    s.x /= spatial; s.y /= spatial; s.z /= spatial; s.w /= spatial;
    st4(y + (size_t)n * cp + cv * 4, s);
}
__global__ void avgpool_bwd_kernel(const float *delta, float *prev, long long total4, int spatial, int cp, int accumulate) {
    pdl_enter();
    long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total4) return;
    const int cvec = cp / 4;
    const int cv = (int)(e % cvec);
    const long long pix = e / cvec;
    const long long n = pix / spatial;
    float4 d = ld4(delta + (size_t)n * cp + cv * 4);
    d.x /= spatial; d.y /= spatial; d.z /= spatial; d.w /= spatial;
    float *dst = prev + (size_t)pix * cp + cv * 4;
    if (accumulate) {
        float4 q = ld4(dst);
        d.x += q.x; d.y += q.y; d.z += q.z; d.w += q.w;
    }
    st4(dst, d);
}

// ---------------------------------------------------------------------------- softmax + cross entropy
// One warp per (sample, group).  Writes probabilities, delta = truth - p, the per-element error and
// one partial loss per warp; softmax_cost_kernel then adds the partials in a fixed tree order.
struct SoftmaxArgs {
    const float *x, *truth;
    float *p, *delta, *loss, *unit_loss;
    int units, groups, n, cp, parity;
    float temp;
};
__global__ void __launch_bounds__(TB) softmax_kernel(const SoftmaxArgs a) {
    pdl_enter();
    const int unit = blockIdx.x * (TB / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (unit >= a.units) return;
    const int b = unit / a.groups, g = unit - b * a.groups;
    const size_t base = (size_t)b * a.cp + (size_t)g * a.n;
    float largest = a.parity == AET_PARITY_CPU ? -FLT_MAX : -INFINITY;
    for (int i = lane; i < a.n; i += 32) {
        float v = a.x[base + i];
        if (a.parity != AET_PARITY_CPU) v = (float)(int)v;   // the MTCS kernel compares through an int
        largest = fmaxf(largest, v);
    }
    for (int o = 16; o; o >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, o));
    float sum = 0.f;
    for (int i = lane; i < a.n; i += 32) {
        float e = expf(a.x[base + i] / a.temp - largest / a.temp);
        a.p[base + i] = e;
        sum += e;
    }
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float l = 0.f;
    for (int i = lane; i < a.n; i += 32) {
        float q = a.p[base + i] / sum;
        a.p[base + i] = q;
        if (a.truth) {
            float t = a.truth[base + i];
            float err = t ? -logf(q) : 0.f;
            a.loss[base + i] = err;
            a.delta[base + i] = t - q;
            l += err;
        }
    }
    for (int o = 16; o; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) a.unit_loss[unit] = l;
}
__global__ void __launch_bounds__(1024) softmax_cost_kernel(const float *unit_loss, int units, float *cost, float inv_batch,
                                                            float *mean_loss) {
    pdl_enter();
    __shared__ float sh[1024];
    float s = 0.f;
    for (int i = threadIdx.x; i < units; i += 1024) s += unit_loss[i];
    sh[threadIdx.x] = s;
    __syncthreads();
    for (int o = 512; o; o >>= 1) {
        if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        cost[0] = sh[0];
        if (mean_loss) mean_loss[0] = sh[0] * inv_batch;
    }
}

// ---------------------------------------------------------------------------- fused classifier head
// conv (no BN, linear) -> global average pool -> softmax + cross entropy, up to 32 classes: one block,
// one warp per sample (lane = class).  The forward kernel replaces avgpool_fwd + softmax + cost, the
// backward kernel replaces softmax backward + avgpool backward + the convolution's bias gradient.
struct HeadArgs {
    const float *y;        // conv output       [N][spatial][cp]
    float *avg;            // avg-pool output   [N][cp]
    float *p, *sm_delta, *loss;   // softmax output / delta / per-element error  [N][cp]
    const float *truth;    // [N][cp] or null
    float *cost;           // {sum, mean}
    float *avg_delta;      // [N][cp]
    float *conv_delta;     // [N][spatial][cp]
    float *bias_grad;      // [cp], accumulated
    int N, spatial, classes, cp, parity;
    float temp, loss_scale;
};
__global__ void __launch_bounds__(1024) head_forward_kernel(const HeadArgs a) {
    pdl_enter();
    __shared__ float warp_loss[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float lsum = 0.f;
    // Phase 1: the average pool with one (sample, class) pair per thread, so that the whole block has
    // its loads in flight at once; the pixels of a pair are summed in index order as the layer does.
    for (int e = threadIdx.x; e < a.N * a.cp; e += 1024) {
        const int n = e / a.cp, c = e - n * a.cp;
        if (c >= a.classes) continue;
        const float *src = a.y + (size_t)n * a.spatial * a.cp + c;
        float v = 0.f;
        int i = 0;
        for (; i + 8 <= a.spatial; i += 8) {
            float t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) t[u] = src[(size_t)(i + u) * a.cp];
#pragma unroll
            for (int u = 0; u < 8; ++u) v += t[u];
        }
        for (; i < a.spatial; ++i) v += src[(size_t)i * a.cp];
        a.avg[e] = v / a.spatial;
    }
    __syncthreads();   // the block's own global writes are visible to it after the barrier
    for (int n = warp; n < a.N; n += 32) {
        const float v = lane < a.classes ? a.avg[(size_t)n * a.cp + lane] : 0.f;
        float m = lane < a.classes ? (a.parity == AET_PARITY_CPU ? v : (float)(int)v) : -INFINITY;
        if (a.parity == AET_PARITY_CPU && lane >= a.classes) m = -FLT_MAX;
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float e = lane < a.classes ? expf(v / a.temp - m / a.temp) : 0.f;
        float sum = e;
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        float err = 0.f;
        if (lane < a.classes) {
            const float q = e / sum;
            a.p[(size_t)n * a.cp + lane] = q;
            if (a.truth) {
                const float t = a.truth[(size_t)n * a.cp + lane];
                err = t ? -logf(q) : 0.f;
                a.loss[(size_t)n * a.cp + lane] = err;
                a.sm_delta[(size_t)n * a.cp + lane] = t - q;
            }
        }
        for (int o = 16; o; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
        lsum += err;
    }
    if (lane == 0) warp_loss[warp] = lsum;
    __syncthreads();
    if (threadIdx.x == 0 && a.truth) {
        float c = 0.f;
        for (int w = 0; w < 32; ++w) c += warp_loss[w];
        a.cost[0] = c;
        a.cost[1] = c / a.N;
    }
}
__global__ void __launch_bounds__(1024) head_backward_kernel(const HeadArgs a) {
    pdl_enter();
    __shared__ float part[32][33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float bsum = 0.f;
    for (int n = warp; n < a.N; n += 32) {
        if (lane < a.classes) {
            const float d = a.loss_scale * a.sm_delta[(size_t)n * a.cp + lane];   // softmax backward into the avg-pool delta
            a.avg_delta[(size_t)n * a.cp + lane] = d;
            const float g = d / a.spatial;                                        // avg-pool backward into the conv delta
            float *dst = a.conv_delta + (size_t)n * a.spatial * a.cp + lane;
            for (int i = 0; i < a.spatial; ++i) { dst[(size_t)i * a.cp] = g; bsum += g; }
        }
    }
    part[warp][lane] = bsum;
    __syncthreads();
    if (warp == 0 && lane < a.classes && a.bias_grad) {
        float t = 0.f;
        for (int w = 0; w < 32; ++w) t += part[w][lane];
        a.bias_grad[lane] += t;
    }
}

// ---------------------------------------------------------------------------- small utilities
// ---------------------------------------------------------------------------- linear classifier head
// 1x1 convolution (bias, no activation) -> global average pool -> softmax + cross entropy is linear up
// to the softmax, so a network's training pass runs it on the pooled vectors instead of on the feature
// map: logits[n] = W * mean_px(x[n]) + b (exact FP32, S times fewer multiplies than the convolution),
// and backward: dx[n][px] = W^T g[n] / S for every pixel, dW = sum_n g[n] xbar[n]^T, db = sum_n g[n],
// with g = loss_scale * (truth - p).  The convolution's own output and delta tensors are only formed
// when a host tap asks for them.
struct LinHeadArgs {
    const float *x;        // convolution input [N][S][cp]
    const float *w, *b;    // weights [classes][cp], bias
    float *xbar;           // [N][cp] pooled input, kept for the weight gradient
    float *avg;            // avg-pool output = logits [N][ocp]
    float *p, *sm_delta, *loss;
    const float *truth;
    float *unit_loss;      // [N]
    float *cost;           // {sum, mean}
    unsigned int *ticket;
    float *avg_delta;      // [N][ocp]
    float *pd;             // delta of the convolution's input [N][S][cp], overwritten
    float *gw, *gb;        // weight / bias gradient accumulators
    int N, S, cp, classes, ocp, parity;
    float temp, loss_scale;
};

__global__ void __launch_bounds__(256) linhead_forward_kernel(const LinHeadArgs a) {
    pdl_enter();
    extern __shared__ float xs[];           // cp pooled inputs, then 32 logits
    __shared__ bool last;
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *xn = a.x + (size_t)n * a.S * a.cp;
    for (int c = threadIdx.x; c < a.cp; c += 256) {
        float s = 0.f;
        int px = 0;
        for (; px + 8 <= a.S; px += 8) {   // eight loads in flight; the sum keeps the pixel order
            float t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) t[u] = xn[(size_t)(px + u) * a.cp + c];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += t[u];
        }
        for (; px < a.S; ++px) s += xn[(size_t)px * a.cp + c];
        s /= a.S;
        xs[c] = s;
        a.xbar[(size_t)n * a.cp + c] = s;
    }
    float *lg = xs + a.cp;
    __syncthreads();
    for (int k = warp; k < a.classes; k += 8) {
        const float *wk = a.w + (size_t)k * a.cp;
        float d = 0.f;
        for (int c = lane; c < a.cp; c += 32) d += wk[c] * xs[c];
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) lg[k] = d + a.b[k];
    }
    __syncthreads();
    if (warp == 0) {
        const float v = lane < a.classes ? lg[lane] : 0.f;
        if (lane < a.ocp) a.avg[(size_t)n * a.ocp + lane] = lane < a.classes ? v : 0.f;
        float m = lane < a.classes ? (a.parity == AET_PARITY_CPU ? v : (float)(int)v) : -INFINITY;
        if (a.parity == AET_PARITY_CPU && lane >= a.classes) m = -FLT_MAX;
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float e = lane < a.classes ? expf(v / a.temp - m / a.temp) : 0.f;
        float sum = e;
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        float err = 0.f;
        if (lane < a.classes) {
            const float q = e / sum;
            a.p[(size_t)n * a.ocp + lane] = q;
            if (a.truth) {
                const float t = a.truth[(size_t)n * a.ocp + lane];
                err = t ? -logf(q) : 0.f;
                a.loss[(size_t)n * a.ocp + lane] = err;
                a.sm_delta[(size_t)n * a.ocp + lane] = t - q;
            }
        }
        for (int o = 16; o; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
        if (lane == 0) {
            a.unit_loss[n] = err;
            __threadfence();
            last = atomicAdd(a.ticket, 1u) == (unsigned)(a.N - 1);
        }
    }
    __syncthreads();
    if (!last || !a.truth) {
        if (last && threadIdx.x == 0) *a.ticket = 0u;
        return;
    }
    // the block that finished last adds the per-sample losses in index order
    __threadfence();
    if (warp == 0) {   // lane i adds samples i, i+32, ...; the lanes are combined by a fixed xor tree
        float c = 0.f;
        for (int i = lane; i < a.N; i += 32) c += __ldcg(a.unit_loss + i);
        for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) {
            a.cost[0] = c;
            a.cost[1] = c / a.N;
            *a.ticket = 0u;
        }
    }
}

__global__ void __launch_bounds__(256) linhead_backward_kernel(const LinHeadArgs a) {
    pdl_enter();
    __shared__ float g[32];
    extern __shared__ float gs[];   // weight-gradient blocks: g of every sample [N][classes], then the lane sums
    if ((int)blockIdx.x < a.N) {
        const int n = blockIdx.x;
        if (threadIdx.x < 32) {
            const float v = (int)threadIdx.x < a.classes ? a.loss_scale * a.sm_delta[(size_t)n * a.ocp + threadIdx.x] : 0.f;
            g[threadIdx.x] = v;
            if ((int)threadIdx.x < a.ocp) a.avg_delta[(size_t)n * a.ocp + threadIdx.x] = v;
        }
        __syncthreads();
        float *dn = a.pd + (size_t)n * a.S * a.cp;
        for (int c = threadIdx.x; c < a.cp; c += 256) {
            float v = 0.f;
            int k = 0;
            for (; k + 4 <= a.classes; k += 4) {
                const float w0 = a.w[(size_t)k * a.cp + c], w1 = a.w[(size_t)(k + 1) * a.cp + c];
                const float w2 = a.w[(size_t)(k + 2) * a.cp + c], w3 = a.w[(size_t)(k + 3) * a.cp + c];
                v += g[k] * w0; v += g[k + 1] * w1; v += g[k + 2] * w2; v += g[k + 3] * w3;
            }
            for (; k < a.classes; ++k) v += g[k] * a.w[(size_t)k * a.cp + c];
            v /= a.S;
            for (int px = 0; px < a.S; ++px) dn[(size_t)px * a.cp + c] = v;
        }
        return;
    }
    // weight gradient of 32 channels: eight sample lanes per channel, summed in a fixed order
    for (int i = threadIdx.x; i < a.N * a.classes; i += 256) {
        const int n = i / a.classes, k = i - n * a.classes;
        gs[i] = a.loss_scale * a.sm_delta[(size_t)n * a.ocp + k];
    }
    __syncthreads();
    const int cl = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const int c = ((int)blockIdx.x - a.N) * 32 + cl;
    float acc[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) acc[k] = 0.f;
    for (int n0 = 0; n0 < a.N; n0 += 128) {
        float xr[16];   // sixteen samples of this lane's channel, all loads in flight together
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int n = n0 + sl + 8 * u;
            xr[u] = (n < a.N && c < a.cp) ? a.xbar[(size_t)n * a.cp + c] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            if (k >= a.classes) break;
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int n = n0 + sl + 8 * u;
                if (n < a.N) acc[k] += gs[n * a.classes + k] * xr[u];   // the warp shares n: a broadcast read
            }
        }
    }
    float *red3 = gs + a.N * a.classes;   // [classes][8 sample lanes][32 channels]
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        if (k >= a.classes) break;
        red3[(k * 8 + sl) * 32 + cl] = acc[k];
    }
    __syncthreads();
    // warp sl finishes classes sl, sl+8, ...: its read-modify-writes of the gradient are independent
    for (int k = sl; k < a.classes; k += 8) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) t += red3[(k * 8 + q) * 32 + cl];
        if (c < a.cp) a.gw[(size_t)k * a.cp + c] += t;   // sum over pixels of (g / S) * x = g * mean_px(x)
    }
    if (blockIdx.x == (unsigned)a.N && (int)threadIdx.x < a.classes) {
        float t = 0.f;
        for (int n = 0; n < a.N; ++n) t += gs[n * a.classes + threadIdx.x];
        a.gb[threadIdx.x] += t;
    }
}
__global__ void axpy_kernel(float *y, const float *x, float a, size_t n4, int accumulate) {
    pdl_enter();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 v = ld4(x + i * 4);
    v.x *= a; v.y *= a; v.z *= a; v.w *= a;
    if (accumulate) {
        float4 q = ld4(y + i * 4);
        v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
    }
    st4(y + i * 4, v);
}
__global__ void fill_kernel(float *p, float v, size_t n4) {
    pdl_enter();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n4) st4(p + i * 4, make_float4(v, v, v, v));
}
__global__ void step_counter_kernel(unsigned long long *ctr) {
    pdl_enter(); ctr[0] += 1ull; }

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// Counter-based uniforms: u = top 24 bits of mix64(seed + step*A + (index+1)*B).
__global__ void dropout_fwd_kernel(float *x, float *rnd, size_t n, int c, int cp, float prob, float scale,
                                   unsigned long long seed, const unsigned long long *step, int generate) {
    pdl_enter();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float r;
    if (generate) {
        unsigned long long s = seed + step[0] * 0xD1342543DE82EF95ull + (i + 1) * 0x9E3779B97F4A7C15ull;
        r = (float)(mix64(s) >> 40) * (1.0f / 16777216.0f);
        rnd[i] = r;
    } else {
        r = rnd[i];
    }
    if ((int)(i % cp) >= c) return;
    x[i] = r < prob ? 0.f : x[i] * scale;
}
__global__ void dropout_bwd_kernel(float *d, const float *rnd, size_t n, float prob, float scale) {
    pdl_enter();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    d[i] = rnd[i] < prob ? 0.f : d[i] * scale;
}

// ---------------------------------------------------------------------------- SGD with momentum
// u = U + G (+ decay_term * w for weights); w += rate * u; U = momentum * u; G = 0.
// Same operation order as the three reference passes (U += -decay*B*W; W += lr/B*U; U *= momentum).
// The slice of the gradient arena that is summed over the ranks inside the update kernel.
struct TailArgs {
    const float *peer_buf[16];                 // rank q's published slices (parity buffers back to back)
    const volatile unsigned long long *flags;  // local [2][16]: flags[parity][q] = epoch once q has published
    const unsigned long long *epoch;
    unsigned long long lo, n, cap;
    int world;
    int *status;
    int *gate;   // written by tail_wait_kernel: 1 = every rank's slice of this step has arrived, 0 = the wait ran out
};

// Copies this rank's slice into its published buffer and raises its flag in every peer's memory: data,
// system-wide fence, ticket; the block that takes the last ticket writes the flags.  The parity alternates
// with the step, so a rank that runs ahead never overwrites a buffer a slower peer still reads (it cannot
// pass the next step's wait before that peer has published there).  Block 0 advances the epoch; the
// others read it after the ticket of the previous launch has been reset, i.e. epoch + 1 is this launch.
struct PublishArgs {
    unsigned long long *peer_flags[8];
    float *buf_local;
    unsigned long long *epoch;
    unsigned int *ticket;
    int rank;
};
__global__ void __launch_bounds__(1024) tail_publish_kernel(const float *G, const TailArgs t, const PublishArgs p) {
    pdl_enter();
    const unsigned long long e = *p.epoch + 1ull, parity = e & 1ull;   // *epoch is only advanced by the last block, below
    float *dst = p.buf_local + parity * t.cap;
    for (unsigned long long i = ((unsigned long long)blockIdx.x * 1024ull + threadIdx.x) * 4ull; i < t.n; i += (unsigned long long)gridDim.x * 4096ull)
        st4(dst + i, ld4(G + t.lo + i));
    __syncthreads();
    __shared__ bool last;
    if (threadIdx.x == 0) {
        __threadfence_system();   // cumulative: orders the whole block's copies (joined by the barrier) before the ticket
        last = atomicAdd(p.ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    if ((int)threadIdx.x < t.world && threadIdx.x < 8) {
        __threadfence_system();   // after the last ticket every block's copies are ordered before the flags

        volatile unsigned long long *f = p.peer_flags[threadIdx.x] + parity * 16ull + (unsigned long long)p.rank;
        *f = e;
    }
    if (threadIdx.x == 0) { *p.epoch = e; *p.ticket = 0u; }
}

// Limit of the peer-flag wait below (nanoseconds); set per device by elementwise_set_wait_limit.
__constant__ unsigned long long g_flag_wait_limit_ns = 1000000000ull;

// Non-finite scrub of the reference's GPU update.  kind 1 = a weight segment: a NaN/Inf pending update becomes 0
// (resetNanAndInf) and a NaN/Inf weight becomes 1 / (index + 1) (fixNanAndInf), mtcs/MtcsConvLayer.c:586-587,
// mtcs/MtcsTool.c:77-107.  kind 2 = a bias / scale segment of a batch-norm layer with try_fix_nan: the pending
// update becomes 1 / (index + 1), dnn/NLayer.c:318-323.  `index` is the element's position in its segment.
// Returns true when something was replaced.
__device__ __forceinline__ bool scrub1(float &w, float &u, int kind, size_t index) {
    bool hit = false;
    if (kind == 1) {
        if (isnan(u) || isinf(u)) { u = 0.f; hit = true; }
        if (isnan(w) || isinf(w)) { w = 1.0f / ((float)index + 1.f); hit = true; }
    } else if (kind == 2) {
        if (isnan(u) || isinf(u)) { u = 1.0f / ((float)index + 1.f); hit = true; }
    }
    return hit;
}
__device__ __forceinline__ bool scrub4(float4 &w, float4 &u, int kind, size_t index) {
    bool hit = scrub1(w.x, u.x, kind, index);
    hit |= scrub1(w.y, u.y, kind, index + 1);
    hit |= scrub1(w.z, u.z, kind, index + 2);
    hit |= scrub1(w.w, u.w, kind, index + 3);
    return hit;
}

// One warp waits (bounded) until every rank has published its slice of this step and leaves the verdict in `gate`
// for the update kernel that follows: a wait that runs out must stop the WHOLE update, not the blocks that happened
// to notice, or the parameters would be left half updated.
__global__ void tail_wait_kernel(const TailArgs t) {
    pdl_enter();
    const unsigned long long e = *t.epoch, parity = e & 1ull;
    bool ok = true;
    if ((int)threadIdx.x < t.world) {
        const volatile unsigned long long *f = t.flags + parity * 16ull + threadIdx.x;
        unsigned long long t0 = 0;
        unsigned int spins = 0;
        while (*f < e) {
            if ((++spins & 255u) == 0u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                else if (now - t0 > g_flag_wait_limit_ns) { ok = false; break; }   // a peer never arrived: give up
            }
        }
    }
    const bool all_ok = __all_sync(0xffffffffu, ok);
    __threadfence_system();   // acquire: the update kernel reads the peers' slices after their flags
    if (threadIdx.x == 0) {
        *t.gate = all_ok ? 1 : 0;
        if (!all_ok && t.status) atomicOr(t.status, AET_STATUS_TIMEOUT);
    }
}

// seg_table: four floats per segment {learning-rate multiplier, decay flag, scrub kind, first block (int bits)}
__global__ void __launch_bounds__(TB) sgd_arena_kernel(float *W, float *U, float *G, const int *block_seg,
                                                       const float *seg_table, const float *hyper, const TailArgs t, int *status) {
    pdl_enter();
    const int seg = block_seg[blockIdx.x];
    const bool frozen = seg_table[4 * seg] < 0.f;   // not updated now: the gradient joins the pending update, nothing else moves
    const float rate = hyper[0] * seg_table[4 * seg];
    const float momentum = hyper[1];
    const float decay_term = seg_table[4 * seg + 1] != 0.f ? hyper[2] : 0.f;
    const int scrub = (int)seg_table[4 * seg + 2];
    const size_t i = ((size_t)blockIdx.x * TB + threadIdx.x) * 4;
    float4 w = ld4(W + i), u = ld4(U + i), g = ld4(G + i);
    const size_t b0 = (size_t)blockIdx.x * TB * 4;
    if (t.world > 1) {
        // A peer's gradients never arrived (tail_wait_kernel gave up): no block updates anything, so that the
        // parameters of this rank stay those of the last complete step.
        if (*t.gate == 0) return;
        if (b0 >= t.lo && b0 < t.lo + t.n) {
            // this block's gradients are the sum of every rank's published slice, added in rank order
            const unsigned long long parity = *t.epoch & 1ull;
            // (all ranks' loads are issued before the first sum: one NVLink round trip instead of one per rank)
            float4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (q < t.world) v[q] = __ldcv(reinterpret_cast<const float4 *>(t.peer_buf[q] + parity * t.cap + (i - t.lo)));
            g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (q < t.world) { g.x += v[q].x; g.y += v[q].y; g.z += v[q].z; g.w += v[q].w; }
        }
    }
    u.x += g.x; u.y += g.y; u.z += g.z; u.w += g.w;
    if (frozen) {
        st4(U + i, u);
        st4(G + i, make_float4(0.f, 0.f, 0.f, 0.f));
        return;
    }
    if (scrub) {
        const size_t first = (size_t)__float_as_int(seg_table[4 * seg + 3]) * TB * 4;
        if (scrub4(w, u, scrub, i - first) && status) atomicOr(status, AET_STATUS_NAN);
    }
    u.x += decay_term * w.x; u.y += decay_term * w.y; u.z += decay_term * w.z; u.w += decay_term * w.w;
    w.x += rate * u.x; w.y += rate * u.y; w.z += rate * u.z; w.w += rate * u.w;
    u.x *= momentum; u.y *= momentum; u.z *= momentum; u.w *= momentum;
    st4(W + i, w);
    st4(U + i, u);
    st4(G + i, make_float4(0.f, 0.f, 0.f, 0.f));
}
// Adam, mtcs/MtcsConvLayer.c:494-524 (adam_update_gpu), the reference's eight launches per parameter array in one pass:
//   m *= B1; v *= B2; d += (-decay*batch) * w; m += (1-B1) * d; d *= d; v += (1-B2) * d;
//   w += rate * (m / (1-B1^t)) / (sqrtf(v / (1-B2^t)) + eps); d = 0
// The reference applies the same routine, decay included, to weights, biases and scales (:600-612).  d = U + G: the
// pending-update buffer carries nothing between steps under Adam.  hyper[4..7] = {rate, -decay*batch, 1-B1^t, 1-B2^t}.
__global__ void __launch_bounds__(TB) adam_arena_kernel(float *W, float *U, float *G, float *M, float *V, const int *block_seg,
                                                        const float *seg_table, const float *hyper, float B1, float B2, float eps,
                                                        int *status) {
    pdl_enter();
    const int seg = block_seg[blockIdx.x];
    const float rate = hyper[4] * seg_table[4 * seg];
    const float decay_term = hyper[5], c1 = hyper[6], c2 = hyper[7];
    const int scrub = (int)seg_table[4 * seg + 2];
    const size_t i = ((size_t)blockIdx.x * TB + threadIdx.x) * 4;
    float4 w = ld4(W + i), u = ld4(U + i), g = ld4(G + i), m = ld4(M + i), v = ld4(V + i);
    u.x += g.x; u.y += g.y; u.z += g.z; u.w += g.w;
    if (seg_table[4 * seg] < 0.f) {   // not updated now: the gradient joins the pending update, nothing else moves
        st4(U + i, u);
        st4(G + i, make_float4(0.f, 0.f, 0.f, 0.f));
        return;
    }
    if (scrub) {
        const size_t first = (size_t)__float_as_int(seg_table[4 * seg + 3]) * TB * 4;
        if (scrub4(w, u, scrub, i - first) && status) atomicOr(status, AET_STATUS_NAN);
    }
    float *wp = &w.x, *up = &u.x, *mp = &m.x, *vp = &v.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float mm = __fmul_rn(mp[k], B1), vv = __fmul_rn(vp[k], B2);
        float d = __fadd_rn(up[k], __fmul_rn(decay_term, wp[k]));
        mm = __fadd_rn(mm, __fmul_rn(1.f - B1, d));
        d = __fmul_rn(d, d);
        vv = __fadd_rn(vv, __fmul_rn(1.f - B2, d));
        const float mhat = mm / c1, vhat = vv / c2;
        wp[k] = wp[k] + rate * mhat / (sqrtf(vhat) + eps);
        mp[k] = mm; vp[k] = vv;
    }
    st4(W + i, w);
    st4(M + i, m);
    st4(V + i, v);
    st4(U + i, make_float4(0.f, 0.f, 0.f, 0.f));
    st4(G + i, make_float4(0.f, 0.f, 0.f, 0.f));
}

__global__ void sgd_segment_kernel(float *W, float *U, float *G, size_t n4, float rate, float momentum, float decay_term,
                                   int scrub, int *status) {
    pdl_enter();
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x);
    if (i >= n4) return;
    i *= 4;
    float4 w = ld4(W + i), u = ld4(U + i), g = ld4(G + i);
    u.x += g.x; u.y += g.y; u.z += g.z; u.w += g.w;
    if (scrub && scrub4(w, u, scrub, i) && status) atomicOr(status, AET_STATUS_NAN);
    u.x += decay_term * w.x; u.y += decay_term * w.y; u.z += decay_term * w.z; u.w += decay_term * w.w;
    w.x += rate * u.x; w.y += rate * u.y; w.z += rate * u.z; w.w += rate * u.w;
    u.x *= momentum; u.y *= momentum; u.z *= momentum; u.w *= momentum;
    st4(W + i, w);
    st4(U + i, u);
    st4(G + i, make_float4(0.f, 0.f, 0.f, 0.f));
}

__global__ void param_hash_kernel(const float *p, size_t n, unsigned long long *hash) {
    pdl_enter();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long h = 0;
    if (i < n) h = mix64((unsigned long long)__float_as_uint(p[i]) ^ ((i + 1) * 0x9E3779B97F4A7C15ull));
    for (int o = 16; o; o >>= 1) h += __shfl_xor_sync(0xffffffffu, h, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(hash, h);   // integer addition: order-independent
}

// Image augmentation: NImage.rotateCrop + flip + distort (dnn/NImage.c:138-157,201-337,346-362,551-572) fused into one pass,
// one thread per output pixel (all channels).  Source NCHW as uploaded, destination the network input (NHWC, padded).
// The coordinate arithmetic keeps the reference's double intermediates; sampling and colour math are float as there.
__device__ __forceinline__ float aug_pixel(const float *im, int w, int h, int x, int y) {
    return (x < 0 || x >= w || y < 0 || y >= h) ? 0.f : __ldg(im + (size_t)y * w + x);
}
__device__ __forceinline__ float aug_bilinear(const float *im, int w, int h, float x, float y) {
    const int ix = (int)floorf(x), iy = (int)floorf(y);
    const float dx = x - ix, dy = y - iy;
    // products and sums in the reference's order, without contraction into fused multiply-adds
    float val = __fmul_rn(__fmul_rn(1 - dy, 1 - dx), aug_pixel(im, w, h, ix, iy));
    val = __fadd_rn(val, __fmul_rn(__fmul_rn(dy, 1 - dx), aug_pixel(im, w, h, ix, iy + 1)));
    val = __fadd_rn(val, __fmul_rn(__fmul_rn(1 - dy, dx), aug_pixel(im, w, h, ix + 1, iy)));
    val = __fadd_rn(val, __fmul_rn(__fmul_rn(dy, dx), aug_pixel(im, w, h, ix + 1, iy + 1)));
    return val;
}
__global__ void augment_kernel(const float *__restrict__ src, int n, int c, int sh, int sw, float *__restrict__ dst, int size, int cp,
                               const aet_augment *__restrict__ params) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)n * size * size) return;
    const int x = (int)(e % size);
    const int y = (int)((e / size) % size);
    const int b = (int)(e / ((size_t)size * size));
    const aet_augment p = params[b];
    const int w = size, h = size;
    const float cx = (float)(sw / 2.0), cy = (float)(sh / 2.0);
    const float cr = (float)cos((double)p.rad), sr = (float)sin((double)p.rad);
    const float dx1 = p.dx / p.scale * p.aspect, dy1 = p.dy / p.scale;
    const int xs = p.flip ? w - 1 - x : x;      // the flipped crop's pixel x is the crop's pixel w-1-x
    const float rx = (float)((double)cr * (((double)xs - w / 2.) / p.scale * p.aspect + dx1) - (double)sr * (((double)y - h / 2.) / p.scale + dy1) + cx);
    const float ry = (float)((double)sr * (((double)xs - w / 2.) / p.scale * p.aspect + dx1) + (double)cr * (((double)y - h / 2.) / p.scale + dy1) + cy);
    float *out = dst + e * cp;
    const float *img = src + (size_t)b * c * sh * sw;
    if (c != 3) {
        for (int k = 0; k < cp; ++k) out[k] = k < c ? aug_bilinear(img + (size_t)k * sh * sw, sw, sh, rx, ry) : 0.f;
        return;
    }
    float r = aug_bilinear(img, sw, sh, rx, ry), g = aug_bilinear(img + (size_t)sh * sw, sw, sh, rx, ry),
          bl = aug_bilinear(img + (size_t)2 * sh * sw, sw, sh, rx, ry);
    // RGB -> HSV
    const float mx = fmaxf(r, fmaxf(g, bl)), mn = fminf(r, fminf(g, bl));
    const float delta = mx - mn;
    float hh, ss, vv = mx;
    if (mx == 0.f) { ss = 0.f; hh = 0.f; }
    else {
        ss = delta / mx;
        if (r == mx) hh = (g - bl) / delta;
        else if (g == mx) hh = 2.f + (bl - r) / delta;
        else hh = 4.f + (r - g) / delta;
        if (hh < 0.f) hh += 6.f;
        hh = (float)((double)hh / 6.);
    }
    ss = __fmul_rn(ss, p.dsat);
    vv = __fmul_rn(vv, p.dexp);
    hh = __fadd_rn(hh, p.dhue);
    if (hh > 1.f) hh -= 1.f;
    if (hh < 0.f) hh += 1.f;
    // HSV -> RGB
    const float hq = __fmul_rn(6.f, hh);
    if (ss == 0.f) { r = g = bl = vv; }
    else {
        const int index = (int)floorf(hq);
        const float f = hq - index;
        const float pp = __fmul_rn(vv, 1.f - ss);
        const float q = __fmul_rn(vv, 1.f - __fmul_rn(ss, f));
        const float t = __fmul_rn(vv, 1.f - __fmul_rn(ss, 1.f - f));
        if (index == 0) { r = vv; g = t; bl = pp; }
        else if (index == 1) { r = q; g = vv; bl = pp; }
        else if (index == 2) { r = pp; g = vv; bl = t; }
        else if (index == 3) { r = pp; g = q; bl = vv; }
        else if (index == 4) { r = t; g = pp; bl = vv; }
        else { r = vv; g = pp; bl = q; }
    }
    *reinterpret_cast<float4 *>(out) = make_float4(fminf(fmaxf(r, 0.f), 1.f), fminf(fmaxf(g, 0.f), 1.f), fminf(fmaxf(bl, 0.f), 1.f), 0.f);
}

// DnnUtils.topK (dnn/DnnUtils.c:463-477), one thread per sample running the reference's own insertion loop, so ties
// and order come out exactly as there: index[j] = position of the j-th largest score, strict '>' comparisons.
__global__ void top_k_kernel(const float *__restrict__ scores, int samples, int n, int ld, int k, int *__restrict__ index) {
    pdl_enter();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= samples) return;
    const float *a = scores + (size_t)s * ld;
    int *idx = index + (size_t)s * k;
    for (int j = 0; j < k; ++j) idx[j] = -1;
    for (int i = 0; i < n; ++i) {
        int curr = i;
        for (int j = 0; j < k; ++j) {
            if (idx[j] < 0 || a[curr] > a[idx[j]]) {
                const int swap = curr;
                curr = idx[j];
                idx[j] = swap;
            }
            if (curr < 0) break;   // an empty slot was filled: the remaining slots are empty too and stay so
        }
    }
}

struct ReducePlan {
    CMap m;
    int blocks;
    long long pix_per_block;
};
ReducePlan plan_reduce(aet_context *ctx, long long pixels, int cp) {
    ReducePlan p;
    p.m = make_cmap(cp);
    long long want = 4LL * ctx->sm_count / p.m.cslabs;
    if (want < 1) want = 1;
    long long min_pix = (long long)p.m.pl_count * 8;   // at least 8 pixels per thread
    long long maxb = (pixels + min_pix - 1) / min_pix;
    if (want > maxb) want = maxb;
    if (want < 1) want = 1;
    p.pix_per_block = (pixels + want - 1) / want;
    p.blocks = (int)((pixels + p.pix_per_block - 1) / p.pix_per_block);
    return p;
}
ReducePlan plan_apply(aet_context *ctx, long long pixels, int cp) {
    ReducePlan p;
    p.m = make_cmap(cp);
    long long want = 8LL * ctx->sm_count / p.m.cslabs;
    long long min_pix = (long long)p.m.pl_count * 2;
    long long maxb = (pixels + min_pix - 1) / min_pix;
    if (want > maxb) want = maxb;
    if (want < 1) want = 1;
    p.pix_per_block = (pixels + want - 1) / want;
    p.blocks = (int)((pixels + p.pix_per_block - 1) / p.pix_per_block);
    return p;
}

}  // namespace

bool pdl_enabled() {
    static const bool on = []() { const char *e = getenv("AET_NO_PDL"); return !(e && *e && *e != '0'); }();
    return on;
}
static thread_local bool g_pdl_skip = false;
void pdl_skip_next() { g_pdl_skip = true; }
bool pdl_take_skip() {
    const bool s = g_pdl_skip;
    g_pdl_skip = false;
    return s;
}

int aet_check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        aet_set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
        return AET_E_CUDA;
    }
    return AET_OK;
}

// Batch statistics of l->x (the convolution result) into mean / variance / inv_std.
int k_bn_stats(aet_layer *l, int update_rolling, const ConvStats *from_epilogue) {
    aet_context *ctx = l->ctx;
    const long long pixels = (long long)l->batch * l->oh * l->ow;
    ReducePlan p = plan_reduce(ctx, pixels, l->ocp);
    float *partial = nullptr;
    const bool have = from_epilogue && from_epilogue->rows > 0;   // the convolution's epilogue already summed its tiles
    if (have) {
        partial = from_epilogue->partial;
        p.blocks = from_epilogue->rows;
    } else {
        AET_TRY(ctx_scratch(ctx, (size_t)p.blocks * 2 * l->ocp * sizeof(float), &partial));
    }
    // The statistics are accumulated around a per-channel shift so that the one-pass variance does
    // not cancel; any value near the data works, and the previous step's batch mean is already there.
    ReduceArgs a = {};
    a.x = l->x->d; a.shift = l->mean; a.partial = partial; a.pixels = pixels; a.cp = l->ocp;
    a.pix_per_block = p.pix_per_block; a.m = p.m;
    if (!have) {
        LaunchScope s(ctx, "bn_stats", (double)pixels * l->ocp * 4.0, 0);
        launch_k(ctx->stream, dim3(p.blocks, p.m.cslabs), TB, 0, reduce2_kernel<0>, a);
        AET_TRY(aet_check_launch("bn_stats"));
    }
    FinalizeArgs f = {};
    f.partial = partial; f.blocks = p.blocks; f.cp = l->ocp; f.c = l->oc; f.m = pixels;
    f.parity = ctx->parity; f.update_rolling = update_rolling; f.shift = l->mean;
    f.mean = l->mean; f.variance = l->variance; f.inv = l->inv_std;
    f.rolling_mean = l->rolling_mean; f.rolling_variance = l->rolling_variance;
    LaunchScope s(ctx, "bn_stats_finalize", 0, 0);
    launch_k(ctx->stream, (l->ocp + FIN_CH - 1) / FIN_CH, 1024, 0, finalize_kernel<0>, f);
    return aet_check_launch("bn_stats_finalize");
}

// output = act(bn(x)) with the batch statistics (or the rolling ones for inference).
int k_bn_apply(aet_layer *l, int use_rolling) {
    aet_context *ctx = l->ctx;
    const long long pixels = (long long)l->batch * l->oh * l->ow;
    if (use_rolling) {
        LaunchScope s(ctx, "bn_eval_inv", 0, 0);
        launch_k(ctx->stream, (l->ocp + 127) / 128, 128, 0, eval_inv_kernel, l->rolling_variance, l->inv_std, l->oc, l->ocp,
                                                                        ctx->parity);
        AET_TRY(aet_check_launch("bn_eval_inv"));
    }
    ReducePlan p = plan_apply(ctx, pixels, l->ocp);
    ApplyArgs a = {};
    a.x = l->x->d; a.y = l->output->d;
    a.mean = use_rolling ? l->rolling_mean : l->mean; a.inv = l->inv_std;
    a.gamma = layer_s(l); a.beta = layer_b(l);
    a.act = l->act; a.cp = l->ocp; a.pixels = pixels; a.pix_per_block = p.pix_per_block; a.m = p.m;
    LaunchScope s(ctx, "bn_apply_act", (double)pixels * l->ocp * 8.0, 0);
    launch_k(ctx->stream, dim3(p.blocks, p.m.cslabs), TB, 0, bn_apply_kernel, a);
    return aet_check_launch("bn_apply_act");
}

static PoolGather make_pool_gather(const aet_layer *pool) {
    PoolGather g;
    g.delta = pool->delta->d; g.idx = pool->indexes;
    g.C = pool->c; g.H = pool->h; g.W = pool->w; g.OH = pool->oh; g.OW = pool->ow;
    g.size = pool->size; g.sx = pool->stride_x; g.sy = pool->stride_y; g.off = -pool->pad / 2;
    g.simple2 = (g.size == 2 && g.sx == 2 && g.sy == 2 && g.off == 0) ? 1 : 0;
    return g;
}

// output of the following max-pool layer straight from the convolution result: pool(act(bn(x))).
int k_bn_pool_forward(aet_layer *l, aet_layer *pool, int use_rolling) {
    aet_context *ctx = l->ctx;
    if (use_rolling) {
        LaunchScope s(ctx, "bn_eval_inv", 0, 0);
        launch_k(ctx->stream, (l->ocp + 127) / 128, 128, 0, eval_inv_kernel, l->rolling_variance, l->inv_std, l->oc, l->ocp,
                                                                        ctx->parity);
        AET_TRY(aet_check_launch("bn_eval_inv"));
    }
    BnPoolArgs b = {};
    PoolArgs &a = b.p;
    a.x = l->x->d; a.y = pool->output->d; a.idx = pool->indexes;
    a.N = pool->batch; a.C = pool->c; a.H = pool->h; a.W = pool->w; a.cp = pool->cp; a.OH = pool->oh; a.OW = pool->ow;
    a.size = pool->size; a.sx = pool->stride_x; a.sy = pool->stride_y; a.off = -pool->pad / 2; a.parity = ctx->parity;
    a.total = (long long)pool->batch * pool->oh * pool->ow * (pool->cp / 4);
    b.mean = use_rolling ? l->rolling_mean : l->mean; b.inv = l->inv_std; b.gamma = layer_s(l); b.beta = layer_b(l);
    b.act = l->act;
    b.ymax = (l->stem && !use_rolling) ? l->stem_ymax : nullptr;   // eligible layers have even maps: every window takes the 2x2 branch
    b.code = l->stem_code;
    const double bytes = 4.0 * pool->batch * pool->h * pool->w * pool->cp + (b.ymax ? 13.0 : 8.0) * pool->batch * pool->oh * pool->ow * pool->cp;
    LaunchScope s(ctx, "bn_act_maxpool_fwd", bytes, 0);
    launch_k(ctx->stream, (unsigned)((a.total + TB - 1) / TB), TB, 0, bn_pool_fwd_kernel, b);
    return aet_check_launch("bn_act_maxpool_fwd");
}

// delta <- BN backward of (delta * act'(output)); accumulates the scale (and, MTCS parity, shift) gradients.
// With `pool` set, the incoming delta is gathered from that max-pool layer instead of being read.
int k_bn_backward(aet_layer *l, aet_layer *pool) {
    aet_context *ctx = l->ctx;
    const long long pixels = (long long)l->batch * l->oh * l->ow;
    ReducePlan p = plan_reduce(ctx, pixels, l->ocp);
    float *partial = nullptr;
    AET_TRY(ctx_scratch(ctx, (size_t)p.blocks * 2 * l->ocp * sizeof(float), &partial));
    ReduceArgs a = {};
    a.x = l->x->d; a.delta = l->delta->d; a.mean = l->mean; a.inv = l->inv_std;
    a.gamma = layer_s(l); a.beta = layer_b(l); a.partial = partial; a.act = l->act;
    a.pixels = pixels; a.cp = l->ocp; a.pix_per_block = p.pix_per_block; a.m = p.m;
    const double pool_bytes = pool ? 8.0 * pool->batch * pool->oh * pool->ow * pool->cp : 0.0;
    const bool window_major = pool && pool->size == 2 && pool->stride_x == 2 && pool->stride_y == 2 && pool->pad / 2 == 0 &&
                              pool->h % 2 == 0 && pool->w % 2 == 0 && TB % (l->ocp / 4) == 0 &&
                              (long long)pool->batch * pool->oh * pool->ow * (pool->cp / 4) < (1LL << 31);
    PoolWinArgs w = {};
    if (window_major) {
        w.x = l->x->d; w.dx = l->delta->d; w.pdelta = pool->delta->d; w.pidx = pool->indexes;
        w.mean = l->mean; w.inv = l->inv_std; w.gamma = layer_s(l); w.beta = layer_b(l); w.coef = l->bwd_coef;
        w.act = l->act; w.cp = l->ocp; w.C = pool->c; w.H = pool->h; w.W = pool->w; w.OH = pool->oh; w.OW = pool->ow;
        w.total = (unsigned)((long long)pool->batch * pool->oh * pool->ow * (pool->cp / 4));
        // one wave of exactly the blocks that are resident together (the kernel is a grid-stride loop): a
        // partial second wave would run at a fraction of the bandwidth
        int &resident_reduce = ctx->resident_bn_reduce;   // per context: occupancy is a property of the device
        if (!resident_reduce &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_reduce, bn_bwd_poolwin_kernel<false>, TB, 0) != cudaSuccess)
            resident_reduce = 2;
        int blocks = resident_reduce * ctx->sm_count;
        const int maxb = (int)((w.total + TB - 1) / TB);
        if (blocks > maxb) blocks = maxb;
        p.blocks = blocks;
        AET_TRY(ctx_scratch(ctx, (size_t)p.blocks * 2 * l->ocp * sizeof(float), &partial));
        w.partial = partial;
        LaunchScope s(ctx, "bn_bwd_reduce_poolwin", (double)pixels * l->ocp * 4.0 + pool_bytes, 0);
        launch_k(ctx->stream, p.blocks, TB, 0, bn_bwd_poolwin_kernel<false>, w);
        AET_TRY(aet_check_launch("bn_bwd_reduce_poolwin"));
    } else if (pool) {
        a.pool = make_pool_gather(pool);
        LaunchScope s(ctx, "bn_bwd_reduce_pool", (double)pixels * l->ocp * 4.0 + pool_bytes, 0);
        launch_k(ctx->stream, dim3(p.blocks, p.m.cslabs), TB, 0, reduce2_kernel<1, true>, a);
        AET_TRY(aet_check_launch("bn_bwd_reduce_pool"));
    } else {
        LaunchScope s(ctx, "bn_bwd_reduce", (double)pixels * l->ocp * 8.0, 0);
        launch_k(ctx->stream, dim3(p.blocks, p.m.cslabs), TB, 0, reduce2_kernel<1>, a);
        AET_TRY(aet_check_launch("bn_bwd_reduce"));
    }
    FinalizeArgs f = {};
    f.partial = partial; f.blocks = p.blocks; f.cp = l->ocp; f.c = l->oc; f.m = pixels; f.parity = ctx->parity;
    f.variance = l->variance; f.inv = l->inv_std; f.gamma = layer_s(l);
    f.g_gamma = layer_sG(l); f.g_beta = layer_bG(l); f.coef = l->bwd_coef;
    {
        LaunchScope s(ctx, "bn_bwd_finalize", 0, 0);
        launch_k(ctx->stream, (l->ocp + FIN_CH - 1) / FIN_CH, 1024, 0, finalize_kernel<1>, f);
        AET_TRY(aet_check_launch("bn_bwd_finalize"));
    }
    ReducePlan q = plan_apply(ctx, pixels, l->ocp);
    BwdApplyArgs b = {};
    b.x = l->x->d; b.delta = l->delta->d; b.mean = l->mean; b.inv = l->inv_std;
    b.gamma = layer_s(l); b.beta = layer_b(l); b.coef = l->bwd_coef; b.act = l->act; b.cp = l->ocp;
    b.pixels = pixels; b.pix_per_block = q.pix_per_block; b.m = q.m;
    if (window_major) {
        int &resident_apply = ctx->resident_bn_apply;
        if (!resident_apply &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_apply, bn_bwd_poolwin_kernel<true>, TB, 0) != cudaSuccess)
            resident_apply = 2;
        const int want = 2 * resident_apply * ctx->sm_count;   // two full waves
        const int blocks = (int)((w.total + TB - 1) / TB) < want ? (int)((w.total + TB - 1) / TB) : want;
        LaunchScope s(ctx, "bn_bwd_apply_poolwin", (double)pixels * l->ocp * 8.0 + pool_bytes, 0);
        launch_k(ctx->stream, blocks, TB, 0, bn_bwd_poolwin_kernel<true>, w);
        return aet_check_launch("bn_bwd_apply_poolwin");
    }
    if (pool) {
        b.pool = make_pool_gather(pool);
        LaunchScope s(ctx, "bn_bwd_apply_pool", (double)pixels * l->ocp * 8.0 + pool_bytes, 0);
        launch_k(ctx->stream, dim3(q.blocks, q.m.cslabs), TB, 0, bn_bwd_apply_kernel<true>, b);
        return aet_check_launch("bn_bwd_apply_pool");
    }
    LaunchScope s(ctx, "bn_bwd_apply", (double)pixels * l->ocp * 12.0, 0);
    launch_k(ctx->stream, dim3(q.blocks, q.m.cslabs), TB, 0, bn_bwd_apply_kernel<false>, b);
    return aet_check_launch("bn_bwd_apply");
}

// The full-resolution delta of a layer whose backward went through the pool-sized path: the BN backward apply pass with
// the coefficients that pass left behind (host taps only).
int k_stem_delta(aet_layer *l, aet_layer *pool) {
    aet_context *ctx = l->ctx;
    PoolWinArgs w = {};
    w.x = l->x->d; w.dx = l->delta->d; w.pdelta = pool->delta->d; w.pidx = pool->indexes;
    w.mean = l->mean; w.inv = l->inv_std; w.gamma = layer_s(l); w.beta = layer_b(l); w.coef = l->bwd_coef;
    w.act = l->act; w.cp = l->ocp; w.C = pool->c; w.H = pool->h; w.W = pool->w; w.OH = pool->oh; w.OW = pool->ow;
    w.total = (unsigned)((long long)pool->batch * pool->oh * pool->ow * (pool->cp / 4));
    const int blocks = (int)((w.total + TB - 1) / TB) < 8 * ctx->sm_count ? (int)((w.total + TB - 1) / TB) : 8 * ctx->sm_count;
    LaunchScope s(ctx, "bn_bwd_apply_poolwin", 0, 0);
    launch_k(ctx->stream, blocks, TB, 0, bn_bwd_poolwin_kernel<true>, w);
    return aet_check_launch("bn_bwd_apply_poolwin");
}

#include "stem.cuh"

// ---------------------------------------------------------------------------- shortcut (residual add)
struct ShortcutArgs {
    const float *in;        // forward: layer input; backward: unused
    float *out;             // forward: output; backward: this layer's delta (scaled in place by the activation gradient)
    const float *y;         // backward: this layer's output
    float *add[4];          // forward: the sources' outputs; backward: the sources' deltas
    int add_cp[4], add_lazy[4];
    float *pd;              // backward: previous layer's delta (may be null)
    int pd_lazy;
    int n, C, cp, act;
    long long total;        // pixels * cp / 4
};
// out = act(in + sum_i add_i) over the channels both tensors have; pad lanes stay zero.
__global__ void __launch_bounds__(TB) shortcut_fwd_kernel(const ShortcutArgs a) {
    pdl_enter();
    const long long e = (long long)blockIdx.x * TB + threadIdx.x;
    if (e >= a.total) return;
    const int cvec = a.cp / 4;
    const long long p = e / cvec;
    const int c = (int)(e % cvec) * 4;
    float4 v = ld4(a.in + p * a.cp + c);
    for (int i = 0; i < a.n; ++i)
        if (c < a.add_cp[i]) {
            const float4 q = ld4(a.add[i] + p * a.add_cp[i] + c);
            v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
        }
    v.x = c < a.C ? act_fwd(v.x, a.act) : 0.f;
    v.y = c + 1 < a.C ? act_fwd(v.y, a.act) : 0.f;
    v.z = c + 2 < a.C ? act_fwd(v.z, a.act) : 0.f;
    v.w = c + 3 < a.C ? act_fwd(v.w, a.act) : 0.f;
    st4(a.out + p * a.cp + c, v);
}
// d = delta * act'(y) (written back), added to the previous delta and to every source's delta (overwriting where
// nothing has been written yet).  A source with more channels than this layer is zeroed by the host first.
__global__ void __launch_bounds__(TB) shortcut_bwd_kernel(const ShortcutArgs a) {
    pdl_enter();
    const long long e = (long long)blockIdx.x * TB + threadIdx.x;
    if (e >= a.total) return;
    const int cvec = a.cp / 4;
    const long long p = e / cvec;
    const int c = (int)(e % cvec) * 4;
    const size_t o = (size_t)p * a.cp + c;
    float4 d = ld4(a.out + o);
    const float4 y = ld4(a.y + o);
    d.x *= act_grad(y.x, a.act); d.y *= act_grad(y.y, a.act); d.z *= act_grad(y.z, a.act); d.w *= act_grad(y.w, a.act);
    if (c + 1 >= a.C) d.y = 0.f;
    if (c + 2 >= a.C) d.z = 0.f;
    if (c + 3 >= a.C) d.w = 0.f;
    if (a.act != AET_LINEAR) st4(a.out + o, d);
    if (a.pd) {
        float4 q = d;
        if (!a.pd_lazy) { const float4 t = ld4(a.pd + o); q.x += t.x; q.y += t.y; q.z += t.z; q.w += t.w; }
        st4(a.pd + o, q);
    }
    for (int i = 0; i < a.n; ++i)
        if (c < a.add_cp[i]) {
            float *dst = a.add[i] + (size_t)p * a.add_cp[i] + c;
            float4 q = d;
            if (!a.add_lazy[i]) { const float4 t = ld4(dst); q.x += t.x; q.y += t.y; q.z += t.z; q.w += t.w; }
            st4(dst, q);
        }
}

int k_shortcut_forward(aet_layer *l, const float *in) {
    aet_context *ctx = l->ctx;
    ShortcutArgs a = {};
    a.in = in; a.out = l->output->d; a.n = l->n_from; a.C = l->c; a.cp = l->cp; a.act = l->act;
    for (int i = 0; i < l->n_from; ++i) { a.add[i] = l->from[i]->output->d; a.add_cp[i] = l->from[i]->ocp; }
    a.total = (long long)l->batch * l->h * l->w * (l->cp / 4);
    LaunchScope s(ctx, "shortcut_fwd", 4.0 * (2 + l->n_from) * l->batch * l->h * l->w * l->cp, 0);
    launch_k(ctx->stream, (unsigned)((a.total + TB - 1) / TB), TB, 0, shortcut_fwd_kernel, a);
    return aet_check_launch("shortcut_fwd");
}

int k_shortcut_backward(aet_layer *l, aet_tensor *pd) {
    aet_context *ctx = l->ctx;
    ShortcutArgs a = {};
    a.out = l->delta->d; a.y = l->output->d; a.n = l->n_from; a.C = l->c; a.cp = l->cp; a.act = l->act;
    a.pd = pd ? pd->d : nullptr; a.pd_lazy = pd && pd->lazy_zero ? 1 : 0;
    for (int i = 0; i < l->n_from; ++i) {
        aet_tensor *fd = l->from[i]->delta;
        if (fd->lazy_zero && (l->from[i]->ocp > l->cp || fd == pd)) {
            // wider than this layer (its other channels must read as zero), or the very tensor `pd` names (it must
            // receive the delta twice, as the reference adds it twice): start from explicit zeros
            AET_TRY(aet_tensor_zero(fd));
            fd->lazy_zero = false;
            if (fd == pd) a.pd_lazy = 0;
        }
        a.add[i] = fd->d; a.add_cp[i] = l->from[i]->ocp; a.add_lazy[i] = fd->lazy_zero ? 1 : 0;
        fd->lazy_zero = false;
    }
    if (pd) pd->lazy_zero = false;
    a.total = (long long)l->batch * l->h * l->w * (l->cp / 4);
    LaunchScope s(ctx, "shortcut_bwd", 4.0 * (3 + 2 * l->n_from) * l->batch * l->h * l->w * l->cp, 0);
    launch_k(ctx->stream, (unsigned)((a.total + TB - 1) / TB), TB, 0, shortcut_bwd_kernel, a);
    return aet_check_launch("shortcut_bwd");
}

// Convolution without BN: delta *= act'(output) in place and the bias gradient accumulates.
int k_bias_act_backward(aet_layer *l) {
    aet_context *ctx = l->ctx;
    const long long pixels = (long long)l->batch * l->oh * l->ow;
    ReducePlan p = plan_reduce(ctx, pixels, l->ocp);
    float *partial = nullptr;
    AET_TRY(ctx_scratch(ctx, (size_t)p.blocks * 2 * l->ocp * sizeof(float), &partial));
    ReduceArgs a = {};
    a.x = l->output->d; a.delta = l->delta->d; a.partial = partial; a.act = l->act;
    a.pixels = pixels; a.cp = l->ocp; a.pix_per_block = p.pix_per_block; a.m = p.m;
    {
        LaunchScope s(ctx, "bias_act_bwd", (double)pixels * l->ocp * (l->act == AET_LINEAR ? 4.0 : 12.0), 0);
        launch_k(ctx->stream, dim3(p.blocks, p.m.cslabs), TB, 0, reduce2_kernel<2>, a);
        AET_TRY(aet_check_launch("bias_act_bwd"));
    }
    FinalizeArgs f = {};
    f.partial = partial; f.blocks = p.blocks; f.cp = l->ocp; f.c = l->oc; f.m = pixels; f.g_beta = layer_bG(l);
    LaunchScope s(ctx, "bias_bwd_finalize", 0, 0);
    launch_k(ctx->stream, (l->ocp + FIN_CH - 1) / FIN_CH, 1024, 0, finalize_kernel<2>, f);
    return aet_check_launch("bias_bwd_finalize");
}

int k_maxpool_forward(aet_layer *l, const float *x) {
    aet_context *ctx = l->ctx;
    PoolArgs a = {};
    a.x = x; a.y = l->output->d; a.idx = l->indexes;
    a.N = l->batch; a.C = l->c; a.H = l->h; a.W = l->w; a.cp = l->cp; a.OH = l->oh; a.OW = l->ow;
    a.size = l->size; a.sx = l->stride_x; a.sy = l->stride_y; a.off = -l->pad / 2; a.parity = ctx->parity;
    a.total = (long long)l->batch * l->oh * l->ow * (l->cp / 4);
    const double bytes = 4.0 * l->batch * l->h * l->w * l->cp + 8.0 * l->batch * l->oh * l->ow * l->cp;
    LaunchScope s(ctx, "maxpool_fwd", bytes, 0);
    launch_k(ctx->stream, (unsigned)((a.total + TB - 1) / TB), TB, 0, maxpool_fwd_kernel, a);
    return aet_check_launch("maxpool_fwd");
}

int k_maxpool_backward(aet_layer *l, float *prev_delta, int accumulate) {
    aet_context *ctx = l->ctx;
    PoolBwdArgs a = {};
    a.delta = l->delta->d; a.idx = l->indexes; a.prev = prev_delta;
    a.N = l->batch; a.C = l->c; a.H = l->h; a.W = l->w; a.cp = l->cp; a.OH = l->oh; a.OW = l->ow;
    a.size = l->size; a.sx = l->stride_x; a.sy = l->stride_y; a.off = -l->pad / 2; a.accumulate = accumulate;
    a.total = (long long)l->batch * l->h * l->w * (l->cp / 4);
    const double bytes = 8.0 * l->batch * l->oh * l->ow * l->cp + (accumulate ? 8.0 : 4.0) * l->batch * l->h * l->w * l->cp;
    LaunchScope s(ctx, "maxpool_bwd", bytes, 0);
    launch_k(ctx->stream, (unsigned)((a.total + TB - 1) / TB), TB, 0, maxpool_bwd_kernel, a);
    return aet_check_launch("maxpool_bwd");
}

int k_avgpool_forward(aet_layer *l, const float *x) {
    aet_context *ctx = l->ctx;
    const int total = l->batch * (l->cp / 4);
    LaunchScope s(ctx, "avgpool_fwd", 4.0 * l->batch * l->h * l->w * l->cp + 4.0 * l->batch * l->cp, 0);
    launch_k(ctx->stream, (total + 127) / 128, 128, 0, avgpool_fwd_kernel, x, l->output->d, l->batch, l->h * l->w, l->cp);
    return aet_check_launch("avgpool_fwd");
}

int k_avgpool_backward(aet_layer *l, float *prev_delta, int accumulate) {
    aet_context *ctx = l->ctx;
    const long long total4 = (long long)l->batch * l->h * l->w * (l->cp / 4);
    LaunchScope s(ctx, "avgpool_bwd", (accumulate ? 8.0 : 4.0) * l->batch * l->h * l->w * l->cp + 4.0 * l->batch * l->cp, 0);
    launch_k(ctx->stream, (unsigned)((total4 + TB - 1) / TB), TB, 0, avgpool_bwd_kernel, l->delta->d, prev_delta, total4,
                                                                                   l->h * l->w, l->cp, accumulate);
    return aet_check_launch("avgpool_bwd");
}

int k_softmax_forward(aet_layer *l, const float *x, const float *truth) {
    aet_context *ctx = l->ctx;
    SoftmaxArgs a = {};
    a.x = x; a.truth = truth; a.p = l->output->d; a.delta = l->delta->d; a.loss = l->loss; a.unit_loss = l->sample_loss;
    a.groups = l->groups; a.units = l->batch * l->groups; a.n = l->c / l->groups; a.cp = l->cp;
    a.parity = ctx->parity; a.temp = l->temperature;
    {
        LaunchScope s(ctx, "softmax_xent", 20.0 * l->batch * l->c, 0);
        launch_k(ctx->stream, (a.units + TB / 32 - 1) / (TB / 32), TB, 0, softmax_kernel, a);
        AET_TRY(aet_check_launch("softmax_xent"));
    }
    if (truth) {
        float *mean_loss = l->net ? l->cost_dev + 1 : nullptr;
        LaunchScope s(ctx, "softmax_cost", 0, 0);
        launch_k(ctx->stream, 1, 1024, 0, softmax_cost_kernel, l->sample_loss, a.units, l->cost_dev, 1.0f / l->batch, mean_loss);
        AET_TRY(aet_check_launch("softmax_cost"));
    }
    return AET_OK;
}

static HeadArgs make_head(aet_layer *conv, aet_layer *avg, aet_layer *sm, const float *truth) {
    HeadArgs h = {};
    h.y = conv->output->d; h.avg = avg->output->d; h.p = sm->output->d; h.sm_delta = sm->delta->d; h.loss = sm->loss;
    h.truth = truth; h.cost = sm->cost_dev; h.avg_delta = avg->delta->d; h.conv_delta = conv->delta ? conv->delta->d : nullptr;
    h.bias_grad = layer_bG(conv);
    h.N = sm->batch; h.spatial = avg->h * avg->w; h.classes = sm->c; h.cp = sm->cp; h.parity = sm->ctx->parity;
    h.temp = sm->temperature;
    h.loss_scale = (sm->ctx->parity == AET_PARITY_MTCS && sm->net) ? sm->net->loss_scale : 1.0f;
    return h;
}
int k_head_forward(aet_layer *conv, aet_layer *avg, aet_layer *sm, const float *truth) {
    aet_context *ctx = sm->ctx;
    HeadArgs h = make_head(conv, avg, sm, truth);
    LaunchScope s(ctx, "head_avgpool_softmax_xent", 4.0 * conv->batch * conv->oh * conv->ow * conv->ocp + 24.0 * sm->batch * sm->c, 0);
    launch_k(ctx->stream, 1, 1024, 0, head_forward_kernel, h);
    return aet_check_launch("head_avgpool_softmax_xent");
}
int k_head_backward(aet_layer *conv, aet_layer *avg, aet_layer *sm) {
    aet_context *ctx = sm->ctx;
    HeadArgs h = make_head(conv, avg, sm, nullptr);
    LaunchScope s(ctx, "head_backward", 4.0 * conv->batch * conv->oh * conv->ow * conv->ocp + 8.0 * sm->batch * sm->c, 0);
    launch_k(ctx->stream, 1, 1024, 0, head_backward_kernel, h);
    return aet_check_launch("head_backward");
}

static LinHeadArgs make_linhead(aet_layer *conv, aet_layer *avg, aet_layer *sm, const float *x, const float *truth, float *pd) {
    LinHeadArgs h = {};
    h.x = x; h.w = layer_W(conv); h.b = layer_b(conv); h.xbar = conv->lin_xbar;
    h.avg = avg->output->d; h.p = sm->output->d; h.sm_delta = sm->delta->d; h.loss = sm->loss; h.truth = truth;
    h.unit_loss = sm->sample_loss; h.cost = sm->cost_dev; h.ticket = conv->lin_ticket;
    h.avg_delta = avg->delta->d; h.pd = pd; h.gw = layer_G(conv); h.gb = layer_bG(conv);
    h.N = sm->batch; h.S = conv->oh * conv->ow; h.cp = conv->cp; h.classes = sm->c; h.ocp = sm->cp; h.parity = sm->ctx->parity;
    h.temp = sm->temperature;
    h.loss_scale = (sm->ctx->parity == AET_PARITY_MTCS && sm->net) ? sm->net->loss_scale : 1.0f;
    return h;
}
int k_linhead_forward(aet_layer *conv, aet_layer *avg, aet_layer *sm, const float *x, const float *truth) {
    aet_context *ctx = sm->ctx;
    LinHeadArgs h = make_linhead(conv, avg, sm, x, truth, nullptr);
    LaunchScope s(ctx, "linear_head_forward", 4.0 * h.N * h.S * h.cp + 4.0 * h.classes * h.cp, 2.0 * h.N * h.classes * h.cp);
    launch_k(ctx->stream, h.N, 256, (size_t)(h.cp + 32) * sizeof(float), linhead_forward_kernel, h);
    return aet_check_launch("linear_head_forward");
}
int k_linhead_backward(aet_layer *conv, aet_layer *avg, aet_layer *sm, float *pd) {
    aet_context *ctx = sm->ctx;
    LinHeadArgs h = make_linhead(conv, avg, sm, nullptr, nullptr, pd);
    LaunchScope s(ctx, "linear_head_backward", 4.0 * h.N * h.S * h.cp + 8.0 * h.classes * h.cp, 4.0 * h.N * h.classes * h.cp);
    launch_k(ctx->stream, h.N + (h.cp + 31) / 32, 256, (size_t)(h.N + 256) * h.classes * sizeof(float), linhead_backward_kernel, h);
    return aet_check_launch("linear_head_backward");
}
// The convolution delta the fused head never wrote: g / S broadcast over the pixels (no gradient side effects).
int k_linhead_conv_delta(aet_layer *conv, aet_layer *avg, aet_layer *sm) {
    aet_context *ctx = sm->ctx;
    HeadArgs h = make_head(conv, avg, sm, nullptr);
    h.bias_grad = nullptr;
    LaunchScope s(ctx, "head_backward", 4.0 * conv->batch * conv->oh * conv->ow * conv->ocp, 0);
    launch_k(ctx->stream, 1, 1024, 0, head_backward_kernel, h);
    return aet_check_launch("head_backward");
}

int k_axpy(aet_context *ctx, float *y, const float *x, float a, size_t n, int accumulate, const char *name) {
    const size_t n4 = n / 4;
    LaunchScope s(ctx, name, (accumulate ? 12.0 : 8.0) * n, 0);
    launch_k(ctx->stream, (unsigned)((n4 + TB - 1) / TB), TB, 0, axpy_kernel, y, x, a, n4, accumulate);
    return aet_check_launch(name);
}

int k_fill(aet_context *ctx, float *p, float v, size_t n) {
    const size_t n4 = n / 4;
    LaunchScope s(ctx, "fill", 4.0 * n, 0);
    launch_k(ctx->stream, (unsigned)((n4 + TB - 1) / TB), TB, 0, fill_kernel, p, v, n4);
    return aet_check_launch("fill");
}

int k_step_counter(aet_context *ctx, unsigned long long *ctr) {
    LaunchScope s(ctx, "step_counter", 0, 0);
    launch_k(ctx->stream, 1, 1, 0, step_counter_kernel, ctr);
    return aet_check_launch("step_counter");
}

int k_dropout_forward(aet_layer *l, float *x, int generate) {
    aet_context *ctx = l->ctx;
    const size_t n = (size_t)l->batch * l->h * l->w * l->cp;
    LaunchScope s(ctx, "dropout_fwd", 12.0 * n, 0);
    launch_k(ctx->stream, (unsigned)((n + TB - 1) / TB), TB, 0, dropout_fwd_kernel, x, l->rnd, n, l->c, l->cp, l->probability,
                                                                             1.f / (1.f - l->probability), l->seed,
                                                                             l->step_dev, generate);
    return aet_check_launch("dropout_fwd");
}

int k_dropout_backward(aet_layer *l, float *delta) {
    aet_context *ctx = l->ctx;
    const size_t n = (size_t)l->batch * l->h * l->w * l->cp;
    LaunchScope s(ctx, "dropout_bwd", 12.0 * n, 0);
    launch_k(ctx->stream, (unsigned)((n + TB - 1) / TB), TB, 0, dropout_bwd_kernel, delta, l->rnd, n, l->probability,
                                                                             1.f / (1.f - l->probability));
    return aet_check_launch("dropout_bwd");
}

int elementwise_set_wait_limit(unsigned long long ns) {
    AET_CUDA(cudaMemcpyToSymbol(g_flag_wait_limit_ns, &ns, sizeof(ns)));
    return AET_OK;
}

int k_sgd_segment(aet_context *ctx, float *W, float *U, float *G, size_t count, float lr_over_b, float momentum,
                  float decay_term, int scrub) {
    const size_t n4 = count / 4;
    LaunchScope s(ctx, "sgd_segment", 24.0 * count, 0);
    launch_k(ctx->stream, (unsigned)((n4 + TB - 1) / TB), TB, 0, sgd_segment_kernel, W, U, G, n4, lr_over_b, momentum, decay_term,
             scrub, ctx->status_dev);
    return aet_check_launch("sgd_segment");
}

__global__ void comm_stamp_kernel(unsigned long long *d, int after) {
    pdl_enter();
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (!after) d[0] = now;
    else { d[1] += now - d[0]; if (after == 1) d[2] += 1; }   // after == 2: a second bracket of the same step
}
int k_comm_stamp(aet_context *ctx, unsigned long long *dev4, int after) {
    LaunchScope s(ctx, "comm_stamp", 0, 0);
    launch_k(ctx->stream, 1, 1, 0, comm_stamp_kernel, dev4, after);
    return aet_check_launch("comm_stamp");
}

int k_sgd_arena(aet_network *net) {
    aet_context *ctx = net->ctx;
    LaunchScope s(ctx, "sgd_momentum", 24.0 * net->arena.used, 0);
    TailArgs t = {};
    if (net->xchg_active && net->tail_n) {
        for (int q = 0; q < net->world; ++q) t.peer_buf[q] = reinterpret_cast<const float *>(net->xchg_peer[q] + kXchgFlagBytes);
        t.flags = reinterpret_cast<const volatile unsigned long long *>(net->xchg_local);
        t.epoch = net->xchg_epoch; t.lo = net->tail_lo; t.n = net->tail_n; t.cap = net->xchg_cap;
        t.world = net->world; t.status = ctx->status_dev; t.gate = net->xchg_gate;
        // option "comm_stamps": the wait for the peers' slices counts as exposed communication like the wait for a collective
        const bool stamps = ctx->opt[OPT_COMM_STAMPS] != 0 && net->comm_stamp_dev;
        if (stamps) launch_k(ctx->stream, 1, 1, 0, comm_stamp_kernel, net->comm_stamp_dev, 0);
        launch_k(ctx->stream, 1, 32, 0, tail_wait_kernel, t);
        if (stamps) launch_k(ctx->stream, 1, 1, 0, comm_stamp_kernel, net->comm_stamp_dev, net->comm_stamped ? 2 : 1);
        AET_TRY(aet_check_launch("grad_wait"));
    }
    net->comm_stamped = false;
    launch_k(ctx->stream, net->n_blocks, TB, 0, sgd_arena_kernel, net->arena.W, net->arena.U, net->arena.G, net->block_seg,
                                                           net->seg_table, net->hyper_dev, t, ctx->status_dev);
    return aet_check_launch("sgd_momentum");
}

int k_adam_arena(aet_network *net) {
    aet_context *ctx = net->ctx;
    if (net->xchg_active && net->tail_n) { aet_set_error("Adam does not take its gradients through the peer exchange"); return AET_E_INVALID; }
    LaunchScope s(ctx, "adam", 40.0 * net->arena.used, 0);
    launch_k(ctx->stream, net->n_blocks, TB, 0, adam_arena_kernel, net->arena.W, net->arena.U, net->arena.G, net->arena.M, net->arena.V,
             net->block_seg, net->seg_table, net->hyper_dev, net->B1, net->B2, net->eps, ctx->status_dev);
    return aet_check_launch("adam");
}

int k_tail_publish(aet_network *net) {
    aet_context *ctx = net->ctx;
    TailArgs t = {};
    t.lo = net->tail_lo; t.n = net->tail_n; t.cap = net->xchg_cap; t.world = net->world;
    PublishArgs p = {};
    for (int q = 0; q < net->world && q < 8; ++q) p.peer_flags[q] = reinterpret_cast<unsigned long long *>(net->xchg_peer[q]);
    p.buf_local = reinterpret_cast<float *>(net->xchg_local + kXchgFlagBytes);
    p.epoch = net->xchg_epoch; p.ticket = net->xchg_ticket; p.rank = net->rank;
    int blocks = (int)((net->tail_n + 4095) / 4096);
    if (blocks > ctx->sm_count) blocks = ctx->sm_count;
    LaunchScope s(ctx, "grad_publish", 8.0 * net->tail_n, 0);
    launch_k(ctx->stream, blocks, 1024, 0, tail_publish_kernel, net->arena.G, t, p);
    return aet_check_launch("grad_publish");
}

int k_augment(aet_context *ctx, const float *src_nchw, int n, int c, int sh, int sw, float *dst_nhwc, int size, int cp,
              const aet_augment *params_dev) {
    const size_t px = (size_t)n * size * size;
    LaunchScope s(ctx, "augment", 4.0 * n * c * sh * sw + 4.0 * px * cp, 0);
    launch_k(ctx->stream, (unsigned)((px + TB - 1) / TB), TB, 0, augment_kernel, src_nchw, n, c, sh, sw, dst_nhwc, size, cp, params_dev);
    return aet_check_launch("augment");
}

int k_top_k(aet_context *ctx, const float *scores, int samples, int n, int ld, int k, int *index_dev) {
    LaunchScope s(ctx, "top_k", 4.0 * samples * n, 0);
    launch_k(ctx->stream, (unsigned)((samples + 63) / 64), 64, 0, top_k_kernel, scores, samples, n, ld, k, index_dev);
    return aet_check_launch("top_k");
}

int k_param_hash(aet_context *ctx, const float *p, size_t count, uint64_t *hash_dev) {
    LaunchScope s(ctx, "param_hash", 4.0 * count, 0);
    launch_k(ctx->stream, (unsigned)((count + TB - 1) / TB), TB, 0, param_hash_kernel, p, count,
                                                                                reinterpret_cast<unsigned long long *>(hash_dev));
    return aet_check_launch("param_hash");
}

// ---------------------------------------------------------------------------- allocation-free bias gradient
// Some hosts of this library may not allocate device memory once they are running: a training loop
// inside a process whose whole device pool was sized and handed out at start-up, or a service that has
// entered a phase in which cudaMalloc (a device-wide synchronisation) is off limits.  For them the bias
// gradient (the column sums that k_bias_act_backward forms with partials in the context's cudaMalloc'ed
// scratch arena) is also offered with its partials in the fixed array below, which every GPU that loads
// the library holds until exit.
constexpr size_t kStaticScratchFloats = 1u << 18;   // 1 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

namespace {
struct StaticDeviceState {
    std::atomic<bool> ready{false};   // published with release order after `scratch` and `sm_count` are written
    float *scratch = nullptr;         // device address of g_static_scratch on this device
    int sm_count = 0;
};
StaticDeviceState g_static_state[64];
std::mutex g_static_mutex;            // serialises the first call on a device between host threads
}  // namespace

extern "C" int aet_backward_bias_static(const float *delta, float *bias_updates, long long pixels, int channels,
                                        void *cuda_stream) {
    if (!delta || !bias_updates || pixels <= 0 || channels <= 0) {
        aet_set_error("aet_backward_bias_static: null pointer or empty shape");
        return AET_E_INVALID;
    }
    if (channels % 4 != 0 || (reinterpret_cast<uintptr_t>(delta) & 15u) != 0) {
        aet_set_error("aet_backward_bias_static: channels must be a multiple of 4 and delta 16-byte aligned");
        return AET_E_INVALID;
    }
    int dev = -1;
    AET_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        aet_set_error("aet_backward_bias_static: device ordinal %d is outside the supported range", dev);
        return AET_E_INVALID;
    }
    StaticDeviceState &st = g_static_state[dev];
    if (!st.ready.load(std::memory_order_acquire)) {
        // Host code only sees a stand-in for the __device__ array; the kernels need its device address,
        // looked up once per device with that device current.  (With lazy module loading this lookup is
        // also what makes the driver back the array with memory: do it at start-up.)
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!st.ready.load(std::memory_order_relaxed)) {
            float *p = nullptr;
            AET_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_scratch));
            AET_CUDA(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
            st.scratch = p;
            st.ready.store(true, std::memory_order_release);
        }
    }
    ReducePlan p;
    p.m = make_cmap(channels);
    long long want = 2LL * st.sm_count / p.m.cslabs;
    if (want < 1) want = 1;
    const long long min_pix = (long long)p.m.pl_count * 4;
    const long long maxb = (pixels + min_pix - 1) / min_pix;
    if (want > maxb) want = maxb;
    if (want < 1) want = 1;
    p.pix_per_block = (pixels + want - 1) / want;
    p.blocks = (int)((pixels + p.pix_per_block - 1) / p.pix_per_block);
    const size_t need = (size_t)p.blocks * 2 * (size_t)channels;
    if (need > kStaticScratchFloats) {
        aet_set_error("aet_backward_bias_static: %d channels need %zu scratch floats, the static array holds %zu "
                      "(use the layer entry points, which allocate)", channels, need, kStaticScratchFloats);
        return AET_E_INVALID;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    ReduceArgs a = {};
    a.x = delta;                                   // the kernel also loads its 'output' operand; linear ignores the value
    a.delta = const_cast<float *>(delta);          // linear activation: the kernel does not write delta
    a.partial = st.scratch; a.act = AET_LINEAR;
    a.pixels = pixels; a.cp = channels; a.pix_per_block = p.pix_per_block; a.m = p.m;
    launch_k(stream, dim3(p.blocks, p.m.cslabs), TB, 0, reduce2_kernel<2>, a);
    AET_TRY(aet_check_launch("backward_bias_static (partials)"));
    FinalizeArgs f = {};
    f.partial = st.scratch; f.blocks = p.blocks; f.cp = channels; f.c = channels; f.m = pixels; f.g_beta = bias_updates;
    launch_k(stream, (channels + FIN_CH - 1) / FIN_CH, 1024, 0, finalize_kernel<2>, f);
    return aet_check_launch("backward_bias_static (finalize)");
}
