// Backward pass of an image network's first convolution (3x3, stride 1, pad 1, at most 3 input channels) with batch
// norm whose 2x2 / stride-2 max-pool is fused into it, when nothing upstream needs a data gradient.  Included by
// elementwise.cu.
//
// The general path forms the full-resolution delta  dx = ka*q + kb*(y - mean) + kc  (q: the pool's delta routed to the
// argmax input, times the activation gradient; y: the convolution result; ka/kb/kc per output channel) and then runs
// the weight-gradient GEMM over it: three passes over tensors four times the size of the pool's.  Only the weight
// gradient is wanted here, and with patch(p, t) the input value under tap t of output pixel p
//     dW[k][t] = sum_p dx[p][k] * patch(p, t)
//              = ka[k] * sum_p q[p][k] * patch(p, t)                         (q is non-zero at one input per window)
//              + kb[k] * sum_t' W[k][t'] * sum_p (patch(p, t') - pbar[t']) * patch(p, t)     (y - mean = W . (patch - pbar))
//              + kc[k] * sum_p patch(p, t)
// so the first term is a pass over the pool-sized tensors, and the other two need only the 36 x 36 Gram matrix of the
// input patches and their column sums, which depend on the input batch alone and are formed beside the rest of the
// step.  The sums feeding ka/kb/kc and the scale / shift gradients come out of the same pool-sized pass, which reads the
// convolution result at each window's argmax from a pool-sized tensor the fused forward kernel stores.
#pragma once

namespace {

constexpr int STEM_TAPS = 36;          // 3 x 3 taps x 4 (padded) input channels, in the weights' [r][s][c] order
constexpr int STEM_GRAM_ROWS = 8;      // output rows per strip of the Gram kernel = row lanes per block
constexpr int STEM_GRAM_COMBOS = 27;   // (row of tap a, row of tap b, column of tap b): a thread keeps all columns of tap a
constexpr int STEM_GRAM_ENTRY = 28;    // 27 products per combo (+ 1 pad), in the order (column of tap a, channel a, channel b)
constexpr int STEM_GRAM_PART = STEM_GRAM_COMBOS * STEM_GRAM_ENTRY + 28;   // + column sums [(rb, sb)][channel] (27, + 1 pad)
constexpr int STEM_WIN = 16;           // pool windows per work item of the sparse pass
constexpr int STEM_COLS = 2 * STEM_WIN + 2;   // input columns under them, with the border
constexpr int STEM_FIN_LANES = 28;     // threads per tap in the finishing kernel (36 x 28 = 1008 threads)

struct StemSparseArgs {
    const float *x;               // layer input [N][H][W][4]
    const float *pdelta;          // pool delta  [N][OH][OW][ocp]
    const unsigned char *code;    // position of the argmax inside its window (0..3, row-major; 4: none) [N][OH][OW][ocp]
    const float *ymax;            // convolution result at the argmax [N][OH][OW][ocp]
    const float *mean, *inv, *gamma, *beta;
    float *partial_s;             // [blocks][2][ocp]
    float *partial_t;             // [blocks][ocp][36]
    int act, ocp, N, H, W, OH, OW, chunks, items;   // chunks = ceil(OW / 16), items = N * OH * chunks
    unsigned div_chunks_mul, div_chunks_shr, div_oh_mul, div_oh_shr;   // multiply-high division by `chunks` and by OH
    unsigned long long *span;     // profiling: first CTA entry / last CTA exit (null: off)
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool valid) {
    const unsigned bytes = valid ? 16u : 0u;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ unsigned mulhi_div(unsigned n, unsigned mul, unsigned shr) { return mul ? __umulhi(n, mul) >> shr : n; }

// One block = 4 * ocp threads; thread (g, k) owns output channel k and every fourth pool window (g, g+4, ...) of a work
// item, which is 16 consecutive windows of one pool row.  For each of its windows it forms q = pool delta * activation
// gradient, adds q and q * (y - mean) to the BN sums of its channel, and adds q times the nine input pixels (all channels
// at once, 16-byte loads) around the argmax pixel to its 27 accumulators.  The items' inputs arrive by cp.async two
// items ahead into three rotating shared-memory buffers, so one barrier per item is enough: the buffer refilled in
// iteration i was last read in iteration i - 1.
template <int THREADS, int MINB, int UNROLL>
__global__ void __launch_bounds__(THREADS, MINB) stem_bwd_sparse_kernel(const StemSparseArgs a) {
    extern __shared__ float4 stem_smem[];
    span_begin(a.span);
    pdl_enter();
    constexpr int ocp = THREADS / 4;
    // per buffer: dv[16][ocp] floats, ym[16][ocp] floats, px[4][34] float4, code[16][ocp] bytes
    const int buf_bytes = STEM_WIN * ocp * 9 + 4 * STEM_COLS * 16;
    unsigned char *smem = reinterpret_cast<unsigned char *>(stem_smem);
    const int k = threadIdx.x % ocp, g = threadIdx.x / ocp;
    const float mean = a.mean[k], inv = a.inv[k], gam = a.gamma[k], bet = a.beta[k];
    float acc[27];
#pragma unroll
    for (int i = 0; i < 27; ++i) acc[i] = 0.f;
    float s1 = 0.f, s2 = 0.f;

    auto fetch = [&](int item, int slot) {
        if (item < a.items) {
            unsigned char *buf = smem + (size_t)slot * buf_bytes;
            const unsigned row = mulhi_div((unsigned)item, a.div_chunks_mul, a.div_chunks_shr);
            const int chunk = item - (int)row * a.chunks;
            const unsigned n = mulhi_div(row, a.div_oh_mul, a.div_oh_shr);
            const int oh = (int)row - (int)n * a.OH;
            const int ow0 = chunk * STEM_WIN;
            const size_t base = ((size_t)row * a.OW + ow0) * ocp;
            const int e = threadIdx.x;                     // 16-byte piece e of the item's pool delta / result slab
            const bool ok = ow0 + e * 4 / ocp < a.OW;
            cp_async16(buf + e * 16, a.pdelta + (ok ? base + (size_t)e * 4 : 0), ok);
            cp_async16(buf + STEM_WIN * ocp * 4 + e * 16, a.ymax + (ok ? base + (size_t)e * 4 : 0), ok);
            if (e < 4 * STEM_COLS) {
                const int rr = e / STEM_COLS, cc = e - rr * STEM_COLS;
                const int ih = 2 * oh - 1 + rr, iw = 2 * ow0 - 1 + cc;
                const bool in = ih >= 0 && ih < a.H && iw >= 0 && iw < a.W;
                cp_async16(buf + STEM_WIN * ocp * 8 + e * 16, a.x + (in ? ((size_t)((int)n * a.H + ih) * a.W + iw) * 4 : 0), in);
            }
            if (e < ocp) {   // ocp pieces of 16 codes
                const bool okc = ow0 + e * 16 / ocp < a.OW;
                cp_async16(buf + STEM_WIN * ocp * 8 + 4 * STEM_COLS * 16 + e * 16, a.code + (okc ? base + (size_t)e * 16 : 0), okc);
            }
        }
        cp_async_commit();   // an empty group past the last item keeps the wait counts uniform
    };

    fetch(blockIdx.x, 0);
    fetch(blockIdx.x + gridDim.x, 1);
    int slot = 0;
    for (int item = blockIdx.x; item < a.items; item += gridDim.x) {
        cp_async_wait<1>();   // this item's group has landed (the next item's may still be in flight)
        __syncthreads();      // ... for every thread; and every thread is done with the previous item's buffer
        fetch(item + 2 * gridDim.x, slot == 0 ? 2 : slot - 1);
        const unsigned char *buf = smem + (size_t)slot * buf_bytes;
        const float *dvs = reinterpret_cast<const float *>(buf), *yms = dvs + STEM_WIN * ocp;
        const float4 *nb = reinterpret_cast<const float4 *>(buf + STEM_WIN * ocp * 8);
        const unsigned char *cds = buf + STEM_WIN * ocp * 8 + 4 * STEM_COLS * 16;
        const int chunk = item - (int)mulhi_div((unsigned)item, a.div_chunks_mul, a.div_chunks_shr) * a.chunks;
        const int wlim = a.OW - chunk * STEM_WIN;   // windows of this item inside the row
#pragma unroll UNROLL
        for (int u = 0; u < STEM_WIN / 4; ++u) {
            const int w = g + 4 * u;
            const int cd = cds[w * ocp + k];
            const float ym = yms[w * ocp + k], dv = dvs[w * ocp + k];
            const float xm = __fsub_rn(ym, mean);
            const float q = (cd < 4 && w < wlim) ? dv * act_gradient_pre(__fadd_rn(__fmul_rn(__fmul_rn(xm, inv), gam), bet), a.act) : 0.f;
            s1 += q;
            s2 = fmaf(q, xm, s2);
            // the argmax pixel's receptive-field corner in nb: row cd>>1, column 2*window + (cd&1)
            const float4 *base = nb + ((cd >> 1) & 1) * STEM_COLS + 2 * w + (cd & 1);
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int sx = 0; sx < 3; ++sx) {
                    const float4 v = base[r * STEM_COLS + sx];
                    acc[(r * 3 + sx) * 3 + 0] = fmaf(q, v.x, acc[(r * 3 + sx) * 3 + 0]);
                    acc[(r * 3 + sx) * 3 + 1] = fmaf(q, v.y, acc[(r * 3 + sx) * 3 + 1]);
                    acc[(r * 3 + sx) * 3 + 2] = fmaf(q, v.z, acc[(r * 3 + sx) * 3 + 2]);
                }
        }
        slot = slot == 2 ? 0 : slot + 1;
    }
    cp_async_wait<0>();
    __syncthreads();
    // sum the four window groups' accumulators through shared memory (the landing buffers are free now)
    float *redf = reinterpret_cast<float *>(stem_smem);
#pragma unroll
    for (int i = 0; i < 27; ++i) redf[i * THREADS + threadIdx.x] = acc[i];
    redf[27 * THREADS + threadIdx.x] = s1;
    redf[28 * THREADS + threadIdx.x] = s2;
    __syncthreads();
    if (g == 0) {
        float4 *pt = reinterpret_cast<float4 *>(a.partial_t + ((size_t)blockIdx.x * ocp + k) * STEM_TAPS);
#pragma unroll
        for (int tp = 0; tp < 9; ++tp) {
            float v[3];
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) {
                const float *src = redf + (tp * 3 + ch) * THREADS + k;
                v[ch] = (src[0] + src[ocp]) + (src[2 * ocp] + src[3 * ocp]);
            }
            pt[tp] = make_float4(v[0], v[1], v[2], 0.f);
        }
    } else if (g == 1) {
        const float *p1 = redf + 27 * THREADS + k, *p2 = redf + 28 * THREADS + k;
        float *ps = a.partial_s + (size_t)blockIdx.x * 2 * ocp + k;
        ps[0] = (p1[0] + p1[ocp]) + (p1[2 * ocp] + p1[3 * ocp]);
        ps[ocp] = (p2[0] + p2[ocp]) + (p2[2 * ocp] + p2[3 * ocp]);
    }
    span_end(a.span);
}

struct StemGramArgs {
    const float *x;     // [N][H][W][4]
    float *partial;     // [blocks][STEM_GRAM_PART]
    int N, H, W, strips_per_image, strips;
    unsigned long long *span;
};

// Gram matrix of the input patches, G[(ra,sa,ca)][(rb,sb,cb)] = sum over output pixels p of the input under tap (ra,sa),
// channel ca, times the input under tap (rb,sb), channel cb (zero outside the image), and the patches' column sums
// S[(rb,sb,cb)].  A block owns strips of 8 output rows; thread (row, combo) walks along one row and keeps, for its
// combo = (ra, rb, sb), the products of all three columns sa of tap a (a sliding window of three pixels) with the pixel
// under tap b: 27 accumulators for two 16-byte shared-memory loads per pixel.
__global__ void __launch_bounds__(STEM_GRAM_COMBOS * STEM_GRAM_ROWS) stem_gram_kernel(const StemGramArgs a) {
    extern __shared__ float4 stem_img[];   // [STEM_GRAM_ROWS + 2][W + 2], then the reduction buffer
    span_begin(a.span);
    pdl_enter();
    const int combo = threadIdx.x % STEM_GRAM_COMBOS, y = threadIdx.x / STEM_GRAM_COMBOS;
    const int ra = combo / 9, rb = (combo / 3) % 3, sb = combo % 3;
    const int wp = a.W + 2;
    float g[27], cs[3] = {0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 27; ++i) g[i] = 0.f;
    for (int strip = blockIdx.x; strip < a.strips; strip += gridDim.x) {
        const int n = strip / a.strips_per_image, r0 = (strip % a.strips_per_image) * STEM_GRAM_ROWS;
        __syncthreads();
        for (int i = threadIdx.x; i < (STEM_GRAM_ROWS + 2) * wp; i += blockDim.x) {
            const int rr = i / wp, cc = i % wp;
            const int ih = r0 - 1 + rr, iw = cc - 1;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ih >= 0 && ih < a.H && iw >= 0 && iw < a.W) v = ld4(a.x + ((size_t)(n * a.H + ih) * a.W + iw) * 4);
            stem_img[i] = v;
        }
        __syncthreads();
        if (r0 + y < a.H) {
            const float4 *pa = stem_img + (y + ra) * wp, *pb = stem_img + (y + rb) * wp + sb;
            float4 a0 = pa[0], a1 = pa[1];
#pragma unroll 2
            for (int xw = 0; xw < a.W; ++xw) {
                const float4 a2 = pa[xw + 2], vb = pb[xw];
                g[0] = fmaf(a0.x, vb.x, g[0]); g[1] = fmaf(a0.x, vb.y, g[1]); g[2] = fmaf(a0.x, vb.z, g[2]);
                g[3] = fmaf(a0.y, vb.x, g[3]); g[4] = fmaf(a0.y, vb.y, g[4]); g[5] = fmaf(a0.y, vb.z, g[5]);
                g[6] = fmaf(a0.z, vb.x, g[6]); g[7] = fmaf(a0.z, vb.y, g[7]); g[8] = fmaf(a0.z, vb.z, g[8]);
                g[9] = fmaf(a1.x, vb.x, g[9]); g[10] = fmaf(a1.x, vb.y, g[10]); g[11] = fmaf(a1.x, vb.z, g[11]);
                g[12] = fmaf(a1.y, vb.x, g[12]); g[13] = fmaf(a1.y, vb.y, g[13]); g[14] = fmaf(a1.y, vb.z, g[14]);
                g[15] = fmaf(a1.z, vb.x, g[15]); g[16] = fmaf(a1.z, vb.y, g[16]); g[17] = fmaf(a1.z, vb.z, g[17]);
                g[18] = fmaf(a2.x, vb.x, g[18]); g[19] = fmaf(a2.x, vb.y, g[19]); g[20] = fmaf(a2.x, vb.z, g[20]);
                g[21] = fmaf(a2.y, vb.x, g[21]); g[22] = fmaf(a2.y, vb.y, g[22]); g[23] = fmaf(a2.y, vb.z, g[23]);
                g[24] = fmaf(a2.z, vb.x, g[24]); g[25] = fmaf(a2.z, vb.y, g[25]); g[26] = fmaf(a2.z, vb.z, g[26]);
                if (ra == 0) { cs[0] += vb.x; cs[1] += vb.y; cs[2] += vb.z; }   // each (rb, sb) once: the combos with ra = 0
                a0 = a1; a1 = a2;
            }
        }
    }
    // sum over the 8 row lanes through shared memory, then one partial per block
    __syncthreads();
    float *red = reinterpret_cast<float *>(stem_img);   // [8][27][31]
    float *mine = red + (y * STEM_GRAM_COMBOS + combo) * 31;
#pragma unroll
    for (int i = 0; i < 27; ++i) mine[i] = g[i];
    mine[27] = cs[0]; mine[28] = cs[1]; mine[29] = cs[2];
    __syncthreads();
    float *dst = a.partial + (size_t)blockIdx.x * STEM_GRAM_PART;
    for (int i = threadIdx.x; i < STEM_GRAM_COMBOS * 30; i += blockDim.x) {
        const int cb = i / 30, j = i % 30;
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < STEM_GRAM_ROWS; ++q) v += red[(q * STEM_GRAM_COMBOS + cb) * 31 + j];
        if (j < 27) dst[cb * STEM_GRAM_ENTRY + j] = v;
        else if (cb < 9) dst[STEM_GRAM_COMBOS * STEM_GRAM_ENTRY + cb * 3 + (j - 27)] = v;   // ra = 0: cb = rb * 3 + sb
    }
    span_end(a.span);
}

// Sums the Gram partials of all blocks, in double and in a fixed order: 32 threads per entry, four independent loads
// in flight per thread.
__global__ void __launch_bounds__(1024) stem_gram_finish_kernel(const float *partial, int blocks, double *gram) {
    pdl_enter();
    __shared__ double part[32][33];
    const int i = threadIdx.x & 31, lane = threadIdx.x >> 5;
    const int e = blockIdx.x * 32 + i;
    double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
    if (e < STEM_GRAM_PART) {
        const float *src = partial + e;
        int b = lane;
        for (; b + 96 < blocks; b += 128) {
            const float v0 = __ldg(src + (size_t)b * STEM_GRAM_PART), v1 = __ldg(src + (size_t)(b + 32) * STEM_GRAM_PART);
            const float v2 = __ldg(src + (size_t)(b + 64) * STEM_GRAM_PART), v3 = __ldg(src + (size_t)(b + 96) * STEM_GRAM_PART);
            s0 += (double)v0; s1 += (double)v1; s2 += (double)v2; s3 += (double)v3;
        }
        for (; b < blocks; b += 32) s0 += (double)__ldg(src + (size_t)b * STEM_GRAM_PART);
    }
    part[lane][i] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (lane == 0 && e < STEM_GRAM_PART) {
        double t[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
        for (int q = 0; q < 32; ++q) t[q & 3] += part[q][i];
        gram[e] = (t[0] + t[1]) + (t[2] + t[3]);
    }
}

struct StemFinishArgs {
    const float *partial_t;   // [blocks][ocp][36]
    const float *partial_s;   // [blocks][2][ocp]
    const float *w;           // [oc][36] weights
    const double *gram;       // [STEM_GRAM_PART] raw Gram sums and column sums
    const float *variance, *inv, *gamma;
    float *g_gamma, *g_beta, *coef;   // scale / shift gradients (accumulated), coef [3][ocp] (kept for a later delta tap)
    float *dw;                // [oc][36]
    double pixels;
    int blocks, ocp, accumulate, parity;
};

// BN backward coefficients and the scale / shift gradients of one channel from the sums S1 = sum q, S2 = sum q (y - mean).
__device__ __forceinline__ void bn_bwd_channel(double s1, double s2, double m, int parity, float var, float gam, float inv,
                                               float *g_gamma, float *g_beta, float &ka, float &kb, float &kc) {
    const float S1 = (float)s1, S2 = (float)s2;
    *g_gamma += S2 * inv;
    float md, vd, k1;
    // v^(-3/2) is formed as 1 / (v * sqrt(v)) in double: it agrees with pow() to the last few bits of
    // the double, far below the float the product is rounded to, and costs a fraction of pow()
    if (parity == AET_PARITY_CPU) {
        const double v = (double)(var + .00001f), rs = sqrt(v);
        md = (float)((double)(gam * S1) * (-1. / rs));
        vd = (float)((double)(gam * S2) * (-.5 / (v * rs)));
        k1 = (float)(1. / rs);
    } else {
        *g_beta += S1;
        const float v = var + .000001f;
        md = (gam * S1) * (-1.f / sqrtf(v));
        vd = (float)((double)(gam * S2) * (-.5 * (double)(1.f / (v * sqrtf(v)))));
        k1 = 1.f / (sqrtf(var) + .000001f);
    }
    ka = gam * k1;
    kb = (float)((double)vd * 2. / m);
    kc = (float)((double)md / m);
}

// One block per output channel k: the channel's BN sums -> coefficients and scale / shift gradients, then
// dW[k][t] = ka * T1[k][t] + kb * sum_u W[k][u] (G[u][t] - S[u] S[t] / pixels) + kc * S[t].
__global__ void __launch_bounds__(STEM_TAPS * STEM_FIN_LANES) stem_bwd_finish_kernel(const StemFinishArgs a) {
    pdl_enter();
    __shared__ double gram[STEM_GRAM_PART];
    __shared__ double part[STEM_FIN_LANES][STEM_TAPS];
    __shared__ float wk[STEM_TAPS];
    __shared__ double ssum[2][2];
    __shared__ float kcoef[3];
    const int k = blockIdx.x, t = threadIdx.x % STEM_TAPS, lane = threadIdx.x / STEM_TAPS;
    const int warp = threadIdx.x >> 5, wl = threadIdx.x & 31;
    for (int i = threadIdx.x; i < STEM_GRAM_PART; i += blockDim.x) gram[i] = a.gram[i];
    if (lane == 0) wk[t] = a.w[(size_t)k * STEM_TAPS + t];
    {
        const float *src = a.partial_t + (size_t)k * STEM_TAPS + t;
        const size_t stride = (size_t)a.ocp * STEM_TAPS;
        double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;
        int b = lane;
        for (; b + 3 * STEM_FIN_LANES < a.blocks; b += 4 * STEM_FIN_LANES) {
            const float v0 = __ldg(src + b * stride), v1 = __ldg(src + (b + STEM_FIN_LANES) * stride);
            const float v2 = __ldg(src + (b + 2 * STEM_FIN_LANES) * stride), v3 = __ldg(src + (b + 3 * STEM_FIN_LANES) * stride);
            s0 += (double)v0; s1 += (double)v1; s2 += (double)v2; s3 += (double)v3;
        }
        for (; b < a.blocks; b += STEM_FIN_LANES) s0 += (double)__ldg(src + b * stride);
        part[lane][t] = (s0 + s1) + (s2 + s3);
    }
    if (warp < 4) {   // the first four warps also form S1 and S2, two warps each
        const int which = warp >> 1, half = warp & 1;
        const float *src = a.partial_s + which * a.ocp + k;
        double v0 = 0.0, v1 = 0.0;
        int b = half * 32 + wl;
        for (; b + 64 < a.blocks; b += 128) {
            const float x0 = __ldg(src + (size_t)b * 2 * a.ocp), x1 = __ldg(src + (size_t)(b + 64) * 2 * a.ocp);
            v0 += (double)x0; v1 += (double)x1;
        }
        for (; b < a.blocks; b += 64) v0 += (double)__ldg(src + (size_t)b * 2 * a.ocp);
        double v = v0 + v1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (wl == 0) ssum[which][half] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float ka, kb, kc;
        bn_bwd_channel(ssum[0][0] + ssum[0][1], ssum[1][0] + ssum[1][1], a.pixels, a.parity, a.variance[k], a.gamma[k], a.inv[k],
                       a.g_gamma + k, a.g_beta + k, ka, kb, kc);
        kcoef[0] = ka; kcoef[1] = kb; kcoef[2] = kc;
        a.coef[k] = ka; a.coef[a.ocp + k] = kb; a.coef[2 * a.ocp + k] = kc;
    }
    __syncthreads();
    if (lane != 0) return;
    double t1 = 0.0;
#pragma unroll
    for (int q = 0; q < STEM_FIN_LANES; ++q) t1 += part[q][t];
    const double *colsum = gram + STEM_GRAM_COMBOS * STEM_GRAM_ENTRY;   // [(r, s)][3]
    const int rb = t / 12, sb = (t >> 2) % 3, cb = t & 3;
    double wg = 0.0, ws = 0.0;
    if (cb < 3) {
        for (int u = 0; u < STEM_TAPS; ++u) {
            if ((u & 3) == 3) continue;
            const int ra = u / 12, sa = (u >> 2) % 3, ca = u & 3;
            const double wu = (double)wk[u];
            wg += wu * gram[((ra * 3 + rb) * 3 + sb) * STEM_GRAM_ENTRY + (sa * 3 + ca) * 3 + cb];
            ws += wu * colsum[(u >> 2) * 3 + ca];
        }
    }
    const double st = cb < 3 ? colsum[(t >> 2) * 3 + cb] : 0.0;
    const double t2 = wg - ws * st / a.pixels;
    float v = cb == 3 ? 0.f : (float)((double)kcoef[0] * t1 + (double)kcoef[1] * t2 + (double)kcoef[2] * st);
    float *dst = a.dw + (size_t)k * STEM_TAPS + t;
    if (a.accumulate) v += *dst;
    *dst = v;
}

}  // namespace

static void stem_fastdiv(unsigned d, unsigned &mul, unsigned &shr) {
    mul = 0; shr = 0;   // d == 1: identity
    if (d > 1) {
        unsigned lg = 0;
        while ((1ull << lg) < d) ++lg;
        const unsigned p = 31 + lg;
        mul = (unsigned)(((1ull << p) + d - 1) / d);   // round-up method: exact for dividends below 2^31
        shr = p - 32;
    }
}

bool stem_backward_eligible(const aet_layer *l, const aet_layer *pool) {
    return l->type == AET_CONVOLUTIONAL && l->bn && pool && pool->indexes && l->size == 3 && l->stride_x == 1 && l->stride_y == 1 &&
           l->pad == 1 && l->dilation == 1 && l->groups == 1 && l->c <= 3 && l->cp == 4 && (l->ocp == 64 || l->ocp == 128) &&
           pool->size == 2 && pool->stride_x == 2 && pool->stride_y == 2 && pool->pad / 2 == 0 && pool->h % 2 == 0 && pool->w % 2 == 0 &&
           l->w <= 190 && l->delta && l->ctx->opt[OPT_STEM];
}

// Gram matrix and column sums of the input batch (launched on the side stream when the pass overlaps).
int k_stem_gram(aet_layer *l, const float *x_in) {
    aet_context *ctx = l->ctx;
    StemGramArgs g = {};
    g.x = x_in; g.N = l->batch; g.H = l->h; g.W = l->w;
    g.strips_per_image = (l->h + STEM_GRAM_ROWS - 1) / STEM_GRAM_ROWS;
    g.strips = g.strips_per_image * l->batch;
    const int blocks = g.strips < l->stem_gram_blocks ? g.strips : l->stem_gram_blocks;
    g.partial = l->stem_gram_partial;
    size_t smem = (size_t)(STEM_GRAM_ROWS + 2) * (l->w + 2) * sizeof(float4);
    const size_t red = (size_t)STEM_GRAM_ROWS * STEM_GRAM_COMBOS * 31 * sizeof(float);
    if (smem < red) smem = red;
    {
        LaunchScope s(ctx, "stem_gram", 16.0 * l->batch * l->h * l->w, 2.0 * l->batch * l->h * l->w * 27.0 * 27.0);
        g.span = ctx->span_ptr;
        launch_k(ctx->stream, blocks, STEM_GRAM_COMBOS * STEM_GRAM_ROWS, smem, stem_gram_kernel, g);
        AET_TRY(aet_check_launch("stem_gram"));
    }
    LaunchScope s(ctx, "stem_gram_finish", 0, 0);
    launch_k(ctx->stream, (STEM_GRAM_PART + 31) / 32, 1024, 0, stem_gram_finish_kernel, (const float *)l->stem_gram_partial, blocks, l->stem_gram);
    return aet_check_launch("stem_gram_finish");
}

static size_t stem_sparse_smem(const aet_layer *l) {
    const size_t threads = 4 * (size_t)l->ocp;
    const size_t landing = 3 * ((size_t)STEM_WIN * l->ocp * 9 + 4 * STEM_COLS * 16);
    const size_t reduce = 29 * threads * sizeof(float);   // the final sums reuse the region from its start
    return landing > reduce ? landing : reduce;
}

// The pool-sized pass: per-block BN sums and first-term sums.
int k_stem_backward(aet_layer *l, aet_layer *pool, const float *x_in) {
    aet_context *ctx = l->ctx;
    const int threads = 4 * l->ocp;
    const size_t smem = stem_sparse_smem(l);
    StemSparseArgs a = {};
    a.chunks = (pool->ow + STEM_WIN - 1) / STEM_WIN;
    a.items = l->batch * pool->oh * a.chunks;
    stem_fastdiv((unsigned)a.chunks, a.div_chunks_mul, a.div_chunks_shr);
    stem_fastdiv((unsigned)pool->oh, a.div_oh_mul, a.div_oh_shr);
    void (*kernel)(const StemSparseArgs) = threads <= 256 ? stem_bwd_sparse_kernel<256, 3, 1> : stem_bwd_sparse_kernel<512, 1, 2>;
    AET_TRY(ctx_smem_attr(ctx, kernel, 160 * 1024));
    if (!l->stem_resident &&
        (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&l->stem_resident, kernel, threads, smem) != cudaSuccess || l->stem_resident < 1))
        l->stem_resident = 1;
    int blocks = l->stem_resident * ctx->sm_count;
    if (blocks > a.items) blocks = a.items;
    if (blocks > l->stem_blocks) blocks = l->stem_blocks;
    a.x = x_in; a.pdelta = pool->delta->d; a.code = l->stem_code; a.ymax = l->stem_ymax;
    a.mean = l->mean; a.inv = l->inv_std; a.gamma = layer_s(l); a.beta = layer_b(l);
    a.partial_s = l->stem_partial; a.partial_t = l->stem_partial + (size_t)l->stem_blocks * 2 * l->ocp;
    a.act = l->act; a.ocp = l->ocp; a.N = l->batch; a.H = l->h; a.W = l->w; a.OH = pool->oh; a.OW = pool->ow;
    const double bytes = 9.0 * l->batch * pool->oh * pool->ow * l->ocp + 16.0 * l->batch * l->h * l->w;
    LaunchScope s(ctx, "stem_bwd_sparse", bytes, 2.0 * l->batch * pool->oh * pool->ow * l->ocp * 27.0);
    a.span = ctx->span_ptr;
    launch_k(ctx->stream, blocks, threads, smem, kernel, a);
    AET_TRY(aet_check_launch("stem_bwd_sparse"));
    l->stem_blocks_used = blocks;
    return AET_OK;
}

// BN coefficients, scale / shift gradients and the weight gradient, once the Gram matrix is there.
int k_stem_finish(aet_layer *l, float *dw, int accumulate) {
    aet_context *ctx = l->ctx;
    StemFinishArgs a = {};
    a.partial_s = l->stem_partial;
    a.partial_t = l->stem_partial + (size_t)l->stem_blocks * 2 * l->ocp;
    a.w = layer_W(l); a.gram = l->stem_gram;
    a.variance = l->variance; a.inv = l->inv_std; a.gamma = layer_s(l);
    a.g_gamma = layer_sG(l); a.g_beta = layer_bG(l); a.coef = l->bwd_coef;
    a.dw = dw; a.blocks = l->stem_blocks_used; a.ocp = l->ocp; a.accumulate = accumulate; a.parity = ctx->parity;
    a.pixels = (double)l->batch * l->h * l->w;
    LaunchScope s(ctx, "stem_bwd_finish", 0, 0);
    launch_k(ctx->stream, l->oc, STEM_TAPS * STEM_FIN_LANES, 0, stem_bwd_finish_kernel, a);
    return aet_check_launch("stem_bwd_finish");
}

int stem_alloc(aet_layer *l, aet_layer *pool) {
    aet_context *ctx = l->ctx;
    l->stem_blocks = 4 * ctx->sm_count;
    l->stem_gram_blocks = 4 * ctx->sm_count;
    const size_t pooled = (size_t)l->batch * pool->oh * pool->ow * l->ocp;
    const size_t part = (size_t)l->stem_blocks * (2 + STEM_TAPS) * l->ocp;
    AET_CUDA(cudaMalloc(&l->stem_ymax, pooled * sizeof(float)));
    AET_CUDA(cudaMalloc(&l->stem_code, pooled));
    AET_CUDA(cudaMalloc(&l->stem_partial, part * sizeof(float)));
    AET_CUDA(cudaMalloc(&l->stem_gram_partial, (size_t)l->stem_gram_blocks * STEM_GRAM_PART * sizeof(float)));
    AET_CUDA(cudaMalloc(&l->stem_gram, (size_t)STEM_GRAM_PART * sizeof(double)));
    AET_CUDA(cudaMemset(l->stem_ymax, 0, pooled * sizeof(float)));
    AET_CUDA(cudaMemset(l->stem_code, 4, pooled));
    return AET_OK;
}
