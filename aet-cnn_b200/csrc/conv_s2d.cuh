// Strided first-layer convolutions whose filter is too large for the persistent thin-K kernel (an 11x11 / stride-4
// layer on 3 channels: K = 484), rewritten as a stride-1 convolution the TMA kernels can run.  Included by conv.cu.
//
// With stride s, input pixel (oh*s + r - pad, ow*s + c - pad) of output pixel (oh, ow) and filter tap (r, c) is, in an
// input regrouped into s x s blocks of pixels, block (oh + r/s, ow + c/s), position (r % s, c % s).  So
//     y[n][oh][ow][k] = sum over block taps (ry, rx), positions (dy, dx), channels ch of
//                       xb[n][oh + ry][ow + rx][(dy*s + dx)*4 + ch] * wb[k][ry][rx][(dy*s + dx)*4 + ch]
// is a ceil(R/s) x ceil(R/s) convolution with stride 1 and no padding over s*s*4 channels (rounded up to a multiple
// of 32 with zeros), where xb is the regrouped, zero-padded input and wb the regrouped filter (zero where r or c
// falls outside the R x R filter).  The products are the same ones the strided convolution forms, plus zeros.  The
// weight gradient of the regrouped layer holds every element of the real one exactly once, so it is folded back by
// a gather (done where the regrouped gradient can run on a TMA kernel; otherwise the weight gradient keeps its own
// path).  The data gradient is not rewritten: a first layer has none.
#pragma once

namespace {

struct S2dGeom {
    int s, rb, hb, wb, cpad, cells;   // stride, block taps per side, regrouped map, regrouped channels, 16-byte cells of a block
};

bool s2d_geom(const aet_layer *l, S2dGeom *out) {
    const aet_context *ctx = l->ctx;
    if (!ctx->opt[OPT_S2D] || ctx->conv_path != 0 || l->groups != 1 || l->dilation != 1 || l->cp != 4) return false;
    if (l->stride_x != l->stride_y || l->stride_x < 2 || l->size <= l->stride_x) return false;
    if (l->size * l->size * l->cp <= THIN_MAX_CELLS * 4) return false;   // the thin-K kernels take it as it is
    S2dGeom g;
    g.s = l->stride_x;
    g.rb = (l->size + g.s - 1) / g.s;
    g.hb = l->oh + g.rb - 1;
    g.wb = l->ow + g.rb - 1;
    g.cells = g.s * g.s;
    g.cpad = round_up(g.cells * 4, 32);
    if (g.wb > 128 || g.cpad > 256) return false;                         // the TMA kernels' map width; a sane channel count
    if ((double)l->batch * g.hb * g.wb * g.cpad >= 2147483648.0) return false;
    *out = g;
    return true;
}

// regrouped input: one thread per 16-byte cell of xb, cells of one block pixel consecutive
__global__ void __launch_bounds__(256) s2d_input_kernel(const float *__restrict__ x, float *__restrict__ xb, int N, int H, int W, int pad,
                                                        int s, int hb, int wb, int cpad, long long total) {
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int per = cpad / 4;
    const int cell = (int)(i % per);
    long long q = i / per;
    const int bx = (int)(q % wb); q /= wb;
    const int by = (int)(q % hb);
    const int n = (int)(q / hb);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cell < s * s) {
        const int iy = by * s + cell / s - pad, ix = bx * s + cell % s - pad;
        if (iy >= 0 && iy < H && ix >= 0 && ix < W) v = ldg4(x + ((size_t)((size_t)n * H + iy) * W + ix) * 4);
    }
    *reinterpret_cast<float4 *>(xb + (size_t)i * 4) = v;
}

// regrouped filter: wb[k][ry][rx][cell] = w[k][ry*s + dy][rx*s + dx] (16 bytes = the 4 padded channels of a tap)
__global__ void __launch_bounds__(256) s2d_weight_kernel(const float *__restrict__ w, float *__restrict__ wbk, int K, int R, int s, int rb,
                                                         int cpad, int total) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int per = cpad / 4;
    const int cell = i % per;
    int q = i / per;
    const int rx = q % rb; q /= rb;
    const int ry = q % rb;
    const int k = q / rb;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cell < s * s) {
        const int r = ry * s + cell / s, c = rx * s + cell % s;
        if (r < R && c < R) v = ldg4(w + ((size_t)((size_t)k * R + r) * R + c) * 4);
    }
    *reinterpret_cast<float4 *>(wbk + (size_t)i * 4) = v;
}

// weight gradient folded back: every tap of the real filter sits in exactly one cell of the regrouped gradient
__global__ void __launch_bounds__(256) s2d_fold_kernel(const float *__restrict__ gb, float *__restrict__ dw, int K, int R, int s, int rb,
                                                       int cpad, int accumulate, int total) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = i % R, r = (i / R) % R, k = i / (R * R);
    const int cell = (r % s) * s + c % s;
    float4 v = ldg4(gb + ((size_t)((size_t)k * rb + r / s) * rb + c / s) * cpad + cell * 4);
    float4 *dst = reinterpret_cast<float4 *>(dw + (size_t)i * 4);
    if (accumulate) {
        const float4 o = *dst;
        v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
    }
    *dst = v;
}

// The regrouped layer: an aet_layer that carries only what the convolution launchers read (geometry, weights, the
// tensor-map cache); it owns no activations.
int s2d_shadow(aet_layer *l, const S2dGeom &g, aet_layer **out) {
    if (l->s2d) { *out = l->s2d; return AET_OK; }
    aet_layer *sh = new aet_layer();
    sh->ctx = l->ctx; sh->type = AET_CONVOLUTIONAL; sh->index = l->index;
    sh->batch = l->batch; sh->c = g.cpad; sh->h = g.hb; sh->w = g.wb; sh->cp = g.cpad;
    sh->oc = l->oc; sh->oh = l->oh; sh->ow = l->ow; sh->ocp = l->ocp;
    sh->size = g.rb; sh->stride_x = sh->stride_y = 1; sh->pad = 0;
    sh->bn = 0; sh->act = l->act; sh->train = l->train;
    sh->groups = 1; sh->dilation = 1; sh->cg = g.cpad; sh->cgp = g.cpad;
    const size_t wfloats = round_up_sz((size_t)l->oc * g.rb * g.rb * g.cpad, 1024);
    const size_t xfloats = (size_t)l->batch * g.hb * g.wb * g.cpad;
    ParamArena &a = sh->own_arena;
    a.capacity = a.used = wfloats;
    a.owns = true;
    if (cudaMalloc(&a.W, wfloats * sizeof(float)) != cudaSuccess || cudaMalloc(&a.G, wfloats * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&l->s2d_x, xfloats * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        if (a.W) cudaFree(a.W);
        if (a.G) cudaFree(a.G);
        if (l->s2d_x) { cudaFree(l->s2d_x); l->s2d_x = nullptr; }
        delete sh;
        aet_set_error("convolutional: allocation of the regrouped first-layer buffers failed");
        return AET_E_NOMEM;
    }
    sh->arena = &a;
    sh->seg_w.offset = 0; sh->seg_w.count = (size_t)l->oc * g.rb * g.rb * g.cpad; sh->seg_w.padded = wfloats;
    l->s2d = sh;
    *out = sh;
    return AET_OK;
}

int s2d_regroup_input(aet_layer *l, const S2dGeom &g, const float *x) {
    aet_context *ctx = l->ctx;
    const long long total = (long long)l->batch * g.hb * g.wb * (g.cpad / 4);
    LaunchScope scope(ctx, "conv_s2d_input", (double)l->batch * l->h * l->w * 16.0 + (double)total * 16.0, 0);
    launch_k(ctx->stream, (unsigned)((total + 255) / 256), 256, 0, s2d_input_kernel, x, l->s2d_x, l->batch, l->h, l->w, l->pad, g.s, g.hb,
             g.wb, g.cpad, total);
    return aet_check_launch("conv_s2d_input");
}

// 1 = the layer is not of this kind
int s2d_fprop(aet_layer *l, const float *x, float *y, const float *bias, int act_in_epilogue, ConvStats *stats) {
    S2dGeom g;
    if (!s2d_geom(l, &g)) return 1;
    aet_context *ctx = l->ctx;
    if (ctx->math != AET_MATH_TF32) return 1;   // the TMA kernels are the point of the regrouping, and they are TF32 only
    {
        // ... and they must be able to tile the output map (tiny maps stay with the gather kernel as they are)
        cuuint32_t bw, bh, bi;
        int rows_t, per_img;
        const bool dense = pixel_box(BM, l->oh, l->ow, &bw, &bh, &bi) && (int)bw == l->ow;
        if (!dense && !(ctx->opt[OPT_RAGGED] && ragged_box(BM, l->oh, l->ow, &rows_t, &per_img))) return 1;
    }
    aet_layer *sh = nullptr;
    AET_TRY(s2d_shadow(l, g, &sh));
    AET_TRY(s2d_regroup_input(l, g, x));
    l->s2d_src = x;
    {
        const int total = l->oc * g.rb * g.rb * (g.cpad / 4);
        LaunchScope scope(ctx, "conv_s2d_weights", (double)total * 32.0, 0);
        launch_k(ctx->stream, (unsigned)((total + 255) / 256), 256, 0, s2d_weight_kernel, (const float *)layer_W(l), layer_W(sh), l->oc,
                 l->size, g.s, g.rb, g.cpad, total);
        AET_TRY(aet_check_launch("conv_s2d_weights"));
    }
    sh->act = l->act;
    return conv_fprop(sh, l->s2d_x, y, bias, act_in_epilogue, stats);
}

int s2d_wgrad(aet_layer *l, const float *x, const float *dy, float *dw, int accumulate) {
    S2dGeom g;
    if (!s2d_geom(l, &g)) return 1;
    aet_context *ctx = l->ctx;
    {
        // worth it only where the regrouped weight gradient runs on a TMA kernel: its 32-pixel K slabs must tile the
        // output map or its rows must be wider than a slab (small odd maps stay with the gather kernel as they are)
        cuuint32_t bw, bh, bi;
        const bool tiles = pixel_box(BK, l->oh, l->ow, &bw, &bh, &bi) || (ctx->opt[OPT_RAGGED] && l->ow > BK);
        if (ctx->math != AET_MATH_TF32 || !tiles || (l->ocp % 32 && l->ocp >= 32)) return 1;
    }
    aet_layer *sh = nullptr;
    AET_TRY(s2d_shadow(l, g, &sh));
    // inside a network's step the forward pass has just regrouped this very input
    if (!(ctx->in_network_pass && l->s2d_src == x)) AET_TRY(s2d_regroup_input(l, g, x));
    AET_TRY(conv_wgrad(sh, l->s2d_x, dy, layer_G(sh), 0));
    const int total = l->oc * l->size * l->size;
    LaunchScope scope(ctx, "conv_s2d_fold", (double)total * 48.0, 0);
    launch_k(ctx->stream, (unsigned)((total + 255) / 256), 256, 0, s2d_fold_kernel, (const float *)layer_G(sh), dw, l->oc, l->size, g.s, g.rb,
             g.cpad, accumulate, total);
    return aet_check_launch("conv_s2d_fold");
}

void s2d_release(aet_layer *l) {
    if (l->s2d) {
        tma_release(l->s2d);
        if (l->s2d->own_arena.W) cudaFree(l->s2d->own_arena.W);
        if (l->s2d->own_arena.G) cudaFree(l->s2d->own_arena.G);
        delete l->s2d;
        l->s2d = nullptr;
    }
    if (l->s2d_x) { cudaFree(l->s2d_x); l->s2d_x = nullptr; }
}

}  // namespace
