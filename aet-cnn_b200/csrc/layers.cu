// Host-side layer objects: the C restatement of the reference's NLayer subclasses.  Each layer
// owns its output / delta tensors and its parameters exactly as the reference's constructors do
// (dnn/ConvolutionalLayer.c:60-230, dnn/MaxPoolLayer.c:12-56, dnn/AvgPoolLayer.c:17-27,
// dnn/SoftMaxLayer.c:20-45, dnn/DropoutLayer.c:20-50); forward / backward / update keep the
// reference's call order and write semantics:
//   conv forward overwrites its output; conv backward overwrites the previous delta;
//   pool / avg-pool / softmax ADD into the previous delta; gradients ACCUMULATE until update().
#include <math.h>
#include <string.h>

#include "common.h"
#include "activation.cuh"

namespace {

int fail_invalid(const char *msg) {
    aet_set_error("%s", msg);
    return AET_E_INVALID;
}

int arena_create(ParamArena *a, size_t floats) {
    a->capacity = floats;
    a->used = 0;
    a->owns = true;
    if (floats == 0) return AET_OK;
    AET_CUDA(cudaMalloc(&a->W, floats * sizeof(float)));
    AET_CUDA(cudaMalloc(&a->U, floats * sizeof(float)));
    AET_CUDA(cudaMalloc(&a->G, floats * sizeof(float)));
    AET_CUDA(cudaMemset(a->W, 0, floats * sizeof(float)));
    AET_CUDA(cudaMemset(a->U, 0, floats * sizeof(float)));
    AET_CUDA(cudaMemset(a->G, 0, floats * sizeof(float)));
    AET_CUDA(cudaDeviceSynchronize());   // the context stream does not order against the legacy stream
    return AET_OK;
}

ParamSegment arena_take(ParamArena *a, size_t count) {
    ParamSegment s;
    s.offset = a->used;
    s.count = count;
    s.padded = round_up_sz(count, 1024);
    a->used += s.padded;
    return s;
}

uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

int read_tensor_or_zero(aet_tensor *t, float *host) {
    if (t->lazy_zero) {
        memset(host, 0, t->count() * sizeof(float));
        return AET_OK;
    }
    return aet_tensor_read(t, host);
}

}  // namespace

size_t conv_param_floats(int c, int n, int size, int batch_normalize, int groups) {
    c /= groups > 0 ? groups : 1;
    const int cp = round_up(c, 4);
    size_t total = round_up_sz((size_t)n * size * size * cp, 1024) + round_up_sz((size_t)round_up(n, 4), 1024);
    if (batch_normalize) total += round_up_sz((size_t)round_up(n, 4), 1024);
    return total;
}

void arena_destroy(ParamArena *a) {
    if (a->owns) {
        if (a->W) cudaFree(a->W);
        if (a->U) cudaFree(a->U);
        if (a->G) cudaFree(a->G);
        if (a->M) cudaFree(a->M);
        if (a->V) cudaFree(a->V);
    }
    a->W = a->U = a->G = a->M = a->V = nullptr;
}

int arena_create_public(ParamArena *a, size_t floats) { return arena_create(a, floats); }

// ---------------------------------------------------------------------------- constructors
aet_layer *conv_layer_create_in(aet_context *ctx, ParamArena *arena, int batch, int h, int w, int c, int n, int groups,
                                int size, int stride_x, int stride_y, int dilation, int padding, aet_activation activation,
                                int batch_normalize, int train, int index) {
    if (!ctx) { aet_set_error("null context"); return nullptr; }
    if (groups < 1 || dilation < 1) { aet_set_error("convolutional: groups and dilation must be positive"); return nullptr; }
    if (groups > 1 && (c % groups || n % groups || (c / groups) % 4 || (n / groups) % 4)) {
        aet_set_error("convolutional: groups=%d needs channels/groups and filters/groups to be multiples of 4 (got %d, %d)", groups, c, n);
        return nullptr;
    }
    if (dilation > 1 && (size % 2 == 0 || padding != size / 2)) {
        // the reference sizes the output from `padding` but gathers with padding * dilation (dnn/ConvolutionalLayer.c:337-343,
        // 795-801): the two only agree for odd filters padded by size / 2, which is what its cfgs use
        aet_set_error("convolutional: dilation > 1 needs an odd size with padding = size/2");
        return nullptr;
    }
    if (batch_normalize != 0 && batch_normalize != 1) { aet_set_error("convolutional: batch_normalize must be 0 or 1"); return nullptr; }
    if ((int)activation < 0 || (int)activation >= AET_ACTIVATION_COUNT) { aet_set_error("convolutional: unsupported activation"); return nullptr; }
    if (act_needs_input(activation) && !batch_normalize) {
        aet_set_error("convolutional: swish / mish need batch_normalize=1 (their gradient is formed from the value before the "
                      "activation, which only the batch-norm backward kernels recompute)");
        return nullptr;
    }
    if (batch <= 0 || h <= 0 || w <= 0 || c <= 0 || n <= 0 || size <= 0 || stride_x <= 0 || stride_y <= 0 || padding < 0) {
        aet_set_error("convolutional: bad geometry");
        return nullptr;
    }
    const int oh = (h + 2 * padding - size) / stride_y + 1, ow = (w + 2 * padding - size) / stride_x + 1;
    if (oh <= 0 || ow <= 0) { aet_set_error("convolutional: empty output"); return nullptr; }
    aet_layer *l = new aet_layer();
    l->ctx = ctx; l->type = AET_CONVOLUTIONAL; l->index = index;
    l->batch = batch; l->c = c; l->h = h; l->w = w; l->cp = round_up(c, 4);
    l->oc = n; l->oh = oh; l->ow = ow; l->ocp = round_up(n, 4);
    l->size = size; l->stride_x = stride_x; l->stride_y = stride_y; l->pad = padding;
    l->bn = batch_normalize; l->act = activation; l->train = train;
    l->groups = groups; l->dilation = dilation; l->cg = c / groups; l->cgp = round_up(c / groups, 4);
    if (!arena) {
        if (arena_create(&l->own_arena, conv_param_floats(c, n, size, batch_normalize, groups)) != AET_OK) { delete l; return nullptr; }
        arena = &l->own_arena;
    }
    l->arena = arena;
    l->seg_w = arena_take(arena, (size_t)n * size * size * l->cgp);
    l->seg_b = arena_take(arena, (size_t)l->ocp);
    if (batch_normalize) l->seg_s = arena_take(arena, (size_t)l->ocp);
    if (arena->used > arena->capacity) { aet_set_error("parameter arena overflow"); delete l; return nullptr; }
    l->output = aet_tensor_create(ctx, batch, n, oh, ow);
    l->delta = train ? aet_tensor_create(ctx, batch, n, oh, ow) : nullptr;
    if (!l->output || (train && !l->delta)) { aet_layer_destroy(l); return nullptr; }
    if (batch_normalize) {
        l->x = aet_tensor_create(ctx, batch, n, oh, ow);
        float *blk = nullptr;
        if (!l->x || cudaMalloc(&blk, (size_t)9 * l->ocp * sizeof(float)) != cudaSuccess) {
            aet_set_error("convolutional: BN buffer allocation failed");
            aet_layer_destroy(l);
            return nullptr;
        }
        cudaMemset(blk, 0, (size_t)9 * l->ocp * sizeof(float));
        l->mean = blk; l->variance = blk + l->ocp; l->rolling_mean = blk + 2 * l->ocp;
        l->rolling_variance = blk + 3 * l->ocp; l->inv_std = blk + 4 * l->ocp; l->shift = blk + 5 * l->ocp;
        l->bwd_coef = blk + 6 * l->ocp;
        std::vector<float> ones(l->ocp, 0.f);
        for (int i = 0; i < n; ++i) ones[i] = 1.f;
        cudaMemcpy(layer_s(l), ones.data(), l->ocp * sizeof(float), cudaMemcpyHostToDevice);
        cudaDeviceSynchronize();
    }
    // Initial weights: scale * U(-1,1), scale = sqrt(2/(size*size*c)) as dnn/WeightData.c:153-167,
    // from a counter-based generator instead of rand().
    {
        std::vector<float> wts((size_t)n * (c / groups) * size * size);
        const float scale = sqrtf(2.f / (size * size * c / groups));   // dnn/ConvolutionalLayer.c:233
        for (size_t i = 0; i < wts.size(); ++i) {
            uint64_t z = mix64(0xA17C0DEULL + (uint64_t)index * 0x632BE59BD9B4E019ULL + (i + 1) * 0x9E3779B97F4A7C15ULL);
            float u = (float)(z >> 40) * (1.0f / 16777216.0f);
            wts[i] = scale * (2.f * u - 1.f);
        }
        if (tensor_upload_nchw(ctx, layer_W(l), wts.data(), n, c / groups, size, size, l->cgp, false) != AET_OK) {
            aet_layer_destroy(l);
            return nullptr;
        }
    }
    return l;
}

extern "C" aet_layer *aet_convolutional_layer_create(aet_context *ctx, int batch, int h, int w, int c, int n, int groups,
                                                     int size, int stride_x, int stride_y, int dilation, int padding,
                                                     aet_activation activation, int batch_normalize, int train) {
    ctx_enter(ctx);
    return conv_layer_create_in(ctx, nullptr, batch, h, w, c, n, groups, size, stride_x, stride_y, dilation, padding,
                                activation, batch_normalize, train, 0);
}

extern "C" aet_layer *aet_maxpool_layer_create(aet_context *ctx, int batch, int h, int w, int c, int size, int stride_x,
                                               int stride_y, int padding, int train) {
    ctx_enter(ctx);
    if (!ctx || batch <= 0 || h <= 0 || w <= 0 || c <= 0 || size <= 0 || stride_x <= 0 || stride_y <= 0 || padding < 0) {
        aet_set_error("maxpool: bad geometry");
        return nullptr;
    }
    const int oh = (h + padding - size) / stride_y + 1, ow = (w + padding - size) / stride_x + 1;  // dnn/MaxPoolLayer.c:40-41
    if (oh <= 0 || ow <= 0) { aet_set_error("maxpool: empty output"); return nullptr; }
    aet_layer *l = new aet_layer();
    l->ctx = ctx; l->type = AET_MAXPOOL;
    l->batch = batch; l->c = c; l->h = h; l->w = w; l->cp = round_up(c, 4);
    l->oc = c; l->oh = oh; l->ow = ow; l->ocp = l->cp;
    l->size = size; l->stride_x = stride_x; l->stride_y = stride_y; l->pad = padding; l->train = train;
    l->output = aet_tensor_create(ctx, batch, c, oh, ow);
    l->delta = train ? aet_tensor_create(ctx, batch, c, oh, ow) : nullptr;
    bool ok = l->output && (!train || l->delta);
    if (ok && train) {
        ok = cudaMalloc(&l->indexes, l->output->elems() * sizeof(int)) == cudaSuccess &&
             cudaMemset(l->indexes, 0xFF, l->output->elems() * sizeof(int)) == cudaSuccess;
        if (!ok) aet_set_error("maxpool: index allocation failed");
    }
    if (!ok) { aet_layer_destroy(l); return nullptr; }
    cudaDeviceSynchronize();
    return l;
}

extern "C" aet_layer *aet_avgpool_layer_create(aet_context *ctx, int batch, int w, int h, int c) {
    ctx_enter(ctx);
    if (!ctx || batch <= 0 || h <= 0 || w <= 0 || c <= 0) { aet_set_error("avgpool: bad geometry"); return nullptr; }
    aet_layer *l = new aet_layer();
    l->ctx = ctx; l->type = AET_AVGPOOL;
    l->batch = batch; l->c = c; l->h = h; l->w = w; l->cp = round_up(c, 4);
    l->oc = c; l->oh = 1; l->ow = 1; l->ocp = l->cp;
    l->output = aet_tensor_create(ctx, batch, c, 1, 1);
    l->delta = aet_tensor_create(ctx, batch, c, 1, 1);
    if (!l->output || !l->delta) { aet_layer_destroy(l); return nullptr; }
    return l;
}

extern "C" aet_layer *aet_softmax_layer_create(aet_context *ctx, int batch, int inputs, int groups, float temperature) {
    ctx_enter(ctx);
    if (!ctx || batch <= 0 || inputs <= 0 || groups <= 0 || inputs % groups || !(temperature > 0.f)) {
        aet_set_error("softmax: bad arguments");
        return nullptr;
    }
    aet_layer *l = new aet_layer();
    l->ctx = ctx; l->type = AET_SOFTMAX;
    l->batch = batch; l->c = inputs; l->h = 1; l->w = 1; l->cp = round_up(inputs, 4);
    l->oc = inputs; l->oh = 1; l->ow = 1; l->ocp = l->cp;
    l->groups = groups; l->temperature = temperature;
    l->output = aet_tensor_create(ctx, batch, inputs, 1, 1);
    l->delta = aet_tensor_create(ctx, batch, inputs, 1, 1);
    bool ok = l->output && l->delta;
    const size_t n = (size_t)batch * l->cp;
    ok = ok && cudaMalloc(&l->loss, n * sizeof(float)) == cudaSuccess && cudaMemset(l->loss, 0, n * sizeof(float)) == cudaSuccess;
    ok = ok && cudaMalloc(&l->sample_loss, (size_t)batch * groups * sizeof(float)) == cudaSuccess;
    ok = ok && cudaMalloc(&l->cost_base, 8 * sizeof(float)) == cudaSuccess && cudaMemset(l->cost_base, 0, 8 * sizeof(float)) == cudaSuccess;
    l->cost_dev = l->cost_base;
    if (!ok) { aet_set_error("softmax: allocation failed"); aet_layer_destroy(l); return nullptr; }
    cudaDeviceSynchronize();
    return l;
}

extern "C" aet_layer *aet_dropout_layer_create(aet_context *ctx, int batch, int inputs, float probability, aet_layer *prev) {
    ctx_enter(ctx);
    if (!ctx || !prev || !prev->output || batch != prev->batch || inputs != prev->oc * prev->oh * prev->ow ||
        !(probability >= 0.f && probability < 1.f)) {
        aet_set_error("dropout: bad arguments (needs the previous layer and a matching input count)");
        return nullptr;
    }
    aet_layer *l = new aet_layer();
    l->ctx = ctx; l->type = AET_DROPOUT; l->prev = prev;
    l->batch = batch; l->c = prev->oc; l->h = prev->oh; l->w = prev->ow; l->cp = prev->ocp;
    l->oc = l->c; l->oh = l->h; l->ow = l->w; l->ocp = l->cp;
    l->probability = probability;
    l->output = prev->output;   // aliases, not owned
    l->delta = prev->delta;
    const size_t n = prev->output->elems();
    bool ok = cudaMalloc(&l->rnd, n * sizeof(float)) == cudaSuccess && cudaMemset(l->rnd, 0, n * sizeof(float)) == cudaSuccess;
    ok = ok && cudaMalloc(&l->step_dev, sizeof(unsigned long long)) == cudaSuccess &&
         cudaMemset(l->step_dev, 0, sizeof(unsigned long long)) == cudaSuccess;
    if (!ok) { aet_set_error("dropout: allocation failed"); aet_layer_destroy(l); return nullptr; }
    cudaDeviceSynchronize();
    l->seed = 0xD509ULL;
    return l;
}

extern "C" aet_layer *aet_shortcut_layer_create(aet_context *ctx, int batch, int h, int w, int c, int n, aet_layer *const *from,
                                                aet_activation activation, int train) {
    ctx_enter(ctx);
    if (!ctx || batch <= 0 || h <= 0 || w <= 0 || c <= 0 || n < 1 || n > 4 || !from) {
        aet_set_error("shortcut: bad arguments (1 to 4 source layers)");
        return nullptr;
    }
    if ((int)activation < 0 || (int)activation >= AET_ACTIVATION_COUNT || act_needs_input(activation)) {
        aet_set_error("shortcut: unsupported activation (swish / mish are not restated for shortcut layers)");
        return nullptr;
    }
    for (int i = 0; i < n; ++i) {
        const aet_layer *f = from[i];
        if (!f || !f->output || f->batch != batch || f->oh != h || f->ow != w) {   // dnn/NetworkFactory.c:234
            aet_set_error("shortcut: source %d must be a layer with a %dx%d output map", i, h, w);
            return nullptr;
        }
        if (train && !f->delta) { aet_set_error("shortcut: source %d has no delta (created with train=0)", i); return nullptr; }
    }
    aet_layer *l = new aet_layer();
    l->ctx = ctx; l->type = AET_SHORTCUT; l->act = activation; l->train = train;
    l->batch = batch; l->c = c; l->h = h; l->w = w; l->cp = round_up(c, 4);
    l->oc = c; l->oh = h; l->ow = w; l->ocp = l->cp;
    l->n_from = n;
    for (int i = 0; i < n; ++i) l->from[i] = from[i];
    l->output = aet_tensor_create(ctx, batch, c, h, w);
    if (train) l->delta = aet_tensor_create(ctx, batch, c, h, w);
    if (!l->output || (train && !l->delta)) { aet_layer_destroy(l); return nullptr; }
    return l;
}

extern "C" void aet_layer_destroy(aet_layer *l) {
    ctx_enter(l ? l->ctx : nullptr);
    if (!l) return;
    if (l->ctx) cudaStreamSynchronize(l->ctx->stream);
    conv_release(l);
    if (l->type != AET_DROPOUT) {
        aet_tensor_destroy(l->output);
        aet_tensor_destroy(l->delta);
    }
    aet_tensor_destroy(l->x);
    if (l->mean) cudaFree(l->mean);
    if (l->indexes) cudaFree(l->indexes);
    if (l->loss) cudaFree(l->loss);
    if (l->sample_loss) cudaFree(l->sample_loss);
    if (l->stem_ymax) cudaFree(l->stem_ymax);
    if (l->stem_code) cudaFree(l->stem_code);
    if (l->stem_partial) cudaFree(l->stem_partial);
    if (l->stem_gram_partial) cudaFree(l->stem_gram_partial);
    if (l->stem_gram) cudaFree(l->stem_gram);
    if (l->lin_xbar) cudaFree(l->lin_xbar);
    if (l->lin_ticket) cudaFree(l->lin_ticket);
    if (l->cost_base) cudaFree(l->cost_base);
    if (l->rnd) cudaFree(l->rnd);
    if (l->step_dev) cudaFree(l->step_dev);
    arena_destroy(&l->own_arena);
    delete l;
}

// ---------------------------------------------------------------------------- forward
static int check_input(const aet_layer *l, const aet_tensor *in) {
    if (!in) return fail_invalid("layer forward/backward: state.input is NULL");
    if (in->n != l->batch || in->c != l->c || in->h != l->h || in->w != l->w) {
        aet_set_error("layer %d: input is %dx%dx%dx%d, expected %dx%dx%dx%d", l->index, in->n, in->c, in->h, in->w, l->batch,
                      l->c, l->h, l->w);
        return AET_E_INVALID;
    }
    return AET_OK;
}

extern "C" int aet_layer_forward(aet_layer *l, aet_state state) {
    ctx_enter(l ? l->ctx : nullptr);
    if (!l) return fail_invalid("null layer");
    l->ctx->prof_tag = l->net ? l->index : -1;
    AET_TRY(check_input(l, state.input));
    switch (l->type) {
    case AET_CONVOLUTIONAL:
        if (l->bn) {
            ConvStats cs = {l->mean, nullptr, 0};
            AET_TRY(conv_fprop(l, state.input->d, l->x->d, nullptr, 0, state.train ? &cs : nullptr));
            if (state.train) AET_TRY(k_bn_stats(l, 1, &cs));
            l->last_forward_train = state.train != 0;
            aet_layer *pool = l->fused_pool;
            if (pool && (pool->indexes || !state.train)) {
                // the following max-pool is produced here; the full-resolution activated output is
                // only materialised if a host tap asks for it
                l->stem_gram_ready = false;
                l->stem_delta_stale = false;
                if (l->stem && state.train && l->ctx->in_network_pass && l->ctx->opt[OPT_OVERLAP_WGRAD]) {
                    // the Gram matrix of the input patches depends on the input alone: it runs beside the forward pass
                    AET_TRY(side_begin(l->ctx));
                    const int gr = k_stem_gram(l, state.input->d);
                    side_end(l->ctx);
                    AET_TRY(gr);
                    l->stem_gram_ready = true;
                }
                AET_TRY(k_bn_pool_forward(l, pool, state.train ? 0 : 1));
                l->output_stale = true;
                pool->fused_ready = true;
                pool->output->lazy_zero = false;
            } else {
                AET_TRY(k_bn_apply(l, state.train ? 0 : 1));
                l->output_stale = false;
            }
        } else {
            l->lin_used = false; l->lin_out_stale = false; l->lin_delta_stale = false; l->lin_bwd_pending = false;
            if (l->lin_head && l->ctx->in_network_pass && state.train && state.truth) {
                // classifier head of a network in training: folded into the softmax layer's call
                l->lin_fwd_pending = true;
                l->lin_input = state.input;
                l->output->lazy_zero = false;
                return AET_OK;
            }
            l->lin_fwd_pending = false;
            AET_TRY(conv_fprop(l, state.input->d, l->output->d, layer_b(l), 1));
        }
        l->output->lazy_zero = false;
        return AET_OK;
    case AET_MAXPOOL:
        if (l->fused_ready && l->fused_into && state.input == l->fused_into->output) {
            l->fused_ready = false;   // already computed by the convolution's fused kernel
            return AET_OK;
        }
        l->fused_ready = false;
        l->output->lazy_zero = false;
        return k_maxpool_forward(l, state.input->d);
    case AET_AVGPOOL:
        l->output->lazy_zero = false;
        l->head_forward_pending = false;
        if (l->head_softmax && state.input == l->head_softmax->head_conv->output) {
            l->head_forward_pending = true;    // produced by the softmax layer's fused head kernel
            return AET_OK;
        }
        return k_avgpool_forward(l, state.input->d);
    case AET_SOFTMAX: {
        const float *truth = nullptr;
        if (state.truth) {
            if (state.truth->n != l->batch || state.truth->c * state.truth->h * state.truth->w != l->c)
                return fail_invalid("softmax: truth tensor shape does not match");
            truth = state.truth->d;
        }
        l->cost_valid = false;
        if (l->head_conv && l->head_conv->lin_fwd_pending) {
            aet_layer *cv = l->head_conv;
            cv->lin_fwd_pending = false;
            if (l->head_avg->head_forward_pending && state.input == l->head_avg->output && truth) {
                l->head_avg->head_forward_pending = false;
                AET_TRY(k_linhead_forward(cv, l->head_avg, l, cv->lin_input->d, truth));
                cv->lin_used = true;
                cv->lin_out_stale = true;
                l->delta->lazy_zero = false;
                return AET_OK;
            }
            AET_TRY(conv_fprop(cv, cv->lin_input->d, cv->output->d, layer_b(cv), 1));   // not the fused call pattern after all
        }
        if (l->head_avg && l->head_avg->head_forward_pending && state.input == l->head_avg->output) {
            l->head_avg->head_forward_pending = false;
            AET_TRY(k_head_forward(l->head_conv, l->head_avg, l, truth));
        } else {
            if (l->head_avg && l->head_avg->head_forward_pending) {   // not the fused call pattern after all
                l->head_avg->head_forward_pending = false;
                AET_TRY(k_avgpool_forward(l->head_avg, l->head_conv->output->d));
            }
            AET_TRY(k_softmax_forward(l, state.input->d, truth));
        }
        if (truth) l->delta->lazy_zero = false;
        return AET_OK;
    }
    case AET_SHORTCUT:
        l->output->lazy_zero = false;
        return k_shortcut_forward(l, state.input->d);
    case AET_DROPOUT:
        if (!state.train) return AET_OK;
        if (state.input != l->prev->output) return fail_invalid("dropout: state.input must be the previous layer's output");
        if (!l->rnd_fixed) AET_TRY(k_step_counter(l->ctx, l->step_dev));
        return k_dropout_forward(l, l->prev->output->d, l->rnd_fixed ? 0 : 1);
    }
    return fail_invalid("unknown layer type");
}

// ---------------------------------------------------------------------------- backward
extern "C" int aet_layer_backward(aet_layer *l, aet_state state) {
    ctx_enter(l ? l->ctx : nullptr);
    if (!l) return fail_invalid("null layer");
    l->ctx->prof_tag = l->net ? l->index : -1;
    if (l->net && !l->ctx->in_network_pass) l->net->grad_clean = false;   // a caller's own backward call accumulates into the arena
    if (!l->delta) return fail_invalid("layer was created with train=0");
    aet_tensor *pd = state.delta;
    if (pd && (pd->n != l->batch || pd->c != l->c || pd->h != l->h || pd->w != l->w))
        return fail_invalid("layer backward: state.delta shape does not match the layer input");
    switch (l->type) {
    case AET_CONVOLUTIONAL: {
        AET_TRY(check_input(l, state.input));
        if (l->lin_bwd_pending) {
            // fused linear head: softmax and avg-pool backward, this layer's data, weight and bias gradients in one kernel
            l->lin_bwd_pending = false;
            if (!pd) return fail_invalid("linear head backward needs the previous layer's delta");
            AET_TRY(k_linhead_backward(l, l->head_softmax->head_avg, l->head_softmax, pd->d));
            pd->lazy_zero = false;
            l->delta->lazy_zero = false;
            l->lin_delta_stale = true;
            l->head_softmax->head_avg->delta->lazy_zero = false;
            return AET_OK;
        }
        if (l->head_backward_done) {
            l->head_backward_done = false;    // delta and bias gradient came from the fused head kernel
        } else if (l->gather_pending && l->bn && l->fused_pool && l->stem && !pd && l->ctx->in_network_pass && l->last_forward_train) {
            // first layer: scale / shift gradients and the weight gradient straight from the pool-sized tensors
            l->gather_pending = false;
            if (!l->stem_gram_ready) AET_TRY(k_stem_gram(l, state.input->d));
            l->stem_gram_ready = false;
            AET_TRY(k_stem_backward(l, l->fused_pool, state.input->d));
            // The Gram kernels were queued on the side stream during the forward pass and the later layers' weight
            // gradients behind them; this is the last kernel of the backward pass, so the streams join here.
            AET_TRY(side_join(l->ctx));
            AET_TRY(k_stem_finish(l, layer_G(l), 1));
            l->delta->lazy_zero = false;
            l->stem_delta_stale = true;
            return AET_OK;
        } else if (l->gather_pending && l->bn && l->fused_pool) {
            // the max-pool's backward was deferred: gather its delta inside the BN backward kernels
            l->gather_pending = false;
            AET_TRY(k_bn_backward(l, l->fused_pool));
            l->delta->lazy_zero = false;
        } else {
            if (l->delta->lazy_zero) {   // nothing upstream wrote a gradient: materialise the zeros
                AET_TRY(aet_tensor_zero(l->delta));
                l->delta->lazy_zero = false;
            }
            if (l->bn) AET_TRY(k_bn_backward(l, nullptr));
            else AET_TRY(k_bias_act_backward(l));
        }
        // In a network's backward pass the weight gradient runs on the side stream, beside the
        // data-gradient chain of this and the earlier layers (both only read this layer's delta).
        if (l->ctx->overlap_wgrad) AET_TRY(side_begin(l->ctx));
        const int wr = conv_wgrad(l, state.input->d, l->delta->d, layer_G(l), l->ctx->wgrad_fresh ? 0 : 1);
        side_end(l->ctx);
        AET_TRY(wr);
        if (pd) {
            AET_TRY(conv_dgrad(l, l->delta->d, pd->d));
            pd->lazy_zero = false;
        }
        return AET_OK;
    }
    case AET_MAXPOOL:
        if (!pd) return AET_OK;
        if (l->delta->lazy_zero) { AET_TRY(aet_tensor_zero(l->delta)); l->delta->lazy_zero = false; }
        if (l->fused_into && pd == l->fused_into->delta && pd->lazy_zero && l->indexes) {
            l->fused_into->gather_pending = true;   // the convolution's BN backward gathers from this layer
            return AET_OK;
        }
        AET_TRY(k_maxpool_backward(l, pd->d, pd->lazy_zero ? 0 : 1));
        pd->lazy_zero = false;
        return AET_OK;
    case AET_AVGPOOL:
        if (!pd) return AET_OK;
        if (l->head_backward_done) { l->head_backward_done = false; return AET_OK; }
        if (l->head_softmax && l->head_softmax->head_conv->lin_bwd_pending) return AET_OK;   // done by the convolution's backward call
        if (l->delta->lazy_zero) { AET_TRY(aet_tensor_zero(l->delta)); l->delta->lazy_zero = false; }
        AET_TRY(k_avgpool_backward(l, pd->d, pd->lazy_zero ? 0 : 1));
        pd->lazy_zero = false;
        return AET_OK;
    case AET_SOFTMAX: {
        if (!pd) return AET_OK;
        if (pd->cp != l->cp) return fail_invalid("softmax backward: previous delta layout mismatch");
        if (l->head_conv && l->head_conv->lin_used && l->ctx->in_network_pass && pd == l->head_avg->delta && pd->lazy_zero &&
            l->head_conv->delta->lazy_zero && !l->delta->lazy_zero && l->head_conv->index > 0) {
            l->head_conv->lin_bwd_pending = true;   // everything happens in the convolution's backward call
            return AET_OK;
        }
        if (l->head_avg && pd == l->head_avg->delta && pd->lazy_zero && l->head_conv->delta && l->head_conv->delta->lazy_zero &&
            !l->delta->lazy_zero) {
            AET_TRY(k_head_backward(l->head_conv, l->head_avg, l));
            l->head_avg->head_backward_done = true;
            l->head_conv->head_backward_done = true;
            pd->lazy_zero = false;
            l->head_conv->delta->lazy_zero = false;
            return AET_OK;
        }
        // CPU path scales by 1, MTCS path by loss_scale (dnn/SoftMaxLayer.c:293-314)
        const float ls = (l->ctx->parity == AET_PARITY_MTCS && l->net) ? l->net->loss_scale : 1.0f;
        AET_TRY(k_axpy(l->ctx, pd->d, l->delta->d, ls, (size_t)l->batch * l->cp, pd->lazy_zero ? 0 : 1, "softmax_bwd"));
        pd->lazy_zero = false;
        return AET_OK;
    }
    case AET_SHORTCUT:
        if (l->delta->lazy_zero) { AET_TRY(aet_tensor_zero(l->delta)); l->delta->lazy_zero = false; }
        return k_shortcut_backward(l, pd);
    case AET_DROPOUT:
        if (!pd) return AET_OK;
        if (pd != l->prev->delta) return fail_invalid("dropout: state.delta must be the previous layer's delta");
        if (pd->lazy_zero) return AET_OK;
        return k_dropout_backward(l, pd->d);
    }
    return fail_invalid("unknown layer type");
}

// ---------------------------------------------------------------------------- update
extern "C" int aet_layer_update(aet_layer *l, int batch, float learning_rate, float momentum, float decay, float loss_scale) {
    ctx_enter(l ? l->ctx : nullptr);
    if (!l) return fail_invalid("null layer");
    if (l->type != AET_CONVOLUTIONAL) return AET_OK;
    if (batch <= 0 || !(loss_scale > 0.f)) return fail_invalid("update: batch and loss_scale must be positive");
    // mtcs/MtcsConvLayer.c:582,618-631
    const float lr = learning_rate * l->lr_scale / loss_scale;
    const float rate = lr / batch;
    // the GPU update scrubs non-finite weights and pending weight updates first (mtcs/MtcsConvLayer.c:586-587); the
    // CPU update does not (dnn/ConvolutionalLayer.c:959-980)
    const int scrub_w = l->ctx->parity == AET_PARITY_MTCS ? 1 : 0;
    const int scrub_bn = (l->bn && l->net && l->net->try_fix_nan && l->ctx->parity == AET_PARITY_MTCS) ? 2 : 0;
    AET_TRY(k_sgd_segment(l->ctx, layer_W(l), layer_U(l), layer_G(l), l->seg_w.padded, rate, momentum, -decay * batch * loss_scale, scrub_w));
    AET_TRY(k_sgd_segment(l->ctx, layer_b(l), layer_bU(l), layer_bG(l), l->seg_b.padded, rate, momentum, 0.f, scrub_bn));
    if (l->bn) AET_TRY(k_sgd_segment(l->ctx, layer_s(l), layer_sU(l), layer_sG(l), l->seg_s.padded, rate, momentum, 0.f, scrub_bn));
    return AET_OK;
}

// ConvolutionalLayer.fuseConvBatchnorm (dnn/ConvolutionalLayer.c:983-1003): the rolling statistics and the scale are
// folded into biases and weights, in double on the host exactly as the reference computes them (a one-off step before
// inference, not a hot path), and the layer becomes a plain convolution + bias + activation.
int conv_layer_fuse_batchnorm(aet_layer *l) {
    if (!l || l->type != AET_CONVOLUTIONAL || !l->bn) return AET_OK;
    const size_t nw = aet_layer_param_count(l, AET_P_WEIGHTS);
    std::vector<float> b(l->oc), s(l->oc), rm(l->oc), rv(l->oc), w(nw);
    AET_TRY(aet_layer_read(l, AET_P_BIASES, b.data()));
    AET_TRY(aet_layer_read(l, AET_P_SCALES, s.data()));
    AET_TRY(aet_layer_read(l, AET_P_ROLLING_MEAN, rm.data()));
    AET_TRY(aet_layer_read(l, AET_P_ROLLING_VARIANCE, rv.data()));
    AET_TRY(aet_layer_read(l, AET_P_WEIGHTS, w.data()));
    const size_t filter_size = nw / (size_t)l->oc;
    for (int f = 0; f < l->oc; ++f) {
        b[f] = b[f] - (double)s[f] * rm[f] / (sqrt((double)rv[f] + .00001));
        const double precomputed = s[f] / (sqrt((double)rv[f] + .00001));
        for (size_t i = 0; i < filter_size; ++i) w[(size_t)f * filter_size + i] *= precomputed;
    }
    AET_TRY(aet_layer_write(l, AET_P_BIASES, b.data()));
    AET_TRY(aet_layer_write(l, AET_P_WEIGHTS, w.data()));
    l->bn = 0;
    l->output_stale = false;
    if (l->fused_pool) { l->fused_pool->fused_into = nullptr; l->fused_pool->fused_ready = false; l->fused_pool = nullptr; }
    return AET_OK;
}

extern "C" int aet_layer_init_delta(aet_layer *l) {
    if (!l) return fail_invalid("null layer");
    if (!l->delta || l->type == AET_DROPOUT) return AET_OK;
    AET_TRY(aet_tensor_zero(l->delta));
    l->delta->lazy_zero = false;
    return AET_OK;
}

extern "C" aet_tensor *aet_layer_output(aet_layer *l) { return l ? l->output : nullptr; }
extern "C" aet_tensor *aet_layer_delta(aet_layer *l) { return l ? l->delta : nullptr; }
extern "C" aet_layer_type aet_layer_kind(const aet_layer *l) { return l ? l->type : AET_CONVOLUTIONAL; }
extern "C" int aet_layer_out_shape(const aet_layer *l, int *c, int *h, int *w) {
    if (!l) return fail_invalid("null layer");
    if (c) *c = l->oc;
    if (h) *h = l->oh;
    if (w) *w = l->ow;
    return AET_OK;
}

extern "C" float aet_layer_cost(aet_layer *l) {
    ctx_enter(l ? l->ctx : nullptr);
    if (!l || l->type != AET_SOFTMAX) return 0.f;
    if (!l->cost_valid) {
        float v = 0.f;
        if (vector_download(l->ctx, l->cost_dev, &v, 1) != AET_OK) return NAN;
        l->cost_host = v;
        l->cost_valid = true;
    }
    return l->cost_host;
}

// ---------------------------------------------------------------------------- parameter taps
extern "C" size_t aet_layer_param_count(const aet_layer *l, aet_param which) {
    if (!l) return 0;
    const size_t act = (size_t)l->batch * l->oc * l->oh * l->ow;
    switch (which) {
    case AET_P_WEIGHTS: case AET_P_WEIGHT_UPDATES:
        return l->type == AET_CONVOLUTIONAL ? (size_t)l->oc * l->cg * l->size * l->size : 0;
    case AET_P_BIASES: case AET_P_BIAS_UPDATES:
        return l->type == AET_CONVOLUTIONAL ? (size_t)l->oc : 0;
    case AET_P_SCALES: case AET_P_SCALE_UPDATES: case AET_P_ROLLING_MEAN: case AET_P_ROLLING_VARIANCE:
    case AET_P_MEAN: case AET_P_VARIANCE:
        return (l->type == AET_CONVOLUTIONAL && l->bn) ? (size_t)l->oc : 0;
    case AET_P_OUTPUT: return act;
    case AET_P_DELTA: return l->delta ? act : 0;
    case AET_P_X: case AET_P_X_NORM: return l->x ? act : 0;
    case AET_P_INDEXES: return l->indexes ? act : 0;
    case AET_P_LOSS: return l->loss ? act : 0;
    case AET_P_RAND: return l->rnd ? act : 0;
    }
    return 0;
}

static int read_vec_sum(aet_layer *l, const float *a, const float *b, float *host, size_t n) {
    AET_TRY(vector_download(l->ctx, a, host, n));
    if (b) {
        std::vector<float> t(n);
        AET_TRY(vector_download(l->ctx, b, t.data(), n));
        for (size_t i = 0; i < n; ++i) host[i] += t[i];
    }
    return AET_OK;
}

extern "C" int aet_layer_read(aet_layer *l, aet_param which, void *host_v) {
    ctx_enter(l ? l->ctx : nullptr);
    if (!l || !host_v) return fail_invalid("aet_layer_read: null argument");
    if (aet_layer_param_count(l, which) == 0) return fail_invalid("aet_layer_read: this layer has no such buffer");
    float *host = static_cast<float *>(host_v);
    aet_context *ctx = l->ctx;
    const size_t nw = (size_t)l->oc * l->cg * l->size * l->size;
    switch (which) {
    case AET_P_WEIGHTS:
        return tensor_download_nchw(ctx, layer_W(l), host, l->oc, l->cg, l->size, l->size, l->cgp);
    case AET_P_WEIGHT_UPDATES: {
        // what the reference's weight_updates holds: carried momentum plus the pending gradient
        AET_TRY(tensor_download_nchw(ctx, layer_U(l), host, l->oc, l->cg, l->size, l->size, l->cgp));
        std::vector<float> g(nw);
        AET_TRY(tensor_download_nchw(ctx, layer_G(l), g.data(), l->oc, l->cg, l->size, l->size, l->cgp));
        for (size_t i = 0; i < nw; ++i) host[i] += g[i];
        return AET_OK;
    }
    case AET_P_BIASES: return vector_download(ctx, layer_b(l), host, l->oc);
    case AET_P_BIAS_UPDATES: return read_vec_sum(l, layer_bU(l), layer_bG(l), host, l->oc);
    case AET_P_SCALES: return vector_download(ctx, layer_s(l), host, l->oc);
    case AET_P_SCALE_UPDATES: return read_vec_sum(l, layer_sU(l), layer_sG(l), host, l->oc);
    case AET_P_ROLLING_MEAN: return vector_download(ctx, l->rolling_mean, host, l->oc);
    case AET_P_ROLLING_VARIANCE: return vector_download(ctx, l->rolling_variance, host, l->oc);
    case AET_P_MEAN: return vector_download(ctx, l->mean, host, l->oc);
    case AET_P_VARIANCE: return vector_download(ctx, l->variance, host, l->oc);
    case AET_P_OUTPUT:
        if (l->output_stale) {   // fused forward skipped the full-resolution output: form it now
            AET_TRY(k_bn_apply(l, l->last_forward_train ? 0 : 1));
            l->output_stale = false;
        }
        if (l->lin_out_stale) {  // the linear head never ran the convolution itself
            AET_TRY(conv_fprop(l, l->lin_input->d, l->output->d, layer_b(l), 1));
            l->lin_out_stale = false;
        }
        return read_tensor_or_zero(l->output, host);
    case AET_P_DELTA:
        if (l->stem_delta_stale) {
            AET_TRY(k_stem_delta(l, l->fused_pool));
            l->stem_delta_stale = false;
        }
        if (l->lin_delta_stale) {
            AET_TRY(k_linhead_conv_delta(l, l->head_softmax->head_avg, l->head_softmax));
            l->lin_delta_stale = false;
        }
        return read_tensor_or_zero(l->delta, host);
    case AET_P_X: return aet_tensor_read(l->x, host);
    case AET_P_X_NORM: {
        AET_TRY(aet_tensor_read(l->x, host));
        std::vector<float> mean(l->oc), inv(l->oc);
        AET_TRY(vector_download(ctx, l->mean, mean.data(), l->oc));
        AET_TRY(vector_download(ctx, l->inv_std, inv.data(), l->oc));
        const size_t sp = (size_t)l->oh * l->ow;
        for (int b = 0; b < l->batch; ++b)
            for (int c = 0; c < l->oc; ++c) {
                float *p = host + ((size_t)b * l->oc + c) * sp;
                for (size_t i = 0; i < sp; ++i) p[i] = (p[i] - mean[c]) * inv[c];
            }
        return AET_OK;
    }
    case AET_P_INDEXES:
        return tensor_download_nchw_int(ctx, l->indexes, static_cast<int *>(host_v), l->batch, l->oc, l->oh, l->ow, l->ocp);
    case AET_P_LOSS:
        return tensor_download_nchw(ctx, l->loss, host, l->batch, l->oc, 1, 1, l->ocp);
    case AET_P_RAND:
        return tensor_download_nchw(ctx, l->rnd, host, l->batch, l->oc, l->oh, l->ow, l->ocp);
    }
    return fail_invalid("aet_layer_read: unknown selector");
}

static int write_vec(aet_layer *l, float *dev, const float *host, size_t n, float *zero_also) {
    AET_TRY(vector_upload(l->ctx, dev, host, n));
    if (zero_also) AET_CUDA(cudaMemsetAsync(zero_also, 0, n * sizeof(float), l->ctx->stream));
    return AET_OK;
}

extern "C" int aet_layer_write(aet_layer *l, aet_param which, const void *host_v) {
    ctx_enter(l ? l->ctx : nullptr);
    if (!l || !host_v) return fail_invalid("aet_layer_write: null argument");
    if (aet_layer_param_count(l, which) == 0) return fail_invalid("aet_layer_write: this layer has no such buffer");
    const float *host = static_cast<const float *>(host_v);
    aet_context *ctx = l->ctx;
    switch (which) {
    case AET_P_WEIGHTS:
        return tensor_upload_nchw(ctx, layer_W(l), host, l->oc, l->cg, l->size, l->size, l->cgp, false);
    case AET_P_WEIGHT_UPDATES:
        AET_TRY(tensor_upload_nchw(ctx, layer_U(l), host, l->oc, l->cg, l->size, l->size, l->cgp, false));
        AET_CUDA(cudaMemsetAsync(layer_G(l), 0, l->seg_w.padded * sizeof(float), ctx->stream));
        return AET_OK;
    case AET_P_BIASES: return write_vec(l, layer_b(l), host, l->oc, nullptr);
    case AET_P_BIAS_UPDATES: return write_vec(l, layer_bU(l), host, l->oc, layer_bG(l));
    case AET_P_SCALES: return write_vec(l, layer_s(l), host, l->oc, nullptr);
    case AET_P_SCALE_UPDATES: return write_vec(l, layer_sU(l), host, l->oc, layer_sG(l));
    case AET_P_ROLLING_MEAN: return write_vec(l, l->rolling_mean, host, l->oc, nullptr);
    case AET_P_ROLLING_VARIANCE: return write_vec(l, l->rolling_variance, host, l->oc, nullptr);
    case AET_P_MEAN: return write_vec(l, l->mean, host, l->oc, nullptr);
    case AET_P_VARIANCE: return write_vec(l, l->variance, host, l->oc, nullptr);
    case AET_P_OUTPUT:
        l->output->lazy_zero = false;
        l->output_stale = false;
        l->lin_out_stale = false;
        return aet_tensor_write(l->output, host);
    case AET_P_DELTA:
        l->delta->lazy_zero = false;
        l->lin_delta_stale = false;
        l->stem_delta_stale = false;
        return aet_tensor_write(l->delta, host);
    case AET_P_X: return aet_tensor_write(l->x, host);
    case AET_P_RAND:
        l->rnd_fixed = true;
        return tensor_upload_nchw(ctx, l->rnd, host, l->batch, l->oc, l->oh, l->ow, l->ocp, false);
    default: break;
    }
    return fail_invalid("aet_layer_write: this buffer is read-only");
}

// ---------------------------------------------------------------------------- weights file records
// dnn/ConvolutionalLayer.c:422-430 (save) and :456-486 (load): biases, then for BN layers scales,
// rolling mean, rolling variance, then the weights [n][c][size][size].
extern "C" int aet_layer_save_weights(aet_layer *l, void *fpv) {
    FILE *fp = static_cast<FILE *>(fpv);
    if (!l || !fp) return fail_invalid("aet_layer_save_weights: null argument");
    if (l->type != AET_CONVOLUTIONAL) return AET_OK;
    std::vector<float> v(l->oc);
    const aet_param order[4] = {AET_P_BIASES, AET_P_SCALES, AET_P_ROLLING_MEAN, AET_P_ROLLING_VARIANCE};
    for (int i = 0; i < (l->bn ? 4 : 1); ++i) {
        AET_TRY(aet_layer_read(l, order[i], v.data()));
        if (fwrite(v.data(), sizeof(float), v.size(), fp) != v.size()) { aet_set_error("weights file: short write"); return AET_E_IO; }
    }
    std::vector<float> wts(aet_layer_param_count(l, AET_P_WEIGHTS));
    AET_TRY(aet_layer_read(l, AET_P_WEIGHTS, wts.data()));
    if (fwrite(wts.data(), sizeof(float), wts.size(), fp) != wts.size()) { aet_set_error("weights file: short write"); return AET_E_IO; }
    return AET_OK;
}

extern "C" int aet_layer_load_weights(aet_layer *l, void *fpv) {
    FILE *fp = static_cast<FILE *>(fpv);
    if (!l || !fp) return fail_invalid("aet_layer_load_weights: null argument");
    if (l->type != AET_CONVOLUTIONAL) return AET_OK;
    std::vector<float> v(l->oc);
    const aet_param order[4] = {AET_P_BIASES, AET_P_SCALES, AET_P_ROLLING_MEAN, AET_P_ROLLING_VARIANCE};
    for (int i = 0; i < ((l->bn && !l->dontloadscales) ? 4 : 1); ++i) {   // dontloadscales: no batch-norm block (dnn/ConvolutionalLayer.c:468)
        if (fread(v.data(), sizeof(float), v.size(), fp) != v.size()) { aet_set_error("weights file: unexpected end (layer %d)", l->index); return AET_E_IO; }
        AET_TRY(aet_layer_write(l, order[i], v.data()));
    }
    std::vector<float> wts(aet_layer_param_count(l, AET_P_WEIGHTS));
    if (fread(wts.data(), sizeof(float), wts.size(), fp) != wts.size()) { aet_set_error("weights file: unexpected end (layer %d weights)", l->index); return AET_E_IO; }
    if (l->flipped) {   // stored as [(c * size * size) rows][filters]: transposeMatrix of dnn/ConvolutionalLayer.c:444-454,483-485
        const size_t rows = (size_t)l->cg * l->size * l->size, cols = (size_t)l->oc;
        std::vector<float> t(wts.size());
        for (size_t x = 0; x < rows; ++x)
            for (size_t y = 0; y < cols; ++y) t[y * rows + x] = wts[x * cols + y];
        wts.swap(t);
    }
    return aet_layer_write(l, AET_P_WEIGHTS, wts.data());
}
