// Network runtime: cfg reader + factory (dnn/NetworkFactory.c:77-173,328-354,543-601,671-824,
// 830-1013 and dnn/ConfigFile.c), the forward / backward / update loops of dnn/NNetwork.c:382-396,
// 627-654,667-716,740-813, the learning-rate schedule (:215-246), the Darknet .weights container
// (:64-147), plus what the reference does not have: a CUDA graph of the whole training step, a flat
// parameter arena updated by one fused kernel, and the NCCL gradient all-reduce for batch
// data-parallel training (issued per bucket on a side stream while backward continues).
#include <dlfcn.h>
#include <limits.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <map>

#include "common.h"

aet_layer *conv_layer_create_in(aet_context *ctx, ParamArena *arena, int batch, int h, int w, int c, int n, int groups,
                                int size, int stride_x, int stride_y, int dilation, int padding, aet_activation activation,
                                int batch_normalize, int train, int index);
size_t conv_param_floats(int c, int n, int size, int batch_normalize, int groups);
int conv_layer_fuse_batchnorm(aet_layer *l);
void arena_destroy(ParamArena *a);
int arena_create_public(ParamArena *a, size_t floats);

namespace {

// ---------------------------------------------------------------------------- cfg text
struct Section {
    std::string name;
    std::map<std::string, std::string> kv;
    int line = 0;
};

std::string trim(const std::string &s) {
    size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
    return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
}

int parse_cfg(const char *text, std::vector<Section> &out) {
    std::string all(text), line;
    size_t pos = 0;
    int lineno = 0;
    while (pos <= all.size()) {
        size_t nl = all.find('\n', pos);
        if (nl == std::string::npos) nl = all.size();
        line = trim(all.substr(pos, nl - pos));
        pos = nl + 1;
        ++lineno;
        if (line.empty() || line[0] == '#' || line[0] == ';') continue;
        if (line[0] == '[') {
            size_t close = line.find(']');
            if (close == std::string::npos) { aet_set_error("cfg line %d: missing ']'", lineno); return AET_E_IO; }
            Section s;
            s.name = trim(line.substr(1, close - 1));
            s.line = lineno;
            out.push_back(s);
            continue;
        }
        size_t eq = line.find('=');
        if (eq == std::string::npos || out.empty()) { aet_set_error("cfg line %d: expected key=value inside a section", lineno); return AET_E_IO; }
        out.back().kv[trim(line.substr(0, eq))] = trim(line.substr(eq + 1));
    }
    return AET_OK;
}

int opt_int(const Section &s, const char *key, int def) {
    auto it = s.kv.find(key);
    return it == s.kv.end() ? def : atoi(it->second.c_str());
}
float opt_float(const Section &s, const char *key, float def) {
    auto it = s.kv.find(key);
    return it == s.kv.end() ? def : (float)atof(it->second.c_str());
}
std::string opt_str(const Section &s, const char *key, const char *def) {
    auto it = s.kv.find(key);
    return it == s.kv.end() ? std::string(def) : it->second;
}

int parse_activation(const std::string &a, aet_activation *out) {
    // dnn/Activation.c:105-124, restricted to the types this library restates
    static const struct { const char *name; aet_activation act; } table[] = {
        {"linear", AET_LINEAR}, {"relu", AET_RELU}, {"leaky", AET_LEAKY}, {"logistic", AET_LOGISTIC}, {"relu6", AET_RELU6},
        {"relie", AET_RELIE}, {"ramp", AET_RAMP}, {"tanh", AET_TANH}, {"plse", AET_PLSE}, {"elu", AET_ELU}, {"loggy", AET_LOGGY},
        {"hardtan", AET_HARDTAN}, {"lhtan", AET_LHTAN}, {"selu", AET_SELU}, {"swish", AET_SWISH}, {"mish", AET_MISH}};
    for (const auto &e : table)
        if (a == e.name) { *out = e.act; return AET_OK; }
    aet_set_error("activation '%s' is outside the supported set (linear, relu, leaky, logistic, relu6, relie, ramp, tanh, plse, "
                  "elu, loggy, hardtan, lhtan, selu, swish, mish)", a.c_str());
    return AET_E_INVALID;
}

const char *kUnsupportedConvKeys[] = {"binary", "xnor", "bin_output", "sway", "rotate", "stretch", "stretch_sway",
                                      "antialiasing", "assisted_excitation", "cbn", "coordconv", "grad_centr", "reverse",
                                      "share_index"};

// ---------------------------------------------------------------------------- NCCL through dlopen
struct NcclUniqueId { char internal[128]; };
typedef int (*nccl_get_unique_id_t)(NcclUniqueId *);
typedef int (*nccl_comm_init_rank_t)(void **, int, NcclUniqueId, int);
// Leading fields of ncclConfig_t as NCCL 2.18 published them; NCCL reads `size` and `version` and takes its own
// defaults for the fields a caller's older layout does not have.
struct NcclConfig218 {
    size_t size;
    unsigned int magic, version;
    int blocking, cgaClusterSize, minCTAs, maxCTAs;
    const char *netName;
    int splitShare;
};
typedef int (*nccl_comm_init_rank_config_t)(void **, int, NcclUniqueId, int, NcclConfig218 *);
typedef int (*nccl_all_reduce_t)(const void *, void *, size_t, int, int, void *, cudaStream_t);
typedef int (*nccl_comm_destroy_t)(void *);
typedef const char *(*nccl_get_error_string_t)(int);
struct NcclApi {
    void *handle = nullptr;
    nccl_get_unique_id_t get_unique_id = nullptr;
    nccl_comm_init_rank_t comm_init_rank = nullptr;
    nccl_comm_init_rank_config_t comm_init_rank_config = nullptr;   // optional
    nccl_all_reduce_t all_reduce = nullptr;
    nccl_comm_destroy_t comm_destroy = nullptr;
    nccl_get_error_string_t error_string = nullptr;
};
NcclApi *nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (api.handle) {
            api.get_unique_id = (nccl_get_unique_id_t)dlsym(api.handle, "ncclGetUniqueId");
            api.comm_init_rank = (nccl_comm_init_rank_t)dlsym(api.handle, "ncclCommInitRank");
            api.comm_init_rank_config = (nccl_comm_init_rank_config_t)dlsym(api.handle, "ncclCommInitRankConfig");
            api.all_reduce = (nccl_all_reduce_t)dlsym(api.handle, "ncclAllReduce");
            api.comm_destroy = (nccl_comm_destroy_t)dlsym(api.handle, "ncclCommDestroy");
            api.error_string = (nccl_get_error_string_t)dlsym(api.handle, "ncclGetErrorString");
        }
    }
    if (!api.handle || !api.get_unique_id || !api.comm_init_rank || !api.all_reduce || !api.comm_destroy) {
        aet_set_error("NCCL (libnccl.so.2) could not be loaded: %s", dlerror() ? dlerror() : "missing symbols");
        return nullptr;
    }
    return &api;
}
int nccl_fail(NcclApi *api, int code, const char *what) {
    aet_set_error("%s failed: %s", what, api->error_string ? api->error_string(code) : "NCCL error");
    return AET_E_NCCL;
}

// ---------------------------------------------------------------------------- helpers
float current_rate(const aet_network *net) {
    // dnn/NNetwork.c:215-246, with its types: batch_num is a size_t, so the divisions, the burn-in comparison and the
    // sig policy's `batch_num - step` are unsigned (the difference wraps while batch_num < step, which drives the
    // rate to 0 for gamma > 0 exactly as the reference's expression does), and pow / exp are the double functions.
    const size_t batch_num = (size_t)(net->seen / ((int64_t)net->batch * net->subdivisions));
    if (batch_num < (size_t)net->burn_in) return (float)(net->learning_rate * pow((float)batch_num / net->burn_in, net->power));
    switch (net->policy) {
    case 0: return net->learning_rate;
    case 1: return (float)(net->learning_rate * pow(net->scale, batch_num / (size_t)net->step));
    case 2: {
        float rate = net->learning_rate;
        for (int i = 0; i < net->num_steps; ++i) {
            if ((size_t)net->steps[i] > batch_num) return rate;
            rate *= net->scales[i];
        }
        return rate;
    }
    case 3: return (float)(net->learning_rate * pow(net->gamma, (int)batch_num));
    case 4: return (float)(net->learning_rate * pow(1 - (float)batch_num / net->max_batches, net->power));
    case 5: return (float)(net->learning_rate * (1. / (1. + exp(net->gamma * (batch_num - (size_t)net->step)))));
    default: return net->learning_rate;
    }
}

int build_sgd_tables(aet_network *net) {
    std::vector<int> block_seg;
    std::vector<float> seg_table;
    int seg_id = 0;
    for (aet_layer *l : net->layers) {
        if (l->type != AET_CONVOLUTIONAL) continue;
        const ParamSegment *segs[3] = {&l->seg_w, &l->seg_b, l->bn ? &l->seg_s : nullptr};
        for (int k = 0; k < 3; ++k) {
            if (!segs[k]) continue;
            if (segs[k]->offset != block_seg.size() * 1024) { aet_set_error("internal: arena segments are not contiguous"); return AET_E_INVALID; }
            const int first_block = (int)block_seg.size();
            for (size_t b = 0; b < segs[k]->padded / 1024; ++b) block_seg.push_back(seg_id);
            // {learning-rate multiplier, decay flag, non-finite scrub kind, first block of the segment (int bits)}
            const bool mtcs = net->ctx->parity == AET_PARITY_MTCS;
            float first_bits;
            memcpy(&first_bits, &first_block, sizeof(float));
            seg_table.push_back(l->lr_scale);
            seg_table.push_back(k == 0 ? 1.f : 0.f);
            seg_table.push_back(!mtcs ? 0.f : (k == 0 ? 1.f : ((l->bn && net->try_fix_nan) ? 2.f : 0.f)));
            seg_table.push_back(first_bits);
            net->seg_layer.push_back(l);
            ++seg_id;
        }
    }
    net->n_blocks = (int)block_seg.size();
    net->n_segments = seg_id;
    if (net->n_blocks == 0) return AET_OK;
    AET_CUDA(cudaMalloc(&net->block_seg, block_seg.size() * sizeof(int)));
    AET_CUDA(cudaMalloc(&net->seg_table, seg_table.size() * sizeof(float)));
    AET_CUDA(cudaMemcpy(net->block_seg, block_seg.data(), block_seg.size() * sizeof(int), cudaMemcpyHostToDevice));
    AET_CUDA(cudaMemcpy(net->seg_table, seg_table.data(), seg_table.size() * sizeof(float), cudaMemcpyHostToDevice));
    net->seg_host = seg_table;
    net->seg_skip.assign(seg_id, 0);
    return AET_OK;
}

// Which layers the coming update leaves alone (dnn/NNetwork.c:667-709): layers with train == 0 in both paths; in the GPU
// path also a layer whose dont_update is not yet below the iteration number.  A skipped segment keeps its weights and adds
// the step's gradient to its pending update, which is what the reference's single weight_updates buffer does when
// update() is not called.  The table changes rarely; the copy is ordered on the main stream like the kernels that read it.
int refresh_update_mask(aet_network *net) {
    if (net->seg_layer.empty()) return AET_OK;
    // (an update asked for before any training call counts as iteration 1, so that a bare aet_network_update still updates)
    const int64_t iteration = std::max<int64_t>(1, net->seen / ((int64_t)net->batch * net->subdivisions));
    const bool mtcs = net->ctx->parity == AET_PARITY_MTCS;
    bool changed = false;
    for (size_t sgi = 0; sgi < net->seg_layer.size(); ++sgi) {
        const aet_layer *l = net->seg_layer[sgi];
        const unsigned char skip = (l->train == 0 || (mtcs && !((int64_t)l->dont_update < iteration))) ? 1 : 0;
        if (skip != net->seg_skip[sgi]) { net->seg_skip[sgi] = skip; changed = true; }
    }
    if (!changed) return AET_OK;
    std::vector<float> t = net->seg_host;
    for (size_t sgi = 0; sgi < net->seg_skip.size(); ++sgi)
        if (net->seg_skip[sgi]) t[4 * sgi] = -1.f;
    // pageable source: the runtime stages it before the call returns, the copy itself runs in stream order
    AET_CUDA(cudaMemcpyAsync(net->seg_table, t.data(), t.size() * sizeof(float), cudaMemcpyHostToDevice, net->ctx->stream));
    return AET_OK;
}

aet_layer *softmax_layer(aet_network *net) {
    for (size_t i = net->layers.size(); i-- > 0;)
        if (net->layers[i]->type == AET_SOFTMAX) return net->layers[i];
    return nullptr;
}

int upload_hyper(aet_network *net) {
    AET_TRY(refresh_update_mask(net));
    const int world = net->world > 0 ? net->world : 1;
    const int update_batch = net->batch * net->subdivisions * world;
    const float rate = current_rate(net);
    float h[8] = {rate / net->loss_scale / update_batch, net->momentum, -net->decay * update_batch * net->loss_scale, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (net->adam) {
        // adam_update_gpu(w, d, m, v, B1, B2, eps, decay, learning_rate, n, batch, t), mtcs/MtcsConvLayer.c:494-524: the rate is
        // not divided by the batch, the decay term is -decay*batch, t is the current batch number (NNetwork.c:700)
        const int t = (int)(net->seen / ((int64_t)net->batch * net->subdivisions));
        h[4] = rate / net->loss_scale;
        h[5] = -net->decay * update_batch;
        h[6] = 1.f - powf(net->B1, (float)t);
        h[7] = 1.f - powf(net->B2, (float)t);
    }
    if (memcmp(h, net->hyper_host, sizeof(h)) == 0) return AET_OK;
    memcpy(net->hyper_host, h, sizeof(h));
    // The copy is asynchronous and the host may be many steps ahead of the device: every change of the rate is
    // staged in its own pinned slot, reused only after the copy that read it has run.
    const int slot = net->hyper_next;
    net->hyper_next = (slot + 1) % kHyperSlots;
    if (!net->hyper_ev[slot]) AET_CUDA(cudaEventCreateWithFlags(&net->hyper_ev[slot], cudaEventDisableTiming));
    if (net->hyper_used[slot]) AET_CUDA(cudaEventSynchronize(net->hyper_ev[slot]));
    float *stage = net->loss_pinned + 16 + 8 * slot;
    memcpy(stage, h, sizeof(h));
    AET_CUDA(cudaMemcpyAsync(net->hyper_dev, stage, sizeof(h), cudaMemcpyHostToDevice, net->ctx->stream));
    AET_CUDA(cudaEventRecord(net->hyper_ev[slot], net->ctx->stream));
    net->hyper_used[slot] = true;
    return AET_OK;
}

int net_forward(aet_network *net, aet_state state) {
    // dnn/NNetwork.c:382-396
    net->ctx->in_network_pass = true;
    int rc = AET_OK;
    for (size_t i = 0; i < net->layers.size() && rc == AET_OK; ++i) {
        aet_layer *l = net->layers[i];
        state.index = (int)i;
        if (l->delta && state.train && l->type != AET_DROPOUT) l->delta->lazy_zero = true;   // initDelta, without the memset
        rc = aet_layer_forward(l, state);
        state.input = l->output;
    }
    net->ctx->in_network_pass = false;
    return rc;
}

int issue_allreduce(aet_network *net, size_t lo, size_t hi, int slot) {
    NcclApi *api = nccl_api();
    if (!api) return AET_E_NCCL;
    aet_context *ctx = net->ctx;
    AET_CUDA(cudaEventRecord(net->ev_grad_ready[slot], ctx->stream));
    AET_CUDA(cudaStreamWaitEvent(net->comm_stream, net->ev_grad_ready[slot], 0));
    if (ctx->side_pending) {   // the weight gradients of the bucket were queued on the side stream
        AET_CUDA(cudaEventRecord(net->ev_grad_ready_side[slot], ctx->side_stream));
        AET_CUDA(cudaStreamWaitEvent(net->comm_stream, net->ev_grad_ready_side[slot], 0));
    }
    float *g = net->arena.G + lo;
    int r = api->all_reduce(g, g, hi - lo, 7 /* ncclFloat32 */, 0 /* ncclSum */, net->comm, net->comm_stream);
    if (r != 0) return nccl_fail(api, r, "ncclAllReduce");
    return AET_OK;
}

// `exchange`: this backward pass completes a gradient (the last call of a `subdivisions` group): only then
// are the accumulated gradients summed over the ranks.
int net_backward(aet_network *net, aet_state state, bool exchange = true) {
    // dnn/NNetwork.c:627-654
    aet_tensor *original_input = state.input, *original_delta = state.delta;
    const bool dp = net->comm != nullptr && net->world > 1 && exchange;
    const size_t bucket_floats = 64 * 1024;
    size_t pend_lo = 0, pend_hi = 0;
    int slot = 0;
    aet_context *ctx = net->ctx;
    ctx->overlap_wgrad = ctx->opt[OPT_OVERLAP_WGRAD] != 0;
    ctx->in_network_pass = true;
    // A gradient arena that fits the peer-exchange buffer is exchanged in one piece at the end of backward
    // (one synchronisation of the ranks per step, no collective kernels beside the backward pass).
    const bool whole = dp && net->xchg_active && net->arena.used <= net->xchg_cap;
    for (int i = (int)net->layers.size() - 1; i >= 0; --i) {
        aet_layer *l = net->layers[i];
        state.index = i;
        if (i == 0) { state.input = original_input; state.delta = original_delta; }
        else { state.input = net->layers[i - 1]->output; state.delta = net->layers[i - 1]->delta; }
        if (l->stopbackward) break;      // dnn/NNetwork.c:648-651
        if (l->onlyforward) continue;
        int br = aet_layer_backward(l, state);
        if (br == AET_OK && dp && !whole && l->type == AET_CONVOLUTIONAL) {
            const ParamSegment &last = l->bn ? l->seg_s : l->seg_b;
            const size_t lo = l->seg_w.offset, hi = last.offset + last.padded;
            if (pend_hi == pend_lo) { pend_lo = lo; pend_hi = hi; }
            else pend_lo = lo;   // layers are laid out in order, so walking backwards extends the range downwards
            // A bucket is sent as soon as it is full, unless what is left below it is small: the collectives of one
            // communicator run one after the other, so a separate small last bucket would queue behind this one and
            // add its whole latency to the end of the step; together they are one collective.
            if (br == AET_OK && pend_hi - pend_lo >= bucket_floats && (pend_lo >= bucket_floats / 2 || !ctx->opt[OPT_MERGE_TAIL]) && slot < 7) {
                br = issue_allreduce(net, pend_lo, pend_hi, slot++);
                pend_lo = pend_hi = 0;
            }
        }
        if (br != AET_OK) {   // leave the streams joined and the context in its plain state
            ctx->in_network_pass = false;
            ctx->overlap_wgrad = false;
            side_join(ctx);
            return br;
        }
    }
    ctx->overlap_wgrad = false;
    ctx->in_network_pass = false;
    // The last bucket holds the first layers' gradients, complete only now: a collective here would be fully
    // exposed, so with a peer exchange attached the ranks publish it and the update kernel sums it.
    net->tail_n = 0;
    if (whole) { net->tail_lo = 0; net->tail_n = net->arena.used; }
    else if (dp && pend_hi > pend_lo) {
        if (net->xchg_active && pend_hi - pend_lo <= net->xchg_cap) { net->tail_lo = pend_lo; net->tail_n = pend_hi - pend_lo; }
        else AET_TRY(issue_allreduce(net, pend_lo, pend_hi, slot++));
    }
    AET_TRY(side_join(ctx));
    if (dp && slot > 0) {
        // Option "comm_stamps": one-thread kernels read %globaltimer before and after the wait for the collectives, and
        // the second adds the difference to a running sum - how long the main stream sat idle for communication.
        const bool stamps = ctx->opt[OPT_COMM_STAMPS] != 0 && net->comm_stamp_dev;
        if (stamps) AET_TRY(k_comm_stamp(ctx, net->comm_stamp_dev, 0));
        AET_CUDA(cudaEventRecord(net->ev_comm_done, net->comm_stream));
        AET_CUDA(cudaStreamWaitEvent(net->ctx->stream, net->ev_comm_done, 0));
        pdl_skip_next();   // the kernel after a cross-stream wait is launched plainly
        if (stamps) AET_TRY(k_comm_stamp(ctx, net->comm_stamp_dev, 1));
        net->comm_stamped = stamps;
    }
    if (net->tail_n) AET_TRY(k_tail_publish(net));
    return AET_OK;
}

// One call of NNetwork.train(InputData*, TruthData*) (dnn/NNetwork.c:740-760) and, when `final`, the update
// that NNetwork.train(ImageData*) runs after its `subdivisions` calls (dnn/NNetwork.c:762-774).
int run_step(aet_network *net, bool final) {
    aet_state st = {};
    st.truth = net->truth; st.input = net->input; st.delta = nullptr; st.train = 1;
    AET_TRY(net_forward(net, st));
    st.input = net->input;
    // every update leaves the gradient arena zero, so without subdivisions this backward pass is the only writer of G
    net->ctx->wgrad_fresh = net->subdivisions == 1 && net->grad_clean;
    const int br = net_backward(net, st, final);
    net->ctx->wgrad_fresh = false;
    AET_TRY(br);
    net->grad_clean = false;
    if (!final) return AET_OK;   // gradients keep accumulating in the arena until the group's last call
    net->ctx->prof_tag = -1;   // the update belongs to no single layer
    if (net->n_blocks) AET_TRY(net->adam ? k_adam_arena(net) : k_sgd_arena(net));
    net->tail_n = 0;           // the published slices are consumed: a second update must not add them again
    net->grad_clean = true;
    return AET_OK;
}

void graph_drop(aet_network *net) {
    for (int k = 0; k < 4; ++k) {
        if (net->graph_exec[k]) {
            cudaGraphExecDestroy(net->graph_exec[k]);
            net->graph_exec[k] = nullptr;
        }
    }
    net->eager_runs[0] = net->eager_runs[1] = 0;
}

// Queues the read-back of {cost, mean loss} and of the device status word into three pinned floats.
int queue_loss_readback(aet_network *net, float *pinned3, cudaStream_t stream = nullptr) {
    aet_layer *sm = softmax_layer(net);
    cudaStream_t s = stream ? stream : net->ctx->stream;
    if (sm) AET_CUDA(cudaMemcpyAsync(pinned3, sm->cost_dev, 2 * sizeof(float), cudaMemcpyDeviceToHost, s));
    else pinned3[0] = pinned3[1] = 0.f;
    AET_CUDA(cudaMemcpyAsync(pinned3 + 2, net->ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
    return AET_OK;
}

// Turns the status word that came back with a loss into the call's return code.  A timed-out wait leaves the
// step incomplete (tiles unwritten, the update partly applied): the caller must treat the weights as lost and
// reload a checkpoint.  The non-finite flag is informational and is left for aet_context_check.
int status_to_code(aet_network *net, const float *pinned3) {
    int st;
    memcpy(&st, pinned3 + 2, sizeof(int));
    if (st & AET_STATUS_TIMEOUT) {
        cudaMemsetAsync(net->ctx->status_dev, 0, sizeof(int), net->ctx->stream);
        aet_set_error("a bounded device-side wait expired during the training step (status %d): the step is incomplete, "
                      "the weights must be reloaded", st);
        return AET_E_TIMEOUT;
    }
    return AET_OK;
}

bool host_pinned(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return at.type == cudaMemoryTypeHost;
}

}  // namespace

// ---------------------------------------------------------------------------- creation
extern "C" aet_network *aet_network_create_ex(aet_context *ctx, const char *cfg_text, int train, int batch_override) {
    ctx_enter(ctx);
    if (!ctx || !cfg_text) { aet_set_error("aet_network_create: null argument"); return nullptr; }
    std::vector<Section> secs;
    if (parse_cfg(cfg_text, secs) != AET_OK) return nullptr;
    if (secs.empty() || (secs[0].name != "net" && secs[0].name != "network")) {
        aet_set_error("cfg: the first section must be [net] or [network]");
        return nullptr;
    }
    aet_network *net = new aet_network();
    net->ctx = ctx; net->train = train;
    const Section &ns = secs[0];
    // dnn/NetworkFactory.c:671-824
    net->max_batches = opt_int(ns, "max_batches", 0);
    net->batch = opt_int(ns, "batch", 1);
    net->learning_rate = opt_float(ns, "learning_rate", .001f);
    net->momentum = opt_float(ns, "momentum", .9f);
    net->decay = opt_float(ns, "decay", .0001f);
    const int subdivs = opt_int(ns, "subdivisions", 1);
    net->batch /= subdivs > 0 ? subdivs : 1;
    net->subdivisions = subdivs > 0 ? subdivs : 1;
    if (batch_override > 0) { net->batch = batch_override; net->subdivisions = 1; }
    net->loss_scale = opt_float(ns, "loss_scale", 1.f);
    net->try_fix_nan = opt_int(ns, "try_fix_nan", 0);
    net->adam = opt_int(ns, "adam", 0);               // dnn/NetworkFactory.c:719-724
    if (net->adam) {
        net->B1 = opt_float(ns, "B1", .9f);
        net->B2 = opt_float(ns, "B2", .999f);
        net->eps = opt_float(ns, "eps", .000001f);
    }
    net->h = opt_int(ns, "height", 0); net->w = opt_int(ns, "width", 0); net->c = opt_int(ns, "channels", 0);
    net->power = opt_float(ns, "power", 4.f);
    net->burn_in = opt_int(ns, "burn_in", 0);
    const std::string policy = opt_str(ns, "policy", "constant");
    if (policy == "constant") net->policy = 0;
    else if (policy == "step") { net->policy = 1; net->step = opt_int(ns, "step", 1); net->scale = opt_float(ns, "scale", 1.f); }
    else if (policy == "steps") {
        net->policy = 2;
        std::string l = opt_str(ns, "steps", ""), p = opt_str(ns, "scales", "");
        if (l.empty() || p.empty()) { aet_set_error("cfg: STEPS policy must have steps and scales"); delete net; return nullptr; }
        char *sv = nullptr;
        for (char *tok = strtok_r(&l[0], ",", &sv); tok; tok = strtok_r(nullptr, ",", &sv)) net->steps.push_back(atoi(tok));
        for (char *tok = strtok_r(&p[0], ",", &sv); tok; tok = strtok_r(nullptr, ",", &sv)) net->scales.push_back((float)atof(tok));
        net->num_steps = (int)(net->steps.size() < net->scales.size() ? net->steps.size() : net->scales.size());
    }
    else if (policy == "exp") { net->policy = 3; net->gamma = opt_float(ns, "gamma", 1.f); }
    else if (policy == "poly") net->policy = 4;
    else if (policy == "sig") { net->policy = 5; net->gamma = opt_float(ns, "gamma", 1.f); net->step = opt_int(ns, "step", 1); }
    else { aet_set_error("cfg: unsupported learning-rate policy '%s'", policy.c_str()); delete net; return nullptr; }
    const std::string parity = opt_str(ns, "parity", "");
    if (parity == "cpu") ctx->parity = AET_PARITY_CPU;
    else if (parity == "mtcs") ctx->parity = AET_PARITY_MTCS;
    if (net->batch <= 0 || net->h <= 0 || net->w <= 0 || net->c <= 0) {
        aet_set_error("cfg: [net] needs positive batch, height, width and channels");
        delete net;
        return nullptr;
    }

    // first pass: parameter arena size
    size_t arena_floats = 0;
    {
        int c = net->c, h = net->h, w = net->w;
        for (size_t i = 1; i < secs.size(); ++i) {
            const Section &s = secs[i];
            if (s.name == "convolutional" || s.name == "conv") {
                const int n = opt_int(s, "filters", 1), size = opt_int(s, "size", 1);
                int stride = opt_int(s, "stride", 1), sx = opt_int(s, "stride_x", -1), sy = opt_int(s, "stride_y", -1);
                if (sx < 1) sx = stride;
                if (sy < 1) sy = stride;
                int padding = opt_int(s, "padding", 0);
                if (opt_int(s, "pad", 0)) padding = size / 2;
                arena_floats += conv_param_floats(c, n, size, opt_int(s, "batch_normalize", 0), opt_int(s, "groups", 1));
                h = (h + 2 * padding - size) / (sy > 0 ? sy : 1) + 1;
                w = (w + 2 * padding - size) / (sx > 0 ? sx : 1) + 1;
                c = n;
            } else if (s.name == "maxpool" || s.name == "max") {
                const int stride = opt_int(s, "stride", 1), sx = opt_int(s, "stride_x", stride), sy = opt_int(s, "stride_y", stride);
                const int size = opt_int(s, "size", stride), padding = opt_int(s, "padding", size - 1);
                h = (h + padding - size) / (sy > 0 ? sy : 1) + 1;
                w = (w + padding - size) / (sx > 0 ? sx : 1) + 1;
            } else if (s.name == "avgpool" || s.name == "avg") {
                h = w = 1;
            }
        }
    }
    if (arena_create_public(&net->arena, arena_floats) != AET_OK) { aet_network_destroy(net); return nullptr; }

    // second pass: layers (dnn/NetworkFactory.c:615-666)
    int c = net->c, h = net->h, w = net->w;
    for (size_t i = 1; i < secs.size(); ++i) {
        const Section &s = secs[i];
        aet_layer *l = nullptr;
        const int index = (int)net->layers.size();
        if (s.name == "convolutional" || s.name == "conv") {
            for (const char *k : kUnsupportedConvKeys)
                if (opt_float(s, k, 0.f) != 0.f && !(strcmp(k, "share_index") == 0 && opt_int(s, k, -1000000000) == -1000000000)) {
                    aet_set_error("cfg line %d: convolutional option '%s' is outside the supported hot path", s.line, k);
                    aet_network_destroy(net);
                    return nullptr;
                }
            const int n = opt_int(s, "filters", 1), groups = opt_int(s, "groups", 1), size = opt_int(s, "size", 1);
            int stride = opt_int(s, "stride", 1), sx = opt_int(s, "stride_x", -1), sy = opt_int(s, "stride_y", -1);
            if (sx < 1) sx = stride;
            if (sy < 1) sy = stride;
            int dilation = opt_int(s, "dilation", 1);
            if (size == 1) dilation = 1;
            int padding = opt_int(s, "padding", 0);
            if (opt_int(s, "pad", 0)) padding = size / 2;
            aet_activation act;
            if (parse_activation(opt_str(s, "activation", "logistic"), &act) != AET_OK) { aet_network_destroy(net); return nullptr; }
            l = conv_layer_create_in(ctx, &net->arena, net->batch, h, w, c, n, groups, size, sx, sy, dilation, padding, act,
                                     opt_int(s, "batch_normalize", 0), train, index);
            if (l) {
                l->lr_scale = opt_float(s, "learning_rate", 1.f);
                l->flipped = opt_int(s, "flipped", 0);
            }
        } else if (s.name == "maxpool" || s.name == "max") {
            const int stride = opt_int(s, "stride", 1), sx = opt_int(s, "stride_x", stride), sy = opt_int(s, "stride_y", stride);
            const int size = opt_int(s, "size", stride), padding = opt_int(s, "padding", size - 1);
            if (opt_int(s, "maxpool_depth", 0) || opt_int(s, "antialiasing", 0) || opt_int(s, "maxpool_zero_nonmax", 0)) {
                aet_set_error("cfg line %d: maxpool_depth / antialiasing / maxpool_zero_nonmax are outside the supported hot path", s.line);
                aet_network_destroy(net);
                return nullptr;
            }
            l = aet_maxpool_layer_create(ctx, net->batch, h, w, c, size, sx, sy, padding, train);
        } else if (s.name == "avgpool" || s.name == "avg") {
            l = aet_avgpool_layer_create(ctx, net->batch, w, h, c);
        } else if (s.name == "softmax" || s.name == "soft") {
            if (h != 1 || w != 1) { aet_set_error("cfg line %d: softmax input must be 1x1 spatial (got %dx%d)", s.line, h, w); aet_network_destroy(net); return nullptr; }
            if (opt_int(s, "spatial", 0) || !opt_str(s, "tree", "").empty()) { aet_set_error("cfg line %d: spatial / tree softmax are outside the supported hot path", s.line); aet_network_destroy(net); return nullptr; }
            l = aet_softmax_layer_create(ctx, net->batch, c, opt_int(s, "groups", 1), opt_float(s, "temperature", 1.f));
        } else if (s.name == "dropout") {
            if (net->layers.empty()) { aet_set_error("cfg line %d: dropout cannot be the first layer", s.line); aet_network_destroy(net); return nullptr; }
            if (opt_int(s, "dropblock", 0)) { aet_set_error("cfg line %d: dropblock is outside the supported hot path", s.line); aet_network_destroy(net); return nullptr; }
            l = aet_dropout_layer_create(ctx, net->batch, c * h * w, opt_float(s, "probability", .2f), net->layers.back());
            if (l) l->seed = 0xD509ULL + 0x9E3779B97F4A7C15ULL * (uint64_t)(index + 1);
        } else if (s.name == "shortcut") {
            // dnn/NetworkFactory.c:175-246: from = i[,j...] (negative = relative to this layer), activation default linear
            if (net->layers.empty()) { aet_set_error("cfg line %d: shortcut cannot be the first layer", s.line); aet_network_destroy(net); return nullptr; }
            if (opt_str(s, "weights_type", "none") != "none") { aet_set_error("cfg line %d: shortcut weights are outside the supported hot path", s.line); aet_network_destroy(net); return nullptr; }
            aet_activation a;
            if (parse_activation(opt_str(s, "activation", "linear"), &a) != AET_OK) { aet_network_destroy(net); return nullptr; }
            std::string from = opt_str(s, "from", "");
            aet_layer *src[4];
            int nsrc = 0;
            size_t pos = 0;
            while (pos < from.size() && nsrc < 5) {
                size_t comma = from.find(',', pos);
                std::string tok = from.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
                pos = comma == std::string::npos ? from.size() : comma + 1;
                if (tok.empty()) continue;
                int idx = atoi(tok.c_str());
                if (idx < 0) idx += index;
                if (idx < 0 || idx >= index || nsrc == 4) { nsrc = 5; break; }
                src[nsrc++] = net->layers[idx];
            }
            if (nsrc < 1 || nsrc > 4) { aet_set_error("cfg line %d: shortcut needs from = 1 to 4 earlier layers", s.line); aet_network_destroy(net); return nullptr; }
            for (int q = 0; q < nsrc; ++q) {
                // a source's full-resolution output and delta must exist: it leaves the call-pattern fusions
                aet_layer *f = src[q];
                if (f->fused_pool) { f->fused_pool->fused_into = nullptr; f->fused_pool = nullptr; f->stem = false; }
                f->lin_head = false;
            }
            {   // so does the layer in front of the shortcut (its output is this layer's input and its delta receives ours)
                aet_layer *f = net->layers.back();
                if (f->fused_pool) { f->fused_pool->fused_into = nullptr; f->fused_pool = nullptr; f->stem = false; }
            }
            l = aet_shortcut_layer_create(ctx, net->batch, h, w, c, nsrc, src, a, train);
        } else {
            aet_set_error("cfg line %d: layer type [%s] is outside the supported hot path", s.line, s.name.c_str());
            aet_network_destroy(net);
            return nullptr;
        }
        if (!l) { aet_network_destroy(net); return nullptr; }
        l->net = net;
        l->index = index;
        // keys every layer type takes (dnn/NetworkFactory.c:926-934)
        l->stopbackward = opt_int(s, "stopbackward", 0) == 1;
        l->dont_update = opt_int(s, "dont_update", 0);
        l->dontload = opt_int(s, "dontload", 0);
        l->dontloadscales = opt_int(s, "dontloadscales", 0);
        for (const char *k : {"onlyforward", "train_only_bn", "burnin_update", "clip"})
            if (opt_float(s, k, 0.f) != 0.f) {
                net->layers.push_back(l);   // owned by the network from here on
                aet_set_error("cfg line %d: layer option '%s' is outside the supported hot path", s.line, k);
                aet_network_destroy(net);
                return nullptr;
            }
        if (l->type == AET_MAXPOOL && !net->layers.empty() && ctx->opt[OPT_FUSE]) {
            aet_layer *prev = net->layers.back();
            if (prev->type == AET_CONVOLUTIONAL && prev->bn) {
                prev->fused_pool = l; l->fused_into = prev;
                if (prev->index == 0 && stem_backward_eligible(prev, l) && stem_alloc(prev, l) == AET_OK) prev->stem = true;
            }
        }
        net->layers.push_back(l);
        if (l->type == AET_SOFTMAX && net->layers.size() >= 3 && ctx->opt[OPT_FUSE]) {
            aet_layer *avg = net->layers[net->layers.size() - 2], *cv = net->layers[net->layers.size() - 3];
            if (avg->type == AET_AVGPOOL && cv->type == AET_CONVOLUTIONAL && !cv->bn && cv->act == AET_LINEAR && cv->delta &&
                l->groups == 1 && l->c <= 32) {
                l->head_conv = cv; l->head_avg = avg;
                avg->head_softmax = l; cv->head_softmax = l;
                // 1x1 classifier: the head is linear up to the softmax and can run on the pooled vectors
                if (cv->size == 1 && cv->stride_x == 1 && cv->stride_y == 1 && cv->pad == 0 && ctx->opt[OPT_LINEAR_HEAD] &&
                    (size_t)(cv->batch + 256) * l->c * sizeof(float) <= 40 * 1024 && (size_t)(cv->cp + 32) * sizeof(float) <= 40 * 1024 &&
                    cudaMalloc(&cv->lin_xbar, (size_t)cv->batch * cv->cp * sizeof(float)) == cudaSuccess &&
                    cudaMalloc(&cv->lin_ticket, sizeof(unsigned int)) == cudaSuccess &&
                    cudaMemset(cv->lin_ticket, 0, sizeof(unsigned int)) == cudaSuccess)
                    cv->lin_head = true;
            }
        }
        c = l->oc; h = l->oh; w = l->ow;
    }
    if (net->layers.empty()) { aet_set_error("cfg: no layers"); aet_network_destroy(net); return nullptr; }
    if (train) {
        // dnn/NetworkFactory.c:883-896,979-991: the layers in front of the LAST stopbackward layer only run forward and are
        // never updated; that layer itself keeps train = 1 (its update runs on gradients nothing ever writes)
        int last_stop = -1;
        for (aet_layer *l : net->layers)
            if (l->stopbackward) last_stop = l->index;
        for (int k = 0; k < last_stop; ++k) { net->layers[k]->onlyforward = 1; net->layers[k]->train = 0; }
        // the fused classifier head computes three layers' backward in the softmax layer's call: undo it when the walk
        // stops inside the head
        aet_layer *sm = softmax_layer(net);
        if (sm && sm->head_conv && last_stop >= sm->head_conv->index) {
            sm->head_conv->lin_head = false;
            sm->head_conv->head_softmax = nullptr;
            sm->head_avg->head_softmax = nullptr;
            sm->head_conv = nullptr; sm->head_avg = nullptr;
        }
        // so does the first layer's backward from the pool-sized tensors, which the pool layer's call prepares
        for (aet_layer *l : net->layers)
            if (l->index <= last_stop && l->stem) l->stem = false;
    }
    net->input = aet_tensor_create(ctx, net->batch, net->c, net->h, net->w);
    net->truth = aet_tensor_create(ctx, net->batch, c * h * w, 1, 1);
    bool ok = net->input && net->truth && build_sgd_tables(net) == AET_OK;
    ok = ok && cudaMalloc(&net->hyper_dev, 8 * sizeof(float)) == cudaSuccess;
    if (ok && net->adam) {
        ok = cudaMalloc(&net->arena.M, net->arena.capacity * sizeof(float)) == cudaSuccess &&
             cudaMalloc(&net->arena.V, net->arena.capacity * sizeof(float)) == cudaSuccess &&
             cudaMemset(net->arena.M, 0, net->arena.capacity * sizeof(float)) == cudaSuccess &&
             cudaMemset(net->arena.V, 0, net->arena.capacity * sizeof(float)) == cudaSuccess;
        cudaDeviceSynchronize();
    }
    ok = ok && cudaMallocHost(&net->loss_pinned, kPinnedFloats * sizeof(float)) == cudaSuccess;
    if (!ok) {
        if (!strlen(aet_last_error())) aet_set_error("network allocation failed");
        aet_network_destroy(net);
        return nullptr;
    }
    memset(net->loss_pinned, 0, kPinnedFloats * sizeof(float));
    net->hyper_host[1] = -1.f;   // force the first upload
    cudaStreamSynchronize(ctx->stream);
    return net;
}

extern "C" aet_network *aet_network_create_from_string(aet_context *ctx, const char *cfg_text, int train) {
    return aet_network_create_ex(ctx, cfg_text, train, 0);
}

extern "C" aet_network *aet_network_create(aet_context *ctx, const char *cfg_path, int train) {
    if (!cfg_path) { aet_set_error("aet_network_create: null path"); return nullptr; }
    FILE *fp = fopen(cfg_path, "rb");
    if (!fp) { aet_set_error("cannot open cfg file %s", cfg_path); return nullptr; }
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), fp)) > 0) text.append(buf, n);
    fclose(fp);
    return aet_network_create_ex(ctx, text.c_str(), train, 0);
}

extern "C" void aet_network_destroy(aet_network *net) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net) return;
    if (net->ctx) cudaStreamSynchronize(net->ctx->stream);
    aet_network_comm_destroy(net);
    graph_drop(net);
    for (size_t i = net->layers.size(); i-- > 0;) aet_layer_destroy(net->layers[i]);
    aet_tensor_destroy(net->input);
    aet_tensor_destroy(net->truth);
    if (net->input_alt) aet_tensor_destroy(net->input_alt);
    if (net->truth_alt) aet_tensor_destroy(net->truth_alt);
    arena_destroy(&net->arena);
    if (net->block_seg) cudaFree(net->block_seg);
    if (net->seg_table) cudaFree(net->seg_table);
    if (net->hyper_dev) cudaFree(net->hyper_dev);
    if (net->loss_pinned) cudaFreeHost(net->loss_pinned);
    for (int k = 0; k < kHyperSlots; ++k) if (net->hyper_ev[k]) cudaEventDestroy(net->hyper_ev[k]);
    for (int k = 0; k < 2; ++k) {
        if (net->stage_dev[k]) cudaFree(net->stage_dev[k]);
        if (net->stage_host[k]) cudaFreeHost(net->stage_host[k]);
        if (net->ev_staged[k]) cudaEventDestroy(net->ev_staged[k]);
        if (net->ev_consumed[k]) cudaEventDestroy(net->ev_consumed[k]);
        if (net->ev_loss[k]) cudaEventDestroy(net->ev_loss[k]);
    }
    if (net->copy_stream) cudaStreamDestroy(net->copy_stream);
    if (net->loss_stream) cudaStreamDestroy(net->loss_stream);
    delete net;
}

extern "C" int aet_network_layer_count(const aet_network *net) { return net ? (int)net->layers.size() : 0; }
extern "C" aet_layer *aet_network_layer(aet_network *net, int index) {
    if (!net || index < 0 || index >= (int)net->layers.size()) { aet_set_error("layer index out of range"); return nullptr; }
    return net->layers[index];
}
extern "C" int aet_network_batch(const aet_network *net) { return net ? net->batch : 0; }
extern "C" int aet_network_input_shape(const aet_network *net, int *c, int *h, int *w) {
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    if (c) *c = net->c;
    if (h) *h = net->h;
    if (w) *w = net->w;
    return AET_OK;
}
extern "C" int aet_network_outputs(const aet_network *net) {
    if (!net || net->layers.empty()) return 0;
    const aet_layer *l = net->layers.back();
    return l->oc * l->oh * l->ow;
}
extern "C" aet_tensor *aet_network_input(aet_network *net) { return net ? net->input : nullptr; }
extern "C" aet_tensor *aet_network_truth(aet_network *net) { return net ? net->truth : nullptr; }
extern "C" float aet_network_learning_rate(const aet_network *net) { return net ? current_rate(net) : 0.f; }
extern "C" int aet_network_set_hyper(aet_network *net, float learning_rate, float momentum, float decay) {
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    net->learning_rate = learning_rate; net->momentum = momentum; net->decay = decay;
    return AET_OK;
}
extern "C" int64_t aet_network_seen(const aet_network *net) { return net ? net->seen : 0; }

// ---------------------------------------------------------------------------- forward / backward / update
extern "C" int aet_network_forward(aet_network *net, aet_state state) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    return net_forward(net, state);
}
extern "C" int aet_network_backward(aet_network *net, aet_state state) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    net->grad_clean = false;
    return net_backward(net, state);
}
extern "C" int aet_network_update(aet_network *net) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    AET_TRY(upload_hyper(net));
    net->ctx->prof_tag = -1;   // the update belongs to no single layer
    if (net->n_blocks) AET_TRY(net->adam ? k_adam_arena(net) : k_sgd_arena(net));
    net->tail_n = 0;           // the published slices are consumed: a second update must not add them again
    net->grad_clean = true;
    return AET_OK;
}
extern "C" float aet_network_cost(aet_network *net) {
    ctx_enter(net ? net->ctx : nullptr);
    // dnn/NNetwork.c:611-624
    if (!net) return 0.f;
    float sum = 0.f;
    int count = 0;
    for (aet_layer *l : net->layers)
        if (l->type == AET_SOFTMAX) { sum += aet_layer_cost(l); ++count; }
    return count ? sum / count : 0.f;
}

extern "C" int aet_network_train_step_device(aet_network *net, float *loss) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    if (!net->train) { aet_set_error("network was created with train=0"); return AET_E_INVALID; }
    if (net->bn_fused) { aet_set_error("batch-norm layers were fused into their convolutions: this network only predicts"); return AET_E_INVALID; }
    aet_context *ctx = net->ctx;
    net->seen += net->batch;           // dnn/NNetwork.c:742
    // The reference runs `subdivisions` of these calls, then ONE update with update_batch = batch * subdivisions
    // (dnn/NNetwork.c:762-774, 667-680): weight gradients accumulate over the group's calls, and only its last
    // call exchanges them between ranks and applies them.
    const bool final = (net->seen / net->batch) % net->subdivisions == 0;
    if (final) {
        net->cur_iteration += 1;       // :773
        AET_TRY(upload_hyper(net));
    }
    const int kind = final ? 1 : 0;
    aet_layer *sm = softmax_layer(net);
    if (sm) {
        sm->cost_valid = false;
        sm->cost_dev = sm->cost_base + 4 * net->cur_slot;   // each input slot's graph writes a cost record of its own
    }
    const long before = ctx->launches;
    const int gi = kind + 2 * net->cur_slot;   // a graph holds its tensors' addresses: one per input slot
    const bool clean_now = net->subdivisions == 1 && net->grad_clean;
    if (net->use_graph && net->graph_exec[gi] && !ctx->profiling && net->graph_clean[gi] == clean_now) {
        AET_CUDA(cudaGraphLaunch(net->graph_exec[gi], ctx->stream));
        ctx->launches += net->graph_launches[gi];
        net->grad_clean = final;
    } else if (net->use_graph && net->eager_runs[kind] > 0 && !ctx->profiling) {
        // an eager step of this kind has sized every scratch buffer; capture this one
        if (net->graph_exec[gi]) { cudaGraphExecDestroy(net->graph_exec[gi]); net->graph_exec[gi] = nullptr; }   // captured in the other arena state
        cudaGraph_t graph = nullptr;
        AET_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        ctx->capturing = true;
        int r = run_step(net, final);
        ctx->capturing = false;
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        if (r != AET_OK) { if (graph) cudaGraphDestroy(graph); return r; }
        if (e != cudaSuccess) { aet_set_error("graph capture failed: %s", cudaGetErrorString(e)); return AET_E_CUDA; }
        net->graph_launches[gi] = ctx->launches - before;
        net->graph_clean[gi] = clean_now;
        e = cudaGraphInstantiate(&net->graph_exec[gi], graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) { aet_set_error("graph instantiate failed: %s", cudaGetErrorString(e)); net->graph_exec[gi] = nullptr; return AET_E_CUDA; }
        AET_CUDA(cudaGraphLaunch(net->graph_exec[gi], ctx->stream));
    } else {
        AET_TRY(run_step(net, final));
        net->eager_runs[kind] += 1;
    }
    if (final) net->launches_per_step = ctx->launches - before;
    if (loss) return aet_network_last_loss(net, loss);
    return AET_OK;
}

extern "C" int aet_network_last_loss(aet_network *net, float *loss) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !loss) { aet_set_error("null argument"); return AET_E_INVALID; }
    aet_layer *sm = softmax_layer(net);
    AET_TRY(queue_loss_readback(net, net->loss_pinned));
    AET_CUDA(cudaStreamSynchronize(net->ctx->stream));
    if (sm) {
        sm->cost_host = net->loss_pinned[0];
        sm->cost_valid = true;
    }
    *loss = net->loss_pinned[1];
    return status_to_code(net, net->loss_pinned);
}

extern "C" int aet_network_train_step(aet_network *net, const float *host_x, const float *host_truth, float *loss) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !host_x || !host_truth) { aet_set_error("aet_network_train_step: null argument"); return AET_E_INVALID; }
    aet_context *ctx = net->ctx;
    const size_t nx = net->input->count(), nt = net->truth->count();
    AET_TRY(ctx_staging(ctx, (nx + nt) * sizeof(float)));
    // Page-locked caller buffers (cudaHostAlloc / cudaHostRegister / a pinned torch tensor) are copied
    // by DMA straight from where they are; pageable ones go through the context's pinned mirror.
    const bool pinned = host_pinned(host_x) && host_pinned(host_truth);
    if (pinned) {
        AET_CUDA(cudaMemcpyAsync(ctx->staging, host_x, nx * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        AET_CUDA(cudaMemcpyAsync(ctx->staging + nx, host_truth, nt * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
        if (!loss) {   // the caller may reuse its buffers as soon as this returns: wait for the two copies (not for the step)
            if (!net->ev_uploaded) AET_CUDA(cudaEventCreateWithFlags(&net->ev_uploaded, cudaEventDisableTiming));
            AET_CUDA(cudaEventRecord(net->ev_uploaded, ctx->stream));
        }
    } else {
        // both uploads share the pinned mirror: stage x and truth back to back in it
        AET_CUDA(cudaStreamSynchronize(ctx->stream));
        memcpy(ctx->pinned, host_x, nx * sizeof(float));
        memcpy(ctx->pinned + nx, host_truth, nt * sizeof(float));
        AET_CUDA(cudaMemcpyAsync(ctx->staging, ctx->pinned, (nx + nt) * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    }
    AET_TRY(tensor_upload_staged(ctx, net->input->d, ctx->staging, net->input->n, net->input->c, net->input->h, net->input->w, net->input->cp));
    AET_TRY(tensor_upload_staged(ctx, net->truth->d, ctx->staging + nx, net->truth->n, net->truth->c, 1, 1, net->truth->cp));
    const int r = aet_network_train_step_device(net, loss);
    if (!loss && net->ev_uploaded && pinned) AET_CUDA(cudaEventSynchronize(net->ev_uploaded));
    return r;
}

// Pipelined form of aet_network_train_step.  The reference keeps the GPU fed with a host-side double buffer that
// loader threads fill while the previous batch trains (dnn/ImageData.c:169-202) and uploads each batch before
// its step (mtcs/MtcsIOData.c:50-52); here the double buffer is on the device: the copy of THIS call's batch
// runs on a copy stream while the PREVIOUS call's step still computes, and nothing waits for this step.
extern "C" int aet_network_train_step_async(aet_network *net, const float *host_x, const float *host_truth, float *previous_loss) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !host_x || !host_truth) { aet_set_error("aet_network_train_step_async: null argument"); return AET_E_INVALID; }
    if (!net->train) { aet_set_error("network was created with train=0"); return AET_E_INVALID; }
    aet_context *ctx = net->ctx;
    const size_t nx = net->input->count(), nt = net->truth->count();
    if (!net->copy_stream) {
        AET_CUDA(cudaSetDevice(ctx->device));
        AET_CUDA(cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking));
        AET_CUDA(cudaStreamCreateWithFlags(&net->loss_stream, cudaStreamNonBlocking));
        for (int k = 0; k < 2; ++k) {
            AET_CUDA(cudaMalloc(&net->stage_dev[k], (nx + nt) * sizeof(float)));
            AET_CUDA(cudaEventCreateWithFlags(&net->ev_staged[k], cudaEventDisableTiming));
            AET_CUDA(cudaEventCreateWithFlags(&net->ev_consumed[k], cudaEventDisableTiming));
            AET_CUDA(cudaEventCreateWithFlags(&net->ev_loss[k], cudaEventDisableTiming));
        }
        net->stage_floats = nx + nt;
    }
    const int slot = (int)(net->async_steps & 1), prev = slot ^ 1;
    const bool reused = net->async_steps >= 2;
    const float *src_x = host_x, *src_t = host_truth;
    if (!(host_pinned(host_x) && host_pinned(host_truth))) {
        // pageable buffers: through this slot's pinned mirror, free again once the copy of two calls ago has run
        if (!net->stage_host[slot]) AET_CUDA(cudaMallocHost(&net->stage_host[slot], (nx + nt) * sizeof(float)));
        if (reused) AET_CUDA(cudaEventSynchronize(net->ev_staged[slot]));
        memcpy(net->stage_host[slot], host_x, nx * sizeof(float));
        memcpy(net->stage_host[slot] + nx, host_truth, nt * sizeof(float));
        src_x = net->stage_host[slot]; src_t = net->stage_host[slot] + nx;
    }
    // Slot 1 has input and truth tensors of its own, so that the copy stream can also TRANSPOSE the batch of the
    // next step while this step still reads its input (the first layer's backward does, to the end of the step).
    if (slot == 1 && !net->input_alt) {
        net->input_alt = aet_tensor_create(ctx, net->input->n, net->input->c, net->input->h, net->input->w);
        net->truth_alt = aet_tensor_create(ctx, net->truth->n, net->truth->c, 1, 1);
        if (!net->input_alt || !net->truth_alt) return AET_E_NOMEM;
    }
    aet_tensor *in = slot ? net->input_alt : net->input, *tr = slot ? net->truth_alt : net->truth;
    if (reused) AET_CUDA(cudaStreamWaitEvent(net->copy_stream, net->ev_consumed[slot], 0));
    AET_CUDA(cudaMemcpyAsync(net->stage_dev[slot], src_x, nx * sizeof(float), cudaMemcpyHostToDevice, net->copy_stream));
    AET_CUDA(cudaMemcpyAsync(net->stage_dev[slot] + nx, src_t, nt * sizeof(float), cudaMemcpyHostToDevice, net->copy_stream));
    AET_TRY(tensor_upload_staged(ctx, in->d, net->stage_dev[slot], in->n, in->c, in->h, in->w, in->cp, net->copy_stream));
    AET_TRY(tensor_upload_staged(ctx, tr->d, net->stage_dev[slot] + nx, tr->n, tr->c, 1, 1, tr->cp, net->copy_stream));
    in->lazy_zero = false; tr->lazy_zero = false;
    AET_CUDA(cudaEventRecord(net->ev_staged[slot], net->copy_stream));
    AET_CUDA(cudaStreamWaitEvent(ctx->stream, net->ev_staged[slot], 0));
    pdl_skip_next();   // the kernel after a cross-stream wait is launched plainly
    // the step overwrites this slot's cost record: the read-back of two calls ago (long finished) must have run; the
    // previous step's read-back uses the other record, so the steps stay back to back
    if (reused) AET_CUDA(cudaStreamWaitEvent(ctx->stream, net->ev_loss[slot], 0));
    aet_tensor *in0 = net->input, *tr0 = net->truth;
    net->input = in; net->truth = tr; net->cur_slot = slot;
    const int sr = aet_network_train_step_device(net, nullptr);
    net->input = in0; net->truth = tr0; net->cur_slot = 0;
    AET_TRY(sr);
    AET_CUDA(cudaEventRecord(net->ev_consumed[slot], ctx->stream));   // the step has read the slot's tensors to its end
    // The loss travels back on a stream of its own, so that the steps stay back to back on the main stream.
    float *ring = net->loss_pinned + 8 + 4 * slot;
    AET_CUDA(cudaStreamWaitEvent(net->loss_stream, net->ev_consumed[slot], 0));
    AET_TRY(queue_loss_readback(net, ring, net->loss_stream));
    AET_CUDA(cudaEventRecord(net->ev_loss[slot], net->loss_stream));
    const bool have_prev = net->async_steps >= 1;
    net->async_steps += 1;
    if (!have_prev) {
        if (previous_loss) *previous_loss = NAN;
        return AET_OK;
    }
    // the previous step's result: its successor is already queued, so waiting here never idles the device
    AET_CUDA(cudaEventSynchronize(net->ev_loss[prev]));
    const float *pr = net->loss_pinned + 8 + 4 * prev;
    if (previous_loss) *previous_loss = pr[1];
    return status_to_code(net, pr);
}

extern "C" int aet_network_predict(aet_network *net, const float *host_x, float *host_out) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !host_x || !host_out) { aet_set_error("aet_network_predict: null argument"); return AET_E_INVALID; }
    AET_TRY(aet_tensor_write(net->input, host_x));
    aet_state st = {};
    st.input = net->input; st.train = 0;
    AET_TRY(net_forward(net, st));
    return aet_tensor_read(net->layers.back()->output, host_out);
}

// NNetwork.fuseConvBatchnorm (dnn/NNetwork.c:272-290), the convolutional branch.
extern "C" int aet_network_fuse_conv_batchnorm(aet_network *net) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    graph_drop(net);
    for (aet_layer *l : net->layers)
        if (l->type == AET_CONVOLUTIONAL && l->bn) AET_TRY(conv_layer_fuse_batchnorm(l));
    net->bn_fused = true;
    return AET_OK;
}

// Forward with train = 0 on a host batch, then DnnUtils.topK (dnn/DnnUtils.c:463-477) per sample on the device.
extern "C" int aet_network_predict_topk(aet_network *net, const float *host_x, int k, int *host_indexes) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !host_x || !host_indexes || k <= 0) { aet_set_error("aet_network_predict_topk: bad argument"); return AET_E_INVALID; }
    aet_layer *last = net->layers.back();
    const int classes = last->oc * last->oh * last->ow;
    if (last->oh != 1 || last->ow != 1) { aet_set_error("aet_network_predict_topk: the last layer must be 1x1 spatial"); return AET_E_INVALID; }
    if (k > classes) k = classes;
    AET_TRY(aet_tensor_write(net->input, host_x));
    aet_state st = {};
    st.input = net->input; st.train = 0;
    AET_TRY(net_forward(net, st));
    float *scratch = nullptr;
    AET_TRY(ctx_scratch(net->ctx, (size_t)net->batch * k * sizeof(int), &scratch));
    int *idx = reinterpret_cast<int *>(scratch);
    AET_TRY(k_top_k(net->ctx, last->output->d, net->batch, classes, last->ocp, k, idx));
    AET_CUDA(cudaMemcpyAsync(host_indexes, idx, (size_t)net->batch * k * sizeof(int), cudaMemcpyDeviceToHost, net->ctx->stream));
    AET_CUDA(cudaStreamSynchronize(net->ctx->stream));
    return AET_OK;
}

// The accuracy loop of Classifier.validateSingle (dnn/Classifier.c:359-464) over images already decoded, resized
// and cropped by the caller: predict, top-k, count hits.  top1 = avg_acc / count, topk = avg_topk / count.
extern "C" int aet_network_validate(aet_network *net, const float *host_images, const int *class_ids, int count, int k,
                                    float *top1, float *topk) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !host_images || !class_ids || count <= 0 || k <= 0) { aet_set_error("aet_network_validate: bad argument"); return AET_E_INVALID; }
    const size_t per = (size_t)net->c * net->h * net->w;
    aet_layer *last = net->layers.back();
    const int classes = last->oc;
    if (k > classes) k = classes;       // "if (topk > classes) topk = classes", :399-400
    std::vector<float> batch(per * net->batch, 0.f);
    std::vector<int> idx((size_t)net->batch * k);
    double avg_acc = 0, avg_topk = 0;
    for (int base = 0; base < count; base += net->batch) {
        const int n = count - base < net->batch ? count - base : net->batch;
        memcpy(batch.data(), host_images + (size_t)base * per, (size_t)n * per * sizeof(float));
        if (n < net->batch) memset(batch.data() + (size_t)n * per, 0, (size_t)(net->batch - n) * per * sizeof(float));
        AET_TRY(aet_network_predict_topk(net, batch.data(), k, idx.data()));
        for (int i = 0; i < n; ++i) {
            const int *ix = idx.data() + (size_t)i * k;
            if (ix[0] == class_ids[base + i]) avg_acc += 1;
            for (int j = 0; j < k; ++j)
                if (ix[j] == class_ids[base + i]) avg_topk += 1;
        }
    }
    if (top1) *top1 = (float)(avg_acc / count);
    if (topk) *topk = (float)(avg_topk / count);
    return AET_OK;
}

// The augmentation chain of ImageData.loadImageAugmentPaths (dnn/ImageData.c:56-73) on the device: upload the source
// images and the per-image draws, one kernel writes the network's input tensor.
extern "C" int aet_network_augment_input(aet_network *net, const float *host_src, int src_h, int src_w, const aet_augment *params) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !host_src || !params || src_h <= 0 || src_w <= 0) { aet_set_error("aet_network_augment_input: bad argument"); return AET_E_INVALID; }
    if (net->w != net->h) { aet_set_error("aet_network_augment_input: only square network inputs (the crop is size x size)"); return AET_E_INVALID; }
    aet_context *ctx = net->ctx;
    const size_t src_floats = (size_t)net->batch * net->c * src_h * src_w;
    const size_t par_floats = ((size_t)net->batch * sizeof(aet_augment) + sizeof(float) - 1) / sizeof(float);
    AET_TRY(ctx_staging(ctx, (src_floats + par_floats) * sizeof(float)));
    const bool pinned = host_pinned(host_src);
    if (pinned) {
        AET_CUDA(cudaMemcpyAsync(ctx->staging, host_src, src_floats * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    } else {
        AET_CUDA(cudaStreamSynchronize(ctx->stream));
        memcpy(ctx->pinned, host_src, src_floats * sizeof(float));
        AET_CUDA(cudaMemcpyAsync(ctx->staging, ctx->pinned, src_floats * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    }
    memcpy(ctx->pinned + src_floats, params, (size_t)net->batch * sizeof(aet_augment));
    AET_CUDA(cudaMemcpyAsync(ctx->staging + src_floats, ctx->pinned + src_floats, par_floats * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AET_TRY(k_augment(ctx, ctx->staging, net->batch, net->c, src_h, src_w, net->input->d, net->w, net->input->cp,
                      reinterpret_cast<const aet_augment *>(ctx->staging + src_floats)));
    net->input->lazy_zero = false;
    AET_CUDA(cudaStreamSynchronize(ctx->stream));   // the pinned mirror and the caller's buffers are free again
    return AET_OK;
}

extern "C" int aet_network_use_graph(aet_network *net, int enable) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    net->use_graph = enable != 0;
    if (!enable) graph_drop(net);
    return AET_OK;
}

// ---------------------------------------------------------------------------- weights container
extern "C" int aet_network_save_weights(aet_network *net, const char *path) {
    if (!net || !path) { aet_set_error("null argument"); return AET_E_INVALID; }
    FILE *fp = fopen(path, "wb");
    if (!fp) { aet_set_error("cannot open %s for writing", path); return AET_E_IO; }
    const int32_t header[3] = {0, 2, 5};
    const uint64_t seen = (uint64_t)net->cur_iteration * net->batch * net->subdivisions;   // dnn/NNetwork.c:126
    bool ok = fwrite(header, sizeof(int32_t), 3, fp) == 3 && fwrite(&seen, sizeof(uint64_t), 1, fp) == 1;
    int r = ok ? AET_OK : AET_E_IO;
    for (size_t i = 0; r == AET_OK && i < net->layers.size(); ++i) r = aet_layer_save_weights(net->layers[i], fp);
    fclose(fp);
    if (!ok) aet_set_error("weights file: short write");
    return r;
}

extern "C" int aet_network_load_weights(aet_network *net, const char *path) { return aet_network_load_weights_upto(net, path, -1); }

extern "C" int aet_network_load_weights_upto(aet_network *net, const char *path, int cutoff) {
    if (!net || !path) { aet_set_error("null argument"); return AET_E_INVALID; }
    FILE *fp = fopen(path, "rb");
    if (!fp) { aet_set_error("cannot open weights file %s", path); return AET_E_IO; }
    int32_t header[3];
    if (fread(header, sizeof(int32_t), 3, fp) != 3) { fclose(fp); aet_set_error("weights file: short header"); return AET_E_IO; }
    if (header[0] * 10 + header[1] >= 2) {
        uint64_t seen = 0;
        if (fread(&seen, sizeof(uint64_t), 1, fp) != 1) { fclose(fp); aet_set_error("weights file: short header"); return AET_E_IO; }
        net->seen = (int64_t)seen;
    } else {
        int32_t seen = 0;
        if (fread(&seen, sizeof(int32_t), 1, fp) != 1) { fclose(fp); aet_set_error("weights file: short header"); return AET_E_IO; }
        net->seen = seen;
    }
    // (the reference derives a whole-file `transpose` flag from major/minor > 1000 at dnn/NNetwork.c:92 and never uses
    // it; transposed records are a per-layer property, the cfg key `flipped`)
    net->cur_iteration = net->seen / ((int64_t)net->batch * net->subdivisions);
    int r = AET_OK;
    // dnn/NNetwork.c:93-108: layers marked dontload are passed over without consuming anything, and a file that ends at a
    // record boundary (a backbone cut off with `partial`) leaves the remaining layers as they are
    const size_t upto = cutoff < 0 ? net->layers.size() : std::min(net->layers.size(), (size_t)cutoff);
    for (size_t i = 0; r == AET_OK && i < upto; ++i) {
        aet_layer *l = net->layers[i];
        if (l->dontload || l->type != AET_CONVOLUTIONAL) continue;
        const int ch = fgetc(fp);
        if (ch == EOF) break;
        ungetc(ch, fp);
        r = aet_layer_load_weights(l, fp);
    }
    fclose(fp);
    return r;
}

// Momentum side file.  The .weights container carries no momentum buffers, so a run resumed from it differs from an
// uninterrupted one (dnn/NNetwork.c:112-147 saves only biases, scales, rolling statistics and weights).  This optional
// file holds what is missing: "AETM", int32 version = 1, uint64 seen, then per convolutional layer in layer order the
// records bias_updates[K], then for batch-norm layers scale_updates[K] and the last batch mean[K] (the next step's
// statistics are accumulated around it, so it decides their rounding), then weight_updates[K*C/groups*k*k], all FP32
// in the .weights file's element order.
extern "C" int aet_network_save_momentum(aet_network *net, const char *path) {
    if (!net || !path) { aet_set_error("null argument"); return AET_E_INVALID; }
    FILE *fp = fopen(path, "wb");
    if (!fp) { aet_set_error("cannot open %s for writing", path); return AET_E_IO; }
    const int32_t version = 1;
    const uint64_t seen = (uint64_t)net->seen;
    bool ok = fwrite("AETM", 1, 4, fp) == 4 && fwrite(&version, sizeof(version), 1, fp) == 1 && fwrite(&seen, sizeof(seen), 1, fp) == 1;
    int r = AET_OK;
    std::vector<float> v;
    for (size_t i = 0; ok && r == AET_OK && i < net->layers.size(); ++i) {
        aet_layer *l = net->layers[i];
        if (l->type != AET_CONVOLUTIONAL) continue;
        const aet_param order[4] = {AET_P_BIAS_UPDATES, AET_P_SCALE_UPDATES, AET_P_MEAN, AET_P_WEIGHT_UPDATES};
        for (int k = 0; k < 4 && ok && r == AET_OK; ++k) {
            if ((k == 1 || k == 2) && !l->bn) continue;
            v.resize(aet_layer_param_count(l, order[k]));
            r = aet_layer_read(l, order[k], v.data());
            if (r == AET_OK) ok = fwrite(v.data(), sizeof(float), v.size(), fp) == v.size();
        }
    }
    fclose(fp);
    if (!ok) { aet_set_error("momentum file: short write"); return AET_E_IO; }
    return r;
}

extern "C" int aet_network_load_momentum(aet_network *net, const char *path) {
    if (!net || !path) { aet_set_error("null argument"); return AET_E_INVALID; }
    FILE *fp = fopen(path, "rb");
    if (!fp) { aet_set_error("cannot open momentum file %s", path); return AET_E_IO; }
    char magic[4];
    int32_t version = 0;
    uint64_t seen = 0;
    if (fread(magic, 1, 4, fp) != 4 || memcmp(magic, "AETM", 4) != 0 || fread(&version, sizeof(version), 1, fp) != 1 || version != 1 ||
        fread(&seen, sizeof(seen), 1, fp) != 1) {
        fclose(fp);
        aet_set_error("momentum file %s: bad header", path);
        return AET_E_IO;
    }
    int r = AET_OK;
    std::vector<float> v;
    for (size_t i = 0; r == AET_OK && i < net->layers.size(); ++i) {
        aet_layer *l = net->layers[i];
        if (l->type != AET_CONVOLUTIONAL) continue;
        const aet_param order[4] = {AET_P_BIAS_UPDATES, AET_P_SCALE_UPDATES, AET_P_MEAN, AET_P_WEIGHT_UPDATES};
        for (int k = 0; k < 4 && r == AET_OK; ++k) {
            if ((k == 1 || k == 2) && !l->bn) continue;
            v.resize(aet_layer_param_count(l, order[k]));
            if (fread(v.data(), sizeof(float), v.size(), fp) != v.size()) { aet_set_error("momentum file: unexpected end (layer %d)", l->index); r = AET_E_IO; break; }
            r = aet_layer_write(l, order[k], v.data());
        }
    }
    fclose(fp);
    return r;
}

extern "C" int aet_network_param_hash(aet_network *net, uint64_t *hash) {
    ctx_enter(net ? net->ctx : nullptr);
    if (!net || !hash) { aet_set_error("null argument"); return AET_E_INVALID; }
    aet_context *ctx = net->ctx;
    uint64_t *dev = nullptr;
    AET_CUDA(cudaMalloc(&dev, sizeof(uint64_t)));
    AET_CUDA(cudaMemsetAsync(dev, 0, sizeof(uint64_t), ctx->stream));
    int r = k_param_hash(ctx, net->arena.W, net->arena.used, dev);
    if (r == AET_OK) r = k_param_hash(ctx, net->arena.U, net->arena.used, dev);
    if (r == AET_OK) {
        cudaError_t e = cudaMemcpyAsync(hash, dev, sizeof(uint64_t), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) { aet_set_error("param hash read-back failed: %s", cudaGetErrorString(e)); r = AET_E_CUDA; }
    }
    cudaFree(dev);
    return r;
}

// ---------------------------------------------------------------------------- profiling
extern "C" int aet_network_profile(aet_network *net, int enable) {
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    return aet_context_profile(net->ctx, enable);
}
extern "C" int aet_network_profile_read(aet_network *net, aet_kernel_time *table, int capacity, int *count) {
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    return aet_context_profile_read(net->ctx, table, capacity, count);
}

extern "C" int aet_network_launches_per_step(const aet_network *net) { return net ? (int)net->launches_per_step : 0; }

// ---------------------------------------------------------------------------- data parallel
extern "C" int aet_comm_unique_id(void *unique_id_128) {
    if (!unique_id_128) { aet_set_error("null argument"); return AET_E_INVALID; }
    NcclApi *api = nccl_api();
    if (!api) return AET_E_NCCL;
    NcclUniqueId id;
    int r = api->get_unique_id(&id);
    if (r != 0) return nccl_fail(api, r, "ncclGetUniqueId");
    memcpy(unique_id_128, &id, sizeof(id));
    return AET_OK;
}

extern "C" int aet_network_comm_init(aet_network *net, const void *unique_id_128, int rank, int world) {
    if (!net || !unique_id_128 || world < 1 || rank < 0 || rank >= world) { aet_set_error("aet_network_comm_init: bad arguments"); return AET_E_INVALID; }
    if (net->comm) { aet_set_error("communicator already initialised"); return AET_E_INVALID; }
    NcclApi *api = nccl_api();
    if (!api) return AET_E_NCCL;
    AET_CUDA(cudaSetDevice(net->ctx->device));
    NcclUniqueId id;
    memcpy(&id, unique_id_128, sizeof(id));
    void *comm = nullptr;
    // The gradient buckets are small and overlap the backward pass, whose convolution kernels are sized to one CTA
    // per SM: the collective can be capped to a few CTAs (option "nccl_max_ctas", 0 = NCCL's own choice) through this
    // communicator's configuration, which leaves the process environment and other communicators alone.
    int r = -1;
    const int max_ctas = net->ctx->opt[OPT_NCCL_MAX_CTAS];   // 0 (the default): NCCL's own choice
    if (max_ctas > 0 && api->comm_init_rank_config) {
        NcclConfig218 cfg;
        cfg.size = sizeof(cfg); cfg.magic = 0xcafebeef; cfg.version = 21800;
        cfg.blocking = INT_MIN; cfg.cgaClusterSize = INT_MIN; cfg.minCTAs = INT_MIN; cfg.maxCTAs = max_ctas;
        cfg.netName = nullptr; cfg.splitShare = INT_MIN;
        r = api->comm_init_rank_config(&comm, world, id, rank, &cfg);
        net->comm_capped = r == 0;
    }
    if (r != 0) r = api->comm_init_rank(&comm, world, id, rank);
    if (r != 0) return nccl_fail(api, r, "ncclCommInitRank");
    net->comm = comm; net->rank = rank; net->world = world;
    AET_CUDA(cudaStreamCreateWithFlags(&net->comm_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 8; ++i) AET_CUDA(cudaEventCreateWithFlags(&net->ev_grad_ready[i], cudaEventDisableTiming));
    for (int i = 0; i < 8; ++i) AET_CUDA(cudaEventCreateWithFlags(&net->ev_grad_ready_side[i], cudaEventDisableTiming));
    AET_CUDA(cudaEventCreateWithFlags(&net->ev_comm_done, cudaEventDisableTiming));
    AET_CUDA(cudaMalloc(&net->comm_stamp_dev, 4 * sizeof(unsigned long long)));
    AET_CUDA(cudaMemset(net->comm_stamp_dev, 0, 4 * sizeof(unsigned long long)));
    graph_drop(net);
    net->hyper_host[1] = -1.f;
    return AET_OK;
}

// Mean time per step the main stream waited for the gradient collectives since the last call (context option
// "comm_stamps" = 1, set before the step's graph is captured); resets the counters.
extern "C" int aet_network_comm_exposed(aet_network *net, double *mean_microseconds, long long *steps) {
    if (!net || !mean_microseconds) { aet_set_error("aet_network_comm_exposed: null argument"); return AET_E_INVALID; }
    ctx_enter(net->ctx);
    *mean_microseconds = 0.0;
    if (steps) *steps = 0;
    if (!net->comm_stamp_dev) return AET_OK;
    unsigned long long h[4] = {0, 0, 0, 0};
    AET_CUDA(cudaStreamSynchronize(net->ctx->stream));
    AET_CUDA(cudaMemcpy(h, net->comm_stamp_dev, sizeof(h), cudaMemcpyDeviceToHost));
    AET_CUDA(cudaMemset(net->comm_stamp_dev, 0, sizeof(h)));
    if (h[2]) *mean_microseconds = (double)h[1] / (double)h[2] / 1000.0;
    if (steps) *steps = (long long)h[2];
    return AET_OK;
}

// ---- peer exchange of the last gradient bucket
struct XchgBlob {            // what a rank hands to its peers (80 bytes)
    cudaIpcMemHandle_t handle;
    unsigned char uuid[16];  // ranks must sit on different GPUs: their update kernels wait for one another
};
static_assert(sizeof(XchgBlob) == 80, "exchange blob layout");

extern "C" int aet_network_comm_exchange_export(aet_network *net, void *blob_80) {
    if (!net || !blob_80) { aet_set_error("aet_network_comm_exchange_export: null argument"); return AET_E_INVALID; }
    if (!net->comm || net->world < 2 || net->world > 8) { aet_set_error("peer exchange needs an initialised communicator of 2..8 ranks"); return AET_E_INVALID; }
    AET_CUDA(cudaSetDevice(net->ctx->device));
    if (!net->xchg_local) {
        net->xchg_cap = 1024 * 1024;   // floats per parity buffer: gradient arenas up to 4 MB are exchanged whole
        {   // tuning aid (option "xchg_cap_floats"): a small value leaves only the last bucket to the exchange
            const long v = net->ctx->opt[OPT_XCHG_CAP_FLOATS];
            if (v >= 1024 && v <= 16 * 1024 * 1024) net->xchg_cap = (size_t)v / 1024 * 1024;
        }
        const size_t bytes = kXchgFlagBytes + 2 * net->xchg_cap * sizeof(float);
        AET_CUDA(cudaMalloc(&net->xchg_local, bytes));
        AET_CUDA(cudaMemset(net->xchg_local, 0, bytes));
        AET_CUDA(cudaMalloc(&net->xchg_epoch, sizeof(unsigned long long)));
        AET_CUDA(cudaMemset(net->xchg_epoch, 0, sizeof(unsigned long long)));
        AET_CUDA(cudaMalloc(&net->xchg_ticket, sizeof(unsigned int)));
        AET_CUDA(cudaMemset(net->xchg_ticket, 0, sizeof(unsigned int)));
        AET_CUDA(cudaMalloc(&net->xchg_gate, sizeof(int)));
        AET_CUDA(cudaMemset(net->xchg_gate, 0, sizeof(int)));
        AET_CUDA(cudaDeviceSynchronize());
    }
    XchgBlob b;
    memset(&b, 0, sizeof(b));
    AET_CUDA(cudaIpcGetMemHandle(&b.handle, net->xchg_local));
    cudaDeviceProp prop;
    AET_CUDA(cudaGetDeviceProperties(&prop, net->ctx->device));
    memcpy(b.uuid, &prop.uuid, 16);
    memcpy(blob_80, &b, sizeof(b));
    return AET_OK;
}

extern "C" int aet_network_comm_exchange_attach(aet_network *net, const void *blobs_world_x_80) {
    if (!net || !blobs_world_x_80 || !net->xchg_local) { aet_set_error("aet_network_comm_exchange_attach: export first"); return AET_E_INVALID; }
    if (net->adam) { aet_set_error("peer exchange refused: the Adam update takes its gradients from the collectives only"); return AET_E_INVALID; }
    const XchgBlob *b = static_cast<const XchgBlob *>(blobs_world_x_80);
    for (int p = 0; p < net->world; ++p)
        for (int q = p + 1; q < net->world; ++q)
            if (memcmp(b[p].uuid, b[q].uuid, 16) == 0) {
                aet_set_error("peer exchange refused: ranks %d and %d share a GPU (their kernels would wait for one another on one device)", p, q);
                return AET_E_INVALID;
            }
    AET_CUDA(cudaSetDevice(net->ctx->device));
    for (int q = 0; q < net->world; ++q) {
        if (q == net->rank) { net->xchg_peer[q] = net->xchg_local; continue; }
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, b[q].handle, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            aet_set_error("cudaIpcOpenMemHandle for rank %d failed: %s", q, cudaGetErrorString(e));
            cudaGetLastError();
            return AET_E_CUDA;
        }
        net->xchg_peer[q] = static_cast<unsigned char *>(ptr);
    }
    net->xchg_active = true;
    graph_drop(net);
    return AET_OK;
}

// Back to the collectives alone (the mapped buffers stay until the network is destroyed).  Every rank must take the
// same path, so a launcher whose attach failed on any rank detaches on all of them.
extern "C" int aet_network_comm_exchange_detach(aet_network *net) {
    if (!net) { aet_set_error("null network"); return AET_E_INVALID; }
    ctx_enter(net->ctx);
    if (net->xchg_active) {
        AET_CUDA(cudaStreamSynchronize(net->ctx->stream));
        net->xchg_active = false;
        graph_drop(net);
    }
    return AET_OK;
}

static void xchg_release(aet_network *net) {
    net->xchg_active = false;
    for (int q = 0; q < 16; ++q) {
        if (net->xchg_peer[q] && net->xchg_peer[q] != net->xchg_local) cudaIpcCloseMemHandle(net->xchg_peer[q]);
        net->xchg_peer[q] = nullptr;
    }
    if (net->xchg_local) { cudaFree(net->xchg_local); net->xchg_local = nullptr; }
    if (net->xchg_epoch) { cudaFree(net->xchg_epoch); net->xchg_epoch = nullptr; }
    if (net->xchg_ticket) { cudaFree(net->xchg_ticket); net->xchg_ticket = nullptr; }
    if (net->xchg_gate) { cudaFree(net->xchg_gate); net->xchg_gate = nullptr; }
}

extern "C" int aet_network_comm_destroy(aet_network *net) {
    if (!net || !net->comm) return AET_OK;
    cudaStreamSynchronize(net->ctx->stream);
    cudaStreamSynchronize(net->comm_stream);
    graph_drop(net);
    xchg_release(net);
    NcclApi *api = nccl_api();
    if (api) api->comm_destroy(net->comm);
    net->comm = nullptr; net->world = 1; net->rank = 0;
    for (int i = 0; i < 8; ++i) if (net->ev_grad_ready[i]) { cudaEventDestroy(net->ev_grad_ready[i]); net->ev_grad_ready[i] = nullptr; }
    for (int i = 0; i < 8; ++i) if (net->ev_grad_ready_side[i]) { cudaEventDestroy(net->ev_grad_ready_side[i]); net->ev_grad_ready_side[i] = nullptr; }
    if (net->ev_uploaded) { cudaEventDestroy(net->ev_uploaded); net->ev_uploaded = nullptr; }
    if (net->ev_comm_done) { cudaEventDestroy(net->ev_comm_done); net->ev_comm_done = nullptr; }
    if (net->comm_stamp_dev) { cudaFree(net->comm_stamp_dev); net->comm_stamp_dev = nullptr; }
    if (net->comm_stream) { cudaStreamDestroy(net->comm_stream); net->comm_stream = nullptr; }
    return AET_OK;
}

extern "C" int aet_network_grad_arena(aet_network *net, void **device_ptr, size_t *count) {
    if (!net || !device_ptr || !count) { aet_set_error("null argument"); return AET_E_INVALID; }
    *device_ptr = net->arena.G;
    *count = net->arena.used;
    return AET_OK;
}
