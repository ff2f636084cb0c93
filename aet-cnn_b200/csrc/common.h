// Internal definitions shared by the host-side C layer and the CUDA kernels.
//
// Device storage convention: every activation tensor is NHWC with the channel count padded
// up to a multiple of 4 (`cp`), so that each pixel row is a whole number of 16-byte cells and is
// a legal TMA / vector-load operand.  Pad channels always hold 0.  Weights use the same
// convention with (n=filters, h=w=size, c=input channels): [filter][tap][cp].
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>

#include "../../include/aet_b200.h"
#include <utility>

// bits of the device status word
#define AET_STATUS_TIMEOUT 1   // a bounded wait expired
#define AET_STATUS_NAN 2       // the update found (and scrubbed) non-finite values
constexpr int kPinnedFloats = 16 + 8 * 8;
constexpr int kHyperSlots = 8;

void aet_set_error(const char *fmt, ...);

#define AET_CUDA(call)                                                                              \
    do {                                                                                            \
        cudaError_t e__ = (call);                                                                   \
        if (e__ != cudaSuccess) {                                                                   \
            aet_set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
            return AET_E_CUDA;                                                                      \
        }                                                                                           \
    } while (0)

#define AET_TRY(call)                  \
    do {                               \
        int r__ = (call);              \
        if (r__ != AET_OK) return r__; \
    } while (0)

static inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
static inline size_t round_up_sz(size_t v, size_t m) { return (v + m - 1) / m * m; }

// Device-side duration of a profiled launch: the kernels that support it record the earliest entry and the latest
// exit of their CTAs (%globaltimer) in a slot of this array, so that the table can show, beside the event-bracketed
// time of a launch, how long its CTAs were actually on the machine.
constexpr int kMaxSpanSlots = 4096;
struct ProfileRecord {
    int span_slot;        // index into the context's span array, or -1
    char name[40];        // kernel label, with ".variant" appended when the launcher chose among code paths
    int tag;              // index of the network layer the launch belongs to, or -1
    double bytes, flops;
    cudaEvent_t e0, e1;
};

// Behaviour switches of a context (kernel choice, fusions, overlap).  Each has a name for
// aet_context_set_option and an environment variable that is read ONCE, when the context is created, and only
// supplies the initial value; nothing on a launch path reads the environment.
enum AetOption {
    OPT_ROWS = 0,          // row-sharing TMA kernels                         AET_NO_ROWS
    OPT_ROWS_FPROP,        //   ... for the forward pass (off: the plain TMA kernel measures faster there)   AET_ROWS_F
    OPT_ROWS_DGRAD,        //   ... for the data gradient                     AET_NO_ROWS_D
    OPT_SMERGE,            // column taps merged into the MMA's N (narrow data gradients)   AET_NO_SMERGE
    OPT_KSPLIT,            // K range split over a two-CTA cluster            AET_NO_KSPLIT
    OPT_MT2,               // two pixel tiles per CTA                         AET_NO_MT2
    OPT_ROWS_MULTI,        // allow the row-sharing kernels more than one wave    AET_ROWS_MULTI
    OPT_PAR_EPILOGUE,      // second epilogue warp group                      AET_NO_PAR_EPILOGUE
    OPT_FC_ALIAS,          // whole-map filters run as 1x1 convolutions       AET_NO_FC_ALIAS
    OPT_EPILOGUE_STATS,    // batch-norm statistics gathered by the convolution's epilogue   AET_NO_EPILOGUE_STATS
    OPT_THIN,              // persistent first-layer kernels                  AET_NO_THIN
    OPT_OVERLAP_WGRAD,     // weight-gradient kernels on a second stream      AET_NO_OVERLAP
    OPT_WGRAD_SPLITS,      // forced K-split count of the row-sharing weight gradient (0 = automatic)   AET_WGRAD_SPLITS
    OPT_BN_TILE,           // forced N tile of the gather / plain TMA kernels (0 = automatic)           AET_BN
    OPT_FUSE,              // network-level fusions (BN + pool, classifier head), read when a network is built   AET_NO_FUSE
    OPT_LINEAR_HEAD,       // classifier head on the pooled vectors, read when a network is built          AET_NO_LINEAR_HEAD
    OPT_XCHG_CAP_FLOATS,   // capacity of the peer-exchange buffer (0 = default)   AET_XCHG_CAP_FLOATS
    OPT_NCCL_MAX_CTAS,     // CTA cap of the gradient all-reduce's communicator (0 = NCCL's choice)   AET_NCCL_MAX_CTAS
    OPT_DUAL_ACC,          // two accumulators per tile when a CTA owns one tile (row-sharing kernels; off by default)   AET_DUAL_ACC
    OPT_ROTATE,            // CTAs start their K loops at different slabs (row-sharing kernels)   AET_NO_ROTATE
    OPT_STEM,              // first convolution + BN + 2x2 max-pool: weight gradient from the pool-sized tensors   AET_NO_STEM
    OPT_COMM_STAMPS,       // time the main stream's wait for the gradient collectives (aet_network_comm_exposed)   AET_COMM_STAMPS
    OPT_MERGE_TAIL,        // a small last gradient bucket rides with the one before it   AET_NO_MERGE_TAIL
    OPT_RAGGED,            // TMA kernels on maps whose rows do not divide the tile (13x13, 27x27)   AET_NO_RAGGED
    OPT_PAIR,              // CTA pairs sharing the weight tiles (cta_group::2 MMAs) in the row-sharing kernels; off by default   AET_PAIR
    OPT_S2D,               // large strided first-layer filters regrouped into stride-1 convolutions                AET_NO_S2D
    OPT_FD_SPLIT,          // forward / data gradient of layers with few tiles and a long K loop split over the grid   AET_NO_FD_SPLIT
    OPT_COUNT
};

struct aet_context {
    int device = 0;
    int opt[OPT_COUNT] = {0};
    std::vector<const void *> smem_attr_done;   // kernels whose dynamic shared-memory limit was raised on this device
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    aet_parity_mode parity = AET_PARITY_MTCS;
    aet_math_mode math = AET_MATH_TF32;
    int conv_path = 0;  // 0 auto (TMA where the shape allows), 1 force gather producer
    // staging buffer for NCHW <-> NHWC host taps
    float *staging = nullptr;
    size_t staging_bytes = 0;
    float *pinned = nullptr;  // pinned host mirror used by async uploads
    size_t pinned_bytes = 0;
    // scratch arena (split-K partials, reduction partials)
    float *scratch = nullptr;
    size_t scratch_bytes = 0;
    int *status_dev = nullptr;  // device status word written by bounded waits
    // Second stream of a network's backward pass: the weight-gradient kernels of a layer run there,
    // beside the data-gradient chain on `stream`, with their own scratch arena.  side_begin() forks it
    // from `stream` and makes it the launch stream; side_end() restores `stream`; side_join() makes
    // `stream` wait for everything queued on it.
    cudaStream_t side_stream = nullptr, main_stream_saved = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    bool overlap_wgrad = false;   // set by the network around its backward pass
    bool wgrad_fresh = false;     // set by a training step without subdivisions: the gradient arena is zero when backward starts, the weight gradients may overwrite
    bool on_side = false, side_pending = false;
    int resident_bn_reduce = 0, resident_bn_apply = 0;   // resident blocks per SM of the window-major BN backward kernels (queried once)
    float *scratch_side = nullptr;
    size_t scratch_side_bytes = 0;
    // profiling
    bool profiling = false;
    unsigned long long *span_dev = nullptr;   // [kMaxSpanSlots][2]: first CTA entry, last CTA exit (ns)
    unsigned long long *span_ptr = nullptr;   // slot of the launch being issued (null: not profiling / table full)
    std::vector<ProfileRecord> records;
    std::vector<cudaEvent_t> event_pool;
    size_t event_next = 0;
    long launches = 0;
    int prof_tag = -1;    // layer index stamped on profile records ("name#index" in the table)
    bool in_network_pass = false;   // set by the network around its forward/backward loops (enables call-pattern fusions)
    bool capturing = false;
};

struct aet_tensor {
    aet_context *ctx = nullptr;
    int n = 0, c = 0, h = 0, w = 0, cp = 0;
    float *d = nullptr;
    bool owns = true;
    // Logically all-zero without having been cleared: the next writer overwrites instead of
    // accumulating, and host reads return zeros.  Lets the network skip one memset per layer.
    bool lazy_zero = false;
    size_t count() const { return (size_t)n * c * h * w; }
    size_t elems() const { return (size_t)n * h * w * cp; }  // device floats
    size_t pixels() const { return (size_t)n * h * w; }
};

// One contiguous run of parameters inside the arena, a multiple of 1024 floats long.
struct ParamSegment {
    size_t offset = 0, count = 0, padded = 0;
};

struct ParamArena {
    float *W = nullptr, *U = nullptr, *G = nullptr;  // values, momentum, per-step gradient
    float *M = nullptr, *V = nullptr;                // Adam's first and second moments (allocated for adam=1 networks)
    size_t capacity = 0, used = 0;
    bool owns = false;
};

struct aet_layer {
    aet_context *ctx = nullptr;
    aet_network *net = nullptr;
    aet_layer_type type = AET_CONVOLUTIONAL;
    int index = 0;
    int batch = 0, c = 0, h = 0, w = 0, cp = 0;         // input
    int oc = 0, oh = 0, ow = 0, ocp = 0;                // output
    int size = 1, stride_x = 1, stride_y = 1, pad = 0;  // conv / pool (pool: pad = padding)
    int dilation = 1;                                   // conv: tap spacing (`groups`, below, is a convolution's channel groups too:
                                                        // dnn/ConvolutionalLayer.c:716-722)
    int cg = 0, cgp = 0;                                // conv: input channels of one group and their padded count
    int bn = 0, train = 1;
    int flipped = 0;      // the weights record of a .weights file is stored transposed (dnn/ConvolutionalLayer.c:483-485)
    aet_activation act = AET_LINEAR;
    float lr_scale = 1.0f;
    // generic per-layer cfg keys (dnn/NetworkFactory.c:926-934): stopbackward ends the network's backward walk before this
    // layer (dnn/NNetwork.c:648); the layers in front of the last such layer only run forward and are never updated
    // (dnn/NetworkFactory.c:979-991: onlyforward = 1, train = 0); dont_update = N skips the update while the iteration
    // number is <= N (dnn/NNetwork.c:703, the GPU path only); dontload skips the layer's record of a .weights file
    // (dnn/NNetwork.c:95), dontloadscales its batch-norm block (dnn/ConvolutionalLayer.c:468)
    int stopbackward = 0, onlyforward = 0, dont_update = 0, dontload = 0, dontloadscales = 0;
    aet_tensor *output = nullptr, *delta = nullptr, *x = nullptr;  // x: conv result before BN
    // parameters (slices of an arena)
    ParamArena *arena = nullptr;
    ParamArena own_arena;
    ParamSegment seg_w, seg_b, seg_s;
    float *mean = nullptr, *variance = nullptr, *rolling_mean = nullptr, *rolling_variance = nullptr;
    float *inv_std = nullptr;            // per-channel 1/std in the parity mode's form
    float *bwd_coef = nullptr;           // [3][ocp] coefficients of the BN backward apply pass
    float *shift = nullptr;              // BN statistics shift (first pixel of each channel)
    // pooling
    int *indexes = nullptr;
    // softmax
    int groups = 1;
    float temperature = 1.0f;
    float *loss = nullptr, *sample_loss = nullptr, *cost_dev = nullptr;
    float *cost_base = nullptr;   // two {cost, mean loss} records, one per input slot of the asynchronous step; cost_dev points at the one in use
    float cost_host = 0.0f;
    bool cost_valid = false;
    // dropout
    float probability = 0.0f;
    float *rnd = nullptr;
    bool rnd_fixed = false;  // uniforms were supplied by the caller; forward does not regenerate
    aet_layer *prev = nullptr;
    uint64_t seed = 0;
    unsigned long long *step_dev = nullptr;
    // Network-level fusion: a BN convolution followed by a max-pool computes the pool's output in
    // its own forward and gathers the pool's delta in its own backward; the pool layer then idles.
    aet_layer *fused_pool = nullptr;   // set on the convolution
    aet_layer *fused_into = nullptr;   // set on the max-pool
    bool output_stale = false;         // conv output not materialised (recomputed on a host read)
    bool last_forward_train = true;
    bool fused_ready = false;          // pool: output already produced by the convolution this pass
    bool gather_pending = false;       // conv: the pool deferred its backward to this layer
    // Network-level fusion of the classifier head conv(linear) -> avgpool -> softmax (<= 32 classes)
    aet_layer *head_conv = nullptr, *head_avg = nullptr;   // set on the softmax layer
    aet_layer *head_softmax = nullptr;                     // set on the avg-pool and the convolution
    // Linear head (1x1 convolution folded into the pooled vectors; network training passes only), on the convolution:
    bool lin_head = false;           // eligible (set when the network is wired)
    bool lin_fwd_pending = false;    // forward deferred to the softmax layer's call
    bool lin_used = false;           // the last forward went through the fused kernel
    bool lin_out_stale = false;      // output tensor not formed (a host tap runs the convolution)
    bool lin_bwd_pending = false;    // softmax/avg-pool backward deferred to this layer's backward call
    bool lin_delta_stale = false;    // delta tensor not formed (a host tap broadcasts it)
    aet_tensor *lin_input = nullptr; // input of the deferred forward
    float *lin_xbar = nullptr;       // [batch][cp] pooled input
    unsigned int *lin_ticket = nullptr;
    bool head_forward_pending = false;  // avg-pool: forward deferred to the softmax layer's fused kernel
    bool head_backward_done = false;    // avg-pool / conv: delta (and bias gradient) already produced
    // First convolution of an image network with BN and a fused 2x2 max-pool (network training passes): the weight
    // gradient is formed from the pool-sized tensors and the Gram matrix of the input patches; the full-resolution
    // delta is never written.
    bool stem = false;               // eligible (set when the network is wired)
    bool stem_gram_ready = false;    // this pass's Gram matrix is queued (on the side stream when the pass overlaps)
    bool stem_delta_stale = false;   // delta tensor not formed (a host tap runs the BN backward apply pass)
    float *stem_ymax = nullptr;      // [batch][pool oh][pool ow][ocp] convolution result at each window's argmax
    unsigned char *stem_code = nullptr;   // same shape: the argmax's position inside its window (0..3 row-major, 4: none)
    int stem_resident = 0;           // resident blocks per SM of the pool-sized pass (queried once)
    float *stem_partial = nullptr;   // per block: BN sums [2][ocp], then first-term sums [ocp][36]
    float *stem_gram_partial = nullptr;   // per-block Gram sums [blocks][81][16]
    double *stem_gram = nullptr;          // Gram sums over the batch [81][16]
    int stem_blocks = 0, stem_blocks_used = 0, stem_gram_blocks = 0;
    // shortcut: the layers whose outputs are added to the input
    aet_layer *from[4] = {nullptr, nullptr, nullptr, nullptr};
    int n_from = 0;
    // TMA descriptors are built lazily per (layer, pass, operand address)
    void *tma_cache = nullptr;
    // large strided first-layer filter run as a stride-1 convolution over a regrouped input (conv_s2d.cuh)
    aet_layer *s2d = nullptr;        // the regrouped layer: geometry, regrouped weights and their gradient
    float *s2d_x = nullptr;          // the regrouped input
    const float *s2d_src = nullptr;  // which input s2d_x was last made from
};

struct aet_network {
    aet_context *ctx = nullptr;
    std::vector<aet_layer *> layers;
    int batch = 1, subdivisions = 1, c = 0, h = 0, w = 0, train = 1;
    float learning_rate = 0.001f, momentum = 0.9f, decay = 0.0001f;
    int policy = 0;  // 0 constant 1 step 2 steps 3 exp 4 poly 5 sig
    int burn_in = 0, max_batches = 0, step = 1, num_steps = 0;
    float power = 4.0f, gamma = 1.0f, scale = 1.0f;
    std::vector<int> steps;
    std::vector<float> scales;
    int64_t seen = 0, cur_iteration = 0;
    bool grad_clean = true;          // the gradient arena is all zero (creation, or an update ran last)
    bool graph_clean[4] = {true, true, true, true};   // ... as it was when each step graph was captured
    bool bn_fused = false;   // fuseConvBatchnorm ran: inference only from here on
    float loss_scale = 1.0f;
    int try_fix_nan = 0;
    aet_tensor *input = nullptr, *truth = nullptr;
    ParamArena arena;
    // SGD launch tables
    int *block_seg = nullptr;    // per 1024-float block: segment id
    float *seg_table = nullptr;  // per segment: lr multiplier (negative: the segment is not updated now), decay flag, ...
    std::vector<float> seg_host;         // host copy of seg_table with the layers' own multipliers
    std::vector<aet_layer *> seg_layer;  // owner of each segment
    std::vector<unsigned char> seg_skip; // which segments the device table currently marks as not updated
    int n_blocks = 0, n_segments = 0;
    float *hyper_dev = nullptr;  // {lr/B, momentum, -decay*B*loss_scale, unused, then for Adam: rate, -decay*B, 1-B1^t, 1-B2^t}
    float hyper_host[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int adam = 0;                // [net] adam=1: Adam instead of SGD with momentum (mtcs/MtcsConvLayer.c:494-524,600-612)
    float B1 = .9f, B2 = .999f, eps = .000001f;
    // Pinned host block (kPinnedFloats floats): [0..3] cost, mean loss, status word of a synchronous loss read;
    // [8..15] the same triple for each of the two slots of the asynchronous step; [16..] a ring of kHyperSlots
    // staged hyper-parameter quadruples (one per change of the learning rate, each with its own event).
    float *loss_pinned = nullptr;
    cudaEvent_t hyper_ev[8] = {nullptr};
    bool hyper_used[8] = {false};
    int hyper_next = 0;
    // CUDA graphs of one train step: [1] forward + backward + exchange + update, [0] forward + backward only
    // (the calls of a `subdivisions` group that only accumulate gradients)
    bool use_graph = false;
    // and each of them once per input slot (the asynchronous step alternates between two input / truth tensors)
    cudaGraphExec_t graph_exec[4] = {nullptr, nullptr, nullptr, nullptr};
    long graph_launches[4] = {0, 0, 0, 0};
    int cur_slot = 0;                                          // input slot of the step being queued
    aet_tensor *input_alt = nullptr, *truth_alt = nullptr;     // slot 1 (slot 0 = `input`, `truth`)
    int eager_runs[2] = {0, 0};
    // Double-buffered input staging of aet_network_train_step_async: the host->device copy of step s+1 runs on
    // `copy_stream` while step s computes; `ev_staged` orders the step after its copy, `ev_consumed` orders the
    // next copy into a slot after the transposing kernels that read it, `ev_loss` marks a step's loss read-back.
    cudaStream_t copy_stream = nullptr, loss_stream = nullptr;
    float *stage_dev[2] = {nullptr, nullptr};
    float *stage_host[2] = {nullptr, nullptr};   // pinned mirrors, used when the caller's buffers are pageable
    size_t stage_floats = 0;
    cudaEvent_t ev_staged[2] = {nullptr, nullptr}, ev_consumed[2] = {nullptr, nullptr}, ev_loss[2] = {nullptr, nullptr};
    uint64_t async_steps = 0;
    int update_batch_world = 0;  // batch * world for data parallel
    // data parallel
    void *comm = nullptr;
    bool comm_capped = false;   // the communicator took the CTA cap
    int rank = 0, world = 1;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_grad_ready[8] = {nullptr}, ev_grad_ready_side[8] = {nullptr}, ev_comm_done = nullptr;
    // Peer exchange of the last gradient bucket (the first layers' gradients, ready only at the very end
    // of backward, where a collective's latency would be fully exposed): every rank publishes its slice
    // in a buffer its peers have mapped, and the update kernel sums the ranks' slices itself.
    bool xchg_active = false;
    unsigned char *xchg_local = nullptr;        // [2][16] u64 flags, then two parity buffers of xchg_cap floats
    unsigned char *xchg_peer[16] = {nullptr};   // the same region of every rank (own entry = xchg_local)
    size_t xchg_cap = 0;
    unsigned long long *xchg_epoch = nullptr;   // device-side step counter
    unsigned int *xchg_ticket = nullptr;        // blocks of the publish kernel that have finished
    unsigned long long *comm_stamp_dev = nullptr;   // {last stamp, summed wait in ns, waits counted, unused}
    bool comm_stamped = false;                  // this step's backward already bracketed a wait for collectives
    int *xchg_gate = nullptr;                   // 1 / 0: this step's slices of all ranks arrived / the wait ran out
    size_t tail_lo = 0, tail_n = 0;             // arena range summed through the exchange this step (0: none)
    cudaEvent_t ev_uploaded = nullptr;   // after the H2D copies of a train step fed from the caller's pinned buffers
    long launches_per_step = 0;
};

// ---- launch bookkeeping -----------------------------------------------------------------
void prof_begin(aet_context *ctx, const char *name, double bytes, double flops, const char *variant = nullptr);
void prof_end(aet_context *ctx);
struct LaunchScope {
    aet_context *ctx;
    // `variant` names the code path a launcher picked (tile shape, split, epilogue form); it is appended to the
    // label as "name.variant" so that a test can assert which path it exercised.
    LaunchScope(aet_context *c, const char *name, double bytes, double flops, const char *variant = nullptr) : ctx(c) {
        ctx->launches++;
        if (ctx->profiling) prof_begin(ctx, name, bytes, flops, variant);
    }
    ~LaunchScope() {
        if (ctx->profiling) prof_end(ctx);
        ctx->span_ptr = nullptr;
    }
};
int aet_check_launch(const char *what);

// Every kernel of the library is launched with programmatic stream serialization: its CTAs may be
// scheduled (and run their prologue: barrier setup, TMEM allocation, descriptor prefetch) while the
// previous kernel of the stream drains.  The contract each kernel keeps: no global-memory access
// before pdl_wait(), which returns once every earlier kernel of the stream has completed and its
// writes are visible.  pdl_trigger() after the wait lets the next kernel start scheduling, so at
// most one kernel waits behind the running one.  AET_NO_PDL=1 in the environment launches plainly.
bool pdl_enabled();
void pdl_skip_next();   // the next launch_k on this thread is a plain launch (after a cross-stream event wait)
bool pdl_take_skip();
template <typename... KArgs, typename... Args>
inline void launch_k(cudaStream_t stream, dim3 grid, dim3 block, size_t smem, void (*kernel)(KArgs...), Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl_enabled() && !pdl_take_skip()) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);   // errors surface in aet_check_launch
}
// The same with a thread-block cluster of `cluster_x` x 1 x `cluster_z` CTAs: along z the CTAs that split one
// tile's K range (distributed shared memory), along x the CTA pair that shares its B tiles (cta_group::2 MMAs).
template <typename... KArgs, typename... Args>
inline void launch_k_cluster(cudaStream_t stream, dim3 grid, dim3 block, size_t smem, int cluster_x, int cluster_z,
                             void (*kernel)(KArgs...), Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)cluster_z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl_enabled() && !pdl_take_skip()) ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#ifdef __CUDACC__
// first CTA entry / last CTA exit of a profiled launch (see kMaxSpanSlots); one thread per CTA, two atomics in all
__device__ __forceinline__ void span_begin(unsigned long long *span) {
    if (span && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        atomicMin(span, t);
    }
}
__device__ __forceinline__ void span_end(unsigned long long *span) {
    if (span && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        atomicMax(span + 1, t);
    }
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// the usual kernel opening: wait for the stream's earlier kernels, then let the next one schedule
__device__ __forceinline__ void pdl_enter() { pdl_wait(); pdl_trigger(); }
#endif
int ctx_scratch(aet_context *ctx, size_t bytes, float **out);
// Raises a kernel's dynamic shared-memory limit once per context (the attribute is per device, and a context is
// one device; a process-wide flag would leave a second device's kernels at the 48 KB default).
int ctx_smem_attr_impl(aet_context *ctx, const void *func, int bytes);
template <typename F>
inline int ctx_smem_attr(aet_context *ctx, F *func, int bytes = 220 * 1024) {
    return ctx_smem_attr_impl(ctx, reinterpret_cast<const void *>(func), bytes);
}
int side_begin(aet_context *ctx);
void side_end(aet_context *ctx);
int side_join(aet_context *ctx);
// Entry points make their context's device the calling thread's current one: a process may hold contexts on several
// GPUs (or another library may have switched the device), and allocations and launches follow the current device.
static inline void ctx_enter(const aet_context *ctx) {
    int d = -1;
    if (ctx && cudaGetDevice(&d) == cudaSuccess && d != ctx->device) cudaSetDevice(ctx->device);
}
int ctx_staging(aet_context *ctx, size_t bytes);

// ---- layout taps (tensor.cu) ------------------------------------------------------------------
int tensor_upload_nchw(aet_context *ctx, float *dev_nhwc, const float *host, int n, int c, int h, int w, int cp,
                       bool async_pinned);
int tensor_upload_staged(aet_context *ctx, float *dev_nhwc, const float *dev_nchw, int n, int c, int h, int w, int cp,
                         cudaStream_t stream = nullptr);   // stream: null = the context's
int tensor_download_nchw(aet_context *ctx, const float *dev_nhwc, float *host, int n, int c, int h, int w, int cp);
int tensor_download_nchw_int(aet_context *ctx, const int *dev_nhwc, int *host, int n, int c, int h, int w, int cp);
int vector_upload(aet_context *ctx, float *dev, const float *host, size_t count);
int vector_download(aet_context *ctx, const float *dev, float *host, size_t count);

// ---- kernels (launchers return AET_OK or an error) ----------------------------------------------
struct ConvGeom {
    int N, C, H, W, cp;      // input activation (C, cp: the channels one GEMM sees -- one group's)
    int K, OH, OW, kp;       // output activation (K, kp: one group's filters)
    int R, S, sy, sx, pad;
    int xs, ys;              // floats between consecutive pixels of the input / output tensors (the whole layer's padded
                             // channel counts; equal to cp / kp unless the layer has channel groups)
    int dil;                 // spacing of the filter taps; the padding in pixels is pad * dil (dnn/Im2Col.c:65-103)
};
// Batch-norm statistics gathered by the forward epilogue: in `shift` (per-channel, near the data);
// out `partial` (scratch arena, rows x [2][ocp]: sum and sum of squares of y - shift) and `rows`
// (0 when the launch could not gather them: bias or activation in the epilogue, 3xTF32).
struct ConvStats {
    const float *shift;
    float *partial;
    int rows;
};
int conv_fprop(aet_layer *l, const float *x, float *y, const float *bias, int act_in_epilogue, ConvStats *stats = nullptr);
int conv_dgrad(aet_layer *l, const float *dy, float *dx);
int conv_wgrad(aet_layer *l, const float *x, const float *dy, float *dw, int accumulate);
void conv_release(aet_layer *l);

int k_bn_stats(aet_layer *l, int update_rolling, const ConvStats *from_epilogue = nullptr);
int k_bn_apply(aet_layer *l, int use_rolling);
int k_bn_backward(aet_layer *l, aet_layer *pool);
int k_bn_pool_forward(aet_layer *l, aet_layer *pool, int use_rolling);
int k_shortcut_forward(aet_layer *l, const float *in);
int k_shortcut_backward(aet_layer *l, aet_tensor *pd);
int k_comm_stamp(aet_context *ctx, unsigned long long *dev4, int after);
bool stem_backward_eligible(const aet_layer *l, const aet_layer *pool);
int stem_alloc(aet_layer *l, aet_layer *pool);
int k_stem_gram(aet_layer *l, const float *x_in);
int k_stem_backward(aet_layer *l, aet_layer *pool, const float *x_in);
int k_stem_finish(aet_layer *l, float *dw, int accumulate);
int k_stem_delta(aet_layer *l, aet_layer *pool);
int k_bias_act_backward(aet_layer *l);
int k_maxpool_forward(aet_layer *l, const float *x);
int k_maxpool_backward(aet_layer *l, float *prev_delta, int accumulate);
int k_avgpool_forward(aet_layer *l, const float *x);
int k_avgpool_backward(aet_layer *l, float *prev_delta, int accumulate);
int k_softmax_forward(aet_layer *l, const float *x, const float *truth);
int k_head_forward(aet_layer *conv, aet_layer *avg, aet_layer *sm, const float *truth);
int k_head_backward(aet_layer *conv, aet_layer *avg, aet_layer *sm);
int k_linhead_forward(aet_layer *conv, aet_layer *avg, aet_layer *sm, const float *x, const float *truth);
int k_linhead_backward(aet_layer *conv, aet_layer *avg, aet_layer *sm, float *pd);
int k_linhead_conv_delta(aet_layer *conv, aet_layer *avg, aet_layer *sm);
int k_axpy(aet_context *ctx, float *y, const float *x, float a, size_t n, int accumulate, const char *name);
int k_dropout_forward(aet_layer *l, float *x, int generate);
int k_dropout_backward(aet_layer *l, float *delta);
int k_fill(aet_context *ctx, float *p, float v, size_t n);
int k_step_counter(aet_context *ctx, unsigned long long *ctr);
int k_sgd_segment(aet_context *ctx, float *W, float *U, float *G, size_t count, float lr_over_b, float momentum,
                  float decay_term, int scrub);   // scrub: 0 none, 1 weights, 2 batch-norm bias / scale with try_fix_nan
int k_sgd_arena(aet_network *net);
int k_adam_arena(aet_network *net);
int conv_set_wait_limit(unsigned long long ns);          // conv.cu: limit of the mbarrier waits of the convolution kernels
int elementwise_set_wait_limit(unsigned long long ns);   // elementwise.cu: limit of the peer-flag wait of the update kernel
int conv_wait_probe(aet_context *ctx);                   // conv.cu: a wait nobody satisfies (self-test of the bounded waits)
int k_tail_publish(aet_network *net);
constexpr size_t kXchgFlagBytes = 1024;   // 2 x 16 u64 flags, padded
int k_param_hash(aet_context *ctx, const float *p, size_t count, uint64_t *hash_dev);
int k_augment(aet_context *ctx, const float *src_nchw, int n, int c, int sh, int sw, float *dst_nhwc, int size, int cp,
              const aet_augment *params_dev);
int k_top_k(aet_context *ctx, const float *scores, int samples, int n, int ld, int k, int *index_dev);

// parameter pointers
static inline float *layer_W(aet_layer *l) { return l->arena->W + l->seg_w.offset; }
static inline float *layer_U(aet_layer *l) { return l->arena->U + l->seg_w.offset; }
static inline float *layer_G(aet_layer *l) { return l->arena->G + l->seg_w.offset; }
static inline float *layer_b(aet_layer *l) { return l->arena->W + l->seg_b.offset; }
static inline float *layer_bU(aet_layer *l) { return l->arena->U + l->seg_b.offset; }
static inline float *layer_bG(aet_layer *l) { return l->arena->G + l->seg_b.offset; }
static inline float *layer_s(aet_layer *l) { return l->arena->W + l->seg_s.offset; }
static inline float *layer_sU(aet_layer *l) { return l->arena->U + l->seg_s.offset; }
static inline float *layer_sG(aet_layer *l) { return l->arena->G + l->seg_s.offset; }
