/*
 * aet_b200.h -- C ABI of the B200-native replacement for the AET-CNN training hot path.
 *
 * Every entry point replaces one seam of the reference (paths are inside the reference
 * project; dnn/ = src/com/ai/dnn/, mtcs/ = src/com/ai/dnn/mtcs/).  The reference selects its
 * back end by subclassing: mtcs/MtcsConvLayer.h:20, mtcs/MtcsIOData.h:12 override the CPU
 * classes' virtual forward/backward/update (dnn/NLayer.h:159-166).  This header restates that
 * seam as plain C: opaque handles, plain pointers and sizes, int status codes.
 *
 * Conventions
 *   - Host-visible tensor layout is the reference's: FP32, NCHW, contiguous
 *     (dnn/NData.h:14-68).  Device storage is private (NHWC, channel-padded to 4).
 *   - Every function returning int returns AET_OK (0) or a negative AET_E_* code; the
 *     message is available from aet_last_error().  Nothing aborts the process and no device
 *     code traps: device-side waits are bounded and report through the status code.
 *   - One host thread drives one context (as in the reference: mtcs/MtcsTool.c:22-30).
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails with
 *     AET_E_CUDA.
 */
#ifndef AET_B200_H
#define AET_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AET_OK            0
#define AET_E_INVALID   (-1)   /* bad argument / unsupported configuration */
#define AET_E_CUDA      (-2)   /* CUDA runtime or driver error */
#define AET_E_NOMEM     (-3)
#define AET_E_IO        (-4)   /* cfg or weights file */
#define AET_E_TIMEOUT   (-5)   /* a bounded device-side wait expired */
#define AET_E_NCCL      (-6)
#define AET_E_NAN       (-7)   /* non-finite values detected (try_fix_nan diagnostics) */

/* dnn/Activation.h:15-19.  The first fourteen have gradients that are functions of the OUTPUT (dnn/Activation.h:41-113);
 * the first three are the hot path's; cfg names are the reference's ("logistic", "relu6", "relie", "ramp", "tanh",
 * "plse", "elu", "loggy", "hardtan", "lhtan", "selu").  swish and mish (dnn/IOData.c:75-105, dnn/Activation.c:303-330)
 * need the value BEFORE the activation for their gradient: they are taken by batch-normalised convolutions, whose
 * backward kernels recompute that value from the stored convolution result; other layers reject them.  stair, gelu,
 * hard_mish and the channel normalisations are not built. */
typedef enum { AET_LINEAR = 0, AET_RELU = 1, AET_LEAKY = 2, AET_LOGISTIC = 3, AET_RELU6 = 4, AET_RELIE = 5, AET_RAMP = 6,
               AET_TANH = 7, AET_PLSE = 8, AET_ELU = 9, AET_LOGGY = 10, AET_HARDTAN = 11, AET_LHTAN = 12, AET_SELU = 13,
               AET_SWISH = 14, AET_MISH = 15 } aet_activation;
#define AET_ACTIVATION_COUNT 16
/* dnn/NLayer.c:30-60 layer kinds that NetworkFactory.createLayer instantiates on the hot path */
typedef enum { AET_CONVOLUTIONAL = 0, AET_MAXPOOL = 1, AET_AVGPOOL = 2, AET_SOFTMAX = 3, AET_DROPOUT = 4, AET_SHORTCUT = 5 } aet_layer_type;
/* Which of the reference's two numerically different back ends the formulas follow:
 * the CPU classes (dnn/NormData.c, dnn/DeltaData.c, ...) or the MTCS kernels (mtcs/...). */
typedef enum { AET_PARITY_CPU = 0, AET_PARITY_MTCS = 1 } aet_parity_mode;
/* Tensor-core input precision of the implicit-GEMM kernels (accumulation is always FP32). */
typedef enum { AET_MATH_TF32 = 0, AET_MATH_3XTF32 = 1 } aet_math_mode;

/* Parameter / buffer selectors for aet_layer_read / aet_layer_write. */
typedef enum {
    AET_P_WEIGHTS = 0,       /* [n][c][size][size]   dnn/WeightData.h:24-82 */
    AET_P_WEIGHT_UPDATES,    /* same shape; momentum buffer plus pending gradient */
    AET_P_BIASES,            /* [n]                  dnn/BiasData.h */
    AET_P_BIAS_UPDATES,
    AET_P_SCALES,            /* [n] BN gamma         dnn/ScaleData.h */
    AET_P_SCALE_UPDATES,
    AET_P_ROLLING_MEAN,      /* dnn/NormData.h:20-40 */
    AET_P_ROLLING_VARIANCE,
    AET_P_MEAN,
    AET_P_VARIANCE,
    AET_P_OUTPUT,            /* layer output  [batch][c][h][w]; for a BN convolution followed by a max-pool inside a
                              * network it is formed on demand from the saved convolution result with the layer's
                              * current scale / shift: read it before the next update */
    AET_P_DELTA,             /* layer delta   [batch][c][h][w] */
    AET_P_X,                 /* BN input saved by normalize (dnn/NormData.c:244-282) */
    AET_P_X_NORM,            /* recomputed on read: (x-mean)*inv_std */
    AET_P_INDEXES,           /* max-pool argmax, int32, reference numbering (dnn/MaxPoolLayer.c:250-270) */
    AET_P_LOSS,              /* per-element cross entropy (dnn/SoftMaxLayer.c:47-55) */
    AET_P_RAND               /* dropout uniforms (dnn/DropoutLayer.c:55-70) */
} aet_param;

typedef struct aet_context aet_context;
typedef struct aet_tensor  aet_tensor;    /* NData / IOData / DeltaData / TruthData */
typedef struct aet_layer   aet_layer;     /* NLayer and subclasses */
typedef struct aet_network aet_network;   /* NNetwork */

/* dnn/NLayer.h:21-29 NetworkState, passed by value exactly like the reference does. */
typedef struct aet_state {
    aet_tensor *truth;
    aet_tensor *input;
    aet_tensor *delta;      /* previous layer's delta; NULL for the first layer */
    float      *workspace;  /* device scratch; NULL lets the layer use the context's */
    int         train;
    int         index;
} aet_state;

/* ------------------------------------------------------------------ context
 * Replaces the MtcsTool / MtcsStream / MtcsMem singletons (call sites mtcs/MtcsTool.c:22-30,
 * mtcs/MtcsIOData.c:21,47-51).  One context = one device + one stream + one scratch arena. */
const char  *aet_last_error(void);
const char  *aet_version(void);
aet_context *aet_context_create(int device);
void         aet_context_destroy(aet_context *ctx);
/* Use an externally owned cudaStream_t (NULL = a stream the context creates itself). */
int          aet_context_set_stream(aet_context *ctx, void *cuda_stream);
void        *aet_context_stream(aet_context *ctx);
int          aet_context_set_parity(aet_context *ctx, aet_parity_mode mode);
int          aet_context_set_math(aet_context *ctx, aet_math_mode mode);
int          aet_context_synchronize(aet_context *ctx);
/* Behaviour switches (kernel choice, fusions, stream overlap), by name: "rows", "rows_fprop", "rows_dgrad",
 * "smerge", "ksplit", "mt2", "rows_multi", "par_epilogue", "fc_alias", "epilogue_stats", "thin", "pair", "rotate", "dual_acc",
 * "overlap_wgrad", "wgrad_splits", "bn_tile", "gather_only" (take effect at the next launch), "fuse",
 * "linear_head", "xchg_cap_floats" (read when a network is built / the exchange is exported).  The matching
 * AET_* environment variables only give the initial values and are read once, in aet_context_create. */
int          aet_context_set_option(aet_context *ctx, const char *name, int value);
int          aet_context_get_option(const aet_context *ctx, const char *name, int *value);
/* Reads and clears the device status word; AET_OK, AET_E_TIMEOUT (a bounded wait expired: results of the work
 * in flight are incomplete) or AET_E_NAN (the update found non-finite weights or gradients and replaced them
 * as the reference does, mtcs/MtcsConvLayer.c:586-587 -- informational, training continued). */
int          aet_context_check(aet_context *ctx);
/* Limit of every device-side wait (mbarrier waits of the convolution kernels, the peer-flag wait of the update
 * kernel), in nanoseconds; one second by default.  Applies to the context's device.  After the limit a kernel
 * gives up, frees what it holds, sets the status word and returns: nothing traps and the context stays usable.
 * A data-parallel job whose ranks can be further apart than the limit (a rank writing a checkpoint) raises it. */
int          aet_context_set_wait_limit(aet_context *ctx, unsigned long long nanoseconds);
/* Self-test of that path: launches one warp that waits on a barrier nothing arrives at.  After the limit the
 * kernel returns and aet_context_check reports AET_E_TIMEOUT. */
int          aet_context_wait_probe(aet_context *ctx);
/* Per-kernel device timing (CUDA events on the context stream around every launch the library
 * makes): enable, run work, read the table grouped by kernel name.  Replaces the reference's
 * wall-clock prints (dnn/Classifier.c:255,312-319). */
typedef struct aet_kernel_time {
    char   name[48];
    int    launches;
    double total_ms;
    double algo_bytes;   /* algorithmic bytes moved per launch (HBM-bound kernels), else 0 */
    double algo_flops;   /* algorithmic FLOPs per launch (tensor-bound kernels), else 0 */
    double span_ms;      /* convolution kernels: sum over the launches of (last CTA exit - first CTA entry) on the device's
                          * own clock, i.e. the time without launch latency and event brackets; 0 where not recorded */
} aet_kernel_time;
int          aet_context_profile(aet_context *ctx, int enable);
int          aet_context_profile_read(aet_context *ctx, aet_kernel_time *table, int capacity, int *count);
long         aet_context_launch_count(const aet_context *ctx);

/* ------------------------------------------------------------------ tensors
 * Replaces DataFactory.createOutputData/createDeltaData/createInputData/createTruthData
 * (dnn/DataFactory.h:24-39) and the H2D/D2H taps of mtcs/MtcsIOData.c:47-52. */
aet_tensor *aet_tensor_create(aet_context *ctx, int batch, int c, int h, int w);
void        aet_tensor_destroy(aet_tensor *t);
int         aet_tensor_shape(const aet_tensor *t, int *batch, int *c, int *h, int *w);
int         aet_tensor_write(aet_tensor *t, const float *host_nchw);  /* InputData.setImageData */
int         aet_tensor_read(const aet_tensor *t, float *host_nchw);
int         aet_tensor_zero(aet_tensor *t);                             /* NData.setZero dnn/NData.c:232 */
size_t      aet_tensor_count(const aet_tensor *t);                      /* batch*c*h*w */

/* ------------------------------------------------------------------ layers
 * Constructors keep the reference's argument order, restricted to the supported branch
 * (groups=1, dilation=1, no binary/xnor/antialias/deform): dnn/ConvolutionalLayer.h:87-91,
 * dnn/MaxPoolLayer.h:29-30, dnn/AvgPoolLayer.c:17, dnn/SoftMaxLayer.h:27-28,
 * dnn/DropoutLayer.c:20-50.  `padding` is the resolved value (cfg `pad=1` => size/2). */
aet_layer *aet_convolutional_layer_create(aet_context *ctx, int batch, int h, int w, int c, int n, int groups,
                                          int size, int stride_x, int stride_y, int dilation, int padding,
                                          aet_activation activation, int batch_normalize, int train);
aet_layer *aet_maxpool_layer_create(aet_context *ctx, int batch, int h, int w, int c, int size, int stride_x,
                                    int stride_y, int padding, int train);
aet_layer *aet_avgpool_layer_create(aet_context *ctx, int batch, int w, int h, int c);
aet_layer *aet_softmax_layer_create(aet_context *ctx, int batch, int inputs, int groups, float temperature);
/* Dropout works in place on `prev`'s output and delta (dnn/NetworkFactory.c:644-650). */
aet_layer *aet_dropout_layer_create(aet_context *ctx, int batch, int inputs, float probability, aet_layer *prev);
/* ShortcutLayer without weights (dnn/ShortcutLayer.c:272-407 forward, :132-250 backward; factory dnn/NetworkFactory.c:175-246
 * with weights_type = none): output = activation(input + sum of the outputs of `from[0..n)`), n <= 4; a source with fewer
 * channels adds to the first of them, one with more contributes its first `c` channels (the reference compares flat
 * NCHW indices with the source's output count); all maps must be h x w.  backward: delta *= activation gradient, then
 * delta is ADDED to state.delta and to every source layer's delta.  The swish / mish forms are not restated. */
aet_layer *aet_shortcut_layer_create(aet_context *ctx, int batch, int h, int w, int c, int n, aet_layer *const *from,
                                     aet_activation activation, int train);
void       aet_layer_destroy(aet_layer *l);

/* NLayer.forward / backward / update / initDelta (dnn/NLayer.h:159-173). */
int aet_layer_forward(aet_layer *l, aet_state state);
int aet_layer_backward(aet_layer *l, aet_state state);
int aet_layer_update(aet_layer *l, int batch, float learning_rate, float momentum, float decay, float loss_scale);
int aet_layer_init_delta(aet_layer *l);
aet_tensor *aet_layer_output(aet_layer *l);      /* NLayer.getOutputData */
aet_tensor *aet_layer_delta(aet_layer *l);       /* NLayer.deltaData     */
aet_layer_type aet_layer_kind(const aet_layer *l);
int   aet_layer_out_shape(const aet_layer *l, int *c, int *h, int *w);
float aet_layer_cost(aet_layer *l);              /* OutputLayer.getCost dnn/SoftMaxLayer.c:321 */
size_t aet_layer_param_count(const aet_layer *l, aet_param which);
int   aet_layer_read(aet_layer *l, aet_param which, void *host);        /* float, int32 for AET_P_INDEXES */
int   aet_layer_write(aet_layer *l, aet_param which, const void *host);
/* ConvolutionalLayer.loadWeights/saveWeights (dnn/ConvolutionalLayer.c:422-486): the `fp`
 * is a C FILE* positioned at this layer's record. */
int   aet_layer_load_weights(aet_layer *l, void *fp);
int   aet_layer_save_weights(aet_layer *l, void *fp);

/* ------------------------------------------------------------------ network
 * NetworkFactory.createNetwork (dnn/NetworkFactory.c:830-1013) + NNetwork (dnn/NNetwork.h:141-195). */
aet_network *aet_network_create(aet_context *ctx, const char *cfg_path, int train);
aet_network *aet_network_create_from_string(aet_context *ctx, const char *cfg_text, int train);
/* batch > 0 overrides the cfg's [net] batch (createNetwork(cfg,batch,time_steps), dnn/NetworkFactory.c:1023). */
aet_network *aet_network_create_ex(aet_context *ctx, const char *cfg_text, int train, int batch);
void         aet_network_destroy(aet_network *net);
int          aet_network_layer_count(const aet_network *net);
aet_layer   *aet_network_layer(aet_network *net, int index);
int          aet_network_batch(const aet_network *net);
int          aet_network_input_shape(const aet_network *net, int *c, int *h, int *w);
int          aet_network_outputs(const aet_network *net);   /* NNetwork.getOuputSize */
aet_tensor  *aet_network_input(aet_network *net);           /* NNetwork.inputData */
aet_tensor  *aet_network_truth(aet_network *net);           /* NNetwork.truthData */
float        aet_network_learning_rate(const aet_network *net);   /* NNetwork.getCurrentRate dnn/NNetwork.c:215-246 */
int          aet_network_set_hyper(aet_network *net, float learning_rate, float momentum, float decay);
int64_t      aet_network_seen(const aet_network *net);

/* NNetwork.forward / backward / update (dnn/NNetwork.c:382-396,627-654,667-716). */
int   aet_network_forward(aet_network *net, aet_state state);
int   aet_network_backward(aet_network *net, aet_state state);
int   aet_network_update(aet_network *net);
float aet_network_cost(aet_network *net);                      /* getNetworkCost dnn/NNetwork.c:611-624 */
/* NNetwork.train(InputData*,TruthData*) (dnn/NNetwork.c:740-760): host NCHW batch and one-hot truth in, mean
 * loss of this batch out (cost / batch).  With [net] subdivisions = S > 1 the weight gradients accumulate over S
 * calls and the S-th call runs the update with update_batch = batch * S, as NNetwork.train(ImageData*) does
 * (dnn/NNetwork.c:762-774).  Copies are asynchronous on the context stream; the loss read-back is the only host
 * synchronisation; AET_E_TIMEOUT is returned when a bounded device-side wait expired during the step. */
int   aet_network_train_step(aet_network *net, const float *host_x, const float *host_truth, float *loss);
/* Same step on data already resident in the network's input/truth tensors.  When `loss` is NULL
 * nothing is read back (the loss stays in device memory until aet_network_last_loss). */
int   aet_network_train_step_device(aet_network *net, float *loss);
int   aet_network_last_loss(aet_network *net, float *loss);
/* Pipelined aet_network_train_step: the device-side double buffer that stands for the reference's loader double
 * buffer (dnn/ImageData.c:169-202) and per-step upload (mtcs/MtcsIOData.c:50-52).  The host->device copy of this
 * call's batch runs on a copy stream while the previous call's step computes; the call waits for nothing of its
 * own step and returns the PREVIOUS call's mean loss in `previous_loss` (NaN on the first call; NULL to skip).
 * Page-locked buffers are read by DMA until the NEXT call (or aet_network_last_loss) returns: keep them
 * unchanged until then (alternate two); pageable buffers are copied before the call returns.
 * aet_network_last_loss drains the pipeline.  The first call allocates the two staging slots.
 * Returns AET_E_TIMEOUT when the previous step's kernels gave up a bounded wait. */
int   aet_network_train_step_async(aet_network *net, const float *host_x, const float *host_truth, float *previous_loss);
/* NNetwork.predict (dnn/NNetwork.c:411-428): forward with train=0, copy the last layer's output. */
int   aet_network_predict(aet_network *net, const float *host_x, float *host_out);
/* NNetwork.fuseConvBatchnorm (dnn/NNetwork.c:272-290, dnn/ConvolutionalLayer.c:983-1003): folds every batch-norm
 * layer's rolling statistics and scale into its convolution's biases and weights; afterwards the network only
 * predicts (training calls return AET_E_INVALID).  Run it after aet_network_load_weights, as the reference's
 * validation and prediction entry points do (dnn/Classifier.c:372-374). */
int   aet_network_fuse_conv_batchnorm(aet_network *net);
/* predict + DnnUtils.topK (dnn/DnnUtils.c:463-477): host_indexes[batch][k] = class indexes by descending score. */
int   aet_network_predict_topk(aet_network *net, const float *host_x, int k, int *host_indexes);
/* The accuracy loop of Classifier.validateSingle (dnn/Classifier.c:431-462) over `count` images the caller has
 * already decoded and cropped to the network's input ([count][c][h][w]); class_ids[count] are the true classes.
 * top1 = share of images whose best class is right, topk = share with the right class among the best k. */
int   aet_network_validate(aet_network *net, const float *host_images, const int *class_ids, int count, int k,
                           float *top1, float *topk);
/* Device-side image augmentation: the per-image chain of ImageData.loadImageAugmentPaths (dnn/ImageData.c:56-73) --
 * NImage.rotateCrop with bilinear sampling (dnn/NImage.c:138-157,551-572), NImage.flip (:346-362), NImage.distort in HSV
 * (:201-337) -- as ONE kernel that reads the uploaded source images and writes the network's input tensor, instead of
 * the reference's host loops followed by an upload of the finished batch.  The random draws stay with the caller
 * (one aet_augment per image, drawn as the reference draws them: :1016-1035 for rad/scale/dx/dy/aspect, :339-344 for
 * dhue/dsat/dexp), so a run is reproducible and checkable.  Source images: host FP32 [batch][c][src_h][src_w], all of
 * one size; the crop is net width x net height (square networks: the reference's final resize is then the identity). */
typedef struct aet_augment {
    float rad, scale, dx, dy, aspect;   /* rotateCrop(rad, scale, size, size, dx, dy, aspect) */
    int   flip;                         /* mirror left-right */
    float dhue, dsat, dexp;             /* distort(dhue, dsat, dexp); ignored unless channels == 3 */
} aet_augment;
int   aet_network_augment_input(aet_network *net, const float *host_src, int src_h, int src_w, const aet_augment *params);
/* Capture forward+backward+update into a CUDA graph that later train steps replay (0 = off). */
int   aet_network_use_graph(aet_network *net, int enable);
/* NNetwork.loadWeights / saveWeights (dnn/NNetwork.c:64-147): Darknet .weights container. */
int   aet_network_load_weights(aet_network *net, const char *path);
/* loadWeights(filename, cutoff) (dnn/NNetwork.c:64-110): only the layers in front of index `cutoff` are read (-1: all).
 * Layers whose cfg section says dontload = 1 are passed over; dontloadscales = 1 skips a layer's batch-norm block; a
 * file that ends at a layer boundary leaves the remaining layers untouched. */
int   aet_network_load_weights_upto(aet_network *net, const char *path, int cutoff);
int   aet_network_save_weights(aet_network *net, const char *path);
/* Optional side file with the step-to-step state the .weights container leaves out (bias / scale / weight updates and,
 * for batch-norm layers, the last batch mean, per convolutional layer in the .weights file's order), so that a run
 * resumed from both files continues bit for bit.
 * No reference counterpart: dnn/NNetwork.c:112-147 does not save them. */
int   aet_network_save_momentum(aet_network *net, const char *path);
int   aet_network_load_momentum(aet_network *net, const char *path);
/* 64-bit hash of all weights, biases, scales and momentum buffers (data-parallel consistency check). */
int   aet_network_param_hash(aet_network *net, uint64_t *hash);
/* Per-kernel device timing of the next train steps (aet_context_profile on the network's context;
 * enabling it also suspends graph replay so that every launch is visible). */
int   aet_network_profile(aet_network *net, int enable);
int   aet_network_profile_read(aet_network *net, aet_kernel_time *table, int capacity, int *count);
int   aet_network_launches_per_step(const aet_network *net);

/* ------------------------------------------------------------------ data parallel
 * The reference is single GPU (dnn/Classifier.c:142, `ngpus = 1`); these entry points add the
 * batch-data-parallel exchange: one NCCL all-reduce of the per-step gradient arena, issued per
 * layer bucket during backward on a side stream.  `unique_id` is the 128-byte ncclUniqueId. */
int   aet_comm_unique_id(void *unique_id_128);
int   aet_network_comm_init(aet_network *net, const void *unique_id_128, int rank, int world);
/* Measurement aid: mean time per step (microseconds) the main stream waited for the gradient collectives since the last
 * call, and the number of steps counted.  Needs the context option "comm_stamps" = 1 before the step's graph is
 * captured (two one-thread kernels per step read the device clock around the wait). */
int   aet_network_comm_exposed(aet_network *net, double *mean_microseconds, long long *steps);
/* Optional, after aet_network_comm_init on 2..8 ranks that sit on DIFFERENT GPUs of one box (no counterpart in
 * the reference, which is single-GPU): the last gradient bucket of a step (the first layers', complete only when
 * backward ends) is summed over the ranks inside the update kernel through peer-mapped buffers instead of by a
 * collective whose latency nothing could hide.  Every rank exports an 80-byte blob (CUDA IPC handle + device
 * UUID), the caller gathers the blobs in rank order by any host channel and hands all of them to attach.  Attach
 * refuses ranks that share a GPU.  Without attach the bucket goes through the all-reduce like the others. */
int   aet_network_comm_exchange_export(aet_network *net, void *blob_80);
int   aet_network_comm_exchange_attach(aet_network *net, const void *blobs_world_x_80);
/* Back to the collectives alone.  Every rank must take the same path: when the attach failed on any rank, all detach. */
int   aet_network_comm_exchange_detach(aet_network *net);
int   aet_network_comm_destroy(aet_network *net);
/* Device pointer and float count of the gradient arena (for callers that run their own collective). */
int   aet_network_grad_arena(aet_network *net, void **device_ptr, size_t *count);

/* ------------------------------------------------------------------ allocation-free entry point
 * No counterpart in the reference (its kernels need no scratch; ours reduce in two stages).
 * For callers that must not allocate device memory while they run -- a process whose whole device
 * pool is sized and handed out at start-up, a service inside a phase where cudaMalloc (which
 * synchronises the device) is off limits -- this computes the bias gradient
 *     bias_updates[c] += sum over p of delta[p][c]
 * with the stage-one partial sums held in a fixed 1 MiB __device__ array inside the library instead
 * of the context's cudaMalloc'ed scratch arena.  It calls no cudaMalloc / cudaFree.
 *   delta         device pointer, FP32 [pixels][channels] row-major, 16-byte aligned
 *   bias_updates  device pointer, FP32 [channels], accumulated into
 *   channels      multiple of 4; the launch plan must fit the array: blocks * 2 * channels floats
 *                 with up to 2 * SMs blocks (so up to ~440 channels at full grid on a 148-SM
 *                 part, more when `pixels` is small), otherwise AET_E_INVALID
 *   cuda_stream   cudaStream_t to launch on (NULL = the legacy default stream)
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress) with
 * that device current; under lazy module loading that lookup is also when the driver backs the
 * array with memory.  So make one warm-up call per device at start-up, while allocation is still
 * allowed and outside any stream capture; host threads may race on it (it is serialised inside).
 * The address is cached for the life of the process: do not call cudaDeviceReset between calls.
 * All calls on a device share the one array: calls whose kernels may overlap on the GPU (different
 * streams) race -- serialise them.  Nothing in the array has to be cleared between calls. */
int   aet_backward_bias_static(const float *delta, float *bias_updates, long long pixels, int channels, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* AET_B200_H */
