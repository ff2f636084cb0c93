/*
 * TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement of the AET-CNN training hot path (reference tree src/com/ai/dnn,
 * cited per function in aet_oracle.c).  It exists to CHECK the CUDA library and to
 * provide the timed CPU baseline; the product library never links, loads or calls it.
 *
 * PARITY UNPINNED by the reference's own tests: the reference ships no tests, golden
 * vectors or fixtures for this path, and its sources (AET dialect) cannot be compiled
 * here.  The oracle is instead pinned by (a) hand-computable cases, (b) fixtures from an
 * independent float64 implementation of the same published operators (tests/golden),
 * (c) finite-difference gradient checks and the im2col/col2im adjoint identity.
 *
 * All tensors are FP32, NCHW, contiguous, exactly as the reference stores them.
 * `mode` selects which of the reference's two numerically different back ends is
 * restated: AETO_MODE_CPU (the dnn/ classes) or AETO_MODE_MTCS (the dnn/mtcs/ kernels).
 */
#ifndef AET_ORACLE_H
#define AET_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { AETO_LINEAR = 0, AETO_RELU = 1, AETO_LEAKY = 2 };
enum { AETO_MODE_CPU = 0, AETO_MODE_MTCS = 1 };
enum { AETO_CONV = 0, AETO_MAXPOOL = 1, AETO_AVGPOOL = 2, AETO_SOFTMAX = 3, AETO_DROPOUT = 4, AETO_SHORTCUT = 5 };

/* ---- primitives ---- */
void aeto_gemm(int TA, int TB, int M, int N, int K, float ALPHA, const float *A, int lda,
               const float *B, int ldb, float BETA, float *C, int ldc);
void aeto_im2col(const float *im, int channels, int height, int width, int ksize_h, int ksize_w,
                 int pad_h, int pad_w, int stride_h, int stride_w, float *col);
void aeto_col2im(const float *col, int channels, int height, int width, int ksize_h, int ksize_w,
                 int pad_h, int pad_w, int stride_h, int stride_w, float *im);
int  aeto_conv_out(int in, int size, int stride, int pad);
size_t aeto_conv_workspace(int c, int h, int w, int size, int stride_x, int stride_y, int pad);

/* ---- convolution (groups=1, dilation=1) ---- */
void aeto_conv_forward(const float *x, const float *weights, float *y, float *workspace,
                       int batch, int c, int h, int w, int n, int size, int stride_x, int stride_y, int pad);
/* dx may be NULL (first layer). dw accumulates (beta=1); dx is overwritten. */
void aeto_conv_backward(const float *x, const float *weights, const float *delta, float *dw, float *dx,
                        float *workspace, int batch, int c, int h, int w, int n, int size,
                        int stride_x, int stride_y, int pad);
void aeto_add_bias(float *y, const float *biases, int batch, int n, int spatial);
void aeto_backward_bias(float *bias_updates, const float *delta, int batch, int n, int spatial);
void aeto_activate(float *y, size_t count, int activation, int mode);
void aeto_gradient(const float *y, size_t count, int activation, float *delta);
/* swish (14) and mish (15): delta *= f'(v) formed as dnn/Activation.c:303-330 does, from the output y and the value
 * before the activation v. */
void aeto_gradient_input(const float *y, const float *v, size_t count, int activation, float *delta);

/* ---- batch norm ---- */
void aeto_bn_forward(int mode, int train, float *y, int batch, int c, int spatial,
                     const float *scales, const float *biases, float *mean, float *variance,
                     float *rolling_mean, float *rolling_variance, float *x, float *x_norm);
void aeto_bn_backward(int mode, float *delta, const float *x, const float *x_norm, const float *mean,
                      const float *variance, const float *scales, float *scale_updates,
                      float *bias_updates, float *mean_delta, float *variance_delta,
                      int batch, int c, int spatial);

/* ---- pooling ---- */
int  aeto_maxpool_out(int in, int size, int stride, int padding);
void aeto_maxpool_forward(int mode, const float *x, float *y, int *indexes, int batch, int c, int h, int w,
                          int size, int stride_x, int stride_y, int padding);
void aeto_maxpool_backward(const float *delta, const int *indexes, float *prev_delta, size_t out_count);
void aeto_avgpool_forward(const float *x, float *y, int batch, int c, int spatial);
void aeto_avgpool_backward(const float *delta, float *prev_delta, int batch, int c, int spatial);

/* ---- softmax + cross entropy ---- */
float aeto_softmax_forward(int mode, const float *x, float *p, const float *truth, float *delta, float *loss,
                           int batch, int inputs, int groups, float temperature);
void aeto_softmax_backward(const float *delta, float *prev_delta, size_t count, float loss_scale);

/* ---- dropout: r[] holds the uniform draws ---- */
void aeto_dropout_forward(float *x, const float *r, size_t count, float probability);
void aeto_dropout_backward(float *delta, const float *r, size_t count, float probability);

/* ---- shortcut without weights: dnn/ShortcutLayer.c:272-407 (forward), :132-250 (backward), per sample ----
 * out[j] = in[j] + sum_i add_i[j] for j < add_outputs_i, then the activation; backward: delta *= gradient(out),
 * delta_out[j] += delta[j], layer_delta_i[j] += delta[j] for j < add_outputs_i. */
void aeto_shortcut_forward(const float *in, float *out, int batch, size_t outputs, int n, const float *const *add,
                           const size_t *add_outputs);
void aeto_shortcut_backward(const float *delta, float *delta_out, int batch, size_t outputs, int n, float *const *layer_delta,
                            const size_t *add_outputs);

/* ---- SGD with momentum ---- */
void aeto_sgd_weights(float *w, float *u, size_t count, int batch, float lr, float momentum, float decay);
void aeto_sgd_plain(float *p, float *u, size_t count, int batch, float lr, float momentum);

/* ---- whole network (restates NNetwork.forward/backward/update) ---- */
typedef struct aeto_layer_spec {
    int type;            /* AETO_CONV ... */
    int filters, size, stride_x, stride_y, pad; /* conv: pad = resolved padding; pool: padding */
    int batch_normalize, activation;
    float probability;   /* dropout */
    float temperature;   /* softmax */
    int groups;          /* softmax groups */
    float learning_rate_scale;
    int n_from, from[4]; /* shortcut: absolute indexes of the layers whose outputs are added */
    int stopbackward;    /* dnn/NNetwork.c:648: the backward walk ends before this layer; the layers in front of the LAST
                          * such layer only run forward and are never updated (dnn/NetworkFactory.c:979-991) */
    int dont_update;     /* dnn/NNetwork.c:703 (GPU path only): no update while the iteration number is <= this */
} aeto_layer_spec;

typedef struct aeto_net aeto_net;
enum { AETO_P_WEIGHTS = 0, AETO_P_WEIGHT_UPDATES, AETO_P_BIASES, AETO_P_BIAS_UPDATES, AETO_P_SCALES,
       AETO_P_SCALE_UPDATES, AETO_P_ROLLING_MEAN, AETO_P_ROLLING_VARIANCE, AETO_P_MEAN, AETO_P_VARIANCE,
       AETO_P_OUTPUT, AETO_P_DELTA, AETO_P_X, AETO_P_X_NORM, AETO_P_INDEXES, AETO_P_LOSS, AETO_P_RAND };

aeto_net *aeto_net_create(const aeto_layer_spec *specs, int nlayers, int batch, int c, int h, int w,
                          int mode, int threads);
void   aeto_net_free(aeto_net *net);
int    aeto_net_layers(const aeto_net *net);
/* Returns a pointer into the oracle's own storage and its element count (0 / NULL when absent). */
float *aeto_net_param(aeto_net *net, int layer, int which, size_t *count);
void   aeto_net_out_shape(const aeto_net *net, int layer, int *c, int *h, int *w);
void   aeto_net_forward(aeto_net *net, const float *x, const float *truth, int train);
/* input_delta may be NULL (layer 0 then skips dgrad, as NNetwork.backward does). */
void   aeto_net_backward(aeto_net *net, const float *x, float *input_delta);
void   aeto_net_update(aeto_net *net, int update_batch, float lr, float momentum, float decay);
float  aeto_net_cost(const aeto_net *net);
/* forward + backward + update; returns cost / batch like NNetwork.train (subdivisions = 1). */
float  aeto_net_train_step(aeto_net *net, const float *x, const float *truth, float lr, float momentum, float decay);

/* NNetwork.getCurrentRate, dnn/NNetwork.c:215-246 (policy: 0 constant, 1 step, 2 steps, 3 exp, 4 poly, 5 sig;
 * the RANDOM policy is not restated).  batch_num = seen / (batch * subdivisions). */
float  aeto_current_rate(size_t batch_num, int policy, float learning_rate, int burn_in, float power, int step, float scale,
                         const int *steps, const float *scales, int num_steps, float gamma, int max_batches);
/* fix_nan_and_inf / reset_nan_and_inf of the GPU update, mtcs/MtcsTool.c:77-107 */
void   aeto_fix_nan_and_inf(float *v, size_t n);
void   aeto_reset_nan_and_inf(float *v, size_t n);

/* ConvolutionalLayer.fuseConvBatchnorm, dnn/ConvolutionalLayer.c:983-1003: folds the rolling statistics and the
 * scale into biases and weights (inference). */
void   aeto_fuse_conv_batchnorm(float *biases, const float *scales, const float *rolling_mean, const float *rolling_variance,
                                float *weights, int filters, size_t filter_size);
/* DnnUtils.topK, dnn/DnnUtils.c:463-477: indexes of the k largest of a[0..n) in descending order (strict >). */
void   aeto_top_k(const float *a, int n, int k, int *index);
/* ConvolutionalLayer.transposeMatrix, dnn/ConvolutionalLayer.c:444-454 (the `flipped` weights layout). */
void   aeto_transpose_matrix(float *a, int rows, int cols);

/* The per-image augmentation chain of ImageData.loadImageAugmentPaths (dnn/ImageData.c:56-73) with its random draws
 * given as inputs: NImage.rotateCrop (dnn/NImage.c:551-572, bilinear sampling :138-157) into a size x size crop,
 * NImage.flip (:346-362) when `flip`, NImage.distort (:323-337: RGB->HSV :201-243, scale S and V, shift hue,
 * HSV->RGB :245-291, clamp to [0,1]) for 3-channel images.  src [c][sh][sw] -> dst [c][size][size]. */
void   aeto_augment_image(const float *src, int c, int sh, int sw, float *dst, int size, float rad, float scale, float dx, float dy,
                          float aspect, int flip, float dhue, float dsat, float dexp);

/* Convolution with channel groups and dilated taps: dnn/ConvolutionalLayer.c:703-806 (forward) and :909-947 (backward)
 * with im2col_cpu_ext / col2im_cpu_ext (dnn/Im2Col.c:65-103,155-192; padding in pixels = pad * dilation).
 * weights [n][c/groups][size][size].  The output size is the layer's own formula (aeto_conv_out with `pad`). */
void   aeto_conv_forward_ex(const float *x, const float *weights, float *y, float *workspace, int batch, int c, int h, int w,
                            int n, int size, int stride_x, int stride_y, int pad, int groups, int dilation);
void   aeto_conv_backward_ex(const float *x, const float *weights, const float *delta, float *dw, float *dx, float *workspace,
                             int batch, int c, int h, int w, int n, int size, int stride_x, int stride_y, int pad, int groups,
                             int dilation);

/* adam_update_gpu, mtcs/MtcsConvLayer.c:494-524: one parameter array; d (the pending update) is zeroed. */
void   aeto_adam_update(float *w, float *d, float *m, float *v, float B1, float B2, float eps, float decay, float rate, size_t n,
                        int batch, int t);

/* synthetic tensors (aet_rng.h) exposed for bindings */
void aeto_fill_uniform(float *dst, size_t n, uint64_t seed, uint64_t tensor_id);
void aeto_fill_normal(float *dst, size_t n, uint64_t seed, uint64_t tensor_id, float mean, float stddev);

#ifdef __cplusplus
}
#endif
#endif
