/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the AET-CNN training hot path.
 * See aet_oracle.h for what this is and is not.  Reference citations are paths inside the
 * reference project (src/com/ai/dnn/...), abbreviated dnn/ and dnn/mtcs/.
 *
 * Build variants:
 *   default        float accumulators, loop orders as the reference writes them
 *   -DAETO_ACC64   the same formulas with double accumulators in every reduction; used
 *                  by tests that need an error bar tighter than FP32 summation noise.
 */
#include "aet_oracle.h"
#include "aet_rng.h"
#include <float.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>

#ifdef AETO_ACC64
typedef double acc_t;
#else
typedef float acc_t;
#endif

static void *xcalloc(size_t n, size_t sz) {
    void *p = calloc(n ? n : 1, sz);
    if (!p) { fprintf(stderr, "aet_oracle: out of memory\n"); abort(); }
    return p;
}

/* ------------------------------------------------------------------ GEMM
 * dnn/Gemm.c:53-144.  C is scaled by BETA first, then rows are processed one at a time;
 * NN and TN update C in axpy order (k outer, j inner), NT and TT form a dot product. */
static void gemm_row_nn(int N, int K, float ALPHA, const float *A, const float *B, int ldb, float *C) {
#ifdef AETO_ACC64
    double *acc = (double *)xcalloc((size_t)N, sizeof(double));
    for (int k = 0; k < K; ++k) {
        double a = (double)ALPHA * A[k];
        for (int j = 0; j < N; ++j) acc[j] += a * B[(size_t)k * ldb + j];
    }
    for (int j = 0; j < N; ++j) C[j] = (float)(C[j] + acc[j]);
    free(acc);
#else
    for (int k = 0; k < K; ++k) {
        float a = ALPHA * A[k];
        for (int j = 0; j < N; ++j) C[j] += a * B[(size_t)k * ldb + j];
    }
#endif
}
static void gemm_row_tn(int N, int K, float ALPHA, const float *A, int lda, const float *B, int ldb, float *C) {
#ifdef AETO_ACC64
    double *acc = (double *)xcalloc((size_t)N, sizeof(double));
    for (int k = 0; k < K; ++k) {
        double a = (double)ALPHA * A[(size_t)k * lda];
        for (int j = 0; j < N; ++j) acc[j] += a * B[(size_t)k * ldb + j];
    }
    for (int j = 0; j < N; ++j) C[j] = (float)(C[j] + acc[j]);
    free(acc);
#else
    for (int k = 0; k < K; ++k) {
        float a = ALPHA * A[(size_t)k * lda];
        for (int j = 0; j < N; ++j) C[j] += a * B[(size_t)k * ldb + j];
    }
#endif
}
static void gemm_row_nt(int N, int K, float ALPHA, const float *A, const float *B, int ldb, float *C) {
    for (int j = 0; j < N; ++j) {
        acc_t sum = 0;
        for (int k = 0; k < K; ++k) sum += ALPHA * A[k] * B[(size_t)j * ldb + k];
        C[j] += (float)sum;
    }
}
static void gemm_row_tt(int N, int K, float ALPHA, const float *A, int lda, const float *B, int ldb, float *C) {
    for (int j = 0; j < N; ++j) {
        acc_t sum = 0;
        for (int k = 0; k < K; ++k) sum += ALPHA * A[(size_t)k * lda] * B[(size_t)j * ldb + k];
        C[j] += (float)sum;
    }
}

void aeto_gemm(int TA, int TB, int M, int N, int K, float ALPHA, const float *A, int lda,
               const float *B, int ldb, float BETA, float *C, int ldc) {
    if (BETA != 1) {
        for (int i = 0; i < M; ++i)
            for (int j = 0; j < N; ++j) C[(size_t)i * ldc + j] *= BETA;
    }
    for (int t = 0; t < M; ++t) {
        float *c = C + (size_t)t * ldc;
        if (!TA && !TB)      gemm_row_nn(N, K, ALPHA, A + (size_t)t * lda, B, ldb, c);
        else if (TA && !TB)  gemm_row_tn(N, K, ALPHA, A + t, lda, B, ldb, c);
        else if (!TA && TB)  gemm_row_nt(N, K, ALPHA, A + (size_t)t * lda, B, ldb, c);
        else                 gemm_row_tt(N, K, ALPHA, A + t, lda, B, ldb, c);
    }
}

/* ------------------------------------------------------------------ im2col / col2im
 * dnn/Im2Col.c:20-22,65-103 (im2col) and :155-192 (col2im).  Column-matrix rows are ordered
 * (channel, kernel_row, kernel_col), columns (out_row, out_col); taps outside the image read 0.
 * col2im first zeroes the image, then accumulates. Dilation is fixed at 1 (hot-path scope). */
int aeto_conv_out(int in, int size, int stride, int pad) { return (in + 2 * pad - size) / stride + 1; }

size_t aeto_conv_workspace(int c, int h, int w, int size, int stride_x, int stride_y, int pad) {
    return (size_t)c * size * size * aeto_conv_out(h, size, stride_y, pad) * aeto_conv_out(w, size, stride_x, pad);
}

void aeto_im2col(const float *im, int channels, int height, int width, int ksize_h, int ksize_w,
                 int pad_h, int pad_w, int stride_h, int stride_w, float *col) {
    const int out_h = (height + 2 * pad_h - ksize_h) / stride_h + 1;
    const int out_w = (width + 2 * pad_w - ksize_w) / stride_w + 1;
    for (int ch = 0; ch < channels; ++ch) {
        const float *plane = im + (size_t)ch * height * width;
        for (int kr = 0; kr < ksize_h; ++kr)
            for (int kc = 0; kc < ksize_w; ++kc)
                for (int orow = 0; orow < out_h; ++orow) {
                    int irow = orow * stride_h - pad_h + kr;
                    if ((unsigned)irow >= (unsigned)height) {
                        for (int ocol = 0; ocol < out_w; ++ocol) *col++ = 0;
                        continue;
                    }
                    for (int ocol = 0; ocol < out_w; ++ocol) {
                        int icol = ocol * stride_w - pad_w + kc;
                        *col++ = ((unsigned)icol < (unsigned)width) ? plane[(size_t)irow * width + icol] : 0.0f;
                    }
                }
    }
}

void aeto_col2im(const float *col, int channels, int height, int width, int ksize_h, int ksize_w,
                 int pad_h, int pad_w, int stride_h, int stride_w, float *im) {
    const int out_h = (height + 2 * pad_h - ksize_h) / stride_h + 1;
    const int out_w = (width + 2 * pad_w - ksize_w) / stride_w + 1;
    memset(im, 0, sizeof(float) * (size_t)channels * height * width);
    for (int ch = 0; ch < channels; ++ch) {
        float *plane = im + (size_t)ch * height * width;
        for (int kr = 0; kr < ksize_h; ++kr)
            for (int kc = 0; kc < ksize_w; ++kc)
                for (int orow = 0; orow < out_h; ++orow) {
                    int irow = orow * stride_h - pad_h + kr;
                    if ((unsigned)irow >= (unsigned)height) { col += out_w; continue; }
                    for (int ocol = 0; ocol < out_w; ++ocol, ++col) {
                        int icol = ocol * stride_w - pad_w + kc;
                        if ((unsigned)icol < (unsigned)width) plane[(size_t)irow * width + icol] += *col;
                    }
                }
    }
}

/* ------------------------------------------------------------------ convolution
 * Forward: dnn/ConvolutionalLayer.c:684-806 (FP32 branch): Y = 0; per image col = im2col(X_i)
 * (skipped for 1x1 stride-1, :789-790); Y_i += W * col. */
void aeto_conv_forward(const float *x, const float *weights, float *y, float *workspace,
                       int batch, int c, int h, int w, int n, int size, int stride_x, int stride_y, int pad) {
    const int out_h = aeto_conv_out(h, size, stride_y, pad), out_w = aeto_conv_out(w, size, stride_x, pad);
    const int m = n, k = size * size * c, nn = out_h * out_w;
    memset(y, 0, sizeof(float) * (size_t)batch * m * nn);
    for (int i = 0; i < batch; ++i) {
        const float *im = x + (size_t)i * c * h * w;
        const float *b = im;
        if (!(size == 1 && stride_x == 1 && stride_y == 1)) {
            aeto_im2col(im, c, h, w, size, size, pad, pad, stride_y, stride_x, workspace);
            b = workspace;
        }
        aeto_gemm(0, 0, m, nn, k, 1, weights, k, b, nn, 1, y + (size_t)i * m * nn, nn);
    }
}

/* Backward: dnn/ConvolutionalLayer.c:909-947.  Per image: col = im2col(X_i) (always, even 1x1);
 * dW += delta_i * col^T; if a previous delta exists: col = W^T * delta_i (beta 0); dX_i = col2im(col). */
void aeto_conv_backward(const float *x, const float *weights, const float *delta, float *dw, float *dx,
                        float *workspace, int batch, int c, int h, int w, int n, int size,
                        int stride_x, int stride_y, int pad) {
    const int out_h = aeto_conv_out(h, size, stride_y, pad), out_w = aeto_conv_out(w, size, stride_x, pad);
    const int m = n, nn = size * size * c, k = out_h * out_w;
    for (int i = 0; i < batch; ++i) {
        const float *a = delta + (size_t)i * m * k;
        const float *im = x + (size_t)i * c * h * w;
        aeto_im2col(im, c, h, w, size, size, pad, pad, stride_y, stride_x, workspace);
        aeto_gemm(0, 1, m, nn, k, 1, a, k, workspace, k, 1, dw, nn);
        if (dx) {
            aeto_gemm(1, 0, nn, k, m, 1, weights, nn, a, k, 0, workspace, k);
            aeto_col2im(workspace, c, h, w, size, size, pad, pad, stride_y, stride_x, dx + (size_t)i * c * h * w);
        }
    }
}

/* dnn/IOData.c:43-55 */
void aeto_add_bias(float *y, const float *biases, int batch, int n, int spatial) {
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < n; ++i)
            for (int j = 0; j < spatial; ++j) y[((size_t)b * n + i) * spatial + j] += biases[i];
}

/* dnn/BiasData.c:40-57 with dnn/DnnUtils.c:113-119: per image, per channel partial sum, then add. */
void aeto_backward_bias(float *bias_updates, const float *delta, int batch, int n, int spatial) {
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < n; ++i) {
            const float *d = delta + (size_t)spatial * (i + (size_t)b * n);
            acc_t sum = 0;
            for (int j = 0; j < spatial; ++j) sum += d[j];
            bias_updates[i] += (float)sum;
        }
}

/* dnn/Activation.h:53,56,61 (CPU scalar definitions; `.1*x` is a double product) and
 * dnn/mtcs/MtcsActivation.c:112-117 (`.1f*x`). */
/* Scalar activations, dnn/Activation.h:41-113 (CPU, double intermediates where the reference's literals are double)
 * and mtcs/MtcsActivation.c:17-103 (GPU, float).  Numbering: AETO_LINEAR 0, RELU 1, LEAKY 2, then LOGISTIC 3,
 * RELU6 4, RELIE 5, RAMP 6, TANH 7, PLSE 8, ELU 9, LOGGY 10, HARDTAN 11, LHTAN 12, SELU 13. */
/* dnn/Activation.h:108-113 (softplus_activate) and :69 (tanh_activate) */
static float softplus_ref(float x, float threshold) {
    if (x > threshold) return x;
    else if (x < -threshold) return expf(x);
    return logf(expf(x) + 1);
}
static float tanh_ref(float x) { return (2 / (1 + expf(-2 * x)) - 1); }

static float act_cpu(float x, int a) {
    switch (a) {
    case 0: return x;
    case 1: return x * (x > 0);
    case 2: return (x > 0) ? x : .1 * x;
    case 3: return 1. / (1. + exp(-x));
    case 4: return fminf(fmaxf(x, 0), 6);                       /* the CPU class has no relu6; GPU form */
    case 5: return (x > 0) ? x : .01 * x;
    case 6: return x * (x > 0) + .1 * x;
    case 7: return (exp(2 * x) - 1) / (exp(2 * x) + 1);
    case 8: if (x < -4) return .01 * (x + 4); if (x > 4) return .01 * (x - 4) + 1; return .125 * x + .5;
    case 9: return (x >= 0) * x + (x < 0) * (exp(x) - 1);
    case 10: return 2. / (1. + exp(-x)) - 1;
    case 11: if (x < -1) return -1; if (x > 1) return 1; return x;
    case 12: if (x < 0) return .001 * x; if (x > 1) return .001 * (x - 1) + 1; return x;
    case 13: return (x >= 0) * 1.0507 * x + (x < 0) * 1.0507 * 1.6732 * (exp(x) - 1);
    case 14: { float sg = 1. / (1. + exp(-x)); return x * sg; }                                  /* dnn/IOData.c:75-88 */
    case 15: return x * tanh_ref(softplus_ref(x, 20));                                          /* dnn/IOData.c:92-105 */
    default: return x;
    }
}
static float act_mtcs(float x, int a) {
    switch (a) {
    case 0: return x;
    case 1: return x * (x > 0);
    case 2: return (x > 0) ? x : .1f * x;
    case 3: return 1.f / (1.f + expf(-x));
    case 4: return fminf(fmaxf(x, 0), 6);
    case 5: return (x > 0) ? x : .01f * x;
    case 6: return x * (x > 0) + .1f * x;
    case 7: return (2 / (1 + expf(-2 * x)) - 1);
    case 8: if (x < -4) return .01f * (x + 4); if (x > 4) return .01f * (x - 4) + 1; return .125f * x + .5f;
    case 9: return (x >= 0) * x + (x < 0) * (expf(x) - 1);
    case 10: return 2.f / (1.f + expf(-x)) - 1;
    case 11: if (x < -1) return -1; if (x > 1) return 1; return x;
    case 12: if (x < 0) return .001 * x; if (x > 1) return .001 * (x - 1) + 1; return x;
    case 13: return (x >= 0) * 1.0507f * x + (x < 0) * 1.0507f * 1.6732f * (expf(x) - 1);
    case 14: { float sg = 1.f / (1.f + expf(-x)); return x * sg; }
    case 15: return x * tanh_ref(softplus_ref(x, 20));
    default: return x;
    }
}
static float act_grad(float x, int a) {   /* on the activation's output; the same in both back ends */
    switch (a) {
    case 0: return 1;
    case 1: return (x > 0);
    case 2: return (x > 0) ? 1 : .1;
    case 3: return (1 - x) * x;
    case 4: return (x > 0 && x < 6);
    case 5: return (x > 0) ? 1 : .01;
    case 6: return (x > 0) + .1;
    case 7: return 1 - x * x;
    case 8: return (x < 0 || x > 1) ? .01 : .125;
    case 9: return (x >= 0) + (x < 0) * (x + 1);
    case 10: { float y = (x + 1.) / 2.; return 2 * (1 - y) * y; }
    case 11: if (x > -1 && x < 1) return 1; return 0;
    case 12: if (x > 0 && x < 1) return 1; return .001;
    case 13: return (x >= 0) * 1.0507 + (x < 0) * (x + 1.0507 * 1.6732);
    default: return 1;
    }
}

void aeto_activate(float *y, size_t count, int activation, int mode) {
    if (activation == AETO_LINEAR) return;
    for (size_t i = 0; i < count; ++i) y[i] = mode == AETO_MODE_CPU ? act_cpu(y[i], activation) : act_mtcs(y[i], activation);
}

/* dnn/Activation.h:87-113 and dnn/Activation.c:233-239: delta *= f'(output). */
void aeto_gradient(const float *y, size_t count, int activation, float *delta) {
    if (activation == AETO_LINEAR) return;
    for (size_t i = 0; i < count; ++i) delta[i] *= act_grad(y[i], activation);
}

/* swish and mish, dnn/Activation.c:303-330: the gradient needs what the forward pass kept in `activation_input`
 * (sigmoid(v) for swish, v itself for mish); here `v` is the value before the activation for both. */
void aeto_gradient_input(const float *y, const float *v, size_t count, int activation, float *delta) {
    for (size_t i = 0; i < count; ++i) {
        if (activation == 14) {
            float sigmoid = 1.f / (1.f + expf(-v[i]));   /* logistic_activate, as activateArraySwish stored it */
            float swish = y[i];
            delta[i] *= swish + sigmoid * (1 - swish);
        } else if (activation == 15) {
            const float MISH_THRESHOLD = 20.0f;
            float inp = v[i];
            const float sp = softplus_ref(inp, MISH_THRESHOLD);
            const float grad_sp = 1 - exp(-sp);
            const float tsp = tanh(sp);
            const float grad_tsp = (1 - tsp * tsp) * grad_sp;
            const float grad = inp * grad_tsp + tsp;
            delta[i] *= grad;
        }
    }
}

/* ------------------------------------------------------------------ batch norm forward
 * CPU : dnn/NLayer.c:141-162; statistics dnn/NormData.c:141-186 (one pass, divisor m-1),
 *       rolling .9/.1 dnn/NormData.c:224-229, normalise dnn/NormData.c:244-282
 *       (x saved, x_hat = (x-mean) * 1/(sqrt(var)+1e-6), y = x_hat*gamma + beta),
 *       eval branch dnn/NormData.c:291-325.
 * MTCS: dnn/NLayer.c:224-226; statistics dnn/mtcs/MtcsNormData.c:54-133 (two pass, divisor m),
 *       rolling .99/.01 dnn/mtcs/MtcsNormData.c:193-232, normalise :336-347
 *       (x_hat = (x-mean)/sqrtf(var+1e-5)), eval branch :481-491. */
void aeto_bn_forward(int mode, int train, float *y, int batch, int c, int spatial,
                     const float *scales, const float *biases, float *mean, float *variance,
                     float *rolling_mean, float *rolling_variance, float *x, float *x_norm) {
    const size_t size = (size_t)c * spatial;
    if (train) {
        if (mode == AETO_MODE_CPU) {
            acc_t *t0 = (acc_t *)xcalloc((size_t)batch * c, sizeof(acc_t));
            acc_t *t1 = (acc_t *)xcalloc((size_t)batch * c, sizeof(acc_t));
            acc_t *t2 = (acc_t *)xcalloc((size_t)batch * c, sizeof(acc_t));
            for (int i = 0; i < batch; ++i)
                for (int j = 0; j < c; ++j)
                    for (int k = 0; k < spatial; ++k) {
                        float v = y[(size_t)i * size + (size_t)j * spatial + k];
                        t0[i * c + j] += v;
                        t1[i * c + j] += v * v;
                        t2[i * c + j] += -2 * v;
                    }
            float scale = 1. / (batch * spatial);
            for (int i = 0; i < c; ++i) {
                acc_t s = 0;
                for (int j = 0; j < batch; ++j) s += t0[j * c + i];
                mean[i] = (float)(s * scale);
            }
            scale = 1. / (batch * spatial - 1);
            for (int i = 0; i < c; ++i) {
                acc_t a = 0, b = 0;
                for (int j = 0; j < batch; ++j) { a += t1[j * c + i]; b += t2[j * c + i]; }
                acc_t v = a + b * mean[i] + (acc_t)mean[i] * mean[i] * batch * spatial;
                variance[i] = (float)(v * scale);
            }
            free(t0); free(t1); free(t2);
            for (int i = 0; i < c; ++i) {
                rolling_mean[i] *= .9f;      rolling_mean[i] += .1f * mean[i];
                rolling_variance[i] *= .9f;  rolling_variance[i] += .1f * variance[i];
            }
        } else {
            for (int f = 0; f < c; ++f) {
                acc_t s = 0;
                for (int j = 0; j < batch; ++j)
                    for (int k = 0; k < spatial; ++k) s += y[(size_t)j * size + (size_t)f * spatial + k];
                mean[f] = (float)(s / (spatial * batch));
                acc_t v = 0;
                for (int j = 0; j < batch; ++j)
                    for (int k = 0; k < spatial; ++k) {
                        float d = y[(size_t)j * size + (size_t)f * spatial + k] - mean[f];
                        v += d * d;
                    }
                variance[f] = (float)(v / (spatial * batch));
            }
            for (int i = 0; i < c; ++i) {
                rolling_mean[i] *= .99f;     rolling_mean[i] += .01f * mean[i];
                rolling_variance[i] *= .99f; rolling_variance[i] += .01f * variance[i];
            }
        }
    }
    const float *mu = train ? mean : rolling_mean;
    const float *var = train ? variance : rolling_variance;
    for (int b = 0; b < batch; ++b)
        for (int f = 0; f < c; ++f) {
            float inv = (mode == AETO_MODE_CPU) ? (float)(1.0 / (sqrt(var[f]) + .000001f)) : 0.0f;
            for (int i = 0; i < spatial; ++i) {
                size_t idx = (size_t)b * size + (size_t)f * spatial + i;
                float v = y[idx];
                if (x) x[idx] = v;
                if (mode == AETO_MODE_CPU) v = (v - mu[f]) * inv;
                else v = (v - mu[f]) / sqrtf(var[f] + .00001f);
                if (train && x_norm) x_norm[idx] = v;
                y[idx] = v * scales[f] + biases[f];
            }
        }
}

/* ------------------------------------------------------------------ batch norm backward
 * CPU : dnn/NLayer.c:246-278 -> dnn/ScaleData.c:76-107 (dgamma += sum delta*x_hat),
 *       dnn/NData.c:238-248 (delta *= gamma), dnn/DeltaData.c:23-38 (mean delta, eps 1e-5),
 *       :41-58 (variance delta), :64-80 (normalise delta).  The shift gradient is NOT computed.
 * MTCS: dnn/NLayer.c:281-324 -> dnn/mtcs/MtcsBiasData.c:27-45 (dbeta += sum delta) first, then the
 *       same sequence with the constants of dnn/mtcs/MtcsDeltaData.c:112,183,234. */
void aeto_bn_backward(int mode, float *delta, const float *x, const float *x_norm, const float *mean,
                      const float *variance, const float *scales, float *scale_updates,
                      float *bias_updates, float *mean_delta, float *variance_delta,
                      int batch, int c, int spatial) {
    const size_t size = (size_t)c * spatial;
    if (mode == AETO_MODE_MTCS) aeto_backward_bias(bias_updates, delta, batch, c, spatial);
    for (int f = 0; f < c; ++f) {
        acc_t sum = 0;
        for (int b = 0; b < batch; ++b)
            for (int i = 0; i < spatial; ++i) {
                size_t idx = (size_t)i + spatial * ((size_t)f + (size_t)c * b);
                sum += delta[idx] * x_norm[idx];
            }
        scale_updates[f] += (float)sum;
    }
    for (int b = 0; b < batch; ++b)
        for (int f = 0; f < c; ++f)
            for (int i = 0; i < spatial; ++i) delta[(size_t)b * size + (size_t)f * spatial + i] *= scales[f];
    for (int f = 0; f < c; ++f) {
        acc_t s = 0, v = 0;
        for (int b = 0; b < batch; ++b)
            for (int i = 0; i < spatial; ++i) {
                size_t idx = (size_t)b * size + (size_t)f * spatial + i;
                s += delta[idx];
                v += delta[idx] * (x[idx] - mean[f]);
            }
        if (mode == AETO_MODE_CPU) {
            mean_delta[f] = (float)(s * (-1. / sqrt(variance[f] + .00001f)));
            variance_delta[f] = (float)(v * (-.5 * pow(variance[f] + .00001f, (float)(-3. / 2.))));
        } else {
            mean_delta[f] = (float)s * (-1.F / sqrtf(variance[f] + .000001f));
            variance_delta[f] = (float)((float)v * (-.5 * powf(variance[f] + .000001f, (float)(-3. / 2.))));
        }
    }
    const int m = spatial * batch;
    for (int b = 0; b < batch; ++b)
        for (int f = 0; f < c; ++f)
            for (int i = 0; i < spatial; ++i) {
                size_t idx = (size_t)b * size + (size_t)f * spatial + i;
                if (mode == AETO_MODE_CPU)
                    delta[idx] = (float)(delta[idx] * 1. / (sqrt(variance[f] + .00001f))
                                         + variance_delta[f] * 2. * (x[idx] - mean[f]) / m + mean_delta[f] / m);
                else
                    delta[idx] = (float)(delta[idx] * 1.F / (sqrtf(variance[f]) + .000001f)
                                         + variance_delta[f] * 2. * (x[idx] - mean[f]) / m + mean_delta[f] / m);
            }
}

/* ------------------------------------------------------------------ max pool
 * dnn/MaxPoolLayer.c:40-41 (output size), :237-272 (forward, strict '>' in row/col scan order,
 * index = flat offset into the whole NCHW input, -1 when nothing beats the start value),
 * :318-331 (backward scatter-add).  Pad value: -FLT_MAX on CPU (:260), -INFINITY in
 * dnn/mtcs/MtcsMaxPoolLayer.c:82,92. */
int aeto_maxpool_out(int in, int size, int stride, int padding) { return (in + padding - size) / stride + 1; }

void aeto_maxpool_forward(int mode, const float *x, float *y, int *indexes, int batch, int c, int h, int w,
                          int size, int stride_x, int stride_y, int padding) {
    const int oh = aeto_maxpool_out(h, size, stride_y, padding), ow = aeto_maxpool_out(w, size, stride_x, padding);
    const int w_offset = -padding / 2, h_offset = -padding / 2;
    const float lowest = (mode == AETO_MODE_CPU) ? -FLT_MAX : -INFINITY;
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k)
            for (int i = 0; i < oh; ++i)
                for (int j = 0; j < ow; ++j) {
                    size_t out_index = (size_t)j + ow * ((size_t)i + oh * ((size_t)k + (size_t)c * b));
                    float max = lowest;
                    int max_i = -1;
                    for (int n = 0; n < size; ++n)
                        for (int m = 0; m < size; ++m) {
                            int cur_h = h_offset + i * stride_y + n, cur_w = w_offset + j * stride_x + m;
                            int index = cur_w + w * (cur_h + h * (k + b * c));
                            int valid = cur_h >= 0 && cur_h < h && cur_w >= 0 && cur_w < w;
                            float val = valid ? x[index] : lowest;
                            if (val > max) { max_i = index; max = val; }
                        }
                    y[out_index] = max;
                    if (indexes) indexes[out_index] = max_i;
                }
}

void aeto_maxpool_backward(const float *delta, const int *indexes, float *prev_delta, size_t out_count) {
    for (size_t i = 0; i < out_count; ++i)
        if (indexes[i] >= 0) prev_delta[indexes[i]] += delta[i];   /* the reference does not guard -1 */
}

/* dnn/AvgPoolLayer.c:29-46 (forward) and :73-88 (backward, += delta/(H*W)). */
void aeto_avgpool_forward(const float *x, float *y, int batch, int c, int spatial) {
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k) {
            acc_t s = 0;
            for (int i = 0; i < spatial; ++i) s += x[(size_t)i + spatial * ((size_t)k + (size_t)b * c)];
            y[k + (size_t)b * c] = (float)(s / spatial);
        }
}
void aeto_avgpool_backward(const float *delta, float *prev_delta, int batch, int c, int spatial) {
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k)
            for (int i = 0; i < spatial; ++i)
                prev_delta[(size_t)i + spatial * ((size_t)k + (size_t)b * c)] += delta[k + (size_t)b * c] / spatial;
}

/* ------------------------------------------------------------------ softmax + cross entropy
 * CPU : dnn/SoftMaxLayer.c:67-83 (max-subtracted, exp() in double, float running sum), :47-55
 *       (error = t ? -logf(p) : 0, delta = t - p), :99-119; cost = sum(error).
 * MTCS: dnn/SoftMaxLayer.c:122-139 (the running max is assigned through an `int`, i.e. each
 *       logit is truncated toward zero before the comparison; expf), :191-199; cost via
 *       dnn/mtcs/MtcsData.c:20-29 (host sum of the error array). */
float aeto_softmax_forward(int mode, const float *x, float *p, const float *truth, float *delta, float *loss,
                           int batch, int inputs, int groups, float temperature) {
    const int n = inputs / groups;
    for (int b = 0; b < batch; ++b)
        for (int g = 0; g < groups; ++g) {
            const float *in = x + (size_t)b * inputs + (size_t)g * n;
            float *out = p + (size_t)b * inputs + (size_t)g * n;
            float largest = (mode == AETO_MODE_CPU) ? -FLT_MAX : -INFINITY;
            for (int i = 0; i < n; ++i) {
                if (mode == AETO_MODE_CPU) { if (in[i] > largest) largest = in[i]; }
                else { int val = (int)in[i]; largest = (val > largest) ? (float)val : largest; }
            }
            acc_t sum = 0;
            for (int i = 0; i < n; ++i) {
                float e = (mode == AETO_MODE_CPU) ? (float)exp(in[i] / temperature - largest / temperature)
                                                  : expf(in[i] / temperature - largest / temperature);
                sum += e;
                out[i] = e;
            }
            for (int i = 0; i < n; ++i) out[i] = (float)(out[i] / (float)sum);
        }
    float cost = 0;
    if (truth) {
        acc_t s = 0;
        for (size_t i = 0; i < (size_t)batch * inputs; ++i) {
            float t = truth[i], q = p[i];
            loss[i] = t ? -logf(q) : 0;
            delta[i] = t - q;
            s += loss[i];
        }
        cost = (float)s;
    }
    return cost;
}

/* dnn/SoftMaxLayer.c:291-316: prev_delta += loss_scale * delta (loss_scale is 1 on the CPU path). */
void aeto_softmax_backward(const float *delta, float *prev_delta, size_t count, float loss_scale) {
    for (size_t i = 0; i < count; ++i) prev_delta[i] += loss_scale * delta[i];
}

/* ------------------------------------------------------------------ dropout
 * dnn/DropoutLayer.c:55-86; scale = 1/(1-p) (constructor).  The uniform draws are an input so that
 * the device generator and the oracle share one mask. */
void aeto_dropout_forward(float *x, const float *r, size_t count, float probability) {
    const float scale = 1.f / (1.f - probability);
    for (size_t i = 0; i < count; ++i) x[i] = (r[i] < probability) ? 0 : x[i] * scale;
}
void aeto_dropout_backward(float *delta, const float *r, size_t count, float probability) {
    const float scale = 1.f / (1.f - probability);
    for (size_t i = 0; i < count; ++i) delta[i] = (r[i] < probability) ? 0 : delta[i] * scale;
}

/* ------------------------------------------------------------------ SGD with momentum
 * dnn/ConvolutionalLayer.c:959-980: U += (-decay*batch) W; W += (lr/batch) U; U *= momentum for
 * weights; biases and BN scales skip the decay term. */
void aeto_sgd_weights(float *w, float *u, size_t count, int batch, float lr, float momentum, float decay) {
    const float a = -decay * batch, s = lr / batch;
    for (size_t i = 0; i < count; ++i) u[i] += a * w[i];
    for (size_t i = 0; i < count; ++i) w[i] += s * u[i];
    for (size_t i = 0; i < count; ++i) u[i] *= momentum;
}
void aeto_sgd_plain(float *p, float *u, size_t count, int batch, float lr, float momentum) {
    const float s = lr / batch;
    for (size_t i = 0; i < count; ++i) p[i] += s * u[i];
    for (size_t i = 0; i < count; ++i) u[i] *= momentum;
}

/* ================================================================== whole network
 * Restates dnn/NNetwork.c:382-396 (forward: zero each layer's delta, run it, hand its output on),
 * :627-654 (backward: last layer first, previous layer's output/delta as input/delta, layer 0 gets
 * the caller's delta which may be NULL), :611-624 (cost), :667-680 (update), :740-758 (train). */
typedef struct olayer {
    aeto_layer_spec s;
    int c, h, w, oc, oh, ow;
    size_t inputs, outputs, nweights;
    float *output, *delta;
    float *weights, *weight_updates, *biases, *bias_updates, *scales, *scale_updates;
    float *mean, *variance, *rolling_mean, *rolling_variance, *mean_delta, *variance_delta, *x, *x_norm;
    float *act_input;   /* swish / mish: the value before the activation */
    int *indexes;
    float *loss, *rnd;
    float cost;
} olayer;

struct aeto_net {
    int n, batch, c, h, w, mode, threads;
    olayer *l;
    float *workspace;
    size_t workspace_elems;
    const float *truth;
    int last_stop;        /* index of the last layer with stopbackward (-1: none) */
    long iteration;       /* updates requested so far through aeto_net_train_step (seen / batch) */
};

aeto_net *aeto_net_create(const aeto_layer_spec *specs, int nlayers, int batch, int c, int h, int w,
                          int mode, int threads) {
    aeto_net *net = (aeto_net *)xcalloc(1, sizeof(*net));
    net->n = nlayers; net->batch = batch; net->c = c; net->h = h; net->w = w; net->mode = mode;
    net->threads = threads < 1 ? 1 : threads;
    net->l = (olayer *)xcalloc((size_t)nlayers, sizeof(olayer));
    net->last_stop = -1;
    for (int i = 0; i < nlayers; ++i)
        if (specs[i].stopbackward == 1) net->last_stop = i;
    int cc = c, hh = h, ww = w;
    for (int i = 0; i < nlayers; ++i) {
        olayer *L = &net->l[i];
        L->s = specs[i];
        L->c = cc; L->h = hh; L->w = ww;
        L->inputs = (size_t)cc * hh * ww;
        switch (L->s.type) {
        case AETO_CONV:
            L->oc = L->s.filters;
            L->oh = aeto_conv_out(hh, L->s.size, L->s.stride_y, L->s.pad);
            L->ow = aeto_conv_out(ww, L->s.size, L->s.stride_x, L->s.pad);
            L->nweights = (size_t)L->s.filters * cc * L->s.size * L->s.size;
            L->weights = (float *)xcalloc(L->nweights, sizeof(float));
            L->weight_updates = (float *)xcalloc(L->nweights, sizeof(float));
            L->biases = (float *)xcalloc((size_t)L->oc, sizeof(float));
            L->bias_updates = (float *)xcalloc((size_t)L->oc, sizeof(float));
            if (L->s.batch_normalize) {
                L->scales = (float *)xcalloc((size_t)L->oc, sizeof(float));
                for (int k = 0; k < L->oc; ++k) L->scales[k] = 1;
                L->scale_updates = (float *)xcalloc((size_t)L->oc, sizeof(float));
                L->mean = (float *)xcalloc((size_t)L->oc, sizeof(float));
                L->variance = (float *)xcalloc((size_t)L->oc, sizeof(float));
                L->rolling_mean = (float *)xcalloc((size_t)L->oc, sizeof(float));
                L->rolling_variance = (float *)xcalloc((size_t)L->oc, sizeof(float));
                L->mean_delta = (float *)xcalloc((size_t)L->oc, sizeof(float));
                L->variance_delta = (float *)xcalloc((size_t)L->oc, sizeof(float));
            }
            {
                size_t ws = aeto_conv_workspace(cc, hh, ww, L->s.size, L->s.stride_x, L->s.stride_y, L->s.pad);
                if (ws > net->workspace_elems) net->workspace_elems = ws;
            }
            break;
        case AETO_MAXPOOL:
            L->oc = cc;
            L->oh = aeto_maxpool_out(hh, L->s.size, L->s.stride_y, L->s.pad);
            L->ow = aeto_maxpool_out(ww, L->s.size, L->s.stride_x, L->s.pad);
            break;
        case AETO_AVGPOOL: L->oc = cc; L->oh = 1; L->ow = 1; break;
        default:           L->oc = cc; L->oh = hh; L->ow = ww; break;
        }
        L->outputs = (size_t)L->oc * L->oh * L->ow;
        if (L->s.type == AETO_DROPOUT) {
            /* dnn/NetworkFactory.c:644-650: dropout works in place on its predecessor's buffers. */
            L->output = net->l[i - 1].output;
            L->delta = net->l[i - 1].delta;
            L->rnd = (float *)xcalloc((size_t)batch * L->inputs, sizeof(float));
        } else {
            L->output = (float *)xcalloc((size_t)batch * L->outputs, sizeof(float));
            L->delta = (float *)xcalloc((size_t)batch * L->outputs, sizeof(float));
        }
        if (L->s.type == AETO_CONV && L->s.batch_normalize) {
            L->x = (float *)xcalloc((size_t)batch * L->outputs, sizeof(float));
            L->x_norm = (float *)xcalloc((size_t)batch * L->outputs, sizeof(float));
        }
        if (L->s.type == AETO_MAXPOOL) L->indexes = (int *)xcalloc((size_t)batch * L->outputs, sizeof(int));
        if (L->s.type == AETO_SOFTMAX) L->loss = (float *)xcalloc((size_t)batch * L->outputs, sizeof(float));
        cc = L->oc; hh = L->oh; ww = L->ow;
    }
    net->workspace = (float *)xcalloc(net->workspace_elems * (size_t)net->threads, sizeof(float));
    return net;
}

void aeto_net_free(aeto_net *net) {
    if (!net) return;
    for (int i = 0; i < net->n; ++i) {
        olayer *L = &net->l[i];
        if (L->s.type != AETO_DROPOUT) { free(L->output); free(L->delta); }
        free(L->weights); free(L->weight_updates); free(L->biases); free(L->bias_updates);
        free(L->scales); free(L->scale_updates); free(L->mean); free(L->variance);
        free(L->rolling_mean); free(L->rolling_variance); free(L->mean_delta); free(L->variance_delta);
        free(L->x); free(L->x_norm); free(L->indexes); free(L->loss); free(L->rnd); free(L->act_input);
    }
    free(net->l); free(net->workspace); free(net);
}

int aeto_net_layers(const aeto_net *net) { return net->n; }

void aeto_net_out_shape(const aeto_net *net, int layer, int *c, int *h, int *w) {
    *c = net->l[layer].oc; *h = net->l[layer].oh; *w = net->l[layer].ow;
}

float *aeto_net_param(aeto_net *net, int layer, int which, size_t *count) {
    olayer *L = &net->l[layer];
    size_t act = (size_t)net->batch * L->outputs, ch = (size_t)L->oc;
    float *p = NULL; size_t n = 0;
    switch (which) {
    case AETO_P_WEIGHTS:          p = L->weights; n = L->nweights; break;
    case AETO_P_WEIGHT_UPDATES:   p = L->weight_updates; n = L->nweights; break;
    case AETO_P_BIASES:           p = L->biases; n = ch; break;
    case AETO_P_BIAS_UPDATES:     p = L->bias_updates; n = ch; break;
    case AETO_P_SCALES:           p = L->scales; n = ch; break;
    case AETO_P_SCALE_UPDATES:    p = L->scale_updates; n = ch; break;
    case AETO_P_ROLLING_MEAN:     p = L->rolling_mean; n = ch; break;
    case AETO_P_ROLLING_VARIANCE: p = L->rolling_variance; n = ch; break;
    case AETO_P_MEAN:             p = L->mean; n = ch; break;
    case AETO_P_VARIANCE:         p = L->variance; n = ch; break;
    case AETO_P_OUTPUT:           p = L->output; n = act; break;
    case AETO_P_DELTA:            p = L->delta; n = act; break;
    case AETO_P_X:                p = L->x; n = act; break;
    case AETO_P_X_NORM:           p = L->x_norm; n = act; break;
    case AETO_P_INDEXES:          p = (float *)L->indexes; n = act; break;
    case AETO_P_LOSS:             p = L->loss; n = act; break;
    case AETO_P_RAND:             p = L->rnd; n = (size_t)net->batch * L->inputs; break;
    default: break;
    }
    if (!p) n = 0;
    if (count) *count = n;
    return p;
}

/* Batch-parallel variants used only by the timed multi-core baseline: images are independent in
 * the reference's per-image loops, so each worker thread owns a workspace slice and a contiguous
 * range of images; weight gradients are summed per thread and then combined in thread order. */
typedef struct conv_job {
    aeto_net *net; olayer *L; const float *in; float *prev_delta; float *dws; int tid, lo, hi, backward;
} conv_job;

static void *conv_worker(void *arg) {
    conv_job *j = (conv_job *)arg;
    aeto_net *net = j->net; olayer *L = j->L;
    const size_t in_sz = L->inputs, out_sz = L->outputs;
    float *ws = net->workspace + (size_t)j->tid * net->workspace_elems;
    if (j->hi <= j->lo) return NULL;
    if (!j->backward)
        aeto_conv_forward(j->in + (size_t)j->lo * in_sz, L->weights, L->output + (size_t)j->lo * out_sz, ws,
                          j->hi - j->lo, L->c, L->h, L->w, L->s.filters, L->s.size, L->s.stride_x, L->s.stride_y, L->s.pad);
    else
        aeto_conv_backward(j->in + (size_t)j->lo * in_sz, L->weights, L->delta + (size_t)j->lo * out_sz,
                           j->dws + (size_t)j->tid * L->nweights,
                           j->prev_delta ? j->prev_delta + (size_t)j->lo * in_sz : NULL, ws, j->hi - j->lo,
                           L->c, L->h, L->w, L->s.filters, L->s.size, L->s.stride_x, L->s.stride_y, L->s.pad);
    return NULL;
}

static void conv_run_threads(aeto_net *net, olayer *L, const float *in, float *prev_delta, float *dws, int backward) {
    const int T = net->threads;
    pthread_t *th = (pthread_t *)xcalloc((size_t)T, sizeof(pthread_t));
    conv_job *jobs = (conv_job *)xcalloc((size_t)T, sizeof(conv_job));
    for (int t = 0; t < T; ++t) {
        jobs[t] = (conv_job){net, L, in, prev_delta, dws, t, (int)((long)net->batch * t / T),
                             (int)((long)net->batch * (t + 1) / T), backward};
        if (pthread_create(&th[t], NULL, conv_worker, &jobs[t]) != 0) { fprintf(stderr, "aet_oracle: pthread_create failed\n"); abort(); }
    }
    for (int t = 0; t < T; ++t) pthread_join(th[t], NULL);
    free(th); free(jobs);
}

static void conv_forward_mt(aeto_net *net, olayer *L, const float *in) {
    if (net->threads > 1) { conv_run_threads(net, L, in, NULL, NULL, 0); return; }
    aeto_conv_forward(in, L->weights, L->output, net->workspace, net->batch, L->c, L->h, L->w,
                      L->s.filters, L->s.size, L->s.stride_x, L->s.stride_y, L->s.pad);
}

static void conv_backward_mt(aeto_net *net, olayer *L, const float *in, float *prev_delta) {
    if (net->threads > 1) {
        float *dws = (float *)xcalloc(L->nweights * (size_t)net->threads, sizeof(float));
        conv_run_threads(net, L, in, prev_delta, dws, 1);
        for (int t = 0; t < net->threads; ++t)
            for (size_t j = 0; j < L->nweights; ++j) L->weight_updates[j] += dws[(size_t)t * L->nweights + j];
        free(dws);
        return;
    }
    aeto_conv_backward(in, L->weights, L->delta, L->weight_updates, prev_delta, net->workspace, net->batch,
                       L->c, L->h, L->w, L->s.filters, L->s.size, L->s.stride_x, L->s.stride_y, L->s.pad);
}

/* dnn/ShortcutLayer.c:272-353 with weights == NULL: the per-sample loops of forwardMultilayer */
void aeto_shortcut_forward(const float *in, float *out, int batch, size_t outputs, int n, const float *const *add,
                           const size_t *add_outputs) {
    for (int b = 0; b < batch; ++b)
        for (size_t j = 0; j < outputs; ++j) {
            float v = in[(size_t)b * outputs + j];
            for (int i = 0; i < n; ++i)
                if (j < add_outputs[i]) v += add[i][(size_t)b * add_outputs[i] + j];
            out[(size_t)b * outputs + j] = v;
        }
}
/* dnn/ShortcutLayer.c:132-230 with weights == NULL */
void aeto_shortcut_backward(const float *delta, float *delta_out, int batch, size_t outputs, int n, float *const *layer_delta,
                            const size_t *add_outputs) {
    for (int b = 0; b < batch; ++b)
        for (size_t j = 0; j < outputs; ++j) {
            const float d = delta[(size_t)b * outputs + j];
            if (delta_out) delta_out[(size_t)b * outputs + j] += d;
            for (int i = 0; i < n; ++i)
                if (j < add_outputs[i]) layer_delta[i][(size_t)b * add_outputs[i] + j] += d;
        }
}

void aeto_net_forward(aeto_net *net, const float *x, const float *truth, int train) {
    const float *in = x;
    net->truth = truth;
    for (int i = 0; i < net->n; ++i) {
        olayer *L = &net->l[i];
        const size_t act = (size_t)net->batch * L->outputs;
        if (train && L->s.type != AETO_DROPOUT) memset(L->delta, 0, act * sizeof(float));
        switch (L->s.type) {
        case AETO_CONV:
            conv_forward_mt(net, L, in);
            if (L->s.batch_normalize)
                aeto_bn_forward(net->mode, train, L->output, net->batch, L->oc, L->oh * L->ow, L->scales, L->biases,
                                L->mean, L->variance, L->rolling_mean, L->rolling_variance, L->x, L->x_norm);
            else
                aeto_add_bias(L->output, L->biases, net->batch, L->oc, L->oh * L->ow);
            if (L->s.activation >= 14) {   /* swish / mish keep the value before the activation (dnn/ConvolutionalLayer.c:764-772) */
                if (!L->act_input) L->act_input = (float *)xcalloc(act, sizeof(float));
                memcpy(L->act_input, L->output, act * sizeof(float));
            }
            aeto_activate(L->output, act, L->s.activation, net->mode);
            break;
        case AETO_MAXPOOL:
            aeto_maxpool_forward(net->mode, in, L->output, L->indexes, net->batch, L->c, L->h, L->w,
                                 L->s.size, L->s.stride_x, L->s.stride_y, L->s.pad);
            break;
        case AETO_AVGPOOL:
            aeto_avgpool_forward(in, L->output, net->batch, L->c, L->h * L->w);
            break;
        case AETO_SOFTMAX:
            L->cost = aeto_softmax_forward(net->mode, in, L->output, truth, L->delta, L->loss, net->batch,
                                           (int)L->inputs, L->s.groups > 0 ? L->s.groups : 1,
                                           L->s.temperature > 0 ? L->s.temperature : 1.0f);
            break;
        case AETO_DROPOUT:
            if (train) aeto_dropout_forward(L->output, L->rnd, (size_t)net->batch * L->inputs, L->s.probability);
            break;
        case AETO_SHORTCUT: {
            const float *add[4];
            size_t add_outputs[4];
            for (int q = 0; q < L->s.n_from; ++q) { add[q] = net->l[L->s.from[q]].output; add_outputs[q] = net->l[L->s.from[q]].outputs; }
            aeto_shortcut_forward(in, L->output, net->batch, L->outputs, L->s.n_from, add, add_outputs);
            aeto_activate(L->output, act, L->s.activation, net->mode);
            break;
        }
        }
        in = L->output;
    }
}

void aeto_net_backward(aeto_net *net, const float *x, float *input_delta) {
    for (int i = net->n - 1; i >= 0; --i) {
        olayer *L = &net->l[i];
        const float *in = (i == 0) ? x : net->l[i - 1].output;
        float *pd = (i == 0) ? input_delta : net->l[i - 1].delta;
        const size_t act = (size_t)net->batch * L->outputs;
        if (L->s.stopbackward == 1) break;     /* dnn/NNetwork.c:648 */
        if (i < net->last_stop) continue;      /* onlyforward, dnn/NNetwork.c:650 with dnn/NetworkFactory.c:979-991 */
        switch (L->s.type) {
        case AETO_CONV:
            if (L->s.activation >= 14) aeto_gradient_input(L->output, L->act_input, act, L->s.activation, L->delta);
            else aeto_gradient(L->output, act, L->s.activation, L->delta);
            if (L->s.batch_normalize)
                aeto_bn_backward(net->mode, L->delta, L->x, L->x_norm, L->mean, L->variance, L->scales,
                                 L->scale_updates, L->bias_updates, L->mean_delta, L->variance_delta,
                                 net->batch, L->oc, L->oh * L->ow);
            else
                aeto_backward_bias(L->bias_updates, L->delta, net->batch, L->oc, L->oh * L->ow);
            conv_backward_mt(net, L, in, pd);
            break;
        case AETO_MAXPOOL:
            if (pd) aeto_maxpool_backward(L->delta, L->indexes, pd, act);
            break;
        case AETO_AVGPOOL:
            if (pd) aeto_avgpool_backward(L->delta, pd, net->batch, L->c, L->h * L->w);
            break;
        case AETO_SOFTMAX:
            if (pd) aeto_softmax_backward(L->delta, pd, act, 1.0f);
            break;
        case AETO_DROPOUT:
            if (pd) aeto_dropout_backward(pd, L->rnd, (size_t)net->batch * L->inputs, L->s.probability);
            break;
        case AETO_SHORTCUT: {
            float *ld[4];
            size_t add_outputs[4];
            for (int q = 0; q < L->s.n_from; ++q) { ld[q] = net->l[L->s.from[q]].delta; add_outputs[q] = net->l[L->s.from[q]].outputs; }
            aeto_gradient(L->output, act, L->s.activation, L->delta);   /* dnn/ShortcutLayer.c:232-243 */
            aeto_shortcut_backward(L->delta, pd, net->batch, L->outputs, L->s.n_from, ld, add_outputs);
            break;
        }
        }
    }
}

void aeto_net_update(aeto_net *net, int update_batch, float lr, float momentum, float decay) {
    for (int i = 0; i < net->n; ++i) {
        olayer *L = &net->l[i];
        if (L->s.type != AETO_CONV) continue;
        if (i < net->last_stop) continue;      /* train == 0, dnn/NNetwork.c:672,688 */
        /* dnn/NNetwork.c:703, updateMTCS only: updateCPU (:667-680) does not look at dont_update */
        /* (an update asked for before any training call counts as iteration 1, so that a bare update still updates) */
        if (net->mode == AETO_MODE_MTCS && !((long)L->s.dont_update < (net->iteration > 0 ? net->iteration : 1))) continue;
        float rate = lr * (L->s.learning_rate_scale != 0 ? L->s.learning_rate_scale : 1.0f);
        aeto_sgd_weights(L->weights, L->weight_updates, L->nweights, update_batch, rate, momentum, decay);
        aeto_sgd_plain(L->biases, L->bias_updates, (size_t)L->oc, update_batch, rate, momentum);
        if (L->scales) aeto_sgd_plain(L->scales, L->scale_updates, (size_t)L->oc, update_batch, rate, momentum);
    }
}

float aeto_net_cost(const aeto_net *net) {
    float sum = 0; int count = 0;
    for (int i = 0; i < net->n; ++i)
        if (net->l[i].s.type == AETO_SOFTMAX) { sum += net->l[i].cost; ++count; }
    return count ? sum / count : 0;
}

float aeto_net_train_step(aeto_net *net, const float *x, const float *truth, float lr, float momentum, float decay) {
    aeto_net_forward(net, x, truth, 1);
    aeto_net_backward(net, x, NULL);
    float cost = aeto_net_cost(net);
    net->iteration += 1;   /* seen += batch before forward (dnn/NNetwork.c:742); iteration_num = seen / batch at the update */
    aeto_net_update(net, net->batch, lr, momentum, decay);
    return cost / net->batch;
}

void aeto_fill_uniform(float *dst, size_t n, uint64_t seed, uint64_t tensor_id) {
    aet_rng_fill_uniform(dst, n, seed, tensor_id);
}
void aeto_fill_normal(float *dst, size_t n, uint64_t seed, uint64_t tensor_id, float mean, float stddev) {
    aet_rng_fill_normal(dst, n, seed, tensor_id, mean, stddev);
}

/* ------------------------------------------------------------------ learning-rate schedule
 * dnn/NNetwork.c:215-246, expression by expression: batch_num is a size_t there, so `batch_num / step`,
 * `batch_num < burn_in` and `batch_num - step` are unsigned arithmetic (the sig policy's difference wraps
 * while batch_num < step), and pow / exp are the double functions. */
float aeto_current_rate(size_t batch_num, int policy, float learning_rate, int burn_in, float power, int step, float scale,
                        const int *steps, const float *scales, int num_steps, float gamma, int max_batches) {
    int i;
    float rate;
    if (batch_num < (size_t)burn_in) return (float)(learning_rate * pow((float)batch_num / burn_in, power));
    switch (policy) {
    case 0: return learning_rate;
    case 1: return (float)(learning_rate * pow(scale, batch_num / step));
    case 2:
        rate = learning_rate;
        for (i = 0; i < num_steps; ++i) {
            if ((size_t)steps[i] > batch_num) return rate;
            rate *= scales[i];
        }
        return rate;
    case 3: return (float)(learning_rate * pow(gamma, (int)batch_num));
    case 4: return (float)(learning_rate * pow(1 - (float)batch_num / max_batches, power));
    case 5: return (float)(learning_rate * (1. / (1. + exp(gamma * (batch_num - step)))));
    default: return learning_rate;
    }
}

/* mtcs/MtcsTool.c:77-107 */
void aeto_fix_nan_and_inf(float *v, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (isnan(v[i]) || isinf(v[i])) v[i] = 1.0f / (fabsf((float)i) + 1);
}
void aeto_reset_nan_and_inf(float *v, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (isnan(v[i]) || isinf(v[i])) v[i] = 0;
}

/* dnn/ConvolutionalLayer.c:983-1003 */
void aeto_fuse_conv_batchnorm(float *biases, const float *scales, const float *rolling_mean, const float *rolling_variance,
                              float *weights, int filters, size_t filter_size) {
    for (int f = 0; f < filters; ++f) {
        biases[f] = biases[f] - (double)scales[f] * rolling_mean[f] / (sqrt((double)rolling_variance[f] + .00001));
        double precomputed = scales[f] / (sqrt((double)rolling_variance[f] + .00001));
        for (size_t i = 0; i < filter_size; ++i) {
            size_t w_index = (size_t)f * filter_size + i;
            weights[w_index] *= precomputed;
        }
    }
}

/* dnn/DnnUtils.c:463-477 */
void aeto_top_k(const float *a, int n, int k, int *index) {
    int i, j;
    for (j = 0; j < k; ++j) index[j] = -1;
    for (i = 0; i < n; ++i) {
        int curr = i;
        for (j = 0; j < k; ++j) {
            if ((index[j] < 0) || a[curr] > a[index[j]]) {
                int swap = curr;
                curr = index[j];
                index[j] = swap;
            }
        }
    }
}

/* dnn/ConvolutionalLayer.c:444-454 */
void aeto_transpose_matrix(float *a, int rows, int cols) {
    float *transpose = (float *)calloc((size_t)rows * cols, sizeof(float));
    for (int x = 0; x < rows; ++x)
        for (int y = 0; y < cols; ++y) transpose[(size_t)y * rows + x] = a[(size_t)x * cols + y];
    memcpy(a, transpose, (size_t)rows * cols * sizeof(float));
    free(transpose);
}

/* ------------------------------------------------------------------ image augmentation (dnn/NImage.c) */
static float img_pixel_extend(const float *im, int w, int h, int c, int x, int y, int k) {   /* :138-144 */
    if (x < 0 || x >= w || y < 0 || y >= h) return 0;
    if (k < 0 || k >= c) return 0;
    return im[(size_t)k * h * w + (size_t)y * w + x];
}
static float img_bilinear(const float *im, int w, int h, int c, float x, float y, int k) {     /* :146-157 */
    int ix = (int)floorf(x);
    int iy = (int)floorf(y);
    float dx = x - ix;
    float dy = y - iy;
    float val = (1 - dy) * (1 - dx) * img_pixel_extend(im, w, h, c, ix, iy, k) +
                dy * (1 - dx) * img_pixel_extend(im, w, h, c, ix, iy + 1, k) +
                (1 - dy) * dx * img_pixel_extend(im, w, h, c, ix + 1, iy, k) +
                dy * dx * img_pixel_extend(im, w, h, c, ix + 1, iy + 1, k);
    return val;
}
static float three_way_max(float a, float b, float c) { return (a > b) ? ((a > c) ? a : c) : ((b > c) ? b : c); }
static float three_way_min(float a, float b, float c) { return (a < b) ? ((a < c) ? a : c) : ((b < c) ? b : c); }

void aeto_augment_image(const float *src, int c, int sh, int sw, float *dst, int size, float rad, float s, float dx, float dy,
                        float aspect, int flip, float dhue, float dsat, float dexp) {
    const int w = size, h = size;
    /* rotateCrop :551-572 */
    float cx = sw / 2.0;
    float cy = sh / 2.0;
    float cr = cos(rad);
    float sr = sin(rad);
    float dx1 = dx / s * aspect;
    float dy1 = dy / s;
    for (int k = 0; k < c; ++k)
        for (int y = 0; y < h; ++y)
            for (int x = 0; x < w; ++x) {
                float rx = cr * ((x - w / 2.) / s * aspect + dx1) - sr * ((y - h / 2.) / s + dy1) + cx;
                float ry = sr * ((x - w / 2.) / s * aspect + dx1) + cr * ((y - h / 2.) / s + dy1) + cy;
                dst[(size_t)k * h * w + (size_t)y * w + x] = img_bilinear(src, sw, sh, c, rx, ry, k);
            }
    /* flip :346-362 */
    if (flip)
        for (int k = 0; k < c; ++k)
            for (int i = 0; i < h; ++i)
                for (int j = 0; j < w / 2; ++j) {
                    size_t index = j + (size_t)w * (i + (size_t)h * k), fl = (w - j - 1) + (size_t)w * (i + (size_t)h * k);
                    float swap = dst[fl];
                    dst[fl] = dst[index];
                    dst[index] = swap;
                }
    if (c != 3) return;
    /* distort :323-337 */
    const size_t wh = (size_t)w * h;
    for (size_t p = 0; p < wh; ++p) {
        float r = dst[p], g = dst[wh + p], b = dst[2 * wh + p];
        float hh, ss, vv;
        /* rgbToHsv :201-243 */
        float max = three_way_max(r, g, b);
        float min = three_way_min(r, g, b);
        float delta = max - min;
        vv = max;
        if (max == 0) {
            ss = 0;
            hh = 0;
        } else {
            ss = delta / max;
            if (r == max) hh = (g - b) / delta;
            else if (g == max) hh = 2 + (b - r) / delta;
            else hh = 4 + (r - g) / delta;
            if (hh < 0) hh += 6;
            hh = hh / 6.;
        }
        ss = ss * dsat;       /* scaleChannel(1, sat) */
        vv = vv * dexp;       /* scaleChannel(2, val) */
        hh = hh + dhue;
        if (hh > 1) hh -= 1;
        if (hh < 0) hh += 1;
        /* hsvToRgb :245-291 */
        float hq = 6 * hh;
        if (ss == 0) {
            r = g = b = vv;
        } else {
            int index = floor(hq);
            float f = hq - index;
            float pp = vv * (1 - ss);
            float q = vv * (1 - ss * f);
            float t = vv * (1 - ss * (1 - f));
            if (index == 0) { r = vv; g = t; b = pp; }
            else if (index == 1) { r = q; g = vv; b = pp; }
            else if (index == 2) { r = pp; g = vv; b = t; }
            else if (index == 3) { r = pp; g = q; b = vv; }
            else if (index == 4) { r = t; g = pp; b = vv; }
            else { r = vv; g = pp; b = q; }
        }
        /* constrainImage :309-318 */
        float out[3] = {r, g, b};
        for (int k = 0; k < 3; ++k) {
            if (out[k] < 0) out[k] = 0;
            if (out[k] > 1) out[k] = 1;
            dst[k * wh + p] = out[k];
        }
    }
}

/* ------------------------------------------------------------------ groups and dilation
 * im2col_cpu_ext / col2im_cpu_ext, dnn/Im2Col.c:65-103 and :155-192. */
static void im2col_ext(const float *data_im, int channels, int height, int width, int kernel_h, int kernel_w, int pad_h, int pad_w,
                       int stride_h, int stride_w, int dilation_h, int dilation_w, float *data_col) {
    const int output_h = (height + 2 * pad_h - (dilation_h * (kernel_h - 1) + 1)) / stride_h + 1;
    const int output_w = (width + 2 * pad_w - (dilation_w * (kernel_w - 1) + 1)) / stride_w + 1;
    const int channel_size = height * width;
    for (int channel = channels; channel--; data_im += channel_size)
        for (int kernel_row = 0; kernel_row < kernel_h; kernel_row++)
            for (int kernel_col = 0; kernel_col < kernel_w; kernel_col++) {
                int input_row = -pad_h + kernel_row * dilation_h;
                for (int output_rows = output_h; output_rows; output_rows--) {
                    if ((unsigned)input_row >= (unsigned)height) {
                        for (int output_col = output_w; output_col; output_col--) *(data_col++) = 0;
                    } else {
                        int input_col = -pad_w + kernel_col * dilation_w;
                        for (int output_col = output_w; output_col; output_col--) {
                            *(data_col++) = ((unsigned)input_col < (unsigned)width) ? data_im[input_row * width + input_col] : 0;
                            input_col += stride_w;
                        }
                    }
                    input_row += stride_h;
                }
            }
}
static void col2im_ext(const float *data_col, int channels, int height, int width, int kernel_h, int kernel_w, int pad_h, int pad_w,
                       int stride_h, int stride_w, int dilation_h, int dilation_w, float *data_im) {
    memset(data_im, 0, sizeof(float) * (size_t)height * width * channels);
    const int output_h = (height + 2 * pad_h - (dilation_h * (kernel_h - 1) + 1)) / stride_h + 1;
    const int output_w = (width + 2 * pad_w - (dilation_w * (kernel_w - 1) + 1)) / stride_w + 1;
    const int channel_size = height * width;
    for (int channel = channels; channel--; data_im += channel_size)
        for (int kernel_row = 0; kernel_row < kernel_h; kernel_row++)
            for (int kernel_col = 0; kernel_col < kernel_w; kernel_col++) {
                int input_row = -pad_h + kernel_row * dilation_h;
                for (int output_rows = output_h; output_rows; output_rows--) {
                    if ((unsigned)input_row >= (unsigned)height) {
                        data_col += output_w;
                    } else {
                        int input_col = -pad_w + kernel_col * dilation_w;
                        for (int output_col = output_w; output_col; output_col--) {
                            if ((unsigned)input_col < (unsigned)width) data_im[input_row * width + input_col] += *data_col;
                            data_col++;
                            input_col += stride_w;
                        }
                    }
                    input_row += stride_h;
                }
            }
}

/* dnn/ConvolutionalLayer.c:703-806, FP32 branch */
void aeto_conv_forward_ex(const float *x, const float *weights, float *y, float *workspace, int batch, int c, int h, int w,
                          int nf, int size, int stride_x, int stride_y, int pad, int groups, int dilation) {
    const int out_h = aeto_conv_out(h, size, stride_y, pad), out_w = aeto_conv_out(w, size, stride_x, pad);
    const int m = nf / groups, k = size * size * c / groups, n = out_h * out_w;
    const size_t nweights = (size_t)nf * k;
    memset(y, 0, sizeof(float) * (size_t)batch * nf * n);
    for (int i = 0; i < batch; ++i)
        for (int j = 0; j < groups; ++j) {
            const float *im = x + (size_t)(i * groups + j) * (c / groups) * h * w;
            const float *a = weights + j * nweights / groups;
            const float *b = im;
            float *cc = y + (size_t)(i * groups + j) * n * m;
            if (!(size == 1 && stride_x == 1 && stride_y == 1 && dilation == 1)) {
                im2col_ext(im, c / groups, h, w, size, size, pad * dilation, pad * dilation, stride_y, stride_x, dilation, dilation, workspace);
                b = workspace;
            }
            aeto_gemm(0, 0, m, n, k, 1, a, k, b, n, 1, cc, n);
        }
}

/* dnn/ConvolutionalLayer.c:909-947 */
void aeto_conv_backward_ex(const float *x, const float *weights, const float *delta, float *dw, float *dx, float *workspace,
                           int batch, int c, int h, int w, int nf, int size, int stride_x, int stride_y, int pad, int groups,
                           int dilation) {
    const int out_h = aeto_conv_out(h, size, stride_y, pad), out_w = aeto_conv_out(w, size, stride_x, pad);
    const int m = nf / groups, n = size * size * c / groups, k = out_h * out_w;
    const size_t nweights = (size_t)nf * n;
    for (int i = 0; i < batch; ++i)
        for (int j = 0; j < groups; ++j) {
            const float *a = delta + (size_t)(i * groups + j) * m * k;
            float *cc = dw + j * nweights / groups;
            const float *im = x + (size_t)(i * groups + j) * (c / groups) * h * w;
            im2col_ext(im, c / groups, h, w, size, size, pad * dilation, pad * dilation, stride_y, stride_x, dilation, dilation, workspace);
            aeto_gemm(0, 1, m, n, k, 1, a, k, workspace, k, 1, cc, n);
            if (dx) {
                const float *wa = weights + j * nweights / groups;
                aeto_gemm(1, 0, n, k, m, 1, wa, n, a, k, 0, workspace, k);
                col2im_ext(workspace, c / groups, h, w, size, size, pad * dilation, pad * dilation, stride_y, stride_x, dilation, dilation,
                           dx + (size_t)(i * groups + j) * (c / groups) * h * w);
            }
        }
}

/* mtcs/MtcsConvLayer.c:494-524 (scal, scal, axpy, axpy, mul, axpy, adam_kernel, fill), element by element */
void aeto_adam_update(float *w, float *d, float *m, float *v, float B1, float B2, float eps, float decay, float rate, size_t n,
                      int batch, int t) {
    for (size_t i = 0; i < n; ++i) {
        m[i] *= B1;
        v[i] *= B2;
        d[i] += (-decay * batch) * w[i];
        m[i] += (1 - B1) * d[i];
        d[i] = d[i] * d[i];
        v[i] += (1 - B2) * d[i];
        float mhat = m[i] / (1.f - powf(B1, t));
        float vhat = v[i] / (1.f - powf(B2, t));
        w[i] = w[i] + rate * mhat / (sqrtf(vhat) + eps);
        d[i] = 0;
    }
}
