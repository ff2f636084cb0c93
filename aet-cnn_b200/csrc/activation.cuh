// Activation functions and their gradients, one definition for the convolution epilogues and the streaming
// kernels.  Formulas are the reference's GPU ones (mtcs/MtcsActivation.c:17-103 forward, :393-470 gradients;
// CPU twins dnn/Activation.h:41-113): every gradient is a function of the activation's OUTPUT, which is what lets
// the backward kernels recompute it from the stored result (dnn/Activation.c:233-239).
#pragma once
#include "../../include/aet_b200.h"

// The rarely used types live in functions of their own that are never inlined: the hot kernels apply an activation
// per element inside unrolled loops, and a fourteen-way switch inlined there costs them a third of their speed.
__host__ __device__ __noinline__ static float act_forward_other(float x, int act) {
    switch (act) {
    case AET_LOGISTIC: return 1.f / (1.f + expf(-x));
    case AET_RELU6: return fminf(fmaxf(x, 0.f), 6.f);
    case AET_RELIE: return x > 0.f ? x : .01f * x;
    case AET_RAMP: return x * (x > 0.f) + .1f * x;
    case AET_TANH: return 2.f / (1.f + expf(-2.f * x)) - 1.f;
    case AET_PLSE: return x < -4.f ? .01f * (x + 4.f) : (x > 4.f ? .01f * (x - 4.f) + 1.f : .125f * x + .5f);
    case AET_ELU: return (x >= 0.f) * x + (x < 0.f) * (expf(x) - 1.f);
    case AET_LOGGY: return 2.f / (1.f + expf(-x)) - 1.f;
    case AET_HARDTAN: return x < -1.f ? -1.f : (x > 1.f ? 1.f : x);
    case AET_LHTAN: return x < 0.f ? .001f * x : (x > 1.f ? .001f * (x - 1.f) + 1.f : x);
    case AET_SELU: return (x >= 0.f) * 1.0507f * x + (x < 0.f) * 1.0507f * 1.6732f * (expf(x) - 1.f);
    case AET_SWISH: return x * (1.f / (1.f + expf(-x)));                                  // dnn/IOData.c:75-88
    case AET_MISH: {                                                                      // dnn/IOData.c:92-105
        const float sp = x > 20.f ? x : (x < -20.f ? expf(x) : logf(expf(x) + 1.f));       // softplus, threshold 20
        return x * (2.f / (1.f + expf(-2.f * sp)) - 1.f);
    }
    default: return x;
    }
}
__host__ __device__ __forceinline__ float act_forward(float x, int act) {
    if (act == AET_LEAKY) return x > 0.f ? x : 0.1f * x;
    if (act == AET_RELU) return x > 0.f ? x : 0.f;
    if (act == AET_LINEAR) return x;
    return act_forward_other(x, act);
}

// d activation / d input, evaluated on the activation's output y
__host__ __device__ __noinline__ static float act_gradient_other(float y, int act) {
    switch (act) {
    case AET_LOGISTIC: return (1.f - y) * y;
    case AET_RELU6: return (y > 0.f && y < 6.f) ? 1.f : 0.f;
    case AET_RELIE: return y > 0.f ? 1.f : .01f;
    case AET_RAMP: return (y > 0.f) + .1f;
    case AET_TANH: return 1.f - y * y;
    case AET_PLSE: return (y < 0.f || y > 1.f) ? .01f : .125f;
    case AET_ELU: return (y >= 0.f) + (y < 0.f) * (y + 1.f);
    case AET_LOGGY: { const float t = (y + 1.f) / 2.f; return 2.f * (1.f - t) * t; }
    case AET_HARDTAN: return (y > -1.f && y < 1.f) ? 1.f : 0.f;
    case AET_LHTAN: return (y > 0.f && y < 1.f) ? 1.f : .001f;
    case AET_SELU: return (y >= 0.f) * 1.0507f + (y < 0.f) * (y + 1.0507f * 1.6732f);
    default: return 1.f;
    }
}
__host__ __device__ __forceinline__ float act_gradient(float y, int act) {
    if (act == AET_LEAKY) return y > 0.f ? 1.f : 0.1f;
    if (act == AET_RELU) return y > 0.f ? 1.f : 0.f;
    if (act == AET_LINEAR) return 1.f;
    return act_gradient_other(y, act);
}

// swish and mish: d activation / d input as a function of the INPUT v (dnn/Activation.c:303-330; the reference keeps
// sigmoid(v), respectively v, in a side buffer for this, the kernels here recompute v)
__host__ __device__ __noinline__ static float act_gradient_input_other(float v, int act) {
    if (act == AET_SWISH) {
        const float sg = 1.f / (1.f + expf(-v)), sw = v * sg;
        return sw + sg * (1.f - sw);
    }
    const float sp = v > 20.f ? v : (v < -20.f ? expf(v) : logf(expf(v) + 1.f));
    const float grad_sp = 1.f - expf(-sp);
    const float tsp = tanhf(sp);
    const float grad_tsp = (1.f - tsp * tsp) * grad_sp;
    return v * grad_tsp + tsp;
}
__host__ __device__ __forceinline__ bool act_needs_input(int act) { return act >= AET_SWISH; }
// gradient of any supported activation from the value before the activation
__host__ __device__ __forceinline__ float act_gradient_pre(float v, int act) {
    if (act < AET_SWISH) return act_gradient(act_forward(v, act), act);
    return act_gradient_input_other(v, act);
}
