// Pointwise objective math shared by the derivative, leaf-estimation and metric kernels.
// der = -dLoss/dApprox (the ascent direction CatBoost calls "der"), hess = d2Loss/dApprox2 >= 0.
// Formulas follow catboost/private/libs/algo_helpers/error_functions.h (RMSE :191, Logloss/CrossEntropy,
// Poisson, Quantile, MAPE, Huber, Lq, Expectile, Tweedie, LogCosh) and
// catboost/cuda/targets/kernel/pointwise_targets.cu:246-327.
#pragma once
#include "cb_common.cuh"

enum CbLoss : int {
    CB_LOSS_RMSE = 0,
    CB_LOSS_LOGLOSS = 1,
    CB_LOSS_CROSSENTROPY = 2,
    CB_LOSS_POISSON = 3,
    CB_LOSS_MAE = 4,
    CB_LOSS_QUANTILE = 5,
    CB_LOSS_LOGLINQUANTILE = 6,
    CB_LOSS_MAPE = 7,
    CB_LOSS_HUBER = 8,
    CB_LOSS_LQ = 9,
    CB_LOSS_EXPECTILE = 10,
    CB_LOSS_TWEEDIE = 11,
    CB_LOSS_LOGCOSH = 12,
    CB_LOSS_EXTERNAL = 100,   // der/hess supplied by the host side (ranking, multiclass, custom objectives)
};

struct CbLossOut {
    float der;
    float hess;
    float value;
};

__device__ __forceinline__ CbLossOut cb_loss_eval(int loss, float p0, float p1, float a, float y) {
    CbLossOut o;
    switch (loss) {
        default:
        case CB_LOSS_RMSE: {
            float d = y - a;
            o.der = d; o.hess = 1.0f; o.value = d * d;
            break;
        }
        case CB_LOSS_LOGLOSS:
        case CB_LOSS_CROSSENTROPY: {
            float p = 1.0f / (1.0f + __expf(-a));
            o.der = y - p;
            o.hess = fmaxf(p * (1.0f - p), 1e-16f);
            // log(1+e^a) - y a, stable for both signs
            // softplus, stable for both signs; the fast logarithm is off by at most 6e-8 per document (the reported loss
            // is a mean of these)
            float sp = fmaxf(a, 0.0f) + __logf(1.0f + __expf(-fabsf(a)));
            o.value = sp - y * a;
            break;
        }
        case CB_LOSS_POISSON: {
            float e = __expf(a);
            o.der = y - e; o.hess = e; o.value = e - y * a;
            break;
        }
        case CB_LOSS_MAE: {
            float d = y - a;
            o.der = (d > 0.0f) ? 1.0f : ((d < 0.0f) ? -1.0f : 0.0f);
            o.hess = 1.0f; o.value = fabsf(d);
            break;
        }
        case CB_LOSS_QUANTILE: {   // p0 = alpha, p1 = delta
            float d = y - a;
            bool up = d > p1, dn = d < -p1;
            o.der = up ? p0 : (dn ? -(1.0f - p0) : 0.0f);
            o.hess = 1.0f;
            o.value = up ? p0 * d : (dn ? -(1.0f - p0) * d : 0.0f);
            break;
        }
        case CB_LOSS_LOGLINQUANTILE: {
            float e = __expf(a);
            float d = y - e;
            o.der = (d > 0.0f) ? p0 * e : -(1.0f - p0) * e;
            o.hess = 1.0f;
            o.value = (d > 0.0f) ? p0 * d : -(1.0f - p0) * d;
            break;
        }
        case CB_LOSS_MAPE: {
            float d = y - a;
            float s = 1.0f / fmaxf(1.0f, fabsf(y));
            o.der = ((d > 0.0f) ? 1.0f : ((d < 0.0f) ? -1.0f : 0.0f)) * s;
            o.hess = 1.0f; o.value = fabsf(d) * s;
            break;
        }
        case CB_LOSS_HUBER: {      // p0 = delta
            float d = y - a;
            float ad = fabsf(d);
            if (ad <= p0) { o.der = d; o.hess = 1.0f; o.value = 0.5f * d * d; }
            else { o.der = (d > 0.0f) ? p0 : -p0; o.hess = 1e-6f; o.value = p0 * (ad - 0.5f * p0); }
            break;
        }
        case CB_LOSS_LQ: {         // p0 = q
            float d = y - a;
            float ad = fabsf(d);
            o.value = __powf(ad, p0);
            o.der = p0 * __powf(ad, p0 - 1.0f) * ((d > 0.0f) ? 1.0f : -1.0f);
            o.hess = (p0 >= 2.0f) ? p0 * (p0 - 1.0f) * __powf(ad, p0 - 2.0f) : 1.0f;
            if (ad == 0.0f) { o.der = 0.0f; o.hess = (p0 == 2.0f) ? 2.0f : 1.0f; }
            break;
        }
        case CB_LOSS_EXPECTILE: {  // p0 = alpha
            float d = y - a;
            float w = (d > 0.0f) ? p0 : (1.0f - p0);
            o.der = 2.0f * w * d; o.hess = 2.0f * w; o.value = w * d * d;
            break;
        }
        case CB_LOSS_TWEEDIE: {    // p0 = variance power in (1,2)
            float e1 = __expf((1.0f - p0) * a);
            float e2 = __expf((2.0f - p0) * a);
            o.der = y * e1 - e2;
            o.hess = fmaxf(-y * (1.0f - p0) * e1 + (2.0f - p0) * e2, 1e-16f);
            o.value = -y * e1 / (1.0f - p0) + e2 / (2.0f - p0);
            break;
        }
        case CB_LOSS_LOGCOSH: {
            float d = y - a;
            float t = tanhf(d);
            o.der = t; o.hess = fmaxf(1.0f - t * t, 1e-6f);
            float ad = fabsf(d);
            o.value = ad + log1pf(__expf(-2.0f * ad)) - 0.69314718056f;
            break;
        }
    }
    return o;
}
