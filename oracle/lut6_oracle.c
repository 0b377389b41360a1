/* TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement, in plain C, of the arithmetic of BinaryBrain's 6-input LUT layer family.
 * It is the checker the CUDA kernels are compared with; the product never links, imports or
 * executes it.  Every function names the reference code (file:line inside ryuz/BinaryBrain
 * v4.3.2) whose results it restates.
 *
 * Parity status: PINNED.  tests/test_oracle_pin.py compares every function below with the
 * unmodified reference headers compiled into oracle/_ref/libbbref.so (oracle/ref_driver.cpp),
 * and with the committed fixtures under tests/golden/ that were produced by that library.
 *
 * Layouts (host memory):
 *   fp32 frames : row per node, `stride` floats per row, frame f at row[f]
 *   bit frames  : row per node, `stride` uint32 per row, frame f = bit (f & 31) of word (f >> 5)
 *                 (include/bb/DataType.h:612-647, LSB first)
 *   wiring      : idx[node*6 + k]                         (include/bb/FixedSizeConnectionTable.h:24-216)
 *   W           : W[node*64 + i], bit k of i <-> input k  (include/bb/StochasticOperation.h:95-114)
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <math.h>
#include <float.h>

typedef struct {
    int   binary;        /* x -> 0.5 +/- bias by (x > 0.5)  (fp32 input only; bit input always is) */
    int   lut_binarize;  /* W -> {0,1} by (W > 0.5) */
    float bias;          /* unbinarize_bias, 0.25 in the reference */
} lut_mode_t;

static inline int get_bit(uint32_t const *row, int f) { return (int)((row[f >> 5] >> (f & 31)) & 1u); }

static inline void set_bit(uint32_t *row, int f, int v)
{
    uint32_t m = 1u << (f & 31);
    if (v) row[f >> 5] |= m; else row[f >> 5] &= ~m;
}

/* Input conditioning shared by every CPU branch:
 * include/bb/DifferentiableLutN.h:779-786 and include/bb/StochasticLutN.h:527-535. */
static inline void fetch_x(float xv[6], int bit_input, void const *x, size_t x_stride, int const *idx6, int f, lut_mode_t const *m)
{
    for (int i = 0; i < 6; ++i) {
        float v;
        if (bit_input) v = (float)get_bit((uint32_t const *)x + (size_t)idx6[i] * x_stride, f);
        else           v = ((float const *)x)[(size_t)idx6[i] * x_stride + f];
        if (bit_input || m->binary) xv[i] = 0.5f + ((v > 0.5f) ? +m->bias : -m->bias);
        else                        xv[i] = fminf(1.0f, fmaxf(0.0f, v));
    }
}

static inline void fetch_W(float Wv[64], float const *W, int node, lut_mode_t const *m)
{
    for (int i = 0; i < 64; ++i) {
        float w = W[(size_t)node * 64 + i];
        Wv[i] = m->lut_binarize ? ((w > 0.5f) ? 1.0f : 0.0f) : w;    /* DifferentiableLutN.h:765-771 */
    }
}

/* include/bb/StochasticOperation.h:95-114  StochasticOperation_Lut_Forward */
static inline float lut_forward(float const x[6], float const W[64])
{
    float acc = 0.0f;
    for (int i = 0; i < 64; ++i) {
        float w = W[i];
        for (int j = 0; j < 6; ++j) w *= ((i >> j) & 1) ? x[j] : (1.0f - x[j]);
        acc += w;
    }
    return acc;
}

/* include/bb/StochasticOperation.h:118-152  StochasticOperation_Lut_Backward */
static inline void lut_backward(float const x[6], float dx[6], float dy, float const W[64], float dW[64])
{
    for (int i = 0; i < 64; ++i) {
        float dw = dy;
        for (int j = 0; j < 6; ++j) dw *= ((i >> j) & 1) ? x[j] : (1.0f - x[j]);
        dW[i] += dw;
    }
    for (int i = 0; i < 6; ++i) {
        dx[i] = 0.0f;
        for (int j = 0; j < 64; ++j) {
            float w = ((j >> i) & 1) ? +W[j] : -W[j];
            for (int k = 0; k < 6; ++k) if (i != k) w *= ((j >> k) & 1) ? x[k] : (1.0f - x[k]);
            dx[i] += w;
        }
        dx[i] *= dy;
    }
}

/* ------------------------------------------------------------------------------------------
 * StochasticLut6 (no batch norm)
 * forward : include/bb/StochasticLutN.h:512-559 (generic), StochasticLutSimd.h:25-190 (AVX2)
 *           y = clip(lut(x), 0, 1); y_bit_out packs (y > 0.5) as DifferentiableLutN.h:990-993 does
 * backward: include/bb/StochasticLutN.h:668-752; dx = sum over consuming nodes; dW accumulated
 * ------------------------------------------------------------------------------------------ */
void oracle_sl6_forward(int bit_input, void const *x, size_t x_stride, float *y, size_t y_stride, uint32_t *y_bits, size_t yb_stride,
                        int const *idx, float const *W, int O, int F, int binary, int lut_binarize, float bias)
{
    lut_mode_t m = { binary, lut_binarize, bias };
    #pragma omp parallel for
    for (int node = 0; node < O; ++node) {
        float Wv[64]; fetch_W(Wv, W, node, &m);
        for (int f = 0; f < F; ++f) {
            float xv[6]; fetch_x(xv, bit_input, x, x_stride, idx + node * 6, f, &m);
            float v = lut_forward(xv, Wv);
            if (y_bits) set_bit(y_bits + (size_t)node * yb_stride, f, v > 0.5f);
            v = fmaxf(0.0f, v); v = fminf(1.0f, v);
            if (y) y[(size_t)node * y_stride + f] = v;
        }
    }
}

void oracle_sl6_backward(int bit_input, void const *x, size_t x_stride, float const *dy, size_t dy_stride, float *dx, size_t dx_stride,
                         int const *idx, float const *W, float *dW, int I, int O, int F, int binary, int lut_binarize, float bias)
{
    lut_mode_t m = { binary, lut_binarize, bias };
    for (int i = 0; i < I; ++i) memset(dx + (size_t)i * dx_stride, 0, sizeof(float) * F);
    for (int node = 0; node < O; ++node) {
        float Wv[64]; fetch_W(Wv, W, node, &m);
        float dWv[64] = {0};
        for (int f = 0; f < F; ++f) {
            float xv[6]; fetch_x(xv, bit_input, x, x_stride, idx + node * 6, f, &m);
            float dxv[6];
            lut_backward(xv, dxv, dy[(size_t)node * dy_stride + f], Wv, dWv);
            for (int i = 0; i < 6; ++i) dx[(size_t)idx[node * 6 + i] * dx_stride + f] += dxv[i];
        }
        for (int i = 0; i < 64; ++i) dW[(size_t)node * 64 + i] += dWv[i];
    }
}

/* ------------------------------------------------------------------------------------------
 * DifferentiableLut6 = LUT6 + scalar-gamma/beta batch norm over frames + hard-tanh / binarize
 * training forward : include/bb/DifferentiableLutN.h:747-845
 * inference forward: include/bb/DifferentiableLutN.h:847-905
 * backward         : include/bb/DifferentiableLutN.h:1157-1266
 * y (fp32) gets {0,1} in binary mode, clip(.,0,1) otherwise; y_bits (optional) packs (y_bn > 0.5).
 * y_pre (optional) receives the batch-normalised value before binarize/clip so that callers can
 * tell a genuine mismatch from a value sitting on a decision threshold.
 * ------------------------------------------------------------------------------------------ */
void oracle_dl6_forward_train(int bit_input, void const *x, size_t x_stride, float *y, size_t y_stride, uint32_t *y_bits, size_t yb_stride,
                              float *y_pre, int const *idx, float const *W,
                              float *mean_out, float *rstd_out, float *running_mean, float *running_var,
                              float gamma, float beta, float momentum, float bias,
                              int O, int F, int lut_binarize, int binary)
{
    lut_mode_t m = { binary, lut_binarize, bias };
    float rF = 1.0f / (float)F;
    #pragma omp parallel for
    for (int node = 0; node < O; ++node) {
        float Wv[64]; fetch_W(Wv, W, node, &m);
        /* Kahan sums of y and y*y: DifferentiableLutN.h:775-802 */
        float s1 = 0, c1 = 0, y1, t1, s2 = 0, c2 = 0, y2, t2;
        for (int f = 0; f < F; ++f) {
            float xv[6]; fetch_x(xv, bit_input, x, x_stride, idx + node * 6, f, &m);
            float v = lut_forward(xv, Wv);
            y1 = v - c1;       t1 = s1 + y1; c1 = (t1 - s1) - y1; s1 = t1;
            y2 = (v * v) - c2; t2 = s2 + y2; c2 = (t2 - s2) - y2; s2 = t2;
        }
        float mean = s1 * rF;
        /* DifferentiableLutN.h:805 writes (s2*rF) - (mean*mean); with the reference's own build flags
         * (-O2 -mfma, GCC's default -ffp-contract=fast) that is one fused multiply-subtract, spelled
         * out here so that the result does not depend on this file's compiler. */
        float var  = fmaxf(1.0e-5f, fmaf(s2, rF, -(mean * mean)));
        float rstd = 1.0f / sqrtf(var);
        running_mean[node] = running_mean[node] * momentum + mean * (1.0f - momentum);
        running_var[node]  = running_var[node]  * momentum + var  * (1.0f - momentum);
        mean_out[node] = mean;
        rstd_out[node] = rstd;
        for (int f = 0; f < F; ++f) {
            float xv[6]; fetch_x(xv, bit_input, x, x_stride, idx + node * 6, f, &m);
            float v = lut_forward(xv, Wv);
            v = (v - mean) * rstd;
            v = v * gamma + beta;
            if (y_pre)  y_pre[(size_t)node * y_stride + f] = v;
            if (y_bits) set_bit(y_bits + (size_t)node * yb_stride, f, v > 0.5f);
            if (binary) v = (v > 0.5f) ? 1.0f : 0.0f;
            else { v = fminf(v, 1.0f); v = fmaxf(v, 0.0f); }
            if (y) y[(size_t)node * y_stride + f] = v;
        }
    }
}

void oracle_dl6_forward_infer(int bit_input, void const *x, size_t x_stride, float *y, size_t y_stride, uint32_t *y_bits, size_t yb_stride,
                              float *y_pre, int const *idx, float const *W,
                              float const *running_mean, float const *running_var,
                              float gamma, float beta, float bias, int O, int F, int lut_binarize, int binary)
{
    lut_mode_t m = { binary, lut_binarize, bias };
    #pragma omp parallel for
    for (int node = 0; node < O; ++node) {
        float Wv[64]; fetch_W(Wv, W, node, &m);
        float mean = running_mean[node];
        float rstd = 1.0f / sqrtf(running_var[node]);       /* DifferentiableLutN.h:866-868 */
        for (int f = 0; f < F; ++f) {
            float xv[6]; fetch_x(xv, bit_input, x, x_stride, idx + node * 6, f, &m);
            float v = lut_forward(xv, Wv);
            v = (v - mean) * rstd;
            v = v * gamma + beta;
            if (y_pre)  y_pre[(size_t)node * y_stride + f] = v;
            if (y_bits) set_bit(y_bits + (size_t)node * yb_stride, f, v > 0.5f);
            if (binary) v = (v > 0.5f) ? 1.0f : 0.0f;
            else { v = fminf(v, 1.0f); v = fmaxf(v, 0.0f); }
            if (y) y[(size_t)node * y_stride + f] = v;
        }
    }
}

void oracle_dl6_backward(int bit_input, void const *x, size_t x_stride, float const *dy, size_t dy_stride, float *dx, size_t dx_stride,
                         int const *idx, float const *W, float *dW, float const *mean_in, float const *rstd_in,
                         float gamma, float beta, float bias, int I, int O, int F, int lut_binarize, int binary)
{
    lut_mode_t m = { binary, lut_binarize, bias };
    float rF = 1.0f / (float)F;
    for (int i = 0; i < I; ++i) memset(dx + (size_t)i * dx_stride, 0, sizeof(float) * F);
    for (int node = 0; node < O; ++node) {
        float Wv[64]; fetch_W(Wv, W, node, &m);
        float dWv[64] = {0};
        float mean = mean_in[node], rstd = rstd_in[node], rstd2 = rstd * rstd;
        float dmeanx = 0, dstd = 0;
        for (int f = 0; f < F; ++f) {           /* DifferentiableLutN.h:1190-1220 */
            float xv[6]; fetch_x(xv, bit_input, x, x_stride, idx + node * 6, f, &m);
            float v = lut_forward(xv, Wv);
            float tanh_x = ((v - mean) * rstd) * gamma + beta;
            float g = dy[(size_t)node * dy_stride + f];
            if (tanh_x <= 0.0f) g = 0.0f;
            if (tanh_x >= 1.0f) g = 0.0f;
            float xc = v - mean, dxn = gamma * g;
            dstd   += -(dxn * xc * rstd2);
            dmeanx += -(dxn * rstd);
        }
        float dvar  = dstd * rstd;
        float dmean = (dmeanx - (mean * dvar)) * rF;
        for (int f = 0; f < F; ++f) {           /* DifferentiableLutN.h:1225-1258 */
            float xv[6]; fetch_x(xv, bit_input, x, x_stride, idx + node * 6, f, &m);
            float v = lut_forward(xv, Wv);
            float tanh_x = ((v - mean) * rstd) * gamma + beta;
            float g = dy[(size_t)node * dy_stride + f];
            if (tanh_x <= 0.0f) g = 0.0f;
            if (tanh_x >= 1.0f) g = 0.0f;
            float dxn = g * gamma, dxc = dxn * rstd;
            float gg  = dxc + dmean + (v * dvar * rF);
            float dxv[6];
            lut_backward(xv, dxv, gg, Wv, dWv);
            for (int i = 0; i < 6; ++i) dx[(size_t)idx[node * 6 + i] * dx_stride + f] += dxv[i];
        }
        for (int i = 0; i < 64; ++i) dW[(size_t)node * 64 + i] += dWv[i];
    }
}

/* ------------------------------------------------------------------------------------------
 * StochasticBatchNormalization (stand-alone), generic CPU branch
 * training forward : include/bb/StochasticBatchNormalization.h:521-594 (two-pass variance,
 *                    var = max(0,var), rstd = 1/(sqrt(var)+1e-7))
 * re-forward       : include/bb/StochasticBatchNormalization.h:655-682
 * inference forward: include/bb/StochasticBatchNormalization.h:596-614 written as gain*x+offset.
 *                    The reference takes the offset's mean from its per-batch mean tensor
 *                    (:603); the operator ABI only carries the running statistics
 *                    (include/bbcu/bbcu.h:911-923), so `mean` here is whatever the caller passes.
 * backward         : include/bb/StochasticBatchNormalization.h:808-852
 * ------------------------------------------------------------------------------------------ */
void oracle_sbn_forward_train(float const *x, float *y, size_t stride, float *mean_out, float *rstd_out,
                              float *running_mean, float *running_var, float gamma, float beta, float momentum, int O, int F)
{
    #pragma omp parallel for
    for (int node = 0; node < O; ++node) {
        float const *xr = x + (size_t)node * stride;
        float mean = 0;
        for (int f = 0; f < F; ++f) mean += xr[f];
        mean /= (float)F;
        float var = 0;
        for (int f = 0; f < F; ++f) { float xc = xr[f] - mean; var += xc * xc; }
        var /= (float)F;
        var = fmaxf(0.0f, var);
        float rstd = 1.0f / (sqrtf(var) + 1.0e-7f);
        running_mean[node] = running_mean[node] * momentum + mean * (1.0f - momentum);
        running_var[node]  = running_var[node]  * momentum + var  * (1.0f - momentum);
        mean_out[node] = mean; rstd_out[node] = rstd;
        for (int f = 0; f < F; ++f) {
            float v = (xr[f] - mean) * rstd;
            y[(size_t)node * stride + f] = v * gamma + beta;
        }
    }
}

void oracle_sbn_reforward(float const *x, float *y, size_t stride, float const *mean, float const *rstd, float gamma, float beta, int O, int F)
{
    for (int node = 0; node < O; ++node)
        for (int f = 0; f < F; ++f) {
            float v = (x[(size_t)node * stride + f] - mean[node]) * rstd[node];
            y[(size_t)node * stride + f] = v * gamma + beta;
        }
}

void oracle_sbn_forward_infer(float const *x, float *y, size_t stride, float const *mean, float const *var, float gamma, float beta, int O, int F)
{
    for (int node = 0; node < O; ++node) {
        float gain   = gamma / (sqrtf(var[node]) + 1.0e-7f);
        float offset = beta - (gamma * mean[node] / (sqrtf(var[node]) + 1.0e-7f));
        for (int f = 0; f < F; ++f) y[(size_t)node * stride + f] = gain * x[(size_t)node * stride + f] + offset;
    }
}

void oracle_sbn_backward(float const *x, float const *dy, float *dx, size_t stride, float const *mean_in, float const *rstd_in, float gamma, int O, int F)
{
    #pragma omp parallel for
    for (int node = 0; node < O; ++node) {
        float mean = mean_in[node], rstd = rstd_in[node], dmeanx = 0, dstd = 0;
        for (int f = 0; f < F; ++f) {
            float xc = x[(size_t)node * stride + f] - mean;
            float dxn = gamma * dy[(size_t)node * stride + f];
            dstd   += -(dxn * xc * (rstd * rstd));
            dmeanx += -(dxn * rstd);
        }
        float dvar  = dstd * rstd;
        float dmean = (dmeanx - (mean * dvar)) / (float)F;
        for (int f = 0; f < F; ++f) {
            float dxn = dy[(size_t)node * stride + f] * gamma;
            float dxc = dxn * rstd;
            dx[(size_t)node * stride + f] = dxc + dmean + (x[(size_t)node * stride + f] * dvar / (float)F);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * BinaryLut6 bit-packed inference forward
 * include/bb/BinaryLutN.h:436-463 (generic) and :322-433 (AVX2): index bit k = input k,
 * y = bit `index` of the node's 64-bit table stored as two int32 (BinaryLutN.h:43-46,279-284).
 * Frames >= F inside the last word are written as 0 here; callers compare F frames only.
 * ------------------------------------------------------------------------------------------ */
void oracle_binary_lut6_forward(uint32_t const *x, uint32_t *y, size_t stride, int const *idx, int32_t const *table, int O, int F)
{
    #pragma omp parallel for
    for (int node = 0; node < O; ++node) {
        uint64_t t = ((uint64_t)(uint32_t)table[node * 2 + 1] << 32) | (uint32_t)table[node * 2];
        uint32_t *yr = y + (size_t)node * stride;
        memset(yr, 0, sizeof(uint32_t) * ((F + 31) / 32));
        for (int f = 0; f < F; ++f) {
            int index = 0;
            for (int k = 0; k < 6; ++k) index |= get_bit(x + (size_t)idx[node * 6 + k] * stride, f) << k;
            if ((t >> index) & 1u) yr[f >> 5] |= 1u << (f & 31);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Adam as the layer's optimizer applies it (include/bb/OptimizerAdam.h:142-184 CPU branch):
 *   lr_t = lr * sqrt(1 - b2^t) / (1 - b1^t);  m += (1-b1)(g-m);  v += (1-b2)(g*g-v);
 *   p -= lr_t * m / (sqrt(v) + 1e-7);  then the gradient is zeroed (include/bb/Optimizer.h:29-33).
 * b1t / b2t are the running powers, updated by the caller's state here.
 * ------------------------------------------------------------------------------------------ */
void oracle_adam_update(float *p, float *g, float *mbuf, float *vbuf, size_t n, float lr, float beta1, float beta2, float *b1t, float *b2t)
{
    *b1t *= beta1; *b2t *= beta2;
    float lr_t = lr * sqrtf(1.0f - *b2t) / (1.0f - *b1t);
    for (size_t i = 0; i < n; ++i) {
        mbuf[i] += (1.0f - beta1) * (g[i] - mbuf[i]);
        vbuf[i] += (1.0f - beta2) * (g[i] * g[i] - vbuf[i]);
        p[i] -= lr_t * mbuf[i] / (sqrtf(vbuf[i]) + 1.0e-7f);
        g[i] = 0.0f;
    }
}

/* ------------------------------------------------------------------------------------------
 * Neighbours used by whole-step parity: bb::Reduce, the two losses.
 * Reduce                  include/bb/Reduce.h:200-220 (forward), :250-268 (backward)
 * LossSoftmaxCrossEntropy include/bb/LossSoftmaxCrossEntropy.h:151-205 (pix_size = 1 form)
 * LossMeanSquaredError    include/bb/LossMeanSquaredError.h:153-172 (mean reduction)
 * ------------------------------------------------------------------------------------------ */
void oracle_reduce_forward(float const *x, float *y, int in_nodes, int out_nodes, int F)
{
    int mux = in_nodes / out_nodes;
    for (int o = 0; o < out_nodes; ++o)
        for (int f = 0; f < F; ++f) {
            float sum = 0;
            for (int i = 0; i < mux; ++i) sum += x[(size_t)(out_nodes * i + o) * F + f];
            y[(size_t)o * F + f] = sum / (float)mux;
        }
}

void oracle_reduce_backward(float const *dy, float *dx, int in_nodes, int out_nodes, int F)
{
    int mux = in_nodes / out_nodes;
    for (int o = 0; o < out_nodes; ++o)
        for (int f = 0; f < F; ++f) {
            float g = dy[(size_t)o * F + f] / (float)mux;
            for (int i = 0; i < mux; ++i) dx[(size_t)(out_nodes * i + o) * F + f] = g;
        }
}

double oracle_softmax_cross_entropy(float const *y, float const *t, float *dy, int nodes, int F)
{
    float eps = 1.0e-7f, t_sum = 0;
    for (int f = 0; f < F; ++f) for (int n = 0; n < nodes; ++n) t_sum += t[(size_t)n * F + f];
    double loss_sum = 0;
    for (int f = 0; f < F; ++f) {
        float c = -3.402823466e+38f;
        for (int n = 0; n < nodes; ++n) c = fmaxf(c, y[(size_t)n * F + f]);
        float y_sum = 0, t_max = 0;
        for (int n = 0; n < nodes; ++n) { y_sum += expf(y[(size_t)n * F + f] - c); t_max += t[(size_t)n * F + f]; }
        if (y_sum <= eps) y_sum = eps;
        float lf = 0;
        for (int n = 0; n < nodes; ++n) {
            float softmax = expf(y[(size_t)n * F + f] - c) / y_sum, tv = t[(size_t)n * F + f];
            if (tv > 0) lf += logf(softmax + eps) * t_max;
            dy[(size_t)n * F + f] = (t_max * softmax - tv) / t_sum;
        }
        loss_sum += lf;
    }
    return -loss_sum / t_sum;
}

double oracle_mean_squared_error(float const *y, float const *t, float *dy, int nodes, int F, int batch_size)
{
    float grad_reduction = 1.0f / (float)(nodes * batch_size);
    double loss = 0;
    for (int f = 0; f < F; ++f)
        for (int n = 0; n < nodes; ++n) {
            float g = y[(size_t)n * F + f] - t[(size_t)n * F + f];
            dy[(size_t)n * F + f] = 2 * g * grad_reduction;
            float e = g * g;
            if (!isnan(e)) loss += e * (1.0 / nodes);
        }
    return loss / F;
}

/* ------------------------------------------------------------------------------------------
 * Binary modulation
 * RealToBinary  include/bb/RealToBinary.h:309-345 (th == NULL: deterministic) and :352-398 (th[node][out_frame] given)
 * BinaryToReal  include/bb/BinaryToReal.h:247-276 (forward), :312-330 (backward)
 * Layout: x [x_depth * point_size][frames] fp32, y bit rows of `ys` words; output node = (depth * depth_mod + d) * point_size + p.
 * ------------------------------------------------------------------------------------------ */
void oracle_real_to_binary(float const *x, uint32_t *y, size_t ys, float const *th, int x_depth, int point_size, int frames, int frame_mod,
                           int depth_mod, float lo, float hi)
{
    float frame_step = 1.0f / (float)frame_mod, depth_step = 1.0f / (float)depth_mod, scale = 1.0f / (hi - lo);
    int out_frames = frames * frame_mod, nodes = x_depth * point_size;
    for (int n = 0; n < nodes * depth_mod; ++n) memset(y + (size_t)n * ys, 0, sizeof(uint32_t) * ((out_frames + 31) / 32));
    for (int fi = 0; fi < frames; ++fi)
        for (int f = 0; f < frame_mod; ++f) {
            int of = fi * frame_mod + f;
            for (int depth = 0; depth < x_depth; ++depth)
                for (int p = 0; p < point_size; ++p) {
                    int in_node = depth * point_size + p;
                    float xv = (x[(size_t)in_node * frames + fi] - lo) * scale;
                    for (int d = 0; d < depth_mod; ++d) {
                        int on = (depth * depth_mod + d) * point_size + p;
                        float v = (xv - (float)(d * depth_step)) * (float)depth_mod;
                        int bit;
                        if (th) bit = v > th[(size_t)in_node * out_frames + of];
                        else {
                            v = (v - (float)(f * frame_step)) * (float)frame_mod;
                            v = fmaxf(0.0f, fminf(1.0f, v));
                            bit = v > 0.5f;
                        }
                        if (bit) y[(size_t)on * ys + (of >> 5)] |= 1u << (of & 31);
                    }
                }
        }
}

void oracle_binary_to_real_forward(uint32_t const *x, size_t xs, float *y, int x_nodes, int y_nodes, int y_frames, int frame_mux)
{
    for (int f = 0; f < y_frames; ++f)
        for (int n = 0; n < y_nodes; ++n) {
            float v = 0; int cnt = 0;
            for (int xn = n; xn < x_nodes; xn += y_nodes)
                for (int i = 0; i < frame_mux; ++i) { v += (float)get_bit(x + (size_t)xn * xs, f * frame_mux + i); ++cnt; }
            y[(size_t)n * y_frames + f] = v / (float)cnt;
        }
}

void oracle_binary_to_real_backward(float const *dy, float *dx, int x_nodes, int y_nodes, int y_frames, int frame_mux)
{
    float gain = (float)y_nodes / ((float)x_nodes * (float)frame_mux);
    for (int n = 0; n < x_nodes; ++n)
        for (int f = 0; f < y_frames; ++f)
            for (int i = 0; i < frame_mux; ++i)
                dx[(size_t)n * y_frames * frame_mux + f * frame_mux + i] = dy[(size_t)(n % y_nodes) * y_frames + f] * gain;
}

/* ------------------------------------------------------------------------------------------------
 * Convolution lowering: Im2Col, Col2Im, MaxPooling (CPU paths of the reference).
 * Dense arrays: fp32 [node][frames], bits [node][words] with an explicit word stride.
 * ---------------------------------------------------------------------------------------------- */

enum { ORACLE_BORDER_CONSTANT = 0, ORACLE_BORDER_REFLECT = 1, ORACLE_BORDER_REFLECT_101 = 2, ORACLE_BORDER_REPLICATE = 3, ORACLE_BORDER_WRAP = 4 };

/* include/bb/ConvolutionIm2Col.h:253-288 */
static int im2col_border(int mode, int *x, int *y, int w, int h)
{
    switch (mode) {
    case ORACLE_BORDER_REFLECT:
        if (*x < 0) *x = -*x - 1;
        if (*y < 0) *y = -*y - 1;
        if (*x >= w) *x = (w - 1) - (*x - w);
        if (*y >= h) *y = (h - 1) - (*y - h);
        return 1;
    case ORACLE_BORDER_REFLECT_101:
        if (*x < 0) *x = -*x;
        if (*y < 0) *y = -*y;
        if (*x >= w) *x = (w - 2) - (*x - w);
        if (*y >= h) *y = (h - 2) - (*y - h);
        return 1;
    case ORACLE_BORDER_REPLICATE:
        if (*x < 0) *x = 0;
        if (*y < 0) *y = 0;
        if (*x >= w) *x = w - 1;
        if (*y >= h) *y = h - 1;
        return 1;
    case ORACLE_BORDER_WRAP:
        if (*x < 0) *x += w;
        if (*y < 0) *y += h;
        if (*x >= w) *x -= w;
        if (*y >= h) *y -= h;
        return 1;
    default:
        return 0;
    }
}

/* Source of output element (output_frame, node (c, fy, fx)): returns the input node or -1 for the border value.
 * include/bb/ConvolutionIm2Col.h:368-391 */
static int im2col_source(int output_frame, int c, int fy, int fx, int x_stride, int y_stride, int x_offset, int y_offset, int in_w, int in_h,
                         int out_w, int out_h, int border_mode, int *input_frame)
{
    int output_size = out_w * out_h;
    int f = output_frame % output_size;
    *input_frame = output_frame / output_size;
    int iy = (f / out_w) * y_stride - y_offset + fy;
    int ix = (f % out_w) * x_stride - x_offset + fx;
    if (iy >= 0 && iy < in_h && ix >= 0 && ix < in_w) return (c * in_h + iy) * in_w + ix;
    if (im2col_border(border_mode, &ix, &iy, in_w, in_h)) return (c * in_h + iy) * in_w + ix;
    return -1;
}

void oracle_im2col_forward_f32(float const *x, float *y, int x_stride, int y_stride, int x_offset, int y_offset, int in_frames, int in_w, int in_h,
                               int in_c, int out_w, int out_h, int filter_w, int filter_h, int border_mode, float border_value)
{
    int out_frames = in_frames * out_w * out_h;
    for (int c = 0; c < in_c; ++c)
        for (int fy = 0; fy < filter_h; ++fy)
            for (int fx = 0; fx < filter_w; ++fx) {
                int on = (c * filter_h + fy) * filter_w + fx;
                for (int of = 0; of < out_frames; ++of) {
                    int fi, in = im2col_source(of, c, fy, fx, x_stride, y_stride, x_offset, y_offset, in_w, in_h, out_w, out_h, border_mode, &fi);
                    y[(size_t)on * out_frames + of] = in < 0 ? border_value : x[(size_t)in * in_frames + fi];
                }
            }
}

/* Bit frames: the border value of the Bit specialisation is 0. */
void oracle_im2col_forward_bit(uint32_t const *x, size_t xs, uint32_t *y, size_t ys, int x_stride, int y_stride, int x_offset, int y_offset,
                               int in_frames, int in_w, int in_h, int in_c, int out_w, int out_h, int filter_w, int filter_h, int border_mode)
{
    int out_frames = in_frames * out_w * out_h;
    for (int c = 0; c < in_c; ++c)
        for (int fy = 0; fy < filter_h; ++fy)
            for (int fx = 0; fx < filter_w; ++fx) {
                int on = (c * filter_h + fy) * filter_w + fx;
                memset(y + (size_t)on * ys, 0, sizeof(uint32_t) * ((out_frames + 31) / 32));
                for (int of = 0; of < out_frames; ++of) {
                    int fi, in = im2col_source(of, c, fy, fx, x_stride, y_stride, x_offset, y_offset, in_w, in_h, out_w, out_h, border_mode, &fi);
                    if (in >= 0 && ((x[(size_t)in * xs + (fi >> 5)] >> (fi & 31)) & 1u)) y[(size_t)on * ys + (of >> 5)] |= 1u << (of & 31);
                }
            }
}

/* include/bb/ConvolutionIm2Col.h:439-482: only positions inside the image receive gradient (border copies send none back). */
void oracle_im2col_backward_f32(float const *dy, float *dx, int x_stride, int y_stride, int x_offset, int y_offset, int in_frames, int in_w, int in_h,
                                int in_c, int out_w, int out_h, int filter_w, int filter_h)
{
    int out_frames = in_frames * out_w * out_h;
    int iy_limit = (out_h - 1) * y_stride, ix_limit = (out_w - 1) * x_stride;
    for (int c = 0; c < in_c; ++c)
        for (int y = 0; y < in_h; ++y)
            for (int x = 0; x < in_w; ++x) {
                int in = (c * in_h + y) * in_w + x;
                int x_align = x % x_stride, y_align = y % y_stride;
                for (int fi = 0; fi < in_frames; ++fi) {
                    float g = 0;
                    for (int fy = y_align; fy < filter_h; fy += y_stride) {
                        int iy = y - fy + y_offset;
                        if (iy < 0 || iy > iy_limit) continue;
                        for (int fx = x_align; fx < filter_w; fx += x_stride) {
                            int ix = x - fx + x_offset;
                            if (ix < 0 || ix > ix_limit) continue;
                            int of = (fi * out_h + iy / y_stride) * out_w + ix / x_stride;
                            int on = (c * filter_h + fy) * filter_w + fx;
                            g += dy[(size_t)on * out_frames + of];
                        }
                    }
                    dx[(size_t)in * in_frames + fi] = 0.0f + g;
                }
            }
}

/* include/bb/ConvolutionCol2Im.h:205-221: y[c*hw + xy][fo] = x[c][fo*hw + xy] */
void oracle_col2im_forward_f32(float const *x, float *y, int w, int h, int c_size, int out_frames)
{
    int hw = w * h, in_frames = out_frames * hw;
    for (int c = 0; c < c_size; ++c)
        for (int xy = 0; xy < hw; ++xy)
            for (int fo = 0; fo < out_frames; ++fo) y[(size_t)(c * hw + xy) * out_frames + fo] = x[(size_t)c * in_frames + (size_t)fo * hw + xy];
}

void oracle_col2im_forward_bit(uint32_t const *x, size_t xs, uint32_t *y, size_t ys, int w, int h, int c_size, int out_frames)
{
    int hw = w * h;
    for (int c = 0; c < c_size; ++c)
        for (int xy = 0; xy < hw; ++xy) {
            uint32_t *row = y + (size_t)(c * hw + xy) * ys;
            memset(row, 0, sizeof(uint32_t) * ((out_frames + 31) / 32));
            for (int fo = 0; fo < out_frames; ++fo) {
                size_t fi = (size_t)fo * hw + xy;
                if ((x[(size_t)c * xs + (fi >> 5)] >> (fi & 31)) & 1u) row[fo >> 5] |= 1u << (fo & 31);
            }
        }
}

/* include/bb/ConvolutionCol2Im.h:283-299 */
void oracle_col2im_backward_f32(float const *dy, float *dx, int w, int h, int c_size, int out_frames)
{
    int hw = w * h, in_frames = out_frames * hw;
    for (int c = 0; c < c_size; ++c)
        for (int xy = 0; xy < hw; ++xy)
            for (int fo = 0; fo < out_frames; ++fo) dx[(size_t)c * in_frames + (size_t)fo * hw + xy] = dy[(size_t)(c * hw + xy) * out_frames + fo];
}

/* include/bb/MaxPooling.h:286-322: strict '>' from the lowest float, so the first maximum wins; argmax counts the in-range
 * positions of the window in scan order. */
void oracle_maxpool_forward_f32(float const *x, float *y, int32_t *argmax, int filter_h, int filter_w, int in_w, int in_h, int c_size, int frames)
{
    int out_w = (in_w + filter_w - 1) / filter_w, out_h = (in_h + filter_h - 1) / filter_h;
    for (int c = 0; c < c_size; ++c)
        for (int oy = 0; oy < out_h; ++oy)
            for (int ox = 0; ox < out_w; ++ox) {
                size_t on = ((size_t)c * out_h + oy) * out_w + ox;
                for (int f = 0; f < frames; ++f) {
                    float best = -FLT_MAX;
                    int32_t am = 0, arg = 0;
                    for (int fy = 0; fy < filter_h; ++fy) {
                        int iy = oy * filter_h + fy;
                        if (iy >= in_h) continue;
                        for (int fx = 0; fx < filter_w; ++fx) {
                            int ix = ox * filter_w + fx;
                            if (ix >= in_w) continue;
                            float v = x[(((size_t)c * in_h + iy) * in_w + ix) * frames + f];
                            if (v > best) { best = v; am = arg; }
                            ++arg;
                        }
                    }
                    y[on * frames + f] = best;
                    if (argmax) argmax[on * frames + f] = am;
                }
            }
}

/* include/bb/MaxPooling.h:369-394: OR of the window */
void oracle_maxpool_forward_bit(uint32_t const *x, uint32_t *y, size_t stride, int filter_h, int filter_w, int in_w, int in_h, int c_size, int frames)
{
    int out_w = (in_w + filter_w - 1) / filter_w, out_h = (in_h + filter_h - 1) / filter_h, words = (frames + 31) / 32;
    for (int c = 0; c < c_size; ++c)
        for (int oy = 0; oy < out_h; ++oy)
            for (int ox = 0; ox < out_w; ++ox) {
                uint32_t *row = y + (((size_t)c * out_h + oy) * out_w + ox) * stride;
                for (int wd = 0; wd < words; ++wd) {
                    uint32_t m = 0;
                    for (int fy = 0; fy < filter_h; ++fy)
                        for (int fx = 0; fx < filter_w; ++fx) {
                            int iy = oy * filter_h + fy, ix = ox * filter_w + fx;
                            if (iy < in_h && ix < in_w) m |= x[(((size_t)c * in_h + iy) * in_w + ix) * stride + wd];
                        }
                    row[wd] = m;
                }
            }
}

/* include/bb/MaxPooling.h:600-629 */
void oracle_maxpool_backward_f32(int32_t const *argmax, float const *dy, float *dx, int filter_h, int filter_w, int in_w, int in_h, int c_size, int frames)
{
    int out_w = (in_w + filter_w - 1) / filter_w, out_h = (in_h + filter_h - 1) / filter_h;
    for (int c = 0; c < c_size; ++c)
        for (int oy = 0; oy < out_h; ++oy)
            for (int ox = 0; ox < out_w; ++ox) {
                size_t on = ((size_t)c * out_h + oy) * out_w + ox;
                for (int f = 0; f < frames; ++f) {
                    int32_t arg = 0, am = argmax[on * frames + f];
                    float g = dy[on * frames + f];
                    for (int fy = 0; fy < filter_h; ++fy) {
                        int iy = oy * filter_h + fy;
                        if (iy >= in_h) continue;
                        for (int fx = 0; fx < filter_w; ++fx) {
                            int ix = ox * filter_w + fx;
                            if (ix >= in_w) continue;
                            dx[(((size_t)c * in_h + iy) * in_w + ix) * frames + f] = (arg == am) ? g : 0.0f;
                            ++arg;
                        }
                    }
                }
            }
}

/* include/bb/MaxPooling.h:681-708: the first set input bit of the window takes the gradient */
void oracle_maxpool_backward_bit_f32(uint32_t const *x, size_t xs, float const *dy, float *dx, int filter_h, int filter_w, int in_w, int in_h,
                                     int c_size, int frames)
{
    int out_w = (in_w + filter_w - 1) / filter_w, out_h = (in_h + filter_h - 1) / filter_h;
    for (int c = 0; c < c_size; ++c)
        for (int oy = 0; oy < out_h; ++oy)
            for (int ox = 0; ox < out_w; ++ox) {
                size_t on = ((size_t)c * out_h + oy) * out_w + ox;
                for (int f = 0; f < frames; ++f) {
                    float g = dy[on * frames + f];
                    for (int fy = 0; fy < filter_h; ++fy) {
                        int iy = oy * filter_h + fy;
                        if (iy >= in_h) continue;
                        for (int fx = 0; fx < filter_w; ++fx) {
                            int ix = ox * filter_w + fx;
                            if (ix >= in_w) continue;
                            size_t in = ((size_t)c * in_h + iy) * in_w + ix;
                            int bit = (x[in * xs + (f >> 5)] >> (f & 31)) & 1u;
                            dx[in * frames + f] = bit ? g : 0.0f;
                            if (bit) g = 0.0f;
                        }
                    }
                }
            }
}
