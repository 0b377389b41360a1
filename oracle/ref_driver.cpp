// TEST INFRASTRUCTURE ONLY -- never linked into, imported by or executed from the product path.
//
// Thin extern "C" driver around the *unmodified* BinaryBrain header-only CPU implementation.
// It is compiled against the reference's own headers where they lie (-I<reference>/include, no
// BB_WITH_CUDA) by oracle/Makefile into oracle/_ref/libbbref.so.  Nothing of the reference is
// copied here: this file only instantiates the reference's public classes, feeds them caller
// supplied wiring / tables / frames, and copies the results back out.
//
// Used for: (1) pinning oracle/lut6_oracle.c, (2) generating tests/golden/*.npz,
//           (3) the "reference" CPU-baseline arm of bench.py.
//
// Dense array conventions of this driver (all host memory):
//   fp32 frames  : [node][frame]  contiguous, no padding
//   bit frames   : [node][words]  32 frames per uint32, LSB first, words = ceil(frames/32)
//   wiring       : [out_node][6]  int32
//   W            : [out_node][64] fp32
//   binary table : [out_node][2]  int32 (bit i of the 64-bit table = output for input index i)

#include <cstdint>
#include <cstring>
#include <chrono>
#include <vector>
#include <sstream>
#include <string>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "bb/StochasticLutN.h"
#include "bb/DifferentiableLutN.h"
#include "bb/BinaryLutN.h"
#include "bb/StochasticBatchNormalization.h"
#include "bb/OptimizerAdam.h"
#include "bb/Sequential.h"
#include "bb/Reduce.h"
#include "bb/LossSoftmaxCrossEntropy.h"
#include "bb/LossMeanSquaredError.h"
#include "bb/RealToBinary.h"
#include "bb/BinaryToReal.h"
#include "bb/UniformDistributionGenerator.h"
#include "bb/ConvolutionIm2Col.h"
#include "bb/ConvolutionCol2Im.h"
#include "bb/MaxPooling.h"
#include "bb/Convolution2d.h"

namespace {

using clk = std::chrono::steady_clock;
inline double secs(clk::time_point a, clk::time_point b) { return std::chrono::duration<double>(b - a).count(); }

void put_fp32(bb::FrameBuffer &buf, float const *src, int nodes, int frames)
{
    auto ptr = buf.Lock<float>(true);
    for (int n = 0; n < nodes; ++n) {
        std::memcpy(ptr.GetAddr(n), src + (size_t)n * frames, sizeof(float) * frames);
    }
}

void get_fp32(bb::FrameBuffer const &buf, float *dst, int nodes, int frames)
{
    auto ptr = buf.LockConst<float>();
    for (int n = 0; n < nodes; ++n) {
        std::memcpy(dst + (size_t)n * frames, ptr.GetAddr(n), sizeof(float) * frames);
    }
}

void put_bit(bb::FrameBuffer &buf, std::uint32_t const *src, int nodes, int frames)
{
    int words = (frames + 31) / 32;
    auto mem  = buf.LockMemory(true);
    auto base = (std::uint8_t *)mem.GetAddr();
    auto stride = buf.GetFrameStride();
    for (int n = 0; n < nodes; ++n) {
        std::memset(base + (size_t)n * stride, 0, stride);
        std::memcpy(base + (size_t)n * stride, src + (size_t)n * words, sizeof(std::uint32_t) * words);
    }
}

void get_bit(bb::FrameBuffer const &buf, std::uint32_t *dst, int nodes, int frames)
{
    int words = (frames + 31) / 32;
    auto mem  = buf.LockMemoryConst();
    auto base = (std::uint8_t const *)mem.GetAddr();
    auto stride = buf.GetFrameStride();
    for (int n = 0; n < nodes; ++n) {
        std::memcpy(dst + (size_t)n * words, base + (size_t)n * stride, sizeof(std::uint32_t) * words);
        if (frames % 32) {   // padding bits are not part of the result
            dst[(size_t)n * words + words - 1] &= (1u << (frames % 32)) - 1u;
        }
    }
}

template <class Layer>
void set_wiring(Layer &lut, int const *idx, int out_nodes)
{
    for (int n = 0; n < out_nodes; ++n)
        for (int i = 0; i < 6; ++i)
            lut->SetNodeConnectionIndex(n, i, idx[n * 6 + i]);
}

template <class Layer>
void set_W(Layer &lut, float const *W, int out_nodes)
{
    auto p = lut->lock_W();
    for (int n = 0; n < out_nodes; ++n)
        for (int i = 0; i < 64; ++i)
            p(n, i) = W[n * 64 + i];
}

template <class Layer>
void get_dW(Layer &lut, float *dW, int out_nodes)
{
    auto p = lut->lock_dW_const();
    for (int n = 0; n < out_nodes; ++n)
        for (int i = 0; i < 64; ++i)
            dW[n * 64 + i] = p(n, i);
}

template <class Layer>
void set_dW(Layer &lut, float const *dW, int out_nodes)
{
    auto p = lut->lock_dW();
    for (int n = 0; n < out_nodes; ++n)
        for (int i = 0; i < 64; ++i)
            p(n, i) = dW[n * 64 + i];
}

template <typename BinType>
int run_stochastic(void const *x, int I, int O, int F, int const *idx, float const *W,
                   int binary, int lut_binarize, int host_simd,
                   float *y, float const *dy, float *dx, float *dW, double *t)
{
    auto lut = bb::StochasticLutN<6, BinType, float>::Create(O);
    lut->SendCommand("host_only true");
    lut->SendCommand(binary ? "binary true" : "binary false");
    lut->SendCommand(lut_binarize ? "lut_binarize true" : "lut_binarize false");
    lut->SendCommand(host_simd ? "host_simd true" : "host_simd false");

    bb::FrameBuffer x_buf(F, {I}, bb::DataType<BinType>::type, true);
    lut->SetInputShape(x_buf.GetShape());
    set_wiring(lut, idx, O);
    set_W(lut, W, O);
    if (std::is_same<BinType, float>::value) put_fp32(x_buf, (float const *)x, I, F);
    else                                     put_bit(x_buf, (std::uint32_t const *)x, I, F);

    auto t0 = clk::now();
    auto y_buf = lut->Forward(x_buf, true);
    auto t1 = clk::now();
    if (y) get_fp32(y_buf, y, O, F);
    if (t) t[0] = secs(t0, t1);

    if (dy) {
        bb::FrameBuffer dy_buf(F, {O}, BB_TYPE_FP32, true);
        put_fp32(dy_buf, dy, O, F);
        if (dW) set_dW(lut, dW, O);          // dW is accumulated into: start from the caller's values
        auto t2 = clk::now();
        auto dx_buf = lut->Backward(dy_buf);
        auto t3 = clk::now();
        if (dx) get_fp32(dx_buf, dx, I, F);
        if (dW) get_dW(lut, dW, O);
        if (t) t[1] = secs(t2, t3);
    }
    return 0;
}

template <typename BinType>
int run_differentiable(void const *x, int I, int O, int F, int const *idx, float const *W,
                       int batch_norm, int binary, int lut_binarize,
                       float gamma, float beta, float momentum,
                       float *running_mean, float *running_var, int train,
                       void *y, float *mean, float *rstd,
                       float const *dy, float *dx, float *dW, double *t)
{
    using Layer = bb::DifferentiableLutN<6, BinType, float>;
    typename Layer::create_t c;
    c.output_shape = {O};
    c.batch_norm   = batch_norm != 0;
    c.binary       = binary != 0;
    c.momentum     = momentum;
    c.gamma        = gamma;
    c.beta         = beta;
    auto lut = Layer::Create(c);
    lut->SendCommand("host_only true");
    lut->SendCommand(lut_binarize ? "lut_binarize true" : "lut_binarize false");

    bb::FrameBuffer x_buf(F, {I}, bb::DataType<BinType>::type, true);
    lut->SetInputShape(x_buf.GetShape());
    set_wiring(lut, idx, O);
    set_W(lut, W, O);
    if (running_mean && running_var) {
        auto m = lut->lock_mean();
        auto v = lut->lock_var();
        for (int n = 0; n < O; ++n) { m[n] = running_mean[n]; v[n] = running_var[n]; }
    }
    if (std::is_same<BinType, float>::value) put_fp32(x_buf, (float const *)x, I, F);
    else                                     put_bit(x_buf, (std::uint32_t const *)x, I, F);

    auto t0 = clk::now();
    auto y_buf = lut->Forward(x_buf, train != 0);
    auto t1 = clk::now();
    if (t) t[0] = secs(t0, t1);
    if (y) {
        if (std::is_same<BinType, float>::value) get_fp32(y_buf, (float *)y, O, F);
        else                                     get_bit(y_buf, (std::uint32_t *)y, O, F);
    }
    if (train && batch_norm) {
        auto m = lut->lock_tmp_mean_const();
        auto r = lut->lock_tmp_rstd_const();
        for (int n = 0; n < O; ++n) { if (mean) mean[n] = m[n]; if (rstd) rstd[n] = r[n]; }
    }
    if (running_mean && running_var) {
        auto m = lut->lock_mean_const();
        auto v = lut->lock_var_const();
        for (int n = 0; n < O; ++n) { running_mean[n] = m[n]; running_var[n] = v[n]; }
    }

    if (train && dy) {
        bb::FrameBuffer dy_buf(F, {O}, BB_TYPE_FP32, true);
        put_fp32(dy_buf, dy, O, F);
        if (dW) set_dW(lut, dW, O);
        auto t2 = clk::now();
        auto dx_buf = lut->Backward(dy_buf);
        auto t3 = clk::now();
        if (dx) get_fp32(dx_buf, dx, I, F);
        if (dW) get_dW(lut, dW, O);
        if (t) t[1] = secs(t2, t3);
    }
    return 0;
}

}   // namespace


namespace {
template <class L> void fill_sparse(L &lut, int I, int O, int const *idx, float const *W)
{
    lut->SetInputShape({I});
    set_wiring(lut, idx, O);
    set_W(lut, W, O);
}
template <class L> long long dump_to(L &lut, unsigned char *buf, long long cap)
{
    std::ostringstream os(std::ios::binary);
    lut->DumpObject(os);
    std::string bytes = os.str();
    if ((long long)bytes.size() > cap) return -(long long)bytes.size();
    std::memcpy(buf, bytes.data(), bytes.size());
    return (long long)bytes.size();
}
template <class L> void read_sparse(L &lut, int O, int *idx, float *W)
{
    for (int n = 0; n < O; ++n)
        for (int k = 0; k < 6; ++k) idx[n * 6 + k] = (int)lut->GetNodeConnectionIndex(n, k);
    auto Wp = lut->lock_W_const();
    for (int n = 0; n < O; ++n)
        for (int i = 0; i < 64; ++i) W[n * 64 + i] = Wp(n, i);
}
}   // namespace

extern "C" {

// bb::StochasticLutN<6,float|Bit,float>::Forward (+Backward when dy != NULL), CPU branch.
int bbref_stochastic_lut6(int bit_input, void const *x, int I, int O, int F, int const *idx, float const *W,
                          int binary, int lut_binarize, int host_simd,
                          float *y, float const *dy, float *dx, float *dW, double *t)
{
    if (bit_input) return run_stochastic<bb::Bit>(x, I, O, F, idx, W, 1, lut_binarize, host_simd, y, dy, dx, dW, t);
    return run_stochastic<float>(x, I, O, F, idx, W, binary, lut_binarize, host_simd, y, dy, dx, dW, t);
}

// bb::DifferentiableLutN<6,float|Bit,float>::Forward (+Backward when dy != NULL), generic CPU branch.
int bbref_differentiable_lut6(int bit_io, void const *x, int I, int O, int F, int const *idx, float const *W,
                              int batch_norm, int binary, int lut_binarize,
                              float gamma, float beta, float momentum,
                              float *running_mean, float *running_var, int train,
                              void *y, float *mean, float *rstd,
                              float const *dy, float *dx, float *dW, double *t)
{
    if (bit_io) return run_differentiable<bb::Bit>(x, I, O, F, idx, W, batch_norm, 1, lut_binarize, gamma, beta, momentum,
                                                  running_mean, running_var, train, y, mean, rstd, dy, dx, dW, t);
    return run_differentiable<float>(x, I, O, F, idx, W, batch_norm, binary, lut_binarize, gamma, beta, momentum,
                                     running_mean, running_var, train, y, mean, rstd, dy, dx, dW, t);
}

// bb::BinaryLutN<6,bb::Bit>::Forward, AVX2 (host_simd=1) or generic (host_simd=0) CPU branch.
int bbref_binary_lut6(std::uint32_t const *x, int I, int O, int F, int const *idx, std::int32_t const *table,
                      int host_simd, std::uint32_t *y, double *t)
{
    auto lut = bb::BinaryLutN<6, bb::Bit, float>::Create(O);
    lut->SendCommand("host_only true");
    lut->SendCommand(host_simd ? "host_simd true" : "host_simd false");
    bb::FrameBuffer x_buf(F, {I}, BB_TYPE_BIT, true);
    lut->SetInputShape(x_buf.GetShape());
    for (int n = 0; n < O; ++n) {
        for (int i = 0; i < 6; ++i) lut->SetNodeConnectionIndex(n, i, idx[n * 6 + i]);
        for (int i = 0; i < 64; ++i) lut->SetLutTable(n, i, ((table[n * 2 + (i >> 5)] >> (i & 31)) & 1) != 0);
    }
    put_bit(x_buf, x, I, F);
    auto t0 = clk::now();
    auto y_buf = lut->Forward(x_buf, false);
    auto t1 = clk::now();
    if (t) t[0] = secs(t0, t1);
    if (y) get_bit(y_buf, y, O, F);
    return 0;
}

// bb::StochasticBatchNormalization<float>: mode 0 = Forward(train), 1 = Forward(inference), 2 = ReForward.
// Backward runs after a training forward when dy != NULL.
int bbref_stochastic_bn(float const *x, int O, int F, float gamma, float beta, float momentum,
                        float *running_mean, float *running_var, int mode,
                        float *y, float *mean, float *rstd, float const *dy, float *dx)
{
    auto bn = bb::StochasticBatchNormalization<float>::Create(momentum, gamma, beta);
    bn->SendCommand("host_only true");
    bb::FrameBuffer x_buf(F, {O}, BB_TYPE_FP32, true);
    bn->SetInputShape(x_buf.GetShape());
    put_fp32(x_buf, x, O, F);
    if (running_mean && running_var) {
        auto m = bn->lock_mean();
        auto v = bn->lock_var();
        for (int n = 0; n < O; ++n) { m[n] = running_mean[n]; v[n] = running_var[n]; }
    }
    bb::FrameBuffer y_buf;
    if (mode == 2) {
        y_buf = bn->Forward(x_buf, true);      // establishes mean/rstd
        bn->Backward(bb::FrameBuffer(F, {O}, BB_TYPE_FP32, true));
        y_buf = bn->ReForward(x_buf);
    } else {
        y_buf = bn->Forward(x_buf, mode == 0);
    }
    if (y) get_fp32(y_buf, y, O, F);
    {
        auto m = bn->lock_tmp_mean_const();
        auto r = bn->lock_tmp_rstd_const();
        for (int n = 0; n < O; ++n) { if (mean) mean[n] = m[n]; if (rstd) rstd[n] = r[n]; }
    }
    if (running_mean && running_var) {
        auto m = bn->lock_mean_const();
        auto v = bn->lock_var_const();
        for (int n = 0; n < O; ++n) { running_mean[n] = m[n]; running_var[n] = v[n]; }
    }
    if (dy && mode != 1) {
        bb::FrameBuffer dy_buf(F, {O}, BB_TYPE_FP32, true);
        put_fp32(dy_buf, dy, O, F);
        auto dx_buf = bn->Backward(dy_buf);
        if (dx) get_fp32(dx_buf, dx, O, F);
    }
    return 0;
}

// The reference's seeded wiring and table initialisation of a fresh layer
// (FixedSizeConnectionTable::InitializeConnection + Tensor::InitNormalDistribution).
int bbref_init_layer(int I, int O, std::uint64_t seed, char const *connection, int *idx, float *W)
{
    bb::DifferentiableLutN<6, float, float>::create_t c;
    c.output_shape = {O};
    c.seed         = seed;
    c.connection   = connection ? connection : "";
    auto lut = bb::DifferentiableLutN<6, float, float>::Create(c);
    lut->SetInputShape({I});
    for (int n = 0; n < O; ++n)
        for (int i = 0; i < 6; ++i)
            idx[n * 6 + i] = (int)lut->GetNodeConnectionIndex(n, i);
    auto p = lut->lock_W_const();
    for (int n = 0; n < O; ++n)
        for (int i = 0; i < 64; ++i)
            W[n * 64 + i] = p(n, i);
    return 0;
}

// The wiring a fresh reference layer draws for node shapes of `dims` axes (in_shape / out_shape) under a connection rule
// ("", "random", "serial", "pointwise", "depthwise", "gauss").
int bbref_init_connection(int dims, int const *in_shape, int const *out_shape, std::uint64_t seed, char const *connection, int *idx)
{
    bb::DifferentiableLutN<6, float, float>::create_t c;
    c.output_shape = bb::indices_t(out_shape, out_shape + dims);
    c.seed         = seed;
    c.connection   = connection ? connection : "";
    auto lut = bb::DifferentiableLutN<6, float, float>::Create(c);
    lut->SetInputShape(bb::indices_t(in_shape, in_shape + dims));
    const int O = (int)lut->GetOutputNodeSize();
    for (int n = 0; n < O; ++n)
        for (int i = 0; i < 6; ++i)
            idx[n * 6 + i] = (int)lut->GetNodeConnectionIndex(n, i);
    return 0;
}

// steps x { DifferentiableLutN forward(train) -> backward(dy) -> OptimizerAdam::Update } on fixed x, dy.
int bbref_differentiable_lut6_adam(float const *x, int I, int O, int F, int const *idx, float *W,
                                   int batch_norm, int binary, int lut_binarize,
                                   float gamma, float beta, float momentum,
                                   float const *dy, int steps, float lr, float beta1, float beta2,
                                   float *y_last, float *running_mean, float *running_var)
{
    using Layer = bb::DifferentiableLutN<6, float, float>;
    Layer::create_t c;
    c.output_shape = {O};
    c.batch_norm = batch_norm != 0; c.binary = binary != 0;
    c.momentum = momentum; c.gamma = gamma; c.beta = beta;
    auto lut = Layer::Create(c);
    lut->SendCommand("host_only true");
    lut->SendCommand(lut_binarize ? "lut_binarize true" : "lut_binarize false");
    bb::FrameBuffer x_buf(F, {I}, BB_TYPE_FP32, true);
    lut->SetInputShape(x_buf.GetShape());
    set_wiring(lut, idx, O);
    set_W(lut, W, O);
    put_fp32(x_buf, x, I, F);
    bb::FrameBuffer dy_buf(F, {O}, BB_TYPE_FP32, true);
    put_fp32(dy_buf, dy, O, F);

    bb::OptimizerAdam<float>::create_t oc;
    oc.learning_rate = lr; oc.beta1 = beta1; oc.beta2 = beta2;
    auto opt = bb::OptimizerAdam<float>::Create(oc);
    opt->SetVariables(lut->GetParameters(), lut->GetGradients());

    bb::FrameBuffer y_buf;
    for (int s = 0; s < steps; ++s) {
        y_buf = lut->Forward(x_buf, true);
        lut->Backward(dy_buf);
        opt->Update();
    }
    if (y_last) get_fp32(y_buf, y_last, O, F);
    {
        auto p = lut->lock_W_const();
        for (int n = 0; n < O; ++n) for (int i = 0; i < 64; ++i) W[n * 64 + i] = p(n, i);
    }
    if (running_mean && running_var) {
        auto m = lut->lock_mean_const();
        auto v = lut->lock_var_const();
        for (int n = 0; n < O; ++n) { running_mean[n] = m[n]; running_var[n] = v[n]; }
    }
    return 0;
}

// One training step of a stack of DifferentiableLutN<6,float> layers (fp32, batch norm on, non-binary) followed by bb::Reduce to
// `classes` outputs, LossSoftmaxCrossEntropy (use_mse = 0) or LossMeanSquaredError (use_mse = 1) and OptimizerAdam:
// forward(train) -> loss -> backward -> Update.  idx / W are the concatenated wiring and tables of the layers (in: initial, out:
// W after the step); widths[0] is the input width, widths[1..layers] the layer widths.  classes == widths[layers] skips the Reduce.
int bbref_lut_mlp_step(float const *x, float const *t, int frames, int layers, int const *widths, int classes, int const *idx, float *W,
                       int use_mse, float lr, float *y_out, double *loss_out, float *dx_out)
{
    auto net = bb::Sequential::Create();
    std::vector<std::shared_ptr<bb::DifferentiableLutN<6, float, float>>> luts;
    for (int l = 0; l < layers; ++l) {
        bb::DifferentiableLutN<6, float, float>::create_t c;
        c.output_shape = {widths[l + 1]};
        c.binary = false;
        auto lut = bb::DifferentiableLutN<6, float, float>::Create(c);
        lut->SendCommand("host_only true");
        luts.push_back(lut);
        net->Add(lut);
    }
    if (classes != widths[layers]) net->Add(bb::Reduce<float, float>::Create(bb::indices_t({classes})));
    net->SetInputShape({widths[0]});
    size_t io = 0, wo = 0;
    for (int l = 0; l < layers; ++l) {
        set_wiring(luts[l], idx + io, widths[l + 1]);
        set_W(luts[l], W + wo, widths[l + 1]);
        io += (size_t)widths[l + 1] * 6;
        wo += (size_t)widths[l + 1] * 64;
    }
    bb::FrameBuffer x_buf(frames, {widths[0]}, BB_TYPE_FP32, true);
    put_fp32(x_buf, x, widths[0], frames);
    bb::FrameBuffer t_buf(frames, {classes}, BB_TYPE_FP32, true);
    put_fp32(t_buf, t, classes, frames);

    bb::OptimizerAdam<float>::create_t oc;
    oc.learning_rate = lr;
    auto opt = bb::OptimizerAdam<float>::Create(oc);
    opt->SetVariables(net->GetParameters(), net->GetGradients());

    auto y_buf = net->Forward(x_buf, true);
    bb::FrameBuffer dy_buf;
    if (use_mse) {
        auto loss = bb::LossMeanSquaredError<float>::Create();
        dy_buf = loss->CalculateLoss(y_buf, t_buf, frames);
        if (loss_out) *loss_out = loss->GetLoss();
    } else {
        auto loss = bb::LossSoftmaxCrossEntropy<float>::Create();
        dy_buf = loss->CalculateLoss(y_buf, t_buf, frames);
        if (loss_out) *loss_out = loss->GetLoss();
    }
    auto dx_buf = net->Backward(dy_buf);
    opt->Update();
    if (y_out) get_fp32(y_buf, y_out, classes, frames);
    if (dx_out) get_fp32(dx_buf, dx_out, widths[0], frames);
    wo = 0;
    for (int l = 0; l < layers; ++l) {
        auto p = luts[l]->lock_W_const();
        for (int n = 0; n < widths[l + 1]; ++n) for (int i = 0; i < 64; ++i) W[wo + (size_t)n * 64 + i] = p(n, i);
        wo += (size_t)widths[l + 1] * 64;
    }
    return 0;
}

// The LUT-CNN as one bb::Sequential of the reference's own classes, forward (training mode) and backward of a given dy:
//   Convolution2d(3x3 same; per-pixel DifferentiableLut6 27 -> 216 -> 36 -> 32), Convolution2d(288 -> 216 -> 36 -> 32), MaxPooling 2x2,
//   Convolution2d(288 -> 384 -> 64), Convolution2d(576 -> 384 -> 64), MaxPooling 2x2, DifferentiableLut6 4096 -> 1024 -> 420 -> 70 -> 10
// on images {3, hw, hw} (hw = 32 gives the widths above; the first dense layer reads 64 * (hw/4)^2 nodes).  idx / W hold the wiring and
// tables of the 14 LUT layers in network order; dW_out receives their table gradients, y_out [10][frames], dx_out [3*hw*hw][frames].
int bbref_lut_cnn_step(float const *x, float const *dy, int frames, int hw, int const *idx, float const *W, float *y_out, float *dx_out,
                       float *dW_out)
{
    using Lut = bb::DifferentiableLutN<6, float, float>;
    static const int widths[14] = {216, 36, 32, 216, 36, 32, 384, 64, 384, 64, 1024, 420, 70, 10};
    std::vector<std::shared_ptr<Lut>> luts;
    auto make = [&](int w) {
        Lut::create_t c;
        c.output_shape = {w};
        c.binary = false;
        auto l = Lut::Create(c);
        luts.push_back(l);
        return l;
    };
    auto conv = [&](int first, int count) {
        auto seq = bb::Sequential::Create();
        for (int k = 0; k < count; ++k) seq->Add(make(widths[first + k]));
        return bb::Convolution2d<float, float>::Create(seq, 3, 3, 1, 1, "same");
    };
    auto net = bb::Sequential::Create();
    net->Add(conv(0, 3));
    net->Add(conv(3, 3));
    net->Add(bb::MaxPooling<float, float>::Create(2, 2));
    net->Add(conv(6, 2));
    net->Add(conv(8, 2));
    net->Add(bb::MaxPooling<float, float>::Create(2, 2));
    for (int k = 10; k < 14; ++k) net->Add(make(widths[k]));
    net->SendCommand("host_only true");
    net->SetInputShape({3, hw, hw});
    size_t io = 0, wo = 0;
    for (int l = 0; l < 14; ++l) {
        set_wiring(luts[l], idx + io, widths[l]);
        set_W(luts[l], W + wo, widths[l]);
        io += (size_t)widths[l] * 6;
        wo += (size_t)widths[l] * 64;
    }
    bb::FrameBuffer x_buf(frames, {3, hw, hw}, BB_TYPE_FP32, true);
    put_fp32(x_buf, x, 3 * hw * hw, frames);
    auto y_buf = net->Forward(x_buf, true);
    if (y_out) get_fp32(y_buf, y_out, 10, frames);
    bb::FrameBuffer dy_buf(frames, {10}, BB_TYPE_FP32, true);
    put_fp32(dy_buf, dy, 10, frames);
    auto dx_buf = net->Backward(dy_buf);
    if (dx_out) get_fp32(dx_buf, dx_out, 3 * hw * hw, frames);
    wo = 0;
    for (int l = 0; l < 14; ++l) {
        if (dW_out) get_dW(luts[l], dW_out + wo, widths[l]);
        wo += (size_t)widths[l] * 64;
    }
    return 0;
}

// bb::RealToBinary<bb::Bit,float>::Forward on an input of node shape {depth, point_size}.  seed == 0: deterministic modulation;
// otherwise thresholds come from UniformDistributionGenerator<float>(0, 1, seed), data-wise, and th_out [node][out_frame]
// receives the threshold each comparison used (the same generator is replayed in the draw order of RealToBinary.h:360-392).
int bbref_real_to_binary(float const *x, int depth, int point_size, int frames, int frame_mod, int depth_mod, std::uint64_t seed,
                         std::uint32_t *y_bits, float *th_out)
{
    std::shared_ptr<bb::ValueGenerator<float>> gen;
    if (seed) gen = bb::UniformDistributionGenerator<float>::Create(0.0f, 1.0f, seed);
    auto r2b = bb::RealToBinary<bb::Bit, float>::Create(frame_mod, depth_mod, gen, false);
    r2b->SendCommand("host_only true");
    const int nodes = depth * point_size;
    bb::FrameBuffer x_buf(frames, {depth, point_size}, BB_TYPE_FP32, true);
    put_fp32(x_buf, x, nodes, frames);
    auto y_buf = r2b->Forward(x_buf, true);
    get_bit(y_buf, y_bits, nodes * depth_mod, frames * frame_mod);
    if (seed && th_out) {
        auto replay = bb::UniformDistributionGenerator<float>::Create(0.0f, 1.0f, seed);
        int out_frames = frames * frame_mod;
        for (int of = 0; of < out_frames; ++of) {
            float th = replay->GetValue();
            for (int n = 0; n < nodes; ++n) {
                th_out[(size_t)n * out_frames + of] = th;
                th = replay->GetValue();
            }
        }
    }
    return 0;
}

// bb::BinaryToReal<bb::Bit,float>: forward of bit frames [x_nodes][y_frames * frame_mux] to fp32 [y_nodes][y_frames], then backward of dy.
int bbref_binary_to_real(std::uint32_t const *x_bits, int x_nodes, int y_nodes, int y_frames, int frame_mux, float *y, float const *dy, float *dx)
{
    auto b2r = bb::BinaryToReal<bb::Bit, float>::Create(frame_mux, bb::indices_t({y_nodes}));
    b2r->SendCommand("host_only true");
    bb::FrameBuffer x_buf(y_frames * frame_mux, {x_nodes}, BB_TYPE_BIT, true);
    put_bit(x_buf, x_bits, x_nodes, y_frames * frame_mux);
    auto y_buf = b2r->Forward(x_buf, true);
    if (y) get_fp32(y_buf, y, y_nodes, y_frames);
    if (dy && dx) {
        bb::FrameBuffer dy_buf(y_frames, {y_nodes}, BB_TYPE_FP32, true);
        put_fp32(dy_buf, dy, y_nodes, y_frames);
        auto dx_buf = b2r->Backward(dy_buf);
        get_fp32(dx_buf, dx, x_nodes, y_frames * frame_mux);
    }
    return 0;
}

// bb::ConvolutionIm2Col: forward of x [c*h*w][frames] to y [c*fh*fw][frames*oh*ow], then (fp32 only) backward of dy.
// bit != 0 runs the <bb::Bit, float> instantiation on packed words (forward only).
int bbref_im2col(int bit, void const *x, int c, int h, int w, int frames, int fh, int fw, int y_stride, int x_stride, char const *padding,
                 char const *border_mode, void *y, float const *dy, float *dx, int *out_hw)
{
    const int in_nodes = c * h * w, out_nodes = c * fh * fw;
    if (bit) {
        auto layer = bb::ConvolutionIm2Col<bb::Bit, float>::Create(fh, fw, y_stride, x_stride, padding, border_mode);
        layer->SendCommand("host_only true");
        bb::FrameBuffer x_buf(frames, {c, h, w}, BB_TYPE_BIT, true);
        put_bit(x_buf, (std::uint32_t const *)x, in_nodes, frames);
        auto y_buf = layer->Forward(x_buf, true);
        if (out_hw) *out_hw = (int)(y_buf.GetFrameSize() / frames);
        if (y) get_bit(y_buf, (std::uint32_t *)y, out_nodes, (int)y_buf.GetFrameSize());
        return 0;
    }
    auto layer = bb::ConvolutionIm2Col<float, float>::Create(fh, fw, y_stride, x_stride, padding, border_mode);
    layer->SendCommand("host_only true");
    bb::FrameBuffer x_buf(frames, {c, h, w}, BB_TYPE_FP32, true);
    put_fp32(x_buf, (float const *)x, in_nodes, frames);
    auto y_buf = layer->Forward(x_buf, true);
    const int out_frames = (int)y_buf.GetFrameSize();
    if (out_hw) *out_hw = out_frames / frames;
    if (y) get_fp32(y_buf, (float *)y, out_nodes, out_frames);
    if (dy && dx) {
        bb::FrameBuffer dy_buf(out_frames, {c, fh, fw}, BB_TYPE_FP32, true);
        put_fp32(dy_buf, dy, out_nodes, out_frames);
        auto dx_buf = layer->Backward(dy_buf);
        get_fp32(dx_buf, dx, in_nodes, frames);
    }
    return 0;
}

// bb::ConvolutionCol2Im: x [c][out_frames*h*w] to y [c*h*w][out_frames]; (fp32 only) backward of dy.
int bbref_col2im(int bit, void const *x, int c, int h, int w, int out_frames, void *y, float const *dy, float *dx)
{
    const int in_frames = out_frames * h * w, out_nodes = c * h * w;
    if (bit) {
        auto layer = bb::ConvolutionCol2Im<bb::Bit, float>::Create(h, w);
        layer->SendCommand("host_only true");
        layer->SetInputShape({c});                       // Forward() does not derive the channel count itself
        bb::FrameBuffer x_buf(in_frames, {c}, BB_TYPE_BIT, true);
        put_bit(x_buf, (std::uint32_t const *)x, c, in_frames);
        auto y_buf = layer->Forward(x_buf, true);
        if (y) get_bit(y_buf, (std::uint32_t *)y, out_nodes, out_frames);
        return 0;
    }
    auto layer = bb::ConvolutionCol2Im<float, float>::Create(h, w);
    layer->SendCommand("host_only true");
    layer->SetInputShape({c});
    bb::FrameBuffer x_buf(in_frames, {c}, BB_TYPE_FP32, true);
    put_fp32(x_buf, (float const *)x, c, in_frames);
    auto y_buf = layer->Forward(x_buf, true);
    if (y) get_fp32(y_buf, (float *)y, out_nodes, out_frames);
    if (dy && dx) {
        bb::FrameBuffer dy_buf(out_frames, {c, h, w}, BB_TYPE_FP32, true);
        put_fp32(dy_buf, dy, out_nodes, out_frames);
        auto dx_buf = layer->Backward(dy_buf);
        get_fp32(dx_buf, dx, c, in_frames);
    }
    return 0;
}

// bb::MaxPooling: forward of x [c*h*w][frames] to y [c*oh*ow][frames] and backward of dy.
int bbref_maxpool(int bit, void const *x, int c, int h, int w, int frames, int fh, int fw, void *y, float const *dy, float *dx)
{
    const int oh = (h + fh - 1) / fh, ow = (w + fw - 1) / fw;
    const int in_nodes = c * h * w, out_nodes = c * oh * ow;
    bb::FrameBuffer dy_buf;
    if (dy) {
        dy_buf = bb::FrameBuffer(frames, {c, oh, ow}, BB_TYPE_FP32, true);
        put_fp32(dy_buf, dy, out_nodes, frames);
    }
    if (bit) {
        auto layer = bb::MaxPooling<bb::Bit, float>::Create(fh, fw);
        layer->SendCommand("host_only true");
        bb::FrameBuffer x_buf(frames, {c, h, w}, BB_TYPE_BIT, true);
        put_bit(x_buf, (std::uint32_t const *)x, in_nodes, frames);
        auto y_buf = layer->Forward(x_buf, true);
        if (y) get_bit(y_buf, (std::uint32_t *)y, out_nodes, frames);
        if (dy && dx) get_fp32(layer->Backward(dy_buf), dx, in_nodes, frames);
        return 0;
    }
    auto layer = bb::MaxPooling<float, float>::Create(fh, fw);
    layer->SendCommand("host_only true");
    bb::FrameBuffer x_buf(frames, {c, h, w}, BB_TYPE_FP32, true);
    put_fp32(x_buf, (float const *)x, in_nodes, frames);
    auto y_buf = layer->Forward(x_buf, true);
    if (y) get_fp32(y_buf, (float *)y, out_nodes, frames);
    if (dy && dx) get_fp32(layer->Backward(dy_buf), dx, in_nodes, frames);
    return 0;
}

// Serialisation.  kind: 0 DifferentiableLutN<6,float>, 1 DifferentiableLutN<6,Bit>, 2 StochasticLutN<6,float>, 3 BinaryLutN<6,Bit>.
// dump: build a layer with the given state (tables: W [O][64] fp32, or [O][2] int32 truth tables for kind 3) and write its DumpObject
// bytes into buf (returns the byte count, negated when cap is too small).  load: LoadObject from bytes, read the state back out.
long long bbref_layer_dump(int kind, int I, int O, int const *idx, void const *tables, float const *rmean, float const *rvar, int batch_norm,
                           int binary, int lut_binarize, float gamma, float beta, float momentum, unsigned char *buf, long long cap)
{
    if (kind == 0 || kind == 1) {
        auto make = [&](auto tag) {
            using L = bb::DifferentiableLutN<6, decltype(tag)>;
            typename L::create_t c;
            c.output_shape = {O};
            c.batch_norm = batch_norm != 0; c.binary = binary != 0;
            c.momentum = momentum; c.gamma = gamma; c.beta = beta;
            auto lut = L::Create(c);
            lut->SendCommand(lut_binarize ? "lut_binarize true" : "lut_binarize false");
            fill_sparse(lut, I, O, idx, (float const *)tables);
            auto m = lut->lock_mean(); auto v = lut->lock_var();
            for (int n = 0; n < O; ++n) { m[n] = rmean[n]; v[n] = rvar[n]; }
            return dump_to(lut, buf, cap);
        };
        return kind == 0 ? make(float()) : make(bb::Bit());
    }
    if (kind == 2) {
        auto lut = bb::StochasticLutN<6, float>::Create(O);
        lut->SendCommand(binary ? "binary true" : "binary false");
        lut->SendCommand(lut_binarize ? "lut_binarize true" : "lut_binarize false");
        fill_sparse(lut, I, O, idx, (float const *)tables);
        return dump_to(lut, buf, cap);
    }
    auto lut = bb::BinaryLutN<6, bb::Bit>::Create(O);
    lut->SetInputShape({I});
    std::int32_t const *t = (std::int32_t const *)tables;
    for (int n = 0; n < O; ++n) {
        for (int k = 0; k < 6; ++k) lut->SetNodeConnectionIndex(n, k, idx[n * 6 + k]);
        for (int i = 0; i < 64; ++i) lut->SetLutTable(n, i, (t[n * 2 + (i >> 5)] >> (i & 31)) & 1);
    }
    return dump_to(lut, buf, cap);
}

// flags_out: [lut_binarize, binary, batch_norm]; params_out: [gamma, beta, momentum]
int bbref_layer_load(int kind, unsigned char const *buf, long long size, int I, int O, int *idx, void *tables, float *rmean, float *rvar,
                     int *flags_out, float *params_out)
{
    std::istringstream is(std::string((char const *)buf, (size_t)size), std::ios::binary);
    if (kind == 0 || kind == 1) {
        auto run = [&](auto tag) {
            using L = bb::DifferentiableLutN<6, decltype(tag)>;
            auto lut = L::Create(O);
            lut->LoadObject(is);
            if ((int)lut->GetInputNodeSize() != I || (int)lut->GetOutputNodeSize() != O) return 1;
            read_sparse(lut, O, idx, (float *)tables);
            auto m = lut->lock_mean_const(); auto v = lut->lock_var_const();
            for (int n = 0; n < O; ++n) { rmean[n] = m[n]; rvar[n] = v[n]; }
            std::ostringstream info;
            lut->PrintInfo(1, info);                // the flags are only exposed through the printed summary
            std::string txt = info.str();
            flags_out[0] = txt.find("lut_binarize : 1") != std::string::npos;
            flags_out[1] = txt.find("binary : 1") != std::string::npos;
            flags_out[2] = txt.find("batch_norm : 1") != std::string::npos;
            params_out[0] = (float)lut->GetGamma(); params_out[1] = (float)lut->GetBeta(); params_out[2] = 0.0f;
            return 0;
        };
        return kind == 0 ? run(float()) : run(bb::Bit());
    }
    if (kind == 2) {
        auto lut = bb::StochasticLutN<6, float>::Create(O);
        lut->LoadObject(is);
        if ((int)lut->GetInputNodeSize() != I || (int)lut->GetOutputNodeSize() != O) return 1;
        read_sparse(lut, O, idx, (float *)tables);
        return 0;
    }
    auto lut = bb::BinaryLutN<6, bb::Bit>::Create(O);
    lut->LoadObject(is);
    if ((int)lut->GetInputNodeSize() != I || (int)lut->GetOutputNodeSize() != O) return 1;
    std::int32_t *t = (std::int32_t *)tables;
    for (int n = 0; n < O; ++n) {
        t[n * 2] = t[n * 2 + 1] = 0;
        for (int k = 0; k < 6; ++k) idx[n * 6 + k] = (int)lut->GetNodeConnectionIndex(n, k);
        for (int i = 0; i < 64; ++i) if (lut->GetLutTable(n, i)) t[n * 2 + (i >> 5)] |= (std::int32_t)(1u << (i & 31));
    }
    return 0;
}

// LoadObject `buf` into a fresh reference layer of the kind and DumpObject it again: equal bytes mean the reference read every field.
long long bbref_layer_redump(int kind, unsigned char const *buf, long long size, int O, unsigned char *out, long long cap)
{
    std::istringstream is(std::string((char const *)buf, (size_t)size), std::ios::binary);
    if (kind == 0) { auto l = bb::DifferentiableLutN<6, float>::Create(O);   l->LoadObject(is); return dump_to(l, out, cap); }
    if (kind == 1) { auto l = bb::DifferentiableLutN<6, bb::Bit>::Create(O); l->LoadObject(is); return dump_to(l, out, cap); }
    if (kind == 2) { auto l = bb::StochasticLutN<6, float>::Create(O);       l->LoadObject(is); return dump_to(l, out, cap); }
    auto l = bb::BinaryLutN<6, bb::Bit>::Create(O);
    l->LoadObject(is);
    return dump_to(l, out, cap);
}

int bbref_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// A launcher may have exported OMP_NUM_THREADS=1 to this process (torch.distributed.run does): the timed legs set the team size themselves.
void bbref_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}   // extern "C"
