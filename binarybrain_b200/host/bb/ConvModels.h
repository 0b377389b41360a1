// Host-side classes of the convolution lowering, in BinaryBrain's style, over the C ABI (no CPU branch behind them):
//   bb::ConvolutionIm2Col<FT,BT>   include/bb/ConvolutionIm2Col.h:25-565
//   bb::ConvolutionCol2Im<FT,BT>   include/bb/ConvolutionCol2Im.h:24-370
//   bb::MaxPooling<FT,BT>          include/bb/MaxPooling.h:24-741
//   bb::Convolution2d<FT,BT>       include/bb/Convolution2d.h:30-410  (Im2Col -> per-pixel layer -> Col2Im)
// FT = float or bb::Bit (frame type of the forward pass), BT = float (gradients).
#pragma once

#include <stack>

#include "LutModels.h"

namespace bb {

enum { BB_BORDER_CONSTANT = 0, BB_BORDER_REFLECT = 1, BB_BORDER_REFLECT_101 = 2, BB_BORDER_REPLICATE = 3, BB_BORDER_WRAP = 4 };

template <typename FT> struct frame_type_of            { static constexpr int value = BB_TYPE_FP32; };
template <>            struct frame_type_of<Bit>       { static constexpr int value = BB_TYPE_BIT; };

template <typename FT = float, typename BT = float>
class ConvolutionIm2Col : public Model
{
    indices_t m_input_shape, m_output_shape;
    index_t m_input_frame_size = 1;
    index_t m_c = 1, m_h = 1, m_w = 1, m_fh = 1, m_fw = 1, m_ys = 1, m_xs = 1, m_yo = 0, m_xo = 0, m_oh = 1, m_ow = 1;
    std::string m_padding = "valid";
    int   m_border_mode  = BB_BORDER_REFLECT_101;
    float m_border_value = 0.0f;

    static int BorderConv(std::string const &mode)
    {
        if (mode == "constant")    return BB_BORDER_CONSTANT;
        if (mode == "reflect")     return BB_BORDER_REFLECT;
        if (mode == "reflect_101") return BB_BORDER_REFLECT_101;
        if (mode == "replicate")   return BB_BORDER_REPLICATE;
        if (mode == "wrap")        return BB_BORDER_WRAP;
        throw std::runtime_error("unknown border mode " + mode);
    }

public:
    struct create_t {
        index_t filter_h_size = 1, filter_w_size = 1, x_stride = 1, y_stride = 1;
        std::string padding = "valid", border_mode = "reflect_101";
        float border_value = 0.0f;
    };
    explicit ConvolutionIm2Col(create_t const &c)
        : m_fh(c.filter_h_size), m_fw(c.filter_w_size), m_ys(c.y_stride), m_xs(c.x_stride), m_padding(c.padding),
          m_border_mode(BorderConv(c.border_mode)), m_border_value(c.border_value) {}
    static std::shared_ptr<ConvolutionIm2Col> Create(create_t const &c) { return std::make_shared<ConvolutionIm2Col>(c); }
    static std::shared_ptr<ConvolutionIm2Col> Create(index_t filter_h_size, index_t filter_w_size, index_t y_stride = 1, index_t x_stride = 1,
                                                     std::string padding = "valid", std::string border_mode = "reflect_101")
    {
        create_t c;
        c.filter_h_size = filter_h_size; c.filter_w_size = filter_w_size; c.y_stride = y_stride; c.x_stride = x_stride;
        c.padding = padding; c.border_mode = border_mode;
        return Create(c);
    }
    std::string GetModelName() const override { return "ConvolutionIm2Col"; }
    indices_t GetInputShape()  const override { return m_input_shape; }
    indices_t GetOutputShape() const override { return m_output_shape; }
    index_t GetOutputHeight() const { return m_oh; }
    index_t GetOutputWidth()  const { return m_ow; }

    // include/bb/ConvolutionIm2Col.h:188-228
    indices_t SetInputShape(indices_t shape) override
    {
        if (shape == m_input_shape) return m_output_shape;
        BB_ASSERT(shape.size() == 3);
        m_input_shape = shape;
        m_c = shape[0]; m_h = shape[1]; m_w = shape[2];
        if (m_padding == "valid") {
            m_oh = ((m_h - m_fh + 1) + (m_ys - 1)) / m_ys;
            m_ow = ((m_w - m_fw + 1) + (m_xs - 1)) / m_xs;
            m_yo = 0; m_xo = 0;
        } else if (m_padding == "same") {
            m_oh = (m_h + (m_ys - 1)) / m_ys;
            m_ow = (m_w + (m_xs - 1)) / m_xs;
            m_yo = (m_fh - 1) / 2; m_xo = (m_fw - 1) / 2;
        } else {
            throw std::runtime_error("unknown padding " + m_padding);
        }
        m_output_shape = indices_t({m_c, m_fh, m_fw});
        return m_output_shape;
    }

    FrameBuffer Forward(FrameBuffer x_buf, bool /*train*/ = true) override
    {
        BB_ASSERT(x_buf.GetType() == frame_type_of<FT>::value);
        if (x_buf.GetShape() != m_input_shape) SetInputShape(x_buf.GetShape());
        m_input_frame_size = x_buf.GetFrameSize();
        FrameBuffer y_buf(m_input_frame_size * m_oh * m_ow, m_output_shape, x_buf.GetType());
        int xs = (int)(x_buf.GetFrameStride() / 4), ys = (int)(y_buf.GetFrameStride() / 4);
        if (x_buf.GetType() == BB_TYPE_FP32)
            BBCU_CHECK(bbcu_fp32_Im2Col_Forward((float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), (int)m_xs, (int)m_ys,
                                                (int)m_xo, (int)m_yo, (int)m_input_frame_size, xs, (int)m_w, (int)m_h, (int)m_c, (int)m_ow, (int)m_oh, ys,
                                                (int)m_fw, (int)m_fh, m_border_mode, m_border_value, Manager::Stream()));
        else
            BBCU_CHECK(bbcu_bit_Im2Col_Forward((int const *)x_buf.LockDeviceMemoryConst(), (int *)y_buf.LockDeviceMemory(true), (int)m_xs, (int)m_ys, (int)m_xo,
                                               (int)m_yo, (int)m_input_frame_size, xs, (int)m_w, (int)m_h, (int)m_c, (int)m_ow, (int)m_oh, ys, (int)m_fw,
                                               (int)m_fh, m_border_mode, Manager::Stream()));
        return y_buf;
    }

    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        if (dy_buf.Empty()) return dy_buf;
        BB_ASSERT(dy_buf.GetType() == BB_TYPE_FP32);
        FrameBuffer dx_buf(m_input_frame_size, m_input_shape, BB_TYPE_FP32);
        BBCU_CHECK(bbcu_fp32_Im2Col_Backward((float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), (int)m_xs, (int)m_ys,
                                             (int)m_xo, (int)m_yo, (int)m_input_frame_size, (int)(dx_buf.GetFrameStride() / 4), (int)m_w, (int)m_h, (int)m_c,
                                             (int)m_ow, (int)m_oh, (int)(dy_buf.GetFrameStride() / 4), (int)m_fw, (int)m_fh, Manager::Stream()));
        return dx_buf;
    }
};


template <typename FT = float, typename BT = float>
class ConvolutionCol2Im : public Model
{
    indices_t m_input_shape;
    index_t m_c = 1, m_h = 1, m_w = 1;

public:
    struct create_t { index_t h_size = 1, w_size = 1; };
    explicit ConvolutionCol2Im(create_t const &c) : m_h(c.h_size), m_w(c.w_size) {}
    static std::shared_ptr<ConvolutionCol2Im> Create(create_t const &c) { return std::make_shared<ConvolutionCol2Im>(c); }
    static std::shared_ptr<ConvolutionCol2Im> Create(index_t h_size = 1, index_t w_size = 1) { create_t c; c.h_size = h_size; c.w_size = w_size; return Create(c); }
    std::string GetModelName() const override { return "ConvolutionCol2Im"; }
    void SetOutputSize(index_t h_size, index_t w_size) { m_h = h_size; m_w = w_size; }
    indices_t SetInputShape(indices_t shape) override { m_input_shape = shape; m_c = CalcShapeSize(shape); return GetOutputShape(); }
    indices_t GetInputShape()  const override { return m_input_shape; }
    indices_t GetOutputShape() const override { return indices_t({m_c, m_h, m_w}); }

    FrameBuffer Forward(FrameBuffer x_buf, bool /*train*/ = true) override
    {
        BB_ASSERT(x_buf.GetType() == frame_type_of<FT>::value);
        if (x_buf.GetShape() != m_input_shape) SetInputShape(x_buf.GetShape());
        BB_ASSERT(x_buf.GetFrameSize() % (m_h * m_w) == 0);
        index_t out_frames = x_buf.GetFrameSize() / (m_h * m_w);
        FrameBuffer y_buf(out_frames, GetOutputShape(), x_buf.GetType());
        int xs = (int)(x_buf.GetFrameStride() / 4), ys = (int)(y_buf.GetFrameStride() / 4);
        if (x_buf.GetType() == BB_TYPE_FP32)
            BBCU_CHECK(bbcu_fp32_Col2Im_Forward((float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), (int)m_w, (int)m_h, (int)m_c,
                                                xs, (int)out_frames, ys, Manager::Stream()));
        else
            BBCU_CHECK(bbcu_bit_Col2Im_Forward((int const *)x_buf.LockDeviceMemoryConst(), (int *)y_buf.LockDeviceMemory(true), (int)m_w, (int)m_h, (int)m_c, xs,
                                               (int)out_frames, ys, Manager::Stream()));
        return y_buf;
    }

    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        if (dy_buf.Empty()) return dy_buf;
        BB_ASSERT(dy_buf.GetType() == BB_TYPE_FP32);
        index_t out_frames = dy_buf.GetFrameSize();
        FrameBuffer dx_buf(out_frames * m_h * m_w, indices_t({m_c}), BB_TYPE_FP32);
        BBCU_CHECK(bbcu_fp32_Col2Im_Backward((float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), (int)m_w, (int)m_h, (int)m_c,
                                             (int)(dx_buf.GetFrameStride() / 4), (int)out_frames, (int)(dy_buf.GetFrameStride() / 4), Manager::Stream()));
        return dx_buf;
    }
};


template <typename FT = float, typename BT = float>
class MaxPooling : public Model
{
    indices_t m_input_shape, m_output_shape;
    index_t m_fh = 1, m_fw = 1, m_c = 1, m_h = 1, m_w = 1, m_oh = 1, m_ow = 1;
    std::stack<std::shared_ptr<Memory>> m_argmax;           // fp32 layer: int32 [c*oh*ow][frame stride], kept for backward

public:
    struct create_t { index_t filter_h_size = 1, filter_w_size = 1; };
    explicit MaxPooling(create_t const &c) : m_fh(c.filter_h_size), m_fw(c.filter_w_size) {}
    static std::shared_ptr<MaxPooling> Create(create_t const &c) { return std::make_shared<MaxPooling>(c); }
    static std::shared_ptr<MaxPooling> Create(index_t filter_h_size = 1, index_t filter_w_size = 1)
    {
        create_t c; c.filter_h_size = filter_h_size; c.filter_w_size = filter_w_size;
        return Create(c);
    }
    std::string GetModelName() const override { return "MaxPooling"; }
    indices_t GetInputShape()  const override { return m_input_shape; }
    indices_t GetOutputShape() const override { return m_output_shape; }

    // include/bb/MaxPooling.h:118-137: output size rounded up
    indices_t SetInputShape(indices_t shape) override
    {
        if (shape == m_input_shape) return m_output_shape;
        BB_ASSERT(shape.size() == 3);
        m_input_shape = shape;
        m_c = shape[0]; m_h = shape[1]; m_w = shape[2];
        m_ow = (m_w + m_fw - 1) / m_fw;
        m_oh = (m_h + m_fh - 1) / m_fh;
        m_output_shape = indices_t({m_c, m_oh, m_ow});
        return m_output_shape;
    }

    FrameBuffer Forward(FrameBuffer x_buf, bool train = true) override
    {
        BB_ASSERT(x_buf.GetType() == frame_type_of<FT>::value);
        if (x_buf.GetShape() != m_input_shape) SetInputShape(x_buf.GetShape());
        FrameBuffer y_buf(x_buf.GetFrameSize(), m_output_shape, x_buf.GetType());
        int F = (int)x_buf.GetFrameSize(), s = (int)(x_buf.GetFrameStride() / 4);
        if (x_buf.GetType() == BB_TYPE_BIT) {
            if (train) PushFrameBuffer(x_buf);              // the bit layer's backward re-reads its input (MaxPooling.h:329-333)
            BBCU_CHECK(bbcu_bit_MaxPooling_Forward((int const *)x_buf.LockDeviceMemoryConst(), (int *)y_buf.LockDeviceMemory(true), (int)m_fh, (int)m_fw, (int)m_w,
                                                   (int)m_h, (int)m_ow, (int)m_oh, (int)m_c, F, s, Manager::Stream()));
            return y_buf;
        }
        std::shared_ptr<Memory> argmax;
        if (train) {
            argmax = std::make_shared<Memory>((std::size_t)(y_buf.GetFrameStride() * y_buf.GetNodeSize()));
            m_argmax.push(argmax);
        }
        BBCU_CHECK(bbcu_fp32_MaxPooling_Forward((float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true),
                                                argmax ? (int *)argmax->Dev(true) : nullptr, (int)m_fh, (int)m_fw, (int)m_w, (int)m_h, (int)m_ow, (int)m_oh,
                                                (int)m_c, F, s, Manager::Stream()));
        return y_buf;
    }

    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        if (dy_buf.Empty()) return dy_buf;
        BB_ASSERT(dy_buf.GetType() == BB_TYPE_FP32);
        FrameBuffer dx_buf(dy_buf.GetFrameSize(), m_input_shape, BB_TYPE_FP32);
        int F = (int)dy_buf.GetFrameSize(), s = (int)(dy_buf.GetFrameStride() / 4);
        if (frame_type_of<FT>::value == BB_TYPE_BIT) {
            FrameBuffer x_buf = PopFrameBuffer();
            BBCU_CHECK(bbcu_bit_fp32_MaxPooling_Backward((int const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(),
                                                         (float *)dx_buf.LockDeviceMemory(true), (int)m_fh, (int)m_fw, (int)m_w, (int)m_h, (int)m_ow, (int)m_oh,
                                                         (int)m_c, F, (int)(x_buf.GetFrameStride() / 4), s, Manager::Stream()));
            return dx_buf;
        }
        BB_ASSERT(!m_argmax.empty());
        std::shared_ptr<Memory> argmax = m_argmax.top();
        m_argmax.pop();
        BBCU_CHECK(bbcu_fp32_MaxPooling_Backward((int const *)argmax->DevConst(), (float const *)dy_buf.LockDeviceMemoryConst(),
                                                 (float *)dx_buf.LockDeviceMemory(true), (int)m_fh, (int)m_fw, (int)m_w, (int)m_h, (int)m_ow, (int)m_oh, (int)m_c, F, s,
                                                 Manager::Stream()));
        return dx_buf;
    }
};


// bb::Sequential (include/bb/Sequential.h): forward in order, backward in reverse.
class Sequential : public Model
{
    std::vector<std::shared_ptr<Model>> m_layers;

public:
    static std::shared_ptr<Sequential> Create() { return std::make_shared<Sequential>(); }
    std::string GetModelName() const override { return "Sequential"; }
    void Add(std::shared_ptr<Model> layer) { m_layers.push_back(layer); }
    index_t GetSize() const { return (index_t)m_layers.size(); }
    std::shared_ptr<Model> Get(index_t i) const { return m_layers.at((std::size_t)i); }
    indices_t SetInputShape(indices_t shape) override
    {
        for (auto &l : m_layers) shape = l->SetInputShape(shape);
        return shape;
    }
    indices_t GetInputShape()  const override { return m_layers.empty() ? indices_t() : m_layers.front()->GetInputShape(); }
    indices_t GetOutputShape() const override { return m_layers.empty() ? indices_t() : m_layers.back()->GetOutputShape(); }
    FrameBuffer Forward(FrameBuffer x_buf, bool train = true) override
    {
        for (auto &l : m_layers) x_buf = l->Forward(x_buf, train);
        return x_buf;
    }
    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        for (auto it = m_layers.rbegin(); it != m_layers.rend(); ++it) dy_buf = (*it)->Backward(dy_buf);
        return dy_buf;
    }
};


// Im2Col -> layer -> Col2Im.  `layer` sees {c, fh, fw} inputs and one output pixel per frame.
template <typename FT = float, typename BT = float>
class Convolution2d : public Model
{
    std::shared_ptr<ConvolutionIm2Col<FT, BT>> m_im2col;
    std::shared_ptr<Model>                     m_layer;
    std::shared_ptr<ConvolutionCol2Im<FT, BT>> m_col2im;
    indices_t m_input_shape;

public:
    struct create_t {
        std::shared_ptr<Model> layer;
        index_t filter_h_size = 1, filter_w_size = 1, x_stride = 1, y_stride = 1;
        std::string padding = "valid", border_mode = "reflect_101";
        float border_value = 0.0f;
    };
    explicit Convolution2d(create_t const &c) : m_layer(c.layer)
    {
        typename ConvolutionIm2Col<FT, BT>::create_t ic;
        ic.filter_h_size = c.filter_h_size; ic.filter_w_size = c.filter_w_size; ic.x_stride = c.x_stride; ic.y_stride = c.y_stride;
        ic.padding = c.padding; ic.border_mode = c.border_mode; ic.border_value = c.border_value;
        m_im2col = ConvolutionIm2Col<FT, BT>::Create(ic);
        m_col2im = ConvolutionCol2Im<FT, BT>::Create();     // its size follows from the input shape (Convolution2d.h:91)
    }
    static std::shared_ptr<Convolution2d> Create(create_t const &c) { return std::make_shared<Convolution2d>(c); }
    static std::shared_ptr<Convolution2d> Create(std::shared_ptr<Model> layer, index_t filter_h_size, index_t filter_w_size, index_t y_stride = 1,
                                                 index_t x_stride = 1, std::string padding = "valid", std::string border_mode = "reflect_101")
    {
        create_t c;
        c.layer = layer; c.filter_h_size = filter_h_size; c.filter_w_size = filter_w_size; c.y_stride = y_stride; c.x_stride = x_stride;
        c.padding = padding; c.border_mode = border_mode;
        return Create(c);
    }
    std::string GetModelName() const override { return "Convolution2d"; }
    std::shared_ptr<Model> GetLayer() const { return m_layer; }
    indices_t GetInputShape()  const override { return m_input_shape; }
    indices_t GetOutputShape() const override { return m_col2im->GetOutputShape(); }

    // include/bb/Convolution2d.h:213-247
    indices_t SetInputShape(indices_t shape) override
    {
        m_input_shape = shape;
        indices_t s = m_im2col->SetInputShape(shape);
        m_col2im->SetOutputSize(m_im2col->GetOutputHeight(), m_im2col->GetOutputWidth());
        s = m_layer->SetInputShape(s);
        return m_col2im->SetInputShape(s);
    }

    FrameBuffer Forward(FrameBuffer x_buf, bool train = true) override
    {
        if (x_buf.GetShape() != m_input_shape) SetInputShape(x_buf.GetShape());
        x_buf = m_im2col->Forward(x_buf, train);
        x_buf = m_layer->Forward(x_buf, train);
        return m_col2im->Forward(x_buf, train);
    }

    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        if (dy_buf.Empty()) return dy_buf;
        dy_buf = m_col2im->Backward(dy_buf);
        dy_buf = m_layer->Backward(dy_buf);
        return m_im2col->Backward(dy_buf);
    }
};

}   // namespace bb
