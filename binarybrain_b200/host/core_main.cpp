// pybind11 module `binarybrain_b200.core`: BinaryBrain's Python-facing class names for the LUT path
// (python/binarybrain/src/core_main.cpp:153-190,572-652,674-709,940-1067 in the reference), implemented by
// the C++ host classes of host/bb/*.h over the bbcu_* C ABI.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>

#include "bb/LutModels.h"
#include "bb/ConvModels.h"

namespace py = pybind11;
using namespace bb;

using DifferentiableLut6_fp32_fp32 = DifferentiableLutN<6, float, float>;
using DifferentiableLut6_bit_fp32  = DifferentiableLutN<6, Bit, float>;
using StochasticLut6_fp32_fp32     = StochasticLutN<6, float, float>;
using StochasticLut6_bit_fp32      = StochasticLutN<6, Bit, float>;
using BinaryLut6_bit_fp32          = BinaryLutN<6, Bit, float>;
using StochasticBatchNormalization_fp32 = StochasticBatchNormalization<float>;
using OptimizerAdam_fp32           = OptimizerAdam<float>;
using ConvolutionIm2Col_fp32_fp32   = ConvolutionIm2Col<float, float>;
using ConvolutionIm2Col_bit_fp32    = ConvolutionIm2Col<Bit, float>;
using ConvolutionCol2Im_fp32_fp32   = ConvolutionCol2Im<float, float>;
using ConvolutionCol2Im_bit_fp32    = ConvolutionCol2Im<Bit, float>;
using MaxPooling_fp32_fp32          = MaxPooling<float, float>;
using MaxPooling_bit_fp32           = MaxPooling<Bit, float>;
using Convolution2d_fp32_fp32       = Convolution2d<float, float>;
using Convolution2d_bit_fp32        = Convolution2d<Bit, float>;

static py::array_t<float> tensor_numpy(Tensor &t)
{
    indices_t shp = t.GetShape();
    py::array_t<float> a(std::vector<py::ssize_t>(shp.begin(), shp.end()));
    std::memcpy(a.mutable_data(), t.HostConst(), sizeof(float) * (size_t)t.GetSize());
    return a;
}

static void tensor_set_numpy(Tensor &t, py::array_t<float, py::array::c_style | py::array::forcecast> a)
{
    if ((index_t)a.size() != t.GetSize()) throw std::runtime_error("Tensor.set_numpy: size mismatch");
    std::memcpy(t.Host(true), a.data(), sizeof(float) * (size_t)a.size());
}

template <class L, class PyClass>
static void def_sparse(PyClass &c)
{
    c.def("W", [](L &l) { return l.GetParameters(); })
     .def("dW", [](L &l) { return l.GetGradients(); })
     .def("get_node_connection_size", &L::GetNodeConnectionSize)
     .def("get_node_connection_index", &L::GetNodeConnectionIndex)
     .def("set_node_connection_index", &L::SetNodeConnectionIndex)
     .def("get_connection", [](L &l) {
         index_t O = l.GetOutputNodeSize();
         py::array_t<std::int32_t> a(std::vector<py::ssize_t>{(py::ssize_t)O, (py::ssize_t)6});
         auto p = a.mutable_data();
         for (index_t o = 0; o < O; ++o) for (int i = 0; i < 6; ++i) p[o * 6 + i] = (std::int32_t)l.GetNodeConnectionIndex(o, i);
         return a;
     })
     .def("set_connection", [](L &l, py::array_t<std::int32_t, py::array::c_style | py::array::forcecast> a) {
         index_t O = l.GetOutputNodeSize();
         if (a.size() != O * 6) throw std::runtime_error("set_connection: expected [nodes, 6]");
         for (index_t o = 0; o < O; ++o) for (int i = 0; i < 6; ++i) l.SetNodeConnectionIndex(o, i, a.data()[o * 6 + i]);
     });
}

PYBIND11_MODULE(core, m)
{
    m.doc() = "BinaryBrain LUT6 hot path on B200: C++ host classes over libbbcu_b200";
    m.attr("TYPE_BIT")  = BB_TYPE_BIT;
    m.attr("TYPE_FP32") = BB_TYPE_FP32;

    m.def("get_device_count", &Manager::GetDeviceCount);
    m.def("set_device", &Manager::SetDevice);
    m.def("is_device_available", &Manager::IsDeviceAvailable);
    m.def("set_host_only", &Manager::SetHostOnly);
    m.def("synchronize", []() { BB_CUDA_CHECK(cudaStreamSynchronize(Manager::Stream())); });
    m.def("set_stream", [](std::uintptr_t s) { Manager::Stream() = reinterpret_cast<cudaStream_t>(s); },
          "install the CUDA stream (as an integer handle) every layer enqueues on");
    m.def("heap_allocated_size", []() { return bbcu_LocalHeap_GetAllocatedSize(); });
    m.def("heap_max_alloc_size", []() { return bbcu_LocalHeap_GetMaxAllocSize(); });
    m.def("heap_garbage_collect", []() { bbcu_LocalHeap_GarbageCollect(); });

    py::class_<Tensor, std::shared_ptr<Tensor>>(m, "Tensor")
        .def("get_shape", &Tensor::GetShape)
        .def("numpy", &tensor_numpy)
        .def("set_numpy", &tensor_set_numpy)
        .def("fill_zero", &Tensor::FillZero);

    py::class_<FrameBuffer>(m, "FrameBuffer")
        .def(py::init<>())
        .def(py::init<index_t, indices_t, int, bool>(), py::arg("frame_size"), py::arg("shape"), py::arg("data_type") = BB_TYPE_FP32,
             py::arg("host_only") = false)
        .def("empty", &FrameBuffer::Empty)
        .def("get_type", &FrameBuffer::GetType)
        .def("get_frame_size", &FrameBuffer::GetFrameSize)
        .def("get_frame_stride", &FrameBuffer::GetFrameStride)
        .def("get_node_size", &FrameBuffer::GetNodeSize)
        .def("get_node_shape", &FrameBuffer::GetShape)
        .def("fill_zero", &FrameBuffer::FillZero)
        .def("clone", &FrameBuffer::Clone)
        .def("copy_to", &FrameBuffer::CopyTo, py::arg("dst"), py::arg("frame_size") = 0, py::arg("src_frame_offset") = 0, py::arg("dst_frame_offset") = 0,
             py::arg("node_size") = 0, py::arg("src_node_offset") = 0, py::arg("dst_node_offset") = 0)
        .def("frame_range", &FrameBuffer::FrameRange, py::arg("size"), py::arg("offset") = 0)
        .def("range", &FrameBuffer::Range, py::arg("size"), py::arg("offset") = 0)
        .def("concatenate", &FrameBuffer::Concatenate)
        .def("convert_to", &FrameBuffer::ConvertTo)
        .def("is_host_pinned", &FrameBuffer::IsHostPinned)
        .def("lock_device", [](FrameBuffer &b) { return (std::uintptr_t)b.LockDeviceMemory(); })
        .def("get_fp32", &FrameBuffer::GetFP32)
        .def("set_fp32", &FrameBuffer::SetFP32)
        .def_static("calc_frame_stride", &FrameBuffer::CalcFrameStride)
        // numpy arrays carry frames on axis 0 and the node shape on the other axes (FrameBuffer.h:347-358)
        .def_static("from_numpy_fp32", [](py::array_t<float, py::array::c_style | py::array::forcecast> a, int data_type) {
            if (a.ndim() < 2) throw std::runtime_error("from_numpy: expected [frames, nodes...]");
            indices_t shape;
            for (py::ssize_t d = 1; d < a.ndim(); ++d) shape.push_back(a.shape(d));
            FrameBuffer b(a.shape(0), shape, data_type);
            b.SetFrameMajor(a.data());
            return b;
        }, py::arg("ndarray"), py::arg("data_type") = BB_TYPE_FP32)
        .def("numpy_fp32", [](FrameBuffer &b) {
            std::vector<py::ssize_t> shape{(py::ssize_t)b.GetFrameSize()};
            for (auto s : b.GetShape()) shape.push_back((py::ssize_t)s);
            py::array_t<float> a(shape);
            b.GetFrameMajor(a.mutable_data());
            return a;
        });

    py::class_<Model, std::shared_ptr<Model>>(m, "Model")
        .def("get_model_name", &Model::GetModelName)
        .def("get_object_name", &Model::GetObjectName)
        .def("set_name", &Model::SetName)
        .def("get_name", &Model::GetName)
        .def("dump_bytes", [](Model &m) { return py::bytes(m.DumpObjectBytes()); })
        .def("load_bytes", [](Model &m, py::bytes b) { m.LoadObjectBytes(std::string(b)); })
        .def("send_command", &Model::SendCommand, py::arg("command"))
        .def("get_input_shape", &Model::GetInputShape)
        .def("set_input_shape", &Model::SetInputShape)
        .def("get_output_shape", &Model::GetOutputShape)
        .def("get_input_node_size", &Model::GetInputNodeSize)
        .def("get_output_node_size", &Model::GetOutputNodeSize)
        .def("forward", &Model::Forward, py::arg("x_buf"), py::arg("train") = true)
        .def("backward", &Model::Backward)
        .def("clear", &Model::Clear);

    {
        py::class_<DifferentiableLut6_fp32_fp32, Model, std::shared_ptr<DifferentiableLut6_fp32_fp32>> c(m, "DifferentiableLut6_fp32_fp32");
        c.def_static("create", &DifferentiableLut6_fp32_fp32::CreatePy, py::arg("output_shape"), py::arg("batch_norm") = true, py::arg("binary") = true,
                     py::arg("connection") = "", py::arg("momentum") = 0.0, py::arg("gamma") = 0.3, py::arg("beta") = 0.5, py::arg("seed") = 1)
         .def("get_mean", [](DifferentiableLut6_fp32_fp32 &l) -> Tensor & { return l.running_mean(); }, py::return_value_policy::reference_internal)
         .def("get_var", [](DifferentiableLut6_fp32_fp32 &l) -> Tensor & { return l.running_var(); }, py::return_value_policy::reference_internal)
         .def("set_frame_shard", [](DifferentiableLut6_fp32_fp32 &l, index_t total_frames, py::object allreduce_sums, py::object allreduce_grads) {
             // the callbacks receive (device pointer, element count, stream) as integers, e.g. to wrap the memory for torch.distributed
             DifferentiableLut6_fp32_fp32::AllReduceF64 f64;
             DifferentiableLut6_fp32_fp32::AllReduceF32 f32;
             if (!allreduce_sums.is_none())
                 f64 = [allreduce_sums](double *p, std::size_t n, cudaStream_t s) { allreduce_sums((std::uintptr_t)p, n, (std::uintptr_t)s); };
             if (!allreduce_grads.is_none())
                 f32 = [allreduce_grads](float *p, std::size_t n, cudaStream_t s) { allreduce_grads((std::uintptr_t)p, n, (std::uintptr_t)s); };
             l.SetFrameShard(total_frames, f64, f32);
         }, py::arg("total_frames"), py::arg("allreduce_sums"), py::arg("allreduce_grads") = py::none())
         .def("get_total_frames", &DifferentiableLut6_fp32_fp32::GetTotalFrames)
         .def("get_gamma", &DifferentiableLut6_fp32_fp32::GetGamma)
         .def("get_beta", &DifferentiableLut6_fp32_fp32::GetBeta)
         .def("forward_node", &DifferentiableLut6_fp32_fp32::ForwardNode, py::arg("node"), py::arg("input_value"));
        def_sparse<DifferentiableLut6_fp32_fp32>(c);
    }
    {
        py::class_<DifferentiableLut6_bit_fp32, Model, std::shared_ptr<DifferentiableLut6_bit_fp32>> c(m, "DifferentiableLut6_bit_fp32");
        c.def_static("create", &DifferentiableLut6_bit_fp32::CreatePy, py::arg("output_shape"), py::arg("batch_norm") = true, py::arg("binary") = true,
                     py::arg("connection") = "", py::arg("momentum") = 0.0, py::arg("gamma") = 0.3, py::arg("beta") = 0.5, py::arg("seed") = 1)
         .def("get_mean", [](DifferentiableLut6_bit_fp32 &l) -> Tensor & { return l.running_mean(); }, py::return_value_policy::reference_internal)
         .def("get_var", [](DifferentiableLut6_bit_fp32 &l) -> Tensor & { return l.running_var(); }, py::return_value_policy::reference_internal)
         .def("forward_node", &DifferentiableLut6_bit_fp32::ForwardNode, py::arg("node"), py::arg("input_value"));
        def_sparse<DifferentiableLut6_bit_fp32>(c);
    }
    {
        py::class_<StochasticLut6_fp32_fp32, Model, std::shared_ptr<StochasticLut6_fp32_fp32>> c(m, "StochasticLut6_fp32_fp32");
        c.def_static("create", &StochasticLut6_fp32_fp32::CreatePy, py::arg("output_shape"), py::arg("connection") = "", py::arg("seed") = 1);
        def_sparse<StochasticLut6_fp32_fp32>(c);
    }
    {
        py::class_<StochasticLut6_bit_fp32, Model, std::shared_ptr<StochasticLut6_bit_fp32>> c(m, "StochasticLut6_bit_fp32");
        c.def_static("create", &StochasticLut6_bit_fp32::CreatePy, py::arg("output_shape"), py::arg("connection") = "", py::arg("seed") = 1);
        def_sparse<StochasticLut6_bit_fp32>(c);
    }
    py::class_<BinaryLut6_bit_fp32, Model, std::shared_ptr<BinaryLut6_bit_fp32>>(m, "BinaryLut6_bit_fp32")
        .def_static("create", &BinaryLut6_bit_fp32::CreatePy, py::arg("output_shape"), py::arg("connection") = "", py::arg("seed") = 1)
        .def("get_node_connection_index", &BinaryLut6_bit_fp32::GetNodeConnectionIndex)
        .def("set_node_connection_index", &BinaryLut6_bit_fp32::SetNodeConnectionIndex)
        .def("get_lut_table_size", &BinaryLut6_bit_fp32::GetLutTableSize)
        .def("get_lut_table", &BinaryLut6_bit_fp32::GetLutTable)
        .def("set_lut_table", &BinaryLut6_bit_fp32::SetLutTable)
        .def("import_layer", [](BinaryLut6_bit_fp32 &b, DifferentiableLut6_fp32_fp32 &src) { b.ImportLayer(src); })
        .def("import_layer", [](BinaryLut6_bit_fp32 &b, DifferentiableLut6_bit_fp32 &src) { b.ImportLayer(src); })
        .def("import_layer", [](BinaryLut6_bit_fp32 &b, StochasticLut6_fp32_fp32 &src) { b.ImportLayer(src); });

    py::class_<StochasticBatchNormalization_fp32, Model, std::shared_ptr<StochasticBatchNormalization_fp32>>(m, "StochasticBatchNormalization_fp32")
        .def_static("create", &StochasticBatchNormalization_fp32::Create, py::arg("momentum") = 0.9f, py::arg("gamma") = 0.2f, py::arg("beta") = 0.5f)
        .def("reforward", &StochasticBatchNormalization_fp32::ReForward)
        .def("get_mean", [](StochasticBatchNormalization_fp32 &l) -> Tensor & { return l.running_mean(); }, py::return_value_policy::reference_internal)
        .def("get_var", [](StochasticBatchNormalization_fp32 &l) -> Tensor & { return l.running_var(); }, py::return_value_policy::reference_internal);

    // convolution lowering (python/binarybrain/src/core_main.cpp of the reference registers the same names)
    py::class_<Sequential, Model, std::shared_ptr<Sequential>>(m, "Sequential")
        .def_static("create", &Sequential::Create)
        .def("add", &Sequential::Add)
        .def("get_size", &Sequential::GetSize)
        .def("get", &Sequential::Get);
#define BB200_DEF_CONV(FT)                                                                                                                      \
    py::class_<ConvolutionIm2Col_##FT, Model, std::shared_ptr<ConvolutionIm2Col_##FT>>(m, "ConvolutionIm2Col_" #FT)                              \
        .def_static("create", [](index_t fh, index_t fw, index_t ys, index_t xs, std::string padding, std::string border) {                     \
            return ConvolutionIm2Col_##FT::Create(fh, fw, ys, xs, padding, border); },                                                          \
            py::arg("filter_h_size"), py::arg("filter_w_size"), py::arg("y_stride") = 1, py::arg("x_stride") = 1,                               \
            py::arg("padding") = "valid", py::arg("border_mode") = "reflect_101");                                                              \
    py::class_<ConvolutionCol2Im_##FT, Model, std::shared_ptr<ConvolutionCol2Im_##FT>>(m, "ConvolutionCol2Im_" #FT)                              \
        .def_static("create", [](index_t h, index_t w) { return ConvolutionCol2Im_##FT::Create(h, w); }, py::arg("h_size"), py::arg("w_size")); \
    py::class_<MaxPooling_##FT, Model, std::shared_ptr<MaxPooling_##FT>>(m, "MaxPooling_" #FT)                                                   \
        .def_static("create", [](index_t fh, index_t fw) { return MaxPooling_##FT::Create(fh, fw); }, py::arg("filter_h_size"),                 \
                    py::arg("filter_w_size"));                                                                                                  \
    py::class_<Convolution2d_##FT, Model, std::shared_ptr<Convolution2d_##FT>>(m, "Convolution2d_" #FT)                                          \
        .def_static("create", [](std::shared_ptr<Model> layer, index_t fh, index_t fw, index_t ys, index_t xs, std::string padding,             \
                                 std::string border) { return Convolution2d_##FT::Create(layer, fh, fw, ys, xs, padding, border); },            \
            py::arg("layer"), py::arg("filter_h_size"), py::arg("filter_w_size"), py::arg("y_stride") = 1, py::arg("x_stride") = 1,             \
            py::arg("padding") = "valid", py::arg("border_mode") = "reflect_101")                                                               \
        .def("get_layer", &Convolution2d_##FT::GetLayer);
    BB200_DEF_CONV(fp32_fp32)
    BB200_DEF_CONV(bit_fp32)
#undef BB200_DEF_CONV

    py::class_<OptimizerAdam_fp32, std::shared_ptr<OptimizerAdam_fp32>>(m, "OptimizerAdam_fp32")
        .def_static("create", &OptimizerAdam_fp32::Create, py::arg("learning_rate") = 0.001f, py::arg("beta1") = 0.9f, py::arg("beta2") = 0.999f)
        .def("set_learning_rate", &OptimizerAdam_fp32::SetLearningRate)
        .def("add_variables", &OptimizerAdam_fp32::AddVariables)
        .def("set_variables", [](OptimizerAdam_fp32 &o, std::shared_ptr<Tensor> p, std::shared_ptr<Tensor> g) { o.AddVariables(p, g); })
        .def("step", &OptimizerAdam_fp32::Step)
        .def("zero_grad", &OptimizerAdam_fp32::ZeroGrad)
        .def("update", &OptimizerAdam_fp32::Update);
}
