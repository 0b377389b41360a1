// The C++ usage shown in the integration notes, as a translation unit of its own: the header-only host classes over the C ABI.
// Compiled and linked by tests/test_host_headers_compile.py; it is not run there (it needs a GPU).
#include <vector>

#include "bb/ConvModels.h"

using namespace bb;

int main()
{
    const index_t batch = 64;
    auto net = Sequential::Create();
    std::vector<std::shared_ptr<DifferentiableLutN<6, float>>> layers;
    for (index_t n : {1024, 420, 70}) {
        layers.push_back(DifferentiableLutN<6, float>::Create(n));
        net->Add(layers.back());
    }
    net->SetInputShape({784});
    auto opt = OptimizerAdam<float>::Create();
    for (auto &l : layers) opt->AddVariables(l->GetParameters(), l->GetGradients());

    std::vector<float> images((std::size_t)batch * 784, 0.5f), grad((std::size_t)batch * 70, 0.01f);
    FrameBuffer x(batch, {784}, BB_TYPE_FP32), dy(batch, {70}, BB_TYPE_FP32);
    x.SetFrameMajor(images.data());
    dy.SetFrameMajor(grad.data());
    FrameBuffer y = net->Forward(x, true);
    FrameBuffer dx = net->Backward(dy);
    opt->Update();
    std::vector<float> out((std::size_t)batch * 70);
    y.GetFrameMajor(out.data());
    return dx.Empty() ? 1 : 0;
}
