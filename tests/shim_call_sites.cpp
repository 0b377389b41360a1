// Translation unit for tests/test_shim_compiles.py: BinaryBrain's own layer classes, compiled with BB_WITH_CUDA against
// BinaryBrain's include/bbcu/bbcu.h followed by include/bbcu_b200_shim.h.  Explicit instantiation compiles every member
// function, i.e. every call site of the bbcu_* operators (bb::BinaryLutN is used instead: one of its never-called members does
// not compile in the reference, include/bb/BinaryLutN.h:229).
#define BB_WITH_CUDA
#include "bbcu/bbcu.h"
#include "bbcu_b200_shim.h"
#include "bb/DifferentiableLutN.h"
#include "bb/StochasticLutN.h"
#include "bb/BinaryLutN.h"
#include "bb/StochasticBatchNormalization.h"
#include "bb/OptimizerAdam.h"
#include "bb/Convolution2d.h"
#include "bb/MaxPooling.h"
#include "bb/LossMeanSquaredError.h"
#include "bb/BinaryToReal.h"
template class bb::DifferentiableLutN<6, float, float>;
template class bb::DifferentiableLutN<6, bb::Bit, float>;
template class bb::StochasticLutN<6, float, float>;
template class bb::StochasticLutN<6, bb::Bit, float>;
void use_binary_lut() { auto l = bb::BinaryLutN<6, bb::Bit, float>::Create(16); bb::FrameBuffer x(32, {16}, BB_TYPE_BIT); l->SetInputShape(x.GetShape()); l->Forward(x, false); }
template class bb::StochasticBatchNormalization<float>;
template class bb::OptimizerAdam<float>;
template class bb::ConvolutionIm2Col<float, float>;
template class bb::ConvolutionIm2Col<bb::Bit, float>;
template class bb::ConvolutionCol2Im<float, float>;
template class bb::ConvolutionCol2Im<bb::Bit, float>;
template class bb::MaxPooling<float, float>;
template class bb::MaxPooling<bb::Bit, float>;
template class bb::LossMeanSquaredError<float>;
template class bb::BinaryToReal<float, float>;
template class bb::BinaryToReal<bb::Bit, float>;
