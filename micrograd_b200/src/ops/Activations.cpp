// relu, sigmoid, tanh (reference: src/ops/Activations.cpp) and exp (addition).
// relu's backward masks on the forward input, sigmoid/tanh/exp use the forward
// output, as the reference's closures do.
#include "mg_cuda.h"
#include "micrograd/Tensor.h"

std::shared_ptr<Tensor> Tensor::relu() { return unary_op(MG_RELU, "relu", 0.0); }

std::shared_ptr<Tensor> Tensor::sigmoid() { return unary_op(MG_SIGMOID, "sigmoid", 0.0); }

std::shared_ptr<Tensor> Tensor::tanh() { return unary_op(MG_TANH, "tanh", 0.0); }

std::shared_ptr<Tensor> Tensor::exp() { return unary_op(MG_EXP, "exp", 0.0); }
