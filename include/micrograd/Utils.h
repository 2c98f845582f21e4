#pragma once
// Debug helpers, same two entry points as the reference's
// include/micrograd/Utils.h:5-6.
#include <memory>
#include <string>

#include "Tensor.h"

// Graphviz dump of the graph that produced `tensor`.
std::string to_dot(const std::shared_ptr<Tensor> &tensor);
// "<op> <scalar with two decimals>", the label of tensor-scalar ops.
std::string format_scalar(const std::string &op, double scalar);
