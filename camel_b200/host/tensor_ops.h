// Entry points of the B200 `tensor` plugin: the 31 operators of the reference module under
// their reference names (modules/tensor/operators.h:31-63) plus the operators this plugin adds.
#pragma once

#include "camel/core/operator.h"

#include <string>
#include <unordered_map>
#include <vector>

namespace ctx = camel::core::context;

#define CAMEL_TENSOR_DECLARE(name) slot_t name(ArgsView &with, ArgsView &norm, ctx::Context &ctx);
CAMEL_TENSOR_DECLARE(__tensor_add__)
CAMEL_TENSOR_DECLARE(__tensor_subtract__)
CAMEL_TENSOR_DECLARE(__tensor_multiply__)
CAMEL_TENSOR_DECLARE(__tensor_divide__)
CAMEL_TENSOR_DECLARE(__tensor_pow__)
CAMEL_TENSOR_DECLARE(__tensor_matmul__)
CAMEL_TENSOR_DECLARE(__tensor_idx__)
CAMEL_TENSOR_DECLARE(__tensor_idx2d__)
CAMEL_TENSOR_DECLARE(__tensor_lt__)
CAMEL_TENSOR_DECLARE(__tensor_le__)
CAMEL_TENSOR_DECLARE(__tensor_gt__)
CAMEL_TENSOR_DECLARE(__tensor_ge__)
CAMEL_TENSOR_DECLARE(__tensor_eq__)
CAMEL_TENSOR_DECLARE(__tensor_empty__)
CAMEL_TENSOR_DECLARE(__tensor_zeros__)
CAMEL_TENSOR_DECLARE(__tensor_ones__)
CAMEL_TENSOR_DECLARE(__tensor_full__)
CAMEL_TENSOR_DECLARE(__tensor_random__)
CAMEL_TENSOR_DECLARE(__tensor_range__)
CAMEL_TENSOR_DECLARE(__tensor_eye__)
CAMEL_TENSOR_DECLARE(__tensor_shape__)
CAMEL_TENSOR_DECLARE(__tensor_sum__)
CAMEL_TENSOR_DECLARE(__tensor_sum_axis__)
CAMEL_TENSOR_DECLARE(__tensor_max_axis__)
CAMEL_TENSOR_DECLARE(__tensor_argmax_axis__)
CAMEL_TENSOR_DECLARE(__tensor_exp__)
CAMEL_TENSOR_DECLARE(__tensor_log__)
CAMEL_TENSOR_DECLARE(__tensor_transpose__)
CAMEL_TENSOR_DECLARE(__tensor_concat__)
CAMEL_TENSOR_DECLARE(__tensor_reshape__)
CAMEL_TENSOR_DECLARE(__tensor_show__)
// added: fused forms of compositions the reference writes in .cml (svm.cml:31, mnist.cml:13-25,
// lr.cml:19-21) and the convolution / pooling operators it lacks
CAMEL_TENSOR_DECLARE(__tensor_relu__)
CAMEL_TENSOR_DECLARE(__tensor_softmax__)
CAMEL_TENSOR_DECLARE(__tensor_dense__)
CAMEL_TENSOR_DECLARE(__tensor_dense_relu__)
CAMEL_TENSOR_DECLARE(__tensor_dense_softmax__)
CAMEL_TENSOR_DECLARE(__tensor_conv2d__)
CAMEL_TENSOR_DECLARE(__tensor_conv2d_relu__)
CAMEL_TENSOR_DECLARE(__tensor_maxpool2d__)
CAMEL_TENSOR_DECLARE(__tensor_flatten__)
CAMEL_TENSOR_DECLARE(__tensor_conv2d_relu_maxpool2__)
CAMEL_TENSOR_DECLARE(__tensor_matmul_tn__)
CAMEL_TENSOR_DECLARE(__tensor_scaled_sub__)
#undef CAMEL_TENSOR_DECLARE

// URI suffix -> body; what the module's executor dispatches on (modules/tensor/executor.cpp:36-61).
std::unordered_map<std::string, operator_t> getTensorOpsMap();
// Operator groups exported by the module (modules/tensor/module.cpp:30-38).
const std::vector<oper_group_ptr_t> &getTensorOperatorGroups();
