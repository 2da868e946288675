// Registration tables of the B200 `tensor` plugin.  Group names, URIs, arities and signature
// strings of the first 37 entries are those of the reference (modules/tensor/operators.cpp:
// 196-583) - they are the surface `.cml` programs resolve against and must not drift; the table
// is checked entry by entry against the compiled reference in the tests.
#include "tensor_ops.h"

#include "camel/core/type/composite/array.h"
#include "device_tensor.h"
#include "type.h"

#include <optional>

using namespace camel::core::type;
using camel::tensor::TensorType;

namespace {

Type *tensorOf(Type *dtype = nullptr) { return TensorType::Dynamic(dtype ? dtype : Type::Float32()); }
bool isTensor(Type *t) { return t && t->code() == TensorType::typeCode(); }
bool isArray(Type *t) { return t && t->code() == TypeCode::Array; }
bool isScalar(Type *t) { return t && camel::tensor::isSupportedTensorScalar(t->code()); }
bool isInt(Type *t) { return t && (t->code() == TypeCode::Int32 || t->code() == TypeCode::Int64); }

using Check = std::optional<Type *> (*)(const type_vec_t &with, const type_vec_t &norm);

// One URI of a group: arity of the `with` and `norm` lists (-1: variadic), signature, check.
struct Entry {
    const char *uri;
    int withCount, normCount;
    const char *signature;
    Check check;
};

resolver_ptr_t makeResolver(const Entry &e) {
    std::vector<bool> wf(e.withCount > 0 ? e.withCount : 0, false), nf(e.normCount > 0 ? e.normCount : 0, false);
    Check check = e.check;
    return DynamicFuncTypeResolver::create(
        {{e.withCount, wf}, {e.normCount, nf}}, std::string(e.signature),
        [check](const type_vec_t &with, const type_vec_t &norm, const ModifierSet &) { return check(with, norm); });
}

oper_group_ptr_t group(const char *name, std::initializer_list<Entry> entries) {
    std::vector<std::pair<std::string, resolver_ptr_t>> resolvers;
    for (const Entry &e : entries)
        resolvers.emplace_back(e.uri, makeResolver(e));
    return OperatorGroup::create(name, resolvers);
}

std::optional<Type *> some(Type *t) { return std::optional<Type *>{t}; }

// -- checks (what each reference resolver accepts) --
std::optional<Type *> binaryCheck(const type_vec_t &, const type_vec_t &n) {
    if (n.size() != 2)
        return std::nullopt;
    bool l = isTensor(n[0]), r = isTensor(n[1]);
    return ((l && r) || (l && isScalar(n[1])) || (r && isScalar(n[0]))) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> powCheck(const type_vec_t &, const type_vec_t &n) {
    return isTensor(n[0]) && (isTensor(n[1]) || isScalar(n[1])) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> compareCheck(const type_vec_t &, const type_vec_t &n) {
    if (n.size() != 2)
        return std::nullopt;
    bool l = isTensor(n[0]), r = isTensor(n[1]);
    bool ok = (l && r) || (l && isScalar(n[1])) || (r && isScalar(n[0])) || (isArray(n[0]) && isScalar(n[1])) ||
              (isScalar(n[0]) && isArray(n[1]));
    return ok ? some(tensorOf(Type::Bool())) : std::nullopt;
}
std::optional<Type *> idxCheck(const type_vec_t &, const type_vec_t &n) {
    return isTensor(n[0]) && n[1]->code() == TypeCode::Int64 ? some(Type::Float64()) : std::nullopt;
}
std::optional<Type *> idx2dCheck(const type_vec_t &, const type_vec_t &n) {
    return isTensor(n[0]) && n[1]->code() == TypeCode::Int64 && n[2]->code() == TypeCode::Int64
               ? some(Type::Float64()) : std::nullopt;
}
std::optional<Type *> shapeCtorCheck(const type_vec_t &, const type_vec_t &n) {
    return n.size() == 1 && isArray(n[0]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> fullCheck(const type_vec_t &, const type_vec_t &n) {
    return isArray(n[0]) && isScalar(n[1]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> randomCheck(const type_vec_t &, const type_vec_t &n) {
    return isArray(n[0]) && isScalar(n[1]) && isScalar(n[2]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> rangeCheck(const type_vec_t &, const type_vec_t &n) {
    if (n.empty() || n.size() > 3)
        return std::nullopt;
    for (Type *t : n)
        if (!isInt(t))
            return std::nullopt;
    return some(tensorOf(Type::Int64()));
}
std::optional<Type *> eyeCheck(const type_vec_t &, const type_vec_t &n) {
    return isInt(n[0]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> shapeCheck(const type_vec_t &, const type_vec_t &n) {
    static ArrayType *ints = ArrayType::create(Type::Int64());
    return isTensor(n[0]) ? some(ints) : std::nullopt;
}
std::optional<Type *> sumCheck(const type_vec_t &, const type_vec_t &n) {
    return isTensor(n[0]) ? some(Type::Float64()) : std::nullopt;
}
std::optional<Type *> axisCheck(const type_vec_t &, const type_vec_t &n) {
    return n.size() == 2 && isTensor(n[0]) && isInt(n[1]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> argmaxCheck(const type_vec_t &, const type_vec_t &n) {
    return n.size() == 2 && isTensor(n[0]) && isInt(n[1]) ? some(tensorOf(Type::Int64())) : std::nullopt;
}
std::optional<Type *> unaryCheck(const type_vec_t &, const type_vec_t &n) {
    return isTensor(n[0]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> concatCheck(const type_vec_t &, const type_vec_t &n) {
    if (n.size() != 3 || n[2]->code() != TypeCode::Int64)
        return std::nullopt;
    bool l = isTensor(n[0]) || isArray(n[0]), r = isTensor(n[1]) || isArray(n[1]);
    return l && r ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> reshapeCheck(const type_vec_t &, const type_vec_t &n) {
    return (isTensor(n[0]) || isArray(n[0])) && isArray(n[1]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> showCheck(const type_vec_t &, const type_vec_t &n) {
    return (isTensor(n[0]) || isArray(n[0])) ? some(Type::Void()) : std::nullopt;
}
// -- added operators --
std::optional<Type *> denseCheck(const type_vec_t &w, const type_vec_t &n) {
    return w.size() == 2 && isTensor(w[0]) && isTensor(w[1]) && n.size() == 1 && isTensor(n[0]) ? some(tensorOf())
                                                                                               : std::nullopt;
}
std::optional<Type *> convCheck(const type_vec_t &w, const type_vec_t &n) {
    return w.size() == 4 && isTensor(w[0]) && isTensor(w[1]) && isInt(w[2]) && isInt(w[3]) && n.size() == 1 &&
                   isTensor(n[0])
               ? some(tensorOf())
               : std::nullopt;
}
std::optional<Type *> matmulTnCheck(const type_vec_t &, const type_vec_t &n) {
    return n.size() == 2 && isTensor(n[0]) && isTensor(n[1]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> scaledSubCheck(const type_vec_t &, const type_vec_t &n) {
    return n.size() == 3 && isTensor(n[0]) && isTensor(n[1]) && isScalar(n[2]) ? some(tensorOf()) : std::nullopt;
}
std::optional<Type *> poolCheck(const type_vec_t &, const type_vec_t &n) {
    return n.size() == 2 && isTensor(n[0]) && isInt(n[1]) ? some(tensorOf()) : std::nullopt;
}

constexpr const char *kBinarySig  = "(lhs: Tensor | number, rhs: Tensor | number) => Tensor";
constexpr const char *kCompareSig = "(lhs: Tensor | number, rhs: Tensor | number) => Tensor<bool>";
constexpr const char *kPowSig     = "(base: Tensor, exponent: Tensor | number) => Tensor";
constexpr const char *kShapeSig   = "(shape: int[]) => Tensor";
constexpr const char *kAxisSig    = "(t: Tensor, axis: int) => Tensor";
constexpr const char *kUnarySig   = "(t: Tensor) => Tensor";

oper_group_ptr_t matmulGroup(const char *name) {
    return OperatorGroup::create(
        name, {{"tensor:matmul",
                StaticFuncTypeResolver::create({}, {{tensorOf(), false}, {tensorOf(), false}}, tensorOf())}});
}

} // namespace

std::unordered_map<std::string, operator_t> getTensorOpsMap() {
    return {
        {"add", __tensor_add__}, {"subtract", __tensor_subtract__}, {"multiply", __tensor_multiply__},
        {"divide", __tensor_divide__}, {"pow", __tensor_pow__}, {"matmul", __tensor_matmul__},
        {"idx", __tensor_idx__}, {"idx2d", __tensor_idx2d__}, {"lt", __tensor_lt__}, {"le", __tensor_le__},
        {"gt", __tensor_gt__}, {"ge", __tensor_ge__}, {"eq", __tensor_eq__}, {"empty", __tensor_empty__},
        {"zeros", __tensor_zeros__}, {"ones", __tensor_ones__}, {"full", __tensor_full__},
        {"random", __tensor_random__}, {"range", __tensor_range__}, {"eye", __tensor_eye__},
        {"shape", __tensor_shape__}, {"sum", __tensor_sum__}, {"sum_axis", __tensor_sum_axis__},
        {"max_axis", __tensor_max_axis__}, {"argmax_axis", __tensor_argmax_axis__}, {"exp", __tensor_exp__},
        {"log", __tensor_log__}, {"transpose", __tensor_transpose__}, {"concat", __tensor_concat__},
        {"reshape", __tensor_reshape__}, {"show", __tensor_show__},
        // added
        {"relu", __tensor_relu__}, {"softmax", __tensor_softmax__}, {"dense", __tensor_dense__},
        {"dense_relu", __tensor_dense_relu__}, {"dense_softmax", __tensor_dense_softmax__},
        {"conv2d", __tensor_conv2d__}, {"conv2d_relu", __tensor_conv2d_relu__},
        {"maxpool2d", __tensor_maxpool2d__}, {"flatten", __tensor_flatten__},
        {"matmul_tn", __tensor_matmul_tn__}, {"scaled_sub", __tensor_scaled_sub__},
        {"conv2d_relu_maxpool2", __tensor_conv2d_relu_maxpool2__},
    };
}

const std::vector<oper_group_ptr_t> &getTensorOperatorGroups() {
    static const std::vector<oper_group_ptr_t> groups = {
        group("__add__", {{"tensor:add", 0, 2, kBinarySig, binaryCheck}}),
        group("__sub__", {{"tensor:subtract", 0, 2, kBinarySig, binaryCheck}}),
        group("__mul__", {{"tensor:multiply", 0, 2, kBinarySig, binaryCheck}}),
        group("__div__", {{"tensor:divide", 0, 2, kBinarySig, binaryCheck}}),
        group("__pow__", {{"tensor:pow", 0, 2, kPowSig, powCheck}}),
        matmulGroup("__mat__"),
        group("__idx__", {{"tensor:idx", 0, 2, "(t: Tensor, i: int) => float", idxCheck},
                          {"tensor:idx2d", 0, 3, "(t: Tensor, i: int, j: int) => float", idx2dCheck}}),
        group("__lt__", {{"tensor:lt", 0, 2, kCompareSig, compareCheck}}),
        group("__le__", {{"tensor:le", 0, 2, kCompareSig, compareCheck}}),
        group("__gt__", {{"tensor:gt", 0, 2, kCompareSig, compareCheck}}),
        group("__ge__", {{"tensor:ge", 0, 2, kCompareSig, compareCheck}}),
        group("__eq__", {{"tensor:eq", 0, 2, kCompareSig, compareCheck}}),
        group("empty", {{"tensor:empty", 0, 1, kShapeSig, shapeCtorCheck}}),
        group("zeros", {{"tensor:zeros", 0, 1, kShapeSig, shapeCtorCheck}}),
        group("ones", {{"tensor:ones", 0, 1, kShapeSig, shapeCtorCheck}}),
        group("full", {{"tensor:full", 0, 2, "(shape: int[], value: number) => Tensor", fullCheck}}),
        group("random", {{"tensor:random", 0, 3, "(shape: int[], low: number, high: number) => Tensor", randomCheck}}),
        group("range", {{"tensor:range", 0, -1, "(start: int, stop?: int, step?: int) => Tensor", rangeCheck}}),
        group("eye", {{"tensor:eye", 0, 1, "(n: int) => Tensor", eyeCheck}}),
        group("shape", {{"tensor:shape", 0, 1, "(t: Tensor) => int[]", shapeCheck}}),
        group("sum", {{"tensor:sum", 0, 1, "(t: Tensor) => float", sumCheck},
                      {"tensor:sum_axis", 0, 2, kAxisSig, axisCheck}}),
        group("max", {{"tensor:max_axis", 0, 2, kAxisSig, axisCheck}}),
        group("argmax", {{"tensor:argmax_axis", 0, 2, kAxisSig, argmaxCheck}}),
        group("exp", {{"tensor:exp", 0, 1, kUnarySig, unaryCheck}}),
        group("log", {{"tensor:log", 0, 1, kUnarySig, unaryCheck}}),
        group("transpose", {{"tensor:transpose", 0, 1, kUnarySig, unaryCheck}}),
        group("concat", {{"tensor:concat", 0, 3, "(a: Tensor | number[], b: Tensor | number[], axis: int) => Tensor",
                          concatCheck}}),
        group("reshape", {{"tensor:reshape", 0, 2, "(t: Tensor | number[], shape: int[]) => Tensor", reshapeCheck}}),
        group("show", {{"tensor:show", 0, 1, "(t: Tensor | number[]) => void", showCheck}}),
        group("add", {{"tensor:add", 0, 2, kBinarySig, binaryCheck}}),
        group("subtract", {{"tensor:subtract", 0, 2, kBinarySig, binaryCheck}}),
        group("multiply", {{"tensor:multiply", 0, 2, kBinarySig, binaryCheck}}),
        group("divide", {{"tensor:divide", 0, 2, kBinarySig, binaryCheck}}),
        group("pow", {{"tensor:pow", 0, 2, kPowSig, powCheck}}),
        matmulGroup("matmul"),
        // ---- added by this plugin ----
        group("relu", {{"tensor:relu", 0, 1, kUnarySig, unaryCheck}}),
        group("softmax", {{"tensor:softmax", 0, 1, kUnarySig, unaryCheck}}),
        group("dense", {{"tensor:dense", 2, 1, "<w: Tensor, b: Tensor>(x: Tensor) => Tensor", denseCheck}}),
        group("dense_relu", {{"tensor:dense_relu", 2, 1, "<w: Tensor, b: Tensor>(x: Tensor) => Tensor", denseCheck}}),
        group("dense_softmax",
              {{"tensor:dense_softmax", 2, 1, "<w: Tensor, b: Tensor>(x: Tensor) => Tensor", denseCheck}}),
        group("conv2d", {{"tensor:conv2d", 4, 1,
                          "<w: Tensor, b: Tensor, stride: int, pad: int>(x: Tensor) => Tensor", convCheck}}),
        group("conv2d_relu", {{"tensor:conv2d_relu", 4, 1,
                               "<w: Tensor, b: Tensor, stride: int, pad: int>(x: Tensor) => Tensor", convCheck}}),
        group("maxpool2d", {{"tensor:maxpool2d", 0, 2, "(t: Tensor, window: int) => Tensor", poolCheck}}),
        group("flatten", {{"tensor:flatten", 0, 1, kUnarySig, unaryCheck}}),
        group("conv2d_relu_maxpool2",
              {{"tensor:conv2d_relu_maxpool2", 4, 1,
                "<w: Tensor, b: Tensor, stride: int, pad: int>(x: Tensor) => Tensor", convCheck}}),
        group("matmul_tn", {{"tensor:matmul_tn", 0, 2, "(a: Tensor, b: Tensor) => Tensor", matmulTnCheck}}),
        group("scaled_sub",
              {{"tensor:scaled_sub", 0, 3, "(w: Tensor, g: Tensor, lr: number) => Tensor", scaledSubCheck}}),
    };
    return groups;
}
