// Node classes of the fused-layer path: shape rules on the host, compute through the C ABI.
#include <algorithm>
#include <sstream>

#include "dynet_shim.h"

namespace dynet_b200 {

#define ARG_CHECK(cond, msg)                       \
  do {                                             \
    if (!(cond)) {                                 \
      std::ostringstream oss__;                    \
      oss__ << msg;                                \
      throw std::invalid_argument(oss__.str());    \
    }                                              \
  } while (0)

void throw_status(const Device_GPU& dev, int status) {
  if (status == DYB200_OK) return;
  std::string what = dyb200_last_error(dev.ctx);
  switch (status) {
    case DYB200_EINVAL: throw std::invalid_argument(what);
    case DYB200_ENOMEM: throw out_of_memory(what);
    case DYB200_ECUDA: throw cuda_exception(what);
    default: throw std::runtime_error(what);
  }
}

dyb200_tensor to_c(const Tensor& t) {
  dyb200_tensor c;
  c.v = t.v;
  for (unsigned k = 0; k < 7; ++k) c.d[k] = k < t.d.nd ? t.d.d[k] : 1;
  c.nd = t.d.nd;
  c.bd = t.d.bd;
  return c;
}

void call_fwd(fwd_fn f, const Device_GPU& dev, const std::vector<const Tensor*>& xs, Tensor& fx, const void* attrs, void* aux) {
  std::vector<dyb200_tensor> cx(xs.size());
  for (size_t k = 0; k < xs.size(); ++k) cx[k] = to_c(*xs[k]);
  dyb200_tensor cf = to_c(fx);
  throw_status(dev, f(xs.empty() ? nullptr : cx.data(), (int)xs.size(), &cf, attrs, aux, dev.ctx));
}
void call_bwd(bwd_fn f, const Device_GPU& dev, const std::vector<const Tensor*>& xs, const Tensor& fx, const Tensor& dEdf,
              unsigned i, Tensor& dEdxi, const void* attrs, void* aux) {
  std::vector<dyb200_tensor> cx(xs.size());
  for (size_t k = 0; k < xs.size(); ++k) cx[k] = to_c(*xs[k]);
  dyb200_tensor cf = to_c(fx), cd = to_c(dEdf), co = to_c(dEdxi);
  throw_status(dev, f(xs.empty() ? nullptr : cx.data(), (int)xs.size(), &cf, &cd, i, &co, attrs, aux, dev.ctx));
}

#define SIMPLE_NODE(CLS, CNAME, ...)                                                                             \
  void CLS::forward_dev_impl(const Device_GPU& dev, const std::vector<const Tensor*>& xs, Tensor& fx) const {    \
    __VA_ARGS__;                                                                                                 \
    call_fwd(dyb200_##CNAME##_fwd, dev, xs, fx, attrs_ptr, aux_mem);                                             \
  }                                                                                                              \
  void CLS::backward_dev_impl(const Device_GPU& dev, const std::vector<const Tensor*>& xs, const Tensor& fx,    \
                              const Tensor& dEdf, unsigned i, Tensor& dEdxi) const {                             \
    __VA_ARGS__;                                                                                                 \
    call_bwd(dyb200_##CNAME##_bwd, dev, xs, fx, dEdf, i, dEdxi, attrs_ptr, aux_mem);                             \
  }
#define NO_ATTRS const void* attrs_ptr = nullptr

// ---- unary: result has the shape of the argument ----
#define UNARY_DIM(CLS)                                                   \
  Dim CLS::dim_forward(const std::vector<Dim>& xs) const {               \
    ARG_CHECK(xs.size() == 1, "Failed input count check in " #CLS);      \
    return xs[0];                                                        \
  }
UNARY_DIM(Tanh) SIMPLE_NODE(Tanh, tanh, NO_ATTRS)
UNARY_DIM(LogisticSigmoid) SIMPLE_NODE(LogisticSigmoid, logistic, NO_ATTRS)
UNARY_DIM(Rectify) SIMPLE_NODE(Rectify, rectify, NO_ATTRS)
UNARY_DIM(ExponentialLinearUnit)
SIMPLE_NODE(ExponentialLinearUnit, elu, dyb200_elu_attrs at = {alpha, lambda}; const void* attrs_ptr = &at)

// ---- cwise binary: per-dimension and batch broadcasting (dynet/nodes-arith-cwise.cc:20-34, :168-182, :319-333) ----
static Dim broadcast_dim(const std::vector<Dim>& xs, const char* name, bool right_only) {
  ARG_CHECK(xs.size() == 2, "Failed input count check in " << name);
  Dim r;
  unsigned lo = std::min(xs[0].nd, xs[1].nd), hi = std::max(xs[0].nd, xs[1].nd);
  for (unsigned i = 0; i < lo; ++i) {
    bool ok = right_only ? (xs[0].d[i] == xs[1].d[i] || xs[1].d[i] == 1)
                         : (xs[0].d[i] == xs[1].d[i] || std::min(xs[0].d[i], xs[1].d[i]) == 1);
    ARG_CHECK(ok, name << ": For each dimension, the dim size needs to match or equal 1.");
  }
  ARG_CHECK(xs[0].bd == xs[1].bd || (right_only ? xs[1].bd == 1 : std::min(xs[0].bd, xs[1].bd) == 1),
            name << ": batch size must match or equal 1");
  for (unsigned i = 0; i < hi; ++i)
    r.d[r.nd++] = i < lo ? std::max(xs[0].d[i], xs[1].d[i]) : (i < xs[0].nd ? xs[0].d[i] : xs[1].d[i]);
  r.bd = std::max(xs[0].bd, xs[1].bd);
  return r;
}
Dim CwiseMultiply::dim_forward(const std::vector<Dim>& xs) const { return broadcast_dim(xs, "CwiseMultiply", false); }
Dim CwiseSum::dim_forward(const std::vector<Dim>& xs) const { return broadcast_dim(xs, "CwiseSum", false); }
Dim CwiseQuotient::dim_forward(const std::vector<Dim>& xs) const { return broadcast_dim(xs, "CwiseQuotient", true); }
SIMPLE_NODE(CwiseMultiply, cmult, NO_ATTRS)
SIMPLE_NODE(CwiseSum, csum, NO_ATTRS)
SIMPLE_NODE(CwiseQuotient, cdiv, NO_ATTRS)

// ---- softmax family ----
Dim Softmax::dim_forward(const std::vector<Dim>& xs) const {     // dynet/nodes-softmaxes.cc:21-26
  ARG_CHECK(xs.size() == 1, "Failed input count check in Softmax");
  ARG_CHECK(xs[0].nd <= 2, "Bad input dimensions in Softmax, must be 2 or fewer");
  ARG_CHECK(dimension < xs[0].nd, "reduction dimension must be < number of dimensions, was " << dimension);
  return xs[0];
}
SIMPLE_NODE(Softmax, softmax, dyb200_dim_attrs at = {dimension}; const void* attrs_ptr = &at)
Dim LogSoftmax::dim_forward(const std::vector<Dim>& xs) const {  // dynet/nodes-softmaxes.cc:144-148
  ARG_CHECK(xs.size() == 1, "Failed input count check in LogSoftmax");
  ARG_CHECK(xs[0].nd <= 2, "Bad input dimensions in LogSoftmax, must be 2 or fewer");
  return xs[0];
}
SIMPLE_NODE(LogSoftmax, log_softmax, NO_ATTRS)
Dim LogSumExp::dim_forward(const std::vector<Dim>& xs) const {   // dynet/nodes-logsumexp.cc:25-33
  ARG_CHECK(!xs.empty(), "LogSumExp needs at least one argument");
  Dim d = xs[0];
  for (size_t i = 1; i < xs.size(); ++i) {
    ARG_CHECK(d.batch_size() == xs[i].batch_size(), "Mismatched input dimensions in LogSumExp");
    d.bd = std::max(xs[i].bd, d.bd);
  }
  return d;
}
SIMPLE_NODE(LogSumExp, logsumexp, NO_ATTRS)
Dim LogSumExpDimension::dim_forward(const std::vector<Dim>& xs) const {  // dynet/nodes-logsumexp.cc:112-121
  ARG_CHECK(xs.size() == 1, "LogSumExpDimension takes only one argument");
  ARG_CHECK(xs[0].nd <= 2, "LogSumExpDimension, expects 2 or fewer dimensions");
  ARG_CHECK(xs[0].nd > dimension, "LogSumExpDimension, expects its dimension argument (" << dimension
                                      << ") to be smaller than the number of elements in the input");
  Dim d;
  for (unsigned k = 0; k < xs[0].nd; ++k) if (k != dimension) d.d[d.nd++] = xs[0].d[k];
  if (d.nd == 0) d.d[d.nd++] = 1;   // Dim::delete_dim of the only dimension leaves a size-1 vector (dynet/dim.h:212-228)
  d.bd = xs[0].bd;
  return d;
}
SIMPLE_NODE(LogSumExpDimension, logsumexp_dim, dyb200_dim_attrs at = {dimension}; const void* attrs_ptr = &at)

Dim PickNegLogSoftmax::dim_forward(const std::vector<Dim>& xs) const {   // dynet/nodes-pickneglogsoftmax.cc:32-44
  ARG_CHECK(xs.size() == 1, "Failed input count check in PickNegLogSoftmax");
  ARG_CHECK(xs[0].cols() == 1 && xs[0].nd <= 2, "Bad input dimensions in PickNegLogSoftmax");
  ARG_CHECK(pvals == nullptr || xs[0].bd == pvals->size(),
            "The number of IDs passed to PickNegLogSoftmax (" << (pvals ? pvals->size() : 0)
                << "), did not match the number of mini-batch elements in the expression under consideration (" << xs[0].bd
                << "). These numbers must match.");
  return Dim({1}, xs[0].bd);
}
SIMPLE_NODE(PickNegLogSoftmax, pickneglogsoftmax,
            dyb200_pick_attrs at = {pvals ? pvals->data() : nullptr, pvals ? (uint32_t)pvals->size() : (uint32_t)xs[0]->d.bd};
            const void* attrs_ptr = &at)

// ---- normalisation ----
Dim WeightNormalization::dim_forward(const std::vector<Dim>& xs) const {  // dynet/nodes-normalization.cc:20-24
  ARG_CHECK(xs.size() == 2, "Failed input count check in WeightNormalization");
  ARG_CHECK(1 == xs[1].size(), " Size of gain parameter in WeightNormalization should be 1, received " << xs[1].size());
  return xs[0];
}
SIMPLE_NODE(WeightNormalization, weight_norm, NO_ATTRS)

static Dim moment_dim(const Dim& x, const std::vector<unsigned>& dims, bool include_batch, const char* name) {
  ARG_CHECK(x.nd <= 3, name << " implemented up to tensors of order 3 (with minibatch) for now");
  ARG_CHECK(dims.size() <= 2, "Number of dimensions to reduce (excluding batch dimension) implemented up to 2 in " << name);
  if (dims.empty()) ARG_CHECK(include_batch, "At least one dimension has to be reduced (including batch dimension) in " << name);
  for (unsigned d : dims) ARG_CHECK(d < x.nd, "dimension " << d << " is out of bounds of tensor of order " << x.nd << " in " << name);
  Dim r;
  for (unsigned k = 0; k < x.nd; ++k)
    if (std::find(dims.begin(), dims.end(), k) == dims.end()) r.d[r.nd++] = x.d[k];
  if (r.nd == 0) r.d[r.nd++] = 1;   // Dim::delete_dims keeps a size-1 vector
  r.bd = include_batch ? 1 : x.bd;
  return r;
}
static dyb200_moment_attrs moment_attrs(const std::vector<unsigned>& dims, unsigned order, bool ib, unsigned on) {
  dyb200_moment_attrs a = {{0, 0}, (uint32_t)dims.size(), order, ib ? 1 : 0, on};
  for (size_t k = 0; k < dims.size() && k < 2; ++k) a.dims[k] = dims[k];
  return a;
}
Dim MomentDimension::dim_forward(const std::vector<Dim>& xs) const {
  ARG_CHECK(xs.size() == 1, "Failed input count check in MomentDimension");
  ARG_CHECK(order >= 1, "Order of moment should be >=1 in MomentDimension (received " << order << ")");
  return moment_dim(xs[0], dims, include_batch_dim, "MomentDimension");
}
SIMPLE_NODE(MomentDimension, moment_dim, dyb200_moment_attrs at = moment_attrs(dims, order, include_batch_dim, overwrite_n); const void* attrs_ptr = &at)
Dim StdDimension::dim_forward(const std::vector<Dim>& xs) const {
  ARG_CHECK(xs.size() == 1, "Failed input count check in StdDimension");
  return moment_dim(xs[0], dims, include_batch_dim, "StdDimension");
}
SIMPLE_NODE(StdDimension, std_dim, dyb200_moment_attrs at = moment_attrs(dims, 2, include_batch_dim, overwrite_n); const void* attrs_ptr = &at)

Dim LayerNormFused::dim_forward(const std::vector<Dim>& xs) const {
  ARG_CHECK(xs.size() == 3, "layer_norm expects (x, g, b)");
  ARG_CHECK(xs[1].size() == xs[0].batch_size() && xs[2].size() == xs[0].batch_size(), "layer_norm: gain/bias must match one batch element of x");
  return xs[0];
}
SIMPLE_NODE(LayerNormFused, layer_norm, NO_ATTRS)

// ---- embedding ----
Dim LookupNode::dim_forward(const std::vector<Dim>&) const { return dim; }   // dynet/param-nodes.cc:164-166
void LookupNode::forward_dev_impl(const Device_GPU& dev, const std::vector<const Tensor*>& xs, Tensor& fx) const {
  dyb200_lookup_attrs at = {all_values.v, all_values.d.bd, ids_preloaded ? nullptr : pindices->data(), dim.bd, weight_decay};
  call_fwd(dyb200_lookup_fwd, dev, xs, fx, &at, aux_mem);
}
void LookupNode::backward_dev_impl(const Device_GPU&, const std::vector<const Tensor*>&, const Tensor&, const Tensor&,
                                   unsigned i, Tensor&) const {
  std::ostringstream oss;
  oss << "called backward() on arity 0 node: i = " << i;   // dynet/param-nodes.cc:331-339
  throw std::runtime_error(oss.str());
}
void LookupNode::accumulate_grad(const Device_GPU& dev, const Tensor& g, Tensor& all_grads) const {
  throw_status(dev, dyb200_lookup_accumulate_grads(dim.bd, ids_preloaded ? nullptr : pindices->data(), (const unsigned*)aux_mem,
                                                   g.v, all_grads.v, (unsigned)all_grads.d.batch_size(), all_grads.d.bd, dev.ctx));
}

// ---- fused LSTM ----
Dim VanillaLSTMGates::dim_forward(const std::vector<Dim>& xs) const {   // dynet/nodes-lstm.cc:24-59
  ARG_CHECK(xs.size() >= (dropout ? 7u : 5u), "Failed input count check in VanillaLSTMGates");
  unsigned num_inputs = dropout ? xs.size() - 6 : xs.size() - 4;
  unsigned hidden_dim = xs[num_inputs][0], input_dim = xs[num_inputs + 1][1], batch_size = xs[0].bd, sum = 0;
  for (unsigned i = 0; i < num_inputs; ++i) {
    ARG_CHECK(xs[i].ndims() == 1, "VanillaLSTMGates: x_t[" << i << "] expected to be a vector");
    ARG_CHECK(xs[i].bd == batch_size, "VanillaLSTMGates: x_t has inconsistent batch size");
    sum += xs[i][0];
  }
  ARG_CHECK(sum == input_dim, "VanillaLSTMGates: x_t has inconsistent dimension");
  ARG_CHECK(xs[num_inputs + 1][0] == hidden_dim * 4, "VanillaLSTMGates: Wx dim 0 expected " << hidden_dim * 4);
  ARG_CHECK(xs[num_inputs + 2][0] == hidden_dim * 4 && xs[num_inputs + 2][1] == hidden_dim, "VanillaLSTMGates: Wh expected " << hidden_dim * 4 << " x " << hidden_dim);
  ARG_CHECK(xs[num_inputs + 3][0] == hidden_dim * 4, "VanillaLSTMGates: b dim expected " << hidden_dim * 4);
  return Dim({hidden_dim * 4}, batch_size);
}
SIMPLE_NODE(VanillaLSTMGates, vanilla_lstm_gates,
            dyb200_lstm_gates_attrs at = {dropout ? 1 : 0, weightnoise_std, forget_gate_bias}; const void* attrs_ptr = &at)
static Dim lstm_ch_dim(const std::vector<Dim>& xs, const char* name) {   // dynet/nodes-lstm.cc:541-548, :629-636
  ARG_CHECK(xs.size() == 2, "Failed input count check in " << name);
  ARG_CHECK(xs[0].ndims() == 1 && xs[1].ndims() == 1, name << ": c and gates_t expected to be vectors");
  ARG_CHECK(xs[0].size() * 4 == xs[1].size(), name << ": gates_t expected 4 times as big as c_t, but " << xs[0].size() << "*4 != " << xs[1].size());
  ARG_CHECK(xs[0].bd == xs[1].bd, name << ": gates_t and c_t expected to have equal batch size");
  return xs[0];
}
Dim VanillaLSTMC::dim_forward(const std::vector<Dim>& xs) const { return lstm_ch_dim(xs, "VanillaLSTMC"); }
Dim VanillaLSTMH::dim_forward(const std::vector<Dim>& xs) const { return lstm_ch_dim(xs, "VanillaLSTMH"); }
SIMPLE_NODE(VanillaLSTMC, vanilla_lstm_c, NO_ATTRS)
SIMPLE_NODE(VanillaLSTMH, vanilla_lstm_h, NO_ATTRS)

// ---- glue nodes ----
Dim PickRange::dim_forward(const std::vector<Dim>& xs) const {         // dynet/nodes-select.cc:206-212
  ARG_CHECK(xs.size() == 1, "Failed input count check in PickRange");
  ARG_CHECK(dim < xs[0].nd && start < end && xs[0][dim] >= end, "Bad input dimensions or range in PickRange: range(" << start << ", " << end << ") with dim=" << dim);
  Dim ret = xs[0];
  ret.d[dim] = end - start;
  return ret;
}
SIMPLE_NODE(PickRange, pick_range, dyb200_pick_range_attrs at = {start, end, dim}; const void* attrs_ptr = &at)
Dim Concatenate::dim_forward(const std::vector<Dim>& xs) const {       // dynet/nodes-concat.cc:25-40
  ARG_CHECK(!xs.empty(), "Concatenate needs at least one argument");
  unsigned new_rows = 0;
  Dim dr = xs[0];
  if (dr.nd < dimension + 1) { for (unsigned k = dr.nd; k < dimension + 1; ++k) dr.d[k] = 1; dr.nd = dimension + 1; }
  for (Dim c : xs) {
    if (c.nd < dr.nd) { for (unsigned k = c.nd; k < dr.nd; ++k) c.d[k] = 1; c.nd = dr.nd; }
    ARG_CHECK(c.nd == dr.nd, "Bad input dimensions in Concatenate");
    new_rows += c[dimension];
    for (unsigned k = 0; k < dr.nd; ++k) ARG_CHECK(k == dimension || c.d[k] == dr.d[k], "Bad input dimensions in Concatenate");
    dr.bd = std::max(dr.bd, c.bd);
  }
  dr.d[dimension] = new_rows;
  return dr;
}
SIMPLE_NODE(Concatenate, concatenate, dyb200_dim_attrs at = {dimension}; const void* attrs_ptr = &at)
Dim Sum::dim_forward(const std::vector<Dim>& xs) const {               // dynet/nodes-arith-sum.cc:22-33
  ARG_CHECK(xs.size() > 0, "Zero-length vector passed to Sum");
  Dim d = xs[0];
  for (size_t i = 1; i < xs.size(); ++i) {
    ARG_CHECK(d.batch_size() == xs[i].batch_size(), "Mismatched input dimensions in Sum");
    d.bd = std::max(xs[i].bd, d.bd);
  }
  return d;
}
SIMPLE_NODE(Sum, sum, NO_ATTRS)
Dim SumDimension::dim_forward(const std::vector<Dim>& xs) const {      // dynet/nodes-arith-sum.cc:182-193
  ARG_CHECK(xs.size() == 1, "Failed input count check in SumDimension");
  ARG_CHECK(xs[0].nd <= 3, "SumDimension implemented up to tensors of order 3 (with minibatch) for now");
  ARG_CHECK(dims.size() <= 2, "Number of dimensions to reduce (excluding batch dimension) implemented up to 2 in SumDimension");
  ARG_CHECK(!dims.empty() || include_batch_dim, "At least one dimension has to be reduced (including batch dimension) in SumDimension");
  Dim ret;
  for (unsigned d : dims) ARG_CHECK(d < xs[0].nd, "dimension " << d << " is out of bounds of tensor of order " << xs[0].nd << " in SumDimension");
  for (unsigned k = 0; k < xs[0].nd; ++k) {
    bool removed = false;
    for (unsigned d : dims) removed = removed || d == k;
    if (!removed) ret.d[ret.nd++] = xs[0].d[k];
  }
  if (ret.nd == 0) ret.d[ret.nd++] = 1;   // Dim::delete_dims keeps a size-1 vector (dynet/dim.h:234-256)
  ret.bd = include_batch_dim ? 1 : xs[0].bd;
  return ret;
}
static dyb200_sum_dim_attrs sum_dim_attrs(const std::vector<unsigned>& dims, bool b) {
  dyb200_sum_dim_attrs a = {{0, 0}, (unsigned)dims.size(), b ? 1 : 0};
  for (size_t k = 0; k < dims.size() && k < 2; ++k) a.dims[k] = dims[k];
  return a;
}
SIMPLE_NODE(SumDimension, sum_dim, dyb200_sum_dim_attrs at = sum_dim_attrs(dims, include_batch_dim); const void* attrs_ptr = &at)
Dim SquaredNorm::dim_forward(const std::vector<Dim>& xs) const {       // dynet/nodes-norms.cc:22-25
  ARG_CHECK(xs.size() == 1, "Failed input count check in SquaredNorm");
  return Dim({1}, xs[0].bd);
}
SIMPLE_NODE(SquaredNorm, squared_norm, NO_ATTRS)
UNARY_DIM(Negate) SIMPLE_NODE(Negate, negate, NO_ATTRS)
UNARY_DIM(ConstantPlusX) SIMPLE_NODE(ConstantPlusX, constant_plus_x, dyb200_const_attrs at = {c}; const void* attrs_ptr = &at)
UNARY_DIM(ConstantMinusX) SIMPLE_NODE(ConstantMinusX, constant_minus_x, dyb200_const_attrs at = {c}; const void* attrs_ptr = &at)

// ---- MatrixMultiply / AffineTransform ----
Dim MatrixMultiply::dim_forward(const std::vector<Dim>& xs) const {   // dynet/nodes-matrixmultiply.cc:21-27
  ARG_CHECK(xs.size() == 2, "Failed input count check in MatrixMultiply");
  ARG_CHECK(xs[0].cols() == xs[1].rows(), "Mismatched input dimensions in MatrixMultiply");
  ARG_CHECK(xs[0].nd <= 2 && xs[1].nd <= 2, "Cannot multiply tensors of dimension higher than 2");
  if (xs[1].ndims() == 1) return Dim({xs[0].rows()}, std::max(xs[0].bd, xs[1].bd));
  return Dim({xs[0].rows(), xs[1].cols()}, std::max(xs[0].bd, xs[1].bd));
}
SIMPLE_NODE(MatrixMultiply, matmul, NO_ATTRS)
Dim AffineTransform::dim_forward(const std::vector<Dim>& xs) const {  // dynet/nodes-affinetransform.cc:23-38
  ARG_CHECK((xs.size() - 1) % 2 == 0, "Bad number of inputs in AffineTransform");
  if (xs.size() == 1) return xs[0];
  ARG_CHECK(xs[0].rows() == xs[1].rows() && xs[1].cols() == xs[2].rows(), "Bad dimensions for AffineTransform");
  unsigned bd = std::max(std::max(xs[0].bd, xs[1].bd), xs[2].bd);
  Dim d = xs[2].cols() != 1 ? Dim({xs[0].rows(), xs[2].cols()}, bd) : Dim({xs[0].rows()}, bd);
  for (size_t i = 3; i < xs.size(); i += 2) {
    ARG_CHECK(xs[i].cols() == xs[i + 1].rows() && d.rows() == xs[i].rows() && d.cols() == xs[i + 1].cols(),
              "Bad dimensions for AffineTransform");
    d.bd = std::max(std::max(d.bd, xs[i].bd), xs[i + 1].bd);
  }
  return d;
}
SIMPLE_NODE(AffineTransform, affine_transform, NO_ATTRS)

namespace gpu {
void parallel_memcpy(const Device_GPU& dev, int num_seqs, int max_len, float** src, float** trg, size_t* len) {
  throw_status(dev, dyb200_parallel_memcpy(num_seqs, max_len, src, trg, len, dev.ctx));
}
void parallel_accumulate(const Device_GPU& dev, int num_seqs, int max_len, float** src, float** trg, size_t* len) {
  throw_status(dev, dyb200_parallel_accumulate(num_seqs, max_len, src, trg, len, dev.ctx));
}
}  // namespace gpu

}  // namespace dynet_b200

// ---- shape rules without a device: dim_forward of a node by name --------------------------------------------------------
// xs: the argument shapes (the `v` fields are ignored); iargs: the node's integer constructor arguments (Softmax /
// LogSumExpDimension / Concatenate: dimension; PickRange: start, end, dim; SumDimension: include_batch_dim, dims...;
// MomentDimension: order, include_batch_dim, dims...; StdDimension: include_batch_dim, dims...; VanillaLSTMGates: dropout;
// LookupNode: E, n).  Returns DYB200_OK and the result shape, or DYB200_EINVAL with the reference's message in `err`.
extern "C" int dyb200h_dim_forward(const char* node, const dyb200_tensor* xs, int nxs, const int32_t* iargs, int niargs,
                                   dyb200_tensor* out, char* err, size_t errlen) {
  using namespace dynet_b200;
  auto arg = [&](int k) -> unsigned { return k < niargs ? (unsigned)iargs[k] : 0u; };
  std::vector<Dim> dims;
  for (int k = 0; k < nxs; ++k) {
    Dim d;
    d.nd = xs[k].nd; d.bd = xs[k].bd;
    for (unsigned q = 0; q < d.nd && q < 7; ++q) d.d[q] = xs[k].d[q];
    dims.push_back(d);
  }
  const std::string n = node ? node : "";
  try {
    Dim r;
    std::vector<unsigned> rest;
    if (n == "Tanh") r = Tanh().dim_forward(dims);
    else if (n == "LogisticSigmoid") r = LogisticSigmoid().dim_forward(dims);
    else if (n == "Rectify") r = Rectify().dim_forward(dims);
    else if (n == "ExponentialLinearUnit") r = ExponentialLinearUnit().dim_forward(dims);
    else if (n == "CwiseMultiply") r = CwiseMultiply().dim_forward(dims);
    else if (n == "CwiseSum") r = CwiseSum().dim_forward(dims);
    else if (n == "CwiseQuotient") r = CwiseQuotient().dim_forward(dims);
    else if (n == "Softmax") r = Softmax(arg(0)).dim_forward(dims);
    else if (n == "LogSoftmax") r = LogSoftmax().dim_forward(dims);
    else if (n == "LogSumExp") r = LogSumExp().dim_forward(dims);
    else if (n == "LogSumExpDimension") r = LogSumExpDimension(arg(0)).dim_forward(dims);
    else if (n == "PickNegLogSoftmax") { std::vector<unsigned> ids(arg(0), 0u); r = PickNegLogSoftmax(&ids).dim_forward(dims); }
    else if (n == "WeightNormalization") r = WeightNormalization().dim_forward(dims);
    else if (n == "MomentDimension") { for (int k = 2; k < niargs; ++k) rest.push_back(arg(k)); r = MomentDimension(rest, arg(0), arg(1) != 0).dim_forward(dims); }
    else if (n == "StdDimension") { for (int k = 1; k < niargs; ++k) rest.push_back(arg(k)); r = StdDimension(rest, arg(0) != 0).dim_forward(dims); }
    else if (n == "LayerNormFused") r = LayerNormFused().dim_forward(dims);
    else if (n == "LookupNode") { Tensor t(Dim({arg(0)}, 1), nullptr); r = LookupNode(t, nullptr, arg(1)).dim_forward(dims); }
    else if (n == "VanillaLSTMGates") r = VanillaLSTMGates(arg(0) != 0).dim_forward(dims);
    else if (n == "VanillaLSTMC") r = VanillaLSTMC().dim_forward(dims);
    else if (n == "VanillaLSTMH") r = VanillaLSTMH().dim_forward(dims);
    else if (n == "PickRange") r = PickRange(arg(0), arg(1), arg(2)).dim_forward(dims);
    else if (n == "Concatenate") r = Concatenate(arg(0)).dim_forward(dims);
    else if (n == "Sum") r = Sum().dim_forward(dims);
    else if (n == "SumDimension") { for (int k = 1; k < niargs; ++k) rest.push_back(arg(k)); r = SumDimension(rest, arg(0) != 0).dim_forward(dims); }
    else if (n == "SquaredNorm") r = SquaredNorm().dim_forward(dims);
    else if (n == "Negate") r = Negate().dim_forward(dims);
    else if (n == "ConstantPlusX") r = ConstantPlusX(0.f).dim_forward(dims);
    else if (n == "ConstantMinusX") r = ConstantMinusX(0.f).dim_forward(dims);
    else if (n == "MatrixMultiply") r = MatrixMultiply().dim_forward(dims);
    else if (n == "AffineTransform") r = AffineTransform().dim_forward(dims);
    else { if (err && errlen) snprintf(err, errlen, "unknown node %s", n.c_str()); return DYB200_ERUNTIME; }
    if (out) {
      out->v = nullptr; out->nd = r.nd; out->bd = r.bd;
      for (unsigned q = 0; q < 7; ++q) out->d[q] = q < r.nd ? r.d[q] : 0;
    }
    return DYB200_OK;
  } catch (const std::invalid_argument& e) {
    if (err && errlen) snprintf(err, errlen, "%s", e.what());
    return DYB200_EINVAL;
  }
}
