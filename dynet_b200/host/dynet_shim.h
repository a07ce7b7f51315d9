// Host-side mirror of the reference's node interface for the fused-layer path.
//
// DyNet declares, for every node (dynet/nodes-def-macros.h:44-62),
//   template<class MyDevice> void forward_dev_impl(const MyDevice&, const std::vector<const Tensor*>& xs, Tensor& fx) const;
//   template<class MyDevice> void backward_dev_impl(const MyDevice&, const std::vector<const Tensor*>& xs,
//                                                   const Tensor& fx, const Tensor& dEdf, unsigned i, Tensor& dEdxi) const;
// and instantiates them for Device_GPU in its CUDA build (dynet/nodes-impl-macros.h:13-21).
// The classes below carry the same names, constructor arguments, aux_storage_size() and
// dim_forward() rules, and implement those two members by unpacking the tensors and calling
// the C ABI of libdyb200.so.  Inside a DyNet tree the same bodies become the explicit
// `template<> void NodeT::forward_dev_impl<Device_GPU>(...)` specialisations.
//
// Errors: a non-zero C status is turned into the exception type the reference throws at the
// same place (std::invalid_argument, std::runtime_error, cuda_exception, out_of_memory).
#pragma once
#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/dyb200.h"

namespace dynet_b200 {

struct cuda_exception : public std::runtime_error {          // dynet/cuda.h:20-24
  explicit cuda_exception(const std::string& what) : std::runtime_error(what) {}
};
struct out_of_memory : public std::runtime_error {           // dynet/except.h:11-14
  explicit out_of_memory(const std::string& what) : std::runtime_error(what) {}
};

// dynet::Dim (dynet/dim.h:24-303): up to 7 dims plus the batch size.
struct Dim {
  unsigned d[7] = {0, 0, 0, 0, 0, 0, 0};
  unsigned nd = 0;
  unsigned bd = 1;
  Dim() {}
  Dim(std::initializer_list<unsigned> x, unsigned b = 1) : nd(0), bd(b) { for (auto v : x) d[nd++] = v; }
  unsigned operator[](unsigned i) const { return i < nd ? d[i] : 1; }
  unsigned ndims() const { return nd; }
  unsigned batch_elems() const { return bd; }
  size_t batch_size() const { size_t p = 1; for (unsigned i = 0; i < nd; ++i) p *= d[i]; return p; }
  size_t size() const { return batch_size() * bd; }
  unsigned rows() const { return (*this)[0]; }
  unsigned cols() const { return nd > 1 ? d[1] : 1; }
  bool operator==(const Dim& o) const {
    if (nd != o.nd || bd != o.bd) return false;
    for (unsigned i = 0; i < nd; ++i) if (d[i] != o.d[i]) return false;
    return true;
  }
};

// dynet::Tensor (dynet/tensor.h:44-130): a non-owning view.
struct Tensor {
  Dim d;
  float* v = nullptr;
  Tensor() {}
  Tensor(const Dim& dim, float* ptr) : d(dim), v(ptr) {}
};

// dynet::Device_GPU (dynet/devices.h:46-61), reduced to what the kernels need.
struct Device_GPU {
  int cuda_device_id = 0;
  dyb200_ctx* ctx = nullptr;
};

void throw_status(const Device_GPU& dev, int status);
dyb200_tensor to_c(const Tensor& t);

// dynet::Node (dynet/dynet.h:526-775), the part the executors use on this path.
struct Node {
  mutable void* aux_mem = nullptr;   // set by the caller to aux_storage_size() bytes of device memory
  Dim dim;                           // result of dim_forward, cached by the graph in the reference
  virtual ~Node() {}
  virtual const char* name() const = 0;
  virtual Dim dim_forward(const std::vector<Dim>& xs) const = 0;
  virtual size_t aux_storage_size() const { return 0; }
  virtual bool supports_multibatch() const { return true; }
  virtual void forward_dev_impl(const Device_GPU& dev, const std::vector<const Tensor*>& xs, Tensor& fx) const = 0;
  virtual void backward_dev_impl(const Device_GPU& dev, const std::vector<const Tensor*>& xs, const Tensor& fx,
                                 const Tensor& dEdf, unsigned i, Tensor& dEdxi) const = 0;
};

typedef int (*fwd_fn)(const dyb200_tensor*, int, dyb200_tensor*, const void*, void*, dyb200_ctx*);
typedef int (*bwd_fn)(const dyb200_tensor*, int, const dyb200_tensor*, const dyb200_tensor*, unsigned, dyb200_tensor*,
                      const void*, void*, dyb200_ctx*);
void call_fwd(fwd_fn f, const Device_GPU& dev, const std::vector<const Tensor*>& xs, Tensor& fx, const void* attrs, void* aux);
void call_bwd(bwd_fn f, const Device_GPU& dev, const std::vector<const Tensor*>& xs, const Tensor& fx, const Tensor& dEdf,
              unsigned i, Tensor& dEdxi, const void* attrs, void* aux);

#define DYB200_NODE_COMMON(NAME)                                                                              \
  const char* name() const override { return #NAME; }                                                         \
  Dim dim_forward(const std::vector<Dim>& xs) const override;                                                 \
  void forward_dev_impl(const Device_GPU& dev, const std::vector<const Tensor*>& xs, Tensor& fx) const override; \
  void backward_dev_impl(const Device_GPU& dev, const std::vector<const Tensor*>& xs, const Tensor& fx,       \
                         const Tensor& dEdf, unsigned i, Tensor& dEdxi) const override;

// ---- activations (dynet/nodes-trig.h, dynet/nodes-activations.h) ----
struct Tanh : Node { DYB200_NODE_COMMON(Tanh) };
struct LogisticSigmoid : Node { DYB200_NODE_COMMON(LogisticSigmoid) };
struct Rectify : Node { DYB200_NODE_COMMON(Rectify) };
struct ExponentialLinearUnit : Node {
  float lambda, alpha;  // argument order of the reference constructor (nodes-activations.h:46-53)
  explicit ExponentialLinearUnit(float lambda = 1.f, float alpha = 1.f) : lambda(lambda), alpha(alpha) {}
  DYB200_NODE_COMMON(ExponentialLinearUnit)
};
// ---- cwise binary (dynet/nodes-arith-cwise.h) ----
struct CwiseMultiply : Node { DYB200_NODE_COMMON(CwiseMultiply) };
struct CwiseSum : Node { DYB200_NODE_COMMON(CwiseSum) };
struct CwiseQuotient : Node { DYB200_NODE_COMMON(CwiseQuotient) };
// ---- softmax family (dynet/nodes-softmaxes.h, nodes-logsumexp.h, nodes-pickneglogsoftmax.h) ----
struct Softmax : Node {
  unsigned dimension;
  explicit Softmax(unsigned d = 0) : dimension(d) {}
  DYB200_NODE_COMMON(Softmax)
};
struct LogSoftmax : Node {
  size_t aux_storage_size() const override { return 2 * dim.size() / dim.rows() * sizeof(float); }
  DYB200_NODE_COMMON(LogSoftmax)
};
struct LogSumExp : Node { DYB200_NODE_COMMON(LogSumExp) };
struct LogSumExpDimension : Node {
  unsigned dimension;
  explicit LogSumExpDimension(unsigned d = 0) : dimension(d) {}
  DYB200_NODE_COMMON(LogSumExpDimension)
};
struct PickNegLogSoftmax : Node {
  const std::vector<unsigned>* pvals;   // host ids, one per batch element (pval is the size-1 case)
  const unsigned* ids_dev_preloaded;    // non-null: ids already sit in aux_mem on the device
  explicit PickNegLogSoftmax(const std::vector<unsigned>* ids) : pvals(ids), ids_dev_preloaded(nullptr) {}
  size_t aux_storage_size() const override { return 2 * dim.batch_elems() * sizeof(float) + dim.batch_elems() * sizeof(unsigned); }
  DYB200_NODE_COMMON(PickNegLogSoftmax)
};
// ---- normalisation (dynet/nodes-normalization.h, nodes-moments.h) ----
struct WeightNormalization : Node { DYB200_NODE_COMMON(WeightNormalization) };
struct MomentDimension : Node {
  std::vector<unsigned> dims; unsigned order; bool include_batch_dim; unsigned overwrite_n;
  MomentDimension(const std::vector<unsigned>& dims, unsigned order, bool include_batch_dim = false, unsigned overwrite_n = 0)
      : dims(dims), order(order), include_batch_dim(include_batch_dim), overwrite_n(overwrite_n) {}
  bool supports_multibatch() const override { return true; }
  DYB200_NODE_COMMON(MomentDimension)
};
struct StdDimension : Node {
  std::vector<unsigned> dims; bool include_batch_dim; unsigned overwrite_n;
  StdDimension(const std::vector<unsigned>& dims, bool include_batch_dim = false, unsigned overwrite_n = 0)
      : dims(dims), include_batch_dim(include_batch_dim), overwrite_n(overwrite_n) {}
  DYB200_NODE_COMMON(StdDimension)
};
// The 8-node composite of dynet/expr.cc:248-253 as one node (xs = x, g, b).
struct LayerNormFused : Node { DYB200_NODE_COMMON(LayerNormFused) };
// ---- embedding (dynet/param-nodes.h:84-110) ----
struct LookupNode : Node {
  Tensor all_values;                     // Dim({E}, V)
  const std::vector<unsigned>* pindices; // host ids (pindex is the size-1 case); null when preloaded
  float weight_decay;                    // params.current_weight_decay()
  bool ids_preloaded;                    // ids already sit in aux_mem on the device
  LookupNode(const Tensor& table, const std::vector<unsigned>* ids, unsigned n, float wd = 1.f)
      : all_values(table), pindices(ids), weight_decay(wd), ids_preloaded(ids == nullptr) {
    dim = Dim({(unsigned)table.d.batch_size()}, n);
  }
  size_t aux_storage_size() const override { return dim.bd * sizeof(unsigned); }
  DYB200_NODE_COMMON(LookupNode)
  // LookupNode::accumulate_grad -> LookupParameterStorage::accumulate_grads (dynet/param-nodes.cc:168-175)
  void accumulate_grad(const Device_GPU& dev, const Tensor& g, Tensor& all_grads) const;
};
// ---- fused LSTM (dynet/nodes-lstm.h) ----
struct VanillaLSTMGates : Node {
  bool dropout; float weightnoise_std; float forget_gate_bias;
  explicit VanillaLSTMGates(bool dropout, float weightnoise_std = 0.f) : dropout(dropout), weightnoise_std(weightnoise_std), forget_gate_bias(1.f) {}
  DYB200_NODE_COMMON(VanillaLSTMGates)
};
struct VanillaLSTMC : Node { DYB200_NODE_COMMON(VanillaLSTMC) };
struct PickRange : Node {                                                 // dynet/nodes-select.h
  unsigned start, end, dim;
  PickRange(unsigned s, unsigned e, unsigned d = 0) : start(s), end(e), dim(d) {}
  DYB200_NODE_COMMON(PickRange)
};
struct Concatenate : Node {                                               // dynet/nodes-concat.h
  unsigned dimension;
  explicit Concatenate(unsigned d = 0) : dimension(d) {}
  DYB200_NODE_COMMON(Concatenate)
};
struct Sum : Node { DYB200_NODE_COMMON(Sum) };                            // dynet/nodes-arith-sum.h
struct SumDimension : Node {
  std::vector<unsigned> dims; bool include_batch_dim;
  SumDimension(const std::vector<unsigned>& d, bool b) : dims(d), include_batch_dim(b) {}
  DYB200_NODE_COMMON(SumDimension)
};
struct SquaredNorm : Node { DYB200_NODE_COMMON(SquaredNorm) };            // dynet/nodes-norms.h
struct Negate : Node { DYB200_NODE_COMMON(Negate) };                      // dynet/nodes-arith-unary.h
struct ConstantPlusX : Node {                                             // dynet/nodes-arith-const.h
  float c;
  explicit ConstantPlusX(float v) : c(v) {}
  DYB200_NODE_COMMON(ConstantPlusX)
};
struct ConstantMinusX : Node {
  float c;
  explicit ConstantMinusX(float v) : c(v) {}
  DYB200_NODE_COMMON(ConstantMinusX)
};
struct MatrixMultiply : Node { DYB200_NODE_COMMON(MatrixMultiply) };     // dynet/nodes-matrixmultiply.h
struct AffineTransform : Node { DYB200_NODE_COMMON(AffineTransform) };   // dynet/nodes-affinetransform.h
struct VanillaLSTMH : Node { DYB200_NODE_COMMON(VanillaLSTMH) };

// dynet::gpu::parallel_memcpy / parallel_accumulate (dynet/gpu-ops.h:14-15)
namespace gpu {
void parallel_memcpy(const Device_GPU& dev, int num_seqs, int max_len, float** src, float** trg, size_t* len);
void parallel_accumulate(const Device_GPU& dev, int num_seqs, int max_len, float** src, float** trg, size_t* len);
}  // namespace gpu

}  // namespace dynet_b200
