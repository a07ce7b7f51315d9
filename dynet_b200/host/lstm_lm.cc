// One training step of the batched LSTM language model, driven node by node.
//
// Graph (examples/batching/rnnlm-batch.h:110-151 over CompactVanillaLSTMBuilder,
// dynet/lstm.cc:1044-1080): per time step  x = lookup(C, tok[t]); per layer gates -> c -> h
// (vanilla_lstm_gates[_dropout], vanilla_lstm_c, vanilla_lstm_h); r = bias + R * h;
// err_t = pickneglogsoftmax(r, tok[t+1]); loss = sum_batches(sum_t err_t).
// Forward calls each node's forward_dev_impl in topological order; backward walks the nodes in
// reverse and calls backward_dev_impl once per differentiable argument, accumulating (+=) into
// gradient memory that was zeroed once (dynet/exec.cc:166-284); the lookup gradients are
// scattered after the reverse pass in time order (exec.cc:277-282).
// Parameters are read in place (weight decay is 1).  With `fused` set, Gates + C + H of a step are one call,
// weight gradients are deferred to one product per parameter, and the output layer (affine_transform +
// pickneglogsoftmax), which does not feed back into the recurrence, runs once over all T*B columns.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "dynet_shim.h"

using namespace dynet_b200;

extern "C" {
typedef struct {
  uint32_t V, E, H, L, T, B;
  float lr, clip;
  int32_t dropout;  // 0: vanilla_lstm_gates, 1: vanilla_lstm_gates_dropout (masks are inputs)
  int32_t fused;    // 0: one call per node and argument; 1: dyb200_vanilla_lstm_{fwd,bwd}_fused per layer and step
} dyb200h_lm_config;
}

namespace {

struct Arena {
  char* base; size_t size, off;
  template <class Tp> Tp* take(size_t n) {
    off = (off + 255) & ~(size_t)255;
    Tp* p = (Tp*)(base + off);
    off += n * sizeof(Tp);
    return p;
  }
};

size_t param_sizes(const dyb200h_lm_config& c, std::vector<size_t>* sizes) {
  size_t total = 0;
  auto add = [&](size_t n) { if (sizes) sizes->push_back(n); total += n; };
  add((size_t)c.E * c.V);
  for (uint32_t l = 0; l < c.L; ++l) {
    add((size_t)4 * c.H * (l == 0 ? c.E : c.H));
    add((size_t)4 * c.H * c.H);
    add((size_t)4 * c.H);
  }
  add((size_t)c.V * c.H);
  add(c.V);
  return total;
}

struct Lm {
  dyb200h_lm_config c;
  Device_GPU dev;
  std::string err;
  float *params, *grads;
  std::vector<float*> p, g;       // per-tensor views into the flat buffers
  // activations
  uint32_t* tok;                  // (T+1) x B ids on the device
  float *x, *gates, *cs, *hs, *r, *aux, *errs, *zeros, *ones;
  // gradients of activations
  float *dact, *dx, *dh, *dc, *dgates, *dr;
  size_t dact_bytes;
  float* scalars;                 // [0] = squared gradient norm
  cudaStream_t stream;
  // fused driver: weight-gradient products deferred to the end of the backward pass (one per parameter)
  std::vector<dyb200_wgrad*> wg_layer;   // per layer: A = gate gradient, B0 = x .* mask_x, B1 = h_tm1 .* mask_h
  // CUDA-graph replay of the whole forward + backward pass (optional): the ~1400 launches of a step are
  // captured once and re-issued with one cudaGraphLaunch; inputs live at fixed addresses (tok, mask_buf).
  bool use_graph = false;
  bool time_major = false;               // fused driver: time step by time step (the reference's order) instead of layer by layer
  std::vector<cudaGraphExec_t> graph_exec;   // [0]: the whole step; [1 + p]: phase p (see step_body)
  float* graph_loss = nullptr;
  uint64_t graph_launches = 0;
  std::vector<float*> mask_buf;          // 2L buffers: mask_x_l (I_l x B), mask_h_l (H x B)
  void drop_graphs() {
    for (auto& g : graph_exec) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
  }
  ~Lm() {
    drop_graphs();
    for (auto w : wg_layer) dyb200_wgrad_destroy(w);
  }
};

size_t plan(const dyb200h_lm_config& c, Lm* m, char* base, size_t size) {
  Arena a{base, size, 0};
  const size_t HB = (size_t)c.H * c.B, GB = 4 * HB, VB = (size_t)c.V * c.B, EB = (size_t)c.E * c.B, TL = (size_t)c.T * c.L;
  uint32_t* tok = a.take<uint32_t>((size_t)(c.T + 1) * c.B);
  float* x = a.take<float>(c.T * EB);
  float* gates = a.take<float>(TL * GB);
  float* cs = a.take<float>(TL * HB);
  float* hs = a.take<float>(TL * HB);
  float* r = a.take<float>(c.T * VB);
  float* aux = a.take<float>((size_t)c.T * 3 * c.B);
  float* errs = a.take<float>((size_t)c.T * c.B);
  float* zeros = a.take<float>(HB);
  float* ones = a.take<float>((size_t)c.T * c.B);
  float* scalars = a.take<float>(64);
  std::vector<float*> mask_buf;
  for (uint32_t l = 0; l < c.L; ++l) {
    mask_buf.push_back(a.take<float>((size_t)(l == 0 ? c.E : c.H) * c.B));
    mask_buf.push_back(a.take<float>(HB));
  }
  float* dr = a.take<float>(c.fused ? c.T * VB : VB);   // d(logits): all steps at once in the fused driver
  // everything below is zeroed by one memset per backward
  a.off = (a.off + 255) & ~(size_t)255;
  size_t d0 = a.off;
  float* dx = a.take<float>(c.T * EB);
  float* dh = a.take<float>(TL * HB);
  float* dc = a.take<float>(TL * HB);
  float* dgates = a.take<float>(TL * GB);
  size_t d1 = a.off;
  if (m) {
    m->tok = tok; m->x = x; m->gates = gates; m->cs = cs; m->hs = hs; m->r = r; m->aux = aux; m->errs = errs;
    m->zeros = zeros; m->ones = ones; m->scalars = scalars; m->dr = dr; m->dx = dx; m->dh = dh; m->dc = dc; m->dgates = dgates;
    m->dact = (float*)(base + d0);
    m->dact_bytes = d1 - d0;
    m->mask_buf = mask_buf;
  }
  return a.off + 256;
}

#define CU(expr)                                                                              \
  do {                                                                                        \
    cudaError_t e__ = (expr);                                                                 \
    if (e__ != cudaSuccess) throw cuda_exception(std::string(#expr) + ": " + cudaGetErrorString(e__)); \
  } while (0)

// Everything of a step after its inputs are in place (token ids in m.tok, masks at `masks`).
// phase < 0: the whole step.  The fused layer-by-layer driver can also run it in L + 1 pieces, so that a data-parallel
// caller can start reducing the gradients that are already final while the rest of the backward pass runs:
//   phase 0      forward, loss, backward of the output layer   -> gradients of R and bias final
//   phase p >= 1 backward of layer L - p over all time steps and its weight-gradient products -> that layer's gradients final
//   phase L      also scatters the embedding gradients         -> gradients of the table final
void step_body(Lm& m, const float* const* masks, float* loss_dev, int phase = -1) {
  const bool do_fwd = phase <= 0;
  const dyb200h_lm_config& c = m.c;
  const uint32_t V = c.V, E = c.E, H = c.H, L = c.L, T = c.T, B = c.B;
  const size_t HB = (size_t)H * B, GB = 4 * HB, VB = (size_t)V * B, EB = (size_t)E * B;
  const Device_GPU& dev = m.dev;
  cudaStream_t st = m.stream;
  const uint32_t TB = T * B;
  // activations of layer l at time t sit at block l * T + t: every layer's states are one H x (T*B) matrix
  auto at = [T](uint32_t t, uint32_t l) { return (size_t)l * T + t; };
  // place the target ids where PickNegLogSoftmax expects them: aux = {z[n], m[n], ids[n]} with n = B per step,
  // or n = T*B when the output layer runs once over all time steps
  if (!do_fwd) {}
  else if (c.fused)
    CU(cudaMemcpyAsync(m.aux + 2 * (size_t)TB, m.tok + B, (size_t)TB * sizeof(uint32_t), cudaMemcpyDeviceToDevice, st));
  else
    CU(cudaMemcpy2DAsync(m.aux + 2 * (size_t)B, 3 * (size_t)B * sizeof(float), m.tok + B, (size_t)B * sizeof(uint32_t),
                         (size_t)B * sizeof(uint32_t), T, cudaMemcpyDeviceToDevice, st));

  Tensor tC(Dim({E}, V), m.p[0]), tR(Dim({V, H}), m.p[1 + 3 * L]), tbias(Dim({V}), m.p[2 + 3 * L]);
  Tensor tZero(Dim({H}, B), m.zeros);
  VanillaLSTMGates gates_node(c.dropout != 0);
  VanillaLSTMC c_node;
  VanillaLSTMH h_node;
  AffineTransform affine;
  PickNegLogSoftmax pnls(nullptr);
  pnls.dim = Dim({1}, B);

  auto layer_xs = [&](uint32_t t, uint32_t l, Tensor* store, std::vector<const Tensor*>& xs) {
    // store: [in, h_prev, Wx, Wh, b, mx, mh]
    uint32_t I = l == 0 ? E : H;
    store[0] = Tensor(Dim({I}, B), l == 0 ? m.x + t * EB : m.hs + at(t, l - 1) * HB);
    store[1] = t == 0 ? tZero : Tensor(Dim({H}, B), m.hs + at(t - 1, l) * HB);
    store[2] = Tensor(Dim({4 * H, I}), m.p[1 + 3 * l]);
    store[3] = Tensor(Dim({4 * H, H}), m.p[2 + 3 * l]);
    store[4] = Tensor(Dim({4 * H}), m.p[3 + 3 * l]);
    xs = {&store[0], &store[1], &store[2], &store[3], &store[4]};
    if (c.dropout) {
      store[5] = Tensor(Dim({I}, B), const_cast<float*>(masks[2 * l]));
      store[6] = Tensor(Dim({H}, B), const_cast<float*>(masks[2 * l + 1]));
      xs.push_back(&store[5]);
      xs.push_back(&store[6]);
    }
  };

  // ---------------- forward ----------------
  if (do_fwd && c.fused) {   // the T lookups read one table: one gather over the T*B ids
    LookupNode look(tC, nullptr, TB);
    look.aux_mem = m.tok;
    Tensor xall(Dim({E}, TB), m.x);
    look.forward_dev_impl(dev, {}, xall);
  }
  // Order of the (time step, layer) calls.  The node-by-node driver goes time step by time step like the reference's
  // graph.  The fused driver finishes a layer over all time steps before it starts the next one (layer l at step t needs
  // layer l - 1 at step t and layer l at step t - 1, which both orders provide): the split weight planes of one layer
  // (50 and 67 MB) then stay in the 126 MB L2 from step to step instead of alternating with the other layer's, which
  // matters when the per-GPU batch is small and the products are bound by weight traffic.  Same values either way
  // (dyb200h_lm_set_time_major restores the reference's order).
  const bool layer_major = c.fused && !m.time_major;
  if (phase > 0 && !layer_major) throw std::invalid_argument("the step runs in phases only in the fused layer-by-layer driver");
  if (do_fwd && layer_major) {
    // One call per layer: the inputs of a layer for all time steps are complete before it starts (embeddings, or the layer
    // below), so they are split into operand planes in one launch and the T steps run inside one kernel whose CTAs hand
    // h_t over on the device (dyb200_vanilla_lstm_seq_fwd; it makes the per-step calls itself when the shape does not allow that).
    for (uint32_t l = 0; l < L; ++l) {
      const uint32_t I = l == 0 ? E : H;
      Tensor xall(Dim({I}, TB), l == 0 ? m.x : m.hs + at(0, l - 1) * HB);
      Tensor gall(Dim({4 * H}, TB), m.gates + at(0, l) * GB), call(Dim({H}, TB), m.cs + at(0, l) * HB), hall_l(Dim({H}, TB), m.hs + at(0, l) * HB);
      Tensor tWx(Dim({4 * H, I}), m.p[1 + 3 * l]), tWh(Dim({4 * H, H}), m.p[2 + 3 * l]), tb(Dim({4 * H}), m.p[3 + 3 * l]);
      Tensor mxl(Dim({I}, B), c.dropout ? const_cast<float*>(masks[2 * l]) : nullptr), mhl(Dim({H}, B), c.dropout ? const_cast<float*>(masks[2 * l + 1]) : nullptr);
      dyb200_tensor cxa = to_c(xall), ch0 = to_c(tZero), cc0 = to_c(tZero), cWx = to_c(tWx), cWh = to_c(tWh), cb = to_c(tb), cmx = to_c(mxl),
                    cmh = to_c(mhl), cg = to_c(gall), cc = to_c(call), ch = to_c(hall_l);
      dyb200_lstm_gates_attrs at = {c.dropout ? 1 : 0, 0.f, 1.f};
      throw_status(dev, dyb200_vanilla_lstm_seq_fwd(&cxa, &ch0, &cc0, &cWx, &cWh, &cb, c.dropout ? &cmx : nullptr, c.dropout ? &cmh : nullptr,
                                                    &at, &cg, &cc, &ch, m.wg_layer[l], T, dev.ctx));
    }
  }
  for (uint32_t t = 0; t < ((layer_major || !do_fwd) ? 0u : T); ++t) {
    if (!c.fused) {
      LookupNode look(tC, nullptr, B);
      look.aux_mem = m.tok + (size_t)t * B;
      Tensor xt(Dim({E}, B), m.x + t * EB);
      look.forward_dev_impl(dev, {}, xt);
    }
    for (uint32_t l = 0; l < L; ++l) {
      size_t idx = at(t, l);
      Tensor store[7];
      std::vector<const Tensor*> xs;
      layer_xs(t, l, store, xs);
      Tensor tg(Dim({4 * H}, B), m.gates + idx * GB), tc(Dim({H}, B), m.cs + idx * HB), th(Dim({H}, B), m.hs + idx * HB);
      Tensor cprev = t == 0 ? tZero : Tensor(Dim({H}, B), m.cs + at(t - 1, l) * HB);
      if (c.fused) {
        dyb200_tensor cx = to_c(store[0]), chp = to_c(store[1]), ccp = to_c(cprev), cWx = to_c(store[2]), cWh = to_c(store[3]),
                      cb = to_c(store[4]), cmx, cmh, cg = to_c(tg), cc = to_c(tc), ch = to_c(th);
        if (c.dropout) { cmx = to_c(store[5]); cmh = to_c(store[6]); }
        dyb200_lstm_gates_attrs at = {c.dropout ? 1 : 0, 0.f, 1.f};
        // (the inputs of this step are also placed in the layer's weight-gradient accumulator, at the step's columns)
        throw_status(dev, dyb200_vanilla_lstm_fwd_fused_at(&cx, &chp, &ccp, &cWx, &cWh, &cb, c.dropout ? &cmx : nullptr,
                                                           c.dropout ? &cmh : nullptr, &at, &cg, &cc, &ch, m.wg_layer[l], t * B, dev.ctx));
        continue;
      }
      gates_node.forward_dev_impl(dev, xs, tg);
      c_node.forward_dev_impl(dev, {&cprev, &tg}, tc);
      h_node.forward_dev_impl(dev, {&tc, &tg}, th);
    }
    if (c.fused) continue;
    Tensor htop(Dim({H}, B), m.hs + at(t, L - 1) * HB), rt(Dim({V}, B), m.r + t * VB);
    // r = affine_transform({bias, R, h}) (examples/batching/rnnlm-batch.h:132)
    affine.forward_dev_impl(dev, {&tbias, &tR, &htop}, rt);
    pnls.aux_mem = m.aux + (size_t)t * 3 * B;
    Tensor et(Dim({1}, B), m.errs + (size_t)t * B);
    pnls.forward_dev_impl(dev, {&rt}, et);
  }
  // The output layer does not feed back into the recurrence: in the fused driver it runs once over the
  // H x (T*B) matrix of top-layer states (same values per column as the per-step nodes).
  Tensor hall(Dim({H}, TB), m.hs + at(0, L - 1) * HB), rall(Dim({V}, TB), m.r), eall(Dim({1}, TB), m.errs);
  const dyb200_affine_attrs R_is_param = {DYB200_GEMM_A_IS_PARAM};
  if (do_fwd && c.fused) {
    dyb200_tensor cxs[3] = {to_c(tbias), to_c(tR), to_c(hall)}, cr = to_c(rall);
    throw_status(dev, dyb200_affine_transform_fwd(cxs, 3, &cr, &R_is_param, nullptr, dev.ctx));
    pnls.dim = Dim({1}, TB);
    pnls.aux_mem = m.aux;
    pnls.forward_dev_impl(dev, {&rall}, eall);
  }
  if (do_fwd) throw_status(dev, dyb200_sum_all(m.errs, (size_t)T * B, loss_dev, 0, dev.ctx));

  // ---------------- backward ----------------
  if (do_fwd) CU(cudaMemsetAsync(m.dact, 0, m.dact_bytes, st));
  Tensor tgR(Dim({V, H}), m.g[1 + 3 * L]), tgbias(Dim({V}), m.g[2 + 3 * L]);
  if (do_fwd && c.fused) {
    Tensor tones(Dim({1}, TB), m.ones), tdr(Dim({V}, TB), m.dr), tdhall(Dim({H}, TB), m.dh + at(0, L - 1) * HB);
    // PickNegLogSoftmax backward and the three AffineTransform backward calls (dbias += sum_columns dr, dR += dr h^T,
    // dh += R^T dr) in one: dr is written straight into the operand layouts of the two products
    dyb200_tensor cr = to_c(rall), ch = to_c(hall), cR = to_c(tR), cones = to_c(tones), cdr = to_c(tdr);
    dyb200_tensor cgb = to_c(tgbias), cgR = to_c(tgR), cdh = to_c(tdhall);
    throw_status(dev, dyb200_softmax_output_bwd_fused(&cr, &ch, &cR, &cones, m.aux, &cgR, &cgb, &cdh, &cdr, DYB200_GEMM_A_IS_PARAM, dev.ctx));
  }
  Tensor tones(Dim({1}, B), m.ones);
  const uint32_t pass0 = phase < 0 ? 0u : (phase == 0 ? L : (uint32_t)phase - 1), pass1 = phase < 0 ? (layer_major ? L : 1u) : (phase == 0 ? L : (uint32_t)phase);
  for (uint32_t pass = pass0; pass < pass1; ++pass) {
  if (layer_major) {
    // One call per layer, top layer first: dE/dh of all its steps is complete (output layer, or the layer above), and the
    // steps T-1 .. 1 run inside one kernel whose CTAs hand dE/dh_{t-1} over on the device (dyb200_vanilla_lstm_seq_bwd; it
    // makes the per-step calls itself when the shape does not allow that).
    const uint32_t l = L - 1 - pass, I = l == 0 ? E : H;
    Tensor xall(Dim({I}, TB), l == 0 ? m.x : m.hs + at(0, l - 1) * HB);
    Tensor gall(Dim({4 * H}, TB), m.gates + at(0, l) * GB), call(Dim({H}, TB), m.cs + at(0, l) * HB), hall_l(Dim({H}, TB), m.hs + at(0, l) * HB);
    Tensor dhall(Dim({H}, TB), m.dh + at(0, l) * HB), dcall(Dim({H}, TB), m.dc + at(0, l) * HB);
    Tensor dxall(Dim({I}, TB), l == 0 ? m.dx : m.dh + at(0, l - 1) * HB);
    Tensor tWx(Dim({4 * H, I}), m.p[1 + 3 * l]), tWh(Dim({4 * H, H}), m.p[2 + 3 * l]);
    Tensor gWx(Dim({4 * H, I}), m.g[1 + 3 * l]), gWh(Dim({4 * H, H}), m.g[2 + 3 * l]), gb(Dim({4 * H}), m.g[3 + 3 * l]);
    Tensor mxl(Dim({I}, B), c.dropout ? const_cast<float*>(masks[2 * l]) : nullptr), mhl(Dim({H}, B), c.dropout ? const_cast<float*>(masks[2 * l + 1]) : nullptr);
    dyb200_tensor cxa = to_c(xall), ch0 = to_c(tZero), cc0 = to_c(tZero), cWx = to_c(tWx), cWh = to_c(tWh), cmx = to_c(mxl), cmh = to_c(mhl),
                  cg = to_c(gall), cc = to_c(call), ch = to_c(hall_l), cdh = to_c(dhall), cdc = to_c(dcall), cdx = to_c(dxall),
                  cgWx = to_c(gWx), cgWh = to_c(gWh), cgb = to_c(gb);
    dyb200_lstm_gates_attrs at = {c.dropout ? 1 : 0, 0.f, 1.f};
    throw_status(dev, dyb200_vanilla_lstm_seq_bwd(&cxa, &ch0, &cc0, &cWx, &cWh, c.dropout ? &cmx : nullptr, c.dropout ? &cmh : nullptr, &at,
                                                  &cg, &cc, &ch, &cdh, &cdc, &cdx, &cgWx, &cgWh, &cgb, m.wg_layer[l], T, dev.ctx));
  } else
  for (uint32_t tt = T; tt-- > 0;) {
    if (!c.fused) {
      Tensor rt(Dim({V}, B), m.r + tt * VB), et(Dim({1}, B), m.errs + (size_t)tt * B), tdr(Dim({V}, B), m.dr);
      Tensor htop(Dim({H}, B), m.hs + at(tt, L - 1) * HB), tdhtop(Dim({H}, B), m.dh + at(tt, L - 1) * HB);
      CU(cudaMemsetAsync(m.dr, 0, VB * sizeof(float), st));
      pnls.aux_mem = m.aux + (size_t)tt * 3 * B;
      pnls.backward_dev_impl(dev, {&rt}, et, tones, 0, tdr);
      affine.backward_dev_impl(dev, {&tbias, &tR, &htop}, rt, tdr, 0, tgbias);   // dbias += sum_b dr
      affine.backward_dev_impl(dev, {&tbias, &tR, &htop}, rt, tdr, 1, tgR);      // dR += dr h^T
      affine.backward_dev_impl(dev, {&tbias, &tR, &htop}, rt, tdr, 2, tdhtop);   // dh += R^T dr
    }
    for (uint32_t l = layer_major ? L - pass : L; l-- > (layer_major ? L - pass - 1 : 0u);) {
      size_t idx = at(tt, l);
      Tensor store[7];
      std::vector<const Tensor*> xs;
      layer_xs(tt, l, store, xs);
      Tensor tg(Dim({4 * H}, B), m.gates + idx * GB), tc(Dim({H}, B), m.cs + idx * HB), th(Dim({H}, B), m.hs + idx * HB);
      Tensor tdh(Dim({H}, B), m.dh + idx * HB), tdc(Dim({H}, B), m.dc + idx * HB), tdg(Dim({4 * H}, B), m.dgates + idx * GB);
      Tensor cprev = tt == 0 ? tZero : Tensor(Dim({H}, B), m.cs + at(tt - 1, l) * HB);
      if (c.fused) {
        uint32_t I2 = l == 0 ? E : H;
        Tensor tdin2(Dim({I2}, B), l == 0 ? m.dx + tt * EB : m.dh + at(tt, l - 1) * HB);
        Tensor tdhp2(Dim({H}, B), tt > 0 ? m.dh + at(tt - 1, l) * HB : nullptr);
        Tensor tdcp2(Dim({H}, B), tt > 0 ? m.dc + at(tt - 1, l) * HB : nullptr);
        Tensor gWx2(Dim({4 * H, I2}), m.g[1 + 3 * l]), gWh2(Dim({4 * H, H}), m.g[2 + 3 * l]), gb2(Dim({4 * H}), m.g[3 + 3 * l]);
        dyb200_tensor cx = to_c(store[0]), chp = to_c(store[1]), ccp = to_c(cprev), cWx = to_c(store[2]), cWh = to_c(store[3]), cmx, cmh,
                      cg = to_c(tg), cc = to_c(tc), cdh = to_c(tdh), cdc = to_c(tdc), cdx = to_c(tdin2), cdhp = to_c(tdhp2),
                      cdcp = to_c(tdcp2), cgWx = to_c(gWx2), cgWh = to_c(gWh2), cgb = to_c(gb2);
        if (c.dropout) { cmx = to_c(store[5]); cmh = to_c(store[6]); }
        dyb200_lstm_gates_attrs at = {c.dropout ? 1 : 0, 0.f, 1.f};
        throw_status(dev, dyb200_vanilla_lstm_bwd_fused_at(&cx, &chp, &ccp, &cWx, &cWh, c.dropout ? &cmx : nullptr, c.dropout ? &cmh : nullptr,
                                                           &cg, &cc, &cdh, &cdc, &cdx, tt > 0 ? &cdhp : nullptr, tt > 0 ? &cdcp : nullptr,
                                                           &cgWx, &cgWh, &cgb, &at, m.wg_layer[l], tt * B, dev.ctx));
        continue;
      }
      h_node.backward_dev_impl(dev, {&tc, &tg}, th, tdh, 0, tdc);
      h_node.backward_dev_impl(dev, {&tc, &tg}, th, tdh, 1, tdg);
      if (tt > 0) {
        Tensor tdcp(Dim({H}, B), m.dc + at(tt - 1, l) * HB);
        c_node.backward_dev_impl(dev, {&cprev, &tg}, tc, tdc, 0, tdcp);
      }
      c_node.backward_dev_impl(dev, {&cprev, &tg}, tc, tdc, 1, tdg);
      uint32_t I = l == 0 ? E : H;
      Tensor tdin(Dim({I}, B), l == 0 ? m.dx + tt * EB : m.dh + at(tt, l - 1) * HB);
      gates_node.backward_dev_impl(dev, xs, tg, tdg, 0, tdin);
      if (tt > 0) {
        Tensor tdhp(Dim({H}, B), m.dh + at(tt - 1, l) * HB);
        gates_node.backward_dev_impl(dev, xs, tg, tdg, 1, tdhp);
      }
      Tensor gWx(Dim({4 * H, I}), m.g[1 + 3 * l]), gWh(Dim({4 * H, H}), m.g[2 + 3 * l]), gb(Dim({4 * H}), m.g[3 + 3 * l]);
      gates_node.backward_dev_impl(dev, xs, tg, tdg, 2, gWx);
      gates_node.backward_dev_impl(dev, xs, tg, tdg, 3, gWh);
      gates_node.backward_dev_impl(dev, xs, tg, tdg, 4, gb);
    }
  }
    // the deferred weight-gradient products of the layer whose reverse pass just ended: one per parameter matrix, K = T * B
    if (layer_major) {
      const uint32_t l = L - 1 - pass;
      throw_status(dev, dyb200_wgrad_flush(m.wg_layer[l], m.g[1 + 3 * l], 4 * H, m.g[2 + 3 * l], 4 * H, dev.ctx));
    }
  }
  if (phase >= 0 && (uint32_t)phase != L) return;
  Tensor tgC(Dim({E}, V), m.g[0]);
  if (c.fused) {
    if (!layer_major)
      for (uint32_t l = 0; l < L; ++l)
        throw_status(dev, dyb200_wgrad_flush(m.wg_layer[l], m.g[1 + 3 * l], 4 * H, m.g[2 + 3 * l], 4 * H, dev.ctx));
    // All T lookups share the table, so their accumulate_grads calls fold into one over the T*B ids in time
    // order: each table row still receives its rows in the order of the per-step calls.
    LookupNode look(tC, nullptr, T * B);
    look.aux_mem = m.tok;
    Tensor tdx(Dim({E}, T * B), m.dx);
    look.accumulate_grad(dev, tdx, tgC);
  } else {
    for (uint32_t t = 0; t < T; ++t) {
      LookupNode look(tC, nullptr, B);
      look.aux_mem = m.tok + (size_t)t * B;
      Tensor tdx(Dim({E}, B), m.dx + t * EB);
      look.accumulate_grad(dev, tdx, tgC);
    }
  }
}

void forward_backward(Lm& m, const uint32_t* tokens, int on_device, const float* const* masks, float* loss_dev, int phase = -1) {
  const dyb200h_lm_config& c = m.c;
  cudaStream_t st = m.stream;
  if (phase > (int)c.L) throw std::invalid_argument("phase out of range");
  if (c.dropout && !masks) throw std::invalid_argument("dropout is on but no masks were given");
  if (phase <= 0)
    CU(cudaMemcpyAsync(m.tok, tokens, (size_t)(c.T + 1) * c.B * sizeof(uint32_t), on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, st));
  if (!m.use_graph) { step_body(m, masks, loss_dev, phase); return; }

  // graph mode: masks are staged into the driver's own buffers so that the captured kernels see fixed addresses
  std::vector<const float*> fixed;
  if (c.dropout) {
    for (uint32_t l = 0; l < c.L; ++l)
      for (int k = 0; k < 2; ++k) {
        float* dst = m.mask_buf[2 * l + k];
        size_t n = (size_t)(k == 0 ? (l == 0 ? c.E : c.H) : c.H) * c.B;
        if (phase <= 0 && masks[2 * l + k] != dst) CU(cudaMemcpyAsync(dst, masks[2 * l + k], n * sizeof(float), cudaMemcpyDeviceToDevice, st));
        fixed.push_back(dst);
      }
  }
  if (m.graph_loss != loss_dev) m.drop_graphs();
  if (m.graph_exec.size() < c.L + 2) m.graph_exec.resize(c.L + 2, nullptr);
  cudaGraphExec_t& gexec = m.graph_exec[phase + 1];
  if (!gexec) {
    if (st == nullptr) throw std::runtime_error("graph mode needs a non-default stream (the legacy stream cannot be captured)");
    uint64_t l0 = dyb200_ctx_launch_count(m.dev.ctx);
    // The launches that split the weights into operand planes are issued only when the parameter cache is stale, a
    // decision taken on the host while capturing.  Marking the cache stale here puts them into every graph, whatever
    // happened before the capture, so a replay after an update never multiplies with the planes of old weights.
    dyb200_ctx_params_changed(m.dev.ctx);
    CU(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    cudaGraph_t graph = nullptr;
    try {
      step_body(m, c.dropout ? fixed.data() : nullptr, loss_dev, phase);
    } catch (...) {
      cudaStreamEndCapture(st, &graph);
      if (graph) cudaGraphDestroy(graph);
      throw;
    }
    CU(cudaStreamEndCapture(st, &graph));
    cudaError_t e = cudaGraphInstantiate(&gexec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) throw cuda_exception(std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
    m.graph_loss = loss_dev;
    if (phase <= 0) m.graph_launches = 0;
    m.graph_launches += dyb200_ctx_launch_count(m.dev.ctx) - l0;
  }
  CU(cudaGraphLaunch(gexec, st));
}

}  // namespace

extern "C" {

size_t dyb200h_lm_num_params(const dyb200h_lm_config* c) { return param_sizes(*c, nullptr); }
size_t dyb200h_lm_workspace_bytes(const dyb200h_lm_config* c) { return plan(*c, nullptr, nullptr, 0); }
// Offsets (in floats) of the 3L+3 parameter tensors inside the flat buffer; returns their count.
int dyb200h_lm_param_offsets(const dyb200h_lm_config* c, size_t* offsets, size_t* sizes, int cap) {
  std::vector<size_t> sz;
  param_sizes(*c, &sz);
  size_t off = 0;
  for (size_t k = 0; k < sz.size() && (int)k < cap; ++k) { offsets[k] = off; sizes[k] = sz[k]; off += sz[k]; }
  return (int)sz.size();
}

int dyb200h_lm_create(const dyb200h_lm_config* c, float* params, float* grads, void* workspace, size_t ws_bytes,
                      dyb200_ctx* ctx, void* stream, void** out) {
  if (!c || !params || !grads || !workspace || !ctx || !out) return DYB200_EINVAL;
  if (ws_bytes < plan(*c, nullptr, nullptr, 0)) return DYB200_ENOMEM;
  Lm* m = new Lm();
  m->c = *c;
  m->dev.ctx = ctx;
  m->params = params;
  m->grads = grads;
  m->stream = (cudaStream_t)stream;
  std::vector<size_t> sz;
  param_sizes(*c, &sz);
  size_t off = 0;
  for (size_t n : sz) { m->p.push_back(params + off); m->g.push_back(grads + off); off += n; }
  plan(*c, m, (char*)workspace, ws_bytes);
  // this driver owns the parameter updates (dyb200h_lm_update -> dyb200_sgd_update), so the packed
  // copies of the weights can be reused across the time steps of a training step
  dyb200_ctx_param_cache(ctx, 1);
  // Programmatic dependent launch measured no gain for this step (the graph replay already chains the kernels
  // tightly: 5.95 vs 6.00 ms at batch 64, 19.9 vs 20.1 ms at batch 512), so this driver leaves it as the caller set it
  // on the context (dyb200_ctx_dependent_launch; off by default).
  int rc = DYB200_OK;
  if (c->fused) {
    for (uint32_t l = 0; l < c->L && !rc; ++l) {
      dyb200_wgrad* w = nullptr;
      rc = dyb200_wgrad_create(ctx, 4 * c->H, l == 0 ? c->E : c->H, c->H, c->T * c->B, &w);
      if (!rc) m->wg_layer.push_back(w);
    }

    if (rc) { delete m; return rc; }
  }
  rc = dyb200_fill(m->zeros, (size_t)c->H * c->B, 0.f, ctx);
  if (!rc) rc = dyb200_fill(m->ones, (size_t)c->T * c->B, 1.f, ctx);
  if (rc) { delete m; return rc; }
  *out = m;
  return DYB200_OK;
}

void dyb200h_lm_destroy(void* h) { delete (Lm*)h; }
const char* dyb200h_lm_error(void* h) { return h ? ((Lm*)h)->err.c_str() : "null handle"; }

static int guarded(Lm* m, void (*fn)(Lm&, void*), void* arg) {
  try {
    fn(*m, arg);
    return DYB200_OK;
  } catch (const std::invalid_argument& e) { m->err = e.what(); return DYB200_EINVAL;
  } catch (const out_of_memory& e) { m->err = e.what(); return DYB200_ENOMEM;
  } catch (const cuda_exception& e) { m->err = e.what(); return DYB200_ECUDA;
  } catch (const std::exception& e) { m->err = e.what(); return DYB200_ERUNTIME; }
}

struct FbArgs { const uint32_t* tokens; int on_device; const float* const* masks; float* loss_dev; int phase; };

// tokens: (T+1) x B ids (host, or device when tokens_on_device); masks: 2L device pointers
// {mask_x_0, mask_h_0, mask_x_1, ...} each I_l x B / H x B, or NULL when dropout is off;
// loss_dev: device scalar that receives sum_batches(sum_t err_t).  Gradients accumulate into `grads`.
int dyb200h_lm_forward_backward(void* h, const uint32_t* tokens, int tokens_on_device, const float* const* masks,
                                float* loss_dev) {
  FbArgs a{tokens, tokens_on_device, masks, loss_dev, -1};
  return guarded((Lm*)h, [](Lm& m, void* p) {
    FbArgs* a = (FbArgs*)p;
    forward_backward(m, a->tokens, a->on_device, a->masks, a->loss_dev, a->phase);
  }, &a);
}

// The same step in pieces, for a data-parallel caller that reduces gradients while the backward pass still runs (fused
// layer-by-layer driver only).  dyb200h_lm_num_phases returns L + 1, or 1 when the driver cannot split the step.  Call the
// phases 0 .. L in order with the same arguments; after phase p the gradients of the tensors dyb200h_lm_phase_grad_range
// names are final: phase 0 -> R and bias (the tail of the flat buffer), phase p (0 < p < L) -> Wx, Wh, b of layer L - p,
// phase L -> the embedding table and layer 0 (the head of the buffer).  Results are those of dyb200h_lm_forward_backward.
int dyb200h_lm_num_phases(void* h) {
  Lm* m = (Lm*)h;
  return (m->c.fused && !m->time_major) ? (int)m->c.L + 1 : 1;
}
int dyb200h_lm_phase_grad_range(void* h, int phase, size_t* offset, size_t* count) {
  Lm* m = (Lm*)h;
  const uint32_t L = m->c.L;
  if (phase < 0 || phase > (int)L || !offset || !count) return DYB200_EINVAL;
  std::vector<size_t> sz;
  param_sizes(m->c, &sz);
  std::vector<size_t> off(sz.size() + 1, 0);
  for (size_t k = 0; k < sz.size(); ++k) off[k + 1] = off[k] + sz[k];
  size_t first, last;   // tensor indices [first, last)
  if (phase == 0) { first = 1 + 3 * L; last = 3 + 3 * L; }
  else if ((uint32_t)phase == L) { first = 0; last = 4; }
  else { first = 1 + 3 * (L - phase); last = first + 3; }
  *offset = off[first];
  *count = off[last] - off[first];
  return DYB200_OK;
}
int dyb200h_lm_forward_backward_phase(void* h, int phase, const uint32_t* tokens, int tokens_on_device, const float* const* masks,
                                      float* loss_dev) {
  Lm* m = (Lm*)h;
  if (phase < 0 || phase >= dyb200h_lm_num_phases(h)) { m->err = "phase out of range"; return DYB200_EINVAL; }
  FbArgs a{tokens, tokens_on_device, masks, loss_dev, dyb200h_lm_num_phases(h) == 1 ? -1 : phase};
  return guarded(m, [](Lm& mm, void* p) {
    FbArgs* a = (FbArgs*)p;
    forward_backward(mm, a->tokens, a->on_device, a->masks, a->loss_dev, a->phase);
  }, &a);
}

// Squared L2 norm of the local gradients into a device scalar (reduce it over ranks before update).
int dyb200h_lm_grad_sumsq(void* h, float** scalar_dev_out) {
  Lm* m = (Lm*)h;
  size_t n = param_sizes(m->c, nullptr);
  int rc = dyb200_squared_norm(m->grads, n, m->scalars, 0, m->dev.ctx);
  if (rc) { m->err = dyb200_last_error(m->dev.ctx); return rc; }
  if (scalar_dev_out) *scalar_dev_out = m->scalars;
  return DYB200_OK;
}

// SimpleSGD update with gradient clipping from the scalar computed by dyb200h_lm_grad_sumsq; zeroes the gradients.
int dyb200h_lm_update(void* h) {
  Lm* m = (Lm*)h;
  size_t n = param_sizes(m->c, nullptr);
  int rc = dyb200_sgd_update(m->params, m->grads, n, m->c.lr, m->c.clip, m->scalars, m->dev.ctx);
  if (rc) m->err = dyb200_last_error(m->dev.ctx);
  return rc;
}

// Graph mode: capture forward + backward once (on the next call) and replay it afterwards.  Call it after at least one
// eager step (scratch arena and parameter cache at their final sizes) and only with a non-default stream; while it is on,
// the library's per-launch GEMM timing must be off.  Returns the kernels per replay through dyb200h_lm_graph_launches.
int dyb200h_lm_set_graph(void* h, int enable) {
  Lm* m = (Lm*)h;
  m->use_graph = enable != 0;
  if (!enable) m->drop_graphs();
  return DYB200_OK;
}
uint64_t dyb200h_lm_graph_launches(void* h) { return ((Lm*)h)->graph_launches; }
// Fused driver only: 1 = run the (time step, layer) calls time step by time step, as the reference's graph orders them;
// 0 (default) = layer by layer.  Same values either way; drops a captured graph.
int dyb200h_lm_set_time_major(void* h, int enable) {
  Lm* m = (Lm*)h;
  m->time_major = enable != 0;
  m->drop_graphs();
  return DYB200_OK;
}
// Device pointers of the 2L mask buffers the graph reads (write the masks there to avoid the staging copy).
int dyb200h_lm_mask_buffers(void* h, float** out, int cap) {
  Lm* m = (Lm*)h;
  int n = (int)m->mask_buf.size();
  for (int k = 0; k < n && k < cap; ++k) out[k] = m->mask_buf[k];
  return n;
}

// Device pointer of the hidden states h[t][l] (T x L x H x B), for parity checks.
const float* dyb200h_lm_hidden_states(void* h) { return ((Lm*)h)->hs; }

}  // extern "C"
