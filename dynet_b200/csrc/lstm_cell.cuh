// Backward arithmetic of one LSTM cell element, shared by the per-step cell pass (lstm.cu) and the sequence kernel
// (lstm_seq_bwd.cu).  Every operation is written as an explicit round-to-nearest intrinsic so that both kernels round
// identically wherever the compiler inlines this (no context-dependent multiply-add contraction).
//   VanillaLSTMH backward  (dynet/nodes-lstm.cc:530-580): dc  = dh o (1 - tanh(c)^2) [+ dE/dc],  do_pre = dh tanh(c) o (1 - o)
//   VanillaLSTMC backward  (dynet/nodes-lstm.cc:415-470): dc_prev += dc f,  di_pre = dc g i (1 - i),  df_pre = dc c_prev f (1 - f),
//                                                         dg_pre = dc i (1 - g^2)
#pragma once

__device__ __forceinline__ float sigmoid_grad(float g, float d) { return __fmul_rn(__fmul_rn(d, g), __fsub_rn(1.f, g)); }
__device__ __forceinline__ float tanh_grad(float g, float d) { return __fmul_rn(d, __fmaf_rn(-g, g, 1.f)); }

// gi / gf / go / gg: the saved gate activations; c, cp: c_t and c_{t-1}; dh, dci: dE/dh_t and dE/dc_t (has_dc: dci is given);
// dcp: dE/dc_{t-1}, accumulated; pi / pf / po / pg: the gradients of the four pre-activations.
__device__ __forceinline__ void lstm_cell_grad(float gi, float gf, float go, float gg, float c, float cp, float dh, float dci,
                                               bool has_dc, float& dcp, float& pi, float& pf, float& po, float& pg) {
  const float t = tanhf(c);
  float dc = __fmul_rn(__fmul_rn(dh, go), __fmaf_rn(-t, t, 1.f));
  if (has_dc) dc = __fadd_rn(dc, dci);
  dcp = __fmaf_rn(dc, gf, dcp);
  pi = sigmoid_grad(gi, __fmul_rn(dc, gg));
  pf = sigmoid_grad(gf, __fmul_rn(dc, cp));
  po = sigmoid_grad(go, __fmul_rn(dh, t));
  pg = tanh_grad(gg, __fmul_rn(dc, gi));
}
