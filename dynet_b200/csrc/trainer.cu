// Trainer update rules as one pass over a flat parameter buffer, with gradient clipping folded in.
//   Trainer::clip_gradients          dynet/training.cc:168-183
//   SimpleSGD / CyclicalSGD rule     dynet/training.cc:619-622, :646-649
//   MomentumSGD                      dynet/training.cc:669-673
//   Adagrad                          dynet/training.cc:735-739
//   Adadelta                         dynet/training.cc:802-808
//   RMSProp                          dynet/training.cc:883-888
//   Adam                             dynet/training.cc:955-961
//   Amsgrad                          dynet/training.cc:1034-1041
// The reference runs 1-5 Eigen kernels per parameter per rule and copies one norm per parameter to the host
// when clipping; here the squared gradient norm stays on the device (dyb200_squared_norm) and one kernel
// applies clip scale, rule, weight-decay divisor and the clearing of the gradient
// (ParameterStorage::clear, dynet/model.cc:111-117).
#include "common.cuh"

namespace {

constexpr int kBlock = 256;

struct RuleArgs {
  float* p; float* g; float* s0; float* s1; float* s2;
  size_t n;
  dyb200_trainer_hyper h;
  float lr_t;            // Adam / Amsgrad: learning rate with both bias corrections and the weight-decay divisor
  const float* sumsq;    // squared global gradient norm (device), or null: no clipping
  int zero_grads;
};

template <int RULE>
__device__ __forceinline__ void apply(float& p, float& g, float& s0, float& s1, float& s2, const dyb200_trainer_hyper& h,
                                      float gscale, float lr_t) {
  const float wd = h.weight_decay;
  if (RULE == DYB200_RULE_SGD) {
    p -= g * (h.learning_rate * gscale / wd);
  } else if (RULE == DYB200_RULE_MOMENTUM) {
    s0 = s0 * h.momentum - g * (h.learning_rate * gscale);
    p += s0 / wd;
  } else if (RULE == DYB200_RULE_ADAGRAD) {
    g = g * gscale;
    s0 += g * g;
    p += g / sqrtf(s0 + h.epsilon) * (-h.learning_rate / wd);
  } else if (RULE == DYB200_RULE_ADADELTA) {
    g = g * gscale;
    s0 = s0 * h.rho + g * g * (1.f - h.rho);
    g = -g * sqrtf(s1 + h.epsilon) / sqrtf(s0 + h.epsilon);
    s1 = s1 * h.rho + g * g * (1.f - h.rho);
    p += g / wd;
  } else if (RULE == DYB200_RULE_RMSPROP) {
    g = g * gscale;
    s0 = s0 * h.rho + g * g * (1.f - h.rho);
    g = -g / sqrtf(s0 + h.epsilon);
    p += h.learning_rate * g / wd;
  } else if (RULE == DYB200_RULE_ADAM) {
    g = g * gscale;
    s0 = s0 * h.beta_1 + g * (1.f - h.beta_1);
    s1 = s1 * h.beta_2 + g * g * (1.f - h.beta_2);
    p -= s0 / (sqrtf(s1) + h.epsilon) * lr_t;
  } else {   // DYB200_RULE_AMSGRAD
    g = g * gscale;
    s0 = s0 * h.beta_1 + g * (1.f - h.beta_1);
    s1 = s1 * h.beta_2 + g * g * (1.f - h.beta_2);
    s2 = fmaxf(s2, s1);
    p -= s0 / (sqrtf(s2) + h.epsilon) * lr_t;
  }
}

template <int RULE> struct NStates { static constexpr int v = RULE == DYB200_RULE_SGD ? 0 : (RULE == DYB200_RULE_MOMENTUM || RULE == DYB200_RULE_ADAGRAD || RULE == DYB200_RULE_RMSPROP) ? 1 : RULE == DYB200_RULE_AMSGRAD ? 3 : 2; };

template <int RULE>
__global__ void __launch_bounds__(kBlock) k_trainer_update(const RuleArgs a) {
  dyb_grid_dep_sync();
  float gscale = 1.f;
  if (a.sumsq && a.h.clip_threshold > 0.f) {
    const float gg = sqrtf(a.sumsq[0]);
    if (gg > a.h.clip_threshold) gscale = a.h.clip_threshold / gg;
  }
  constexpr int NS = NStates<RULE>::v;
  bool vec = aligned16(a.p) && aligned16(a.g) && (NS < 1 || aligned16(a.s0)) && (NS < 2 || aligned16(a.s1)) && (NS < 3 || aligned16(a.s2));
  const size_t n4 = vec ? a.n / 4 : 0;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n4; i += (size_t)gridDim.x * kBlock) {
    float4 p = ld4(a.p + 4 * i), g = ld4(a.g + 4 * i);
    float4 s0 = NS >= 1 ? ld4(a.s0 + 4 * i) : zero4, s1 = NS >= 2 ? ld4(a.s1 + 4 * i) : zero4, s2 = NS >= 3 ? ld4(a.s2 + 4 * i) : zero4;
    apply<RULE>(p.x, g.x, s0.x, s1.x, s2.x, a.h, gscale, a.lr_t);
    apply<RULE>(p.y, g.y, s0.y, s1.y, s2.y, a.h, gscale, a.lr_t);
    apply<RULE>(p.z, g.z, s0.z, s1.z, s2.z, a.h, gscale, a.lr_t);
    apply<RULE>(p.w, g.w, s0.w, s1.w, s2.w, a.h, gscale, a.lr_t);
    st4(a.p + 4 * i, p);
    if (NS >= 1) st4(a.s0 + 4 * i, s0);
    if (NS >= 2) st4(a.s1 + 4 * i, s1);
    if (NS >= 3) st4(a.s2 + 4 * i, s2);
    if (a.zero_grads) st4(a.g + 4 * i, zero4);
    else if (RULE != DYB200_RULE_SGD && RULE != DYB200_RULE_MOMENTUM) st4(a.g + 4 * i, g);   // these rules rewrite the gradient
  }
  for (size_t i = 4 * n4 + (size_t)blockIdx.x * kBlock + threadIdx.x; i < a.n; i += (size_t)gridDim.x * kBlock) {
    float p = a.p[i], g = a.g[i];
    float s0 = NS >= 1 ? a.s0[i] : 0.f, s1 = NS >= 2 ? a.s1[i] : 0.f, s2 = NS >= 3 ? a.s2[i] : 0.f;
    apply<RULE>(p, g, s0, s1, s2, a.h, gscale, a.lr_t);
    a.p[i] = p;
    if (NS >= 1) a.s0[i] = s0;
    if (NS >= 2) a.s1[i] = s1;
    if (NS >= 3) a.s2[i] = s2;
    if (a.zero_grads) a.g[i] = 0.f;
    else if (RULE != DYB200_RULE_SGD && RULE != DYB200_RULE_MOMENTUM) a.g[i] = g;
  }
}

template <int RULE>
int launch(dyb200_ctx* ctx, const RuleArgs& a) {
  dyb_launch(k_trainer_update<RULE>, stream_grid(ctx, a.n / 4 + 1, kBlock * 2), kBlock, 0, ctx, a);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

}  // namespace

extern "C" int dyb200_trainer_update(int rule, float* params, float* grads, float* state0, float* state1, float* state2, size_t n,
                                     const dyb200_trainer_hyper* hyper, const float* grad_sumsq, int zero_grads, dyb200_ctx* ctx) {
  if (n == 0) return DYB200_OK;
  DYB_CHECK_ARG(ctx, params && grads && hyper, "trainer_update: null pointer");
  DYB_CHECK_ARG(ctx, rule >= DYB200_RULE_SGD && rule <= DYB200_RULE_AMSGRAD, "trainer_update: unknown rule %d", rule);
  DYB_CHECK_ARG(ctx, hyper->weight_decay > 0.f, "trainer_update: the weight-decay divisor must be positive (1 when unused)");
  const int ns = rule == DYB200_RULE_SGD ? 0 : (rule == DYB200_RULE_MOMENTUM || rule == DYB200_RULE_ADAGRAD || rule == DYB200_RULE_RMSPROP) ? 1
                 : rule == DYB200_RULE_AMSGRAD ? 3 : 2;
  DYB_CHECK_ARG(ctx, (ns < 1 || state0) && (ns < 2 || state1) && (ns < 3 || state2), "trainer_update: rule %d needs %d state buffers", rule, ns);
  RuleArgs a{params, grads, state0, state1, state2, n, *hyper, 0.f, grad_sumsq, zero_grads};
  if (rule == DYB200_RULE_ADAM || rule == DYB200_RULE_AMSGRAD) {
    // float lr_t = learning_rate * sqrt(1 - beta_2^(updates+1)) / (1 - beta_1^(updates+1)) / weight_decay, in double then rounded
    const double t = (double)hyper->updates + 1.0;
    a.lr_t = (float)(hyper->learning_rate * sqrt(1.0 - pow((double)hyper->beta_2, t)) / (1.0 - pow((double)hyper->beta_1, t)) / hyper->weight_decay);
  }
  int rc;
  switch (rule) {
    case DYB200_RULE_SGD: rc = launch<DYB200_RULE_SGD>(ctx, a); break;
    case DYB200_RULE_MOMENTUM: rc = launch<DYB200_RULE_MOMENTUM>(ctx, a); break;
    case DYB200_RULE_ADAGRAD: rc = launch<DYB200_RULE_ADAGRAD>(ctx, a); break;
    case DYB200_RULE_ADADELTA: rc = launch<DYB200_RULE_ADADELTA>(ctx, a); break;
    case DYB200_RULE_RMSPROP: rc = launch<DYB200_RULE_RMSPROP>(ctx, a); break;
    case DYB200_RULE_ADAM: rc = launch<DYB200_RULE_ADAM>(ctx, a); break;
    default: rc = launch<DYB200_RULE_AMSGRAD>(ctx, a); break;
  }
  if (rc) return rc;
  ctx->param_version++;   // packed copies of the parameters in the cache are stale now
  return DYB200_OK;
}
