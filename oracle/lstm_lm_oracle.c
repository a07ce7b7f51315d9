/*
 * CPU oracle for one training step of the batched LSTM language model:
 * TEST INFRASTRUCTURE ONLY (parity checker and timed CPU baseline).
 *
 * Graph: examples/batching/rnnlm-batch.h:110-151 over a CompactVanillaLSTMBuilder
 * (dynet/lstm.cc:1044-1080), i.e. per time step
 *   x = lookup(C, tok[t-1]); per layer: gates -> c -> h (fused LSTM nodes);
 *   r = bias + R * h; err_t = pickneglogsoftmax(r, tok[t]);
 * loss = sum_batches(sum_t err_t).  Backward visits the nodes in reverse order
 * and accumulates (+=) into every gradient, as dynet/exec.cc:166-284 does; the
 * lookup gradients are scattered after the reverse pass in time order
 * (exec.cc:277-282).  Dropout masks are inputs (the reference draws them with a
 * CPU RNG that no GPU run can reproduce, dynet/tensor.cc:261-265).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* node-level oracle functions from dynet_oracle.c */
int orc_lookup_fwd(const float*, uint32_t, uint32_t, const uint32_t*, uint32_t, float, float*);
void orc_lookup_accumulate_grads(float*, uint32_t, const uint32_t*, uint32_t, const float*);
void orc_lstm_gates_fwd(const float* const*, const uint32_t*, unsigned, const float*, const float*,
                        const float*, const float*, const float*, uint32_t, const float*, uint32_t,
                        uint32_t, uint32_t, uint32_t, float, int, int, float*);
void orc_lstm_gates_bwd(const float* const*, const uint32_t*, unsigned, const float*, const float*,
                        const float*, const float*, uint32_t, const float*, uint32_t, uint32_t,
                        uint32_t, uint32_t, const float*, const float*, unsigned, float*);
void orc_lstm_c_fwd(const float*, const float*, uint32_t, uint32_t, float*);
void orc_lstm_c_bwd(const float*, const float*, uint32_t, uint32_t, const float*, unsigned, float*);
void orc_lstm_h_fwd(const float*, const float*, uint32_t, uint32_t, float*);
void orc_lstm_h_bwd(const float*, const float*, uint32_t, uint32_t, const float*, unsigned, float*);
int orc_pnls_fwd(const float*, uint32_t, uint32_t, const uint32_t*, float*, float*, float*);
void orc_pnls_bwd(const float*, uint32_t, uint32_t, const uint32_t*, const float*, const float*, float*);
void orc_gemm_nn_acc(const float*, const float*, float*, size_t, size_t, size_t);
void orc_gemm_tn_acc(const float*, const float*, float*, size_t, size_t, size_t);
void orc_gemm_nt_acc(const float*, const float*, float*, size_t, size_t, size_t);

typedef struct {
  uint32_t V, E, H, L, T, B;
} orc_lm_dims;

/* Parameter / gradient block, one pointer per tensor:
 *   p[0] = C (E x V), then per layer l: p[1+3l] = Wx (4H x I_l), p[2+3l] = Wh (4H x H),
 *   p[3+3l] = b (4H); p[1+3L] = R (V x H); p[2+3L] = bias (V).
 * tokens: (T+1) x B, tokens[t*B + b].  masks: per layer mask_x (I_l x B), mask_h
 * (H x B), or NULL for no dropout.  h_out (optional): T x L x H x B hidden states.
 * Returns 0, or -1 for an out-of-range token id. */
ORC_API int orc_lstm_lm_fwdbwd(const orc_lm_dims* d, const float* const* p, float* const* g,
                               const uint32_t* tokens, const float* const* mask_x,
                               const float* const* mask_h, float* loss_out, float* h_out) {
  const uint32_t V = d->V, E = d->E, H = d->H, L = d->L, T = d->T, B = d->B;
  const size_t HB = (size_t)H * B, GB = (size_t)4 * H * B, VB = (size_t)V * B, EB = (size_t)E * B;
  const float* C = p[0];
  const float* R = p[1 + 3 * L];
  const float* bias = p[2 + 3 * L];
  int rc = 0;

  float* x = (float*)malloc(T * EB * sizeof(float));
  float* gates = (float*)malloc((size_t)T * L * GB * sizeof(float));
  float* cs = (float*)malloc((size_t)T * L * HB * sizeof(float));
  float* hs = (float*)malloc((size_t)T * L * HB * sizeof(float));
  float* r = (float*)malloc((size_t)T * VB * sizeof(float));
  float* z = (float*)malloc((size_t)T * B * sizeof(float));
  float* m = (float*)malloc((size_t)B * sizeof(float));
  float* err = (float*)malloc((size_t)T * B * sizeof(float));
  float* zeros = (float*)calloc(HB, sizeof(float));

  /* ---------------- forward ---------------- */
  for (uint32_t t = 0; t < T && rc == 0; ++t) {
    float* xt = x + t * EB;
    rc = orc_lookup_fwd(C, E, V, tokens + (size_t)t * B, B, 1.0f, xt);
    if (rc) break;
    const float* in = xt;
    uint32_t I = E;
    for (uint32_t l = 0; l < L; ++l) {
      size_t idx = (size_t)t * L + l;
      const float* h_prev = t == 0 ? zeros : hs + ((size_t)(t - 1) * L + l) * HB;
      const float* c_prev = t == 0 ? zeros : cs + ((size_t)(t - 1) * L + l) * HB;
      const float* ins[1] = {in};
      uint32_t idims[1] = {I};
      orc_lstm_gates_fwd(ins, idims, 1, h_prev, p[1 + 3 * l], p[2 + 3 * l], p[3 + 3 * l],
                         mask_x ? mask_x[l] : NULL, B, mask_x ? mask_h[l] : NULL, B, H, I, B,
                         1.0f, 0, 8, gates + idx * GB);
      orc_lstm_c_fwd(c_prev, gates + idx * GB, H, B, cs + idx * HB);
      orc_lstm_h_fwd(cs + idx * HB, gates + idx * GB, H, B, hs + idx * HB);
      in = hs + idx * HB;
      I = H;
    }
    /* r = bias + R * h: MatrixMultiply then CwiseSum with the batch-1 bias */
    float* rt = r + t * VB;
    memset(rt, 0, VB * sizeof(float));
    orc_gemm_nn_acc(R, in, rt, V, H, B);
    for (uint32_t b = 0; b < B; ++b)
      for (uint32_t v = 0; v < V; ++v) rt[(size_t)b * V + v] = bias[v] + rt[(size_t)b * V + v];
    rc = orc_pnls_fwd(rt, V, B, tokens + (size_t)(t + 1) * B, err + (size_t)t * B, z + (size_t)t * B, m);
  }
  if (rc == 0) {
    /* sum(errs) then sum_batches */
    float total = 0.f;
    for (uint32_t b = 0; b < B; ++b) {
      float s = 0.f;
      for (uint32_t t = 0; t < T; ++t) s += err[(size_t)t * B + b];
      total += s;
    }
    *loss_out = total;
    if (h_out) memcpy(h_out, hs, (size_t)T * L * HB * sizeof(float));
  }

  /* ---------------- backward ---------------- */
  if (rc == 0 && g) {
    float* dh = (float*)calloc((size_t)T * L * HB, sizeof(float));
    float* dc = (float*)calloc((size_t)T * L * HB, sizeof(float));
    float* dgates = (float*)malloc(GB * sizeof(float));
    float* dx = (float*)calloc(T * EB, sizeof(float));
    float* dr = (float*)malloc(VB * sizeof(float));
    float* ones = (float*)malloc(B * sizeof(float));
    for (uint32_t b = 0; b < B; ++b) ones[b] = 1.f;
    float* gR = g[1 + 3 * L];
    float* gbias = g[2 + 3 * L];
    for (uint32_t tt = T; tt-- > 0;) {
      const float* rt = r + tt * VB;
      size_t top = (size_t)tt * L + (L - 1);
      memset(dr, 0, VB * sizeof(float));
      orc_pnls_bwd(rt, V, B, tokens + (size_t)(tt + 1) * B, z + (size_t)tt * B, ones, dr);
      /* CwiseSum backward: dbias += sum_b dr (column by column); dprod = dr */
      for (uint32_t b = 0; b < B; ++b)
        for (uint32_t v = 0; v < V; ++v) gbias[v] += dr[(size_t)b * V + v];
      /* MatrixMultiply backward: dR += dr * h^T ; dh += R^T dr */
      orc_gemm_nt_acc(dr, hs + top * HB, gR, V, B, H);
      orc_gemm_tn_acc(R, dr, dh + top * HB, V, H, B);
      for (uint32_t l = L; l-- > 0;) {
        size_t idx = (size_t)tt * L + l;
        const float* h_prev = tt == 0 ? zeros : hs + ((size_t)(tt - 1) * L + l) * HB;
        const float* c_prev = tt == 0 ? zeros : cs + ((size_t)(tt - 1) * L + l) * HB;
        const float* in = l == 0 ? x + tt * EB : hs + ((size_t)tt * L + l - 1) * HB;
        uint32_t I = l == 0 ? E : H;
        const float* ins[1] = {in};
        uint32_t idims[1] = {I};
        const float* mx = mask_x ? mask_x[l] : NULL;
        const float* mh = mask_x ? mask_h[l] : NULL;
        memset(dgates, 0, GB * sizeof(float));
        /* h node: args (c_t, gates) */
        orc_lstm_h_bwd(cs + idx * HB, gates + idx * GB, H, B, dh + idx * HB, 0, dc + idx * HB);
        orc_lstm_h_bwd(cs + idx * HB, gates + idx * GB, H, B, dh + idx * HB, 1, dgates);
        /* c node: args (c_tm1, gates) */
        if (tt > 0)
          orc_lstm_c_bwd(c_prev, gates + idx * GB, H, B, dc + idx * HB, 0,
                         dc + ((size_t)(tt - 1) * L + l) * HB);
        orc_lstm_c_bwd(c_prev, gates + idx * GB, H, B, dc + idx * HB, 1, dgates);
        /* gates node: args (x, h_tm1, Wx, Wh, b) */
        float* dxin = l == 0 ? dx + tt * EB : dh + ((size_t)tt * L + l - 1) * HB;
        orc_lstm_gates_bwd(ins, idims, 1, h_prev, p[1 + 3 * l], p[2 + 3 * l], mx, B, mh, B, H, I, B,
                           gates + idx * GB, dgates, 0, dxin);
        if (tt > 0)
          orc_lstm_gates_bwd(ins, idims, 1, h_prev, p[1 + 3 * l], p[2 + 3 * l], mx, B, mh, B, H, I,
                             B, gates + idx * GB, dgates, 1, dh + ((size_t)(tt - 1) * L + l) * HB);
        orc_lstm_gates_bwd(ins, idims, 1, h_prev, p[1 + 3 * l], p[2 + 3 * l], mx, B, mh, B, H, I, B,
                           gates + idx * GB, dgates, 2, g[1 + 3 * l]);
        orc_lstm_gates_bwd(ins, idims, 1, h_prev, p[1 + 3 * l], p[2 + 3 * l], mx, B, mh, B, H, I, B,
                           gates + idx * GB, dgates, 3, g[2 + 3 * l]);
        orc_lstm_gates_bwd(ins, idims, 1, h_prev, p[1 + 3 * l], p[2 + 3 * l], mx, B, mh, B, H, I, B,
                           gates + idx * GB, dgates, 4, g[3 + 3 * l]);
      }
    }
    for (uint32_t t = 0; t < T; ++t)
      orc_lookup_accumulate_grads(g[0], E, tokens + (size_t)t * B, B, dx + t * EB);
    free(dh); free(dc); free(dgates); free(dx); free(dr); free(ones);
  }
  free(x); free(gates); free(cs); free(hs); free(r); free(z); free(m); free(err); free(zeros);
  return rc;
}

/* SimpleSGD step with DyNet's default gradient clipping (dynet/training.cc:168-183,
 * :195-224, :619-622; norm as in dynet/model.cc:806-848): scale = clip/||g|| when
 * ||g|| > clip; p -= g * lr * scale; g = 0.  sizes[i] = element count of tensor i. */
ORC_API float orc_sgd_update(float* const* p, float* const* g, const size_t* sizes, unsigned n,
                             float lr, float clip_threshold) {
  float total = 0.f;
  for (unsigned i = 0; i < n; ++i) {
    float s = 0.f;
    for (size_t k = 0; k < sizes[i]; ++k) s += g[i][k] * g[i][k];
    total += s;
  }
  float gg = sqrtf(total), gscale = 1.f;
  if (clip_threshold > 0.f && gg > clip_threshold) gscale = clip_threshold / gg;
  for (unsigned i = 0; i < n; ++i) {
    for (size_t k = 0; k < sizes[i]; ++k) {
      p[i][k] -= g[i][k] * (lr * gscale);
      g[i][k] = 0.f;
    }
  }
  return gg;
}

/* Trainer update rules, one statement per reference statement, each rounded to float32
 * (dynet/training.cc: SimpleSGD :619-622, MomentumSGD :669-673, Adagrad :735-739, Adadelta :802-808,
 * RMSProp :883-888, Adam :955-961, Amsgrad :1034-1041).  rule: 0 sgd, 1 momentum, 2 adagrad, 3 adadelta,
 * 4 rmsprop, 5 adam, 6 amsgrad.  gscale is Trainer::clip_gradients' factor (:168-183); wd the
 * weight-decay divisor; updates the number of updates done before this one.  The gradient is left as the
 * rule leaves it (rules 2-6 rewrite it). */
ORC_API void orc_trainer_update(int rule, float* p, float* g, float* s0, float* s1, float* s2, size_t n, float lr,
                                float gscale, float wd, float momentum, float eps, float rho, float beta_1,
                                float beta_2, unsigned long long updates) {
  float lr_t = (float)(lr * sqrt(1 - pow(beta_2, (double)updates + 1)) / (1 - pow(beta_1, (double)updates + 1)) / wd);
  for (size_t k = 0; k < n; ++k) {
    switch (rule) {
      case 0: p[k] -= g[k] * (lr * gscale / wd); break;
      case 1:
        s0[k] = s0[k] * momentum - g[k] * (lr * gscale);
        p[k] += s0[k] / wd;
        break;
      case 2:
        g[k] = g[k] * gscale;
        s0[k] += g[k] * g[k];
        p[k] += g[k] / sqrtf(s0[k] + eps) * (-lr / wd);
        break;
      case 3:
        g[k] = g[k] * gscale;
        s0[k] = s0[k] * rho + g[k] * g[k] * (1.f - rho);
        g[k] = -g[k] * sqrtf(s1[k] + eps) / sqrtf(s0[k] + eps);
        s1[k] = s1[k] * rho + g[k] * g[k] * (1.f - rho);
        p[k] += g[k] / wd;
        break;
      case 4:
        g[k] = g[k] * gscale;
        s0[k] = s0[k] * rho + g[k] * g[k] * (1.f - rho);
        g[k] = -g[k] / sqrtf(s0[k] + eps);
        p[k] += lr * g[k] / wd;
        break;
      case 5:
        g[k] = g[k] * gscale;
        s0[k] = s0[k] * beta_1 + g[k] * (1.f - beta_1);
        s1[k] = s1[k] * beta_2 + g[k] * g[k] * (1.f - beta_2);
        p[k] -= s0[k] / (sqrtf(s1[k]) + eps) * lr_t;
        break;
      default:
        g[k] = g[k] * gscale;
        s0[k] = s0[k] * beta_1 + g[k] * (1.f - beta_1);
        s1[k] = s1[k] * beta_2 + g[k] * g[k] * (1.f - beta_2);
        s2[k] = s2[k] > s1[k] ? s2[k] : s1[k];
        p[k] -= s0[k] / (sqrtf(s2[k]) + eps) * lr_t;
        break;
    }
  }
}
