// One training pass of the BiLSTM tagger over a mini-batch of ragged sentences, run the way DyNet's autobatching
// executor schedules it.
//
// Graph per sentence (examples/tagger/train_tag-bilstm.cc:60-117, without the input noise): x_t = lookup(p_w, w_t);
// forward and backward CompactVanillaLSTM over the sentence; per token th = tanh(thbias + l2th * fwd_t + r2th * rev_t),
// logits = tbias + th2t * th, err = pickneglogsoftmax(logits, tag_t); loss = sum of all errs.
//
// With --dynet-autobatch 1 the batched executor (dynet/exec.cc:481-895) runs nodes of equal depth together: the k-th
// LSTM step of every sentence that is at least k + 1 words long is ONE batched node, so the batch shrinks with the step
// (sentences sorted by length, longest first: the sentences still running at step k are the first B_k).  The per-token
// nodes of the tag layer are batched over ALL tokens; their inputs, the hidden states of (sentence, position), sit in
// the outputs of different LSTM steps and are gathered into one contiguous matrix by combine_tensors (exec.cc:298-361 ->
// gpu::parallel_memcpy); the gradients go back through accumulate_tensors (exec.cc:363-411 -> gpu::parallel_accumulate).
// This driver makes exactly those calls.  The pointer tables of the movers are built on the host per mini-batch and
// uploaded, as the executor does (exec.cc:346-356).
//
// Device layout: per direction the columns of all steps sit side by side in step order ("step-major"): column
// prefix[k] + s holds sentence s at step k.  The token-major matrices of the tag layer have token n = (s, t) at column
// tok0[s] + t.
#include <cuda_runtime.h>

#include <chrono>
#include <cstring>
#include <string>
#include <vector>

#include "dynet_shim.h"

using namespace dynet_b200;

extern "C" {
typedef struct {
  uint32_t V, E, H, TH, NT;   // vocabulary, embedding width, hidden units per direction, tag-hidden width, tags
  float lr, clip;
} dyb200h_tagger_config;
}

namespace {

#define CU(expr)                                                                              \
  do {                                                                                        \
    cudaError_t e__ = (expr);                                                                 \
    if (e__ != cudaSuccess) throw cuda_exception(std::string(#expr) + ": " + cudaGetErrorString(e__)); \
  } while (0)

// parameter order in the flat buffers
enum { P_EMB = 0, P_WXF, P_WHF, P_BF, P_WXR, P_WHR, P_BR, P_L2TH, P_R2TH, P_THB, P_TH2T, P_TB, P_COUNT };

size_t tagger_sizes(const dyb200h_tagger_config& c, size_t* sz) {
  const size_t G = 4 * (size_t)c.H;
  size_t s[P_COUNT] = {(size_t)c.E * c.V, G * c.E, G * c.H, G, G * c.E, G * c.H, G,
                       (size_t)c.TH * c.H, (size_t)c.TH * c.H, c.TH, (size_t)c.NT * c.TH, c.NT};
  size_t total = 0;
  for (int k = 0; k < P_COUNT; ++k) { if (sz) sz[k] = s[k]; total += s[k]; }
  return total;
}

struct Arena {
  char* base; size_t off;
  template <class Tp> Tp* take(size_t n) {
    off = (off + 255) & ~(size_t)255;
    Tp* p = (Tp*)(base + off);
    off += n * sizeof(Tp);
    return p;
  }
};

struct Dir {   // one direction's step-major activations, N columns each
  float *x, *gates, *c, *h, *dh, *dc, *dx;
  uint32_t* ids;      // word of every column
  dyb200_wgrad* wg;   // deferred dWx / dWh products
};

struct Tagger {
  dyb200h_tagger_config c;
  Device_GPU dev;
  std::string err;
  float *params, *grads;
  float *p[P_COUNT], *g[P_COUNT];
  cudaStream_t stream;
  uint32_t max_sent, max_tok, max_len;
  Dir d[2];
  float *hf, *hr, *dhf, *dhr, *pre, *th, *dth, *dpre, *logits, *dlogits, *errs, *aux, *ones, *zeros, *scalars;
  // pointer / length tables of the four mover calls (device) and their pinned host staging
  float** tbl_dev; size_t* len_dev;
  float** tbl_host;   // pinned: 8 N pointers, N lengths, then the ids (2 N words + N tags)
  size_t dact_off0, dact_off1;
  char* ws;
  bool time_movers = false;
  cudaEvent_t ev[8];
  cudaEvent_t upload_ev = nullptr;
  bool upload_pending = false;
  // The two directions are independent chains of small launches: the reverse direction runs on a stream (and a library
  // context: scratch arena, split-weight cache) of its own, beside the forward direction on the caller's stream.
  Device_GPU dev2;
  cudaStream_t stream2 = nullptr;
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
  double host_schedule_ms = 0.0;
  ~Tagger() {
    for (int k = 0; k < 2; ++k) if (d[k].wg) dyb200_wgrad_destroy(d[k].wg);
    if (tbl_host) cudaFreeHost(tbl_host);
    for (auto& e : ev) if (e) cudaEventDestroy(e);
    if (upload_ev) cudaEventDestroy(upload_ev);
    if (fork_ev) cudaEventDestroy(fork_ev);
    if (join_ev) cudaEventDestroy(join_ev);
    if (dev2.ctx) dyb200_ctx_destroy(dev2.ctx);
    if (stream2) cudaStreamDestroy(stream2);
  }
};

size_t plan(const dyb200h_tagger_config& c, uint32_t S, uint32_t N, Tagger* t, char* base) {
  Arena a{base, 0};
  const size_t E = c.E, H = c.H, G = 4 * H;
  Dir d[2];
  for (int k = 0; k < 2; ++k) {
    d[k].x = a.take<float>(E * N); d[k].gates = a.take<float>(G * N); d[k].c = a.take<float>(H * N); d[k].h = a.take<float>(H * N);
    d[k].ids = a.take<uint32_t>(N);
    d[k].wg = nullptr;
  }
  float* hf = a.take<float>(H * N); float* hr = a.take<float>(H * N);
  float* pre = a.take<float>((size_t)c.TH * N); float* th = a.take<float>((size_t)c.TH * N);
  float* logits = a.take<float>((size_t)c.NT * N);
  float* errs = a.take<float>(N); float* aux = a.take<float>(3 * (size_t)N); float* ones = a.take<float>(N);
  float* zeros = a.take<float>(H * S); float* scalars = a.take<float>(64);
  float** tbl = a.take<float*>(8 * (size_t)N); size_t* len = a.take<size_t>(N);
  // everything below is zeroed by one memset per pass
  a.off = (a.off + 255) & ~(size_t)255;
  const size_t z0 = a.off;
  for (int k = 0; k < 2; ++k) { d[k].dh = a.take<float>(H * N); d[k].dc = a.take<float>(H * N); d[k].dx = a.take<float>(E * N); }
  float* dhf = a.take<float>(H * N); float* dhr = a.take<float>(H * N);
  float* dth = a.take<float>((size_t)c.TH * N); float* dpre = a.take<float>((size_t)c.TH * N);
  float* dlogits = a.take<float>((size_t)c.NT * N);
  const size_t z1 = a.off;
  if (t) {
    for (int k = 0; k < 2; ++k) { dyb200_wgrad* keep = t->d[k].wg; t->d[k] = d[k]; t->d[k].wg = keep; }
    t->hf = hf; t->hr = hr; t->dhf = dhf; t->dhr = dhr; t->pre = pre; t->th = th; t->dth = dth; t->dpre = dpre;
    t->logits = logits; t->dlogits = dlogits; t->errs = errs; t->aux = aux; t->ones = ones; t->zeros = zeros; t->scalars = scalars;
    t->tbl_dev = tbl; t->len_dev = len; t->dact_off0 = z0; t->dact_off1 = z1; t->ws = base;
  }
  return a.off + 256;
}

}  // namespace

namespace {

struct PassArgs { uint32_t S; const uint32_t* lens; const uint32_t* words; const uint32_t* tags; float* loss_dev; };

void tagger_pass(Tagger& m, const PassArgs& a) {
  const dyb200h_tagger_config& c = m.c;
  const uint32_t E = c.E, H = c.H, TH = c.TH, NT = c.NT, V = c.V, S = a.S;
  const Device_GPU& dev = m.dev;
  const Device_GPU* dv[2] = {&m.dev, &m.dev2};   // library context of each direction
  const cudaStream_t st2 = m.stream2;
  cudaStream_t st = m.stream;
  if (S == 0) throw std::invalid_argument("tagger: empty mini-batch");
  if (S > m.max_sent) throw std::invalid_argument("tagger: more sentences than the workspace was planned for");
  // ---- host side: the batched executor's schedule for this mini-batch ----
  // (the pinned staging buffers are reused from pass to pass: the previous pass's uploads must have left them)
  if (m.upload_pending) { CU(cudaEventSynchronize(m.upload_ev)); m.upload_pending = false; }
  const auto t_host0 = std::chrono::steady_clock::now();
  const uint32_t Lmax = a.lens[0];
  if (Lmax == 0 || Lmax > m.max_len) throw std::invalid_argument("tagger: sentence length out of range");
  std::vector<uint32_t> tok0(S + 1, 0);
  for (uint32_t s = 0; s < S; ++s) {
    if (s && a.lens[s] > a.lens[s - 1]) throw std::invalid_argument("tagger: sentences must be sorted by length, longest first");
    if (a.lens[s] == 0) throw std::invalid_argument("tagger: empty sentence");
    tok0[s + 1] = tok0[s] + a.lens[s];
  }
  const uint32_t N = tok0[S];
  if (N > m.max_tok) throw std::invalid_argument("tagger: more tokens than the workspace was planned for");
  std::vector<uint32_t> Bk(Lmax), prefix(Lmax + 1, 0);
  {
    uint32_t b = S;
    for (uint32_t k = 0; k < Lmax; ++k) {
      while (b > 0 && a.lens[b - 1] <= k) --b;     // sentences 0 .. b-1 are longer than k
      Bk[k] = b;
      prefix[k + 1] = prefix[k] + b;
    }
  }
  float** tbl = m.tbl_host;
  size_t* lens_host = (size_t*)(m.tbl_host + 8 * (size_t)m.max_tok);
  uint32_t* ids_host = (uint32_t*)(lens_host + m.max_tok);
  uint32_t *ids_f = ids_host, *ids_r = ids_host + N, *tag_ids = ids_host + 2 * (size_t)N;
  for (uint32_t s = 0; s < S; ++s) {
    const uint32_t len = a.lens[s];
    for (uint32_t t = 0; t < len; ++t) {
      const uint32_t n = tok0[s] + t, w = a.words[n];
      if (w >= V) throw std::invalid_argument("Out-of-bounds attempt to access index " + std::to_string(w) + " for LookupParameter of size " + std::to_string(V));
      if (a.tags[n] >= NT) throw std::invalid_argument("Index error in PickNegLogSoftmax: tag " + std::to_string(a.tags[n]));
      const uint32_t cf = prefix[t] + s, cr = prefix[len - 1 - t] + s;   // column of (s, t) in the two directions
      ids_f[cf] = w; ids_r[cr] = w; tag_ids[n] = a.tags[n];
      tbl[n] = m.d[0].h + (size_t)cf * H;               tbl[N + n] = m.hf + (size_t)n * H;
      tbl[2 * (size_t)N + n] = m.d[1].h + (size_t)cr * H;  tbl[3 * (size_t)N + n] = m.hr + (size_t)n * H;
      tbl[4 * (size_t)N + n] = m.dhf + (size_t)n * H;     tbl[5 * (size_t)N + n] = m.d[0].dh + (size_t)cf * H;
      tbl[6 * (size_t)N + n] = m.dhr + (size_t)n * H;     tbl[7 * (size_t)N + n] = m.d[1].dh + (size_t)cr * H;
      lens_host[n] = H;
    }
  }
  m.host_schedule_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_host0).count();
  CU(cudaMemcpyAsync(m.tbl_dev, tbl, 8 * (size_t)N * sizeof(float*), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(m.len_dev, lens_host, (size_t)N * sizeof(size_t), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(m.d[0].ids, ids_f, (size_t)N * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(m.d[1].ids, ids_r, (size_t)N * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(m.aux + 2 * (size_t)N, tag_ids, (size_t)N * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
  CU(cudaEventRecord(m.upload_ev, st));
  m.upload_pending = true;

  Tensor tEmb(Dim({E}, V), m.p[P_EMB]);
  const dyb200_lstm_gates_attrs at = {0, 0.f, 1.f};
  auto col = [](float* base, uint32_t rows, uint32_t c0, uint32_t n) { return Tensor(Dim({rows}, n), base + (size_t)c0 * rows); };

  // ---------------- forward ----------------
  CU(cudaEventRecord(m.fork_ev, st));          // (the uploads above are on the caller's stream)
  CU(cudaStreamWaitEvent(st2, m.fork_ev, 0));
  for (int dr = 0; dr < 2; ++dr) {
    Dir& d = m.d[dr];
    const Device_GPU& dev = *dv[dr];
    LookupNode look(tEmb, nullptr, N);       // all lookups of a direction are one batched node
    look.aux_mem = d.ids;
    Tensor xall(Dim({E}, N), d.x);
    look.forward_dev_impl(dev, {}, xall);
    // the inputs of all steps of the direction exist now: one launch splits them into the operand planes of the gate products
    // and of the weight-gradient product; each step's epilogue then leaves h_t as the next step's operand planes, so the
    // steps launch no operand split of their own
    const dyb200_tensor cxall = to_c(xall);
    throw_status(dev, dyb200_wgrad_pack_inputs(d.wg, &cxall, nullptr, 0, dev.ctx));
    Tensor tWx(Dim({4 * H, E}), m.p[P_WXF + 3 * dr]), tWh(Dim({4 * H, H}), m.p[P_WHF + 3 * dr]), tb(Dim({4 * H}), m.p[P_BF + 3 * dr]);
    const dyb200_tensor cWx = to_c(tWx), cWh = to_c(tWh), cb = to_c(tb);
    for (uint32_t k = 0; k < Lmax; ++k) {
      const uint32_t B = Bk[k];
      const dyb200_tensor cx = to_c(col(d.x, E, prefix[k], B));
      const dyb200_tensor chp = to_c(k ? col(d.h, H, prefix[k - 1], B) : Tensor(Dim({H}, B), m.zeros));
      const dyb200_tensor ccp = to_c(k ? col(d.c, H, prefix[k - 1], B) : Tensor(Dim({H}, B), m.zeros));
      dyb200_tensor cg = to_c(col(d.gates, 4 * H, prefix[k], B)), cc = to_c(col(d.c, H, prefix[k], B)), ch = to_c(col(d.h, H, prefix[k], B));
      throw_status(dev, dyb200_vanilla_lstm_fwd_fused_at(&cx, &chp, &ccp, &cWx, &cWh, &cb, nullptr, nullptr, &at, &cg, &cc, &ch, d.wg, prefix[k], dev.ctx));
    }
  }
  CU(cudaEventRecord(m.join_ev, st2));
  CU(cudaStreamWaitEvent(st, m.join_ev, 0));
  // combine_tensors: the hidden states of all tokens, token-major
  for (int dr = 0; dr < 2; ++dr) {
    if (m.time_movers) CU(cudaEventRecord(m.ev[2 * dr], st));
    gpu::parallel_memcpy(dev, (int)N, (int)H, m.tbl_dev + 2 * (size_t)dr * N, m.tbl_dev + (2 * (size_t)dr + 1) * N, m.len_dev);
    if (m.time_movers) CU(cudaEventRecord(m.ev[2 * dr + 1], st));
  }
  Tensor thb(Dim({TH}), m.p[P_THB]), l2th(Dim({TH, H}), m.p[P_L2TH]), r2th(Dim({TH, H}), m.p[P_R2TH]);
  Tensor th2t(Dim({NT, TH}), m.p[P_TH2T]), tbias(Dim({NT}), m.p[P_TB]);
  Tensor thf(Dim({H}, N), m.hf), thr(Dim({H}, N), m.hr), tpre(Dim({TH}, N), m.pre), tth(Dim({TH}, N), m.th), tlog(Dim({NT}, N), m.logits);
  Tensor terrs(Dim({1}, N), m.errs), tones(Dim({1}, N), m.ones);
  AffineTransform affine;
  Tanh tanh_node;
  PickNegLogSoftmax pnls(nullptr);
  pnls.dim = Dim({1}, N);
  pnls.aux_mem = m.aux;
  const std::vector<const Tensor*> xs1 = {&thb, &l2th, &thf, &r2th, &thr}, xs2 = {&tbias, &th2t, &tth};
  affine.forward_dev_impl(dev, xs1, tpre);
  tanh_node.forward_dev_impl(dev, {&tpre}, tth);
  affine.forward_dev_impl(dev, xs2, tlog);
  pnls.forward_dev_impl(dev, {&tlog}, terrs);
  throw_status(dev, dyb200_sum_all(m.errs, N, a.loss_dev, 0, dev.ctx));

  // ---------------- backward ----------------
  CU(cudaMemsetAsync(m.ws + m.dact_off0, 0, m.dact_off1 - m.dact_off0, st));
  Tensor tdlog(Dim({NT}, N), m.dlogits), tdth(Dim({TH}, N), m.dth), tdpre(Dim({TH}, N), m.dpre), tdhf(Dim({H}, N), m.dhf), tdhr(Dim({H}, N), m.dhr);
  Tensor gthb(Dim({TH}), m.g[P_THB]), gl2th(Dim({TH, H}), m.g[P_L2TH]), gr2th(Dim({TH, H}), m.g[P_R2TH]);
  Tensor gth2t(Dim({NT, TH}), m.g[P_TH2T]), gtbias(Dim({NT}), m.g[P_TB]);
  pnls.backward_dev_impl(dev, {&tlog}, terrs, tones, 0, tdlog);
  affine.backward_dev_impl(dev, xs2, tlog, tdlog, 0, gtbias);
  affine.backward_dev_impl(dev, xs2, tlog, tdlog, 1, gth2t);
  affine.backward_dev_impl(dev, xs2, tlog, tdlog, 2, tdth);
  tanh_node.backward_dev_impl(dev, {&tpre}, tth, tdth, 0, tdpre);
  affine.backward_dev_impl(dev, xs1, tpre, tdpre, 0, gthb);
  affine.backward_dev_impl(dev, xs1, tpre, tdpre, 1, gl2th);
  affine.backward_dev_impl(dev, xs1, tpre, tdpre, 2, tdhf);
  affine.backward_dev_impl(dev, xs1, tpre, tdpre, 3, gr2th);
  affine.backward_dev_impl(dev, xs1, tpre, tdpre, 4, tdhr);
  // accumulate_tensors: the token-major gradients back into the steps' dE/dh
  for (int dr = 0; dr < 2; ++dr) {
    if (m.time_movers) CU(cudaEventRecord(m.ev[4 + 2 * dr], st));
    gpu::parallel_accumulate(dev, (int)N, (int)H, m.tbl_dev + (4 + 2 * (size_t)dr) * N, m.tbl_dev + (5 + 2 * (size_t)dr) * N, m.len_dev);
    if (m.time_movers) CU(cudaEventRecord(m.ev[5 + 2 * dr], st));
  }
  Tensor gEmb(Dim({E}, V), m.g[P_EMB]);
  CU(cudaEventRecord(m.fork_ev, st));
  CU(cudaStreamWaitEvent(st2, m.fork_ev, 0));
  for (int dr = 0; dr < 2; ++dr) {
    Dir& d = m.d[dr];
    const Device_GPU& dev = *dv[dr];
    Tensor tWx(Dim({4 * H, E}), m.p[P_WXF + 3 * dr]), tWh(Dim({4 * H, H}), m.p[P_WHF + 3 * dr]);
    Tensor gb(Dim({4 * H}), m.g[P_BF + 3 * dr]);
    const dyb200_tensor cWx = to_c(tWx), cWh = to_c(tWh);
    dyb200_tensor cgb = to_c(gb);
    for (uint32_t k = Lmax; k-- > 0;) {
      const uint32_t B = Bk[k];
      const dyb200_tensor cx = to_c(col(d.x, E, prefix[k], B));
      const dyb200_tensor chp = to_c(k ? col(d.h, H, prefix[k - 1], B) : Tensor(Dim({H}, B), m.zeros));
      const dyb200_tensor ccp = to_c(k ? col(d.c, H, prefix[k - 1], B) : Tensor(Dim({H}, B), m.zeros));
      const dyb200_tensor cg = to_c(col(d.gates, 4 * H, prefix[k], B)), cc = to_c(col(d.c, H, prefix[k], B));
      const dyb200_tensor cdh = to_c(col(d.dh, H, prefix[k], B)), cdc = to_c(col(d.dc, H, prefix[k], B));
      dyb200_tensor cdx = to_c(col(d.dx, E, prefix[k], B));
      dyb200_tensor cdhp = to_c(k ? col(d.dh, H, prefix[k - 1], B) : Tensor()), cdcp = to_c(k ? col(d.dc, H, prefix[k - 1], B) : Tensor());
      // (weight gradients: the gate gradient of this step goes to the step's columns of the direction's accumulator, where the
      // forward pass left the inputs; one product at the end)
      throw_status(dev, dyb200_vanilla_lstm_bwd_fused_at(&cx, &chp, &ccp, &cWx, &cWh, nullptr, nullptr, &cg, &cc, &cdh, &cdc, &cdx,
                                                         k ? &cdhp : nullptr, k ? &cdcp : nullptr, nullptr, nullptr, &cgb, &at, d.wg,
                                                         prefix[k], dev.ctx));
    }
    throw_status(dev, dyb200_wgrad_flush(d.wg, m.g[P_WXF + 3 * dr], 4 * H, m.g[P_WHF + 3 * dr], 4 * H, dev.ctx));
  }
  CU(cudaEventRecord(m.join_ev, st2));
  CU(cudaStreamWaitEvent(st, m.join_ev, 0));
  // the lookups' accumulate_grad calls, folded into one per direction over its columns (step order); both add into the one
  // table gradient, so they run one after the other on the caller's stream
  for (int dr = 0; dr < 2; ++dr) {
    Dir& d = m.d[dr];
    LookupNode look(tEmb, nullptr, N);
    look.aux_mem = d.ids;
    Tensor tdx(Dim({E}, N), d.dx);
    look.accumulate_grad(dev, tdx, gEmb);
  }
}

int guarded(Tagger* m, const PassArgs& a) {
  try {
    tagger_pass(*m, a);
    return DYB200_OK;
  } catch (const std::invalid_argument& e) { m->err = e.what(); return DYB200_EINVAL;
  } catch (const out_of_memory& e) { m->err = e.what(); return DYB200_ENOMEM;
  } catch (const cuda_exception& e) { m->err = e.what(); return DYB200_ECUDA;
  } catch (const std::exception& e) { m->err = e.what(); return DYB200_ERUNTIME; }
}

}  // namespace

extern "C" {

size_t dyb200h_tagger_num_params(const dyb200h_tagger_config* c) { return tagger_sizes(*c, nullptr); }
// Offsets (in floats) of the 12 parameter tensors in the flat buffer, in the order emb, (Wx, Wh, b) forward, (Wx, Wh, b)
// backward, l2th, r2th, thbias, th2t, tbias; returns their count.
int dyb200h_tagger_param_offsets(const dyb200h_tagger_config* c, size_t* offsets, size_t* sizes, int cap) {
  size_t sz[P_COUNT], off = 0;
  tagger_sizes(*c, sz);
  for (int k = 0; k < P_COUNT && k < cap; ++k) { offsets[k] = off; sizes[k] = sz[k]; off += sz[k]; }
  return P_COUNT;
}
size_t dyb200h_tagger_workspace_bytes(const dyb200h_tagger_config* c, uint32_t max_sentences, uint32_t max_tokens) {
  return plan(*c, max_sentences, max_tokens, nullptr, nullptr);
}

int dyb200h_tagger_create(const dyb200h_tagger_config* c, float* params, float* grads, void* workspace, size_t ws_bytes,
                          uint32_t max_sentences, uint32_t max_tokens, uint32_t max_len, dyb200_ctx* ctx, void* stream, void** out) {
  if (!c || !params || !grads || !workspace || !ctx || !out || max_sentences == 0 || max_tokens == 0) return DYB200_EINVAL;
  if (ws_bytes < plan(*c, max_sentences, max_tokens, nullptr, nullptr)) return DYB200_ENOMEM;
  Tagger* m = new Tagger();
  m->c = *c; m->dev.ctx = ctx; m->params = params; m->grads = grads; m->stream = (cudaStream_t)stream;
  m->max_sent = max_sentences; m->max_tok = max_tokens; m->max_len = max_len;
  m->d[0].wg = m->d[1].wg = nullptr; m->tbl_host = nullptr;
  for (auto& e : m->ev) e = nullptr;
  size_t sz[P_COUNT], off = 0;
  tagger_sizes(*c, sz);
  for (int k = 0; k < P_COUNT; ++k) { m->p[k] = params + off; m->g[k] = grads + off; off += sz[k]; }
  plan(*c, max_sentences, max_tokens, m, (char*)workspace);
  dyb200_ctx_param_cache(ctx, 1);   // this driver owns the updates (dyb200h_tagger_update), so split weights can be reused
  int rc = DYB200_OK;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) rc = DYB200_ECUDA;
  if (!rc && cudaStreamCreateWithFlags(&m->stream2, cudaStreamNonBlocking) != cudaSuccess) rc = DYB200_ECUDA;
  if (!rc) rc = dyb200_ctx_create(device, m->stream2, &m->dev2.ctx);
  if (!rc) dyb200_ctx_param_cache(m->dev2.ctx, 1);
  if (!rc && (cudaEventCreateWithFlags(&m->fork_ev, cudaEventDisableTiming) != cudaSuccess ||
              cudaEventCreateWithFlags(&m->join_ev, cudaEventDisableTiming) != cudaSuccess)) rc = DYB200_ECUDA;
  for (int k = 0; k < 2 && !rc; ++k) rc = dyb200_wgrad_create(k ? m->dev2.ctx : ctx, 4 * c->H, c->E, c->H, max_tokens, &m->d[k].wg);
  const size_t host_bytes = 8 * (size_t)max_tokens * sizeof(float*) + (size_t)max_tokens * sizeof(size_t) + 3 * (size_t)max_tokens * sizeof(uint32_t);
  if (!rc && cudaMallocHost((void**)&m->tbl_host, host_bytes) != cudaSuccess) { cudaGetLastError(); rc = DYB200_ENOMEM; }
  for (auto& e : m->ev) if (!rc && cudaEventCreate(&e) != cudaSuccess) rc = DYB200_ECUDA;
  if (!rc && cudaEventCreateWithFlags(&m->upload_ev, cudaEventDisableTiming) != cudaSuccess) rc = DYB200_ECUDA;
  if (!rc) rc = dyb200_fill(m->zeros, (size_t)c->H * max_sentences, 0.f, ctx);
  if (!rc) rc = dyb200_fill(m->ones, max_tokens, 1.f, ctx);
  if (rc) { delete m; return rc; }
  *out = m;
  return DYB200_OK;
}

void dyb200h_tagger_destroy(void* h) { delete (Tagger*)h; }
const char* dyb200h_tagger_error(void* h) { return h ? ((Tagger*)h)->err.c_str() : "null handle"; }

// One mini-batch: n_sent sentences sorted by length (longest first), lens[n_sent], words / tags concatenated sentence by
// sentence (host arrays).  loss_dev receives the summed loss; gradients ACCUMULATE into the flat gradient buffer.
int dyb200h_tagger_forward_backward(void* h, uint32_t n_sent, const uint32_t* lens, const uint32_t* words, const uint32_t* tags,
                                    float* loss_dev) {
  if (!h || !lens || !words || !tags || !loss_dev) return DYB200_EINVAL;
  PassArgs a{n_sent, lens, words, tags, loss_dev};
  return guarded((Tagger*)h, a);
}

int dyb200h_tagger_grad_sumsq(void* h, float** scalar_dev_out) {
  Tagger* m = (Tagger*)h;
  int rc = dyb200_squared_norm(m->grads, tagger_sizes(m->c, nullptr), m->scalars, 0, m->dev.ctx);
  if (rc) { m->err = dyb200_last_error(m->dev.ctx); return rc; }
  if (scalar_dev_out) *scalar_dev_out = m->scalars;
  return DYB200_OK;
}
int dyb200h_tagger_update(void* h) {
  Tagger* m = (Tagger*)h;
  int rc = dyb200_sgd_update(m->params, m->grads, tagger_sizes(m->c, nullptr), m->c.lr, m->c.clip, m->scalars, m->dev.ctx);
  if (rc) m->err = dyb200_last_error(m->dev.ctx);
  dyb200_ctx_params_changed(m->dev2.ctx);   // (the second direction's context keeps its own split weights)
  return rc;
}

// Launch count and device error flags of the second direction's context (the caller's context reports its own).
int dyb200h_tagger_side_stats(void* h, uint64_t* launches, uint32_t* error_flags) {
  Tagger* m = (Tagger*)h;
  if (!m) return DYB200_EINVAL;
  if (launches) *launches = dyb200_ctx_launch_count(m->dev2.ctx);
  if (error_flags) return dyb200_ctx_check_device_errors(m->dev2.ctx, error_flags);
  return DYB200_OK;
}

// Measurement hooks: with timing on, the four mover calls of a pass are bracketed by CUDA events; dyb200h_tagger_mover_ms
// waits for the pass and returns {copy fwd, copy bwd direction, accumulate fwd, accumulate bwd direction} in ms, plus the host
// time spent building the schedule and the pointer tables of the last pass.
int dyb200h_tagger_time_movers(void* h, int enable) { ((Tagger*)h)->time_movers = enable != 0; return DYB200_OK; }
int dyb200h_tagger_mover_ms(void* h, float ms_out[4], double* host_schedule_ms) {
  Tagger* m = (Tagger*)h;
  if (cudaStreamSynchronize(m->stream) != cudaSuccess) return DYB200_ECUDA;
  for (int k = 0; k < 4; ++k) {
    float t = 0.f;
    if (m->time_movers && cudaEventElapsedTime(&t, m->ev[2 * k], m->ev[2 * k + 1]) != cudaSuccess) { cudaGetLastError(); t = 0.f; }
    ms_out[k] = t;
  }
  if (host_schedule_ms) *host_schedule_ms = m->host_schedule_ms;
  return DYB200_OK;
}

}  // extern "C"
