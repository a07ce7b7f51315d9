// Fused LSTM nodes: VanillaLSTMGates, VanillaLSTMC, VanillaLSTMH.
//
// Gates forward is ONE GEMM launch: both products (Wx*x and Wh*h) accumulate into the same
// output tile, dropout masks are applied to the activations as they are loaded, and the
// epilogue adds the bias (+ forget-gate bias on rows [H,2H)) and applies sigmoid / tanh.
// Gates backward forms the gate pre-activation gradient dgate once per call in scratch and
// then runs one transposed GEMM (dx, dh: mask fused in the epilogue) or one outer-product
// GEMM over the batch (dWx, dWh: mask fused in the operand load), or a deterministic batch
// reduction (db).  C and H are single-pass 128-bit elementwise kernels over gate slices.
#include "common.cuh"
#include "gemm.cuh"
#include "lstm_cell.cuh"
#include "reduce.cuh"

namespace {

constexpr int kThreads = 256;

// dgate = dE * g * (1 - g) on rows [0, 3H), dE * (1 - g^2) on rows [3H, 4H)
__device__ __forceinline__ float gate_deriv(float g, float d, bool is_tanh) {
  return is_tanh ? d * (1.f - g * g) : d * g * (1.f - g);
}
__global__ void __launch_bounds__(kThreads) k_gate_deriv(const float* __restrict__ fx, const float* __restrict__ dEdf,
                                                        float* __restrict__ dg, uint32_t H, size_t total, int vec) {
  dyb_grid_dep_sync();
  const uint32_t G = 4 * H;
  if (vec) {
    size_t n4 = total / 4;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += (size_t)gridDim.x * kThreads) {
      float4 g = ld4(fx + 4 * i), d = ld4(dEdf + 4 * i);
      bool t = (uint32_t)((4 * i) % G) >= 3 * H;  // H % 4 == 0, so a vector never straddles gates
      st4(dg + 4 * i, make_float4(gate_deriv(g.x, d.x, t), gate_deriv(g.y, d.y, t), gate_deriv(g.z, d.z, t), gate_deriv(g.w, d.w, t)));
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kThreads)
      dg[i] = gate_deriv(fx[i], dEdf[i], (uint32_t)(i % G) >= 3 * H);
  }
}
struct GateDerivSum {  // db[r] += sum_b dgate[r, b]
  const float *fx, *dEdf;
  uint32_t H;
  __device__ float operator()(size_t r, uint32_t b) const {
    size_t k = (size_t)b * 4 * H + r;
    return gate_deriv(fx[k], dEdf[k], r >= 3u * H);
  }
};

// weightnoise_std > 0: the reference skips both products, so the output is act(bias) only.
__global__ void __launch_bounds__(kThreads) k_gates_bias_only(const float* __restrict__ bias, float* __restrict__ fx,
                                                             uint32_t H, size_t total, float forget_bias) {
  dyb_grid_dep_sync();
  const uint32_t G = 4 * H;
  for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kThreads) {
    uint32_t r = (uint32_t)(i % G);
    float v = bias[r] + ((r >= H && r < 2 * H) ? forget_bias : 0.f);
    fx[i] = r < 3 * H ? gate_sigmoid(v) : gate_tanh(v);
  }
}

// Concatenate k inputs along dim 0 into one I x B matrix (only used when k > 1).
__global__ void __launch_bounds__(kThreads) k_concat_rows(const float* __restrict__ src, uint32_t d, uint32_t off,
                                                         uint32_t I, uint32_t B, float* __restrict__ dst) {
  dyb_grid_dep_sync();
  size_t total = (size_t)d * B;
  for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < total; e += (size_t)gridDim.x * kThreads) {
    size_t b = e / d, r = e % d;
    dst[b * I + off + r] = src[e];
  }
}

// ---- C and H ---------------------------------------------------------------------------
// MODE 0: c = i*g + f*c_tm1                     (VanillaLSTMC forward)
// MODE 1: h = o * tanh(c)                       (VanillaLSTMH forward)
template <int MODE, int VEC>
__global__ void __launch_bounds__(kThreads) k_lstm_ch_fwd(const float* __restrict__ st, const float* __restrict__ gates,
                                                         float* __restrict__ out, uint32_t H, size_t total) {
  dyb_grid_dep_sync();
  constexpr int W = VEC ? 4 : 1;
  for (size_t e = ((size_t)blockIdx.x * kThreads + threadIdx.x) * W; e < total; e += (size_t)gridDim.x * kThreads * W) {
    size_t b = e / H, j = e % H;
    const float* g = gates + b * 4 * H;
    if (VEC) {
      float4 s = ld4_stream(st + e), r;
      if (MODE == 0) {
        float4 gi = ld4_stream(g + j), gf = ld4_stream(g + H + j), gg = ld4_stream(g + 3 * H + j);
        r = make_float4(lstm_cell_c(gi.x, gg.x, gf.x, s.x), lstm_cell_c(gi.y, gg.y, gf.y, s.y), lstm_cell_c(gi.z, gg.z, gf.z, s.z), lstm_cell_c(gi.w, gg.w, gf.w, s.w));
      } else {
        float4 go = ld4_stream(g + 2 * H + j);
        r = make_float4(lstm_cell_h(go.x, s.x), lstm_cell_h(go.y, s.y), lstm_cell_h(go.z, s.z), lstm_cell_h(go.w, s.w));
      }
      st4(out + e, r);
    } else {
      out[e] = MODE == 0 ? lstm_cell_c(g[j], g[3 * H + j], g[H + j], st[e]) : lstm_cell_h(g[2 * H + j], st[e]);
    }
  }
}
// Backward, scalar index math shared by the vector and scalar variants.
// C, i=0: dc_tm1 += dc * f.   C, i=1: di += dc*g ; df += dc*c_tm1 ; dg += dc*i.
// H, i=0: dc += dh * o * (1 - tanh(c)^2).   H, i=1: do += dh * tanh(c).
template <int NODE, int VEC>
__global__ void __launch_bounds__(kThreads) k_lstm_ch_bwd(const float* __restrict__ st, const float* __restrict__ gates,
                                                         const float* __restrict__ d, unsigned i,
                                                         float* __restrict__ dxi, uint32_t H, size_t total) {
  dyb_grid_dep_sync();
  constexpr int W = VEC ? 4 : 1;
  for (size_t e = ((size_t)blockIdx.x * kThreads + threadIdx.x) * W; e < total; e += (size_t)gridDim.x * kThreads * W) {
    size_t b = e / H, j = e % H;
    const float* g = gates + b * 4 * H;
    float* og = dxi + b * 4 * H;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      float dv = d[e + w];
      if (NODE == 0) {
        if (i == 0) dxi[e + w] += dv * g[H + j + w];
        else {
          og[j + w] += dv * g[3 * H + j + w];
          og[H + j + w] += dv * st[e + w];
          og[3 * H + j + w] += dv * g[j + w];
        }
      } else {
        float t = tanhf(st[e + w]);
        if (i == 0) dxi[e + w] += dv * g[2 * H + j + w] * (1.f - t * t);
        else og[2 * H + j + w] += dv * t;
      }
    }
  }
}


// ---- fused cell kernels (used by the *_fused entry points) ---------------------------------------
// Forward: c = i*g + f*c_tm1 and h = o*tanh(c) in one pass over the gates.
template <int VEC>
__global__ void __launch_bounds__(kThreads) k_lstm_cell_fwd(const float* __restrict__ c_tm1, const float* __restrict__ gates,
                                                           float* __restrict__ c_t, float* __restrict__ h_t, uint32_t H,
                                                           size_t total) {
  dyb_grid_dep_sync();
  constexpr int W = VEC ? 4 : 1;
  for (size_t e = ((size_t)blockIdx.x * kThreads + threadIdx.x) * W; e < total; e += (size_t)gridDim.x * kThreads * W) {
    size_t b = e / H, j = e % H;
    const float* g = gates + b * 4 * H;
    if (VEC) {
      float4 cp = ld4_stream(c_tm1 + e), gi = ld4_stream(g + j), gf = ld4_stream(g + H + j), go = ld4_stream(g + 2 * H + j),
             gg = ld4_stream(g + 3 * H + j);
      float4 c = make_float4(lstm_cell_c(gi.x, gg.x, gf.x, cp.x), lstm_cell_c(gi.y, gg.y, gf.y, cp.y), lstm_cell_c(gi.z, gg.z, gf.z, cp.z), lstm_cell_c(gi.w, gg.w, gf.w, cp.w));
      st4(c_t + e, c);
      st4(h_t + e, make_float4(lstm_cell_h(go.x, c.x), lstm_cell_h(go.y, c.y), lstm_cell_h(go.z, c.z), lstm_cell_h(go.w, c.w)));
    } else {
      float c = lstm_cell_c(g[j], g[3 * H + j], g[H + j], c_tm1[e]);
      c_t[e] = c;
      h_t[e] = lstm_cell_h(g[2 * H + j], c);
    }
  }
}

// Backward of the H node, the C node and the gate non-linearities in one pass:
//   dc = dEdc + dEdh * o * (1 - tanh(c)^2);  dc_tm1 += dc * f
//   dpre_i = dc*g * i(1-i); dpre_f = dc*c_tm1 * f(1-f); dpre_o = dEdh*tanh(c) * o(1-o); dpre_g = dc*i * (1-g^2)
//   db[r] += sum_b dpre[r, b]
// One CTA owns 8 hidden units for the whole batch (thread = unit x batch lane), so the bias gradient
// is a complete, fixed-order sum and needs no second pass.
constexpr int kJT = 8;
__global__ void __launch_bounds__(256) k_lstm_cell_bwd(const float* __restrict__ c_t, const float* __restrict__ c_tm1,
                                                      const float* __restrict__ gates, const float* __restrict__ dEdh,
                                                      const float* __restrict__ dEdc, float* __restrict__ dc_tm1,
                                                      float* __restrict__ dpre, float* __restrict__ db, uint32_t H, uint32_t B) {
  dyb_grid_dep_sync();
  __shared__ float red[8][4][kJT];
  const int jj = threadIdx.x % kJT, bl = threadIdx.x / kJT;   // 32 batch lanes
  const uint32_t j = blockIdx.x * kJT + jj;
  const bool live = j < H;
  float si = 0.f, sf = 0.f, so = 0.f, sg = 0.f;
  if (live) {
    for (uint32_t b = bl; b < B; b += 32) {
      const size_t e = (size_t)b * H + j;
      const float* g = gates + (size_t)b * 4 * H;
      const float gi = g[j], gf = g[H + j], go = g[2 * H + j], gg = g[3 * H + j];
      const float c = c_t[e], cp = c_tm1[e], dh = dEdh[e];
      const float t = tanhf(c);
      float dc = dh * go * (1.f - t * t);
      if (dEdc) dc += dEdc[e];
      if (dc_tm1) dc_tm1[e] += dc * gf;
      const float pi = gate_deriv(gi, dc * gg, false), pf = gate_deriv(gf, dc * cp, false);
      const float po = gate_deriv(go, dh * t, false), pg = gate_deriv(gg, dc * gi, true);
      float* o = dpre + (size_t)b * 4 * H;
      o[j] = pi; o[H + j] = pf; o[2 * H + j] = po; o[3 * H + j] = pg;
      si += pi; sf += pf; so += po; sg += pg;
    }
  }
  // lanes of a warp: jj = lane % 8, four batch lanes -> fold the batch lanes, then the 8 warps
#pragma unroll
  for (int off = 8; off < 32; off <<= 1) {
    si += __shfl_xor_sync(0xffffffffu, si, off); sf += __shfl_xor_sync(0xffffffffu, sf, off);
    so += __shfl_xor_sync(0xffffffffu, so, off); sg += __shfl_xor_sync(0xffffffffu, sg, off);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane < kJT) { red[warp][0][lane] = si; red[warp][1][lane] = sf; red[warp][2][lane] = so; red[warp][3][lane] = sg; }
  __syncthreads();
  if (threadIdx.x < 4 * kJT) {
    const int gate = threadIdx.x / kJT, u = threadIdx.x % kJT;
    float acc = 0.f;
    for (int w = 0; w < 8; ++w) acc += red[w][gate][u];
    const uint32_t jo = blockIdx.x * kJT + u;
    if (jo < H) db[(size_t)gate * H + jo] += acc;
  }
}

// The same pass for shapes with H % 64 == 0 and B % 32 == 0, laid out for bandwidth: a CTA owns a tile of 64 hidden
// units x 32 batch columns; threads read float4 along the hidden index (coalesced), and the tile of gate gradients
// goes through shared memory for its row sums.  Outputs, each optional except dc_tm1's accumulate: dpre (fp32,
// [4H x B]); the TF32 hi / lo planes of dpre (dn: rows = batch, K = 4H, same indexing as dpre - the K-major right operand
// of the dx / dh product and, read MN-major, the left operand of the weight-gradient products), which saves the packing
// pass over dpre; db += row sums, formed as per-tile partial sums that the last
// CTA of each 64-unit stripe to arrive adds in ascending tile order (deterministic; counters[] returns to zero).
constexpr int kCT_J = 64, kCT_B = 32;
// JT = hidden units per tile: 64 (two columns per thread) or, for grids that would leave most SMs idle, 32 (one column)
template <int JT>
__global__ void __launch_bounds__(256) k_lstm_cell_bwd_tiled(const float* __restrict__ c_t, const float* __restrict__ c_tm1,
                                                            const float* __restrict__ gates, const float* __restrict__ dEdh,
                                                            const float* __restrict__ dEdc, float* __restrict__ dc_tm1,
                                                            float* __restrict__ dpre, float* __restrict__ dn_hi, float* __restrict__ dn_lo,
                                                            uint32_t dn_pitch, float* __restrict__ db, float* __restrict__ part,
                                                            uint32_t* __restrict__ counters, uint32_t H, uint32_t B) {
  dyb_grid_dep_sync();
  __shared__ float tile[4][JT][kCT_B + 1];
  __shared__ uint32_t is_last;
  constexpr int kQuads = JT / 4, kLanes = 256 / kQuads, kCols = kCT_B / kLanes;   // 16 x 16 x 2 or 8 x 32 x 1
  const uint32_t j0 = blockIdx.x * JT, b0 = blockIdx.y * kCT_B;
  const uint32_t tq = threadIdx.x % kQuads, tb = threadIdx.x / kQuads;   // hidden-unit quad, batch lane
  const uint32_t j = j0 + 4 * tq;
#pragma unroll
  for (int half = 0; half < kCols; ++half) {
    const uint32_t bl = tb + kLanes * half, b = b0 + bl;
    const bool live = b < B;   // (the last tile of a batch that is not a multiple of 32 columns: zeros in, nothing out)
    const size_t e = (size_t)(live ? b : 0) * H + j;
    const float* g = gates + (size_t)(live ? b : 0) * 4 * H + j;
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 gi = live ? ld4(g) : z4, gf = live ? ld4(g + H) : z4, go = live ? ld4(g + 2 * H) : z4, gg = live ? ld4(g + 3 * H) : z4;
    const float4 c = live ? ld4(c_t + e) : z4, cp = live ? ld4(c_tm1 + e) : z4, dh = live ? ld4(dEdh + e) : z4;
    const float4 dcin = (dEdc && live) ? ld4(dEdc + e) : z4;
    float4 dcp = (dc_tm1 && live) ? ld4(dc_tm1 + e) : z4;
    float pi[4], pf[4], po[4], pg[4];
    const float gi_[4] = {gi.x, gi.y, gi.z, gi.w}, gf_[4] = {gf.x, gf.y, gf.z, gf.w}, go_[4] = {go.x, go.y, go.z, go.w},
                gg_[4] = {gg.x, gg.y, gg.z, gg.w}, c_[4] = {c.x, c.y, c.z, c.w}, cp_[4] = {cp.x, cp.y, cp.z, cp.w},
                dh_[4] = {dh.x, dh.y, dh.z, dh.w}, dci_[4] = {dcin.x, dcin.y, dcin.z, dcin.w};
    float dcp_[4] = {dcp.x, dcp.y, dcp.z, dcp.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      lstm_cell_grad(gi_[q], gf_[q], go_[q], gg_[q], c_[q], cp_[q], dh_[q], dci_[q], dEdc != nullptr, dcp_[q], pi[q], pf[q], po[q], pg[q]);
      tile[0][4 * tq + q][bl] = pi[q]; tile[1][4 * tq + q][bl] = pf[q];
      tile[2][4 * tq + q][bl] = po[q]; tile[3][4 * tq + q][bl] = pg[q];
    }
    if (dc_tm1 && live) st4(dc_tm1 + e, make_float4(dcp_[0], dcp_[1], dcp_[2], dcp_[3]));
    if (dpre && live) {
      float* o = dpre + (size_t)b * 4 * H + j;
      st4(o, make_float4(pi[0], pi[1], pi[2], pi[3])); st4(o + H, make_float4(pf[0], pf[1], pf[2], pf[3]));
      st4(o + 2 * H, make_float4(po[0], po[1], po[2], po[3])); st4(o + 3 * H, make_float4(pg[0], pg[1], pg[2], pg[3]));
    }
    if (dn_hi && live) {
      const size_t o = (size_t)b * dn_pitch + j;
      float hi[4], lo[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) split_tf32(pi[q], hi[q], lo[q]);
      st4(dn_hi + o, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(dn_lo + o, make_float4(lo[0], lo[1], lo[2], lo[3]));
#pragma unroll
      for (int q = 0; q < 4; ++q) split_tf32(pf[q], hi[q], lo[q]);
      st4(dn_hi + o + H, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(dn_lo + o + H, make_float4(lo[0], lo[1], lo[2], lo[3]));
#pragma unroll
      for (int q = 0; q < 4; ++q) split_tf32(po[q], hi[q], lo[q]);
      st4(dn_hi + o + 2 * H, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(dn_lo + o + 2 * H, make_float4(lo[0], lo[1], lo[2], lo[3]));
#pragma unroll
      for (int q = 0; q < 4; ++q) split_tf32(pg[q], hi[q], lo[q]);
      st4(dn_hi + o + 3 * H, make_float4(hi[0], hi[1], hi[2], hi[3])); st4(dn_lo + o + 3 * H, make_float4(lo[0], lo[1], lo[2], lo[3]));
    }
  }
  __syncthreads();
  // row sums: warp w takes rows w, w + 8, ... of the 256 (gate, unit) rows; lane = batch column
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t r = warp; r < 4 * JT; r += 8) {
    const uint32_t gate = r / JT, jl = r % JT;
    const float v = tile[gate][jl][lane];
    const size_t row = (size_t)gate * H + j0 + jl;
    const float s = warp_sum(v);
    if (lane == 0) part[(size_t)blockIdx.y * 4 * H + row] = s;
  }
  // the last CTA of this stripe of hidden units adds the partial sums of all batch tiles, in tile order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t seen = atomicAdd(&counters[blockIdx.x], 1u);
    is_last = seen == gridDim.y - 1;
    if (is_last) counters[blockIdx.x] = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < 4 * JT) {
    __threadfence();
    const uint32_t r = threadIdx.x;   // one thread per (gate, unit) row of the stripe
    const size_t row = (size_t)(r / JT) * H + j0 + r % JT;
    float acc = 0.f;
    uint32_t t = 0;
    for (; t + 8 <= gridDim.y; t += 8) {   // eight loads in flight, added in tile order
      float v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = __ldcg(part + (size_t)(t + q) * 4 * H + row);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc += v[q];
    }
    for (; t < gridDim.y; ++t) acc += __ldcg(part + (size_t)t * 4 * H + row);
    db[row] += acc;
  }
}

struct GatesArgs {
  unsigned k;                 // number of x inputs
  const dyb200_tensor *h, *Wx, *Wh, *b, *mx, *mh;
  uint32_t H, I, B;
};

int parse_gates(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, const dyb200_lstm_gates_attrs* a, GatesArgs* g) {
  DYB_CHECK_ARG(ctx, a != nullptr, "VanillaLSTMGates: attrs required");
  const int fixed = a->dropout ? 6 : 4;
  DYB_CHECK_ARG(ctx, nxs >= fixed + 1, "Failed input count check in VanillaLSTMGates");
  g->k = (unsigned)(nxs - fixed);
  g->h = &xs[g->k]; g->Wx = &xs[g->k + 1]; g->Wh = &xs[g->k + 2]; g->b = &xs[g->k + 3];
  g->mx = a->dropout ? &xs[g->k + 4] : nullptr;
  g->mh = a->dropout ? &xs[g->k + 5] : nullptr;
  g->H = t_dim(g->h, 0);
  g->I = t_dim(g->Wx, 1);
  g->B = xs[0].bd;
  uint32_t sum = 0;
  for (unsigned j = 0; j < g->k; ++j) {
    DYB_CHECK_ARG(ctx, xs[j].nd == 1, "VanillaLSTMGates: x_t[%u] expected to be a vector", j);
    DYB_CHECK_ARG(ctx, xs[j].bd == g->B, "VanillaLSTMGates: x_t has inconsistent batch size");
    sum += xs[j].d[0];
  }
  DYB_CHECK_ARG(ctx, sum == g->I, "VanillaLSTMGates: x_t has inconsistent dimension");
  DYB_CHECK_ARG(ctx, g->h->nd == 1 && g->h->bd == g->B, "VanillaLSTMGates: h_tm1 expected to be a vector with the batch size of x_t");
  DYB_CHECK_ARG(ctx, g->Wx->nd == 2 && g->Wx->bd == 1, "VanillaLSTMGates: Wx expected to be a matrix");
  DYB_CHECK_ARG(ctx, g->Wh->nd == 2 && g->Wh->bd == 1, "VanillaLSTMGates: Wh expected to be a matrix");
  DYB_CHECK_ARG(ctx, g->b->nd == 1 && g->b->bd == 1, "VanillaLSTMGates: b expected to be a vector");
  DYB_CHECK_ARG(ctx, g->Wx->d[0] == 4 * g->H, "VanillaLSTMGates: Wx dim 0 expected %u, was %u", 4 * g->H, g->Wx->d[0]);
  DYB_CHECK_ARG(ctx, g->Wh->d[0] == 4 * g->H, "VanillaLSTMGates: Wh dim 0 expected %u, was %u", 4 * g->H, g->Wh->d[0]);
  DYB_CHECK_ARG(ctx, g->Wh->d[1] == g->H, "VanillaLSTMGates: Wh dim 1 expected %u, was %u", g->H, g->Wh->d[1]);
  DYB_CHECK_ARG(ctx, g->b->d[0] == 4 * g->H, "VanillaLSTMGates: b dim expected %u, was %u", 4 * g->H, g->b->d[0]);
  if (a->dropout) {
    DYB_CHECK_ARG(ctx, g->mx->nd == 1 && g->mh->nd == 1, "VanillaLSTMGates: dropout masks expected to be vectors");
    DYB_CHECK_ARG(ctx, g->mx->bd == g->B || g->mx->bd == 1, "VanillaLSTMGates: dropout_mask_x expected to have batch size 1 or %u, was %u", g->B, g->mx->bd);
    DYB_CHECK_ARG(ctx, g->mh->bd == g->B || g->mh->bd == 1, "VanillaLSTMGates: dropout_mask_h expected to have batch size 1 or %u, was %u", g->B, g->mh->bd);
    DYB_CHECK_ARG(ctx, g->mx->d[0] == g->I, "VanillaLSTMGates: dropout_mask_x dim 1 expected %u, was %u", g->I, g->mx->d[0]);
    DYB_CHECK_ARG(ctx, g->mh->d[0] == g->H, "VanillaLSTMGates: dropout_mask_h dim 1 expected %u, was %u", g->H, g->mh->d[0]);
  }
  return DYB200_OK;
}

// x as one I x B matrix: the single input itself, or a concatenation built in `scratch`.
int gather_x(dyb200_ctx* ctx, const dyb200_tensor* xs, const GatesArgs& g, float* scratch, const float** x_out) {
  if (g.k == 1) { *x_out = xs[0].v; return DYB200_OK; }
  uint32_t off = 0;
  for (unsigned j = 0; j < g.k; ++j) {
    size_t total = (size_t)xs[j].d[0] * g.B;
    if (total) {
      dyb_launch(k_concat_rows, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, xs[j].v, xs[j].d[0], off, g.I, g.B, scratch);
      DYB_LAUNCHED(ctx);
    }
    off += xs[j].d[0];
  }
  *x_out = scratch;
  return DYB200_OK;
}

int ch_check(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, const char* name) {
  DYB_CHECK_ARG(ctx, nxs == 2, "Failed input count check in %s", name);
  DYB_CHECK_ARG(ctx, xs[0].nd == 1 && xs[1].nd == 1, "%s: c and gates_t expected to be vectors", name);
  DYB_CHECK_ARG(ctx, t_batch_size(&xs[0]) * 4 == t_batch_size(&xs[1]), "%s: gates_t expected 4 times as big as c_t, but %zu*4 != %zu", name, t_batch_size(&xs[0]), t_batch_size(&xs[1]));
  DYB_CHECK_ARG(ctx, xs[0].bd == xs[1].bd, "%s: gates_t and c_t expected to have equal batch size, but %u != %u", name, xs[0].bd, xs[1].bd);
  return DYB200_OK;
}

template <int MODE>
int ch_fwd(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, dyb200_tensor* fx, const char* name) {
  int rc = ch_check(ctx, xs, nxs, name);
  if (rc) return rc;
  uint32_t H = xs[0].d[0];
  size_t total = (size_t)H * xs[0].bd;
  DYB_CHECK_ARG(ctx, t_size(fx) == total, "%s: output size mismatch", name);
  if (total == 0) return DYB200_OK;
  bool vec = H % 4 == 0 && aligned16(xs[0].v) && aligned16(xs[1].v) && aligned16(fx->v);
  if (vec) dyb_launch(k_lstm_ch_fwd<MODE, 1>, stream_grid(ctx, total / 4, kThreads), kThreads, 0, ctx, xs[0].v, xs[1].v, fx->v, H, total);
  else dyb_launch(k_lstm_ch_fwd<MODE, 0>, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, xs[0].v, xs[1].v, fx->v, H, total);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}
template <int NODE>
int ch_bwd(dyb200_ctx* ctx, const dyb200_tensor* xs, int nxs, const dyb200_tensor* dEdf, unsigned i, dyb200_tensor* dEdxi,
           const char* name) {
  int rc = ch_check(ctx, xs, nxs, name);
  if (rc) return rc;
  DYB_CHECK_ARG(ctx, i < 2, "%s::backward: argument index %u out of range", name, i);
  uint32_t H = xs[0].d[0];
  size_t total = (size_t)H * xs[0].bd;
  DYB_CHECK_ARG(ctx, t_size(dEdf) == total && t_size(dEdxi) == (i == 0 ? total : 4 * total), "%s::backward: size mismatch", name);
  if (total == 0) return DYB200_OK;
  if (H % 4 == 0) dyb_launch(k_lstm_ch_bwd<NODE, 1>, stream_grid(ctx, total / 4, kThreads), kThreads, 0, ctx, xs[0].v, xs[1].v, dEdf->v, i, dEdxi->v, H, total);
  else dyb_launch(k_lstm_ch_bwd<NODE, 0>, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, xs[0].v, xs[1].v, dEdf->v, i, dEdxi->v, H, total);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

}  // namespace

extern "C" {

int dyb200_vanilla_lstm_gates_fwd(DYB200_FWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem;
  const dyb200_lstm_gates_attrs* a = (const dyb200_lstm_gates_attrs*)attrs;
  GatesArgs g;
  int rc = parse_gates(ctx, xs, nxs, a, &g);
  if (rc) return rc;
  const uint32_t G = 4 * g.H;
  DYB_CHECK_ARG(ctx, t_size(fx) == (size_t)G * g.B, "VanillaLSTMGates: output must be Dim({%u}, %u)", G, g.B);
  if ((size_t)G * g.B == 0) return DYB200_OK;
  if (a->weightnoise_std > 0.f) {
    // Reference behaviour (dynet/nodes-lstm.cc:200-219): the noisy copies are built and never used.
    size_t total = (size_t)G * g.B;
    dyb_launch(k_gates_bias_only, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, g.b->v, fx->v, g.H, total, a->forget_gate_bias);
    DYB_LAUNCHED(ctx);
    return DYB200_OK;
  }
  const float* x = nullptr;
  void* scratch = nullptr;
  if (g.k > 1) {
    rc = dyb200_scratch(ctx, (size_t)g.I * g.B * sizeof(float), &scratch);
    if (rc) return rc;
  }
  rc = gather_x(ctx, xs, g, (float*)scratch, &x);
  if (rc) return rc;
  GemmPair pairs[2] = {
      {g.Wx->v, G, 0, x, g.I, 0, g.I, g.mx ? g.mx->v : nullptr, g.I, g.mx ? g.mx->bd == g.B : 0, 1},
      {g.Wh->v, G, 0, g.h->v, g.H, 0, g.H, g.mh ? g.mh->v : nullptr, g.H, g.mh ? g.mh->bd == g.B : 0, 1}};
  GemmEpilogue epi{EPI_GATES, fx->v, G, g.b->v, g.H, a->forget_gate_bias, nullptr, 0, 0};
  return dyb200_gemm_fused(ctx, G, g.B, 2, pairs, epi);
}

int dyb200_vanilla_lstm_gates_bwd(DYB200_BWD_ARGS) {
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  (void)aux_mem;
  const dyb200_lstm_gates_attrs* a = (const dyb200_lstm_gates_attrs*)attrs;
  GatesArgs g;
  int rc = parse_gates(ctx, xs, nxs, a, &g);
  if (rc) return rc;
  const uint32_t G = 4 * g.H;
  const size_t total = (size_t)G * g.B;
  DYB_CHECK_ARG(ctx, i < g.k + 4, "VanillaLSTMGates::backward: no gradient for argument %u", i);
  DYB_CHECK_ARG(ctx, t_size(fx) == total && t_size(dEdf) == total, "VanillaLSTMGates::backward: gates size mismatch");
  if (total == 0) return DYB200_OK;
  if (i == g.k + 3) {  // db
    DYB_CHECK_ARG(ctx, t_size(dEdxi) == G, "VanillaLSTMGates::backward: db size mismatch");
    GateDerivSum f{fx->v, dEdf->v, g.H};
    return batch_reduce_add(ctx, f, G, g.B, dEdxi->v);
  }
  // scratch: dgate (G x B) [+ concatenated x (I x B)]
  size_t dg_bytes = (total * sizeof(float) + 255) & ~(size_t)255;
  bool need_x = (i == g.k + 1) && g.k > 1;
  void* scratch;
  rc = dyb200_scratch(ctx, dg_bytes + (need_x ? (size_t)g.I * g.B * sizeof(float) : 0), &scratch);
  if (rc) return rc;
  float* dg = (float*)scratch;
  int vec = g.H % 4 == 0 && aligned16(fx->v) && aligned16(dEdf->v);
  dyb_launch(k_gate_deriv, stream_grid(ctx, vec ? total / 4 : total, kThreads), kThreads, 0, ctx, fx->v, dEdf->v, dg, g.H, total, vec);
  DYB_LAUNCHED(ctx);
  if (i < g.k) {  // dx_i = Wx[:, slice_i]^T dgate (.* mask slice)
    uint32_t off = 0, di = xs[i].d[0];
    for (unsigned j = 0; j < i; ++j) off += xs[j].d[0];
    DYB_CHECK_ARG(ctx, t_size(dEdxi) == (size_t)di * g.B, "VanillaLSTMGates::backward: dx size mismatch");
    GemmPair p{g.Wx->v + (size_t)off * G, G, 1, dg, G, 0, G, nullptr, 0, 0, 1};
    GemmEpilogue e{g.mx ? EPI_ACCUM_MASK : EPI_ACCUM, dEdxi->v, di, nullptr, 0, 0.f, g.mx ? g.mx->v + off : nullptr, g.I, g.mx ? g.mx->bd == g.B : 0};
    return dyb200_gemm_fused(ctx, di, g.B, 1, &p, e);
  }
  if (i == g.k) {  // dh = Wh^T dgate (.* mask_h)
    DYB_CHECK_ARG(ctx, t_size(dEdxi) == (size_t)g.H * g.B, "VanillaLSTMGates::backward: dh size mismatch");
    GemmPair p{g.Wh->v, G, 1, dg, G, 0, G, nullptr, 0, 0, 1};
    GemmEpilogue e{g.mh ? EPI_ACCUM_MASK : EPI_ACCUM, dEdxi->v, g.H, nullptr, 0, 0.f, g.mh ? g.mh->v : nullptr, g.H, g.mh ? g.mh->bd == g.B : 0};
    return dyb200_gemm_fused(ctx, g.H, g.B, 1, &p, e);
  }
  if (i == g.k + 1) {  // dWx += dgate (x .* mask_x)^T, summed over the batch
    DYB_CHECK_ARG(ctx, t_size(dEdxi) == (size_t)G * g.I, "VanillaLSTMGates::backward: dWx size mismatch");
    const float* x = nullptr;
    rc = gather_x(ctx, xs, g, (float*)((char*)scratch + dg_bytes), &x);
    if (rc) return rc;
    GemmPair p{dg, G, 0, x, g.I, 1, g.B, g.mx ? g.mx->v : nullptr, g.I, g.mx ? g.mx->bd == g.B : 0, 0};
    GemmEpilogue e{EPI_ACCUM, dEdxi->v, G, nullptr, 0, 0.f, nullptr, 0, 0};
    return dyb200_gemm_fused(ctx, G, g.I, 1, &p, e);
  }
  // i == k + 2: dWh += dgate (h .* mask_h)^T
  DYB_CHECK_ARG(ctx, t_size(dEdxi) == (size_t)G * g.H, "VanillaLSTMGates::backward: dWh size mismatch");
  GemmPair p{dg, G, 0, g.h->v, g.H, 1, g.B, g.mh ? g.mh->v : nullptr, g.H, g.mh ? g.mh->bd == g.B : 0, 0};
  GemmEpilogue e{EPI_ACCUM, dEdxi->v, G, nullptr, 0, 0.f, nullptr, 0, 0};
  return dyb200_gemm_fused(ctx, G, g.H, 1, &p, e);
}


// ---- fused entry points: the gates -> c -> h chain of one layer and time step in fewer launches ----
int dyb200_vanilla_lstm_fwd_fused(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                  const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* b,
                                  const dyb200_tensor* mask_x, const dyb200_tensor* mask_h,
                                  const dyb200_lstm_gates_attrs* attrs, dyb200_tensor* gates, dyb200_tensor* c_t,
                                  dyb200_tensor* h_t, dyb200_ctx* ctx) {
  return dyb200_vanilla_lstm_fwd_fused_at(x, h_tm1, c_tm1, Wx, Wh, b, mask_x, mask_h, attrs, gates, c_t, h_t, nullptr, 0, ctx);
}

int dyb200_vanilla_lstm_fwd_fused_at(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                     const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* b,
                                     const dyb200_tensor* mask_x, const dyb200_tensor* mask_h,
                                     const dyb200_lstm_gates_attrs* attrs, dyb200_tensor* gates, dyb200_tensor* c_t,
                                     dyb200_tensor* h_t, dyb200_wgrad* deferred, uint32_t deferred_col, dyb200_ctx* ctx) {
  DYB_CHECK_ARG(ctx, x && h_tm1 && c_tm1 && Wx && Wh && b && attrs && gates && c_t && h_t, "lstm_fwd_fused: null argument");
  DYB_CHECK_ARG(ctx, (attrs->dropout != 0) == (mask_x != nullptr && mask_h != nullptr), "lstm_fwd_fused: masks must be given exactly when dropout is set");
  dyb200_tensor xs[7] = {*x, *h_tm1, *Wx, *Wh, *b};
  int nxs = 5;
  if (attrs->dropout) { xs[5] = *mask_x; xs[6] = *mask_h; nxs = 7; }
  const uint32_t H = c_tm1->d[0];
  const size_t total = (size_t)H * c_tm1->bd;
  DYB_CHECK_ARG(ctx, t_size(c_t) == total && t_size(h_t) == total, "lstm_fwd_fused: c_t / h_t size mismatch");
  {
    // W x + U h on the tensor pipe with interleaved gate rows, so that bias + sigmoid / tanh AND the c / h update run in
    // the product's epilogue: inside the MMA kernel when K is not split, else in the split-K reduction.
    const uint32_t I = t_dim(x, 0), B = x->bd, G = 4 * H;
    const bool shapes_ok = x->nd == 1 && h_tm1->nd == 1 && t_dim(h_tm1, 0) == H && h_tm1->bd == B && c_tm1->bd == B && Wx->nd == 2 &&
                           Wx->d[0] == G && Wx->d[1] == I && Wh->nd == 2 && Wh->d[0] == G && Wh->d[1] == H && t_size(b) == G &&
                           t_size(gates) == (size_t)G * B &&
                           (!attrs->dropout || ((mask_x->bd == B || mask_x->bd == 1) && (mask_h->bd == B || mask_h->bd == 1) &&
                                                t_dim(mask_x, 0) == I && t_dim(mask_h, 0) == H));
    const uint32_t kb = (I + 31) / 32 + (H + 31) / 32;
    (void)kb;
    if (shapes_ok && attrs->weightnoise_std == 0.f && H % 32 == 0 && I > 0 && B > 0 && dyb200_tc_eligible(G, B, 2.0 * G * B * (I + H)) &&
        aligned16(gates->v) && aligned16(b->v) && aligned16(c_tm1->v) && aligned16(c_t->v) && aligned16(h_t->v)) {
      { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
      PackedOp A[2], Bp[2];
      int rc;
      if ((rc = dyb200_tc_param_gates(ctx, Wx->v, G, G, I, &A[0]))) return rc;
      if ((rc = dyb200_tc_param_gates(ctx, Wh->v, G, G, H, &A[1]))) return rc;
      PackJobs batch;
      dyb200_tc_pack_begin(&batch);
      const float* mx = attrs->dropout ? mask_x->v : nullptr;
      const float* mh = attrs->dropout ? mask_h->v : nullptr;
      const int mx_full = mx ? mask_x->bd == B : 0, mh_full = mh ? mask_h->bd == B : 0;
      if (deferred) DYB_CHECK_ARG(ctx, dyb200_wgrad_rows(deferred) == G, "lstm_fwd_fused: the deferred accumulator has %u rows, the layer %u", dyb200_wgrad_rows(deferred), G);
      // Inputs that dyb200_wgrad_pack_inputs (x, all steps at once) or the previous step's epilogue (h) already wrote as
      // operand planes are used as they are; the others are split here, also into the weight-gradient accumulator.
      const bool x_pre = deferred && dyb200_wgrad_x_planes(deferred, deferred_col, B, &Bp[0]);
      const bool h_pre = x_pre && dyb200_wgrad_h_planes(deferred, deferred_col, B, &Bp[1]);
      if (!x_pre && (rc = dyb200_tc_pack(ctx, x->v, I, true, B, I, mx, I, mx_full, &Bp[0], &batch))) return rc;
      if (!h_pre && (rc = dyb200_tc_pack(ctx, h_tm1->v, H, true, B, H, mh, H, mh_full, &Bp[1], &batch))) return rc;
      if (deferred && !(x_pre && h_pre)) {   // the same inputs, transposed, are the B operands of this step's weight-gradient products
        if ((rc = dyb200_wgrad_push_b_at(deferred, deferred_col, B, x_pre ? nullptr : x->v, I, mx, mx_full, h_tm1->v, H, mh, mh_full, ctx, &batch))) return rc;
      }
      if ((rc = dyb200_tc_pack_flush(ctx, &batch))) return rc;
      GemmEpilogue e{EPI_LSTM_CELL, gates->v, G, b->v, H, attrs->forget_gate_bias, nullptr, 0, 0};
      e.c_prev = c_tm1->v; e.c_out = c_t->v; e.h_out = h_t->v;
      // with pre-split inputs this step's epilogue also writes h_t .* mask_h as the operand planes of the next step
      if (x_pre && (!mh || aligned16(mh)) && dyb200_wgrad_next_h(deferred, deferred_col, B, &e)) { e.hmask = mh; e.hmask_ld = H; e.hmask_full = mh_full; }
      return dyb200_tc_gemm_packed(ctx, G, B, 2, A, Bp, e);
    }
  }
  int rc = dyb200_vanilla_lstm_gates_fwd(xs, nxs, gates, attrs, nullptr, ctx);
  if (rc) return rc;
  if (deferred) {
    PackJobs batch;
    dyb200_tc_pack_begin(&batch);
    const float* mx = attrs->dropout ? mask_x->v : nullptr;
    const float* mh = attrs->dropout ? mask_h->v : nullptr;
    if ((rc = dyb200_wgrad_push_b_at(deferred, deferred_col, x->bd, x->v, t_dim(x, 0), mx, mx ? mask_x->bd == x->bd : 0, h_tm1->v,
                                     t_dim(h_tm1, 0), mh, mh ? mask_h->bd == x->bd : 0, ctx, &batch))) return rc;
    if ((rc = dyb200_tc_pack_flush(ctx, &batch))) return rc;
  }
  dyb200_tensor ch[2] = {*c_tm1, *gates};
  rc = ch_check(ctx, ch, 2, "VanillaLSTMC");
  if (rc) return rc;
  if (total == 0) return DYB200_OK;
  bool vec = H % 4 == 0 && aligned16(c_tm1->v) && aligned16(gates->v) && aligned16(c_t->v) && aligned16(h_t->v);
  if (vec) dyb_launch(k_lstm_cell_fwd<1>, stream_grid(ctx, total / 4, kThreads), kThreads, 0, ctx, c_tm1->v, gates->v, c_t->v, h_t->v, H, total);
  else dyb_launch(k_lstm_cell_fwd<0>, stream_grid(ctx, total, kThreads), kThreads, 0, ctx, c_tm1->v, gates->v, c_t->v, h_t->v, H, total);
  DYB_LAUNCHED(ctx);
  return DYB200_OK;
}

int dyb200_vanilla_lstm_bwd_fused(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                  const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* mask_x,
                                  const dyb200_tensor* mask_h, const dyb200_tensor* gates, const dyb200_tensor* c_t,
                                  const dyb200_tensor* dEdh, const dyb200_tensor* dEdc, dyb200_tensor* dx,
                                  dyb200_tensor* dh_tm1, dyb200_tensor* dc_tm1, dyb200_tensor* dWx, dyb200_tensor* dWh,
                                  dyb200_tensor* db, const dyb200_lstm_gates_attrs* attrs, dyb200_wgrad* deferred,
                                  dyb200_ctx* ctx) {
  return dyb200_vanilla_lstm_bwd_fused_at(x, h_tm1, c_tm1, Wx, Wh, mask_x, mask_h, gates, c_t, dEdh, dEdc, dx, dh_tm1, dc_tm1, dWx, dWh, db,
                                          attrs, deferred, DYB200_WGRAD_APPEND, ctx);
}

int dyb200_vanilla_lstm_bwd_fused_at(const dyb200_tensor* x, const dyb200_tensor* h_tm1, const dyb200_tensor* c_tm1,
                                     const dyb200_tensor* Wx, const dyb200_tensor* Wh, const dyb200_tensor* mask_x,
                                     const dyb200_tensor* mask_h, const dyb200_tensor* gates, const dyb200_tensor* c_t,
                                     const dyb200_tensor* dEdh, const dyb200_tensor* dEdc, dyb200_tensor* dx,
                                     dyb200_tensor* dh_tm1, dyb200_tensor* dc_tm1, dyb200_tensor* dWx, dyb200_tensor* dWh,
                                     dyb200_tensor* db, const dyb200_lstm_gates_attrs* attrs, dyb200_wgrad* deferred,
                                     uint32_t deferred_col, dyb200_ctx* ctx) {
  // deferred_col == DYB200_WGRAD_APPEND: this call appends the gate gradient AND the layer inputs to the accumulator;
  // otherwise the inputs of this step were placed at that column by dyb200_vanilla_lstm_fwd_fused_at and only the gate
  // gradient is written there.
  const bool at_col = deferred && deferred_col != DYB200_WGRAD_APPEND;
  { int rc0__ = dyb200_scratch_begin(ctx); if (rc0__) return rc0__; }
  DYB_CHECK_ARG(ctx, x && h_tm1 && c_tm1 && Wx && Wh && gates && c_t && dEdh && (deferred || (dWx && dWh)) && db && attrs, "lstm_bwd_fused: null argument");
  DYB_CHECK_ARG(ctx, (attrs->dropout != 0) == (mask_x != nullptr && mask_h != nullptr), "lstm_bwd_fused: masks must be given exactly when dropout is set");
  DYB_CHECK_ARG(ctx, attrs->weightnoise_std == 0.f, "lstm_bwd_fused: weight noise is not supported by the fused path");
  const uint32_t H = t_dim(h_tm1, 0), I = t_dim(x, 0), B = x->bd, G = 4 * H;
  DYB_CHECK_ARG(ctx, x->nd == 1 && h_tm1->nd == 1 && h_tm1->bd == B && c_tm1->bd == B && t_dim(c_tm1, 0) == H, "lstm_bwd_fused: x / h_tm1 / c_tm1 shape mismatch");
  DYB_CHECK_ARG(ctx, Wx->nd == 2 && Wx->d[0] == G && Wx->d[1] == I && Wh->nd == 2 && Wh->d[0] == G && Wh->d[1] == H, "lstm_bwd_fused: weight shape mismatch");
  const size_t HB = (size_t)H * B;
  DYB_CHECK_ARG(ctx, t_size(gates) == 4 * HB && t_size(c_t) == HB && t_size(dEdh) == HB && (!dEdc || t_size(dEdc) == HB), "lstm_bwd_fused: state size mismatch");
  DYB_CHECK_ARG(ctx, (!dx || t_size(dx) == (size_t)I * B) && (!dh_tm1 || t_size(dh_tm1) == HB) && (!dc_tm1 || t_size(dc_tm1) == HB), "lstm_bwd_fused: gradient size mismatch");
  DYB_CHECK_ARG(ctx, (deferred || (t_size(dWx) == (size_t)G * I && t_size(dWh) == (size_t)G * H)) && t_size(db) == G, "lstm_bwd_fused: parameter gradient size mismatch");
  if (attrs->dropout) DYB_CHECK_ARG(ctx, (mask_x->bd == B || mask_x->bd == 1) && (mask_h->bd == B || mask_h->bd == 1) && t_dim(mask_x, 0) == I && t_dim(mask_h, 0) == H, "lstm_bwd_fused: mask shape mismatch");
  if (HB == 0) return DYB200_OK;
  const float* mx = attrs->dropout ? mask_x->v : nullptr;
  const float* mh = attrs->dropout ? mask_h->v : nullptr;
  const int mx_full = attrs->dropout ? mask_x->bd == B : 0, mh_full = attrs->dropout ? mask_h->bd == B : 0;
  const double flops_small = 2.0 * (I < H ? I : H) * (double)B * G;
  const bool tensor_path = dyb200_tc_eligible(I < H ? I : H, B, flops_small) && dyb200_tc_eligible(G, I < H ? I : H, flops_small);
  int rc;
  PackJobs batch;   // every operand split of this call goes out in one launch
  dyb200_tc_pack_begin(&batch);
  PackedOp dn, dt, wxT, whT, xt, ht;
  // Bandwidth-shaped pass for whole tiles: it writes the split planes of the gate gradient itself.
  // (any batch size: the last 32-column tile may be partly filled; any column position in the accumulator)
  const bool tiled = tensor_path && H % kCT_J == 0 && H / kCT_J <= DYB200_DEV_COUNTERS && aligned16(c_t->v) &&
                     aligned16(c_tm1->v) && aligned16(gates->v) && aligned16(dEdh->v) && (!dEdc || aligned16(dEdc->v)) &&
                     (!dc_tm1 || aligned16(dc_tm1->v));
  float* dpre = nullptr;
  if (tiled) {
    // The planes of the gate gradient (row = batch column, K = 4H) are the right operand of the dx / dh product below and,
    // read MN-major, the left operand of the weight-gradient products: with a deferred accumulator they are written straight
    // into its A planes at this step's columns.
    if (deferred) {
      DYB_CHECK_ARG(ctx, dyb200_wgrad_rows(deferred) == G, "lstm_bwd_fused: the deferred accumulator has %u rows, the layer %u", dyb200_wgrad_rows(deferred), G);
      dn.rows = B; dn.K = G;
      if (at_col) rc = dyb200_wgrad_reserve_a_at(deferred, deferred_col, B, &dn.hi, &dn.lo, &dn.pitch, ctx);
      else rc = dyb200_wgrad_reserve(deferred, B, &dn.hi, &dn.lo, &dn.pitch, x->v, I, mx, mx_full, h_tm1->v, H, mh, mh_full, ctx, &batch);
      if (rc) return rc;
    } else {
      if ((rc = dyb200_tc_planes(ctx, B, G, &dn))) return rc;
    }
    void* pp;
    const uint32_t btiles = (B + kCT_B - 1) / kCT_B;
    if ((rc = dyb200_scratch(ctx, (size_t)btiles * G * sizeof(float), &pp))) return rc;
    // half-height tiles when full ones would leave most SMs without a CTA (small per-GPU batches)
    const bool small_grid = (H / kCT_J) * btiles < (uint32_t)ctx->sm_count && H / 32 <= DYB200_DEV_COUNTERS;
    if (small_grid)
      dyb_launch(k_lstm_cell_bwd_tiled<32>, dim3(H / 32, btiles), 256, 0, ctx,
                 c_t->v, c_tm1->v, gates->v, dEdh->v, dEdc ? dEdc->v : nullptr, dc_tm1 ? dc_tm1->v : nullptr, nullptr, dn.hi, dn.lo, dn.pitch,
                 db->v, (float*)pp, ctx->dev_flags + DYB200_DEV_COUNTER0, H, B);
    else
      dyb_launch(k_lstm_cell_bwd_tiled<kCT_J>, dim3(H / kCT_J, btiles), 256, 0, ctx,
                 c_t->v, c_tm1->v, gates->v, dEdh->v, dEdc ? dEdc->v : nullptr, dc_tm1 ? dc_tm1->v : nullptr, nullptr, dn.hi, dn.lo, dn.pitch,
                 db->v, (float*)pp, ctx->dev_flags + DYB200_DEV_COUNTER0, H, B);
    DYB_LAUNCHED(ctx);
  } else {
    void* sp;
    if ((rc = dyb200_scratch(ctx, 4 * HB * sizeof(float), &sp))) return rc;
    dpre = (float*)sp;
    dyb_launch(k_lstm_cell_bwd, (H + kJT - 1) / kJT, 256, 0, ctx, c_t->v, c_tm1->v, gates->v, dEdh->v, dEdc ? dEdc->v : nullptr,
                                                                dc_tm1 ? dc_tm1->v : nullptr, dpre, db->v, H, B);
    DYB_LAUNCHED(ctx);
    if (deferred) {
      // weight gradients: append (dgate, x .* mask_x, h .* mask_h) to the accumulator; one product at flush time
      if (at_col) rc = dyb200_wgrad_pack_a_at(deferred, deferred_col, B, dpre, G, ctx, &batch);
      else rc = dyb200_wgrad_push_batched(deferred, B, dpre, G, x->v, I, mx, mx_full, h_tm1->v, H, mh, mh_full, ctx, &batch);
      if (rc) return rc;
    }
    if (tensor_path && (rc = dyb200_tc_pack(ctx, dpre, G, true, B, G, nullptr, 0, 0, &dn, &batch))) return rc;    // rows = batch, K = 4H
  }
  if (tiled && !deferred) {   // the immediate weight-gradient products need (x .* mask_x)^T and (h .* mask_h)^T
    if ((rc = dyb200_tc_pack(ctx, x->v, I, false, I, B, mx, I, mx_full, &xt, &batch))) return rc;
    if ((rc = dyb200_tc_pack(ctx, h_tm1->v, H, false, H, B, mh, H, mh_full, &ht, &batch))) return rc;
  }
  if ((rc = dyb200_tc_pack_flush(ctx, &batch))) return rc;
  if (tensor_path) {
    // the gate gradient is split once per layout and shared by the four products
    // (K splits: those of the sequence kernel where it could run this shape, so that the two forms add the same partial
    // sums in the same order and agree bit for bit; the cost model's choice otherwise)
    LstmBwdTiling tl;
    const uint32_t fs = (tiled && attrs->weightnoise_std == 0.f && dyb200_lstm_bwd_tiling(ctx, I, H, B, &tl)) ? tl.S : 0;
    if (dx && dh_tm1) {
      // dx and dh_tm1 in one product: [Wx; Wh]^T (I + H rows) times the gate gradient, rows routed to the two tensors
      if ((rc = dyb200_tc_param2(ctx, Wx->v, I, Wh->v, H, G, true, G, &wxT))) return rc;
      GemmEpilogue e{mx ? EPI_ACCUM_MASK : EPI_ACCUM, dx->v, I, nullptr, 0, 0.f, mx, I, mx_full};
      e.split_m = I; e.C2 = dh_tm1->v; e.ldc2 = H; e.maskC2 = mh; e.maskc2_ld = H; e.maskc2_full = mh_full;
      if ((rc = dyb200_tc_gemm_packed(ctx, I + H, B, 1, &wxT, &dn, e, fs))) return rc;
    } else if (dx) {
      if ((rc = dyb200_tc_param(ctx, Wx->v, G, true, I, G, &wxT))) return rc;
      GemmEpilogue e{mx ? EPI_ACCUM_MASK : EPI_ACCUM, dx->v, I, nullptr, 0, 0.f, mx, I, mx_full};
      if ((rc = dyb200_tc_gemm_packed(ctx, I, B, 1, &wxT, &dn, e, fs))) return rc;
    } else if (dh_tm1) {
      if ((rc = dyb200_tc_param(ctx, Wh->v, G, true, H, G, &whT))) return rc;
      GemmEpilogue e{mh ? EPI_ACCUM_MASK : EPI_ACCUM, dh_tm1->v, H, nullptr, 0, 0.f, mh, H, mh_full};
      if ((rc = dyb200_tc_gemm_packed(ctx, H, B, 1, &whT, &dn, e))) return rc;
    }
    if (deferred) return DYB200_OK;
    if (tiled) {    // (the planes of the tiled pass, read MN-major; xt / ht went out with the batch above)
      dt = dn; dt.rows = G; dt.K = B; dt.mn_major = 1;
    } else {
      if ((rc = dyb200_tc_pack(ctx, dpre, G, false, G, B, nullptr, 0, 0, &dt))) return rc;   // rows = 4H, K = batch
      if ((rc = dyb200_tc_pack(ctx, x->v, I, false, I, B, mx, I, mx_full, &xt))) return rc;       // (x .* mask_x)^T : rows = I, K = batch
      if ((rc = dyb200_tc_pack(ctx, h_tm1->v, H, false, H, B, mh, H, mh_full, &ht))) return rc;
    }
    GemmEpilogue ex{EPI_ACCUM, dWx->v, G, nullptr, 0, 0.f, nullptr, 0, 0};
    if ((rc = dyb200_tc_gemm_packed(ctx, G, I, 1, &dt, &xt, ex))) return rc;
    GemmEpilogue eh{EPI_ACCUM, dWh->v, G, nullptr, 0, 0.f, nullptr, 0, 0};
    return dyb200_tc_gemm_packed(ctx, G, H, 1, &dt, &ht, eh);
  }
  // small shapes: the same four products on the CUDA-core kernel
  if (dx) {
    GemmPair p{Wx->v, G, 1, dpre, G, 0, G, nullptr, 0, 0, 1};
    GemmEpilogue e{mx ? EPI_ACCUM_MASK : EPI_ACCUM, dx->v, I, nullptr, 0, 0.f, mx, I, mx_full};
    if ((rc = dyb200_gemm_fused(ctx, I, B, 1, &p, e))) return rc;
  }
  if (dh_tm1) {
    GemmPair p{Wh->v, G, 1, dpre, G, 0, G, nullptr, 0, 0, 1};
    GemmEpilogue e{mh ? EPI_ACCUM_MASK : EPI_ACCUM, dh_tm1->v, H, nullptr, 0, 0.f, mh, H, mh_full};
    if ((rc = dyb200_gemm_fused(ctx, H, B, 1, &p, e))) return rc;
  }
  if (deferred) return DYB200_OK;
  {
    GemmPair p{dpre, G, 0, x->v, I, 1, B, mx, I, mx_full, 0};
    GemmEpilogue e{EPI_ACCUM, dWx->v, G, nullptr, 0, 0.f, nullptr, 0, 0};
    if ((rc = dyb200_gemm_fused(ctx, G, I, 1, &p, e))) return rc;
  }
  GemmPair p{dpre, G, 0, h_tm1->v, H, 1, B, mh, H, mh_full, 0};
  GemmEpilogue e{EPI_ACCUM, dWh->v, G, nullptr, 0, 0.f, nullptr, 0, 0};
  return dyb200_gemm_fused(ctx, G, H, 1, &p, e);
}

int dyb200_vanilla_lstm_c_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return ch_fwd<0>(ctx, xs, nxs, fx, "VanillaLSTMC"); }
int dyb200_vanilla_lstm_c_bwd(DYB200_BWD_ARGS) { (void)fx; (void)attrs; (void)aux_mem; return ch_bwd<0>(ctx, xs, nxs, dEdf, i, dEdxi, "VanillaLSTMC"); }
int dyb200_vanilla_lstm_h_fwd(DYB200_FWD_ARGS) { (void)attrs; (void)aux_mem; return ch_fwd<1>(ctx, xs, nxs, fx, "VanillaLSTMH"); }
int dyb200_vanilla_lstm_h_bwd(DYB200_BWD_ARGS) { (void)fx; (void)attrs; (void)aux_mem; return ch_bwd<1>(ctx, xs, nxs, dEdf, i, dEdxi, "VanillaLSTMH"); }

}  // extern "C"
