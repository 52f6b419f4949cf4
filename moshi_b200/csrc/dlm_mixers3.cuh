// Further mechanisms of the decoder-LM handle (dlm.cu), first used by the Dibulix design: pre-norm sublayers on several residual
// streams with learned read / write weights, the preparation of a latent attention whose cache row is [latent | rotated key
// part], a per-row sigmoid gate, an element-wise gated recurrence (minGRU), and the preparation of the gated delta rule with one
// decay per key channel.
//   T = activation / weight / cache type (bf16, or float in the all-fp32 mode).  The streams, norms, positions and angles,
//   gates, decays, unit norms and every recurrent state are fp32 in both modes.
#pragma once

#include "dlm_mixers2.cuh"

namespace b200 {
namespace dlm {

// x = table[token] -> every one of the S residual streams (fp32);  u = sum_s in[s] x_s (hc_in null: u = x);
// h = u / sqrt(mean(u^2) + eps) * w1 -> T.  One CTA per token; xs is [tokens][S][W].
template <typename T>
__global__ void __launch_bounds__(256) embed_streams_kernel(const int* __restrict__ tokens, const T* __restrict__ table, int vocab, int W, int S,
                                                            const float* __restrict__ hc_in, const float* __restrict__ w1, float* __restrict__ xs,
                                                            T* __restrict__ h, float eps, int* __restrict__ err) {
  extern __shared__ float u[];
  __shared__ float red[32];
  const long long t = blockIdx.x;
  int id = tokens[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad) { if (threadIdx.x == 0) atomicOr(err, ERR_TOKEN); id = 0; }
  const T* row = table + (long long)id * W;
  float a = 0.f;
  for (int s = 0; s < S; ++s) a += hc_in ? hc_in[s] : 1.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = bad ? 0.f : to_f(row[i]);
    for (int s = 0; s < S; ++s) xs[(t * S + s) * W + i] = v;
    u[i] = hc_in ? a * v : v;
  }
  __syncthreads();
  const float r = block_rrms(u, W, eps, red);
  for (int i = threadIdx.x; i < W; i += blockDim.x) h[t * W + i] = from_f<T>(u[i] * r * w1[i]);
}

// End of a pre-norm sublayer on S residual streams, one CTA per token:
//   y     = s0 * y0 (+ s1 * y1: two mixers side by side)
//   x_t  <- sum_s mix[s][t] x_s + out[t] y   for every stream t, from the old streams (mix null: the one stream gets x + y)
//   trace = sum_t x_t (per-layer dump), xsum likewise (what the output norm reads after the last sublayer)
//   u     = sum_t in_next[t] x_t;  h = u / sqrt(mean(u^2) + eps) * w_next -> T   (what the next sublayer reads)
template <typename T, int S>
__global__ void __launch_bounds__(256) streams_end_kernel(float* __restrict__ xs, const T* __restrict__ y0, float s0, const T* __restrict__ y1, float s1,
                                                          const float* __restrict__ mix, const float* __restrict__ out, float* __restrict__ trace,
                                                          float* __restrict__ xsum, const float* __restrict__ in_next, const float* __restrict__ w_next,
                                                          T* __restrict__ h, int W, float eps) {
  extern __shared__ float u[];
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float m[S][S], o[S], a[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    o[s] = out ? out[s] : 1.f;
    a[s] = in_next ? in_next[s] : 1.f;
#pragma unroll
    for (int q = 0; q < S; ++q) m[s][q] = mix ? mix[s * S + q] : (s == q ? 1.f : 0.f);
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float y = s0 * to_f(y0[t * W + i]);
    if (y1) y = fmaf(s1, to_f(y1[t * W + i]), y);
    float old[S], sum = 0.f, un = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) old[s] = xs[(t * S + s) * W + i];
#pragma unroll
    for (int q = 0; q < S; ++q) {
      float v = o[q] * y;
#pragma unroll
      for (int s = 0; s < S; ++s) v = fmaf(m[s][q], old[s], v);
      xs[(t * S + q) * W + i] = v;
      sum += v;
      un = fmaf(a[q], v, un);
    }
    if (trace) trace[t * W + i] = sum;
    if (xsum) xsum[t * W + i] = sum;
    u[i] = un;
  }
  if (w_next) {
    __syncthreads();
    const float r = block_rrms(u, W, eps, red);
    for (int i = threadIdx.x; i < W; i += blockDim.x) h[t * W + i] = from_f<T>(u[i] * r * w_next[i]);
  }
}

// Preparation of the latent attention with a rotated part, one CTA per token, on the projections proj T [tokens][ld]
// (q at off_q: H heads of [dim unrotated | rd rotated]; dkv at off_dkv: r latent elements, then rd of the rotated key part):
//   cache row [rp] <- [ rms_norm(latent) * w | rope(rotated key part) | zeros ]
//   qa[t][h][r .. r + rd) <- rope(rotated query part of head h) * scale, zeros up to rp
// (the first r elements of a qa row are the query folded through W_uk, written by a product of its own).  Rotation by halves or
// adjacent pairs over all rd dimensions, angle pos * freq[i], cos and sin times amp.
template <typename T>
__global__ void __launch_bounds__(128) latent_rope_append_kernel(const T* __restrict__ proj, long long ld, int off_q, int off_dkv, const float* __restrict__ w,
                                                                 T* __restrict__ cache, int cap, int r, int rd, int rp, int H, int dim, int adjacent,
                                                                 const double* __restrict__ freq, float amp, float scale, float* __restrict__ qa,
                                                                 const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, float eps) {
  extern __shared__ float rot[];        // [rd / 2] cosines, [rd / 2] sines
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int pos = tok_pos[t], half = rd / 2;
  const T* row = proj + t * ld;
  rotary_fill(rot, half, pos, freq, amp);
  float s = 0.f;
  for (int i = threadIdx.x; i < r; i += blockDim.x) { const float v = to_f(row[off_dkv + i]); s += v * v; }
  const float rs = 1.f / sqrtf(block_sum(s, red) / (float)r + eps);      // block_sum synchronises: rot is complete below
  T* dst = cache + ((long long)tok_slot[t] * cap + pos) * rp;
  for (int i = threadIdx.x; i < rp; i += blockDim.x) {
    float v = 0.f;
    if (i < r) v = to_f(row[off_dkv + i]) * rs * w[i];
    else if (i < r + rd) v = rotary_at(row + off_dkv + r, i - r, half, adjacent, rot);
    dst[i] = from_f<T>(v);
  }
  const int tail = rp - r;
  for (int i = threadIdx.x; i < H * tail; i += blockDim.x) {
    const int hh = i / tail, d = i - hh * tail;
    qa[(t * H + hh) * rp + r + d] = d < rd ? rotary_at(row + off_q + hh * (dim + rd) + dim, d, half, adjacent, rot) * scale : 0.f;
  }
}

// minGRU over the step's portions: per channel S <- (1 - z) S + z c with z = sigmoid(pz + bz), c = u + 1/2 where u = px + bx >= 0
// and sigmoid(u) below; out = S * silu(pg) -> T.  The state [slots][N] is fp32, starts from zero at position 0 and is carried
// between steps.  A CTA owns 32 channels of one portion; its warps cut the portion's tokens into segments that run side by
// side: the recurrence is linear in S, so a segment's end is A S_start + B with A = prod (1 - z) and B its end from zero.  Pass 1
// leaves (A, B) per segment, every warp folds the segments in front of it into its own start state, pass 2 walks the segment
// again and writes the results.  Grid: (ceil(N / 32), entries), block (32, warps).
template <typename T>
__global__ void __launch_bounds__(1024, 1) mingru_kernel(const T* __restrict__ proj, long long ld, int off_z, int off_x, int off_g, const float* __restrict__ bz,
                                                      const float* __restrict__ bx, float* __restrict__ state, T* __restrict__ out, long long ld_out, int N,
                                                      const int* __restrict__ ent_tok0, const int* __restrict__ ent_ntok, const int* __restrict__ ent_slot,
                                                      const int* __restrict__ ent_pos0) {
  __shared__ float sa[32][32], sb[32][32];
  const int lane = threadIdx.x, w = threadIdx.y, nw = blockDim.y, ent = blockIdx.y;
  const int c = blockIdx.x * 32 + lane;
  const bool live = c < N;
  const int tok0 = ent_tok0[ent], nt = ent_ntok[ent];
  const int len = (nt + nw - 1) / nw, t0 = min(nt, w * len), t1 = min(nt, t0 + len);
  const float bzc = live && bz ? bz[c] : 0.f, bxc = live && bx ? bx[c] : 0.f;
  float a = 1.f, b = 0.f;
  if (live && nw > 1) {
#pragma unroll 8
    for (int i = t0; i < t1; ++i) {      // the loads do not depend on the state, so several tokens' loads may be in flight at once
      const T* row = proj + (long long)(tok0 + i) * ld;
      const float z = sigmoidf(to_f(row[off_z + c]) + bzc);
      const float u = to_f(row[off_x + c]) + bxc;
      b = fmaf(z, (u >= 0.f ? u + 0.5f : sigmoidf(u)) - b, b);
      a *= 1.f - z;
    }
  }
  sa[w][lane] = a; sb[w][lane] = b;
  __syncthreads();
  if (!live) return;
  float* sp = state + (long long)ent_slot[ent] * N + c;
  float S = ent_pos0[ent] > 0 ? *sp : 0.f;
  for (int u = 0; u < w; ++u) S = fmaf(sa[u][lane], S, sb[u][lane]);
#pragma unroll 8
  for (int i = t0; i < t1; ++i) {
    const T* row = proj + (long long)(tok0 + i) * ld;
    const float z = sigmoidf(to_f(row[off_z + c]) + bzc);
    const float u = to_f(row[off_x + c]) + bxc;
    S = fmaf(z, (u >= 0.f ? u + 0.5f : sigmoidf(u)) - S, S);
    out[(long long)(tok0 + i) * ld_out + c] = from_f<T>(S * siluf(to_f(row[off_g + c])));
  }
  if (t1 == nt && t0 < t1) *sp = S;      // the warp that owns the portion's last token
}

// Preparation of the gated delta rule with one decay per head and key channel for matrix_memory_scan_kernel<MODE_CHDELTA>, one
// CTA per token, on the convolved projections c fp32 [tokens][2 * G * dim + heads * vdim] (q, k, v before their activation):
//   q <- unit(silu(q)) * qscale,  k <- unit(silu(k))   per query/key head, unit(x) = x / sqrt(sum x^2 + 1e-6);
//   value head h reads query/key head h / (heads / G);   v <- silu(v);
//   g[h][d] = exp(-exp(A_log[h]) * softplus(za[h * dim + d] + dt_bias[h * dim + d])),  beta[h] = sigmoid(zb[h])
// prep row of (token, head): [q | k | g | beta] (plain or lane-ordered, as scan_prep_kernel lays rows out).
__global__ void __launch_bounds__(256) chdelta_prep_kernel(ScanParams p, const float* __restrict__ conv, int G, const float* __restrict__ A_log,
                                                           const float* __restrict__ dt_bias, const float* __restrict__ za, const float* __restrict__ zb,
                                                           long long ldzb, int store_log) {      // store_log: log g instead of g (the chunked form sums them)
  extern __shared__ float rinv[];       // [2 * G] inverse lengths of the q and k heads
  const long long t = blockIdx.x;
  const int heads = p.heads, dim = p.dim, vdim = p.vdim, rep = heads / G;
  const int C = 2 * G * dim + heads * vdim;
  const float* c = conv + t * C;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int u = warp; u < 2 * G; u += 8) {
    float s = 0.f;
    for (int d = lane; d < dim; d += 32) { const float v = siluf(c[u * dim + d]); s += v * v; }
    s = warp_sum(s);
    if (lane == 0) rinv[u] = 1.f / sqrtf(s + 1e-6f);
  }
  __syncthreads();
  const int R = p.rows, Dp = p.lpc > 0 ? p.lpc * p.rows : dim;
  float* dst = p.prep + t * heads * p.prow;
  for (int i = threadIdx.x; i < heads * Dp; i += 256) {
    const int h = i / Dp, d = i - h * Dp, g = h / rep;
    int at = d;
    if (p.lpc > 0) { const int gg = d / R, w = d - gg * R; at = ((w >> 2) * p.lpc + gg) * 4 + (w & 3); }
    float* o = dst + h * p.prow;
    const bool live = d < dim;
    o[at] = live ? siluf(c[g * dim + d]) * rinv[g] * p.qscale : 0.f;
    o[Dp + at] = live ? siluf(c[(G + g) * dim + d]) * rinv[G + g] : 0.f;
    const float lg = live ? -expf(A_log[h]) * softplusf(za[t * heads * dim + h * dim + d] + dt_bias[h * dim + d]) : 0.f;
    o[2 * Dp + at] = store_log ? lg : (live ? expf(lg) : 0.f);
  }
  for (int h = threadIdx.x; h < heads; h += 256) dst[h * p.prow + 3 * Dp] = sigmoidf(zb[t * ldzb + h]);
  for (int i = threadIdx.x; i < heads * vdim; i += 256) p.vprep[t * heads * vdim + i] = siluf(c[2 * G * dim + i]);
}

// The chunked delta rule (dlm_mixers2.cuh) with one decay per key channel.  With L_t[d] the chunk's running sum of log g[d]:
//   A[t][i] = beta_t sum_d k_t[d] k_i[d] e^(L_t[d] - L_i[d])  (i < t),    P[t][i] = sum_d q_t[d] k_i[d] e^(L_t[d] - L_i[d])  (i <= t)
//   b_t = beta_t (v_t - S_0^T (e^(L_t) k_t)),  o_t = S_0^T (e^(L_t) q_t) + sum_i P[t][i] u_i,  S_end = e^(L_end) S_0 + sum_t (e^(L_end - L_t) k_t) u_t^T
// so the walk is the scalar one on three row sets per token (rows3) with unit scalar factors, and a decay per state row at the
// chunk's end (gend).  Every exponent is <= 0.  One CTA per (chunk, head), off the chain; prep rows are plain: q | k | log g | beta.
__global__ void __launch_bounds__(256) chdelta_gram_kernel(DeltaChunkParams p) {
  constexpr int C = DELTA_CH;
  extern __shared__ float gsm[];
  const int ck = blockIdx.x, head = blockIdx.y, dim = p.dim, DS = dim + 1;
  float* ks = gsm;                     // [C][DS]
  float* qs = ks + C * DS;             // [C][DS]
  float* Ls = qs + C * DS;             // [C][DS] running sums of log g
  float* be = Ls + C * DS;             // [C]
  float* As = be + C;                  // [C][C]
  const int tok0 = p.chunk_tok0[ck], nt = p.chunk_nt[ck];
  for (int i = threadIdx.x; i < C * dim; i += 256) {
    const int t = i / dim, d = i - t * dim;
    const float* row = p.prep + ((long long)(tok0 + t) * p.heads + head) * p.prow;
    qs[t * DS + d] = t < nt ? row[d] : 0.f;
    ks[t * DS + d] = t < nt ? row[dim + d] : 0.f;
    Ls[t * DS + d] = t < nt ? row[2 * dim + d] : 0.f;
  }
  if (threadIdx.x < C) be[threadIdx.x] = threadIdx.x < nt ? p.prep[((long long)(tok0 + threadIdx.x) * p.heads + head) * p.prow + 3 * dim] : 0.f;
  __syncthreads();
  for (int d = threadIdx.x; d < dim; d += 256) {
    float acc = 0.f;
    for (int t = 0; t < C; ++t) { acc += Ls[t * DS + d]; Ls[t * DS + d] = acc; }
  }
  __syncthreads();
  float* g = p.gram + ((long long)ck * p.heads + head) * (2 * C + 2 * C * C);
  if (threadIdx.x < C) { g[threadIdx.x] = 0.f; g[C + threadIdx.x] = be[threadIdx.x]; }      // no scalar decay: the walk's e^(L) factors are 1
  g += C;
  // the rows the walk takes, and the state's decay over the chunk
  for (int i = threadIdx.x; i < nt * dim; i += 256) {
    const int t = i / dim, d = i - t * dim;
    const float lt = Ls[t * DS + d], e = expf(lt);
    float* r3 = p.rows3 + ((long long)(tok0 + t) * p.heads + head) * 3 * dim;
    r3[d] = e * qs[t * DS + d];
    r3[dim + d] = e * ks[t * DS + d];
    r3[2 * dim + d] = expf(Ls[(nt - 1) * DS + d] - lt) * ks[t * DS + d];
  }
  for (int d = threadIdx.x; d < dim; d += 256) p.gend[((long long)ck * p.heads + head) * dim + d] = expf(Ls[(nt - 1) * DS + d]);
  for (int i = threadIdx.x; i < C * C; i += 256) {
    const int t = i / C, j = i - t * C;
    float a = 0.f, pq = 0.f;
    if (j <= t && t < nt) {
      float kk = 0.f, kq = 0.f;
      if (j == t) {
        for (int d = 0; d < dim; ++d) kq = fmaf(ks[j * DS + d], qs[t * DS + d], kq);
      } else {
        for (int d = 0; d < dim; ++d) {
          const float kd = ks[j * DS + d] * expf(Ls[t * DS + d] - Ls[j * DS + d]);
          kk = fmaf(ks[t * DS + d], kd, kk);
          kq = fmaf(qs[t * DS + d], kd, kq);
        }
      }
      pq = kq;
      if (j < t) a = be[t] * kk;
    }
    As[i] = a;
    g[C + C * C + i] = pq;
  }
  __syncthreads();
  // T = (I + A)^-1, unit lower triangular: lane j of warp 0 solves (I + A) x = e_j by forward substitution
  if (threadIdx.x < C) {
    const int j = threadIdx.x;
    float x[C];
#pragma unroll
    for (int t = 0; t < C; ++t) {
      float acc = t == j ? 1.f : 0.f;
#pragma unroll
      for (int i = 0; i < t; ++i) acc = fmaf(-As[t * C + i], x[i], acc);
      x[t] = acc;
      g[C + t * C + j] = acc;
    }
  }
}

// rows of logits times a constant: bf16 rows with a padded stride (in_bf given) or fp32 in place -> fp32 [rows][V]
__global__ void scale_rows_kernel(const bf16* __restrict__ in_bf, long long ld, float* __restrict__ out, int V, long long n, float scale) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const long long row = i / V;
  const float v = in_bf ? __bfloat162float(in_bf[row * ld + (i - row * V)]) : out[i];
  out[i] = v * scale;
}

__global__ void identity_kernel(float* __restrict__ m, int n) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n * n) m[i] = (i / n == i % n) ? 1.f : 0.f;
}

}  // namespace dlm
}  // namespace b200
