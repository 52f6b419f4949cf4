// Further mechanisms of the decoder-LM handle (dlm.cu), first used by the Govuvik design: RMS-norm sandwiches around every
// sublayer, per-channel causal convolutions with carried inputs, rotary positions with wavelength-dependent rescaling,
// sliding-window attention whose heads' scores are mixed before the softmax (with a sink), two recurrent matrix memories
// (per-channel decay; stabilised exponential gates), and a routed mixture of experts.
//   T = activation / weight / cache type (bf16, or float in the all-fp32 mode).  Norms, positions and angles, scores and
//   softmax, routers, gates, decays, the recurrent state and the residual stream are fp32 in both modes.
#pragma once

#include "dlm_kernels.cuh"

namespace b200 {
namespace dlm {

__device__ __forceinline__ float siluf(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float log_sigmoidf(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// rms-normalises one fp32 row held in shared memory (or global): returns 1 / sqrt(mean(x^2) + eps)
__device__ __forceinline__ float block_rrms(const float* __restrict__ x, int W, float eps, float* red) {
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += x[i] * x[i];
  return 1.f / sqrtf(block_sum(s, red) / (float)W + eps);
}

// x = rms_norm(table[token]) * w_embed -> residual stream; h = rms_norm(x) * w_next -> what the first layer reads (fp32)
template <typename T>
__global__ void __launch_bounds__(256) embed_norm_kernel(const int* __restrict__ tokens, const T* __restrict__ table, int vocab, int W,
                                                         const float* __restrict__ w_embed, const float* __restrict__ w_next,
                                                         float* __restrict__ xin, float* __restrict__ h, float eps, int* __restrict__ err) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  int id = tokens[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad) { if (threadIdx.x == 0) atomicOr(err, ERR_TOKEN); id = 0; }
  const T* row = table + (long long)id * W;
  float* x = xin + t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) x[i] = bad ? 0.f : to_f(row[i]);
  __syncthreads();
  const float r0 = block_rrms(x, W, eps, red);
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += blockDim.x) x[i] = x[i] * r0 * w_embed[i];
  __syncthreads();
  const float r1 = block_rrms(x, W, eps, red);
  for (int i = threadIdx.x; i < W; i += blockDim.x) h[t * W + i] = x[i] * r1 * w_next[i];
}

// out[row] = rms_norm(x[rows ? rows[row] : row]) * w
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                                           T* __restrict__ out, int W, float eps) {
  __shared__ float red[32];
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* xr = x + src * W;
  const float r = block_rrms(xr, W, eps, red);
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[(long long)blockIdx.x * W + i] = from_f<T>(xr[i] * r * w[i]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Causal convolution over time on every channel, with the last taps - 1 inputs of a sequence carried between steps.
//   y[t][c] = (residual ? u[t][c] : 0) + sum_j w[c][j] * u[t - taps + 1 + j][c],  inputs before position 0 are zero
// The step's tokens are rows of `in`; a tap that reaches in front of the step's first token of the request reads the carried
// inputs hist[slot][p mod (taps - 1)][c] (p = absolute position).  The carried inputs are written by conv_carry_kernel AFTER
// this kernel, so that no token of the step reads a row that another one has replaced.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) causal_conv_kernel(const TI* __restrict__ in, long long ld_in, const float* __restrict__ hist,
                                                          const float* __restrict__ w, TO* __restrict__ out, long long ld_out, int C,
                                                          int taps, int residual, const int* __restrict__ tok_slot,
                                                          const int* __restrict__ tok_pos, const int* __restrict__ tok_first) {
  const long long t = blockIdx.x;
  const int pos = tok_pos[t], slot = tok_slot[t], back_in_step = (int)t - tok_first[t];   // tokens of this request in front of t
  const int keep = taps - 1;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float u = to_f(in[t * ld_in + c]);
    if (w == nullptr) { out[t * ld_out + c] = from_f<TO>(u); continue; }      // no convolution: the values pass as they are
    float acc = w[(long long)c * taps + keep] * u;
    for (int b = 1; b <= keep; ++b) {
      if (b > pos) break;                                  // in front of the sequence: zero
      const float v = b <= back_in_step ? to_f(in[(t - b) * ld_in + c]) : hist[((long long)slot * keep + (pos - b) % keep) * C + c];
      acc = fmaf(w[(long long)c * taps + keep - b], v, acc);
    }
    out[t * ld_out + c] = from_f<TO>(residual ? u + acc : acc);
  }
}

// the last taps - 1 inputs of every request of the step go into its carried rows (by position mod (taps - 1))
template <typename TI>
__global__ void __launch_bounds__(256) conv_carry_kernel(const TI* __restrict__ in, long long ld_in, float* __restrict__ hist, int C, int keep,
                                                         const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                                         const int* __restrict__ tok_last) {
  const long long t = blockIdx.x;
  if (tok_last[t] - (int)t >= keep) return;                // not among the request's last taps - 1 tokens of this step
  float* dst = hist + ((long long)tok_slot[t] * keep + tok_pos[t] % keep) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] = to_f(in[t * ld_in + c]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Query / key preparation of the window attention, one CTA per token, on the convolved projections qkv fp32 [T][Nq + Nk + Nv]:
//   q <- rope(rms_norm(q over all Nq) * wq)   (kept in place, fp32: the scores are fp32 products)
//   k <- rope(rms_norm(k over all Nk) * wk)   -> key cache row of the token;  v -> value cache row
// Rotary: the first 2 * half dimensions of every head, dimension i with i + half, angle = pos * freq[i]; the angle and its sine
// and cosine are evaluated in double once per (token, i) so that a position in the thousands costs no digits, then kept as fp32.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(float* __restrict__ qkv, long long ld, int Nq, int Nk, int Nv, int dim, int half,
                                                           const float* __restrict__ wq, const float* __restrict__ wk,
                                                           const double* __restrict__ freq, T* __restrict__ kcache, T* __restrict__ vcache,
                                                           int cap, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, float eps) {
  __shared__ float red[32];
  extern __shared__ float rot[];        // [half] cosines, [half] sines
  const long long t = blockIdx.x;
  float* q = qkv + t * ld;
  float* k = q + Nq;
  const float* v = k + Nk;
  const int pos = tok_pos[t];
  const long long crow = (long long)tok_slot[t] * cap + pos;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, cs;
    sincos((double)pos * freq[i], &sn, &cs);
    rot[i] = (float)cs; rot[half + i] = (float)sn;
  }
  const float rq = block_rrms(q, Nq, eps, red);
  __syncthreads();
  const float rk = block_rrms(k, Nk, eps, red);
  // every (head, i < half) pair or unrotated element is owned by one thread: no hazards in place
  for (int e = threadIdx.x; e < Nq; e += blockDim.x) {
    const int d = e % dim;
    if (d < half) {
      const float cs = rot[d], sn = rot[half + d];
      const float a = q[e] * rq * wq[e], b = q[e + half] * rq * wq[e + half];
      q[e] = a * cs - b * sn;
      q[e + half] = b * cs + a * sn;
    } else if (d >= 2 * half) {
      q[e] = q[e] * rq * wq[e];
    }
  }
  T* kc = kcache + crow * Nk;
  for (int e = threadIdx.x; e < Nk; e += blockDim.x) {
    const int d = e % dim;
    if (d < half) {
      const float cs = rot[d], sn = rot[half + d];
      const float a = k[e] * rk * wk[e], b = k[e + half] * rk * wk[e + half];
      kc[e] = from_f<T>(a * cs - b * sn);
      kc[e + half] = from_f<T>(b * cs + a * sn);
    } else if (d >= 2 * half) {
      kc[e] = from_f<T>(k[e] * rk * wk[e]);
    }
  }
  T* vc = vcache + crow * Nv;
  for (int e = threadIdx.x; e < Nv; e += blockDim.x) vc[e] = from_f<T>(v[e]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Sliding-window attention with grouped keys / values, mixed heads and a sink.  A tile is up to QT consecutive tokens of ONE
// request with all H query heads (the mix needs every head's score of a (token, key) pair in one place).
//   raw[h][j] = q_h . k_{h / (H / G)}[j]                            fp32
//   s[h][j]   = sum_g mix[h][g] * raw[g][j]                         mix = talk[h][g] * temp[g] * scale, folded at load
//   token at position p sees keys j with 0 <= p - j < window
//   p[h][j]   = exp(s[h][j]) / (exp(sink[h]) + sum_j' exp(s[h][j']))  online over key tiles of KT keys, state (m, l) starts at (sink, 1)
//   out[h]    = sum_j p[h][j] v_{h / (H / G)}[j]
// nsplit > 1 (grid.y): the tile's key tiles are dealt over the splits, which leave (m, l, unnormalised sums) per (token, head)
// row for latent_attn_merge_kernel; the sink enters in split 0 only.
// ---------------------------------------------------------------------------------------------------------------------------
struct WindowAttnParams {
  const float* q;           // [tokens][ldq], the H * dim query values first
  long long ldq;
  const void* kcache;       // T [slots][cap][G * dim]
  const void* vcache;       // T [slots][cap][G * vdim]
  const float* mix;         // [H][H]
  const float* sink;        // [H]
  const int* tile_row0;     // first (token, head) row of the tile = first token * H
  const int* tile_rows;     // rows of the tile = tokens * H
  const int* tile_slot;
  const int* tok_pos;
  void* out;                // T [tokens][H * vdim]
  float* part;              // nsplit > 1: [tile][split][QT * H][vdim + 2]
  int cap, H, G, dim, vdim, window, QT, KT, nsplit, kstride;      // kstride: elements between staged key rows (odd number of words)
  int vec;                  // key and value rows are multiples of 16 bytes: staged with 16-byte loads
};

template <typename T>
__global__ void __launch_bounds__(256) window_attn_kernel(WindowAttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, G = p.G, dim = p.dim, vdim = p.vdim, QT = p.QT, KT = p.KT, rep = H / G;
  const int Nq = H * dim, Nk = G * dim, Nv = G * vdim, KS = KT + 1;
  float* qs = reinterpret_cast<float*>(smem_raw);                  // [QT][Nq]
  float* oacc = qs + QT * Nq;                                      // [QT][H * vdim]
  float* sraw = oacc + QT * H * vdim;                              // [QT * H][KS]
  float* sp = sraw + QT * H * KS;                                  // [QT * H][KS] mixed scores, then weights
  float* mixs = sp + QT * H * KS;                                  // [H][H]
  float* rm = mixs + H * H;                                        // [QT * H] running maximum
  float* rl = rm + QT * H;                                         // [QT * H] running sum
  float* rc = rl + QT * H;                                         // [QT * H] rescale factor of the current key tile
  T* vs = reinterpret_cast<T*>(smem_raw + (((size_t)((rc + QT * H) - qs) * 4 + 15) / 16) * 16);     // [KT][Nv], on 16 bytes
  T* ks = vs + (size_t)KT * Nv;                                    // [KT][kstride]
  const int tile = blockIdx.x, split = blockIdx.y;
  const int tok0 = p.tile_row0[tile] / H, nt = p.tile_rows[tile] / H;
  const int p0 = p.tok_pos[tok0];                                  // positions p0 .. p0 + nt - 1
  const T* kc = static_cast<const T*>(p.kcache) + (long long)p.tile_slot[tile] * p.cap * Nk;
  const T* vc = static_cast<const T*>(p.vcache) + (long long)p.tile_slot[tile] * p.cap * Nv;
  const int kmin = max(0, p0 - p.window + 1), kmax = p0 + nt - 1;
  const int n_kt = (kmax - kmin) / KT + 1;
  const int per = (n_kt + p.nsplit - 1) / p.nsplit;
  const int kt0 = split * per, kt1 = min(n_kt, kt0 + per);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < QT * Nq; i += 256) {
    const int qt = i / Nq;
    qs[i] = qt < nt ? p.q[(long long)(tok0 + qt) * p.ldq + (i - qt * Nq)] : 0.f;
  }
  for (int i = threadIdx.x; i < QT * H * vdim; i += 256) oacc[i] = 0.f;
  for (int i = threadIdx.x; i < H * H; i += 256) mixs[i] = p.mix[i];
  for (int i = threadIdx.x; i < QT * H; i += 256) {
    if (split == 0) { rm[i] = p.sink[i % H]; rl[i] = 1.f; }        // the sink: one unit of weight at logit sink[h], no value
    else { rm[i] = -INFINITY; rl[i] = 0.f; }
  }

  for (int kt = kt0; kt < kt1; ++kt) {
    const int kb = kmin + kt * KT;
    const int nk = min(KT, kmax + 1 - kb);
    __syncthreads();
    if (p.vec) {        // rows start on 16 bytes in the cache: 16-byte loads, 4-byte stores into the (odd-word strided) key rows
      const int kw = Nk * (int)sizeof(T) / 16, vw = Nv * (int)sizeof(T) / 16;
      const uint4* k4 = reinterpret_cast<const uint4*>(kc + (long long)kb * Nk);
      const uint4* v4 = reinterpret_cast<const uint4*>(vc + (long long)kb * Nv);
      uint32_t* ksw = reinterpret_cast<uint32_t*>(ks);
      const int kstw = p.kstride * (int)sizeof(T) / 4;
#pragma unroll 4
      for (int i = threadIdx.x; i < nk * kw; i += 256) {
        const int j = i / kw, e = i - j * kw;
        const uint4 v = k4[i];
        uint32_t* d = ksw + j * kstw + e * 4;
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
      }
#pragma unroll 4
      for (int i = threadIdx.x; i < nk * vw; i += 256) reinterpret_cast<uint4*>(vs)[i] = v4[i];
    } else {
      for (int i = threadIdx.x; i < nk * Nk; i += 256) { const int j = i / Nk, e = i - j * Nk; ks[j * p.kstride + e] = kc[(long long)(kb + j) * Nk + e]; }
      for (int i = threadIdx.x; i < nk * Nv; i += 256) vs[i] = vc[(long long)kb * Nv + i];
    }
    __syncthreads();
    // raw scores: item (row = qt * H + h, key j), keys fastest
    for (int i = threadIdx.x; i < QT * H * KT; i += 256) {
      const int row = i / KT, j = i - row * KT;
      float acc = 0.f;
      if (j < nk && row / H < nt) {
        const float* qv = qs + (row / H) * Nq + (row % H) * dim;
        const T* kv = ks + j * p.kstride + ((row % H) / rep) * dim;
        for (int d = 0; d < dim; ++d) acc = fmaf(qv[d], to_f(kv[d]), acc);
      }
      sraw[row * KS + j] = acc;
    }
    __syncthreads();
    // mix over heads, mask, online softmax: one warp per row, lanes over keys
    for (int row = warp; row < nt * H; row += 8) {
      const int qt = row / H, h = row - qt * H;
      const int pos = p0 + qt;
      float mx = -INFINITY;
      for (int j = lane; j < KT; j += 32) {
        float s = -INFINITY;
        const int kj = kb + j;
        if (j < nk && qt < nt && kj <= pos && pos - kj < p.window) {
          s = 0.f;
          for (int g = 0; g < H; ++g) s = fmaf(mixs[h * H + g], sraw[(qt * H + g) * KS + j], s);
        }
        sp[row * KS + j] = s;
        mx = fmaxf(mx, s);
      }
      mx = warp_max(mx);
      const float mo = rm[row], mn = fmaxf(mo, mx);
      float sum = 0.f;
      for (int j = lane; j < KT; j += 32) {
        const float s = sp[row * KS + j];
        const float w = s > -INFINITY ? expf(s - mn) : 0.f;
        sp[row * KS + j] = w;
        sum += w;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float corr = mn > -INFINITY ? expf(mo - mn) : 1.f;  // mo = -inf, mn finite -> 0; both -inf: nothing seen yet
        rc[row] = corr;
        rl[row] = rl[row] * corr + sum;
        rm[row] = mn;
      }
    }
    __syncthreads();
    // weighted sum of the values: item (row, c), c fastest
    for (int i = threadIdx.x; i < nt * H * vdim; i += 256) {
      const int row = i / vdim, c = i - row * vdim;
      const T* vv = vs + ((row % H) / rep) * vdim + c;
      const float* w = sp + row * KS;
      float acc = oacc[i] * rc[row];
      for (int j = 0; j < nk; ++j) acc = fmaf(w[j], to_f(vv[j * Nv]), acc);
      oacc[i] = acc;
    }
  }
  __syncthreads();
  if (p.nsplit == 1) {
    T* out = static_cast<T*>(p.out);
    for (int i = threadIdx.x; i < nt * H * vdim; i += 256) out[(long long)tok0 * H * vdim + i] = from_f<T>(oacc[i] / rl[i / vdim]);
  } else {
    float* dst = p.part + ((long long)tile * p.nsplit + split) * (QT * H) * (vdim + 2);
    for (int i = threadIdx.x; i < nt * H * vdim; i += 256) { const int row = i / vdim; dst[(long long)row * (vdim + 2) + (i - row * vdim)] = oacc[i]; }
    for (int row = threadIdx.x; row < nt * H; row += 256) { dst[(long long)row * (vdim + 2) + vdim] = rm[row]; dst[(long long)row * (vdim + 2) + vdim + 1] = rl[row]; }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores for bf16 caches (dim and vdim multiples of 16): a tile is 16 consecutive tokens of one
// request with all H heads, a key tile 32 keys.  Per key tile: (1) raw scores Q_h K_g^T per head as mma.sync m16n8k16 (queries
// rounded to bf16 once, fp32 accumulate) into shared memory; (2) head mix, window mask and online softmax in fp32, one warp
// per (head, token) row, the weights going back as bf16; (3) O_h += P_h V_g on the tensor cores, the accumulators of a warp's
// NI items (head, 64 value columns) in registers.  Split keys and the sink as in window_attn_kernel; rows of `part` are
// (token, head) pairs, head fastest, as latent_attn_merge_kernel wants them.
// ---------------------------------------------------------------------------------------------------------------------------
template <int NI>
__global__ void __launch_bounds__(256) window_attn_mma_kernel(WindowAttnParams p) {
  constexpr int QT = 16, KT = 32, SS = 40, PS = 40;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, G = p.G, dim = p.dim, vdim = p.vdim, rep = H / G;
  const int Nq = H * dim, Nk = G * dim, Nv = G * vdim, QS = Nq + 8, KS = Nk + 8, VS = Nv + 8, VC = (vdim + 63) / 64;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                   // [16][QS]
  bf16* Ks = Qs + QT * QS;                                        // [32][KS]
  bf16* Vs = Ks + KT * KS;                                        // [32][VS]
  bf16* pb = Vs + KT * VS;                                        // [H][16][PS] softmax weights of the key tile
  float* sraw = reinterpret_cast<float*>(pb + H * QT * PS);       // [H][16][SS] raw scores
  float* mixs = sraw + H * QT * SS;                               // [H][max(H, 16)]
  float* rm = mixs + H * max(H, 16);                              // [H * 16] running maximum, row = h * 16 + token
  float* rl = rm + H * QT;
  float* rc = rl + H * QT;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, t4 = lane & 3, mi = lane >> 3;
  const int tok0 = p.tile_row0[tile] / H, nt = p.tile_rows[tile] / H;
  const int p0 = p.tok_pos[tok0];
  const bf16* kc = static_cast<const bf16*>(p.kcache) + (long long)p.tile_slot[tile] * p.cap * Nk;
  const bf16* vc = static_cast<const bf16*>(p.vcache) + (long long)p.tile_slot[tile] * p.cap * Nv;
  const int kmin = max(0, p0 - p.window + 1), kmax = p0 + nt - 1;
  const int n_kt = (kmax - kmin) / KT + 1;
  const int per = (n_kt + p.nsplit - 1) / p.nsplit;
  const int kt0 = split * per, kt1 = min(n_kt, kt0 + per);

  for (int i = threadIdx.x; i < QT * (Nq / 2); i += 256) {
    const int qt = i / (Nq / 2), e = (i - qt * (Nq / 2)) * 2;
    float2 v = make_float2(0.f, 0.f);
    if (qt < nt) v = *reinterpret_cast<const float2*>(p.q + (long long)(tok0 + qt) * p.ldq + e);
    *reinterpret_cast<unsigned*>(Qs + qt * QS + e) = pack_bf16(v.x, v.y);
  }
  if (H <= 16) {      // rows padded to 16 entries (zeros) for the register-blocked mix
    for (int i = threadIdx.x; i < H * 16; i += 256) mixs[i] = (i & 15) < H ? p.mix[(i >> 4) * H + (i & 15)] : 0.f;
  } else {
    for (int i = threadIdx.x; i < H * H; i += 256) mixs[i] = p.mix[i];
  }
  for (int i = threadIdx.x; i < H * QT; i += 256) {
    if (split == 0) { rm[i] = p.sink[i / QT]; rl[i] = 1.f; }
    else { rm[i] = -INFINITY; rl[i] = 0.f; }
  }
  float oacc[NI][8][4];
#pragma unroll
  for (int a = 0; a < NI; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) { oacc[a][b][0] = oacc[a][b][1] = oacc[a][b][2] = oacc[a][b][3] = 0.f; }

  for (int kt = kt0; kt < kt1; ++kt) {
    const int kb = kmin + kt * KT;
    const int nk = min(KT, kmax + 1 - kb);
    __syncthreads();
    {   // keys and values of the tile: 16-byte loads; rows past the last key are zero (their weights are zero, they must be finite)
      const int kw = Nk / 8, vw = Nv / 8;
      const uint4* k4 = reinterpret_cast<const uint4*>(kc + (long long)kb * Nk);
      const uint4* v4 = reinterpret_cast<const uint4*>(vc + (long long)kb * Nv);
#pragma unroll 4
      for (int i = threadIdx.x; i < KT * kw; i += 256) {
        const int j = i / kw, e = i - j * kw;
        *reinterpret_cast<uint4*>(Ks + j * KS + e * 8) = j < nk ? k4[i] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll 4
      for (int i = threadIdx.x; i < KT * vw; i += 256) {
        const int j = i / vw, e = i - j * vw;
        *reinterpret_cast<uint4*>(Vs + j * VS + e * 8) = j < nk ? v4[i] : make_uint4(0u, 0u, 0u, 0u);
      }
    }
    __syncthreads();
    // (1) raw scores, one head at a time per warp
    for (int h = warp; h < H; h += 8) {
      const bf16* qh = Qs + h * dim;
      const bf16* kh = Ks + (h / rep) * dim;
      float sacc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f; }
      for (int ks = 0; ks < dim / 16; ++ks) {
        unsigned a[4];
        ldmatrix_x4(a, qh + ((mi & 1) * 8 + (lane & 7)) * QS + ks * 16 + (mi >> 1) * 8);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          unsigned b[4];
          ldmatrix_x4(b, kh + (np * 16 + (mi >> 1) * 8 + (lane & 7)) * KS + ks * 16 + (mi & 1) * 8);
          mma_bf16_16816(sacc[2 * np], a, b[0], b[1]);
          mma_bf16_16816(sacc[2 * np + 1], a, b[2], b[3]);
        }
      }
      float* dst = sraw + h * QT * SS;
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        *reinterpret_cast<float2*>(dst + g8 * SS + nb * 8 + 2 * t4) = make_float2(sacc[nb][0], sacc[nb][1]);
        *reinterpret_cast<float2*>(dst + (g8 + 8) * SS + nb * 8 + 2 * t4) = make_float2(sacc[nb][2], sacc[nb][3]);
      }
    }
    __syncthreads();
    // (2) mix over heads, mask, online softmax; lane = key.  Up to 16 heads: a warp takes a token, keeps the token's raw scores
    // of all heads in registers and reads each row of the mix matrix (padded to 16) as four 16-byte broadcasts.
    if (H <= 16) {
      for (int qt = warp; qt < QT; qt += 8) {
        const int pos = p0 + qt, kj = kb + lane;
        const bool vis = lane < nk && qt < nt && kj <= pos && pos - kj < p.window;
        float raw[16];
#pragma unroll
        for (int g = 0; g < 16; ++g) raw[g] = g < H ? sraw[(g * QT + qt) * SS + lane] : 0.f;
        for (int h = 0; h < H; ++h) {
          const float4* mr = reinterpret_cast<const float4*>(mixs + h * 16);
          float s = 0.f;
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) {
            const float4 mv = mr[g4];
            s = fmaf(mv.x, raw[4 * g4], s); s = fmaf(mv.y, raw[4 * g4 + 1], s); s = fmaf(mv.z, raw[4 * g4 + 2], s); s = fmaf(mv.w, raw[4 * g4 + 3], s);
          }
          if (!vis) s = -INFINITY;
          const int row = h * QT + qt;
          const float mo = rm[row], mn = fmaxf(mo, warp_max(s));
          const float w = s > -INFINITY ? expf(s - mn) : 0.f;
          const float sum = warp_sum(w);
          pb[row * PS + lane] = __float2bfloat16_rn(w);
          if (lane == 0) {
            const float corr = mn > -INFINITY ? expf(mo - mn) : 1.f;
            rc[row] = corr;
            rl[row] = rl[row] * corr + sum;
            rm[row] = mn;
          }
        }
      }
    } else {
      for (int row = warp; row < H * QT; row += 8) {
        const int h = row / QT, qt = row - h * QT;
        const int pos = p0 + qt, kj = kb + lane;
        float s = -INFINITY;
        if (lane < nk && qt < nt && kj <= pos && pos - kj < p.window) {
          s = 0.f;
          for (int g = 0; g < H; ++g) s = fmaf(mixs[h * H + g], sraw[(g * QT + qt) * SS + lane], s);
        }
        const float mo = rm[row], mn = fmaxf(mo, warp_max(s));
        const float w = s > -INFINITY ? expf(s - mn) : 0.f;
        const float sum = warp_sum(w);
        pb[row * PS + lane] = __float2bfloat16_rn(w);
        if (lane == 0) {
          const float corr = mn > -INFINITY ? expf(mo - mn) : 1.f;
          rc[row] = corr;
          rl[row] = rl[row] * corr + sum;
          rm[row] = mn;
        }
      }
    }
    __syncthreads();
    // (3) weighted sums of the values
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
      const int it = warp + 8 * ii;
      if (it >= H * VC) break;
      const int h = it / VC, c0 = (it - h * VC) * 64;
      const float corr0 = rc[h * QT + g8], corr1 = rc[h * QT + g8 + 8];
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) { oacc[ii][nb][0] *= corr0; oacc[ii][nb][1] *= corr0; oacc[ii][nb][2] *= corr1; oacc[ii][nb][3] *= corr1; }
      const bf16* vh = Vs + (h / rep) * vdim + c0;
#pragma unroll
      for (int k2 = 0; k2 < 2; ++k2) {
        unsigned pf[4];
        ldmatrix_x4(pf, pb + h * QT * PS + ((lane & 7) + 8 * ((lane >> 3) & 1)) * PS + 16 * k2 + 8 * (lane >> 4));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          if (c0 + np * 16 < vdim) {
            unsigned b[4];
            ldmatrix_x4_trans(b, vh + (k2 * 16 + (mi & 1) * 8 + (lane & 7)) * VS + np * 16 + (mi >> 1) * 8);
            mma_bf16_16816(oacc[ii][2 * np], pf, b[0], b[1]);
            mma_bf16_16816(oacc[ii][2 * np + 1], pf, b[2], b[3]);
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int ii = 0; ii < NI; ++ii) {
    const int it = warp + 8 * ii;
    if (it >= H * VC) break;
    const int h = it / VC, c0 = (it - h * VC) * 64;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int qt = g8 + 8 * hf;
      if (qt >= nt) continue;
      if (p.nsplit == 1) {
        const float inv = 1.f / rl[h * QT + qt];
        bf16* dst = static_cast<bf16*>(p.out) + ((long long)(tok0 + qt) * H + h) * vdim + c0;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
          if (c0 + nb * 8 < vdim)
            *reinterpret_cast<unsigned*>(dst + nb * 8 + 2 * t4) = pack_bf16(oacc[ii][nb][2 * hf] * inv, oacc[ii][nb][2 * hf + 1] * inv);
      } else {
        float* dst = p.part + (((long long)tile * p.nsplit + split) * (QT * H) + qt * H + h) * (vdim + 2);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
          if (c0 + nb * 8 < vdim)
            *reinterpret_cast<float2*>(dst + c0 + nb * 8 + 2 * t4) = make_float2(oacc[ii][nb][2 * hf], oacc[ii][nb][2 * hf + 1]);
        if (c0 == 0 && t4 == 0) { dst[vdim] = rm[h * QT + qt]; dst[vdim + 1] = rl[h * QT + qt]; }
      }
    }
  }
}

// fp32 rows -> T (the merged splits of the window attention)
template <typename T>
__global__ void rows_from_f32_kernel(const float* __restrict__ in, T* __restrict__ out, long long n) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i < n) out[i] = from_f<T>(in[i]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Small projections whose result must be fp32 (gates of a recurrence, router logits): out[t][n] = x[t] . w[n] + b[n], one CTA
// per token, the row in shared memory, one warp per output.  The sum over k has a fixed order whatever else is in the step.
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) small_proj_f32_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w, const float* __restrict__ b,
                                                             float* __restrict__ out, int N, int K) {
  extern __shared__ float xrow[];
  const long long t = blockIdx.x;
  for (int i = threadIdx.x; i < K; i += blockDim.x) xrow[i] = to_f(x[t * ldx + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int n = warp; n < N; n += 8) {
    const T* wr = w + (long long)n * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(xrow[k], to_f(wr[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) out[t * N + n] = acc + (b ? b[n] : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Recurrent matrix memories.  Per (request, head): S [dim][vdim] fp32, carried between steps (stored column-major,
// St[slot][head][vdim][dim], so that a thread's rows of a column are contiguous); a sequence starts from zero (position 0).
//   MODE_DECAY (gated linear attention): S <- diag(a_t) S + k_t v_t^T,  o_t = S^T q_t,   a_t = sigmoid(z_t + bz)^(1 / tau)
//   MODE_EXPGATE (stabilised exponential gating, the matrix memory of xLSTM):
//       i_t = cap tanh(gi / cap), f_t = logsigmoid(cap tanh(gf / cap)),  m_t = max(f_t + m_{t-1}, i_t)   (m starts at 0)
//       S <- e^(f_t + m_{t-1} - m_t) S + e^(i_t - m_t) k_t v_t^T,  n likewise with k_t alone
//       o_t = S^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
// q is scaled by qscale.  scan_prep_kernel lays out what a token contributes; matrix_memory_scan_kernel runs the recurrence.
// ---------------------------------------------------------------------------------------------------------------------------
//   MODE_DELTA (the gated delta rule): S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//       (g, beta per head and token; a column of S depends on no other column, so the columns are dealt over threads as above)
//   MODE_CHDELTA: the same with one decay per key channel, S <- diag(g_t) S (prep row [q | k | g | beta])
enum { MODE_DECAY = 0, MODE_EXPGATE = 1, MODE_DELTA = 2, MODE_CHDELTA = 3 };

struct ScanParams {
  const void* proj;         // T [tokens][ld]: q at off_q, k at off_k, v at off_v (heads x dim / vdim each)
  long long ld;
  int off_q, off_k, off_v;
  const float* z;           // MODE_DECAY: [tokens][heads * dim] decay logits;  MODE_EXPGATE: [tokens][2 * heads] gate inputs (i then f, biased)
  const float* zb;          // MODE_DECAY: bias [heads * dim]
  float inv_tau, cap, qscale;
  float* prep;              // [tokens][heads][nvec * dim (+ 2 gates, padded to 4)] fp32: what the recurrence reads per token and head
  float* vprep;             // [tokens][heads * vdim] fp32
  int prow;                 // floats per (token, head) row of prep
  float* St;                // [slots][heads][vdim][dim]
  float* nvec;              // MODE_EXPGATE: [2][slots][heads][dim]: two generations, so that no CTA of a head reads what another
  float* mval;              // MODE_EXPGATE: [2][slots][heads]                has already replaced
  const int* ent_par;       // per entry: the generation to read (the other one is written)
  int slots;
  // Long portions are cut into segments that run as entries of their own, in parallel (ent_seg = index of the segment in its
  // portion, ent_nseg = segments of the portion, ent_buf = its row of the segment buffers).  Segment 0 continues the slot's
  // state; the others start from nothing and leave what scan_chain_kernel and the correction need:
  //   segS  [buf][heads][vdim + 1][dim]  the segment's end state (row vdim: mLSTM's n), later replaced by its true start state
  //   segB  [buf][heads][dim]            MODE_DECAY: product of the decays over the segment
  //   segM  [buf][heads][4]              MODE_EXPGATE: sum of the log forget gates, local maximum at the end, (chain: true maximum at the start)
  //   qb    [tokens][heads * dim]        q times the product of the decays from the segment's start to the token (MODE_EXPGATE: q)
  //   tokM  [tokens][heads][4]           MODE_EXPGATE: log forget sum so far, local maximum, local n . q
  const int* ent_seg; const int* ent_nseg; const int* ent_buf;
  float *segS, *segB, *segM, *qb, *tokM;
  const int* ent_tok0;      // per entry: first token of the step, number of tokens, slot, position of the first token
  const int* ent_ntok;
  const int* ent_slot;
  const int* ent_pos0;
  float* out;               // [tokens][heads * vdim]
  int heads, dim, vdim, stage, vec;      // vec: rows of prep and the 16-column slices of vprep start on 16 bytes
  int lpc = 0, rows = 0;    // lane-ordered prep rows for the kernel variant that reads four rows per load (0: plain rows)
  // MODE_DECAY with one fixed decay per head (retention) instead of the per-channel sigmoid decay, keys scaled by kscale, and
  // rotary positions on q and k (rot_half > 0): angle pos * freq[i], cos and sin times rot_amp, pairs by halves or adjacent
  const float* head_decay = nullptr;
  const double* freq = nullptr;
  const int* tok_pos = nullptr;
  int rot_half = 0, rot_adjacent = 0;
  float rot_amp = 1.f, kscale = 1.f;
};

// Everything the recurrence reads, as fp32 rows that its CTAs can copy asynchronously: per (token, head)
//   MODE_DECAY:   [q * qscale | k | a = sigmoid(z + bz)^(1 / tau)]
//   MODE_EXPGATE: [q * qscale | k | i, f]   with i = cap tanh(gi / cap), f = logsigmoid(cap tanh(gf / cap))
// and the values as fp32.  One CTA per token.
template <typename T, int MODE>
__global__ void __launch_bounds__(256) scan_prep_kernel(ScanParams p) {
  extern __shared__ float prep_rot[];   // [rot_half] cosines, [rot_half] sines of the token's position
  const long long t = blockIdx.x;
  const int heads = p.heads, dim = p.dim;
  const int half = p.rot_half;
  if (half > 0) {
    const int pos = p.tok_pos[t];
    for (int i = threadIdx.x; i < half; i += 256) {
      double sn, cs;
      sincos((double)pos * p.freq[i], &sn, &cs);
      prep_rot[i] = (float)cs * p.rot_amp; prep_rot[half + i] = (float)sn * p.rot_amp;
    }
    __syncthreads();
  }
  // element d of head h of the projection at `off`, turned by the token's position when the mixer has rotary positions
  auto turned = [&](const T* row, int off, int h, int d) -> float {
    const T* hd = row + off + h * dim;
    const float own = to_f(hd[d]);
    if (d >= 2 * half) return own;
    int i, partner; bool first;
    if (p.rot_adjacent) { i = d >> 1; first = (d & 1) == 0; partner = d ^ 1; }
    else { first = d < half; i = first ? d : d - half; partner = first ? d + half : d - half; }
    const float other = to_f(hd[partner]);
    return first ? own * prep_rot[i] - other * prep_rot[half + i] : own * prep_rot[i] + other * prep_rot[half + i];
  };
  // plain rows (lpc = 0): q, k, a of `dim` elements each.  Lane-ordered rows (lpc > 0, for the recurrence kernel that reads four
  // rows per load): each padded with zeros to Dp = lpc * rows; lane g of a column owns rows g * rows .. g * rows + rows - 1 and
  // row g * rows + 4 c + j sits at (c * lpc + g) * 4 + j, so that a quarter-warp's 16-byte loads fall in distinct banks.
  const int R = p.rows, Dp = p.lpc > 0 ? p.lpc * p.rows : dim;
  const T* row = static_cast<const T*>(p.proj) + t * p.ld;
  float* dst = p.prep + t * heads * p.prow;
  for (int i = threadIdx.x; i < heads * Dp; i += 256) {
    const int h = i / Dp, d = i - h * Dp;
    int at = d;
    if (p.lpc > 0) { const int g = d / R, w = d - g * R; at = ((w >> 2) * p.lpc + g) * 4 + (w & 3); }
    float* o = dst + h * p.prow;
    const bool live = d < dim;
    o[at] = live ? turned(row, p.off_q, h, d) * p.qscale : 0.f;
    o[Dp + at] = live ? turned(row, p.off_k, h, d) * p.kscale : 0.f;
    if (MODE == MODE_DECAY) {
      if (p.head_decay) o[2 * Dp + at] = live ? p.head_decay[h] : 0.f;
      else o[2 * Dp + at] = live ? expf(log_sigmoidf(p.z[t * heads * dim + h * dim + d] + p.zb[h * dim + d]) * p.inv_tau) : 0.f;
    }
  }
  if (MODE == MODE_EXPGATE) {
    for (int i = threadIdx.x; i < 2 * heads; i += 256) {
      const int which = i / heads, h = i - which * heads;
      const float g = p.cap * tanhf(p.z[t * 2 * heads + i] / p.cap);
      dst[h * p.prow + 2 * Dp + which] = which ? log_sigmoidf(g) : g;
    }
  }
  for (int i = threadIdx.x; i < heads * p.vdim; i += 256) p.vprep[t * heads * p.vdim + i] = to_f(row[p.off_v + i]);
}

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* src, bool vec4) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  if (vec4) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

// The recurrence itself.  A CTA owns 128 / LPC * CB columns of one (request, head) and walks the request's new tokens in order;
// LPC lanes share CB adjacent columns (row = lane's group + LPC * i, held in registers), so a column's dot product with q closes
// with log2(LPC) shuffles, and every q, k and decay element a thread reads from shared memory serves CB columns.  Batches of
// requests: LPC = 8 (many CTAs, state rows read in full sectors); a few long requests: LPC = 16 (twice the CTAs, half the chain
// per token).  CB = 1 is what runs: the kernel is bound by the chain from token to token, and more columns per thread mean
// fewer warps to overlap it.  Tokens arrive in stages of `stage` tokens,
// copied asynchronously into one of two shared-memory buffers while the other is being consumed.  mLSTM's n and m exist once
// per (slot, head) in two generations: every CTA reads generation `par` of its entry, the CTA of the first columns writes
// generation `par ^ 1`.  Grid: (entries * heads, ceil(vdim / (128 / LPC * CB))).
template <int MODE, int R, int LPC, int CB, bool VL = false>      // R rows per thread (dim <= LPC * R), CB adjacent columns per thread
__global__ void __launch_bounds__(128) matrix_memory_scan_kernel(ScanParams p) {      // VL: a thread's rows are adjacent, read four at a time from lane-ordered prep rows
  constexpr int NC = 128 / LPC * CB;                  // columns per CTA
  constexpr int Dp = LPC * R;
  const int TT = p.stage;
  extern __shared__ __align__(16) float sm[];
  const int dim = p.dim, vdim = p.vdim, heads = p.heads, prow = p.prow;
  const int srow = prow + NC;                         // a staged token: its prep row, then its values
  const int ent = blockIdx.x / heads, head = blockIdx.x - ent * heads;
  const int tok0 = p.ent_tok0[ent], nt = p.ent_ntok[ent], slot = p.ent_slot[ent], pos0 = p.ent_pos0[ent];
  const int rg = threadIdx.x & (LPC - 1), cl = threadIdx.x / LPC * CB, col = blockIdx.y * NC + cl;      // first of the thread's columns
  float* Sbase = p.St + ((long long)slot * heads + head) * vdim * dim;
  const int par = MODE == MODE_EXPGATE ? p.ent_par[ent] : 0;
  const int seg = p.ent_seg[ent], nseg = p.ent_nseg[ent];
  const long long sbuf = (long long)p.ent_buf[ent] * heads + head;      // row of the segment buffers (when nseg > 1)
  const bool lead = blockIdx.y == 0 && cl == 0;                          // the threads that write what exists once per head
  const long long sh = (long long)slot * heads + head;
  const float* nin = MODE == MODE_EXPGATE ? p.nvec + ((long long)par * p.slots * heads + sh) * dim : nullptr;
  float* nout = MODE == MODE_EXPGATE ? p.nvec + ((long long)(par ^ 1) * p.slots * heads + sh) * dim : nullptr;
  float S[R][CB], nv[R], m = 0.f;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = VL ? rg * R + i : rg + LPC * i;
    const bool live = pos0 > 0 && seg == 0 && r < dim;
#pragma unroll
    for (int j = 0; j < CB; ++j) S[i][j] = live && col + j < vdim ? Sbase[(long long)(col + j) * dim + r] : 0.f;
    nv[i] = (MODE == MODE_EXPGATE && live) ? nin[r] : 0.f;
  }
  if (MODE == MODE_EXPGATE && pos0 > 0 && seg == 0) m = p.mval[(long long)par * p.slots * heads + sh];
  if (MODE == MODE_EXPGATE && seg > 0) m = -INFINITY;        // a later segment: nothing seen yet (the first token sets the maximum)
  float bdec[MODE == MODE_DECAY ? R : 1], logF = 0.f;         // later segments: decay products per row; sum of the log forget gates
#pragma unroll
  for (int i = 0; i < (MODE == MODE_DECAY ? R : 1); ++i) bdec[i] = 1.f;

  auto issue = [&](int t0, int buf) {
    const int tn = min(TT, nt - t0);
    float* base = sm + buf * TT * srow;
    if (p.vec) {
      const int pw = prow / 4, vw = NC / 4;
      for (int i = threadIdx.x; i < tn * (pw + vw); i += 128) {
        const int tt = i / (pw + vw), e = i - tt * (pw + vw);
        const long long tok = tok0 + t0 + tt;
        if (e < pw) cp_async_f32(base + tt * srow + e * 4, p.prep + (tok * heads + head) * prow + e * 4, true);
        else if (blockIdx.y * NC + (e - pw) * 4 < vdim) cp_async_f32(base + tt * srow + prow + (e - pw) * 4, p.vprep + tok * heads * vdim + head * vdim + blockIdx.y * NC + (e - pw) * 4, true);
      }
    } else {
      for (int i = threadIdx.x; i < tn * srow; i += 128) {
        const int tt = i / srow, e = i - tt * srow;
        const long long tok = tok0 + t0 + tt;
        if (e < prow) cp_async_f32(base + tt * srow + e, p.prep + (tok * heads + head) * prow + e, false);
        else if (blockIdx.y * NC + (e - prow) < vdim) cp_async_f32(base + tt * srow + e, p.vprep + tok * heads * vdim + head * vdim + blockIdx.y * NC + (e - prow), false);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  issue(0, 0);
  for (int t0 = 0, st = 0; t0 < nt; t0 += TT, ++st) {
    const int tn = min(TT, nt - t0);
    if (t0 + TT < nt) { issue(t0 + TT, (st + 1) & 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    const float* base = sm + (st & 1) * TT * srow;
#pragma unroll 2
    for (int tt = 0; tt < tn; ++tt) {
      const float* qq = base + tt * srow;
      const float* kk = qq + (VL ? Dp : dim);
      const float* aa = kk + (VL ? Dp : dim);
      float v[CB], acc[CB], nq = 0.f, fa = 1.f, fb = 1.f, m2 = 0.f;
#pragma unroll
      for (int j = 0; j < CB; ++j) { v[j] = col + j < vdim ? qq[prow + cl + j] : 0.f; acc[j] = 0.f; }
      if (MODE == MODE_EXPGATE) {
        const float il = aa[0], fl = aa[1];
        m2 = fmaxf(fl + m, il);
        fa = expf(fl + m - m2);                      // m = -inf (nothing seen yet) gives 0
        fb = expf(il - m2);
        m = m2;
        logF += fl;
      }
      if (MODE == MODE_DELTA || MODE == MODE_CHDELTA) {      // two passes over the thread's rows: decay and S^T k, then the write and the read-out
        const float gl = aa[0], be = MODE == MODE_CHDELTA ? aa[VL ? Dp : dim] : aa[1];
        float dot[CB], u[CB];
#pragma unroll
        for (int j = 0; j < CB; ++j) dot[j] = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int r = VL ? rg * R + i : rg + LPC * i;
          const float kv = VL ? kk[((i >> 2) * LPC + rg) * 4 + (i & 3)] : (r < dim ? kk[r] : 0.f);
          const float gr = MODE == MODE_CHDELTA ? (VL ? aa[((i >> 2) * LPC + rg) * 4 + (i & 3)] : (r < dim ? aa[r] : 0.f)) : gl;      // the row's own decay
#pragma unroll
          for (int j = 0; j < CB; ++j) { S[i][j] *= gr; dot[j] = fmaf(S[i][j], kv, dot[j]); }
        }
#pragma unroll
        for (int j = 0; j < CB; ++j) {
#pragma unroll
          for (int o = 1; o < LPC; o <<= 1) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], o);
          u[j] = be * (v[j] - dot[j]);
        }
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int r = VL ? rg * R + i : rg + LPC * i;
          const int at = VL ? ((i >> 2) * LPC + rg) * 4 + (i & 3) : r;
          const bool live = VL || r < dim;
          const float kv = live ? kk[at] : 0.f, qv = live ? qq[at] : 0.f;
#pragma unroll
          for (int j = 0; j < CB; ++j) { S[i][j] = fmaf(kv, u[j], S[i][j]); acc[j] = fmaf(S[i][j], qv, acc[j]); }
        }
      } else if (VL) {
#pragma unroll
        for (int c4 = 0; c4 < R / 4; ++c4) {         // rows past dim are zeros in q, k and a: they stay zero and add nothing
          const float4 q4 = *reinterpret_cast<const float4*>(qq + (c4 * LPC + rg) * 4);
          const float4 k4 = *reinterpret_cast<const float4*>(kk + (c4 * LPC + rg) * 4);
          const float qv4[4] = {q4.x, q4.y, q4.z, q4.w}, kv4[4] = {k4.x * fb, k4.y * fb, k4.z * fb, k4.w * fb};
          float av4[4] = {fa, fa, fa, fa};
          if (MODE == MODE_DECAY) {
            const float4 a4 = *reinterpret_cast<const float4*>(aa + (c4 * LPC + rg) * 4);
            av4[0] = a4.x; av4[1] = a4.y; av4[2] = a4.z; av4[3] = a4.w;
          }
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const int i = 4 * c4 + w;
            if (seg > 0) {      // what the carried state is multiplied with: q times the decays so far, or q itself
              if (MODE == MODE_DECAY) bdec[i] *= av4[w];
              if (lead && rg * R + i < dim) p.qb[(long long)(tok0 + t0 + tt) * heads * dim + head * dim + rg * R + i] = MODE == MODE_DECAY ? qv4[w] * bdec[i] : qv4[w];
            }
#pragma unroll
            for (int j = 0; j < CB; ++j) {
              S[i][j] = fmaf(av4[w], S[i][j], kv4[w] * v[j]);
              acc[j] = fmaf(S[i][j], qv4[w], acc[j]);
            }
            if (MODE == MODE_EXPGATE) {
              nv[i] = fmaf(fa, nv[i], kv4[w]);
              nq = fmaf(nv[i], qv4[w], nq);
            }
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int r = rg + LPC * i;
          if (r < dim) {
            const float kv = kk[r] * fb, qv = qq[r];
            const float ar = MODE == MODE_DECAY ? aa[r] : fa;
            if (seg > 0) {
              if (MODE == MODE_DECAY) bdec[i] *= ar;
              if (lead) p.qb[(long long)(tok0 + t0 + tt) * heads * dim + head * dim + r] = MODE == MODE_DECAY ? qv * bdec[i] : qv;
            }
#pragma unroll
            for (int j = 0; j < CB; ++j) {
              S[i][j] = fmaf(ar, S[i][j], kv * v[j]);
              acc[j] = fmaf(S[i][j], qv, acc[j]);
            }
            if (MODE == MODE_EXPGATE) {
              nv[i] = fmaf(fa, nv[i], kv);
              nq = fmaf(nv[i], qv, nq);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < CB; ++j)
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
      if (MODE == MODE_EXPGATE) {
#pragma unroll
        for (int o = 1; o < LPC; o <<= 1) nq += __shfl_xor_sync(0xffffffffu, nq, o);
        if (seg == 0) {
          const float den = 1.f / (fmaxf(fabsf(nq), expf(-m2)) + 1e-6f);
#pragma unroll
          for (int j = 0; j < CB; ++j) acc[j] *= den;
        } else if (lead && rg == 0) {      // numerators stay as they are; the correction divides
          float* tm = p.tokM + ((long long)(tok0 + t0 + tt) * heads + head) * 4;
          tm[0] = logF; tm[1] = m2; tm[2] = nq;
        }
      }
      if (rg == 0) {
        float* o = p.out + (long long)(tok0 + t0 + tt) * heads * vdim + head * vdim + col;
#pragma unroll
        for (int j = 0; j < CB; ++j) if (col + j < vdim) o[j] = acc[j];
      }
    }
    __syncthreads();
  }
  if (nseg > 1) {      // a segment of a long portion: its end state goes to the segment buffers, scan_chain_kernel finishes the slot
    float* dst = p.segS + sbuf * (vdim + 1) * dim;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = VL ? rg * R + i : rg + LPC * i;
      if (r < dim) {
#pragma unroll
        for (int j = 0; j < CB; ++j) if (col + j < vdim) dst[(long long)(col + j) * dim + r] = S[i][j];
        if (MODE == MODE_EXPGATE && lead) dst[(long long)vdim * dim + r] = nv[i];
        if (MODE == MODE_DECAY && lead) p.segB[sbuf * dim + r] = bdec[i];
      }
    }
    if (MODE == MODE_EXPGATE && lead && rg == 0) { p.segM[sbuf * 4] = logF; p.segM[sbuf * 4 + 1] = m; }
    return;
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = VL ? rg * R + i : rg + LPC * i;
    if (r < dim) {
#pragma unroll
      for (int j = 0; j < CB; ++j) if (col + j < vdim) Sbase[(long long)(col + j) * dim + r] = S[i][j];
      if (MODE == MODE_EXPGATE && lead) nout[r] = nv[i];
    }
  }
  if (MODE == MODE_EXPGATE && lead && rg == 0) p.mval[(long long)(par ^ 1) * p.slots * heads + sh] = m;
}

// After the segments of a long portion have run side by side: walks them in order, per (portion, head) and state element,
//   MODE_DECAY:   start_p = S;  S <- B_p * S + end_p                                   (B_p: the segment's decay product, per row)
//   MODE_EXPGATE: start_p = S;  m' = max(F_p + m, ml_p);  S <- e^(F_p + m - m') S + e^(ml_p - m') end_p   (n likewise; F_p: log forget sum)
// leaving every later segment's true start state in its row of segS (and its starting maximum in segM[2]) for the correction, and
// the state after the last segment in the slot.  Grid: (entries * heads, state elements / 256); the CTAs of a segment other
// than a first one return.
template <int MODE>
__global__ void __launch_bounds__(256) scan_chain_kernel(ScanParams p) {
  const int ent = blockIdx.x / p.heads, head = blockIdx.x - ent * p.heads;
  const int nseg = p.ent_nseg[ent];
  if (p.ent_seg[ent] != 0 || nseg < 2) return;
  const int heads = p.heads, dim = p.dim, vdim = p.vdim, slot = p.ent_slot[ent], buf0 = p.ent_buf[ent];
  const long long sh = (long long)slot * heads + head;
  const int par = MODE == MODE_EXPGATE ? p.ent_par[ent] : 0;
  const int rows = MODE == MODE_EXPGATE ? vdim + 1 : vdim;
  const long long bstride = (long long)heads * (vdim + 1) * dim;
  float* s0 = p.segS + ((long long)buf0 * heads + head) * (vdim + 1) * dim;
  const int e = blockIdx.y * 256 + threadIdx.x;      // one state element per thread: the walk over the segments is a chain of loads
  if (e < rows * dim) {
    const int r = e % dim;
    float S = s0[e];
    float m = MODE == MODE_EXPGATE ? p.segM[((long long)buf0 * heads + head) * 4 + 1] : 0.f;
    for (int q = 1; q < nseg; ++q) {
      const long long sb = (long long)(buf0 + q) * heads + head;
      const float end = s0[q * bstride + e];
      s0[q * bstride + e] = S;
      if (MODE == MODE_DECAY) {
        S = fmaf(p.segB[sb * dim + r], S, end);
      } else {
        const float F = p.segM[sb * 4], ml = p.segM[sb * 4 + 1];
        const float m2 = fmaxf(F + m, ml);
        S = expf(F + m - m2) * S + expf(ml - m2) * end;
        if (e == 0) p.segM[sb * 4 + 2] = m;        // the maximum this segment truly starts from
        m = m2;
      }
    }
    if (e < vdim * dim) p.St[sh * vdim * dim + e] = S;
    else p.nvec[((long long)(par ^ 1) * p.slots * heads + sh) * dim + r] = S;
    if (MODE == MODE_EXPGATE && e == 0) p.mval[(long long)(par ^ 1) * p.slots * heads + sh] = m;
  }
}

// mLSTM, tokens of a later segment: the carried part corr = [S_start^T q | n_start . q] (one small product per segment) meets the
// local numerators:  m = max(F_t + m_start, ml_t);  a = e^(F_t + m_start - m), b = e^(ml_t - m);
//   out = (a corr + b local) / (max(|a corr_n + b local_n|, e^(-m)) + 1e-6).  One warp per (token, head).
__global__ void __launch_bounds__(128) mlstm_combine_kernel(float* __restrict__ out, const float* __restrict__ corr, const float* __restrict__ tokM,
                                                            const float* __restrict__ segM_row, int heads, int vdim, long long rows) {
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int h = (int)(row % heads);
  const float* tm = tokM + row * 4;
  const float ms = segM_row[h * 4 + 2];
  const float m = fmaxf(tm[0] + ms, tm[1]);
  const float a = expf(tm[0] + ms - m), b = expf(tm[1] - m);
  const float* c = corr + row * (vdim + 1);
  const float den = 1.f / (fmaxf(fabsf(a * c[vdim] + b * tm[2]), expf(-m)) + 1e-6f);
  float* o = out + row * vdim;
  for (int i = lane; i < vdim; i += 32) o[i] = (a * c[i] + b * o[i]) * den;
}

// what leaves a recurrent mixer: per head rms_norm over vdim (weight w[h * wstride + c]: wstride = 0 shares one row between
// the heads, w = null: no weight), times a gate computed from the projection g (act 0: sigmoid, 1: silu) -> T.  One warp per (token, head).
template <typename T, typename TG = T>      // TG: type of the gate's pre-activations (fp32 when they come from a product of their own)
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int wstride,
                                                             const TG* __restrict__ proj, long long ld, int off_g, int act, T* __restrict__ out,
                                                             int heads, int vdim, long long rows, float eps) {
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads; const int h = (int)(row - t * heads);
  const float* src = o + row * vdim;
  float s = 0.f;
  for (int c = lane; c < vdim; c += 32) s += src[c] * src[c];
  const float r = 1.f / sqrtf(warp_sum(s) / (float)vdim + eps);
  for (int c = lane; c < vdim; c += 32) {
    const float g = to_f(proj[t * ld + off_g + h * vdim + c]);
    out[row * vdim + c] = from_f<T>(src[c] * r * (w ? w[(long long)h * wstride + c] : 1.f) * (act ? siluf(g) : sigmoidf(g)));
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// End of a sublayer in the sandwich arrangement, one CTA per token:
//   y = branch0                                                 (one mixer)
//     | factor * (rms_norm(branch0) * w0 + rms_norm(branch1) * w1)   (two mixers side by side, each normed over the width)
//     | sum_k ew[t][k] * branch0[t * top + k]                   (routed experts: weighted sum of the chosen experts' rows)
//   x <- x + rms_norm(y) * w_post;  optional copy of x (per-layer trace);  optional h = rms_norm(x) * w_next as fp32 and / or T
// ---------------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) sublayer_end_kernel(float* __restrict__ xin, const T* __restrict__ b0, const float* __restrict__ w0,
                                                           const T* __restrict__ b1, const float* __restrict__ w1, float factor,
                                                           const float* __restrict__ ew, int top, const float* __restrict__ w_post,
                                                           float* __restrict__ trace, const float* __restrict__ w_next,
                                                           float* __restrict__ h32, T* __restrict__ hT, int W, float eps) {
  extern __shared__ float y[];
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float* x = xin + t * W;
  if (ew) {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float acc = 0.f;
      for (int k = 0; k < top; ++k) acc = fmaf(ew[t * top + k], to_f(b0[(t * top + k) * W + i]), acc);
      y[i] = acc;
    }
  } else if (b1) {
    float s0 = 0.f, s1 = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float a = to_f(b0[t * W + i]), b = to_f(b1[t * W + i]); s0 += a * a; s1 += b * b; }
    const float r0 = 1.f / sqrtf(block_sum(s0, red) / (float)W + eps);
    const float r1 = 1.f / sqrtf(block_sum(s1, red) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) y[i] = factor * (to_f(b0[t * W + i]) * r0 * w0[i] + to_f(b1[t * W + i]) * r1 * w1[i]);
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) y[i] = to_f(b0[t * W + i]);
  }
  __syncthreads();
  const float ry = block_rrms(y, W, eps, red);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = x[i] + y[i] * ry * w_post[i];
    x[i] = v;
    y[i] = v;
    if (trace) trace[t * W + i] = v;
  }
  if (w_next) {
    __syncthreads();
    const float rx = block_rrms(y, W, eps, red);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = y[i] * rx * w_next[i];
      if (h32) h32[t * W + i] = v;
      if (hT) hT[t * W + i] = from_f<T>(v);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Routed experts.  moe_route_kernel: per token (one warp) the `top` largest router logits (ties: the lower index) and the
// softmax over those alone.  moe_group_kernel (ONE CTA): sorts the (token, choice) pairs by expert: pos-th row of the grouped
// order is pair perm[pos] of token row_tok[pos], and cuts every expert's rows into tiles of tile_m for the grouped products
// (tile -> expert, first row, rows); n_tiles[0] = number of tiles.  The order inside an expert follows the atomics and may
// differ from run to run; a row's result does not depend on it (every row of a product is summed on its own).
// ---------------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int E, int top, int* __restrict__ idx,
                                                        float* __restrict__ wts, int n_tok) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tok) return;
  const float* z = logits + (long long)t * E;
  float zmax = 0.f, den = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= idx[(long long)t * top + j] == e;
      const float v = z[e];
      if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (k == 0) zmax = best;
    const float w = expf(best - zmax);
    den += w;
    if (lane == 0) { idx[(long long)t * top + k] = bi; wts[(long long)t * top + k] = w; }
    __syncwarp();
  }
  __syncwarp();
  if (lane < top) wts[(long long)t * top + lane] /= den;
}

__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ idx, int n_pairs, int top, int E, int* __restrict__ rank,
                                                         int* __restrict__ perm, int* __restrict__ row_tok, int* __restrict__ tile_expert,
                                                         int* __restrict__ tile_row0, int* __restrict__ tile_rows, int* __restrict__ n_tiles, int tile_m) {
  extern __shared__ int cnt[];          // [E] counts, then [E] offsets
  int* off = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) rank[i] = atomicAdd(&cnt[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      for (int r0 = 0; r0 < cnt[e]; r0 += tile_m) { tile_expert[nt] = e; tile_row0[nt] = o + r0; tile_rows[nt] = min(tile_m, cnt[e] - r0); ++nt; }
      o += cnt[e];
    }
    n_tiles[0] = nt;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int pos = off[idx[i]] + rank[i];
    perm[pos] = i;
    row_tok[pos] = i / top;
  }
}

// Grouped product of the routed experts: for tile (expert e, rows pos0 .. pos0 + n - 1 of the grouped order)
//   C[c_rows ? c_rows[pos] : pos][:] = act( A[a_rows ? a_rows[pos] : pos][:] . B[e]^T ),  B[e] = B + e * sb, [N][K];  act 1: relu(.)^2
// CUDA cores, fp32 FMA, k in order (the all-fp32 mode, and shapes the tensor-core kernel does not take).
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256) grouped_gemm_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ a_rows,
                                                           const TB* __restrict__ B, long long ldb, long long sb, TC* __restrict__ C,
                                                           long long ldc, const int* __restrict__ c_rows, const int* __restrict__ tile_expert,
                                                           const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                                                           const int* __restrict__ n_tiles, int N, int K, int act) {
  constexpr int BM = 64, BN = 64, BK = 16;
  if ((int)blockIdx.y >= n_tiles[0]) return;
  __shared__ float As[BK][BM + 1], Bs[BK][BN + 1];
  __shared__ int arow[BM];
  const int pos0 = tile_row0[blockIdx.y], M = tile_rows[blockIdx.y];
  B += (long long)tile_expert[blockIdx.y] * sb;
  const int n0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  if (threadIdx.x < BM) arow[threadIdx.x] = threadIdx.x < M ? (a_rows ? a_rows[pos0 + threadIdx.x] : pos0 + threadIdx.x) : 0;
  __syncthreads();
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rr = ty + 16 * i, kk = k0 + tx;
      As[tx][rr] = (rr < M && kk < K) ? to_f(A[(long long)arow[rr] * lda + kk]) : 0.f;
      Bs[tx][rr] = (n0 + rr < N && kk < K) ? to_f(B[(long long)(n0 + rr) * ldb + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[k][ty + 16 * i]; b[i] = Bs[k][tx + 16 * i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = ty + 16 * i, n = n0 + tx + 16 * j;
      if (m < M && n < N) {
        float v = acc[i][j];
        if (act) { v = fmaxf(v, 0.f); v = v * v; }
        const long long crow = c_rows ? c_rows[pos0 + m] : pos0 + m;
        C[crow * ldc + n] = from_f<TC>(v);
      }
    }
}

// The same grouped product on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 accumulate): K a multiple of 16, rows of A
// and B on 16-byte boundaries; act 2: gate and value rows of B alternate and the epilogue writes
// min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1) into column n / 2.  CTA tile 128 x 128 (tiles of 128 rows in the tile table), 8 warps of 32 x 64, 64-element
// k-steps through two shared-memory buffers filled by cp.async (chunks outside M, N or K are zero-filled by a copy of size 0).
__device__ __forceinline__ void cp_async_16_or_zero(void* smem_dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

constexpr int GG_BM = 128, GG_BN = 128, GG_BK = 64, GG_ST = GG_BK + 8;
constexpr size_t GG_SMEM = (size_t)2 * (GG_BM + GG_BN) * GG_ST * 2 + GG_BM * 4;

__global__ void __launch_bounds__(256, 2) grouped_gemm_mma_kernel(const bf16* __restrict__ A, long long lda, const int* __restrict__ a_rows,
                                                                  const bf16* __restrict__ B, long long ldb, long long sb, bf16* __restrict__ C,
                                                                  long long ldc, const int* __restrict__ c_rows, const int* __restrict__ tile_expert,
                                                                  const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                                                                  const int* __restrict__ n_tiles, int N, int K, int act, float limit = 0.f) {
  constexpr int BM = GG_BM, BN = GG_BN, BK = GG_BK, ST = GG_ST;
  if ((int)blockIdx.y >= n_tiles[0]) return;
  extern __shared__ __align__(16) unsigned char gg_smem[];
  bf16 (*As)[BM][ST] = reinterpret_cast<bf16 (*)[BM][ST]>(gg_smem);                                  // [2][BM][ST]
  bf16 (*Bs)[BN][ST] = reinterpret_cast<bf16 (*)[BN][ST]>(gg_smem + (size_t)2 * BM * ST * 2);        // [2][BN][ST]
  int* arow = reinterpret_cast<int*>(gg_smem + (size_t)2 * (BM + BN) * ST * 2);
  const int pos0 = tile_row0[blockIdx.y], M = tile_rows[blockIdx.y];
  B += (long long)tile_expert[blockIdx.y] * sb;
  const int n0 = blockIdx.x * BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3, mi = lane >> 3;
  const int wm = (warp & 3) * 32, wn = (warp >> 2) * 64;
  if (threadIdx.x < BM) arow[threadIdx.x] = threadIdx.x < M ? (a_rows ? a_rows[pos0 + threadIdx.x] : pos0 + threadIdx.x) : 0;
  __syncthreads();
  float acc[2][8][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) { acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f; }
  auto load = [&](int k0, int buf) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = threadIdx.x + 256 * j;
      const int rr = c >> 3, kk = (c & 7) * 8;
      const bool va = rr < M && k0 + kk < K, vb = n0 + rr < N && k0 + kk < K;
      cp_async_16_or_zero(&As[buf][rr][kk], va ? A + (long long)arow[rr] * lda + k0 + kk : A, va);
      cp_async_16_or_zero(&Bs[buf][rr][kk], vb ? B + (long long)(n0 + rr) * ldb + k0 + kk : B, vb);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load(0, 0);
  for (int k0 = 0, it = 0; k0 < K; k0 += BK, ++it) {
    const int buf = it & 1;
    if (k0 + BK < K) { load(k0 + BK, buf ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      unsigned a[2][4];
#pragma unroll
      for (int mf = 0; mf < 2; ++mf) ldmatrix_x4(a[mf], &As[buf][wm + mf * 16 + (mi & 1) * 8 + (lane & 7)][ks * 16 + (mi >> 1) * 8]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        unsigned b[4];
        ldmatrix_x4(b, &Bs[buf][wn + np * 16 + (mi >> 1) * 8 + (lane & 7)][ks * 16 + (mi & 1) * 8]);
#pragma unroll
        for (int mf = 0; mf < 2; ++mf) {
          mma_bf16_16816(acc[mf][2 * np], a[mf], b[0], b[1]);
          mma_bf16_16816(acc[mf][2 * np + 1], a[mf], b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  const bool pair_ok = (ldc & 1) == 0 && (reinterpret_cast<uintptr_t>(C) & 3) == 0;      // two columns in one 4-byte store
#pragma unroll
  for (int mf = 0; mf < 2; ++mf)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int m = wm + mf * 16 + g + 8 * hf;
      if (m >= M) continue;
      const long long crow = c_rows ? c_rows[pos0 + m] : pos0 + m;
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        const int n = n0 + wn + nb * 8 + 2 * t4;
        float v0 = acc[mf][nb][2 * hf], v1 = acc[mf][nb][2 * hf + 1];
        if (act == 2) {      // rows of B interleave gate and value: columns (n, n + 1) are one output, column n / 2 of C
          if (n + 1 < N) {
            const float g = fminf(v0, limit), u = fminf(fmaxf(v1, -limit), limit);
            C[crow * ldc + (n >> 1)] = __float2bfloat16_rn(g / (1.f + expf(-1.702f * g)) * (u + 1.f));
          }
          continue;
        }
        if (act) { v0 = fmaxf(v0, 0.f); v0 *= v0; v1 = fmaxf(v1, 0.f); v1 *= v1; }
        if (n + 1 < N && pair_ok) {
          *reinterpret_cast<unsigned*>(C + crow * ldc + n) = pack_bf16(v0, v1);
        } else {
          if (n < N) C[crow * ldc + n] = __float2bfloat16_rn(v0);
          if (n + 1 < N) C[crow * ldc + n + 1] = __float2bfloat16_rn(v1);
        }
      }
    }
}

// logits <- cap * tanh(logits / cap) on fp32 rows; `in` may be the padded bf16 rows of the tensor-core head (ld elements per row)
__global__ void softcap_rows_kernel(const bf16* __restrict__ in_bf, long long ld, float* __restrict__ out, int V, long long n, float cap) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const long long row = i / V;
  const float v = in_bf ? __bfloat162float(in_bf[row * ld + (i - row * V)]) : out[i];
  out[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

}  // namespace dlm
}  // namespace b200
