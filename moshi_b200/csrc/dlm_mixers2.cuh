// Further mechanisms of the decoder-LM handle (dlm.cu), first used by the Namalix design: a parallel block on a zero-centred
// RMS norm, causal attention whose weights are sigmoids mixed over heads after the sigmoid (no softmax, no normaliser), rotary
// positions on halves or on adjacent pairs with the index-ramp rescaling, values blended with those of an earlier layer, the
// preparation of a fixed-decay retention and of the gated delta rule for the matrix-memory kernel, a gated tanh-GELU
// feed-forward, and routed experts with clamped gates behind a sigmoid router.
//   T = activation / weight / cache type (bf16, or float in the all-fp32 mode).  Norms, positions and angles, scores and
//   attention weights, routers, gates, decays, unit norms, the recurrent state and the residual stream are fp32 in both modes.
#pragma once

#include "dlm_mixers.cuh"

namespace b200 {
namespace dlm {

__device__ __forceinline__ float softplusf(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanhf(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
// gate bounded above, value bounded on both sides: g * sigmoid(1.702 g) * (u + 1)
__device__ __forceinline__ float clamped_gluf(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * sigmoidf(1.702f * g) * (u + 1.f);
}

// x = table[token] * scale -> residual stream (fp32);  h = x / sqrt(mean(x^2) + eps) * w1 -> T   (w1 = 1 + the stored weight)
template <typename T>
__global__ void __launch_bounds__(256) embed_scale_norm_kernel(const int* __restrict__ tokens, const T* __restrict__ table, int vocab, int W, float scale,
                                                               const float* __restrict__ w1, float* __restrict__ xin, T* __restrict__ h, float eps,
                                                               int* __restrict__ err) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  int id = tokens[t];
  const bool bad = id < 0 || id >= vocab;
  if (bad) { if (threadIdx.x == 0) atomicOr(err, ERR_TOKEN); id = 0; }
  const T* row = table + (long long)id * W;
  float* x = xin + t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) x[i] = bad ? 0.f : to_f(row[i]) * scale;
  __syncthreads();
  const float r = block_rrms(x, W, eps, red);
  for (int i = threadIdx.x; i < W; i += blockDim.x) h[t * W + i] = from_f<T>(x[i] * r * w1[i]);
}

// End of a parallel block, one CTA per token:  x <- x + mix + ff,  ff = a dense feed-forward's row | sum_k ew[t][k] * rows of
// the chosen experts | nothing;  optional copy of x (per-layer trace);  optional h = rms_norm(x) * w_next for the next layer.
template <typename T>
__global__ void __launch_bounds__(256) parallel_block_end_kernel(float* __restrict__ xin, const T* __restrict__ mix, const T* __restrict__ ff,
                                                                 const T* __restrict__ yexp, const float* __restrict__ ew, int top,
                                                                 float* __restrict__ trace, const float* __restrict__ w_next, T* __restrict__ h,
                                                                 int W, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float* x = xin + t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float y = to_f(mix[t * W + i]);
    if (ff) y += to_f(ff[t * W + i]);
    if (yexp) {
      float acc = 0.f;
      for (int k = 0; k < top; ++k) acc = fmaf(ew[t * top + k], to_f(yexp[(t * top + k) * W + i]), acc);
      y += acc;
    }
    const float v = x[i] + y;
    x[i] = v;
    if (trace) trace[t * W + i] = v;
  }
  if (w_next) {
    __syncthreads();
    const float r = block_rrms(x, W, eps, red);
    for (int i = threadIdx.x; i < W; i += blockDim.x) h[t * W + i] = from_f<T>(x[i] * r * w_next[i]);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Rotary positions.  rot[] holds, per token, cos and sin of pos * freq[i] (i < half), evaluated in double and multiplied by
// `amp`.  Pairing B200_ROT_HALVES: dimension i turns with i + half; B200_ROT_ADJACENT: 2i with 2i + 1.  The pair (u, v) becomes
// (u cos - v sin, v cos + u sin); dimensions from 2 * half on pass unchanged.
// ---------------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void rotary_fill(float* rot, int half, int pos, const double* __restrict__ freq, float amp) {
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, cs;
    sincos((double)pos * freq[i], &sn, &cs);
    rot[i] = (float)cs * amp; rot[half + i] = (float)sn * amp;
  }
}

// element d of a head after rotation; `head` points at the head's first element
template <typename T>
__device__ __forceinline__ float rotary_at(const T* __restrict__ head, int d, int half, int adjacent, const float* __restrict__ rot,
                                           const float* __restrict__ hb = nullptr) {      // hb: the head's bias, added before the rotation
  const float own = to_f(head[d]) + (hb ? hb[d] : 0.f);
  if (d >= 2 * half) return own;
  int i, partner; bool first;
  if (adjacent) { i = d >> 1; first = (d & 1) == 0; partner = d ^ 1; }
  else { first = d < half; i = first ? d : d - half; partner = first ? d + half : d - half; }
  const float other = to_f(head[partner]) + (hb ? hb[partner] : 0.f);
  return first ? own * rot[i] - other * rot[half + i] : own * rot[i] + other * rot[half + i];
}

// Query / key / value preparation of the sigmoid attention, one CTA per token, on the projections proj T [tokens][ld]:
//   q <- rope(q) * qscale -> qout fp32 [tokens][Nq];   k <- rope(k) -> key cache row;
//   v <- (1 - lambda) v + lambda v_first (when v_first is given) -> value cache row;   v -> v_keep (when given: this layer's
//   values are what later layers blend in).  Also the preparation of a window attention without norms or convolution.
template <typename T>
__global__ void __launch_bounds__(256) attn_rope_cache_kernel(const T* __restrict__ proj, long long ld, int off_q, int off_k, int off_v, int Nq, int Nk,
                                                              int Nv, int dim, int half, int adjacent, const double* __restrict__ freq, float amp,
                                                              float qscale, float* __restrict__ qout, T* __restrict__ kcache, T* __restrict__ vcache,
                                                              int cap, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                                              const T* __restrict__ v_first, const float* __restrict__ lambda, T* __restrict__ v_keep,
                                                              const float* __restrict__ bias = nullptr) {      // bias: fp32 [Nq | Nk | Nv], added to the projections
  extern __shared__ float rot[];        // [half] cosines, [half] sines
  const long long t = blockIdx.x;
  const T* row = proj + t * ld;
  const int pos = tok_pos[t];
  const long long crow = (long long)tok_slot[t] * cap + pos;
  rotary_fill(rot, half, pos, freq, amp);
  __syncthreads();
  for (int e = threadIdx.x; e < Nq; e += blockDim.x) {
    const int hh = e / dim, d = e - hh * dim;
    qout[t * Nq + e] = rotary_at(row + off_q + hh * dim, d, half, adjacent, rot, bias ? bias + hh * dim : nullptr) * qscale;
  }
  T* kc = kcache + crow * Nk;
  for (int e = threadIdx.x; e < Nk; e += blockDim.x) {
    const int hh = e / dim, d = e - hh * dim;
    kc[e] = from_f<T>(rotary_at(row + off_k + hh * dim, d, half, adjacent, rot, bias ? bias + Nq + hh * dim : nullptr));
  }
  T* vc = vcache + crow * Nv;
  const float lam = v_first ? lambda[0] : 0.f;
  for (int e = threadIdx.x; e < Nv; e += blockDim.x) {
    T raw = row[off_v + e];
    if (bias) raw = from_f<T>(to_f(raw) + bias[Nq + Nk + e]);
    if (v_keep) v_keep[t * Nv + e] = raw;
    vc[e] = v_first ? from_f<T>((1.f - lam) * to_f(raw) + lam * to_f(v_first[t * Nv + e])) : raw;
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Causal attention with sigmoid weights and grouped keys / values.  A tile is up to QT consecutive tokens of ONE request with
// all H query heads (the mix needs every head's weight of a (token, key) pair in one place).
//   s[g][j]  = q_g . k_{g / (H / G)}[j]             (q carries the score scale), capped: softcap * tanh(s / softcap)
//   w[g][j]  = sigmoid(s[g][j] + bias[g])  for keys j <= the token's position, else 0;   no normalisation over keys
//   w'[h][j] = sum_g mix[h][g] * w[g][j]
//   out[h]   = gate[h] * sum_j w'[h][j] v_{h / (H / G)}[j],   gate[h] = sigmoid(gate_in[token][h])
// There is no running maximum or sum: key tiles simply add up.  nsplit > 1 (grid.y): the key tiles are dealt over the splits,
// which leave plain partial sums per (token, head) row for sigmoid_attn_merge_kernel.
// ---------------------------------------------------------------------------------------------------------------------------
struct SigmoidAttnParams {
  const float* q;           // [tokens][ldq]
  long long ldq;
  const void* kcache;       // T [slots][cap][G * dim]
  const void* vcache;       // T [slots][cap][G * vdim]
  const float* mix;         // [H][H]
  const float* bias;        // [H]
  const float* gate_in;     // [tokens][ldg], the H gate pre-activations first
  long long ldg;
  const int* tile_row0;     // first (token, head) row of the tile = first token * H
  const int* tile_rows;     // rows of the tile = tokens * H
  const int* tile_slot;
  const int* tok_pos;
  void* out;                // T [tokens][H * vdim]
  float* part;              // nsplit > 1: [tile][split][QT * H][vdim]
  int cap, H, G, dim, vdim, QT, KT, nsplit, kstride;      // kstride: elements between staged key rows (odd number of words)
  int vec;                  // key and value rows are multiples of 16 bytes: staged with 16-byte loads
  float softcap;            // <= 0: none
};

__device__ __forceinline__ float sigmoid_weight(float s, float softcap, float bias) {
  if (softcap > 0.f) s = softcap * tanhf(s / softcap);
  return sigmoidf(s + bias);
}

template <typename T>
__global__ void __launch_bounds__(256) sigmoid_attn_kernel(SigmoidAttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, G = p.G, dim = p.dim, vdim = p.vdim, QT = p.QT, KT = p.KT, rep = H / G;
  const int Nq = H * dim, Nk = G * dim, Nv = G * vdim, KS = KT + 1;
  float* qs = reinterpret_cast<float*>(smem_raw);                  // [QT][Nq]
  float* oacc = qs + QT * Nq;                                      // [QT][H * vdim]
  float* sw = oacc + QT * H * vdim;                                // [QT * H][KS] weights of every head
  float* sp = sw + QT * H * KS;                                    // [QT * H][KS] mixed weights
  float* mixs = sp + QT * H * KS;                                  // [H][H]
  float* bs = mixs + H * H;                                        // [H]
  T* vs = reinterpret_cast<T*>(smem_raw + (((size_t)((bs + H) - qs) * 4 + 15) / 16) * 16);     // [KT][Nv], on 16 bytes
  T* ks = vs + (size_t)KT * Nv;                                    // [KT][kstride]
  const int tile = blockIdx.x, split = blockIdx.y;
  const int tok0 = p.tile_row0[tile] / H, nt = p.tile_rows[tile] / H;
  const int p0 = p.tok_pos[tok0];                                  // positions p0 .. p0 + nt - 1
  const T* kc = static_cast<const T*>(p.kcache) + (long long)p.tile_slot[tile] * p.cap * Nk;
  const T* vc = static_cast<const T*>(p.vcache) + (long long)p.tile_slot[tile] * p.cap * Nv;
  const int kmax = p0 + nt - 1;
  const int n_kt = kmax / KT + 1;
  const int per = (n_kt + p.nsplit - 1) / p.nsplit;
  const int kt0 = split * per, kt1 = min(n_kt, kt0 + per);

  for (int i = threadIdx.x; i < QT * Nq; i += 256) {
    const int qt = i / Nq;
    qs[i] = qt < nt ? p.q[(long long)(tok0 + qt) * p.ldq + (i - qt * Nq)] : 0.f;
  }
  for (int i = threadIdx.x; i < QT * H * vdim; i += 256) oacc[i] = 0.f;
  for (int i = threadIdx.x; i < H * H; i += 256) mixs[i] = p.mix[i];
  for (int i = threadIdx.x; i < H; i += 256) bs[i] = p.bias[i];

  for (int kt = kt0; kt < kt1; ++kt) {
    const int kb = kt * KT;
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
    // weights of every head: item (row = qt * H + g, key j), keys fastest
    for (int i = threadIdx.x; i < QT * H * KT; i += 256) {
      const int row = i / KT, j = i - row * KT;
      const int qt = row / H, g = row - qt * H;
      float w = 0.f;
      if (j < nk && qt < nt && kb + j <= p0 + qt) {
        const float* qv = qs + qt * Nq + g * dim;
        const T* kv = ks + j * p.kstride + (g / rep) * dim;
        float acc = 0.f;
        for (int d = 0; d < dim; ++d) acc = fmaf(qv[d], to_f(kv[d]), acc);
        w = sigmoid_weight(acc, p.softcap, bs[g]);
      }
      sw[row * KS + j] = w;
    }
    __syncthreads();
    // mix over heads (a key the token does not see has weight 0 in every head, so the mix leaves it 0)
    for (int i = threadIdx.x; i < nt * H * KT; i += 256) {
      const int row = i / KT, j = i - row * KT;
      const int qt = row / H, h = row - qt * H;
      float s = 0.f;
      for (int g = 0; g < H; ++g) s = fmaf(mixs[h * H + g], sw[(qt * H + g) * KS + j], s);
      sp[row * KS + j] = s;
    }
    __syncthreads();
    // weighted sum of the values: item (row, c), c fastest
    for (int i = threadIdx.x; i < nt * H * vdim; i += 256) {
      const int row = i / vdim, c = i - row * vdim;
      const T* vv = vs + ((row % H) / rep) * vdim + c;
      const float* w = sp + row * KS;
      float acc = oacc[i];
      for (int j = 0; j < nk; ++j) acc = fmaf(w[j], to_f(vv[j * Nv]), acc);
      oacc[i] = acc;
    }
  }
  __syncthreads();
  if (p.nsplit == 1) {
    T* out = static_cast<T*>(p.out);
    for (int i = threadIdx.x; i < nt * H * vdim; i += 256) {
      const int row = i / vdim;
      const float gate = sigmoidf(p.gate_in[(long long)(tok0 + row / H) * p.ldg + row % H]);
      out[(long long)tok0 * H * vdim + i] = from_f<T>(oacc[i] * gate);
    }
  } else {
    float* dst = p.part + ((long long)tile * p.nsplit + split) * (QT * H) * vdim;
    for (int i = threadIdx.x; i < nt * H * vdim; i += 256) dst[i] = oacc[i];
  }
}

// sums the key splits of one (token, head) row in split order and applies the head's gate; grid (tiles, rows per tile)
template <typename T>
__global__ void __launch_bounds__(128) sigmoid_attn_merge_kernel(const float* __restrict__ part, const int* __restrict__ tile_row0,
                                                                 const int* __restrict__ tile_rows, const float* __restrict__ gate_in, long long ldg,
                                                                 T* __restrict__ out, int H, int vdim, int nsplit, int rows_per_tile) {
  const int tile = blockIdx.x, lr = blockIdx.y;
  if (lr >= tile_rows[tile]) return;
  const long long row = tile_row0[tile] + lr;
  const float gate = sigmoidf(gate_in[(row / H) * ldg + row % H]);
  const float* base = part + ((long long)tile * nsplit * rows_per_tile + lr) * vdim;
  const long long ss = (long long)rows_per_tile * vdim;
  for (int c = threadIdx.x; c < vdim; c += 128) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) acc += base[s * ss + c];
    out[row * vdim + c] = from_f<T>(acc * gate);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores for bf16 caches (dim and vdim multiples of 16): a tile is 16 consecutive tokens of one
// request with all H heads, a key tile 32 keys.  Per key tile: (1) scores Q_g K^T per head as mma.sync m16n8k16 (queries rounded
// to bf16 once, fp32 accumulate), cap, bias and sigmoid in fp32 on the accumulator registers, weights into shared memory as
// fp32; (2) the mix over heads in fp32, one warp per token, lane = key, the mixed weights going back as bf16; (3) O_h += W'_h V
// on the tensor cores, the accumulators of a warp's NI items (head, 64 value columns) in registers.  16 warps per CTA when that
// leaves a warp at most two items, else 8.
// ---------------------------------------------------------------------------------------------------------------------------
// the same weight with the hardware exponential and reciprocal (2 ulp each: far below the bf16 rounding of the operands around it)
__device__ __forceinline__ float sigmoid_weight_fast(float s, float softcap, float inv_cap, float bias) {
  if (softcap > 0.f) s = softcap * (1.f - __fdividef(2.f, 1.f + __expf(2.f * s * inv_cap)));      // tanh(z) = 1 - 2 / (1 + e^2z)
  return __fdividef(1.f, 1.f + __expf(-(s + bias)));
}

// Keys of a tile are copied asynchronously while the previous tile's mix and weighted sums run, values while the tile's own
// scores and mix run: K and V have one buffer each and no thread waits for a load it has just issued.
template <int NI, int NW>      // accumulator items per warp, warps per CTA
__global__ void __launch_bounds__(NW * 32) sigmoid_attn_mma_kernel(SigmoidAttnParams p) {
  constexpr int QT = 16, KT = 32, SS = 40, PS = 40, NT = NW * 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, G = p.G, dim = p.dim, vdim = p.vdim, rep = H / G;
  const int Nq = H * dim, Nk = G * dim, Nv = G * vdim, QS = Nq + 8, KS = Nk + 8, VS = Nv + 8, VC = (vdim + 63) / 64;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                   // [16][QS]
  bf16* Ks = Qs + QT * QS;                                        // [32][KS]
  bf16* Vs = Ks + KT * KS;                                        // [32][VS]
  bf16* pb = Vs + KT * VS;                                        // [H][16][PS] mixed weights of the key tile
  float* sw = reinterpret_cast<float*>(pb + H * QT * PS);         // [H][16][SS] weights of every head
  float* mixs = sw + H * QT * SS;                                 // [H][max(H, 16)]
  float* bs = mixs + H * max(H, 16);                              // [H]
  // the last tiles of a prompt see the most keys: they are started first, so that the short ones fill the end of the launch
  const int tile = gridDim.x - 1 - blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, t4 = lane & 3, mi = lane >> 3;
  const int tok0 = p.tile_row0[tile] / H, nt = p.tile_rows[tile] / H;
  const int p0 = p.tok_pos[tok0];
  const bf16* kc = static_cast<const bf16*>(p.kcache) + (long long)p.tile_slot[tile] * p.cap * Nk;
  const bf16* vc = static_cast<const bf16*>(p.vcache) + (long long)p.tile_slot[tile] * p.cap * Nv;
  const int kmax = p0 + nt - 1;
  const int n_kt = kmax / KT + 1;
  const int per = (n_kt + p.nsplit - 1) / p.nsplit;
  const int kt0 = split * per, kt1 = min(n_kt, kt0 + per);
  const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
  const int kw = Nk / 8, vw = Nv / 8;
  // rows past the last key are zero-filled (their weights are zero, they must be finite)
  auto load_keys = [&](int kt) {
    const int kb = kt * KT, nk = min(KT, kmax + 1 - kb);
    const bf16* src = kc + (long long)kb * Nk;
    for (int i = threadIdx.x; i < KT * kw; i += NT) {
      const int j = i / kw, e = i - j * kw;
      cp_async_16_or_zero(Ks + j * KS + e * 8, j < nk ? src + (long long)j * Nk + e * 8 : kc, j < nk);
    }
  };
  auto load_values = [&](int kt) {
    const int kb = kt * KT, nk = min(KT, kmax + 1 - kb);
    const bf16* src = vc + (long long)kb * Nv;
    for (int i = threadIdx.x; i < KT * vw; i += NT) {
      const int j = i / vw, e = i - j * vw;
      cp_async_16_or_zero(Vs + j * VS + e * 8, j < nk ? src + (long long)j * Nv + e * 8 : vc, j < nk);
    }
  };
  if (kt0 < kt1) load_keys(kt0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  for (int i = threadIdx.x; i < QT * (Nq / 2); i += NT) {
    const int qt = i / (Nq / 2), e = (i - qt * (Nq / 2)) * 2;
    float2 v = make_float2(0.f, 0.f);
    if (qt < nt) v = *reinterpret_cast<const float2*>(p.q + (long long)(tok0 + qt) * p.ldq + e);
    *reinterpret_cast<unsigned*>(Qs + qt * QS + e) = pack_bf16(v.x, v.y);
  }
  if (H <= 16) {      // rows padded to 16 entries (zeros) for the register-blocked mix
    for (int i = threadIdx.x; i < H * 16; i += NT) mixs[i] = (i & 15) < H ? p.mix[(i >> 4) * H + (i & 15)] : 0.f;
  } else {
    for (int i = threadIdx.x; i < H * H; i += NT) mixs[i] = p.mix[i];
  }
  for (int i = threadIdx.x; i < H; i += NT) bs[i] = p.bias[i];
  for (int i = threadIdx.x; i < H * QT * PS / 2; i += NT) reinterpret_cast<unsigned*>(pb)[i] = 0u;
  float oacc[NI][8][4];
#pragma unroll
  for (int a = 0; a < NI; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) { oacc[a][b][0] = oacc[a][b][1] = oacc[a][b][2] = oacc[a][b][3] = 0.f; }

  for (int kt = kt0; kt < kt1; ++kt) {
    const int kb = kt * KT;
    const int nk = min(KT, kmax + 1 - kb);
    __syncthreads();                                              // the previous tile's weighted sums are done with the values
    load_values(kt);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");          // this tile's keys (issued a tile ago) have landed
    __syncthreads();
    // (1) scores and weights, one head at a time per warp
    for (int h = warp; h < H; h += NW) {
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
      float* dst = sw + h * QT * SS;
      const float bias = bs[h];
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        const int j = nb * 8 + 2 * t4;      // keys j, j + 1 of the tile; rows g8 and g8 + 8
        float w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qt = g8 + 8 * (e >> 1), kj = kb + j + (e & 1);
          const bool vis = j + (e & 1) < nk && qt < nt && kj <= p0 + qt;
          w[e] = vis ? sigmoid_weight_fast(sacc[nb][e], p.softcap, inv_cap, bias) : 0.f;
        }
        *reinterpret_cast<float2*>(dst + g8 * SS + j) = make_float2(w[0], w[1]);
        *reinterpret_cast<float2*>(dst + (g8 + 8) * SS + j) = make_float2(w[2], w[3]);
      }
    }
    __syncthreads();
    if (kt + 1 < kt1) load_keys(kt + 1);                          // every warp is done with this tile's keys
    asm volatile("cp.async.commit_group;" ::: "memory");
    // (2) mix over heads; lane = key
    if (H <= 16) {
      for (int qt = warp; qt < nt; qt += NW) {                    // rows past the tile's tokens stay zero
        float raw[16];
#pragma unroll
        for (int g = 0; g < 16; ++g) raw[g] = g < H ? sw[(g * QT + qt) * SS + lane] : 0.f;
        for (int h = 0; h < H; ++h) {
          const float4* mr = reinterpret_cast<const float4*>(mixs + h * 16);
          float s = 0.f;
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4) {
            const float4 mv = mr[g4];
            s = fmaf(mv.x, raw[4 * g4], s); s = fmaf(mv.y, raw[4 * g4 + 1], s); s = fmaf(mv.z, raw[4 * g4 + 2], s); s = fmaf(mv.w, raw[4 * g4 + 3], s);
          }
          pb[(h * QT + qt) * PS + lane] = __float2bfloat16_rn(s);
        }
      }
    } else {
      for (int row = warp; row < H * QT; row += NW) {
        const int h = row / QT, qt = row - h * QT;
        if (qt >= nt) continue;
        float s = 0.f;
        for (int g = 0; g < H; ++g) s = fmaf(mixs[h * H + g], sw[(g * QT + qt) * SS + lane], s);
        pb[row * PS + lane] = __float2bfloat16_rn(s);
      }
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");          // this tile's values have landed (the next keys may still fly)
    __syncthreads();
    // (3) weighted sums of the values
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
      const int it = warp + NW * ii;
      if (it >= H * VC) break;
      const int h = it / VC, c0 = (it - h * VC) * 64;
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
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int ii = 0; ii < NI; ++ii) {
    const int it = warp + NW * ii;
    if (it >= H * VC) break;
    const int h = it / VC, c0 = (it - h * VC) * 64;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int qt = g8 + 8 * hf;
      if (qt >= nt) continue;
      if (p.nsplit == 1) {
        const float gate = sigmoidf(p.gate_in[(long long)(tok0 + qt) * p.ldg + h]);
        bf16* dst = static_cast<bf16*>(p.out) + ((long long)(tok0 + qt) * H + h) * vdim + c0;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
          if (c0 + nb * 8 < vdim)
            *reinterpret_cast<unsigned*>(dst + nb * 8 + 2 * t4) = pack_bf16(oacc[ii][nb][2 * hf] * gate, oacc[ii][nb][2 * hf + 1] * gate);
      } else {
        float* dst = p.part + (((long long)tile * p.nsplit + split) * (QT * H) + qt * H + h) * vdim;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
          if (c0 + nb * 8 < vdim)
            *reinterpret_cast<float2*>(dst + c0 + nb * 8 + 2 * t4) = make_float2(oacc[ii][nb][2 * hf], oacc[ii][nb][2 * hf + 1]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Preparation of the gated delta rule for matrix_memory_scan_kernel<MODE_DELTA>, one CTA per token, on the convolved projections
// c fp32 [tokens][2 * G * dim + heads * vdim] (q, k, v before their activation):
//   q <- unit(silu(q)) * dim^-1/2,  k <- unit(silu(k))   per query/key head, unit(x) = x / sqrt(sum x^2 + 1e-6);
//   value head h reads query/key head h / (heads / G);   v <- silu(v);
//   beta = sigmoid(z[h]),  g = exp(-exp(A_log[h]) * softplus(z[heads + h] + dt_bias[h]))   (z: the two gate projections, fp32)
// prep row of (token, head): [q | k | g, beta] (plain or lane-ordered, as scan_prep_kernel lays rows out).
// ---------------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) delta_prep_kernel(ScanParams p, const float* __restrict__ conv, int G, const float* __restrict__ A_log,
                                                         const float* __restrict__ dt_bias, long long ldz) {
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
  }
  for (int h = threadIdx.x; h < heads; h += 256) {
    const float* z = p.z + t * ldz;
    const float lg = -expf(A_log[h]) * softplusf(z[heads + h] + dt_bias[h]), be = sigmoidf(z[h]);
    dst[h * p.prow + 2 * Dp] = expf(lg);
    dst[h * p.prow + 2 * Dp + 1] = be;
    if (p.tokM) { p.tokM[(t * heads + h) * 4] = lg; p.tokM[(t * heads + h) * 4 + 1] = be; }      // the chunked form reads the logarithm
  }
  for (int i = threadIdx.x; i < heads * vdim; i += 256) p.vprep[t * heads * vdim + i] = siluf(c[2 * G * dim + i]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// The gated delta rule over a portion, in chunks of DELTA_CH tokens (prompts; single tokens keep matrix_memory_scan_kernel).
// With S_0 the state in front of a chunk, L_t the sum of log g over the chunk's tokens up to t, and u_t what token t writes:
//   S_t = e^(L_t) S_0 + sum_{i <= t} e^(L_t - L_i) k_i u_i^T
//   u_t + sum_{i < t} A[t][i] u_i = b_t,   b_t = beta_t (v_t - e^(L_t) S_0^T k_t),   A[t][i] = beta_t e^(L_t - L_i) (k_t . k_i)
//   i.e. U = T B with T = (I + A)^-1, unit lower triangular, which depends on the chunk's keys and gates alone
//   o_t = e^(L_t) S_0^T q_t + sum_{i <= t} P[t][i] u_i,                       P[t][i] = e^(L_t - L_i) (k_i . q_t)
// so a chunk costs three products against the state (K S_0, Q S_0 and the state's update) and two small triangular products
// (T B and P U), all of which run over the chunk's tokens at once.  Every exponent is <= 0: no decay is ever inverted.
// delta_gram_kernel computes L, T and P for every (chunk, head) side by side (the forward substitution that inverts I + A runs
// there, off the chain); delta_chunk_kernel walks a request's chunks in order.
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int DELTA_CH = 32;

struct DeltaChunkParams {
  const float* prep;        // [tokens][heads][prow]: q (scaled) | k, plain rows of `dim` each
  const float* vprep;       // [tokens][heads * vdim]
  const float* gates;       // [tokens][heads][4]: log g, beta
  int prow;
  float* gram;              // [chunks][heads][2 * DELTA_CH + 2 * DELTA_CH * DELTA_CH]: L | beta | T | P
  const int* chunk_tok0;    // per chunk: first token of the step, tokens
  const int* chunk_nt;
  const int* ent_chunk0;    // per entry: its first chunk
  const int* ent_tok0; const int* ent_ntok; const int* ent_slot; const int* ent_pos0;
  float* St;                // [slots][heads][vdim][dim]
  float* out;               // [tokens][heads * vdim]
  int heads, dim, vdim;
  // one decay per key channel (prep rows q | k | log g | beta): the gram kernel leaves, per token, the rows the walk multiplies the
  // state with, rows3 [tokens][heads][3 dim] = e^(L_t) q | e^(L_t) k | e^(L_end - L_t) k, and per chunk gend [chunks][heads][dim] = e^(L_end)
  float* rows3 = nullptr;
  float* gend = nullptr;
};

__global__ void __launch_bounds__(256) delta_gram_kernel(DeltaChunkParams p) {
  constexpr int C = DELTA_CH;
  extern __shared__ float gsm[];
  const int ck = blockIdx.x, head = blockIdx.y, dim = p.dim, DS = dim + 1;
  float* ks = gsm;                     // [C][DS]
  float* qs = ks + C * DS;             // [C][DS]
  float* L = qs + C * DS;              // [C]
  float* be = L + C;                   // [C]
  const int tok0 = p.chunk_tok0[ck], nt = p.chunk_nt[ck];
  for (int i = threadIdx.x; i < C * dim; i += 256) {
    const int t = i / dim, d = i - t * dim;
    const float* row = p.prep + ((long long)(tok0 + t) * p.heads + head) * p.prow;
    qs[t * DS + d] = t < nt ? row[d] : 0.f;
    ks[t * DS + d] = t < nt ? row[dim + d] : 0.f;
  }
  if (threadIdx.x == 0) {
    float acc = 0.f;
    for (int t = 0; t < C; ++t) {
      if (t < nt) acc += p.gates[((long long)(tok0 + t) * p.heads + head) * 4];
      L[t] = acc;
      be[t] = t < nt ? p.gates[((long long)(tok0 + t) * p.heads + head) * 4 + 1] : 0.f;
    }
  }
  __syncthreads();
  float* g = p.gram + ((long long)ck * p.heads + head) * (2 * C + 2 * C * C);
  if (threadIdx.x < C) { g[threadIdx.x] = L[threadIdx.x]; g[C + threadIdx.x] = be[threadIdx.x]; }
  g += C;
  float* As = be + C;                  // [C][C]
  for (int i = threadIdx.x; i < C * C; i += 256) {
    const int t = i / C, j = i - t * C;
    float a = 0.f, pq = 0.f;
    if (j <= t && t < nt) {
      float kk = 0.f, kq = 0.f;
      for (int d = 0; d < dim; ++d) { kk = fmaf(ks[t * DS + d], ks[j * DS + d], kk); kq = fmaf(ks[j * DS + d], qs[t * DS + d], kq); }
      const float dec = expf(L[t] - L[j]);
      pq = dec * kq;
      if (j < t) a = be[t] * dec * kk;
    }
    As[i] = a;
    g[C + C * C + i] = pq;
  }
  __syncthreads();
  // T = (I + A)^-1, unit lower triangular: lane j of warp 0 solves (I + A) x = e_j by forward substitution (x_t = 0 above the diagonal)
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

// A CTA owns 32 columns of one (request, head): lane = column, warp w (of 8) owns rows [w * 4 R4, (w + 1) * 4 R4) of the state in
// registers.  Grid: (entries * heads, ceil(vdim / 32)).
template <int R4, bool CHD = false>      // float4 groups of rows per thread: dim <= 32 R4; CHD: one decay per key channel (rows3, gend)
__global__ void __launch_bounds__(256) delta_chunk_kernel(DeltaChunkParams p) {
  constexpr int C = DELTA_CH, R = 4 * R4, NW = 8, DP = NW * R;        // rows per thread, warps, padded key size
  constexpr int NBUF = R4 <= 4 ? 2 : 1;                               // what a chunk reads is staged one chunk ahead when two buffers fit
  constexpr int NROW = CHD ? 3 : 2;                                   // row sets per token: q, k (and the keys as the state's update takes them)
  constexpr int GM = 2 * C + 2 * C * C, STAGE = NROW * C * DP + C * 32 + GM;
  extern __shared__ __align__(16) float csm[];
  float* wp = csm + NBUF * STAGE;      // [NW][C][32] partial K S_0
  float* op = wp + NW * C * 32;        // [NW][C][32] partial Q S_0, then [0]: e^(L_t) Q S_0
  float* us = op + NW * C * 32;        // [C][32] what the tokens write
  float* uw = us + C * 32;             // [C][32] the same, decayed to the chunk's end
  float* bs = uw + C * 32;             // [C][32] right-hand sides b_t
  float* eL = bs + C * 32;             // [C] e^(L_t): the decay from the chunk's start to token t
  float* eW = eL + C;                  // [C] e^(L_end - L_t): from token t to the chunk's end
  const int heads = p.heads, dim = p.dim, vdim = p.vdim;
  const int ent = blockIdx.x / heads, head = blockIdx.x - ent * heads;
  const int tok0 = p.ent_tok0[ent], ntok = p.ent_ntok[ent], slot = p.ent_slot[ent], pos0 = p.ent_pos0[ent], chunk0 = p.ent_chunk0[ent];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, col = blockIdx.y * 32 + lane, row0 = warp * R;
  const bool live_col = col < vdim;
  float* Sbase = p.St + ((long long)slot * heads + head) * vdim * dim;
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = (pos0 > 0 && live_col && row0 + i < dim) ? Sbase[(long long)col * dim + row0 + i] : 0.f;

  const int n_chunks = (ntok + C - 1) / C;
  const bool vec = (dim & 3) == 0 && (vdim & 3) == 0;      // rows of q, k and the column slice of v start on 16 bytes
  // chunk ck into buffer b: q and k rows (zero beyond the chunk's tokens and the key size), the values of this CTA's columns, L | beta | A | P
  auto stage = [&](int ck, int b) {
    float* ks = csm + b * STAGE;       // [C][DP]
    float* qs = ks + C * DP;           // [C][DP]
    float* k2 = qs + C * DP;           // CHD: [C][DP] keys decayed to the chunk's end
    float* vs = qs + (NROW - 1) * C * DP;      // [C][32]
    float* gm = vs + C * 32;
    const int t0 = tok0 + ck * C, nt = min(C, ntok - ck * C);
    const float* gl = p.gram + ((long long)(chunk0 + ck) * heads + head) * GM;
    const float* rows = CHD ? p.rows3 : p.prep;
    const int rstride = CHD ? 3 * dim : p.prow;
    if (vec) {
      for (int i = threadIdx.x; i < C * (DP / 4); i += 256) {
        const int t = i / (DP / 4), d = (i - t * (DP / 4)) * 4;
        const bool ok = t < nt && d < dim;
        const float* row = rows + ((long long)(t0 + (ok ? t : 0)) * heads + head) * rstride;
        cp_async_16_or_zero(qs + t * DP + d, ok ? row + d : row, ok);
        cp_async_16_or_zero(ks + t * DP + d, ok ? row + dim + d : row, ok);
        if (CHD) cp_async_16_or_zero(k2 + t * DP + d, ok ? row + 2 * dim + d : row, ok);
      }
      for (int i = threadIdx.x; i < C * 8; i += 256) {
        const int t = i >> 3, c = blockIdx.y * 32 + (i & 7) * 4;
        const bool ok = t < nt && c < vdim;
        const float* src = p.vprep + (long long)(t0 + (ok ? t : 0)) * heads * vdim + head * vdim + (ok ? c : 0);
        cp_async_16_or_zero(vs + t * 32 + (i & 7) * 4, src, ok);
      }
      for (int i = threadIdx.x; i < GM / 4; i += 256) cp_async_16_or_zero(gm + 4 * i, gl + 4 * i, true);
    } else {
      for (int i = threadIdx.x; i < C * DP; i += 256) {
        const int t = i / DP, d = i - t * DP;
        const bool ok = t < nt && d < dim;
        const float* row = rows + ((long long)(t0 + (ok ? t : 0)) * heads + head) * rstride;
        qs[i] = ok ? row[d] : 0.f;
        ks[i] = ok ? row[dim + d] : 0.f;
        if (CHD) k2[i] = ok ? row[2 * dim + d] : 0.f;
      }
      for (int i = threadIdx.x; i < C * 32; i += 256) {
        const int t = i >> 5, c = blockIdx.y * 32 + (i & 31);
        vs[i] = (t < nt && c < vdim) ? p.vprep[(long long)(t0 + t) * heads * vdim + head * vdim + c] : 0.f;
      }
      for (int i = threadIdx.x; i < GM; i += 256) gm[i] = gl[i];
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage(0, 0);
  for (int ck = 0; ck < n_chunks; ++ck) {
    const int t0 = tok0 + ck * C, nt = min(C, ntok - ck * C), buf = NBUF == 2 ? (ck & 1) : 0;
    const float* ks = csm + buf * STAGE;
    const float* qs = ks + C * DP;
    const float* kw = CHD ? qs + C * DP : ks;      // the keys as the state's update takes them
    const float* vs = qs + (NROW - 1) * C * DP;
    const float* gm = vs + C * 32;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                   // this chunk has landed for every thread, and every thread is done with the previous one
    if (NBUF == 2 && ck + 1 < n_chunks) stage(ck + 1, buf ^ 1);
    if (threadIdx.x < C) {
      const float lt = gm[threadIdx.x], le = gm[nt - 1];
      eL[threadIdx.x] = expf(lt);
      eW[threadIdx.x] = expf(le - lt);
    }
    const float* Bt = gm + C;
    const float* A = gm + 2 * C;             // T = (I + A)^-1
    const float* P = gm + 2 * C + C * C;
    // (1) this warp's share of K S_0 and Q S_0 for every token of the chunk (rows of tokens past the chunk's end are zero)
#pragma unroll 2
    for (int t = 0; t < C; t += 2) {
      float a0 = 0.f, b0 = 0.f, a1 = 0.f, b1 = 0.f;
#pragma unroll
      for (int j = 0; j < R4; ++j) {
        const float4 k0 = *reinterpret_cast<const float4*>(ks + t * DP + row0 + 4 * j), k1 = *reinterpret_cast<const float4*>(ks + (t + 1) * DP + row0 + 4 * j);
        const float4 q0 = *reinterpret_cast<const float4*>(qs + t * DP + row0 + 4 * j), q1 = *reinterpret_cast<const float4*>(qs + (t + 1) * DP + row0 + 4 * j);
        a0 = fmaf(k0.x, S[4 * j], a0); a0 = fmaf(k0.y, S[4 * j + 1], a0); a0 = fmaf(k0.z, S[4 * j + 2], a0); a0 = fmaf(k0.w, S[4 * j + 3], a0);
        b0 = fmaf(q0.x, S[4 * j], b0); b0 = fmaf(q0.y, S[4 * j + 1], b0); b0 = fmaf(q0.z, S[4 * j + 2], b0); b0 = fmaf(q0.w, S[4 * j + 3], b0);
        a1 = fmaf(k1.x, S[4 * j], a1); a1 = fmaf(k1.y, S[4 * j + 1], a1); a1 = fmaf(k1.z, S[4 * j + 2], a1); a1 = fmaf(k1.w, S[4 * j + 3], a1);
        b1 = fmaf(q1.x, S[4 * j], b1); b1 = fmaf(q1.y, S[4 * j + 1], b1); b1 = fmaf(q1.z, S[4 * j + 2], b1); b1 = fmaf(q1.w, S[4 * j + 3], b1);
      }
      wp[(warp * C + t) * 32 + lane] = a0; wp[(warp * C + t + 1) * 32 + lane] = a1;
      op[(warp * C + t) * 32 + lane] = b0; op[(warp * C + t + 1) * 32 + lane] = b1;
      if (t + 2 >= nt) break;
    }
    __syncthreads();
    // (2) tokens dealt over the warps: b_t and e^(L_t) Q S_0 from the partial sums, then U = T B (four running sums)
    for (int t = warp; t < nt; t += NW) {
      float w = 0.f, o = 0.f;
#pragma unroll
      for (int g = 0; g < NW; ++g) { w += wp[(g * C + t) * 32 + lane]; o += op[(g * C + t) * 32 + lane]; }
      bs[t * 32 + lane] = Bt[t] * (vs[t * 32 + lane] - eL[t] * w);
      op[t * 32 + lane] = eL[t] * o;          // row t of part 0 is read by this thread alone
    }
    __syncthreads();
    for (int t = warp; t < nt; t += NW) {
      float u0 = bs[t * 32 + lane], u1 = 0.f, u2 = 0.f, u3 = 0.f;
      int i = 0;
      for (; i + 4 <= t; i += 4) {
        u0 = fmaf(A[t * C + i], bs[i * 32 + lane], u0); u1 = fmaf(A[t * C + i + 1], bs[(i + 1) * 32 + lane], u1);
        u2 = fmaf(A[t * C + i + 2], bs[(i + 2) * 32 + lane], u2); u3 = fmaf(A[t * C + i + 3], bs[(i + 3) * 32 + lane], u3);
      }
      for (; i < t; ++i) u0 = fmaf(A[t * C + i], bs[i * 32 + lane], u0);
      const float u = (u0 + u1) + (u2 + u3);
      us[t * 32 + lane] = u;
      uw[t * 32 + lane] = eW[t] * u;
    }
    __syncthreads();
    // (3) read-outs (tokens dealt over the warps, four running sums) and the state at the chunk's end
    for (int t = warp; t < nt; t += NW) {
      float o0 = op[t * 32 + lane], o1 = 0.f, o2 = 0.f, o3 = 0.f;
      int i = 0;
      for (; i + 3 <= t; i += 4) {
        o0 = fmaf(P[t * C + i], us[i * 32 + lane], o0); o1 = fmaf(P[t * C + i + 1], us[(i + 1) * 32 + lane], o1);
        o2 = fmaf(P[t * C + i + 2], us[(i + 2) * 32 + lane], o2); o3 = fmaf(P[t * C + i + 3], us[(i + 3) * 32 + lane], o3);
      }
      for (; i <= t; ++i) o0 = fmaf(P[t * C + i], us[i * 32 + lane], o0);
      if (live_col) p.out[(long long)(t0 + t) * heads * vdim + head * vdim + col] = (o0 + o1) + (o2 + o3);
    }
    if (CHD) {      // every row of the state has its own decay over the chunk (the gram kernel leaves L = 0: the factors above are 1)
      const float* ge = p.gend + ((long long)(chunk0 + ck) * heads + head) * dim;
#pragma unroll
      for (int i = 0; i < R; ++i) S[i] *= row0 + i < dim ? __ldg(ge + row0 + i) : 0.f;
    } else {
      const float gall = expf(gm[nt - 1]);
#pragma unroll
      for (int i = 0; i < R; ++i) S[i] *= gall;
    }
#pragma unroll 4
    for (int t = 0; t < nt; ++t) {
      const float w = uw[t * 32 + lane];
#pragma unroll
      for (int j = 0; j < R4; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(kw + t * DP + row0 + 4 * j);
        S[4 * j] = fmaf(k4.x, w, S[4 * j]); S[4 * j + 1] = fmaf(k4.y, w, S[4 * j + 1]); S[4 * j + 2] = fmaf(k4.z, w, S[4 * j + 2]); S[4 * j + 3] = fmaf(k4.w, w, S[4 * j + 3]);
      }
    }
    if (NBUF == 1 && ck + 1 < n_chunks) {      // one buffer: the next chunk is staged once every thread has left this one
      __syncthreads();
      stage(ck + 1, 0);
    }
  }
  if (live_col) {
#pragma unroll
    for (int i = 0; i < R; ++i) if (row0 + i < dim) Sbase[(long long)col * dim + row0 + i] = S[i];
  }
}

// out = gelu_tanh(gate) * up on the two halves of a concatenated projection
template <typename T>
__global__ void __launch_bounds__(256) gated_gelu_kernel(const T* __restrict__ proj, long long ldp, int off_gate, int off_up, T* __restrict__ out, int F, long long n) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const long long t = i / F; const int f = (int)(i - t * F);
  out[i] = from_f<T>(gelu_tanhf(to_f(proj[t * ldp + off_gate + f])) * to_f(proj[t * ldp + off_up + f]));
}

// out[r][f] = clamped_glu(in[r][2f], in[r][2f + 1]): the experts' first product with gate and value rows interleaved
template <typename T>
__global__ void __launch_bounds__(256) clamped_glu_kernel(const T* __restrict__ in, T* __restrict__ out, int F, long long n, float limit) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const long long r = i / F; const int f = (int)(i - r * F);
  out[i] = from_f<T>(clamped_gluf(to_f(in[r * 2 * F + 2 * f]), to_f(in[r * 2 * F + 2 * f + 1]), limit));
}

// Router with sigmoid scores, per token (one warp): s = sigmoid(logit); the `top` experts with the largest s + correction are
// chosen (ties: the lower index); their weights are s / (sum of the chosen s + 1e-20) * out_scale.
__global__ void __launch_bounds__(128) moe_route_sigmoid_kernel(const float* __restrict__ logits, long long ldl, const float* __restrict__ correction,
                                                                int E, int top, float out_scale, int* __restrict__ idx, float* __restrict__ wts, int n_tok) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= n_tok) return;
  const float* z = logits + (long long)t * ldl;
  float den = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY, bs = 0.f; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= idx[(long long)t * top + j] == e;
      const float s = sigmoidf(z[e]), v = s + correction[e];
      if (!taken && (v > best || (v == best && e < bi))) { best = v; bi = e; bs = s; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, bs, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; bs = os; }
    }
    den += bs;
    if (lane == 0) { idx[(long long)t * top + k] = bi; wts[(long long)t * top + k] = bs; }
    __syncwarp();
  }
  __syncwarp();
  if (lane < top) wts[(long long)t * top + lane] = wts[(long long)t * top + lane] / (den + 1e-20f) * out_scale;
}

// w <- 1 + w (a norm weight stored around zero), once at load
__global__ void add_one_kernel(float* __restrict__ w, int n) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n) w[i] += 1.f;
}

}  // namespace dlm
}  // namespace b200
