// Kernels of the decoder-LM handle (dlm.cu): the mechanisms a layer-list language model is assembled from.
//   T = activation / weight / cache type (bf16, or float for the all-fp32 mode); every reduction, norm, score, softmax,
//   gate, the residual stream and the depth average are fp32 in both modes.
#pragma once

#include "common.cuh"
#include "tc_prims.cuh"

namespace b200 {
namespace dlm {

using bf16 = __nv_bfloat16;

enum { ERR_TOKEN = 1, ERR_WAIT = 2 };      // device error flags: a token id outside the embedding table; a copy into shared memory that never arrived

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// sum over the block (blockDim.x a multiple of 32, <= 1024); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }

// layer norm with weight and bias of one fp32 row (two passes: mean, then the mean of squared deviations) -> T
template <typename T>
__device__ __forceinline__ void block_layernorm(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                                T* __restrict__ out, int W, float eps, float* red) {
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += x[i];
  const float mean = block_sum(s, red) / (float)W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) { const float d = x[i] - mean; q += d * d; }
  const float rstd = 1.f / sqrtf(block_sum(q, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[i] = from_f<T>((x[i] - mean) * rstd * w[i] + b[i]);
}

// x = table[token] * scale -> the layer-input stream and slot 0 of the per-layer result stack
template <typename T>
__global__ void __launch_bounds__(256) embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, int vocab, int W, float scale,
                                                    float* __restrict__ xin, float* __restrict__ x0, int* __restrict__ err) {
  const int t = blockIdx.x;
  int id = tokens[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, ERR_TOKEN);
    id = 0;
  }
  const T* row = table + (long long)id * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = to_f(row[i]) * scale;
    xin[(long long)t * W + i] = v;
    x0[(long long)t * W + i] = v;
  }
}

// h[row] = layernorm(x[rows ? rows[row] : row])
template <typename T>
__global__ void __launch_bounds__(256) layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                                        const float* __restrict__ b, T* __restrict__ out, int W, float eps) {
  __shared__ float red[32];
  const int src = rows ? rows[blockIdx.x] : blockIdx.x;
  block_layernorm<T>(x + (long long)src * W, w, b, out + (long long)blockIdx.x * W, W, eps, red);
}

// End of a parallel block with gated residuals and a depth-weighted average, one CTA per token:
//   X_new = x + mult * (mix * sigmoid(g1 + b1) + ff * sigmoid(g2 + b2));  stack[li + 1] = X_new
//   x    <- sum_{j <= li + 1} avg[j] * stack[j]            (what the next layer, or the output norm, reads)
//   h    <- layernorm(x) with the NEXT layer's norm (when given)
template <typename T>
__global__ void __launch_bounds__(256) block_end_kernel(float* __restrict__ xin, const T* __restrict__ mix, const T* __restrict__ ff,
                                                        const T* __restrict__ proj, long long ldp, int off_g1, int off_g2,
                                                        const float* __restrict__ b1, const float* __restrict__ b2, float mult,
                                                        float* __restrict__ stack, long long stack_stride, int li,
                                                        const float* __restrict__ avg, float* __restrict__ trace,
                                                        const float* __restrict__ nw, const float* __restrict__ nb, T* __restrict__ h,
                                                        int W, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  float* x = xin + t * W;
  const T* pr = proj + t * ldp;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = to_f(mix[t * W + i]) * sigmoidf(to_f(pr[off_g1 + i]) + b1[i]);
    if (ff) v += to_f(ff[t * W + i]) * sigmoidf(to_f(pr[off_g2 + i]) + b2[i]);
    const float xn = x[i] + mult * v;
    stack[(long long)(li + 1) * stack_stride + t * W + i] = xn;
    float acc = 0.f;
    for (int j = 0; j <= li; ++j) acc += avg[j] * stack[(long long)j * stack_stride + t * W + i];
    acc += avg[li + 1] * xn;
    x[i] = acc;
    if (trace) trace[t * W + i] = acc;
  }
  if (nw) {
    __syncthreads();
    block_layernorm<T>(x, nw, nb, h + t * W, W, eps, red);
  }
}

// latent of the new tokens: c = raw / sqrt(mean(raw^2) + eps) * w, appended to the slot's cache rows; one warp per token
template <typename T>
__global__ void __launch_bounds__(128) latent_append_kernel(const T* __restrict__ proj, long long ldp, int off, const float* __restrict__ w,
                                                            T* __restrict__ cache, int cap, int r, const int* __restrict__ tok_slot,
                                                            const int* __restrict__ tok_pos, int n_tok, float eps) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), l = threadIdx.x & 31;
  if (t >= n_tok) return;
  const T* raw = proj + (long long)t * ldp + off;
  float s = 0.f;
  for (int i = l; i < r; i += 32) { const float v = to_f(raw[i]); s += v * v; }
  const float rs = 1.f / sqrtf(warp_sum(s) / (float)r + eps);
  T* dst = cache + ((long long)tok_slot[t] * cap + tok_pos[t]) * r;
  for (int i = l; i < r; i += 32) dst[i] = from_f<T>(to_f(raw[i]) * rs * w[i]);
}

// out = relu(x)^2
template <typename T>
__global__ void __launch_bounds__(256) relu2_kernel(const T* __restrict__ proj, long long ldp, int off, T* __restrict__ out, int F, long long n) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const long long t = i / F; const int f = (int)(i - t * F);
  const float v = fmaxf(to_f(proj[t * ldp + off + f]), 0.f);
  out[i] = from_f<T>(v * v);
}

// C[z][M][N] = alpha * A[z][M][K] . B[z][N][K]^T on the CUDA cores (fp32 FMA; inputs converted on load): the all-fp32 mode's
// linear, the per-head products around the latent attention, and the bf16 mode's linear for shapes the tcgen05 GEMM does not take.
// A row's sum runs over k in order whatever M is: a token's result does not depend on what else is in the step.
// accumulate: C += instead of C =.
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256) gemm_nt_kernel(const TA* __restrict__ A, long long lda, long long sa, const TB* __restrict__ B,
                                                      long long ldb, long long sb, TC* __restrict__ C, long long ldc, long long sc,
                                                      int M, int N, int K, float alpha, int accumulate = 0, int zdiv = 0,
                                                      long long sa2 = 0, long long sb2 = 0, long long sc2 = 0) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 1], Bs[BK][BN + 1];
  {   // batch index z, or (z / zdiv, z % zdiv) with strides of their own for the outer index (zdiv > 0)
    const long long z1 = zdiv > 0 ? blockIdx.z % zdiv : blockIdx.z, z2 = zdiv > 0 ? blockIdx.z / zdiv : 0;
    A += z1 * sa + z2 * sa2; B += z1 * sb + z2 * sb2; C += z1 * sc + z2 * sc2;
  }
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int rr = ty + 16 * i, kk = k0 + tx;
      As[tx][rr] = (m0 + rr < M && kk < K) ? to_f(A[(long long)(m0 + rr) * lda + kk]) : 0.f;
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
      const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (m < M && n < N) C[(long long)m * ldc + n] = from_f<TC>(alpha * acc[i][j] + (accumulate ? to_f(C[(long long)m * ldc + n]) : 0.f));
    }
}

// [H*d][r] -> [H][r][d] (per-head transpose, done once at load: the query-side fold of W_uk wants it k-major)
template <typename T>
__global__ void head_transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int H, int d, int r) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= (long long)H * d * r) return;
  const int c = (int)(i % r); const long long hd = i / r; const int dd = (int)(hd % d); const int hh = (int)(hd / d);
  out[((long long)hh * r + c) * d + dd] = in[i];
}

template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i < n) out[i] = from_f<TO>(to_f(in[i]));
}

// ---------------------------------------------------------------------------------------------------------------------------
// Latent attention.  Rows are (token, head) pairs, head fastest; a tile is up to 4 * RPW consecutive rows of ONE cache slot.
// qa[row][r] is the query folded through W_uk and the score scale, so that score(row, j) = qa[row] . c[j] against the cached
// latents themselves and the value side is out[row] = sum_j p_j c[j] (W_uv is applied afterwards).  Causal: key j <= the
// row's position.  The softmax denominator holds one extra term exp(sink[head]) that has no value.
//   lane l owns latent elements l, l + 32, ...; a 32-key tile is staged in shared memory and shared by the CTA's 4 warps;
//   per row and key tile: 32 partial dots are transposed-reduced (8 keys at a time) so that lane L ends with the score of
//   key (L & 3) * 8 + (L >> 2); then one online-softmax update and the weighted sum.
//   nsplit > 1: CTA (tile, s) covers a contiguous share of the key tiles and leaves (m, l, unnormalised sum) for the merge.
// ---------------------------------------------------------------------------------------------------------------------------
struct AttnParams {
  const float* qa;          // [rows][r]
  const void* cache;        // T [slots][cap][r]
  const float* sink;        // [H]
  const int* tile_row0;     // first row of the tile
  const int* tile_rows;     // rows in the tile
  const int* tile_slot;
  const int* tok_pos;       // position of every token of the step in its slot
  float* out;               // [rows][r]
  float* part;              // nsplit > 1: [tile][split][rows_per_tile][r + 2]
  int cap, r, H, nsplit;
  int* err = nullptr;       // device error flags (may be null)
  // sink = null: an ordinary softmax.  window > 0: the row at position p sees keys j with 0 <= p - j < window.  gate != null:
  // row (token, head) is multiplied by sigmoid(gate[token * ldg + head]).
  int window = 0;
  const float* gate = nullptr;
  int ldg = 0;
};

template <typename T, int NCH, int RPW>
__global__ void __launch_bounds__(128) latent_attn_kernel(AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* cs = reinterpret_cast<T*>(smem_raw);            // [32][r]
  constexpr int KT = 32;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = p.r, H = p.H;
  const int row0 = p.tile_row0[tile], nrows = p.tile_rows[tile];
  const T* cbase = static_cast<const T*>(p.cache) + (long long)p.tile_slot[tile] * p.cap * r;
  const int kmax = p.tok_pos[(row0 + nrows - 1) / H];          // rows are ordered by token: the last row sees the most keys
  const int kt_lo = p.window > 0 ? max(0, p.tok_pos[row0 / H] - p.window + 1) / KT : 0;      // the first row's window starts lowest
  const int n_kt = kmax / KT + 1 - kt_lo;
  const int per = (n_kt + p.nsplit - 1) / p.nsplit;
  const int kt0 = kt_lo + split * per, kt1 = min(kt_lo + n_kt, kt0 + per);

  float q[RPW][NCH], o[RPW][NCH], m[RPW], lsum[RPW];
  int pos[RPW];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int lr = warp * RPW + i;
    const bool valid = lr < nrows;
    const int g = row0 + (valid ? lr : 0);
    pos[i] = valid ? p.tok_pos[g / H] : -1;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int e = lane + 32 * c;
      q[i][c] = (valid && e < r) ? p.qa[(long long)g * r + e] : 0.f;
      o[i][c] = 0.f;
    }
    // the sink enters once: the first split starts from (m = sink, l = 1); the others from nothing
    if (split == 0 && valid && p.sink) { m[i] = p.sink[g % H]; lsum[i] = lane == 0 ? 1.f : 0.f; }
    else { m[i] = -INFINITY; lsum[i] = 0.f; }
  }

  for (int kt = kt0; kt < kt1; ++kt) {
    const int j0 = kt * KT;
    const int nk = min(KT, kmax + 1 - j0);
    __syncthreads();
    {   // stage keys j0 .. j0 + nk - 1: one contiguous span of the slot's cache
      const T* src = cbase + (long long)j0 * r;
      const int n = nk * r;
      if (((r * (int)sizeof(T)) & 15) == 0) {
        const int n16 = n * (int)sizeof(T) / 16;
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(cs);
        for (int i = threadIdx.x; i < n16; i += 128) d4[i] = s4[i];
      } else {
        for (int i = threadIdx.x; i < n; i += 128) cs[i] = src[i];
      }
    }
    __syncthreads();
    float sc[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) sc[i] = 0.f;
#pragma unroll
    for (int g8 = 0; g8 < 4; ++g8) {
      if (g8 * 8 >= nk) break;                                   // uniform over the CTA
      float part[RPW][8];
#pragma unroll
      for (int i = 0; i < RPW; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) part[i][k] = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int e = lane + 32 * c;
        if (e < r) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int kk = g8 * 8 + k;
            const float cv = kk < nk ? to_f(cs[kk * r + e]) : 0.f;
#pragma unroll
            for (int i = 0; i < RPW; ++i) part[i][k] = fmaf(q[i][c], cv, part[i][k]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        float v4[4], v2[2];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float send = (lane & 16) ? part[i][k] : part[i][k + 4];
          const float keep = (lane & 16) ? part[i][k + 4] : part[i][k];
          v4[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float send = (lane & 8) ? v4[k] : v4[k + 2];
          const float keep = (lane & 8) ? v4[k + 2] : v4[k];
          v2[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
        const float send = (lane & 4) ? v2[0] : v2[1];
        const float keep = (lane & 4) ? v2[1] : v2[0];
        float v1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
        // every lane now holds the score of key g8 * 8 + (lane >> 2); lanes with (lane & 3) == g8 keep it
        if ((lane & 3) == g8) sc[i] = v1;
      }
    }
    const int mykey = j0 + (lane & 3) * 8 + (lane >> 2);
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      const bool seen = mykey <= pos[i] && mykey <= kmax && (p.window <= 0 || pos[i] - mykey < p.window);
      const float s = seen ? sc[i] : -INFINITY;
      const float mn = fmaxf(m[i], warp_max(s));
      float pj = 0.f;
      if (mn > -INFINITY) {                                       // uniform over the warp
        const float corr = expf(m[i] - mn);                       // m = -inf -> 0
        pj = seen ? expf(s - mn) : 0.f;
        lsum[i] = lsum[i] * corr + pj;
#pragma unroll
        for (int c = 0; c < NCH; ++c) o[i][c] *= corr;
        m[i] = mn;
      }
      sc[i] = pj;
    }
    for (int k = 0; k < nk; ++k) {
      const int srcl = ((k & 7) << 2) | (k >> 3);
      float pk[RPW];
      bool any = false;
#pragma unroll
      for (int i = 0; i < RPW; ++i) { pk[i] = __shfl_sync(0xffffffffu, sc[i], srcl); any |= pk[i] != 0.f; }
      if (!any) continue;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int e = lane + 32 * c;
        if (e < r) {
          const float cv = to_f(cs[k * r + e]);
#pragma unroll
          for (int i = 0; i < RPW; ++i) o[i][c] = fmaf(pk[i], cv, o[i][c]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int lr = warp * RPW + i;
    if (lr >= nrows) continue;
    const float l = warp_sum(lsum[i]);
    if (p.nsplit == 1) {
      const float inv = (p.gate ? sigmoidf(p.gate[(long long)((row0 + lr) / H) * p.ldg + (row0 + lr) % H]) : 1.f) / l;
      float* dst = p.out + (long long)(row0 + lr) * r;
#pragma unroll
      for (int c = 0; c < NCH; ++c) { const int e = lane + 32 * c; if (e < r) dst[e] = o[i][c] * inv; }
    } else {
      float* dst = p.part + (((long long)tile * p.nsplit + split) * (4 * RPW) + lr) * (r + 2);
#pragma unroll
      for (int c = 0; c < NCH; ++c) { const int e = lane + 32 * c; if (e < r) dst[e] = o[i][c]; }
      if (lane == 0) { dst[r] = m[i]; dst[r + 1] = l; }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores, for bf16 latents whose size is a multiple of 64 (<= 512): both products of a 16-row
// tile against a 32-key tile run as mma.sync m16n8k16 (bf16 in, fp32 accumulate).  The CTA's four warps cut the LATENT axis:
// warp w owns elements [w * r/4, (w + 1) * r/4) of every latent, for the scores (a partial dot over its share, summed over
// the warps through shared memory) as well as for the weighted sum (its share of the output columns), so that the query
// fragments and the output accumulators stay in registers and every warp reads only its own columns of the key tile.
// The softmax (fp32, with the sink) is done by every warp on the summed scores; the weights enter the second product as bf16.
// Key tiles are double-buffered with cp.async; rows of the tile beyond the last key are zero-filled.
// ---------------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem_row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Waits for a phase of an mbarrier, at most about two seconds (wall clock, sampled every 1024 polls); false when it gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  uint32_t done, spins = 0;
  uint64_t t0 = 0;
  for (;;) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((++spins & 1023u) == 0u) {
      const uint64_t now = tcp::global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) return false;
    }
  }
}

template <int NKS>      // 16-element steps of a warp's share of the latent: r = 64 * NKS
__global__ void __launch_bounds__(128, 3) latent_attn_mma_kernel(AttnParams p) {
  // r = 512: 75 KB per CTA, three CTAs per SM.  Keys arrive by bulk copies (one per key, issued by the lanes of warp 0) that
  // complete on an mbarrier per buffer, so no thread spends instructions on staging.  A row of partial scores is 32 floats; its 8-float blocks are permuted by the
  // row (block ^ (row & 3)) so that neither the stores nor the loads meet in a bank.
  constexpr int KT = 32, R = 64 * NKS, SL = 16 * NKS, STRIDE = R + 8, SPS = 32, PST = 40;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* cs = reinterpret_cast<bf16*>(smem_raw);                                     // [2][KT][STRIDE] keys
  float* sp = reinterpret_cast<float*>(smem_raw + (size_t)2 * KT * STRIDE * 2);     // [4 warps][16][SPS] partial scores
  bf16* pb = reinterpret_cast<bf16*>(sp + 4 * 16 * SPS);                            // [16][PST] softmax weights of the tile
  float* stat = reinterpret_cast<float*>(pb + 16 * PST);                            // [3][16]: rescale factor, maximum, sum
  const uint32_t bars = tcp::smem_u32(stat + 48);                                   // [2] mbarriers: keys of a buffer have landed
  const int tile = blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int H = p.H;
  const int row0 = p.tile_row0[tile], nrows = p.tile_rows[tile];
  const bf16* cbase = static_cast<const bf16*>(p.cache) + (long long)p.tile_slot[tile] * p.cap * R;
  const int kmax = p.tok_pos[(row0 + nrows - 1) / H];
  const int kt_lo = p.window > 0 ? max(0, p.tok_pos[row0 / H] - p.window + 1) / KT : 0;      // the first row's window starts lowest
  const int n_kt = kmax / KT + 1;
  const int per = (n_kt - kt_lo + p.nsplit - 1) / p.nsplit;
  const int kt0 = kt_lo + split * per, kt1 = min(n_kt, kt0 + per);
  const int col0 = warp * SL;

  // query fragments of rows g and g + 8, this warp's share of the latent
  unsigned qf[NKS][4];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int lr = g + 8 * hf;
    const bool valid = lr < nrows;
    const float* qrow = p.qa + (long long)(row0 + (valid ? lr : 0)) * R + col0;
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks) {
      const float2 a = valid ? *reinterpret_cast<const float2*>(qrow + ks * 16 + 2 * t4) : make_float2(0.f, 0.f);
      const float2 b = valid ? *reinterpret_cast<const float2*>(qrow + ks * 16 + 2 * t4 + 8) : make_float2(0.f, 0.f);
      qf[ks][hf] = pack_bf16(a.x, a.y);
      qf[ks][2 + hf] = pack_bf16(b.x, b.y);
    }
  }
  // softmax state of one row: warp w owns rows 4w .. 4w + 3, eight lanes per row, lane kq of them keys 4 kq .. 4 kq + 3 of a tile
  const int orow = 4 * warp + (lane >> 3), kq = lane & 7;
  int opos; float om, ol;
  {
    const bool valid = orow < nrows;
    const int gr = row0 + (valid ? orow : 0);
    opos = valid ? p.tok_pos[gr / H] : -1;
    if (valid && split == 0 && p.sink) { om = p.sink[gr % H]; ol = 1.f; }      // the sink: weight exp(sink) in the denominator, no value
    else { om = valid ? -INFINITY : 0.f; ol = 0.f; }
  }
  float oacc[2 * NKS][4];
#pragma unroll
  for (int i = 0; i < 2 * NKS; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }

  // Keys past the request's last one are masked, but their (zero) weights still multiply what the buffer holds: make it finite.
  if (kt1 == n_kt && kt0 < kt1) {
    const int nk = kmax + 1 - (n_kt - 1) * KT;
    bf16* dst = cs + (size_t)((n_kt - 1 - kt0) & 1) * KT * STRIDE + nk * STRIDE;
    for (int c = threadIdx.x; c < (KT - nk) * STRIDE / 8; c += 128) reinterpret_cast<uint4*>(dst)[c] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (threadIdx.x == 0) {
    tcp::mbar_init(bars, 1);
    tcp::mbar_init(bars + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  auto issue = [&](int kt, int buf) {                       // warp 0: lane j copies key j of the tile
    const int j0 = kt * KT, nk = min(KT, kmax + 1 - j0);
    const uint32_t bar = bars + 8 * buf;
    if (lane == 0) tcp::mbar_expect_tx(bar, (uint32_t)nk * R * 2);
    __syncwarp();
    if (lane < nk) tcp::bulk_load(tcp::smem_u32(cs + ((size_t)buf * KT + lane) * STRIDE), cbase + (long long)(j0 + lane) * R, R * 2, bar);
  };

  if (warp == 0 && kt0 < kt1) issue(kt0, 0);
  bool arrived = true;
  for (int kt = kt0; kt < kt1; ++kt) {
    const int buf = (kt - kt0) & 1;
    if (arrived) arrived = mbar_wait_bounded(bars + 8 * buf, ((kt - kt0) >> 1) & 1);
    const bf16* ct = cs + (size_t)buf * KT * STRIDE;
    // partial scores of this warp's share of the latent: [16 rows][32 keys]
    float sacc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks) {
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        unsigned b[4];
        const int mi = lane >> 3;
        ldmatrix_x4(b, ct + (np * 16 + (mi >> 1) * 8 + (lane & 7)) * STRIDE + col0 + ks * 16 + (mi & 1) * 8);
        mma_bf16_16816(sacc[2 * np], qf[ks], b[0], b[1]);
        mma_bf16_16816(sacc[2 * np + 1], qf[ks], b[2], b[3]);
      }
    }
    float* mine = sp + warp * 16 * SPS;
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
      const int col = ((nb ^ (g & 3)) << 3) + 2 * t4;
      *reinterpret_cast<float2*>(mine + g * SPS + col) = make_float2(sacc[nb][0], sacc[nb][1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * SPS + col) = make_float2(sacc[nb][2], sacc[nb][3]);
    }
    __syncthreads();
    if (warp == 0 && kt + 1 < kt1) issue(kt + 1, buf ^ 1);      // every warp is done with the other buffer (tile kt - 1)
    // softmax update of the owned row on the summed scores, once per row; the weights go back as bf16
    {
      const int pc = (((kq >> 1) ^ (orow & 3)) << 3) + (kq & 1) * 4;
      float4 a = *reinterpret_cast<const float4*>(sp + orow * SPS + pc);
#pragma unroll
      for (int w = 1; w < 4; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(sp + (w * 16 + orow) * SPS + pc);
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
      }
      const int key = kt * KT + 4 * kq;                    // the mask also hides the zero-filled keys past the last one
      const int klow = p.window > 0 ? opos - p.window + 1 : 0;      // the window's lower end
      float s0 = key <= opos && key >= klow ? a.x : -INFINITY, s1 = key + 1 <= opos && key + 1 >= klow ? a.y : -INFINITY;
      float s2 = key + 2 <= opos && key + 2 >= klow ? a.z : -INFINITY, s3 = key + 3 <= opos && key + 3 >= klow ? a.w : -INFINITY;
      float mx = fmaxf(fmaxf(s0, s1), fmaxf(s2, s3));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float mn = fmaxf(om, mx);
      const float mu = mn == -INFINITY ? 0.f : mn;
      const float corr = __expf(om - mu);                  // om = -inf -> 0 (nothing accumulated yet)
      s0 = __expf(s0 - mu); s1 = __expf(s1 - mu); s2 = __expf(s2 - mu); s3 = __expf(s3 - mu);
      float sum = (s0 + s1) + (s2 + s3);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      ol = ol * corr + sum;
      om = mn;
      *reinterpret_cast<uint2*>(pb + orow * PST + 4 * kq) = make_uint2(pack_bf16(s0, s1), pack_bf16(s2, s3));
      if (kq == 0) stat[orow] = corr;
    }
    __syncthreads();
    const float corr0 = stat[g], corr1 = stat[g + 8];
    if (__any_sync(0xffffffffu, corr0 != 1.f || corr1 != 1.f)) {      // a running maximum moved somewhere in the warp
#pragma unroll
      for (int i = 0; i < 2 * NKS; ++i) { oacc[i][0] *= corr0; oacc[i][1] *= corr0; oacc[i][2] *= corr1; oacc[i][3] *= corr1; }
    }
    // weighted sum over this warp's output columns; A fragments of the weights: k-step 0 = keys 0..15, k-step 1 = keys 16..31
#pragma unroll
    for (int k2 = 0; k2 < 2; ++k2) {
      unsigned pf[4];
      ldmatrix_x4(pf, pb + ((lane & 7) + 8 * ((lane >> 3) & 1)) * PST + 16 * k2 + 8 * (lane >> 4));
#pragma unroll
      for (int np = 0; np < NKS; ++np) {
        unsigned b[4];
        const int mi = lane >> 3;
        ldmatrix_x4_trans(b, ct + (k2 * 16 + (mi & 1) * 8 + (lane & 7)) * STRIDE + col0 + np * 16 + (mi >> 1) * 8);
        mma_bf16_16816(oacc[2 * np], pf, b[0], b[1]);
        mma_bf16_16816(oacc[2 * np + 1], pf, b[2], b[3]);
      }
    }
  }

  if (!arrived && p.err != nullptr) atomicOr(p.err, ERR_WAIT);
  if (kq == 0) { stat[16 + orow] = om; stat[32 + orow] = ol; }
  __syncthreads();
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int lr = g + 8 * hf;
    if (lr >= nrows) continue;
    const float mt = stat[16 + lr], lt = stat[32 + lr];
    if (p.nsplit == 1) {
      const float inv = (p.gate ? sigmoidf(p.gate[(long long)((row0 + lr) / H) * p.ldg + (row0 + lr) % H]) : 1.f) / lt;
      float* dst = p.out + (long long)(row0 + lr) * R + col0;
#pragma unroll
      for (int nb = 0; nb < 2 * NKS; ++nb)
        *reinterpret_cast<float2*>(dst + nb * 8 + 2 * t4) = make_float2(oacc[nb][2 * hf] * inv, oacc[nb][2 * hf + 1] * inv);
    } else {
      float* dst = p.part + (((long long)tile * p.nsplit + split) * 16 + lr) * (R + 2);
#pragma unroll
      for (int nb = 0; nb < 2 * NKS; ++nb)
        *reinterpret_cast<float2*>(dst + col0 + nb * 8 + 2 * t4) = make_float2(oacc[nb][2 * hf], oacc[nb][2 * hf + 1]);
      if (warp == 0 && t4 == 0) { dst[R] = mt; dst[R + 1] = lt; }
    }
  }
}

// merges the splits of one row: out = sum_s o_s exp(m_s - M) / sum_s l_s exp(m_s - M); one CTA per row, grid (tiles, rows).
// Every warp computes the split weights (lane s owns splits s and s + 32); then a thread owns element pairs of the row and
// sums them over the splits with independent 8-byte loads (scalar loads when the latent size is odd).
__global__ void __launch_bounds__(128) latent_attn_merge_kernel(const float* __restrict__ part, const int* __restrict__ tile_row0,
                                                                const int* __restrict__ tile_rows, float* __restrict__ out, int r,
                                                                int nsplit, int rows_per_tile, const float* __restrict__ gate = nullptr,
                                                                int ldg = 0, int H = 1) {      // gate: row (token, head) times sigmoid(gate[token * ldg + head])
  __shared__ float wsm[64];
  const int tile = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int lr = blockIdx.y;
  if (lr >= tile_rows[tile]) return;
  const float* base = part + ((long long)tile * nsplit * rows_per_tile + lr) * (r + 2);
  const long long ss = (long long)rows_per_tile * (r + 2);
  float ms[2], ls[2], w[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int s = lane + 32 * i;
    ms[i] = s < nsplit ? base[s * ss + r] : -INFINITY;
    ls[i] = s < nsplit ? base[s * ss + r + 1] : 0.f;
  }
  const float M = warp_max(fmaxf(ms[0], ms[1]));
  float L = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    w[i] = ms[i] > -INFINITY ? expf(ms[i] - M) : 0.f;
    L += ls[i] * w[i];
  }
  float inv = 1.f / warp_sum(L);
  if (gate) { const int row = tile_row0[tile] + lr; inv *= sigmoidf(gate[(long long)(row / H) * ldg + row % H]); }
  if (warp == 0) { wsm[lane] = w[0]; wsm[lane + 32] = w[1]; }
  __syncthreads();
  float* dst = out + (long long)(tile_row0[tile] + lr) * r;
  if ((r & 1) == 0) {       // rows of r + 2 floats start on 8-byte boundaries
    for (int e = threadIdx.x * 2; e < r; e += 256) {
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll 8
      for (int s = 0; s < nsplit; ++s) {
        const float2 v = *reinterpret_cast<const float2*>(base + s * ss + e);
        acc.x = fmaf(v.x, wsm[s], acc.x); acc.y = fmaf(v.y, wsm[s], acc.y);
      }
      *reinterpret_cast<float2*>(dst + e) = make_float2(acc.x * inv, acc.y * inv);
    }
  } else {
    for (int e = threadIdx.x; e < r; e += 128) {
      float acc = 0.f;
#pragma unroll 8
      for (int s = 0; s < nsplit; ++s) acc = fmaf(base[s * ss + e], wsm[s], acc);
      dst[e] = acc * inv;
    }
  }
}

// C[z][M][N] = alpha * A[z][M][K] . B[z][N][K]^T on the tensor cores (mma.sync m16n8k16, bf16 in, fp32 accumulate) for the
// per-head products around the latent attention in bfloat16: A is bf16 or fp32 (rounded to bf16 on its way into shared
// memory), B bf16, C fp32 or bf16.  K a multiple of 16; M and N are free (zero-filled edges).  CTA tile 64 x 64, 4 warps of
// 16 rows x 64 columns, 32-element k-steps through shared memory.
template <typename TA, typename TC>
__global__ void __launch_bounds__(128) gemm_nt_mma_kernel(const TA* __restrict__ A, long long lda, long long sa, const bf16* __restrict__ B,
                                                          long long ldb, long long sb, TC* __restrict__ C, long long ldc, long long sc,
                                                          int M, int N, int K, float alpha) {
  constexpr int BM = 64, BN = 64, BK = 32, ST = BK + 8;
  __shared__ __align__(16) bf16 As[BM][ST];
  __shared__ __align__(16) bf16 Bs[BN][ST];
  A += (long long)blockIdx.z * sa; B += (long long)blockIdx.z * sb; C += (long long)blockIdx.z * sc;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  // 64 rows x 32 k of each operand per step, fetched with 16-byte loads into registers one step ahead (the launcher checks
  // that K is a multiple of 16 and that rows start on 16-byte boundaries, so a chunk lies inside K or outside it as a whole)
  constexpr int ACH = sizeof(TA) == 2 ? 2 : 4;        // chunks of A per thread: 8 bf16 or 4 floats each
  uint4 ra[ACH], rb[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int j = 0; j < ACH; ++j) {
      const int c = threadIdx.x + 128 * j;
      const int per_row = sizeof(TA) == 2 ? 4 : 8, el = sizeof(TA) == 2 ? 8 : 4;
      const int rr = c / per_row, kk = (c % per_row) * el;
      ra[j] = (m0 + rr < M && k0 + kk < K) ? *reinterpret_cast<const uint4*>(A + (long long)(m0 + rr) * lda + k0 + kk) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c = threadIdx.x + 128 * j;
      const int rr = c / 4, kk = (c % 4) * 8;
      rb[j] = (n0 + rr < N && k0 + kk < K) ? *reinterpret_cast<const uint4*>(B + (long long)(n0 + rr) * ldb + k0 + kk) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < ACH; ++j) {
      const int c = threadIdx.x + 128 * j;
      if constexpr (sizeof(TA) == 2) {
        *reinterpret_cast<uint4*>(&As[c / 4][(c % 4) * 8]) = ra[j];
      } else {
        const float4 f = *reinterpret_cast<const float4*>(&ra[j]);
        *reinterpret_cast<uint2*>(&As[c / 8][(c % 8) * 4]) = make_uint2(pack_bf16(f.x, f.y), pack_bf16(f.z, f.w));
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c = threadIdx.x + 128 * j;
      *reinterpret_cast<uint4*>(&Bs[c / 4][(c % 4) * 8]) = rb[j];
    }
    __syncthreads();
    if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      unsigned a[4];
      const int mi = lane >> 3;
      ldmatrix_x4(a, &As[warp * 16 + (mi & 1) * 8 + (lane & 7)][ks * 16 + (mi >> 1) * 8]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        unsigned b[4];
        ldmatrix_x4(b, &Bs[np * 16 + (mi >> 1) * 8 + (lane & 7)][ks * 16 + (mi & 1) * 8]);
        mma_bf16_16816(acc[2 * np], a, b[0], b[1]);
        mma_bf16_16816(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int nb = 0; nb < 8; ++nb)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int m = m0 + warp * 16 + g + 8 * hf, n = n0 + nb * 8 + 2 * t4;
      if (m < M) {
        if (n < N) C[(long long)m * ldc + n] = from_f<TC>(alpha * acc[nb][2 * hf]);
        if (n + 1 < N) C[(long long)m * ldc + n + 1] = from_f<TC>(alpha * acc[nb][2 * hf + 1]);
      }
    }
}

// bf16 rows with a padded stride -> fp32 [rows][V]
__global__ void rows_to_f32_kernel(const bf16* __restrict__ in, long long ld, float* __restrict__ out, int V, long long n) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const long long row = i / V;
  out[i] = __bfloat162float(in[row * ld + (i - row * V)]);
}

// greedy choice on the fp32 logits themselves: first maximum of every row; one CTA per row
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ logits, int V, long long* __restrict__ out) {
  __shared__ float bv[8];
  __shared__ int bi[8];
  const float* row = logits + (long long)blockIdx.x * V;
  float best = -INFINITY; int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += 256) { const float v = row[i]; if (v > best || (v == best && i < idx)) { best = v; idx = i; } }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
    out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}

// logits f32 -> bf16 rows for the LM's sampler
__global__ void logits_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, long long n) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}

}  // namespace dlm
}  // namespace b200
