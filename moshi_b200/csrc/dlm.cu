// Decoder-LM handle: a language model given as a list of layers (mixer + feed-forward per layer), its weights under the
// checkpoint's names, a slot cache per layer (latents, or keys and values, plus the carried inputs of convolutions and the
// state of recurrent mixers), and the ragged step (any number of new tokens per slot) that both prompt portions and
// single-token decoding go through.  Two block arrangements are registered: gated parallel sublayers with a depth-weighted
// average (the Likosun design), RMS-norm sandwiches around mixer and feed-forward in turn (the Govuvik design), and a plain
// parallel block on one zero-centred RMS norm (the Namalix design).
#include <algorithm>

#include <cmath>

#include "dlm_kernels.cuh"
#include "dlm_mixers.cuh"
#include "dlm_mixers2.cuh"
#include "dlm_mixers3.cuh"
#include "gemm_sk.cuh"
#include "lm_kernels.cuh"

using namespace b200;
using namespace b200::dlm;

namespace {

// a linear's weight: row-major [N][K] of the compute type, or (bf16, eligible shape) the packed tiles of the tcgen05 GEMM
struct Weight {
  void* rm = nullptr;
  void* tiles = nullptr;
  int N = 0, K = 0;
};

struct Layer {
  b200_dlm_layer c;
  int ncat = 0, ldp = 0, off_q = 0, off_dkv = 0, off_up = 0, off_g1 = 0, off_g2 = 0;
  Weight cat, o, down;                 // [q | dkv | up | gate1 | gate2] x width;  width x (heads * vdim);  width x ff
  void *ukT = nullptr, *uv = nullptr;  // [H][r][dim] (transposed per head), [H * vdim][r]
  float *n1w = nullptr, *n1b = nullptr, *cnorm = nullptr, *sink = nullptr, *b1 = nullptr, *b2 = nullptr, *avg = nullptr;
  void* cache = nullptr;               // [slots][cap][r]
  int sig = 0;                         // index of the layer's attention tile list
  // ---- sandwich block (norms around every sublayer); a = the only mixer or the left one, b = the right one of a parallel pair
  float *n2w = nullptr, *n1bw = nullptr, *n2bw = nullptr, *canon = nullptr, *canon_hist = nullptr;
  // window attention (a)
  int a_q = 0, a_k = 0, a_v = 0, a_g = 0;         // offsets into the concatenated projection
  int Nq = 0, Nk = 0, Nv = 0, QT = 0, KT = 0, kstride = 0; size_t attn_smem = 0;
  int sig_mma = -1, mma_items = 0; size_t mma_smem = 0;
  int sig_one = -1, KT_one = 0, kstride_one = 0; size_t smem_one = 0;      // single-token requests: tiles of one token, less shared memory, more CTAs per SM      // tensor-core window attention: tile list of 16 tokens, items per warp
  float *qnorm = nullptr, *knorm = nullptr, *qkv_conv = nullptr, *qkv_hist = nullptr, *mixhh = nullptr; double* freq = nullptr;
  void *kcache = nullptr, *vcache = nullptr;
  Weight a_o;
  float *a_out = nullptr, *b_out = nullptr;       // norms of the two outputs of a parallel pair
  // recurrent mixers: GLA (b of a parallel pair) and mLSTM (a)
  int r_q = 0, r_k = 0, r_v = 0, r_g = 0, r_a1 = 0, decay_rank = 0;
  void *a2 = nullptr, *w_if = nullptr;            // T [heads * dim][decay_rank];  T [2 * heads][width]
  float *a2b = nullptr, *if_b = nullptr, *rnorm = nullptr;
  float *St = nullptr, *nvec = nullptr, *mval = nullptr;
  Weight r_o;
  // routed experts
  void *router = nullptr, *ups = nullptr, *downs = nullptr;      // T [E][width]; T [E][ff][width]; T [E][width][ff]
  // ---- parallel-residual block: one mixer (a) beside the feed-forward, both on the same norm.  The concatenated projection is
  // [q | k | v | (g) | (ff gate | ff up)]; what must be fp32 before an activation (the attention's head gates, the delta rule's
  // beta and step size, router logits) comes from one small projection w_small, T [nsmall][width]
  int p_q = 0, p_k = 0, p_v = 0, p_g = 0, p_ffg = 0, p_ffu = 0;
  int s_gate = 0, s_ba = 0, s_router = 0, nsmall = 0;
  void* w_small = nullptr;
  float *pbias = nullptr, *vlambda = nullptr, *head_decay = nullptr, *A_log = nullptr, *dt_bias = nullptr, *correction = nullptr;
  float rot_amp = 1.f;
  std::vector<float> decay;            // retention: the configuration's decays (copied at create)
  // ---- pre-norm streams block: mixer and feed-forward on norms of their own; per sublayer the read, write and mixing weights of
  // the residual streams.  Latent attention with a rotated part: cache rows of rp elements [latent | rotated key part | padding].
  // Parallel pair: window attention (a) beside a minGRU (b), projection [q | k | v | z | x | g].  Channel delta: [q | k | v | a1 | g1].
  float *hc_in[2] = {nullptr, nullptr}, *hc_out[2] = {nullptr, nullptr}, *hc_mix[2] = {nullptr, nullptr};
  Weight up;
  int rp = 0;
  int g_z = 0, g_x = 0, g_g = 0, c_a1 = 0, c_g1 = 0, gate_rank = 0;
  float *qkv_bias = nullptr, *zx_bias = nullptr, *gru = nullptr;      // gru: [slots][channels] state of the minGRU
  void* g2 = nullptr;                  // T [heads * vdim][gate_rank]
};

// attention tile list of one (heads, rows per tile) combination
struct TileSig {
  int H, rpt;
  int off_row0 = 0, off_rows = 0, off_slot = 0;     // offsets into the step's metadata block (ints)
  int count = 0;
};

}  // namespace

struct b200_dlm {
  b200_dlm_config cfg;
  std::vector<Layer> layers;
  TensorStore store;
  Arena weights, state;
  bool finalized = false, f32 = false;
  int device = -1;
  int use_tc = 1, trace_layers = 0, attn_split = 0, attn_tc = 1;
  // option "time_kernels": CUDA events around every operation of a step, summed per class (bench.py's per-kernel roofline)
  int time_kernels = 0;
  std::vector<cudaEvent_t> ev_pool; std::vector<int> ev_class; size_t ev_used = 0;
  double class_ms[6] = {0, 0, 0, 0, 0, 0};
  void *embed = nullptr;
  Weight head;
  float *fnw = nullptr, *fnb = nullptr;
  int64_t weight_bytes = 0;
  // cache and step buffers
  int slots = 0, cap = 0, tmax = 0, wmax = 0;
  std::vector<int> len;                // tokens held per slot
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_meta = nullptr;
  int *meta_dev = nullptr, *meta_pin = nullptr; int meta_ints = 0;
  int off_tok = 0, off_slot = 0, off_pos = 0, off_want = 0;
  std::vector<TileSig> sigs;
  float *xin = nullptr, *stack = nullptr, *trace = nullptr, *qa = nullptr, *ol = nullptr, *part = nullptr, *logits = nullptr;
  void *hbuf = nullptr, *proj = nullptr, *obuf = nullptr, *mixo = nullptr, *act = nullptr, *ffo = nullptr, *hf = nullptr;
  bf16 *logits_bf = nullptr, *head_bf = nullptr;
  size_t part_floats = 0;
  int last_tokens = 0, last_want = 0;
  int* err = nullptr;
  // sandwich block: step metadata per token (first / last token of its request in the step) and per entry, further buffers
  int off_first = 0, off_last = 0, off_ent_tok0 = 0, off_ent_ntok = 0, off_ent_slot = 0, off_ent_pos0 = 0, off_ent_par = 0, n_entries = 0, max_entry_tokens = 0;
  std::vector<char> par;               // per slot: which generation of mLSTM's n and m is current
  // recurrences: portions of at least 2 * scan_seg tokens run as segments of scan_seg tokens side by side (units = entries after the cut)
  int scan_seg = 256, n_units = 0, max_seg_units = 0, off_ent_seg = 0, off_ent_nseg = 0, off_ent_buf = 0;
  struct ScanUnit { int tok0, ntok, seg, buf; };
  std::vector<ScanUnit> units;
  float *segS = nullptr, *segB = nullptr, *segM = nullptr, *tokM = nullptr, *corr = nullptr;
  float *embw = nullptr, *h32 = nullptr, *qkv32 = nullptr, *scan32 = nullptr, *gate32 = nullptr, *attn32 = nullptr, *route32 = nullptr, *moe_w = nullptr, *scan_prep = nullptr, *scan_v = nullptr;
  void *mixo2 = nullptr, *obuf2 = nullptr, *yexp = nullptr;
  int *moe_idx = nullptr, *moe_rank = nullptr, *moe_perm = nullptr, *moe_row_tok = nullptr, *moe_tile_e = nullptr, *moe_tile_r0 = nullptr,
      *moe_tile_n = nullptr, *moe_ntiles = nullptr;
  float* sk_ws = nullptr; int* sk_counters = nullptr;
  tc::GemmPlanCache plans;
  // parallel-residual block: recurrences that cannot run as segments (the delta rule) take the step's entries whole
  int off_whole_tok0 = 0, off_whole_ntok = 0, off_whole_slot = 0, off_whole_pos0 = 0, off_zero = 0, off_one = 0;
  int off_chunk_tok0 = 0, off_chunk_nt = 0, off_whole_chunk0 = 0, n_chunks = 0, max_chunks = 0;      // the delta rule's chunks of a step
  int delta_chunk = 1;                 // option: portions of at least 16 tokens take the chunked delta rule
  float* gram = nullptr;               // [chunks][heads][2 DELTA_CH + 2 DELTA_CH^2]
  int vmix_first = -1;                 // the first attention layer that blends values: the later ones blend its values in
  float* small32 = nullptr;            // [tokens][nsmall] fp32 results of the small projection
  float* xs = nullptr;                 // pre-norm streams block: the residual streams [tokens][streams][width]
  float *rows3 = nullptr, *gend = nullptr;      // chunked delta rule with a decay per key channel: [tokens][heads][3 dim], [chunks][heads][dim]
  void *vfirst = nullptr, *act2 = nullptr;      // T [tokens][G * vdim] values of layer vmix_first; T [tokens * top][2 ff] experts' first product
};

namespace {

size_t esize(const b200_dlm* h) { return h->f32 ? 4 : 2; }
int rows_per_tile(int r) { return r <= 576 ? 16 : 8; }

template <typename TO>
int convert_into(const Tensor* t, TO* dst) {
  const long long n = t->numel();
  const unsigned g = (unsigned)ceil_div64(n, 256);
  if (t->dtype == B200_BF16) B200_LAUNCH(convert_kernel, g, 256, 0, nullptr, static_cast<const bf16*>(t->data), dst, n);
  else if (t->dtype == B200_F32) B200_LAUNCH(convert_kernel, g, 256, 0, nullptr, static_cast<const float*>(t->data), dst, n);
  else B200_FAIL(B200_ERR_SHAPE, "decoder LM: weights must be bfloat16 or float32");
  return check_launch("convert");
}

int find_tensor(b200_dlm* h, const std::string& name, std::vector<int64_t> shape, const Tensor** out) {
  const Tensor* t = h->store.find(name);
  if (!t) B200_FAIL(B200_ERR_MISSING, "decoder LM finalize: tensor '%s' was not loaded", name.c_str());
  if (t->shape != shape) {
    std::string got;
    for (auto s : t->shape) got += std::to_string(s) + ",";
    B200_FAIL(B200_ERR_SHAPE, "decoder LM tensor '%s' has shape [%s]", name.c_str(), got.c_str());
  }
  *out = t;
  return B200_OK;
}

// small vectors always live in fp32
int get_f32(b200_dlm* h, const std::string& name, int64_t n, float** out) {
  const Tensor* t = nullptr;
  B200_TRY(find_tensor(h, name, {n}, &t));
  B200_TRY(h->weights.alloc_t(out, (size_t)n, false));
  h->weight_bytes += n * 4;
  return convert_into(t, *out);
}

// matrix rows [rows][K] of the compute type written at dst (row offset inside a concatenation)
int put_matrix(b200_dlm* h, const std::string& name, int64_t rows, int64_t K, void* dst) {
  const Tensor* t = nullptr;
  B200_TRY(find_tensor(h, name, {rows, K}, &t));
  return h->f32 ? convert_into(t, static_cast<float*>(dst)) : convert_into(t, static_cast<bf16*>(dst));
}

// bf16 mode + eligible shape: the row-major matrix is replaced by the tcgen05 GEMM's packed tiles
int seal_weight(b200_dlm* h, Weight& w, void* rm, int N, int K, std::vector<void*>& drop, int ld_out = 0) {
  w.rm = rm; w.N = N; w.K = K; w.tiles = nullptr;
  h->weight_bytes += (int64_t)N * K * esize(h);
  if (!h->f32 && h->use_tc && K >= 8 && K % 8 == 0 && ld_out % 8 == 0 && (N + 127) / 128 <= tc::SK_MAX_TILES) {
    B200_TRY(h->weights.alloc(&w.tiles, tc::sk_packed_bytes(N, K, 0, 0), false));
    B200_TRY(tc::sk_pack_weights(static_cast<const bf16*>(rm), w.tiles, N, K, 0, 0, nullptr));
    drop.push_back(rm);
    w.rm = nullptr;
  }
  return B200_OK;
}

template <typename TA, typename TB, typename TC>
int gemm_nt(cudaStream_t st, const TA* A, long long lda, long long sa, const TB* B, long long ldb, long long sb, TC* C, long long ldc,
            long long sc, int M, int N, int K, int batch, float alpha, int accumulate = 0, int outer = 1, long long sa2 = 0, long long sb2 = 0,
            long long sc2 = 0) {
  dim3 grid(ceil_div(N, 64), ceil_div(M, 64), batch * outer);
  B200_LAUNCH((gemm_nt_kernel<TA, TB, TC>), grid, 256, 0, st, A, lda, sa, B, ldb, sb, C, ldc, sc, M, N, K, alpha, accumulate, outer > 1 ? batch : 0, sa2, sb2, sc2);
  return check_launch("gemm_nt");
}

// the per-head products around the latent attention: tensor cores for bf16 weights (K a multiple of 16), else CUDA cores
template <typename TA, typename TB, typename TC>
int head_gemm(cudaStream_t st, const TA* A, long long lda, long long sa, const TB* B, long long ldb, long long sb, TC* C, long long ldc,
              long long sc, int M, int N, int K, int batch, float alpha, bool tensor_cores) {
  if constexpr (sizeof(TB) == 2) {
    constexpr long long AE = 16 / (long long)sizeof(TA);       // elements of A per 16 bytes
    const bool aligned = lda % AE == 0 && sa % AE == 0 && ldb % 8 == 0 && sb % 8 == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)B % 16 == 0;
    if (tensor_cores && K % 16 == 0 && aligned) {
      dim3 grid(ceil_div(N, 64), ceil_div(M, 64), batch);
      B200_LAUNCH((gemm_nt_mma_kernel<TA, TC>), grid, 128, 0, st, A, lda, sa, B, ldb, sb, C, ldc, sc, M, N, K, alpha);
      return check_launch("gemm_nt_mma");
    }
  }
  return gemm_nt(st, A, lda, sa, B, ldb, sb, C, ldc, sc, M, N, K, batch, alpha);
}

// y[M][N] = x[M][K] . W^T in the compute type
template <typename T>
int linear(b200_dlm* h, const T* x, long long ldx, const Weight& w, T* y, long long ldy, int M);

template <>
int linear<float>(b200_dlm* h, const float* x, long long ldx, const Weight& w, float* y, long long ldy, int M) {
  return gemm_nt(h->stream, x, ldx, 0, static_cast<const float*>(w.rm), (long long)w.K, 0, y, ldy, 0, M, w.N, w.K, 1, 1.f);
}

template <>
int linear<bf16>(b200_dlm* h, const bf16* x, long long ldx, const Weight& w, bf16* y, long long ldy, int M) {
  if (w.tiles && ldx % 8 == 0 && ldy % 8 == 0) {
    tc::SkTuning t;
    for (int m0 = 0; m0 < M; m0 += 256) {          // the LM's GEMM takes up to 256 rows per launch
      const int m = std::min(256, M - m0);
      B200_TRY(tc::sk_linear(h->plans, x + (long long)m0 * ldx, ldx, w.tiles, y + (long long)m0 * ldy, ldy, nullptr, 0, m, w.N, w.K, 0, 0,
                             h->sk_ws, h->sk_counters, t, h->stream));
    }
    return B200_OK;
  }
  if (!w.rm) B200_FAIL(B200_ERR_STATE, "decoder LM: a packed linear met an unaligned activation stride");
  return gemm_nt(h->stream, x, ldx, 0, static_cast<const bf16*>(w.rm), (long long)w.K, 0, y, ldy, 0, M, w.N, w.K, 1, 1.f);
}

template <typename T, int NCH, int RPW>
int launch_attn(cudaStream_t st, const AttnParams& p, int tiles, int nsplit) {
  const size_t smem = (size_t)32 * p.r * sizeof(T);
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    B200_CUDA(cudaFuncSetAttribute(latent_attn_kernel<T, NCH, RPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set = true;
  }
  B200_LAUNCH((latent_attn_kernel<T, NCH, RPW>), dim3(tiles, nsplit), 128, smem, st, p);
  return check_launch("latent_attn");
}

// keys are cut over `nsplit` CTAs per tile when the tiles alone cannot fill the GPU (decoding, short portions)
int pick_split(int forced, int tiles, int max_ctx, int rpt, int r, size_t part_floats) {
  const int key_tiles = ceil_div(max_ctx, 32);
  // one wave: registers allow three CTAs of the tensor-core kernel per SM, its two key tiles of rows of r elements may allow fewer
  const size_t cta_smem = (size_t)2 * 32 * (r + 8) * 2 + 11 * 1024;
  const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(3, (size_t)227 * 1024 / cta_smem));
  int nsplit = 1;
  if (forced > 0) nsplit = std::min(forced, 64);
  else if (tiles < 148) nsplit = std::min(std::max(148 * per_sm / tiles, 1), 64);
  nsplit = std::max(1, std::min(nsplit, key_tiles));
  nsplit = ceil_div(key_tiles, ceil_div(key_tiles, nsplit));                   // no split without a key tile
  while (nsplit > 1 && (size_t)tiles * nsplit * rpt * (r + 2) > part_floats) --nsplit;
  return nsplit;
}

template <int NKS>
int launch_attn_mma(cudaStream_t st, const AttnParams& p, int tiles) {
  const size_t smem = (size_t)2 * 32 * (p.r + 8) * 2 + (size_t)4 * 16 * 32 * 4 + (size_t)16 * 40 * 2 + (size_t)3 * 16 * 4 + 16;      // keys, partial scores, weights, row state, mbarriers
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(latent_attn_mma_kernel<NKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    attr_set = true;
  }
  B200_LAUNCH(latent_attn_mma_kernel<NKS>, dim3(tiles, p.nsplit), 128, smem, st, p);
  return check_launch("latent_attn_mma");
}

// bf16 rows of 64, 128, .., 576 elements (512 of latent + 64 of a rotated key part) take the tensor-core kernel
inline bool attn_mma_takes(int r, int rpt, bool bf16_latents) { return bf16_latents && rpt == 16 && r % 64 == 0 && r <= 576; }

template <typename T>
int run_attention(cudaStream_t st, AttnParams p, int tiles, int rpt, bool tensor_cores = true) {
  const int r = p.r;
  if (tensor_cores && attn_mma_takes(r, rpt, sizeof(T) == 2)) {
    switch (r / 64) {
      case 1: B200_TRY(launch_attn_mma<1>(st, p, tiles)); break;
      case 2: B200_TRY(launch_attn_mma<2>(st, p, tiles)); break;
      case 3: B200_TRY(launch_attn_mma<3>(st, p, tiles)); break;
      case 4: B200_TRY(launch_attn_mma<4>(st, p, tiles)); break;
      case 5: B200_TRY(launch_attn_mma<5>(st, p, tiles)); break;
      case 6: B200_TRY(launch_attn_mma<6>(st, p, tiles)); break;
      case 7: B200_TRY(launch_attn_mma<7>(st, p, tiles)); break;
      case 8: B200_TRY(launch_attn_mma<8>(st, p, tiles)); break;
      default: B200_TRY(launch_attn_mma<9>(st, p, tiles)); break;
    }
  }
  else if (r <= 64) B200_TRY((launch_attn<T, 2, 4>(st, p, tiles, p.nsplit)));
  else if (r <= 128) B200_TRY((launch_attn<T, 4, 4>(st, p, tiles, p.nsplit)));
  else if (r <= 256) B200_TRY((launch_attn<T, 8, 4>(st, p, tiles, p.nsplit)));
  else if (r <= 512) B200_TRY((launch_attn<T, 16, 4>(st, p, tiles, p.nsplit)));
  else if (r <= 576) B200_TRY((launch_attn<T, 18, 4>(st, p, tiles, p.nsplit)));
  else B200_TRY((launch_attn<T, 32, 2>(st, p, tiles, p.nsplit)));
  if (p.nsplit > 1) {
    B200_LAUNCH(latent_attn_merge_kernel, dim3(tiles, rpt), 128, 0, st, p.part, p.tile_row0, p.tile_rows, p.out, r, p.nsplit, rpt, p.gate, p.ldg, p.H);
    B200_TRY(check_launch("latent_attn_merge"));
  }
  return B200_OK;
}

template <typename T>
int attention(b200_dlm* h, const Layer& L, int max_ctx) {
  const TileSig& s = h->sigs[L.sig];
  AttnParams p;
  p.qa = h->qa; p.cache = L.cache; p.sink = L.sink;
  p.tile_row0 = h->meta_dev + s.off_row0; p.tile_rows = h->meta_dev + s.off_rows; p.tile_slot = h->meta_dev + s.off_slot;
  p.tok_pos = h->meta_dev + h->off_pos;
  p.out = h->ol; p.part = h->part; p.cap = h->cap; p.r = L.c.a.kv_rank; p.H = L.c.a.heads; p.err = h->err;
  p.nsplit = pick_split(h->attn_split, s.count, max_ctx, s.rpt, p.r, h->part_floats);
  return run_attention<T>(h->stream, p, s.count, s.rpt, h->attn_tc != 0);
}

enum { CLS_LINEAR = 0, CLS_ATTN = 1, CLS_FOLD = 2, CLS_ELEMENTWISE = 3, CLS_RECURRENT = 4, CLS_EXPERTS = 5 };

int mark(b200_dlm* h, int cls) {       // cls >= 0 opens an interval of that class, -1 closes the open one
  if (!h->time_kernels) return B200_OK;
  if (h->ev_used == h->ev_pool.size()) {
    cudaEvent_t e;
    B200_CUDA(cudaEventCreate(&e));
    h->ev_pool.push_back(e); h->ev_class.push_back(0);
  }
  h->ev_class[h->ev_used] = cls;
  B200_CUDA(cudaEventRecord(h->ev_pool[h->ev_used++], h->stream));
  return B200_OK;
}
#define TIMED(cls, ...) do { B200_TRY(mark(h, cls)); __VA_ARGS__; B200_TRY(mark(h, -1)); } while (0)

template <typename T>
int step_body(b200_dlm* h, int n_tok, int n_want, int max_ctx, float* logits_out) {
  const b200_dlm_config& c = h->cfg;
  const int W = c.width;
  cudaStream_t st = h->stream;
  const int* meta = h->meta_dev;
  const long long stride = (long long)h->tmax * W;
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(embed_kernel<T>, n_tok, 256, 0, st, meta + h->off_tok, static_cast<const T*>(h->embed), c.vocab, W, c.embedding_scale,
              h->xin, h->stack, h->err));
  T* hb = static_cast<T*>(h->hbuf);
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(layernorm_kernel<T>, n_tok, 256, 0, st, h->xin, (const int*)nullptr, h->layers[0].n1w, h->layers[0].n1b, hb, W, c.norm_eps));
  for (int li = 0; li < c.n_layers; ++li) {
    const Layer& L = h->layers[li];
    const int H = L.c.a.heads, dk = L.c.a.dim, dv = L.c.a.vdim, r = L.c.a.kv_rank;
    T* proj = static_cast<T*>(h->proj);
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, hb, W, L.cat, proj, L.ldp, n_tok)));
    // mixer: latent attention
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(latent_append_kernel<T>, ceil_div(n_tok, 4), 128, 0, st, proj, (long long)L.ldp, L.off_dkv, L.cnorm, static_cast<T*>(L.cache),
                h->cap, r, meta + h->off_slot, meta + h->off_pos, n_tok, c.norm_eps));
    // query folded through W_uk (and the score scale): qa[t][h][:] = scale * q[t][h][:] . W_uk[h]
    TIMED(CLS_FOLD, B200_TRY(head_gemm(st, proj + L.off_q, (long long)L.ldp, (long long)dk, static_cast<const T*>(L.ukT), (long long)dk, (long long)r * dk, h->qa,
                     (long long)H * r, (long long)r, n_tok, r, dk, H, L.c.a.scale, h->attn_tc != 0)));
    TIMED(CLS_ATTN, B200_TRY(attention<T>(h, L, max_ctx)));
    // values: o[t][h][:] = W_uv[h] . (sum_j p_j c_j)
    T* ob = static_cast<T*>(h->obuf);
    TIMED(CLS_FOLD, B200_TRY(head_gemm(st, h->ol, (long long)H * r, (long long)r, static_cast<const T*>(L.uv), (long long)r, (long long)dv * r, ob, (long long)H * dv,
                     (long long)dv, n_tok, dv, r, H, 1.f, h->attn_tc != 0)));
    T* mixo = static_cast<T*>(h->mixo);
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob, (long long)H * dv, L.o, mixo, W, n_tok)));
    // feed-forward
    T* ffo = nullptr;
    if (L.c.mlp == B200_MLP_DENSE_RELU2) {
      T* act = static_cast<T*>(h->act);
      const long long n = (long long)n_tok * L.c.ff;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(relu2_kernel<T>, (unsigned)ceil_div64(n, 256), 256, 0, st, proj, (long long)L.ldp, L.off_up, act, L.c.ff, n));
      ffo = static_cast<T*>(h->ffo);
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, act, L.c.ff, L.down, ffo, W, n_tok)));
    }
    const bool last = li + 1 == c.n_layers;
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(block_end_kernel<T>, n_tok, 256, 0, st, h->xin, mixo, ffo, proj, (long long)L.ldp, L.off_g1, L.off_g2, L.b1, L.b2, c.residual_mult,
                h->stack, stride, li, L.avg, h->trace_layers ? h->trace + (long long)li * stride : nullptr,
                last ? nullptr : h->layers[li + 1].n1w, last ? nullptr : h->layers[li + 1].n1b, hb, W, c.norm_eps));
  }
  B200_TRY(check_launch("decoder LM layers"));
  if (n_want > 0) {
    T* hf = static_cast<T*>(h->hf);
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(layernorm_kernel<T>, n_want, 256, 0, st, h->xin, meta + h->off_want, h->fnw, h->fnb, hf, W, c.norm_eps));
    if (h->head.tiles) {
      const int ldl = (c.vocab + 7) / 8 * 8;
      TIMED(CLS_LINEAR, B200_TRY(linear<bf16>(h, reinterpret_cast<const bf16*>(hf), W, h->head, h->head_bf, ldl, n_want)));
      const long long n = (long long)n_want * c.vocab;
      B200_LAUNCH(rows_to_f32_kernel, (unsigned)ceil_div64(n, 256), 256, 0, st, h->head_bf, (long long)ldl, h->logits, c.vocab, n);
    } else {
      TIMED(CLS_LINEAR, B200_TRY(gemm_nt(st, hf, (long long)W, 0, static_cast<const T*>(h->head.rm), (long long)W, 0, h->logits, (long long)c.vocab, 0, n_want, c.vocab, W, 1, 1.f)));
    }
    if (logits_out)
      B200_CUDA(cudaMemcpyAsync(logits_out, h->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToDevice, st));
  }
  return check_launch("decoder LM step");
}


// ---------------------------------------------------------------------------------------------------------------------------
// Sandwich block: norm -> (canon convolution) -> mixer -> norm -> residual, then norm -> feed-forward -> norm -> residual
// ---------------------------------------------------------------------------------------------------------------------------

// a small tensor of any shape as fp32
int get_f32_shaped(b200_dlm* h, const std::string& name, std::vector<int64_t> shape, float** out) {
  const Tensor* t = nullptr;
  B200_TRY(find_tensor(h, name, shape, &t));
  B200_TRY(h->weights.alloc_t(out, (size_t)t->numel(), false));
  h->weight_bytes += t->numel() * 4;
  return convert_into(t, *out);
}

__global__ void fold_head_mix_kernel(const float* __restrict__ talk, const float* __restrict__ temp, float scale, float* __restrict__ out, int H) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < H * H) out[i] = talk[i] * temp[i % H] * scale;
}

// rotary frequencies base^(-2i/dims), rescaled by wavelength (short waves kept, long waves divided by `factor`, linear blend between)
std::vector<double> rotary_frequencies(const b200_dlm_mixer& m) {
  const int half = m.rot_dims / 2;
  std::vector<double> f((size_t)std::max(half, 1), 0.0);
  const double two_pi = 6.283185307179586476925;
  for (int i = 0; i < half; ++i) {
    double v = std::pow((double)m.rot_base, -2.0 * i / m.rot_dims);
    if (m.rot_factor > 0.f) {
      const double wave = two_pi / v, orig = m.rot_original;
      if (wave < orig / m.rot_high) {
      } else if (wave > orig / m.rot_low) {
        v /= m.rot_factor;
      } else {
        const double sm = (orig / wave - m.rot_low) / ((double)m.rot_high - m.rot_low);
        v = (1.0 - sm) * v / m.rot_factor + sm * v;
      }
    }
    f[i] = v;
  }
  return f;
}

size_t window_attn_smem(const b200_dlm_mixer& m, int QT, int KT, size_t es, int* kstride) {
  const size_t Nq = (size_t)m.heads * m.dim, Nk = (size_t)m.kv_heads * m.dim, Nv = (size_t)m.kv_heads * m.vdim, rows = (size_t)QT * m.heads;
  const size_t words = ((Nk * es + 3) / 4) | 1;           // an odd number of 32-bit words between staged key rows
  *kstride = (int)(words * 4 / es);
  return 4 * (QT * Nq + rows * m.vdim + 2 * rows * (KT + 1) + (size_t)m.heads * m.heads + 3 * rows) + es * ((size_t)KT * *kstride + KT * Nv) + 32;
}

int add_sig(b200_dlm* h, int H, int rpt) {
  for (size_t k = 0; k < h->sigs.size(); ++k) if (h->sigs[k].H == H && h->sigs[k].rpt == rpt) return (int)k;
  TileSig s; s.H = H; s.rpt = rpt; h->sigs.push_back(s);
  return (int)h->sigs.size() - 1;
}

// which window attention kernels a layer's head shapes take: the tile of query tokens and of keys that fits shared memory for
// the CUDA-core kernel (also with tiles of one token, for single-token steps), and the tensor-core kernel when it fits
int plan_window_attention(b200_dlm* h, Layer& L, int i) {
  const b200_dlm_mixer& a = L.c.a;
  const size_t es = esize(h);
  L.QT = 0;
  for (int kt : {32, 16, 8}) {
    for (int qt : {4, 2, 1}) {
      int ks = 0;
      const size_t sm = window_attn_smem(a, qt, kt, es, &ks);
      if (sm <= 200 * 1024) { L.QT = qt; L.KT = kt; L.kstride = ks; L.attn_smem = sm; break; }
    }
    if (L.QT) break;
  }
  if (!L.QT) B200_FAIL(B200_ERR_SHAPE, "decoder LM: layer %d: the window attention's heads do not fit shared memory", i);
  L.sig = add_sig(h, a.heads, L.QT * a.heads);
  for (int kt : {32, 16, 8}) {
    int ks = 0;
    const size_t sm = window_attn_smem(a, 1, kt, es, &ks);
    if (sm <= 200 * 1024) { L.sig_one = add_sig(h, a.heads, a.heads); L.KT_one = kt; L.kstride_one = ks; L.smem_one = sm; break; }
  }
  if (!h->f32 && a.dim % 16 == 0 && a.vdim % 16 == 0) {     // bf16 cache, fragment-sized heads: the tensor-core kernel, if it fits
    const size_t Hh = a.heads, QS = L.Nq + 8, KS = L.Nk + 8, VS = L.Nv + 8;
    const size_t sm = 2 * (16 * QS + 32 * KS + 32 * VS + Hh * 16 * 40) + 4 * (Hh * 16 * 40 + Hh * std::max<size_t>(Hh, 16) + 3 * Hh * 16);
    const int items = ceil_div(a.heads * ceil_div(a.vdim, 64), 8);
    if (sm <= 220 * 1024 && items <= 4) { L.sig_mma = add_sig(h, a.heads, 16 * a.heads); L.mma_items = items <= 2 ? items : 4; L.mma_smem = sm; }
  }
  return B200_OK;
}

int finalize_sandwich_layer(b200_dlm* h, int i, std::vector<void*>& drop) {
  Layer& L = h->layers[i];
  const b200_dlm_config& c = h->cfg;
  const int64_t W = c.width;
  const size_t es = esize(h);
  const std::string p = "l" + std::to_string(i) + ".";
  auto matrix = [&](const std::string& name, int64_t rows, int64_t K, void** out) -> int {
    B200_TRY(h->weights.alloc(out, (size_t)rows * K * es, false));
    h->weight_bytes += rows * K * es;
    return put_matrix(h, name, rows, K, *out);
  };
  B200_TRY(get_f32(h, p + "norm1", W, &L.n1w));
  B200_TRY(get_f32(h, p + "norm1b", W, &L.n1bw));
  if (c.canon_taps > 0) B200_TRY(get_f32_shaped(h, p + "canon1", {W, c.canon_taps}, &L.canon));
  void* cat = nullptr;
  auto at = [&](int off) { return static_cast<char*>(cat) + (size_t)off * W * es; };
  if (L.c.mixer == B200_MIXER_PARALLEL) {
    const b200_dlm_mixer &a = L.c.a, &b = L.c.b;
    const std::string l = p + "mix.left.", r = p + "mix.right.";
    L.Nq = a.heads * a.dim; L.Nk = a.kv_heads * a.dim; L.Nv = a.kv_heads * a.vdim;
    const int Rq = b.heads * b.dim, Rv = b.heads * b.vdim;
    const Tensor* a1 = h->store.find(r + "a1");
    if (!a1 || a1->shape.size() != 2 || a1->shape[1] != W) B200_FAIL(B200_ERR_MISSING, "decoder LM finalize: tensor '%sa1' [rank, width] was not loaded", r.c_str());
    L.decay_rank = (int)a1->shape[0];
    L.a_q = 0; L.a_k = L.Nq; L.a_v = L.a_k + L.Nk;
    L.r_q = L.a_v + L.Nv; L.r_k = L.r_q + Rq; L.r_v = L.r_k + Rq; L.r_g = L.r_v + Rv; L.r_a1 = (L.r_g + Rv + 7) / 8 * 8;    // the decay's inner projection starts on 16 bytes
    L.ncat = L.r_a1 + L.decay_rank;
    L.ldp = (L.ncat + 7) / 8 * 8;
    B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, true));
    B200_TRY(put_matrix(h, l + "q", L.Nq, W, at(L.a_q)));
    B200_TRY(put_matrix(h, l + "k", L.Nk, W, at(L.a_k)));
    B200_TRY(put_matrix(h, l + "v", L.Nv, W, at(L.a_v)));
    B200_TRY(put_matrix(h, r + "q", Rq, W, at(L.r_q)));
    B200_TRY(put_matrix(h, r + "k", Rq, W, at(L.r_k)));
    B200_TRY(put_matrix(h, r + "v", Rv, W, at(L.r_v)));
    B200_TRY(put_matrix(h, r + "g", Rv, W, at(L.r_g)));
    B200_TRY(put_matrix(h, r + "a1", L.decay_rank, W, at(L.r_a1)));
    B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
    // left: window attention
    B200_TRY(get_f32(h, l + "q.norm", L.Nq, &L.qnorm));
    B200_TRY(get_f32(h, l + "k.norm", L.Nk, &L.knorm));
    if (a.conv_taps >= 1) {
      const int C = L.Nq + L.Nk + L.Nv, taps = a.conv_taps;
      B200_TRY(h->weights.alloc_t(&L.qkv_conv, (size_t)C * taps, false));
      const Tensor* t = nullptr;
      int off = 0;
      for (const char* nm : {"q", "k", "v"}) {
        const int rows = nm[0] == 'q' ? L.Nq : nm[0] == 'k' ? L.Nk : L.Nv;
        B200_TRY(find_tensor(h, l + nm + ".conv", {rows, taps}, &t));
        B200_TRY(convert_into(t, L.qkv_conv + (size_t)off * taps));
        off += rows;
      }
      h->weight_bytes += (int64_t)C * taps * 4;
    }
    float *talk = nullptr, *temp = nullptr;
    B200_TRY(get_f32_shaped(h, l + "talk", {a.heads, a.heads}, &talk));
    B200_TRY(get_f32(h, l + "temp", a.heads, &temp));
    B200_TRY(get_f32(h, l + "sink", a.heads, &L.sink));
    B200_TRY(h->weights.alloc_t(&L.mixhh, (size_t)a.heads * a.heads, false));
    B200_LAUNCH(fold_head_mix_kernel, ceil_div(a.heads * a.heads, 256), 256, 0, nullptr, talk, temp, a.scale, L.mixhh, a.heads);
    B200_TRY(check_launch("fold_head_mix"));
    const std::vector<double> fr = rotary_frequencies(a);
    B200_TRY(h->weights.alloc_t(&L.freq, fr.size(), false));
    B200_CUDA(cudaMemcpy(L.freq, fr.data(), fr.size() * sizeof(double), cudaMemcpyHostToDevice));
    void* wo = nullptr;
    B200_TRY(matrix(l + "o", W, (int64_t)a.heads * a.vdim, &wo));
    h->weight_bytes -= W * a.heads * a.vdim * es;
    B200_TRY(seal_weight(h, L.a_o, wo, (int)W, a.heads * a.vdim, drop, (int)W));
    B200_TRY(get_f32(h, l + "out", W, &L.a_out));
    B200_TRY(get_f32(h, r + "out", W, &L.b_out));
    B200_TRY(plan_window_attention(h, L, i));
    // right: gated linear attention
    B200_TRY(matrix(r + "a2", Rq, L.decay_rank, &L.a2));
    B200_TRY(get_f32(h, r + "a2.b", Rq, &L.a2b));
    B200_TRY(get_f32(h, r + "norm", b.vdim, &L.rnorm));
    void* wo2 = nullptr;
    B200_TRY(matrix(r + "o", W, Rv, &wo2));
    h->weight_bytes -= W * Rv * es;
    B200_TRY(seal_weight(h, L.r_o, wo2, (int)W, Rv, drop, (int)W));
  } else {      // B200_MIXER_MLSTM
    const b200_dlm_mixer& a = L.c.a;
    const std::string m = p + "mix.";
    const int Rq = a.heads * a.dim, Rv = a.heads * a.vdim;
    L.r_q = 0; L.r_k = Rq; L.r_v = 2 * Rq; L.r_g = L.r_v + Rv; L.ncat = L.r_g + Rv;
    L.ldp = (L.ncat + 7) / 8 * 8;
    B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, false));
    B200_TRY(put_matrix(h, m + "q", Rq, W, at(L.r_q)));
    B200_TRY(put_matrix(h, m + "k", Rq, W, at(L.r_k)));
    B200_TRY(put_matrix(h, m + "v", Rv, W, at(L.r_v)));
    B200_TRY(put_matrix(h, m + "g", Rv, W, at(L.r_g)));
    B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
    B200_TRY(h->weights.alloc(&L.w_if, (size_t)2 * a.heads * W * es, false));
    B200_TRY(put_matrix(h, m + "i", a.heads, W, L.w_if));
    B200_TRY(put_matrix(h, m + "f", a.heads, W, static_cast<char*>(L.w_if) + (size_t)a.heads * W * es));
    h->weight_bytes += 2 * a.heads * W * es;
    B200_TRY(h->weights.alloc_t(&L.if_b, (size_t)2 * a.heads, false));
    const Tensor* t = nullptr;
    B200_TRY(find_tensor(h, m + "i.b", {a.heads}, &t));
    B200_TRY(convert_into(t, L.if_b));
    B200_TRY(find_tensor(h, m + "f.b", {a.heads}, &t));
    B200_TRY(convert_into(t, L.if_b + a.heads));
    B200_TRY(get_f32(h, m + "norm", Rv, &L.rnorm));
    void* wo = nullptr;
    B200_TRY(matrix(m + "o", W, Rv, &wo));
    h->weight_bytes -= W * Rv * es;
    B200_TRY(seal_weight(h, L.r_o, wo, (int)W, Rv, drop, (int)W));
  }
  if (L.c.mlp == B200_MLP_MOE_RELU2) {
    const int64_t E = L.c.experts, F = L.c.ff;
    B200_TRY(get_f32(h, p + "norm2", W, &L.n2w));
    B200_TRY(get_f32(h, p + "norm2b", W, &L.n2bw));
    B200_TRY(matrix(p + "mlp.router", E, W, &L.router));
    B200_TRY(h->weights.alloc(&L.ups, (size_t)E * F * W * es, false));
    B200_TRY(h->weights.alloc(&L.downs, (size_t)E * W * F * es, false));
    for (int64_t e = 0; e < E; ++e) {
      const std::string q = p + "mlp.e" + std::to_string(e) + ".";
      B200_TRY(put_matrix(h, q + "up", F, W, static_cast<char*>(L.ups) + (size_t)e * F * W * es));
      B200_TRY(put_matrix(h, q + "down", W, F, static_cast<char*>(L.downs) + (size_t)e * W * F * es));
    }
    h->weight_bytes += 2 * E * F * W * es;
  }
  return B200_OK;
}

template <typename T>
int small_proj(b200_dlm* h, const T* x, long long ldx, const void* w, const float* b, float* out, int M, int N, int K) {
  B200_LAUNCH(small_proj_f32_kernel<T>, M, 256, (size_t)K * 4, h->stream, x, ldx, static_cast<const T*>(w), b, out, N, K);
  return check_launch("small_proj_f32");
}

template <int MODE, int R, int LPC, int CB, bool VL = false>
int launch_scan_r(cudaStream_t st, const ScanParams& p, int n_entries) {
  constexpr int NC = 128 / LPC * CB;
  const dim3 grid(n_entries * p.heads, ceil_div(p.vdim, NC));
  const size_t smem = (size_t)2 * p.stage * (p.prow + NC) * 4;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute((matrix_memory_scan_kernel<MODE, R, LPC, CB, VL>), cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    attr_set = true;
  }
  B200_LAUNCH((matrix_memory_scan_kernel<MODE, R, LPC, CB, VL>), grid, 128, smem, st, p);
  return check_launch("matrix_memory_scan");
}

// How the recurrence kernel is laid out for this step, set in p: 16 or 8 lanes per column, rows per thread, plain or
// lane-ordered prep rows and their length.  whole: the step's entries are taken as they are (no segments).
struct ScanLayout { bool wide, lanes4; int rows, nu; };

template <int MODE>
ScanLayout scan_layout(b200_dlm* h, ScanParams& p, bool whole) {
  p.prep = h->scan_prep; p.vprep = h->scan_v;
  p.vec = p.vdim % 4 == 0;
  p.stage = 8;      // short stages: less shared memory per CTA, more CTAs per SM to overlap the chains
  p.ent_par = h->meta_dev + h->off_ent_par; p.slots = h->slots;
  if (whole) {
    p.ent_tok0 = h->meta_dev + h->off_whole_tok0; p.ent_ntok = h->meta_dev + h->off_whole_ntok; p.ent_slot = h->meta_dev + h->off_whole_slot;
    p.ent_pos0 = h->meta_dev + h->off_whole_pos0;
    p.ent_seg = h->meta_dev + h->off_zero; p.ent_nseg = h->meta_dev + h->off_one; p.ent_buf = h->meta_dev + h->off_zero;
  } else {
    p.ent_tok0 = h->meta_dev + h->off_ent_tok0; p.ent_ntok = h->meta_dev + h->off_ent_ntok; p.ent_slot = h->meta_dev + h->off_ent_slot;
    p.ent_pos0 = h->meta_dev + h->off_ent_pos0;
    p.ent_seg = h->meta_dev + h->off_ent_seg; p.ent_nseg = h->meta_dev + h->off_ent_nseg; p.ent_buf = h->meta_dev + h->off_ent_buf;
  }
  p.segS = h->segS; p.segB = h->segB; p.segM = h->segM; p.qb = h->gate32; p.tokM = h->tokM;      // the decay logits are spent once prep has run
  // a few long requests: 16 lanes per column (twice the CTAs, half the chain per token); batches and single tokens: 8 lanes per
  // column (state rows read in full sectors).  Portions of more than 8 tokens: the variant whose threads own adjacent rows and
  // read q, k and the decay four rows per load from lane-ordered prep rows (a third of the instructions per token; its state
  // accesses are scattered, which costs nothing once per portion but would cost single-token steps twice their time).
  ScanLayout L;
  L.nu = whole ? h->n_entries : h->n_units;
  L.wide = h->max_entry_tokens > 8 && L.nu * p.heads * ceil_div(p.vdim, 16) < 2 * 148 && p.dim > 16;
  L.lanes4 = h->max_entry_tokens > 8;
  const int lpc = L.wide ? 16 : 8;
  L.rows = L.wide ? (p.dim <= 64 ? 4 : p.dim <= 128 ? 8 : 16) : (p.dim <= 32 ? 4 : p.dim <= 64 ? 8 : p.dim <= 128 ? 16 : 32);
  p.lpc = L.lanes4 ? lpc : 0; p.rows = L.rows;
  const int Dp = L.lanes4 ? lpc * L.rows : p.dim;
  p.prow = ((MODE == MODE_DECAY || MODE == MODE_CHDELTA ? 3 : 2) * Dp + (MODE == MODE_DECAY ? 0 : 2) + 3) / 4 * 4;
  return L;
}

// the recurrence per (request, head) on prepared rows; long portions run as segments side by side, are chained, and their later
// segments get the carried state's share added
template <int MODE>
int scan_run(b200_dlm* h, const ScanParams& p, const ScanLayout& L, bool whole) {
  cudaStream_t st = h->stream;
  const int nu = L.nu, rows = L.rows;
  int rc;
  if (L.wide) {
    if (rows == 4) rc = launch_scan_r<MODE, 4, 16, 1, true>(st, p, nu);
    else if (rows == 8) rc = launch_scan_r<MODE, 8, 16, 1, true>(st, p, nu);
    else rc = launch_scan_r<MODE, 16, 16, 1, true>(st, p, nu);
  } else if (L.lanes4) {
    if (rows == 4) rc = launch_scan_r<MODE, 4, 8, 1, true>(st, p, nu);
    else if (rows == 8) rc = launch_scan_r<MODE, 8, 8, 1, true>(st, p, nu);
    else if (rows == 16) rc = launch_scan_r<MODE, 16, 8, 1, true>(st, p, nu);
    else rc = launch_scan_r<MODE, 32, 8, 1, true>(st, p, nu);
  } else {
    if (rows == 4) rc = launch_scan_r<MODE, 4, 8, 1>(st, p, nu);
    else if (rows == 8) rc = launch_scan_r<MODE, 8, 8, 1>(st, p, nu);
    else if (rows == 16) rc = launch_scan_r<MODE, 16, 8, 1>(st, p, nu);
    else rc = launch_scan_r<MODE, 32, 8, 1>(st, p, nu);
  }
  B200_TRY(rc);
  if constexpr (MODE != MODE_DELTA && MODE != MODE_CHDELTA) {
  bool any = false;
  for (auto& u : h->units) any |= u.buf >= 0;
  if (!any || whole) return B200_OK;
  B200_LAUNCH(scan_chain_kernel<MODE>, dim3(nu * p.heads, ceil_div((p.vdim + 1) * p.dim, 256)), 256, 0, st, p);
  B200_TRY(check_launch("scan_chain"));
  // the carried state's share for the later segments: runs of segments of one portion with equal length go as one batched product
  const long long H = p.heads, D = p.dim, V = p.vdim;
  for (size_t i = 0; i < h->units.size();) {
    const auto& u = h->units[i];
    if (u.buf < 0 || u.seg == 0) { ++i; continue; }
    size_t j = i + 1;
    while (j < h->units.size() && h->units[j].buf == h->units[j - 1].buf + 1 && h->units[j].seg == h->units[j - 1].seg + 1 && h->units[j].ntok == u.ntok) ++j;
    const int run = (int)(j - i);
    const float* start = h->segS + (long long)u.buf * H * (V + 1) * D;        // the segments' true start states, [run][heads][vdim + 1][dim]
    float* out = p.out + (long long)u.tok0 * H * V;
    if (MODE == MODE_DECAY) {      // out += (q . decay so far) S_start
      B200_TRY(gemm_nt(st, h->gate32 + (long long)u.tok0 * H * D, H * D, D, start, D, (V + 1) * D, out, H * V, V, u.ntok, (int)V, (int)D, (int)H, 1.f, 1,
                       run, (long long)u.ntok * H * D, H * (V + 1) * D, (long long)u.ntok * H * V));
    } else {                       // [S_start^T q | n_start . q], then the weighted meeting with the local numerators
      float* corr = h->corr + (long long)u.tok0 * H * (V + 1);
      B200_TRY(gemm_nt(st, h->gate32 + (long long)u.tok0 * H * D, H * D, D, start, D, (V + 1) * D, corr, H * (V + 1), V + 1, u.ntok,
                       (int)V + 1, (int)D, (int)H, 1.f, 0, run, (long long)u.ntok * H * D, H * (V + 1) * D, (long long)u.ntok * H * (V + 1)));
      for (size_t k = i; k < j; ++k) {
        const auto& w = h->units[k];
        const long long rows2 = (long long)w.ntok * H;
        B200_LAUNCH(mlstm_combine_kernel, (unsigned)ceil_div64(rows2, 4), 128, 0, st, p.out + (long long)w.tok0 * H * V, h->corr + (long long)w.tok0 * H * (V + 1),
                    h->tokM + (long long)w.tok0 * H * 4, h->segM + (long long)w.buf * H * 4, (int)H, (int)V, rows2);
      }
      B200_TRY(check_launch("mlstm_combine"));
    }
    i = j;
  }
  }
  return B200_OK;
}

// prep rows (q, k and the decay or the two gates, fp32) for every token of the step, then the recurrence
template <typename T, int MODE>
int launch_scan(b200_dlm* h, ScanParams p, int n_tok) {
  const ScanLayout L = scan_layout<MODE>(h, p, false);
  B200_LAUNCH((scan_prep_kernel<T, MODE>), n_tok, 256, (size_t)2 * p.rot_half * sizeof(float), h->stream, p);
  B200_TRY(check_launch("scan_prep"));
  return scan_run<MODE>(h, p, L, false);
}

template <typename T>
int window_attention(b200_dlm* h, const Layer& L, int n_tok, int max_ctx, long long ldq = 0) {      // ldq: row stride of the fp32 queries (0: q, k, v side by side)
  const b200_dlm_mixer& a = L.c.a;
  bool mma = false;
  if constexpr (sizeof(T) == 2) mma = h->attn_tc && L.sig_mma >= 0 && (h->max_entry_tokens > 1 || h->attn_tc > 1);      // single tokens: a 16-row fragment tile would be all padding
  const bool one = !mma && h->max_entry_tokens == 1 && L.sig_one >= 0;
  const TileSig& s = h->sigs[mma ? L.sig_mma : one ? L.sig_one : L.sig];
  const int QT = mma ? 16 : one ? 1 : L.QT, KT = mma ? 32 : one ? L.KT_one : L.KT;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(window_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    B200_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    B200_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    B200_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  WindowAttnParams p;
  p.q = h->qkv32; p.ldq = ldq > 0 ? ldq : L.Nq + L.Nk + L.Nv; p.kcache = L.kcache; p.vcache = L.vcache; p.mix = L.mixhh; p.sink = L.sink;
  p.tile_row0 = h->meta_dev + s.off_row0; p.tile_rows = h->meta_dev + s.off_rows; p.tile_slot = h->meta_dev + s.off_slot;
  p.tok_pos = h->meta_dev + h->off_pos; p.out = h->obuf; p.part = h->part;
  p.cap = h->cap; p.H = a.heads; p.G = a.kv_heads; p.dim = a.dim; p.vdim = a.vdim; p.window = a.window; p.QT = QT; p.KT = KT; p.kstride = one ? L.kstride_one : L.kstride;
  p.vec = ((size_t)L.Nk * sizeof(T)) % 16 == 0 && ((size_t)L.Nv * sizeof(T)) % 16 == 0;
  // keys are cut over several CTAs per tile when the tiles alone cannot fill the GPU (decoding, short portions)
  const int key_tiles = ceil_div(std::min(a.window, max_ctx) + QT - 1, KT);
  int nsplit = 1;
  if (h->attn_split > 0) nsplit = std::min(h->attn_split, 64);
  else if (s.count < 148) nsplit = std::min(std::max((one ? 444 : 296) / std::max(s.count, 1), 1), 64);
  nsplit = std::max(1, std::min(nsplit, key_tiles));
  const int rpt = QT * a.heads;
  while (nsplit > 1 && (size_t)s.count * nsplit * rpt * (a.vdim + 2) > h->part_floats) --nsplit;
  p.nsplit = nsplit;
  if (mma) {
    const dim3 grid(s.count, nsplit);
    if (L.mma_items == 1) B200_LAUNCH(window_attn_mma_kernel<1>, grid, 256, L.mma_smem, h->stream, p);
    else if (L.mma_items == 2) B200_LAUNCH(window_attn_mma_kernel<2>, grid, 256, L.mma_smem, h->stream, p);
    else B200_LAUNCH(window_attn_mma_kernel<4>, grid, 256, L.mma_smem, h->stream, p);
  } else {
    B200_LAUNCH(window_attn_kernel<T>, dim3(s.count, nsplit), 256, one ? L.smem_one : L.attn_smem, h->stream, p);
  }
  B200_TRY(check_launch("window_attn"));
  if (nsplit > 1) {
    float* merged = h->f32 ? static_cast<float*>(h->obuf) : h->attn32;
    B200_LAUNCH(latent_attn_merge_kernel, dim3(s.count, rpt), 128, 0, h->stream, h->part, p.tile_row0, p.tile_rows, merged, a.vdim, nsplit, rpt);
    B200_TRY(check_launch("window_attn merge"));
    if (!h->f32) {
      const long long n = (long long)n_tok * a.heads * a.vdim;
      B200_LAUNCH(rows_from_f32_kernel<T>, (unsigned)ceil_div64(n, 256), 256, 0, h->stream, merged, static_cast<T*>(h->obuf), n);
      B200_TRY(check_launch("rows_from_f32"));
    }
  }
  return B200_OK;
}

// routed experts on the rows of hb -> yexp [tokens * top][W] (row t * top + k = the k-th chosen expert's output for token t)
template <typename T>
int routed_experts(b200_dlm* h, const Layer& L, const T* hb, int n_tok) {
  const int W = h->cfg.width, E = L.c.experts, top = L.c.top, F = L.c.ff, pairs = n_tok * top;
  cudaStream_t st = h->stream;
  B200_TRY(small_proj<T>(h, hb, W, L.router, nullptr, h->route32, n_tok, E, W));
  B200_LAUNCH(moe_route_kernel, ceil_div(n_tok, 4), 128, 0, st, h->route32, E, top, h->moe_idx, h->moe_w, n_tok);
  bool mma = false;
  if constexpr (sizeof(T) == 2) mma = h->attn_tc && W % 16 == 0 && F % 16 == 0;
  const int tile_m = mma ? 128 : 64;
  B200_LAUNCH(moe_group_kernel, 1, 1024, (size_t)2 * E * sizeof(int), st, h->moe_idx, pairs, top, E, h->moe_rank, h->moe_perm, h->moe_row_tok,
              h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, tile_m);
  B200_TRY(check_launch("moe route / group"));
  const int max_tiles = ceil_div(pairs, tile_m) + std::min(E, pairs);
  T* act = static_cast<T*>(h->act);
  T* yexp = static_cast<T*>(h->yexp);
  const T* ups = static_cast<const T*>(L.ups);
  const T* downs = static_cast<const T*>(L.downs);
  if (mma) {
    if constexpr (sizeof(T) == 2) {
      static bool attr_set = false;
      if (!attr_set) {
        B200_CUDA(cudaFuncSetAttribute(grouped_gemm_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GG_SMEM));
        attr_set = true;
      }
      B200_LAUNCH(grouped_gemm_mma_kernel, dim3(ceil_div(F, 128), max_tiles), 256, GG_SMEM, st, hb, (long long)W, h->moe_row_tok, ups, (long long)W, (long long)F * W,
                  act, (long long)F, (const int*)nullptr, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, F, W, 1);
      B200_LAUNCH(grouped_gemm_mma_kernel, dim3(ceil_div(W, 128), max_tiles), 256, GG_SMEM, st, act, (long long)F, (const int*)nullptr, downs, (long long)F, (long long)W * F,
                  yexp, (long long)W, h->moe_perm, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, W, F, 0);
    }
  } else {
    B200_LAUNCH((grouped_gemm_kernel<T, T, T>), dim3(ceil_div(F, 64), max_tiles), 256, 0, st, hb, (long long)W, h->moe_row_tok, ups, (long long)W, (long long)F * W,
                act, (long long)F, (const int*)nullptr, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, F, W, 1);
    B200_LAUNCH((grouped_gemm_kernel<T, T, T>), dim3(ceil_div(W, 64), max_tiles), 256, 0, st, act, (long long)F, (const int*)nullptr, downs, (long long)F, (long long)W * F,
                yexp, (long long)W, h->moe_perm, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, W, F, 0);
  }
  return check_launch("grouped expert products");
}

template <typename T>
int step_sandwich(b200_dlm* h, int n_tok, int n_want, int max_ctx, float* logits_out) {
  const b200_dlm_config& c = h->cfg;
  const int W = c.width;
  cudaStream_t st = h->stream;
  const int* meta = h->meta_dev;
  const int *tok_slot = meta + h->off_slot, *tok_pos = meta + h->off_pos, *tok_first = meta + h->off_first, *tok_last = meta + h->off_last;
  const long long stride = (long long)h->tmax * W;
  const size_t ysm = (size_t)W * 4;
  T* hb = static_cast<T*>(h->hbuf);
  T* proj = static_cast<T*>(h->proj);
  T* ob = static_cast<T*>(h->obuf);
  T* ob2 = static_cast<T*>(h->obuf2);
  T* mixo = static_cast<T*>(h->mixo);
  T* mixo2 = static_cast<T*>(h->mixo2);
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(embed_norm_kernel<T>, n_tok, 256, 0, st, meta + h->off_tok, static_cast<const T*>(h->embed), c.vocab, W, h->embw,
                                     h->layers[0].n1w, h->xin, h->h32, c.norm_eps, h->err));
  for (int li = 0; li < c.n_layers; ++li) {
    const Layer& L = h->layers[li];
    const bool last = li + 1 == c.n_layers;
    const bool mlp = L.c.mlp != B200_MLP_NONE;
    // what the mixer reads: h + conv(h) over time
    if (c.canon_taps > 0) {
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH((causal_conv_kernel<float, T>), n_tok, 256, 0, st, h->h32, (long long)W, L.canon_hist, L.canon, hb, (long long)W, W, c.canon_taps,
                                         1, tok_slot, tok_pos, tok_first);
            if (c.canon_taps > 1) B200_LAUNCH(conv_carry_kernel<float>, n_tok, 256, 0, st, h->h32, (long long)W, L.canon_hist, W, c.canon_taps - 1, tok_slot, tok_pos, tok_last));
    } else {
      const long long n = (long long)n_tok * W;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(rows_from_f32_kernel<T>, (unsigned)ceil_div64(n, 256), 256, 0, st, h->h32, hb, n));
    }
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, hb, W, L.cat, proj, L.ldp, n_tok)));
    const float* w_after = mlp ? L.n2w : (last ? nullptr : h->layers[li + 1].n1w);      // the norm whose input this sublayer completes
    float* trace = (h->trace_layers && !mlp) ? h->trace + (long long)li * stride : nullptr;
    if (L.c.mixer == B200_MIXER_PARALLEL) {
      const b200_dlm_mixer &a = L.c.a, &b = L.c.b;
      const int C = L.Nq + L.Nk + L.Nv;
      // left: convolution on q, k, v, then norm and rotation, keys and values into the cache
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH((causal_conv_kernel<T, float>), n_tok, 256, 0, st, proj, (long long)L.ldp, L.qkv_hist, L.qkv_conv, h->qkv32, (long long)C, C,
                                         std::max(a.conv_taps, 1), 0, tok_slot, tok_pos, tok_first);
            if (a.conv_taps > 1) B200_LAUNCH(conv_carry_kernel<T>, n_tok, 256, 0, st, proj, (long long)L.ldp, L.qkv_hist, C, a.conv_taps - 1, tok_slot, tok_pos, tok_last);
            B200_LAUNCH(qk_norm_rope_kernel<T>, n_tok, 256, (size_t)a.rot_dims * 4 + 4, st, h->qkv32, (long long)C, L.Nq, L.Nk, L.Nv, a.dim, a.rot_dims / 2, L.qnorm, L.knorm, L.freq,
                        static_cast<T*>(L.kcache), static_cast<T*>(L.vcache), h->cap, tok_slot, tok_pos, c.norm_eps));
      TIMED(CLS_ATTN, B200_TRY(window_attention<T>(h, L, n_tok, max_ctx)));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob, (long long)a.heads * a.vdim, L.a_o, mixo, W, n_tok)));
      // right: decay logits, the recurrence, head norm and gate
      const int Rq = b.heads * b.dim, Rv = b.heads * b.vdim;
      TIMED(CLS_FOLD, B200_TRY(head_gemm(st, proj + L.r_a1, (long long)L.ldp, 0, static_cast<const T*>(L.a2), (long long)L.decay_rank, 0, h->gate32, (long long)Rq, 0,
                                         n_tok, Rq, L.decay_rank, 1, 1.f, h->attn_tc != 0)));
      ScanParams sp;
      sp.proj = proj; sp.ld = L.ldp; sp.off_q = L.r_q; sp.off_k = L.r_k; sp.off_v = L.r_v; sp.z = h->gate32; sp.zb = L.a2b;
      sp.inv_tau = 1.f / b.tau; sp.cap = 0.f; sp.qscale = 1.f / sqrtf((float)b.dim); sp.St = L.St; sp.nvec = nullptr; sp.mval = nullptr;
      sp.ent_tok0 = meta + h->off_ent_tok0; sp.ent_ntok = meta + h->off_ent_ntok; sp.ent_slot = meta + h->off_ent_slot; sp.ent_pos0 = meta + h->off_ent_pos0;
      sp.out = h->scan32; sp.heads = b.heads; sp.dim = b.dim; sp.vdim = b.vdim;
      TIMED(CLS_RECURRENT, B200_TRY((launch_scan<T, MODE_DECAY>(h, sp, n_tok))));
      const long long rows = (long long)n_tok * b.heads;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(head_norm_gate_kernel<T>, (unsigned)ceil_div64(rows, 4), 128, 0, st, h->scan32, L.rnorm, 0, proj, (long long)L.ldp, L.r_g, 1, ob2,
                                         b.heads, b.vdim, rows, c.norm_eps));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob2, (long long)Rv, L.r_o, mixo2, W, n_tok)));
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(sublayer_end_kernel<T>, n_tok, 256, ysm, st, h->xin, mixo, L.a_out, mixo2, L.b_out, 0.5f, (const float*)nullptr, 0, L.n1bw, trace,
                                         w_after, mlp ? nullptr : h->h32, mlp ? hb : nullptr, W, c.norm_eps));
    } else {
      const b200_dlm_mixer& a = L.c.a;
      const int Rv = a.heads * a.vdim;
      TIMED(CLS_FOLD, B200_TRY(small_proj<T>(h, hb, W, L.w_if, L.if_b, h->gate32, n_tok, 2 * a.heads, W)));
      ScanParams sp;
      sp.proj = proj; sp.ld = L.ldp; sp.off_q = L.r_q; sp.off_k = L.r_k; sp.off_v = L.r_v; sp.z = h->gate32; sp.zb = nullptr;
      sp.inv_tau = 0.f; sp.cap = a.gate_cap; sp.qscale = 1.f / sqrtf((float)a.dim); sp.St = L.St; sp.nvec = L.nvec; sp.mval = L.mval;
      sp.ent_tok0 = meta + h->off_ent_tok0; sp.ent_ntok = meta + h->off_ent_ntok; sp.ent_slot = meta + h->off_ent_slot; sp.ent_pos0 = meta + h->off_ent_pos0;
      sp.out = h->scan32; sp.heads = a.heads; sp.dim = a.dim; sp.vdim = a.vdim;
      TIMED(CLS_RECURRENT, B200_TRY((launch_scan<T, MODE_EXPGATE>(h, sp, n_tok))));
      const long long rows = (long long)n_tok * a.heads;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(head_norm_gate_kernel<T>, (unsigned)ceil_div64(rows, 4), 128, 0, st, h->scan32, L.rnorm, a.vdim, proj, (long long)L.ldp, L.r_g, 0, ob2,
                                         a.heads, a.vdim, rows, c.norm_eps));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob2, (long long)Rv, L.r_o, mixo, W, n_tok)));
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(sublayer_end_kernel<T>, n_tok, 256, ysm, st, h->xin, mixo, (const float*)nullptr, (const T*)nullptr, (const float*)nullptr, 1.f,
                                         (const float*)nullptr, 0, L.n1bw, trace, w_after, mlp ? nullptr : h->h32, mlp ? hb : nullptr, W, c.norm_eps));
    }
    if (mlp) {
      TIMED(CLS_EXPERTS, B200_TRY(routed_experts<T>(h, L, hb, n_tok)));
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(sublayer_end_kernel<T>, n_tok, 256, ysm, st, h->xin, static_cast<const T*>(h->yexp), (const float*)nullptr, (const T*)nullptr,
                                         (const float*)nullptr, 1.f, h->moe_w, L.c.top, L.n2bw, h->trace_layers ? h->trace + (long long)li * stride : nullptr,
                                         last ? nullptr : h->layers[li + 1].n1w, h->h32, (T*)nullptr, W, c.norm_eps));
    }
  }
  B200_TRY(check_launch("decoder LM layers"));
  if (n_want > 0) {
    T* hf = static_cast<T*>(h->hf);
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(rmsnorm_rows_kernel<T>, n_want, 256, 0, st, h->xin, meta + h->off_want, h->fnw, hf, W, c.norm_eps));
    const long long n = (long long)n_want * c.vocab;
    if (h->head.tiles) {
      const int ldl = (c.vocab + 7) / 8 * 8;
      TIMED(CLS_LINEAR, B200_TRY(linear<bf16>(h, reinterpret_cast<const bf16*>(hf), W, h->head, h->head_bf, ldl, n_want)));
      B200_LAUNCH(softcap_rows_kernel, (unsigned)ceil_div64(n, 256), 256, 0, st, h->head_bf, (long long)ldl, h->logits, c.vocab, n, c.logit_softcap);
    } else {
      TIMED(CLS_LINEAR, B200_TRY(gemm_nt(st, hf, (long long)W, 0, static_cast<const T*>(h->head.rm), (long long)W, 0, h->logits, (long long)c.vocab, 0, n_want, c.vocab, W, 1, 1.f)));
      if (c.logit_softcap > 0.f)
        B200_LAUNCH(softcap_rows_kernel, (unsigned)ceil_div64(n, 256), 256, 0, st, (const bf16*)nullptr, 0LL, h->logits, c.vocab, n, c.logit_softcap);
    }
    if (logits_out)
      B200_CUDA(cudaMemcpyAsync(logits_out, h->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToDevice, st));
  }
  return check_launch("decoder LM step");
}


// ---------------------------------------------------------------------------------------------------------------------------
// Parallel-residual block: h = rms(x) (1 + w);  x <- x + mixer(h) + ff(h)
// ---------------------------------------------------------------------------------------------------------------------------

// rotary frequencies with the index-ramp rescaling: the index at which a wave makes t turns over `original` positions is
// d(t) = dims ln(original / (2 pi t)) / (2 ln base); the ramp rises from 0 at lo = floor(d(fast)) to 1 at hi = ceil(d(slow));
// f_i <- f_i / factor * ramp + f_i * (1 - ramp); cos and sin are multiplied by 0.1 ln(factor) + 1 (returned in *amp)
std::vector<double> rotary_frequencies_ramp(const b200_dlm_mixer& m, float* amp) {
  const int dims = m.rot_dims, half = dims / 2;
  std::vector<double> f((size_t)std::max(half, 1), 0.0);
  const double two_pi = 6.283185307179586476925, base = m.rot_base, orig = m.rot_original, factor = m.rot_factor;
  auto index_of = [&](double turns) { return dims * std::log(orig / (two_pi * turns)) / (2.0 * std::log(base)); };
  const double lo = std::max(std::floor(index_of(m.rot_fast)), 0.0), hi = std::min(std::ceil(index_of(m.rot_slow)), (double)dims - 1.0);
  for (int i = 0; i < half; ++i) {
    const double v = std::pow(base, -2.0 * i / dims);
    const double ramp = std::min(std::max((i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
    f[i] = v / factor * ramp + v * (1.0 - ramp);
  }
  *amp = (float)(0.1 * std::log(factor) + 1.0);
  return f;
}

template <typename T>
__global__ void interleave_rows_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long long rows, long long K) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= rows * K) return;
  const long long r = i / K, k = i - r * K;
  out[(2 * r) * K + k] = a[i];
  out[(2 * r + 1) * K + k] = b[i];
}

size_t sigmoid_attn_smem(const b200_dlm_mixer& m, int QT, int KT, size_t es, int* kstride) {
  const size_t Nq = (size_t)m.heads * m.dim, Nk = (size_t)m.kv_heads * m.dim, Nv = (size_t)m.kv_heads * m.vdim, rows = (size_t)QT * m.heads;
  const size_t words = ((Nk * es + 3) / 4) | 1;           // an odd number of 32-bit words between staged key rows
  *kstride = (int)(words * 4 / es);
  return 4 * (QT * Nq + rows * m.vdim + 2 * rows * (KT + 1) + (size_t)m.heads * m.heads + m.heads) + es * ((size_t)KT * *kstride + KT * Nv) + 32;
}

int finalize_parallel_layer(b200_dlm* h, int i, std::vector<void*>& drop) {
  Layer& L = h->layers[i];
  const b200_dlm_config& c = h->cfg;
  const b200_dlm_mixer& a = L.c.a;
  const int64_t W = c.width;
  const size_t es = esize(h);
  const std::string p = "l" + std::to_string(i) + ".", m = p + "mix.";
  auto matrix = [&](const std::string& name, int64_t rows, int64_t K, void** out) -> int {
    B200_TRY(h->weights.alloc(out, (size_t)rows * K * es, false));
    return put_matrix(h, name, rows, K, *out);
  };
  B200_TRY(get_f32(h, p + "norm1", W, &L.n1w));
  B200_LAUNCH(add_one_kernel, ceil_div((int)W, 256), 256, 0, nullptr, L.n1w, (int)W);
  const bool attn = L.c.mixer == B200_MIXER_SIGMOID_ATTENTION, ret = L.c.mixer == B200_MIXER_RETENTION, delta = L.c.mixer == B200_MIXER_DELTA;
  const int H = a.heads, G = attn || delta ? a.kv_heads : a.heads;
  L.Nq = (attn ? H : G) * a.dim; L.Nk = G * a.dim; L.Nv = (attn ? G : H) * a.vdim;
  const int Ng = attn ? 0 : H * a.vdim;                    // the recurrent mixers' output gate is as wide as their result
  const bool dense = L.c.mlp == B200_MLP_DENSE_GATED_GELU, moe = L.c.mlp == B200_MLP_MOE_CLAMPED_GLU;
  const int F = L.c.ff, E = L.c.experts;
  L.p_q = 0; L.p_k = L.Nq; L.p_v = L.p_k + L.Nk; L.p_g = L.p_v + L.Nv; L.p_ffg = L.p_g + Ng; L.p_ffu = L.p_ffg + (dense ? F : 0);
  L.ncat = L.p_ffu + (dense ? F : 0);
  L.ldp = (L.ncat + 7) / 8 * 8;
  void* cat = nullptr;
  B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, false));
  auto at = [&](int off) { return static_cast<char*>(cat) + (size_t)off * W * es; };
  B200_TRY(put_matrix(h, m + "q", L.Nq, W, at(L.p_q)));
  B200_TRY(put_matrix(h, m + "k", L.Nk, W, at(L.p_k)));
  B200_TRY(put_matrix(h, m + "v", L.Nv, W, at(L.p_v)));
  if (Ng) B200_TRY(put_matrix(h, m + "g", Ng, W, at(L.p_g)));
  if (dense) {
    B200_TRY(put_matrix(h, p + "mlp.gate", F, W, at(L.p_ffg)));
    B200_TRY(put_matrix(h, p + "mlp.up", F, W, at(L.p_ffu)));
  }
  B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
  // the small fp32 projection: head gates | beta, step size | router logits
  L.s_gate = 0; L.s_ba = attn ? H : 0; L.s_router = L.s_ba + (delta ? 2 * H : 0); L.nsmall = L.s_router + (moe ? E : 0);
  if (L.nsmall) {
    B200_TRY(h->weights.alloc(&L.w_small, (size_t)L.nsmall * W * es, false));
    auto sat = [&](int off) { return static_cast<char*>(L.w_small) + (size_t)off * W * es; };
    if (attn) B200_TRY(put_matrix(h, m + "g", H, W, sat(L.s_gate)));
    if (delta) {
      B200_TRY(put_matrix(h, m + "b", H, W, sat(L.s_ba)));
      B200_TRY(put_matrix(h, m + "a", H, W, sat(L.s_ba + H)));
    }
    if (moe) B200_TRY(put_matrix(h, p + "mlp.router", E, W, sat(L.s_router)));
    h->weight_bytes += (int64_t)L.nsmall * W * es;
  }
  if (a.rot_dims > 0) {
    std::vector<double> fr;
    if (a.rot_scaling == B200_ROT_RAMP) fr = rotary_frequencies_ramp(a, &L.rot_amp);
    else fr = rotary_frequencies(a);
    B200_TRY(h->weights.alloc_t(&L.freq, fr.size(), false));
    B200_CUDA(cudaMemcpy(L.freq, fr.data(), fr.size() * sizeof(double), cudaMemcpyHostToDevice));
  }
  if (attn) {
    B200_TRY(get_f32_shaped(h, m + "talk", {H, H}, &L.mixhh));
    B200_TRY(get_f32(h, m + "pb", H, &L.pbias));
    if (a.v_mix) {
      if (h->vmix_first < 0) h->vmix_first = i;
      else {
        const b200_dlm_mixer& f = h->layers[h->vmix_first].c.a;
        if (f.kv_heads != a.kv_heads || f.vdim != a.vdim)
          B200_FAIL(B200_ERR_SHAPE, "decoder LM: layer %d blends its values with layer %d's, whose key/value heads or value size differ", i, h->vmix_first);
        B200_TRY(get_f32_shaped(h, m + "vmix", {}, &L.vlambda));
      }
    }
    // tile of query tokens and of keys that fits shared memory
    L.QT = 0;
    for (int kt : {32, 16, 8}) {
      for (int qt : {4, 2, 1}) {
        int ks = 0;
        const size_t sm = sigmoid_attn_smem(a, qt, kt, es, &ks);
        if (sm <= 200 * 1024) { L.QT = qt; L.KT = kt; L.kstride = ks; L.attn_smem = sm; break; }
      }
      if (L.QT) break;
    }
    if (!L.QT) B200_FAIL(B200_ERR_SHAPE, "decoder LM: layer %d: the attention's heads do not fit shared memory", i);
    L.sig = add_sig(h, H, L.QT * H);
    for (int kt : {32, 16, 8}) {
      int ks = 0;
      const size_t sm = sigmoid_attn_smem(a, 1, kt, es, &ks);
      if (sm <= 200 * 1024) { L.sig_one = add_sig(h, H, H); L.KT_one = kt; L.kstride_one = ks; L.smem_one = sm; break; }
    }
    if (!h->f32 && a.dim % 16 == 0 && a.vdim % 16 == 0) {     // bf16 cache, fragment-sized heads: the tensor-core kernel, if it fits
      const size_t Hh = H, QS = L.Nq + 8, KS = L.Nk + 8, VS = L.Nv + 8;
      const size_t sm = 2 * (16 * QS + 32 * KS + 32 * VS + Hh * 16 * 40) + 4 * (Hh * 16 * 40 + Hh * std::max<size_t>(Hh, 16) + Hh);
      const int items16 = ceil_div(H * ceil_div(a.vdim, 64), 16), items8 = ceil_div(H * ceil_div(a.vdim, 64), 8);
      // 16 warps when that leaves a warp at most two accumulator items (128 registers per thread), else 8 warps with up to four
      if (sm <= 220 * 1024 && items8 <= 4) { L.sig_mma = add_sig(h, H, 16 * H); L.mma_items = items16 <= 2 ? -items16 : (items8 <= 2 ? items8 : 4); L.mma_smem = sm; }
    }
  } else if (ret) {
    B200_TRY(h->weights.alloc_t(&L.head_decay, (size_t)H, false));
    B200_CUDA(cudaMemcpy(L.head_decay, L.decay.data(), (size_t)H * sizeof(float), cudaMemcpyHostToDevice));
  } else {
    const int C = 2 * L.Nq + L.Nv, taps = a.conv_taps;
    B200_TRY(h->weights.alloc_t(&L.qkv_conv, (size_t)C * taps, false));
    const Tensor* t = nullptr;
    int off = 0;
    for (const char* nm : {"q", "k", "v"}) {
      const int rows = nm[0] == 'v' ? L.Nv : L.Nq;
      B200_TRY(find_tensor(h, m + nm + ".conv", {rows, taps}, &t));
      B200_TRY(convert_into(t, L.qkv_conv + (size_t)off * taps));
      off += rows;
    }
    h->weight_bytes += (int64_t)C * taps * 4;
    B200_TRY(get_f32(h, m + "A_log", H, &L.A_log));
    B200_TRY(get_f32(h, m + "dt_bias", H, &L.dt_bias));
    B200_TRY(get_f32(h, m + "norm", a.vdim, &L.rnorm));
  }
  void* wo = nullptr;
  B200_TRY(matrix(m + "o", W, (int64_t)H * a.vdim, &wo));
  B200_TRY(seal_weight(h, L.o, wo, (int)W, H * a.vdim, drop, (int)W));
  if (dense) {
    void* wd = nullptr;
    B200_TRY(matrix(p + "mlp.down", W, F, &wd));
    B200_TRY(seal_weight(h, L.down, wd, (int)W, F, drop, (int)W));
  } else if (moe) {
    B200_TRY(get_f32(h, p + "mlp.correction", E, &L.correction));
    B200_TRY(h->weights.alloc(&L.ups, (size_t)E * 2 * F * W * es, false));      // rows 2f / 2f + 1 of an expert: gate f / value f
    B200_TRY(h->weights.alloc(&L.downs, (size_t)E * W * F * es, false));
    void *tg = nullptr, *tu = nullptr;
    B200_CUDA(cudaMalloc(&tg, (size_t)F * W * es));
    B200_CUDA(cudaMalloc(&tu, (size_t)F * W * es));
    int rc = B200_OK;
    for (int64_t e = 0; e < E && rc == B200_OK; ++e) {
      const std::string q = p + "mlp.e" + std::to_string(e) + ".";
      rc = put_matrix(h, q + "gate", F, W, tg);
      if (rc == B200_OK) rc = put_matrix(h, q + "up", F, W, tu);
      if (rc != B200_OK) break;
      char* dst = static_cast<char*>(L.ups) + (size_t)e * 2 * F * W * es;
      const unsigned g = (unsigned)ceil_div64((int64_t)F * W, 256);
      if (h->f32) interleave_rows_kernel<float><<<g, 256>>>(static_cast<const float*>(tg), static_cast<const float*>(tu), reinterpret_cast<float*>(dst), F, W);
      else interleave_rows_kernel<bf16><<<g, 256>>>(static_cast<const bf16*>(tg), static_cast<const bf16*>(tu), reinterpret_cast<bf16*>(dst), F, W);
      rc = check_launch("interleave_rows");
      if (rc == B200_OK) rc = put_matrix(h, q + "down", W, F, static_cast<char*>(L.downs) + (size_t)e * W * F * es);
    }
    cudaDeviceSynchronize();
    cudaFree(tg); cudaFree(tu);
    B200_TRY(rc);
    h->weight_bytes += 3 * (int64_t)E * F * W * es;
  }
  return B200_OK;
}

template <typename T>
int sigmoid_attention(b200_dlm* h, const Layer& L, int n_tok, int max_ctx) {
  const b200_dlm_mixer& a = L.c.a;
  bool mma = false;
  // single tokens on a short history: the CUDA-core kernel on one-token tiles; on a long one the tensor-core kernel wins although 15
  // of its 16 fragment rows are padding (measured at 32 requests x 2048 keys: 0.14 against 0.19 ms per layer)
  if constexpr (sizeof(T) == 2) mma = h->attn_tc && L.sig_mma >= 0 && (h->max_entry_tokens > 1 || h->attn_tc > 1 || max_ctx >= 512);
  const bool one = !mma && h->max_entry_tokens == 1 && L.sig_one >= 0;
  const TileSig& s = h->sigs[mma ? L.sig_mma : one ? L.sig_one : L.sig];
  const int QT = mma ? 16 : one ? 1 : L.QT, KT = mma ? 32 : one ? L.KT_one : L.KT;
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(sigmoid_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    B200_CUDA(cudaFuncSetAttribute((sigmoid_attn_mma_kernel<1, 16>), cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    B200_CUDA(cudaFuncSetAttribute((sigmoid_attn_mma_kernel<2, 16>), cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    B200_CUDA(cudaFuncSetAttribute((sigmoid_attn_mma_kernel<4, 8>), cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set = true;
  }
  SigmoidAttnParams p;
  p.q = h->qkv32; p.ldq = L.Nq; p.kcache = L.kcache; p.vcache = L.vcache; p.mix = L.mixhh; p.bias = L.pbias;
  p.gate_in = h->small32 + L.s_gate; p.ldg = L.nsmall;
  p.tile_row0 = h->meta_dev + s.off_row0; p.tile_rows = h->meta_dev + s.off_rows; p.tile_slot = h->meta_dev + s.off_slot;
  p.tok_pos = h->meta_dev + h->off_pos; p.out = h->obuf; p.part = h->part;
  p.cap = h->cap; p.H = a.heads; p.G = a.kv_heads; p.dim = a.dim; p.vdim = a.vdim; p.QT = QT; p.KT = KT; p.kstride = one ? L.kstride_one : L.kstride;
  p.vec = ((size_t)L.Nk * sizeof(T)) % 16 == 0 && ((size_t)L.Nv * sizeof(T)) % 16 == 0;
  p.softcap = a.softcap;
  // keys are cut over several CTAs per tile when the tiles alone cannot fill the GPU (decoding, short portions)
  const int key_tiles = ceil_div(max_ctx, KT);
  int nsplit = 1;
  if (h->attn_split > 0) nsplit = std::min(h->attn_split, 64);
  else if (mma && h->max_entry_tokens > 1 && s.count < 592) nsplit = ceil_div(592, std::max(s.count, 1));      // prompts: four CTAs per SM in turn even out the causal triangle
  else if (s.count < 148) nsplit = std::min(std::max((one ? 444 : 296) / std::max(s.count, 1), 1), 64);
  nsplit = std::max(1, std::min(nsplit, key_tiles));
  const int rpt = QT * a.heads;
  while (nsplit > 1 && (size_t)s.count * nsplit * rpt * a.vdim > h->part_floats) --nsplit;
  p.nsplit = nsplit;
  if (mma) {
    if constexpr (sizeof(T) == 2) {
      const dim3 grid(s.count, nsplit);
      if (L.mma_items == -1) B200_LAUNCH((sigmoid_attn_mma_kernel<1, 16>), grid, 512, L.mma_smem, h->stream, p);
      else if (L.mma_items == -2) B200_LAUNCH((sigmoid_attn_mma_kernel<2, 16>), grid, 512, L.mma_smem, h->stream, p);
      else B200_LAUNCH((sigmoid_attn_mma_kernel<4, 8>), grid, 256, L.mma_smem, h->stream, p);
    }
  } else {
    B200_LAUNCH(sigmoid_attn_kernel<T>, dim3(s.count, nsplit), 256, one ? L.smem_one : L.attn_smem, h->stream, p);
  }
  B200_TRY(check_launch("sigmoid_attn"));
  if (nsplit > 1) {
    B200_LAUNCH(sigmoid_attn_merge_kernel<T>, dim3(s.count, rpt), 128, 0, h->stream, h->part, p.tile_row0, p.tile_rows, p.gate_in, p.ldg, static_cast<T*>(h->obuf),
                a.heads, a.vdim, nsplit, rpt);
    B200_TRY(check_launch("sigmoid_attn merge"));
  }
  return B200_OK;
}

// routed experts with clamped gates on the rows of hb -> yexp [tokens * top][W]; the router's logits are in small32
template <typename T>
int routed_experts_glu(b200_dlm* h, const Layer& L, const T* hb, int n_tok) {
  const int W = h->cfg.width, E = L.c.experts, top = L.c.top, F = L.c.ff, pairs = n_tok * top;
  cudaStream_t st = h->stream;
  B200_LAUNCH(moe_route_sigmoid_kernel, ceil_div(n_tok, 4), 128, 0, st, h->small32 + L.s_router, (long long)L.nsmall, L.correction, E, top, L.c.router_scale,
              h->moe_idx, h->moe_w, n_tok);
  bool mma = false;
  if constexpr (sizeof(T) == 2) mma = h->attn_tc && W % 16 == 0 && F % 16 == 0;
  const int tile_m = mma ? 128 : 64;
  B200_LAUNCH(moe_group_kernel, 1, 1024, (size_t)2 * E * sizeof(int), st, h->moe_idx, pairs, top, E, h->moe_rank, h->moe_perm, h->moe_row_tok,
              h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, tile_m);
  B200_TRY(check_launch("moe route / group"));
  const int max_tiles = ceil_div(pairs, tile_m) + std::min(E, pairs);
  T* act = static_cast<T*>(h->act);
  T* act2 = static_cast<T*>(h->act2);
  T* yexp = static_cast<T*>(h->yexp);
  const T* ups = static_cast<const T*>(L.ups);
  const T* downs = static_cast<const T*>(L.downs);
  const long long n = (long long)pairs * F;
  if (mma) {
    if constexpr (sizeof(T) == 2) {
      static bool attr_set = false;
      if (!attr_set) {
        B200_CUDA(cudaFuncSetAttribute(grouped_gemm_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GG_SMEM));
        attr_set = true;
      }
      // gate and value rows of an expert are interleaved, so the first product's epilogue holds both of an output in one thread
      B200_LAUNCH(grouped_gemm_mma_kernel, dim3(ceil_div(2 * F, 128), max_tiles), 256, GG_SMEM, st, hb, (long long)W, h->moe_row_tok, ups, (long long)W, (long long)2 * F * W,
                  act, (long long)F, (const int*)nullptr, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, 2 * F, W, 2, L.c.expert_limit);
      B200_LAUNCH(grouped_gemm_mma_kernel, dim3(ceil_div(W, 128), max_tiles), 256, GG_SMEM, st, act, (long long)F, (const int*)nullptr, downs, (long long)F, (long long)W * F,
                  yexp, (long long)W, h->moe_perm, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, W, F, 0, 0.f);
    }
  } else {
    B200_LAUNCH((grouped_gemm_kernel<T, T, T>), dim3(ceil_div(2 * F, 64), max_tiles), 256, 0, st, hb, (long long)W, h->moe_row_tok, ups, (long long)W, (long long)2 * F * W,
                act2, (long long)2 * F, (const int*)nullptr, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, 2 * F, W, 0);
    B200_LAUNCH(clamped_glu_kernel<T>, (unsigned)ceil_div64(n, 256), 256, 0, st, act2, act, F, n, L.c.expert_limit);
    B200_LAUNCH((grouped_gemm_kernel<T, T, T>), dim3(ceil_div(W, 64), max_tiles), 256, 0, st, act, (long long)F, (const int*)nullptr, downs, (long long)F, (long long)W * F,
                yexp, (long long)W, h->moe_perm, h->moe_tile_e, h->moe_tile_r0, h->moe_tile_n, h->moe_ntiles, W, F, 0);
  }
  return check_launch("grouped expert products");
}

template <int R4, bool CHD = false>
int launch_delta_chunk(cudaStream_t st, const DeltaChunkParams& p, int n_entries) {
  constexpr int C = DELTA_CH, DP = 32 * R4;
  const size_t smem = (size_t)((R4 <= 4 ? 2 : 1) * ((CHD ? 3 : 2) * C * DP + C * 32 + 2 * C + 2 * C * C) + 16 * C * 32 + 3 * C * 32 + 2 * C) * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute((delta_chunk_kernel<R4, CHD>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set = true;
  }
  B200_LAUNCH((delta_chunk_kernel<R4, CHD>), dim3(n_entries * p.heads, ceil_div(p.vdim, 32)), 256, smem, st, p);
  return check_launch("delta_chunk");
}

// the delta rule of a step's portions in chunks: the chunks' decay sums and the two triangular matrices side by side, then the
// walk over each request's chunks
int delta_chunks(b200_dlm* h, const ScanParams& sp) {
  DeltaChunkParams p;
  p.prep = sp.prep; p.vprep = sp.vprep; p.gates = sp.tokM; p.prow = sp.prow; p.gram = h->gram;
  p.chunk_tok0 = h->meta_dev + h->off_chunk_tok0; p.chunk_nt = h->meta_dev + h->off_chunk_nt; p.ent_chunk0 = h->meta_dev + h->off_whole_chunk0;
  p.ent_tok0 = h->meta_dev + h->off_whole_tok0; p.ent_ntok = h->meta_dev + h->off_whole_ntok; p.ent_slot = h->meta_dev + h->off_whole_slot;
  p.ent_pos0 = h->meta_dev + h->off_whole_pos0;
  p.St = sp.St; p.out = sp.out; p.heads = sp.heads; p.dim = sp.dim; p.vdim = sp.vdim;
  const size_t gsm = (size_t)(2 * DELTA_CH * (sp.dim + 1) + 2 * DELTA_CH + DELTA_CH * DELTA_CH) * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(delta_gram_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((2 * DELTA_CH * 257 + 2 * DELTA_CH + DELTA_CH * DELTA_CH) * sizeof(float))));
    attr_set = true;
  }
  B200_LAUNCH(delta_gram_kernel, dim3(h->n_chunks, sp.heads), 256, gsm, h->stream, p);
  B200_TRY(check_launch("delta_gram"));
  const int d = sp.dim;
  if (d <= 32) return launch_delta_chunk<1>(h->stream, p, h->n_entries);
  if (d <= 64) return launch_delta_chunk<2>(h->stream, p, h->n_entries);
  if (d <= 128) return launch_delta_chunk<4>(h->stream, p, h->n_entries);
  return launch_delta_chunk<8>(h->stream, p, h->n_entries);
}

// the same for the delta rule with a decay per key channel: the gram kernel also leaves the rows the walk multiplies the state with
int chdelta_chunks(b200_dlm* h, const ScanParams& sp) {
  DeltaChunkParams p;
  p.prep = sp.prep; p.vprep = sp.vprep; p.gates = nullptr; p.prow = sp.prow; p.gram = h->gram; p.rows3 = h->rows3; p.gend = h->gend;
  p.chunk_tok0 = h->meta_dev + h->off_chunk_tok0; p.chunk_nt = h->meta_dev + h->off_chunk_nt; p.ent_chunk0 = h->meta_dev + h->off_whole_chunk0;
  p.ent_tok0 = h->meta_dev + h->off_whole_tok0; p.ent_ntok = h->meta_dev + h->off_whole_ntok; p.ent_slot = h->meta_dev + h->off_whole_slot;
  p.ent_pos0 = h->meta_dev + h->off_whole_pos0;
  p.St = sp.St; p.out = sp.out; p.heads = sp.heads; p.dim = sp.dim; p.vdim = sp.vdim;
  const size_t gsm = (size_t)(3 * DELTA_CH * (sp.dim + 1) + DELTA_CH + DELTA_CH * DELTA_CH) * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA(cudaFuncSetAttribute(chdelta_gram_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((3 * DELTA_CH * 257 + DELTA_CH + DELTA_CH * DELTA_CH) * sizeof(float))));
    attr_set = true;
  }
  B200_LAUNCH(chdelta_gram_kernel, dim3(h->n_chunks, sp.heads), 256, gsm, h->stream, p);
  B200_TRY(check_launch("chdelta_gram"));
  const int d = sp.dim;
  if (d <= 32) return launch_delta_chunk<1, true>(h->stream, p, h->n_entries);
  if (d <= 64) return launch_delta_chunk<2, true>(h->stream, p, h->n_entries);
  if (d <= 128) return launch_delta_chunk<4, true>(h->stream, p, h->n_entries);
  return launch_delta_chunk<8, true>(h->stream, p, h->n_entries);
}

template <typename T>
int step_parallel(b200_dlm* h, int n_tok, int n_want, int max_ctx, float* logits_out) {
  const b200_dlm_config& c = h->cfg;
  const int W = c.width;
  cudaStream_t st = h->stream;
  const int* meta = h->meta_dev;
  const int *tok_slot = meta + h->off_slot, *tok_pos = meta + h->off_pos, *tok_first = meta + h->off_first, *tok_last = meta + h->off_last;
  const long long stride = (long long)h->tmax * W;
  T* hb = static_cast<T*>(h->hbuf);
  T* proj = static_cast<T*>(h->proj);
  T* ob = static_cast<T*>(h->obuf);
  T* mixo = static_cast<T*>(h->mixo);
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(embed_scale_norm_kernel<T>, n_tok, 256, 0, st, meta + h->off_tok, static_cast<const T*>(h->embed), c.vocab, W, c.embedding_scale,
                                     h->layers[0].n1w, h->xin, hb, c.norm_eps, h->err));
  for (int li = 0; li < c.n_layers; ++li) {
    const Layer& L = h->layers[li];
    const b200_dlm_mixer& a = L.c.a;
    const bool last = li + 1 == c.n_layers;
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, hb, W, L.cat, proj, L.ldp, n_tok)));
    if (L.nsmall) TIMED(CLS_FOLD, B200_TRY(small_proj<T>(h, hb, W, L.w_small, nullptr, h->small32, n_tok, L.nsmall, W)));
    const int Rv = a.heads * a.vdim;
    if (L.c.mixer == B200_MIXER_SIGMOID_ATTENTION) {
      const bool blend = a.v_mix && li != h->vmix_first, keep = a.v_mix && li == h->vmix_first;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(attn_rope_cache_kernel<T>, n_tok, 256, (size_t)a.rot_dims * 4 + 4, st, proj, (long long)L.ldp, L.p_q, L.p_k, L.p_v, L.Nq, L.Nk, L.Nv,
                                         a.dim, a.rot_dims / 2, a.rot_pairing == B200_ROT_ADJACENT, L.freq, L.rot_amp, a.scale, h->qkv32, static_cast<T*>(L.kcache),
                                         static_cast<T*>(L.vcache), h->cap, tok_slot, tok_pos, blend ? static_cast<const T*>(h->vfirst) : (const T*)nullptr, L.vlambda,
                                         keep ? static_cast<T*>(h->vfirst) : (T*)nullptr));
      TIMED(CLS_ATTN, B200_TRY(sigmoid_attention<T>(h, L, n_tok, max_ctx)));
    } else {
      ScanParams sp;
      sp.proj = proj; sp.ld = L.ldp; sp.off_q = L.p_q; sp.off_k = L.p_k; sp.off_v = L.p_v; sp.z = nullptr; sp.zb = nullptr;
      sp.inv_tau = 0.f; sp.cap = 0.f; sp.St = L.St; sp.nvec = nullptr; sp.mval = nullptr;
      sp.out = h->scan32; sp.heads = a.heads; sp.dim = a.dim; sp.vdim = a.vdim;
      const long long rows = (long long)n_tok * a.heads;
      if (L.c.mixer == B200_MIXER_RETENTION) {
        sp.qscale = 1.f; sp.kscale = 1.f / sqrtf((float)a.dim); sp.head_decay = L.head_decay;
        sp.freq = L.freq; sp.tok_pos = tok_pos; sp.rot_half = a.rot_dims / 2; sp.rot_adjacent = a.rot_pairing == B200_ROT_ADJACENT; sp.rot_amp = L.rot_amp;
        TIMED(CLS_RECURRENT, B200_TRY((launch_scan<T, MODE_DECAY>(h, sp, n_tok))));
        TIMED(CLS_ELEMENTWISE, B200_LAUNCH(head_norm_gate_kernel<T>, (unsigned)ceil_div64(rows, 4), 128, 0, st, h->scan32, (const float*)nullptr, 0, proj, (long long)L.ldp, L.p_g, 1, ob,
                                           a.heads, a.vdim, rows, c.norm_eps));
      } else {
        const int C = 2 * L.Nq + L.Nv;
        TIMED(CLS_ELEMENTWISE, B200_LAUNCH((causal_conv_kernel<T, float>), n_tok, 256, 0, st, proj, (long long)L.ldp, L.qkv_hist, L.qkv_conv, h->qkv32, (long long)C, C,
                                           a.conv_taps, 0, tok_slot, tok_pos, tok_first);
              if (a.conv_taps > 1) B200_LAUNCH(conv_carry_kernel<T>, n_tok, 256, 0, st, proj, (long long)L.ldp, L.qkv_hist, C, a.conv_taps - 1, tok_slot, tok_pos, tok_last));
        sp.qscale = 1.f / sqrtf((float)a.dim); sp.z = h->small32 + L.s_ba;
        const ScanLayout lay = scan_layout<MODE_DELTA>(h, sp, true);
        const bool chunked = h->delta_chunk && h->max_entry_tokens >= 16 && h->gram != nullptr;      // prompts: chunks of tokens at once; single tokens: the scan
        if (chunked) { sp.lpc = 0; sp.rows = 0; sp.prow = (2 * a.dim + 2 + 3) / 4 * 4; }            // plain rows
        TIMED(CLS_RECURRENT, B200_LAUNCH(delta_prep_kernel, n_tok, 256, (size_t)2 * a.kv_heads * sizeof(float), st, sp, h->qkv32, a.kv_heads, L.A_log, L.dt_bias, (long long)L.nsmall);
              B200_TRY(check_launch("delta_prep"));
              if (chunked) B200_TRY(delta_chunks(h, sp)); else B200_TRY(scan_run<MODE_DELTA>(h, sp, lay, true)));
        TIMED(CLS_ELEMENTWISE, B200_LAUNCH(head_norm_gate_kernel<T>, (unsigned)ceil_div64(rows, 4), 128, 0, st, h->scan32, L.rnorm, 0, proj, (long long)L.ldp, L.p_g, 1, ob,
                                           a.heads, a.vdim, rows, c.norm_eps));
      }
    }
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob, (long long)Rv, L.o, mixo, W, n_tok)));
    const T *ffo = nullptr, *yexp = nullptr;
    if (L.c.mlp == B200_MLP_DENSE_GATED_GELU) {
      T* act = static_cast<T*>(h->act);
      const long long n = (long long)n_tok * L.c.ff;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(gated_gelu_kernel<T>, (unsigned)ceil_div64(n, 256), 256, 0, st, proj, (long long)L.ldp, L.p_ffg, L.p_ffu, act, L.c.ff, n));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, act, L.c.ff, L.down, static_cast<T*>(h->ffo), W, n_tok)));
      ffo = static_cast<const T*>(h->ffo);
    } else if (L.c.mlp == B200_MLP_MOE_CLAMPED_GLU) {
      TIMED(CLS_EXPERTS, B200_TRY(routed_experts_glu<T>(h, L, hb, n_tok)));
      yexp = static_cast<const T*>(h->yexp);
    }
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(parallel_block_end_kernel<T>, n_tok, 256, 0, st, h->xin, mixo, ffo, yexp, h->moe_w, L.c.top,
                                       h->trace_layers ? h->trace + (long long)li * stride : nullptr, last ? nullptr : h->layers[li + 1].n1w, hb, W, c.norm_eps));
  }
  B200_TRY(check_launch("decoder LM layers"));
  if (n_want > 0) {
    T* hf = static_cast<T*>(h->hf);
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(rmsnorm_rows_kernel<T>, n_want, 256, 0, st, h->xin, meta + h->off_want, h->fnw, hf, W, c.norm_eps));
    if (h->head.tiles) {
      const int ldl = (c.vocab + 7) / 8 * 8;
      TIMED(CLS_LINEAR, B200_TRY(linear<bf16>(h, reinterpret_cast<const bf16*>(hf), W, h->head, h->head_bf, ldl, n_want)));
      const long long n = (long long)n_want * c.vocab;
      B200_LAUNCH(rows_to_f32_kernel, (unsigned)ceil_div64(n, 256), 256, 0, st, h->head_bf, (long long)ldl, h->logits, c.vocab, n);
    } else {
      TIMED(CLS_LINEAR, B200_TRY(gemm_nt(st, hf, (long long)W, 0, static_cast<const T*>(h->head.rm), (long long)W, 0, h->logits, (long long)c.vocab, 0, n_want, c.vocab, W, 1, 1.f)));
    }
    if (logits_out)
      B200_CUDA(cudaMemcpyAsync(logits_out, h->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToDevice, st));
  }
  return check_launch("decoder LM step");
}


// ---------------------------------------------------------------------------------------------------------------------------
// Pre-norm sublayers on residual streams: u = sum_s in[s] x_s;  y = f(rms(u) * w);  x_t <- sum_s mix[s][t] x_s + out[t] y
// ---------------------------------------------------------------------------------------------------------------------------

int finalize_streams_layer(b200_dlm* h, int i, std::vector<void*>& drop) {
  Layer& L = h->layers[i];
  const b200_dlm_config& c = h->cfg;
  const b200_dlm_mixer &a = L.c.a, &b = L.c.b;
  const int64_t W = c.width;
  const size_t es = esize(h);
  const std::string p = "l" + std::to_string(i) + ".", m = p + "mix.";
  const bool mlp = L.c.mlp != B200_MLP_NONE;
  auto matrix = [&](const std::string& name, int64_t rows, int64_t K, void** out) -> int {
    B200_TRY(h->weights.alloc(out, (size_t)rows * K * es, false));
    return put_matrix(h, name, rows, K, *out);
  };
  auto sealed = [&](const std::string& name, int64_t rows, int64_t K, Weight& w, int ld_out) -> int {
    void* rm = nullptr;
    B200_TRY(matrix(name, rows, K, &rm));
    return seal_weight(h, w, rm, (int)rows, (int)K, drop, ld_out);
  };
  B200_TRY(get_f32(h, p + "norm1", W, &L.n1w));
  if (mlp) B200_TRY(get_f32(h, p + "norm2", W, &L.n2w));
  for (int q = 0; q < (mlp ? 2 : 1) && c.streams > 0; ++q) {
    const std::string hc = p + "hc" + std::to_string(q + 1) + ".";
    B200_TRY(get_f32(h, hc + "in", c.streams, &L.hc_in[q]));
    B200_TRY(get_f32(h, hc + "out", c.streams, &L.hc_out[q]));
    B200_TRY(get_f32_shaped(h, hc + "mix", {c.streams, c.streams}, &L.hc_mix[q]));
  }
  void* cat = nullptr;
  auto at = [&](int off) { return static_cast<char*>(cat) + (size_t)off * W * es; };
  auto pad8 = [](int v) { return (v + 7) / 8 * 8; };
  auto frequencies = [&](const b200_dlm_mixer& mx) -> int {
    if (mx.rot_dims <= 0) return B200_OK;
    std::vector<double> fr;
    if (mx.rot_scaling == B200_ROT_RAMP) fr = rotary_frequencies_ramp(mx, &L.rot_amp);
    else fr = rotary_frequencies(mx);
    B200_TRY(h->weights.alloc_t(&L.freq, fr.size(), false));
    B200_CUDA(cudaMemcpy(L.freq, fr.data(), fr.size() * sizeof(double), cudaMemcpyHostToDevice));
    return B200_OK;
  };
  if (L.c.mixer == B200_MIXER_LATENT_ATTENTION) {
    const int64_t H = a.heads, dq = a.dim + a.rot_dims, r = a.kv_rank, rd = a.rot_dims;
    L.Nq = (int)(H * dq);
    L.off_q = 0; L.off_dkv = pad8(L.Nq); L.ncat = L.off_dkv + (int)(r + rd);
    L.ldp = pad8(L.ncat);
    L.rp = pad8((int)(r + rd));
    {   // bf16: rows padded to a multiple of 64 take the tensor-core kernel, when that costs at most a third more cache
      const int rp64 = (int)(r + rd + 63) / 64 * 64;
      if (!h->f32 && h->use_tc && rp64 <= 576 && (int64_t)rp64 * 3 <= (r + rd) * 4) L.rp = rp64;
    }
    B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, true));
    B200_TRY(put_matrix(h, m + "q", H * dq, W, at(L.off_q)));
    B200_TRY(put_matrix(h, m + "dkv", r + rd, W, at(L.off_dkv)));
    B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
    B200_TRY(get_f32(h, m + "dkv.norm", r, &L.cnorm));
    if (a.head_gate) {
      L.nsmall = (int)H; L.s_gate = 0;
      B200_TRY(matrix(m + "g", H, W, &L.w_small));
      h->weight_bytes += H * W * es;
    }
    if (a.sink == B200_SINK_LEARNED) B200_TRY(get_f32(h, m + "sink", H, &L.sink));
    else if (a.sink == B200_SINK_UNIT) B200_TRY(h->weights.alloc_t(&L.sink, (size_t)H, true));
    {   // W_uk [H * dim][r] -> per head [r][dim]
      void* uk = nullptr;
      B200_TRY(matrix(m + "uk", H * a.dim, r, &uk));
      B200_TRY(h->weights.alloc(&L.ukT, (size_t)H * a.dim * r * es, false));
      const long long n = H * a.dim * r;
      if (h->f32) B200_LAUNCH(head_transpose_kernel<float>, (unsigned)ceil_div64(n, 256), 256, 0, nullptr, static_cast<const float*>(uk), static_cast<float*>(L.ukT), (int)H, a.dim, (int)r);
      else B200_LAUNCH(head_transpose_kernel<bf16>, (unsigned)ceil_div64(n, 256), 256, 0, nullptr, static_cast<const bf16*>(uk), static_cast<bf16*>(L.ukT), (int)H, a.dim, (int)r);
      B200_TRY(check_launch("head_transpose"));
      drop.push_back(uk);
      h->weight_bytes += n * es;
    }
    B200_TRY(matrix(m + "uv", H * a.vdim, r, &L.uv));
    h->weight_bytes += H * a.vdim * r * es;
    B200_TRY(sealed(m + "o", W, H * a.vdim, L.o, (int)W));
    B200_TRY(frequencies(a));
    L.sig = add_sig(h, (int)H, rows_per_tile(L.rp));
  } else if (L.c.mixer == B200_MIXER_PARALLEL) {
    const std::string l = m + "left.", r = m + "right.";
    const int N = b.dim;
    L.Nq = a.heads * a.dim; L.Nk = a.kv_heads * a.dim; L.Nv = a.kv_heads * a.vdim;
    L.p_q = 0; L.p_k = L.Nq; L.p_v = L.p_k + L.Nk; L.g_z = L.p_v + L.Nv; L.g_x = L.g_z + N; L.g_g = L.g_x + N; L.ncat = L.g_g + N;
    L.ldp = pad8(L.ncat);
    B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, false));
    B200_TRY(put_matrix(h, l + "q", L.Nq, W, at(L.p_q)));
    B200_TRY(put_matrix(h, l + "k", L.Nk, W, at(L.p_k)));
    B200_TRY(put_matrix(h, l + "v", L.Nv, W, at(L.p_v)));
    B200_TRY(put_matrix(h, r + "z", N, W, at(L.g_z)));
    B200_TRY(put_matrix(h, r + "x", N, W, at(L.g_x)));
    B200_TRY(put_matrix(h, r + "g", N, W, at(L.g_g)));
    B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
    if (a.bias) {
      const int C = L.Nq + L.Nk + L.Nv;
      B200_TRY(h->weights.alloc_t(&L.qkv_bias, (size_t)C, false));
      const Tensor* t = nullptr;
      int off = 0;
      for (const char* nm : {"q", "k", "v"}) {
        const int rows = nm[0] == 'q' ? L.Nq : nm[0] == 'k' ? L.Nk : L.Nv;
        B200_TRY(find_tensor(h, l + nm + ".b", {rows}, &t));
        B200_TRY(convert_into(t, L.qkv_bias + off));
        off += rows;
      }
      h->weight_bytes += (int64_t)C * 4;
    }
    if (b.bias) {
      B200_TRY(h->weights.alloc_t(&L.zx_bias, (size_t)2 * N, false));
      const Tensor* t = nullptr;
      B200_TRY(find_tensor(h, r + "z.b", {N}, &t));
      B200_TRY(convert_into(t, L.zx_bias));
      B200_TRY(find_tensor(h, r + "x.b", {N}, &t));
      B200_TRY(convert_into(t, L.zx_bias + N));
      h->weight_bytes += (int64_t)2 * N * 4;
    }
    // the score scale goes into the rotated queries; the head mix of the kernel is the identity
    B200_TRY(h->weights.alloc_t(&L.mixhh, (size_t)a.heads * a.heads, false));
    B200_LAUNCH(identity_kernel, ceil_div(a.heads * a.heads, 256), 256, 0, nullptr, L.mixhh, a.heads);
    B200_TRY(check_launch("identity"));
    if (a.sink == B200_SINK_LEARNED) B200_TRY(get_f32(h, l + "sink", a.heads, &L.sink));
    else B200_TRY(h->weights.alloc_t(&L.sink, (size_t)a.heads, true));      // a unit in the denominator = a sink of logit 0
    B200_TRY(frequencies(a));
    B200_TRY(sealed(l + "o", W, (int64_t)a.heads * a.vdim, L.a_o, (int)W));
    B200_TRY(sealed(r + "o", W, N, L.r_o, (int)W));
    B200_TRY(plan_window_attention(h, L, i));
  } else {      // B200_MIXER_CHANNEL_DELTA
    const int H = a.heads, G = a.kv_heads, taps = a.conv_taps;
    L.Nq = G * a.dim; L.Nk = G * a.dim; L.Nv = H * a.vdim;
    const int Nd = H * a.dim;
    const Tensor *a1 = h->store.find(m + "a1"), *g1 = h->store.find(m + "g1");
    if (!a1 || a1->shape.size() != 2 || a1->shape[1] != W || !g1 || g1->shape.size() != 2 || g1->shape[1] != W)
      B200_FAIL(B200_ERR_MISSING, "decoder LM finalize: tensors '%sa1' / '%sg1' [rank, width] were not loaded", m.c_str(), m.c_str());
    L.decay_rank = (int)a1->shape[0]; L.gate_rank = (int)g1->shape[0];
    L.p_q = 0; L.p_k = L.Nq; L.p_v = L.p_k + L.Nk; L.c_a1 = pad8(L.p_v + L.Nv); L.c_g1 = pad8(L.c_a1 + L.decay_rank); L.ncat = L.c_g1 + L.gate_rank;
    L.ldp = pad8(L.ncat);
    B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, true));
    B200_TRY(put_matrix(h, m + "q", L.Nq, W, at(L.p_q)));
    B200_TRY(put_matrix(h, m + "k", L.Nk, W, at(L.p_k)));
    B200_TRY(put_matrix(h, m + "v", L.Nv, W, at(L.p_v)));
    B200_TRY(put_matrix(h, m + "a1", L.decay_rank, W, at(L.c_a1)));
    B200_TRY(put_matrix(h, m + "g1", L.gate_rank, W, at(L.c_g1)));
    B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
    L.nsmall = H; L.s_ba = 0;
    B200_TRY(matrix(m + "b", H, W, &L.w_small));
    h->weight_bytes += (int64_t)H * W * es;
    B200_TRY(matrix(m + "a2", Nd, L.decay_rank, &L.a2));
    B200_TRY(matrix(m + "g2", L.Nv, L.gate_rank, &L.g2));
    h->weight_bytes += ((int64_t)Nd * L.decay_rank + (int64_t)L.Nv * L.gate_rank) * es;
    const int C = 2 * L.Nq + L.Nv;
    B200_TRY(h->weights.alloc_t(&L.qkv_conv, (size_t)C * taps, false));
    const Tensor* t = nullptr;
    int off = 0;
    for (const char* nm : {"q", "k", "v"}) {
      const int rows = nm[0] == 'v' ? L.Nv : L.Nq;
      B200_TRY(find_tensor(h, m + nm + ".conv", {rows, taps}, &t));
      B200_TRY(convert_into(t, L.qkv_conv + (size_t)off * taps));
      off += rows;
    }
    h->weight_bytes += (int64_t)C * taps * 4;
    B200_TRY(get_f32(h, m + "A_log", H, &L.A_log));
    B200_TRY(get_f32(h, m + "dt_bias", Nd, &L.dt_bias));
    B200_TRY(get_f32(h, m + "norm", a.vdim, &L.rnorm));
    B200_TRY(sealed(m + "o", W, L.Nv, L.o, (int)W));
  }
  if (mlp) {
    B200_TRY(sealed(p + "mlp.up", L.c.ff, W, L.up, L.c.ff));
    B200_TRY(sealed(p + "mlp.down", W, L.c.ff, L.down, (int)W));
  }
  return B200_OK;
}

// the end of a sublayer for any number of streams (a plain residual counts as one stream without weights)
template <typename T>
int streams_end(b200_dlm* h, const T* y0, float s0, const T* y1, float s1, const float* mix, const float* out, float* trace, float* xsum,
                const float* in_next, const float* w_next, int n_tok) {
  const int W = h->cfg.width, S = std::max(h->cfg.streams, 1);
  const size_t sm = (size_t)W * 4;
  T* hb = static_cast<T*>(h->hbuf);
#define B200_STREAMS_CASE(N) case N: B200_LAUNCH((streams_end_kernel<T, N>), n_tok, 256, sm, h->stream, h->xs, y0, s0, y1, s1, mix, out, trace, xsum, in_next, w_next, hb, W, h->cfg.norm_eps); break;
  switch (S) {
    B200_STREAMS_CASE(1) B200_STREAMS_CASE(2) B200_STREAMS_CASE(3) B200_STREAMS_CASE(4) B200_STREAMS_CASE(5) B200_STREAMS_CASE(6) B200_STREAMS_CASE(7)
    default: B200_LAUNCH((streams_end_kernel<T, 8>), n_tok, 256, sm, h->stream, h->xs, y0, s0, y1, s1, mix, out, trace, xsum, in_next, w_next, hb, W, h->cfg.norm_eps);
  }
#undef B200_STREAMS_CASE
  return check_launch("streams_end");
}

// latent attention over cache rows [latent | rotated key part]: the queries' first r elements are folded through W_uk, the rest
// are the rotated query part; the sums over the rows' first r elements go through W_uv
template <typename T>
int latent_rope_attention(b200_dlm* h, const Layer& L, int n_tok, int max_ctx) {
  const b200_dlm_mixer& a = L.c.a;
  const int H = a.heads, dk = a.dim, dv = a.vdim, r = a.kv_rank, rd = a.rot_dims, rp = L.rp;
  cudaStream_t st = h->stream;
  const int* meta = h->meta_dev;
  T* proj = static_cast<T*>(h->proj);
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(latent_rope_append_kernel<T>, n_tok, 128, (size_t)rd * 4 + 4, st, proj, (long long)L.ldp, L.off_q, L.off_dkv, L.cnorm,
                                     static_cast<T*>(L.cache), h->cap, r, rd, rp, H, dk, a.rot_pairing == B200_ROT_ADJACENT, L.freq, L.rot_amp, a.scale, h->qa,
                                     meta + h->off_slot, meta + h->off_pos, h->cfg.norm_eps));
  TIMED(CLS_FOLD, B200_TRY(head_gemm(st, proj + L.off_q, (long long)L.ldp, (long long)(dk + rd), static_cast<const T*>(L.ukT), (long long)dk, (long long)r * dk, h->qa,
                                     (long long)H * rp, (long long)rp, n_tok, r, dk, H, a.scale, h->attn_tc != 0)));
  const TileSig& s = h->sigs[L.sig];
  AttnParams p;
  p.qa = h->qa; p.cache = L.cache; p.sink = a.sink == B200_SINK_NONE ? nullptr : L.sink;
  p.tile_row0 = meta + s.off_row0; p.tile_rows = meta + s.off_rows; p.tile_slot = meta + s.off_slot;
  p.tok_pos = meta + h->off_pos;
  p.out = h->ol; p.part = h->part; p.cap = h->cap; p.r = rp; p.H = H; p.err = h->err;
  p.window = a.window;
  if (a.head_gate) { p.gate = h->small32 + L.s_gate; p.ldg = L.nsmall; }
  const int seen = a.window > 0 ? std::min(max_ctx, a.window + 32) : max_ctx;
  p.nsplit = pick_split(h->attn_split, s.count, seen, s.rpt, rp, h->part_floats);
  TIMED(CLS_ATTN, B200_TRY(run_attention<T>(st, p, s.count, s.rpt, h->attn_tc != 0)));
  T* ob = static_cast<T*>(h->obuf);
  TIMED(CLS_FOLD, B200_TRY(head_gemm(st, h->ol, (long long)H * rp, (long long)rp, static_cast<const T*>(L.uv), (long long)r, (long long)dv * r, ob, (long long)H * dv,
                                     (long long)dv, n_tok, dv, r, H, 1.f, h->attn_tc != 0)));
  return B200_OK;
}

template <typename T>
int step_streams(b200_dlm* h, int n_tok, int n_want, int max_ctx, float* logits_out) {
  const b200_dlm_config& c = h->cfg;
  const int W = c.width, S = std::max(c.streams, 1);
  cudaStream_t st = h->stream;
  const int* meta = h->meta_dev;
  const int *tok_slot = meta + h->off_slot, *tok_pos = meta + h->off_pos, *tok_first = meta + h->off_first, *tok_last = meta + h->off_last;
  const long long stride = (long long)h->tmax * W;
  T* hb = static_cast<T*>(h->hbuf);
  T* proj = static_cast<T*>(h->proj);
  T* ob = static_cast<T*>(h->obuf);
  T* ob2 = static_cast<T*>(h->obuf2);
  T* mixo = static_cast<T*>(h->mixo);
  T* mixo2 = static_cast<T*>(h->mixo2);
  TIMED(CLS_ELEMENTWISE, B200_LAUNCH(embed_streams_kernel<T>, n_tok, 256, (size_t)W * 4, st, meta + h->off_tok, static_cast<const T*>(h->embed), c.vocab, W, S,
                                     h->layers[0].hc_in[0], h->layers[0].n1w, h->xs, hb, c.norm_eps, h->err));
  for (int li = 0; li < c.n_layers; ++li) {
    const Layer& L = h->layers[li];
    const b200_dlm_mixer &a = L.c.a, &b = L.c.b;
    const bool last = li + 1 == c.n_layers, mlp = L.c.mlp != B200_MLP_NONE;
    TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, hb, W, L.cat, proj, L.ldp, n_tok)));
    if (L.nsmall) TIMED(CLS_FOLD, B200_TRY(small_proj<T>(h, hb, W, L.w_small, nullptr, h->small32, n_tok, L.nsmall, W)));
    const T* y1 = nullptr;
    float s0 = 1.f, s1 = 0.f;
    if (L.c.mixer == B200_MIXER_LATENT_ATTENTION) {
      B200_TRY(latent_rope_attention<T>(h, L, n_tok, max_ctx));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob, (long long)a.heads * a.vdim, L.o, mixo, W, n_tok)));
    } else if (L.c.mixer == B200_MIXER_PARALLEL) {
      // left: bias, rotation and score scale on the queries (fp32), keys and values into the cache, then the window attention
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(attn_rope_cache_kernel<T>, n_tok, 256, (size_t)a.rot_dims * 4 + 4, st, proj, (long long)L.ldp, L.p_q, L.p_k, L.p_v, L.Nq, L.Nk, L.Nv,
                                         a.dim, a.rot_dims / 2, a.rot_pairing == B200_ROT_ADJACENT, L.freq, L.rot_amp, a.scale, h->qkv32, static_cast<T*>(L.kcache),
                                         static_cast<T*>(L.vcache), h->cap, tok_slot, tok_pos, (const T*)nullptr, (const float*)nullptr, (T*)nullptr, L.qkv_bias));
      TIMED(CLS_ATTN, B200_TRY(window_attention<T>(h, L, n_tok, max_ctx, L.Nq)));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob, (long long)a.heads * a.vdim, L.a_o, mixo, W, n_tok)));
      // right: the minGRU
      const int N = b.dim;
      const int nw = std::min(32, std::max(1, ceil_div(h->max_entry_tokens, 8)));      // warps per CTA: segments of at least 8 tokens
      TIMED(CLS_RECURRENT, B200_LAUNCH(mingru_kernel<T>, dim3(ceil_div(N, 32), h->n_entries), dim3(32, nw), 0, st, proj, (long long)L.ldp, L.g_z, L.g_x, L.g_g, L.zx_bias,
                                       L.zx_bias ? L.zx_bias + N : nullptr, L.gru, ob2, (long long)N, N, meta + h->off_whole_tok0, meta + h->off_whole_ntok,
                                       meta + h->off_whole_slot, meta + h->off_whole_pos0));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob2, (long long)N, L.r_o, mixo2, W, n_tok)));
      y1 = mixo2; s0 = L.c.a_scale; s1 = L.c.b_scale;
    } else {
      const int C = 2 * L.Nq + L.Nv, Nd = a.heads * a.dim;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH((causal_conv_kernel<T, float>), n_tok, 256, 0, st, proj, (long long)L.ldp, L.qkv_hist, L.qkv_conv, h->qkv32, (long long)C, C,
                                         a.conv_taps, 0, tok_slot, tok_pos, tok_first);
            if (a.conv_taps > 1) B200_LAUNCH(conv_carry_kernel<T>, n_tok, 256, 0, st, proj, (long long)L.ldp, L.qkv_hist, C, a.conv_taps - 1, tok_slot, tok_pos, tok_last));
      // decay and gate pre-activations through their bottlenecks, fp32 out
      TIMED(CLS_FOLD, B200_TRY(head_gemm(st, proj + L.c_a1, (long long)L.ldp, 0, static_cast<const T*>(L.a2), (long long)L.decay_rank, 0, h->gate32, (long long)Nd, 0,
                                         n_tok, Nd, L.decay_rank, 1, 1.f, h->attn_tc != 0));
            B200_TRY(head_gemm(st, proj + L.c_g1, (long long)L.ldp, 0, static_cast<const T*>(L.g2), (long long)L.gate_rank, 0, h->attn32, (long long)L.Nv, 0,
                               n_tok, L.Nv, L.gate_rank, 1, 1.f, h->attn_tc != 0)));
      ScanParams sp;
      sp.proj = proj; sp.ld = L.ldp; sp.off_q = L.p_q; sp.off_k = L.p_k; sp.off_v = L.p_v; sp.z = nullptr; sp.zb = nullptr;
      sp.inv_tau = 0.f; sp.cap = 0.f; sp.St = L.St; sp.nvec = nullptr; sp.mval = nullptr;
      sp.out = h->scan32; sp.heads = a.heads; sp.dim = a.dim; sp.vdim = a.vdim;
      sp.qscale = 1.f / sqrtf((float)a.dim);
      const ScanLayout lay = scan_layout<MODE_CHDELTA>(h, sp, true);
      const bool chunked = h->delta_chunk && h->max_entry_tokens >= 16 && h->gram != nullptr;      // prompts: chunks of tokens at once; single tokens: the scan
      if (chunked) { sp.lpc = 0; sp.rows = 0; sp.prow = (3 * a.dim + 2 + 3) / 4 * 4; }            // plain rows, the decays as logarithms
      TIMED(CLS_RECURRENT, B200_LAUNCH(chdelta_prep_kernel, n_tok, 256, (size_t)2 * a.kv_heads * sizeof(float), st, sp, h->qkv32, a.kv_heads, L.A_log, L.dt_bias, h->gate32,
                                       h->small32 + L.s_ba, (long long)L.nsmall, chunked ? 1 : 0);
            B200_TRY(check_launch("chdelta_prep"));
            if (chunked) B200_TRY(chdelta_chunks(h, sp)); else B200_TRY(scan_run<MODE_CHDELTA>(h, sp, lay, true)));
      const long long rows = (long long)n_tok * a.heads;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH((head_norm_gate_kernel<T, float>), (unsigned)ceil_div64(rows, 4), 128, 0, st, h->scan32, L.rnorm, 0, h->attn32, (long long)L.Nv, 0, 0, ob,
                                         a.heads, a.vdim, rows, c.norm_eps));
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, ob, (long long)L.Nv, L.o, mixo, W, n_tok)));
    }
    const Layer* nx = last ? nullptr : &h->layers[li + 1];
    float* trace = h->trace_layers ? h->trace + (long long)li * stride : nullptr;
    if (mlp) {
      TIMED(CLS_ELEMENTWISE, B200_TRY(streams_end<T>(h, mixo, s0, y1, s1, L.hc_mix[0], L.hc_out[0], nullptr, nullptr, L.hc_in[1], L.n2w, n_tok)));
      T* act = static_cast<T*>(h->act);
      T* upb = static_cast<T*>(h->act2);
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, hb, W, L.up, upb, L.c.ff, n_tok)));
      const long long n = (long long)n_tok * L.c.ff;
      TIMED(CLS_ELEMENTWISE, B200_LAUNCH(relu2_kernel<T>, (unsigned)ceil_div64(n, 256), 256, 0, st, upb, (long long)L.c.ff, 0, act, L.c.ff, n));
      T* ffo = static_cast<T*>(h->ffo);
      TIMED(CLS_LINEAR, B200_TRY(linear<T>(h, act, L.c.ff, L.down, ffo, W, n_tok)));
      TIMED(CLS_ELEMENTWISE, B200_TRY(streams_end<T>(h, ffo, 1.f, (const T*)nullptr, 0.f, L.hc_mix[1], L.hc_out[1], trace, last ? h->xin : nullptr, nx ? nx->hc_in[0] : nullptr,
                                                     nx ? nx->n1w : nullptr, n_tok)));
    } else {
      TIMED(CLS_ELEMENTWISE, B200_TRY(streams_end<T>(h, mixo, s0, y1, s1, L.hc_mix[0], L.hc_out[0], trace, last ? h->xin : nullptr, nx ? nx->hc_in[0] : nullptr,
                                                     nx ? nx->n1w : nullptr, n_tok)));
    }
  }
  B200_TRY(check_launch("decoder LM layers"));
  if (n_want > 0) {
    T* hf = static_cast<T*>(h->hf);
    TIMED(CLS_ELEMENTWISE, B200_LAUNCH(rmsnorm_rows_kernel<T>, n_want, 256, 0, st, h->xin, meta + h->off_want, h->fnw, hf, W, c.norm_eps));
    const long long n = (long long)n_want * c.vocab;
    if (h->head.tiles) {
      const int ldl = (c.vocab + 7) / 8 * 8;
      TIMED(CLS_LINEAR, B200_TRY(linear<bf16>(h, reinterpret_cast<const bf16*>(hf), W, h->head, h->head_bf, ldl, n_want)));
      B200_LAUNCH(scale_rows_kernel, (unsigned)ceil_div64(n, 256), 256, 0, st, h->head_bf, (long long)ldl, h->logits, c.vocab, n, c.logit_scale);
    } else {
      TIMED(CLS_LINEAR, B200_TRY(gemm_nt(st, hf, (long long)W, 0, static_cast<const T*>(h->head.rm), (long long)W, 0, h->logits, (long long)c.vocab, 0, n_want, c.vocab, W, 1, c.logit_scale)));
    }
    if (logits_out)
      B200_CUDA(cudaMemcpyAsync(logits_out, h->logits, (size_t)n_want * c.vocab * 4, cudaMemcpyDeviceToDevice, st));
  }
  return check_launch("decoder LM step");
}

}  // namespace

extern "C" {

int b200_dlm_create(const b200_dlm_config* cfg, b200_dlm** out) {
  if (!cfg || !out || !cfg->layers) B200_FAIL(B200_ERR_INVALID, "dlm_create: null argument");
  if (cfg->vocab < 1 || cfg->width < 1 || cfg->n_layers < 1) B200_FAIL(B200_ERR_INVALID, "dlm_create: vocab, width and n_layers must be positive");
  if (cfg->compute_dtype != B200_BF16 && cfg->compute_dtype != B200_F32) B200_FAIL(B200_ERR_INVALID, "dlm_create: compute_dtype must be bf16 or f32");
  if (cfg->block != B200_BLOCK_GATED_DEPTH_AVERAGE && cfg->block != B200_BLOCK_SANDWICH && cfg->block != B200_BLOCK_PARALLEL_RESIDUAL &&
      cfg->block != B200_BLOCK_PRE_NORM_STREAMS)
    B200_FAIL(B200_ERR_INVALID, "dlm_create: unknown block arrangement %d", cfg->block);
  if (cfg->block == B200_BLOCK_PRE_NORM_STREAMS && (cfg->streams < 0 || cfg->streams > B200_DLM_MAX_STREAMS))
    B200_FAIL(B200_ERR_INVALID, "dlm_create: streams must be in 0..%d", B200_DLM_MAX_STREAMS);
  if (cfg->tied_head && cfg->block != B200_BLOCK_PRE_NORM_STREAMS) B200_FAIL(B200_ERR_INVALID, "dlm_create: a tied head is registered for the pre-norm streams block only");
  if (cfg->canon_taps < 0 || cfg->canon_taps > 64) B200_FAIL(B200_ERR_INVALID, "dlm_create: canon_taps must be in 0..64");
  for (int i = 0; i < cfg->n_layers; ++i) {
    const b200_dlm_layer& l = cfg->layers[i];
    const b200_dlm_mixer &a = l.a, &b = l.b;
    if (cfg->block == B200_BLOCK_PRE_NORM_STREAMS) {
      if (a.heads < 1 || a.dim < 1 || a.vdim < 1) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: heads, dim and vdim must be positive", i);
      if (a.rot_dims < 0 || a.rot_dims % 2) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: rot_dims must be even", i);
      if (a.rot_dims > 0 && a.rot_scaling == B200_ROT_RAMP && (!(a.rot_factor > 0.f) || !(a.rot_original > 0.f) || !(a.rot_fast > 0.f) || !(a.rot_slow > 0.f) || !(a.rot_base > 1.f)))
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: the rotary ramp wants positive factor, original, fast and slow", i);
      if (a.window < 0) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: the window must not be negative", i);
      if (l.mixer == B200_MIXER_LATENT_ATTENTION) {
        if (a.kv_rank < 1 || (a.kv_rank + a.rot_dims + 7) / 8 * 8 > 1024) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: kv_rank + rot_dims in 1..1024", i);
      } else if (l.mixer == B200_MIXER_PARALLEL) {
        if (a.kind != B200_MIXER_WINDOW_ATTENTION || b.kind != B200_MIXER_MINGRU)
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: a parallel pair of this block is window attention beside a minGRU", i);
        if (a.kv_heads < 1 || a.heads % a.kv_heads || a.window < 1 || a.rot_dims > a.dim || a.conv_taps > 1)
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: window attention wants heads a multiple of kv_heads, a positive window, rot_dims <= dim and no convolution", i);
        if (b.dim < 1) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: the minGRU wants a positive width", i);
      } else if (l.mixer == B200_MIXER_CHANNEL_DELTA) {
        if (a.dim > 256 || a.kv_heads < 1 || a.heads % a.kv_heads || a.conv_taps < 1 || a.conv_taps > 64)
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: the delta rule wants dim in 1..256, heads a multiple of kv_heads and conv_taps in 1..64", i);
      } else {
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mixer %d is not registered for this block arrangement", i, l.mixer);
      }
      if (l.mlp != B200_MLP_NONE && l.mlp != B200_MLP_DENSE_RELU2) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mlp kind %d is not registered for this block arrangement", i, l.mlp);
    } else if (cfg->block == B200_BLOCK_PARALLEL_RESIDUAL) {
      if (a.heads < 1 || a.dim < 1 || a.vdim < 1) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: heads, dim and vdim must be positive", i);
      if (a.rot_dims < 0 || a.rot_dims % 2 || a.rot_dims > a.dim) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: rot_dims must be even and at most dim", i);
      if (a.rot_dims > 0 && a.rot_scaling == B200_ROT_RAMP && (!(a.rot_factor > 0.f) || !(a.rot_original > 0.f) || !(a.rot_fast > 0.f) || !(a.rot_slow > 0.f) || !(a.rot_base > 1.f)))
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: the rotary ramp wants positive factor, original, fast and slow", i);
      if (l.mixer == B200_MIXER_SIGMOID_ATTENTION) {
        if (a.kv_heads < 1 || a.heads % a.kv_heads) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: attention wants heads a multiple of kv_heads", i);
      } else if (l.mixer == B200_MIXER_RETENTION) {
        if (a.dim > 256 || !a.decay || a.heads > B200_DLM_MAX_DECAY_HEADS) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: retention wants dim in 1..256 and one decay per head", i);
      } else if (l.mixer == B200_MIXER_DELTA) {
        if (a.dim > 256 || a.kv_heads < 1 || a.heads % a.kv_heads || a.conv_taps < 1 || a.conv_taps > 64)
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: the delta rule wants dim in 1..256, heads a multiple of kv_heads and conv_taps in 1..64", i);
      } else {
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mixer %d is not registered for this block arrangement", i, l.mixer);
      }
      if (l.mlp != B200_MLP_NONE && l.mlp != B200_MLP_DENSE_GATED_GELU && l.mlp != B200_MLP_MOE_CLAMPED_GLU)
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mlp kind %d is not registered for this block arrangement", i, l.mlp);
      if (l.mlp == B200_MLP_MOE_CLAMPED_GLU && (l.experts < 1 || l.experts > 4096 || l.top < 1 || l.top > l.experts || l.top > 32 || !(l.expert_limit > 0.f)))
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: experts in 1..4096, top in 1..min(experts, 32) and a positive limit", i);
    } else if (cfg->block == B200_BLOCK_GATED_DEPTH_AVERAGE) {
      if (l.mixer != B200_MIXER_LATENT_ATTENTION) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mixer %d is not registered for this block arrangement", i, l.mixer);
      if (a.heads < 1 || a.dim < 1 || a.vdim < 1 || a.kv_rank < 1 || a.kv_rank > 1024)
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: heads, dim, vdim must be positive and kv_rank in 1..1024", i);
      if (l.mlp != B200_MLP_NONE && l.mlp != B200_MLP_DENSE_RELU2) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mlp kind %d is not registered for this block arrangement", i, l.mlp);
    } else {
      if (l.mixer == B200_MIXER_PARALLEL) {
        if (a.kind != B200_MIXER_WINDOW_ATTENTION || b.kind != B200_MIXER_GLA)
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: a parallel pair is window attention beside gated linear attention", i);
        if (a.heads < 1 || a.kv_heads < 1 || a.heads % a.kv_heads || a.dim < 1 || a.vdim < 1 || a.window < 1)
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: window attention wants heads a multiple of kv_heads, positive dim, vdim and window", i);
        if (a.rot_dims < 0 || a.rot_dims % 2 || a.rot_dims > a.dim) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: rot_dims must be even and at most dim", i);
        if (a.conv_taps < 0 || a.conv_taps > 64) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: conv_taps must be in 0..64", i);
        if (b.heads < 1 || b.dim < 1 || b.dim > 256 || b.vdim < 1 || !(b.tau > 0.f))
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: gated linear attention wants positive heads, vdim, tau and dim in 1..256", i);
      } else if (l.mixer == B200_MIXER_MLSTM) {
        if (a.heads < 1 || a.dim < 1 || a.dim > 256 || a.vdim < 1 || !(a.gate_cap > 0.f))
          B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mLSTM wants positive heads, vdim, gate_cap and dim in 1..256", i);
      } else {
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mixer %d is not registered for this block arrangement", i, l.mixer);
      }
      if (l.mlp != B200_MLP_NONE && l.mlp != B200_MLP_MOE_RELU2) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: mlp kind %d is not registered for this block arrangement", i, l.mlp);
      if (l.mlp == B200_MLP_MOE_RELU2 && (l.experts < 1 || l.experts > 4096 || l.top < 1 || l.top > l.experts || l.top > 32))
        B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: experts in 1..4096 and top in 1..min(experts, 32)", i);
    }
    if (l.mlp != B200_MLP_NONE && l.ff < 1) B200_FAIL(B200_ERR_INVALID, "dlm_create: layer %d: ff must be positive", i);
  }
  auto* h = new b200_dlm();
  h->cfg = *cfg;
  h->layers.resize(cfg->n_layers);
  for (int i = 0; i < cfg->n_layers; ++i) {
    Layer& L = h->layers[i];
    L.c = cfg->layers[i];
    if (L.c.a.decay) L.decay.assign(L.c.a.decay, L.c.a.decay + L.c.a.heads);      // the caller's array does not outlive this call
    L.c.a.decay = L.c.b.decay = nullptr;
  }
  h->cfg.layers = nullptr;
  h->f32 = cfg->compute_dtype == B200_F32;
  if (cudaGetDevice(&h->device) != cudaSuccess) h->device = -1;
  *out = h;
  return B200_OK;
}

int b200_dlm_load_tensor(b200_dlm* h, const char* name, const void* data_dev, int dtype, int ndim, const int64_t* shape) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_load_tensor: null handle");
  if (h->finalized) B200_FAIL(B200_ERR_STATE, "dlm_load_tensor: the model is finalized");
  DeviceGuard g(h->device);
  return h->store.put(name, data_dev, dtype, ndim, shape);
}

int b200_dlm_set_option(b200_dlm* h, const char* name, int value) {
  if (!h || !name) B200_FAIL(B200_ERR_INVALID, "dlm_set_option: null argument");
  const std::string n(name);
  if (n == "use_tc") {
    if (h->finalized) B200_FAIL(B200_ERR_STATE, "dlm_set_option: use_tc is fixed once the weights are packed");
    h->use_tc = value != 0;
  } else if (n == "trace_layers") {
    if (h->slots) B200_FAIL(B200_ERR_STATE, "dlm_set_option: trace_layers must be set before cache_begin");
    h->trace_layers = value != 0;
  } else if (n == "attn_tc") {
    h->attn_tc = value < 0 ? 0 : value;      // 2: the tensor-core window attention also for single-token requests
  } else if (n == "time_kernels") {
    h->time_kernels = value != 0;
  } else if (n == "scan_segment") {
    h->scan_seg = value < 8 ? 8 : value;
  } else if (n == "delta_chunk") {
    h->delta_chunk = value != 0;
  } else if (n == "attn_split") {
    h->attn_split = value < 0 ? 0 : value;
  } else {
    B200_FAIL(B200_ERR_INVALID, "dlm_set_option: unknown option '%s'", name);
  }
  return B200_OK;
}

int b200_dlm_finalize(b200_dlm* h) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_finalize: null handle");
  if (h->finalized) return B200_OK;
  DeviceGuard g(h->device);
  const b200_dlm_config& c = h->cfg;
  const int64_t W = c.width;
  const size_t es = esize(h);
  std::vector<void*> drop;
  auto matrix = [&](const std::string& name, int64_t rows, int64_t K, void** out) -> int {
    B200_TRY(h->weights.alloc(out, (size_t)rows * K * es, false));
    return put_matrix(h, name, rows, K, *out);
  };
  B200_TRY(matrix("embed", c.vocab, W, &h->embed));
  h->weight_bytes += (int64_t)c.vocab * W * es;
  const bool sandwich = c.block == B200_BLOCK_SANDWICH, parallel = c.block == B200_BLOCK_PARALLEL_RESIDUAL, streams = c.block == B200_BLOCK_PRE_NORM_STREAMS;
  if (streams)
    for (int i = 0; i < c.n_layers; ++i) B200_TRY(finalize_streams_layer(h, i, drop));
  if (sandwich) {
    B200_TRY(get_f32(h, "embed.norm", W, &h->embw));
    for (int i = 0; i < c.n_layers; ++i) B200_TRY(finalize_sandwich_layer(h, i, drop));
  }
  if (parallel) {
    h->vmix_first = -1;
    for (int i = 0; i < c.n_layers; ++i) B200_TRY(finalize_parallel_layer(h, i, drop));
  }
  for (int i = 0; i < c.n_layers && !sandwich && !parallel && !streams; ++i) {
    Layer& L = h->layers[i];
    const std::string p = "l" + std::to_string(i) + ".";
    const int64_t H = L.c.a.heads, dk = L.c.a.dim, dv = L.c.a.vdim, r = L.c.a.kv_rank, F = L.c.ff;
    const bool mlp = L.c.mlp != B200_MLP_NONE;
    B200_TRY(get_f32(h, p + "norm1", W, &L.n1w));
    B200_TRY(get_f32(h, p + "norm1.b", W, &L.n1b));
    // one matrix for everything that reads the normed input: q | latent | up | gate of the mixer | gate of the feed-forward
    L.off_q = 0; L.off_dkv = (int)(H * dk); L.off_up = L.off_dkv + (int)r; L.off_g1 = L.off_up + (mlp ? (int)F : 0);
    L.off_g2 = L.off_g1 + (int)W; L.ncat = L.off_g2 + (mlp ? (int)W : 0);
    L.ldp = (L.ncat + 7) / 8 * 8;
    void* cat = nullptr;
    B200_TRY(h->weights.alloc(&cat, (size_t)L.ncat * W * es, false));
    auto at = [&](int off) { return static_cast<char*>(cat) + (size_t)off * W * es; };
    B200_TRY(put_matrix(h, p + "mix.q", H * dk, W, at(L.off_q)));
    B200_TRY(put_matrix(h, p + "mix.dkv", r, W, at(L.off_dkv)));
    if (mlp) B200_TRY(put_matrix(h, p + "mlp.up", F, W, at(L.off_up)));
    B200_TRY(put_matrix(h, p + "rg1", W, W, at(L.off_g1)));
    if (mlp) B200_TRY(put_matrix(h, p + "rg2", W, W, at(L.off_g2)));
    B200_TRY(seal_weight(h, L.cat, cat, L.ncat, (int)W, drop));
    B200_TRY(get_f32(h, p + "rg1.b", W, &L.b1));
    if (mlp) B200_TRY(get_f32(h, p + "rg2.b", W, &L.b2));
    B200_TRY(get_f32(h, p + "mix.dkv.norm", r, &L.cnorm));
    B200_TRY(get_f32(h, p + "mix.sink", H, &L.sink));
    {   // W_uk [H * dim][r] -> per head [r][dim]
      void* uk = nullptr;
      B200_TRY(matrix(p + "mix.uk", H * dk, r, &uk));
      B200_TRY(h->weights.alloc(&L.ukT, (size_t)H * dk * r * es, false));
      const long long n = H * dk * r;
      if (h->f32) B200_LAUNCH(head_transpose_kernel<float>, (unsigned)ceil_div64(n, 256), 256, 0, nullptr, static_cast<const float*>(uk), static_cast<float*>(L.ukT), (int)H, (int)dk, (int)r);
      else B200_LAUNCH(head_transpose_kernel<bf16>, (unsigned)ceil_div64(n, 256), 256, 0, nullptr, static_cast<const bf16*>(uk), static_cast<bf16*>(L.ukT), (int)H, (int)dk, (int)r);
      B200_TRY(check_launch("head_transpose"));
      drop.push_back(uk);
      h->weight_bytes += n * es;
    }
    B200_TRY(matrix(p + "mix.uv", H * dv, r, &L.uv));
    h->weight_bytes += H * dv * r * es;
    void* wo = nullptr;
    B200_TRY(matrix(p + "mix.o", W, H * dv, &wo));
    B200_TRY(seal_weight(h, L.o, wo, (int)W, (int)(H * dv), drop, (int)W));
    if (mlp) {
      void* wd = nullptr;
      B200_TRY(matrix(p + "mlp.down", W, F, &wd));
      B200_TRY(seal_weight(h, L.down, wd, (int)W, (int)F, drop, (int)W));
    }
    B200_TRY(get_f32(h, p + "dwa", i + 2, &L.avg));
    int sig = -1;
    const int rpt = rows_per_tile((int)r);
    for (size_t k = 0; k < h->sigs.size(); ++k) if (h->sigs[k].H == H && h->sigs[k].rpt == rpt) sig = (int)k;
    if (sig < 0) { TileSig s; s.H = (int)H; s.rpt = rpt; h->sigs.push_back(s); sig = (int)h->sigs.size() - 1; }
    L.sig = sig;
  }
  B200_TRY(get_f32(h, "final.norm", W, &h->fnw));
  if (parallel) B200_LAUNCH(add_one_kernel, ceil_div((int)W, 256), 256, 0, nullptr, h->fnw, (int)W);      // stored around zero
  if (!sandwich && !parallel && !streams) B200_TRY(get_f32(h, "final.norm.b", W, &h->fnb));
  if (c.tied_head) {      // the logits come from the embedding table: its rows stay (the gather), a packed copy serves the product
    h->head.rm = h->embed; h->head.N = c.vocab; h->head.K = (int)W;
    if (!h->f32 && h->use_tc && W % 8 == 0 && (c.vocab + 127) / 128 <= tc::SK_MAX_TILES) {
      B200_TRY(h->weights.alloc(&h->head.tiles, tc::sk_packed_bytes(c.vocab, (int)W, 0, 0), false));
      B200_TRY(tc::sk_pack_weights(static_cast<const bf16*>(h->embed), h->head.tiles, c.vocab, (int)W, 0, 0, nullptr));
    }
  } else {
    void* hd = nullptr;
    B200_TRY(matrix("head", c.vocab, W, &hd));
    B200_TRY(seal_weight(h, h->head, hd, c.vocab, (int)W, drop));
  }
  B200_CUDA(cudaDeviceSynchronize());
  for (void* p : drop) {
    auto it = std::find(h->weights.ptrs.begin(), h->weights.ptrs.end(), p);
    if (it != h->weights.ptrs.end()) h->weights.ptrs.erase(it);
    cudaFree(p);
  }
  h->store.release_all();
  h->finalized = true;
  return B200_OK;
}

int b200_dlm_cache_end(b200_dlm* h) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_cache_end: null handle");
  DeviceGuard g(h->device);
  if (h->slots) cudaStreamSynchronize(h->stream);
  h->state.free_all();
  if (h->meta_pin) { cudaFreeHost(h->meta_pin); h->meta_pin = nullptr; }
  for (auto e : h->ev_pool) cudaEventDestroy(e);
  h->ev_pool.clear(); h->ev_class.clear(); h->ev_used = 0;
  if (h->ev_meta) { cudaEventDestroy(h->ev_meta); h->ev_meta = nullptr; }
  h->plans.clear();
  h->slots = h->cap = h->tmax = h->wmax = 0;
  h->len.clear();
  return B200_OK;
}

int b200_dlm_destroy(b200_dlm* h) {
  if (!h) return B200_OK;
  b200_dlm_cache_end(h);
  DeviceGuard g(h->device);
  h->weights.free_all();
  h->store.release_all();
  delete h;
  return B200_OK;
}

int b200_dlm_set_stream(b200_dlm* h, void* stream) {
  if (!h) B200_FAIL(B200_ERR_INVALID, "dlm_set_stream: null handle");
  h->stream = static_cast<cudaStream_t>(stream);
  return B200_OK;
}

int b200_dlm_cache_begin(b200_dlm* h, int slots, int capacity, int max_step_tokens, int max_want, void* stream) {
  if (!h || !h->finalized) B200_FAIL(B200_ERR_STATE, "dlm_cache_begin: finalize the model first");
  if (h->slots) B200_FAIL(B200_ERR_STATE, "dlm_cache_begin: the cache exists already");
  if (slots < 1 || capacity < 1 || max_step_tokens < 1 || max_want < 1) B200_FAIL(B200_ERR_INVALID, "dlm_cache_begin: sizes must be positive");
  DeviceGuard g(h->device);
  const b200_dlm_config& c = h->cfg;
  Arena& A = h->state;
  const size_t es = esize(h);
  const size_t T = (size_t)max_step_tokens, W = (size_t)c.width;
  h->stream = static_cast<cudaStream_t>(stream);
  const bool sandwich = c.block == B200_BLOCK_SANDWICH, parallel = c.block == B200_BLOCK_PARALLEL_RESIDUAL, streams = c.block == B200_BLOCK_PRE_NORM_STREAMS;
  size_t max_ldp = 0, max_hr = 0, max_hv = 0, max_ff = 1, max_r = 0, max_tiles = 0, max_qkv = 1, max_rv = 1, max_gate = 1, max_e = 1, max_top = 0, max_part = 0, max_prep = 4, max_segrow = 1, max_heads = 1;
  size_t max_small = 1, max_eff = 0, max_nv = 1;
  for (auto& L : h->layers) {
    const b200_dlm_mixer &a = L.c.a, &b = L.c.b;
    max_ldp = std::max(max_ldp, (size_t)L.ldp);
    max_hv = std::max(max_hv, (size_t)a.heads * a.vdim);
    max_ff = std::max(max_ff, (size_t)L.c.ff);
    if (streams) {
      // per request: latents with the rotated key part; keys, values and the minGRU's vector; the matrix memory and the convolutions' last inputs
      if (L.c.mixer == B200_MIXER_LATENT_ATTENTION) {
        B200_TRY(A.alloc(&L.cache, (size_t)slots * capacity * L.rp * es));
        max_hr = std::max(max_hr, (size_t)a.heads * L.rp);
        max_r = std::max(max_r, (size_t)L.rp);
      } else if (L.c.mixer == B200_MIXER_PARALLEL) {
        B200_TRY(A.alloc(&L.kcache, (size_t)slots * capacity * L.Nk * es));
        B200_TRY(A.alloc(&L.vcache, (size_t)slots * capacity * L.Nv * es));
        B200_TRY(A.alloc_t(&L.gru, (size_t)slots * b.dim));
        max_qkv = std::max(max_qkv, (size_t)L.Nq);
        max_rv = std::max(max_rv, (size_t)b.dim);
        max_part = std::max(max_part, (size_t)(L.sig_mma >= 0 ? 16 : L.QT) * a.heads * (a.vdim + 2));
      } else {
        const size_t C = (size_t)2 * L.Nq + L.Nv;
        B200_TRY(A.alloc_t(&L.St, (size_t)slots * a.heads * a.vdim * a.dim));
        if (a.conv_taps > 1) B200_TRY(A.alloc_t(&L.qkv_hist, (size_t)slots * (a.conv_taps - 1) * C));
        max_qkv = std::max(max_qkv, C);
        max_rv = std::max(max_rv, (size_t)a.heads * a.vdim);
        max_gate = std::max(max_gate, (size_t)a.heads * a.dim);
        max_prep = std::max(max_prep, (size_t)a.heads * (3 * (size_t)std::max(2 * a.dim, 64) + 4));
        max_heads = std::max(max_heads, (size_t)a.heads);
      }
      max_small = std::max(max_small, (size_t)L.nsmall);
      continue;
    }
    if (parallel) {
      // per request: keys and values of an attention layer; the matrix memory of a recurrent one and its convolutions' last inputs
      if (L.c.mixer == B200_MIXER_SIGMOID_ATTENTION) {
        B200_TRY(A.alloc(&L.kcache, (size_t)slots * capacity * L.Nk * es));
        B200_TRY(A.alloc(&L.vcache, (size_t)slots * capacity * L.Nv * es));
        max_qkv = std::max(max_qkv, (size_t)L.Nq);
        max_nv = std::max(max_nv, (size_t)L.Nv);
        max_part = std::max(max_part, (size_t)(L.sig_mma >= 0 ? 16 : L.QT) * a.heads * a.vdim);
      } else {
        B200_TRY(A.alloc_t(&L.St, (size_t)slots * a.heads * a.vdim * a.dim));
        if (L.c.mixer == B200_MIXER_DELTA) {
          const size_t C = (size_t)2 * L.Nq + L.Nv;
          if (a.conv_taps > 1) B200_TRY(A.alloc_t(&L.qkv_hist, (size_t)slots * (a.conv_taps - 1) * C));
          max_qkv = std::max(max_qkv, C);
        }
        max_rv = std::max(max_rv, (size_t)a.heads * a.vdim);
        max_gate = std::max(max_gate, (size_t)a.heads * a.dim);
        max_prep = std::max(max_prep, (size_t)a.heads * (3 * (size_t)std::max(2 * a.dim, 64) + 4));
        max_segrow = std::max(max_segrow, (size_t)a.heads * (a.vdim + 1) * a.dim);
        max_heads = std::max(max_heads, (size_t)a.heads);
      }
      if (L.c.mlp == B200_MLP_MOE_CLAMPED_GLU) {
        max_e = std::max(max_e, (size_t)L.c.experts); max_top = std::max(max_top, (size_t)L.c.top);
        max_eff = std::max(max_eff, (size_t)L.c.top * L.c.ff);
      }
      max_small = std::max(max_small, (size_t)L.nsmall);
      continue;
    }
    if (!sandwich) {
      B200_TRY(A.alloc(&L.cache, (size_t)slots * capacity * a.kv_rank * es));
      max_hr = std::max(max_hr, (size_t)a.heads * a.kv_rank);
      max_r = std::max(max_r, (size_t)a.kv_rank);
      continue;
    }
    // per request: the last inputs of the convolutions, keys and values of the window attention, the matrix memories
    if (c.canon_taps > 1) B200_TRY(A.alloc_t(&L.canon_hist, (size_t)slots * (c.canon_taps - 1) * W));
    if (L.c.mixer == B200_MIXER_PARALLEL) {
      const size_t C = (size_t)L.Nq + L.Nk + L.Nv;
      if (a.conv_taps > 1) B200_TRY(A.alloc_t(&L.qkv_hist, (size_t)slots * (a.conv_taps - 1) * C));
      B200_TRY(A.alloc(&L.kcache, (size_t)slots * capacity * L.Nk * es));
      B200_TRY(A.alloc(&L.vcache, (size_t)slots * capacity * L.Nv * es));
      B200_TRY(A.alloc_t(&L.St, (size_t)slots * b.heads * b.vdim * b.dim));
      max_qkv = std::max(max_qkv, C);
      max_rv = std::max(max_rv, (size_t)b.heads * b.vdim);
      max_gate = std::max(max_gate, (size_t)b.heads * b.dim);
      max_prep = std::max(max_prep, (size_t)b.heads * (3 * (size_t)std::max(2 * b.dim, 64) + 4));
      max_segrow = std::max(max_segrow, (size_t)b.heads * (b.vdim + 1) * b.dim);
      max_heads = std::max(max_heads, (size_t)b.heads);
      max_part = std::max(max_part, (size_t)(L.sig_mma >= 0 ? 16 : L.QT) * a.heads * (a.vdim + 2));
    } else {
      B200_TRY(A.alloc_t(&L.St, (size_t)slots * a.heads * a.vdim * a.dim));
      B200_TRY(A.alloc_t(&L.nvec, (size_t)2 * slots * a.heads * a.dim));
      B200_TRY(A.alloc_t(&L.mval, (size_t)2 * slots * a.heads));
      max_rv = std::max(max_rv, (size_t)a.heads * a.vdim);
      max_gate = std::max(max_gate, (size_t)2 * a.heads);
      max_prep = std::max(max_prep, (size_t)a.heads * (2 * (size_t)std::max(2 * a.dim, 64) + 8));
      max_segrow = std::max(max_segrow, (size_t)a.heads * (a.vdim + 1) * a.dim);
      max_heads = std::max(max_heads, (size_t)a.heads);
      max_gate = std::max(max_gate, (size_t)a.heads * a.dim);
    }
    if (L.c.mlp == B200_MLP_MOE_RELU2) { max_e = std::max(max_e, (size_t)L.c.experts); max_top = std::max(max_top, (size_t)L.c.top); }
  }
  B200_TRY(A.alloc_t(&h->xin, T * W));
  if (streams) {
    B200_TRY(A.alloc_t(&h->xs, T * (size_t)std::max(c.streams, 1) * W));
    B200_TRY(A.alloc_t(&h->qkv32, T * max_qkv));
    B200_TRY(A.alloc_t(&h->small32, T * max_small));
    B200_TRY(A.alloc_t(&h->scan32, T * max_rv));
    B200_TRY(A.alloc_t(&h->scan_v, T * max_rv));
    B200_TRY(A.alloc_t(&h->scan_prep, T * max_prep));
    B200_TRY(A.alloc_t(&h->gate32, T * max_gate));
    B200_TRY(A.alloc_t(&h->attn32, T * max_hv));
    B200_TRY(A.alloc_t(&h->qa, T * std::max(max_hr, (size_t)1)));
    B200_TRY(A.alloc_t(&h->ol, T * std::max(max_hr, (size_t)1)));
    B200_TRY(A.alloc(&h->obuf2, T * max_rv * es));
    B200_TRY(A.alloc(&h->mixo2, T * W * es));
    B200_TRY(A.alloc(&h->ffo, T * W * es));
    B200_TRY(A.alloc(&h->act2, T * max_ff * es));
    h->part_floats = (size_t)600 * std::max(std::max(max_part, (size_t)16 * (max_r + 2)), (size_t)1);
    bool any_delta = false;
    for (auto& L : h->layers) any_delta |= L.c.mixer == B200_MIXER_CHANNEL_DELTA;
    if (any_delta) {      // the delta rule's chunks of a step, their triangular matrices and the rows of the walk
      h->max_chunks = max_step_tokens / DELTA_CH + std::min(slots, max_step_tokens) + 1;
      B200_TRY(A.alloc_t(&h->gram, (size_t)h->max_chunks * max_heads * (2 * DELTA_CH + 2 * DELTA_CH * DELTA_CH)));
      B200_TRY(A.alloc_t(&h->rows3, T * 3 * max_gate));
      B200_TRY(A.alloc_t(&h->gend, (size_t)h->max_chunks * max_gate));
    }
  } else if (parallel) {
    const size_t nseg = (size_t)(max_step_tokens / std::max(h->scan_seg, 8) + 2);
    B200_TRY(A.alloc_t(&h->qkv32, T * max_qkv));
    B200_TRY(A.alloc_t(&h->small32, T * max_small));
    B200_TRY(A.alloc_t(&h->scan32, T * max_rv));
    B200_TRY(A.alloc_t(&h->scan_v, T * max_rv));
    B200_TRY(A.alloc_t(&h->scan_prep, T * max_prep));
    B200_TRY(A.alloc_t(&h->segS, nseg * max_segrow));
    B200_TRY(A.alloc_t(&h->segB, nseg * max_gate));
    B200_TRY(A.alloc_t(&h->segM, nseg * max_heads * 4));
    B200_TRY(A.alloc_t(&h->tokM, T * max_heads * 4));
    h->max_seg_units = (int)nseg;
    h->max_chunks = max_step_tokens / DELTA_CH + std::min(slots, max_step_tokens) + 1;
    bool any_delta = false;
    for (auto& L : h->layers) any_delta |= L.c.mixer == B200_MIXER_DELTA;
    if (any_delta) B200_TRY(A.alloc_t(&h->gram, (size_t)h->max_chunks * max_heads * (2 * DELTA_CH + 2 * DELTA_CH * DELTA_CH)));
    B200_TRY(A.alloc_t(&h->gate32, T * max_gate));
    B200_TRY(A.alloc(&h->ffo, T * W * es));
    B200_TRY(A.alloc(&h->vfirst, T * max_nv * es));
    h->part_floats = (size_t)600 * std::max(max_part, (size_t)1);
    if (max_top) {
      const size_t pairs = T * max_top, tiles = pairs / 64 + max_e + 2;
      B200_TRY(A.alloc_t(&h->moe_w, pairs));
      B200_TRY(A.alloc_t(&h->moe_idx, pairs));
      B200_TRY(A.alloc_t(&h->moe_rank, pairs));
      B200_TRY(A.alloc_t(&h->moe_perm, pairs));
      B200_TRY(A.alloc_t(&h->moe_row_tok, pairs));
      B200_TRY(A.alloc_t(&h->moe_tile_e, tiles));
      B200_TRY(A.alloc_t(&h->moe_tile_r0, tiles));
      B200_TRY(A.alloc_t(&h->moe_tile_n, tiles));
      B200_TRY(A.alloc_t(&h->moe_ntiles, 1));
      B200_TRY(A.alloc(&h->yexp, pairs * W * es));
      B200_TRY(A.alloc(&h->act2, T * 2 * max_eff * es));
      max_ff = std::max(max_ff, max_eff);       // the experts' hidden rows: one per (token, chosen expert)
    }
  } else if (!sandwich) {
    B200_TRY(A.alloc_t(&h->stack, (size_t)(c.n_layers + 1) * T * W));
    B200_TRY(A.alloc_t(&h->qa, T * max_hr));
    B200_TRY(A.alloc_t(&h->ol, T * max_hr));
    h->part_floats = (size_t)600 * 16 * (max_r + 2);
    B200_TRY(A.alloc(&h->ffo, T * W * es));
  } else {
    B200_TRY(A.alloc_t(&h->h32, T * W));
    B200_TRY(A.alloc_t(&h->qkv32, T * max_qkv));
    B200_TRY(A.alloc_t(&h->scan32, T * max_rv));
    B200_TRY(A.alloc_t(&h->scan_v, T * max_rv));
    B200_TRY(A.alloc_t(&h->scan_prep, T * max_prep));
    B200_TRY(A.alloc_t(&h->segS, (size_t)(max_step_tokens / std::max(h->scan_seg, 8) + 2) * max_segrow));
    B200_TRY(A.alloc_t(&h->segB, (size_t)(max_step_tokens / std::max(h->scan_seg, 8) + 2) * max_gate));
    B200_TRY(A.alloc_t(&h->segM, (size_t)(max_step_tokens / std::max(h->scan_seg, 8) + 2) * max_heads * 4));
    B200_TRY(A.alloc_t(&h->tokM, T * max_heads * 4));
    B200_TRY(A.alloc_t(&h->corr, T * (max_rv + max_heads)));
    h->max_seg_units = max_step_tokens / std::max(h->scan_seg, 8) + 2;
    B200_TRY(A.alloc_t(&h->gate32, T * max_gate));
    B200_TRY(A.alloc_t(&h->attn32, T * max_hv));
    B200_TRY(A.alloc(&h->obuf2, T * max_rv * es));
    B200_TRY(A.alloc(&h->mixo2, T * W * es));
    h->part_floats = (size_t)600 * std::max(max_part, (size_t)1);
    if (max_top) {
      const size_t pairs = T * max_top, tiles = pairs / 64 + max_e + 2;
      B200_TRY(A.alloc_t(&h->route32, T * max_e));
      B200_TRY(A.alloc_t(&h->moe_w, pairs));
      B200_TRY(A.alloc_t(&h->moe_idx, pairs));
      B200_TRY(A.alloc_t(&h->moe_rank, pairs));
      B200_TRY(A.alloc_t(&h->moe_perm, pairs));
      B200_TRY(A.alloc_t(&h->moe_row_tok, pairs));
      B200_TRY(A.alloc_t(&h->moe_tile_e, tiles));
      B200_TRY(A.alloc_t(&h->moe_tile_r0, tiles));
      B200_TRY(A.alloc_t(&h->moe_tile_n, tiles));
      B200_TRY(A.alloc_t(&h->moe_ntiles, 1));
      B200_TRY(A.alloc(&h->yexp, pairs * W * es));
      max_ff *= max_top;        // the experts' hidden rows: one per (token, chosen expert)
    }
  }
  if (h->trace_layers) B200_TRY(A.alloc_t(&h->trace, (size_t)c.n_layers * T * W));
  B200_TRY(A.alloc_t(&h->part, h->part_floats));
  B200_TRY(A.alloc(&h->hbuf, T * W * es));
  B200_TRY(A.alloc(&h->proj, T * max_ldp * es));
  B200_TRY(A.alloc(&h->obuf, T * max_hv * es));
  B200_TRY(A.alloc(&h->mixo, T * W * es));
  B200_TRY(A.alloc(&h->act, T * max_ff * es));
  B200_TRY(A.alloc(&h->hf, (size_t)max_want * W * es));
  B200_TRY(A.alloc_t(&h->logits, (size_t)max_want * c.vocab));
  B200_TRY(A.alloc_t(&h->logits_bf, (size_t)max_want * c.vocab));
  B200_TRY(A.alloc_t(&h->head_bf, (size_t)max_want * ((c.vocab + 7) / 8 * 8)));
  B200_TRY(A.alloc_t(&h->err, 1));
  B200_TRY(A.alloc(reinterpret_cast<void**>(&h->sk_ws), tc::sk_workspace_bytes(256), false));
  B200_TRY(A.alloc_t(&h->sk_counters, tc::SK_MAX_TILES));
  // step metadata: tokens | slot | position per token, wanted rows, then one tile list per (heads, rows per tile) combination
  int off = 0;
  h->off_tok = off; off += max_step_tokens;
  h->off_slot = off; off += max_step_tokens;
  h->off_pos = off; off += max_step_tokens;
  h->off_want = off; off += max_want;
  h->off_first = off; off += max_step_tokens;
  h->off_last = off; off += max_step_tokens;
  const int max_entries = std::min(slots, max_step_tokens) + max_step_tokens / 8 + 2;      // entries, and the segments long portions are cut into
  h->off_ent_seg = off; off += max_entries;
  h->off_ent_nseg = off; off += max_entries;
  h->off_ent_buf = off; off += max_entries;
  h->off_ent_tok0 = off; off += max_entries;
  h->off_ent_ntok = off; off += max_entries;
  h->off_ent_slot = off; off += max_entries;
  h->off_ent_pos0 = off; off += max_entries;
  h->off_ent_par = off; off += max_entries;
  h->off_whole_tok0 = off; off += max_entries;
  h->off_whole_ntok = off; off += max_entries;
  h->off_whole_slot = off; off += max_entries;
  h->off_whole_pos0 = off; off += max_entries;
  h->off_zero = off; off += max_entries;
  h->off_one = off; off += max_entries;
  h->off_whole_chunk0 = off; off += max_entries;
  h->off_chunk_tok0 = off; off += std::max(h->max_chunks, 1);
  h->off_chunk_nt = off; off += std::max(h->max_chunks, 1);
  for (auto& s : h->sigs) {
    max_tiles = (size_t)ceil_div64((int64_t)max_step_tokens * s.H, s.rpt) + (size_t)std::min(slots, max_step_tokens);
    s.off_row0 = off; off += (int)max_tiles;
    s.off_rows = off; off += (int)max_tiles;
    s.off_slot = off; off += (int)max_tiles;
  }
  h->meta_ints = off;
  B200_TRY(A.alloc_t(&h->meta_dev, (size_t)off));
  B200_CUDA(cudaMallocHost(&h->meta_pin, (size_t)off * sizeof(int)));
  B200_CUDA(cudaEventCreateWithFlags(&h->ev_meta, cudaEventDisableTiming));
  h->slots = slots; h->cap = capacity; h->tmax = max_step_tokens; h->wmax = max_want;
  h->len.assign(slots, 0);
  h->par.assign(slots, 0);
  h->last_tokens = h->last_want = 0;
  if (!h->f32 && h->use_tc) B200_TRY(tc::prepare_plans(h->plans));
  B200_CUDA(cudaDeviceSynchronize());
  return B200_OK;
}

int b200_dlm_release(b200_dlm* h, int slot) {
  if (!h || slot < 0 || slot >= h->slots) B200_FAIL(B200_ERR_INVALID, "dlm_release: slot %d does not exist", slot);
  h->len[slot] = 0;
  return B200_OK;
}

int b200_dlm_slot_length(b200_dlm* h, int slot) {
  if (!h || slot < 0 || slot >= h->slots) return -1;
  return h->len[slot];
}

int b200_dlm_step(b200_dlm* h, int n_entries, const int32_t* slots_host, const int32_t* counts_host, const int32_t* tokens_host,
                  int n_want, const int32_t* want_host, float* logits_dev) {
  if (!h || !h->slots) B200_FAIL(B200_ERR_STATE, "dlm_step: no cache (call cache_begin)");
  if (n_entries < 1 || !slots_host || !counts_host || !tokens_host || (n_want > 0 && !want_host)) B200_FAIL(B200_ERR_INVALID, "dlm_step: null argument");
  DeviceGuard g(h->device);
  long long total = 0;
  std::vector<char> used(h->slots, 0);
  for (int e = 0; e < n_entries; ++e) {
    const int s = slots_host[e], n = counts_host[e];
    if (s < 0 || s >= h->slots) B200_FAIL(B200_ERR_INVALID, "dlm_step: slot %d does not exist", s);
    if (used[s]) B200_FAIL(B200_ERR_INVALID, "dlm_step: slot %d appears twice in one step", s);
    used[s] = 1;
    if (n < 1) B200_FAIL(B200_ERR_INVALID, "dlm_step: entry %d brings no token", e);
    if (h->len[s] + n > h->cap) B200_FAIL(B200_ERR_STATE, "dlm_step: slot %d would hold %d tokens, capacity is %d", s, h->len[s] + n, h->cap);
    total += n;
  }
  if (total > h->tmax) B200_FAIL(B200_ERR_SHAPE, "dlm_step: %lld tokens in one step, the buffers take %d", total, h->tmax);
  if (n_want > h->wmax) B200_FAIL(B200_ERR_SHAPE, "dlm_step: %d logit rows wanted, the buffers take %d", n_want, h->wmax);
  for (int i = 0; i < n_want; ++i)
    if (want_host[i] < 0 || want_host[i] >= total) B200_FAIL(B200_ERR_INVALID, "dlm_step: wanted row %d is outside the step", want_host[i]);
  // the previous step's metadata copy must have left the pinned block
  B200_CUDA(cudaEventSynchronize(h->ev_meta));
  int* m = h->meta_pin;
  int t = 0, max_ctx = 0, n_seg_units = 0, n_chunks = 0;
  h->units.clear();
  for (auto& s : h->sigs) s.count = 0;
  for (int e = 0; e < n_entries; ++e) {
    const int s = slots_host[e], n = counts_host[e], base = h->len[s];
    for (auto& sg : h->sigs) {
      const int rows = n * sg.H;
      for (int r0 = 0; r0 < rows; r0 += sg.rpt) {
        m[sg.off_row0 + sg.count] = t * sg.H + r0;
        m[sg.off_rows + sg.count] = std::min(sg.rpt, rows - r0);
        m[sg.off_slot + sg.count] = s;
        ++sg.count;
      }
    }
    {   // the recurrences' units: the entry itself, or its segments when it is long
      const int seg_len = h->scan_seg, nseg = (h->cfg.block != B200_BLOCK_GATED_DEPTH_AVERAGE && n >= 2 * seg_len && n_seg_units + ceil_div(n, seg_len) <= h->max_seg_units) ? ceil_div(n, seg_len) : 1;
      for (int q = 0; q < nseg; ++q) {
        const int u = (int)h->units.size();
        const int u_tok0 = t + q * seg_len, u_n = nseg == 1 ? n : std::min(seg_len, n - q * seg_len);
        m[h->off_ent_tok0 + u] = u_tok0; m[h->off_ent_ntok + u] = u_n; m[h->off_ent_slot + u] = s; m[h->off_ent_pos0 + u] = base;
        m[h->off_ent_par + u] = h->par[s];
        m[h->off_ent_seg + u] = q; m[h->off_ent_nseg + u] = nseg; m[h->off_ent_buf + u] = nseg > 1 ? n_seg_units : 0;
        h->units.push_back({u_tok0, u_n, q, nseg > 1 ? n_seg_units : -1});
        if (nseg > 1) ++n_seg_units;
      }
    }
    m[h->off_whole_tok0 + e] = t; m[h->off_whole_ntok + e] = n; m[h->off_whole_slot + e] = s; m[h->off_whole_pos0 + e] = base;
    m[h->off_zero + e] = 0; m[h->off_one + e] = 1;
    if (h->max_chunks) {
      m[h->off_whole_chunk0 + e] = n_chunks;
      for (int c0 = 0; c0 < n; c0 += DELTA_CH, ++n_chunks) { m[h->off_chunk_tok0 + n_chunks] = t + c0; m[h->off_chunk_nt + n_chunks] = std::min(DELTA_CH, n - c0); }
    }
    const int first = t, lastt = t + n - 1;
    for (int i = 0; i < n; ++i, ++t) {
      m[h->off_tok + t] = tokens_host[t];
      m[h->off_slot + t] = s;
      m[h->off_pos + t] = base + i;
      m[h->off_first + t] = first;
      m[h->off_last + t] = lastt;
    }
    max_ctx = std::max(max_ctx, base + n);
  }
  for (int i = 0; i < n_want; ++i) m[h->off_want + i] = want_host[i];
  B200_CUDA(cudaMemcpyAsync(h->meta_dev, m, (size_t)h->meta_ints * sizeof(int), cudaMemcpyHostToDevice, h->stream));
  B200_CUDA(cudaEventRecord(h->ev_meta, h->stream));
  h->n_entries = n_entries;
  h->n_units = (int)h->units.size();
  h->n_chunks = n_chunks;
  h->max_entry_tokens = 0;
  for (int e = 0; e < n_entries; ++e) h->max_entry_tokens = std::max(h->max_entry_tokens, (int)counts_host[e]);
  int rc;
  if (h->cfg.block == B200_BLOCK_PRE_NORM_STREAMS) rc = h->f32 ? step_streams<float>(h, t, n_want, max_ctx, logits_dev) : step_streams<bf16>(h, t, n_want, max_ctx, logits_dev);
  else if (h->cfg.block == B200_BLOCK_PARALLEL_RESIDUAL) rc = h->f32 ? step_parallel<float>(h, t, n_want, max_ctx, logits_dev) : step_parallel<bf16>(h, t, n_want, max_ctx, logits_dev);
  else if (h->cfg.block == B200_BLOCK_SANDWICH) rc = h->f32 ? step_sandwich<float>(h, t, n_want, max_ctx, logits_dev) : step_sandwich<bf16>(h, t, n_want, max_ctx, logits_dev);
  else rc = h->f32 ? step_body<float>(h, t, n_want, max_ctx, logits_dev) : step_body<bf16>(h, t, n_want, max_ctx, logits_dev);
  if (rc != B200_OK) return rc;
  if (h->time_kernels && h->ev_used) {      // diagnostics only: waits for the step and sums its intervals per class
    B200_CUDA(cudaStreamSynchronize(h->stream));
    for (size_t i = 0; i + 1 < h->ev_used; i += 2) {
      float ms = 0.f;
      B200_CUDA(cudaEventElapsedTime(&ms, h->ev_pool[i], h->ev_pool[i + 1]));
      h->class_ms[h->ev_class[i]] += ms;
    }
    h->ev_used = 0;
  }
  for (int e = 0; e < n_entries; ++e) { h->len[slots_host[e]] += counts_host[e]; h->par[slots_host[e]] ^= 1; }
  h->last_tokens = t; h->last_want = n_want;
  return B200_OK;
}

int b200_dlm_sample(b200_dlm* h, const float* noise_dev, int use_sampling, float temp, int top_k, int64_t* out_dev) {
  using namespace b200::lm;
  if (!h || !h->slots || h->last_want < 1 || !out_dev) B200_FAIL(B200_ERR_STATE, "dlm_sample: the last step left no logits");
  const int V = h->cfg.vocab;
  DeviceGuard g(h->device);
  if (!use_sampling || temp <= 0.f) {        // greedy: on the fp32 logits, whatever the vocabulary's size
    B200_LAUNCH(argmax_rows_kernel, h->last_want, 256, 0, h->stream, h->logits, V, reinterpret_cast<long long*>(out_dev));
    return check_launch("dlm_sample (greedy)");
  }
  if (V + 1 > 65535) B200_FAIL(B200_ERR_SHAPE, "dlm_sample: the sampler takes vocabularies up to 65534");
  if (top_k < 1) top_k = 1;
  if (top_k > SAMPLE_MAX_K) B200_FAIL(B200_ERR_SHAPE, "dlm_sample: top_k above %d", SAMPLE_MAX_K);
  if (!noise_dev) B200_FAIL(B200_ERR_INVALID, "dlm_sample: sampling needs noise");
  const long long n = (long long)h->last_want * V;
  B200_LAUNCH(logits_to_bf16_kernel, (unsigned)ceil_div64(n, 256), 256, 0, h->stream, h->logits, h->logits_bf, n);
  const int k = top_k < V ? top_k : V;
  B200_LAUNCH(sample_kernel, h->last_want, SAMPLE_THREADS, 0, h->stream, h->logits_bf, (long long)V, noise_dev, (long long)k,
              reinterpret_cast<long long*>(out_dev), V, use_sampling, temp, top_k);
  return check_launch("dlm_sample");
}

int b200_dlm_read_buffer(b200_dlm* h, const char* name, void* dst_dev, int64_t capacity_bytes, int64_t* nbytes) {
  if (!h || !h->slots || !name) B200_FAIL(B200_ERR_STATE, "dlm_read_buffer: no cache");
  DeviceGuard g(h->device);
  const std::string n(name);
  const size_t W = h->cfg.width;
  if (n == "logits") {
    const int64_t bytes = (int64_t)h->last_want * h->cfg.vocab * 4;
    if (nbytes) *nbytes = bytes;
    if (!dst_dev) return B200_OK;
    if (capacity_bytes < bytes) B200_FAIL(B200_ERR_SHAPE, "dlm_read_buffer: '%s' needs %lld bytes", name, (long long)bytes);
    B200_CUDA(cudaMemcpyAsync(dst_dev, h->logits, (size_t)bytes, cudaMemcpyDeviceToDevice, h->stream));
    return B200_OK;
  }
  if (n == "layers") {
    if (!h->trace) B200_FAIL(B200_ERR_STATE, "dlm_read_buffer: 'layers' needs option trace_layers = 1 before cache_begin");
    const int64_t row = (int64_t)h->last_tokens * W * 4;
    const int64_t bytes = row * h->cfg.n_layers;
    if (nbytes) *nbytes = bytes;
    if (!dst_dev) return B200_OK;
    if (capacity_bytes < bytes) B200_FAIL(B200_ERR_SHAPE, "dlm_read_buffer: '%s' needs %lld bytes", name, (long long)bytes);
    B200_CUDA(cudaMemcpy2DAsync(dst_dev, (size_t)row, h->trace, (size_t)h->tmax * W * 4, (size_t)row, (size_t)h->cfg.n_layers,
                                cudaMemcpyDeviceToDevice, h->stream));
    return B200_OK;
  }
  if (n == "error_flags") {
    if (nbytes) *nbytes = 4;
    if (!dst_dev) return B200_OK;
    if (capacity_bytes < 4) B200_FAIL(B200_ERR_SHAPE, "dlm_read_buffer: 'error_flags' needs 4 bytes");
    B200_CUDA(cudaMemcpyAsync(dst_dev, h->err, 4, cudaMemcpyDeviceToDevice, h->stream));
    return B200_OK;
  }
  B200_FAIL(B200_ERR_INVALID, "dlm_read_buffer: unknown buffer '%s'", name);
}

int b200_dlm_read_timers(b200_dlm* h, double* ms6_host, int reset) {
  if (!h || !ms6_host) B200_FAIL(B200_ERR_INVALID, "dlm_read_timers: null argument");
  for (int i = 0; i < 6; ++i) { ms6_host[i] = h->class_ms[i]; if (reset) h->class_ms[i] = 0; }
  return B200_OK;
}

// weights once + what the new tokens read of the cache and state + what they write.  `context` = cached tokens over all
// requests of the step; the sandwich block also needs `tokens` = requests when decoding (one state per request), which is what
// the caller passes there.  Routed experts: every expert's weights count once when the step has at least `experts` (token,
// choice) pairs, else tokens * top experts.
int64_t b200_dlm_algorithmic_bytes(b200_dlm* h, int tokens, int context) {
  if (!h) return 0;
  const int64_t es = esize(h), W = h->cfg.width;
  int64_t b = h->weight_bytes - (int64_t)h->cfg.vocab * W * es;     // the embedding is gathered, not streamed
  if (h->cfg.block == B200_BLOCK_PRE_NORM_STREAMS) {      // `tokens` = requests when decoding; the embedding table is streamed once, as the head
    b = h->weight_bytes;
    for (auto& L : h->layers) {
      const b200_dlm_mixer &a = L.c.a, &m = L.c.b;
      const int64_t per = tokens > 0 ? (int64_t)context / tokens : 0;
      const int64_t seen = (a.window > 0 ? std::min<int64_t>(per, a.window) : per) * tokens;      // decoding: every request reads its window
      if (L.c.mixer == B200_MIXER_LATENT_ATTENTION) b += (seen + tokens) * L.rp * es;
      else if (L.c.mixer == B200_MIXER_PARALLEL) b += (seen + tokens) * (L.Nk + L.Nv) * es + 2 * (int64_t)tokens * m.dim * 4;
      else b += 2 * (int64_t)tokens * a.heads * a.dim * a.vdim * 4;                                // the matrix memories, read and written
    }
    return b + (int64_t)tokens * W * es;
  }
  if (h->cfg.block == B200_BLOCK_PARALLEL_RESIDUAL) {      // `tokens` = requests when decoding, as for the sandwich block
    for (auto& L : h->layers) {
      const b200_dlm_mixer& a = L.c.a;
      if (L.c.mixer == B200_MIXER_SIGMOID_ATTENTION) b += ((int64_t)context + tokens) * (L.Nk + L.Nv) * es;      // every cached key and value once
      else b += 2 * (int64_t)tokens * a.heads * a.dim * a.vdim * 4;                                              // the matrix memories, read and written
      if (L.c.mlp == B200_MLP_MOE_CLAMPED_GLU) {
        const int64_t used = std::min<int64_t>(L.c.experts, (int64_t)tokens * L.c.top);
        b -= (int64_t)(L.c.experts - used) * 3 * L.c.ff * W * es;
      }
    }
    return b + (int64_t)tokens * W * es;
  }
  if (h->cfg.block != B200_BLOCK_SANDWICH) {
    for (auto& L : h->layers) b += ((int64_t)context + tokens) * L.c.a.kv_rank * es;
    return b + (int64_t)tokens * W * es;
  }
  for (auto& L : h->layers) {
    const b200_dlm_mixer &a = L.c.a, &m = L.c.mixer == B200_MIXER_PARALLEL ? L.c.b : L.c.a;
    if (L.c.mixer == B200_MIXER_PARALLEL) {
      const int64_t seen = tokens > 0 ? std::min<int64_t>((int64_t)context / tokens, a.window) * tokens : 0;      // decoding: every request reads its window
      b += (seen + tokens) * (L.Nk + L.Nv) * es;
    }
    b += 2 * (int64_t)tokens * m.heads * m.dim * m.vdim * 4;        // the matrix memories, read and written
    if (L.c.mlp == B200_MLP_MOE_RELU2) {
      const int64_t used = std::min<int64_t>(L.c.experts, (int64_t)tokens * L.c.top);
      b -= (int64_t)(L.c.experts - used) * 2 * L.c.ff * W * es;
    }
  }
  return b + (int64_t)tokens * W * es;
}

// multiply-adds x 2 of the linears and of attention in the form the kernels run it (scores and sums against the latent; the
// window attention over the keys a token sees; routed experts for the chosen ones only; the recurrences' update and read-out)
int64_t b200_dlm_algorithmic_flops(b200_dlm* h, int tokens, int context) {
  if (!h) return 0;
  const int64_t T = tokens, W = h->cfg.width;
  int64_t f = 0;
  for (auto& L : h->layers) {
    if (h->cfg.block == B200_BLOCK_PRE_NORM_STREAMS) {
      const b200_dlm_mixer &a = L.c.a, &m = L.c.b;
      int64_t pairs = 0;       // (query, key) pairs of one prompt of T tokens on top of `context`
      for (int64_t t = 0; t < T; ++t) pairs += a.window > 0 ? std::min<int64_t>(context + t + 1, a.window) : context + t + 1;
      f += 2 * T * W * L.ncat + 2 * T * W * L.nsmall + 2 * T * W * a.heads * a.vdim;
      if (L.c.mixer == B200_MIXER_LATENT_ATTENTION) f += 2 * T * a.heads * (a.dim + a.vdim) * a.kv_rank + 4 * pairs * a.heads * (a.kv_rank + a.rot_dims);
      else if (L.c.mixer == B200_MIXER_PARALLEL) f += 2 * pairs * a.heads * (a.dim + a.vdim) + 2 * T * W * m.dim;
      else f += 8 * T * a.heads * a.dim * a.vdim + 2 * T * ((int64_t)L.decay_rank * a.heads * a.dim + (int64_t)L.gate_rank * a.heads * a.vdim);
      if (L.c.mlp != B200_MLP_NONE) f += 4 * T * W * L.c.ff;
      continue;
    }
    if (h->cfg.block == B200_BLOCK_PARALLEL_RESIDUAL) {
      const b200_dlm_mixer& a = L.c.a;
      f += 2 * T * W * L.ncat + 2 * T * W * L.nsmall + 2 * T * W * a.heads * a.vdim;
      if (L.c.mixer == B200_MIXER_SIGMOID_ATTENTION) f += 2 * a.heads * (a.dim + a.vdim + a.heads) * (T * context + T * (T + 1) / 2);      // scores, head mix, sums
      else f += (L.c.mixer == B200_MIXER_DELTA ? 8 : 4) * T * a.heads * a.dim * a.vdim;
      if (L.c.mlp == B200_MLP_DENSE_GATED_GELU) f += 2 * T * W * L.c.ff;                   // the down-projection (gate and value are inside ncat)
      if (L.c.mlp == B200_MLP_MOE_CLAMPED_GLU) f += 6 * T * L.c.top * W * L.c.ff;
      continue;
    }
    if (h->cfg.block == B200_BLOCK_SANDWICH) {
      const b200_dlm_mixer &a = L.c.a, &m = L.c.mixer == B200_MIXER_PARALLEL ? L.c.b : L.c.a;
      f += 2 * T * W * L.ncat + 2 * T * W * m.heads * m.vdim + 4 * T * m.heads * m.dim * m.vdim;
      if (L.c.mixer == B200_MIXER_PARALLEL) {
        int64_t pairs = 0;       // (query, key) pairs of one prompt of T tokens on top of `context`
        for (int64_t t = 0; t < T; ++t) pairs += std::min<int64_t>(context + t + 1, a.window);
        f += 2 * pairs * a.heads * (a.dim + a.vdim) + 2 * T * W * a.heads * a.vdim + 2 * T * L.decay_rank * m.heads * m.dim;
      }
      if (L.c.mlp == B200_MLP_MOE_RELU2) f += 4 * T * L.c.top * W * L.c.ff + 2 * T * W * L.c.experts;
      continue;
    }
    const int64_t H = L.c.a.heads, dk = L.c.a.dim, dv = L.c.a.vdim, r = L.c.a.kv_rank;
    f += 2 * T * W * L.ncat + 2 * T * H * dk * r + 2 * T * H * dv * r + 2 * T * W * H * dv;
    if (L.c.mlp != B200_MLP_NONE) f += 2 * T * W * L.c.ff;
    f += 4 * H * r * (T * context + T * (T + 1) / 2);
  }
  return f + 2 * T * W * h->cfg.vocab;
}

int b200_op_latent_attention(const float* qa_dev, const void* latents_dev, int dtype, const float* sink_dev, float* out_dev,
                             int T, int H, int r, int pos0, int nsplit, int tensor_cores, void* stream) {
  if (!qa_dev || !latents_dev || !sink_dev || !out_dev) B200_FAIL(B200_ERR_INVALID, "op_latent_attention: null pointer");
  if (T < 1 || H < 1 || r < 1 || r > 1024 || pos0 < 0) B200_FAIL(B200_ERR_SHAPE, "op_latent_attention: bad shape");
  if (dtype != B200_F32 && dtype != B200_BF16) B200_FAIL(B200_ERR_INVALID, "op_latent_attention: latents must be f32 or bf16");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rpt = rows_per_tile(r), rows = T * H, tiles = ceil_div(rows, rpt);
  std::vector<int> meta((size_t)3 * tiles + T);
  for (int i = 0; i < tiles; ++i) { meta[i] = i * rpt; meta[tiles + i] = std::min(rpt, rows - i * rpt); meta[2 * tiles + i] = 0; }
  for (int t = 0; t < T; ++t) meta[3 * tiles + t] = pos0 + t;
  int* meta_dev = nullptr; float* part = nullptr;
  B200_CUDA(cudaMalloc(&meta_dev, meta.size() * sizeof(int)));
  B200_CUDA(cudaMemcpyAsync(meta_dev, meta.data(), meta.size() * sizeof(int), cudaMemcpyHostToDevice, st));
  AttnParams p;
  p.qa = qa_dev; p.cache = latents_dev; p.sink = sink_dev; p.tile_row0 = meta_dev; p.tile_rows = meta_dev + tiles; p.tile_slot = meta_dev + 2 * tiles;
  p.tok_pos = meta_dev + 3 * tiles; p.out = out_dev; p.cap = pos0 + T; p.r = r; p.H = H;
  const size_t part_floats = (size_t)600 * 16 * (r + 2);
  p.nsplit = pick_split(nsplit, tiles, pos0 + T, rpt, r, nsplit > 0 ? (size_t)tiles * nsplit * rpt * (r + 2) : part_floats);
  const size_t need = (size_t)tiles * p.nsplit * rpt * (r + 2);
  B200_CUDA(cudaMalloc(&part, std::max(need, (size_t)1) * sizeof(float)));
  p.part = part;
  int rc = dtype == B200_F32 ? run_attention<float>(st, p, tiles, rpt) : run_attention<bf16>(st, p, tiles, rpt, tensor_cores != 0);
  cudaError_t e = cudaStreamSynchronize(st);
  cudaFree(meta_dev); cudaFree(part);
  if (rc == B200_OK && e != cudaSuccess) { set_error("op_latent_attention: %s", cudaGetErrorString(e)); rc = B200_ERR_CUDA; }
  return rc;
}

}  // extern "C"
