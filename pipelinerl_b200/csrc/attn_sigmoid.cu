// Causal attention WITHOUT a softmax over a paged KV cache, with the heads' weights mixed by a matrix:
//
//     s_h(i, j)  = (q_h(i) . k_c(h)(j)) * scale * temp(pos_i),     temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)
//     s_h       <- cap * tanh(s_h / cap)                           (cap > 0)
//     w_h(i, j)  = sigmoid(s_h(i, j) + bias_h)  for j <= i, else 0 (never normalised over j)
//     m_h(i, j)  = sum_g talk[h][g] w_g(i, j)                      (talk NULL: m = w)
//     o_h(i)     = sum_j m_h(i, j) v_c(h)(j)                       c(h) = h / (H / G)
//
// The mixing couples all heads of a (query, key) pair, so a CTA owns RQ query rows of one segment with ALL their heads.
// It streams the sequence's keys and values in tiles of 32 (all G key/value heads, converted to fp32) through shared
// memory.  Per tile: (1) every (row, head) scores the 32 keys, one key per lane, and stores the sigmoid weights;
// (2) the weights are mixed over the heads; (3) every (row, head) adds the tile's weighted values to its accumulator,
// which lives in shared memory ([RQ][H][vdim] fp32) because the head count is a run-time number.  The eight warps of
// a CTA are split evenly over the RQ rows; the warps of a row take its heads in turn.  RQ is chosen at launch
// (8, 4, 2 or 1: what the segment lengths ask for and shared memory holds).  Key tiles start at absolute multiples
// of 32 and every sum runs in ascending key order, so a token's result does not depend on how its prompt was cut or
// batched.  Everything is fp32; T is only the storage type of q, the cache and (optionally) the output.
//
// K pool: [page][kv head][page_size][dim], V pool: [page][kv head][page_size][vdim]; block_table[slot][j] = j-th page.
#include "prl_common.cuh"
#include <math.h>

namespace prl {
namespace {

constexpr int kWarps = 8;
constexpr int kKeys = 32;

template <typename T> __device__ __forceinline__ float cvt(T v);
template <> __device__ __forceinline__ float cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ float cvt<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ void put(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void put<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void put<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

struct SigmoidAttnArgs {
  const void* q;
  const void* k_pool;
  const void* v_pool;
  const int32_t* block_table;
  int max_blocks, page_size;
  const int32_t* seg_start;
  const int32_t* seg_len;
  const int32_t* seg_pos0;
  const int32_t* seg_slot;
  int H, G, dim, vdim;
  float scale, softcap, temp_coef, temp_every;
  const float* head_bias;
  const float* talk;
  int rq;
  void* out;
};

__host__ __device__ inline size_t sigmoid_attn_floats(int rq, int H, int G, int dim, int vdim) {
  return (size_t)rq * H * dim + (size_t)G * kKeys * (dim + 1) + (size_t)G * kKeys * vdim + 2 * (size_t)rq * H * kKeys +
         (size_t)rq * H * vdim + (size_t)H * H + H + rq;
}

template <typename T, typename TOUT>
__global__ void __launch_bounds__(32 * kWarps) attn_sigmoid_kernel(SigmoidAttnArgs a) {
  pdl_wait();
  extern __shared__ float sm[];
  const int seg = blockIdx.y, RQ = a.rq;
  const int len = a.seg_len[seg];
  const int i0 = blockIdx.x * RQ;
  if (i0 >= len) return;
  const int H = a.H, G = a.G, dim = a.dim, vdim = a.vdim, dimp = dim + 1;
  float* qs = sm;                                   // [RQ][H][dim]
  float* ks = qs + (size_t)RQ * H * dim;            // [G][32][dim + 1]
  float* vs = ks + (size_t)G * kKeys * dimp;        // [G][32][vdim]
  float* wt = vs + (size_t)G * kKeys * vdim;        // [RQ][H][32] sigmoid weights
  float* mx = wt + (size_t)RQ * H * kKeys;          // [RQ][H][32] mixed weights
  float* acc = mx + (size_t)RQ * H * kKeys;         // [RQ][H][vdim]
  float* tk = acc + (size_t)RQ * H * vdim;          // [H][H]
  float* pb = tk + (size_t)H * H;                   // [H]
  float* srow = pb + H;                             // [RQ] score scale of the row (scale * temperature)
  const T* q = (const T*)a.q;
  const T* k_pool = (const T*)a.k_pool;
  const T* v_pool = (const T*)a.v_pool;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wpr = kWarps / RQ, r = warp / wpr, sub = warp % wpr;
  const int slot = a.seg_slot[seg], pos0 = a.seg_pos0[seg];
  const int64_t row0 = a.seg_start[seg];
  const int rows = min(RQ, len - i0);
  const int last_pos = pos0 + i0 + rows - 1;        // the last key any row of the CTA sees

  for (int e = tid; e < RQ * H * dim; e += blockDim.x) {
    const int rr = e / (H * dim);
    qs[e] = rr < rows ? cvt(q[(row0 + i0) * H * dim + e]) : 0.f;
  }
  for (int e = tid; e < RQ * H * vdim; e += blockDim.x) acc[e] = 0.f;
  for (int e = tid; e < H * H; e += blockDim.x) tk[e] = a.talk ? a.talk[e] : ((e / H == e % H) ? 1.f : 0.f);
  for (int e = tid; e < H; e += blockDim.x) pb[e] = a.head_bias ? a.head_bias[e] : 0.f;
  if (tid < RQ) {
    float t = 1.f;
    if (a.temp_coef != 0.f)
      t = 1.f + a.temp_coef * (float)log(floor((double)(pos0 + i0 + tid + 1) / (double)a.temp_every) + 1.0);
    srow[tid] = a.scale * t;
  }
  const int my_pos = pos0 + i0 + r;                 // position of this warp's row (r < rows: a real row)
  const int rep = H / G;
  const int n_tiles = last_pos / kKeys + 1;
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int k0 = kt * kKeys;
    __syncthreads();                                // the previous tile's readers are done (and the setup above is visible)
    const int page = a.block_table[(int64_t)slot * a.max_blocks + k0 / a.page_size];
    const int in_page = k0 % a.page_size;
    for (int e = tid; e < G * kKeys * dim; e += blockDim.x) {
      const int g = e / (kKeys * dim), rest = e - g * kKeys * dim, j = rest / dim, d = rest - j * dim;
      ks[((size_t)g * kKeys + j) * dimp + d] =
          k0 + j <= last_pos ? cvt(k_pool[(((int64_t)page * G + g) * a.page_size + in_page + j) * dim + d]) : 0.f;
    }
    for (int e = tid; e < G * kKeys * vdim; e += blockDim.x) {
      const int g = e / (kKeys * vdim), rest = e - g * kKeys * vdim, j = rest / vdim;
      vs[e] = k0 + j <= last_pos ? cvt(v_pool[(((int64_t)page * G + g) * a.page_size + in_page) * vdim + rest]) : 0.f;
    }
    __syncthreads();
    // (1) weights: lane = key
    const bool seen = r < rows && k0 + lane <= my_pos;
    for (int h = sub; h < H; h += wpr) {
      const float* qh = qs + ((size_t)r * H + h) * dim;
      const float* kj = ks + ((size_t)(h / rep) * kKeys + lane) * dimp;
      float s0 = 0.f, s1 = 0.f;
      int d = 0;
      for (; d + 1 < dim; d += 2) { s0 = fmaf(qh[d], kj[d], s0); s1 = fmaf(qh[d + 1], kj[d + 1], s1); }
      if (d < dim) s0 = fmaf(qh[d], kj[d], s0);
      float s = (s0 + s1) * srow[r];
      if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
      wt[((size_t)r * H + h) * kKeys + lane] = seen ? 1.f / (1.f + expf(-(s + pb[h]))) : 0.f;
    }
    __syncthreads();
    // (2) mix over the heads
    for (int h = sub; h < H; h += wpr) {
      float m = 0.f;
      for (int g = 0; g < H; ++g) m = fmaf(tk[h * H + g], wt[((size_t)r * H + g) * kKeys + lane], m);
      mx[((size_t)r * H + h) * kKeys + lane] = m;
    }
    __syncthreads();
    // (3) weighted values: lane = value channel
    if (r < rows) {
      const int nk = min(kKeys, my_pos - k0 + 1);   // keys of this tile the row sees (<= 0: none)
      for (int h = sub; h < H; h += wpr) {
        const float* mh = mx + ((size_t)r * H + h) * kKeys;
        const float* vh = vs + (size_t)(h / rep) * kKeys * vdim;
        float* ah = acc + ((size_t)r * H + h) * vdim;
        for (int e = lane; e < vdim; e += 32) {
          float o = ah[e];
          for (int j = 0; j < nk; ++j) o = fmaf(mh[j], vh[j * vdim + e], o);
          ah[e] = o;
        }
      }
    }
  }
  __syncthreads();
  TOUT* out = (TOUT*)a.out;
  for (int e = tid; e < rows * H * vdim; e += blockDim.x) put(out, (row0 + i0) * H * vdim + e, acc[e]);
}

}  // namespace
}  // namespace prl

using namespace prl;

// q [n][H][dim] and the pools in fp32 (f32) or bf16; head_bias [H] and talk [H][H] fp32 (NULL: no bias / no mixing);
// out [n][H][vdim] in the cache's element type (out_is_t) or fp32.  temp_coef == 0: no query temperature.
extern "C" int prl_attn_sigmoid(const void* q, const void* k_pool, const void* v_pool, int32_t f32, const int32_t* block_table,
                                int32_t max_blocks, int32_t page_size, const int32_t* seg_start, const int32_t* seg_len,
                                const int32_t* seg_pos0, const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H,
                                int32_t G, int32_t dim, int32_t vdim, float scale, float softcap, float temp_coef,
                                float temp_every, const float* head_bias, const float* talk, int32_t out_is_t, void* out,
                                prl_stream_t st) {
  PRL_CHECK_ARG(q && k_pool && v_pool && block_table && seg_start && seg_len && seg_pos0 && seg_slot && out,
                "prl_attn_sigmoid: NULL argument");
  PRL_CHECK_ARG(n_seg >= 1 && n_seg <= 65535 && max_q >= 1 && H >= 1 && G >= 1 && H % G == 0 && dim >= 1 && vdim >= 1 &&
                page_size >= kKeys && page_size % kKeys == 0 && max_blocks >= 1 && softcap >= 0.f &&
                (temp_coef == 0.f || temp_every > 0.f),
                "prl_attn_sigmoid: bad shape (H=%d G=%d dim=%d vdim=%d page=%d)", H, G, dim, vdim, page_size);
  int rq = 8;
  while (rq > 1 && rq / 2 >= max_q) rq /= 2;                                   // short segments: more warps per row
  const size_t budget = 200 * 1024;
  while (rq > 1 && sigmoid_attn_floats(rq, H, G, dim, vdim) * sizeof(float) > budget) rq /= 2;
  const size_t smem = sigmoid_attn_floats(rq, H, G, dim, vdim) * sizeof(float);
  PRL_CHECK_ARG(smem <= budget, "prl_attn_sigmoid: %d heads of %d + %d channels do not fit in shared memory", H, dim, vdim);
  SigmoidAttnArgs a{q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                    H, G, dim, vdim, scale, softcap, temp_coef, temp_every, head_bias, talk, rq, out};
  dim3 grid((max_q + rq - 1) / rq, n_seg);
  cudaStream_t s = (cudaStream_t)st;
  static SmemAttr attr[3] = {};
#define PRL_SIG(T, TOUT, I)                                                                        \
  do {                                                                                             \
    PRL_CUDA(ensure_smem((attn_sigmoid_kernel<T, TOUT>), (int)smem, attr[I]));                     \
    PRL_CUDA(launch_pdl((attn_sigmoid_kernel<T, TOUT>), grid, dim3(32 * kWarps), smem, s, a));     \
  } while (0)
  if (f32) PRL_SIG(float, float, 0);
  else if (out_is_t) PRL_SIG(__nv_bfloat16, __nv_bfloat16, 1);
  else PRL_SIG(__nv_bfloat16, float, 2);
#undef PRL_SIG
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}
