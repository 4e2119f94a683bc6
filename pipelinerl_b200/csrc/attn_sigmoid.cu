// Causal attention WITHOUT a softmax over a paged KV cache, with the heads' weights mixed by a matrix:
//
//     s_h(i, j)  = (q_h(i) . k_c(h)(j)) * scale * temp(pos_i),     temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)
//     s_h       <- cap * tanh(s_h / cap)                           (cap > 0)
//     w_h(i, j)  = sigmoid(s_h(i, j) + bias_h)  for j <= i, else 0 (never normalised over j)
//     m_h(i, j)  = sum_g talk[h][g] w_g(i, j)                      (talk NULL: m = w)
//     o_h(i)     = sum_j m_h(i, j) v_c(h)(j)                       c(h) = h / (H / G)
//
// The mixing couples all heads of a (query, key) pair, so a CTA owns RQ query rows of one segment with ALL their heads.
// It streams the sequence's keys and values in tiles of 32 (all G key/value heads at once, or one at a time when they
// do not fit; converted to fp32) through shared memory.  Per tile: (1) every (row, head) scores the 32 keys, one key per lane, and stores the sigmoid weights;
// (2) the weights are mixed over the heads; (3) every (row, head) adds the tile's weighted values to its accumulator,
// which lives in shared memory ([RQ][H][vdim] fp32) because the head count is a run-time number.  The eight warps of
// a CTA are split evenly over the RQ rows; the warps of a row take its heads in turn.  RQ is chosen at launch
// (8, 4, 2 or 1: what the segment lengths ask for and shared memory holds).  Key tiles start at absolute multiples
// of 32 and every sum runs in ascending key order, so a token's result does not depend on how its prompt was cut or
// batched.  Everything is fp32; T is only the storage type of q, the cache and (optionally) the output.
//
// Tensor-core variant (bf16 cache, dim and vdim multiples of 16, vdim <= 128): CTA = eight warps on ONE tile of 16
// query rows with all heads.  Per key tile of 32: (1) the warps take the source heads in turn, S = Q K^T by mma.sync
// m16n8k16 with operands read by ldmatrix from padded rows, temperature, cap, bias, sigmoid and mask in fp32, the
// weights to shared memory ([H][16][32] fp32); (2) every warp mixes the weights of its own output heads (a dot product
// over the source heads per element, read in the A-operand layout of the next product) and rounds them to bf16;
// (3) O += M V on the tensor cores, the accumulators of the warp's output heads in registers.  More output heads than
// eight warps hold are split over CTAs that repeat the scores.  When the queries of all heads do not fit in shared memory
// beside the tiles (32 heads of 128), their fragments are read from L2 in every tile instead.  A batch of short segments (a decode step) spreads the
// key tiles of a segment over several CTAs: nothing is normalised, so their shares are simply added, by a second
// launch in a fixed order.
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
  int kv_stage;          // CUDA-core kernel: key / value heads staged at a time (G, or 1 when all of them do not fit)
};

__host__ __device__ inline size_t sigmoid_attn_floats(int rq, int H, int G, int dim, int vdim) {   // G: heads staged at a time
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
  const int GS = a.kv_stage;                        // key / value heads in shared memory at a time
  float* qs = sm;                                   // [RQ][H][dim]
  float* ks = qs + (size_t)RQ * H * dim;            // [GS][32][dim + 1]
  float* vs = ks + (size_t)GS * kKeys * dimp;       // [GS][32][vdim]
  float* wt = vs + (size_t)GS * kKeys * vdim;       // [RQ][H][32] sigmoid weights
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
    const int page = a.block_table[(int64_t)slot * a.max_blocks + k0 / a.page_size];
    const int in_page = k0 % a.page_size;
    const bool seen = r < rows && k0 + lane <= my_pos;
    // (1) weights, the key heads staged GS at a time: lane = key
    for (int c0 = 0; c0 < G; c0 += GS) {
      __syncthreads();                              // the previous readers of ks are done (and the setup above is visible)
      for (int e = tid; e < GS * kKeys * dim; e += blockDim.x) {
        const int g = e / (kKeys * dim), rest = e - g * kKeys * dim, j = rest / dim, d = rest - j * dim;
        ks[((size_t)g * kKeys + j) * dimp + d] =
            k0 + j <= last_pos ? cvt(k_pool[(((int64_t)page * G + c0 + g) * a.page_size + in_page + j) * dim + d]) : 0.f;
      }
      __syncthreads();
      for (int h = c0 * rep + sub; h < (c0 + GS) * rep; h += wpr) {
        const float* qh = qs + ((size_t)r * H + h) * dim;
        const float* kj = ks + ((size_t)(h / rep - c0) * kKeys + lane) * dimp;
        float s0 = 0.f, s1 = 0.f;
        int d = 0;
        for (; d + 1 < dim; d += 2) { s0 = fmaf(qh[d], kj[d], s0); s1 = fmaf(qh[d + 1], kj[d + 1], s1); }
        if (d < dim) s0 = fmaf(qh[d], kj[d], s0);
        float s = (s0 + s1) * srow[r];
        if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        wt[((size_t)r * H + h) * kKeys + lane] = seen ? 1.f / (1.f + expf(-(s + pb[h]))) : 0.f;
      }
    }
    __syncthreads();
    // (2) mix over the heads
    for (int h = sub; h < H; h += wpr) {
      float m = 0.f;
      for (int g = 0; g < H; ++g) m = fmaf(tk[h * H + g], wt[((size_t)r * H + g) * kKeys + lane], m);
      mx[((size_t)r * H + h) * kKeys + lane] = m;
    }
    // (3) weighted values, the value heads staged likewise: lane = value channel
    const int nk = min(kKeys, my_pos - k0 + 1);     // keys of this tile the row sees (<= 0: none)
    for (int c0 = 0; c0 < G; c0 += GS) {
      __syncthreads();                              // mx is written; the previous readers of vs are done
      for (int e = tid; e < GS * kKeys * vdim; e += blockDim.x) {
        const int g = e / (kKeys * vdim), rest = e - g * kKeys * vdim, j = rest / vdim;
        vs[e] = k0 + j <= last_pos ? cvt(v_pool[(((int64_t)page * G + c0 + g) * a.page_size + in_page) * vdim + rest]) : 0.f;
      }
      __syncthreads();
      if (r < rows) {
        for (int h = c0 * rep + sub; h < (c0 + GS) * rep; h += wpr) {
          const float* mh = mx + ((size_t)r * H + h) * kKeys;
          const float* vh = vs + (size_t)(h / rep - c0) * kKeys * vdim;
          float* ah = acc + ((size_t)r * H + h) * vdim;
          for (int e = lane; e < vdim; e += 32) {
            float o = ah[e];
            for (int j = 0; j < nk; ++j) o = fmaf(mh[j], vh[j * vdim + e], o);
            ah[e] = o;
          }
        }
      }
    }
  }
  __syncthreads();
  TOUT* out = (TOUT*)a.out;
  for (int e = tid; e < rows * H * vdim; e += blockDim.x) put(out, (row0 + i0) * H * vdim + e, acc[e]);
}


// ---- tensor-core variant -------------------------------------------------------------------------------------------
typedef __nv_bfloat16 bf16;
constexpr int kTcRows = 16;      // query rows per CTA: one m16 tile
constexpr int kTcWarps = 8;
constexpr int kPadH = 8;         // padding halves per staged row (ldmatrix reads stay conflict-free)
constexpr int kWtLd = 40;        // floats per row of a weight tile (32 keys + padding: 64-bit accesses of a half-warp spread over the banks)

__device__ __forceinline__ void cp16z(void* dst, const void* src, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

struct SigmoidTcArgs {
  SigmoidAttnArgs a;
  int splits;            // CTAs that share the key tiles of a row tile (their shares go to ws and are added afterwards)
  int64_t n_rows;        // rows of the batch: the stride between the splits' shares in ws
  float* ws;             // [splits][n_rows][H][vdim] fp32 when splits > 1
  int q_global;          // the queries of all heads do not fit in shared memory beside the tiles: their fragments come from L2
};

__host__ __device__ inline size_t sigmoid_tc_smem(int H, int G, int dim, int vdim, bool q_staged = true) {
  return ((q_staged ? (size_t)kTcRows * (H * dim + kPadH) : 0) + (size_t)G * kKeys * (dim + kPadH) + (size_t)G * kKeys * (vdim + kPadH)) * sizeof(bf16) +
         ((size_t)H * kTcRows * kWtLd + (size_t)H * H + H + kTcRows) * sizeof(float);
}

// Output heads per warp for a value size: as many as 128 accumulator registers per thread hold, at most 8
__host__ __device__ constexpr int sigmoid_tc_hpw(int vdim) { return 256 / vdim > 8 ? 8 : 256 / vdim; }

// NV = vdim / 8 accumulator tiles per head, HPW output heads per warp (NV * HPW <= 32: 128 accumulator registers)
template <int NV, int HPW>
__global__ void __launch_bounds__(32 * kTcWarps, 1) attn_sigmoid_tc_kernel(SigmoidTcArgs ta) {
  pdl_wait();
  const SigmoidAttnArgs& a = ta.a;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int seg = blockIdx.y;
  const int len = a.seg_len[seg];
  const int i0 = blockIdx.x * kTcRows;
  if (i0 >= len) return;
  const int split = blockIdx.z % ta.splits, hgroup = blockIdx.z / ta.splits;
  const int H = a.H, G = a.G, dim = a.dim;
  constexpr int vdim = NV * 8;
  const int ldq = H * dim + kPadH, ldk = dim + kPadH, ldv = vdim + kPadH;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][ldq]: all heads of the CTA's rows
  bf16* Ks = Qs + (ta.q_global ? 0 : kTcRows * ldq);            // [G][32][ldk]
  bf16* Vs = Ks + (size_t)G * kKeys * ldk;                      // [G][32][ldv]
  float* Wt = reinterpret_cast<float*>(Vs + (size_t)G * kKeys * ldv);   // [H][16][kWtLd] sigmoid weights of the tile
  float* tk = Wt + (size_t)H * kTcRows * kWtLd;                 // [H][H]
  float* pb = tk + H * H;                                       // [H]
  float* srow = pb + H;                                         // [16] score scale of the row (scale * temperature)
  const bf16* q = (const bf16*)a.q;
  const bf16* k_pool = (const bf16*)a.k_pool;
  const bf16* v_pool = (const bf16*)a.v_pool;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = a.seg_slot[seg], pos0 = a.seg_pos0[seg];
  const int64_t row0 = a.seg_start[seg];
  const int rows = min(kTcRows, len - i0);
  const int last_pos = pos0 + i0 + rows - 1;
  const int32_t* bt = a.block_table + (int64_t)slot * a.max_blocks;
  const int tiles_total = last_pos / kKeys + 1;
  const int per = (tiles_total + ta.splits - 1) / ta.splits;
  const int t_begin = split * per, t_end = min(tiles_total, t_begin + per);

  const int chq = ta.q_global ? 0 : H * dim / 8;
  for (int c = tid; c < kTcRows * chq; c += blockDim.x) {
    const int r = c / chq, cc = c - r * chq;
    const bool ok = r < rows;
    cp16z(Qs + r * ldq + cc * 8, q + (row0 + i0 + (ok ? r : 0)) * H * dim + cc * 8, ok ? 16 : 0);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int e = tid; e < H * H; e += blockDim.x) tk[e] = a.talk ? a.talk[e] : 0.f;
  for (int e = tid; e < H; e += blockDim.x) pb[e] = a.head_bias ? a.head_bias[e] : 0.f;
  if (tid < kTcRows) {
    float t = 1.f;
    if (a.temp_coef != 0.f)
      t = 1.f + a.temp_coef * (float)log(floor((double)(pos0 + i0 + tid + 1) / (double)a.temp_every) + 1.0);
    srow[tid] = a.scale * t;
  }
  const int gid = lane >> 2, t2 = (lane & 3) * 2;
  const int pos_r[2] = {gid < rows ? pos0 + i0 + gid : -1, gid + 8 < rows ? pos0 + i0 + gid + 8 : -1};   // -1: no such row
  const int rep = H / G;
  const int h_base = (hgroup * kTcWarps + warp) * HPW;          // this warp's output heads: h_base .. h_base + HPW - 1
  float o[HPW][NV][4];
#pragma unroll
  for (int i = 0; i < HPW; ++i)
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[i][j][e] = 0.f;

  const int chk = dim / 8, chv = vdim / 8;
  // The K and V tiles are copied as groups of their own: V of a tile arrives while its scores are formed, K of the next
  // tile while this tile's weights meet the values.
  auto stage_k = [&](int t) {
    if (t < t_end) {
      const int k0 = t * kKeys;
      const int64_t page = bt[k0 / a.page_size];
      const int in_page = k0 % a.page_size;
      for (int c = tid; c < G * kKeys * chk; c += blockDim.x) {
        const int row = c / chk, cc = c - row * chk, g = row / kKeys, j = row - g * kKeys;
        const bool ok = k0 + j <= last_pos;
        cp16z(Ks + (size_t)row * ldk + cc * 8, k_pool + ((page * G + g) * a.page_size + in_page + (ok ? j : 0)) * dim + cc * 8, ok ? 16 : 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto stage_v = [&](int t) {
    const int k0 = t * kKeys;
    const int64_t page = bt[k0 / a.page_size];
    const int in_page = k0 % a.page_size;
    for (int c = tid; c < G * kKeys * chv; c += blockDim.x) {
      const int row = c / chv, cc = c - row * chv, g = row / kKeys, j = row - g * kKeys;
      const bool ok = k0 + j <= last_pos;
      cp16z(Vs + (size_t)row * ldv + cc * 8, v_pool + ((page * G + g) * a.page_size + in_page + (ok ? j : 0)) * vdim + cc * 8, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage_k(t_begin);
  for (int t = t_begin; t < t_end; ++t) {
    const int k0 = t * kKeys;
    __syncthreads();                                            // the previous tile's values are read
    stage_v(t);
    asm volatile("cp.async.wait_group 1;" ::: "memory");        // the queries and this tile's keys are here
    __syncthreads();
    // (1) the sigmoid weights of the source heads, 16 rows x 32 keys each
    for (int g = warp; g < H; g += kTcWarps) {
      float s[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
      const bf16* qa = Qs + (lane & 15) * ldq + g * dim + (lane >> 4) * 8;
      // without staged queries: the A fragment's four registers straight from the query rows (rows gid, gid + 8; the
      // row past the segment's end reads row 0 and is masked below)
      const bf16* qg0 = q + ((row0 + i0 + (gid < rows ? gid : 0)) * H + g) * dim + t2;
      const bf16* qg1 = q + ((row0 + i0 + (gid + 8 < rows ? gid + 8 : 0)) * H + g) * dim + t2;
      const bf16* kb = Ks + ((size_t)(g / rep) * kKeys + ((lane >> 4) << 3) + (lane & 7)) * ldk + ((lane >> 3) & 1) * 8;
      for (int c = 0; c < dim; c += 16) {
        uint32_t af[4], b01[4], b23[4];
        if (ta.q_global) {
          af[0] = *reinterpret_cast<const uint32_t*>(qg0 + c);
          af[1] = *reinterpret_cast<const uint32_t*>(qg1 + c);
          af[2] = *reinterpret_cast<const uint32_t*>(qg0 + c + 8);
          af[3] = *reinterpret_cast<const uint32_t*>(qg1 + c + 8);
        } else {
          ldsm4(af, qa + c);
        }
        ldsm4(b01, kb + c);                 // keys 0..15: (b0, b1) of n-tile 0, (b0, b1) of n-tile 1
        ldsm4(b23, kb + 16 * ldk + c);      // keys 16..31
        mma16816(s[0], af, b01[0], b01[1]);
        mma16816(s[1], af, b01[2], b01[3]);
        mma16816(s[2], af, b23[0], b23[1]);
        mma16816(s[3], af, b23[2], b23[3]);
      }
      const float bias = pb[g], cap_inv = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
      float* wg = Wt + (size_t)g * kTcRows * kWtLd;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float w[2] = {0.f, 0.f};
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const int key = k0 + 8 * j + t2 + b;
            if (key <= pos_r[u]) {                              // (no such row: pos_r = -1)
              float v = s[j][2 * u + b] * srow[gid + 8 * u];
              // tanh(x) = 1 - 2 / (e^(2x) + 1) and the sigmoid through the exponential unit: absolute errors of a few
              // 1e-7, far below the bf16 rounding of the weights that follows
              if (a.softcap > 0.f) v = a.softcap * (1.f - __fdividef(2.f, __expf(2.f * v * cap_inv) + 1.f));
              w[b] = __fdividef(1.f, 1.f + __expf(-(v + bias)));
            }
          }
          *reinterpret_cast<float2*>(wg + (gid + 8 * u) * kWtLd + 8 * j + t2) = make_float2(w[0], w[1]);
        }
    }
    __syncthreads();                                            // the weights are written, the keys are read
    stage_k(t + 1);
    asm volatile("cp.async.wait_group 1;" ::: "memory");        // this tile's values are here
    __syncthreads();
    // (2) + (3) this warp's output heads: mix, round, multiply with the values
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      const int h = h_base + i;
      if (h >= H) break;                                        // warp-uniform
      float m[2][4][2];                                         // [16-key step][A-operand register][pair]
      const int at = gid * kWtLd + t2;
      if (a.talk) {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
          for (int x = 0; x < 4; ++x) m[kk][x][0] = m[kk][x][1] = 0.f;
        for (int g = 0; g < H; ++g) {
          const float coef = tk[h * H + g];
          const float* wg = Wt + (size_t)g * kTcRows * kWtLd + at;
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
#pragma unroll
            for (int x = 0; x < 4; ++x) {                       // x: (row gid, keys +0), (gid + 8, +0), (gid, +8), (gid + 8, +8)
              const float2 w = *reinterpret_cast<const float2*>(wg + (x & 1) * 8 * kWtLd + 16 * kk + (x >> 1) * 8);
              m[kk][x][0] = fmaf(coef, w.x, m[kk][x][0]);
              m[kk][x][1] = fmaf(coef, w.y, m[kk][x][1]);
            }
        }
      } else {
        const float* wg = Wt + (size_t)h * kTcRows * kWtLd + at;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float2 w = *reinterpret_cast<const float2*>(wg + (x & 1) * 8 * kWtLd + 16 * kk + (x >> 1) * 8);
            m[kk][x][0] = w.x;
            m[kk][x][1] = w.y;
          }
      }
      const bf16* vb = Vs + ((size_t)(h / rep) * kKeys + ((lane >> 3) & 1) * 8 + (lane & 7)) * ldv + (lane >> 4) * 8;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        uint32_t pf[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) pf[x] = pack_bf16(m[kk][x][0], m[kk][x][1]);
#pragma unroll
        for (int j = 0; j < NV; j += 2) {
          uint32_t vf[4];
          ldsm4_t(vf, vb + kk * 16 * ldv + j * 8);
          mma16816(o[i][j], pf, vf[0], vf[1]);
          mma16816(o[i][j + 1], pf, vf[2], vf[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");          // a CTA without tiles still has its query copies in flight
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int h = h_base + i;
    if (h >= H) break;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (gid + 8 * u >= rows) continue;
      const int64_t at = ((row0 + i0 + gid + 8 * u) * H + h) * vdim + t2;
      if (ta.splits == 1) {
        bf16* dst = reinterpret_cast<bf16*>(a.out) + at;
#pragma unroll
        for (int j = 0; j < NV; ++j) *reinterpret_cast<uint32_t*>(dst + 8 * j) = pack_bf16(o[i][j][2 * u], o[i][j][2 * u + 1]);
      } else {
        float* dst = ta.ws + (int64_t)split * ta.n_rows * H * vdim + at;
#pragma unroll
        for (int j = 0; j < NV; ++j) *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(o[i][j][2 * u], o[i][j][2 * u + 1]);
      }
    }
  }
}

// out[e] = bf16(sum over the splits of ws[split][e]) in split order
__global__ void attn_sigmoid_merge_kernel(const float* __restrict__ ws, int64_t n, int splits, bf16* __restrict__ out) {
  pdl_wait();
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  float v = 0.f;
  for (int z = 0; z < splits; ++z) v += ws[z * n + e];
  out[e] = __float2bfloat16_rn(v);
}

}  // namespace
}  // namespace prl

using namespace prl;

// 1 if the tensor-core kernel runs this geometry in bf16 (else prl_attn_sigmoid takes the CUDA-core kernel)
extern "C" int32_t prl_attn_sigmoid_tc_fits(int32_t H, int32_t G, int32_t dim, int32_t vdim) {
  return H >= 1 && G >= 1 && H % G == 0 && dim >= 16 && dim % 16 == 0 && vdim >= 16 && vdim % 16 == 0 && vdim <= 128 &&
         sigmoid_tc_smem(H, G, dim, vdim, false) <= 226 * 1024;
}

// CTAs that share the key tiles of a row tile when the batch has fewer row tiles than the GPU has SMs (a decode step, a
// short prompt portion), and the fp32 workspace their shares need: [splits][n_rows][H][vdim]
static int sigmoid_splits(int n_seg, int max_q, int H, int vdim) {
  const int per_cta = kTcWarps * sigmoid_tc_hpw(vdim);          // output heads one CTA holds
  const int64_t units = (int64_t)n_seg * ((max_q + kTcRows - 1) / kTcRows) * ((H + per_cta - 1) / per_cta);
  const int64_t s = num_sms() / (units > 0 ? units : 1);
  return s < 1 ? 1 : (s > 8 ? 8 : (int)s);
}
extern "C" size_t prl_attn_sigmoid_workspace_bytes(int32_t n_rows, int32_t n_seg, int32_t max_q, int32_t H, int32_t vdim) {
  const int splits = sigmoid_splits(n_seg, max_q, H, vdim);
  return splits > 1 ? (size_t)splits * n_rows * H * vdim * sizeof(float) : 0;
}

// q [n][H][dim] and the pools in fp32 (f32) or bf16; head_bias [H] and talk [H][H] fp32 (NULL: no bias / no mixing);
// out [n][H][vdim] in the cache's element type (out_is_t) or fp32.  temp_coef == 0: no query temperature.
// allow_tc: bf16 with out_is_t and a geometry of prl_attn_sigmoid_tc_fits takes the tensor-core kernel; a batch with few
// row tiles then splits their keys over CTAs if ws holds prl_attn_sigmoid_workspace_bytes (n_rows = rows of q and out).
extern "C" int prl_attn_sigmoid(const void* q, const void* k_pool, const void* v_pool, int32_t f32, const int32_t* block_table,
                                int32_t max_blocks, int32_t page_size, const int32_t* seg_start, const int32_t* seg_len,
                                const int32_t* seg_pos0, const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H,
                                int32_t G, int32_t dim, int32_t vdim, float scale, float softcap, float temp_coef,
                                float temp_every, const float* head_bias, const float* talk, int32_t out_is_t, void* out,
                                int32_t n_rows, int32_t allow_tc, void* ws, size_t ws_bytes, prl_stream_t st) {
  PRL_CHECK_ARG(q && k_pool && v_pool && block_table && seg_start && seg_len && seg_pos0 && seg_slot && out,
                "prl_attn_sigmoid: NULL argument");
  PRL_CHECK_ARG(n_seg >= 1 && n_seg <= 65535 && max_q >= 1 && H >= 1 && G >= 1 && H % G == 0 && dim >= 1 && vdim >= 1 &&
                page_size >= kKeys && page_size % kKeys == 0 && max_blocks >= 1 && softcap >= 0.f &&
                (temp_coef == 0.f || temp_every > 0.f),
                "prl_attn_sigmoid: bad shape (H=%d G=%d dim=%d vdim=%d page=%d)", H, G, dim, vdim, page_size);
  cudaStream_t s = (cudaStream_t)st;
  if (!f32 && out_is_t && allow_tc && prl_attn_sigmoid_tc_fits(H, G, dim, vdim) &&
      ((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0) && ((uintptr_t)out & 3) == 0) {
    const int per_cta = kTcWarps * sigmoid_tc_hpw(vdim);
    const int groups = (H + per_cta - 1) / per_cta;
    int splits = sigmoid_splits(n_seg, max_q, H, vdim);
    if (!ws || n_rows < 1 || ws_bytes < prl_attn_sigmoid_workspace_bytes(n_rows, n_seg, max_q, H, vdim)) splits = 1;
    SigmoidTcArgs ta{{q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                      H, G, dim, vdim, scale, softcap, temp_coef, temp_every, head_bias, talk, 0, out, G},
                     splits, (int64_t)n_rows, (float*)ws, 0};
    ta.q_global = sigmoid_tc_smem(H, G, dim, vdim) > 200 * 1024;
    const size_t smem = sigmoid_tc_smem(H, G, dim, vdim, !ta.q_global);
    dim3 grid((max_q + kTcRows - 1) / kTcRows, n_seg, splits * groups);
    static SmemAttr attr[8] = {};
#define PRL_SIGTC(NV)                                                                                               \
  case NV * 8:                                                                                                      \
    PRL_CUDA(ensure_smem((attn_sigmoid_tc_kernel<NV, sigmoid_tc_hpw(NV * 8)>), (int)smem, attr[NV / 2 - 1]));       \
    PRL_CUDA(launch_pdl((attn_sigmoid_tc_kernel<NV, sigmoid_tc_hpw(NV * 8)>), grid, dim3(32 * kTcWarps), smem, s, ta)); \
    break
    switch (vdim) {
      PRL_SIGTC(2); PRL_SIGTC(4); PRL_SIGTC(6); PRL_SIGTC(8); PRL_SIGTC(10); PRL_SIGTC(12); PRL_SIGTC(14); PRL_SIGTC(16);
    }
#undef PRL_SIGTC
    PRL_LAUNCH_CHECK();
    if (splits > 1) {
      const int64_t n = (int64_t)n_rows * H * vdim;
      PRL_CUDA(launch_pdl(attn_sigmoid_merge_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, s, (const float*)ws, n,
                          splits, (bf16*)out));
      PRL_LAUNCH_CHECK();
    }
    return PRL_OK;
  }
  int rq = 8;
  while (rq > 1 && rq / 2 >= max_q) rq /= 2;                                   // short segments: more warps per row
  const size_t budget = 200 * 1024;
  while (rq > 1 && sigmoid_attn_floats(rq, H, G, dim, vdim) * sizeof(float) > budget) rq /= 2;
  int kv_stage = G;                                 // all key / value heads of a tile at once, or one at a time
  if (sigmoid_attn_floats(rq, H, G, dim, vdim) * sizeof(float) > budget) {
    kv_stage = 1;
    rq = 8;
    while (rq > 1 && rq / 2 >= max_q) rq /= 2;
    while (rq > 1 && sigmoid_attn_floats(rq, H, 1, dim, vdim) * sizeof(float) > budget) rq /= 2;
  }
  const size_t smem = sigmoid_attn_floats(rq, H, kv_stage, dim, vdim) * sizeof(float);
  PRL_CHECK_ARG(smem <= budget, "prl_attn_sigmoid: %d heads of %d + %d channels do not fit in shared memory", H, dim, vdim);
  SigmoidAttnArgs a{q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                    H, G, dim, vdim, scale, softcap, temp_coef, temp_every, head_bias, talk, rq, out, kv_stage};
  dim3 grid((max_q + rq - 1) / rq, n_seg);
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
