// Tensor-core attention over a latent cache (bf16): every query head of a token attends to the SAME key rows
// [latent (rank) | rotated shared part (rot)] of size kd = rank + rot, and the values are the first `rank` channels of
// those rows, so a staged key tile is also the value tile.  Since the heads share their keys, the H heads of a token
// are stacked into the M dimension of the products: the query buffer [n][H][kd] is read as a matrix of n*H rows, row m
// belonging to token m / H and head m % H.  A per-head sink logit (optional) joins the softmax denominator only.
//
// Work unit = 16 stacked rows (one m16 tile of mma.sync m16n8k16).  Keys are walked in tiles of 32 at absolute
// multiples of 32 (a tile lies inside one page, and the order of summation never depends on how a prompt was cut).
//   S = Q K^T   (bf16 in, fp32 out; Q and K read by ldmatrix from padded, conflict-free rows)
//   scale, causal mask, fp32 online softmax per row (the four lanes of a row exchange by shuffles)
//   O += P V    (P rounded to bf16 straight from the accumulator registers; V = the key tile read through ldmatrix.trans)
//
// Two kernels share the tile routine:
//   rows:  CTA = 4 warps = 4 consecutive work units of one segment; the CTA stages each key tile once (cp.async double
//          buffer) for all four.  Prompt portions.
//   split: CTA = 8 warps on ONE work unit; the warps take the key tiles round-robin, each staging its own tiles, and
//          their partial softmaxes are merged through shared memory.  Batches of single tokens (a decode step), where
//          a segment has only H stacked rows but thousands of keys.
#include "prl_common.cuh"
#include <math.h>

namespace prl {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int kKeys = 32;      // keys per tile
constexpr int kPadH = 8;       // padding halves per staged row
constexpr int kRowWarps = 4;
constexpr int kSplitWarps = 8;
constexpr float kNegBig = -1e30f;

__device__ __forceinline__ void cp16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
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

// Running softmax state of a thread: rows g = lane / 4 and g + 8 of the work unit, NV value n-tiles (8 channels each).
template <int NV>
struct Acc {
  float o[NV][4];
  float m[2], l[2];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    m[0] = m[1] = kNegBig;
    l[0] = l[1] = 0.f;
  }
};

// One key tile (32 keys starting at absolute key k0, rows Ks[key][ld]) against the warp's 16 stacked query rows Qs[16][ld].
// pos[i]: the position of the token of row g + 8 i (keys lo[i] .. pos[i] are visible; pos -1 hides everything: a padding
// row; lo is 0 without a sliding window, else pos - window + 1).
template <int NV>
__device__ __forceinline__ void tile_step(Acc<NV>& a, const bf16* Qs, const bf16* Ks, int ld, int kd, int rank, int k0,
                                          const int (&pos)[2], const int (&lo)[2], float scale, int lane) {
  float s[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
  const bf16* qa = Qs + (lane & 15) * ld + (lane >> 4) * 8;
  const bf16* kb = Ks + (((lane >> 4) << 3) + (lane & 7)) * ld + ((lane >> 3) & 1) * 8;
  for (int c = 0; c < kd; c += 16) {
    uint32_t af[4], b01[4], b23[4];
    ldsm4(af, qa + c);
    ldsm4(b01, kb + c);                 // keys 0..15: (b0, b1) of n-tile 0, (b0, b1) of n-tile 1
    ldsm4(b23, kb + 16 * ld + c);       // keys 16..31
    mma16816(s[0], af, b01[0], b01[1]);
    mma16816(s[1], af, b01[2], b01[3]);
    mma16816(s[2], af, b23[0], b23[1]);
    mma16816(s[3], af, b23[2], b23[3]);
  }
  const int t2 = (lane & 3) * 2;
  float mx[2] = {kNegBig, kNegBig};
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = k0 + 8 * j + t2 + (e & 1);
      const int i = e >> 1;
      const float v = (key <= pos[i] && key >= lo[i]) ? s[j][e] * scale : -INFINITY;
      s[j][e] = v;
      mx[i] = fmaxf(mx[i], v);
    }
  float corr[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    const float m_new = fmaxf(a.m[i], mx[i]);
    corr[i] = expf(a.m[i] - m_new);
    a.m[i] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      const float p = expf(s[j][e] - a.m[i]);         // exp(-inf) = 0 for hidden keys
      s[j][e] = p;
      sum[i] += p;
    }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
    sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
    a.l[i] = a.l[i] * corr[i] + sum[i];
  }
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    a.o[j][0] *= corr[0]; a.o[j][1] *= corr[0];
    a.o[j][2] *= corr[1]; a.o[j][3] *= corr[1];
  }
  // O += P V: two k-steps of 16 keys; V[key][channel] = Ks[key][channel], channel < rank
  const bf16* vb = Ks + (((lane >> 3) & 1) * 8 + (lane & 7)) * ld + (lane >> 4) * 8;
#pragma unroll
  for (int kk = 0; kk < 2; ++kk) {
    uint32_t pf[4];
    pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int j = 0; j < NV; j += 2) {
      if (j * 8 < rank) {
        uint32_t vf[4];
        ldsm4_t(vf, vb + kk * 16 * ld + j * 8);
        mma16816(a.o[j], pf, vf[0], vf[1]);
        mma16816(a.o[j + 1], pf, vf[2], vf[3]);
      }
    }
  }
}

// rows of the key tile starting at absolute key k0 of sequence `bt` into Ks (16-byte chunks spread over `nthr` threads);
// rows past `last_key` are zero-filled (their scores are masked, their values must not be NaN)
__device__ __forceinline__ void stage_keys(bf16* Ks, int ld, const bf16* pool, const int32_t* bt, int page_size, int kd, int k0,
                                           int last_key, int tid, int nthr) {
  const int ch = kd / 8;
  const int page = bt[k0 / page_size];
  const bf16* src = pool + ((int64_t)page * page_size + k0 % page_size) * kd;
  for (int i = tid; i < kKeys * ch; i += nthr) {
    const int r = i / ch, c = i - r * ch;
    if (k0 + r <= last_key) cp16(Ks + r * ld + c * 8, src + (int64_t)r * kd + c * 8);
    else *reinterpret_cast<uint4*>(Ks + r * ld + c * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <int NV>
__device__ __forceinline__ void finish_rows(Acc<NV>& a, const float* sink, int H, int rank, int m0, int m_total, int64_t row0,
                                            bf16* out, int lane) {
  const int g = lane >> 2, t2 = (lane & 3) * 2;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + g + 8 * i;
    if (m >= m_total) continue;
    float mm = a.m[i], l = a.l[i], corr = 1.f;
    if (sink) {
      const float sk = sink[m % H];
      const float m_new = fmaxf(mm, sk);
      corr = expf(mm - m_new);
      l = l * corr + expf(sk - m_new);
    }
    const float inv = corr / l;
    bf16* dst = out + (row0 * H + m) * rank;
#pragma unroll
    for (int j = 0; j < NV; ++j)
      if (j * 8 < rank)
        *reinterpret_cast<uint32_t*>(dst + j * 8 + t2) = pack_bf16(a.o[j][2 * i] * inv, a.o[j][2 * i + 1] * inv);
  }
}

template <int NV>
__global__ void __launch_bounds__(kRowWarps * 32) attn_latent_rows_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ pool, const int32_t* __restrict__ block_table, int max_blocks,
    int page_size, const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_len,
    const int32_t* __restrict__ seg_pos0, const int32_t* __restrict__ seg_slot, int H, int kd, int rank, float scale,
    int window, const float* __restrict__ sink, bf16* __restrict__ out) {
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int seg = blockIdx.y;
  const int len = seg_len[seg];
  const int m_total = len * H;
  const int cta_m0 = blockIdx.x * (kRowWarps * 16);
  if (cta_m0 >= m_total) return;
  const int ld = kd + kPadH, ch = kd / 8;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);               // [64][ld]
  bf16* Kb0 = Qs + kRowWarps * 16 * ld;                       // two key tiles of [32][ld]
  const int kb_step = kKeys * ld;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos0 = seg_pos0[seg], slot = seg_slot[seg];
  const int64_t row0 = seg_start[seg];
  const int32_t* bt = block_table + (int64_t)slot * max_blocks;
  const bf16* qsrc = q + (row0 * H + cta_m0) * kd;
  const int m_here = min(kRowWarps * 16, m_total - cta_m0);
  for (int i = tid; i < kRowWarps * 16 * ch; i += blockDim.x) {
    const int r = i / ch, c = i - r * ch;
    if (r < m_here) cp16(Qs + r * ld + c * 8, qsrc + (int64_t)r * kd + c * 8);
    else *reinterpret_cast<uint4*>(Qs + r * ld + c * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  const int last_key = pos0 + (cta_m0 + m_here - 1) / H;      // the CTA's last token sees keys 0 .. last_key
  const int n_tiles = last_key / kKeys + 1;
  // with a sliding window the CTA's first token hides the keys before first_key: whole tiles before it are skipped (the
  // others keep their absolute place, so the order of summation does not depend on the cutting of the prompt)
  const int first_key = window > 0 ? max(pos0 + cta_m0 / H - window + 1, 0) : 0;
  const int t_first = first_key / kKeys;
  stage_keys(Kb0, ld, pool, bt, page_size, kd, t_first * kKeys, last_key, tid, blockDim.x);
  cp_commit();
  const int m0 = cta_m0 + warp * 16, g = lane >> 2;
  int pos[2], lo[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    pos[i] = (m0 + g + 8 * i) < m_total ? pos0 + (m0 + g + 8 * i) / H : -1;
    lo[i] = window > 0 ? pos[i] - window + 1 : 0;
  }
  const int warp_last = m0 < m_total ? pos0 + min(m0 + 15, m_total - 1) / H : -1;      // warp-uniform: the warp's last visible key
  const int warp_first = (window > 0 && m0 < m_total) ? pos0 + m0 / H - window + 1 : 0;  // ... and its first
  Acc<NV> acc;
  acc.init();
  for (int t = t_first; t < n_tiles; ++t) {
    const int b = (t - t_first) & 1;
    if (t + 1 < n_tiles) stage_keys(Kb0 + (b ^ 1) * kb_step, ld, pool, bt, page_size, kd, (t + 1) * kKeys, last_key, tid, blockDim.x);
    cp_commit();
    cp_wait<1>();
    __syncthreads();
    if (t * kKeys <= warp_last && (t + 1) * kKeys > warp_first)
      tile_step<NV>(acc, Qs + warp * 16 * ld, Kb0 + b * kb_step, ld, kd, rank, t * kKeys, pos, lo, scale, lane);
    __syncthreads();
  }
  if (m0 < m_total) finish_rows<NV>(acc, sink, H, rank, m0, m_total, row0, out, lane);
}

template <int NV>
__global__ void __launch_bounds__(kSplitWarps * 32) attn_latent_split_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ pool, const int32_t* __restrict__ block_table, int max_blocks,
    int page_size, const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_len,
    const int32_t* __restrict__ seg_pos0, const int32_t* __restrict__ seg_slot, int H, int kd, int rank, float scale,
    int window, const float* __restrict__ sink, bf16* __restrict__ out, int splits, float* __restrict__ ws) {
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int seg = blockIdx.y, z = blockIdx.z;
  if (seg_len[seg] != 1) return;
  const int m_total = H, m0 = blockIdx.x * 16;
  const int ld = kd + kPadH, ch = kd / 8;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                       // [16][ld]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2;
  bf16* Ks = Qs + (16 + warp * kKeys) * ld;                           // this warp's own key tile
  const int pos_tok = seg_pos0[seg], slot = seg_slot[seg];
  const int64_t row0 = seg_start[seg];
  const int32_t* bt = block_table + (int64_t)slot * max_blocks;
  const int m_here = min(16, m_total - m0);
  for (int i = tid; i < 16 * ch; i += blockDim.x) {
    const int r = i / ch, c = i - r * ch;
    *reinterpret_cast<uint4*>(Qs + r * ld + c * 8) =
        r < m_here ? *reinterpret_cast<const uint4*>(q + (row0 * H + m0 + r) * kd + c * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  int pos[2], lo[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    pos[i] = (m0 + g + 8 * i) < m_total ? pos_tok : -1;
    lo[i] = window > 0 ? pos_tok - window + 1 : 0;
  }
  const int n_tiles = pos_tok / kKeys + 1;
  const int t_first = window > 0 ? max(pos_tok - window + 1, 0) / kKeys : 0;     // tiles before the window are skipped
  Acc<NV> acc;
  acc.init();
  for (int t = t_first + z * kSplitWarps + warp; t < n_tiles; t += kSplitWarps * splits) {     // CTA z of `splits` takes every splits-th turn
    __syncwarp();
    stage_keys(Ks, ld, pool, bt, page_size, kd, t * kKeys, pos_tok, lane, 32);
    cp_commit();
    cp_wait<0>();
    __syncwarp();
    tile_step<NV>(acc, Qs, Ks, ld, kd, rank, t * kKeys, pos, lo, scale, lane);
  }
  __syncthreads();                                                     // the key tiles are dead: their space holds the partials
  // partial of warp w: [16 rows][rank + 2] fp32 = o | m | l
  float* part = reinterpret_cast<float*>(Qs + 16 * ld);
  const int ps = rank + 2;
  float* mine = part + (int64_t)warp * 16 * ps;
  const int t2 = (lane & 3) * 2;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float* pr = mine + (g + 8 * i) * ps;
#pragma unroll
    for (int j = 0; j < NV; ++j)
      if (j * 8 < rank) { pr[j * 8 + t2] = acc.o[j][2 * i]; pr[j * 8 + t2 + 1] = acc.o[j][2 * i + 1]; }
    if ((lane & 3) == 0) { pr[rank] = acc.m[i]; pr[rank + 1] = acc.l[i]; }
  }
  __syncthreads();
  const bool last = splits == 1;                                       // else: this CTA's share goes to the workspace unnormalised
  float* wsp = ws ? ws + (((int64_t)seg * gridDim.x + blockIdx.x) * splits + z) * 16 * ps : nullptr;
  __shared__ float row_w[16][kSplitWarps + 2];                         // per row: the warps' weights | max | denominator
  if (tid < m_here) {                                                  // merge in warp order
    const int r = tid;
    float mx = (sink && last) ? sink[(m0 + r) % H] : kNegBig;
    for (int w = 0; w < kSplitWarps; ++w) mx = fmaxf(mx, part[((int64_t)w * 16 + r) * ps + rank]);
    float den = (sink && last) ? expf(sink[(m0 + r) % H] - mx) : 0.f;
    for (int w = 0; w < kSplitWarps; ++w) {
      const float* pr = part + ((int64_t)w * 16 + r) * ps;
      const float wgt = expf(pr[rank] - mx);                           // a warp without tiles: exp(-1e30 - mx) = 0
      row_w[r][w] = wgt;
      den = fmaf(wgt, pr[rank + 1], den);
    }
    row_w[r][kSplitWarps] = mx;
    row_w[r][kSplitWarps + 1] = den;
    if (!last) { wsp[r * ps + rank] = mx; wsp[r * ps + rank + 1] = den; }
  }
  __syncthreads();
  for (int e = tid; e < m_here * rank; e += blockDim.x) {
    const int r = e / rank, c = e - r * rank;
    float num = 0.f;
#pragma unroll
    for (int w = 0; w < kSplitWarps; ++w) num = fmaf(row_w[r][w], part[((int64_t)w * 16 + r) * ps + c], num);
    if (last) out[(row0 * H + m0 + r) * rank + c] = __float2bfloat16_rn(num / row_w[r][kSplitWarps + 1]);
    else wsp[r * ps + c] = num;
  }
}

// The shares of the `splits` CTAs of a work unit, [seg][unit][split][16][rank + 2] = o | m | l, into the output.
__global__ void attn_latent_merge_kernel(const float* __restrict__ ws, const int32_t* __restrict__ seg_start,
                                         const int32_t* __restrict__ seg_len, int H, int rank, int splits,
                                         const float* __restrict__ sink, bf16* __restrict__ out) {
  pdl_wait();
  const int seg = blockIdx.y, unit = blockIdx.x;
  if (seg_len[seg] != 1) return;
  const int ps = rank + 2, m0 = unit * 16, m_here = min(16, H - m0);
  const int64_t row0 = seg_start[seg];
  const float* base = ws + ((int64_t)seg * gridDim.x + unit) * splits * 16 * ps;
  __shared__ float row_w[16][8 + 1];                                   // per row: the shares' weights | 1 / denominator
  if ((int)threadIdx.x < m_here) {
    const int r = threadIdx.x;
    float mx = sink ? sink[m0 + r] : kNegBig;
    for (int zz = 0; zz < splits; ++zz) mx = fmaxf(mx, base[((int64_t)zz * 16 + r) * ps + rank]);
    float den = sink ? expf(sink[m0 + r] - mx) : 0.f;
    for (int zz = 0; zz < splits; ++zz) {
      const float* pr = base + ((int64_t)zz * 16 + r) * ps;
      const float wgt = expf(pr[rank] - mx);
      row_w[r][zz] = wgt;
      den = fmaf(wgt, pr[rank + 1], den);
    }
    row_w[r][8] = 1.f / den;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < m_here * rank; e += blockDim.x) {
    const int r = e / rank, c = e - r * rank;
    float num = 0.f;
    for (int zz = 0; zz < splits; ++zz) num = fmaf(row_w[r][zz], base[((int64_t)zz * 16 + r) * ps + c], num);
    out[(row0 * H + m0 + r) * rank + c] = __float2bfloat16_rn(num * row_w[r][8]);
  }
}

size_t rows_smem(int kd) { return (size_t)(kRowWarps * 16 + 2 * kKeys) * (kd + kPadH) * sizeof(bf16); }
size_t split_smem(int kd, int rank) {
  const size_t keys = (size_t)(16 + kSplitWarps * kKeys) * (kd + kPadH) * sizeof(bf16);
  const size_t merge = (size_t)16 * (kd + kPadH) * sizeof(bf16) + (size_t)kSplitWarps * 16 * (rank + 2) * sizeof(float);
  return keys > merge ? keys : merge;
}

}  // namespace
}  // namespace prl

using namespace prl;

// 1 if prl_attn_latent runs this geometry (else the caller takes the any-geometry CUDA-core kernel of attn_any.cu)
extern "C" int32_t prl_attn_latent_fits(int32_t kd, int32_t rank, int32_t page_size) {
  return kd % 16 == 0 && rank % 16 == 0 && rank >= 16 && rank <= 256 && rank <= kd && kd <= 576 && page_size % kKeys == 0 &&
         split_smem(kd, rank) <= 200 * 1024;
}

// Key splits of the decode-shaped kernel and the fp32 workspace they need: enough CTAs to cover the SMs, at most 8
extern "C" int32_t prl_attn_latent_splits(int32_t n_seg, int32_t H) {
  const int units = n_seg * ((H + 15) / 16);
  int s = num_sms() / (units > 0 ? units : 1);
  return s < 1 ? 1 : (s > 8 ? 8 : s);
}
extern "C" size_t prl_attn_latent_workspace_bytes(int32_t n_seg, int32_t H, int32_t rank) {
  return (size_t)n_seg * ((H + 15) / 16) * prl_attn_latent_splits(n_seg, H) * 16 * (rank + 2) * sizeof(float);
}

extern "C" int prl_attn_latent(const void* q, const void* pool, const int32_t* block_table, int32_t max_blocks, int32_t page_size,
                               const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_pos0,
                               const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H, int32_t kd, int32_t rank,
                               float scale, int32_t window, const float* sink, void* out, void* ws, size_t ws_bytes,
                               prl_stream_t stream) {
  PRL_CHECK_ARG(q && pool && block_table && seg_start && seg_len && seg_pos0 && seg_slot && out, "prl_attn_latent: NULL argument");
  PRL_CHECK_ARG(n_seg >= 1 && n_seg <= 65535 && max_q >= 1 && H >= 1 && max_blocks >= 1 && window >= 0 && prl_attn_latent_fits(kd, rank, page_size),
                "prl_attn_latent: geometry kd=%d rank=%d page=%d is not built (see prl_attn_latent_fits)", kd, rank, page_size);
  PRL_CHECK_ARG(((uintptr_t)q & 15) == 0 && ((uintptr_t)pool & 15) == 0 && ((uintptr_t)out & 3) == 0, "prl_attn_latent: misaligned buffer");
  cudaStream_t st = (cudaStream_t)stream;
  const bf16 *qq = (const bf16*)q, *pp = (const bf16*)pool;
  bf16* oo = (bf16*)out;
  static SmemAttr attr_rows[3] = {}, attr_split[3] = {};
#define PRL_LAT(KERNEL, ATTR, GRID, THREADS, SMEM)                                                                        \
  do {                                                                                                                    \
    if (rank <= 64) {                                                                                                     \
      PRL_CUDA(ensure_smem(KERNEL<8>, (int)(SMEM), ATTR[0]));                                                             \
      PRL_CUDA(launch_pdl(KERNEL<8>, GRID, dim3(THREADS), (size_t)(SMEM), st, qq, pp, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot, H, kd, rank, scale, window, sink, oo EXTRA)); \
    } else if (rank <= 128) {                                                                                             \
      PRL_CUDA(ensure_smem(KERNEL<16>, (int)(SMEM), ATTR[1]));                                                            \
      PRL_CUDA(launch_pdl(KERNEL<16>, GRID, dim3(THREADS), (size_t)(SMEM), st, qq, pp, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot, H, kd, rank, scale, window, sink, oo EXTRA)); \
    } else {                                                                                                              \
      PRL_CUDA(ensure_smem(KERNEL<32>, (int)(SMEM), ATTR[2]));                                                            \
      PRL_CUDA(launch_pdl(KERNEL<32>, GRID, dim3(THREADS), (size_t)(SMEM), st, qq, pp, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot, H, kd, rank, scale, window, sink, oo EXTRA)); \
    }                                                                                                                     \
  } while (0)
  if (max_q == 1) {
    int splits = prl_attn_latent_splits(n_seg, H);
    if (!ws || ws_bytes < prl_attn_latent_workspace_bytes(n_seg, H, rank)) splits = 1;      // no room for the shares: one CTA per unit
    float* wsf = (float*)ws;
    dim3 grid((H + 15) / 16, n_seg, splits);
#define EXTRA , splits, wsf
    PRL_LAT(attn_latent_split_kernel, attr_split, grid, kSplitWarps * 32, split_smem(kd, rank));
#undef EXTRA
    if (splits > 1) {
      PRL_LAUNCH_CHECK();
      PRL_CUDA(launch_pdl(attn_latent_merge_kernel, dim3((H + 15) / 16, n_seg), dim3(256), (size_t)0, st, (const float*)wsf, seg_start,
                          seg_len, H, rank, splits, sink, oo));
    }
  } else {
    const int64_t m_max = (int64_t)max_q * H;
    dim3 grid((unsigned)((m_max + kRowWarps * 16 - 1) / (kRowWarps * 16)), n_seg);
#define EXTRA
    PRL_LAT(attn_latent_rows_kernel, attr_rows, grid, kRowWarps * 32, rows_smem(kd));
#undef EXTRA
  }
#undef PRL_LAT
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}
