// Causal softmax attention over a paged KV cache for ANY head geometry: query/key size `dim` and value size `vdim`
// are independent run-time numbers (the tcgen05 kernels of attn_tc.cu / paged_attn.cu are built for 128 = 128), the
// softmax scale is a parameter, the cache element type is bf16 or fp32.  Ragged segments: a segment is q_len
// consecutive tokens of one sequence starting at position pos0 (a prompt chunk, or one decoded token); token i of the
// segment sees keys 0 .. pos0 + i of its sequence, all of which are already in the cache.
//
// CTA = 8 warps = 8 (or, for long portions, 32) consecutive query rows of one (segment, query head); the CTA streams the sequence's keys in tiles of
// 32 through shared memory (converted to fp32), a warp scores one key per lane, keeps an fp32 online softmax for its
// row and accumulates vdim / 32 output channels per lane.  Key tiles start at absolute multiples of 32, so the
// summation order for a query never depends on how its prompt was chunked or batched.
//
// Options (all off at 0): `window` > 0 hides keys more than window - 1 positions back, except the first `keep_first`
// tokens of the sequence, which every later token keeps seeing; `softcap` > 0 replaces a score s by
// softcap * tanh(s / softcap) before the softmax.  Key tiles that no row of the CTA can see are skipped whole, the
// others keep their absolute place, so the order of summation still does not depend on the chunking.  The output is
// fp32, or the cache's element type when out_is_t is set (it then feeds a GEMM directly).
//
// K pool: [page][kv head][page_size][dim], V pool: [page][kv head][page_size][vdim]; block_table[slot][j] = j-th page.
#include "prl_common.cuh"
#include <math.h>

namespace prl {

// attn_mma.cu: the tensor-core kernel for prompt portions in bf16 with head sizes it is built for
bool attn_mma_fits(int dim, int vdim, const void* q, const void* k_pool, const void* v_pool);
int attn_mma_launch(const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                    const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H,
                    int G, int dim, int vdim, float scale, int window, int keep_first, float softcap, const float* sink,
                    int out_is_bf16, void* out, cudaStream_t st);

namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kKeysPerTile = 32;

template <typename T> __device__ __forceinline__ float cvt(T v);
template <> __device__ __forceinline__ float cvt<float>(float v) { return v; }
template <> __device__ __forceinline__ float cvt<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, int VR, bool OUT_T, int RW>
__global__ void __launch_bounds__(256) attn_any_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                                       const T* __restrict__ v_pool, const int32_t* __restrict__ block_table,
                                                       int max_blocks, int page_size, const int32_t* __restrict__ seg_start,
                                                       const int32_t* __restrict__ seg_len, const int32_t* __restrict__ seg_pos0,
                                                       const int32_t* __restrict__ seg_slot, int H, int G, int dim, int vdim,
                                                       float scale, int window, int keep_first, float softcap,
                                                       int ldv, const float* __restrict__ sink, void* __restrict__ out_v) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  // RW consecutive query rows per warp (kWarpsPerCta * RW per CTA): a staged key tile is scored against all of them in
  // one pass over the key's channels.  A row's arithmetic is the same for every RW.
  constexpr int kRows = kWarpsPerCta * RW;
  extern __shared__ float sm[];
  const int seg = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
  const int len = seg_len[seg];
  const int i0 = tile * kRows;
  if (i0 >= len) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = h / (H / G);
  const int slot = seg_slot[seg], pos0 = seg_pos0[seg];
  const int64_t row0 = seg_start[seg];
  const int kstride = dim + 1;
  float* Ks = sm;                                  // [32][dim + 1]
  float* Vs = Ks + kKeysPerTile * kstride;         // [32][vdim]
  float* Qs = Vs + kKeysPerTile * vdim;            // [kRows][dim]
  const int rows_here = min(kRows, len - i0);
  const int last_pos = pos0 + i0 + rows_here - 1;  // the CTA needs keys 0 .. last_pos
  // keys the CTA's FIRST row no longer sees end before win_lo; tiles wholly inside [sink_end, win_lo) are skipped
  const int win_lo = window > 0 ? max(0, pos0 + i0 - window + 1) : 0;
  const int sink_end = window > 0 ? min(keep_first, win_lo) : 0;
  const int w_i0 = i0 + warp * RW;                 // this warp's first row
  for (int i = threadIdx.x; i < kRows * dim; i += blockDim.x) {
    const int w = i / dim, d = i - w * dim;
    Qs[i] = w < rows_here ? cvt(q[((row0 + i0 + w) * H + h) * dim + d]) : 0.f;
  }
  float m[RW], l[RW], acc[RW][VR];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < VR; ++i) acc[r][i] = 0.f;
  }
  const int32_t* bt = block_table + (int64_t)slot * max_blocks;
  for (int k0 = 0; k0 <= last_pos; k0 += kKeysPerTile) {
    if (k0 >= sink_end && k0 + kKeysPerTile <= win_lo) continue;     // CTA-uniform
    __syncthreads();
    const int nk = min(kKeysPerTile, last_pos + 1 - k0);
    for (int i = threadIdx.x; i < nk * dim; i += blockDim.x) {
      const int j = i / dim, d = i - j * dim;
      const int kt = k0 + j;
      const int page = bt[kt / page_size], within = kt % page_size;
      Ks[j * kstride + d] = cvt(k_pool[(((int64_t)page * G + g) * page_size + within) * dim + d]);
    }
    for (int i = threadIdx.x; i < nk * vdim; i += blockDim.x) {
      const int j = i / vdim, d = i - j * vdim;
      const int kt = k0 + j;
      const int page = bt[kt / page_size], within = kt % page_size;
      Vs[j * vdim + d] = cvt(v_pool[(((int64_t)page * G + g) * page_size + within) * ldv + d]);
    }
    __syncthreads();
    // which of this warp's rows see anything of the tile (warp-uniform), and which key this lane scores for them
    bool live[RW], mine[RW];
    bool any = false;
    const int kt_mine = k0 + lane;
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const int my_pos = pos0 + w_i0 + r;
      const int my_lo = window > 0 ? my_pos - window + 1 : 0;     // the row sees j >= my_lo, and j < keep_first
      live[r] = w_i0 + r < len && k0 <= my_pos && !(k0 + nk <= my_lo && k0 >= keep_first);
      mine[r] = live[r] && lane < nk && kt_mine <= my_pos && (kt_mine >= my_lo || kt_mine < keep_first);
      any = any || live[r];
    }
    if (!any) continue;
    float dot[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) dot[r] = 0.f;
    if (lane < nk) {
      const float* qr = Qs + (warp * RW) * dim;
      const float* kr = Ks + lane * kstride;
      for (int d = 0; d < dim; ++d) {
        const float kd = kr[d];
#pragma unroll
        for (int r = 0; r < RW; ++r) dot[r] = fmaf(qr[r * dim + d], kd, dot[r]);
      }
    }
    float p[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      p[r] = 0.f;
      if (!live[r]) continue;                      // warp-uniform
      float s = -INFINITY;
      if (mine[r]) {
        s = dot[r] * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      }
      const float m_new = fmaxf(m[r], warp_max(s));   // at least one key of the tile is visible, so m_new is finite
      const float corr = expf(m[r] - m_new);          // exp(-inf) = 0 on the first tile
      p[r] = mine[r] ? expf(s - m_new) : 0.f;
      l[r] = l[r] * corr + warp_sum(p[r]);
      m[r] = m_new;
#pragma unroll
      for (int i = 0; i < VR; ++i) acc[r][i] *= corr;
    }
    // the tile's weighted values are summed on their own and then added to the running output: over a long sequence the
    // rounding error grows with the number of tiles, not of keys
    float tacc[RW][VR];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
      for (int i = 0; i < VR; ++i) tacc[r][i] = 0.f;
    for (int j = 0; j < nk; ++j) {
      float pj[RW];
      bool used = false;
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        pj[r] = __shfl_sync(0xffffffffu, p[r], j);
        used = used || pj[r] != 0.f;
      }
      if (!used) continue;                          // hidden key (warp-uniform)
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        const int c = lane + 32 * i;
        const float v = c < vdim ? Vs[j * vdim + c] : 0.f;
#pragma unroll
        for (int r = 0; r < RW; ++r) tacc[r][i] = fmaf(pj[r], v, tacc[r][i]);
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
      for (int i = 0; i < VR; ++i) acc[r][i] += tacc[r][i];
  }
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    const int my_i = w_i0 + r;
    if (my_i >= len) continue;
    if (sink) {                                      // a logit without key or value: it joins the denominator only
      const float m_new = fmaxf(m[r], sink[h]);
      const float corr = expf(m[r] - m_new);
      l[r] = l[r] * corr + expf(sink[h] - m_new);
#pragma unroll
      for (int i = 0; i < VR; ++i) acc[r][i] *= corr;
    }
    const float inv = 1.f / l[r];
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      const int c = lane + 32 * i;
      if (c < vdim) {
        if constexpr (OUT_T) reinterpret_cast<T*>(out_v)[((row0 + my_i) * H + h) * vdim + c] = T(acc[r][i] * inv);
        else reinterpret_cast<float*>(out_v)[((row0 + my_i) * H + h) * vdim + c] = acc[r][i] * inv;
      }
    }
  }
}

template <typename T, int VR, bool OUT_T, int RW>
int launch_attn_rw(const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                   const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H,
                   int G, int dim, int vdim, float scale, int window, int keep_first, float softcap, int ldv, const float* sink,
                   void* out, cudaStream_t st) {
  constexpr int kRows = kWarpsPerCta * RW;
  const size_t smem = ((size_t)kKeysPerTile * (dim + 1) + (size_t)kKeysPerTile * vdim + (size_t)kRows * dim) * sizeof(float);
  static SmemAttr attr = {};
  if (smem > 48 * 1024) PRL_CUDA(ensure_smem(attn_any_kernel<T, VR, OUT_T, RW>, (int)smem, attr));
  dim3 grid((max_q + kRows - 1) / kRows, H, n_seg);
  PRL_CUDA(launch_pdl((attn_any_kernel<T, VR, OUT_T, RW>), dim3(grid), dim3(256), (size_t)(smem), st, (const T*)q, (const T*)kp, (const T*)vp, bt, max_blocks, page_size, ss, sl,
                      sp, sslot, H, G, dim, vdim, scale, window, keep_first, softcap, ldv, sink, out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

// long portions: four rows per warp (a key tile staged once per 32 rows); short ones: one row per warp, more CTAs
template <typename T, int VR, bool OUT_T>
int launch_attn(const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H,
                int G, int dim, int vdim, float scale, int window, int keep_first, float softcap, int ldv, const float* sink,
                void* out, cudaStream_t st) {
  if (max_q >= 64 && VR <= 4)
    return launch_attn_rw<T, VR, OUT_T, 4>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, vdim,
                                           scale, window, keep_first, softcap, ldv, sink, out, st);
  return launch_attn_rw<T, VR, OUT_T, 1>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, vdim,
                                         scale, window, keep_first, softcap, ldv, sink, out, st);
}

// ---- single-token segments (a decode step) ------------------------------------------------------------------------------
// attn_any_kernel gives a one-row segment to one warp of a CTA that still stages whole key tiles.  Here a CTA owns up to
// kDecHeads query heads that share a key/value head of one segment; its warps take the VISIBLE key tiles (the kept
// first tokens, then the window) round-robin, each lane scoring one key of a tile straight from the cache (16-byte
// loads) for all the CTA's heads, and the warps' partial softmaxes are merged through shared memory.  Same options as
// the kernel above.  Segments that are not exactly one row long are skipped (the host picks this kernel only when
// every segment is one row, or empty).
constexpr int kDecHeads = 4;
constexpr int kDecWarps = 16;

template <typename T> struct Chunk;        // 16 bytes of cache elements
template <> struct Chunk<float> { static constexpr int n = 4; };
template <> struct Chunk<__nv_bfloat16> { static constexpr int n = 8; };

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& u, float (&f)[Chunk<T>::n]);
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& u, float (&f)[4]) {
  f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
}
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}

template <typename T, int VR, bool OUT_T>
__global__ void __launch_bounds__(kDecWarps * 32) attn_decode_any_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool, const int32_t* __restrict__ block_table,
    int max_blocks, int page_size, const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_len,
    const int32_t* __restrict__ seg_pos0, const int32_t* __restrict__ seg_slot, int H, int G, int dim, int vdim, float scale,
    int window, int keep_first, float softcap, int ldv, const float* __restrict__ sink, void* __restrict__ out_v) {
  pdl_wait();
  extern __shared__ float sm[];
  const int seg = blockIdx.y;
  if (seg_len[seg] != 1) return;
  const int qpg = H / G, groups = (qpg + kDecHeads - 1) / kDecHeads;
  const int g = blockIdx.x / groups, h0 = g * qpg + (blockIdx.x % groups) * kDecHeads;
  const int nh = min(kDecHeads, (g + 1) * qpg - h0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = seg_slot[seg], pos = seg_pos0[seg];
  const int64_t row = seg_start[seg];
  float* Qs = sm;                                          // [kDecHeads][dim]
  float* part = Qs + kDecHeads * dim;                      // [warps][kDecHeads][vdim + 2]: acc | m | l
  const int pstride = vdim + 2;
  for (int i = threadIdx.x; i < kDecHeads * dim; i += blockDim.x) {
    const int hh = i / dim, d = i - hh * dim;
    Qs[i] = hh < nh ? cvt(q[(row * H + h0 + hh) * dim + d]) : 0.f;
  }
  __syncthreads();
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;          // the window starts here
  const int sink_end = window > 0 ? min(keep_first, lo) : 0;         // kept first tokens in front of it
  const int tw = lo / kKeysPerTile;                                  // first tile of the window
  const int ts = min((sink_end + kKeysPerTile - 1) / kKeysPerTile, tw);
  const int n_tiles = ts + pos / kKeysPerTile - tw + 1;
  const int32_t* bt = block_table + (int64_t)slot * max_blocks;
  constexpr int E = Chunk<T>::n;
  const bool vec = dim % E == 0;
  float m[kDecHeads], l[kDecHeads], acc[kDecHeads][VR];
#pragma unroll
  for (int hh = 0; hh < kDecHeads; ++hh) {
    m[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
    for (int i = 0; i < VR; ++i) acc[hh][i] = 0.f;
  }
  for (int t = warp; t < n_tiles; t += kDecWarps) {
    const int k0 = (t < ts ? t : tw + t - ts) * kKeysPerTile;
    const int kt = k0 + lane;
    const bool seen = kt <= pos && (kt >= lo || kt < keep_first);
    float dot[kDecHeads];
#pragma unroll
    for (int hh = 0; hh < kDecHeads; ++hh) dot[hh] = 0.f;
    if (seen) {
      const T* kr = k_pool + (((int64_t)bt[kt / page_size] * G + g) * page_size + kt % page_size) * dim;
      if (vec) {
        int d = 0;
        for (; d + 8 * E <= dim; d += 8 * E) {              // eight 16-byte loads in flight per lane
          uint4 raw[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(kr + d + u * E);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            float kf[E];
            unpack16<T>(raw[u], kf);
#pragma unroll
            for (int hh = 0; hh < kDecHeads; ++hh)
#pragma unroll
              for (int e = 0; e < E; ++e) dot[hh] = fmaf(Qs[hh * dim + d + u * E + e], kf[e], dot[hh]);
          }
        }
        for (; d < dim; d += E) {
          float kf[E];
          unpack16<T>(*reinterpret_cast<const uint4*>(kr + d), kf);
#pragma unroll
          for (int hh = 0; hh < kDecHeads; ++hh)
#pragma unroll
            for (int e = 0; e < E; ++e) dot[hh] = fmaf(Qs[hh * dim + d + e], kf[e], dot[hh]);
        }
      } else {
        for (int d = 0; d < dim; ++d) {
          const float kf = cvt(kr[d]);
#pragma unroll
          for (int hh = 0; hh < kDecHeads; ++hh) dot[hh] = fmaf(Qs[hh * dim + d], kf, dot[hh]);
        }
      }
    }
    if (__ballot_sync(0xffffffffu, seen) == 0u) continue;      // cannot happen for a listed tile; keeps m finite
    float p[kDecHeads];
#pragma unroll
    for (int hh = 0; hh < kDecHeads; ++hh) {
      float sc = -INFINITY;
      if (seen) {
        sc = dot[hh] * scale;
        if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
      }
      const float m_new = fmaxf(m[hh], warp_max(sc));
      const float corr = expf(m[hh] - m_new);
      p[hh] = seen ? expf(sc - m_new) : 0.f;
      l[hh] = l[hh] * corr + warp_sum(p[hh]);
      m[hh] = m_new;
#pragma unroll
      for (int i = 0; i < VR; ++i) acc[hh][i] *= corr;
    }
    const uint32_t seen_mask = __ballot_sync(0xffffffffu, seen);
    constexpr int KB = VR <= 4 ? 8 : 4;                        // keys whose value loads are in flight together
    for (int j0 = 0; j0 < kKeysPerTile; j0 += KB) {
      if (!(seen_mask >> j0 & ((1u << KB) - 1u))) continue;    // warp-uniform
      float vv[KB][VR];
#pragma unroll
      for (int u = 0; u < KB; ++u) {
        const int kj = k0 + j0 + u;
        const bool on = seen_mask >> (j0 + u) & 1u;            // hidden keys are not read: their weight is zero anyway
        const T* vr = v_pool + (((int64_t)bt[(on ? kj : k0) / page_size] * G + g) * page_size + (on ? kj : k0) % page_size) * ldv;
#pragma unroll
        for (int i = 0; i < VR; ++i) {
          const int c = lane + 32 * i;
          vv[u][i] = (on && c < vdim) ? cvt(vr[c]) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < KB; ++u)
#pragma unroll
        for (int hh = 0; hh < kDecHeads; ++hh) {
          const float pj = __shfl_sync(0xffffffffu, p[hh], j0 + u);
#pragma unroll
          for (int i = 0; i < VR; ++i) acc[hh][i] = fmaf(pj, vv[u][i], acc[hh][i]);
        }
    }
  }
#pragma unroll
  for (int hh = 0; hh < kDecHeads; ++hh) {
    float* pw = part + ((int64_t)warp * kDecHeads + hh) * pstride;
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      const int c = lane + 32 * i;
      if (c < vdim) pw[c] = acc[hh][i];
    }
    if (lane == 0) { pw[vdim] = m[hh]; pw[vdim + 1] = l[hh]; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nh * vdim; i += blockDim.x) {    // merge the warps' partial softmaxes, in warp order
    const int hh = i / vdim, c = i - hh * vdim;
    float mx = sink ? sink[h0 + hh] : -INFINITY;
    for (int w = 0; w < kDecWarps; ++w) mx = fmaxf(mx, part[((int64_t)w * kDecHeads + hh) * pstride + vdim]);
    float num = 0.f, den = sink ? expf(sink[h0 + hh] - mx) : 0.f;      // the sink logit: denominator only
    for (int w = 0; w < kDecWarps; ++w) {
      const float* pw = part + ((int64_t)w * kDecHeads + hh) * pstride;
      const float wgt = pw[vdim] == -INFINITY ? 0.f : expf(pw[vdim] - mx);
      num = fmaf(wgt, pw[c], num);
      den = fmaf(wgt, pw[vdim + 1], den);
    }
    const int64_t o = (row * H + h0 + hh) * vdim + c;
    if constexpr (OUT_T) reinterpret_cast<T*>(out_v)[o] = T(num / den);
    else reinterpret_cast<float*>(out_v)[o] = num / den;
  }
}

template <typename T, int VR, bool OUT_T>
int launch_attn_decode(const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                       const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int H, int G,
                       int dim, int vdim, float scale, int window, int keep_first, float softcap, int ldv, const float* sink,
                       void* out, cudaStream_t st) {
  const size_t smem = ((size_t)kDecHeads * dim + (size_t)kDecWarps * kDecHeads * (vdim + 2)) * sizeof(float);
  static SmemAttr attr = {};
  if (smem > 48 * 1024) PRL_CUDA(ensure_smem(attn_decode_any_kernel<T, VR, OUT_T>, (int)smem, attr));
  const int groups = (H / G + kDecHeads - 1) / kDecHeads;
  PRL_CUDA(launch_pdl((attn_decode_any_kernel<T, VR, OUT_T>), dim3(G * groups, n_seg), dim3(kDecWarps * 32), smem, st, (const T*)q,
                      (const T*)kp, (const T*)vp, bt, max_blocks, page_size, ss, sl, sp, sslot, H, G, dim, vdim, scale, window,
                      keep_first, softcap, ldv, sink, out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

template <typename T>
int dispatch_attn(int vr, const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                  const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H,
                  int G, int dim, int vdim, float scale, int window, int keep_first, float softcap, int ldv, const float* sink, int out_is_t,
                  void* out, cudaStream_t st) {
#define PRL_ATTN(VR) (out_is_t ? launch_attn<T, VR, true>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, ldv, sink, out, st) \
                               : launch_attn<T, VR, false>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, ldv, sink, out, st))
#define PRL_ATTN_DEC(VR) (out_is_t ? launch_attn_decode<T, VR, true>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, H, G, dim, vdim, scale, window, keep_first, softcap, ldv, sink, out, st) \
                                   : launch_attn_decode<T, VR, false>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, H, G, dim, vdim, scale, window, keep_first, softcap, ldv, sink, out, st))
  if (max_q == 1 && page_size % kKeysPerTile == 0) {          // every segment is one token (or empty): the decode kernel
    if (vr <= 1) return PRL_ATTN_DEC(1);
    if (vr <= 2) return PRL_ATTN_DEC(2);
    if (vr <= 4) return PRL_ATTN_DEC(4);
    if (vr <= 8) return PRL_ATTN_DEC(8);
    return PRL_ATTN_DEC(16);
  }
#undef PRL_ATTN_DEC
  if (vr <= 1) return PRL_ATTN(1);
  if (vr <= 2) return PRL_ATTN(2);
  if (vr <= 4) return PRL_ATTN(4);
  if (vr <= 8) return PRL_ATTN(8);
  return PRL_ATTN(16);
#undef PRL_ATTN
}

}  // namespace
}  // namespace prl

using namespace prl;

constexpr int kMmaMinRows = 16;      // the longest segment of the batch has at least this many rows: tensor-core tiles pay
static int g_attn_tensor_cores = 1;

// Tests compare the tensor-core kernel with the CUDA-core one on the same cache: 0 switches the former off (process-wide).
extern "C" void prl_attn_any_tensor_cores(int32_t on) { g_attn_tensor_cores = on ? 1 : 0; }

static int attn_any_impl(const void* q, const void* k_pool, const void* v_pool, int32_t f32, const int32_t* block_table,
                         int32_t max_blocks, int32_t page_size, const int32_t* seg_start, const int32_t* seg_len,
                         const int32_t* seg_pos0, const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H,
                         int32_t G, int32_t dim, int32_t vdim, float scale, int32_t window, int32_t keep_first,
                         float softcap, int32_t out_is_t, void* out, prl_stream_t st, int32_t ldv = 0,
                         const float* sink = nullptr) {
  if (ldv <= 0) ldv = vdim;
  PRL_CHECK_ARG(ldv >= vdim, "prl_attn_any: value row stride %d below the value size %d", ldv, vdim);
  PRL_CHECK_ARG(q && k_pool && v_pool && block_table && seg_start && seg_len && seg_pos0 && seg_slot && out,
                "prl_attn_any: NULL argument");
  PRL_CHECK_ARG(n_seg >= 1 && n_seg <= 65535 && max_q >= 1 && H >= 1 && H <= 65535 && G >= 1 && H % G == 0 && dim >= 1 &&
                dim <= 1024 && vdim >= 1 && vdim <= 512 && page_size >= 1 && max_blocks >= 1,
                "prl_attn_any: bad shape (H=%d G=%d dim=%d vdim=%d; dim <= 1024, vdim <= 512)", H, G, dim, vdim);
  PRL_CHECK_ARG(window >= 0 && keep_first >= 0 && softcap >= 0.f, "prl_attn_any: bad mask (window=%d keep_first=%d)", window, keep_first);
  const int vr = (vdim + 31) / 32;
  if (!f32 && g_attn_tensor_cores && max_q >= kMmaMinRows && ldv == vdim && attn_mma_fits(dim, vdim, q, k_pool, v_pool))
    return attn_mma_launch(q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot, n_seg,
                           max_q, H, G, dim, vdim, scale, window, keep_first, softcap, sink, out_is_t, out, (cudaStream_t)st);
  if (f32) return dispatch_attn<float>(vr, q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0,
                                       seg_slot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, ldv, sink, out_is_t, out, (cudaStream_t)st);
  return dispatch_attn<__nv_bfloat16>(vr, q, k_pool, v_pool, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0,
                                      seg_slot, n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, ldv, sink, out_is_t, out, (cudaStream_t)st);
}

extern "C" int prl_attn_any(const void* q, const void* k_pool, const void* v_pool, int32_t f32, const int32_t* block_table,
                            int32_t max_blocks, int32_t page_size, const int32_t* seg_start, const int32_t* seg_len,
                            const int32_t* seg_pos0, const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H,
                            int32_t G, int32_t dim, int32_t vdim, float scale, float* out, prl_stream_t st) {
  return attn_any_impl(q, k_pool, v_pool, f32, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                       n_seg, max_q, H, G, dim, vdim, scale, 0, 0, 0.f, 0, out, st);
}

// With a sliding window (0 = none) that keeps the first `keep_first` tokens, a tanh cap on the scores (0 = none) and
// the output in the cache's element type (out_is_t) or fp32.
extern "C" int prl_attn_any_masked(const void* q, const void* k_pool, const void* v_pool, int32_t f32,
                                   const int32_t* block_table, int32_t max_blocks, int32_t page_size,
                                   const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_pos0,
                                   const int32_t* seg_slot, int32_t n_seg, int32_t max_q, int32_t H, int32_t G, int32_t dim,
                                   int32_t vdim, float scale, int32_t window, int32_t keep_first, float softcap,
                                   int32_t out_is_t, void* out, prl_stream_t st) {
  return attn_any_impl(q, k_pool, v_pool, f32, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                       n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, out_is_t, out, st);
}

// As prl_attn_any_masked, with two more freedoms: the value rows have their own stride `ldv` >= vdim (values that are a
// leading slice of wider rows: v_pool may be the key pool itself, so that a latent cache is stored once), and `sink`
// (NULL = none) holds one fp32 logit per query head that enters the softmax denominator without a key or a value.
extern "C" int prl_attn_any_sink(const void* q, const void* k_pool, const void* v_pool, int32_t ldv, int32_t f32,
                                 const int32_t* block_table, int32_t max_blocks, int32_t page_size, const int32_t* seg_start,
                                 const int32_t* seg_len, const int32_t* seg_pos0, const int32_t* seg_slot, int32_t n_seg,
                                 int32_t max_q, int32_t H, int32_t G, int32_t dim, int32_t vdim, float scale, int32_t window,
                                 int32_t keep_first, float softcap, const float* sink, int32_t out_is_t, void* out,
                                 prl_stream_t st) {
  return attn_any_impl(q, k_pool, v_pool, f32, block_table, max_blocks, page_size, seg_start, seg_len, seg_pos0, seg_slot,
                       n_seg, max_q, H, G, dim, vdim, scale, window, keep_first, softcap, out_is_t, out, st, ldv, sink);
}
