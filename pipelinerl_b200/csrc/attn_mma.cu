// Tensor-core variant of the any-geometry paged attention (attn_any.cu) for prompt portions in bf16: key sizes that are
// multiples of 16 (up to 256) and value sizes 16 / 32 / 48 / 64 / 96 / 128, with the same options (sliding window that keeps the first tokens, tanh-capped
// scores, grouped key/value heads, output in bf16 or fp32).
//
// CTA = 4 warps = 64 consecutive query rows of one (segment, query head); a warp owns 16 rows.  Keys are walked in
// tiles of 64 at absolute multiples of 64 (so the order of summation does not depend on how a prompt was cut); tiles
// that no row of the CTA can see -- between the kept first tokens and the window -- are skipped.  Per tile: K and V
// rows come from the paged pools by cp.async (16 bytes per copy, zero fill past the sequence's end), S = Q K^T by
// mma.sync m16n8k16 (bf16 in, fp32 out) with operands read by ldmatrix from padded, conflict-free rows; scale, cap and
// mask in fp32 registers; an fp32 online softmax per row (the four lanes of a row exchange by shuffles); P rounded to
// bf16 straight from the accumulator registers (the accumulator layout of S is the A-operand layout of P V); O += P V
// with V read through ldmatrix.trans.  Everything outside the two products is fp32.
#include "prl_common.cuh"
#include <math.h>

namespace prl {

namespace {

typedef __nv_bfloat16 bf16;
constexpr int kRows = 64;      // query rows per CTA
constexpr int kKeys = 64;      // keys per tile
constexpr int kPadH = 8;       // padding halves per staged row

__device__ __forceinline__ void cp16(void* dst, const void* src, int bytes) {
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

// D: query / key size, a compile-time number for the square geometries (fully unrolled score loop) or 0 = the run-time
// `dim_rt`; DV: value size.
template <int D, int DV, bool OUT_BF16>
__global__ void __launch_bounds__(128) attn_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool,
                                                       const bf16* __restrict__ v_pool, const int32_t* __restrict__ block_table,
                                                       int max_blocks, int page_size, const int32_t* __restrict__ seg_start,
                                                       const int32_t* __restrict__ seg_len, const int32_t* __restrict__ seg_pos0,
                                                       const int32_t* __restrict__ seg_slot, int H, int G, int dim_rt, float scale,
                                                       int window, int keep_first, float softcap, const float* __restrict__ sink,
                                                       void* __restrict__ out_v) {
  pdl_wait();
  const int dim = D ? D : dim_rt;
  const int LD = dim + kPadH;              // halves per staged row: (dim + 8) * 2 bytes, a multiple of 16, odd in 16-byte units
  const int CH = dim / 8;                  // 16-byte chunks per row
  constexpr int LDV = DV + kPadH, CHV = DV / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);      // [64][LD]
  bf16* Ks = Qs + kRows * LD;                        // [64][LD]
  bf16* Vs = Ks + kKeys * LD;                        // [64][LDV]
  const int seg = blockIdx.z, h = blockIdx.y;
  const int len = seg_len[seg];
  const int i0 = blockIdx.x * kRows;
  if (i0 >= len) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = h / (H / G);
  const int slot = seg_slot[seg], pos0 = seg_pos0[seg];
  const int64_t row0 = seg_start[seg];
  const int rows_here = min(kRows, len - i0);
  const int last_pos = pos0 + i0 + rows_here - 1;
  const int win_lo = window > 0 ? max(0, pos0 + i0 - window + 1) : 0;      // the CTA's first row sees from here on
  const int sink_end = window > 0 ? min(keep_first, win_lo) : 0;
  const int32_t* bt = block_table + (int64_t)slot * max_blocks;
  for (int c = tid; c < kRows * CH; c += 128) {
    const int r = c / CH, cc = c - r * CH;
    const bool ok = r < rows_here;
    cp16(Qs + r * LD + cc * 8, q + ((row0 + i0 + (ok ? r : 0)) * H + h) * dim + cc * 8, ok ? 16 : 0);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  // this thread's two rows of the warp's 16: r_lo = lane / 4, r_hi = r_lo + 8
  const int my_row[2] = {warp * 16 + (lane >> 2), warp * 16 + (lane >> 2) + 8};
  int my_pos[2], my_lo[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    my_pos[u] = (i0 + my_row[u] < len) ? pos0 + i0 + my_row[u] : -1;        // -1: no such row, sees nothing
    my_lo[u] = window > 0 ? my_pos[u] - window + 1 : 0;
  }
  const int w_first = pos0 + i0 + warp * 16, w_last = min(w_first + 15, last_pos);    // positions of the warp's rows
  const int w_lo = window > 0 ? w_first - window + 1 : 0;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;

  for (int k0 = 0; k0 <= last_pos; k0 += kKeys) {
    if (k0 >= sink_end && k0 + kKeys <= win_lo) continue;              // CTA-uniform: between the kept tokens and the window
    __syncthreads();                                                   // every warp is done with the previous tile
    for (int c = tid; c < kKeys * CH; c += 128) {
      const int j = c / CH, cc = c - j * CH;
      const int kt = k0 + j;
      const bool ok = kt <= last_pos;
      const int kk = ok ? kt : k0;
      const int64_t at = (((int64_t)bt[kk / page_size] * G + g) * page_size + kk % page_size) * dim + cc * 8;
      cp16(Ks + j * LD + cc * 8, k_pool + at, ok ? 16 : 0);
    }
    for (int c = tid; c < kKeys * CHV; c += 128) {
      const int j = c / CHV, cc = c - j * CHV;
      const int kt = k0 + j;
      const bool ok = kt <= last_pos;
      const int kk = ok ? kt : k0;
      const int64_t at = (((int64_t)bt[kk / page_size] * G + g) * page_size + kk % page_size) * DV + cc * 8;
      cp16(Vs + j * LDV + cc * 8, v_pool + at, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (w_first > last_pos || k0 > w_last) continue;                   // warp-uniform: no rows, or the tile is in the future
    if (k0 + kKeys <= w_lo && k0 >= keep_first) continue;              // hidden from every row of the warp
    // ---- S = Q K^T (16 x 64 per warp)
    float s[kKeys / 8][4];
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < dim; kk += 16) {
      uint32_t a[4];
      ldsm4(a, Qs + (warp * 16 + (lane & 15)) * LD + kk + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < kKeys / 16; ++j) {
        uint32_t b[4];
        ldsm4(b, Ks + (16 * j + (lane & 7) + ((lane >> 4) << 3)) * LD + kk + ((lane >> 3) & 1) * 8);
        mma16816(s[2 * j], a, b[0], b[1]);
        mma16816(s[2 * j + 1], a, b[2], b[3]);
      }
    }
    // ---- scale, cap, mask, online softmax (fp32)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int u = e >> 1;
        const int kt = k0 + 8 * j + (lane & 3) * 2 + (e & 1);
        float v = s[j][e] * scale;
        if (softcap > 0.f) v = softcap * tanhf(v / softcap);
        const bool seen = kt <= my_pos[u] && (kt >= my_lo[u] || kt < keep_first);
        v = seen ? v : -INFINITY;
        s[j][e] = v;
        mx[u] = fmaxf(mx[u], v);
      }
    float corr[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      mx[u] = fmaxf(mx[u], __shfl_xor_sync(0xffffffffu, mx[u], 1));
      mx[u] = fmaxf(mx[u], __shfl_xor_sync(0xffffffffu, mx[u], 2));
      const float m_new = fmaxf(m[u], mx[u]);
      corr[u] = m_new == -INFINITY ? 1.f : expf(m[u] - m_new);       // a row that has seen nothing yet keeps its zeros
      m[u] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int u = e >> 1;
        const float p = s[j][e] == -INFINITY ? 0.f : expf(s[j][e] - m[u]);
        s[j][e] = p;
        sum[u] += p;
      }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], 1);
      sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], 2);
      l[u] = l[u] * corr[u] + sum[u];
    }
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
    // ---- O += P V
#pragma unroll
    for (int t = 0; t < kKeys / 16; ++t) {
      uint32_t a[4] = {pack_bf16(s[2 * t][0], s[2 * t][1]), pack_bf16(s[2 * t][2], s[2 * t][3]),
                       pack_bf16(s[2 * t + 1][0], s[2 * t + 1][1]), pack_bf16(s[2 * t + 1][2], s[2 * t + 1][3])};
#pragma unroll
      for (int j = 0; j < DV / 16; ++j) {
        uint32_t b[4];
        ldsm4_t(b, Vs + (16 * t + (lane & 15)) * LDV + 16 * j + (lane >> 4) * 8);
        mma16816(o[2 * j], a, b[0], b[1]);
        mma16816(o[2 * j + 1], a, b[2], b[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (my_pos[u] < 0) continue;
    float inv = 1.f / l[u];
    if (sink) {                      // a logit per head that joins the denominator only
      const float sk = sink[h], m_new = fmaxf(m[u], sk);
      const float corr = expf(m[u] - m_new);
      inv = corr / (l[u] * corr + expf(sk - m_new));
    }
    const int64_t base = ((row0 + i0 + my_row[u]) * H + h) * DV;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
      const int c = 8 * j + (lane & 3) * 2;
      const float v0 = o[j][2 * u] * inv, v1 = o[j][2 * u + 1] * inv;
      if constexpr (OUT_BF16) {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(out_v) + base + c) = pack_bf16(v0, v1);
      } else {
        float* po = reinterpret_cast<float*>(out_v) + base + c;
        po[0] = v0; po[1] = v1;
      }
    }
  }
}

template <int D, int DV, bool OUT_BF16>
int launch_mma(const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
               const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H, int G,
               int dim, float scale, int window, int keep_first, float softcap, const float* sink, void* out, cudaStream_t st) {
  const size_t smem = ((size_t)(kRows + kKeys) * (dim + kPadH) + (size_t)kKeys * (DV + kPadH)) * sizeof(bf16);
  static SmemAttr attr = {};
  if (smem > 48 * 1024) PRL_CUDA(ensure_smem(attn_mma_kernel<D, DV, OUT_BF16>, (int)smem, attr));
  dim3 grid((max_q + kRows - 1) / kRows, H, n_seg);
  PRL_CUDA(launch_pdl((attn_mma_kernel<D, DV, OUT_BF16>), grid, dim3(128), smem, st, (const bf16*)q, (const bf16*)kp, (const bf16*)vp, bt,
                      max_blocks, page_size, ss, sl, sp, sslot, H, G, dim, scale, window, keep_first, softcap, sink, out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

}  // namespace

// bf16 cache and queries take the tensor-core kernel when the key size is a multiple of 16 up to 256 and the value size
// one of 16 / 32 / 48 / 64 / 96 / 128 (the square geometries 32, 64, 128 with a fully unrolled score loop)
bool attn_mma_fits(int dim, int vdim, const void* q, const void* k_pool, const void* v_pool) {
  const bool vok = vdim == 16 || vdim == 32 || vdim == 48 || vdim == 64 || vdim == 96 || vdim == 128;
  return dim >= 16 && dim % 16 == 0 && dim <= 256 && vok && (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0;
}

int attn_mma_launch(const void* q, const void* kp, const void* vp, const int32_t* bt, int max_blocks, int page_size,
                    const int32_t* ss, const int32_t* sl, const int32_t* sp, const int32_t* sslot, int n_seg, int max_q, int H,
                    int G, int dim, int vdim, float scale, int window, int keep_first, float softcap, const float* sink,
                    int out_is_bf16, void* out, cudaStream_t st) {
#define PRL_MMA(D, DV) (out_is_bf16 ? launch_mma<D, DV, true>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, scale, window, keep_first, softcap, sink, out, st) \
                                    : launch_mma<D, DV, false>(q, kp, vp, bt, max_blocks, page_size, ss, sl, sp, sslot, n_seg, max_q, H, G, dim, scale, window, keep_first, softcap, sink, out, st))
  if (dim == vdim) {
    if (dim == 32) return PRL_MMA(32, 32);
    if (dim == 64) return PRL_MMA(64, 64);
    if (dim == 128) return PRL_MMA(128, 128);
  }
  switch (vdim) {
    case 16: return PRL_MMA(0, 16);
    case 32: return PRL_MMA(0, 32);
    case 48: return PRL_MMA(0, 48);
    case 64: return PRL_MMA(0, 64);
    case 96: return PRL_MMA(0, 96);
    default: return PRL_MMA(0, 128);
  }
#undef PRL_MMA
}

}  // namespace prl
