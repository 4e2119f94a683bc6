// Delta-rule matrix memory with a decay and a removal rate per key channel, over ragged segments with a carried state:
//
//     u_t = k_t / sqrt(sum(k_t^2) + unit_eps)                                  (the key of unit length, per head)
//     w_t = exp(-decay_scale * sigmoid(zw_t + w_bias)),   a_t = sigmoid(za_t + a_bias)       (per head and key channel)
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,        o_t = S_t^T r_t
//
// Both corrections read the old state.  zw, za, r, k, v are fp32 projection outputs; everything here is fp32.
//
// CTA = one (segment, head, tile of kCols value columns); a value column is owned by kLanes lanes of a warp, each
// holding R = ceil(dk / kLanes) key channels of the column in registers (channel = lane + kLanes * j, so the staged
// vectors are read without bank conflicts and the four columns of a warp share each read).  Per token: the column's
// u^T S (R products + a 3-shuffle tree), the update (3 R FMAs), and S^T r (R products + the tree).  The tokens of a
// segment are staged in chunks through shared memory, where the unit key, the decay and the removal rate are formed
// once per (token, channel); nothing but the projections is read from memory.  The arithmetic of a token is the same
// for every chunking of its prompt and every batch: results are bit-identical across schedules.
//
// State: [slot][head][dv][dk] fp32 (a column's key channels contiguous), read at a segment's start, written at its end.
#include "prl_common.cuh"
#include <math.h>

namespace prl {
namespace {

constexpr int kLanes = 8;                    // lanes per value column
constexpr int kColsPerWarp = 32 / kLanes;    // 4
constexpr int kWarps = 4;
constexpr int kCols = kColsPerWarp * kWarps; // 16 value columns per CTA
constexpr int kThreads = 32 * kWarps;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

struct DeltaArgs {
  const float* P;          // projection rows
  int64_t ldp;
  int off_r, off_k, off_v, off_a;
  const float* zw;         // decay logits [row][heads * dk]
  int64_t ldw;
  const float* w_bias;     // [heads * dk]
  const float* a_bias;     // [heads * dk]
  float decay_scale, unit_eps;
  int heads, dk, dv, chunk;
  const int32_t* seg_start;
  const int32_t* seg_len;
  const int32_t* seg_slot;
  float* state;
  float* out;
  int64_t ld_out;
};

template <int R>
__global__ void __launch_bounds__(kThreads) delta_scan_kernel(DeltaArgs a) {
  pdl_wait();
  extern __shared__ float sm[];
  const int seg = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * kCols;
  const int len = a.seg_len[seg];
  if (len <= 0) return;
  const int dk = a.dk, dv = a.dv, TT = a.chunk;
  const int dkp = R * kLanes;                     // padded key size: channels >= dk hold zeros
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane & (kLanes - 1);
  const int col = col0 + warp * kColsPerWarp + lane / kLanes;
  const bool col_on = col < dv;
  const int slot = a.seg_slot[seg];
  const int64_t row0 = a.seg_start[seg];
  // staged per token: u | au | w | k | r, each dkp floats, then kCols values
  const int tok_floats = 5 * dkp + kCols;
  float* S_base = a.state + (((int64_t)slot * a.heads + head) * dv) * dk;
  float S[R];
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int i = sub + kLanes * j;
    S[j] = (col_on && i < dk) ? S_base[(int64_t)col * dk + i] : 0.f;
  }
  const int hoff = head * dk;
  for (int t0 = 0; t0 < len; t0 += TT) {
    const int nt = min(TT, len - t0);
    __syncthreads();
    // ---- stage: one warp per token; a lane takes channels lane, lane + 32, ...
    for (int t = warp; t < nt; t += kWarps) {
      const float* p = a.P + (row0 + t0 + t) * a.ldp;
      float* dst = sm + t * tok_floats;
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) { const float kv = p[a.off_k + hoff + i]; ss = fmaf(kv, kv, ss); }
      ss = warp_sum(ss);
      const float inv = 1.f / sqrtf(ss + a.unit_eps);
      for (int i = lane; i < dkp; i += 32) {
        float u = 0.f, au = 0.f, w = 1.f, kv = 0.f, rv = 0.f;
        if (i < dk) {
          kv = p[a.off_k + hoff + i];
          rv = p[a.off_r + hoff + i];
          u = kv * inv;
          au = sigmoid_f(p[a.off_a + hoff + i] + a.a_bias[hoff + i]) * u;
          w = expf(-a.decay_scale * sigmoid_f(a.zw[(row0 + t0 + t) * a.ldw + hoff + i] + a.w_bias[hoff + i]));
        }
        dst[i] = u; dst[dkp + i] = au; dst[2 * dkp + i] = w; dst[3 * dkp + i] = kv; dst[4 * dkp + i] = rv;
      }
      if (lane < kCols) dst[5 * dkp + lane] = (col0 + lane < dv) ? p[a.off_v + head * dv + col0 + lane] : 0.f;
    }
    __syncthreads();
    // ---- walk the chunk
    for (int t = 0; t < nt; ++t) {
      const float* src = sm + t * tok_floats;
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < R; ++j) dot = fmaf(src[sub + kLanes * j], S[j], dot);
#pragma unroll
      for (int o = kLanes / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float vc = src[5 * dkp + warp * kColsPerWarp + lane / kLanes];
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const int i = sub + kLanes * j;
        float s = src[2 * dkp + i] * S[j];
        s = fmaf(-src[dkp + i], dot, s);
        s = fmaf(src[3 * dkp + i], vc, s);
        S[j] = s;
        acc = fmaf(s, src[4 * dkp + i], acc);
      }
#pragma unroll
      for (int o = kLanes / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (sub == 0 && col_on) a.out[(row0 + t0 + t) * a.ld_out + head * dv + col] = acc;
    }
  }
  if (col_on) {
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int i = sub + kLanes * j;
      if (i < dk) S_base[(int64_t)col * dk + i] = S[j];
    }
  }
}

}  // namespace
}  // namespace prl

using namespace prl;

extern "C" int64_t prl_delta_state_floats(int32_t heads, int32_t dk, int32_t dv) { return (int64_t)heads * dk * dv; }

extern "C" int prl_delta_scan(const float* P, int64_t ldp, int32_t off_r, int32_t off_k, int32_t off_v, int32_t off_a,
                              const float* zw, int64_t ldw, const float* w_bias, const float* a_bias, float decay_scale,
                              float unit_eps, int32_t heads, int32_t dk, int32_t dv, const int32_t* seg_start,
                              const int32_t* seg_len, const int32_t* seg_slot, int32_t n_seg, float* state, float* out,
                              int64_t ld_out, prl_stream_t st) {
  PRL_CHECK_ARG(P && zw && w_bias && a_bias && seg_start && seg_len && seg_slot && state && out, "prl_delta_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && heads <= 65535 && dk >= 1 && dk <= 256 && dv >= 1 && n_seg >= 1 && n_seg <= 65535 &&
                ld_out >= (int64_t)heads * dv && ldw >= (int64_t)heads * dk,
                "prl_delta_scan: bad shape (heads=%d dk=%d dv=%d; dk <= 256)", heads, dk, dv);
  DeltaArgs a{P, ldp, off_r, off_k, off_v, off_a, zw, ldw, w_bias, a_bias, decay_scale, unit_eps, heads, dk, dv, 0,
              seg_start, seg_len, seg_slot, state, out, ld_out};
  const int R = dk <= 32 ? 4 : (dk <= 64 ? 8 : (dk <= 128 ? 16 : 32));
  const int dkp = R * kLanes;
  a.chunk = dk <= 128 ? 16 : 8;
  const size_t smem = (size_t)a.chunk * (5 * dkp + kCols) * sizeof(float);     // <= 42 KB
  dim3 grid((dv + kCols - 1) / kCols, heads, n_seg);
  cudaStream_t s = (cudaStream_t)st;
  switch (R) {
    case 4: PRL_CUDA(launch_pdl(delta_scan_kernel<4>, grid, dim3(kThreads), smem, s, a)); break;
    case 8: PRL_CUDA(launch_pdl(delta_scan_kernel<8>, grid, dim3(kThreads), smem, s, a)); break;
    case 16: PRL_CUDA(launch_pdl(delta_scan_kernel<16>, grid, dim3(kThreads), smem, s, a)); break;
    default: PRL_CUDA(launch_pdl(delta_scan_kernel<32>, grid, dim3(kThreads), smem, s, a)); break;
  }
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}
