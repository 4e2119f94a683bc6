// Delta-rule matrix memory with a decay and a removal rate per key channel, over ragged segments with a carried state:
//
//     u_t = k_t / sqrt(sum(k_t^2) + unit_eps)                                  (the key of unit length, per head)
//     w_t = exp(-decay_scale * sigmoid(zw_t + w_bias)),   a_t = sigmoid(za_t + a_bias)       (per head and key channel)
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,        o_t = S_t^T r_t
//
// Both corrections read the old state.  zw, za, r, k, v are fp32 projection outputs; everything here is fp32.
//
// Two kernels.  delta_prep (one warp per token and head, fully parallel) forms the unit key, the removal rate times the
// unit key (in place of the removal logits) and the decay (in place of the decay logits).  delta_scan walks the tokens:
// CTA = one (segment, head, tile of kCols value columns), four warps.  A value column is owned by kLanes lanes of a
// warp, each holding R = ceil(dk / kLanes) key channels of the column in registers (channels 4 (lane + kLanes jj) .. + 3,
// so the staged vectors are read as conflict-free 128-bit loads that the columns of a warp share).  Per token a warp
// forms the column's u^T S (R products and a shuffle tree: the only cross-lane step on the chain from token to token),
// the update (3 R FMAs) and the lanes' shares of S^T r, which are summed for a whole chunk at once afterwards.  The
// tokens go through shared memory in chunks of 16 over two buffers filled by cp.async: chunk c + 1 arrives while chunk
// c is walked.  The arithmetic of a token is the same for every chunking of its prompt and every batch: results are
// bit-identical across schedules.
//
// State: [slot][head][dv][dk] fp32 (a column's key channels contiguous), read at a segment's start, written at its end.
//
// A second front end, the GATED delta rule with one decay g and one step size beta per head and token,
//
//     S <- g S;   d = beta (v - S^T k);   S <- S + k d^T;   o = S^T q          (q, k of unit length, q times dk^(-1/2))
//
// is the same walk: S_t = g S_(t-1) - (beta g k)(k^T S_(t-1)) + (beta k) v^T, i.e. u = k, a u = beta g k, w = g on
// every channel, and beta k in the key's place.  gated_delta_prep forms these vectors per VALUE head (several value
// heads may share one q / k head) from the convolved q, k and the gate logits.
#include "prl_common.cuh"
#include <math.h>

namespace prl {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = 32 * kWarps;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ void cp4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp16(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct DeltaArgs {
  const float* P;          // projection rows: r, k, v, and (after delta_prep) the removal rate times the unit key
  int64_t ldp;
  int off_r, off_k, off_v, off_a;
  const float* w;          // decays [row][heads * dk] (after delta_prep)
  int64_t ldw;
  const float* u;          // unit keys [row][heads * dk]
  int64_t ldu;
  const float* V;          // values [row][heads * dv] at V + row * ldv (the caller folds the column offset in)
  int64_t ldv;
  int heads, dk, dv, chunk, vec4;
  const int32_t* seg_start;
  const int32_t* seg_len;
  const int32_t* seg_slot;
  float* state;
  float* out;
  int64_t ld_out;
  int n_seg;
};

// One warp per (token, head): u = k / sqrt(sum k^2 + eps) -> u_out; P[off_a] <- sigmoid(P[off_a] + a_bias) * u;
// zw <- exp(-decay_scale * sigmoid(zw + w_bias)).
__global__ void delta_prep_kernel(float* __restrict__ P, int64_t ldp, int off_k, int off_a, float* __restrict__ zw, int64_t ldw,
                                  const float* __restrict__ w_bias, const float* __restrict__ a_bias, float decay_scale,
                                  float unit_eps, int heads, int dk, float* __restrict__ u_out, int64_t ldu) {
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31;
  for (int head = threadIdx.x >> 5; head < heads; head += blockDim.x >> 5) {
    const int hoff = head * dk;
    float* p = P + row * ldp;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) { const float kv = p[off_k + hoff + i]; ss = fmaf(kv, kv, ss); }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss + unit_eps);
    for (int i = lane; i < dk; i += 32) {
      const float u = p[off_k + hoff + i] * inv;
      u_out[row * ldu + hoff + i] = u;
      p[off_a + hoff + i] = sigmoid_f(p[off_a + hoff + i] + a_bias[hoff + i]) * u;
      zw[row * ldw + hoff + i] = expf(-decay_scale * sigmoid_f(zw[row * ldw + hoff + i] + w_bias[hoff + i]));
    }
  }
}

// One warp per (token, value head).  C holds the convolved, activated q | k (kh heads of dk each) of the row; Z the
// logits of beta and of the decay.  D [row][5 * heads * dk] receives u | a u | w | k | r, each [heads][dk]:
//   u = k / sqrt(sum k^2 + unit_eps),  r = q / sqrt(sum q^2 + unit_eps) * dk^(-1/2),
//   beta = sigmoid(Z[off_b + h]),  g = exp(-exp(A_log[h]) * softplus(Z[off_a + h] + dt_bias[h])).
__global__ void gated_delta_prep_kernel(const float* __restrict__ C, int64_t ldc, int off_q, int off_k,
                                        const float* __restrict__ Z, int64_t ldz, int off_b, int off_a,
                                        const float* __restrict__ A_log, const float* __restrict__ dt_bias, float unit_eps,
                                        int heads, int kh, int dk, float* __restrict__ D) {
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int64_t ldd = (int64_t)5 * heads * dk, hd = (int64_t)heads * dk;
  const float q_scale = 1.f / sqrtf((float)dk);
  for (int head = threadIdx.x >> 5; head < heads; head += blockDim.x >> 5) {
    const int src_head = head / (heads / kh);
    const float* q = C + row * ldc + off_q + src_head * dk;
    const float* k = C + row * ldc + off_k + src_head * dk;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < dk; i += 32) { sq = fmaf(q[i], q[i], sq); sk = fmaf(k[i], k[i], sk); }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float inv_q = q_scale / sqrtf(sq + unit_eps), inv_k = 1.f / sqrtf(sk + unit_eps);
    const float beta = sigmoid_f(Z[row * ldz + off_b + head]);
    const float z = Z[row * ldz + off_a + head] + dt_bias[head];
    const float sp = z > 20.f ? z : log1pf(expf(z));
    const float g = expf(-expf(A_log[head]) * sp);
    float* d = D + row * ldd + head * dk;
    for (int i = lane; i < dk; i += 32) {
      const float u = k[i] * inv_k;
      d[i] = u;
      d[hd + i] = beta * g * u;
      d[2 * hd + i] = g;
      d[3 * hd + i] = beta * u;
      d[4 * hd + i] = q[i] * inv_q;
    }
  }
}

// per staged token: u | au | w | k | r, each dkp floats, then kCols values
// kLanes lanes share a value column, R key channels each; kCols = 4 warps x (32 / kLanes) columns per CTA
template <int R, int kLanes>
__global__ void __launch_bounds__(kThreads) delta_scan_kernel(DeltaArgs a) {
  constexpr int kColsPerWarp = 32 / kLanes;
  constexpr int kCols = kColsPerWarp * kWarps;
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int seg = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * kCols;
  const int len = a.seg_len[seg];
  if (len <= 0) return;
  const int dk = a.dk, dv = a.dv, TT = a.chunk;
  constexpr int dkp = R * kLanes;                 // padded key size: channels >= dk hold u = au = k = r = 0, w = 1
  constexpr int tok_floats = 5 * dkp + kCols;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = a.seg_slot[seg];
  const int64_t row0 = a.seg_start[seg];
  const int hoff = head * dk;
  const int buf_floats = TT * tok_floats;
  float* part = sm + 2 * buf_floats;              // [TT][kCols][kLanes]: the lanes' shares of S^T r, summed after the walk
  const int n_chunks = (len + TT - 1) / TT;

  // vectors of chunk c into its buffer: a thread owns fixed pieces (vector, channels) of a token row and walks the
  // chunk's tokens with them, so the copy loop is a pointer increment per token
  const int q = a.vec4 ? 4 : 1, per_vec = dk / q;               // channels per copy, copies per vector
  auto issue = [&](int c) {
    if (c < n_chunks) {
      const int t0 = c * TT, nt = min(TT, len - t0);
      float* buf = sm + (c & 1) * buf_floats;
      for (int i = tid; i < 5 * per_vec; i += kThreads) {
        const int which = i / per_vec, ch = (i - which * per_vec) * q;
        const float* src = which == 0 ? a.u + (row0 + t0) * a.ldu + hoff + ch
                         : which == 1 ? a.P + (row0 + t0) * a.ldp + a.off_a + hoff + ch
                         : which == 2 ? a.w + (row0 + t0) * a.ldw + hoff + ch
                         : which == 3 ? a.P + (row0 + t0) * a.ldp + a.off_k + hoff + ch
                                      : a.P + (row0 + t0) * a.ldp + a.off_r + hoff + ch;
        const int64_t ld = which == 0 ? a.ldu : (which == 2 ? a.ldw : a.ldp);
        float* dst = buf + which * dkp + ch;
        if (a.vec4) { for (int t = 0; t < nt; ++t) cp16(dst + t * tok_floats, src + t * ld); }
        else { for (int t = 0; t < nt; ++t) cp4(dst + t * tok_floats, src + t * ld); }
      }
      for (int i = tid; i < nt * kCols; i += kThreads) {
        const int t = i / kCols, ch = i - t * kCols;
        if (col0 + ch < dv) cp4(buf + t * tok_floats + 5 * dkp + ch, a.V + (row0 + t0 + t) * a.ldv + head * dv + col0 + ch);
      }
    }
    cp_commit();
  };
  if (dkp > dk)                                   // the padding channels, which no copy touches
    for (int i = tid; i < 2 * TT * 5 * (dkp - dk); i += kThreads) {
      const int t = i / (5 * (dkp - dk)), rest = i - t * 5 * (dkp - dk), which = rest / (dkp - dk), ch = dk + rest - which * (dkp - dk);
      sm[t * tok_floats + which * dkp + ch] = which == 2 ? 1.f : 0.f;
    }
  issue(0);

  const int sub = lane & (kLanes - 1);
  const int col = col0 + warp * kColsPerWarp + lane / kLanes;
  const bool col_on = col < dv;
  float* S_base = a.state + (((int64_t)slot * a.heads + head) * dv) * dk;
  float S[R];
#pragma unroll
  for (int jj = 0; jj < R / 4; ++jj)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 4 * (sub + kLanes * jj) + e;
      S[4 * jj + e] = (col_on && i < dk) ? S_base[(int64_t)col * dk + i] : 0.f;
    }
  float* my_part = part + (warp * kColsPerWarp + lane / kLanes) * kLanes + sub;
  const int v_at = 5 * dkp + warp * kColsPerWarp + lane / kLanes;
  for (int c = 0; c < n_chunks; ++c) {
    const int t0 = c * TT, nt = min(TT, len - t0);
    const float* buf = sm + (c & 1) * buf_floats;
    issue(c + 1);                                 // its buffer was walked one chunk ago
    cp_wait<1>();
    __syncthreads();
    // Only u^T S (its shuffle tree) sits on the chain from token to token: the lanes' shares of S^T r go to shared
    // memory unreduced and are summed for all tokens of the chunk afterwards.
    for (int t = 0; t < nt; ++t) {
      const float* src = buf + t * tok_floats;
      float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int jj = 0; jj < R / 4; ++jj) {
        const float4 u = *reinterpret_cast<const float4*>(src + 4 * (sub + kLanes * jj));
        d4[0] = fmaf(u.x, S[4 * jj], d4[0]); d4[1] = fmaf(u.y, S[4 * jj + 1], d4[1]);
        d4[2] = fmaf(u.z, S[4 * jj + 2], d4[2]); d4[3] = fmaf(u.w, S[4 * jj + 3], d4[3]);
      }
      float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
      for (int o = kLanes / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float vc = col_on ? src[v_at] : 0.f;
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int jj = 0; jj < R / 4; ++jj) {
        const int at = 4 * (sub + kLanes * jj);
        const float4 au = *reinterpret_cast<const float4*>(src + dkp + at);
        const float4 w = *reinterpret_cast<const float4*>(src + 2 * dkp + at);
        const float4 k = *reinterpret_cast<const float4*>(src + 3 * dkp + at);
        const float4 r = *reinterpret_cast<const float4*>(src + 4 * dkp + at);
        float s0 = w.x * S[4 * jj], s1 = w.y * S[4 * jj + 1], s2 = w.z * S[4 * jj + 2], s3 = w.w * S[4 * jj + 3];
        s0 = fmaf(-au.x, dot, s0); s1 = fmaf(-au.y, dot, s1); s2 = fmaf(-au.z, dot, s2); s3 = fmaf(-au.w, dot, s3);
        s0 = fmaf(k.x, vc, s0); s1 = fmaf(k.y, vc, s1); s2 = fmaf(k.z, vc, s2); s3 = fmaf(k.w, vc, s3);
        S[4 * jj] = s0; S[4 * jj + 1] = s1; S[4 * jj + 2] = s2; S[4 * jj + 3] = s3;
        a4[0] = fmaf(s0, r.x, a4[0]); a4[1] = fmaf(s1, r.y, a4[1]); a4[2] = fmaf(s2, r.z, a4[2]); a4[3] = fmaf(s3, r.w, a4[3]);
      }
      my_part[t * kCols * kLanes] = (a4[0] + a4[1]) + (a4[2] + a4[3]);
    }
    __syncthreads();
    for (int i = tid; i < nt * kCols; i += kThreads) {
      const int t = i / kCols, ch = i - t * kCols;
      if (col0 + ch < dv) {
        float o = 0.f;
#pragma unroll
        for (int l = 0; l < kLanes; ++l) o += part[i * kLanes + l];
        a.out[(row0 + t0 + t) * a.ld_out + head * dv + col0 + ch] = o;
      }
    }
    // the next chunk's copies overwrite the buffer walked here, and its walk the partial sums: both come behind the
    // barrier that follows the next cp_wait
  }
  if (col_on) {
#pragma unroll
    for (int jj = 0; jj < R / 4; ++jj)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * (sub + kLanes * jj) + e;
        if (i < dk) S_base[(int64_t)col * dk + i] = S[4 * jj + e];
      }
  }
}

}  // namespace
}  // namespace prl

using namespace prl;

// Launch of the walking kernel for prepared vectors (shared by the front ends below).
static int launch_delta_walk(DeltaArgs a, int max_len, cudaStream_t s) {
  const int dk = a.dk, dv = a.dv;
  // (key channels per lane, lanes per value column): four channels per lane up to dk = 128, so that a warp's instruction
  // stream per token is short; the shuffle tree grows with the lanes
  const int lanes = dk <= 16 ? 4 : (dk <= 32 ? 8 : (dk <= 64 ? 16 : 32));
  const int R = dk <= 128 ? 4 : 8;
  const int dkp = R * lanes, cols = (32 / lanes) * kWarps;
  a.chunk = 16;                                       // tokens per staged chunk, two chunks in shared memory
  if (max_len >= 1 && max_len < a.chunk) a.chunk = max_len;     // a decode step stages one token
  // 16-byte copies when every source address is a multiple of 16 bytes
  a.vec4 = dk % 4 == 0 && a.ldp % 4 == 0 && a.ldw % 4 == 0 && a.ldu % 4 == 0 && a.off_r % 4 == 0 && a.off_k % 4 == 0 && a.off_a % 4 == 0 &&
           ((uintptr_t)a.P & 15) == 0 && ((uintptr_t)a.w & 15) == 0 && ((uintptr_t)a.u & 15) == 0;
  const size_t smem = ((size_t)2 * a.chunk * (5 * dkp + cols) + (size_t)a.chunk * cols * lanes) * sizeof(float);   // <= 166 KB
  dim3 grid((dv + cols - 1) / cols, a.heads, a.n_seg);
  static SmemAttr attr[5] = {};
#define PRL_DELTA(RR, LL, I)                                                                  \
  do {                                                                                        \
    PRL_CUDA(ensure_smem((delta_scan_kernel<RR, LL>), (int)smem, attr[I]));                   \
    PRL_CUDA(launch_pdl((delta_scan_kernel<RR, LL>), grid, dim3(kThreads), smem, s, a));      \
  } while (0)
  if (R == 8) PRL_DELTA(8, 32, 4);
  else if (lanes == 4) PRL_DELTA(4, 4, 0);
  else if (lanes == 8) PRL_DELTA(4, 8, 1);
  else if (lanes == 16) PRL_DELTA(4, 16, 2);
  else PRL_DELTA(4, 32, 3);
#undef PRL_DELTA
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int64_t prl_delta_state_floats(int32_t heads, int32_t dk, int32_t dv) { return (int64_t)heads * dk * dv; }

extern "C" int prl_delta_scan(float* P, int64_t ldp, int32_t off_r, int32_t off_k, int32_t off_v, int32_t off_a, float* zw,
                              int64_t ldw, const float* w_bias, const float* a_bias, float decay_scale, float unit_eps,
                              int32_t heads, int32_t dk, int32_t dv, int32_t n_rows, float* unit_keys,
                              const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_slot, int32_t n_seg,
                              int32_t max_len, float* state, float* out, int64_t ld_out, prl_stream_t st) {
  PRL_CHECK_ARG(P && zw && w_bias && a_bias && unit_keys && seg_start && seg_len && seg_slot && state && out, "prl_delta_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && heads <= 65535 && dk >= 1 && dk <= 256 && dv >= 1 && n_seg >= 1 && n_seg <= 65535 && n_rows >= 1 &&
                ld_out >= (int64_t)heads * dv && ldw >= (int64_t)heads * dk,
                "prl_delta_scan: bad shape (heads=%d dk=%d dv=%d; dk <= 256)", heads, dk, dv);
  cudaStream_t s = (cudaStream_t)st;
  const int64_t ldu = (int64_t)heads * dk;
  int pw = heads < 8 ? heads : 8;
  PRL_CUDA(launch_pdl(delta_prep_kernel, dim3(n_rows), dim3(32 * pw), (size_t)0, s, P, ldp, off_k, off_a, zw, ldw, w_bias, a_bias,
                      decay_scale, unit_eps, heads, dk, unit_keys, ldu));
  PRL_LAUNCH_CHECK();
  DeltaArgs a{P, ldp, off_r, off_k, off_v, off_a, zw, ldw, unit_keys, ldu, P + off_v, ldp, heads, dk, dv, 0, 0,
              seg_start, seg_len, seg_slot, state, out, ld_out, n_seg};
  return launch_delta_walk(a, max_len, s);
}

// The gated delta rule over ragged segments.  C [n_rows][ldc]: the convolved and activated q (off_q), k (off_k), both
// kh heads of dk, and v (off_v, `heads` heads of dv); Z [n_rows][ldz]: the logits of beta (off_b) and of the decay
// (off_a), one per value head; scratch [n_rows][5 * heads * dk] fp32; state as prl_delta_state_floats(heads, dk, dv).
extern "C" int prl_gated_delta_scan(const float* C, int64_t ldc, int32_t off_q, int32_t off_k, int32_t off_v, const float* Z,
                                    int64_t ldz, int32_t off_b, int32_t off_a, const float* A_log, const float* dt_bias,
                                    float unit_eps, int32_t heads, int32_t kh, int32_t dk, int32_t dv, int32_t n_rows,
                                    float* scratch, const int32_t* seg_start, const int32_t* seg_len,
                                    const int32_t* seg_slot, int32_t n_seg, int32_t max_len, float* state, float* out,
                                    int64_t ld_out, prl_stream_t st) {
  PRL_CHECK_ARG(C && Z && A_log && dt_bias && scratch && seg_start && seg_len && seg_slot && state && out,
                "prl_gated_delta_scan: NULL argument");
  PRL_CHECK_ARG(heads >= 1 && heads <= 65535 && kh >= 1 && heads % kh == 0 && dk >= 1 && dk <= 256 && dv >= 1 && n_seg >= 1 &&
                n_seg <= 65535 && n_rows >= 1 && ld_out >= (int64_t)heads * dv,
                "prl_gated_delta_scan: bad shape (heads=%d q/k heads=%d dk=%d dv=%d; dk <= 256)", heads, kh, dk, dv);
  cudaStream_t s = (cudaStream_t)st;
  const int pw = heads < 8 ? heads : 8;
  PRL_CUDA(launch_pdl(gated_delta_prep_kernel, dim3(n_rows), dim3(32 * pw), (size_t)0, s, C, ldc, off_q, off_k, Z, ldz, off_b,
                      off_a, A_log, dt_bias, unit_eps, heads, kh, dk, scratch));
  PRL_LAUNCH_CHECK();
  const int hd = heads * dk;
  const int64_t ldd = (int64_t)5 * hd;
  DeltaArgs a{scratch, ldd, 4 * hd, 3 * hd, 0, hd, scratch + 2 * hd, ldd, scratch, ldd, C + off_v, ldc, heads, dk, dv, 0, 0,
              seg_start, seg_len, seg_slot, state, out, ld_out, n_seg};
  return launch_delta_walk(a, max_len, s);
}
