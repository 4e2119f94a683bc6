// Residual stream kept as several parallel copies ("hyper-connections"), the statistics-free tanh norm, per-channel
// layer scale and a sigmoid gate on a sublayer's result, and a token embedding with a hashed token-pair table.
//
// The residual of a row is S streams xs[row][s][W] (fp32).  A sublayer reads
//     u = sum_s w_in[s] xs[s],          h = tanh(alpha u) * gain + shift                       (streams_open)
// and its result y (the sum of `n_split` slices: split-K partials of a GEMM or the choices of a routed feed-forward)
// goes back as
//     y <- y * scale[c] * sigmoid(gate[c] + gate_bias[c])                 (scale / gate optional)
//     xs'[t] = sum_s mix[s][t] xs[s] + w_out[t] y      for every t at once, from the old streams        (streams_close)
// after which the NEXT reader's u and h are formed in the same kernel (its w_in / alpha / gain / shift), so one launch
// per sublayer touches the streams.  S = 1 with mix = [[1]], w_out = [1] is the ordinary residual sum; w_in = ones
// gives the plain sum of the streams (what the model's last norm reads).  Everything is fp32; h is stored in the GEMM
// operand type.  One thread owns a channel of a row, so a row's values never depend on the batch.
#include "prl_common.cuh"
#include <math.h>

namespace prl {
namespace {

constexpr int kMaxStreams = 8;

template <typename T> __device__ __forceinline__ float ldf(const T* p, int64_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

struct TanhNorm {             // h = tanh(alpha[0] u) * gain[c] + shift[c]
  const float* alpha;
  const float* gain;
  const float* shift;
};

// x = embed[token] * scale + pair[row], row = (prev * mul_prev + token * mul_cur) mod buckets, or `buckets` (the extra
// last row) for the first token of a sequence.  prev is the row before in the same segment, or, for a segment's first
// row, the sequence's last token of an earlier batch (prev_state[slot]).  Every stream starts as x; h for the first
// reader (u = x * sum(w_in)) is written too.
template <typename T>
__global__ void embed_pair_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ row_pos,
                                  const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_back,
                                  const int32_t* __restrict__ prev_state, const T* __restrict__ embed,
                                  const T* __restrict__ pair, float scale, int buckets, int mul_prev, int mul_cur, int W,
                                  int vocab, int S, const float* __restrict__ w_in, TanhNorm nm, float* __restrict__ xs,
                                  T* __restrict__ ha) {
  pdl_wait();
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;                                     // an idle slot of the decode step
  int tok = tokens[r];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  int64_t prow = -1;
  if (pair) {
    if (row_pos[r] == 0) prow = buckets;
    else {
      int prev = row_back[r] > 0 ? tokens[r - 1] : prev_state[slot];
      prev = prev < 0 ? 0 : (prev >= vocab ? vocab - 1 : prev);
      prow = ((int64_t)prev * mul_prev + (int64_t)tok * mul_cur) % buckets;
    }
  }
  const float alpha = nm.alpha[0];
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = ldf(embed, (int64_t)tok * W + c) * scale;
    if (prow >= 0) v += ldf(pair, prow * W + c);
    for (int s = 0; s < S; ++s) xs[((int64_t)r * S + s) * W + c] = v;
    float u = 0.f;                                          // the same sum streams_open forms: S terms in stream order
    for (int s = 0; s < S; ++s) u = fmaf(w_in[s], v, u);
    stf(ha, (int64_t)r * W + c, tanhf(alpha * u) * nm.gain[c] + nm.shift[c]);
  }
}

// prev_state[slot] = the segment's last token (run after the embedding of the batch)
__global__ void last_token_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ seg_start,
                                  const int32_t* __restrict__ seg_len, const int32_t* __restrict__ seg_slot, int n_seg,
                                  int32_t* __restrict__ prev_state) {
  pdl_wait();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n_seg) return;
  const int len = seg_len[s];
  if (len <= 0) return;
  prev_state[seg_slot[s]] = tokens[seg_start[s] + len - 1];
}

template <typename T>
__global__ void streams_open_kernel(const float* __restrict__ xs, const int32_t* __restrict__ rows, int S, int W,
                                    const float* __restrict__ w_in, TanhNorm nm, T* __restrict__ ha) {
  pdl_wait();
  const int i = blockIdx.x;
  const int64_t r = rows ? rows[i] : i;
  const float alpha = nm.alpha[0];
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float u = 0.f;
    for (int s = 0; s < S; ++s) u = fmaf(w_in[s], xs[(r * S + s) * W + c], u);
    stf(ha, (int64_t)i * W + c, tanhf(alpha * u) * nm.gain[c] + nm.shift[c]);
  }
}

template <typename T> __device__ __forceinline__ void st4(T* p, int64_t i, const float (&v)[4]);
template <> __device__ __forceinline__ void st4<float>(float* p, int64_t i, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p + i) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// V consecutive channels per thread (V = 4: 128-bit loads and stores; every row stride and base a multiple of 4 floats).
// A channel's arithmetic is the same for both widths.
template <typename T, int V, int SMAX>
__global__ void __launch_bounds__(512) streams_close_kernel(const float* __restrict__ y, int64_t ldy, int n_split, int64_t split_stride,
                                     const float* __restrict__ scale, const float* __restrict__ gate, int64_t ldg,
                                     const float* __restrict__ gate_bias, const float* __restrict__ mix,
                                     const float* __restrict__ w_out, int S, int W, float* __restrict__ xs,
                                     const float* __restrict__ next_in, TanhNorm nm, T* __restrict__ ha) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  __shared__ float sm_mix[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  float* sm_out = sm_mix + kMaxStreams * kMaxStreams;
  float* sm_in = sm_out + kMaxStreams;
  if (threadIdx.x < S * S) sm_mix[threadIdx.x] = mix[threadIdx.x];
  if (threadIdx.x < S) {
    sm_out[threadIdx.x] = w_out[threadIdx.x];
    sm_in[threadIdx.x] = next_in ? next_in[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const float alpha = next_in ? nm.alpha[0] : 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float v[V], old[SMAX][V], h[V];
#pragma unroll
    for (int e = 0; e < V; ++e) v[e] = 0.f;
    for (int k = 0; k < n_split; ++k) {                               // slices in order
      const float* p = y + k * split_stride + r * ldy + c;
      if constexpr (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w; }
      else v[0] += p[0];
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      if (scale) v[e] *= scale[c + e];
      if (gate) v[e] *= sigmoid_f(gate[r * ldg + c + e] + (gate_bias ? gate_bias[c + e] : 0.f));
    }
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      if (s < S) {
        const float* p = xs + (r * S + s) * W + c;
        if constexpr (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); old[s][0] = t.x; old[s][1] = t.y; old[s][2] = t.z; old[s][3] = t.w; }
        else old[s][0] = p[0];
      }
    }
    float u[V];
#pragma unroll
    for (int e = 0; e < V; ++e) u[e] = 0.f;
#pragma unroll
    for (int t = 0; t < SMAX; ++t) {
      if (t >= S) break;
      float a[V];
#pragma unroll
      for (int e = 0; e < V; ++e) {
        a[e] = 0.f;
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < S) a[e] = fmaf(sm_mix[s * S + t], old[s][e], a[e]);
        a[e] = fmaf(sm_out[t], v[e], a[e]);
        u[e] = fmaf(sm_in[t], a[e], u[e]);
      }
      float* p = xs + (r * S + t) * W + c;
      if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1], a[2], a[3]);
      else p[0] = a[0];
    }
    if (next_in) {
#pragma unroll
      for (int e = 0; e < V; ++e) h[e] = tanhf(alpha * u[e]) * nm.gain[c + e] + nm.shift[c + e];
      if constexpr (V == 4) st4(ha, r * W + c, h);
      else stf(ha, r * W + c, h[0]);
    }
  }
}

inline int row_threads(int W) { return W >= 1024 ? 256 : (W >= 256 ? 128 : 64); }

}  // namespace
}  // namespace prl

using namespace prl;
typedef __nv_bfloat16 bf16;

extern "C" int prl_embed_pair(const int32_t* tokens, const int32_t* row_pos, const int32_t* row_slot, const int32_t* row_back,
                              const int32_t* prev_state, const void* embed, const void* pair, int32_t f32, float scale,
                              int32_t buckets, int32_t mul_prev, int32_t mul_cur, int32_t n, int32_t W, int32_t vocab,
                              int32_t S, const float* w_in, const float* alpha, const float* gain, const float* shift,
                              float* xs, void* ha, prl_stream_t st) {
  PRL_CHECK_ARG(tokens && row_pos && row_slot && row_back && embed && w_in && alpha && gain && shift && xs && ha,
                "prl_embed_pair: NULL argument");
  PRL_CHECK_ARG(n >= 1 && W >= 1 && vocab >= 1 && S >= 1 && S <= kMaxStreams && (!pair || (prev_state && buckets >= 1)),
                "prl_embed_pair: bad shape (streams=%d, at most %d)", S, kMaxStreams);
  TanhNorm nm{alpha, gain, shift};
  if (f32) PRL_CUDA(launch_pdl(embed_pair_kernel<float>, dim3(n), dim3(row_threads(W)), (size_t)0, (cudaStream_t)st, tokens, row_pos, row_slot, row_back, prev_state, (const float*)embed, (const float*)pair, scale, buckets, mul_prev, mul_cur, W, vocab, S, w_in, nm, xs, (float*)ha));
  else PRL_CUDA(launch_pdl(embed_pair_kernel<bf16>, dim3(n), dim3(row_threads(W)), (size_t)0, (cudaStream_t)st, tokens, row_pos, row_slot, row_back, prev_state, (const bf16*)embed, (const bf16*)pair, scale, buckets, mul_prev, mul_cur, W, vocab, S, w_in, nm, xs, (bf16*)ha));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_last_token(const int32_t* tokens, const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_slot,
                              int32_t n_seg, int32_t* prev_state, prl_stream_t st) {
  PRL_CHECK_ARG(tokens && seg_start && seg_len && seg_slot && prev_state && n_seg >= 1, "prl_last_token: bad argument");
  PRL_CUDA(launch_pdl(last_token_kernel, dim3((n_seg + 127) / 128), dim3(128), (size_t)0, (cudaStream_t)st, tokens, seg_start, seg_len, seg_slot, n_seg, prev_state));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_streams_open(const float* xs, const int32_t* rows, int32_t n_out, int32_t S, int32_t W, const float* w_in,
                                const float* alpha, const float* gain, const float* shift, void* ha, int32_t f32,
                                prl_stream_t st) {
  PRL_CHECK_ARG(xs && w_in && alpha && gain && shift && ha && n_out >= 1 && W >= 1 && S >= 1 && S <= kMaxStreams,
                "prl_streams_open: bad argument");
  TanhNorm nm{alpha, gain, shift};
  if (f32) PRL_CUDA(launch_pdl(streams_open_kernel<float>, dim3(n_out), dim3(row_threads(W)), (size_t)0, (cudaStream_t)st, xs, rows, S, W, w_in, nm, (float*)ha));
  else PRL_CUDA(launch_pdl(streams_open_kernel<bf16>, dim3(n_out), dim3(row_threads(W)), (size_t)0, (cudaStream_t)st, xs, rows, S, W, w_in, nm, (bf16*)ha));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_streams_close(const float* y, int64_t ldy, int32_t n_split, int64_t split_stride, const float* scale,
                                 const float* gate, int64_t ldg, const float* gate_bias, const float* mix, const float* w_out,
                                 int32_t S, int32_t n, int32_t W, float* xs, const float* next_in, const float* next_alpha,
                                 const float* next_gain, const float* next_shift, void* ha, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(y && mix && w_out && xs && n >= 1 && W >= 1 && S >= 1 && S <= kMaxStreams && n_split >= 1 && ldy >= W,
                "prl_streams_close: bad argument");
  PRL_CHECK_ARG(!next_in || (next_alpha && next_gain && next_shift && ha), "prl_streams_close: the next norm is incomplete");
  PRL_CHECK_ARG(!gate || ldg >= W, "prl_streams_close: bad gate stride");
  TanhNorm nm{next_alpha, next_gain, next_shift};
  const bool v4 = S <= 4 && W % 4 == 0 && ldy % 4 == 0 && split_stride % 4 == 0 && (!gate || ldg % 4 == 0) && ((uintptr_t)y & 15) == 0 &&
                  ((uintptr_t)xs & 15) == 0 && (!gate || ((uintptr_t)gate & 15) == 0) && (!ha || ((uintptr_t)ha & 15) == 0);
  int th = v4 ? (W / 4 + 31) / 32 * 32 : row_threads(W);
  th = th > 512 ? 512 : (th < 96 ? 96 : th);                    // at least S*S + S threads fill the shared tables
#define PRL_CLOSE(TT, VV, SS) PRL_CUDA(launch_pdl((streams_close_kernel<TT, VV, SS>), dim3(n), dim3(th), (size_t)0, (cudaStream_t)st, y, ldy, n_split, split_stride, scale, gate, ldg, gate_bias, mix, w_out, S, W, xs, next_in, nm, (TT*)ha))
  if (f32) { if (S > 4) PRL_CLOSE(float, 1, kMaxStreams); else if (v4) PRL_CLOSE(float, 4, 4); else PRL_CLOSE(float, 1, 4); }
  else { if (S > 4) PRL_CLOSE(bf16, 1, kMaxStreams); else if (v4) PRL_CLOSE(bf16, 4, 4); else PRL_CLOSE(bf16, 1, 4); }
#undef PRL_CLOSE
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}
