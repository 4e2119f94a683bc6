// Row kernels of the hybrid decoder family (models that mix softmax attention, state-space and gated-linear-attention
// mixers and normalise the SUBLAYER OUTPUT instead of its input).  All of them work on a packed batch of n token rows
// that may belong to several sequences ("ragged rows": a prompt chunk next to single decoded tokens), described by
//   row_pos[n]   position of the token in its sequence,
//   row_slot[n]  state / block-table slot of its sequence (< 0: idle row, nothing is read or written for it),
//   row_back[n]  how many rows of the same sequence precede this one inside the batch.
// Arithmetic is fp32 throughout; `T` is only the storage type of what feeds the next GEMM or the KV cache (bf16 when
// the engine serves in bf16, fp32 in the true-fp32 mode).  Small parameter vectors (norm gains, biases, convolution
// taps) are read as fp32 copies the engine keeps beside the weight arena.
#include "prl_common.cuh"

namespace prl {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, int64_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// Sum over the block in a fixed order (warp shuffles, then the warps' partials in index order): the result for a row
// never depends on which other rows are in the launch.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += red[w];
  return t;
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

// x = embed[token] * scale (fp32 residual) and its copy in the GEMM operand type
template <typename T>
__global__ void embed_scale_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ embed, float scale, int W,
                                   int vocab, float* __restrict__ x, T* __restrict__ xa) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  const int r = blockIdx.x;
  int tok = tokens[r];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = ldf(embed, (int64_t)tok * W + c) * scale;
    x[(int64_t)r * W + c] = v;
    stf(xa, (int64_t)r * W + c, v);
  }
}

// Post-norm residual:  y = s0*y0 + s1*y1;  x += y / sqrt(mean(y^2) + eps) * gain;  xa = T(x).
// y0 / y1 may arrive as split-K partial slices [n_split][n][ld] of a GEMM: they are summed here in slice order.
template <typename T>
__global__ void postnorm_residual_kernel(const float* __restrict__ y0, int64_t ld0, float s0, int ns0, int64_t stride0,
                                         const float* __restrict__ y1, int64_t ld1, float s1, int ns1, int64_t stride1,
                                         const float* __restrict__ gain, float eps, int W, int keep, float* __restrict__ x,
                                         T* __restrict__ xa) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  extern __shared__ float ybuf[];    // [W] the row's y between the two passes (empty: recomputed)
  __shared__ float red[32];
  const int r = blockIdx.x;
  auto value = [&](int c) {
    float a = 0.f;
#pragma unroll 4
    for (int k = 0; k < ns0; ++k) a += y0[k * stride0 + (int64_t)r * ld0 + c];
    float y = s0 * a;
    if (y1) {
      float b = 0.f;
#pragma unroll 4
      for (int k = 0; k < ns1; ++k) b += y1[k * stride1 + (int64_t)r * ld1 + c];
      y += s1 * b;
    }
    return y;
  };
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float y = value(c);
    if (keep) ybuf[c] = y;
    ss += y * y;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float y = keep ? ybuf[c] : value(c);      // same thread wrote it
    const float v = x[(int64_t)r * W + c] + y * inv * gain[c];
    x[(int64_t)r * W + c] = v;
    stf(xa, (int64_t)r * W + c, v);
  }
}

// out[i] = T(x[rows[i]] / rms * gain)   (rows == NULL: identity)
template <typename T>
__global__ void rmsnorm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                    const float* __restrict__ gain, float eps, int W, T* __restrict__ out) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  __shared__ float red[32];
  const int i = blockIdx.x;
  const int64_t r = rows ? rows[i] : i;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = x[r * W + c];
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) stf(out, (int64_t)i * W + c, x[r * W + c] * inv * gain[c]);
}

// Gate and (group) norm between a mixer and its output projection.  One block per (row, group) of `gs` channels:
//   gate_first:  v = o * act(g);  out = v / rms_group(v) * gain      (state-space mixer: gate, then grouped RMS norm)
//   otherwise :  out = o / rms_group(o) * gain * act(g)              (linear attention: per-head norm, then gate)
//   norm == 0 :  out = o * act(g)                                    (softmax attention output gate)
// gain index = channel % gain_period (a per-head gain shared by all heads has gain_period = head size).
template <typename T, typename TO>
__global__ void gate_norm_kernel(const TO* __restrict__ o, int64_t ldo, const float* __restrict__ g, int64_t ldg,
                                 const float* __restrict__ gain, int gain_period, int gs, int C, int act_sigmoid,
                                 int gate_first, int norm, float eps, int keep, T* __restrict__ out) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  extern __shared__ float kept[];    // [2][gs]: the values to be normed and the gates between the two passes (keep)
  __shared__ float red[32];
  const int r = blockIdx.x, c0 = blockIdx.y * gs;
  const float* gr = g + (int64_t)r * ldg + c0;
  const int64_t ro = (int64_t)r * ldo + c0;
  float inv = 1.f;
  if (norm) {
    float ss = 0.f;
#pragma unroll 4
    for (int j = threadIdx.x; j < gs; j += blockDim.x) {
      float v = ldf(o, ro + j);
      if (gate_first || keep) {
        const float z = gr[j];
        const float a = act_sigmoid ? sigmoid_f(z) : silu_f(z);
        if (gate_first) v *= a;
        if (keep) { kept[j] = v; kept[gs + j] = a; }      // read back by the same thread
      }
      ss += v * v;
    }
    ss = block_sum(ss, red);
    inv = 1.f / sqrtf(ss / (float)gs + eps);
  }
  const bool kept_here = norm && keep;
#pragma unroll 4
  for (int j = threadIdx.x; j < gs; j += blockDim.x) {
    const int c = c0 + j;
    float a, v;
    if (kept_here) {
      v = kept[j];
      a = kept[gs + j];
    } else {
      const float z = gr[j];
      a = act_sigmoid ? sigmoid_f(z) : silu_f(z);
      v = ldf(o, ro + j);
      if (norm && gate_first) v *= a;
    }
    if (norm) v = gate_first ? v * inv * gain[c % gain_period] : v * inv * gain[c % gain_period] * a;
    else v = v * a;
    stf(out, (int64_t)r * C + c, v);
  }
}

// Clamped gated feed-forward activation: g = min(gate, lim), u = clamp(up, -lim, lim), y = g*sigmoid(beta*g)*(u+1)
template <typename T>
__global__ void glu_clamped_kernel(const float* __restrict__ gu, int64_t ld, int F, float lim, float beta,
                                   T* __restrict__ out) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= F) return;
  const float g = fminf(gu[r * ld + c], lim);
  const float u = fminf(fmaxf(gu[r * ld + F + c], -lim), lim);
  stf(out, r * F + c, g * sigmoid_f(beta * g) * (u + 1.f));
}

// Attention front end for one row: RMS norm over the WHOLE q projection and over the whole k projection (before the
// split into heads), rotary embedding on the first `rot` channels of every head with interleaved pairs (2i, 2i+1),
// q to the query buffer, k / v into the paged cache.  Angles are formed in double (position * frequency) so that a
// position in the tens of thousands keeps full fp32 accuracy in sin / cos.
template <typename T>
__global__ void qk_norm_rope_cache_kernel(const float* __restrict__ P, int64_t ldp, int off_q, int off_k, int off_v,
                                          int H, int G, int dim, int vdim, int rot, const double* __restrict__ freq,
                                          const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                                          const int32_t* __restrict__ row_pos, const int32_t* __restrict__ row_slot,
                                          const int32_t* __restrict__ block_table, int max_blocks, int page_size,
                                          T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  extern __shared__ float cs[];  // [rot/2] cos | [rot/2] sin
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int pos = row_pos[r];
  const float* q = P + (int64_t)r * ldp + off_q;
  const float* k = P + (int64_t)r * ldp + off_k;
  const float* v = P + (int64_t)r * ldp + off_v;
  const int nq = H * dim, nk = G * dim, nv = G * vdim, half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    // angle = position * frequency in double, reduced to [-pi, pi] in double (four double operations), then the
    // fp32 sincos of an argument that small is exact to an ulp; a double sincos would cost more than the rest of the row
    const double ang = (double)pos * freq[i];
    const double turns = rint(ang * 0.15915494309189535);
    const float red_ang = (float)fma(-turns, 6.283185307179586, ang);
    float sn, cn;
    sincosf(red_ang, &sn, &cn);
    cs[i] = cn;
    cs[half + i] = sn;
  }
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) sq += q[i] * q[i];
  for (int i = threadIdx.x; i < nk; i += blockDim.x) sk += k[i] * k[i];
  sq = block_sum(sq, red);
  sk = block_sum(sk, red);
  const float iq = 1.f / sqrtf(sq / (float)nq + eps), ik = 1.f / sqrtf(sk / (float)nk + eps);
  const int page = block_table[(int64_t)slot * max_blocks + pos / page_size], within = pos % page_size;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const bool is_q = i < nq;
    const int e = is_q ? i : i - nq;
    const float* src = is_q ? q : k;
    const float* gn = is_q ? q_gain : k_gain;
    const float inv = is_q ? iq : ik;
    const int head = e / dim, j = e % dim;
    float val = src[e] * inv * gn[e];
    if (j < rot) {
      const int pe = (j & 1) ? e - 1 : e + 1;
      const float other = src[pe] * inv * gn[pe];
      const float c = cs[j >> 1], s = cs[half + (j >> 1)];
      val = (j & 1) ? val * c + other * s : val * c - other * s;
    }
    if (is_q) stf(q_out, (int64_t)r * nq + e, val);
    else stf(k_pool, (((int64_t)page * G + head) * page_size + within) * dim + j, val);
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int head = i / vdim, j = i % vdim;
    stf(v_pool, (((int64_t)page * G + head) * page_size + within) * vdim + j, v[i]);
  }
}

// Causal depthwise convolution + SiLU over ragged rows.  Input channel c of row r is P[r, off + c]; the tap that reaches
// k tokens back reads row r-k if that row belongs to the same sequence inside this batch (k <= row_back[r]) and the
// sequence's carried state otherwise.  state[slot][c][0..taps-2] holds the last taps-1 inputs, oldest first (zeros at
// the start of a sequence).  w[c][taps-1] multiplies the current token.
__global__ void conv_silu_kernel(const float* __restrict__ P, int64_t ldp, int off, int ch, int taps,
                                 const float* __restrict__ w, const float* __restrict__ b,
                                 const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_back,
                                 const float* __restrict__ state, float* __restrict__ out) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int back = row_back[r];
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ch; c += gridDim.y * blockDim.x) {
    float acc = b[c];
    const float* st = state + ((int64_t)slot * ch + c) * (taps - 1);
    for (int k = taps - 1; k >= 0; --k) {   // oldest tap first: a fixed summation order
      const float in = (k <= back) ? P[(int64_t)(r - k) * ldp + off + c] : st[taps - 1 - (k - back)];
      acc = fmaf(w[(int64_t)c * taps + (taps - 1 - k)], in, acc);
    }
    out[(int64_t)r * ch + c] = silu_f(acc);
  }
}

// After the convolution of a batch: shift the sequence's last taps-1 inputs into its state (a segment shorter than
// taps-1 keeps the tail of the old state).  One thread per (segment, channel) reads everything it needs before it writes.
__global__ void conv_state_kernel(const float* __restrict__ P, int64_t ldp, int off, int ch, int taps,
                                  const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_len,
                                  const int32_t* __restrict__ seg_slot, float* __restrict__ state) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  const int s = blockIdx.y;
  const int len = seg_len[s];
  if (len <= 0) return;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ch) return;
  const int keep = taps - 1;
  float* st = state + ((int64_t)seg_slot[s] * ch + c) * keep;
  const int64_t last = (int64_t)seg_start[s] + len - 1;
  constexpr int kMaxKeep = 15;
  float nv[kMaxKeep];
  for (int j = 0; j < keep; ++j) {
    const int e = keep - 1 - j;  // tokens back from the last row of the segment
    nv[j] = (e < len) ? P[(last - e) * ldp + off + c] : st[j + len];
  }
  for (int j = 0; j < keep; ++j) st[j] = nv[j];
}

// Decode step: turn the engine's per-slot state into ragged-row metadata (one row per slot).
__global__ void decode_rows_kernel(const uint8_t* __restrict__ active, int B, int32_t* __restrict__ seg_len,
                                   int32_t* __restrict__ row_slot) {
  pdl_wait();   // launched with the programmatic-serialization attribute like the engine's other step kernels; no early
                // trigger: letting the next grid become resident early measured +3 ms on a 4096-token prefill and +-0 on decode
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int a = active[b] ? 1 : 0;
  seg_len[b] = a;
  row_slot[b] = a ? b : -1;
}

// x = embed[token] * scale + sinusoidal position vector: channel 2i carries sin(pos * freq[i]), channel 2i+1 the cosine
// (freq[i] = base^(-2i/W), given in double; the angle is formed and reduced in double as for the rotary embedding).
// Written to the fp32 residual, to its operand-type copy xa and (x0a != NULL) to a second copy that later layers read
// as "the embedding output".
template <typename T>
__global__ void embed_sinusoid_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ embed, float scale,
                                      const double* __restrict__ freq, const int32_t* __restrict__ row_pos, int W, int vocab,
                                      float* __restrict__ x, T* __restrict__ xa, T* __restrict__ x0a) {
  pdl_wait();
  const int r = blockIdx.x;
  int tok = tokens[r];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const int pos = row_pos[r];
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const double ang = (double)pos * freq[c >> 1];
    const double turns = rint(ang * 0.15915494309189535);
    const float red_ang = (float)fma(-turns, 6.283185307179586, ang);
    float sn, cn;
    sincosf(red_ang, &sn, &cn);
    const float v = ldf(embed, (int64_t)tok * W + c) * scale + ((c & 1) ? cn : sn);
    x[(int64_t)r * W + c] = v;
    stf(xa, (int64_t)r * W + c, v);
    if (x0a) stf(x0a, (int64_t)r * W + c, v);
  }
}

// out[r] = [a[r] | b[r]]  (two row blocks of width W side by side: the operand of a projection that reads both)
template <typename T>
__global__ void concat_rows_kernel(const T* __restrict__ a, const T* __restrict__ b, int W, T* __restrict__ out) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    out[r * 2 * W + c] = a[r * W + c];
    out[r * 2 * W + W + c] = b[r * W + c];
  }
}

// The close of a sublayer whose branches, sum and successor all carry their own RMS norms:
//   b_i = y_i / rms(y_i) * gain_i   (gain_i == NULL: b_i = y_i)              i = 0, 1 (y1 may be absent)
//   v   = s0 b_0 + s1 b_1
//   v   = v / rms(v) * post_gain    (post_gain == NULL: unchanged)
//   x   = (add ? x : 0) + v + bias  (bias == NULL: none)
//   xa  = T(x / rms(x) * next_gain) (next_gain == NULL: T(x)) -- the input of the NEXT sublayer's projection
// y_i may arrive as split-K partial slices [n_split][n][ld] of a GEMM (or as the per-choice outputs of a routed
// feed-forward): they are summed here in slice order.  One block per row; the row stays in shared memory.
template <typename T>
__global__ void sublayer_close_kernel(const float* __restrict__ y0, int64_t ld0, int ns0, int64_t stride0,
                                      const float* __restrict__ gain0, float s0, const float* __restrict__ y1, int64_t ld1,
                                      int ns1, int64_t stride1, const float* __restrict__ gain1, float s1,
                                      const float* __restrict__ post_gain, const float* __restrict__ bias, int add,
                                      const float* __restrict__ next_gain, float eps, int W, float* __restrict__ x,
                                      T* __restrict__ xa) {
  pdl_wait();
  extern __shared__ float rowbuf[];    // [W] y0 (then v, then x) | [W] y1
  __shared__ float red[32];
  float* b0 = rowbuf;
  float* b1 = rowbuf + W;
  const int64_t r = blockIdx.x;
  float ss0 = 0.f, ss1 = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < ns0; ++k) a += y0[k * stride0 + r * ld0 + c];
    b0[c] = a;
    ss0 += a * a;
    if (y1) {
      float b = 0.f;
      for (int k = 0; k < ns1; ++k) b += y1[k * stride1 + r * ld1 + c];
      b1[c] = b;
      ss1 += b * b;
    }
  }
  float i0 = 1.f, i1 = 1.f;
  if (gain0) i0 = 1.f / sqrtf(block_sum(ss0, red) / (float)W + eps);
  if (y1 && gain1) i1 = 1.f / sqrtf(block_sum(ss1, red) / (float)W + eps);
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {        // every thread touches only the columns it wrote
    float v = s0 * (gain0 ? b0[c] * i0 * gain0[c] : b0[c]);
    if (y1) v += s1 * (gain1 ? b1[c] * i1 * gain1[c] : b1[c]);
    b0[c] = v;
    ss += v * v;
  }
  float ip = 1.f;
  if (post_gain) ip = 1.f / sqrtf(block_sum(ss, red) / (float)W + eps);
  float sx = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = post_gain ? b0[c] * ip * post_gain[c] : b0[c];
    if (bias) v += bias[c];
    if (add) v += x[r * W + c];
    x[r * W + c] = v;
    b0[c] = v;
    sx += v * v;
  }
  float in = 1.f;
  if (next_gain) in = 1.f / sqrtf(block_sum(sx, red) / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) stf(xa, r * W + c, next_gain ? b0[c] * in * next_gain[c] : b0[c]);
}

// Attention front end with PER-HEAD unit norms: q and k get their biases (NULL: none), every head of q and of k is
// divided by its own root mean square over `dim` and multiplied by a gain (NULL: none; indexed head * dim + channel);
// q goes to the query buffer, k into the paged cache.  The value written beside it is either the key as projected
// (bias added, BEFORE its norm: off_v < 0, then vdim == dim) or columns off_v.. of P (bias-free).  One warp per head.
template <typename T>
__global__ void qk_headnorm_cache_kernel(const float* __restrict__ P, int64_t ldp, int off_q, int off_k, int off_v, int H,
                                         int G, int dim, int vdim, const float* __restrict__ q_bias,
                                         const float* __restrict__ k_bias, const float* __restrict__ q_gain,
                                         const float* __restrict__ k_gain, float eps, const int32_t* __restrict__ row_pos,
                                         const int32_t* __restrict__ row_slot, const int32_t* __restrict__ block_table,
                                         int max_blocks, int page_size, T* __restrict__ q_out, T* __restrict__ k_pool,
                                         T* __restrict__ v_pool) {
  pdl_wait();
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int pos = row_pos[r];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int page = block_table[(int64_t)slot * max_blocks + pos / page_size], within = pos % page_size;
  for (int hh = warp; hh < H + G; hh += nw) {
    const bool is_q = hh < H;
    const int head = is_q ? hh : hh - H;
    const float* src = P + (int64_t)r * ldp + (is_q ? off_q : off_k) + head * dim;
    const float* bias = is_q ? q_bias : k_bias;
    const float* gain = is_q ? q_gain : k_gain;
    float ss = 0.f;
    for (int j = lane; j < dim; j += 32) {
      const float v = src[j] + (bias ? bias[head * dim + j] : 0.f);
      ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dim + eps);
    for (int j = lane; j < dim; j += 32) {
      const float raw = src[j] + (bias ? bias[head * dim + j] : 0.f);
      const float v = raw * inv * (gain ? gain[head * dim + j] : 1.f);
      if (is_q) {
        stf(q_out, ((int64_t)r * H + head) * dim + j, v);
      } else {
        const int64_t at = (((int64_t)page * G + head) * page_size + within) * dim + j;
        stf(k_pool, at, v);
        if (off_v < 0) stf(v_pool, at, raw);
      }
    }
  }
  if (off_v >= 0) {
    const float* v = P + (int64_t)r * ldp + off_v;
    for (int i = threadIdx.x; i < G * vdim; i += blockDim.x) {
      const int head = i / vdim, j = i % vdim;
      stf(v_pool, (((int64_t)page * G + head) * page_size + within) * vdim + j, v[i]);
    }
  }
}

// In-place activation of a column range of the projection buffer: 0 = SiLU, 1 = tanh
__global__ void act_cols_kernel(float* __restrict__ P, int64_t ld, int off, int C, int act) {
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float* p = P + (int64_t)blockIdx.x * ld + off + c;
  *p = act == 1 ? tanhf(*p) : silu_f(*p);
}

// Feed-forward activations of one input: 0 = relu(z)^2
template <typename T>
__global__ void act_store_kernel(const float* __restrict__ P, int64_t ld, int F, int act, T* __restrict__ out) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= F) return;
  const float z = fmaxf(P[r * ld + c], 0.f);
  stf(out, r * F + c, z * z);
}

// ---- matrix-memory LSTM (mLSTM) --------------------------------------------------------------------------------------
// Gates of the stabilised recurrence, per head:  i = cap tanh((zi + bi) / cap),  f = logsigmoid(cap tanh((zf + bf) / cap))
// (cap == 0: i = zi + bi, f = logsigmoid(zf + bf)),
//   m_t = max(f + m_(t-1), i),   keep_t = exp(f + m_(t-1) - m_t),   take_t = exp(i - m_t)
// so that S_t = keep_t S_(t-1) + take_t k v^T is what prl_decay_scan runs.  m is carried per sequence slot (0 at the
// start); the walk over a segment's tokens is sequential, one warp per head: 32 tokens' transcendentals at a time in
// parallel, the max-chain through shuffles.  gates[row][head] = (keep, take); minv[row][head] = exp(-m_t).
__device__ __forceinline__ float logsigmoid_g(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void mlstm_gates_kernel(const float* __restrict__ P, int64_t ldp, int off_i, int off_f,
                                   const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap, int H,
                                   const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_len,
                                   const int32_t* __restrict__ seg_slot, float* __restrict__ m_state,
                                   float* __restrict__ gates, float* __restrict__ minv) {
  pdl_wait();
  const int seg = blockIdx.x;
  const int len = seg_len[seg];
  if (len <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int64_t row0 = seg_start[seg];
  const int slot = seg_slot[seg];
  for (int h = warp; h < H; h += nw) {
    float m = m_state[(int64_t)slot * H + h];
    for (int t0 = 0; t0 < len; t0 += 32) {
      const int t = t0 + lane;
      float gi = 0.f, gf = 0.f;
      if (t < len) {
        const float* pr = P + (row0 + t) * ldp;
        const float zi = pr[off_i + h] + bias_i[h], zf = pr[off_f + h] + bias_f[h];
        gi = cap > 0.f ? cap * tanhf(zi / cap) : zi;              // cap == 0: the gates are not capped
        gf = logsigmoid_g(cap > 0.f ? cap * tanhf(zf / cap) : zf);
      }
      float m_prev = 0.f, m_mine = 0.f;
      const int nt = min(32, len - t0);
      for (int j = 0; j < nt; ++j) {
        const float fj = __shfl_sync(0xffffffffu, gf, j), ij = __shfl_sync(0xffffffffu, gi, j);
        const float m_new = fmaxf(fj + m, ij);
        if (j == lane) { m_prev = m; m_mine = m_new; }
        m = m_new;
      }
      if (t < len) {
        const int64_t o = (row0 + t) * H + h;
        gates[2 * o] = expf(gf + m_prev - m_mine);
        gates[2 * o + 1] = expf(gi - m_mine);
        minv[o] = expf(-m_mine);
      }
    }
    if (lane == 0) m_state[(int64_t)slot * H + h] = m;
  }
}

// Values of the scan with a ONE appended per head: [row][head][dv + 1], so that the recurrence also carries the
// normaliser n_t = keep n + take k as the last value column and returns n_t . q beside S_t^T q.
__global__ void append_one_kernel(const float* __restrict__ P, int64_t ldp, int off_v, int H, int dv, float* __restrict__ out) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  const int C = H * (dv + 1);
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const int h = i / (dv + 1), c = i - h * (dv + 1);
    out[r * C + i] = c < dv ? P[r * ldp + off_v + h * dv + c] : 1.f;
  }
}

// o = (S^T q) / (max(|n . q|, exp(-m)) + den_eps) per head, divided by its root mean square over the head, times a gain
// over all heads' channels, times sigmoid(g); written in the operand type of the output projection.  Block per (row, head).
template <typename T>
__global__ void mlstm_out_kernel(const float* __restrict__ o_aug, int H, int dv, const float* __restrict__ minv,
                                 float den_eps, const float* __restrict__ g, int64_t ldg, const float* __restrict__ gain,
                                 float eps, T* __restrict__ out) {
  pdl_wait();
  __shared__ float red[32];
  const int64_t r = blockIdx.x;
  const int h = blockIdx.y;
  const float* o = o_aug + (r * H + h) * (dv + 1);
  const float den = fmaxf(fabsf(o[dv]), minv[r * H + h]) + den_eps;
  float ss = 0.f;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    const float v = o[c] / den;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)dv + eps);
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    const int ch = h * dv + c;
    stf(out, r * H * dv + ch, o[c] / den * inv * gain[ch] * sigmoid_f(g[r * ldg + ch]));
  }
}

// Norm AFTER the sum ("post-LN" with a weighted skip):  v = alpha * x + s0 * y0 + s1 * y1 + bias;
// x <- v / sqrt(mean(v^2) + eps) * gain;  xa = T(x).  y0 / y1 may be split-K slices of a projection or the choices of a
// routed feed-forward ([slices][n][ld]), summed here in slice order; y1 and bias may be NULL.
template <typename T>
__global__ void postln_close_kernel(const float* __restrict__ y0, int64_t ld0, float s0, int ns0, int64_t stride0,
                                    const float* __restrict__ y1, int64_t ld1, float s1, int ns1, int64_t stride1,
                                    const float* __restrict__ bias, float alpha, const float* __restrict__ gain, float eps,
                                    int W, int keep, float* __restrict__ x, T* __restrict__ xa) {
  pdl_wait();
  extern __shared__ float vbuf[];    // [W] the row's sum between the two passes (empty: recomputed)
  __shared__ float red[32];
  const int r = blockIdx.x;
  auto value = [&](int c) {
    float a = 0.f;
#pragma unroll 4
    for (int k = 0; k < ns0; ++k) a += y0[k * stride0 + (int64_t)r * ld0 + c];
    float y = s0 * a;
    if (y1) {
      float b = 0.f;
#pragma unroll 4
      for (int k = 0; k < ns1; ++k) b += y1[k * stride1 + (int64_t)r * ld1 + c];
      y += s1 * b;
    }
    if (bias) y += bias[c];
    return fmaf(alpha, x[(int64_t)r * W + c], y);
  };
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = value(c);
    if (keep) vbuf[c] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);     // its barriers also order every thread's reads of x before the writes below
  const float inv = 1.f / sqrtf(ss / (float)W + eps);
  // without the kept copy the second pass reads x again: a thread reads a column before it writes it, and owns it
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = (keep ? vbuf[c] : value(c)) * inv * gain[c];
    x[(int64_t)r * W + c] = v;
    stf(xa, (int64_t)r * W + c, v);
  }
}

// Attention front end with biases, per-head norms, "rotate half" rotary and normed, blended values.  Per row:
//   q, k: + bias (NULL: none); each head divided by its root mean square over `dim` and multiplied by a gain indexed
//         (head * dim + channel) % gain_period (gain NULL: none; qk_norm == 0: no norm at all);
//         the first `rot` channels of each head turned: channel i < rot / 2 pairs with channel i + rot / 2, the pair
//         (u, v) becomes mag * (u cos a - v sin a, v cos a + u sin a), a = pos * freq[i] (double);
//   v:    + bias; v_norm: each head divided by its root mean square over `vdim` (no gain); then
//         v_blend == 1: the row's values are also written to v_first [n][G * vdim] (fp32) for later layers,
//         v_blend == 2: v <- (1 - lambda) v + lambda v_first[row], lambda = *v_lambda.
// q goes to the query buffer [n][H][dim], k and v into the paged cache.  One warp per head.
template <typename T>
__global__ void attn_front_kernel(const float* __restrict__ P, int64_t ldp, int off_q, int off_k, int off_v, int H, int G,
                                  int dim, int vdim, const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                  const float* __restrict__ v_bias, int qk_norm, const float* __restrict__ q_gain,
                                  const float* __restrict__ k_gain, int gain_period, float eps, int rot,
                                  const double* __restrict__ freq, float mag, int v_norm, int v_blend,
                                  const float* __restrict__ v_lambda, float* __restrict__ v_first,
                                  const int32_t* __restrict__ row_pos, const int32_t* __restrict__ row_slot,
                                  const int32_t* __restrict__ block_table, int max_blocks, int page_size,
                                  T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool) {
  pdl_wait();
  extern __shared__ float trig[];    // [rot / 2] cos | [rot / 2] sin of the row's angles, times mag
  const int r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const int pos = row_pos[r];
  const int half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, cs;
    sincos((double)pos * freq[i], &sn, &cs);
    trig[i] = (float)cs * mag;
    trig[half + i] = (float)sn * mag;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int page = block_table[(int64_t)slot * max_blocks + pos / page_size], within = pos % page_size;
  for (int hh = warp; hh < H + 2 * G; hh += nw) {
    if (hh < H + G) {
      const bool is_q = hh < H;
      const int head = is_q ? hh : hh - H;
      const float* src = P + (int64_t)r * ldp + (is_q ? off_q : off_k) + head * dim;
      const float* bias = is_q ? q_bias : k_bias;
      const float* gain = is_q ? q_gain : k_gain;
      float inv = 1.f;
      if (qk_norm) {
        float ss = 0.f;
        for (int j = lane; j < dim; j += 32) {
          const float v = src[j] + (bias ? bias[head * dim + j] : 0.f);
          ss += v * v;
        }
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / (float)dim + eps);
      }
      auto val = [&](int j) {
        const float raw = src[j] + (bias ? bias[head * dim + j] : 0.f);
        return raw * inv * (gain ? gain[(head * dim + j) % gain_period] : 1.f);
      };
      T* dst = is_q ? q_out + ((int64_t)r * H + head) * dim
                    : k_pool + (((int64_t)page * G + head) * page_size + within) * dim;
      for (int i = lane; i < half; i += 32) {
        const float u = val(i), v = val(i + half), cs = trig[i], sn = trig[half + i];
        stf(dst, i, u * cs - v * sn);
        stf(dst, i + half, v * cs + u * sn);
      }
      for (int j = 2 * half + lane; j < dim; j += 32) stf(dst, j, val(j));
    } else {
      const int head = hh - H - G;
      const float* src = P + (int64_t)r * ldp + off_v + head * vdim;
      float inv = 1.f;
      if (v_norm) {
        float ss = 0.f;
        for (int j = lane; j < vdim; j += 32) {
          const float v = src[j] + (v_bias ? v_bias[head * vdim + j] : 0.f);
          ss += v * v;
        }
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / (float)vdim + eps);
      }
      const float lam = v_blend == 2 ? *v_lambda : 0.f;
      float* vf = v_first ? v_first + ((int64_t)r * G + head) * vdim : nullptr;
      T* dst = v_pool + (((int64_t)page * G + head) * page_size + within) * vdim;
      for (int j = lane; j < vdim; j += 32) {
        float v = (src[j] + (v_bias ? v_bias[head * vdim + j] : 0.f)) * inv;
        if (v_blend == 1) vf[j] = v;
        else if (v_blend == 2) v = (1.f - lam) * v + lam * vf[j];
        stf(dst, j, v);
      }
    }
  }
}

// out[r][h * dv + j] = T(o[r][h * dv + j] * sigmoid(g[r][h])): one gate per head on an attention output
template <typename T, typename TO>
__global__ void gate_heads_kernel(const TO* __restrict__ o, int64_t ldo, const float* __restrict__ g, int64_t ldg, int H,
                                  int dv, T* __restrict__ out) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < H * dv; e += gridDim.y * blockDim.x)
    stf(out, r * H * dv + e, ldf(o, r * ldo + e) * sigmoid_f(g[r * ldg + e / dv]));
}

inline int row_threads(int width) {
  int t = ((width + 31) / 32) * 32;
  return t < 32 ? 32 : (t > 256 ? 256 : t);
}

}  // namespace
}  // namespace prl

using namespace prl;
typedef __nv_bfloat16 bf16;

extern "C" int prl_embed_scale(const int32_t* tokens, const void* embed, int32_t f32, float scale, int32_t n, int32_t W,
                               int32_t vocab, float* x, void* xa, prl_stream_t st) {
  PRL_CHECK_ARG(tokens && embed && x && xa && n >= 1 && W >= 1 && vocab >= 1, "prl_embed_scale: bad argument");
  if (f32) PRL_CUDA(launch_pdl(embed_scale_kernel<float>, dim3(n), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, tokens, (const float*)embed, scale, W, vocab, x, (float*)xa));
  else PRL_CUDA(launch_pdl(embed_scale_kernel<bf16>, dim3(n), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, tokens, (const bf16*)embed, scale, W, vocab, x, (bf16*)xa));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_postnorm_residual(const float* y0, int64_t ld0, float s0, int32_t n_split0, const float* y1, int64_t ld1,
                                     float s1, int32_t n_split1, const float* gain, float eps, int32_t n, int32_t W, float* x,
                                     void* xa, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(y0 && gain && x && xa && n >= 1 && W >= 1 && ld0 >= W && (!y1 || ld1 >= W) && n_split0 >= 1 &&
                (!y1 || n_split1 >= 1), "prl_postnorm_residual: bad argument");
  const int64_t st0 = (int64_t)n * ld0, st1 = (int64_t)n * ld1;
  int th = ((W + 31) / 32) * 32;
  const int cap = n <= 256 ? 1024 : 256;     // few rows: more threads per row; many rows: more rows per SM
  th = th > cap ? cap : th;
  const int keep = (size_t)W * sizeof(float) <= 40 * 1024 ? 1 : 0;
  const size_t smem = keep ? (size_t)W * sizeof(float) : 0;
  if (f32) PRL_CUDA(launch_pdl(postnorm_residual_kernel<float>, dim3(n), dim3(th), smem, (cudaStream_t)st, y0, ld0, s0, n_split0, st0, y1, ld1, s1, n_split1, st1, gain, eps, W, keep, x, (float*)xa));
  else PRL_CUDA(launch_pdl(postnorm_residual_kernel<bf16>, dim3(n), dim3(th), smem, (cudaStream_t)st, y0, ld0, s0, n_split0, st0, y1, ld1, s1, n_split1, st1, gain, eps, W, keep, x, (bf16*)xa));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_rmsnorm_rows(const float* x, const int32_t* rows, const float* gain, float eps, int32_t n_out, int32_t W,
                                void* out, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(x && gain && out && n_out >= 1 && W >= 1, "prl_rmsnorm_rows: bad argument");
  if (f32) PRL_CUDA(launch_pdl(rmsnorm_rows_kernel<float>, dim3(n_out), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, x, rows, gain, eps, W, (float*)out));
  else PRL_CUDA(launch_pdl(rmsnorm_rows_kernel<bf16>, dim3(n_out), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, x, rows, gain, eps, W, (bf16*)out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_gate_norm(const void* o, int32_t o_f32, int64_t ldo, const float* g, int64_t ldg, const float* gain,
                             int32_t gain_period, int32_t group_size, int32_t n, int32_t C, int32_t act_sigmoid,
                             int32_t gate_first, int32_t norm, float eps, void* out, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(o && g && out && n >= 1 && C >= 1 && group_size >= 1 && C % group_size == 0 && ldo >= C && ldg >= C,
                "prl_gate_norm: bad argument (C=%d group=%d)", C, group_size);
  PRL_CHECK_ARG(!norm || (gain && gain_period >= 1), "prl_gate_norm: a norm needs its gain");
  dim3 grid(n, C / group_size);
  int th = ((group_size + 31) / 32) * 32;
  const int cap = (int64_t)n * (C / group_size) <= 512 ? 1024 : 256;   // few blocks: more threads per group; many: more groups per SM
  th = th > cap ? cap : th;
  const int keep = norm && 2 * (size_t)group_size * sizeof(float) <= 40 * 1024 ? 1 : 0;
  const size_t smem = keep ? 2 * (size_t)group_size * sizeof(float) : 0;
  cudaStream_t s = (cudaStream_t)st;
#define PRL_GN(T, TO) PRL_CUDA(launch_pdl((gate_norm_kernel<T, TO>), dim3(grid), dim3(th), smem, s, (const TO*)o, ldo, g, ldg, gain, gain_period, group_size, C, \
                                                                   act_sigmoid, gate_first, norm, eps, keep, (T*)out))
  if (f32) { if (o_f32) PRL_GN(float, float); else PRL_GN(float, bf16); }
  else { if (o_f32) PRL_GN(bf16, float); else PRL_GN(bf16, bf16); }
#undef PRL_GN
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_glu_clamped(const float* gate_up, int64_t ld, int32_t n, int32_t F, float limit, float beta, void* out,
                               int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(gate_up && out && n >= 1 && F >= 1 && ld >= 2 * (int64_t)F, "prl_glu_clamped: bad argument");
  dim3 grid(n, (F + 255) / 256);
  if (f32) PRL_CUDA(launch_pdl(glu_clamped_kernel<float>, grid, dim3(256), (size_t)(0), (cudaStream_t)st, gate_up, ld, F, limit, beta, (float*)out));
  else PRL_CUDA(launch_pdl(glu_clamped_kernel<bf16>, grid, dim3(256), (size_t)(0), (cudaStream_t)st, gate_up, ld, F, limit, beta, (bf16*)out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_qk_norm_rope_cache(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, int32_t off_v, int32_t n,
                                      int32_t H, int32_t G, int32_t dim, int32_t vdim, int32_t rot, const double* freq,
                                      const float* q_gain, const float* k_gain, float eps, const int32_t* row_pos,
                                      const int32_t* row_slot, const int32_t* block_table, int32_t max_blocks,
                                      int32_t page_size, void* q_out, void* k_pool, void* v_pool, int32_t f32,
                                      prl_stream_t st) {
  PRL_CHECK_ARG(P && q_gain && k_gain && row_pos && row_slot && block_table && q_out && k_pool && v_pool,
                "prl_qk_norm_rope_cache: NULL argument");
  PRL_CHECK_ARG(n >= 1 && H >= 1 && G >= 1 && dim >= 1 && vdim >= 1 && rot >= 0 && rot <= dim && rot % 2 == 0 &&
                (rot == 0 || freq) && page_size >= 1 && max_blocks >= 1,
                "prl_qk_norm_rope_cache: bad shape (H=%d G=%d dim=%d vdim=%d rot=%d)", H, G, dim, vdim, rot);
  const size_t smem = (size_t)rot * sizeof(float);
  cudaStream_t s = (cudaStream_t)st;
  if (f32) PRL_CUDA(launch_pdl(qk_norm_rope_cache_kernel<float>, dim3(n), dim3(256), (size_t)(smem), s, P, ldp, off_q, off_k, off_v, H, G, dim, vdim, rot, freq, q_gain, k_gain, eps,
        row_pos, row_slot, block_table, max_blocks, page_size, (float*)q_out, (float*)k_pool, (float*)v_pool));
  else PRL_CUDA(launch_pdl(qk_norm_rope_cache_kernel<bf16>, dim3(n), dim3(256), (size_t)(smem), s, P, ldp, off_q, off_k, off_v, H, G, dim, vdim, rot, freq, q_gain, k_gain, eps,
        row_pos, row_slot, block_table, max_blocks, page_size, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_conv_silu(const float* P, int64_t ldp, int32_t off, int32_t n, int32_t ch, int32_t taps, const float* w,
                             const float* b, const int32_t* row_slot, const int32_t* row_back, const float* state,
                             float* out, prl_stream_t st) {
  PRL_CHECK_ARG(P && w && b && row_slot && row_back && state && out && n >= 1 && ch >= 1 && taps >= 1 && taps <= 16,
                "prl_conv_silu: bad argument (taps=%d, at most 16)", taps);
  PRL_CUDA(launch_pdl(conv_silu_kernel, dim3(n, (ch + 255) / 256), dim3(row_threads(ch)), (size_t)(0), (cudaStream_t)st, P, ldp, off, ch, taps, w, b, row_slot, row_back, state, out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_conv_state_update(const float* P, int64_t ldp, int32_t off, int32_t ch, int32_t taps,
                                     const int32_t* seg_start, const int32_t* seg_len, const int32_t* seg_slot,
                                     int32_t n_seg, float* state, prl_stream_t st) {
  PRL_CHECK_ARG(P && seg_start && seg_len && seg_slot && state && ch >= 1 && taps >= 1 && taps <= 16 && n_seg >= 1,
                "prl_conv_state_update: bad argument");
  if (taps == 1) return PRL_OK;
  dim3 grid((ch + 127) / 128, n_seg);
  PRL_CUDA(launch_pdl(conv_state_kernel, dim3(grid), dim3(128), (size_t)(0), (cudaStream_t)st, P, ldp, off, ch, taps, seg_start, seg_len, seg_slot, state));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_decode_rows(const uint8_t* active, int32_t B, int32_t* seg_len, int32_t* row_slot, prl_stream_t st) {
  PRL_CHECK_ARG(active && seg_len && row_slot && B >= 1, "prl_decode_rows: bad argument");
  PRL_CUDA(launch_pdl(decode_rows_kernel, dim3((B + 127) / 128), dim3(128), (size_t)(0), (cudaStream_t)st, active, B, seg_len, row_slot));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_embed_sinusoid(const int32_t* tokens, const void* embed, int32_t f32, float scale, const double* freq,
                                  const int32_t* row_pos, int32_t n, int32_t W, int32_t vocab, float* x, void* xa, void* x0a,
                                  prl_stream_t st) {
  PRL_CHECK_ARG(tokens && embed && freq && row_pos && x && xa && n >= 1 && W >= 1 && vocab >= 1, "prl_embed_sinusoid: bad argument");
  if (f32) PRL_CUDA(launch_pdl(embed_sinusoid_kernel<float>, dim3(n), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, tokens, (const float*)embed, scale, freq, row_pos, W, vocab, x, (float*)xa, (float*)x0a));
  else PRL_CUDA(launch_pdl(embed_sinusoid_kernel<bf16>, dim3(n), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, tokens, (const bf16*)embed, scale, freq, row_pos, W, vocab, x, (bf16*)xa, (bf16*)x0a));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_concat_rows(const void* a, const void* b, int32_t n, int32_t W, void* out, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(a && b && out && n >= 1 && W >= 1, "prl_concat_rows: bad argument");
  if (f32) PRL_CUDA(launch_pdl(concat_rows_kernel<float>, dim3(n), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, (const float*)a, (const float*)b, W, (float*)out));
  else PRL_CUDA(launch_pdl(concat_rows_kernel<bf16>, dim3(n), dim3(row_threads(W)), (size_t)(0), (cudaStream_t)st, (const bf16*)a, (const bf16*)b, W, (bf16*)out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_sublayer_close(const float* y0, int64_t ld0, int32_t n_split0, const float* gain0, float s0,
                                  const float* y1, int64_t ld1, int32_t n_split1, const float* gain1, float s1,
                                  const float* post_gain, const float* bias, int32_t add, const float* next_gain, float eps,
                                  int32_t n, int32_t W, float* x, void* xa, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(y0 && x && xa && n >= 1 && W >= 1 && ld0 >= W && (!y1 || ld1 >= W) && n_split0 >= 1 && (!y1 || n_split1 >= 1),
                "prl_sublayer_close: bad argument");
  const size_t smem = 2 * (size_t)W * sizeof(float);
  PRL_CHECK_ARG(smem <= 200 * 1024, "prl_sublayer_close: a row of %d channels does not fit in shared memory", W);
  const int64_t st0 = (int64_t)n * ld0, st1 = (int64_t)n * ld1;
  int th = ((W + 31) / 32) * 32;
  const int cap = n <= 256 ? 1024 : 256;     // few rows: more threads per row; many rows: more rows per SM
  th = th > cap ? cap : th;
  static SmemAttr attr_f = {}, attr_b = {};
  if (f32) {
    if (smem > 48 * 1024) PRL_CUDA(ensure_smem(sublayer_close_kernel<float>, (int)smem, attr_f));
    PRL_CUDA(launch_pdl(sublayer_close_kernel<float>, dim3(n), dim3(th), smem, (cudaStream_t)st, y0, ld0, n_split0, st0, gain0, s0, y1, ld1, n_split1, st1, gain1, s1, post_gain, bias, add, next_gain, eps, W, x, (float*)xa));
  } else {
    if (smem > 48 * 1024) PRL_CUDA(ensure_smem(sublayer_close_kernel<bf16>, (int)smem, attr_b));
    PRL_CUDA(launch_pdl(sublayer_close_kernel<bf16>, dim3(n), dim3(th), smem, (cudaStream_t)st, y0, ld0, n_split0, st0, gain0, s0, y1, ld1, n_split1, st1, gain1, s1, post_gain, bias, add, next_gain, eps, W, x, (bf16*)xa));
  }
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_qk_headnorm_cache(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, int32_t off_v, int32_t n,
                                     int32_t H, int32_t G, int32_t dim, int32_t vdim, const float* q_bias,
                                     const float* k_bias, const float* q_gain, const float* k_gain, float eps,
                                     const int32_t* row_pos, const int32_t* row_slot, const int32_t* block_table,
                                     int32_t max_blocks, int32_t page_size, void* q_out, void* k_pool, void* v_pool,
                                     int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(P && row_pos && row_slot && block_table && q_out && k_pool && v_pool, "prl_qk_headnorm_cache: NULL argument");
  PRL_CHECK_ARG(n >= 1 && H >= 1 && G >= 1 && dim >= 1 && vdim >= 1 && (off_v >= 0 || vdim == dim) && page_size >= 1 &&
                max_blocks >= 1, "prl_qk_headnorm_cache: bad shape (H=%d G=%d dim=%d vdim=%d)", H, G, dim, vdim);
  int th = 32 * (H + G);
  th = th > 256 ? 256 : th;
  cudaStream_t s = (cudaStream_t)st;
  if (f32) PRL_CUDA(launch_pdl(qk_headnorm_cache_kernel<float>, dim3(n), dim3(th), (size_t)0, s, P, ldp, off_q, off_k, off_v, H, G, dim, vdim, q_bias, k_bias, q_gain, k_gain, eps,
        row_pos, row_slot, block_table, max_blocks, page_size, (float*)q_out, (float*)k_pool, (float*)v_pool));
  else PRL_CUDA(launch_pdl(qk_headnorm_cache_kernel<bf16>, dim3(n), dim3(th), (size_t)0, s, P, ldp, off_q, off_k, off_v, H, G, dim, vdim, q_bias, k_bias, q_gain, k_gain, eps,
        row_pos, row_slot, block_table, max_blocks, page_size, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_act_cols(float* P, int64_t ld, int32_t off, int32_t n, int32_t C, int32_t act, prl_stream_t st) {
  PRL_CHECK_ARG(P && n >= 1 && C >= 1 && off >= 0 && ld >= off + C && (act == 0 || act == 1), "prl_act_cols: bad argument");
  PRL_CUDA(launch_pdl(act_cols_kernel, dim3(n, (C + 255) / 256), dim3(256), (size_t)0, (cudaStream_t)st, P, ld, off, C, act));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_act_store(const float* P, int64_t ld, int32_t n, int32_t F, int32_t act, void* out, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(P && out && n >= 1 && F >= 1 && ld >= F && act == 0, "prl_act_store: bad argument");
  dim3 grid(n, (F + 255) / 256);
  if (f32) PRL_CUDA(launch_pdl(act_store_kernel<float>, grid, dim3(256), (size_t)0, (cudaStream_t)st, P, ld, F, act, (float*)out));
  else PRL_CUDA(launch_pdl(act_store_kernel<bf16>, grid, dim3(256), (size_t)0, (cudaStream_t)st, P, ld, F, act, (bf16*)out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_mlstm_gates(const float* P, int64_t ldp, int32_t off_i, int32_t off_f, const float* bias_i,
                               const float* bias_f, float cap, int32_t H, const int32_t* seg_start, const int32_t* seg_len,
                               const int32_t* seg_slot, int32_t n_seg, float* m_state, float* gates, float* minv,
                               prl_stream_t st) {
  PRL_CHECK_ARG(P && bias_i && bias_f && seg_start && seg_len && seg_slot && m_state && gates && minv && H >= 1 && n_seg >= 1 &&
                cap >= 0.f, "prl_mlstm_gates: bad argument");
  int th = 32 * H;
  th = th > 256 ? 256 : th;
  PRL_CUDA(launch_pdl(mlstm_gates_kernel, dim3(n_seg), dim3(th), (size_t)0, (cudaStream_t)st, P, ldp, off_i, off_f, bias_i, bias_f, cap, H, seg_start, seg_len, seg_slot, m_state, gates, minv));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_append_one(const float* P, int64_t ldp, int32_t off_v, int32_t n, int32_t H, int32_t dv, float* out,
                              prl_stream_t st) {
  PRL_CHECK_ARG(P && out && n >= 1 && H >= 1 && dv >= 1, "prl_append_one: bad argument");
  PRL_CUDA(launch_pdl(append_one_kernel, dim3(n), dim3(row_threads(H * (dv + 1))), (size_t)0, (cudaStream_t)st, P, ldp, off_v, H, dv, out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_mlstm_out(const float* o_aug, int32_t n, int32_t H, int32_t dv, const float* minv, float den_eps,
                             const float* g, int64_t ldg, const float* gain, float eps, void* out, int32_t f32,
                             prl_stream_t st) {
  PRL_CHECK_ARG(o_aug && minv && g && gain && out && n >= 1 && H >= 1 && H <= 65535 && dv >= 1, "prl_mlstm_out: bad argument");
  dim3 grid(n, H);
  const int th = row_threads(dv);
  if (f32) PRL_CUDA(launch_pdl(mlstm_out_kernel<float>, grid, dim3(th), (size_t)0, (cudaStream_t)st, o_aug, H, dv, minv, den_eps, g, ldg, gain, eps, (float*)out));
  else PRL_CUDA(launch_pdl(mlstm_out_kernel<bf16>, grid, dim3(th), (size_t)0, (cudaStream_t)st, o_aug, H, dv, minv, den_eps, g, ldg, gain, eps, (bf16*)out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_postln_close(const float* y0, int64_t ld0, float s0, int32_t n_split0, const float* y1, int64_t ld1,
                                float s1, int32_t n_split1, const float* bias, float alpha, const float* gain, float eps,
                                int32_t n, int32_t W, float* x, void* xa, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(y0 && gain && x && xa && n >= 1 && W >= 1 && ld0 >= W && (!y1 || ld1 >= W) && n_split0 >= 1 &&
                (!y1 || n_split1 >= 1), "prl_postln_close: bad argument");
  const int64_t st0 = (int64_t)n * ld0, st1 = (int64_t)n * ld1;
  int th = ((W + 31) / 32) * 32;
  const int cap = n <= 256 ? 1024 : 256;     // few rows: more threads per row; many rows: more rows per SM
  th = th > cap ? cap : th;
  const int keep = (size_t)W * sizeof(float) <= 40 * 1024 ? 1 : 0;
  const size_t smem = keep ? (size_t)W * sizeof(float) : 0;
  if (f32) PRL_CUDA(launch_pdl(postln_close_kernel<float>, dim3(n), dim3(th), smem, (cudaStream_t)st, y0, ld0, s0, n_split0, st0, y1, ld1, s1, n_split1, st1, bias, alpha, gain, eps, W, keep, x, (float*)xa));
  else PRL_CUDA(launch_pdl(postln_close_kernel<bf16>, dim3(n), dim3(th), smem, (cudaStream_t)st, y0, ld0, s0, n_split0, st0, y1, ld1, s1, n_split1, st1, bias, alpha, gain, eps, W, keep, x, (bf16*)xa));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_attn_front(const float* P, int64_t ldp, int32_t off_q, int32_t off_k, int32_t off_v, int32_t n, int32_t H,
                              int32_t G, int32_t dim, int32_t vdim, const float* q_bias, const float* k_bias,
                              const float* v_bias, int32_t qk_norm, const float* q_gain, const float* k_gain,
                              int32_t gain_period, float eps, int32_t rot, const double* freq, float mag, int32_t v_norm,
                              int32_t v_blend, const float* v_lambda, float* v_first, const int32_t* row_pos,
                              const int32_t* row_slot, const int32_t* block_table, int32_t max_blocks, int32_t page_size,
                              void* q_out, void* k_pool, void* v_pool, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(P && row_pos && row_slot && block_table && q_out && k_pool && v_pool, "prl_attn_front: NULL argument");
  PRL_CHECK_ARG(n >= 1 && H >= 1 && G >= 1 && dim >= 1 && vdim >= 1 && page_size >= 1 && max_blocks >= 1 && rot >= 0 &&
                rot <= dim && rot % 2 == 0 && (rot == 0 || freq) && gain_period >= 1,
                "prl_attn_front: bad shape (H=%d G=%d dim=%d vdim=%d rot=%d)", H, G, dim, vdim, rot);
  PRL_CHECK_ARG(v_blend >= 0 && v_blend <= 2 && (v_blend == 0 || v_first) && (v_blend != 2 || v_lambda),
                "prl_attn_front: blending the values needs the first layer's values and the weight");
  int warps = H + 2 * G;
  warps = warps > 16 ? 16 : warps;
  const size_t smem = (size_t)(rot > 0 ? rot : 1) * sizeof(float);
  if (f32) PRL_CUDA(launch_pdl(attn_front_kernel<float>, dim3(n), dim3(32 * warps), smem, (cudaStream_t)st, P, ldp, off_q, off_k, off_v, H, G, dim, vdim, q_bias, k_bias, v_bias, qk_norm, q_gain, k_gain, gain_period, eps, rot, freq, mag, v_norm, v_blend, v_lambda, v_first, row_pos, row_slot, block_table, max_blocks, page_size, (float*)q_out, (float*)k_pool, (float*)v_pool));
  else PRL_CUDA(launch_pdl(attn_front_kernel<bf16>, dim3(n), dim3(32 * warps), smem, (cudaStream_t)st, P, ldp, off_q, off_k, off_v, H, G, dim, vdim, q_bias, k_bias, v_bias, qk_norm, q_gain, k_gain, gain_period, eps, rot, freq, mag, v_norm, v_blend, v_lambda, v_first, row_pos, row_slot, block_table, max_blocks, page_size, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_gate_heads(const void* o, int32_t o_f32, int64_t ldo, const float* g, int64_t ldg, int32_t n, int32_t H,
                              int32_t dv, void* out, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(o && g && out && n >= 1 && H >= 1 && dv >= 1 && ldo >= (int64_t)H * dv && ldg >= H, "prl_gate_heads: bad argument");
  dim3 grid(n, (H * dv + 1023) / 1024);
  cudaStream_t s = (cudaStream_t)st;
#define PRL_GH(T, TO) PRL_CUDA(launch_pdl((gate_heads_kernel<T, TO>), grid, dim3(256), (size_t)0, s, (const TO*)o, ldo, g, ldg, H, dv, (T*)out))
  if (f32) { if (o_f32) PRL_GH(float, float); else PRL_GH(float, bf16); }
  else { if (o_f32) PRL_GH(bf16, float); else PRL_GH(bf16, bf16); }
#undef PRL_GH
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}
