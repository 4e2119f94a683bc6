// Row kernels of latent attention: keys and values of all heads are expanded from ONE normed low-rank latent per token,
// and only that latent (plus one rotated key part shared by the heads) is cached:
//
//     cache row of a token = [ c = rmsnorm(W_dkv h)[:rank] * gain  |  rotate(W_dkv h [rank:], pos) ]      (rank + rot)
//
// The per-head key expansion is absorbed into the query (q_lat = W_uk,h^T q_h, a per-head GEMM done by the caller), so
// attention runs as one shared "key head" of size rank + rot whose value is the first `rank` channels of the same cache
// row; the per-head value expansion W_uv,h follows on the attention output.
//
// Rotation: channel i of the rotated part pairs with channel i + rot/2 ("rotate half"), or channel 2i with channel 2i + 1
// (`interleaved`); the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * freq[i], freq
// given in double (base^(-2i/rot)); the angle is formed and its sine and cosine taken in double.  A model without a
// query latent passes q_rank = 0 and its full-size query projection to prl_latent_query directly.
#include "prl_common.cuh"
#include <math.h>

namespace prl {
namespace {

template <typename T> __device__ __forceinline__ void stf(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// fixed-order block sum (see hybrid_ops.cu)
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += red[w];
  return t;
}

// One block per row: the query latent (normed, operand type) and the row of the latent cache.
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ P, int64_t ldp, int off_q, int q_rank, int off_kv, int rank,
                                   int rot, const double* __restrict__ freq, const float* __restrict__ q_gain,
                                   const float* __restrict__ kv_gain, float eps, const int32_t* __restrict__ row_pos,
                                   const int32_t* __restrict__ row_slot, const int32_t* __restrict__ block_table,
                                   int max_blocks, int page_size, int interleaved, T* __restrict__ cq_out,
                                   T* __restrict__ pool) {
  pdl_wait();
  __shared__ float red[32];
  const int64_t r = blockIdx.x;
  const int slot = row_slot[r];
  if (slot < 0) return;
  const float* p = P + r * ldp;
  float ss = 0.f;
  if (q_rank > 0) {
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) { const float v = p[off_q + c]; ss = fmaf(v, v, ss); }
    const float inv_q = 1.f / sqrtf(block_sum(ss, red) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) stf(cq_out, r * q_rank + c, p[off_q + c] * inv_q * q_gain[c]);
  }
  ss = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) { const float v = p[off_kv + c]; ss = fmaf(v, v, ss); }
  const float inv_c = 1.f / sqrtf(block_sum(ss, red) / (float)rank + eps);
  const int pos = row_pos[r];
  const int page = block_table[(int64_t)slot * max_blocks + pos / page_size];
  T* dst = pool + ((int64_t)page * page_size + pos % page_size) * (rank + rot);
  for (int c = threadIdx.x; c < rank; c += blockDim.x) stf(dst, c, p[off_kv + c] * inv_c * kv_gain[c]);
  const int half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double sn, cs;
    sincos((double)pos * freq[i], &sn, &cs);
    const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
    const float u = p[off_kv + rank + iu], v = p[off_kv + rank + iv];
    stf(dst, rank + iu, u * (float)cs - v * (float)sn);
    stf(dst, rank + iv, v * (float)cs + u * (float)sn);
  }
  for (int i = 2 * half + threadIdx.x; i < rot; i += blockDim.x) stf(dst, rank + i, p[off_kv + rank + i]);   // odd size: last channel as is
}

// One block per row: a head's query [dim unrotated | rot rotated] -> the unrotated parts packed [n][H*dim] in the
// operand type (the A operand of the per-head absorbing product), the rotated part turned and stored behind the
// `rank` absorbed channels of the attention query [n][H][rank + rot].
template <typename T>
__global__ void latent_query_kernel(const float* __restrict__ Q, int64_t ldq, int H, int dim, int rot, int rank,
                                    const double* __restrict__ freq, const int32_t* __restrict__ row_pos, int interleaved,
                                    T* __restrict__ q_plain, T* __restrict__ q_att) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  const float* q = Q + r * ldq;
  const int pos = row_pos[r];
  const int hd = dim + rot, half = rot / 2;
  for (int e = threadIdx.x; e < H * dim; e += blockDim.x) {
    const int h = e / dim, d = e - h * dim;
    stf(q_plain, r * H * dim + e, q[h * hd + d]);
  }
  for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
    const int h = e / half, i = e - h * half;
    double sn, cs;
    sincos((double)pos * freq[i], &sn, &cs);
    const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
    const float u = q[h * hd + dim + iu], v = q[h * hd + dim + iv];
    T* dst = q_att + (r * H + h) * (rank + rot) + rank;
    stf(dst, iu, u * (float)cs - v * (float)sn);
    stf(dst, iv, v * (float)cs + u * (float)sn);
  }
  if (rot & 1)
    for (int h = threadIdx.x; h < H; h += blockDim.x)
      stf(q_att, (r * H + h) * (rank + rot) + rank + rot - 1, q[h * hd + dim + rot - 1]);
}

// out[r][g][off + c] = T(src[r][g * C + c]) for g < G, c < C: the absorbed query channels into the attention query
// (ld_out = rank + rot, off = 0), or a plain cast of fp32 rows to the operand type (G = 1).
template <typename T>
__global__ void store_groups_kernel(const float* __restrict__ src, int64_t lds, int G, int C, T* __restrict__ out,
                                    int64_t ld_out) {
  pdl_wait();
  const int64_t r = blockIdx.x;
  const int e = blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= G * C) return;
  const int g = e / C, c = e - g * C;
  stf(out, (r * G + g) * ld_out + c, src[r * lds + e]);
}

inline int row_threads(int W) { return W >= 1024 ? 256 : (W >= 256 ? 128 : 64); }

}  // namespace
}  // namespace prl

using namespace prl;
typedef __nv_bfloat16 bf16;

extern "C" int prl_latent_prep(const float* P, int64_t ldp, int32_t off_q, int32_t q_rank, int32_t off_kv, int32_t rank,
                               int32_t rot, const double* freq, const float* q_gain, const float* kv_gain, float eps,
                               const int32_t* row_pos, const int32_t* row_slot, const int32_t* block_table,
                               int32_t max_blocks, int32_t page_size, int32_t n, int32_t interleaved, void* cq_out, void* pool,
                               int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(P && freq && kv_gain && row_pos && row_slot && block_table && pool && (q_rank == 0 || (q_gain && cq_out)),
                "prl_latent_prep: NULL argument");
  PRL_CHECK_ARG(n >= 1 && q_rank >= 0 && rank >= 1 && rot >= 0 && page_size >= 1 && max_blocks >= 1,
                "prl_latent_prep: bad shape");
  const int th = row_threads(q_rank > rank ? q_rank : rank);
  if (f32) PRL_CUDA(launch_pdl(latent_prep_kernel<float>, dim3(n), dim3(th), (size_t)0, (cudaStream_t)st, P, ldp, off_q, q_rank, off_kv, rank, rot, freq, q_gain, kv_gain, eps, row_pos, row_slot, block_table, max_blocks, page_size, interleaved, (float*)cq_out, (float*)pool));
  else PRL_CUDA(launch_pdl(latent_prep_kernel<bf16>, dim3(n), dim3(th), (size_t)0, (cudaStream_t)st, P, ldp, off_q, q_rank, off_kv, rank, rot, freq, q_gain, kv_gain, eps, row_pos, row_slot, block_table, max_blocks, page_size, interleaved, (bf16*)cq_out, (bf16*)pool));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_latent_query(const float* Q, int64_t ldq, int32_t n, int32_t H, int32_t dim, int32_t rot, int32_t rank,
                                const double* freq, const int32_t* row_pos, int32_t interleaved, void* q_plain, void* q_att,
                                int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(Q && freq && row_pos && q_plain && q_att && n >= 1 && H >= 1 && dim >= 1 && rot >= 0 && rank >= 1 &&
                ldq >= (int64_t)H * (dim + rot), "prl_latent_query: bad argument");
  const int th = row_threads(H * dim);
  if (f32) PRL_CUDA(launch_pdl(latent_query_kernel<float>, dim3(n), dim3(th), (size_t)0, (cudaStream_t)st, Q, ldq, H, dim, rot, rank, freq, row_pos, interleaved, (float*)q_plain, (float*)q_att));
  else PRL_CUDA(launch_pdl(latent_query_kernel<bf16>, dim3(n), dim3(th), (size_t)0, (cudaStream_t)st, Q, ldq, H, dim, rot, rank, freq, row_pos, interleaved, (bf16*)q_plain, (bf16*)q_att));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_store_groups(const float* src, int64_t lds, int32_t n, int32_t G, int32_t C, void* out, int64_t ld_out,
                                int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(src && out && n >= 1 && G >= 1 && C >= 1 && lds >= (int64_t)G * C && ld_out >= C, "prl_store_groups: bad argument");
  dim3 grid(n, (G * C + 255) / 256);
  if (f32) PRL_CUDA(launch_pdl(store_groups_kernel<float>, grid, dim3(256), (size_t)0, (cudaStream_t)st, src, lds, G, C, (float*)out, ld_out));
  else PRL_CUDA(launch_pdl(store_groups_kernel<bf16>, grid, dim3(256), (size_t)0, (cudaStream_t)st, src, lds, G, C, (bf16*)out, ld_out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}
