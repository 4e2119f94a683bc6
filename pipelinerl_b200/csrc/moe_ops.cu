// Routed feed-forward (mixture of experts) over a packed batch of n token rows, without a host round trip: the number
// of rows each expert gets stays on the device, so the whole layer can sit in a CUDA graph.
//
//   1. route:  per row, the `top` experts with the largest router logits (ties: the lower index), each with the weight
//              sigmoid(logit) or softmax over the chosen; an optional bias per expert joins the logits first; choice c
//              of row t is the PAIR c * n + t.
//   2. group:  a stable counting sort of the pairs by expert (one CTA): perm[s] = pair at sorted place s, and a table
//              of row tiles (expert, first sorted place, rows <= 64) that the GEMMs walk; its length stays on the device.
//   3. grouped GEMM (twice):  C[row] = A[row'] * W_e^T for every tile, W_e = W + e * expert_stride.  The first product
//              reads the token's row (perm[s] % n) and writes sorted rows; the second reads sorted rows and writes
//              pair rows, i.e. `top` slices [top][n][width] that the sublayer's closing kernel adds up.
//   4. gated activation of an expert with the pair's weight folded in: the weight multiplies the expert's INPUT, and
//              the two first projections are linear, so gate and up are scaled after the product (in fp32).
//
// Two GEMM kernels walk the same tile table.  fp32 operands (and sizes a 16-byte copy cannot express) take the
// CUDA-core kernel of gemm_any.cu with a row indirection: every output element is summed by one thread in ascending k.
// bf16 operands take a tensor-core kernel (mma.sync m16n8k16, fp32 accumulators): 64 x 128 output tile per CTA of eight
// warps, operands staged by cp.async (zero-filled past the edges) into a double buffer and read with ldmatrix.  A
// row's result depends only on the row and the expert's weights, never on which rows share its tile.
#include "prl_common.cuh"

namespace prl {
namespace {

constexpr int kTile = 64;
constexpr int kStepK = 16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// one warp per row; E up to 32 * kMaxPerLane
constexpr int kMaxPerLane = 32;
__global__ void moe_route_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ bias, int n, int E,
                                 int top, int softmax_weights, int32_t* __restrict__ sel, float* __restrict__ wsel) {
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n) return;
  const float* z = logits + (int64_t)t * ld;
  uint32_t taken = 0;            // bit j: expert lane + 32 j already chosen
  float zsel_max = 0.f, denom = 0.f;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e >= E) break;
      if (taken >> j & 1u) continue;
      const float v = z[e] + (bias ? bias[e] : 0.f);
      if (v > best) { best = v; arg = e; }        // ascending e: the lower index wins a tie inside a lane
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if ((arg & 31) == lane) taken |= 1u << (arg >> 5);
    if (c == 0) zsel_max = best;
    denom += expf(best - zsel_max);
    if (lane == 0) {
      sel[(int64_t)c * n + t] = arg;
      wsel[(int64_t)c * n + t] = softmax_weights ? expf(best - zsel_max) : sigmoid_f(best);
    }
  }
  if (softmax_weights == 2) {                    // softmax over ALL experts: the denominator sums every logit
    float all = 0.f;
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e >= E) break;
      all += expf(z[e] + (bias ? bias[e] : 0.f) - zsel_max);
    }
    denom = warp_sum(all);
  }
  if (softmax_weights && lane == 0)
    for (int c = 0; c < top; ++c) wsel[(int64_t)c * n + t] /= denom;
}

// Router and choice in one kernel: logits[e] = x . Wr[e] in fp32 (block per row, the row staged in shared memory, warps
// take experts in turn, a lane sums every 32nd channel, then the warp's shuffle tree: a fixed order), then the top-k
// pass of moe_route_kernel over the logits in shared memory.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) moe_router_kernel(const TX* __restrict__ x, const TW* __restrict__ Wr,
                                                         const float* __restrict__ bias, int n, int W, int E, int top,
                                                         int softmax_weights, int32_t* __restrict__ sel,
                                                         float* __restrict__ wsel) {
  pdl_wait();
  extern __shared__ float rsm[];       // [W] the row | [E] logits
  float* xs = rsm;
  float* z = rsm + W;
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int c = threadIdx.x; c < W; c += blockDim.x) xs[c] = to_f32(x[(int64_t)t * W + c]);
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    const TW* w = Wr + (int64_t)e * W;
    float a = 0.f;
#pragma unroll 8
    for (int c = lane; c < W; c += 32) a = fmaf(xs[c], to_f32(w[c]), a);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) z[e] = a + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  uint32_t taken = 0;
  float zsel_max = 0.f, denom = 0.f;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e >= E) break;
      if (taken >> j & 1u) continue;
      const float v = z[e];
      if (v > best) { best = v; arg = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if ((arg & 31) == lane) taken |= 1u << (arg >> 5);
    if (c == 0) zsel_max = best;
    denom += expf(best - zsel_max);
    if (lane == 0) {
      sel[(int64_t)c * n + t] = arg;
      wsel[(int64_t)c * n + t] = softmax_weights ? expf(best - zsel_max) : sigmoid_f(best);
    }
  }
  if (softmax_weights == 2) {                    // softmax over ALL experts: the denominator sums every logit
    float all = 0.f;
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e >= E) break;
      all += expf(z[e] - zsel_max);
    }
    denom = warp_sum(all);
  }
  if (softmax_weights && lane == 0)
    for (int c = 0; c < top; ++c) wsel[(int64_t)c * n + t] /= denom;
}

// meta[0] = number of tiles; tiles[3 * i + {0, 1, 2}] = expert, first sorted place, rows
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t* __restrict__ sel, int pairs, int E,
                                                         int32_t* __restrict__ perm, int32_t* __restrict__ meta,
                                                         int32_t* __restrict__ tiles) {
  pdl_wait();
  extern __shared__ int32_t cnt[];      // [E] counts, then [E] offsets
  int32_t* off = cnt + E;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = tid; p < pairs; p += blockDim.x) atomicAdd(&cnt[sel[p]], 1);
  __syncthreads();
  if (tid == 0) {
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = at;
      for (int r0 = 0; r0 < cnt[e]; r0 += kTile) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = at + r0;
        tiles[3 * nt + 2] = min(kTile, cnt[e] - r0);
        ++nt;
      }
      at += cnt[e];
    }
    meta[0] = nt;
  }
  __syncthreads();
  for (int e = warp; e < E; e += nw) {     // stable: pairs of an expert keep their order
    int at = off[e];
    for (int p0 = 0; p0 < pairs; p0 += 32) {
      const int p = p0 + lane;
      const bool mine = p < pairs && sel[p] == e;
      const uint32_t mask = __ballot_sync(0xffffffffu, mine);
      if (mine) perm[at + __popc(mask & ((1u << lane) - 1u))] = p;
      at += __popc(mask);
    }
  }
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TA* __restrict__ A, int64_t lda, int a_mod,
                                                       const TW* __restrict__ W, int64_t expert_stride, int64_t ldw,
                                                       const int32_t* __restrict__ perm, const int32_t* __restrict__ meta,
                                                       const int32_t* __restrict__ tiles, int N, int K,
                                                       float* __restrict__ C, int64_t ldc, int c_perm) {
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  __shared__ float As[kStepK][kTile + 4];
  __shared__ float Ws[kStepK][kTile + 4];
  __shared__ int32_t a_row[kTile], c_row[kTile];
  const int e = tiles[3 * tile], s0 = tiles[3 * tile + 1], M = tiles[3 * tile + 2];
  const int tid = threadIdx.x;
  if (tid < kTile) {
    const int s = s0 + min(tid, M - 1);
    const int p = perm[s];
    a_row[tid] = a_mod > 0 ? p % a_mod : s;
    c_row[tid] = c_perm ? p : s;
  }
  __syncthreads();
  const TW* We = W + (int64_t)e * expert_stride;
  const int n0 = blockIdx.x * kTile;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int lr = tid / 4;          // 0..63
  const int lk = (tid % 4) * 4;    // 0,4,8,12
  const int64_t arow = a_row[lr];
  for (int k0 = 0; k0 < K; k0 += kStepK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int nn = n0 + lr;
      As[lk + j][lr] = (lr < M && k < K) ? to_f32(A[arow * lda + k]) : 0.f;
      Ws[lk + j][lr] = (nn < N && k < K) ? to_f32(We[(int64_t)nn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kStepK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (tm + i >= M) continue;
    const int64_t row = c_row[tm + i];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int nn = n0 + tn + j;
      if (nn < N) C[row * ldc + nn] = acc[i][j];
    }
  }
}

// ---- bf16 tensor-core variant ------------------------------------------------------------------------------------------
constexpr int kBN = 128, kBK = 32, kPad = 8;      // tile N, K step, padding (halves) that keeps ldmatrix conflict-free
constexpr int kLds = kBK + kPad;                  // 40 halves = 80 bytes per staged row
constexpr int kStages = 4;                        // cp.async stages in flight: a few-row tile is a pure weight stream
constexpr size_t kMmaSmem = (size_t)kStages * (kTile + kBN) * kLds * sizeof(__nv_bfloat16);

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(256) moe_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, int a_mod,
                                                           const __nv_bfloat16* __restrict__ W, int64_t expert_stride,
                                                           int64_t ldw, const int32_t* __restrict__ perm,
                                                           const int32_t* __restrict__ meta, const int32_t* __restrict__ tiles,
                                                           int N, int K, float* __restrict__ C, int64_t ldc, int c_perm) {
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  extern __shared__ __align__(16) unsigned char mma_smem[];
  typedef __nv_bfloat16 (*ATile)[kTile][kLds];
  typedef __nv_bfloat16 (*BTile)[kBN][kLds];
  ATile As = reinterpret_cast<ATile>(mma_smem);                                           // [kStages][64][40]
  BTile Bs = reinterpret_cast<BTile>(mma_smem + (size_t)kStages * kTile * kLds * sizeof(__nv_bfloat16));   // [kStages][128][40]
  __shared__ int32_t a_row[kTile], c_row[kTile];
  const int e = tiles[3 * tile], s0 = tiles[3 * tile + 1], M = tiles[3 * tile + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kTile) {
    const int s = s0 + min(tid, M - 1);
    const int p = perm[s];
    a_row[tid] = a_mod > 0 ? p % a_mod : s;
    c_row[tid] = c_perm ? p : s;
  }
  __syncthreads();
  const __nv_bfloat16* We = W + (int64_t)e * expert_stride;
  const int n0 = blockIdx.x * kBN;
  const int wm = (warp >> 2) * 32, wn = (warp & 3) * 32;       // warp tile 32 x 32
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;
  // loaders: A 64 rows x 4 chunks of 8 halves (one per thread), B 128 rows x 4 chunks (two per thread)
  const int lr = tid >> 2, lc = (tid & 3) * 8;
  const int64_t a_off = (int64_t)a_row[lr] * lda;
  auto stage = [&](int k0, int buf) {
    const int k = k0 + lc;
    const bool kin = k < K;
    cp_async16_zfill(&As[buf][lr][lc], A + a_off + (kin ? k : 0), (kin && lr < M) ? 16 : 0);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = lr + 64 * h, nn = n0 + r;
      const bool ok = kin && nn < N;
      cp_async16_zfill(&Bs[buf][r][lc], We + (int64_t)(ok ? nn : 0) * ldw + (kin ? k : 0), ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // kStages - 1 steps in flight; a commit per step keeps the group count regular (empty past the end, where `stage`
  // copies nothing but zero fill into a buffer nobody reads)
#pragma unroll
  for (int st = 0; st < kStages - 1; ++st) stage(st * kBK, st);
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += kBK, buf = (buf + 1) % kStages) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
    __syncthreads();            // step k0 has landed for every thread, and every warp is done with the buffer refilled next
    stage(k0 + (kStages - 1) * kBK, (buf + kStages - 1) % kStages);
#pragma unroll
    for (int kk = 0; kk < kBK; kk += 16) {
      uint32_t af[2][4], bf[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) ldsm_x4(af[i], &As[buf][wm + 16 * i + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 2; ++j) ldsm_x4(bf[j], &Bs[buf][wn + 16 * j + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = wm + 16 * i + (lane >> 2) + 8 * half;
      if (m >= M) continue;
      float* crow = C + (int64_t)c_row[m] * ldc;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int nn = n0 + wn + 8 * j + (lane & 3) * 2;
        if (nn < N) crow[nn] = acc[i][j][2 * half];
        if (nn + 1 < N) crow[nn + 1] = acc[i][j][2 * half + 1];
      }
    }
}

// act[s] = g * sigmoid(beta g) * (u + 1),  g = min(w * gate, lim), u = clamp(w * up, -lim, lim),  w = wsel[perm[s]]
template <typename T>
__global__ void moe_glu_kernel(const float* __restrict__ gu, int64_t ld, int F, const int32_t* __restrict__ perm,
                               const float* __restrict__ wsel, float lim, float beta, T* __restrict__ out) {
  pdl_wait();
  const int64_t s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= F) return;
  const float w = wsel[perm[s]];
  const float g = fminf(w * gu[s * ld + c], lim);
  const float u = fminf(fmaxf(w * gu[s * ld + F + c], -lim), lim);
  out[s * F + c] = T(g * sigmoid_f(beta * g) * (u + 1.f));
}

// act[s] = act(gate) * up * (w * wscale), act = SiLU: the pair's weight multiplies the expert's OUTPUT; the second
// projection is linear and has no bias, so the weight is applied to its input instead (in fp32, before the rounding)
template <typename T>
__global__ void moe_glu_out_kernel(const float* __restrict__ gu, int64_t ld, int F, const int32_t* __restrict__ perm,
                                   const float* __restrict__ wsel, float wscale, T* __restrict__ out) {
  pdl_wait();
  const int64_t s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= F) return;
  const float w = wsel[perm[s]] * wscale;
  const float g = gu[s * ld + c];
  out[s * F + c] = T(g * sigmoid_f(g) * gu[s * ld + F + c] * w);
}

}  // namespace
}  // namespace prl

using namespace prl;
typedef __nv_bfloat16 bf16;

extern "C" int64_t prl_moe_max_tiles(int64_t pairs, int32_t experts) { return (pairs + kTile - 1) / kTile + experts; }

extern "C" int prl_moe_route(const float* logits, int64_t ld, const float* bias, int32_t n, int32_t experts, int32_t top,
                             int32_t softmax_weights, int32_t* sel, float* wsel, int32_t* perm, int32_t* meta,
                             int32_t* tiles, prl_stream_t st) {
  PRL_CHECK_ARG(logits && sel && wsel && perm && meta && tiles, "prl_moe_route: NULL argument");
  PRL_CHECK_ARG(n >= 1 && experts >= 1 && experts <= 32 * kMaxPerLane && top >= 1 && top <= experts && ld >= experts,
                "prl_moe_route: bad shape (experts=%d top=%d; at most %d experts)", experts, top, 32 * kMaxPerLane);
  cudaStream_t s = (cudaStream_t)st;
  PRL_CUDA(launch_pdl(moe_route_kernel, dim3((n + 7) / 8), dim3(256), (size_t)0, s, logits, ld, bias, n, experts, top, softmax_weights, sel, wsel));
  PRL_LAUNCH_CHECK();
  PRL_CUDA(launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)(2 * experts * sizeof(int32_t)), s, (const int32_t*)sel, n * top, experts, perm, meta, tiles));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

// Router product, choice and grouping in two launches: x [n, W] and the router matrix [experts, W] in fp32 or bf16.
// Needs (W + experts) * 4 bytes of shared memory; returns PRL_ERR_INVALID beyond 160 KB (use prl_gemm_any + prl_moe_route).
extern "C" int prl_moe_router(const void* x, int32_t x_is_f32, const void* Wr, int32_t w_is_f32, const float* bias, int32_t n, int32_t W,
                              int32_t experts, int32_t top, int32_t softmax_weights, int32_t* sel, float* wsel, int32_t* perm,
                              int32_t* meta, int32_t* tiles, prl_stream_t st) {
  PRL_CHECK_ARG(x && Wr && sel && wsel && perm && meta && tiles, "prl_moe_router: NULL argument");
  PRL_CHECK_ARG(n >= 1 && W >= 1 && experts >= 1 && experts <= 32 * kMaxPerLane && top >= 1 && top <= experts,
                "prl_moe_router: bad shape (experts=%d top=%d; at most %d experts)", experts, top, 32 * kMaxPerLane);
  const size_t smem = ((size_t)W + experts) * sizeof(float);
  PRL_CHECK_ARG(smem <= 160 * 1024, "prl_moe_router: a row of %d channels does not fit in shared memory", W);
  cudaStream_t s = (cudaStream_t)st;
  static SmemAttr attr[4] = {};
#define PRL_RT(TX, TW, I)                                                                                              \
  do {                                                                                                                 \
    if (smem > 48 * 1024) PRL_CUDA(ensure_smem(moe_router_kernel<TX, TW>, (int)smem, attr[I]));                        \
    PRL_CUDA(launch_pdl((moe_router_kernel<TX, TW>), dim3(n), dim3(256), smem, s, (const TX*)x, (const TW*)Wr, bias, n, W, experts, top, \
                        softmax_weights, sel, wsel));                                                                  \
  } while (0)
  if (x_is_f32 && w_is_f32) PRL_RT(float, float, 0);
  else if (x_is_f32) PRL_RT(float, bf16, 1);
  else if (w_is_f32) PRL_RT(bf16, float, 2);
  else PRL_RT(bf16, bf16, 3);
#undef PRL_RT
  PRL_LAUNCH_CHECK();
  PRL_CUDA(launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)(2 * experts * sizeof(int32_t)), s, (const int32_t*)sel, n * top, experts, perm, meta, tiles));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_moe_gemm(const void* A, int32_t a_is_f32, int64_t lda, int32_t a_mod, const void* W, int32_t w_is_f32,
                            int64_t expert_stride, int64_t ldw, const int32_t* perm, const int32_t* meta,
                            const int32_t* tiles, int64_t max_tiles, int64_t N, int64_t K, float* C, int64_t ldc,
                            int32_t c_perm, prl_stream_t st) {
  PRL_CHECK_ARG(A && W && perm && meta && tiles && C, "prl_moe_gemm: NULL argument");
  PRL_CHECK_ARG(max_tiles >= 1 && max_tiles <= 65535 && N >= 1 && K >= 1 && lda >= K && ldw >= K && ldc >= N && a_mod >= 0,
                "prl_moe_gemm: bad shape (tiles=%lld N=%lld K=%lld)", (long long)max_tiles, (long long)N, (long long)K);
  cudaStream_t s = (cudaStream_t)st;
  if (!a_is_f32 && !w_is_f32 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && expert_stride % 8 == 0 &&
      ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) {
    dim3 grid_tc((unsigned)((N + kBN - 1) / kBN), (unsigned)max_tiles);
    static SmemAttr attr = {};
    PRL_CUDA(ensure_smem(moe_gemm_mma_kernel, (int)kMmaSmem, attr));
    PRL_CUDA(launch_pdl(moe_gemm_mma_kernel, grid_tc, dim3(256), kMmaSmem, s, (const bf16*)A, lda, a_mod, (const bf16*)W,
                        expert_stride, ldw, perm, meta, tiles, (int)N, (int)K, C, ldc, c_perm));
    PRL_LAUNCH_CHECK();
    return PRL_OK;
  }
  dim3 grid((unsigned)((N + kTile - 1) / kTile), (unsigned)max_tiles);
#define PRL_MG(TA, TW) PRL_CUDA(launch_pdl((moe_gemm_kernel<TA, TW>), grid, dim3(256), (size_t)0, s, (const TA*)A, lda, a_mod, (const TW*)W, \
                                           expert_stride, ldw, perm, meta, tiles, (int)N, (int)K, C, ldc, c_perm))
  if (a_is_f32 && w_is_f32) PRL_MG(float, float);
  else if (a_is_f32) PRL_MG(float, bf16);
  else if (w_is_f32) PRL_MG(bf16, float);
  else PRL_MG(bf16, bf16);
#undef PRL_MG
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

extern "C" int prl_moe_glu(const float* gate_up, int64_t ld, int64_t pairs, int32_t F, const int32_t* perm,
                           const float* wsel, float limit, float beta, void* out, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(gate_up && perm && wsel && out && pairs >= 1 && F >= 1 && ld >= 2 * (int64_t)F, "prl_moe_glu: bad argument");
  dim3 grid((unsigned)pairs, (F + 255) / 256);
  if (f32) PRL_CUDA(launch_pdl(moe_glu_kernel<float>, grid, dim3(256), (size_t)0, (cudaStream_t)st, gate_up, ld, F, perm, wsel, limit, beta, (float*)out));
  else PRL_CUDA(launch_pdl(moe_glu_kernel<bf16>, grid, dim3(256), (size_t)0, (cudaStream_t)st, gate_up, ld, F, perm, wsel, limit, beta, (bf16*)out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}

// Gated expert activation with the pair's weight on the expert's OUTPUT: out = silu(gate) * up * (wsel * wscale).
extern "C" int prl_moe_glu_out(const float* gate_up, int64_t ld, int64_t pairs, int32_t F, const int32_t* perm,
                               const float* wsel, float wscale, void* out, int32_t f32, prl_stream_t st) {
  PRL_CHECK_ARG(gate_up && perm && wsel && out && pairs >= 1 && F >= 1 && ld >= 2 * (int64_t)F, "prl_moe_glu_out: bad argument");
  dim3 grid((unsigned)pairs, (F + 255) / 256);
  if (f32) PRL_CUDA(launch_pdl(moe_glu_out_kernel<float>, grid, dim3(256), (size_t)0, (cudaStream_t)st, gate_up, ld, F, perm, wsel, wscale, (float*)out));
  else PRL_CUDA(launch_pdl(moe_glu_out_kernel<bf16>, grid, dim3(256), (size_t)0, (cudaStream_t)st, gate_up, ld, F, perm, wsel, wscale, (bf16*)out));
  PRL_LAUNCH_CHECK();
  return PRL_OK;
}
