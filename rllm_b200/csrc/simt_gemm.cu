// Plain matrix product on the CUDA cores, float accumulate, both storage types:
//   C[T, N] = A[T, K] * W[N, K]^T      (weights row-major [out, in], as stored)
// It is the product of the true 32-bit path (float storage, FMA only, no
// reduced-precision matrix mode) and the fallback of the bfloat16 path for
// sizes the tensor-core kernel refuses. Every output element is summed over k
// in ascending order by one thread, so a row's result does not depend on which
// other rows share the batch.
//
// Epilogues: store (activation type), store max(., 0)^2 (activation type), store float (logits),
// accumulate into the float residual stream, and SwiGLU over a gate/up pair of weight tiles
// (W holds [2N, K]: gate rows first, up rows after; out[t, n] = silu(g) * u).
// Reference counterparts: src/gpu/cuda/shaders/matmul.cu:49-77, 216-248 and
// moe.cu:86-147 (fused gate-up).
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

enum : int { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_ACCUM_F32 = 2, EPI_SWIGLU = 3, EPI_RELU2 = 4 };

template <typename TI, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, void* __restrict__ Cv,
                 const TI* __restrict__ bias, int T, int N, int K, int lda, int ldc) {
  pdl_launch();
  pdl_wait();
  constexpr bool DUAL = (EPI == EPI_SWIGLU);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[DUAL ? BK : 1][BN + 4];

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN] = {};
  float acu[DUAL ? TM : 1][TN] = {};

  const int lrow = tid / 4, lk = (tid % 4) * 4;   // each thread stages 4 consecutive k of one row

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + j][lrow] = (am < T && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + j][lrow] = (wn < N && k < K) ? to_f32(W[(size_t)wn * K + k]) : 0.f;
      if (DUAL) Us[lk + j][lrow] = (wn < N && k < K) ? to_f32(W[((size_t)N + wn) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN], u[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
      if (DUAL) {
#pragma unroll
        for (int j = 0; j < TN; ++j) u[j] = Us[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (DUAL) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= T) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += to_f32(bias[n]);
      const size_t o = (size_t)m * ldc + n;
      if (EPI == EPI_STORE) ((TI*)Cv)[o] = from_f32<TI>(v);
      else if (EPI == EPI_STORE_F32) ((float*)Cv)[o] = v;
      else if (EPI == EPI_ACCUM_F32) ((float*)Cv)[o] += v;
      else if (EPI == EPI_RELU2) { const float r = fmaxf(v, 0.f); ((TI*)Cv)[o] = from_f32<TI>(r * r); }   // squared in float, rounded once
      else { float g = v, uu = acu[DUAL ? i : 0][j]; ((TI*)Cv)[o] = from_f32<TI>(g / (1.f + expf(-g)) * uu); }
    }
  }
}

template <typename TI>
int launch(int epi, const void* A, const void* W, void* C, const void* bias, int T, int N, int K,
           int lda, int ldc, cudaStream_t s) {
  dim3 grid((N + BN - 1) / BN, (T + BM - 1) / BM), block(256);
  int rc = 0;
#define GO(E) rc = launch_ex(gemm_simt_kernel<TI, E>, dim3(grid), dim3(block), 0, s, 1, (const TI*)A, (const TI*)W, C, (const TI*)bias, T, N, K, lda, ldc)
  switch (epi) {
    case EPI_STORE: GO(EPI_STORE); break;
    case EPI_STORE_F32: GO(EPI_STORE_F32); break;
    case EPI_ACCUM_F32: GO(EPI_ACCUM_F32); break;
    case EPI_SWIGLU: GO(EPI_SWIGLU); break;
    case EPI_RELU2: GO(EPI_RELU2); break;
    default: return ERR_BAD_SIZE;
  }
#undef GO
  return rc;
}

// Few outputs a row (a gate row, a handful of heads or experts): a CTA a row of A, the threads stride over K
// and keep one sum per output; a row's sums are added in one fixed order whatever else the batch holds.
constexpr int SKINNY_MAX = 8;

template <typename TI> struct Piece {};
template <> struct Piece<float> { static constexpr int N = 4; typedef float4 V;
  static __device__ __forceinline__ void get(const float4& v, float* f) { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; } };
template <> struct Piece<bf16> { static constexpr int N = 8; typedef uint4 V;
  static __device__ __forceinline__ void get(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  } };

// A CTA of `blockDim.x / 32` warps a row; VEC: rows of A and W start on 16 bytes and K is a whole number of 16-byte
// pieces, which the threads then stride over; else element by element. Warp sums, then the warps in order.
template <typename TI, bool VEC>
__global__ void __launch_bounds__(256)
gemm_skinny_kernel(const TI* __restrict__ A, const TI* __restrict__ W, float* __restrict__ C, int T, int N, int K,
                   long long lda, int ldc) {
  pdl_launch();
  pdl_wait();
  __shared__ float part[8][SKINNY_MAX];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const long long t = blockIdx.x;
  const TI* a = A + t * lda;
  float acc[SKINNY_MAX];
#pragma unroll
  for (int n = 0; n < SKINNY_MAX; ++n) acc[n] = 0.f;
  if (VEC) {
    typedef typename Piece<TI>::V V;
    constexpr int PN = Piece<TI>::N;
    const int pieces = K / PN;
    for (int c = threadIdx.x; c < pieces; c += blockDim.x) {
      float x[PN];
      Piece<TI>::get(reinterpret_cast<const V*>(a)[c], x);
#pragma unroll
      for (int n = 0; n < SKINNY_MAX; ++n) {
        if (n < N) {
          float wv[PN];
          Piece<TI>::get(reinterpret_cast<const V*>(W + (size_t)n * K)[c], wv);
#pragma unroll
          for (int i = 0; i < PN; ++i) acc[n] = fmaf(x[i], wv[i], acc[n]);
        }
      }
    }
  } else {
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      const float x = to_f32(a[k]);
#pragma unroll
      for (int n = 0; n < SKINNY_MAX; ++n)
        if (n < N) acc[n] = fmaf(x, to_f32(W[(size_t)n * K + k]), acc[n]);
    }
  }
#pragma unroll
  for (int n = 0; n < SKINNY_MAX; ++n) {
    if (n < N) {
      const float v = warp_sum(acc[n]);
      if (lane == 0) part[warp][n] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < N) {
    float v = 0.f;
    for (int w2 = 0; w2 < nw; ++w2) v += part[w2][threadIdx.x];
    C[t * ldc + threadIdx.x] = v;
  }
}

}  // namespace

// C[T, N] (float, row stride ldc) = A[T, K] (row stride lda) W[N, K]^T for N <= 8.
RLLM_API int rllm_gemm_skinny(int dt, const void* A, const void* W, float* C, int T, int N, int K, long long lda,
                              int ldc, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || N > SKINNY_MAX) return ERR_BAD_SIZE;
  if (T > 2147483647LL) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  const int esz = dt == DT_F32 ? 4 : 2, pn = 16 / esz;
  const bool vec = K % pn == 0 && lda % pn == 0 && !((uintptr_t)A & 15) && !((uintptr_t)W & 15);
  // warps a row: as many as the row has 16-byte pieces for, up to eight (the count depends on K alone)
  int warps = vec ? (K / pn + 31) / 32 : (K + 255) / 256;
  warps = warps < 1 ? 1 : (warps > 8 ? 8 : warps);
  const dim3 grid((unsigned)T), block(32 * warps);
  if (dt == DT_F32)
    return vec ? launch_ex(gemm_skinny_kernel<float, true>, grid, block, 0, s, 1, (const float*)A, (const float*)W, C, T, N, K, lda, ldc)
               : launch_ex(gemm_skinny_kernel<float, false>, grid, block, 0, s, 1, (const float*)A, (const float*)W, C, T, N, K, lda, ldc);
  if (dt == DT_BF16)
    return vec ? launch_ex(gemm_skinny_kernel<bf16, true>, grid, block, 0, s, 1, (const bf16*)A, (const bf16*)W, C, T, N, K, lda, ldc)
               : launch_ex(gemm_skinny_kernel<bf16, false>, grid, block, 0, s, 1, (const bf16*)A, (const bf16*)W, C, T, N, K, lda, ldc);
  return ERR_BAD_DTYPE;
}

// A: [T, K] with row stride lda; W: [N, K] ([2N, K] for the SwiGLU epilogue);
// C: [T, N] with row stride ldc, of the type the epilogue names; bias [N] or null.
RLLM_API int rllm_gemm_simt(int dt, int epi, const void* A, const void* W, void* C, const void* bias,
                            int T, int N, int K, int lda, int ldc, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0) return ERR_BAD_SIZE;
  if ((T + BM - 1) / BM > 65535) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32) return launch<float>(epi, A, W, C, bias, T, N, K, lda, ldc, s);
  if (dt == DT_BF16) return launch<bf16>(epi, A, W, C, bias, T, N, K, lda, ldc, s);
  return ERR_BAD_DTYPE;
}
