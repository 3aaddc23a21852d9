// Many small matrix products in one launch, on the CUDA cores, float accumulate, both storage types:
//   C_g[r, n] = epilogue( sum_k A_g[r, k] * B_g[n, k] )        (B_g row-major [N, K], as weights are stored)
//
// Two ways to say which rows belong to which problem:
//   uniform  every problem g (a head) takes all T rows; its A columns start at g * a_gs, its C columns at
//            g * c_gs, its weights at B + g * b_gs. grid.z = problems.
//   ragged   problems (experts) own segments of a sorted row list; a table written on the device by the
//            routing plan names, per 64-row tile, the problem, the first sorted row and the row count;
//            `rows_in[r]` is the A row a sorted row reads (gather), `rows_out[r]` the C row it writes
//            (scatter), `row_scale[r]` a float factor. CTAs beyond the table's count leave at once, so the
//            launch shape depends on the step's size only and never on the routing.
// Every output element is summed over k in ascending order by one thread: a row's result does not depend
// on where in a list it stands or on what else is in the batch.
//
// Epilogues: store (storage type), store float, relu(x)^2 (storage type). Optional per-(row, problem)
// gate g: the result is multiplied by sigmoid(g) (uniform mode).
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each
enum : int { GEPI_STORE = 0, GEPI_STORE_F32 = 1, GEPI_RELU2 = 2 };

struct GroupedArgs {
  const void* A; long long lda, a_gs;
  const void* B; long long b_gs;
  void* C; long long ldc, c_gs;
  int T, N, K;
  const int* tiles;        // ragged: [max_tiles][3] = problem, first sorted row, rows; null: uniform
  const int* n_tiles;      // ragged: one int on the device
  const int* rows_in;      // ragged, optional
  const int* rows_out;     // ragged, optional
  const float* row_scale;  // ragged, optional
  const void* gate; long long gate_ld;   // uniform, optional: gate[r * gate_ld + g]
};

template <typename TI, int EPI>
__global__ void __launch_bounds__(256) grouped_gemm_kernel(const GroupedArgs p) {
  pdl_launch();
  pdl_wait();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int arow[BM];

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  int g, row0, rows;
  if (p.tiles) {
    if ((int)blockIdx.y >= *p.n_tiles) return;
    g = p.tiles[3 * blockIdx.y]; row0 = p.tiles[3 * blockIdx.y + 1]; rows = p.tiles[3 * blockIdx.y + 2];
  } else {
    g = blockIdx.z; row0 = blockIdx.y * BM; rows = min(BM, p.T - row0);
  }
  const int n0 = blockIdx.x * BN;
  const TI* A = (const TI*)p.A + (p.tiles ? 0 : (long long)g * p.a_gs);
  const TI* B = (const TI*)p.B + (long long)g * p.b_gs;
  if (tid < BM) arow[tid] = tid < rows ? (p.rows_in ? p.rows_in[row0 + tid] : row0 + tid) : -1;
  __syncthreads();

  float acc[TM][TN] = {};
  const int lrow = tid / 4, lk = (tid % 4) * 4;   // each thread stages 4 consecutive k of one row
  const int am = arow[lrow];
  const int wn = n0 + lrow;
  for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      As[lk + j][lrow] = (am >= 0 && k < p.K) ? to_f32(A[(long long)am * p.lda + k]) : 0.f;
      Ws[lk + j][lrow] = (wn < p.N && k < p.K) ? to_f32(B[(long long)wn * p.K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = ty * TM + i;
    if (m >= rows) continue;
    const int r = row0 + m;
    const long long crow = p.rows_out ? p.rows_out[r] : r;
    float f = p.row_scale ? p.row_scale[r] : 1.f;
    if (p.gate) {
      const float gv = to_f32(((const TI*)p.gate)[(long long)r * p.gate_ld + g]);
      f *= 1.f / (1.f + expf(-gv));
    }
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if (EPI == GEPI_RELU2) { v = fmaxf(v, 0.f); v = v * v; }
      v *= f;
      const long long o = crow * p.ldc + (p.tiles ? 0 : (long long)g * p.c_gs) + n;
      if (EPI == GEPI_STORE_F32) ((float*)p.C)[o] = v;
      else ((TI*)p.C)[o] = from_f32<TI>(v);
    }
  }
}

template <typename TI>
int launch(int epi, const GroupedArgs& p, dim3 grid, cudaStream_t s) {
  switch (epi) {
    case GEPI_STORE: return launch_ex(grouped_gemm_kernel<TI, GEPI_STORE>, grid, dim3(256), 0, s, 1, p);
    case GEPI_STORE_F32: return launch_ex(grouped_gemm_kernel<TI, GEPI_STORE_F32>, grid, dim3(256), 0, s, 1, p);
    case GEPI_RELU2: return launch_ex(grouped_gemm_kernel<TI, GEPI_RELU2>, grid, dim3(256), 0, s, 1, p);
  }
  return ERR_BAD_SIZE;
}

}  // namespace

// Uniform problems: A [T, >= G * a_gs] row stride lda; B [G][N, K]; C [T, ...] row stride ldc, problem g at
// column g * c_gs. gate (optional, storage type): [T, gate_ld], problem g at column g.
RLLM_API int rllm_grouped_gemm_uniform(int dt, int epi, const void* A, long long lda, long long a_gs, const void* B,
                                       long long b_gs, void* C, long long ldc, long long c_gs, int T, int G, int N,
                                       int K, const void* gate, long long gate_ld, void* stream) {
  if (T <= 0 || G <= 0 || N <= 0) return 0;
  if (K <= 0) return ERR_BAD_SIZE;
  if ((T + BM - 1) / BM > 65535 || G > 65535) return ERR_TOO_LARGE;
  GroupedArgs p = {A, lda, a_gs, B, b_gs, C, ldc, c_gs, T, N, K, nullptr, nullptr, nullptr, nullptr, nullptr, gate, gate_ld};
  dim3 grid((N + BN - 1) / BN, (T + BM - 1) / BM, G);
  if (dt == DT_F32) return launch<float>(epi, p, grid, (cudaStream_t)stream);
  if (dt == DT_BF16) return launch<bf16>(epi, p, grid, (cudaStream_t)stream);
  return ERR_BAD_DTYPE;
}

// Ragged problems: the tile table (`tiles`, `n_tiles`) comes from rllm_moe_plan; max_tiles bounds the grid.
RLLM_API int rllm_grouped_gemm_ragged(int dt, int epi, const void* A, long long lda, const void* B, long long b_gs,
                                      void* C, long long ldc, int N, int K, const int* tiles, const int* n_tiles,
                                      int max_tiles, const int* rows_in, const int* rows_out, const float* row_scale,
                                      void* stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K <= 0 || !tiles || !n_tiles) return ERR_BAD_SIZE;
  if (max_tiles > 65535) return ERR_TOO_LARGE;
  GroupedArgs p = {A, lda, 0, B, b_gs, C, ldc, 0, 0, N, K, tiles, n_tiles, rows_in, rows_out, row_scale, nullptr, 0};
  dim3 grid((N + BN - 1) / BN, max_tiles, 1);
  if (dt == DT_F32) return launch<float>(epi, p, grid, (cudaStream_t)stream);
  if (dt == DT_BF16) return launch<bf16>(epi, p, grid, (cudaStream_t)stream);
  return ERR_BAD_DTYPE;
}
