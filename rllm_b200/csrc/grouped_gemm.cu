// Many small matrix products in one launch, on the CUDA cores, float accumulate, both storage types:
//   C_g[r, n] = epilogue( sum_k A_g[r, k] * B_g[n, k] )        (B_g row-major [N, K], as weights are stored)
//
// Two ways to say which rows belong to which problem:
//   uniform  every problem g (a head) takes all T rows; its A columns start at g * a_gs, its C columns at
//            g * c_gs, its weights at B + g * b_gs. grid.z = problems.
//   ragged   problems (experts) own segments of a sorted row list; a table written on the device by the
//            routing plan names, per tile of rows, the problem, the first sorted row and the row count;
//            `rows_in[r]` is the A row a sorted row reads (gather), `rows_out[r]` the C row it writes
//            (scatter), `row_scale[r]` a float factor. CTAs beyond the table's count leave at once, so the
//            launch shape depends on the step's size only and never on the routing.
// Every output element is summed over k in ascending order by one thread: a row's result does not depend
// on where in a list it stands or on what else is in the batch.
//
// Epilogues: store (storage type), store float, relu(x)^2 (storage type). Optional per-(row, problem)
// gate g: the result is multiplied by sigmoid(g) (uniform mode).
//
// bfloat16 problems whose rows are 16-byte aligned (K, strides and offsets multiples of 8) run on the
// tensor cores instead (grouped_gemm_mma_kernel, in a shape for long and one for short row lists):
// `mma.sync` m16n8k16 with float accumulators, operands brought by `cp.async` (gathered rows included) through
// a ring of stages and read with `ldmatrix`; a warp leaves out the row tiles of 16 that lie beyond the tile's
// rows, so that a tile with a few rows costs its weights' way through the ring and little else. K runs in ascending blocks of 16 inside one accumulator: a row's result is the
// same wherever it stands. The float path keeps to FMA.
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

// ------------------------------------------------------------------------------------------ tensor cores
// Two shapes of the kernel: LONG for tiles of up to 128 rows (prompt portions: 128 x 128 x 64, three stages,
// eight warps of 64 x 32), FEW for tiles of up to 32 rows (decoding: what counts is the weights' way through
// the ring, so 256 contiguous bytes of a weight row per copy step, four stages, tiles of 64 weight rows so
// that there are CTAs for every SM; four warps of 32 x 16).
struct LongTile { static constexpr int BM = 128, BN = 128, BK = 64, ST = 3, WM = 2, WN = 4, CTAS = 2; };
struct FewTile { static constexpr int BM = 32, BN = 64, BK = 128, ST = 4, WM = 1, WN = 4, CTAS = 2; };
template <typename C> constexpr int mma_smem() { return C::ST * (C::BM + C::BN) * (C::BK + 8) * 2; }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int EPI, typename C>
__global__ void __launch_bounds__(C::WM * C::WN * 32, C::CTAS) grouped_gemm_mma_kernel(const GroupedArgs p) {
  pdl_launch();
  pdl_wait();
  constexpr int BM_ = C::BM, BN_ = C::BN, BK_ = C::BK, ST_ = C::ST, THREADS = C::WM * C::WN * 32;
  constexpr int LDS = BK_ + 8;                                        // rows 16 bytes apart in the banks: ldmatrix meets 8 bank groups
  constexpr int MT = BM_ / C::WM / 16, NT = BN_ / C::WN / 8;          // row tiles of 16 and column tiles of 8 a warp
  constexpr int CPR = BK_ / 8;                                        // 16-byte pieces of a row per block of K
  static_assert(NT % 2 == 0 && (BM_ * CPR) % THREADS == 0 && (BN_ * CPR) % THREADS == 0, "tile shape");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* As = reinterpret_cast<bf16*>(smem_raw);                      // [ST][BM][LDS]
  bf16* Bs = As + ST_ * BM_ * LDS;                                   // [ST][BN][LDS]
  __shared__ int arow[BM_];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp / C::WN, wn = warp % C::WN;
  int g, row0, rows;
  if (p.tiles) {
    if ((int)blockIdx.y >= *p.n_tiles) return;
    g = p.tiles[3 * blockIdx.y]; row0 = p.tiles[3 * blockIdx.y + 1]; rows = p.tiles[3 * blockIdx.y + 2];
  } else {
    g = blockIdx.z; row0 = blockIdx.y * BM_; rows = min(BM_, p.T - row0);
  }
  const int n0 = blockIdx.x * BN_;
  const bf16* A = (const bf16*)p.A + (p.tiles ? 0 : (long long)g * p.a_gs);
  const bf16* B = (const bf16*)p.B + (long long)g * p.b_gs;
  for (int r = tid; r < BM_; r += THREADS) arow[r] = r < rows ? (p.rows_in ? p.rows_in[row0 + r] : row0 + r) : -1;
  __syncthreads();

  const int nk = (p.K + BK_ - 1) / BK_;
  auto load = [&](int kb) {
    const int st = kb % ST_;
#pragma unroll
    for (int i = 0; i < BM_ * CPR / THREADS; ++i) {
      const int c = tid + i * THREADS, r = c / CPR, k = kb * BK_ + (c % CPR) * 8;
      const int ar = arow[r];
      const bool in = ar >= 0 && k < p.K;                            // K is a multiple of 8: a piece is whole or empty
      cp_async16(As + (st * BM_ + r) * LDS + (c % CPR) * 8, A + (in ? (long long)ar * p.lda + k : 0), in ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < BN_ * CPR / THREADS; ++i) {
      const int c = tid + i * THREADS, r = c / CPR, k = kb * BK_ + (c % CPR) * 8;
      const bool in = n0 + r < p.N && k < p.K;
      cp_async16(Bs + (st * BN_ + r) * LDS + (c % CPR) * 8, B + (in ? (long long)(n0 + r) * p.K + k : 0), in ? 16 : 0);
    }
  };
  float acc[MT][NT][4] = {};
  // row tiles of 16 this warp has to compute: those beyond the tile's rows are left out
  const int mt_live = min(MT, max(0, (rows - wm * MT * 16 + 15) / 16));
#pragma unroll
  for (int s = 0; s < ST_ - 1; ++s) {
    if (s < nk) load(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kb = 0; kb < nk; ++kb) {
    asm volatile("cp.async.wait_group %0;" ::"n"(ST_ - 2) : "memory");
    __syncthreads();                                                 // block kb has landed; block kb - 1 is used up
    if (kb + ST_ - 1 < nk) load(kb + ST_ - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bf16* as = As + (kb % ST_) * BM_ * LDS;
    const bf16* bs = Bs + (kb % ST_) * BN_ * LDS;
    // the fragments of the next 16 of K are asked for before the products of the current 16 are issued
    unsigned bfrag[2][NT / 2][4], afrag[2][MT][4];
    auto fetch = [&](int buf, int kk) {
#pragma unroll
      for (int j = 0; j < NT / 2; ++j)
        ldmatrix4(bfrag[buf][j], bs + (wn * NT * 8 + j * 16 + (lane & 7) + ((lane >> 4) << 3)) * LDS + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int i = 0; i < MT; ++i)
        if (i < mt_live) ldmatrix4(afrag[buf][i], as + (wm * MT * 16 + i * 16 + (lane & 15)) * LDS + kk + (lane >> 4) * 8);
    };
    fetch(0, 0);
#pragma unroll
    for (int ks = 0; ks < BK_ / 16; ++ks) {
      if (ks + 1 < BK_ / 16) fetch((ks + 1) & 1, (ks + 1) * 16);
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        if (i < mt_live) {
#pragma unroll
          for (int j = 0; j < NT; ++j)
            mma16816(acc[i][j], afrag[ks & 1][i], bfrag[ks & 1][j >> 1][(j & 1) * 2], bfrag[ks & 1][j >> 1][(j & 1) * 2 + 1]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

#pragma unroll
  for (int i = 0; i < MT; ++i) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = wm * MT * 16 + i * 16 + (lane >> 2) + half * 8;
      if (m >= rows) continue;
      const int r = row0 + m;
      const long long crow = p.rows_out ? p.rows_out[r] : r;
      float f = p.row_scale ? p.row_scale[r] : 1.f;
      if (p.gate) {
        const float gv = to_f32(((const bf16*)p.gate)[(long long)r * p.gate_ld + g]);
        f *= 1.f / (1.f + expf(-gv));
      }
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int n = n0 + wn * NT * 8 + j * 8 + (lane & 3) * 2;
        if (n >= p.N) continue;
        float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
        if (EPI == GEPI_RELU2) { v0 = fmaxf(v0, 0.f); v0 *= v0; v1 = fmaxf(v1, 0.f); v1 *= v1; }
        v0 *= f; v1 *= f;
        const long long o = crow * p.ldc + (p.tiles ? 0 : (long long)g * p.c_gs) + n;
        if (EPI == GEPI_STORE_F32) {
          float* c = (float*)p.C + o;
          if (n + 1 < p.N && !(o & 1)) *reinterpret_cast<float2*>(c) = make_float2(v0, v1);
          else { c[0] = v0; if (n + 1 < p.N) c[1] = v1; }
        } else {
          bf16* c = (bf16*)p.C + o;
          if (n + 1 < p.N && !(o & 1)) *reinterpret_cast<__nv_bfloat162*>(c) = __floats2bfloat162_rn(v0, v1);
          else { c[0] = __float2bfloat16_rn(v0); if (n + 1 < p.N) c[1] = __float2bfloat16_rn(v1); }
        }
      }
    }
  }
}

static inline bool mma_ok(const GroupedArgs& p) {
  return p.K % 8 == 0 && p.lda % 8 == 0 && p.a_gs % 8 == 0 && p.b_gs % 8 == 0 && !((uintptr_t)p.A & 15) &&
         !((uintptr_t)p.B & 15);
}

// grid: the caller's (column tiles and row tiles counted with C's sizes)
template <typename C>
static int launch_mma(int epi, const GroupedArgs& p, dim3 grid, cudaStream_t s) {
  constexpr int SMEM = mma_smem<C>();
#define GO(E)                                                                                          \
  do {                                                                                                 \
    static bool done[64] = {};                                                                         \
    int dev = 0;                                                                                       \
    cudaGetDevice(&dev);                                                                               \
    if (dev >= 0 && dev < 64 && !done[dev]) /* once: as much of an SM as shared memory as there is */  \
      cudaFuncSetAttribute(grouped_gemm_mma_kernel<E, C>, cudaFuncAttributePreferredSharedMemoryCarveout, \
                           (int)cudaSharedmemCarveoutMaxShared);                                       \
    const int rc = allow_dynamic_smem(grouped_gemm_mma_kernel<E, C>, SMEM, done);                      \
    if (rc) return rc;                                                                                 \
    return launch_ex(grouped_gemm_mma_kernel<E, C>, grid, dim3(C::WM * C::WN * 32), (size_t)SMEM, s, 1, p); \
  } while (0)
  switch (epi) {
    case GEPI_STORE: GO(GEPI_STORE);
    case GEPI_STORE_F32: GO(GEPI_STORE_F32);
    case GEPI_RELU2: GO(GEPI_RELU2);
  }
#undef GO
  return ERR_BAD_SIZE;
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
  if (dt == DT_BF16 && mma_ok(p) && T <= FewTile::BM)
    return launch_mma<FewTile>(epi, p, dim3((N + FewTile::BN - 1) / FewTile::BN, 1, G), (cudaStream_t)stream);
  if (dt == DT_BF16 && mma_ok(p) && (T + LongTile::BM - 1) / LongTile::BM <= 65535)
    return launch_mma<LongTile>(epi, p, dim3((N + LongTile::BN - 1) / LongTile::BN, (T + LongTile::BM - 1) / LongTile::BM, G),
                                (cudaStream_t)stream);
  if (dt == DT_F32) return launch<float>(epi, p, grid, (cudaStream_t)stream);
  if (dt == DT_BF16) return launch<bf16>(epi, p, grid, (cudaStream_t)stream);
  return ERR_BAD_DTYPE;
}

// Rows a tile of the plan may have for a ragged problem of this type, shape and number of sorted rows: the tile
// of the kernel that will take it (the plan has to be made with it). Few rows (decoding): tiles of 32.
RLLM_API int rllm_grouped_gemm_tile_rows(int dt, long long lda, int K, int n_rows) {
  if (!(dt == DT_BF16 && K % 8 == 0 && lda % 8 == 0)) return BM;
  return n_rows <= 1024 ? FewTile::BM : LongTile::BM;
}

// Ragged problems: the tile table (`tiles`, `n_tiles`) comes from rllm_moe_plan, made with tiles of
// `tile_rows`; max_tiles bounds the grid.
RLLM_API int rllm_grouped_gemm_ragged(int dt, int epi, const void* A, long long lda, const void* B, long long b_gs,
                                      void* C, long long ldc, int N, int K, const int* tiles, const int* n_tiles,
                                      int max_tiles, int tile_rows, const int* rows_in, const int* rows_out,
                                      const float* row_scale, void* stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K <= 0 || !tiles || !n_tiles) return ERR_BAD_SIZE;
  if (max_tiles > 65535) return ERR_TOO_LARGE;
  GroupedArgs p = {A, lda, 0, B, b_gs, C, ldc, 0, 0, N, K, tiles, n_tiles, rows_in, rows_out, row_scale, nullptr, 0};
  dim3 grid((N + BN - 1) / BN, max_tiles, 1);
  if (dt == DT_BF16 && tile_rows == LongTile::BM && mma_ok(p))
    return launch_mma<LongTile>(epi, p, dim3((N + LongTile::BN - 1) / LongTile::BN, max_tiles, 1), (cudaStream_t)stream);
  if (dt == DT_BF16 && tile_rows == FewTile::BM && mma_ok(p))
    return launch_mma<FewTile>(epi, p, dim3((N + FewTile::BN - 1) / FewTile::BN, max_tiles, 1), (cudaStream_t)stream);
  if (tile_rows != BM) return ERR_BAD_SIZE;                          // the plan was made for the other kernel
  if (dt == DT_F32) return launch<float>(epi, p, grid, (cudaStream_t)stream);
  if (dt == DT_BF16) return launch<bf16>(epi, p, grid, (cudaStream_t)stream);
  return ERR_BAD_DTYPE;
}
