// Attention over a cache of compressed latents, on the CUDA cores, float arithmetic, both storage types.
//
// A cached position is one row [c | r] of `dk = rank + rot` numbers: the normalised latent c (rank) and one
// rotated key part r (rot) that all heads share. With the up-projections folded into the query and the
// output (q' = W_uk^T q per head before, W_uv after: the products of the caller), every head's key at a
// position is the row itself and its value is the row's first `rank` numbers, so one read of a row
// serves all heads, keys and values alike.
//
// latent_prepare (one CTA a token): the latent part of the down-projection is RMS-normed in float
//   (x / sqrt(mean(x^2) + eps) * w), the shared key part is rotated, and both go to the token's cache
//   row; the rotated part of every head's query goes to its place behind the folded part in `qfull`.
//   Rotation: pairs (2i, 2i+1), i < dims/2, by the angle of the step's table (cos, sin per token and i);
//   dimensions from `dims` on pass unchanged.
// latent_attention (one CTA a query token and group of up to 8 heads, a warp a head): keys j with
//   max(0, pos - window + 1) <= j <= pos (window <= 0: from 0), taken 32 at a time in position order from
//   the paged cache, staged once in shared memory for all the CTA's heads; running maximum and sum. A
//   query's result depends on its position and the cache alone, never on how tokens were cut into steps
//   or batched.
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int HG = 8;            // heads (warps) per CTA
constexpr int MAX_RANK = 1024;   // 32 accumulators a lane

template <typename TI>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const TI* __restrict__ proj, long long ld, int q_off, int dkv_off, int H, int dim, int rot,
                      int rank, int dims, const float* __restrict__ wnorm, float eps,
                      const float* __restrict__ table, const int* __restrict__ slots, TI* __restrict__ cache,
                      TI* __restrict__ qfull) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const TI* row = proj + (long long)t * ld;
  const float* tab = table + (long long)t * (dims / 2) * 2;
  const int dk = rank + rot;
  const int slot = slots ? slots[t] : -1;
  // the latent, normalised
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(row[dkv_off + i]); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)rank + eps);
  if (slot >= 0) {
    TI* crow = cache + (long long)slot * dk;
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
      crow[i] = from_f32<TI>(to_f32(row[dkv_off + i]) * r * wnorm[i]);
    // the shared key part, rotated
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
      const float v = to_f32(row[dkv_off + rank + i]);
      float o = v;
      if (i < dims) {
        const float c = tab[(i >> 1) * 2], s = tab[(i >> 1) * 2 + 1];
        const float other = to_f32(row[dkv_off + rank + (i ^ 1)]);
        o = (i & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
      }
      crow[rank + i] = from_f32<TI>(o);
    }
  }
  // every head's rotated query part
  for (int x = threadIdx.x; x < H * rot; x += blockDim.x) {
    const int h = x / rot, i = x % rot;
    const TI* q = row + q_off + (long long)h * (dim + rot) + dim;
    const float v = to_f32(q[i]);
    float o = v;
    if (i < dims) {
      const float c = tab[(i >> 1) * 2], s = tab[(i >> 1) * 2 + 1];
      const float other = to_f32(q[i ^ 1]);
      o = (i & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
    }
    qfull[((long long)t * H + h) * dk + rank + i] = from_f32<TI>(o);
  }
}

template <typename TI, int NACC>      // NACC: accumulators a lane, 32 * NACC >= rank
__global__ void __launch_bounds__(HG * 32)
latent_attention_kernel(const TI* __restrict__ qfull, const TI* __restrict__ cache, TI* __restrict__ out,
                        const int* __restrict__ token_seq, const int* __restrict__ positions,
                        const int* __restrict__ block_table, int bt_stride, int H, int rank, int dk, int page_size,
                        float scale, int window) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float sm[];
  const int ldk = dk | 1;                        // odd: the lanes' key rows meet 32 banks
  float* ks = sm;                                // [32][ldk]
  float* qs = sm + 32 * ldk;                     // [HG][dk]
  __shared__ int key_ok[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, h = blockIdx.y * HG + warp;
  const bool live = h < H;
  const int seq = token_seq[t], pos = positions[t];
  const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* bt = block_table + (long long)seq * bt_stride;
  if (live) {
    const TI* qp = qfull + ((long long)t * H + h) * dk;
    for (int d = lane; d < dk; d += 32) qs[warp * dk + d] = to_f32(qp[d]);
  }
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int nwarps = blockDim.x >> 5;

  for (int base = start; base <= pos; base += 32) {
    __syncthreads();                             // the tile before is used up
    for (int j = warp; j < 32; j += nwarps) {
      const int kj = base + j;
      const int page = kj <= pos ? bt[kj / page_size] : -1;
      if (lane == 0) key_ok[j] = page >= 0;
      if (page >= 0) {
        const TI* kp = cache + ((long long)page * page_size + kj % page_size) * dk;
        for (int d = lane; d < dk; d += 32) ks[j * ldk + d] = to_f32(kp[d]);
      } else {
        for (int d = lane; d < dk; d += 32) ks[j * ldk + d] = 0.f;
      }
    }
    __syncthreads();
    if (!live) continue;
    const bool valid = key_ok[lane] != 0;
    float s = -INFINITY;
    if (valid) {
      const float* kr = ks + lane * ldk;
      const float* q = qs + warp * dk;
      float dsum = 0.f;
      for (int d = 0; d < dk; ++d) dsum = fmaf(q[d], kr[d], dsum);
      s = dsum * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;            // no key of this tile has a page
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);          // first tile: exp(-inf) = 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    const int cnt = min(32, pos - base + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* vr = ks + jj * ldk;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) acc[i] = fmaf(pj, vr[d], acc[i]);
      }
    }
    m = m_new;
  }
  if (!live) return;
  const float inv = l > 0.f ? 1.f / l : 0.f;
  TI* op = out + ((long long)t * H + h) * rank;
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) op[d] = from_f32<TI>(acc[i] * inv);
  }
}

}  // namespace

// proj [T, ld]: head h's query at q_off + h * (dim + rot) as [dim plain | rot to rotate]; the down-projection
// at dkv_off as [rank latent | rot shared key part]. table: float [T, dims/2, 2] (cos, sin). slots [T]: cache
// row of each token (-1: do not write) or null. cache: rows of rank + rot. qfull: [T, H, rank + rot], of which
// this writes the last rot of every head.
RLLM_API int rllm_latent_prepare(int dt, const void* proj, long long ld, int q_off, int dkv_off, int T, int H, int dim,
                                 int rot, int rank, int dims, const float* wnorm, float eps, const float* table,
                                 const int* slots, void* cache, void* qfull, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dim < 0 || rot < 0 || rank <= 0 || dims < 0 || dims > rot || dims % 2) return ERR_BAD_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32)
    return launch_ex(latent_prepare_kernel<float>, dim3(T), dim3(128), 0, s, 1, (const float*)proj, ld, q_off, dkv_off, H,
                     dim, rot, rank, dims, wnorm, eps, table, slots, (float*)cache, (float*)qfull);
  if (dt == DT_BF16)
    return launch_ex(latent_prepare_kernel<bf16>, dim3(T), dim3(128), 0, s, 1, (const bf16*)proj, ld, q_off, dkv_off, H,
                     dim, rot, rank, dims, wnorm, eps, table, slots, (bf16*)cache, (bf16*)qfull);
  return ERR_BAD_DTYPE;
}

// qfull [T, H, dk]; cache [pages * page_size, dk]; out [T, H, rank].
RLLM_API int rllm_latent_attention(int dt, const void* qfull, const void* cache, void* out, const int* token_seq,
                                   const int* positions, const int* block_table, int bt_stride, int T, int H, int rank,
                                   int dk, int page_size, float scale, int window, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || rank <= 0 || rank > MAX_RANK || dk < rank || page_size <= 0) return ERR_BAD_SIZE;
  const int hg = H < HG ? H : HG;
  const int smem = (32 * (dk | 1) + hg * dk) * (int)sizeof(float);
  if (smem > 200 * 1024) return ERR_TOO_LARGE;
  if ((H + hg - 1) / hg > 65535) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(T, (H + HG - 1) / HG), block(hg * 32);
#define GO(TI, NACC)                                                                                                  \
  do {                                                                                                                \
    static bool done[64] = {};                                                                                        \
    if (smem > 48 * 1024) {                                                                                           \
      const int rc = allow_dynamic_smem(latent_attention_kernel<TI, NACC>, 200 * 1024, done);                         \
      if (rc) return rc;                                                                                              \
    }                                                                                                                 \
    return launch_ex(latent_attention_kernel<TI, NACC>, grid, block, (size_t)smem, s, 1, (const TI*)qfull,            \
                     (const TI*)cache, (TI*)out, token_seq, positions, block_table, bt_stride, H, rank, dk, page_size, \
                     scale, window);                                                                                  \
  } while (0)
#define BY_RANK(TI)                                                                                                   \
  do {                                                                                                                \
    if (rank <= 64) GO(TI, 2);                                                                                        \
    if (rank <= 128) GO(TI, 4);                                                                                       \
    if (rank <= 256) GO(TI, 8);                                                                                       \
    if (rank <= 512) GO(TI, 16);                                                                                      \
    GO(TI, 32);                                                                                                       \
  } while (0)
  if (dt == DT_F32) BY_RANK(float);
  if (dt == DT_BF16) BY_RANK(bf16);
#undef BY_RANK
#undef GO
  return ERR_BAD_DTYPE;
}
