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

// ------------------------------------------------------------------------------------------ tensor cores
// bfloat16, dk a multiple of 8, rank a multiple of 16 up to 512. The rows of the problem are the (token, head)
// pairs of a sequence's new tokens, 64 to a CTA: since all heads read the same cache rows, the heads of a
// single decoded token fill a row tile of the tensor core as well as the tokens of a prompt portion do. Keys
// come 32 at a time through two buffers (`cp.async` through the block table); eight warps = four groups of 16
// rows x two halves: for the scores each half takes 16 of the 32 keys (QK^T over dk with `mma.sync` m16n8k16,
// scaled, masked per row by its own position and window, left in shared memory as float), then both halves
// run the same float softmax update over the 32 scores of their rows and each multiplies the bfloat16 weights
// with its half of the value columns (the cache row's first `rank` numbers, read with `ldmatrix.trans`).
// Key tiles begin at the first key that the CTA's first row sees, so where a row's keys fall into tiles, and with it
// the order of its sums, depends on which rows share its CTA: results differ between cuts of a prompt within
// bfloat16 rounding (the float path below has one order per position).
constexpr int QROWS = 64, KT = 32;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix4t(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}

static inline int mma_row_pad(int dk, int nh) {          // numbers per shared-memory row: what ldmatrix may touch, + 8
  const int a = (dk + 15) / 16 * 16, b = 2 * nh * 8;
  return (a > b ? a : b) + 8;
}

template <int NH>     // value columns per half = 8 * NH; rank <= 16 * NH
__global__ void __launch_bounds__(256, 1)
latent_attention_mma_kernel(const bf16* __restrict__ qfull, const bf16* __restrict__ cache, bf16* __restrict__ out,
                            const int* __restrict__ cu_q, const int* __restrict__ positions,
                            const int* __restrict__ block_table, int bt_stride, int num_seqs, int H, int rank, int dk,
                            int ld, int page_size, float scale, int window, int splits, float* __restrict__ pacc,
                            float* __restrict__ pml) {
  pdl_launch();
  pdl_wait();
  // which sequence and which 64 of its (token, head) rows
  int seq = -1, tile = 0;
  {
    int at = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = ((cu_q[s + 1] - cu_q[s]) * H + QROWS - 1) / QROWS;
      if ((int)blockIdx.x < at + n) { seq = s; tile = blockIdx.x - at; break; }
      at += n;
    }
  }
  if (seq < 0) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                      // [64][ld]
  bf16* ks = qs + QROWS * ld;                                        // [2][32][ld]
  float* ss = reinterpret_cast<float*>(ks + 2 * KT * ld);            // [64][33]
  __shared__ int key_ok[2][KT];
  __shared__ int krow[KT];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp >> 1, half = warp & 1;                         // 16 rows each, two halves
  const int tok0 = cu_q[seq], ntok = cu_q[seq + 1] - tok0;
  const int row_first = tile * QROWS, nrows = min(QROWS, ntok * H - row_first);
  const int t_lo = tok0 + row_first / H, t_hi = tok0 + (row_first + nrows - 1) / H;
  const int pos_lo = positions[t_lo], pos_hi = positions[t_hi];
  const int key_first = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
  const int ntiles = (pos_hi - key_first) / KT + 1;
  // with `splits` > 1 (steps of few rows: decoding) the key tiles are dealt out to that many CTAs, which leave
  // their unnormalised sums, maxima and weights' sums for latent_merge_kernel
  const int per_split = (ntiles + splits - 1) / splits;
  const int it0 = blockIdx.y * per_split, it1 = min(ntiles, it0 + per_split);
  const int* bt = block_table + (long long)seq * bt_stride;
  const int cpr = (ld - 8) / 8;                                      // 16-byte pieces a row is filled with
  if (it0 >= it1) {                                                  // no tile left for this CTA: it says so and goes
    for (int r = tid; r < QROWS; r += 256) {
      float* ml = pml + (((long long)blockIdx.x * splits + blockIdx.y) * QROWS + r) * 2;
      ml[0] = -INFINITY; ml[1] = 0.f;
    }
    return;
  }

  // where the next tile's keys lie: one lane a key looks its page up (row of the cache, -1: no such key),
  // before the barrier that lets all warps copy the tile
  auto find_keys = [&](int it) {
    if (tid < KT) {
      const int kj = key_first + it * KT + tid;
      const int page = kj <= pos_hi ? bt[kj / page_size] : -1;
      krow[tid] = page >= 0 ? page * page_size + kj % page_size : -1;
    }
  };
  // a warp copies four keys of the tile, its lanes the 16-byte pieces of a row
  auto load_keys = [&](int it) {
    bf16* dst = ks + ((it - it0) & 1) * KT * ld;
#pragma unroll
    for (int i = 0; i < KT / 8; ++i) {
      const int j = warp + i * 8;
      const int row = krow[j];
      if (lane == 0) key_ok[(it - it0) & 1][j] = row >= 0;
      const bf16* src = cache + (long long)(row < 0 ? 0 : row) * dk;
      for (int piece = lane; piece < cpr; piece += 32) {
        const bool in = row >= 0 && piece * 8 < dk;
        cp_async16(dst + j * ld + piece * 8, src + (in ? piece * 8 : 0), in ? 16 : 0);
      }
    }
  };
  // the queries, once (rows beyond the sequence's: zeros)
  for (int c = tid; c < QROWS * cpr; c += 256) {
    const int r = c / cpr, piece = c % cpr;
    const bool in = r < nrows && piece * 8 < dk;
    cp_async16(qs + r * ld + piece * 8, qfull + (in ? ((long long)tok0 * H + row_first + r) * dk + piece * 8 : 0), in ? 16 : 0);
  }
  find_keys(it0);
  __syncthreads();
  load_keys(it0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  // this thread's two rows (of its warp's 16): their positions and first visible keys
  const int r0 = rg * 16 + (lane >> 2), r1 = r0 + 8;
  int pos0 = -1, pos1 = -1, lo0 = 0, lo1 = 0;
  if (r0 < nrows) { pos0 = positions[tok0 + (row_first + r0) / H]; lo0 = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0; }
  if (r1 < nrows) { pos1 = positions[tok0 + (row_first + r1) / H]; lo1 = (window > 0 && pos1 - window + 1 > 0) ? pos1 - window + 1 : 0; }
  const bool rg_live = rg * 16 < nrows;
  float acc[NH][4];
#pragma unroll
  for (int n = 0; n < NH; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int dk16 = (dk + 15) / 16;

  for (int it = it0; it < it1; ++it) {
    if (it + 1 < it1) find_keys(it + 1);                             // krow was last read before the barrier before
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                                 // tile `it` has landed; tile it - 1 is used up
    if (it + 1 < it1) load_keys(it + 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bf16* kt = ks + ((it - it0) & 1) * KT * ld;
    const int kbase = key_first + it * KT;
    if (rg_live) {
      // scores of this warp's 16 rows against its 16 keys
      float sc[2][4] = {};
#pragma unroll 2
      for (int kk = 0; kk < dk16; ++kk) {
        unsigned a[4], b[4];
        ldmatrix4(a, qs + (rg * 16 + (lane & 15)) * ld + kk * 16 + (lane >> 4) * 8);
        ldmatrix4(b, kt + (half * 16 + (lane & 7) + ((lane >> 4) << 3)) * ld + kk * 16 + ((lane >> 3) & 1) * 8);
        mma16816(sc[0], a, b[0], b[1]);
        mma16816(sc[1], a, b[2], b[3]);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = half * 16 + j * 8 + (lane & 3) * 2 + (e & 1);
          const int kj = kbase + col;
          const bool top = e < 2;
          const bool seen = key_ok[(it - it0) & 1][col] && (top ? (kj >= lo0 && kj <= pos0) : (kj >= lo1 && kj <= pos1));
          ss[(top ? r0 : r1) * (KT + 1) + col] = seen ? sc[j][e] * scale : -INFINITY;
        }
    }
    __syncthreads();
    if (rg_live) {
      // softmax update of rows r0 and r1 over the tile's 32 scores (this lane holds 8 of each row)
      float p0[8], p1[8];
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int col = (q >> 1) * 8 + (lane & 3) * 2 + (q & 1);
        p0[q] = ss[r0 * (KT + 1) + col]; p1[q] = ss[r1 * (KT + 1) + col];
        mx0 = fmaxf(mx0, p0[q]); mx1 = fmaxf(mx1, p1[q]);
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float b0 = n0 == -INFINITY ? 0.f : n0, b1 = n1 == -INFINITY ? 0.f : n1;     // a row that has seen nothing yet
      const float c0 = expf(m0 - b0), c1 = expf(m1 - b1);            // m = -inf: 0
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) { p0[q] = expf(p0[q] - b0); p1[q] = expf(p1[q] - b1); s0 += p0[q]; s1 += p1[q]; }
      s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      l0 = l0 * c0 + s0; l1 = l1 * c1 + s1; m0 = n0; m1 = n1;
#pragma unroll
      for (int n = 0; n < NH; ++n) { acc[n][0] *= c0; acc[n][1] *= c0; acc[n][2] *= c1; acc[n][3] *= c1; }
      // weights as the A operand: keys kk*16 + 2*(lane%4) + {0,1} and + 8
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        unsigned a[4] = {pack_bf16(p0[kk * 4], p0[kk * 4 + 1]), pack_bf16(p1[kk * 4], p1[kk * 4 + 1]),
                         pack_bf16(p0[kk * 4 + 2], p0[kk * 4 + 3]), pack_bf16(p1[kk * 4 + 2], p1[kk * 4 + 3])};
#pragma unroll
        for (int n = 0; n < NH; n += 2) {
          unsigned b[4];
          ldmatrix4t(b, kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + half * NH * 8 + n * 8 + (lane >> 4) * 8);
          mma16816(acc[n], a, b[0], b[1]);
          mma16816(acc[n + 1], a, b[2], b[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (splits > 1) {
    const long long pb = ((long long)blockIdx.x * splits + blockIdx.y) * QROWS;
    if (!rg_live) {                                                  // rows nobody computed: marked empty
      if (half == 0 && (lane & 3) == 0) { pml[(pb + r0) * 2] = -INFINITY; pml[(pb + r0) * 2 + 1] = 0.f;
                                          pml[(pb + r1) * 2] = -INFINITY; pml[(pb + r1) * 2 + 1] = 0.f; }
      return;
    }
    if (half == 0 && (lane & 3) == 0) { pml[(pb + r0) * 2] = m0; pml[(pb + r0) * 2 + 1] = l0;
                                        pml[(pb + r1) * 2] = m1; pml[(pb + r1) * 2 + 1] = l1; }
#pragma unroll
    for (int n = 0; n < NH; ++n) {
      const int col = half * NH * 8 + n * 8 + (lane & 3) * 2;
      if (col >= rank) continue;
      *reinterpret_cast<float2*>(pacc + (pb + r0) * rank + col) = make_float2(acc[n][0], acc[n][1]);
      *reinterpret_cast<float2*>(pacc + (pb + r1) * rank + col) = make_float2(acc[n][2], acc[n][3]);
    }
    return;
  }
  if (!rg_live) return;
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  bf16* o0 = out + ((long long)tok0 * H + row_first + r0) * rank;
  bf16* o1 = out + ((long long)tok0 * H + row_first + r1) * rank;
#pragma unroll
  for (int n = 0; n < NH; ++n) {
    const int col = half * NH * 8 + n * 8 + (lane & 3) * 2;
    if (col >= rank) continue;                                       // rank is even: a pair is in or out
    if (r0 < nrows) *reinterpret_cast<__nv_bfloat162*>(o0 + col) = __floats2bfloat162_rn(acc[n][0] * i0, acc[n][1] * i0);
    if (r1 < nrows) *reinterpret_cast<__nv_bfloat162*>(o1 + col) = __floats2bfloat162_rn(acc[n][2] * i1, acc[n][3] * i1);
  }
}

// The few-rows shape of the kernel above (steps that bring a token or two per sequence): 16 rows a CTA, so that the
// heads of one decoded token are a row tile by themselves; keys 64 at a time through two buffers. All eight warps
// work on the one row tile: for the scores each takes 8 of the 64 keys, then every warp runs the float softmax
// update of the 16 rows (the same numbers in each) and multiplies the weights with its eighth of the value columns.
// rank a multiple of 128 (NW = rank / 64 column tiles of 8 a warp).
constexpr int FROWS = 16, FKT = 64;

template <int NW>
__global__ void __launch_bounds__(256, 1)
latent_attention_few_kernel(const bf16* __restrict__ qfull, const bf16* __restrict__ cache, bf16* __restrict__ out,
                            const int* __restrict__ cu_q, const int* __restrict__ positions,
                            const int* __restrict__ block_table, int bt_stride, int num_seqs, int H, int rank, int dk,
                            int ld, int page_size, float scale, int window, int splits, float* __restrict__ pacc,
                            float* __restrict__ pml) {
  pdl_launch();
  pdl_wait();
  int seq = -1, tile = 0;
  {
    int at = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = ((cu_q[s + 1] - cu_q[s]) * H + FROWS - 1) / FROWS;
      if ((int)blockIdx.x < at + n) { seq = s; tile = blockIdx.x - at; break; }
      at += n;
    }
  }
  if (seq < 0) return;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                      // [16][ld]
  bf16* ks = qs + FROWS * ld;                                        // [2][64][ld]
  float* ss = reinterpret_cast<float*>(ks + 2 * FKT * ld);           // [16][65]
  __shared__ int key_ok[2][FKT];
  __shared__ int krow[FKT];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tok0 = cu_q[seq], ntok = cu_q[seq + 1] - tok0;
  const int row_first = tile * FROWS, nrows = min(FROWS, ntok * H - row_first);
  const int t_lo = tok0 + row_first / H, t_hi = tok0 + (row_first + nrows - 1) / H;
  const int pos_lo = positions[t_lo], pos_hi = positions[t_hi];
  const int key_first = (window > 0 && pos_lo - window + 1 > 0) ? pos_lo - window + 1 : 0;
  const int ntiles = (pos_hi - key_first) / FKT + 1;
  const int per_split = (ntiles + splits - 1) / splits;
  const int it0 = blockIdx.y * per_split, it1 = min(ntiles, it0 + per_split);
  const int* bt = block_table + (long long)seq * bt_stride;
  const int cpr = (ld - 8) / 8;
  const long long pb = ((long long)blockIdx.x * splits + blockIdx.y) * FROWS;
  if (it0 >= it1) {
    if (tid < FROWS) { pml[(pb + tid) * 2] = -INFINITY; pml[(pb + tid) * 2 + 1] = 0.f; }
    return;
  }
  auto find_keys = [&](int it) {
    if (tid < FKT) {
      const int kj = key_first + it * FKT + tid;
      const int page = kj <= pos_hi ? bt[kj / page_size] : -1;
      krow[tid] = page >= 0 ? page * page_size + kj % page_size : -1;
    }
  };
  auto load_keys = [&](int it) {
    bf16* dst = ks + ((it - it0) & 1) * FKT * ld;
#pragma unroll
    for (int i = 0; i < FKT / 8; ++i) {
      const int j = warp + i * 8;
      const int row = krow[j];
      if (lane == 0) key_ok[(it - it0) & 1][j] = row >= 0;
      const bf16* src = cache + (long long)(row < 0 ? 0 : row) * dk;
      for (int piece = lane; piece < cpr; piece += 32) {
        const bool in = row >= 0 && piece * 8 < dk;
        cp_async16(dst + j * ld + piece * 8, src + (in ? piece * 8 : 0), in ? 16 : 0);
      }
    }
  };
  for (int c = tid; c < FROWS * cpr; c += 256) {
    const int r = c / cpr, piece = c % cpr;
    const bool in = r < nrows && piece * 8 < dk;
    cp_async16(qs + r * ld + piece * 8, qfull + (in ? ((long long)tok0 * H + row_first + r) * dk + piece * 8 : 0), in ? 16 : 0);
  }
  find_keys(it0);
  __syncthreads();
  load_keys(it0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  const int r0 = lane >> 2, r1 = r0 + 8;
  int pos0 = -1, pos1 = -1, lo0 = 0, lo1 = 0;
  if (r0 < nrows) { pos0 = positions[tok0 + (row_first + r0) / H]; lo0 = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0; }
  if (r1 < nrows) { pos1 = positions[tok0 + (row_first + r1) / H]; lo1 = (window > 0 && pos1 - window + 1 > 0) ? pos1 - window + 1 : 0; }
  float acc[NW][4];
#pragma unroll
  for (int n = 0; n < NW; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int dk16 = (dk + 15) / 16;

  for (int it = it0; it < it1; ++it) {
    if (it + 1 < it1) find_keys(it + 1);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (it + 1 < it1) load_keys(it + 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bf16* kt = ks + ((it - it0) & 1) * FKT * ld;
    const int kbase = key_first + it * FKT;
    {
      // scores of the 16 rows against this warp's 8 keys
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int kk = 0; kk < dk16; ++kk) {
        unsigned a[4], b[4];
        ldmatrix4(a, qs + (lane & 15) * ld + kk * 16 + (lane >> 4) * 8);
        // x4 over 8 keys x 32 of K would be two steps at once; keep to one step: lanes 16..31 repeat the addresses
        ldmatrix4(b, kt + (warp * 8 + (lane & 7)) * ld + kk * 16 + ((lane >> 3) & 1) * 8);
        mma16816(sc, a, b[0], b[1]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = warp * 8 + (lane & 3) * 2 + (e & 1);
        const int kj = kbase + col;
        const bool top = e < 2;
        const bool seen = key_ok[(it - it0) & 1][col] && (top ? (kj >= lo0 && kj <= pos0) : (kj >= lo1 && kj <= pos1));
        ss[(top ? r0 : r1) * (FKT + 1) + col] = seen ? sc[e] * scale : -INFINITY;
      }
    }
    __syncthreads();
    {
      float p0[16], p1[16];
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        const int col = (q >> 1) * 8 + (lane & 3) * 2 + (q & 1);
        p0[q] = ss[r0 * (FKT + 1) + col]; p1[q] = ss[r1 * (FKT + 1) + col];
        mx0 = fmaxf(mx0, p0[q]); mx1 = fmaxf(mx1, p1[q]);
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
      const float b0 = n0 == -INFINITY ? 0.f : n0, b1 = n1 == -INFINITY ? 0.f : n1;
      const float c0 = expf(m0 - b0), c1 = expf(m1 - b1);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int q = 0; q < 16; ++q) { p0[q] = expf(p0[q] - b0); p1[q] = expf(p1[q] - b1); s0 += p0[q]; s1 += p1[q]; }
      s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      l0 = l0 * c0 + s0; l1 = l1 * c1 + s1; m0 = n0; m1 = n1;
#pragma unroll
      for (int n = 0; n < NW; ++n) { acc[n][0] *= c0; acc[n][1] *= c0; acc[n][2] *= c1; acc[n][3] *= c1; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        unsigned a[4] = {pack_bf16(p0[kk * 4], p0[kk * 4 + 1]), pack_bf16(p1[kk * 4], p1[kk * 4 + 1]),
                         pack_bf16(p0[kk * 4 + 2], p0[kk * 4 + 3]), pack_bf16(p1[kk * 4 + 2], p1[kk * 4 + 3])};
#pragma unroll
        for (int n = 0; n < NW; n += 2) {
          unsigned b[4];
          ldmatrix4t(b, kt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + warp * NW * 8 + n * 8 + (lane >> 4) * 8);
          mma16816(acc[n], a, b[0], b[1]);
          mma16816(acc[n + 1], a, b[2], b[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (splits > 1) {
    if (warp == 0 && (lane & 3) == 0) { pml[(pb + r0) * 2] = m0; pml[(pb + r0) * 2 + 1] = l0;
                                        pml[(pb + r1) * 2] = m1; pml[(pb + r1) * 2 + 1] = l1; }
#pragma unroll
    for (int n = 0; n < NW; ++n) {
      const int col = warp * NW * 8 + n * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(pacc + (pb + r0) * rank + col) = make_float2(acc[n][0], acc[n][1]);
      *reinterpret_cast<float2*>(pacc + (pb + r1) * rank + col) = make_float2(acc[n][2], acc[n][3]);
    }
    return;
  }
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  bf16* o0 = out + ((long long)tok0 * H + row_first + r0) * rank;
  bf16* o1 = out + ((long long)tok0 * H + row_first + r1) * rank;
#pragma unroll
  for (int n = 0; n < NW; ++n) {
    const int col = warp * NW * 8 + n * 8 + (lane & 3) * 2;
    if (r0 < nrows) *reinterpret_cast<__nv_bfloat162*>(o0 + col) = __floats2bfloat162_rn(acc[n][0] * i0, acc[n][1] * i0);
    if (r1 < nrows) *reinterpret_cast<__nv_bfloat162*>(o1 + col) = __floats2bfloat162_rn(acc[n][2] * i1, acc[n][3] * i1);
  }
}

// The splits' parts of every row, merged in split order: out = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s.
// grid.x: the row tiles (of `qrows` rows) as in the kernel that left the parts; grid.y: blocks of 32 columns; a
// warp takes rows, its lanes the columns, all splits' values asked for at once.
__global__ void __launch_bounds__(256)
latent_merge_kernel(const float* __restrict__ pacc, const float* __restrict__ pml, bf16* __restrict__ out,
                    const int* __restrict__ cu_q, int num_seqs, int H, int rank, int splits, int qrows) {
  pdl_launch();
  pdl_wait();
  int seq = -1, tile = 0;
  {
    int at = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = ((cu_q[s + 1] - cu_q[s]) * H + qrows - 1) / qrows;
      if ((int)blockIdx.x < at + n) { seq = s; tile = blockIdx.x - at; break; }
      at += n;
    }
  }
  if (seq < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tok0 = cu_q[seq], ntok = cu_q[seq + 1] - tok0;
  const int row_first = tile * qrows, nrows = min(qrows, ntok * H - row_first);
  const int col = blockIdx.y * 32 + lane;
  for (int r = warp; r < nrows; r += 8) {
    const long long pb = (long long)blockIdx.x * splits * qrows + r;
    const float m = lane < splits ? pml[(pb + (long long)lane * qrows) * 2] : -INFINITY;
    const float l = lane < splits ? pml[(pb + (long long)lane * qrows) * 2 + 1] : 0.f;
    const float M = warp_max(m);
    const float w = (m == -INFINITY) ? 0.f : expf(m - M);
    const float L = warp_sum(w * l);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float v[32];
#pragma unroll
    for (int s = 0; s < 32; ++s) {
      const float ws = __shfl_sync(0xffffffffu, w, s);
      v[s] = (s < splits && ws != 0.f && col < rank) ? ws * pacc[(pb + (long long)s * qrows) * rank + col] : 0.f;
    }
    float a = 0.f;
#pragma unroll
    for (int s = 0; s < 32; ++s) a += v[s];
    if (col < rank) out[((long long)tok0 * H + row_first + r) * rank + col] = __float2bfloat16_rn(a * inv);
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
// cu_q [num_seqs + 1] (row range of each sequence; null: the tensor-core kernel is not used), `tc` 0 forbids it.
// splits > 1 (tensor-core kernels only): the keys of every row tile are dealt out to that many CTAs; pacc: float
// [row tiles, splits, rows, rank], pml: float [row tiles, splits, rows, 2], rows = 64 a tile, or 16 with `few`
// (the shape for steps of a token or two per sequence; taken when rank is a multiple of 128), row tiles =
// ceil(T * H / rows) + num_seqs.
RLLM_API int rllm_latent_attention(int dt, const void* qfull, const void* cache, void* out, const int* token_seq,
                                   const int* positions, const int* block_table, int bt_stride, int T, int H, int rank,
                                   int dk, int page_size, float scale, int window, const int* cu_q, int num_seqs,
                                   int tc, int splits, int few, float* pacc, float* pml, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || rank <= 0 || rank > MAX_RANK || dk < rank || page_size <= 0) return ERR_BAD_SIZE;
  if (tc && dt == DT_BF16 && cu_q && num_seqs > 0 && dk % 8 == 0 && rank % 16 == 0 && rank <= 512 &&
      !((uintptr_t)qfull & 15) && !((uintptr_t)cache & 15) && !((uintptr_t)out & 3)) {
    if (splits < 1 || splits > 32 || (splits > 1 && (!pacc || !pml))) return ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (few && rank % 128 == 0) {
      // 16 rows a CTA: steps of a token or two per sequence
      const int nw = rank / 64;
      const int ld = mma_row_pad(dk, nw * 4);                        // 8 warps x nw tiles of 8 columns = rank
      const int smem = (FROWS + 2 * FKT) * ld * 2 + FROWS * (FKT + 1) * 4;
      const long long blocks = ((long long)T * H + FROWS - 1) / FROWS + num_seqs;
      if (smem <= 220 * 1024 && blocks <= 2147483647LL) {
#define GO(NW)                                                                                                          \
  do {                                                                                                                  \
    static bool done[64] = {};                                                                                          \
    const int rc = allow_dynamic_smem(latent_attention_few_kernel<NW>, 220 * 1024, done);                               \
    if (rc) return rc;                                                                                                  \
    const int rl = launch_ex(latent_attention_few_kernel<NW>, dim3((unsigned)blocks, splits), dim3(256), (size_t)smem,  \
                             s, 1, (const bf16*)qfull, (const bf16*)cache, (bf16*)out, cu_q, positions, block_table,    \
                             bt_stride, num_seqs, H, rank, dk, ld, page_size, scale, window, splits, pacc, pml);        \
    if (rl || splits == 1) return rl;                                                                                   \
    return launch_ex(latent_merge_kernel, dim3((unsigned)blocks, (rank + 31) / 32), dim3(256), 0, s, 1,                 \
                     (const float*)pacc, (const float*)pml, (bf16*)out, cu_q, num_seqs, H, rank, splits, FROWS);        \
  } while (0)
        if (nw == 2) GO(2);
        if (nw == 4) GO(4);
        if (nw == 8) GO(8);
#undef GO
      }
    }
    const int nh = rank <= 64 ? 4 : rank <= 128 ? 8 : rank <= 256 ? 16 : 32;
    const int ld = mma_row_pad(dk, nh);
    const int smem = (QROWS + 2 * KT) * ld * 2 + QROWS * (KT + 1) * 4;
    const long long blocks = ((long long)T * H + QROWS - 1) / QROWS + num_seqs;
    if (smem <= 220 * 1024 && blocks <= 2147483647LL) {
#define GO(NH)                                                                                                          \
  do {                                                                                                                  \
    static bool done[64] = {};                                                                                          \
    const int rc = allow_dynamic_smem(latent_attention_mma_kernel<NH>, 220 * 1024, done);                               \
    if (rc) return rc;                                                                                                  \
    const int rl = launch_ex(latent_attention_mma_kernel<NH>, dim3((unsigned)blocks, splits), dim3(256), (size_t)smem,  \
                             s, 1, (const bf16*)qfull, (const bf16*)cache, (bf16*)out, cu_q, positions, block_table,    \
                             bt_stride, num_seqs, H, rank, dk, ld, page_size, scale, window, splits, pacc, pml);        \
    if (rl || splits == 1) return rl;                                                                                   \
    return launch_ex(latent_merge_kernel, dim3((unsigned)blocks, (rank + 31) / 32), dim3(256), 0, s, 1,                 \
                     (const float*)pacc, (const float*)pml, (bf16*)out, cu_q, num_seqs, H, rank, splits, QROWS);        \
  } while (0)
      if (nh == 4) GO(4);
      if (nh == 8) GO(8);
      if (nh == 16) GO(16);
      GO(32);
#undef GO
    }
  }
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
