// Gated linear attention as a recurrence over a per-request state, float arithmetic throughout.
//
// Per head, with key channels k < dim and value columns v < vdim:
//   alpha_t[k] = sigmoid(z_t[k] + b[k]) ^ (1 / tau)          computed as exp(logsigmoid(.) / tau)   (gla_decay)
//   S_t[k, v]  = alpha_t[k] * S_(t-1)[k, v] + key_t[k] * value_t[v]
//   o_t[v]     = sum_k S_t[k, v] * (query_t[k] * qscale)
// The state S lives in float in a slot per request and is carried from step to step; a step brings any
// number of tokens of a sequence (a prompt portion or one decoded token).
//
// gla_scan (mode WHOLE): one CTA per (sequence, head, 32 value columns); the four warps split the key
//   channels, a lane owns a value column and keeps its share of S in registers while it walks the sequence's
//   tokens, sixteen at a time through shared memory. The four warps' partial sums of o are added in warp order.
//   A position's result is the same bits whether its tokens came one by one or in portions.
// Long portions (the caller decides by the longest portion of the step) are cut into chunks of `chunk` tokens
//   that run side by side, which the recurrence allows because it is linear in S: with A_c the product of
//   a chunk's alphas and B_c the state the chunk builds from zero, S_end = diag(A_c) S_start + B_c.
//   Pass LOCAL computes A_c and B_c per chunk, gla_carry walks the chunks of a sequence once
//   (S_start of each chunk, the final state into the slot), pass FINAL runs each chunk again from its
//   S_start and writes the outputs. Twice the arithmetic, chunks-fold the parallelism; sums are grouped
//   differently than token by token, within float rounding.
// gla_finish: one warp per (token, head): o / sqrt(mean(o^2) + eps) * w over vdim, times silu(gate).
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int CH = 16;           // tokens staged at a time, at most (8 for heads of more than 128 key channels)
constexpr int MAX_DIM = 256;     // key channels per head
enum : int { WHOLE = 0, LOCAL = 1, FINAL = 2 };

__global__ void gla_decay_kernel(float* __restrict__ z, const float* __restrict__ bias, int n, long long total,
                                 float inv_tau) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float zz = z[i] + bias[i % n];
    const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));      // ln sigmoid(zz)
    z[i] = expf(ls * inv_tau);
  }
}

// Which sequence and which of its chunks a CTA of a chunked pass has; false: none.
__device__ __forceinline__ bool find_chunk(const int* cu_q, int num_seqs, int chunk, int b, int& seq, int& c, int& base) {
  int at = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int n = (cu_q[s + 1] - cu_q[s] + chunk - 1) / chunk;
    if (b < at + n) { seq = s; c = b - at; base = at; return true; }
    at += n;
  }
  return false;
}

template <typename TI, int KP, int MODE>   // KP: state registers a thread, 4 * KP >= dim
__global__ void __launch_bounds__(128)
gla_scan_kernel(const TI* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                const float* __restrict__ alpha, float qscale, int H, int dim, int vdim,
                const int* __restrict__ cu_q, int num_seqs, const int* __restrict__ state_slots,
                float* __restrict__ state, float* __restrict__ out, int chunk, float* __restrict__ chunk_state,
                float* __restrict__ chunk_decay, int ch) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) float staged[];              // queries, keys, decays: [ch][dimp] each
  __shared__ float vs[CH][32];
  __shared__ float part[CH][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, v = blockIdx.z * 32 + lane;
  int seq = blockIdx.x, c = 0, base = 0;
  if (MODE != WHOLE && !find_chunk(cu_q, num_seqs, chunk, blockIdx.x, seq, c, base)) return;
  int row0 = cu_q[seq], row1 = cu_q[seq + 1];
  if (MODE != WHOLE) { row0 += c * chunk; row1 = min(row1, row0 + chunk); }
  const int slot = (MODE == WHOLE && state_slots) ? state_slots[seq] : -1;
  const int dimp = (dim + 3) & ~3;               // a staged row, padded to 16 bytes
  float* qs = staged;
  float* ks = qs + ch * dimp;
  float* as = ks + ch * dimp;
  const int kp = (dim + 3) / 4;                  // key channels of a warp
  const int kbase = warp * kp;
  const bool vok = v < vdim;
  const bool vec = kp % 4 == 0 && dim % 4 == 0 && 4 * kp == dim;       // every warp has kp whole channels, in fours
  float S[KP], A[MODE == LOCAL ? KP : 1];
  // where this thread's share of a state lies: the request's slot, or the chunk's place in the scratch
  float* sp = (MODE == WHOLE ? state + ((long long)(slot < 0 ? 0 : slot) * H + h) * dim * vdim
                             : chunk_state + ((long long)(base + c) * H + h) * dim * vdim) + v;
#pragma unroll
  for (int i = 0; i < KP; ++i) {
    const int k = kbase + i;
    const bool mine = vok && i < kp && k < dim;
    S[i] = ((MODE == WHOLE ? slot >= 0 : MODE == FINAL) && mine) ? sp[(long long)k * vdim] : 0.f;
    if (MODE == LOCAL) A[i] = 1.f;
  }
  // bfloat16 rows whose pieces of 8 channels are 16-byte aligned are staged 8 channels a load
  const bool wide = sizeof(TI) == 2 && dim % 8 == 0 && ld % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 &&
                    !((uintptr_t)proj & 15) && !((uintptr_t)alpha & 15);
  for (int c0 = row0; c0 < row1; c0 += ch) {
    const int n = min(ch, row1 - c0);
    if (wide) {
      const int per = dim >> 3;
      for (int x = threadIdx.x; x < n * per; x += 128) {
        const int cc = x / per, k = (x % per) * 8;
        const TI* r = proj + (long long)(c0 + cc) * ld;
        const float4* ap = reinterpret_cast<const float4*>(alpha + (long long)(c0 + cc) * H * dim + h * dim + k);
        const uint4 kq = *reinterpret_cast<const uint4*>(r + k_off + h * dim + k);
        const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kq);
        float* kd = ks + cc * dimp + k;
        float* ad = as + cc * dimp + k;
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(kh[e]); kd[2 * e] = f.x; kd[2 * e + 1] = f.y; }
        *reinterpret_cast<float4*>(ad) = ap[0];
        *reinterpret_cast<float4*>(ad + 4) = ap[1];
        if (MODE != LOCAL) {
          const uint4 qq = *reinterpret_cast<const uint4*>(r + q_off + h * dim + k);
          const __nv_bfloat162* qh = reinterpret_cast<const __nv_bfloat162*>(&qq);
          float* qd = qs + cc * dimp + k;
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(qh[e]); qd[2 * e] = f.x * qscale; qd[2 * e + 1] = f.y * qscale; }
        }
      }
    } else {
      for (int x = threadIdx.x; x < n * dim; x += 128) {
        const int cc = x / dim, k = x % dim;
        const TI* r = proj + (long long)(c0 + cc) * ld;
        if (MODE != LOCAL) qs[cc * dimp + k] = to_f32(r[q_off + h * dim + k]) * qscale;
        ks[cc * dimp + k] = to_f32(r[k_off + h * dim + k]);
        as[cc * dimp + k] = alpha[(long long)(c0 + cc) * H * dim + h * dim + k];
      }
    }
    for (int x = threadIdx.x; x < n * 32; x += 128) {
      const int cc = x >> 5, j = x & 31;
      const int vv = blockIdx.z * 32 + j;
      vs[cc][j] = vv < vdim ? to_f32(proj[(long long)(c0 + cc) * ld + v_off + h * vdim + vv]) : 0.f;
    }
    __syncthreads();
    if (vec) {
      // a warp's key channels are a multiple of 4: decays, keys and queries come four at a time
      for (int cc = 0; cc < n; ++cc) {
        const float val = vs[cc][lane];
        const float4* a4 = reinterpret_cast<const float4*>(as + cc * dimp + kbase);
        const float4* k4 = reinterpret_cast<const float4*>(ks + cc * dimp + kbase);
        const float4* q4 = reinterpret_cast<const float4*>(qs + cc * dimp + kbase);
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < KP; i += 4) {
          if (i < kp) {
            const float4 a = a4[i >> 2], kk = k4[i >> 2];
            S[i] = fmaf(a.x, S[i], kk.x * val); S[i + 1] = fmaf(a.y, S[i + 1], kk.y * val);
            S[i + 2] = fmaf(a.z, S[i + 2], kk.z * val); S[i + 3] = fmaf(a.w, S[i + 3], kk.w * val);
            if (MODE == LOCAL) { A[i] *= a.x; A[i + 1] *= a.y; A[i + 2] *= a.z; A[i + 3] *= a.w; }
            else {
              const float4 q = q4[i >> 2];
              o = fmaf(S[i], q.x, o); o = fmaf(S[i + 1], q.y, o); o = fmaf(S[i + 2], q.z, o); o = fmaf(S[i + 3], q.w, o);
            }
          }
        }
        if (MODE != LOCAL) part[cc][warp][lane] = o;
      }
    } else {
      for (int cc = 0; cc < n; ++cc) {
        const float val = vs[cc][lane];
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < KP; ++i) {
          const int k = kbase + i;
          if (i < kp && k < dim) {
            S[i] = fmaf(as[cc * dimp + k], S[i], ks[cc * dimp + k] * val);
            if (MODE == LOCAL) A[i] *= as[cc * dimp + k];
            else o = fmaf(S[i], qs[cc * dimp + k], o);
          }
        }
        if (MODE != LOCAL) part[cc][warp][lane] = o;
      }
    }
    __syncthreads();
    if (MODE != LOCAL)
      for (int x = threadIdx.x; x < n * 32; x += 128) {
        const int cc = x >> 5, j = x & 31;
        const int vv = blockIdx.z * 32 + j;
        if (vv < vdim)
          out[((long long)(c0 + cc) * H + h) * vdim + vv] = ((part[cc][0][j] + part[cc][1][j]) + part[cc][2][j]) + part[cc][3][j];
      }
  }
  if (MODE != FINAL && vok && !(MODE == WHOLE && slot < 0)) {
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      const int k = kbase + i;
      if (i < kp && k < dim) {
        sp[(long long)k * vdim] = S[i];
        if (MODE == LOCAL && blockIdx.z == 0 && lane == 0) chunk_decay[((long long)(base + c) * H + h) * dim + k] = A[i];
      }
    }
  }
}

// One thread per state element of a (sequence, head): S walks the sequence's chunks; chunk_state[c] turns from
// B_c into the state the chunk starts from, and the slot gets the state after the last chunk.
__global__ void gla_carry_kernel(const int* __restrict__ cu_q, const int* __restrict__ state_slots,
                                 float* __restrict__ state, float* __restrict__ chunk_state,
                                 const float* __restrict__ chunk_decay, int chunk, int H, int dim, int vdim) {
  pdl_launch();
  pdl_wait();
  const int seq = blockIdx.x, h = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (e >= dim * vdim) return;
  int base = 0;
  for (int s = 0; s < seq; ++s) base += (cu_q[s + 1] - cu_q[s] + chunk - 1) / chunk;
  const int n = (cu_q[seq + 1] - cu_q[seq] + chunk - 1) / chunk;
  const int slot = state_slots ? state_slots[seq] : -1;
  float* sp = state + ((long long)(slot < 0 ? 0 : slot) * H + h) * dim * vdim + e;
  float S = slot >= 0 ? *sp : 0.f;
  const int k = e / vdim;
  float* b = chunk_state + ((long long)base * H + h) * dim * vdim + e;
  const float* d = chunk_decay + ((long long)base * H + h) * dim + k;
  const long long bstep = (long long)H * dim * vdim, dstep = (long long)H * dim;
  float bc = n > 0 ? *b : 0.f, dc = n > 0 ? *d : 0.f;
  for (int c = 0; c < n; ++c) {
    float bn = 0.f, dn = 0.f;
    if (c + 1 < n) { bn = b[bstep]; dn = d[dstep]; }                   // the next chunk's, asked for ahead
    *b = S;
    S = fmaf(dc, S, bc);
    bc = bn; dc = dn; b += bstep; d += dstep;
  }
  if (slot >= 0) *sp = S;
}

template <typename TI>
__global__ void __launch_bounds__(128)
gla_finish_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, const TI* __restrict__ proj,
                  long long ld, int g_off, int T, int H, int vdim, TI* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long x = (long long)blockIdx.x * 4 + warp;
  if (x >= (long long)T * H) return;
  const int t = (int)(x / H), h = (int)(x % H);
  const float* orow = o + x * vdim;
  float ss = 0.f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(orow[i], orow[i], ss);
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)vdim + eps);
  const TI* g = proj + (long long)t * ld + g_off + h * vdim;
  TI* dst = out + x * vdim;
  for (int i = lane; i < vdim; i += 32) {
    const float gv = to_f32(g[i]);
    dst[i] = from_f32<TI>(orow[i] * r * w[i] * (gv / (1.f + expf(-gv))));
  }
}

template <typename TI, int MODE>
int scan(dim3 grid, cudaStream_t s, const void* proj, long long ld, int q_off, int k_off, int v_off, const float* alpha,
         float qscale, int H, int dim, int vdim, const int* cu_q, int num_seqs, const int* state_slots, float* state,
         float* out, int chunk, float* chunk_state, float* chunk_decay, int T) {
  const int kp = (dim + 3) / 4;
  // tokens staged at a time: 16 (8 for wide heads), 2 for steps of single tokens (the room goes to more CTAs an SM)
  const int ch = T <= 2 * num_seqs ? 2 : (dim <= 128 ? CH : CH / 2);
  const size_t smem = (size_t)3 * ch * ((dim + 3) & ~3) * sizeof(float);                             // at most 24 KB
#define GO(KP)                                                                                                        \
  return launch_ex(gla_scan_kernel<TI, KP, MODE>, grid, dim3(128), smem, s, 1, (const TI*)proj, ld, q_off, k_off, v_off, \
                   alpha, qscale, H, dim, vdim, cu_q, num_seqs, state_slots, state, out, chunk, chunk_state, chunk_decay, ch)
  if (kp <= 8) GO(8);
  if (kp <= 16) GO(16);
  if (kp <= 32) GO(32);
  GO(64);
#undef GO
}

}  // namespace

// z float [T, n] (n = H * dim) becomes the decays in place: exp(logsigmoid(z + bias) / tau).
RLLM_API int rllm_gla_decay(float* z, const float* bias, int T, int n, float tau, void* stream) {
  if (T <= 0 || n <= 0) return 0;
  if (!(tau > 0.f)) return ERR_BAD_SIZE;
  const long long total = (long long)T * n;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  return launch_ex(gla_decay_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, 1, z, bias, n, total, 1.f / tau);
}

// proj [T, ld] (storage type): queries at q_off, keys at k_off (H x dim each), values at v_off (H x vdim).
// alpha float [T, H * dim]: the decays. cu_q [S + 1]: row range of each sequence; state_slots [S] (-1: the state
// starts at zero and is not kept). state float [slots, H, dim, vdim]. out float [T, H, vdim].
// chunk <= 0: every sequence's rows in one CTA per (head, 32 columns). chunk > 0: the three passes over chunks of
// that many tokens; chunk_state: float [T / chunk + S, H, dim, vdim], chunk_decay: float [T / chunk + S, H, dim].
RLLM_API int rllm_gla_scan(int dt, const void* proj, long long ld, int q_off, int k_off, int v_off, const float* alpha,
                           float qscale, int T, int S, int H, int dim, int vdim, const int* cu_q,
                           const int* state_slots, float* state, float* out, int chunk, float* chunk_state,
                           float* chunk_decay, void* stream) {
  if (S <= 0 || T <= 0) return 0;
  if (H <= 0 || dim <= 0 || dim > MAX_DIM || vdim <= 0) return ERR_BAD_SIZE;
  if (H > 65535 || (vdim + 31) / 32 > 65535) return ERR_TOO_LARGE;
  if (dt != DT_F32 && dt != DT_BF16) return ERR_BAD_DTYPE;
  cudaStream_t s = (cudaStream_t)stream;
  const int vb = (vdim + 31) / 32;
#define SCAN(MODE, GRID)                                                                                            \
  (dt == DT_F32 ? scan<float, MODE>(GRID, s, proj, ld, q_off, k_off, v_off, alpha, qscale, H, dim, vdim, cu_q, S,   \
                                    state_slots, state, out, chunk, chunk_state, chunk_decay, T)                    \
                : scan<bf16, MODE>(GRID, s, proj, ld, q_off, k_off, v_off, alpha, qscale, H, dim, vdim, cu_q, S,    \
                                   state_slots, state, out, chunk, chunk_state, chunk_decay, T))
  if (chunk <= 0) return SCAN(WHOLE, dim3(S, H, vb));
  if (!chunk_state || !chunk_decay) return ERR_BAD_SIZE;
  const int chunks = T / chunk + S;                                  // at least as many as the sequences have
  int rc = SCAN(LOCAL, dim3(chunks, H, vb));
  if (rc) return rc;
  const int per = dim * vdim;
  rc = launch_ex(gla_carry_kernel, dim3(S, H, (per + 255) / 256), dim3(256), 0, s, 1, cu_q, state_slots, state,
                 chunk_state, (const float*)chunk_decay, chunk, H, dim, vdim);
  if (rc) return rc;
  return SCAN(FINAL, dim3(chunks, H, vb));
#undef SCAN
}

// o float [T, H, vdim]; w float [vdim]; gate in proj at g_off (H x vdim, storage type); out [T, H * vdim].
RLLM_API int rllm_gla_finish(int dt, const float* o, const float* w, float eps, const void* proj, long long ld,
                             int g_off, int T, int H, int vdim, void* out, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || vdim <= 0) return ERR_BAD_SIZE;
  const long long blocks = ((long long)T * H + 3) / 4;
  if (blocks > 2147483647LL) return ERR_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32)
    return launch_ex(gla_finish_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, s, 1, o, w, eps, (const float*)proj,
                     ld, g_off, T, H, vdim, (float*)out);
  if (dt == DT_BF16)
    return launch_ex(gla_finish_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, s, 1, o, w, eps, (const bf16*)proj, ld,
                     g_off, T, H, vdim, (bf16*)out);
  return ERR_BAD_DTYPE;
}
