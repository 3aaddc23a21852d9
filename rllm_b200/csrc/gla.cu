// Gated linear attention as a recurrence over a per-request state, float arithmetic throughout.
//
// Per head, with key channels k < dim and value columns v < vdim:
//   alpha_t[k] = sigmoid(z_t[k] + b[k]) ^ (1 / tau)          computed as exp(logsigmoid(.) / tau)
//   S_t[k, v]  = alpha_t[k] * S_(t-1)[k, v] + key_t[k] * value_t[v]
//   o_t[v]     = sum_k S_t[k, v] * (query_t[k] * qscale)
// The state S lives in float in a slot per request and is carried from step to step; a step brings any
// number of tokens of a sequence (a prompt portion or one decoded token): the same kernel, the same order
// of every sum, so the result does not depend on how the tokens were cut into steps.
//
// gla_scan: one CTA per (sequence, head, 32 value columns); the four warps split the key channels, a lane
//   owns a value column and keeps its share of S in registers while it walks the sequence's tokens, eight
//   at a time through shared memory. The four warps' partial sums of o are added in warp order.
// gla_finish: one warp per (token, head): o / sqrt(mean(o^2) + eps) * w over vdim, times silu(gate).
#include "common.cuh"
using namespace rllm;

namespace {

constexpr int CH = 8;            // tokens staged at a time
constexpr int MAX_DIM = 256;     // key channels per head

template <typename TI, int KP>   // KP: state registers a thread, 4 * KP >= dim
__global__ void __launch_bounds__(128)
gla_scan_kernel(const TI* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, const float* __restrict__ z,
                const float* __restrict__ zbias, float inv_tau, float qscale, int H, int dim, int vdim,
                const int* __restrict__ cu_q, const int* __restrict__ state_slots, float* __restrict__ state,
                float* __restrict__ out) {
  pdl_launch();
  pdl_wait();
  __shared__ float qs[CH][MAX_DIM], ks[CH][MAX_DIM], as[CH][MAX_DIM];
  __shared__ float vs[CH][32];
  __shared__ float part[CH][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.x, h = blockIdx.y, v = blockIdx.z * 32 + lane;
  const int row0 = cu_q[seq], row1 = cu_q[seq + 1];
  const int slot = state_slots ? state_slots[seq] : -1;
  const int kp = (dim + 3) / 4;                  // key channels of a warp
  const int kbase = warp * kp;
  const bool vok = v < vdim;
  float S[KP];
  float* sp = state + (((long long)(slot < 0 ? 0 : slot) * H + h) * dim) * vdim + v;
#pragma unroll
  for (int i = 0; i < KP; ++i) {
    const int k = kbase + i;
    S[i] = (slot >= 0 && vok && i < kp && k < dim) ? sp[(long long)k * vdim] : 0.f;
  }
  for (int c0 = row0; c0 < row1; c0 += CH) {
    const int n = min(CH, row1 - c0);
    for (int x = threadIdx.x; x < n * dim; x += 128) {
      const int c = x / dim, k = x % dim;
      const TI* r = proj + (long long)(c0 + c) * ld;
      qs[c][k] = to_f32(r[q_off + h * dim + k]) * qscale;
      ks[c][k] = to_f32(r[k_off + h * dim + k]);
      const float zz = z[(long long)(c0 + c) * H * dim + h * dim + k] + zbias[h * dim + k];
      const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));      // ln sigmoid(zz)
      as[c][k] = expf(ls * inv_tau);
    }
    for (int x = threadIdx.x; x < n * 32; x += 128) {
      const int c = x >> 5, j = x & 31;
      const int vv = blockIdx.z * 32 + j;
      vs[c][j] = vv < vdim ? to_f32(proj[(long long)(c0 + c) * ld + v_off + h * vdim + vv]) : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < n; ++c) {
      const float val = vs[c][lane];
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < KP; ++i) {
        const int k = kbase + i;
        if (i < kp && k < dim) {
          S[i] = fmaf(as[c][k], S[i], ks[c][k] * val);
          o = fmaf(S[i], qs[c][k], o);
        }
      }
      part[c][warp][lane] = o;
    }
    __syncthreads();
    for (int x = threadIdx.x; x < n * 32; x += 128) {
      const int c = x >> 5, j = x & 31;
      const int vv = blockIdx.z * 32 + j;
      if (vv < vdim)
        out[((long long)(c0 + c) * H + h) * vdim + vv] = ((part[c][0][j] + part[c][1][j]) + part[c][2][j]) + part[c][3][j];
    }
  }
  if (slot >= 0 && vok) {
#pragma unroll
    for (int i = 0; i < KP; ++i) {
      const int k = kbase + i;
      if (i < kp && k < dim) sp[(long long)k * vdim] = S[i];
    }
  }
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

}  // namespace

// proj [T, ld] (storage type): queries at q_off, keys at k_off (H x dim each), values at v_off (H x vdim).
// z float [T, H * dim]; zbias float [H * dim]. cu_q [S + 1]: row range of each sequence; state_slots [S]
// (-1: the state starts at zero and is not kept). state float [slots, H, dim, vdim]. out float [T, H, vdim].
RLLM_API int rllm_gla_scan(int dt, const void* proj, long long ld, int q_off, int k_off, int v_off, const float* z,
                           const float* zbias, float tau, float qscale, int S, int H, int dim, int vdim,
                           const int* cu_q, const int* state_slots, float* state, float* out, void* stream) {
  if (S <= 0) return 0;
  if (H <= 0 || dim <= 0 || dim > MAX_DIM || vdim <= 0 || !(tau > 0.f)) return ERR_BAD_SIZE;
  if (H > 65535 || (vdim + 31) / 32 > 65535) return ERR_TOO_LARGE;
  dim3 grid(S, H, (vdim + 31) / 32);
  cudaStream_t s = (cudaStream_t)stream;
  const int kp = (dim + 3) / 4;
#define GO(TI, KP)                                                                                                 \
  return launch_ex(gla_scan_kernel<TI, KP>, grid, dim3(128), 0, s, 1, (const TI*)proj, ld, q_off, k_off, v_off, z, \
                   zbias, 1.f / tau, qscale, H, dim, vdim, cu_q, state_slots, state, out)
#define BY_KP(TI)                \
  do {                           \
    if (kp <= 8) GO(TI, 8);      \
    if (kp <= 16) GO(TI, 16);    \
    if (kp <= 32) GO(TI, 32);    \
    GO(TI, 64);                  \
  } while (0)
  if (dt == DT_F32) BY_KP(float);
  if (dt == DT_BF16) BY_KP(bf16);
#undef BY_KP
#undef GO
  return ERR_BAD_DTYPE;
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
