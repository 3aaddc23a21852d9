// Row-wise work on the float residual stream for layers that norm after the sum, and the small
// activations of their feed-forwards.
//
// postnorm:  s = alpha * h[t] + sum over p of y[t, p, :] (+ sigmoid(zg[t]) * y2[t]);  h[t] = w * s / sqrt(mean(s^2) + eps),
//            float throughout, the parts added in order. Also writes h[t] in the run's storage type (`copy`),
//            which is what the next sublayer's products read.
// cast_rows: the stream in the run's storage type (the first layer's input).
// gated_act: out[r, i] = act(scale_r * g) * (scale_r * u) for gu [R, 2F] (float or storage type), act = silu; the
//            columns of gu come in blocks of `block` gate columns followed by their up columns (block = F: all gate
//            columns, then all up columns). relu2: x <- max(x, 0)^2 in place.
#include "common.cuh"
using namespace rllm;

namespace {

template <typename TO>
__global__ void postnorm_kernel(float* __restrict__ h, const float* __restrict__ y, int parts, const float* __restrict__ y2,
                                const float* __restrict__ zg, int zg_ld, float alpha, const float* __restrict__ w, int H,
                                float eps, TO* __restrict__ copy) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const size_t t = blockIdx.x;
  float* hr = h + t * H;
  const float* yr = y ? y + t * parts * H : nullptr;
  const float* y2r = y2 ? y2 + t * H : nullptr;
  const float g2 = (y2 && zg) ? 1.f / (1.f + expf(-zg[t * zg_ld])) : 1.f;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = alpha * hr[i];
    if (yr)
      for (int p = 0; p < parts; ++p) v += yr[(size_t)p * H + i];
    if (y2r) v = fmaf(g2, y2r[i], v);
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = row[i] * r * w[i];
    hr[i] = v;
    if (copy) copy[t * H + i] = from_f32<TO>(v);
  }
}

// The same for rows of 4 * VPT * blockDim numbers at most: every thread keeps VPT float4 of the row in registers,
// all of a row's loads are in flight together (a step of single tokens is a handful of rows: latency is all).
template <typename TO, int VPT>
__global__ void __launch_bounds__(1024) postnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ y, int parts,
                                                           const float* __restrict__ y2, const float* __restrict__ zg,
                                                           int zg_ld, float alpha, const float* __restrict__ w, int H,
                                                           float eps, TO* __restrict__ copy) {
  pdl_launch();
  pdl_wait();
  __shared__ float red[32];
  const size_t t = blockIdx.x;
  const int n4 = H / 4;
  float4* hr = reinterpret_cast<float4*>(h + t * H);
  const float4* yr = y ? reinterpret_cast<const float4*>(y + t * parts * H) : nullptr;
  const float4* y2r = y2 ? reinterpret_cast<const float4*>(y2 + t * H) : nullptr;
  float4 v[VPT], e[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    v[k] = i < n4 ? hr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    e[k] = (y2r && i < n4) ? y2r[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float g2 = (y2 && zg) ? 1.f / (1.f + expf(-zg[t * zg_ld])) : 1.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) { v[k].x *= alpha; v[k].y *= alpha; v[k].z *= alpha; v[k].w *= alpha; }
  if (yr) {
    for (int p = 0; p < parts; ++p) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) { const float4 a = yr[(size_t)p * n4 + i]; v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w; }
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    if (y2r) { v[k].x = fmaf(g2, e[k].x, v[k].x); v[k].y = fmaf(g2, e[k].y, v[k].y); v[k].z = fmaf(g2, e[k].z, v[k].z); v[k].w = fmaf(g2, e[k].w, v[k].w); }
    ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss); ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < n4) {
      const float4 ww = reinterpret_cast<const float4*>(w)[i];
      const float4 o = make_float4(v[k].x * r * ww.x, v[k].y * r * ww.y, v[k].z * r * ww.z, v[k].w * r * ww.w);
      hr[i] = o;
      if (copy) {
        TO* c = copy + t * H + 4 * (size_t)i;
        c[0] = from_f32<TO>(o.x); c[1] = from_f32<TO>(o.y); c[2] = from_f32<TO>(o.z); c[3] = from_f32<TO>(o.w);
      }
    }
  }
}

template <typename TO>
int launch_postnorm(float* h, const float* y, int parts, const float* y2, const float* zg, int zg_ld, float alpha,
                    const float* w, int T, int H, float eps, TO* copy, cudaStream_t s) {
  const bool vec = H % 4 == 0 && !((uintptr_t)h & 15) && !((uintptr_t)y & 15) && !((uintptr_t)y2 & 15) && !((uintptr_t)w & 15);
  if (vec && H <= 4 * 1024 * 4) {
    const int n4 = H / 4;
    if (n4 <= 1024) {
      const int threads = (n4 + 31) / 32 * 32;
      return launch_ex(postnorm_vec_kernel<TO, 1>, dim3(T), dim3(threads), 0, s, 1, h, y, parts, y2, zg, zg_ld, alpha, w, H, eps, copy);
    }
    const int threads = ((n4 + 3) / 4 + 31) / 32 * 32;
    return launch_ex(postnorm_vec_kernel<TO, 4>, dim3(T), dim3(threads), 0, s, 1, h, y, parts, y2, zg, zg_ld, alpha, w, H, eps, copy);
  }
  static bool done[64] = {};
  const int smem = H * (int)sizeof(float);
  if (smem > 48 * 1024) { const int rc = allow_dynamic_smem(postnorm_kernel<TO>, smem, done); if (rc) return rc; }
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  return launch_ex(postnorm_kernel<TO>, dim3(T), dim3(threads), (size_t)smem, s, 1, h, y, parts, y2, zg, zg_ld, alpha, w, H, eps, copy);
}

__global__ void cast_rows_kernel(const float* __restrict__ x, bf16* __restrict__ out, long long n) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(x[i]);
}

template <typename TI, typename TO>
__global__ void gated_act_kernel(const TI* __restrict__ gu, long long ld, TO* __restrict__ out, int F, int block,
                                 long long n, const float* __restrict__ row_scale) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F;
    const int c = (int)(i % F);
    const float f = row_scale ? row_scale[r] : 1.f;
    const long long at = r * ld + (long long)(c / block) * 2 * block + c % block;     // blocks of gate columns, then their up columns
    const float g = f * to_f32(gu[at]), u = f * to_f32(gu[at + block]);
    out[i] = from_f32<TO>(g / (1.f + expf(-g)) * u);
  }
}

template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, long long n) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_f32(x[i]), 0.f);
    x[i] = from_f32<T>(v * v);
  }
}

__global__ void relu2_bf16x8_kernel(uint4* __restrict__ x, long long n8) {
  pdl_launch();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 v = x[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      f.x = fmaxf(f.x, 0.f); f.y = fmaxf(f.y, 0.f);
      h[k] = __floats2bfloat162_rn(f.x * f.x, f.y * f.y);
    }
    x[i] = v;
  }
}

inline int blocks_for(long long n) { return (int)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368); }

}  // namespace

// h [T, H] float in place; y [T, parts, H] float or null; y2 [T, H] float or null with zg (logits, one per row at
// stride zg_ld) or null; copy [T, H] of type copy_dt or null.
RLLM_API int rllm_postnorm(float* h, const float* y, int parts, const float* y2, const float* zg, int zg_ld, float alpha,
                           const float* w, int T, int H, float eps, void* copy, int copy_dt, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || parts < 0 || (size_t)H * sizeof(float) > 200 * 1024) return ERR_BAD_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (copy && copy_dt == DT_BF16)
    return launch_postnorm<bf16>(h, y, parts, y2, zg, zg_ld, alpha, w, T, H, eps, (bf16*)copy, s);
  if (copy && copy_dt != DT_F32) return ERR_BAD_DTYPE;
  return launch_postnorm<float>(h, y, parts, y2, zg, zg_ld, alpha, w, T, H, eps, (float*)copy, s);
}

RLLM_API int rllm_cast_rows(const float* x, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  return launch_ex(cast_rows_kernel, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, 1, x, (bf16*)out, n);
}

// gu [R, >= 2F] of type in_dt with row stride ld -> out [R, F] of type out_dt; row_scale float [R] or null.
RLLM_API int rllm_gated_act(const void* gu, int in_dt, long long ld, void* out, int out_dt, int R, int F, int block,
                            const float* row_scale, void* stream) {
  if (R <= 0 || F <= 0) return 0;
  if (block <= 0 || F % block) return ERR_BAD_SIZE;
  const long long n = (long long)R * F;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 g(blocks_for(n)), b(256);
  if (in_dt == DT_F32 && out_dt == DT_F32)
    return launch_ex(gated_act_kernel<float, float>, g, b, 0, s, 1, (const float*)gu, ld, (float*)out, F, block, n, row_scale);
  if (in_dt == DT_F32 && out_dt == DT_BF16)
    return launch_ex(gated_act_kernel<float, bf16>, g, b, 0, s, 1, (const float*)gu, ld, (bf16*)out, F, block, n, row_scale);
  if (in_dt == DT_BF16 && out_dt == DT_BF16)
    return launch_ex(gated_act_kernel<bf16, bf16>, g, b, 0, s, 1, (const bf16*)gu, ld, (bf16*)out, F, block, n, row_scale);
  return ERR_BAD_DTYPE;
}

RLLM_API int rllm_relu2(void* x, int dt, long long n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32) return launch_ex(relu2_kernel<float>, dim3(blocks_for(n)), dim3(256), 0, s, 1, (float*)x, n);
  if (dt == DT_BF16 && n % 8 == 0 && !((uintptr_t)x & 15))
    return launch_ex(relu2_bf16x8_kernel, dim3(blocks_for(n / 8)), dim3(256), 0, s, 1, (uint4*)x, n / 8);
  if (dt == DT_BF16) return launch_ex(relu2_kernel<bf16>, dim3(blocks_for(n)), dim3(256), 0, s, 1, (bf16*)x, n);
  return ERR_BAD_DTYPE;
}
