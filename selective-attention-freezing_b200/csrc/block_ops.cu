// LayerNorm of the transformer block around the attention path (LayerNorm.forward, nanogpt/model.py:45-54):
// y = (x - mean) / sqrt(var + eps) * weight (+ bias), statistics in fp32, biased variance as F.layer_norm.
// rms = 1 gives the RMSNorm of the Qwen-shaped blocks instead (the norm the reference's grouped-query adapter
// leaves to the Hugging Face model, qwen/nanogpt/hybrid_prior_attention.py:522-523): no mean, no bias,
// y = x / sqrt(mean(x^2) + eps) * weight.
// HBM-bound: one warp per row, 16-byte loads, the row stays in registers between the two passes.
#include "saf_internal.h"

namespace saf {
namespace {

constexpr int LN_WARPS = 8;
constexpr int LN_MAX_CHUNKS = 8;   // 16-byte chunks per lane held in registers: C <= 2048 on the vector path

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[2 * e] = __uint_as_float(w[e] << 16);
    f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(LN_WARPS * 32) layernorm_bf16_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                                                       const __nv_bfloat16* __restrict__ w,
                                                                       const __nv_bfloat16* __restrict__ b,
                                                                       __nv_bfloat16* __restrict__ out, int64_t ldo, int M,
                                                                       int C, float eps, int rms) {
  const int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const int n_chunks = C >> 3;                     // 8 elements each
  const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)row * ldx);
  float v[LN_MAX_CHUNKS][8];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < LN_MAX_CHUNKS; ++k) {
    const int c = lane + 32 * k;
    if (c < n_chunks) {
      unpack8(xr[c], v[k]);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[k][e];
    }
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  const float mean = rms ? 0.f : s / (float)C;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < LN_MAX_CHUNKS; ++k) {
    if (lane + 32 * k < n_chunks) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = v[k][e] - mean;
        q = fmaf(d, d, q);
      }
    }
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) q += __shfl_xor_sync(0xffffffffu, q, off);
  const float rstd = rsqrtf(q / (float)C + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = reinterpret_cast<const uint4*>(b);
  uint4* orow = reinterpret_cast<uint4*>(out + (int64_t)row * ldo);
#pragma unroll
  for (int k = 0; k < LN_MAX_CHUNKS; ++k) {
    const int c = lane + 32 * k;
    if (c < n_chunks) {
      float wv[8], bv[8];
      unpack8(wr[c], wv);
      if (b) unpack8(br[c], bv);
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float y0 = (v[k][2 * e] - mean) * rstd * wv[2 * e], y1 = (v[k][2 * e + 1] - mean) * rstd * wv[2 * e + 1];
        if (b) {
          y0 += bv[2 * e];
          y1 += bv[2 * e + 1];
        }
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(y0, y1);
        o[e] = *reinterpret_cast<const uint32_t*>(&h2);
      }
      orow[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// any dtype / width / alignment: one warp per row, three passes over the row
template <typename T>
__global__ void __launch_bounds__(LN_WARPS * 32) layernorm_generic_kernel(const T* __restrict__ x, int64_t ldx,
                                                                          const T* __restrict__ w, const T* __restrict__ b,
                                                                          T* __restrict__ out, int64_t ldo, int M, int C,
                                                                          float eps, int rms) {
  const int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const T* xr = x + (int64_t)row * ldx;
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += to_f<T>(xr[c]);
#pragma unroll
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  const float mean = rms ? 0.f : s / (float)C;
  float q = 0.f;
  for (int c = lane; c < C; c += 32) {
    const float d = to_f<T>(xr[c]) - mean;
    q = fmaf(d, d, q);
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) q += __shfl_xor_sync(0xffffffffu, q, off);
  const float rstd = rsqrtf(q / (float)C + eps);
  T* orow = out + (int64_t)row * ldo;
  for (int c = lane; c < C; c += 32) {
    float y = (to_f<T>(xr[c]) - mean) * rstd * to_f<T>(w[c]);
    if (b) y += to_f<T>(b[c]);
    orow[c] = from_f<T>(y);
  }
}

bool ln_al16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

int launch_layernorm(const void* x, int64_t ldx, const void* w, const void* b, void* out, int64_t ldo, int M, int C,
                     float eps, int dtype, int rms, cudaStream_t st) {
  const unsigned grid = (unsigned)((M + LN_WARPS - 1) / LN_WARPS);
  if (dtype == SAF_BF16) {
    const bool vec = C % 8 == 0 && C <= 256 * LN_MAX_CHUNKS && ldx % 8 == 0 && ldo % 8 == 0 && ln_al16(x) && ln_al16(w) &&
                     ln_al16(out) && (!b || ln_al16(b));
    if (vec)
      layernorm_bf16_kernel<<<grid, LN_WARPS * 32, 0, st>>>(
          reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(w),
          reinterpret_cast<const __nv_bfloat16*>(b), reinterpret_cast<__nv_bfloat16*>(out), ldo, M, C, eps, rms);
    else
      layernorm_generic_kernel<__nv_bfloat16><<<grid, LN_WARPS * 32, 0, st>>>(
          reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(w),
          reinterpret_cast<const __nv_bfloat16*>(b), reinterpret_cast<__nv_bfloat16*>(out), ldo, M, C, eps, rms);
  } else {
    layernorm_generic_kernel<float><<<grid, LN_WARPS * 32, 0, st>>>(
        reinterpret_cast<const float*>(x), ldx, reinterpret_cast<const float*>(w), reinterpret_cast<const float*>(b),
        reinterpret_cast<float*>(out), ldo, M, C, eps, rms);
  }
  count_launch();
  return check_launch("layernorm_kernel");
}

}  // namespace saf
