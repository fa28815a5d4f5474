// CUDA-core indexed linear (fp32 accumulate): forward for fp32 / shapes the
// tensor-core GEMM does not take, and both backward products.  Weight rows are
// addressed in place through the slab table; no gathered weight copy exists
// (the reference builds one per call, kernel/indexed_linear.py:93).
//
//   fwd : out[m, n]  = sum_c x[m,c] W[n][c] + b[n]          (kernel/indexed_linear.py:28-38, 86-98)
//   dx  : dx[m, c]   = sum_n dout[m,n] W[n][c]              (:47-49, 107-109)
//   dw  : dW[n][c]   = sum_m dout[m,n] x[m,c], db[n] = sum_m dout[m,n]   (:50-55, 110-121)
// where n = g*slab + r addresses row (row0[g] + r) of weight matrix slab_weight[g].
// Also: the freeze-time row normaliser of decomposed patterns (kernel/fused_attn.py:101-116).
#include "saf_internal.h"

namespace saf {
namespace {

constexpr int MAX_SLABS = 2048;
struct SlabTable {
  int32_t row0[MAX_SLABS];
  uint8_t weight[MAX_SLABS];
  uint8_t rope[MAX_SLABS];
};
struct WeightSet {
  const void* w[SAF_MAX_WEIGHTS];
  const void* b[SAF_MAX_WEIGHTS];
  int64_t ldw[SAF_MAX_WEIGHTS];
  int64_t cdw[SAF_MAX_WEIGHTS];
};

constexpr int TM = 64, TN = 64, TK = 16, GNT = 256;

// pointer to element (row n of the selection, column c)
template <typename T>
__device__ __forceinline__ const T* welem(const WeightSet& ws, const SlabTable& tb, int n, int slab, int c) {
  const int g = n / slab, r = n - g * slab;
  const int w = tb.weight[g];
  return reinterpret_cast<const T*>(ws.w[w]) + (int64_t)(tb.row0[g] + r) * ws.ldw[w] + (int64_t)c * ws.cdw[w];
}

__device__ __forceinline__ void mma_tile(const float (*As)[TM + 1], const float (*Bs)[TN + 1], int ty, int tx,
                                         float (&acc)[4][4]) {
#pragma unroll
  for (int k = 0; k < TK; ++k) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx + 16 * j];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// MODE 0: fwd, MODE 1: dx, MODE 2: dw
template <typename T, int MODE>
__global__ void __launch_bounds__(GNT) linear_generic_kernel(const T* __restrict__ A, int64_t lda,
                                                             const T* __restrict__ X, int64_t ldx, T* __restrict__ Cout,
                                                             int64_t ldc, int M, int C, int N, int slab,
                                                             const __grid_constant__ WeightSet ws,
                                                             const __grid_constant__ SlabTable tb) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  // problem shape (rows I, cols J, depth K) per mode
  const int I = (MODE == 2) ? N : M;
  const int J = (MODE == 0) ? N : C;
  const int K = (MODE == 0) ? C : (MODE == 1 ? N : M);
  const int i0 = blockIdx.y * TM, j0 = blockIdx.x * TN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int idx = tid; idx < TM * TK; idx += GNT) {
      float av = 0.f, bv = 0.f;
      if (MODE == 0 || MODE == 1) {
        // A(i,k): row-major, k contiguous
        const int ii = idx / TK, kk = idx - ii * TK;
        const int i = i0 + ii, k = k0 + kk;
        if (i < I && k < K) av = to_f<T>(A[(int64_t)i * lda + k]);
        As[kk][ii] = av;
      } else {
        // A(i=n, k=m) = dout[m*lda + n]: n contiguous
        const int kk = idx / TM, ii = idx - kk * TM;
        const int i = i0 + ii, k = k0 + kk;
        if (i < I && k < K) av = to_f<T>(A[(int64_t)k * lda + i]);
        As[kk][ii] = av;
      }
      if (MODE == 0) {
        const int jj = idx / TK, kk = idx - jj * TK;
        const int j = j0 + jj, k = k0 + kk;
        if (j < J && k < K) bv = to_f<T>(*welem<T>(ws, tb, j, slab, k));
        Bs[kk][jj] = bv;
      } else if (MODE == 1) {
        // B(j=c, k=n) = W[n][c]: c contiguous
        const int kk = idx / TN, jj = idx - kk * TN;
        const int j = j0 + jj, k = k0 + kk;
        if (j < J && k < K) bv = to_f<T>(*welem<T>(ws, tb, k, slab, j));
        Bs[kk][jj] = bv;
      } else {
        // B(j=c, k=m) = x[m*ldx + c]
        const int kk = idx / TN, jj = idx - kk * TN;
        const int j = j0 + jj, k = k0 + kk;
        if (j < J && k < K) bv = to_f<T>(X[(int64_t)k * ldx + j]);
        Bs[kk][jj] = bv;
      }
    }
    __syncthreads();
    mma_tile(As, Bs, ty, tx, acc);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ii = i0 + ty * 4 + i;
    if (ii >= I) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int jj = j0 + tx + 16 * j;
      if (jj >= J) continue;
      float v = acc[i][j];
      if (MODE == 0) {
        const int g = jj / slab, r = jj - g * slab;
        const int w = tb.weight[g];
        if (ws.b[w]) v += to_f<T>(reinterpret_cast<const T*>(ws.b[w])[tb.row0[g] + r]);
        Cout[(int64_t)ii * ldc + jj] = from_f<T>(v);
      } else if (MODE == 1) {
        if (X) v += to_f<T>(X[jj]);   // optional bias over the output columns
        Cout[(int64_t)ii * ldc + jj] = from_f<T>(v);
      } else {
        *const_cast<T*>(welem<T>(ws, tb, ii, slab, jj)) = from_f<T>(v);
      }
    }
  }
}

// db[n] = sum_m dout[m, n], scattered to bias rows
template <typename T>
__global__ void bias_grad_kernel(const T* __restrict__ dout, int64_t lddo, int M, int N, int slab,
                                 const __grid_constant__ WeightSet ws, const __grid_constant__ SlabTable tb) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const int g = n / slab, r = n - g * slab;
  const int w = tb.weight[g];
  if (!ws.b[w]) return;
  float s = 0.f;
  for (int m = 0; m < M; ++m) s += to_f<T>(dout[(int64_t)m * lddo + n]);
  const_cast<T*>(reinterpret_cast<const T*>(ws.b[w]))[tb.row0[g] + r] = from_f<T>(s);
}

// in-place rotation of the rotated slabs of out (generic path only; the
// tensor-core GEMM rotates in its epilogue)
template <typename T>
__global__ void rope_slabs_kernel(T* __restrict__ out, int64_t ldo, int M, int n_slabs, int slab, int Tlen,
                                  const float* __restrict__ cosT, const float* __restrict__ sinT,
                                  const __grid_constant__ SlabTable tb, float sgn) {
  const int half = slab >> 1;
  const int64_t total = (int64_t)M * n_slabs * half;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(idx % half);
    const int g = (int)((idx / half) % n_slabs);
    const int64_t m = idx / ((int64_t)half * n_slabs);
    if (!tb.rope[g]) continue;
    const int t = (int)(m % Tlen);
    T* p = out + m * ldo + (int64_t)g * slab;
    const float x1 = to_f<T>(p[d]), x2 = to_f<T>(p[d + half]);
    // sgn = -1 gives the adjoint (inverse) rotation; the tables repeat per half
    const float c1 = cosT[(int64_t)t * slab + d], s1 = sgn * sinT[(int64_t)t * slab + d];
    const float c2 = cosT[(int64_t)t * slab + d + half], s2 = sgn * sinT[(int64_t)t * slab + d + half];
    p[d] = from_f<T>(x1 * c1 - x2 * s1);
    p[d + half] = from_f<T>(x2 * c2 + x1 * s2);
  }
}

// bf16, 16-byte accesses: one thread rotates 8 pairs (d .. d+7, d+half .. d+half+7) of one slab of one row
__global__ void __launch_bounds__(256) rope_slabs_vec_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, int M, int n_slabs,
                                                             int slab, int Tlen, const float* __restrict__ cosT,
                                                             const float* __restrict__ sinT,
                                                             const __grid_constant__ SlabTable tb, float sgn) {
  const int half = slab >> 1, per_slab = half >> 3;
  const int64_t total = (int64_t)M * n_slabs * per_slab;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(idx % per_slab) * 8;
    const int g = (int)((idx / per_slab) % n_slabs);
    const int64_t m = idx / ((int64_t)per_slab * n_slabs);
    if (!tb.rope[g]) continue;
    const int t = (int)(m % Tlen);
    __nv_bfloat16* p = out + m * ldo + (int64_t)g * slab + d;
    uint4 lo = *reinterpret_cast<const uint4*>(p), hi = *reinterpret_cast<const uint4*>(p + half);
    const float4* c4 = reinterpret_cast<const float4*>(cosT + (int64_t)t * slab + d);
    const float4* s4 = reinterpret_cast<const float4*>(sinT + (int64_t)t * slab + d);
    const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    const float cc[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float ss[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x1a = __uint_as_float(lw[e] << 16), x1b = __uint_as_float(lw[e] & 0xffff0000u);
      const float x2a = __uint_as_float(hw[e] << 16), x2b = __uint_as_float(hw[e] & 0xffff0000u);
      const float sA = sgn * ss[2 * e], sB = sgn * ss[2 * e + 1];   // the tables repeat per half
      const __nv_bfloat162 l2 = __floats2bfloat162_rn(x1a * cc[2 * e] - x2a * sA, x1b * cc[2 * e + 1] - x2b * sB);
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(x2a * cc[2 * e] + x1a * sA, x2b * cc[2 * e + 1] + x1b * sB);
      lw[e] = *reinterpret_cast<const uint32_t*>(&l2);
      hw[e] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    *reinterpret_cast<uint4*>(p + half) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
  }
}

int fill_tables(const SafIndexedLinearArgs& a, WeightSet* ws, SlabTable* tb) {
  if (a.n_slabs > MAX_SLABS) return fail(SAF_ERR_LIMIT, "n_slabs %d exceeds the limit of %d", a.n_slabs, MAX_SLABS);
  memset(ws, 0, sizeof(*ws));
  memset(tb, 0, sizeof(*tb));
  for (int w = 0; w < a.n_weights; ++w) {
    ws->w[w] = a.weights[w];
    ws->b[w] = a.biases[w];
    ws->ldw[w] = a.ldw[w];
    ws->cdw[w] = a.cdw[w] ? a.cdw[w] : 1;
  }
  for (int g = 0; g < a.n_slabs; ++g) {
    tb->row0[g] = a.slab_row0[g];
    tb->weight[g] = (uint8_t)a.slab_weight[g];
    tb->rope[g] = (uint8_t)(a.slab_rope ? (a.slab_rope[g] != 0) : 0);
  }
  return SAF_OK;
}

template <typename T>
int gemm_generic_typed(const SafIndexedLinearArgs& a, int mode, const void* dout, int64_t lddo, void* dx,
                       int64_t lddx, const void* bias, cudaStream_t st) {
  WeightSet ws;
  SlabTable tb;
  int rc = fill_tables(a, &ws, &tb);
  if (rc) return rc;
  const int N = a.n_slabs * a.slab;
  if (mode == 0) {
    dim3 grid((N + TN - 1) / TN, (a.M + TM - 1) / TM);
    linear_generic_kernel<T, 0><<<grid, GNT, 0, st>>>(reinterpret_cast<const T*>(a.x), a.ldx, nullptr, 0,
                                                      reinterpret_cast<T*>(a.out), a.ldo, a.M, a.C, N, a.slab, ws, tb);
    count_launch();
    if ((rc = check_launch("linear_generic_kernel<fwd>"))) return rc;
    bool any_rope = false;
    for (int g = 0; g < a.n_slabs; ++g) any_rope |= tb.rope[g] != 0;
    if (any_rope) {
      const int64_t total = (int64_t)a.M * a.n_slabs * (a.slab / 2);
      const int blocks = (int)std::min<int64_t>((total + 255) / 256, 148 * 16);
      rope_slabs_kernel<T><<<blocks, 256, 0, st>>>(reinterpret_cast<T*>(a.out), a.ldo, a.M, a.n_slabs, a.slab, a.T,
                                                  a.rope_cos, a.rope_sin, tb, 1.f);
      count_launch();
      if ((rc = check_launch("rope_slabs_kernel"))) return rc;
    }
  } else if (mode == 1) {
    dim3 grid((a.C + TN - 1) / TN, (a.M + TM - 1) / TM);
    linear_generic_kernel<T, 1><<<grid, GNT, 0, st>>>(reinterpret_cast<const T*>(dout), lddo,
                                                      reinterpret_cast<const T*>(bias), 0,
                                                      reinterpret_cast<T*>(dx), lddx, a.M, a.C, N, a.slab, ws, tb);
    count_launch();
    if ((rc = check_launch("linear_generic_kernel<dx>"))) return rc;
  } else {
    dim3 grid((a.C + TN - 1) / TN, (N + TM - 1) / TM);
    linear_generic_kernel<T, 2><<<grid, GNT, 0, st>>>(reinterpret_cast<const T*>(dout), lddo,
                                                      reinterpret_cast<const T*>(a.x), a.ldx, nullptr, 0, a.M, a.C, N,
                                                      a.slab, ws, tb);
    count_launch();
    if ((rc = check_launch("linear_generic_kernel<dw>"))) return rc;
    bool any_bias = false;
    for (int w = 0; w < a.n_weights; ++w) any_bias |= a.biases[w] != nullptr;
    if (any_bias) {
      bias_grad_kernel<T><<<(N + 127) / 128, 128, 0, st>>>(reinterpret_cast<const T*>(dout), lddo, a.M, N, a.slab, ws, tb);
      count_launch();
      if ((rc = check_launch("bias_grad_kernel"))) return rc;
    }
  }
  return SAF_OK;
}

// z[h,i] = logsumexp_{j<=i}(alpha[h,j] + rho[h,i-j]); one warp per row
__global__ void logz_kernel(const float* __restrict__ alpha, const float* __restrict__ rho, float* __restrict__ z,
                            int H, int S, int rows) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= H * S) return;
  const int h = warp / S, i = warp - h * S;
  if (i >= rows) {
    if (lane == 0) z[(int64_t)h * S + i] = 0.f;
    return;
  }
  const float* al = alpha + (int64_t)h * S;
  const float* rh = rho + (int64_t)h * S;
  float m = -INFINITY, s = 0.f;
  for (int j = lane; j <= i; j += 32) {
    const float x = al[j] + rh[i - j];
    if (x > m) {
      s = s * expf(m - x) + 1.f;
      m = x;
    } else if (x > -INFINITY) {
      s += expf(x - m);
    }
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, off), s2 = __shfl_xor_sync(0xffffffffu, s, off);
    const float mm = fmaxf(m, m2);
    if (mm == -INFINITY) {
      s = 0.f;
    } else {
      s = s * expf(m - mm) + s2 * expf(m2 - mm);
    }
    m = mm;
  }
  if (lane == 0) z[(int64_t)h * S + i] = m + logf(s);
}

}  // namespace

int launch_gemm_generic(const SafIndexedLinearArgs& a, cudaStream_t st) {
  if (a.dtype == SAF_F32) return gemm_generic_typed<float>(a, 0, nullptr, 0, nullptr, 0, nullptr, st);
  return gemm_generic_typed<__nv_bfloat16>(a, 0, nullptr, 0, nullptr, 0, nullptr, st);
}
int launch_gemm_bwd_dx(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, void* dx, int64_t lddx,
                       const void* bias, cudaStream_t st) {
  if (a.dtype == SAF_F32) return gemm_generic_typed<float>(a, 1, dout, lddo, dx, lddx, bias, st);
  return gemm_generic_typed<__nv_bfloat16>(a, 1, dout, lddo, dx, lddx, bias, st);
}
int launch_gemm_bwd_dw(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, cudaStream_t st) {
  if (a.dtype == SAF_F32) return gemm_generic_typed<float>(a, 2, dout, lddo, nullptr, 0, nullptr, st);
  return gemm_generic_typed<__nv_bfloat16>(a, 2, dout, lddo, nullptr, 0, nullptr, st);
}
int launch_rope_slabs(void* x, int64_t ld, int M, int n_slabs, int slab, int T, const int32_t* slab_rope,
                      const float* cosT, const float* sinT, int dtype, int inverse, cudaStream_t st) {
  if (n_slabs > MAX_SLABS) return fail(SAF_ERR_LIMIT, "n_slabs %d exceeds the limit of %d", n_slabs, MAX_SLABS);
  SlabTable tb;
  memset(&tb, 0, sizeof(tb));
  for (int g = 0; g < n_slabs; ++g) tb.rope[g] = (uint8_t)(slab_rope ? (slab_rope[g] != 0) : 1);
  const int64_t total = (int64_t)M * n_slabs * (slab / 2);
  const int blocks = (int)std::min<int64_t>((total + 255) / 256, 148 * 16);
  const float sgn = inverse ? -1.f : 1.f;
  const bool vec = dtype == SAF_BF16 && slab % 16 == 0 && ld % 8 == 0 && ((uintptr_t)x & 15) == 0 &&
                   ((uintptr_t)cosT & 15) == 0 && ((uintptr_t)sinT & 15) == 0;
  if (vec) {
    const int64_t tv = (int64_t)M * n_slabs * (slab / 16);
    const int bv = (int)std::min<int64_t>((tv + 255) / 256, 148 * 32);
    rope_slabs_vec_kernel<<<bv, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(x), ld, M, n_slabs, slab, T, cosT, sinT, tb, sgn);
  } else if (dtype == SAF_F32)
    rope_slabs_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<float*>(x), ld, M, n_slabs, slab, T, cosT, sinT, tb, sgn);
  else
    rope_slabs_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(x), ld, M, n_slabs, slab, T,
                                                            cosT, sinT, tb, sgn);
  count_launch();
  return check_launch("rope_slabs_kernel");
}
int launch_logz(const float* alpha, const float* rho, float* z, int H, int S, int rows, cudaStream_t st) {
  const int64_t warps = (int64_t)H * S;
  const int64_t blocks = (warps * 32 + 255) / 256;
  logz_kernel<<<(unsigned)blocks, 256, 0, st>>>(alpha, rho, z, H, S, rows);
  count_launch();
  return check_launch("logz_kernel");
}

}  // namespace saf
