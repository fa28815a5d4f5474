// CUDA-core (fp32 FMA) mixed attention: forward and backward for every head state,
// element type, stride pattern and head_dim <= 128.  This is the path for fp32
// inputs (true fp32 accumulation, the 2e-5 contract of kernel/fused_attn.py:36-37),
// for shapes the tensor-core kernels do not take, and for the backward pass.
//
// Work decomposition follows the reference's Triton kernels
// (kernel/fused_attn.py:228-289 forward, 291-540 backward): one CTA per 64-row
// tile per (batch, head), causal tile skipping, head state read per CTA.
#include "saf_internal.h"

namespace saf {

namespace {

constexpr int BM = 64;      // query rows per CTA
constexpr int BN = 64;      // keys per step
constexpr int PADW = 65;    // padded row length of transposed tiles
constexpr int NT = 256;
constexpr float LOG2E = 1.4426950408889634f;

struct HeadIdx {
  int b, h, state, hq, hk, hv, hp;
};

__device__ __forceinline__ HeadIdx head_index(const SafMixedAttnArgs& a, int bh) {
  HeadIdx x;
  x.b = bh / a.H;
  x.h = bh % a.H;
  x.state = a.force_state >= 0 ? a.force_state : a.frozen[x.h];
  x.hq = a.hidx ? a.hidx[x.h] : x.h;
  if (a.HKV > 0) {
    x.hk = x.hv = a.kvidx ? a.kvidx[x.h] : 0;
  } else {
    x.hk = x.hq;
    x.hv = x.h;
  }
  x.hp = a.pidx ? a.pidx[x.h] : x.h;
  return x;
}

// load one (rows x hd) tile of a (.., T, hd) head into smem, transposed: dst[d*PADW + r]
template <typename T, bool ROPE>
__device__ __forceinline__ void load_tile_T(float* dst, const T* base, int64_t s_row, int64_t s_d, int row0,
                                            int Tlen, int hd, const float* cosT, const float* sinT) {
  for (int idx = threadIdx.x; idx < BM * hd; idx += NT) {
    const int r = idx / hd, d = idx - r * hd;
    const int t = row0 + r;
    float v = 0.f;
    if (t < Tlen) {
      const T* p = base + (int64_t)t * s_row;
      v = to_f<T>(p[(int64_t)d * s_d]);
      if (ROPE) {
        const int half = hd >> 1;
        const float o = (d < half) ? -to_f<T>(p[(int64_t)(d + half) * s_d]) : to_f<T>(p[(int64_t)(d - half) * s_d]);
        v = v * cosT[(int64_t)t * hd + d] + o * sinT[(int64_t)t * hd + d];
      }
    }
    dst[d * PADW + r] = v;
  }
}

// load one (rows x hd) tile row-major: dst[r*hd + d]
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* base, int64_t s_row, int64_t s_d, int row0,
                                          int Tlen, int hd) {
  for (int idx = threadIdx.x; idx < BM * hd; idx += NT) {
    const int r = idx / hd, d = idx - r * hd;
    const int t = row0 + r;
    dst[idx] = (t < Tlen) ? to_f<T>(base[(int64_t)t * s_row + (int64_t)d * s_d]) : 0.f;
  }
}

// pattern tile into Ps[r*PADW + c] for rows i0.., cols j0..; causal + bounds mask.
// TRANSPOSE: Ps[c*PADW + r] (used by the backward, which needs P^T rows)
__device__ __forceinline__ void load_pattern_tile(float* Ps, const SafMixedAttnArgs& a, const HeadIdx& hx, int i0,
                                                  int j0, int state) {
  if (state == SAF_DENSE) {
    const int64_t base = (int64_t)hx.hp * a.patt.stride[0];
    for (int idx = threadIdx.x; idx < BM * BN; idx += NT) {
      const int r = idx / BN, c = idx - r * BN;
      const int i = i0 + r, j = j0 + c;
      float p = 0.f;
      if (i < a.T && j <= i) p = load_rt(a.patt.ptr, base + (int64_t)i * a.patt.stride[1] + (int64_t)j * a.patt.stride[2], a.patt_dtype);
      Ps[r * PADW + c] = p;
    }
  } else {  // SAF_DECOMP
    for (int idx = threadIdx.x; idx < BM * BN; idx += NT) {
      const int r = idx / BN, c = idx - r * BN;
      const int i = i0 + r, j = j0 + c;
      float p = 0.f;
      if (i < a.T && j <= i) {
        const float al = load_rt(a.alpha.ptr, (int64_t)hx.h * a.alpha.stride[0] + (int64_t)j * a.alpha.stride[1], a.dec_dtype);
        const float rh = load_rt(a.rho.ptr, (int64_t)hx.h * a.rho.stride[0] + (int64_t)(i - j) * a.rho.stride[1], a.dec_dtype);
        const float zz = load_rt(a.z.ptr, (int64_t)hx.h * a.z.stride[0] + (int64_t)i * a.z.stride[1], a.dec_dtype);
        p = exp2f((al + rh - zz) * LOG2E);
      }
      Ps[r * PADW + c] = p;
    }
  }
}

// S[i][j] (4x4 per thread) = sum_d At[d][r_i] * Bt[d][c_j];  rows ty*4+i, cols tx+16*j
__device__ __forceinline__ void tile_dot_TT(const float* At, const float* Bt, int hd, int ty, int tx,
                                            float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int d = 0; d < hd; ++d) {
    float av[4], bv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) av[i] = At[d * PADW + ty * 4 + i];
#pragma unroll
    for (int j = 0; j < 4; ++j) bv[j] = Bt[d * PADW + tx + 16 * j];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}

// acc[i][jj] += sum_k Ps[(ty*4+i)*PADW + k] * Vs[k*hd + tx+16*jj]
__device__ __forceinline__ void tile_pv(const float* Ps, const float* Vs, int hd, int ty, int tx,
                                        float (&acc)[4][8]) {
  for (int k = 0; k < BN; ++k) {
    float pv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pv[i] = Ps[(ty * 4 + i) * PADW + k];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int c = tx + 16 * jj;
      if (c < hd) {
        const float v = Vs[k * hd + c];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][jj] = fmaf(pv[i], v, acc[i][jj]);
      }
    }
  }
}

// same with the right operand held transposed: Bt[c*PADW + k]
__device__ __forceinline__ void tile_pv_T(const float* Ps, const float* Bt, int hd, int ty, int tx,
                                          float (&acc)[4][8]) {
  for (int k = 0; k < BN; ++k) {
    float pv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) pv[i] = Ps[(ty * 4 + i) * PADW + k];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int c = tx + 16 * jj;
      if (c < hd) {
        const float v = Bt[c * PADW + k];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i][jj] = fmaf(pv[i], v, acc[i][jj]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT) generic_fwd_kernel(const __grid_constant__ SafMixedAttnArgs a,
                                                         uint32_t states_mask) {
  extern __shared__ float smem[];
  const HeadIdx hx = head_index(a, blockIdx.y);
  if (!((states_mask >> hx.state) & 1u)) return;
  const int mt = gridDim.x - 1 - blockIdx.x;  // heaviest row tiles first
  const int i0 = mt * BM;
  const int hd = a.HD, Tn = a.T;
  float* Qt = smem;                    // [hd][PADW]
  float* Kt = Qt + hd * PADW;          // [hd][PADW]
  float* Vs = Kt + hd * PADW;          // [BN][hd]
  float* Ps = Vs + BN * hd;            // [BM][PADW]
  float* m_s = Ps + BM * PADW;
  float* l_s = m_s + BM;
  float* f_s = l_s + BM;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;

  const T* vb = reinterpret_cast<const T*>(a.v.ptr) + (int64_t)hx.b * a.v.stride[0] + (int64_t)hx.hv * a.v.stride[1];
  const T* qb = nullptr;
  const T* kb = nullptr;
  const bool live = hx.state == SAF_LIVE;
  if (live) {
    qb = reinterpret_cast<const T*>(a.q.ptr) + (int64_t)hx.b * a.q.stride[0] + (int64_t)hx.hq * a.q.stride[1];
    kb = reinterpret_cast<const T*>(a.k.ptr) + (int64_t)hx.b * a.k.stride[0] + (int64_t)hx.hk * a.k.stride[1];
    if (a.rope) load_tile_T<T, true>(Qt, qb, a.q.stride[2], a.q.stride[3], i0, Tn, hd, a.rope_cos, a.rope_sin);
    else load_tile_T<T, false>(Qt, qb, a.q.stride[2], a.q.stride[3], i0, Tn, hd, nullptr, nullptr);
  }
  if (tid < BM) {
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
    f_s[tid] = 1.f;
  }
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) acc[i][jj] = 0.f;
  const float qk_scale = a.sm_scale * LOG2E;
  const int hi = min(i0 + BM, Tn);
  __syncthreads();

  for (int j0 = 0; j0 < hi; j0 += BN) {
    load_tile<T>(Vs, vb, a.v.stride[2], a.v.stride[3], j0, Tn, hd);
    if (live) {
      if (a.rope) load_tile_T<T, true>(Kt, kb, a.k.stride[2], a.k.stride[3], j0, Tn, hd, a.rope_cos, a.rope_sin);
      else load_tile_T<T, false>(Kt, kb, a.k.stride[2], a.k.stride[3], j0, Tn, hd, nullptr, nullptr);
      __syncthreads();
      float s[4][4];
      tile_dot_TT(Qt, Kt, hd, ty, tx, s);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = ty * 4 + i, c = tx + 16 * j;
          const bool ok = (i0 + r) >= (j0 + c) && (j0 + c) < Tn;
          Ps[r * PADW + c] = ok ? s[i][j] * qk_scale : -INFINITY;
        }
      __syncthreads();
      {  // row statistics: 4 threads per row, 16 columns each
        const int r = tid >> 2, qd = tid & 3;
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 16; ++c) mx = fmaxf(mx, Ps[r * PADW + qd * 16 + c]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_old = m_s[r];
        const float m_new = fmaxf(m_old, mx);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float p = exp2f(Ps[r * PADW + qd * 16 + c] - m_safe);
          Ps[r * PADW + qd * 16 + c] = p;
          sum += p;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        __syncwarp();
        if (qd == 0) {
          const float f = (m_old == -INFINITY) ? 0.f : exp2f(m_old - m_safe);
          l_s[r] = l_s[r] * f + sum;
          m_s[r] = m_new;
          f_s[r] = f;
        }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float f = f_s[ty * 4 + i];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) acc[i][jj] *= f;
      }
    } else {
      load_pattern_tile(Ps, a, hx, i0, j0, hx.state);
      __syncthreads();
    }
    tile_pv(Ps, Vs, hd, ty, tx, acc);
    __syncthreads();
  }

  T* ob = reinterpret_cast<T*>(a.out.ptr) + (int64_t)hx.b * a.out.stride[0] + (int64_t)hx.h * a.out.stride[1];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i, t = i0 + r;
    if (t >= Tn) continue;
    float inv = 1.f;
    if (live) {
      const float l = l_s[r];
      inv = 1.f / (l == 0.f ? 1.f : l);
    }
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int c = tx + 16 * jj;
      if (c < hd) ob[(int64_t)t * a.out.stride[2] + (int64_t)c * a.out.stride[3]] = from_f<T>(acc[i][jj] * inv);
    }
  }
  if (live && a.lse.ptr && tid < BM && i0 + tid < Tn) {
    const float m = m_s[tid], l = l_s[tid];
    float* lp = reinterpret_cast<float*>(a.lse.ptr);
    lp[(int64_t)hx.b * a.lse.stride[0] + (int64_t)hx.h * a.lse.stride[1] + (int64_t)(i0 + tid) * a.lse.stride[2]] =
        ((m == -INFINITY) ? 0.f : m) + log2f(l == 0.f ? 1.f : l);
  }
}

// ---------------------------------------------------------------------------
// backward: delta = rowsum(O * dO)      (kernel/fused_attn.py:291-310)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT) generic_delta_kernel(const __grid_constant__ SafMixedAttnBwdArgs g) {
  const SafMixedAttnArgs& a = g.fwd;
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (NT / 32) + warp;
  if (t >= a.T) return;
  const T* o = reinterpret_cast<const T*>(a.out.ptr) + (int64_t)b * a.out.stride[0] + (int64_t)h * a.out.stride[1] + (int64_t)t * a.out.stride[2];
  const T* d = reinterpret_cast<const T*>(g.dout.ptr) + (int64_t)b * g.dout.stride[0] + (int64_t)h * g.dout.stride[1] + (int64_t)t * g.dout.stride[2];
  float s = 0.f;
  for (int c = lane; c < a.HD; c += 32) s += to_f<T>(o[(int64_t)c * a.out.stride[3]]) * to_f<T>(d[(int64_t)c * g.dout.stride[3]]);
#pragma unroll
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0)
    reinterpret_cast<float*>(g.delta.ptr)[(int64_t)b * g.delta.stride[0] + (int64_t)h * g.delta.stride[1] + (int64_t)t * g.delta.stride[2]] = s;
}

// inverse rotation applied to a gradient tile held transposed in smem ([d][PADW]),
// in place: dx = dy*cos - rotate_half(dy)*sin     (adjoint of nanogpt/model.py:63-68)
__device__ __forceinline__ float unrope(const float* Gt, int r, int d, int hd, int t, const float* cosT,
                                        const float* sinT) {
  const int half = hd >> 1;
  const float g = Gt[d * PADW + r];
  // rotate_half(dy)[d] = (d < half) ? -dy[d+half] : dy[d-half]
  const float o = (d < half) ? -Gt[(d + half) * PADW + r] : Gt[(d - half) * PADW + r];
  // adjoint: dx[d] = dy[d]*cos[d] + (d<half ? dy[d+half]*sin[d+half] : -dy[d-half]*sin[d-half]); tables repeat per half
  return g * cosT[(int64_t)t * hd + d] - o * sinT[(int64_t)t * hd + d];
}

// ---------------------------------------------------------------------------
// backward: dK, dV per key tile         (kernel/fused_attn.py:415-481, 314-413)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT) generic_dkdv_kernel(const __grid_constant__ SafMixedAttnBwdArgs g,
                                                          uint32_t states_mask) {
  extern __shared__ float smem[];
  const SafMixedAttnArgs& a = g.fwd;
  const HeadIdx hx = head_index(a, blockIdx.y);
  if (!((states_mask >> hx.state) & 1u)) return;
  const int j0 = blockIdx.x * BN;
  const int hd = a.HD, Tn = a.T;
  float* Kt = smem;                     // [hd][PADW]   keys of this tile (transposed)
  float* Vt = Kt + hd * PADW;           // [hd][PADW]   values of this tile (transposed)
  float* Qt = Vt + hd * PADW;           // [hd][PADW]   query tile (transposed)
  float* Dt = Qt + hd * PADW;           // [hd][PADW]   dO tile (transposed)
  float* Ps = Dt + hd * PADW;           // [BN][PADW]   p^T  : Ps[c*PADW + r]  (key c, query r)
  float* Ds = Ps + BN * PADW;           // [BN][PADW]   ds^T
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const bool live = hx.state == SAF_LIVE;
  const T* vb = reinterpret_cast<const T*>(a.v.ptr) + (int64_t)hx.b * a.v.stride[0] + (int64_t)hx.hv * a.v.stride[1];
  const T* dob = reinterpret_cast<const T*>(g.dout.ptr) + (int64_t)hx.b * g.dout.stride[0] + (int64_t)hx.h * g.dout.stride[1];
  const T* qb = nullptr;
  const T* kb = nullptr;
  if (live) {
    qb = reinterpret_cast<const T*>(a.q.ptr) + (int64_t)hx.b * a.q.stride[0] + (int64_t)hx.hq * a.q.stride[1];
    kb = reinterpret_cast<const T*>(a.k.ptr) + (int64_t)hx.b * a.k.stride[0] + (int64_t)hx.hk * a.k.stride[1];
    if (a.rope) load_tile_T<T, true>(Kt, kb, a.k.stride[2], a.k.stride[3], j0, Tn, hd, a.rope_cos, a.rope_sin);
    else load_tile_T<T, false>(Kt, kb, a.k.stride[2], a.k.stride[3], j0, Tn, hd, nullptr, nullptr);
    load_tile_T<T, false>(Vt, vb, a.v.stride[2], a.v.stride[3], j0, Tn, hd, nullptr, nullptr);
  }
  float dv[4][8], dk[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) dv[i][jj] = dk[i][jj] = 0.f;
  const float qk_scale = a.sm_scale * LOG2E;
  const float* lse = reinterpret_cast<const float*>(a.lse.ptr);
  const float* delta = reinterpret_cast<const float*>(g.delta.ptr);
  __syncthreads();

  for (int i0 = j0; i0 < Tn; i0 += BM) {
    load_tile_T<T, false>(Dt, dob, g.dout.stride[2], g.dout.stride[3], i0, Tn, hd, nullptr, nullptr);
    if (live) {
      if (a.rope) load_tile_T<T, true>(Qt, qb, a.q.stride[2], a.q.stride[3], i0, Tn, hd, a.rope_cos, a.rope_sin);
      else load_tile_T<T, false>(Qt, qb, a.q.stride[2], a.q.stride[3], i0, Tn, hd, nullptr, nullptr);
      __syncthreads();
      // s^T[c][r] = k_c . q_r ; dp^T[c][r] = v_c . do_r      (thread: keys ty*4+i, queries tx+16*j)
      float s[4][4], dp[4][4];
      tile_dot_TT(Kt, Qt, hd, ty, tx, s);
      tile_dot_TT(Vt, Dt, hd, ty, tx, dp);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = ty * 4 + i, r = tx + 16 * j;
          const int qi = i0 + r, kj = j0 + c;
          float p = 0.f, ds = 0.f;
          if (qi < Tn && kj <= qi) {
            const int64_t li = (int64_t)hx.b * a.lse.stride[0] + (int64_t)hx.h * a.lse.stride[1] + (int64_t)qi * a.lse.stride[2];
            const int64_t di = (int64_t)hx.b * g.delta.stride[0] + (int64_t)hx.h * g.delta.stride[1] + (int64_t)qi * g.delta.stride[2];
            p = exp2f(s[i][j] * qk_scale - lse[li]);
            ds = p * (dp[i][j] - delta[di]) * a.sm_scale;
          }
          Ps[c * PADW + r] = p;
          Ds[c * PADW + r] = ds;
        }
      __syncthreads();
      tile_pv_T(Ps, Dt, hd, ty, tx, dv);  // dV[c] += sum_r p[r][c] dO[r]
      tile_pv_T(Ds, Qt, hd, ty, tx, dk);  // dK[c] += sum_r ds[r][c] q[r]
    } else {
      // frozen: P^T tile.  load_pattern_tile gives Ps[r*PADW + c]; transpose through Ds.
      load_pattern_tile(Ds, a, hx, i0, j0, hx.state);
      __syncthreads();
      for (int idx = tid; idx < BM * BN; idx += NT) {
        const int r = idx / BN, c = idx - r * BN;
        Ps[c * PADW + r] = Ds[r * PADW + c];
      }
      __syncthreads();
      tile_pv_T(Ps, Dt, hd, ty, tx, dv);
    }
    __syncthreads();
  }

  T* dvb = reinterpret_cast<T*>(g.dv.ptr) + (int64_t)hx.b * g.dv.stride[0] + (int64_t)hx.hv * g.dv.stride[1];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = j0 + ty * 4 + i;
    if (t >= Tn) continue;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int c = tx + 16 * jj;
      if (c < hd) dvb[(int64_t)t * g.dv.stride[2] + (int64_t)c * g.dv.stride[3]] = from_f<T>(dv[i][jj]);
    }
  }
  if (live) {
    T* dkb = reinterpret_cast<T*>(g.dk.ptr) + (int64_t)hx.b * g.dk.stride[0] + (int64_t)hx.hk * g.dk.stride[1];
    if (a.rope) {
      // stage dK transposed, then un-rotate on store
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int c = tx + 16 * jj;
          if (c < hd) Qt[c * PADW + ty * 4 + i] = dk[i][jj];
        }
      __syncthreads();
      for (int idx = tid; idx < BN * hd; idx += NT) {
        const int r = idx / hd, d = idx - r * hd, t = j0 + r;
        if (t < Tn) dkb[(int64_t)t * g.dk.stride[2] + (int64_t)d * g.dk.stride[3]] = from_f<T>(unrope(Qt, r, d, hd, t, a.rope_cos, a.rope_sin));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = j0 + ty * 4 + i;
        if (t >= Tn) continue;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int c = tx + 16 * jj;
          if (c < hd) dkb[(int64_t)t * g.dk.stride[2] + (int64_t)c * g.dk.stride[3]] = from_f<T>(dk[i][jj]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// backward: dQ per query tile, live heads only   (kernel/fused_attn.py:483-540)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(NT) generic_dq_kernel(const __grid_constant__ SafMixedAttnBwdArgs g) {
  extern __shared__ float smem[];
  const SafMixedAttnArgs& a = g.fwd;
  const HeadIdx hx = head_index(a, blockIdx.y);
  if (hx.state != SAF_LIVE) return;
  const int mt = gridDim.x - 1 - blockIdx.x;
  const int i0 = mt * BM;
  const int hd = a.HD, Tn = a.T;
  float* Qt = smem;                     // [hd][PADW]
  float* Dt = Qt + hd * PADW;           // [hd][PADW]  dO transposed
  float* Kt = Dt + hd * PADW;           // [hd][PADW]
  float* Vt = Kt + hd * PADW;           // [hd][PADW]
  float* Ds = Vt + hd * PADW;           // [BM][PADW]  ds[r][c]
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const T* qb = reinterpret_cast<const T*>(a.q.ptr) + (int64_t)hx.b * a.q.stride[0] + (int64_t)hx.hq * a.q.stride[1];
  const T* kb = reinterpret_cast<const T*>(a.k.ptr) + (int64_t)hx.b * a.k.stride[0] + (int64_t)hx.hk * a.k.stride[1];
  const T* vb = reinterpret_cast<const T*>(a.v.ptr) + (int64_t)hx.b * a.v.stride[0] + (int64_t)hx.hv * a.v.stride[1];
  const T* dob = reinterpret_cast<const T*>(g.dout.ptr) + (int64_t)hx.b * g.dout.stride[0] + (int64_t)hx.h * g.dout.stride[1];
  if (a.rope) load_tile_T<T, true>(Qt, qb, a.q.stride[2], a.q.stride[3], i0, Tn, hd, a.rope_cos, a.rope_sin);
  else load_tile_T<T, false>(Qt, qb, a.q.stride[2], a.q.stride[3], i0, Tn, hd, nullptr, nullptr);
  load_tile_T<T, false>(Dt, dob, g.dout.stride[2], g.dout.stride[3], i0, Tn, hd, nullptr, nullptr);
  float dq[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) dq[i][jj] = 0.f;
  const float qk_scale = a.sm_scale * LOG2E;
  const float* lse = reinterpret_cast<const float*>(a.lse.ptr);
  const float* delta = reinterpret_cast<const float*>(g.delta.ptr);
  float lse_r[4], del_r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int qi = i0 + ty * 4 + i;
    lse_r[i] = del_r[i] = 0.f;
    if (qi < Tn) {
      lse_r[i] = lse[(int64_t)hx.b * a.lse.stride[0] + (int64_t)hx.h * a.lse.stride[1] + (int64_t)qi * a.lse.stride[2]];
      del_r[i] = delta[(int64_t)hx.b * g.delta.stride[0] + (int64_t)hx.h * g.delta.stride[1] + (int64_t)qi * g.delta.stride[2]];
    }
  }
  const int hi = min(i0 + BM, Tn);
  __syncthreads();
  for (int j0 = 0; j0 < hi; j0 += BN) {
    if (a.rope) load_tile_T<T, true>(Kt, kb, a.k.stride[2], a.k.stride[3], j0, Tn, hd, a.rope_cos, a.rope_sin);
    else load_tile_T<T, false>(Kt, kb, a.k.stride[2], a.k.stride[3], j0, Tn, hd, nullptr, nullptr);
    load_tile_T<T, false>(Vt, vb, a.v.stride[2], a.v.stride[3], j0, Tn, hd, nullptr, nullptr);
    __syncthreads();
    float s[4][4], dp[4][4];
    tile_dot_TT(Qt, Kt, hd, ty, tx, s);
    tile_dot_TT(Dt, Vt, hd, ty, tx, dp);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = ty * 4 + i, c = tx + 16 * j;
        const int qi = i0 + r, kj = j0 + c;
        float ds = 0.f;
        if (qi < Tn && kj <= qi) {
          const float p = exp2f(s[i][j] * qk_scale - lse_r[i]);
          ds = p * (dp[i][j] - del_r[i]) * a.sm_scale;
        }
        Ds[r * PADW + c] = ds;
      }
    __syncthreads();
    tile_pv_T(Ds, Kt, hd, ty, tx, dq);
    __syncthreads();
  }
  T* dqb = reinterpret_cast<T*>(g.dq.ptr) + (int64_t)hx.b * g.dq.stride[0] + (int64_t)hx.hq * g.dq.stride[1];
  if (a.rope) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int c = tx + 16 * jj;
        if (c < hd) Kt[c * PADW + ty * 4 + i] = dq[i][jj];
      }
    __syncthreads();
    for (int idx = tid; idx < BM * hd; idx += NT) {
      const int r = idx / hd, d = idx - r * hd, t = i0 + r;
      if (t < Tn) dqb[(int64_t)t * g.dq.stride[2] + (int64_t)d * g.dq.stride[3]] = from_f<T>(unrope(Kt, r, d, hd, t, a.rope_cos, a.rope_sin));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = i0 + ty * 4 + i;
      if (t >= Tn) continue;
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int c = tx + 16 * jj;
        if (c < hd) dqb[(int64_t)t * g.dq.stride[2] + (int64_t)c * g.dq.stride[3]] = from_f<T>(dq[i][jj]);
      }
    }
  }
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return fail(SAF_ERR_CUDA, "cudaFuncSetAttribute(smem=%zu): %s", bytes, cudaGetErrorString(e));
  }
  return SAF_OK;
}

template <typename T>
int fwd_typed(const SafMixedAttnArgs& a, uint32_t mask, cudaStream_t st) {
  const int hd = a.HD;
  const size_t smem = sizeof(float) * ((size_t)2 * hd * PADW + (size_t)BN * hd + (size_t)BM * PADW + 3 * BM);
  int rc = set_smem(generic_fwd_kernel<T>, smem);
  if (rc) return rc;
  dim3 grid((a.T + BM - 1) / BM, a.B * a.H);
  generic_fwd_kernel<T><<<grid, NT, smem, st>>>(a, mask);
  count_launch();
  return check_launch("generic_fwd_kernel");
}

template <typename T>
int bwd_typed(const SafMixedAttnBwdArgs& g, uint32_t mask, cudaStream_t st) {
  const SafMixedAttnArgs& a = g.fwd;
  const int hd = a.HD;
  int rc;
  const bool any_live = (mask & 1u) != 0;
  if (any_live) {
    dim3 gd((a.T + (NT / 32) - 1) / (NT / 32), a.B * a.H);
    generic_delta_kernel<T><<<gd, NT, 0, st>>>(g);
    count_launch();
    if ((rc = check_launch("generic_delta_kernel"))) return rc;
  }
  {
    const size_t smem = sizeof(float) * ((size_t)4 * hd * PADW + (size_t)2 * BN * PADW);
    if ((rc = set_smem(generic_dkdv_kernel<T>, smem))) return rc;
    dim3 grid((a.T + BN - 1) / BN, a.B * a.H);
    generic_dkdv_kernel<T><<<grid, NT, smem, st>>>(g, mask);
    count_launch();
    if ((rc = check_launch("generic_dkdv_kernel"))) return rc;
  }
  if (any_live) {
    const size_t smem = sizeof(float) * ((size_t)4 * hd * PADW + (size_t)BM * PADW);
    if ((rc = set_smem(generic_dq_kernel<T>, smem))) return rc;
    dim3 grid((a.T + BM - 1) / BM, a.B * a.H);
    generic_dq_kernel<T><<<grid, NT, smem, st>>>(g);
    count_launch();
    if ((rc = check_launch("generic_dq_kernel"))) return rc;
  }
  return SAF_OK;
}

}  // namespace

int launch_generic_fwd(const SafMixedAttnArgs& a, uint32_t states_mask, cudaStream_t st) {
  if (a.HD > 128) return fail(SAF_ERR_UNSUPPORTED, "head_dim %d > 128", a.HD);
  if (a.T == 0 || a.B == 0 || a.H == 0) return SAF_OK;
  switch (a.dtype) {
    case SAF_F32: return fwd_typed<float>(a, states_mask, st);
    case SAF_BF16: return fwd_typed<__nv_bfloat16>(a, states_mask, st);
    case SAF_F16: return fwd_typed<__half>(a, states_mask, st);
  }
  return fail(SAF_ERR_INVALID, "unknown dtype %d", a.dtype);
}

int launch_generic_bwd(const SafMixedAttnBwdArgs& g, uint32_t states_mask, cudaStream_t st) {
  const SafMixedAttnArgs& a = g.fwd;
  if (a.HD > 128) return fail(SAF_ERR_UNSUPPORTED, "head_dim %d > 128", a.HD);
  if (a.T == 0 || a.B == 0 || a.H == 0) return SAF_OK;
  switch (a.dtype) {
    case SAF_F32: return bwd_typed<float>(g, states_mask, st);
    case SAF_BF16: return bwd_typed<__nv_bfloat16>(g, states_mask, st);
    case SAF_F16: return bwd_typed<__half>(g, states_mask, st);
  }
  return fail(SAF_ERR_INVALID, "unknown dtype %d", a.dtype);
}

}  // namespace saf
