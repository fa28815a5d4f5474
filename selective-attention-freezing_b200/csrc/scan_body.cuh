// Device code of the structured-pattern scan, shared by the stand-alone scan kernel (scan.cu) and
// by the mixed forward kernel, which runs it in the CTAs of sink+decay heads.
#pragma once
#include "saf_internal.h"

namespace saf {

constexpr int SCAN_NT = 256;
constexpr int SCAN_ROWS = 256;   // rows per block step
constexpr int SCAN_COLS = 64;    // columns per CTA

template <typename T>
__device__ __forceinline__ void load8(const T* p, int64_t sd, bool vec, int ncol, float (&v)[8]) {
  if (vec) {
    if constexpr (sizeof(T) == 2) {
      const uint4 u = *reinterpret_cast<const uint4*>(p);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        T lo, hi;
        const uint16_t l16 = (uint16_t)(w[i] & 0xffffu), h16 = (uint16_t)(w[i] >> 16);
        lo = *reinterpret_cast<const T*>(&l16);
        hi = *reinterpret_cast<const T*>(&h16);
        v[2 * i] = to_f<T>(lo);
        v[2 * i + 1] = to_f<T>(hi);
      }
    } else {
      const float4 x = *reinterpret_cast<const float4*>(p);
      const float4 y = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + 4);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
      v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (i < ncol) ? to_f<T>(p[(int64_t)i * sd]) : 0.f;
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, int64_t sd, bool vec, int ncol, const float (&v)[8]) {
  if (vec) {
    if constexpr (sizeof(T) == 2) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const T lo = from_f<T>(v[2 * i]), hi = from_f<T>(v[2 * i + 1]);
        w[i] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&lo)) | ((uint32_t)(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
      }
      *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < ncol) p[(int64_t)i * sd] = from_f<T>(v[i]);
  }
}

// (1-r) / (1 - r^(n))  =  1 / Z_{n-1};   r == 1 -> 1/n
__device__ __forceinline__ float inv_z(float r, float log_r, int n) {
  if (r >= 1.f) return 1.f / (float)n;
  if (r <= 0.f) return 1.f;
  // r^n below half an fp32 ulp of 1: Z has converged to 1 / (1 - r) (true for all but the first rows of a long
  // sequence, and the test is uniform over almost every warp: the exponential and the division are skipped)
  const float t = (float)n * log_r;
  if (t < -17.5f) return 1.f - r;
  // r^n at most 1/2: 1 - r^n has no cancellation, so the hardware exponential (2 ulp) and reciprocal (1 ulp) keep
  // the quotient within a few fp32 ulp
  if (t < -0.6931472f) return __fdividef(1.f - r, 1.f - exp2f(t * 1.4426950408889634f));
  return (1.f - r) / (-expm1f(t));
}

struct ScanArgs {
  const void* in;      // V (fwd) or dY (bwd)
  void* out;           // Y (fwd) or dV (bwd)
  int64_t si[4], so[4];
  const int32_t* frozen;
  const int32_t* kvidx;   // fwd only: input head = kvidx[h]
  const float* sd_alpha;
  const float* sd_rho;
  int B, H, T, HD, force_state, HKV;
  int vec_ok;
  int n_active;        // host hint: heads that are in the structured state (0 = unknown, all H are assumed)
};

// 256-thread barrier that leaves barrier 0 (and any other warps of the CTA) alone
__device__ __forceinline__ void scan_bar() { asm volatile("bar.sync 15, 256;" ::: "memory"); }

// Where the 64 fp32 words of a chunk's state are parked between the passes of the chunked scan: in the first
// rows of the chunk's own OUTPUT slice (64 columns x sizeof(T) bytes per row), which the last pass overwrites
// only after it has read them.  Word k of the chunk that starts at row p_lo:
template <typename T>
__device__ __forceinline__ float* scan_stash(T* ob_col0, int64_t row_stride, int p_lo, int k) {
  constexpr int PER_ROW = SCAN_COLS * (int)sizeof(T) / 4;       // fp32 words per 64-column row slice
  return reinterpret_cast<float*>(ob_col0 + (int64_t)(p_lo + k / PER_ROW) * row_stride) + (k % PER_ROW);
}

// One CTA-wide pass over positions [p_lo, p_hi) of head (b, h), columns [col0, col0+64).
// Must be called by exactly the first 256 threads of the CTA, all of them.
// MODE 0: the whole job (carry starts at zero, outputs written).
// MODE 1: state at the end of the range from a zero carry, parked in the stash; nothing else is written.
// MODE 2: carry read from the stash (before any output is written), outputs written.
// EXT: the 12.5 KB of carry / column-sum scratch live at `ext` (caller's dynamic shared memory) instead of in
// static shared memory, for kernels whose other roles need every static byte.
template <typename T, bool BWD, int MODE = 0, bool EXT = false>
__device__ __forceinline__ void sink_decay_scan_cta(const ScanArgs& a, int b, int h, int col0, int p_lo = 0,
                                                    int p_hi = -1, float* ext = nullptr) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cg = lane & 7, rl = lane >> 3;
  const int c0 = col0 + cg * 8;
  const int ncol = max(0, min(8, a.HD - c0));
  const bool vec = a.vec_ok && ncol == 8;
  const float alpha = a.sd_alpha[h], r = a.sd_rho[h];
  const float log_r = (r > 0.f && r < 1.f) ? log1pf(r - 1.f) : 0.f;
  const float r2 = r * r, r4 = r2 * r2, r8 = r4 * r4, r16 = r8 * r8, r32 = r16 * r16;
  const int hin = (!BWD && a.HKV > 0) ? (a.kvidx ? a.kvidx[h] : 0) : h;
  const T* ib = reinterpret_cast<const T*>(a.in) + (int64_t)b * a.si[0] + (int64_t)hin * a.si[1] + (int64_t)c0 * a.si[3];
  T* ob = reinterpret_cast<T*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)c0 * a.so[3];

  float (*wtot)[8][SCAN_COLS];              // [2]: double-buffered, one barrier per block step
  float (*colsum)[SCAN_COLS];               // [32]: bwd, per (warp, rl) partial column sums of dY
  float* row0;                              // [64]: bwd, scanned value of row 0
  if constexpr (EXT) {
    wtot = reinterpret_cast<float (*)[8][SCAN_COLS]>(ext);
    colsum = reinterpret_cast<float (*)[SCAN_COLS]>(ext + 2 * 8 * SCAN_COLS);
    row0 = ext + 2 * 8 * SCAN_COLS + 32 * SCAN_COLS;
  } else {
    __shared__ float wtot_s[2][8][SCAN_COLS];
    __shared__ float colsum_s[32][SCAN_COLS];
    __shared__ float row0_s[SCAN_COLS];
    wtot = wtot_s;
    colsum = colsum_s;
    row0 = row0_s;
  }

  float v0[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) v0[c] = 0.f;
  if (!BWD && ncol > 0) load8<T>(ib, a.si[3], vec, ncol, v0);
#pragma unroll
  for (int c = 0; c < 8; ++c) v0[c] *= alpha;            // the sink term a * v_0 of every output row
  float carry[8], csum[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) carry[c] = csum[c] = 0.f;
  // decay from the end of the previous warp to the start of this thread's row group
  float rg = 1.f;  // r^(8*rl)
  for (int i = 0; i < rl; ++i) rg *= r8;

  const int Tn = a.T;
  if (p_hi < 0) p_hi = Tn;
  if (MODE == 2) {
    T* ob0 = reinterpret_cast<T*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)col0 * a.so[3];
#pragma unroll
    for (int c = 0; c < 8; ++c) carry[c] = *scan_stash<T>(ob0, a.so[2], p_lo, cg * 8 + c);
    scan_bar();   // every thread holds its carry before the first output row lands on the stash
  }
  // 16-bit vector path: the next block's rows are fetched (raw 16-byte words) while this block is scanned
  const bool pf = vec && sizeof(T) == 2;
  uint4 nraw[8];
  auto prefetch = [&](int blk) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int p = blk + warp * 32 + rl * 8 + j;
      const int i = BWD ? (Tn - 1 - p) : p;
      nraw[j] = (p < p_hi) ? *reinterpret_cast<const uint4*>(ib + (int64_t)i * a.si[2]) : make_uint4(0, 0, 0, 0);
    }
  };
  if (pf) prefetch(p_lo);
  int buf = 0;
  for (int blk = p_lo; blk < p_hi; blk += SCAN_ROWS, buf ^= 1) {
    const int p0 = blk + warp * 32 + rl * 8;   // scan position of this thread's first row
    float x[8][8];
    if (pf) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t w4[4] = {nraw[j].x, nraw[j].y, nraw[j].z, nraw[j].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint16_t l16 = (uint16_t)(w4[q] & 0xffffu), h16 = (uint16_t)(w4[q] >> 16);
          x[j][2 * q] = to_f<T>(*reinterpret_cast<const T*>(&l16));
          x[j][2 * q + 1] = to_f<T>(*reinterpret_cast<const T*>(&h16));
        }
      }
      if (blk + SCAN_ROWS < p_hi) prefetch(blk + SCAN_ROWS);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int p = p0 + j;
      const int i = BWD ? (Tn - 1 - p) : p;     // memory row
      if (p < p_hi && ncol > 0) {
        if (!pf) load8<T>(ib + (int64_t)i * a.si[2], a.si[3], vec, ncol, x[j]);
        if (BWD) {
          const float w = (1.f - alpha) * inv_z(r, log_r, i + 1);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            csum[c] += x[j][c];
            x[j][c] *= w;
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) x[j][c] = 0.f;
      }
    }
    // local scan over the 8 rows
#pragma unroll
    for (int j = 1; j < 8; ++j)
#pragma unroll
      for (int c = 0; c < 8; ++c) x[j][c] = fmaf(r, x[j - 1][c], x[j][c]);
    // combine the 4 row groups of the warp (inclusive, decay r^8 per group)
    float inc[8], exc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float t = x[7][c];
      float y = __shfl_up_sync(0xffffffffu, t, 8);
      if (rl >= 1) t = fmaf(r8, y, t);
      y = __shfl_up_sync(0xffffffffu, t, 16);
      if (rl >= 2) t = fmaf(r16, y, t);
      inc[c] = t;
      y = __shfl_up_sync(0xffffffffu, t, 8);
      exc[c] = (rl >= 1) ? y : 0.f;
    }
    if (rl == 3) {
#pragma unroll
      for (int c = 0; c < 8; ++c) wtot[buf][warp][cg * 8 + c] = inc[c];
    }
    scan_bar();
    // carry into this warp = sum_{w'<warp} r32^(warp-1-w') wtot[w'] + r32^warp * carry
    float cw[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) cw[c] = carry[c];
    for (int w = 0; w < warp; ++w)
#pragma unroll
      for (int c = 0; c < 8; ++c) cw[c] = fmaf(r32, cw[c], wtot[buf][w][cg * 8 + c]);
    // block carry for the next step (all warps compute the same value)
    {
      float nc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) nc[c] = cw[c];
      for (int w = warp; w < 8; ++w)
#pragma unroll
        for (int c = 0; c < 8; ++c) nc[c] = fmaf(r32, nc[c], wtot[buf][w][cg * 8 + c]);
#pragma unroll
      for (int c = 0; c < 8; ++c) carry[c] = nc[c];
    }
    if (MODE == 1) continue;   // only the running state is wanted
    // state just before this thread's first row
    float cin[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) cin[c] = fmaf(rg, cw[c], exc[c]);
    float rp = r;  // r^(j+1)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int p = p0 + j;
      const int i = BWD ? (Tn - 1 - p) : p;
      float o[8];
      if (!BWD) {
        const float w = (1.f - alpha) * inv_z(r, log_r, i + 1);
#pragma unroll
        for (int c = 0; c < 8; ++c) o[c] = fmaf(w, fmaf(rp, cin[c], x[j][c]), v0[c]);
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) o[c] = fmaf(rp, cin[c], x[j][c]);
      }
      if (p < p_hi && ncol > 0) {
        if (BWD && i == 0) {
#pragma unroll
          for (int c = 0; c < 8; ++c) row0[cg * 8 + c] = o[c];
        } else {
          store8<T>(ob + (int64_t)i * a.so[2], a.so[3], vec, ncol, o);
        }
      }
      rp *= r;
    }
  }
  if (MODE == 1) {
    if (warp == 0 && rl == 0) {
      T* ob0 = reinterpret_cast<T*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)col0 * a.so[3];
#pragma unroll
      for (int c = 0; c < 8; ++c) *scan_stash<T>(ob0, a.so[2], p_lo, cg * 8 + c) = carry[c];
    }
    return;
  }
  if (BWD) {
    // dV_0 = scan value + alpha * sum_i dY_i
#pragma unroll
    for (int c = 0; c < 8; ++c) colsum[warp * 4 + rl][cg * 8 + c] = csum[c];
    scan_bar();
    if (tid < SCAN_COLS) {
      float s = 0.f;
      for (int k = 0; k < 32; ++k) s += colsum[k][tid];
      const int c = col0 + tid;
      if (c < a.HD && Tn > 0) {
        T* o0 = reinterpret_cast<T*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)c * a.so[3];
        *o0 = from_f<T>(row0[tid] + alpha * s);
      }
    }
  }
}

template <typename T, bool BWD>
__global__ void __launch_bounds__(SCAN_NT) sink_decay_scan_kernel(const __grid_constant__ ScanArgs a) {
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
  const int state = a.force_state >= 0 ? a.force_state : a.frozen[h];
  if (state != SAF_SINK_DECAY) return;
  sink_decay_scan_cta<T, BWD>(a, b, h, blockIdx.y * SCAN_COLS);
}

// ---- chunked forward scan: the sequence is cut into chunks of `chunk` rows that run in parallel ----------
//   pass 1  every chunk: its state at the end from a zero carry              (reads V once)
//   pass 2  per head: carries chained over the chunks, each chunk's incoming carry written back in place
//   pass 3  every chunk: scan with its carry, outputs written                 (reads V again, writes Y)
// 3/2 of the sequential scan's bytes, but nf*B*T/chunk CTAs instead of nf*B: bounded by HBM, not by latency.
template <typename T, int MODE>
__global__ void __launch_bounds__(SCAN_NT, 2) sink_decay_chunk_kernel(const __grid_constant__ ScanArgs a, int chunk) {
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
  const int state = a.force_state >= 0 ? a.force_state : a.frozen[h];
  if (state != SAF_SINK_DECAY) return;
  const int p_lo = blockIdx.y * chunk;
  sink_decay_scan_cta<T, false, MODE>(a, b, h, blockIdx.z * SCAN_COLS, p_lo, min(a.T, p_lo + chunk));
}

template <typename T>
__global__ void __launch_bounds__(SCAN_COLS) sink_decay_carry_kernel(const __grid_constant__ ScanArgs a, int chunk,
                                                                     int n_chunks) {
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
  const int state = a.force_state >= 0 ? a.force_state : a.frozen[h];
  if (state != SAF_SINK_DECAY) return;
  const int k = threadIdx.x;                 // column of the slice
  const float r = a.sd_rho[h];
  const float rL = (r <= 0.f) ? 0.f : (r >= 1.f ? 1.f : expf((float)chunk * log1pf(r - 1.f)));   // r^chunk
  T* ob0 = reinterpret_cast<T*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)(blockIdx.y * SCAN_COLS) * a.so[3];
  __shared__ float tot[64][SCAN_COLS];       // host side keeps n_chunks <= 64
  for (int c = 0; c < n_chunks; ++c) tot[c][k] = *scan_stash<T>(ob0, a.so[2], c * chunk, k);   // independent loads
  float carry = 0.f;
  for (int c = 0; c < n_chunks; ++c) {
    *scan_stash<T>(ob0, a.so[2], c * chunk, k) = carry;
    carry = fmaf(rL, carry, tot[c][k]);
  }
}

}  // namespace saf
