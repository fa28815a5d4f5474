// Parameter gradients of decomposed (state 2) heads: the pattern P_ij = exp(alpha_j + rho_{i-j} - z_i), j <= i,
// is a row softmax of the logits alpha_j + rho_{i-j}, so with dP = dO V^T and delta_i = dO_i . O_i
//     dS_ij = P_ij (dP_ij - delta_i),   dalpha_j = sum_i dS_ij,   drho_d = sum_{i-j=d} dS_ij
// summed over the batch (supplement/trainable_pattern_kernels.py:21-58; the dV of these heads is the ordinary
// frozen-head backward).  No T x T buffer: column sums stay in registers, diagonal sums travel through warp
// shuffles into 255 sums per tile pair and one global atomic each.
//
//   tensor-core kernel (bf16, head_dim 64/128): one CTA per (batch, head, 128-key tile j), walks query tiles i >= j
//     dP^T = V_j dO_i^T   SS MMA 128x128xHD -> TMEM, two buffers (keys on lanes, queries on columns)
//     warps 0-15: four warpgroups split the 128 query columns; thread = key row, so dalpha_j is thread-local;
//                 delta_i comes from a small pre-pass (one warp per row)
//     warp 16: TMA producer (dO_i ring), warp 17: MMA issuer
//   generic kernel (any dtype / head_dim): 32x32 tile pairs on the CUDA cores, fp32 throughout.
// Every wait is bounded; on expiry the kernel records a code in *status and falls through.
#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {
namespace {

constexpr float LOG2E_P = 1.4426950408889634f;
constexpr int PG_COMPUTE = 512;                 // 16 warps: four warpgroups, 32 query columns each
constexpr int PG_THREADS = PG_COMPUTE + 64;     // + TMA producer warp + MMA issuer warp

struct PgParams {
  int B, H, T, SD, n_tiles, force_state;
  const int32_t* frozen;
  const float* alpha;
  const float* rho;
  const float* z;
  const float* delta;       // (B, H, T) from the pre-pass
  float* dalpha;
  float* drho;
  int* status;
};

struct PgShared {
  uint64_t v_full, full[4], empty[4], dp_full[2], dp_empty[2];
  uint32_t tmem_base;
  alignas(16) float z[128];          // z_i * log2e of the query tile (+inf past T)
  alignas(16) float dl[128];         // delta_i
  float rw[256];                     // rho_d * log2e for d = D0 - 127 + k (-inf outside [0, T))
  alignas(16) float wb[16][64];      // per warp: 63 diagonal sums of the current tile pair
};

template <int HD>
struct PgCfg {
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int NS = 4;                     // dO_i ring
  static constexpr int SMEM_BYTES = 1024 + TILE_BYTES + NS * TILE_BYTES + (int)sizeof(PgShared) + 64;
  static constexpr int TMEM_COLS = 256;
};

__device__ __forceinline__ float pg_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD>
__device__ __forceinline__ void pg_load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row, int head, int b) {
#pragma unroll
  for (int hh = 0; hh < HD / 64; ++hh) tma_load_4d(dst + hh * 16384, m, bar, hh * 64, row, head, b);
}

// delta[b,h,i] = sum_d dO[b,h,i,d] O[b,h,i,d] for the heads that train; one warp per row
struct PgDeltaParams {
  int B, H, T, HD, force_state;
  const int32_t* frozen;
  const __nv_bfloat16* o;
  const __nv_bfloat16* g;
  int64_t o_s[3], g_s[3];
  float* delta;
};

__global__ void __launch_bounds__(256) pattern_delta_kernel(const PgDeltaParams p) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (int64_t)p.B * p.H * p.T) return;
  const int t = (int)(row % p.T);
  const int h = (int)((row / p.T) % p.H), b = (int)(row / ((int64_t)p.T * p.H));
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  if (state != SAF_DECOMP) return;
  const __nv_bfloat16* o = p.o + b * p.o_s[0] + h * p.o_s[1] + t * p.o_s[2];
  const __nv_bfloat16* g = p.g + b * p.g_s[0] + h * p.g_s[1] + t * p.g_s[2];
  float s = 0.f;
  for (int c = lane * 2; c < p.HD; c += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + c));
    const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + c));
    s = fmaf(a.x, d.x, fmaf(a.y, d.y, s));
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) p.delta[row] = s;
}

template <int HD>
__global__ void __launch_bounds__(PG_THREADS, 1)
pattern_grad_kernel(const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapdO,
                    const __grid_constant__ PgParams p) {
  using C = PgCfg<HD>;
  const int BH = p.B * p.H;
  const int bh = (int)blockIdx.x % BH, jt = (int)blockIdx.x / BH;    // heaviest key tiles (most query tiles) first
  const int b = bh / p.H, h = bh % p.H;
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  if (state != SAF_DECOMP) return;
  const int n = p.n_tiles - jt;
  const int j0 = jt * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sV = smem;
  uint8_t* ring = smem + C::TILE_BYTES;               // dO_i stages
  PgShared* sh = reinterpret_cast<PgShared*>(ring + C::NS * C::TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5;
  constexpr int W_TMA = PG_COMPUTE / 32, W_MMA = W_TMA + 1;

  if (tid == 0) {
    mbar_init(&sh->v_full, 1);
    for (int s = 0; s < C::NS; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);        // the MMA's commit: nothing else reads a dO stage
    }
    for (int k = 0; k < 2; ++k) {
      mbar_init(&sh->dp_full[k], 1);
      mbar_init(&sh->dp_empty[k], PG_COMPUTE / 32);   // one lane of every compute warp
    }
    fence_mbar_init();
  }
  if (warp == W_MMA) {
    tmem_alloc(&sh->tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == W_TMA) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&mapV);
      tma_prefetch_desc(&mapdO);
      mbar_expect_tx(&sh->v_full, C::TILE_BYTES);
      pg_load_tile<HD>(sV, &mapV, &sh->v_full, j0, h, b);
      for (int i = 0; i < n; ++i) {
        const int s = i % C::NS;
        if (!mbar_wait(&sh->empty[s], ((i / C::NS) & 1) ^ 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 70);
          break;
        }
        mbar_expect_tx(&sh->full[s], C::TILE_BYTES);
        pg_load_tile<HD>(ring + s * C::TILE_BYTES, &mapdO, &sh->full[s], (jt + i) * 128, h, b);
      }
    }
  } else if (warp == W_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
    const uint32_t aV = smem_u32(sV), aR = smem_u32(ring);
    bool ok = mbar_wait(&sh->v_full, 0);
    if (!ok) dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 71);
    for (int i = 0; i < n && ok; ++i) {
      const int s = i % C::NS, k = i & 1;
      if (!mbar_wait(&sh->full[s], (i / C::NS) & 1) || !mbar_wait(&sh->dp_empty[k], ((i >> 1) & 1) ^ 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 72);
        break;
      }
      tc_fence_after();
      if (leader) {
        const uint32_t adO = aR + s * C::TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
          umma_ss(tmem + k * 128, umma_smem_desc_sw128(aV + off, 16, 1024), umma_smem_desc_sw128(adO + off, 16, 1024),
                  idesc, ks > 0);
        }
        umma_commit(&sh->dp_full[k]);
        umma_commit(&sh->empty[s]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    const int quarter = warp >> 2;
    const int r = tid & 127;                       // key row of the tile
    const int lane = tid & 31;
    const int cb = quarter * 32;                   // first query column of this group
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int64_t vrow = (int64_t)h * p.SD;
    const float* delta_g = p.delta + ((int64_t)b * p.H + h) * p.T;
    const float a_r = (j0 + r < p.T) ? p.alpha[vrow + j0 + r] * LOG2E_P : -INFINITY;
    float acc_a = 0.f;
    // every thread stages one value of the next tile's vectors: z (threads 0-127), delta (128-255), rho window (256-511)
    auto fetch = [&](int qt) -> float {
      if (tid < 128) {
        const int row = qt * 128 + tid;
        return row < p.T ? p.z[vrow + row] * LOG2E_P : INFINITY;            // +inf: P = 0 past T
      }
      if (tid < 256) {
        const int row = qt * 128 + tid - 128;
        return row < p.T ? delta_g[row] : 0.f;
      }
      const int d = (qt - jt) * 128 - 127 + (tid - 256);
      return (d >= 0 && d < p.T) ? p.rho[vrow + d] * LOG2E_P : -INFINITY;   // -inf: above the diagonal
    };
    float nxt = fetch(jt);
    float* slot = tid < 128 ? &sh->z[tid] : tid < 256 ? &sh->dl[tid - 128] : &sh->rw[tid - 256];
    for (int i = 0; i < n; ++i) {
      const int k = i & 1;
      *slot = nxt;
      named_bar_sync(1, PG_COMPUTE);
      if (i + 1 < n) nxt = fetch(jt + i + 1);
      if (!mbar_wait(&sh->dp_full[k], (i >> 1) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 74);
        break;
      }
      tc_fence_after();
      uint32_t d[32];
      tmem_ld32(tmem + lane_base + k * 128 + cb, d);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->dp_empty[k]);
      // Diagonal sums without atomics: a running sum travels one lane up per column (the cell one column to the
      // right and one row down lies on the same diagonal), so a diagonal's partial sum stays in registers until
      // it leaves lane 31 or the chunk ends; every slot of the warp's array is then written exactly once.
      const float* rw = &sh->rw[cb - r + 127];
      float* wb = sh->wb[warp];
      float run = 0.f;
      float keep[3];
      const float4* Z4 = reinterpret_cast<const float4*>(&sh->z[cb]);
      const float4* D4 = reinterpret_cast<const float4*>(&sh->dl[cb]);
#pragma unroll
      for (int x4 = 0; x4 < 8; ++x4) {
        const float4 Z = Z4[x4], D = D4[x4];
        const float zz[4] = {Z.x, Z.y, Z.z, Z.w}, dd[4] = {D.x, D.y, D.z, D.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int x = x4 * 4 + e;
          const float pe = pg_ex2(a_r + rw[x] - zz[e]);
          const float ds = pe * (__uint_as_float(d[x]) - dd[e]);
          acc_a += ds;
          // lane 31 holds the finished sum of diagonal slot x-1: kept in registers, stored four at a time
          if (x > 0) {
            const int m = x - 1;
            if ((m & 3) == 3) {
              if (lane == 31) *reinterpret_cast<float4*>(&wb[m - 3]) = make_float4(keep[0], keep[1], keep[2], run);
            } else {
              keep[m & 3] = run;
            }
          }
          run = __shfl_up_sync(0xffffffffu, run, 1);
          if (lane == 0) run = 0.f;
          run += ds;
        }
      }
      if (lane == 31) {          // slots 28..30 left in the registers
#pragma unroll
        for (int m = 0; m < 3; ++m) wb[28 + m] = keep[m];
      }
      wb[62 - lane] = run;
      named_bar_sync(1, PG_COMPUTE);
      if (tid < 255) {
        // tile diagonal t = (query column) - (key row) + 127; slot m of a warp is column - lane + 31
        float val = 0.f;
#pragma unroll
        for (int wq = 0; wq < PG_COMPUTE / 32; ++wq) {
          const int m = tid - 96 - 32 * (wq >> 2) + 32 * (wq & 3);
          if (m >= 0 && m < 63) val += sh->wb[wq][m];
        }
        const int dist = i * 128 - 127 + tid;
        if (val != 0.f && dist >= 0 && dist < p.T) atomicAdd(&p.drho[vrow + dist], val);
      }
    }
    if (j0 + r < p.T && acc_a != 0.f) atomicAdd(&p.dalpha[vrow + j0 + r], acc_a);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) tmem_dealloc(tmem, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// CUDA-core version: any dtype, any head_dim <= 256.  One CTA per (32-row query tile, head, batch);
// 16 x 16 threads, each owning a 2 x 2 patch of a 32 x 32 tile pair.
// ---------------------------------------------------------------------------------------------
struct PgGenericParams {
  int B, H, T, HD, SD, force_state, dtype;
  const void* v;
  const void* dout;
  const void* out;
  int64_t v_s[3], do_s[3], o_s[3];
  const int32_t* frozen;
  const float* alpha;
  const float* rho;
  const float* z;
  float* dalpha;
  float* drho;
};

__global__ void __launch_bounds__(256) pattern_grad_generic_kernel(const PgGenericParams p) {
  const int it = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  if (state != SAF_DECOMP) return;
  extern __shared__ float pg_sm[];
  const int ld = p.HD + 1;
  float* sg = pg_sm;                 // dO rows of the query tile
  float* sv = sg + 32 * ld;          // V rows of the key tile
  float* sdelta = sv + 32 * ld;      // 32
  float* sz = sdelta + 32;           // 32
  float* scol = sz + 32;             // 32 column sums
  float* sdiag = scol + 32;          // 63 diagonal sums
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int i0 = it * 32;
  const int64_t vrow = (int64_t)h * p.SD;
  const int64_t gb = (int64_t)b * p.do_s[0] + (int64_t)h * p.do_s[1];
  const int64_t ob = (int64_t)b * p.o_s[0] + (int64_t)h * p.o_s[1];
  const int64_t vb = (int64_t)b * p.v_s[0] + (int64_t)h * p.v_s[1];
  for (int e = tid; e < 32 * p.HD; e += 256) {
    const int rr = e / p.HD, cc = e - rr * p.HD;
    sg[rr * ld + cc] = (i0 + rr < p.T) ? load_rt(p.dout, gb + (int64_t)(i0 + rr) * p.do_s[2] + cc, p.dtype) : 0.f;
  }
  __syncthreads();
  if (tid < 32) {
    float s = 0.f;
    if (i0 + tid < p.T)
      for (int c = 0; c < p.HD; ++c)
        s = fmaf(sg[tid * ld + c], load_rt(p.out, ob + (int64_t)(i0 + tid) * p.o_s[2] + c, p.dtype), s);
    sdelta[tid] = s;
    sz[tid] = (i0 + tid < p.T) ? p.z[vrow + i0 + tid] : INFINITY;
  }
  for (int jt = 0; jt <= it; ++jt) {
    const int j0 = jt * 32;
    __syncthreads();
    for (int e = tid; e < 32 * p.HD; e += 256) {
      const int rr = e / p.HD, cc = e - rr * p.HD;
      sv[rr * ld + cc] = (j0 + rr < p.T) ? load_rt(p.v, vb + (int64_t)(j0 + rr) * p.v_s[2] + cc, p.dtype) : 0.f;
    }
    if (tid < 32) scol[tid] = 0.f;
    if (tid < 63) sdiag[tid] = 0.f;
    __syncthreads();
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int c = 0; c < p.HD; ++c) {
      const float g0 = sg[ty * ld + c], g1 = sg[(ty + 16) * ld + c];
      const float v0 = sv[tx * ld + c], v1 = sv[(tx + 16) * ld + c];
      acc[0][0] = fmaf(g0, v0, acc[0][0]);
      acc[0][1] = fmaf(g0, v1, acc[0][1]);
      acc[1][0] = fmaf(g1, v0, acc[1][0]);
      acc[1][1] = fmaf(g1, v1, acc[1][1]);
    }
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int li = ty + 16 * a, lj = tx + 16 * c;
        const int i = i0 + li, j = j0 + lj;
        if (i < p.T && j <= i) {
          const float pe = expf(p.alpha[vrow + j] + p.rho[vrow + i - j] - sz[li]);
          const float ds = pe * (acc[a][c] - sdelta[li]);
          atomicAdd(&scol[lj], ds);
          atomicAdd(&sdiag[li - lj + 31], ds);
        }
      }
    __syncthreads();
    if (tid < 32 && j0 + tid < p.T && scol[tid] != 0.f) atomicAdd(&p.dalpha[vrow + j0 + tid], scol[tid]);
    if (tid >= 64 && tid < 127) {
      const int k = tid - 64, dist = i0 - j0 + k - 31;
      if (dist >= 0 && dist < p.T && sdiag[k] != 0.f) atomicAdd(&p.drho[vrow + dist], sdiag[k]);
    }
  }
}

template <int HD>
int pg_launch_sm100(const SafPatternGradArgs& a, cudaStream_t st) {
  CUtensorMap mv, mdo;
  int rc;
  if ((rc = make_row_tile_map_bf16(&mv, a.v, a.B, a.H, a.T, HD))) return rc;
  if ((rc = make_row_tile_map_bf16(&mdo, a.dout, a.B, a.H, a.T, HD))) return rc;
  PgDeltaParams d;
  d.B = a.B; d.H = a.H; d.T = a.T; d.HD = HD;
  d.force_state = a.force_state;
  d.frozen = a.frozen;
  d.o = reinterpret_cast<const __nv_bfloat16*>(a.out.ptr);
  d.g = reinterpret_cast<const __nv_bfloat16*>(a.dout.ptr);
  for (int i = 0; i < 3; ++i) {
    d.o_s[i] = a.out.stride[i];
    d.g_s[i] = a.dout.stride[i];
  }
  d.delta = a.delta;
  PgParams p;
  p.B = a.B; p.H = a.H; p.T = a.T; p.SD = a.SD;
  p.n_tiles = (a.T + 127) / 128;
  p.force_state = a.force_state;
  p.frozen = a.frozen;
  p.alpha = a.alpha; p.rho = a.rho; p.z = a.z;
  p.delta = a.delta;
  p.dalpha = a.dalpha; p.drho = a.drho;
  p.status = a.status;
  static PerDeviceOnce smem_once;
  if (int rc2 = ensure_dyn_smem(pattern_grad_kernel<HD>, PgCfg<HD>::SMEM_BYTES, smem_once)) return rc2;
  const int64_t rows = (int64_t)a.B * a.H * a.T;
  const int64_t grid = (int64_t)a.B * a.H * p.n_tiles;
  if (grid > 0x7fffffff || (rows + 7) / 8 > 0x7fffffff) return fail(SAF_ERR_LIMIT, "pattern gradient grid too large");
  pattern_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(d);
  pattern_grad_kernel<HD><<<(unsigned)grid, PG_THREADS, PgCfg<HD>::SMEM_BYTES, st>>>(mv, mdo, p);
  count_launch(2);
  return check_launch("pattern_grad_kernel");
}

int pg_launch_generic(const SafPatternGradArgs& a, cudaStream_t st) {
  if (a.HD > 256) return fail(SAF_ERR_LIMIT, "pattern gradient: head_dim > 256");
  PgGenericParams p;
  p.B = a.B; p.H = a.H; p.T = a.T; p.HD = a.HD; p.SD = a.SD;
  p.force_state = a.force_state;
  p.dtype = a.dtype;
  p.v = a.v.ptr; p.dout = a.dout.ptr; p.out = a.out.ptr;
  for (int i = 0; i < 3; ++i) {
    p.v_s[i] = a.v.stride[i];
    p.do_s[i] = a.dout.stride[i];
    p.o_s[i] = a.out.stride[i];
  }
  p.frozen = a.frozen;
  p.alpha = a.alpha; p.rho = a.rho; p.z = a.z;
  p.dalpha = a.dalpha; p.drho = a.drho;
  const int smem = (2 * 32 * (a.HD + 1) + 32 * 3 + 64) * (int)sizeof(float);
  if (smem > 48 * 1024) {
    // head_dim <= 256 bounds this at 66.8 KB: raise the limit to that maximum once per device
    static PerDeviceOnce smem_once;
    constexpr int SMEM_MAX = (2 * 32 * (256 + 1) + 32 * 3 + 64) * (int)sizeof(float);
    if (int rc2 = ensure_dyn_smem(pattern_grad_generic_kernel, SMEM_MAX, smem_once)) return rc2;
  }
  const int nt = (a.T + 31) / 32;
  if (a.H > 65535 || a.B > 65535) return fail(SAF_ERR_LIMIT, "pattern gradient: B or H > 65535");
  pattern_grad_generic_kernel<<<dim3(nt, a.H, a.B), 256, smem, st>>>(p);
  count_launch();
  return check_launch("pattern_grad_generic_kernel");
}

}  // namespace

int launch_pattern_grad(const SafPatternGradArgs& a, cudaStream_t st) {
  if (a.frozen_host && a.force_state < 0) {
    bool any = false;
    for (int h = 0; h < a.H; ++h) any |= a.frozen_host[h] == SAF_DECOMP;
    if (!any) return SAF_OK;
  }
  const bool tc = a.dtype == SAF_BF16 && (a.HD == 64 || a.HD == 128) && tma_rows_ok(a.v) && tma_rows_ok(a.dout) &&
                  tma_rows_ok(a.out) && a.delta && saf_device_supported();   // the pre-pass reads out / dout as bf16 pairs
  if (tc) return a.HD == 64 ? pg_launch_sm100<64>(a, st) : pg_launch_sm100<128>(a, st);
  return pg_launch_generic(a, st);
}

}  // namespace saf
