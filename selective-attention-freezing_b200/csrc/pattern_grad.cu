// Parameter gradients of decomposed (state 2) heads: the pattern P_ij = exp(alpha_j + rho_{i-j} - z_i), j <= i,
// is a row softmax of the logits alpha_j + rho_{i-j}, so with dP = dO V^T and delta_i = dO_i . O_i
//     dS_ij = P_ij (dP_ij - delta_i),   dalpha_j = sum_i dS_ij,   drho_d = sum_{i-j=d} dS_ij
// summed over the batch (supplement/trainable_pattern_kernels.py:21-58; the dV of these heads is the ordinary
// frozen-head backward).  No T x T buffer: column sums stay in registers, diagonal sums travel through warp
// shuffles into 255 sums per tile pair and one global atomic each.
//
//   tensor-core kernel (bf16, head_dim 64/128): one CTA per (batch, head, 128-key tile j), walks query tiles i >= j
//     dP^T = V_j dO_i^T   SS MMA 128x128xHD -> TMEM, two buffers (keys on lanes, queries on columns)
//     warps 0-7: two warpgroups split the 128 query columns; thread = key row, so dalpha_j is thread-local;
//                delta_i from the dO_i / O_i tiles in shared memory (same swizzle, so bytes pair up as they lie)
//     warp 8: TMA producer ([dO_i | O_i] ring), warp 9: MMA issuer
//   generic kernel (any dtype / head_dim): 32x32 tile pairs on the CUDA cores, fp32 throughout.
// Every wait is bounded; on expiry the kernel records a code in *status and falls through.
#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {
namespace {

constexpr float LOG2E_P = 1.4426950408889634f;
constexpr int PG_THREADS = 320;

struct PgParams {
  int B, H, T, SD, n_tiles, force_state;
  const int32_t* frozen;
  const float* alpha;
  const float* rho;
  const float* z;
  float* dalpha;
  float* drho;
  int* status;
};

struct PgShared {
  uint64_t v_full, full[3], empty[3], dp_full[2], dp_empty[2];
  uint32_t tmem_base;
  alignas(16) float z[2][128];        // z_i * log2e of the query tile (+inf past T)
  alignas(16) float dl[2][2][128];    // the two halves of delta_i
  float rw[2][256];                   // rho_d * log2e for d = D0 - 127 + k (-inf outside [0, T))
  float wb[8][2][64];                 // per warp and 32-column chunk: 63 diagonal sums of the current tile pair
};

template <int HD>
struct PgCfg {
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int NS = (HD == 64) ? 3 : 2;   // stages of [dO_i | O_i]
  static constexpr int SMEM_BYTES = 1024 + TILE_BYTES + NS * 2 * TILE_BYTES + (int)sizeof(PgShared) + 64;
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

// sum over 4 x 16 bytes of products of bf16 pairs lying at the same offsets of two tiles
__device__ __forceinline__ float pg_dot16(const uint8_t* a, const uint8_t* b) {
  const uint4 x = *reinterpret_cast<const uint4*>(a), y = *reinterpret_cast<const uint4*>(b);
  const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    s = fmaf(__uint_as_float(xs[k] << 16), __uint_as_float(ys[k] << 16), s);
    s = fmaf(__uint_as_float(xs[k] & 0xffff0000u), __uint_as_float(ys[k] & 0xffff0000u), s);
  }
  return s;
}

template <int HD>
__global__ void __launch_bounds__(PG_THREADS, 1)
pattern_grad_kernel(const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapdO,
                    const __grid_constant__ CUtensorMap mapO, const __grid_constant__ PgParams p) {
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
  uint8_t* ring = smem + C::TILE_BYTES;               // stage s: [dO_i | O_i]
  PgShared* sh = reinterpret_cast<PgShared*>(ring + C::NS * 2 * C::TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5;

  if (tid == 0) {
    mbar_init(&sh->v_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 257);      // the MMA's commit + every compute thread (delta reads the tiles)
    }
    for (int k = 0; k < 2; ++k) {
      mbar_init(&sh->dp_full[k], 1);
      mbar_init(&sh->dp_empty[k], 256);
    }
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(&sh->tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&mapV);
      tma_prefetch_desc(&mapdO);
      tma_prefetch_desc(&mapO);
      mbar_expect_tx(&sh->v_full, C::TILE_BYTES);
      pg_load_tile<HD>(sV, &mapV, &sh->v_full, j0, h, b);
      for (int i = 0; i < n; ++i) {
        const int s = i % C::NS;
        if (!mbar_wait(&sh->empty[s], ((i / C::NS) & 1) ^ 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 70);
          break;
        }
        uint8_t* dst = ring + s * 2 * C::TILE_BYTES;
        mbar_expect_tx(&sh->full[s], 2 * C::TILE_BYTES);
        pg_load_tile<HD>(dst, &mapdO, &sh->full[s], (jt + i) * 128, h, b);
        pg_load_tile<HD>(dst + C::TILE_BYTES, &mapO, &sh->full[s], (jt + i) * 128, h, b);
      }
    }
  } else if (warp == 9) {
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
        const uint32_t adO = aR + s * 2 * C::TILE_BYTES;
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
    const int half = warp >> 2;
    const int r = tid & 127;                       // key row of the tile
    const int cb = half * 64;                      // first query column of this group
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int64_t vrow = (int64_t)h * p.SD;
    const float a_r = (j0 + r < p.T) ? p.alpha[vrow + j0 + r] * LOG2E_P : -INFINITY;
    float acc_a = 0.f;
    auto fetch_z = [&](int qt) -> float {
      const int row = qt * 128 + r;
      return row < p.T ? p.z[vrow + row] * LOG2E_P : INFINITY;    // +inf: P = 0 past T
    };
    auto fetch_rho = [&](int qt) -> float {
      const int d = (qt - jt) * 128 - 127 + tid;
      return (d >= 0 && d < p.T) ? p.rho[vrow + d] * LOG2E_P : -INFINITY;   // -inf: above the diagonal
    };
    float nz = tid < 128 ? fetch_z(jt) : 0.f;
    float nr = fetch_rho(jt);
    for (int i = 0; i < n; ++i) {
      const int s = i % C::NS, k = i & 1;
      if (!mbar_wait(&sh->full[s], (i / C::NS) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 73);
        break;
      }
      {
        // half of delta_i for row r: both tiles carry the same swizzle, so equal offsets hold equal (row, column)
        const uint8_t* tdo = ring + s * 2 * C::TILE_BYTES;
        const uint8_t* to = tdo + C::TILE_BYTES;
        float dsum = 0.f;
        if (HD == 64) {
          const int o0 = r * 128 + half * 64;
#pragma unroll
          for (int c = 0; c < 4; ++c) dsum += pg_dot16(tdo + o0 + c * 16, to + o0 + c * 16);
        } else {
          const int o0 = half * 16384 + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) dsum += pg_dot16(tdo + o0 + c * 16, to + o0 + c * 16);
        }
        sh->dl[k][half][r] = dsum;
      }
      if (tid < 128) sh->z[k][r] = nz;
      sh->rw[k][tid] = nr;
      named_bar_sync(1, 256);
      mbar_arrive(&sh->empty[s]);
      if (i + 1 < n) {
        if (tid < 128) nz = fetch_z(jt + i + 1);
        nr = fetch_rho(jt + i + 1);
      }
      if (!mbar_wait(&sh->dp_full[k], (i >> 1) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 74);
        break;
      }
      tc_fence_after();
      uint32_t d[2][32];
      tmem_ld32(tmem + lane_base + k * 128 + cb, d[0]);
      tmem_ld32(tmem + lane_base + k * 128 + cb + 32, d[1]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&sh->dp_empty[k]);
      // Diagonal sums without atomics: a running sum travels one lane up per column (the cell one column to the
      // right and one row down lies on the same diagonal), so a diagonal's partial sum stays in registers until
      // it leaves lane 31 or the chunk ends; every slot of the warp's array is then written exactly once.
      // The two 32-column chunks are independent chains, interleaved for latency.
      const float* rw = &sh->rw[k][cb - r + 127];
      float* wb0 = sh->wb[warp][0];
      float* wb1 = sh->wb[warp][1];
      const int lane = tid & 31;
      float run0 = 0.f, run1 = 0.f;
      const float4* Z4 = reinterpret_cast<const float4*>(&sh->z[k][cb]);
      const float4* A4 = reinterpret_cast<const float4*>(&sh->dl[k][0][cb]);
      const float4* B4 = reinterpret_cast<const float4*>(&sh->dl[k][1][cb]);
#pragma unroll
      for (int x4 = 0; x4 < 8; ++x4) {
        const float4 Za = Z4[x4], Aa = A4[x4], Ba = B4[x4];
        const float4 Zb = Z4[8 + x4], Ab = A4[8 + x4], Bb = B4[8 + x4];
        const float z0[4] = {Za.x, Za.y, Za.z, Za.w}, z1[4] = {Zb.x, Zb.y, Zb.z, Zb.w};
        const float d0[4] = {Aa.x + Ba.x, Aa.y + Ba.y, Aa.z + Ba.z, Aa.w + Ba.w};
        const float d1[4] = {Ab.x + Bb.x, Ab.y + Bb.y, Ab.z + Bb.z, Ab.w + Bb.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int x = x4 * 4 + e;
          const float p0 = pg_ex2(a_r + rw[x] - z0[e]);
          const float p1 = pg_ex2(a_r + rw[32 + x] - z1[e]);
          const float ds0 = p0 * (__uint_as_float(d[0][x]) - d0[e]);
          const float ds1 = p1 * (__uint_as_float(d[1][x]) - d1[e]);
          acc_a += ds0 + ds1;
          if (x > 0 && lane == 31) {
            wb0[x - 1] = run0;
            wb1[x - 1] = run1;
          }
          run0 = __shfl_up_sync(0xffffffffu, run0, 1);
          run1 = __shfl_up_sync(0xffffffffu, run1, 1);
          if (lane == 0) run0 = run1 = 0.f;
          run0 += ds0;
          run1 += ds1;
        }
      }
      wb0[62 - lane] = run0;
      wb1[62 - lane] = run1;
      named_bar_sync(1, 256);
      if (tid < 255) {
        // tile diagonal t = (query column) - (key row) + 127; slot m of (warp, chunk) is column - lane + 31
        float val = 0.f;
#pragma unroll
        for (int wq = 0; wq < 8; ++wq)
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            const int m = tid - 96 - 64 * (wq >> 2) - 32 * ch + 32 * (wq & 3);
            if (m >= 0 && m < 63) val += sh->wb[wq][ch][m];
          }
        const int dist = i * 128 - 127 + tid;
        if (val != 0.f && dist >= 0 && dist < p.T) atomicAdd(&p.drho[vrow + dist], val);
      }
    }
    if (j0 + r < p.T && acc_a != 0.f) atomicAdd(&p.dalpha[vrow + j0 + r], acc_a);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::TMEM_COLS);
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

bool pg_tensor_ok(const SafTensor& t) {
  if (!t.ptr || ((uintptr_t)t.ptr & 15) || t.stride[3] != 1) return false;
  for (int i = 0; i < 3; ++i)
    if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
  return true;
}

int pg_map4(CUtensorMap* m, const SafTensor& t, int B, int Hn, int T, int HD) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)T, (uint64_t)Hn, (uint64_t)B};
  uint64_t strides[4] = {0, (uint64_t)t.stride[2] * 2, (uint64_t)t.stride[1] * 2, (uint64_t)t.stride[0] * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tensor_map_bf16(m, t.ptr, 4, dims, strides, box, true);
}

template <int HD>
int pg_launch_sm100(const SafPatternGradArgs& a, cudaStream_t st) {
  CUtensorMap mv, mdo, mo;
  int rc;
  if ((rc = pg_map4(&mv, a.v, a.B, a.H, a.T, HD))) return rc;
  if ((rc = pg_map4(&mdo, a.dout, a.B, a.H, a.T, HD))) return rc;
  if ((rc = pg_map4(&mo, a.out, a.B, a.H, a.T, HD))) return rc;
  PgParams p;
  p.B = a.B; p.H = a.H; p.T = a.T; p.SD = a.SD;
  p.n_tiles = (a.T + 127) / 128;
  p.force_state = a.force_state;
  p.frozen = a.frozen;
  p.alpha = a.alpha; p.rho = a.rho; p.z = a.z;
  p.dalpha = a.dalpha; p.drho = a.drho;
  p.status = a.status;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(pattern_grad_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         PgCfg<HD>::SMEM_BYTES);
    if (e != cudaSuccess) return fail(SAF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  const int64_t grid = (int64_t)a.B * a.H * p.n_tiles;
  if (grid > 0x7fffffff) return fail(SAF_ERR_LIMIT, "pattern gradient grid too large");
  pattern_grad_kernel<HD><<<(unsigned)grid, PG_THREADS, PgCfg<HD>::SMEM_BYTES, st>>>(mv, mdo, mo, p);
  count_launch();
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
  static int attr_bytes = 0;
  if (smem > 48 * 1024 && smem > attr_bytes) {
    cudaError_t e = cudaFuncSetAttribute(pattern_grad_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(SAF_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_bytes = smem;
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
  const bool tc = a.dtype == SAF_BF16 && (a.HD == 64 || a.HD == 128) && pg_tensor_ok(a.v) && pg_tensor_ok(a.dout) &&
                  pg_tensor_ok(a.out) && a.v.stride[3] == 1 && saf_device_supported();
  if (tc) return a.HD == 64 ? pg_launch_sm100<64>(a, st) : pg_launch_sm100<128>(a, st);
  return pg_launch_generic(a, st);
}

}  // namespace saf
