// Backward of the live (flash) heads on tcgen05 / TMEM, fed by TMA.
//
// Same split as the reference (kernel/fused_attn.py:291-540, 593-623: _bwd_preprocess, _bwd_dkdv, _bwd_dq):
// no atomics, deterministic, dq/dk/dv written once.
//
//   delta kernel   delta_i = sum_d O_id dO_id                                   (HBM-bound, 16-byte loads)
//   dK/dV kernel   one CTA per 128-key tile j; walks the query tiles i >= j:
//                    S^T  = K_j Q_i^T            SS MMA 128x128xHD -> TMEM   (keys on lanes, queries on columns)
//                    dP^T = V_j dO_i^T           SS MMA 128x128xHD -> TMEM
//                    P^T  = exp2(S^T scale - lse_i)   , bf16 back into the S^T columns
//                    dS^T = P^T (dP^T - delta_i)      , bf16 back into the dP^T columns
//                    dV_j += P^T  dO_i           TS MMA (A from TMEM, dO_i MN-major from the same smem tile)
//                    dK_j += dS^T Q_i            TS MMA
//                  computing the transposed tiles directly puts P^T / dS^T in the layout the TS MMA wants,
//                  so nothing is transposed through shared memory.
//   dQ kernel      one CTA per 128-row query tile i; walks the key tiles j <= i:
//                    S = Q_i K_j^T, dP = dO_i V_j^T, dS = P (dP - delta), dQ_i += dS K_j   (TS MMA)
//
// CTA = 384 threads: warps 0-3 and 4-7 are two compute warpgroups that split the 128 columns of a tile in
// halves (TMEM lane = row = thread; both groups cover all 128 lanes), warp 8 TMA producer, warp 9 MMA
// issuer (whole warp walks the schedule, one elected lane issues), warps 10-11 complete the third
// warpgroup for the register reallocation.  The bf16 operand the compute warpgroups write lands in the
// first 64 columns of the tile they read (see operand_columns_read); the TS MMA takes K step ks from
// columns 8 ks.
// The sm_scale factor of dS is applied once to the finished dK / dQ accumulators.
// Every wait is bounded; on expiry the kernel records a code in *status and falls through.
#include "saf_internal.h"
#include "dense_pv_body.cuh"
#include "scan_body.cuh"
#include "sm100_prims.cuh"
#include <string.h>

namespace saf {
namespace {

constexpr int BWD_THREADS = 384;
constexpr int BWD_HEAD_GROUP = 8;
constexpr float LOG2E_B = 1.4426950408889634f;

#ifdef SAF_BWD_TRACE
// timing probe (only in specially built libraries): clock64 stamps of one CTA's pipeline events
__device__ long long g_trace[2][8][64];   // [kernel][event][tile]
#define TRACE(kern, evt, tile) do { if (trace_on && (tile) < 64) g_trace[kern][evt][tile] = clock64(); } while (0)
__device__ long long g_wtrace[8][2][64];  // dK/dV kernel, per compute warp: [warp][P^T / dS^T handed over][tile]
#define WTRACE(evt, tile) do { if (wtrace_on && (tile) < 64) g_wtrace[warp][evt][tile] = clock64(); } while (0)
#else
#define TRACE(kern, evt, tile) do { } while (0)
#define WTRACE(evt, tile) do { } while (0)
#endif

template <int HD>
struct BwdCfg {
  static constexpr int TILE_BYTES = 128 * HD * 2;
  // dK/dV kernel: Q_i lives from S^T(i) to dK(i), dO_i from dP^T(i) to dV(i); the Q ring is the one whose
  // refill sits on the critical path, so it gets the third stage even at head_dim 128
  static constexpr int NQ = 3;
  static constexpr int ND = (HD == 64) ? 3 : 2;
  static constexpr int KS = 3;                        // dQ kernel: K ring (a K tile lives until its dQ product)
  static constexpr int VS = (HD == 64) ? 3 : 2;       // dQ kernel: V ring (a V tile is done after its dP product)
  static constexpr int SMEM_DKDV = 1024 + 2 * TILE_BYTES + (NQ + ND) * TILE_BYTES + 256 + 1040;
  // the dK/dV launch also hosts the dense-pattern dV role, which brings its own ring
  static constexpr int SMEM_BYTES = SMEM_DKDV > DpCfg<HD>::SMEM_BYTES ? SMEM_DKDV : DpCfg<HD>::SMEM_BYTES;
  static constexpr int SMEM_BYTES_DQ = 1024 + 2 * TILE_BYTES + (KS + VS) * TILE_BYTES + 512;
  static constexpr int TMEM_COLS = 512;
};

struct BwdParams {
  int B, H, T, n_tiles, force_state;
  float scale_log2, sm_scale;
  const int32_t* frozen;
  const int32_t* hidx;
  const float* lse;
  int64_t lse_s[3];
  float* delta;
  int64_t delta_s[3];
  int* status;
  // structured frozen heads: their reverse scan (dV = P^T dO) runs in the leading CTAs of the dK/dV launch
  int scan_slots;
  ScanArgs scan;
  // dense-stored frozen heads: dV = tril(P)^T dO as a TMA-staged GEMM in the next CTAs of the dK/dV launch
  int dense_slots;
  DpParams dense;
};

struct BwdBars {
  uint64_t res_full;                    // the two resident tiles
  uint64_t ring_full[3], ring_empty[3];
  uint64_t v_full[3], v_empty[3];       // dQ kernel: the V ring (ring_* is its K ring)
  uint64_t s_full[2], dp_full, p_full, ds_full, acc_full;
  uint32_t tmem_base;
};
static_assert(sizeof(BwdBars) <= 256, "barrier block");
// dK/dV kernel only, placed 256 bytes after the barriers: lse and delta of the current query tile (read as float4)
struct BwdVectors {
  alignas(16) float lse[128];
  alignas(16) float dl[128];
};

__device__ __forceinline__ float ex2b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
#ifndef SAF_BWD_POLY_PER_8
#define SAF_BWD_POLY_PER_8 4        // of every 8 exponentials, this many run on the FMA pipe
#endif
// 2^x on the FMA/ALU pipes for x <= 0 (clamped at -126): round to nearest integer with the magic-number
// add, cubic minimax on the fraction, exponent added as an integer shift.  Relative error ~1e-4.
__device__ __forceinline__ float2 exp2_poly2b(float2 x) {
  const float magic = 12582912.f;  // 1.5 * 2^23
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rn(x, make_float2(magic, magic));
  const float2 n = __fadd2_rn(t, make_float2(-magic, -magic));
  const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
  float2 q = __ffma2_rn(f, make_float2(0.0555054f, 0.0555054f), make_float2(0.2402265f, 0.2402265f));
  q = __ffma2_rn(q, f, make_float2(0.6931472f, 0.6931472f));
  q = __ffma2_rn(q, f, make_float2(1.f, 1.f));
  float2 r;
  r.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
  return r;
}
// p = 2^(s*sc - l) for four neighbouring columns; the first SAF_BWD_POLY_PER_8/2 of every four column pairs
// (counted by `pair`) use the polynomial
__device__ __forceinline__ void exp4(float (&o)[4], const uint32_t (&s)[4], float sc, const float4& L, int pair) {
  const float x0 = fmaf(__uint_as_float(s[0]), sc, -L.x), x1 = fmaf(__uint_as_float(s[1]), sc, -L.y);
  const float x2 = fmaf(__uint_as_float(s[2]), sc, -L.z), x3 = fmaf(__uint_as_float(s[3]), sc, -L.w);
  if ((pair & 3) < SAF_BWD_POLY_PER_8 / 2) {
    const float2 e = exp2_poly2b(make_float2(x0, x1));
    o[0] = e.x; o[1] = e.y;
  } else {
    o[0] = ex2b(x0); o[1] = ex2b(x1);
  }
  if (((pair + 1) & 3) < SAF_BWD_POLY_PER_8 / 2) {
    const float2 e = exp2_poly2b(make_float2(x2, x3));
    o[2] = e.x; o[3] = e.y;
  } else {
    o[2] = ex2b(x2); o[3] = ex2b(x3);
  }
}
// The bf16 operand the two compute warpgroups write for the next product lies in the first 64 columns of the fp32 tile
// they have just read: group 0 (columns 0-63 of the tile) writes columns 0-31, group 1 (columns 64-127) writes columns
// 32-63, which group 0 reads.  So group 1 stores only once group 0 has its values in registers: group 0 signals
// after its tcgen05.wait::ld, group 1 waits (named barrier `id`, 256 threads, one-way).  In consecutive columns
// the operand costs the tensor pipe 64 cycles per K step; split over the halves' own columns (0-31 and 64-95) a
// product that follows a shared-memory-operand product took 90 (`saf_selftest_mma_rate` forms 14 / 21).
// Group 0 signals as soon as its loads have landed, group 1 waits only in front of its first store, after the
// arithmetic of its first 32 columns: by then the signal has long been given, also by group 0's slowest warp.
__device__ __forceinline__ void operand_columns_read(int half, int id) {
  if (half == 0) {
    tc_fence_before();
    named_bar_arrive(id, 256);
  }
}
__device__ __forceinline__ void operand_columns_wait(int half, int id) {
  if (half != 0) {
    named_bar_sync(id, 256);
    tc_fence_after();
  }
}
// two fp32 -> packed bf16x2
__device__ __forceinline__ uint32_t bpack(float lo, float hi) {
#ifdef SAF_BWD_PACK_INT
  // round half up on the integer pipe instead of the conversion unit
  const uint32_t a = __float_as_uint(lo) + 0x8000u, b = __float_as_uint(hi) + 0x8000u;
  return __byte_perm(a, b, 0x7632);
#else
  return pack_bf16(lo, hi);
#endif
}
template <int N>
__device__ __forceinline__ void breg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void breg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int HD>
__device__ __forceinline__ void bload_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row, int head, int b) {
#pragma unroll
  for (int hh = 0; hh < HD / 64; ++hh) tma_load_4d(dst + hh * 16384, m, bar, hh * 64, row, head, b);
}

// The issuing lane shares its scheduler with two compute warps that keep it busy, so every instruction between two
// tcgen05.mma costs it tens of cycles: the two descriptors of a product are built once and each K step adds its
// byte offset to their low words.
//
// D[128 x 128] = A[128 x HD] B[128 x HD]^T, both operands K-major tiles in shared memory
template <int HD>
__device__ __forceinline__ void issue_ss(uint32_t d, uint32_t a_smem, uint32_t b_smem, uint32_t idesc) {
  const uint64_t da = umma_smem_desc_sw128(a_smem, 16, 1024), db = umma_smem_desc_sw128(b_smem, 16, 1024);
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
    umma_ss(d, umma_desc_advance(da, off), umma_desc_advance(db, off), idesc, ks > 0);
  }
}
// D[128 x HD] (+)= A[128 x 128] B[128 x HD]; A = bf16 in the first 64 columns of its region in TMEM,
// B = a [128 rows x HD] tile read MN-major
template <int HD>
__device__ __forceinline__ void issue_ts(uint32_t d, uint32_t a_tmem, uint32_t b_smem, uint32_t idesc, bool accumulate) {
  const uint64_t db = umma_smem_desc_sw128(b_smem, 16384, 1024);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    umma_ts(d, a_tmem + ks * 8, umma_desc_advance(db, ks * 2048), idesc, accumulate || ks > 0);
}

// 32 fp32 accumulator columns [c0, c0+32) of row r -> bf16 -> 128-byte-swizzled staging tile
__device__ __forceinline__ void stage_cols(uint8_t* stage, const uint32_t (&o)[32], int c0, int r, float f) {
  uint8_t* dst = stage + (c0 >> 6) * 16384 + r * 128;
  const int cbase = (c0 & 63) >> 3;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q;
    q.x = pack_bf16(__uint_as_float(o[c * 8 + 0]) * f, __uint_as_float(o[c * 8 + 1]) * f);
    q.y = pack_bf16(__uint_as_float(o[c * 8 + 2]) * f, __uint_as_float(o[c * 8 + 3]) * f);
    q.z = pack_bf16(__uint_as_float(o[c * 8 + 4]) * f, __uint_as_float(o[c * 8 + 5]) * f);
    q.w = pack_bf16(__uint_as_float(o[c * 8 + 6]) * f, __uint_as_float(o[c * 8 + 7]) * f);
    *reinterpret_cast<uint4*>(dst + (((cbase + c) ^ (r & 7)) << 4)) = q;
  }
}

// CTA -> (batch, head, tile), heads in groups so CTAs in flight share their streamed tiles in L2,
// heaviest tiles first inside a group.  Returns false when the CTA has nothing to do.
__device__ __forceinline__ bool bwd_cta_coords(const BwdParams& p, int cta, bool heavy_is_low, int& b, int& h, int& tile) {
  const int bh_count = p.B * p.H;
  const int per_group = BWD_HEAD_GROUP * p.n_tiles;
  const int grp = cta / per_group;
  const int gsize = min(BWD_HEAD_GROUP, bh_count - grp * BWD_HEAD_GROUP);
  const int rem = cta - grp * per_group;
  if (rem >= gsize * p.n_tiles) return false;
  const int t = rem / gsize;
  tile = heavy_is_low ? t : p.n_tiles - 1 - t;
  const int bh = grp * BWD_HEAD_GROUP + rem % gsize;
  b = bh / p.H;
  h = bh % p.H;
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  return state == SAF_LIVE;
}

template <int HD>
__device__ __forceinline__ void bwd_setup(BwdBars* bars, int tid, int warp) {
  if (tid == 0) {
    mbar_init(&bars->res_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&bars->ring_full[s], 1);
      mbar_init(&bars->ring_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_full, 256);
    mbar_init(&bars->ds_full, 256);
    mbar_init(&bars->acc_full, 1);
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, BwdCfg<HD>::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

// ---------------------------------------------------------------------------------------------
// dK_j, dV_j
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapdO,
                      const __grid_constant__ CUtensorMap mapdK, const __grid_constant__ CUtensorMap mapdV,
                      const __grid_constant__ CUtensorMap mapP64, const __grid_constant__ CUtensorMap mapdO64,
                      const __grid_constant__ BwdParams p) {
  using C = BwdCfg<HD>;
  if ((int)blockIdx.x < p.scan_slots) {
    // ---- reverse scan of a structured frozen head: one slot per (batch, head, 64-column slice)
    constexpr int PER = HD / SCAN_COLS;
    const int bh = blockIdx.x / PER, col0 = (blockIdx.x % PER) * SCAN_COLS;
    const int sb = bh / p.H, sh = bh % p.H;
    const int state = p.force_state >= 0 ? p.force_state : p.frozen[sh];
    if (state == SAF_SINK_DECAY && threadIdx.x < SCAN_NT) {
      extern __shared__ uint8_t scan_smem_raw[];
      float* scratch = reinterpret_cast<float*>(((uintptr_t)scan_smem_raw + 1023) & ~(uintptr_t)1023);
      sink_decay_scan_cta<__nv_bfloat16, true, 0, true>(p.scan, sb, sh, col0, 0, -1, scratch);
    }
    return;
  }
  if ((int)blockIdx.x < p.scan_slots + p.dense_slots) {
    extern __shared__ uint8_t dense_smem_raw[];
    uint8_t* dsm = (uint8_t*)(((uintptr_t)dense_smem_raw + 1023) & ~(uintptr_t)1023);
    dense_dv_cta<HD>(mapP64, mapdO64, mapdV, p.dense, (int)blockIdx.x - p.scan_slots, dsm);
    return;
  }
  int b, h, jt;
  if (!bwd_cta_coords(p, (int)blockIdx.x - p.scan_slots - p.dense_slots, true, b, h, jt)) return;
  const int hq = p.hidx ? p.hidx[h] : h;
  const int n = p.n_tiles - jt;            // query tiles jt .. n_tiles-1
  const int j0 = jt * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + C::TILE_BYTES;
  uint8_t* ring = smem + 2 * C::TILE_BYTES;           // stage s: [Q_i | dO_i]
  uint8_t* ringdO = ring + C::NQ * C::TILE_BYTES;       // `ring` is the Q ring
  BwdBars* bars = reinterpret_cast<BwdBars*>(ringdO + C::ND * C::TILE_BYTES);
  BwdVectors* vec = reinterpret_cast<BwdVectors*>(reinterpret_cast<uint8_t*>(bars) + 256);
  const int tid = threadIdx.x, warp = tid >> 5;
  bwd_setup<HD>(bars, tid, warp);
  const uint32_t tmem = bars->tmem_base;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + HD;
#ifdef SAF_BWD_TRACE
  const bool trace_on = (b == 0 && h == 0 && jt == 0) && (tid == 0 || tid == 9 * 32);
  const bool wtrace_on = (b == 0 && h == 0 && jt == 0) && (tid & 31) == 0 && tid < 256;
#endif

  if (warp >= 8) {
    breg_dec<56>();
    const bool leader = elect_one();
    if (warp == 8) {
      // ------------------------------------------------------------ TMA producer
      if (leader) {
        tma_prefetch_desc(&mapQ);
        tma_prefetch_desc(&mapK);
        tma_prefetch_desc(&mapV);
        tma_prefetch_desc(&mapdO);
        mbar_expect_tx(&bars->res_full, 2 * C::TILE_BYTES);
        bload_tile<HD>(sK, &mapK, &bars->res_full, j0, hq, b);
        bload_tile<HD>(sV, &mapV, &bars->res_full, j0, h, b);
        // Q_i and dO_i travel in separate rings: dO_i is done after the dV product, Q_i only after the dK
        // product, and S(i+1) must not wait for dO_{i+1}
        for (int i = 0; i < n; ++i) {
          const int sd = i % C::ND, s = i % C::NQ;
          if (!mbar_wait(&bars->v_empty[sd], ((i / C::ND) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 40);
            break;
          }
          mbar_expect_tx(&bars->v_full[sd], C::TILE_BYTES);
          bload_tile<HD>(ringdO + sd * C::TILE_BYTES, &mapdO, &bars->v_full[sd], (jt + i) * 128, h, b);
          if (!mbar_wait(&bars->ring_empty[s], ((i / C::NQ) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 49);
            break;
          }
          uint8_t* dst = ring + s * C::TILE_BYTES;
          mbar_expect_tx(&bars->ring_full[s], C::TILE_BYTES);
          bload_tile<HD>(dst, &mapQ, &bars->ring_full[s], (jt + i) * 128, hq, b);
        }
      }
    } else if (warp == 9) {
      // ------------------------------------------------------------ MMA issuer
      const uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aR = smem_u32(ring), aRd = smem_u32(ringdO);
      bool ok = mbar_wait(&bars->res_full, 0);
      if (!ok) dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 41);
      for (int i = 0; i < n && ok; ++i) {
        const int s = i % C::NQ, sd = i % C::ND;
        const uint32_t aQ = aR + s * C::TILE_BYTES, adO = aRd + sd * C::TILE_BYTES;
        if (i == 0) {
          if (!mbar_wait(&bars->ring_full[0], 0) || !mbar_wait(&bars->v_full[0], 0)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 42);
            break;
          }
          tc_fence_after();
          if (leader) {
            issue_ss<HD>(tmem + COL_S, aK, aQ, idesc_s);
            umma_commit(&bars->s_full[0]);
            issue_ss<HD>(tmem + COL_DP, aV, adO, idesc_s);
            umma_commit(&bars->dp_full);
          }
          __syncwarp();
        }
        if (!mbar_wait(&bars->p_full, i & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 43);
          break;
        }
        tc_fence_after();
        TRACE(0, 4, i);   // issuer saw p_full
        if (leader) {
          issue_ts<HD>(tmem + COL_DV, tmem + COL_S, adO, idesc_o, i > 0);
          umma_commit(&bars->v_empty[sd]);                // dO_i is not read again
        }
        __syncwarp();
        TRACE(0, 6, i);   // dV issued
        const int s2 = (i + 1) % C::NQ, sd2 = (i + 1) % C::ND;
        const uint32_t aQ2 = aR + s2 * C::TILE_BYTES, adO2 = aRd + sd2 * C::TILE_BYTES;
        if (i + 1 < n) {
          if (!mbar_wait(&bars->ring_full[s2], ((i + 1) / C::NQ) & 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 44);
            break;
          }
          tc_fence_after();
          if (leader) {
            issue_ss<HD>(tmem + COL_S, aK, aQ2, idesc_s);   // ordered behind the dV product that read P^T
            umma_commit(&bars->s_full[0]);
          }
          __syncwarp();
          TRACE(0, 7, i);   // next S^T issued
        }
        if (!mbar_wait(&bars->ds_full, i & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 45);
          break;
        }
        tc_fence_after();
        TRACE(0, 5, i);   // issuer saw ds_full
        if (leader) {
          issue_ts<HD>(tmem + COL_DK, tmem + COL_DP, aQ, idesc_o, i > 0);
          umma_commit(&bars->ring_empty[s]);              // Q_i is not read again
        }
        __syncwarp();
        if (i + 1 < n) {
          if (!mbar_wait(&bars->v_full[sd2], ((i + 1) / C::ND) & 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 59);
            break;
          }
          tc_fence_after();
          if (leader) {
            issue_ss<HD>(tmem + COL_DP, aV, adO2, idesc_s);  // ordered behind the dK product that read dS^T
            umma_commit(&bars->dp_full);
          }
          __syncwarp();
        }
      }
      if (leader) umma_commit(&bars->acc_full);
      __syncwarp();
    }
  } else {
    // -------------------------------------------------------------- compute warpgroups
    breg_inc<224>();
    const int half = warp >> 2;
    const int r = tid & 127;                       // key row of the tile
    const int cb = half * 64;                      // first query column of this group
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_base + COL_S, tdP = tmem + lane_base + COL_DP;
    const float sc = p.scale_log2;
    const float* lse_g = p.lse + (int64_t)b * p.lse_s[0] + (int64_t)h * p.lse_s[1];
    const float* dl_g = p.delta + (int64_t)b * p.delta_s[0] + (int64_t)h * p.delta_s[1];
    auto fetch = [&](int qt) -> float {
      const int row = qt * 128 + r;
      if (tid < 128) return row < p.T ? lse_g[(int64_t)row * p.lse_s[2]] : INFINITY;   // +inf: P = 0 past T
      return row < p.T ? dl_g[(int64_t)row * p.delta_s[2]] : 0.f;
    };
    float nxt = fetch(jt);
    // A warp whose wait ran out (decided for the whole warp) stops working but keeps taking part, one-way, in the
    // named barriers of every remaining tile -- two arrivals on barrier 1, one each on 2 and 3 per tile, as a working
    // warp gives -- so the other warps never block on it; they run into their own limits because P^T / dS^T stay
    // incomplete, and all meet again at the epilogue's barrier.
    bool ok = true;
    for (int i = 0; i < n; ++i) {
      if (!ok) {
        named_bar_arrive(1, 256);
        named_bar_arrive(1, 256);
        named_bar_arrive(2, 256);
        named_bar_arrive(3, 256);
        continue;
      }
      named_bar_sync(1, 256);                 // the previous tile's readers are done with the vectors
      if (tid < 128) vec->lse[r] = nxt;
      else vec->dl[r] = nxt;
      named_bar_sync(1, 256);
      if (i + 1 < n) nxt = fetch(jt + i + 1);
      // ---- P^T
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full[0], i & 1))) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 46);
        ok = false;
        named_bar_arrive(2, 256);
        named_bar_arrive(3, 256);
        continue;
      }
      tc_fence_after();
      TRACE(0, 0, i);   // scores visible
      float pf[64];
      {
        // both 32-column halves are requested before the single wait: one TMEM round trip per phase
        uint32_t s[2][32];
        tmem_ld32(tS + cb, s[0]);
        tmem_ld32(tS + cb + 32, s[1]);
        tmem_ld_wait();
        operand_columns_read(half, 2);
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const float4* L4 = reinterpret_cast<const float4*>(&vec->lse[cb + ch * 32]);
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const uint32_t s4[4] = {s[ch][x * 4 + 0], s[ch][x * 4 + 1], s[ch][x * 4 + 2], s[ch][x * 4 + 3]};
            float o4[4];
            exp4(o4, s4, sc, L4[x], 2 * x);
            pf[ch * 32 + x * 4 + 0] = o4[0];
            pf[ch * 32 + x * 4 + 1] = o4[1];
            pf[ch * 32 + x * 4 + 2] = o4[2];
            pf[ch * 32 + x * 4 + 3] = o4[3];
          }
          if (i == 0) {   // diagonal tile: query c sees key r only if c >= r
#pragma unroll
            for (int x = 0; x < 32; ++x)
              if (cb + ch * 32 + x < r) pf[ch * 32 + x] = 0.f;
          }
          uint32_t pk[16];
#pragma unroll
          for (int x = 0; x < 16; ++x) pk[x] = bpack(pf[ch * 32 + 2 * x], pf[ch * 32 + 2 * x + 1]);
          if (ch == 0) operand_columns_wait(half, 2);
          tmem_st16(tS + half * 32 + ch * 16, pk);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_full);
      TRACE(0, 1, i);   // P^T handed over
      WTRACE(0, i);
      // ---- dS^T
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->dp_full, i & 1))) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 47);
        ok = false;
        named_bar_arrive(3, 256);
        continue;
      }
      tc_fence_after();
      TRACE(0, 2, i);   // dP^T visible
      {
        uint32_t d[2][32];
        tmem_ld32(tdP + cb, d[0]);
        tmem_ld32(tdP + cb + 32, d[1]);
        tmem_ld_wait();
        operand_columns_read(half, 3);
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const float4* D4 = reinterpret_cast<const float4*>(&vec->dl[cb + ch * 32]);
          uint32_t pk[16];
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            const float4 D = D4[x];
            const float d0 = pf[ch * 32 + x * 4 + 0] * (__uint_as_float(d[ch][x * 4 + 0]) - D.x);
            const float d1 = pf[ch * 32 + x * 4 + 1] * (__uint_as_float(d[ch][x * 4 + 1]) - D.y);
            const float d2 = pf[ch * 32 + x * 4 + 2] * (__uint_as_float(d[ch][x * 4 + 2]) - D.z);
            const float d3 = pf[ch * 32 + x * 4 + 3] * (__uint_as_float(d[ch][x * 4 + 3]) - D.w);
            pk[2 * x] = bpack(d0, d1);
            pk[2 * x + 1] = bpack(d2, d3);
          }
          if (ch == 0) operand_columns_wait(half, 3);
          tmem_st16(tdP + half * 32 + ch * 16, pk);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->ds_full);
      TRACE(0, 3, i);   // dS^T handed over
      WTRACE(1, i);
    }
    // ---- epilogue: dV_j, dK_j -> bf16 -> swizzled staging (the K / V tiles are no longer read) -> TMA store
    if (ok && !mbar_wait(&bars->acc_full, 0)) {
      dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 48);
      ok = false;
    }
    tc_fence_after();
#pragma unroll
    for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
      uint32_t o[32];
      tmem_ld32(tmem + lane_base + COL_DV + c0, o);
      tmem_ld_wait();
      stage_cols(sV, o, c0, r, 1.f);
      tmem_ld32(tmem + lane_base + COL_DK + c0, o);
      tmem_ld_wait();
      stage_cols(sK, o, c0, r, p.sm_scale);
    }
    fence_proxy_async_smem();
    named_bar_sync(1, 256);
    if (tid == 0 && ok) {
#pragma unroll
      for (int hh = 0; hh < HD / 64; ++hh) {
        tma_store_4d(&mapdV, sV + hh * 16384, hh * 64, j0, h, b);
        tma_store_4d(&mapdK, sK + hh * 16384, hh * 64, j0, hq, b);
      }
      tma_store_commit();
      tma_store_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// dQ_i
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                    const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapdO,
                    const __grid_constant__ CUtensorMap mapdQ, const __grid_constant__ BwdParams p) {
  using C = BwdCfg<HD>;
  int b, h, it;
  if (!bwd_cta_coords(p, (int)blockIdx.x, false, b, h, it)) return;
  const int hq = p.hidx ? p.hidx[h] : h;
  const int n = it + 1;                    // key tiles 0 .. it
  const int i0 = it * 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + C::TILE_BYTES;
  uint8_t* ringK = smem + 2 * C::TILE_BYTES;          // K_j ring, KS tiles
  uint8_t* ringV = ringK + C::KS * C::TILE_BYTES;     // V_j ring, VS tiles
  BwdBars* bars = reinterpret_cast<BwdBars*>(ringV + C::VS * C::TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5;
  bwd_setup<HD>(bars, tid, warp);
  const uint32_t tmem = bars->tmem_base;
  constexpr uint32_t COL_S = 0 /* two buffers */, COL_DP = 256, COL_DQ = 384;
#ifdef SAF_BWD_TRACE
  const bool trace_on = (b == 0 && h == 0 && it == p.n_tiles - 1) && (tid == 0 || tid == 9 * 32);
#endif

  if (warp >= 8) {
    breg_dec<56>();
    const bool leader = elect_one();
    if (warp == 8) {
      // ------------------------------------------------------------ TMA producer
      if (leader) {
        tma_prefetch_desc(&mapQ);
        tma_prefetch_desc(&mapK);
        tma_prefetch_desc(&mapV);
        tma_prefetch_desc(&mapdO);
        mbar_expect_tx(&bars->res_full, 2 * C::TILE_BYTES);
        bload_tile<HD>(sQ, &mapQ, &bars->res_full, i0, hq, b);
        bload_tile<HD>(sdO, &mapdO, &bars->res_full, i0, h, b);
        for (int j = 0; j < n; ++j) {
          const int sk = j % C::KS, sv = j % C::VS;
          if (!mbar_wait(&bars->ring_empty[sk], ((j / C::KS) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 50);
            break;
          }
          mbar_expect_tx(&bars->ring_full[sk], C::TILE_BYTES);
          bload_tile<HD>(ringK + sk * C::TILE_BYTES, &mapK, &bars->ring_full[sk], j * 128, hq, b);
          if (!mbar_wait(&bars->v_empty[sv], ((j / C::VS) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 57);
            break;
          }
          mbar_expect_tx(&bars->v_full[sv], C::TILE_BYTES);
          bload_tile<HD>(ringV + sv * C::TILE_BYTES, &mapV, &bars->v_full[sv], j * 128, h, b);
        }
      }
    } else if (warp == 9) {
      // ------------------------------------------------------------ MMA issuer
      const uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(ringK), aV = smem_u32(ringV);
      bool ok = mbar_wait(&bars->res_full, 0);
      if (!ok) dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 51);
      // scores run up to two key tiles ahead (two score buffers), dP one ahead
      auto issue_scores = [&](int j) -> bool {
        const int s = j % C::KS;
        if (!mbar_wait(&bars->ring_full[s], (j / C::KS) & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 52);
          return false;
        }
        tc_fence_after();
        if (leader) {
          issue_ss<HD>(tmem + COL_S + (j & 1) * 128, aQ, aK + s * C::TILE_BYTES, idesc_s);
          umma_commit(&bars->s_full[j & 1]);
        }
        __syncwarp();
        return true;
      };
      auto issue_dp = [&](int j) -> bool {
        const int s = j % C::VS;
        if (!mbar_wait(&bars->v_full[s], (j / C::VS) & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 58);
          return false;
        }
        tc_fence_after();
        if (leader) {
          issue_ss<HD>(tmem + COL_DP, adO, aV + s * C::TILE_BYTES, idesc_s);
          umma_commit(&bars->dp_full);
          umma_commit(&bars->v_empty[s]);     // V_j is not read again
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_scores(0);
      if (ok) ok = issue_dp(0);
      if (ok && n > 1) ok = issue_scores(1);
      for (int j = 0; j < n && ok; ++j) {
        const int s = j % C::KS;
        if (!mbar_wait(&bars->ds_full, j & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 53);
          break;
        }
        tc_fence_after();
        TRACE(1, 5, j);
        if (leader) {
          issue_ts<HD>(tmem + COL_DQ, tmem + COL_DP, aK + s * C::TILE_BYTES, idesc_o, j > 0);
          umma_commit(&bars->ring_empty[s]);          // K_j is not read again
        }
        __syncwarp();
        if (j + 1 < n) ok = issue_dp(j + 1);          // ordered behind the dQ product that read dS
        if (ok && j + 2 < n) ok = issue_scores(j + 2);   // score buffer j & 1 was read before ds_full(j)
      }
      if (leader) umma_commit(&bars->acc_full);
      __syncwarp();
    }
  } else {
    // -------------------------------------------------------------- compute warpgroups
    breg_inc<224>();
    const int half = warp >> 2;
    const int r = tid & 127;                       // query row of the tile
    const int cb = half * 64;                      // first key column of this group
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tdP = tmem + lane_base + COL_DP;
    const float sc = p.scale_log2;
    const int row = i0 + r;
    float lse_r = INFINITY, dl_r = 0.f;            // +inf: P = 0 for rows past T
    if (row < p.T) {
      lse_r = p.lse[(int64_t)b * p.lse_s[0] + (int64_t)h * p.lse_s[1] + (int64_t)row * p.lse_s[2]];
      dl_r = p.delta[(int64_t)b * p.delta_s[0] + (int64_t)h * p.delta_s[1] + (int64_t)row * p.delta_s[2]];
    }
    // (a warp whose wait ran out keeps giving its one arrival per tile on named barrier 2, as in the dK/dV kernel)
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      if (!ok) {
        named_bar_arrive(2, 256);
        continue;
      }
      const uint32_t tS = tmem + lane_base + COL_S + (j & 1) * 128;
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->s_full[j & 1], (j >> 1) & 1))) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 54);
        ok = false;
        named_bar_arrive(2, 256);
        continue;
      }
      tc_fence_after();
      TRACE(1, 0, j);
      float pf[64];
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t s[32];
        tmem_ld32(tS + cb + ch * 32, s);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const uint32_t s4[4] = {s[x * 4 + 0], s[x * 4 + 1], s[x * 4 + 2], s[x * 4 + 3]};
          float o4[4];
          exp4(o4, s4, sc, make_float4(lse_r, lse_r, lse_r, lse_r), 2 * x);
          pf[ch * 32 + x * 4 + 0] = o4[0];
          pf[ch * 32 + x * 4 + 1] = o4[1];
          pf[ch * 32 + x * 4 + 2] = o4[2];
          pf[ch * 32 + x * 4 + 3] = o4[3];
        }
        if (j == n - 1) {   // diagonal tile: keys after the row do not count
#pragma unroll
          for (int x = 0; x < 32; ++x)
            if (cb + ch * 32 + x > r) pf[ch * 32 + x] = 0.f;
        }
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&bars->dp_full, j & 1))) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 55);
        ok = false;
        named_bar_arrive(2, 256);
        continue;
      }
      tc_fence_after();
      TRACE(1, 2, j);
      {
        uint32_t d[2][32];
        tmem_ld32(tdP + cb, d[0]);
        tmem_ld32(tdP + cb + 32, d[1]);
        tmem_ld_wait();
        operand_columns_read(half, 2);
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t pk[16];
#pragma unroll
          for (int x = 0; x < 16; ++x)
            pk[x] = bpack(pf[ch * 32 + 2 * x] * (__uint_as_float(d[ch][2 * x]) - dl_r),
                          pf[ch * 32 + 2 * x + 1] * (__uint_as_float(d[ch][2 * x + 1]) - dl_r));
          if (ch == 0) operand_columns_wait(half, 2);
          tmem_st16(tdP + half * 32 + ch * 16, pk);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->ds_full);
      TRACE(1, 3, j);
    }
    if (ok && !mbar_wait(&bars->acc_full, 0)) {
      dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 56);
      ok = false;
    }
    tc_fence_after();
#pragma unroll
    for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
      uint32_t o[32];
      tmem_ld32(tmem + lane_base + COL_DQ + c0, o);
      tmem_ld_wait();
      stage_cols(sQ, o, c0, r, p.sm_scale);
    }
    fence_proxy_async_smem();
    named_bar_sync(1, 256);
    if (tid == 0 && ok) {
#pragma unroll
      for (int hh = 0; hh < HD / 64; ++hh) tma_store_4d(&mapdQ, sQ + hh * 16384, hh * 64, i0, hq, b);
      tma_store_commit();
      tma_store_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// delta_i = sum_d O_id dO_id for the live heads (kernel/fused_attn.py:291-310)
// ---------------------------------------------------------------------------------------------
struct DeltaParams {
  const __nv_bfloat16* o;
  const __nv_bfloat16* dout;
  int64_t o_s[3], do_s[3];
  float* delta;
  int64_t delta_s[3];
  const int32_t* frozen;
  int B, H, T, force_state;
  int hd;                       // real head width (<= the kernel's HD)
};

template <int HD>
__global__ void __launch_bounds__(256) flash_bwd_delta_kernel(const __grid_constant__ DeltaParams p) {
  constexpr int TPR = HD / 8;              // threads per row, 16 bytes each
  constexpr int ROWS = 256 / TPR;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  if (state != SAF_LIVE) return;
  const int row = blockIdx.x * ROWS + threadIdx.x / TPR;
  const int c = (threadIdx.x % TPR) * 8;
  float s = 0.f;
  if (row < p.T && c < p.hd) {   // p.hd < HD: head_dim 96 on the 128-column kernels
    const uint4 a = *reinterpret_cast<const uint4*>(p.o + (int64_t)b * p.o_s[0] + (int64_t)h * p.o_s[1] + (int64_t)row * p.o_s[2] + c);
    const uint4 d = *reinterpret_cast<const uint4*>(p.dout + (int64_t)b * p.do_s[0] + (int64_t)h * p.do_s[1] + (int64_t)row * p.do_s[2] + c);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      s = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(dw[e] << 16), s);
      s = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(dw[e] & 0xffff0000u), s);
    }
  }
#pragma unroll
  for (int off = TPR / 2; off; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (row < p.T && (threadIdx.x % TPR) == 0)
    p.delta[(int64_t)b * p.delta_s[0] + (int64_t)h * p.delta_s[1] + (int64_t)row * p.delta_s[2]] = s;
}

bool bwd_aligned16(const void* q) { return ((uintptr_t)q & 15) == 0; }

bool bwd_tma_ok(const SafTensor& t) {
  if (!t.ptr || !bwd_aligned16(t.ptr) || t.stride[3] != 1) return false;
  for (int i = 0; i < 3; ++i)
    if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
  return true;
}

int bwd_map4(CUtensorMap* m, const SafTensor& t, int B, int Hn, int T, int HD) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)T, (uint64_t)Hn, (uint64_t)B};
  uint64_t strides[4] = {0, (uint64_t)t.stride[2] * 2, (uint64_t)t.stride[1] * 2, (uint64_t)t.stride[0] * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tensor_map_bf16(m, t.ptr, 4, dims, strides, box, true);
}

template <int HD>
int bwd_launch_typed(const SafMixedAttnBwdArgs& g, bool live, bool* dense_done, bool* decomp_done, cudaStream_t st) {
  const SafMixedAttnArgs& a = g.fwd;
  CUtensorMap mq, mk, mv, mdo, mdq, mdk, mdv;
  int rc;
  // without live heads (frozen_pv backward) only the roles of the dK/dV launch run: the q/k maps are never used
  const SafTensor& tq = live ? a.q : g.dv;
  const SafTensor& tk = live ? a.k : g.dv;
  const SafTensor& tdq = live ? g.dq : g.dv;
  const SafTensor& tdk = live ? g.dk : g.dv;
  const SafTensor& tv = live ? a.v : g.dv;               // frozen_pv passes no forward tensors
  const int Uq = live ? a.U : a.H;
  if ((rc = bwd_map4(&mq, tq, a.B, Uq, a.T, a.HD))) return rc;
  if ((rc = bwd_map4(&mk, tk, a.B, Uq, a.T, a.HD))) return rc;
  if ((rc = bwd_map4(&mv, tv, a.B, a.H, a.T, a.HD))) return rc;
  if ((rc = bwd_map4(&mdo, g.dout, a.B, a.H, a.T, a.HD))) return rc;
  if ((rc = bwd_map4(&mdq, tdq, a.B, Uq, a.T, a.HD))) return rc;
  if ((rc = bwd_map4(&mdk, tdk, a.B, Uq, a.T, a.HD))) return rc;
  if ((rc = bwd_map4(&mdv, g.dv, a.B, a.H, a.T, a.HD))) return rc;

  DeltaParams d;
  d.o = reinterpret_cast<const __nv_bfloat16*>(a.out.ptr);
  d.dout = reinterpret_cast<const __nv_bfloat16*>(g.dout.ptr);
  for (int i = 0; i < 3; ++i) {
    d.o_s[i] = a.out.stride[i];
    d.do_s[i] = g.dout.stride[i];
    d.delta_s[i] = g.delta.stride[i];
  }
  d.delta = reinterpret_cast<float*>(g.delta.ptr);
  d.frozen = a.frozen;
  d.B = a.B; d.H = a.H; d.T = a.T; d.force_state = a.force_state;
  d.hd = a.HD;
  constexpr int ROWS = 256 / (HD / 8);
  if (live) {
    flash_bwd_delta_kernel<HD><<<dim3((a.T + ROWS - 1) / ROWS, a.B * a.H), 256, 0, st>>>(d);
    count_launch();
    if ((rc = check_launch("flash_bwd_delta_kernel"))) return rc;
  }

  BwdParams p;
  memset(&p, 0, sizeof(p));
  p.B = a.B; p.H = a.H; p.T = a.T; p.force_state = a.force_state;
  p.n_tiles = (a.T + 127) / 128;
  p.sm_scale = a.sm_scale;
  p.scale_log2 = a.sm_scale * LOG2E_B;
  p.frozen = a.frozen; p.hidx = a.hidx;
  p.lse = reinterpret_cast<const float*>(a.lse.ptr);
  p.delta = d.delta;
  for (int i = 0; i < 3; ++i) {
    p.lse_s[i] = a.lse.stride[i];
    p.delta_s[i] = g.delta.stride[i];
  }
  p.status = a.status;
  if (a.sd_alpha && a.sd_rho) {   // (the scan clips its 64-column slices to the real width)
    ScanArgs& sc = p.scan;
    sc.in = g.dout.ptr;
    sc.out = g.dv.ptr;
    for (int i = 0; i < 4; ++i) {
      sc.si[i] = g.dout.stride[i];
      sc.so[i] = g.dv.stride[i];
    }
    sc.frozen = a.frozen; sc.kvidx = nullptr; sc.sd_alpha = a.sd_alpha; sc.sd_rho = a.sd_rho;
    sc.B = a.B; sc.H = a.H; sc.T = a.T; sc.HD = a.HD; sc.force_state = a.force_state; sc.HKV = 0;
    sc.vec_ok = 1;   // bwd_tma_ok() already demands 16-byte aligned bases and strides
    p.scan_slots = a.B * a.H * (HD / SCAN_COLS);
  }
  CUtensorMap mp64, mdo64;
  memset(&mp64, 0, sizeof(mp64));
  memset(&mdo64, 0, sizeof(mdo64));
  {
    bool dense = a.patt.ptr && dense_dv_eligible(g), decomp = a.alpha.ptr && dense_dv_decomp_eligible(g);
    if (a.frozen_host) {
      bool any1 = false, any2 = false;
      for (int hh = 0; hh < a.H; ++hh) {
        any1 |= a.frozen_host[hh] == SAF_DENSE;
        any2 |= a.frozen_host[hh] == SAF_DECOMP;
      }
      dense = dense && any1;
      decomp = decomp && any2;
    }
    if (dense || decomp) {
      CUtensorMap mdv2;
      if ((rc = dense_dv_prepare(g, dense, decomp, &mp64, &mdo64, &mdv2, &p.dense))) return rc;
      p.dense_slots = (int)dense_pv_slots(p.dense);
    }
    *dense_done = dense;
    *decomp_done = decomp;
  }
  static PerDeviceOnce smem_once_dkdv, smem_once_dq;
  if ((rc = ensure_dyn_smem(flash_bwd_dkdv_kernel<HD>, BwdCfg<HD>::SMEM_BYTES, smem_once_dkdv))) return rc;
  if ((rc = ensure_dyn_smem(flash_bwd_dq_kernel<HD>, BwdCfg<HD>::SMEM_BYTES_DQ, smem_once_dq))) return rc;
  const int bh = a.B * a.H;
  const int groups = (bh + BWD_HEAD_GROUP - 1) / BWD_HEAD_GROUP;
  const unsigned grid = live ? (unsigned)(groups * BWD_HEAD_GROUP * p.n_tiles) : 0u;
  if (grid + p.scan_slots + p.dense_slots == 0) return SAF_ERR_UNSUPPORTED;
  flash_bwd_dkdv_kernel<HD><<<grid + p.scan_slots + p.dense_slots, BWD_THREADS, BwdCfg<HD>::SMEM_BYTES, st>>>(
      mq, mk, mv, mdo, mdk, mdv, mp64, mdo64, p);
  count_launch();
  if ((rc = check_launch("flash_bwd_dkdv_kernel"))) return rc;
  p.scan_slots = 0;
  p.dense_slots = 0;
  if (!live) return SAF_OK;
  flash_bwd_dq_kernel<HD><<<grid, BWD_THREADS, BwdCfg<HD>::SMEM_BYTES_DQ, st>>>(mq, mk, mv, mdo, mdq, p);
  count_launch();
  return check_launch("flash_bwd_dq_kernel");
}

}  // namespace

#ifdef SAF_BWD_TRACE
extern "C" int saf_debug_trace(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, g_trace, sizeof(g_trace));
}
extern "C" int saf_debug_wtrace(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, g_wtrace, sizeof(g_wtrace));
}
#endif

// Live heads of a bf16 backward at head_dim 64 / 128 without in-kernel RoPE or GQA; everything else
// stays with the generic kernels.
int launch_flash_bwd_sm100(const SafMixedAttnBwdArgs& g, uint32_t* handled, cudaStream_t st) {
  *handled = 0;
  const SafMixedAttnArgs& a = g.fwd;
  // head_dim 96 rides the 128-column kernels: the tensor maps carry the real width, loads fill the missing columns
  // with zeros and stores clip them
  if (a.dtype != SAF_BF16 || (a.HD != 64 && a.HD != 96 && a.HD != 128) || a.rope || a.HKV > 0) return SAF_ERR_UNSUPPORTED;
  if (!bwd_tma_ok(g.dout) || !bwd_tma_ok(g.dv)) return SAF_ERR_UNSUPPORTED;
  if (!saf_device_supported()) return SAF_ERR_UNSUPPORTED;
  // live heads need the full set of tensors; without them only the frozen-head roles are launched
  bool live = a.U > 0 && a.sm_scale > 0.f && bwd_tma_ok(a.q) && bwd_tma_ok(a.k) && bwd_tma_ok(a.v) && bwd_tma_ok(g.dq) &&
              bwd_tma_ok(g.dk) && bwd_tma_ok(a.out) && a.lse.ptr && g.delta.ptr;
  bool live_present = a.force_state < 0 ? a.U > 0 : a.force_state == SAF_LIVE;
  if (a.frozen_host && a.force_state < 0) {
    live_present = false;
    for (int h = 0; h < a.H; ++h) live_present |= a.frozen_host[h] == SAF_LIVE;
  }
  if (live_present && !live) return SAF_ERR_UNSUPPORTED;   // live heads this launch cannot serve: leave everything
  live = live && live_present;
  if (a.HD == 96 && !live && !(a.sd_alpha && a.sd_rho)) return SAF_ERR_UNSUPPORTED;   // no role of this launch applies
  bool dense_done = false, decomp_done = false;
  const int rc = (a.HD == 64) ? bwd_launch_typed<64>(g, live, &dense_done, &decomp_done, st)
                              : bwd_launch_typed<128>(g, live, &dense_done, &decomp_done, st);
  if (rc == SAF_OK)
    *handled = (live ? (1u << SAF_LIVE) : 0u) | ((a.sd_alpha && a.sd_rho) ? (1u << SAF_SINK_DECAY) : 0u) |
               (dense_done ? (1u << SAF_DENSE) : 0u) | (decomp_done ? (1u << SAF_DECOMP) : 0u);
  return rc;
}

}  // namespace saf
