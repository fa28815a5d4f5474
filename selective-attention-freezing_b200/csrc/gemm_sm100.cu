// Indexed linear on the 5th-generation tensor cores (tcgen05, TMEM accumulators).
//
//   out[m, g*slab + r] = sum_c x[m,c] * W_g[row0_g + r, c]  (+ bias)   [+ RoPE on chosen slabs]
//
// replaces the reference's gather-then-GEMM (kernel/indexed_linear.py:86-98: two
// index_select + cat materialise a (2R, C) weight copy on every call, then cuBLAS;
// RoPE afterwards as 3-4 elementwise kernels, nanogpt/model.py:1007-1008).  Here the
// canonical weights are read in place: every 64-row block of output features has
// its own TMA source (weight matrix, first row), so rows of frozen heads are never
// touched, and the rotation is applied to the fp32 accumulator in the epilogue.
//
// Persistent, warp-specialised CTA (1 per SM):
//   warp 0      TMA producer: x tile 128x64 and four 64x64 weight blocks per stage (128B swizzle)
//   warp 1      MMA issuer: tcgen05.mma 128x256x16, bf16 -> fp32 in TMEM, 2 accumulator buffers (512 columns)
//   warps 2..5  epilogue, 64 columns at a time: TMEM -> registers (bias, RoPE) -> bf16 -> swizzled smem
//               -> TMA store (two staging blocks in flight).  The row's cos/sin values are fetched once
//               per row of tiles, before the accumulator is waited for, so their latency hides behind the MMAs.
// Large products run the same kernel as CTA PAIRS (template parameter PAIR, a cluster of two): one 256x256 tile per
// pair through tcgen05.mma.cta_group::2, each CTA loading its 128 rows of x and half of the weight tile (see GCfg).
// All waits are bounded; a wait that runs out sets *status and the CTA drains.
#include <algorithm>
#include <atomic>

#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {
namespace {

constexpr int GM = 128, GN = 256, GK = 64;   // 128x256 tiles: 96 B/clk/SM of operand traffic at full MMA rate
constexpr int SUBS = GN / 64;                // 64-column blocks per tile
constexpr int A_BYTES = GM * GK * 2;            // 16 KB
constexpr int SUB_BYTES = 64 * GK * 2;          // 8 KB: one 64-row block of weights
constexpr int MAX_STAGES = 6;
// PAIR: two CTAs of a cluster share one 256 x 256 tile through tcgen05 cta_group::2.  Each CTA loads its 128 rows of x
// and HALF of the weight tile (two 64-row blocks), so the operand traffic per SM drops from 96 to 64 bytes per clock at
// the full MMA rate -- what one SM can pull from L2 -- and a stage shrinks to 32 KB (6 stages instead of 4).
template <bool PAIR>
struct GCfg {
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int B_SUBS = PAIR ? 2 : SUBS;                       // weight blocks a CTA loads per stage
  static constexpr int STAGE_BYTES = A_BYTES + B_SUBS * SUB_BYTES;     // 32 KB / 48 KB
  static constexpr int ROWS = PAIR ? 2 * GM : GM;                      // rows of a tile
};
constexpr int OUT_BYTES = 2 * GM * 64 * 2;      // two 16 KB staging blocks for the TMA stores
constexpr int MAX_SUB = 288;                    // 64-row blocks of output features (N <= 18432)
constexpr int GEMM_THREADS = 192;   // TMA warp, MMA warp, one epilogue warpgroup

struct SubTable {
  int32_t row0[MAX_SUB];
  uint8_t weight[MAX_SUB];
  uint8_t rope[MAX_SUB];     // 0: none, 1: this 64-block is the first half of a rotated slab... see kernel
  // slabs that are a multiple of 32 but not of 64 rows (head_dim 96): a 64-column block is two runs of 32 weight
  // rows, each with its own source (first run in row0 / weight, second run here)
  int32_t row0b[MAX_SUB];
  uint8_t weightb[MAX_SUB];
};

struct GemmParams {
  int M, N, K, T, slab;
  int tiles_m, tiles_n;
  const void* bias[SAF_MAX_WEIGHTS];
  const float* cosT;
  const float* sinT;
  int* status;
  int act;                       // SAF_ACT_*
  const __nv_bfloat16* residual; // added to the output, or null
  int64_t ldr;
  int halves;                    // weight blocks arrive as two 32-row TMA boxes (see SubTable)
};

// exact-form GELU, 0.5 x (1 + erf(x / sqrt 2)), with erf from Abramowitz-Stegun 7.1.26 (|error| < 1.5e-7):
// one reciprocal and one exponential on the special-function unit, the rest FMAs
__device__ __forceinline__ float gelu_erf(float x) {
  // Phi(-|x|) = 0.5 erfc(|x| / sqrt 2) = 0.5 t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) exp(-x^2 / 2)
  const float ax = fabsf(x);
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f * 0.70710678118654752f, ax, 1.f)));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(ax * ax * (-0.5f * 1.4426950408889634f)));
  float poly = fmaf(0.5f * 1.061405429f, t, 0.5f * -1.453152027f);
  poly = fmaf(poly, t, 0.5f * 1.421413741f);
  poly = fmaf(poly, t, 0.5f * -0.284496736f);
  poly = fmaf(poly, t, 0.5f * 0.254829592f);
  const float q = poly * t * e;                 // Phi(-|x|)
  return x * (x >= 0.f ? 1.f - q : q);          // x Phi(x)
}

// SiLU gate: g * sigmoid(g) * u, sigmoid through one exponential and one approximate reciprocal
__device__ __forceinline__ float silu_mul(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return g * r * u;
}

struct SmemLayout {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

template <bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
indexed_gemm_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW0,
                    const __grid_constant__ CUtensorMap mapW1, const __grid_constant__ CUtensorMap mapW2,
                    const __grid_constant__ CUtensorMap mapW3, const __grid_constant__ CUtensorMap mapO,
                    const __grid_constant__ GemmParams p, const __grid_constant__ SubTable tb) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  using C = GCfg<PAIR>;
  constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES;
  uint8_t* stage_base = smem;
  uint8_t* out_stage = smem + STAGES * STAGE_BYTES;
  SmemLayout* sl = reinterpret_cast<SmemLayout*>(out_stage + OUT_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KB = (p.K + GK - 1) / GK;
  const int total_tiles = p.tiles_m * p.tiles_n;
  // each CTA walks a contiguous run of tiles (column tile fastest): consecutive tiles share their rows, so the
  // row's cos / sin values stay in registers and the x tile stays hot in L2
  const int rank = PAIR ? (int)cluster_ctarank() : 0;                 // which 128 rows of the tile are this CTA's
  const int unit = PAIR ? blockIdx.x >> 1 : blockIdx.x, n_units = PAIR ? gridDim.x >> 1 : gridDim.x;
  const int tile_lo = (int)((int64_t)unit * total_tiles / n_units);
  const int tile_hi = (int)((int64_t)(unit + 1) * total_tiles / n_units);

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sl->full[s], 1);
      mbar_init(&sl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sl->acc_full[b], 1);
      mbar_init(&sl->acc_empty[b], PAIR ? 8 : 4);       // one arrival per epilogue warp (of both CTAs)
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(&sl->tmem_base, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&sl->tmem_base, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();                 // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem = sl->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      const CUtensorMap* wm[4] = {&mapW0, &mapW1, &mapW2, &mapW3};
      tma_prefetch_desc(&mapX);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = tile_lo; tile < tile_hi && ok; ++tile) {
        const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
        const int nsub = min(SUBS, (p.N - tn * GN) / 64);
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&sl->empty[s], ((it / STAGES) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 10);
            ok = false;
            break;
          }
          uint8_t* a = stage_base + s * STAGE_BYTES;
          uint8_t* b = a + A_BYTES;
          if constexpr (PAIR) {
            // this CTA's 128 rows of x and its two of the tile's four weight blocks.  Every byte of both CTAs is
            // counted on the even CTA's barrier, which its MMA warp waits on: the even CTA's producer announces the
            // pair's bytes there (a local arrive), the odd CTA's producer only issues its loads -- they cannot land
            // before the barrier's previous phase is over, because its own empty barrier opens after that.
            // (a last column tile of two blocks is computed as a 256 x 128 product: one block per CTA)
            const int per = nsub == 2 ? 1 : C::B_SUBS;
            const int mine = max(0, min(per, nsub - rank * per));
            const uint32_t bar = cluster_addr_of(&sl->full[s], 0);
            if (rank == 0) mbar_expect_tx(&sl->full[s], 2 * A_BYTES + nsub * SUB_BYTES);
            tma_load_2d_pair(a, &mapX, bar, kb * GK, tm * C::ROWS + rank * GM);
            for (int u = 0; u < mine; ++u) {
              const int sb = tn * SUBS + rank * per + u;
              tma_load_2d_pair(b + u * SUB_BYTES, wm[tb.weight[sb]], bar, kb * GK, tb.row0[sb]);
              if (p.halves)
                tma_load_2d_pair(b + u * SUB_BYTES + SUB_BYTES / 2, wm[tb.weightb[sb]], bar, kb * GK, tb.row0b[sb]);
            }
          } else {
            mbar_expect_tx(&sl->full[s], A_BYTES + nsub * SUB_BYTES);
            tma_load_2d(a, &mapX, &sl->full[s], kb * GK, tm * GM);
            for (int u = 0; u < nsub; ++u) {
              const int sb = tn * SUBS + u;
              tma_load_2d(b + u * SUB_BYTES, wm[tb.weight[sb]], &sl->full[s], kb * GK, tb.row0[sb]);
              if (p.halves)   // the maps' boxes are 32 rows: the second run lands behind the first (4 swizzle atoms on)
                tma_load_2d(b + u * SUB_BYTES + SUB_BYTES / 2, wm[tb.weightb[sb]], &sl->full[s], kb * GK, tb.row0b[sb]);
            }
          }
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // the whole warp walks the schedule (uniform addresses); one elected lane issues.  In a pair only the even
    // CTA issues: its instructions read both CTAs' stages and write both CTAs' accumulators.
    const bool leader = elect_one();
    const uint32_t idesc_full = umma_idesc_bf16(C::ROWS, GN, 0, 0);
    const uint32_t idesc_half = umma_idesc_bf16(C::ROWS, GN / 2, 0, 0);   // pair: a last column tile of two blocks
    const uint32_t sbase = smem_u32(stage_base);
    uint32_t it = 0, lt = 0;
    bool ok = true;
    for (int tile = tile_lo; tile < tile_hi && ok; ++tile, ++lt) {
      const int buf = lt & 1;
      if (!mbar_wait(&sl->acc_empty[buf], ((lt >> 1) & 1) ^ 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 11);
        break;
      }
      tc_fence_after();
      const uint32_t d = tmem + buf * GN;
      const int tn_ = tile % p.tiles_n;
      const uint32_t idesc = (PAIR && (p.N - tn_ * GN) / 64 == 2) ? idesc_half : idesc_full;
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&sl->full[s], (it / STAGES) & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 12);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a = sbase + s * STAGE_BYTES;
        const uint32_t b = a + A_BYTES;
        if (leader) {
          const uint64_t ad0 = umma_smem_desc_sw128(a, 16, 1024), bd0 = umma_smem_desc_sw128(b, 16, 1024);
#pragma unroll
          for (int k4 = 0; k4 < GK / 16; ++k4) {
            const uint64_t ad = umma_desc_advance(ad0, k4 * 32), bd = umma_desc_advance(bd0, k4 * 32);
            if constexpr (PAIR) umma_ss_pair(d, ad, bd, idesc, (kb | k4) != 0);
            else umma_ss(d, ad, bd, idesc, (kb | k4) != 0);
          }
          if constexpr (PAIR) umma_commit_pair(&sl->empty[s]);      // frees the stage in both CTAs
          else umma_commit(&sl->empty[s]);
        }
        __syncwarp();
      }
      if (ok && leader) {
        if constexpr (PAIR) umma_commit_pair(&sl->acc_full[buf]);
        else umma_commit(&sl->acc_full[buf]);
      }
      __syncwarp();
    }
  } else if (warp >= 2) {
    // epilogue warps 2..5 -> TMEM lane quadrant (warp % 4)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;           // row inside the tile
    const int etid = tid - 64;                  // 0..127
    uint32_t lt = 0;
    uint32_t n_out = 0;                         // output blocks stored so far (staging block = parity)
    int tm_held = -1;                           // row tile whose cos / sin values the registers hold
    float4 cs4[8], sn4[8];
    for (int tile = tile_lo; tile < tile_hi; ++tile, ++lt) {
      const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
      const int nsub = min(SUBS, (p.N - tn * GN) / 64);
      const int buf = lt & 1;
      const int m = tm * C::ROWS + rank * GM + row;
      const int t = (p.T > 0) ? (m % p.T) : 0;
      // head_dim 64: this row's 32 cos and 32 sin values, shared by every rotated block of the tile
      if (p.slab == 64 && p.cosT && tm != tm_held) {
        tm_held = tm;
        const float4* cr4 = reinterpret_cast<const float4*>(p.cosT + (int64_t)t * 64);
        const float4* sr4 = reinterpret_cast<const float4*>(p.sinT + (int64_t)t * 64);
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          cs4[j4] = cr4[j4];
          sn4[j4] = sr4[j4];
        }
      }
      if (!mbar_wait(&sl->acc_full[buf], (lt >> 1) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 13);
        break;
      }
      tc_fence_after();
      const uint32_t tsrc = tmem + ((uint32_t)(quad * 32) << 16) + buf * GN;
      const bool swiglu = p.act == SAF_ACT_SWIGLU;
      for (int u = 0; u < nsub; ++u) {
        // gated MLP: blocks come in (gate, up) pairs; the even block of a pair produces the 64 output columns
        if (swiglu && (u & 1)) continue;
        // the two staging blocks take turns over ALL stores of the CTA (a column tile may hold an odd number of
        // output blocks: alternating by u alone would reuse the block whose store was issued last);
        // the one whose turn it is is free once the store issued two output blocks ago has read it
        const int ob = (n_out++) & 1;
        if (etid == 0) tma_store_wait_read1();
        named_bar_sync(1, 128);
        const int sb = tn * SUBS + u;
        const int w = tb.weight[sb];
        const int rp = tb.rope[sb];
        // column offset of this 64-block inside its slab (slab = 64: 0; slab = 128: 0 or 64)
        const int in_slab = (sb * 64) % p.slab;
        float v[64];
        {
          uint32_t r0[32], r1[32];
          tmem_ld32(tsrc + u * 64, r0);
          tmem_ld32(tsrc + u * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __uint_as_float(r0[j]);
            v[32 + j] = __uint_as_float(r1[j]);
          }
        }
        if (p.halves) {
          const int wb = tb.weightb[sb];
          if (p.bias[w]) {
            const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias[w]) + tb.row0[sb];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(bp[j]);
          }
          if (p.bias[wb]) {
            const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias[wb]) + tb.row0b[sb];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[32 + j] += __bfloat162float(bp[j]);
          }
        } else if (p.bias[w]) {
          const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias[w]) + tb.row0[sb];
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] += __bfloat162float(bp[j]);
        }
        if (p.act == SAF_ACT_GELU) {
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] = gelu_erf(v[j]);
        }
        if (swiglu) {   // v holds the gate block; the up block is the next 64 accumulator columns
          uint32_t q0[32], q1[32];
          tmem_ld32(tsrc + (u + 1) * 64, q0);
          tmem_ld32(tsrc + (u + 1) * 64 + 32, q1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = silu_mul(v[j], __uint_as_float(q0[j]));
            v[32 + j] = silu_mul(v[32 + j], __uint_as_float(q1[j]));
          }
        }
        const int out_col = swiglu ? (tn * GN + u * 64) / 2 : tn * GN + u * 64;
        if (p.residual && m < p.M) {   // this row's 64 residual values: one 128-byte line
          const uint4* rr = reinterpret_cast<const uint4*>(p.residual + (int64_t)m * p.ldr + out_col);
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const uint4 q = rr[c8];
            const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              v[c8 * 8 + 2 * e] += __uint_as_float(w4[e] << 16);
              v[c8 * 8 + 2 * e + 1] += __uint_as_float(w4[e] & 0xffff0000u);
            }
          }
        }
        if (rp) {   // warp-uniform: rows past M are rotated too (t stays a valid table row) and clipped by the store
          const float* cr = p.cosT + (int64_t)t * p.slab;
          const float* sr = p.sinT + (int64_t)t * p.slab;
          if (p.slab == 64) {
            // pairs (d, d+32) live in this block
            // each thread reads its own table row: 16-byte loads (a row is 256 B, 16-byte aligned)
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const float4 c4 = cs4[j4];
              const float4 s4 = sn4[j4];
              const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int j = j4 * 4 + e;
                const float x1 = v[j], x2 = v[32 + j];
                v[j] = x1 * cc[e] - x2 * ss[e];
                v[32 + j] = x2 * cc[e] + x1 * ss[e];
              }
            }
          } else {
            // slab 128: partner block is the other 64-column block of the same tile
            const int pu = u ^ 1;
            uint32_t q0[32], q1[32];
            tmem_ld32(tsrc + pu * 64, q0);
            tmem_ld32(tsrc + pu * 64 + 32, q1);
            tmem_ld_wait();
            const __nv_bfloat16* bp = p.bias[w] ? reinterpret_cast<const __nv_bfloat16*>(p.bias[w]) + tb.row0[tn * SUBS + pu] : nullptr;
#pragma unroll
            for (int j4 = 0; j4 < 16; ++j4) {
              const float4 c4 = reinterpret_cast<const float4*>(cr + in_slab)[j4];
              const float4 s4 = reinterpret_cast<const float4*>(sr + in_slab)[j4];
              const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int j = j4 * 4 + e;
                float o = __uint_as_float(j < 32 ? q0[j] : q1[j - 32]);
                if (bp) o += __bfloat162float(bp[j]);
                // first half: x1*c - x2*s ; second half: x2*c + x1*s
                v[j] = (in_slab == 0) ? (v[j] * cc[e] - o * ss[e]) : (v[j] * cc[e] + o * ss[e]);
              }
            }
          }
        }
        // bf16 pack -> swizzled staging: 16-byte chunk c of row r lands at chunk (c ^ (r & 7))
        uint8_t* dst = out_stage + ob * (OUT_BYTES / 2) + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 q;
          q.x = pack_bf16(v[c * 8 + 0], v[c * 8 + 1]);
          q.y = pack_bf16(v[c * 8 + 2], v[c * 8 + 3]);
          q.z = pack_bf16(v[c * 8 + 4], v[c * 8 + 5]);
          q.w = pack_bf16(v[c * 8 + 6], v[c * 8 + 7]);
          *reinterpret_cast<uint4*>(dst + ((c ^ (row & 7)) << 4)) = q;
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (etid == 0) {
          tma_store_2d(&mapO, out_stage + ob * (OUT_BYTES / 2), out_col, tm * C::ROWS + rank * GM);
          tma_store_commit();
        }
      }
      // accumulator buffer can be overwritten by the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(cluster_addr_of(&sl->acc_empty[buf], 0));   // the even CTA's MMA warp waits
        else mbar_arrive(&sl->acc_empty[buf]);
      }
    }
    if (etid == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {
    cluster_sync_all();               // nothing of the peer's is touched after this point
    if (warp == 1) tmem_dealloc_pair(tmem, 512);
  } else {
    if (warp == 1) tmem_dealloc(tmem, 512);
  }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

int launch_gemm_sm100(const SafIndexedLinearArgs& a, cudaStream_t st) {
  if (a.dtype != SAF_BF16) return SAF_ERR_UNSUPPORTED;
  // slabs of 64 or 128 rows are whole 64-row weight blocks; other multiples of 32 (head_dim 96) are served as runs
  // of 32 rows, two per block, when the total width still fills whole 64-column blocks.  The rotation is fused in
  // the epilogue for the first kind only; for the second it runs as a second launch over the output.
  const bool halves = a.slab != 64 && a.slab != 128;
  if (halves && (a.slab % 32 || (a.n_slabs * a.slab) % 64 || a.act != SAF_ACT_NONE || a.residual)) return SAF_ERR_UNSUPPORTED;
  const int N = a.n_slabs * a.slab;
  if (N / 64 > MAX_SUB) return SAF_ERR_UNSUPPORTED;
  if (a.C % 8 || a.ldx % 8 || a.ldo % 8 || !aligned16(a.x) || !aligned16(a.out)) return SAF_ERR_UNSUPPORTED;
  if ((a.rope_cos && !aligned16(a.rope_cos)) || (a.rope_sin && !aligned16(a.rope_sin))) return SAF_ERR_UNSUPPORTED;
  if (a.residual && (!aligned16(a.residual) || a.ldr % 8)) return SAF_ERR_UNSUPPORTED;
  if (a.act == SAF_ACT_SWIGLU) {
    // (gate, up) pairs of 64-row blocks, no bias, no rotation; every tile holds whole pairs (4 blocks per tile)
    if (a.slab != 64 || a.n_slabs % 2 || a.slab_rope) return SAF_ERR_UNSUPPORTED;
    for (int w = 0; w < a.n_weights; ++w)
      if (a.biases[w]) return SAF_ERR_UNSUPPORTED;
  }
  for (int w = 0; w < a.n_weights; ++w) {
    if (!a.weights[w]) continue;
    if (a.ldw[w] % 8 || (a.cdw[w] != 0 && a.cdw[w] != 1) || !aligned16(a.weights[w])) return SAF_ERR_UNSUPPORTED;
  }
  if (!saf_device_supported()) return SAF_ERR_UNSUPPORTED;

  CUtensorMap mx, mw[4], mo;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)a.C, (uint64_t)a.M};
    uint64_t strides[2] = {0, (uint64_t)a.ldx * 2};
    uint32_t box[2] = {GK, GM};
    if ((rc = make_tensor_map_bf16(&mx, a.x, 2, dims, strides, box, true))) return rc;
  }
  for (int w = 0; w < 4; ++w) {
    const int ww = (w < a.n_weights && a.weights[w]) ? w : 0;
    uint64_t dims[2] = {(uint64_t)a.C, (uint64_t)a.rows_w[ww]};
    uint64_t strides[2] = {0, (uint64_t)a.ldw[ww] * 2};
    uint32_t box[2] = {GK, halves ? 32u : 64u};
    if ((rc = make_tensor_map_bf16(&mw[w], a.weights[ww], 2, dims, strides, box, true))) return rc;
  }
  {
    // gated MLP: the output holds one column per (gate, up) pair
    uint64_t dims[2] = {(uint64_t)(a.act == SAF_ACT_SWIGLU ? N / 2 : N), (uint64_t)a.M};
    uint64_t strides[2] = {0, (uint64_t)a.ldo * 2};
    uint32_t box[2] = {64, GM};
    if ((rc = make_tensor_map_bf16(&mo, a.out, 2, dims, strides, box, false))) return rc;
  }
  SubTable tb;
  memset(&tb, 0, sizeof(tb));
  bool rope_after = false;
  if (halves) {
    for (int hb = 0; hb < N / 32; ++hb) {          // 32-column runs of the output, two per block
      const int g = (hb * 32) / a.slab, r = (hb * 32) % a.slab;
      if (hb & 1) {
        tb.row0b[hb >> 1] = a.slab_row0[g] + r;
        tb.weightb[hb >> 1] = (uint8_t)a.slab_weight[g];
      } else {
        tb.row0[hb >> 1] = a.slab_row0[g] + r;
        tb.weight[hb >> 1] = (uint8_t)a.slab_weight[g];
      }
    }
    if (a.slab_rope)
      for (int g = 0; g < a.n_slabs; ++g) rope_after |= a.slab_rope[g] != 0;
  } else {
    const int per = a.slab / 64;
    for (int g = 0; g < a.n_slabs; ++g)
      for (int u = 0; u < per; ++u) {
        tb.row0[g * per + u] = a.slab_row0[g] + u * 64;
        tb.weight[g * per + u] = (uint8_t)a.slab_weight[g];
        tb.rope[g * per + u] = (uint8_t)(a.slab_rope ? (a.slab_rope[g] != 0) : 0);
      }
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = a.M; p.N = N; p.K = a.C; p.T = a.T; p.slab = a.slab;
  p.tiles_m = (a.M + GM - 1) / GM;
  p.tiles_n = (N + GN - 1) / GN;
  for (int w = 0; w < a.n_weights; ++w) p.bias[w] = a.biases[w];
  p.cosT = a.rope_cos;
  p.sinT = a.rope_sin;
  p.status = a.status;
  p.act = a.act;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ldr = a.ldr;
  p.halves = halves ? 1 : 0;

  const int sm_count = device_sm_count();
  // CTA pairs on 256-row tiles when the product is large enough to fill the machine with them
  const char* pair_env = getenv("SAF_B200_GEMM_PAIR");
  const bool pair_off = pair_env && pair_env[0] == '0' && pair_env[1] == 0;
  if (!pair_off && a.M >= 2 * GM * 32 && N >= GN) {
    constexpr size_t smem_p = 1024 + GCfg<true>::STAGES * GCfg<true>::STAGE_BYTES + OUT_BYTES + sizeof(SmemLayout);
    static_assert(smem_p <= 227 * 1024, "pair kernel shared memory");
    static PerDeviceOnce smem_once_p;
    if ((rc = ensure_dyn_smem(indexed_gemm_kernel<true>, (int)smem_p, smem_once_p))) return rc;
    p.tiles_m = (a.M + 2 * GM - 1) / (2 * GM);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem_p;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // pairs that can be resident at once (an SM without a free neighbour in its GPC stays out)
    static std::atomic<int> pairs_cache[SAF_MAX_DEVICES];
    const int dev = current_device();
    int pairs = (dev >= 0 && dev < SAF_MAX_DEVICES) ? pairs_cache[dev].load(std::memory_order_acquire) : 0;
    if (pairs <= 0) {
      cfg.gridDim = dim3(sm_count & ~1);
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, indexed_gemm_kernel<true>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = sm_count / 2;
      }
      pairs = n;
      if (dev >= 0 && dev < SAF_MAX_DEVICES) pairs_cache[dev].store(pairs, std::memory_order_release);
    }
    pairs = std::min(pairs, p.tiles_m * p.tiles_n);
    cfg.gridDim = dim3(2 * pairs);
    cudaError_t e = cudaLaunchKernelEx(&cfg, indexed_gemm_kernel<true>, mx, mw[0], mw[1], mw[2], mw[3], mo, p, tb);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(SAF_ERR_CUDA, "indexed_gemm_kernel<pair> launch: %s", cudaGetErrorString(e));
    }
    count_launch();
    if ((rc = check_launch("indexed_gemm_kernel<pair>"))) return rc;
  } else {
    constexpr size_t smem = 1024 + GCfg<false>::STAGES * GCfg<false>::STAGE_BYTES + OUT_BYTES + sizeof(SmemLayout);
    static PerDeviceOnce smem_once;
    if ((rc = ensure_dyn_smem(indexed_gemm_kernel<false>, (int)smem, smem_once))) return rc;
    const int grid = std::min(sm_count, p.tiles_m * p.tiles_n);
    indexed_gemm_kernel<false><<<grid, GEMM_THREADS, smem, st>>>(mx, mw[0], mw[1], mw[2], mw[3], mo, p, tb);
    count_launch();
    if ((rc = check_launch("indexed_gemm_kernel"))) return rc;
  }
  if (rope_after)
    return launch_rope_slabs(a.out, a.ldo, a.M, a.n_slabs, a.slab, a.T, a.slab_rope, a.rope_cos, a.rope_sin, a.dtype, 0, st);
  return SAF_OK;
}

}  // namespace saf
