// Device code of the tensor-core scan of structured (sink + decay) heads: shared by the stand-alone launch
// (scan_mma_sm100.cu, which explains the method) and by the mixed-attention launches, whose leading CTAs run it for the
// structured heads of a call while the other CTAs work on the live heads.
#pragma once
#include "saf_internal.h"
#include "scan_body.cuh"
#include "sm100_prims.cuh"

namespace saf {

constexpr int MB = 128;                 // rows per block
constexpr int MS_MAX_STAGES = 11;         // V tiles in flight (the stand-alone kernel; co-scheduled CTAs take fewer)
constexpr int MS_TILE = MB * 64 * 2;    // 16 KB: one V tile, one output tile
constexpr int MS_THREADS = 320;          // TMA warp, MMA warp, two epilogue warpgroups
constexpr int MS_ACC = 4;               // TMEM accumulators
constexpr int MS_OUT = 2;               // staging tiles: one per epilogue warpgroup
constexpr int MS_TL = MS_ACC * 64;      // TMEM column of the Toeplitz operand: bf16 head (64 columns), remainder (64)

struct MsBars {
  uint64_t full[MS_MAX_STAGES], empty[MS_MAX_STAGES], acc_full[MS_ACC], acc_empty[MS_ACC], carry_ready[4], l_ready;
  uint32_t tmem_base;
  alignas(16) float carry[4][64];      // carry[n & 3]: the state block n inherits
  alignas(16) float av0[2][64];        // sink term a * v_0 of each column slice
};
// dynamic shared memory of a CTA with a ring of `stages` V tiles
constexpr int ms_smem_bytes(int stages) { return 1024 + (stages + MS_OUT) * MS_TILE + 2048; }
static_assert(ms_smem_bytes(MS_MAX_STAGES) <= 227 * 1024, "shared memory limit");

#ifdef SAF_SCAN_TRACE
__device__ long long g_strace[12][64];   // (a trace build includes this header in one translation unit only)
#define STRACE(evt, step) do { if (trace_on && (step) < 64) g_strace[evt][step] = clock64(); } while (0)
#else
#define STRACE(evt, step) do { } while (0)
#endif

struct MsParams {
  ScanArgs a;
  int chunk;           // rows per chunk (a multiple of 128)
  int use_stash;       // 1: the chunk's incoming carry sits in its stash; 0: zero carry
  int* status;
};

// Body of one CTA: rows [chunk_idx * p.chunk, ...) of head (b, h), columns [64 slice, 64 (slice + n_slices)), through
// the tensor core.  With n_slices = 2 (zero carry only) the CTA walks the rows once per 64-column slice, back to back
// through the same rings: the running block index goes on, the carry restarts at zero at the slice boundary.  Every thread of the CTA must call it (it holds CTA-wide barriers); the first ten warps work, further warps only
// take part in those barriers.  STAGES V tiles are in flight; `smem_raw` is the CTA's dynamic shared memory, at least
// ms_smem_bytes(STAGES) bytes.
template <int STAGES>
__device__ __forceinline__ void sink_decay_apply_mma_cta(const CUtensorMap& mapV, const CUtensorMap& mapY, const MsParams& p,
                                                         int b, int h, int chunk_idx, int slice, int n_slices, uint8_t* smem_raw) {
  static_assert(STAGES >= 2 && STAGES <= MS_MAX_STAGES, "ring depth");
  constexpr int MS_STAGES = STAGES;
  const ScanArgs& a = p.a;
  const int col0 = slice * SCAN_COLS;
  const int p_lo = chunk_idx * p.chunk, p_hi = min(a.T, p_lo + p.chunk);
  const int blocks_per_slice = (p_hi - p_lo + MB - 1) / MB;
  const int n_blocks = blocks_per_slice * n_slices;                 // running block n = (slice n / bps, block n % bps)
  const int hin = a.HKV > 0 ? (a.kvidx ? a.kvidx[h] : 0) : h;
#ifdef SAF_SCAN_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#endif

  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sV = smem;
  uint8_t* sY = sV + MS_STAGES * MS_TILE;
  MsBars* bars = reinterpret_cast<MsBars*>(sY + MS_OUT * MS_TILE);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < MS_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < MS_ACC; ++i) {
      mbar_init(&bars->acc_full[i], 1);
      mbar_init(&bars->acc_empty[i], 4);              // one arrival per epilogue warp
    }
    for (int i = 0; i < 4; ++i) mbar_init(&bars->carry_ready[i], 1);
    mbar_init(&bars->l_ready, 256);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&mapV);
      for (int n = 0; n < n_blocks; ++n) {
        const int s = n % MS_STAGES;
        if (!mbar_wait(&bars->empty[s], ((n / MS_STAGES) & 1) ^ 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 70);
          break;
        }
        STRACE(0, n);
        mbar_expect_tx(&bars->full[s], MS_TILE);
        tma_load_4d(sV + s * MS_TILE, &mapV, &bars->full[s], col0 + (n / blocks_per_slice) * SCAN_COLS,
                    p_lo + (n % blocks_per_slice) * MB, hin, b);
      }
    }
  } else if (warp == 1) {
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(MB, 64, 0, 1);     // L from TMEM (K-major), V MN-major in shared memory
    const uint32_t vbase = smem_u32(sV);
    bool ok = mbar_wait(&bars->l_ready, 0);
    if (!ok) dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 71);
    tc_fence_after();
    for (int n = 0; n < n_blocks && ok; ++n) {
      const int s = n % MS_STAGES, buf = n % MS_ACC;
      if (!mbar_wait(&bars->full[s], (n / MS_STAGES) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 72);
        break;
      }
      if (leader) STRACE(1, n);
      if (n >= MS_ACC && !mbar_wait(&bars->acc_empty[buf], ((n / MS_ACC) & 1) ^ 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 73);
        break;
      }
      tc_fence_after();
      const uint32_t d = tmem + buf * 64, va = vbase + s * MS_TILE;
      if (leader) {
        STRACE(2, n);
#pragma unroll
        for (int part = 0; part < 2; ++part)
#pragma unroll
          for (int ks = 0; ks < MB / 16; ++ks)            // 16 rows of V = 8 TMEM columns of packed bf16 pairs
            umma_ts(d, tmem + MS_TL + part * 64 + ks * 8, umma_smem_desc_sw128(va + ks * 2048, 16384, 1024), idesc,
                    (part | ks) != 0);
        umma_commit(&bars->empty[s]);
        umma_commit(&bars->acc_full[buf]);
        STRACE(3, n);
      }
      __syncwarp();
    }
  } else if (warp < 10) {
    // ------------------------------------------------- epilogue: two warpgroups take alternate blocks, thread = row
    const int wg = (warp - 2) >> 2;                         // 0: even blocks, 1: odd blocks
    const int et = (tid - 64) & 127;                        // thread of the warpgroup
    const int quad = warp & 3;                              // TMEM lane quadrant of this warp
    const int lrow = quad * 32 + lane;                      // the TMEM lane (block row) this thread reads
    const float alpha = a.sd_alpha[h], r = a.sd_rho[h];
    const float log_r = (r > 0.f && r < 1.f) ? log1pf(r - 1.f) : 0.f;
    const uint32_t tlane = tmem + ((uint32_t)(quad * 32) << 16);
    // incoming carry (read before any output row of this chunk is stored) and v_0 for the sink term: the loads are in
    // flight while the Toeplitz operand is built
    float carry_in = 0.f, v_first = 0.f;
    if (et < 64 * (wg == 0 ? 1 : n_slices - 1)) {          // warpgroup 0: slice 0 (and the stash); warpgroup 1: slice 1
      const int sl = wg;
      const __nv_bfloat16* ob0 = reinterpret_cast<const __nv_bfloat16*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)col0;
      if (p.use_stash && wg == 0) carry_in = *scan_stash<__nv_bfloat16>(const_cast<__nv_bfloat16*>(ob0), a.so[2], p_lo, et);
      const __nv_bfloat16* v0 = reinterpret_cast<const __nv_bfloat16*>(a.in) + (int64_t)b * a.si[0] + (int64_t)hin * a.si[1] +
                                (int64_t)(col0 + sl * SCAN_COLS + et);
      v_first = __bfloat162float(*v0);
    }
    // Toeplitz operand in TMEM, row `lrow`, column k = the bf16 pair (L[2k], L[2k+1]): its bf16 head from warpgroup 0
    // and the bf16 remainder from warpgroup 1
    {
      uint32_t w0[32], w1[32];
      float val = 1.f;                                      // r^(lrow - j), from the diagonal leftwards
#pragma unroll
      for (int k = MB / 2 - 1; k >= 0; --k) {
        float x0 = 0.f, x1 = 0.f;
        if (2 * k + 1 <= lrow) {
          x1 = val;
          val *= r;
        }
        if (2 * k <= lrow) {
          x0 = val;
          val *= r;
        }
        const uint32_t hi = pack_bf16(x0, x1);
        const uint32_t word = wg == 0 ? hi : pack_bf16(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
        if (k < 32) w0[k] = word;
        else w1[k - 32] = word;
      }
      tmem_st32(tlane + MS_TL + wg * 64, w0);
      tmem_st32(tlane + MS_TL + wg * 64 + 32, w1);
      tmem_st_wait();
      tc_fence_before();
    }
    if (et < 64 * (wg == 0 ? 1 : n_slices - 1)) {
      if (wg == 0) bars->carry[0][et] = carry_in;
      bars->av0[wg][et] = alpha * v_first;
    }
    mbar_arrive(&bars->l_ready);
    named_bar_sync(3, 256);                                 // carry[0] and av0 are in place for both warpgroups
    if (wg == 0 && et == 0) mbar_arrive(&bars->carry_ready[0]);
    float pw = r;                                           // r^(lrow + 1)
    for (int i = 0; i < lrow; ++i) pw *= r;
    const uint32_t tsrc = tlane;
    for (int n = wg; n < n_blocks; n += 2) {
      const int buf = n % MS_ACC, slot = n & 3;
      const int sl = n / blocks_per_slice, blk = n - sl * blocks_per_slice;
      const float4* a4 = reinterpret_cast<const float4*>(bars->av0[sl]);
      // the row's weight (1 - a) / Z_i waits for nothing
      const float w = (1.f - alpha) * inv_z(r, log_r, p_lo + blk * MB + lrow + 1);
      bool ok = mbar_wait(&bars->acc_full[buf], (n / MS_ACC) & 1);
      uint32_t s0[32], s1[32];
      if (et == 0) STRACE(4, n);
      if (ok) {
        tc_fence_after();
        tmem_ld32(tsrc + buf * 64, s0);
        tmem_ld32(tsrc + buf * 64 + 32, s1);
        tmem_ld_wait();
        tc_fence_before();
      }
      __syncwarp();
      if (et == 0) STRACE(5, n);
      if (ok && lane == 0) mbar_arrive(&bars->acc_empty[buf]);
      ok = ok && mbar_wait(&bars->carry_ready[slot], (n >> 2) & 1);
      if (et == 0) STRACE(6, n);
      // s_i = (L V)_i + r^(i+1) carry, in place
      if (ok) {
        const float4* c4 = reinterpret_cast<const float4*>(bars->carry[slot]);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {                     // 32 columns at a time: loads first, then the arithmetic
          float4 cc[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) cc[q] = c4[hh * 8 + q];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint32_t* x = (hh == 0 ? s0 : s1) + q * 4;
            x[0] = __float_as_uint(fmaf(pw, cc[q].x, __uint_as_float(x[0])));
            x[1] = __float_as_uint(fmaf(pw, cc[q].y, __uint_as_float(x[1])));
            x[2] = __float_as_uint(fmaf(pw, cc[q].z, __uint_as_float(x[2])));
            x[3] = __float_as_uint(fmaf(pw, cc[q].w, __uint_as_float(x[3])));
          }
        }
        // the state at the end of the block goes out first: the other warpgroup's next block waits for it alone
        if (lrow == MB - 1) {
          uint4* n4 = reinterpret_cast<uint4*>(bars->carry[(n + 1) & 3]);
          const uint32_t keep = blk + 1 == blocks_per_slice ? 0u : 0xffffffffu;   // a new column slice starts from zero
#pragma unroll
          for (int q = 0; q < 8; ++q)
            n4[q] = make_uint4(s0[q * 4] & keep, s0[q * 4 + 1] & keep, s0[q * 4 + 2] & keep, s0[q * 4 + 3] & keep);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            n4[8 + q] = make_uint4(s1[q * 4] & keep, s1[q * 4 + 1] & keep, s1[q * 4 + 2] & keep, s1[q * 4 + 3] & keep);
          mbar_arrive(&bars->carry_ready[(n + 1) & 3]);
          STRACE(7, n);
        }
      }
      // the staging tile is free once this warpgroup's previous store has read it
      if (et == 0) tma_store_wait_read();
      if (named_bar_or(1 + wg, 128, !ok)) {                  // the four warps give up together
        if (!ok) dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 74);
        break;
      }
      if (et == 0) STRACE(8, n);
      uint8_t* dst = sY + wg * MS_TILE + lrow * 128;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {                       // 32 columns at a time: the sink terms, then the stores
        float4 aa[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) aa[q] = a4[hh * 8 + q];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t* xu = (hh == 0 ? s0 : s1) + q * 8;
          float x[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(xu[e]);
          const float4 a0 = aa[q * 2], a1 = aa[q * 2 + 1];
          uint4 o;
          o.x = pack_bf16(fmaf(w, x[0], a0.x), fmaf(w, x[1], a0.y));
          o.y = pack_bf16(fmaf(w, x[2], a0.z), fmaf(w, x[3], a0.w));
          o.z = pack_bf16(fmaf(w, x[4], a1.x), fmaf(w, x[5], a1.y));
          o.w = pack_bf16(fmaf(w, x[6], a1.z), fmaf(w, x[7], a1.w));
          *reinterpret_cast<uint4*>(dst + (((hh * 4 + q) ^ (lrow & 7)) << 4)) = o;
        }
      }
      fence_proxy_async_smem();
      if (et == 0) STRACE(9, n);
      named_bar_sync(1 + wg, 128);
      if (et == 0) {
        tma_store_4d(&mapY, sY + wg * MS_TILE, col0 + sl * SCAN_COLS, p_lo + blk * MB, h, b);
        tma_store_commit();
        STRACE(10, n);
      }
    }
    if (et == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}


}  // namespace saf
