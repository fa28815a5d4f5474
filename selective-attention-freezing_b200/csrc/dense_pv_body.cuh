// Dense-stored frozen heads (state 1) as a TMA-staged lower-triangular GEMM on tcgen05:
//
//   Y[b, h, i, :] = sum_{j <= i} P[pidx[h], i, j] * V[b, h, j, :]
//
// Replaces _acc_dense / _pv_fwd_kernel (kernel/fused_attn.py:125-143, kernel/frozen_attn.py:51-89), which
// stream 64x64 pattern tiles through registers once per batch row.  Here a pattern tile never visits the
// register file: TMA lands it in shared memory in the layout the tensor core reads (A operand, K-major),
// and ONE copy of it multiplies the value tiles of up to 256/head_dim batch rows, so the T^2/2 pattern
// elements -- the only large operand -- cross HBM once per group of batch rows instead of once per row.
//
// CTA = two consecutive 128-row tiles of one head for a group of NB = 256/head_dim batch rows:
// 2 * NB accumulators of head_dim columns fill the 512 TMEM columns.  Keys advance 64 at a time:
//   stage = [P tile 0: 128 x 64 | P tile 1: 128 x 64 | V of NB batch rows: 64 x head_dim each] = 64 KB, 3 stages
//   warp 0      TMA producer
//   warp 1      MMA issuer: O[t][b] += P_t (SS, K-major) * V_b (MN-major), 4 k-steps of 16 keys
//   warps 2-5   zero the above-diagonal entries of the (at most four) diagonal stages in shared memory,
//               then the epilogue: TMEM -> bf16 -> swizzled staging -> TMA store
// Work per stage: 2 * NB * 128 * 64 * head_dim MACs against 32 KB of pattern read from HBM: at head_dim 64
// that is ~1500 tensor cycles per 32 KB per SM, i.e. the kernel sits at the HBM roofline of the pattern.
// All waits are bounded.
#pragma once
#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {

struct DpParams {
  int B, H, T, n_pairs, groups, force_state, HKV;
  int split_from;            // forward: row pairs mp >= split_from run as two CTAs, one per 128-row tile
  const int32_t* frozen;
  const int32_t* pidx;
  const int32_t* kvidx;
  int* status;
  int dense_ok;              // dense-stored heads: pattern tiles come by TMA
  // decomposed heads: pattern tiles exp(alpha_j + rho_{i-j} - z_i) are generated in shared memory
  int dec_ok, dec_dtype;
  const void *alpha, *rho, *z;
  int64_t alpha_s[2], rho_s[2], z_s[2];
};

// can the bf16 TMA-staged kernel serve the dense heads of this call?
inline bool dense_pv_eligible(const SafMixedAttnArgs& a) {
  auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
  auto tma_ok = [&](const SafTensor& t) {
    if (!t.ptr || !al16(t.ptr) || t.stride[3] != 1) return false;
    for (int i = 0; i < 3; ++i)
      if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
    return true;
  };
  if (a.dtype != SAF_BF16 || (a.HD != 64 && a.HD != 128)) return false;
  if (!a.patt.ptr || a.patt_dtype != SAF_BF16 || a.patt.stride[2] != 1 || !al16(a.patt.ptr)) return false;
  if (a.patt.stride[0] % 8 || a.patt.stride[1] % 8 || a.patt.stride[0] <= 0 || a.patt.stride[1] <= 0) return false;
  if (a.S < a.T) return false;
  return tma_ok(a.v) && tma_ok(a.out);
}

// tensor maps (pattern planes, 64-key value tiles, output tiles) and parameters of the dense role
inline int dense_pv_prepare(const SafMixedAttnArgs& a, bool dense, bool decomp, CUtensorMap* mp_, CUtensorMap* mv,
                            CUtensorMap* mo, DpParams* p) {
  int rc;
  memset(mp_, 0, sizeof(*mp_));
  if (dense) {
    // pattern (P, S, S): box 64 keys x 128 rows of one plane; the plane index comes from pidx, its range is
    // the caller's contract
    uint64_t dims[3] = {(uint64_t)a.S, (uint64_t)a.S, (uint64_t)1 << 20};
    uint64_t strides[3] = {0, (uint64_t)a.patt.stride[1] * 2, (uint64_t)a.patt.stride[0] * 2};
    uint32_t box[3] = {64, 128, 1};
    if ((rc = make_tensor_map_bf16(mp_, a.patt.ptr, 3, dims, strides, box, true))) return rc;
  }
  const int Hkv = a.HKV > 0 ? a.HKV : a.H;
  {
    uint64_t dims[4] = {(uint64_t)a.HD, (uint64_t)a.T, (uint64_t)Hkv, (uint64_t)a.B};
    uint64_t strides[4] = {0, (uint64_t)a.v.stride[2] * 2, (uint64_t)a.v.stride[1] * 2, (uint64_t)a.v.stride[0] * 2};
    uint32_t box[4] = {64, 64, 1, 1};
    if ((rc = make_tensor_map_bf16(mv, a.v.ptr, 4, dims, strides, box, true))) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)a.HD, (uint64_t)a.T, (uint64_t)a.H, (uint64_t)a.B};
    uint64_t strides[4] = {0, (uint64_t)a.out.stride[2] * 2, (uint64_t)a.out.stride[1] * 2, (uint64_t)a.out.stride[0] * 2};
    uint32_t box[4] = {64, 128, 1, 1};
    if ((rc = make_tensor_map_bf16(mo, a.out.ptr, 4, dims, strides, box, false))) return rc;
  }
  memset(p, 0, sizeof(*p));
  p->B = a.B; p->H = a.H; p->T = a.T; p->force_state = a.force_state; p->HKV = a.HKV;
  p->n_pairs = (a.T + 255) / 256;
  p->groups = (a.B + 256 / a.HD - 1) / (256 / a.HD);
  p->frozen = a.frozen; p->pidx = a.pidx; p->kvidx = a.kvidx;
  p->status = a.status;
  p->dense_ok = dense ? 1 : 0;
  p->dec_ok = decomp ? 1 : 0;
  // A row pair m walks 4m + 4 key steps for two tiles: the CTAs of a long sequence differ in length by the factor
  // n_pairs, and the longest alone takes 1.5x the average load of an SM when a few heads fill the machine.  The top
  // eighth (quarter at head_dim 128) of the row pairs is therefore cut into its two tiles.  A one-tile CTA costs about
  // 0.7 of a pair's step, not 0.5 (V is read by both), so cutting more loses more than the balance gains: measured
  // 0.294 -> 0.267 ms at c2 (3 heads, T=16384), 0.135 -> 0.112 ms at the c3 shape.
  // Stored patterns only: the generated (decomposed) form builds both tiles with fixed warp groups.
  {
    const int eighths = a.HD == 128 ? 6 : 7;
    p->split_from = (decomp || p->n_pairs < 8) ? p->n_pairs : p->n_pairs * eighths / 8;
  }
  if (decomp) {
    p->alpha = a.alpha.ptr; p->rho = a.rho.ptr; p->z = a.z.ptr;
    for (int i = 0; i < 2; ++i) {
      p->alpha_s[i] = a.alpha.stride[i];
      p->rho_s[i] = a.rho.stride[i];
      p->z_s[i] = a.z.stride[i];
    }
    p->dec_dtype = a.dec_dtype;
  }
  return SAF_OK;
}
// decomposed heads need only the value / output layout the TMA path needs
inline bool dense_pv_decomp_eligible(const SafMixedAttnArgs& a) {
#ifdef SAF_NO_DECOMP_ROLE
  return false;   // comparison builds: decomposed heads stay on the per-batch-row register path
#endif
  auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
  auto tma_ok = [&](const SafTensor& t) {
    if (!t.ptr || !al16(t.ptr) || t.stride[3] != 1) return false;
    for (int i = 0; i < 3; ++i)
      if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
    return true;
  };
  if (a.dtype != SAF_BF16 || (a.HD != 64 && a.HD != 128)) return false;
  if (!a.alpha.ptr || !a.rho.ptr || !a.z.ptr || a.SD < a.T) return false;
  return tma_ok(a.v) && tma_ok(a.out);
}
inline unsigned dense_pv_slots(const DpParams& p) {
  return (unsigned)((p.n_pairs + (p.n_pairs - p.split_from)) * p.H * p.groups);
}

// backward of dense-stored heads, dV = tril(P)^T dO: same role with the pattern read as a transposed (MN-major)
// A operand in 64-query steps.  Maps: pattern in 64 x 64 boxes, dO in 64-row boxes, dV in 128-row boxes.
inline bool dense_dv_eligible(const SafMixedAttnBwdArgs& g) {
  const SafMixedAttnArgs& a = g.fwd;
  auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
  auto tma_ok = [&](const SafTensor& t) {
    if (!t.ptr || !al16(t.ptr) || t.stride[3] != 1) return false;
    for (int i = 0; i < 3; ++i)
      if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
    return true;
  };
  if (a.dtype != SAF_BF16 || (a.HD != 64 && a.HD != 128) || a.HKV > 0) return false;
  if (!a.patt.ptr || a.patt_dtype != SAF_BF16 || a.patt.stride[2] != 1 || !al16(a.patt.ptr)) return false;
  if (a.patt.stride[0] % 8 || a.patt.stride[1] % 8 || a.patt.stride[0] <= 0 || a.patt.stride[1] <= 0) return false;
  if (a.S < a.T) return false;
  return tma_ok(g.dout) && tma_ok(g.dv);
}
// decomposed heads in the backward need only the dO / dV layouts
inline bool dense_dv_decomp_eligible(const SafMixedAttnBwdArgs& g) {
  const SafMixedAttnArgs& a = g.fwd;
  auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
  auto tma_ok = [&](const SafTensor& t) {
    if (!t.ptr || !al16(t.ptr) || t.stride[3] != 1) return false;
    for (int i = 0; i < 3; ++i)
      if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
    return true;
  };
  if (a.dtype != SAF_BF16 || (a.HD != 64 && a.HD != 128) || a.HKV > 0) return false;
  if (!a.alpha.ptr || !a.rho.ptr || !a.z.ptr || a.SD < a.T) return false;
  return tma_ok(g.dout) && tma_ok(g.dv);
}
inline int dense_dv_prepare(const SafMixedAttnBwdArgs& g, bool dense, bool decomp, CUtensorMap* mp_, CUtensorMap* mdo,
                            CUtensorMap* mdv, DpParams* p) {
  const SafMixedAttnArgs& a = g.fwd;
  int rc;
  memset(mp_, 0, sizeof(*mp_));
  if (dense) {
    uint64_t dims[3] = {(uint64_t)a.S, (uint64_t)a.S, (uint64_t)1 << 20};
    uint64_t strides[3] = {0, (uint64_t)a.patt.stride[1] * 2, (uint64_t)a.patt.stride[0] * 2};
    uint32_t box[3] = {64, 64, 1};
    if ((rc = make_tensor_map_bf16(mp_, a.patt.ptr, 3, dims, strides, box, true))) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)a.HD, (uint64_t)a.T, (uint64_t)a.H, (uint64_t)a.B};
    uint64_t strides[4] = {0, (uint64_t)g.dout.stride[2] * 2, (uint64_t)g.dout.stride[1] * 2, (uint64_t)g.dout.stride[0] * 2};
    uint32_t box[4] = {64, 64, 1, 1};
    if ((rc = make_tensor_map_bf16(mdo, g.dout.ptr, 4, dims, strides, box, true))) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)a.HD, (uint64_t)a.T, (uint64_t)a.H, (uint64_t)a.B};
    uint64_t strides[4] = {0, (uint64_t)g.dv.stride[2] * 2, (uint64_t)g.dv.stride[1] * 2, (uint64_t)g.dv.stride[0] * 2};
    uint32_t box[4] = {64, 128, 1, 1};
    if ((rc = make_tensor_map_bf16(mdv, g.dv.ptr, 4, dims, strides, box, false))) return rc;
  }
  memset(p, 0, sizeof(*p));
  p->B = a.B; p->H = a.H; p->T = a.T; p->force_state = a.force_state; p->HKV = 0;
  p->n_pairs = (a.T + 255) / 256;
  p->split_from = p->n_pairs;      // the backward role keeps whole key-tile pairs
  p->groups = (a.B + 256 / a.HD - 1) / (256 / a.HD);
  p->frozen = a.frozen; p->pidx = a.pidx; p->kvidx = nullptr;
  p->status = a.status;
  p->dense_ok = dense ? 1 : 0;
  p->dec_ok = decomp ? 1 : 0;
  if (decomp) {
    p->alpha = a.alpha.ptr; p->rho = a.rho.ptr; p->z = a.z.ptr;
    for (int i = 0; i < 2; ++i) {
      p->alpha_s[i] = a.alpha.stride[i];
      p->rho_s[i] = a.rho.stride[i];
      p->z_s[i] = a.z.stride[i];
    }
    p->dec_dtype = a.dec_dtype;
  }
  return SAF_OK;
}

namespace {

constexpr int DP_THREADS = 192;
constexpr int DP_NST = 3;
constexpr int DP_PATOM = 128 * 64 * 2;     // 16 KB: 128 pattern rows x 64 keys

template <int HD>
struct DpCfg {
  static constexpr int NB = 256 / HD;                 // batch rows per CTA
  static constexpr int V_BYTES = 64 * HD * 2;         // 64 keys x head_dim
  static constexpr int STAGE = 2 * DP_PATOM + NB * V_BYTES;   // 64 KB
  static constexpr int SMEM_BYTES = 1024 + DP_NST * STAGE + 6144;
};

struct DpBars {
  uint64_t full[DP_NST], empty[DP_NST], need_mask, masked, acc_full;
  uint64_t pgen[DP_NST];     // generated pattern tiles of a stage are in place (256 arrivals: both tile groups)
  uint32_t tmem_base;
  // decomposed heads, per tile group and double-buffered over the steps (all x log2 e):
  float ga[2][2][64];        // alpha of the step's 64 keys
  float gr[2][2][192];       // rho over the 191 distances a 128-row tile sees against 64 keys
};
static_assert(sizeof(DpBars) <= 6144, "barrier block");

// Body of one CTA; `slot` counts the CTAs of this role (heaviest row pairs first).  Every thread of the CTA
// must call it (it contains CTA-wide barriers); warps 0-5 work, further warps only take part in the barriers.
template <int HD>
__device__ __forceinline__ void dense_pv_cta(const CUtensorMap& mapP, const CUtensorMap& mapV, const CUtensorMap& mapO,
                                             const DpParams& p, int slot, uint8_t* smem) {
  using C = DpCfg<HD>;
  // CTA -> (head, batch group, row pair [, tile]); heaviest first.  Row pairs from split_from up come as two slots,
  // tile 1 (one key step more) before tile 0.
  const int per_mp = p.H * p.groups;
  const int n_split = p.n_pairs - p.split_from;
  int mp, only_t = -1;                                      // only_t: the one tile this CTA computes, -1 = both
  if (slot < 2 * n_split * per_mp) {
    const int q = slot / per_mp;
    mp = p.n_pairs - 1 - (q >> 1);
    only_t = 1 - (q & 1);
  } else {
    mp = p.split_from - 1 - (slot - 2 * n_split * per_mp) / per_mp;
  }
  const int rem = slot % per_mp;
  const int h = rem / p.groups, grp = rem % p.groups;
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  const bool gen = state == SAF_DECOMP && p.dec_ok;       // pattern tiles generated, not loaded
  if (!gen && !(state == SAF_DENSE && p.dense_ok)) return;
  const int hp = p.pidx ? p.pidx[h] : h;
  const int hv = (p.HKV > 0) ? p.kvidx[h] : h;
  const int b0 = grp * C::NB;
  const int nb = min(C::NB, p.B - b0);
  const int row0 = mp * 256;
  const bool act1 = row0 + 128 < p.T && only_t != 0;
  if (only_t == 1 && !act1) return;                        // the sequence ends inside tile 0
  const int n_half = (p.T + 63) / 64;
  const int nk0 = only_t == 1 ? 0 : min(4 * mp + 2, n_half);   // 64-key steps of tile 0
  const int nkh = act1 ? min(4 * mp + 4, n_half) : nk0;    // and of the CTA
  // steps whose pattern tile holds above-diagonal entries: the two steps that cover a tile's own 128 keys
  auto diag_of = [&](int kh, int t) { return (t == 0 ? nk0 > 0 : act1) && kh >= 4 * mp + 2 * t && kh < 4 * mp + 2 * t + 2; };

  DpBars* bars = reinterpret_cast<DpBars*>(smem + DP_NST * C::STAGE);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < DP_NST; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < DP_NST; ++s) mbar_init(&bars->pgen[s], 256);
    mbar_init(&bars->need_mask, 1);
    mbar_init(&bars->masked, 128);
    mbar_init(&bars->acc_full, 1);
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
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      if (!gen) tma_prefetch_desc(&mapP);
      tma_prefetch_desc(&mapV);
      for (int kh = 0; kh < nkh; ++kh) {
        const int s = kh % DP_NST;
        if (!mbar_wait(&bars->empty[s], ((kh / DP_NST) & 1) ^ 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 70);
          break;
        }
        uint8_t* st = smem + s * C::STAGE;
        const bool t0 = kh < nk0;
        mbar_expect_tx(&bars->full[s], (gen ? 0 : (t0 ? DP_PATOM : 0) + (act1 ? DP_PATOM : 0)) + nb * C::V_BYTES);
        if (!gen && t0) tma_load_3d(st, &mapP, &bars->full[s], kh * 64, row0, hp);
        if (!gen && act1) tma_load_3d(st + DP_PATOM, &mapP, &bars->full[s], kh * 64, row0 + 128, hp);
        for (int bi = 0; bi < nb; ++bi)
#pragma unroll
          for (int hh = 0; hh < HD / 64; ++hh)
            tma_load_4d(st + 2 * DP_PATOM + bi * C::V_BYTES + hh * 8192, &mapV, &bars->full[s], hh * 64, kh * 64, hv,
                        b0 + bi);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(128, HD, 0, 1);
    const uint32_t sbase = smem_u32(smem);
    int n_masked = 0;
    for (int kh = 0; kh < nkh; ++kh) {
      const int s = kh % DP_NST;
      if (!mbar_wait(&bars->full[s], (kh / DP_NST) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 71);
        break;
      }
      if (gen) {
        if (!mbar_wait(&bars->pgen[s], (kh / DP_NST) & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 75);
          break;
        }
      } else if (diag_of(kh, 0) || diag_of(kh, 1)) {
        // the tile has landed: hand it to the mask helpers (they follow this barrier, never the ring's,
        // so they cannot run ahead of or behind the stage they are meant to edit)
        if (leader) mbar_arrive(&bars->need_mask);
        __syncwarp();
        if (!mbar_wait(&bars->masked, n_masked & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 72);
          break;
        }
        ++n_masked;
      }
      tc_fence_after();
      const uint32_t st = sbase + s * C::STAGE;
      if (leader) {
        for (int t = 0; t < 2; ++t) {
          if (t == 0 ? kh >= nk0 : !act1) continue;
          const uint32_t pa = st + t * DP_PATOM;
          for (int bi = 0; bi < nb; ++bi) {
            const uint32_t va = st + 2 * DP_PATOM + bi * C::V_BYTES;
            const uint32_t d = tmem + (t * C::NB + bi) * HD;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_ss(d, umma_smem_desc_sw128(pa + ks * 32, 16, 1024), umma_smem_desc_sw128(va + ks * 2048, 8192, 1024),
                      idesc, (kh | ks) != 0);
          }
        }
        umma_commit(&bars->empty[s]);
      }
      __syncwarp();
    }
    if (leader) umma_commit(&bars->acc_full);
    __syncwarp();
  }
  if (gen && warp >= 2 && warp < 10) {
    // ---------------------------------------------------------------- decomposed head: pattern generation
    // warps 2-5 build tile 0, warps 6-9 tile 1 (needs a CTA of at least 320 threads): thread = row, 64 keys per
    // step.  The step's alpha / rho values are fetched one step ahead into registers and handed over through
    // double-buffered shared memory, so no global latency sits on the step.
    constexpr float L2E = 1.4426950408889634f;
    const int t = (warp - 2) >> 2;                       // tile of this group
    const int gt = (tid - 64) & 127;                     // thread inside the group
    const int r = gt;                                    // row of the tile
    const int i_row = row0 + 128 * t + r;
    const bool t_on = t == 0 || act1;
    const int nk_t = t == 0 ? nk0 : nkh;                 // steps in which this tile takes part
    // +inf: rows past T give exact zeros
    const float zr = (i_row < p.T) ? L2E * load_rt(p.z, (int64_t)h * p.z_s[0] + (int64_t)i_row * p.z_s[1], p.dec_dtype) : INFINITY;
    auto fetch_a = [&](int kh) -> float {                // alpha of key 64 kh + gt   (gt < 64)
      const int key = kh * 64 + gt;
      return (gt < 64 && key < p.T) ? L2E * load_rt(p.alpha, (int64_t)h * p.alpha_s[0] + (int64_t)key * p.alpha_s[1], p.dec_dtype) : 0.f;
    };
    auto fetch_r = [&](int kh, int x) -> float {         // rho at distance (row0 + 128 t - 64 kh - 63) + x
      const int d = row0 + 128 * t - kh * 64 - 63 + x;
      return (x < 191 && d >= 0 && d < p.T) ? L2E * load_rt(p.rho, (int64_t)h * p.rho_s[0] + (int64_t)d * p.rho_s[1], p.dec_dtype) : 0.f;
    };
    float na = 0.f, nr0 = 0.f, nr1 = 0.f;
    if (t_on && nk_t > 0) {
      na = fetch_a(0); nr0 = fetch_r(0, gt); nr1 = fetch_r(0, gt + 128);
    }
    bool ok = true;
    for (int kh = 0; kh < nkh && ok; ++kh) {
      const int s = kh % DP_NST, vb = kh & 1;
      const bool on = t_on && kh < nk_t;
      if (on) {
        // hand this step's vectors over; the buffer was last read two steps ago (one barrier per step in between)
        if (gt < 64) bars->ga[t][vb][gt] = na;
        bars->gr[t][vb][gt] = nr0;
        if (gt + 128 < 192) bars->gr[t][vb][gt + 128] = nr1;
        named_bar_sync(2 + t, 128);
        if (kh + 1 < nk_t) {
          na = fetch_a(kh + 1); nr0 = fetch_r(kh + 1, gt); nr1 = fetch_r(kh + 1, gt + 128);
        }
      }
      if (!mbar_wait(&bars->empty[s], ((kh / DP_NST) & 1) ^ 1)) {      // the stage's previous products are done
        dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 76);
        ok = false;
        break;
      }
      if (on) {
        uint8_t* rowp = smem + s * C::STAGE + t * DP_PATOM + r * 128;
        // distance of key c from this row = d0 + (63 + r - c)
        const float* ga_ = bars->ga[t][vb];
        const float* gr_ = bars->gr[t][vb] + 63 + r;
        const int lim = i_row - kh * 64;                   // keys c <= lim count
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = cc * 8 + 2 * e;
            const float x0 = ga_[c] + gr_[-c] - zr, x1 = ga_[c + 1] + gr_[-c - 1] - zr;
            float p0, p1;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(x0));
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(x1));
            if (c > lim) p0 = 0.f;
            if (c + 1 > lim) p1 = 0.f;
            w[e] = pack_bf16(p0, p1);
          }
          *reinterpret_cast<uint4*>(rowp + ((cc ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async_smem();
      }
      mbar_arrive(&bars->pgen[s]);
    }
  }
  if (warp >= 2 && warp < 6) {
    // ---------------------------------------------------------------- mask helpers, then epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;            // row of the tile == TMEM lane
    const int etid = tid - 64;
    bool ok = true;
    int n_masked = 0;
    for (int kh = gen ? nkh : max(0, nkh - 4); kh < nkh && ok; ++kh) {
      const bool d0 = diag_of(kh, 0), d1 = diag_of(kh, 1);
      if (!d0 && !d1) continue;
      const int s = kh % DP_NST;
      if (!mbar_wait(&bars->need_mask, n_masked & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 73);
        ok = false;
        break;
      }
      ++n_masked;
      const int t = d0 ? 0 : 1;
      // key c of this step is column 64*(kh - first diagonal step) + c of the tile's own 128 keys
      const int koff = (kh - (4 * mp + 2 * t)) * 64;
      uint8_t* rowp = smem + s * C::STAGE + t * DP_PATOM + r * 128;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        const int c_lo = koff + cc * 8;                        // first key of this 16-byte chunk
        if (c_lo + 7 <= r) continue;                            // all eight at or below the diagonal
        uint4* q = reinterpret_cast<uint4*>(rowp + ((cc ^ (r & 7)) << 4));
        uint4 v = *q;
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (c_lo + 2 * e > r) w[e] &= 0xffff0000u;            // low half = key c_lo + 2e
          if (c_lo + 2 * e + 1 > r) w[e] &= 0x0000ffffu;        // high half = key c_lo + 2e + 1
        }
        *q = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&bars->masked);
    }
    if (ok && !mbar_wait(&bars->acc_full, 0)) {
      dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 74);
      ok = false;
    }
    tc_fence_after();
    // accumulators -> bf16 -> staging (the ring is idle now) -> TMA store; two staging tiles in rotation
    int n_st = 0;
    for (int t = 0; t < 2; ++t) {
      if (t == 1 && !act1) break;
      if (t == 0 && nk0 == 0) continue;                   // this CTA computes tile 1 only
      for (int bi = 0; bi < nb; ++bi, ++n_st) {
        uint8_t* stage = smem + (n_st & 1) * (128 * HD * 2);
        if (etid == 0) tma_store_wait_read1();
        named_bar_sync(1, 128);
        const uint32_t tsrc = tmem + ((uint32_t)(quad * 32) << 16) + (t * C::NB + bi) * HD;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tsrc + c0, o);
          tmem_ld_wait();
          uint8_t* dst = stage + (c0 >> 6) * 16384 + r * 128;
          const int cbase = (c0 & 63) >> 3;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 q;
            q.x = pack_bf16(__uint_as_float(o[c * 8 + 0]), __uint_as_float(o[c * 8 + 1]));
            q.y = pack_bf16(__uint_as_float(o[c * 8 + 2]), __uint_as_float(o[c * 8 + 3]));
            q.z = pack_bf16(__uint_as_float(o[c * 8 + 4]), __uint_as_float(o[c * 8 + 5]));
            q.w = pack_bf16(__uint_as_float(o[c * 8 + 6]), __uint_as_float(o[c * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + (((cbase + c) ^ (r & 7)) << 4)) = q;
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (etid == 0 && ok) {
#pragma unroll
          for (int hh = 0; hh < HD / 64; ++hh) tma_store_4d(&mapO, stage + hh * 16384, hh * 64, row0 + t * 128, h, b0 + bi);
          tma_store_commit();
        }
      }
    }
    if (etid == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}


// ---------------------------------------------------------------------------------------------------------
// Backward of dense-stored heads: dV[b, h, j, :] = sum_{i >= j} P[pidx[h], i, j] dO[b, h, i, :]
// (_pv_bwd_kernel, kernel/frozen_attn.py:91-128).  CTA = two consecutive 128-key tiles of one head for NB batch
// rows; queries advance 64 at a time from the tiles' own rows to the end of the sequence.  The pattern block
// [64 queries x 128 keys] lands by TMA as two 64 x 64 boxes and is read by the tensor core as a transposed
// (MN-major) A operand, dO tiles as MN-major B operands: nothing is transposed in shared memory.
// Same calling rules as dense_pv_cta.
template <int HD>
__device__ __forceinline__ void dense_dv_cta(const CUtensorMap& mapP, const CUtensorMap& mapdO, const CUtensorMap& mapdV,
                                             const DpParams& p, int slot, uint8_t* smem) {
  using C = DpCfg<HD>;
  // CTA -> (head, batch group, key pair); heaviest (first) key pairs first
  const int per_kp = p.H * p.groups;
  const int kp = slot / per_kp;
  const int rem = slot % per_kp;
  const int h = rem / p.groups, grp = rem % p.groups;
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  const bool gen = state == SAF_DECOMP && p.dec_ok;       // pattern blocks generated, not loaded
  if (!gen && !(state == SAF_DENSE && p.dense_ok)) return;
  const int hp = p.pidx ? p.pidx[h] : h;
  const int b0 = grp * C::NB;
  const int nb = min(C::NB, p.B - b0);
  const int key0 = kp * 256;
  const bool act1 = key0 + 128 < p.T;
  const int n_half = (p.T + 63) / 64;
  const int qh0 = 4 * kp;                                  // first 64-query step (tile 0's own rows)
  const int n_steps = n_half - qh0;
  // tile 1 starts two steps later; a tile's first two steps hold its above-diagonal entries
  auto tile_on = [&](int st, int t) { return t == 0 ? true : (act1 && st >= 2); };
  auto diag_of = [&](int st, int t) { return st >= 2 * t && st < 2 * t + 2 && (t == 0 || act1); };

  DpBars* bars = reinterpret_cast<DpBars*>(smem + DP_NST * C::STAGE);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < DP_NST; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < DP_NST; ++s) mbar_init(&bars->pgen[s], 256);
    mbar_init(&bars->need_mask, 1);
    mbar_init(&bars->masked, 128);
    mbar_init(&bars->acc_full, 1);
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
      if (!gen) tma_prefetch_desc(&mapP);
      tma_prefetch_desc(&mapdO);
      for (int st = 0; st < n_steps; ++st) {
        const int s = st % DP_NST, qh = qh0 + st;
        if (!mbar_wait(&bars->empty[s], ((st / DP_NST) & 1) ^ 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 80);
          break;
        }
        uint8_t* sp = smem + s * C::STAGE;
        const bool t1 = tile_on(st, 1);
        mbar_expect_tx(&bars->full[s], (gen ? 0 : (t1 ? 2 : 1) * DP_PATOM) + nb * C::V_BYTES);
        for (int t = 0; t < (gen ? 0 : (t1 ? 2 : 1)); ++t)
#pragma unroll
          for (int a = 0; a < 2; ++a)     // two 64-key atoms of [64 queries x 128 bytes]
            tma_load_3d(sp + t * DP_PATOM + a * 8192, &mapP, &bars->full[s], key0 + 128 * t + 64 * a, qh * 64, hp);
        for (int bi = 0; bi < nb; ++bi)
#pragma unroll
          for (int hh = 0; hh < HD / 64; ++hh)
            tma_load_4d(sp + 2 * DP_PATOM + bi * C::V_BYTES + hh * 8192, &mapdO, &bars->full[s], hh * 64, qh * 64, h, b0 + bi);
      }
    }
  } else if (warp == 1) {
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(128, HD, 1, 1);     // A = P^T and B = dO both MN-major
    const uint32_t sbase = smem_u32(smem);
    int n_masked = 0;
    for (int st = 0; st < n_steps; ++st) {
      const int s = st % DP_NST;
      if (!mbar_wait(&bars->full[s], (st / DP_NST) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 81);
        break;
      }
      if (gen) {
        if (!mbar_wait(&bars->pgen[s], (st / DP_NST) & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 85);
          break;
        }
      } else if (diag_of(st, 0) || diag_of(st, 1)) {
        if (leader) mbar_arrive(&bars->need_mask);
        __syncwarp();
        if (!mbar_wait(&bars->masked, n_masked & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 82);
          break;
        }
        ++n_masked;
      }
      tc_fence_after();
      const uint32_t sp = sbase + s * C::STAGE;
      if (leader) {
        for (int t = 0; t < 2; ++t) {
          if (!tile_on(st, t)) continue;
          const uint32_t pa = sp + t * DP_PATOM;
          const bool first = (st == 2 * t);                   // this tile's first product
          for (int bi = 0; bi < nb; ++bi) {
            const uint32_t da = sp + 2 * DP_PATOM + bi * C::V_BYTES;
            const uint32_t d = tmem + (t * C::NB + bi) * HD;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_ss(d, umma_smem_desc_sw128(pa + ks * 2048, 8192, 1024), umma_smem_desc_sw128(da + ks * 2048, 8192, 1024),
                      idesc, !(first && ks == 0));
          }
        }
        umma_commit(&bars->empty[s]);
      }
      __syncwarp();
    }
    if (leader) umma_commit(&bars->acc_full);
    __syncwarp();
  }
  if (gen && warp >= 2 && warp < 10) {
    // ---------------------------------------------------------------- decomposed head: generate P^T blocks
    // warps 2-5 build tile 0, warps 6-9 tile 1; thread -> (64-key atom a, query row q of the step).
    // alpha of the tile's 128 keys is loaded once; rho over the step's 191 distances and z of the thread's
    // query are fetched one step ahead.
    constexpr float L2E = 1.4426950408889634f;
    const int t = (warp - 2) >> 2;
    const int gt = (tid - 64) & 127;
    const int a = gt >> 6, q = gt & 63;
    const int kt0 = key0 + 128 * t;                       // first key of this tile
    const bool t_on = t == 0 || act1;
    {
      const int key = kt0 + gt;                           // ga[t] viewed as 128 consecutive keys
      (&bars->ga[t][0][0])[gt] = (t_on && key < p.T)
          ? L2E * load_rt(p.alpha, (int64_t)h * p.alpha_s[0] + (int64_t)key * p.alpha_s[1], p.dec_dtype) : 0.f;
    }
    auto fetch_r = [&](int st, int x) -> float {          // rho at distance (64 qh - kt0 - 127) + x
      const int d = (qh0 + st) * 64 - kt0 - 127 + x;
      return (x < 191 && d >= 0 && d < p.T) ? L2E * load_rt(p.rho, (int64_t)h * p.rho_s[0] + (int64_t)d * p.rho_s[1], p.dec_dtype) : 0.f;
    };
    auto fetch_z = [&](int st) -> float {                 // +inf: query rows past T give exact zeros
      const int qi = (qh0 + st) * 64 + q;
      return (qi < p.T) ? L2E * load_rt(p.z, (int64_t)h * p.z_s[0] + (int64_t)qi * p.z_s[1], p.dec_dtype) : INFINITY;
    };
    const int st_lo = 2 * t;                              // first step of this tile
    float nr0 = 0.f, nr1 = 0.f, nz = INFINITY;
    if (t_on && st_lo < n_steps) {
      nr0 = fetch_r(st_lo, gt); nr1 = fetch_r(st_lo, gt + 128); nz = fetch_z(st_lo);
    }
    bool ok = true;
    for (int st = 0; st < n_steps && ok; ++st) {
      const int s = st % DP_NST, vb = st & 1;
      const bool on = t_on && st >= st_lo;
      float zq = INFINITY;
      if (on) {
        bars->gr[t][vb][gt] = nr0;
        if (gt + 128 < 192) bars->gr[t][vb][gt + 128] = nr1;
        zq = nz;
        named_bar_sync(2 + t, 128);                        // also orders the one-time alpha stores
        if (st + 1 < n_steps) {
          nr0 = fetch_r(st + 1, gt); nr1 = fetch_r(st + 1, gt + 128); nz = fetch_z(st + 1);
        }
      }
      if (!mbar_wait(&bars->empty[s], ((st / DP_NST) & 1) ^ 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 86);
        ok = false;
        break;
      }
      if (on) {
        uint8_t* rowp = smem + s * C::STAGE + t * DP_PATOM + a * 8192 + q * 128;
        const float* ga_ = &bars->ga[t][0][0] + a * 64;
        // distance of key (64 a + c) from this query = dlo + (127 + q - 64 a - c)
        const float* gr_ = bars->gr[t][vb] + 127 + q - 64 * a;
        const int lim = (qh0 + st) * 64 + q - kt0 - 64 * a;   // keys c <= lim count
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = cc * 8 + 2 * e;
            const float x0 = ga_[c] + gr_[-c] - zq, x1 = ga_[c + 1] + gr_[-c - 1] - zq;
            float p0, p1;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(x0));
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(x1));
            if (c > lim) p0 = 0.f;
            if (c + 1 > lim) p1 = 0.f;
            w[e] = pack_bf16(p0, p1);
          }
          *reinterpret_cast<uint4*>(rowp + ((cc ^ (q & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async_smem();
      }
      mbar_arrive(&bars->pgen[s]);
    }
  }
  if (warp >= 2 && warp < 6) {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;            // key row of the tile == TMEM lane
    const int etid = tid - 64;
    bool ok = true;
    int n_masked = 0;
    for (int st = 0; st < (gen ? 0 : min(n_steps, 4)) && ok; ++st) {
      const bool d0 = diag_of(st, 0), d1 = diag_of(st, 1);
      if (!d0 && !d1) continue;
      const int s = st % DP_NST;
      if (!mbar_wait(&bars->need_mask, n_masked & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 83);
        ok = false;
        break;
      }
      ++n_masked;
      const int t = d0 ? 0 : 1;
      // thread -> (64-key atom a, query row q of the step); query and key both counted from the tile's first row
      const int a = etid >> 6, q = etid & 63;
      const int q_rel = (st - 2 * t) * 64 + q;
      uint8_t* rowp = smem + s * C::STAGE + t * DP_PATOM + a * 8192 + q * 128;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        const int k_lo = a * 64 + cc * 8;                      // first key of this 16-byte chunk
        if (k_lo + 7 <= q_rel) continue;                       // all eight keys at or before the query
        uint4* w4 = reinterpret_cast<uint4*>(rowp + ((cc ^ (q & 7)) << 4));
        uint4 v = *w4;
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (k_lo + 2 * e > q_rel) w[e] &= 0xffff0000u;
          if (k_lo + 2 * e + 1 > q_rel) w[e] &= 0x0000ffffu;
        }
        *w4 = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&bars->masked);
    }
    if (ok && !mbar_wait(&bars->acc_full, 0)) {
      dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 84);
      ok = false;
    }
    tc_fence_after();
    int n_st = 0;
    for (int t = 0; t < 2; ++t) {
      if (t == 1 && (!act1 || n_steps <= 2)) break;           // tile 1 never accumulated anything
      for (int bi = 0; bi < nb; ++bi, ++n_st) {
        uint8_t* stage = smem + (n_st & 1) * (128 * HD * 2);
        if (etid == 0) tma_store_wait_read1();
        named_bar_sync(1, 128);
        const uint32_t tsrc = tmem + ((uint32_t)(quad * 32) << 16) + (t * C::NB + bi) * HD;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tsrc + c0, o);
          tmem_ld_wait();
          uint8_t* dst = stage + (c0 >> 6) * 16384 + r * 128;
          const int cbase = (c0 & 63) >> 3;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 qv;
            qv.x = pack_bf16(__uint_as_float(o[c * 8 + 0]), __uint_as_float(o[c * 8 + 1]));
            qv.y = pack_bf16(__uint_as_float(o[c * 8 + 2]), __uint_as_float(o[c * 8 + 3]));
            qv.z = pack_bf16(__uint_as_float(o[c * 8 + 4]), __uint_as_float(o[c * 8 + 5]));
            qv.w = pack_bf16(__uint_as_float(o[c * 8 + 6]), __uint_as_float(o[c * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + (((cbase + c) ^ (r & 7)) << 4)) = qv;
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (etid == 0 && ok) {
#pragma unroll
          for (int hh = 0; hh < HD / 64; ++hh) tma_store_4d(&mapdV, stage + hh * 16384, hh * 64, key0 + t * 128, h, b0 + bi);
          tma_store_commit();
        }
      }
    }
    if (etid == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace saf
