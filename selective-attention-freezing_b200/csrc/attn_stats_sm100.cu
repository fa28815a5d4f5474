// Attention statistics for the freeze controller without the (B, H, T, T) capture.
//
// The reference measures heads by running the eager path with capture on and reducing the retained
// softmax(QK^T) tensor: batch mean per cell, centred sum of squares reduced per head, and sum p log p per head
// (nanogpt/dynamic_freeze.py:96-127 _centered_batch_reduced_moments, :130-143 _merge_reduced_moments,
// :146-173 _negative_entropy_sum, used by _measure :629-745).  Here a CTA takes one 128 x 128 cell tile of one head
// at a time and walks the batch: S_b = Q_b K_b^T on tcgen05 into TMEM, P_b = exp2(S_b scale - lse_b) with the row
// log-sum-exp of the flash forward, per-cell Welford mean (staging tile) / M2 (registers), then the tile of the running mean is
// Chan-merged in place and the per-head scalars are reduced to one double atomic per CTA.
//
//   warps 0-15: four warpgroups x 32 key columns, thread = query row (TMEM lane)
//   warp 16: TMA producer ([Q_b tile | K_b tile] ring), warp 17: MMA issuer
// Every wait is bounded; on expiry the kernel records a code in *status and falls through.
//
// LOGITS: the same walk over the raw scores q k^T * sm_scale of the whole square (nothing masked, tiles above the
// diagonal included), for the priors that sample logits (`_last_logits`, nanogpt/model.py:828-831, reduced at
// nanogpt/dynamic_freeze.py:721-737 with _centered_batch_moments / _merge_moments, :62-93): running mean per cell and,
// when asked for, the centred squares per cell; no per-head scalars.
#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {
namespace {

constexpr int AS_COMPUTE = 512;
constexpr int AS_THREADS = AS_COMPUTE + 64;
constexpr float AS_LN2 = 0.6931471805599453f;

struct AsParams {
  int B, U, T, n_tiles;
  float scale_log2;
  float scale;                 // LOGITS: sm_scale itself
  float* cell_m2;              // LOGITS: (U, T, T) or null
  const float* lse;
  int64_t lse_s[3];
  float* mean;                 // (U, T, T)
  long long count_prev;
  double* head_m2;
  double* neg_entropy;
  int* status;
};

struct AsShared {
  uint64_t full[3], empty[3], s_full[2], s_empty[2];
  uint32_t tmem_base;
  double red[2][AS_COMPUTE / 32];
};

template <int HD>
struct AsCfg {
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int NS = (HD == 64) ? 3 : 2;
  static constexpr int STAGE_LD = 132;                       // floats per staged row: 128 + 4 keeps 16-byte row writes conflict-free
  static constexpr int STAGE_BYTES = 128 * STAGE_LD * 4;     // the tile's batch mean on its way to coalesced global rows
  static constexpr int SMEM_BYTES = 1024 + NS * 2 * TILE_BYTES + STAGE_BYTES + (int)sizeof(AsShared) + 64;
  static constexpr int TMEM_COLS = 256;
};

__device__ __forceinline__ float as_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int HD>
__device__ __forceinline__ void as_load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row, int head, int b) {
#pragma unroll
  for (int hh = 0; hh < HD / 64; ++hh) tma_load_4d(dst + hh * 16384, m, bar, hh * 64, row, head, b);
}

// Persistent: CTA c owns tiles c, c + gridDim.x, ... of the (head, query tile, key tile) list, so the producer's loads
// for the next tile run under the epilogue of the current one and the set-up is paid once.  `g` counts batch steps
// over all tiles of the CTA; ring stages and TMEM buffers follow it.
struct AsTile {
  int u, it, jt;
};
__device__ __forceinline__ AsTile as_decode(const AsParams& p, int t) {
  const int nn = p.n_tiles * p.n_tiles;
  AsTile x;
  x.u = t / nn;
  const int rem = t - x.u * nn;
  x.it = rem / p.n_tiles;
  x.jt = rem - x.it * p.n_tiles;
  return x;
}

template <int HD, bool LOGITS>
__global__ void __launch_bounds__(AS_THREADS, 1)
attn_stats_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ AsParams p) {
  using C = AsCfg<HD>;
  const int total_tiles = p.U * p.n_tiles * p.n_tiles;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = smem;                                // stage s: [Q_b tile | K_b tile]
  float* stage = reinterpret_cast<float*>(ring + C::NS * 2 * C::TILE_BYTES);
  AsShared* sh = reinterpret_cast<AsShared*>(ring + C::NS * 2 * C::TILE_BYTES + C::STAGE_BYTES);
  constexpr int W_TMA = AS_COMPUTE / 32, W_MMA = W_TMA + 1;

  if (tid == 0) {
    for (int s = 0; s < C::NS; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);                      // the MMA's commit
    }
    for (int k = 0; k < 2; ++k) {
      mbar_init(&sh->s_full[k], 1);
      mbar_init(&sh->s_empty[k], AS_COMPUTE / 32);      // one lane of every compute warp
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
    if (elect_one()) {
      tma_prefetch_desc(&mapQ);
      tma_prefetch_desc(&mapK);
      int g = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const AsTile x = as_decode(p, t);
        if (!LOGITS && x.jt > x.it) continue;
        for (int b = 0; b < p.B; ++b, ++g) {
          const int s = g % C::NS;
          if (!mbar_wait(&sh->empty[s], ((g / C::NS) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 80);
            ok = false;
            break;
          }
          uint8_t* dst = ring + s * 2 * C::TILE_BYTES;
          mbar_expect_tx(&sh->full[s], 2 * C::TILE_BYTES);
          as_load_tile<HD>(dst, &mapQ, &sh->full[s], x.it * 128, x.u, b);
          as_load_tile<HD>(dst + C::TILE_BYTES, &mapK, &sh->full[s], x.jt * 128, x.u, b);
        }
      }
    }
  } else if (warp == W_MMA) {
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(128, 128, 0, 0);
    const uint32_t aR = smem_u32(ring);
    int g = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const AsTile x = as_decode(p, t);
      if (!LOGITS && x.jt > x.it) continue;
      for (int b = 0; b < p.B; ++b, ++g) {
        const int s = g % C::NS, k = g & 1;
        if (!mbar_wait(&sh->full[s], (g / C::NS) & 1) || !mbar_wait(&sh->s_empty[k], ((g >> 1) & 1) ^ 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 81);
          ok = false;
          break;
        }
        tc_fence_after();
        if (leader) {
          const uint32_t aQ = aR + s * 2 * C::TILE_BYTES, aK = aQ + C::TILE_BYTES;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
            umma_ss(tmem + k * 128, umma_smem_desc_sw128(aQ + off, 16, 1024), umma_smem_desc_sw128(aK + off, 16, 1024),
                    idesc, ks > 0);
          }
          umma_commit(&sh->s_full[k]);
          umma_commit(&sh->empty[s]);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    const int quarter = warp >> 2;
    const int r = tid & 127;                        // query row of the tile
    const int cb = quarter * 32;                    // first key column of this group
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const float sc = p.scale_log2;
    const double total = (double)p.count_prev + (double)p.B;
    const float w = (float)((double)p.B / total);
    const bool vec = (p.T & 3) == 0;
    // per-head scalars of this thread, handed to the head's two doubles when the CTA moves to another head
    double m2sum = 0.0, esum = 0.0;
    int cur_u = -1;
    auto flush_head = [&]() {
#pragma unroll
      for (int off = 16; off; off >>= 1) {
        m2sum += __shfl_xor_sync(0xffffffffu, m2sum, off);
        esum += __shfl_xor_sync(0xffffffffu, esum, off);
      }
      named_bar_sync(1, AS_COMPUTE);                // the previous flush has been read
      if (lane == 0) {
        sh->red[0][warp] = m2sum;
        sh->red[1][warp] = esum;
      }
      named_bar_sync(1, AS_COMPUTE);
      if (tid < 2) {
        double tot = 0.0;
        for (int wq = 0; wq < AS_COMPUTE / 32; ++wq) tot += sh->red[tid][wq];
        atomicAdd(tid == 0 ? &p.head_m2[cur_u] : &p.neg_entropy[cur_u], tot);
      }
      m2sum = esum = 0.0;
    };
    int g = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const AsTile x = as_decode(p, t);
      float* mean_u = p.mean + (int64_t)x.u * p.T * p.T;
      if (!LOGITS && x.jt > x.it) {
        // above the diagonal every probability is zero: the first batch writes the zeros, later ones leave them
        if (p.count_prev == 0) {
          for (int e = tid; e < 128 * 128; e += AS_COMPUTE) {
            const int gi = x.it * 128 + (e >> 7), gj = x.jt * 128 + (e & 127);
            if (gi < p.T && gj < p.T) mean_u[(int64_t)gi * p.T + gj] = 0.f;
          }
        }
        continue;
      }
      if (!LOGITS && x.u != cur_u) {
        if (cur_u >= 0) flush_head();
        cur_u = x.u;
      }
      const int gi = x.it * 128 + r;
      const bool row_ok = gi < p.T;
      const int gj0 = x.jt * 128 + cb;
      const bool diag = (x.it == x.jt);
      const float* lse_u = LOGITS ? nullptr : p.lse + (int64_t)x.u * p.lse_s[1] + (int64_t)gi * p.lse_s[2];
      // The running batch mean of the tile lives in the padded staging tile (each thread owns 32 cells of its row
      // until the tile is finished), the centred squares in registers: that leaves room to fetch a sample's 32
      // scores in one TMEM load and to hand the buffer back before the arithmetic.
      float m2[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) m2[c] = 0.f;
      float* srow = stage + r * C::STAGE_LD + cb;
      float ent = 0.f;                                // sum p log2 p of this thread's cells
      float nl = LOGITS ? 0.f : (row_ok ? lse_u[0] : INFINITY);        // +inf: rows past T hold zeros
      named_bar_sync(2, AS_COMPUTE);                  // the previous tile's rows have left the staging tile
      for (int b = 0; b < p.B; ++b, ++g) {
        const int k = g & 1;
        const float L = nl;
        if (!LOGITS && b + 1 < p.B && row_ok) nl = lse_u[(int64_t)(b + 1) * p.lse_s[0]];
        if (!mbar_wait(&sh->s_full[k], (g >> 1) & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 82);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t d[32];
        tmem_ld32(tmem + lane_base + k * 128 + cb, d);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->s_empty[k]);
        const float inv = 1.f / (float)(b + 1);
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          float4 mv = make_float4(0.f, 0.f, 0.f, 0.f);
          if (b > 0) mv = *reinterpret_cast<const float4*>(srow + c4 * 4);
          float mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = c4 * 4 + e;
            float pe;
            if constexpr (LOGITS) {
              pe = __uint_as_float(d[c]) * p.scale;                     // the raw score
            } else {
              float xl = fmaf(__uint_as_float(d[c]), sc, -L);           // log2 of the probability
              if (diag && gj0 + c > gi) xl = -INFINITY;                 // causal mask inside the diagonal tile
              pe = as_ex2(xl);
              ent = fmaf(pe, fmaxf(xl, -200.f), ent);                   // p = 0 there, so the clamp only avoids 0 * inf
            }
            // Welford update of the cell's mean and centred sum of squares over the batch
            const float dlt = pe - mm[e];
            mm[e] = fmaf(dlt, inv, mm[e]);
            m2[c] = fmaf(dlt, pe - mm[e], m2[c]);
          }
          *reinterpret_cast<float4*>(srow + c4 * 4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
        }
      }
      if (!ok) break;
      // ---- merge the tile into the running mean (Chan).  A thread holds 32 cells of one row; written from there the
      // rows of a warp would be 32 separate 16-byte pieces per instruction, so every warp now takes whole 512-byte
      // rows out of the staging tile.
      if constexpr (!LOGITS) {
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4)
          m2sum += (double)(m2[c4 * 4] + m2[c4 * 4 + 1]) + (double)(m2[c4 * 4 + 2] + m2[c4 * 4 + 3]);
      }
      // the old rows are requested before the barrier (the accumulators are dead by now), so their latency and the
      // wait for the slowest warp overlap
      double corr = 0.0;
      const int gjl = x.jt * 128 + lane * 4;
      float4 o[8], pv[8];
      float dl2[LOGITS ? 8 : 1][4];                   // LOGITS: (batch mean - running mean)^2 of this thread's cells
      if constexpr (LOGITS) {
#pragma unroll
        for (int rr = 0; rr < 8; ++rr)
#pragma unroll
          for (int e = 0; e < 4; ++e) dl2[rr][e] = 0.f;
      }
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) {
        pv[rr] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int grow = x.it * 128 + warp * 8 + rr;
        if (!LOGITS && vec && p.count_prev > 0 && grow < p.T && gjl < p.T)   // (LOGITS keeps more state: loaded where used)
          pv[rr] = *reinterpret_cast<const float4*>(mean_u + (int64_t)grow * p.T + gjl);
      }
      named_bar_sync(2, AS_COMPUTE);
#pragma unroll
      for (int rr = 0; rr < 8; ++rr)
        o[rr] = *reinterpret_cast<const float4*>(stage + (warp * 8 + rr) * C::STAGE_LD + lane * 4);
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) {
        const int grow = x.it * 128 + warp * 8 + rr;
        if (grow >= p.T || gjl >= p.T) continue;
        float* dst = mean_u + (int64_t)grow * p.T + gjl;
        float ov[4] = {o[rr].x, o[rr].y, o[rr].z, o[rr].w};
        if (vec) {
          if (p.count_prev > 0) {
            if constexpr (LOGITS) pv[rr] = *reinterpret_cast<const float4*>(dst);
            const float pr[4] = {pv[rr].x, pv[rr].y, pv[rr].z, pv[rr].w};
            float cs = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float dlt = ov[e] - pr[e];
              cs = fmaf(dlt, dlt, cs);
              if constexpr (LOGITS) dl2[rr][e] = dlt * dlt;
              ov[e] = fmaf(dlt, w, pr[e]);
            }
            corr += (double)cs;
          }
          *reinterpret_cast<float4*>(dst) = make_float4(ov[0], ov[1], ov[2], ov[3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (gjl + e >= p.T) continue;
            float v = ov[e];
            if (p.count_prev > 0) {
              const float pr = dst[e];
              const float dlt = v - pr;
              corr += (double)(dlt * dlt);
              if constexpr (LOGITS) dl2[rr][e] = dlt * dlt;
              v = fmaf(dlt, w, pr);
            }
            dst[e] = v;
          }
        }
      }
      if constexpr (LOGITS) {
        if (p.cell_m2) {
          // the centred squares take the same way out: registers -> staging tile -> whole rows, merged per cell
          const float cw = (float)((double)p.count_prev * (double)p.B / total);
          float* m2_u = p.cell_m2 + (int64_t)x.u * p.T * p.T;
          named_bar_sync(2, AS_COMPUTE);              // every warp has taken its mean rows out of the staging tile
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)
            *reinterpret_cast<float4*>(srow + c4 * 4) = make_float4(m2[c4 * 4], m2[c4 * 4 + 1], m2[c4 * 4 + 2], m2[c4 * 4 + 3]);
          named_bar_sync(2, AS_COMPUTE);
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int grow = x.it * 128 + warp * 8 + rr;
            if (grow >= p.T || gjl >= p.T) continue;
            const float4 b2 = *reinterpret_cast<const float4*>(stage + (warp * 8 + rr) * C::STAGE_LD + lane * 4);
            float* dst = m2_u + (int64_t)grow * p.T + gjl;
            float ov[4] = {b2.x, b2.y, b2.z, b2.w};
            if (vec) {
              if (p.count_prev > 0) {
                const float4 old = *reinterpret_cast<const float4*>(dst);
                ov[0] += fmaf(dl2[rr][0], cw, old.x);
                ov[1] += fmaf(dl2[rr][1], cw, old.y);
                ov[2] += fmaf(dl2[rr][2], cw, old.z);
                ov[3] += fmaf(dl2[rr][3], cw, old.w);
              }
              *reinterpret_cast<float4*>(dst) = make_float4(ov[0], ov[1], ov[2], ov[3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (gjl + e >= p.T) continue;
                dst[e] = p.count_prev > 0 ? ov[e] + fmaf(dl2[rr][e], cw, dst[e]) : ov[e];
              }
            }
          }
        }
      } else {
        m2sum += corr * ((double)p.count_prev * (double)p.B / total);
        esum += (double)ent * (double)AS_LN2;          // natural log, as the reference's xlogy
      }
    }
    if (!LOGITS && ok && cur_u >= 0) flush_head();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == W_MMA) tmem_dealloc(tmem, C::TMEM_COLS);
}

template <int HD, bool LOGITS>
int as_launch(const SafAttnStatsArgs& a, cudaStream_t st) {
  CUtensorMap mq, mk;
  int rc;
  if ((rc = make_row_tile_map_bf16(&mq, a.q, a.B, a.U, a.T, HD))) return rc;
  if ((rc = make_row_tile_map_bf16(&mk, a.k, a.B, a.U, a.T, HD))) return rc;
  AsParams p;
  p.B = a.B; p.U = a.U; p.T = a.T;
  p.n_tiles = (a.T + 127) / 128;
  p.scale_log2 = a.sm_scale * 1.4426950408889634f;
  p.scale = a.sm_scale;
  p.cell_m2 = LOGITS ? a.cell_m2 : nullptr;
  p.lse = LOGITS ? nullptr : reinterpret_cast<const float*>(a.lse.ptr);
  for (int i = 0; i < 3; ++i) p.lse_s[i] = LOGITS ? 0 : a.lse.stride[i];
  p.mean = a.mean;
  p.count_prev = a.count_prev;
  p.head_m2 = a.head_m2;
  p.neg_entropy = a.neg_entropy;
  p.status = a.status;
  static PerDeviceOnce smem_once;
  if (int rc2 = ensure_dyn_smem(attn_stats_kernel<HD, LOGITS>, AsCfg<HD>::SMEM_BYTES, smem_once)) return rc2;
  const int64_t tiles = (int64_t)a.U * p.n_tiles * p.n_tiles;
  if (tiles > 0x7fffffff) return fail(SAF_ERR_LIMIT, "attention statistics: too many tiles");
  const int sm_count = device_sm_count();
  const int grid = (int)(tiles < sm_count ? tiles : sm_count);      // one persistent CTA per SM
  attn_stats_kernel<HD, LOGITS><<<(unsigned)grid, AS_THREADS, AsCfg<HD>::SMEM_BYTES, st>>>(mq, mk, p);
  count_launch();
  return check_launch("attn_stats_kernel");
}

}  // namespace

int launch_attn_stats_sm100(const SafAttnStatsArgs& a, cudaStream_t st) {
  if (a.dtype != SAF_BF16 || (a.HD != 64 && a.HD != 128)) return fail(SAF_ERR_UNSUPPORTED, "attention statistics: bf16 with head_dim 64 or 128 only");
  if (!tma_rows_ok(a.q) || !tma_rows_ok(a.k))
    return fail(SAF_ERR_UNSUPPORTED, "attention statistics: q, k need 16-byte aligned rows and unit last stride");
  if ((uintptr_t)a.mean & 15) return fail(SAF_ERR_INVALID, "attention statistics: mean must be 16-byte aligned");
  if (!saf_device_supported()) return fail(SAF_ERR_UNSUPPORTED, "attention statistics need an sm_100 device");
  if ((uintptr_t)a.cell_m2 & 15) return fail(SAF_ERR_INVALID, "attention statistics: cell_m2 must be 16-byte aligned");
  if (a.quantity == SAF_STATS_LOGITS) return a.HD == 64 ? as_launch<64, true>(a, st) : as_launch<128, true>(a, st);
  return a.HD == 64 ? as_launch<64, false>(a, st) : as_launch<128, false>(a, st);
}

}  // namespace saf
