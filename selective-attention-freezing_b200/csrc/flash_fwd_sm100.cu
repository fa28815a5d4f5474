// Mixed-attention forward on tcgen05 / TMEM, fed by TMA: live heads as causal flash attention,
// structured (sink + decay) frozen heads as a co-scheduled scan, all in one launch.
//
// Replaces the reference's fused forward (_fwd_kernel / _acc_flash, kernel/fused_attn.py:182-289:
// 64x64 Triton tiles, pointer loads, 4 warps, no persistence).  A live CTA owns TWO consecutive
// 128-row query tiles of one (batch, head) and walks the causal range of 128-key tiles once for both:
//
//   warps 0-3   softmax of query tile 0 (one thread per row: TMEM lane == row, no shuffles)
//   warps 4-7   softmax of query tile 1
//   warp  8     TMA producer: Q tiles once, then K_j and V_j tiles through two rings of stages
//   warp  9     score MMA issuer:  S_t(j) = Q_t K_j^T   (SS, 128x128xHD)  -> TMEM score buffer
//   warp  10    output MMA issuer: O_t += P_t(j) V_j     (TS: P read from TMEM, V MN-major in smem)
//   warp  11    completes the third warpgroup (register reallocation works per warpgroup)
//
// TMEM (512 columns): score buffers of 128 columns each, then O0, O1 (HD columns each).  P (bf16)
// overwrites the first 64 columns of its score buffer, so scores never touch shared or global memory.
// head_dim 64 leaves room for THREE score buffers shared by the two query tiles in rotation (the k-th
// score tile, k = 2j + t, lives in buffer k mod 3), so S_t(j+1) is computed while P_t(j) is still being
// made and a softmax warpgroup finds its next scores ready when it finishes a tile; head_dim 128 fills
// TMEM with two score buffers, one per tile.  Two issuing warps split the per-tile bookkeeping
// (barrier waits, descriptor updates, commits), which otherwise costs more than the MMAs themselves;
// the whole warp walks the schedule so addresses stay in uniform registers and one elected lane issues.
// The softmax warps take registers from the control warpgroup (setmaxnreg) so a full 128-column score
// row stays in registers; their arithmetic uses the packed f32x2 FMA/ADD and the 3-input max of sm_100.
// The running output is rescaled lazily: only when a row maximum grows by more than 2^8 (exact, because
// the final normaliser l carries the same reference maximum).
//
// Grid order: first one slot per (batch, head) that runs the O(T) scan if that head is frozen on a
// structured pattern (first 256 threads; other heads' slots exit) -- they start at time zero and
// finish long before the live tiles, so frozen heads cost no launch and almost no time.  Then the
// live tiles, in groups of 8 (batch, head) pairs so the CTAs in flight share K/V in L2, heaviest
// row tiles first inside a group.  CTAs of dense / decomposed heads exit (pattern kernels take them).
#include "saf_internal.h"
#include "dense_pv_body.cuh"
#include "scan_body.cuh"
#include "scan_mma_body.cuh"
#include "sm100_prims.cuh"
#include <stdlib.h>
#include <string.h>

#include <algorithm>

namespace saf {
namespace {

// a build-free off switch for measurements: NAME=0 in the environment
bool getenv_off(const char* name) {
  const char* v = getenv(name);
  return v && v[0] == '0' && v[1] == 0;
}

constexpr int FM = 128;             // rows per query tile
constexpr int FN = 128;             // keys per step
constexpr int FLASH_THREADS = 384;
#ifndef SAF_HEAD_GROUP
#define SAF_HEAD_GROUP 8
#endif
constexpr int HEAD_GROUP = SAF_HEAD_GROUP;   // (batch, head) pairs whose tiles are in flight together (K/V shared in L2)
constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;
#ifndef SAF_POLY_EXP_PER_16
#define SAF_POLY_EXP_PER_16 8       // of every 16 exponentials, this many run on the FMA pipe
#endif

#ifdef SAF_FWD_TRACE
// timing probe (only in specially built libraries): clock64 stamps of one CTA's pipeline events
__device__ long long g_ftrace[8][64];   // [event][key step]
#define FTRACE(evt, step) do { if (trace_on && (step) < 64) g_ftrace[evt][step] = clock64(); } while (0)
#else
#define FTRACE(evt, step) do { } while (0)
#endif

template <int HD>
struct Cfg {
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int KSTAGE = (HD == 64) ? 4 : 2;    // K ring and V ring, powers of two
  static constexpr int Q_BYTES = 2 * TILE_BYTES;
  static constexpr int RING_BYTES = 2 * KSTAGE * TILE_BYTES;
  static constexpr int SMEM_FLASH = 1024 + Q_BYTES + RING_BYTES + 4096;
  // the dense-pattern role of the same launch needs its own ring
  static constexpr int SMEM_BYTES = SMEM_FLASH > DpCfg<HD>::SMEM_BYTES ? SMEM_FLASH : DpCfg<HD>::SMEM_BYTES;
  // persistent kernel: Q, rings, barriers; at head_dim 64 two 16 KB output staging buffers as well (at head_dim
  // 128 Q and the rings leave no room: the epilogue stages a tile in its own Q buffer)
  static constexpr bool STAGE_IN_Q = (HD == 128);
  static constexpr int O_STAGING = STAGE_IN_Q ? 0 : 2 * 128 * 128;
  static constexpr int SMEM_PERSIST_OWN = 1024 + Q_BYTES + RING_BYTES + O_STAGING + 1024;
  static constexpr int SMEM_PERSIST = SMEM_PERSIST_OWN > DpCfg<HD>::SMEM_BYTES ? SMEM_PERSIST_OWN : DpCfg<HD>::SMEM_BYTES;
  static_assert(SMEM_PERSIST_OWN + 4096 <= 232448, "persistent kernel exceeds the 227 KB of shared memory per CTA");
  static constexpr int TMEM_COLS = 512;
  static constexpr int NBUF = (HD == 64) ? 3 : 2;      // score buffers
  static constexpr int O_COL = NBUF * 128;
};

// ring depth of the tensor-core scan when it runs in a scan slot of these launches: what their shared memory holds
constexpr int SCAN_ROLE_STAGES = 8;
static_assert(ms_smem_bytes(SCAN_ROLE_STAGES) <= Cfg<64>::SMEM_BYTES && ms_smem_bytes(SCAN_ROLE_STAGES) <= Cfg<64>::SMEM_PERSIST &&
                  ms_smem_bytes(SCAN_ROLE_STAGES) <= Cfg<128>::SMEM_BYTES && ms_smem_bytes(SCAN_ROLE_STAGES) <= Cfg<128>::SMEM_PERSIST,
              "the scan role must fit the launches' dynamic shared memory");

struct FlashParams {
  int B, H, T, HKV, force_state, n_pairs;
  float scale_log2;
  const int32_t* frozen;
  const int32_t* hidx;
  const int32_t* kvidx;
  float* lse;
  int64_t lse_s[3];
  int* status;
  int has_scan;
  ScanArgs scan;
  int dense_slots;           // CTAs of the TMA-staged dense-pattern role, right after the scan slots
  DpParams dense;
  // frozen heads whose pattern is produced by the softmax warps (P -> TMEM -> P V on the tensor core)
  const void* patt;          // dense (P, S, S), state 1
  int64_t patt_s[3];
  int patt_dtype;
  const int32_t* pidx;
  const void *alpha, *rho, *z;   // decomposed (H, S), state 2
  int64_t alpha_s[2], rho_s[2], z_s[2];
  int dec_dtype;
  // persistent live-tile role: dynamic tile queue over the live heads only
  int* sched;                // [0] next item, [1] CTAs that have seen the end; zero on entry, left zero
  int n_items, U, lead;      // live items B * U * n_pairs; live heads; CTAs in front of the persistent ones
  uint8_t live_head[64];     // head of live slot u
};

struct FlashBars {
  uint64_t q_full;
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[3];     // score buffer written by the score MMAs
  uint64_t p_full[3];     // P written by the softmax warpgroup (128 arrivals)
  uint64_t buf_free[3];   // PV product that read P from this buffer has finished
  uint32_t tmem_base;
  float dec_alpha[2][128];   // decomposed heads: alpha of the current key tile, per query tile
  float dec_rho[2][256];     // and the rho values its distances can take
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x on the FMA/ALU pipes for x in [-126, 126]: round to nearest integer with the magic-number
// add, cubic minimax on the fraction in [-0.5, 0.5], exponent added as an integer shift.
// Relative error ~1e-4, far below the bf16 rounding the result goes through.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  const float magic = 12582912.f;  // 1.5 * 2^23
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rn(x, make_float2(magic, magic));
  const float2 n = __fadd2_rn(t, make_float2(-magic, -magic));
  const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
  float2 p = __ffma2_rn(f, make_float2(0.0555054f, 0.0555054f), make_float2(0.2402265f, 0.2402265f));
  p = __ffma2_rn(p, f, make_float2(0.6931472f, 0.6931472f));
  p = __ffma2_rn(p, f, make_float2(1.f, 1.f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  return r;
}

template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int row, int head, int b) {
#pragma unroll
  for (int hh = 0; hh < HD / 64; ++hh) tma_load_4d(dst + hh * 16384, m, bar, hh * 64, row, head, b);
}

template <int HD>
__global__ void __launch_bounds__(FLASH_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                 const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO,
                 const __grid_constant__ CUtensorMap mapP, const __grid_constant__ CUtensorMap mapV64,
                 const __grid_constant__ FlashParams p) {
  using C = Cfg<HD>;
  const int bh_count = p.B * p.H;
  // ---- scan slots ---------------------------------------------------------------------------
  if ((int)blockIdx.x < bh_count) {
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
    if (state == SAF_SINK_DECAY && p.has_scan) {
      {
        // the whole sequence as 128-row Toeplitz products on the tensor core, one 64-column slice after the other
        // (about a third of the time of the register scan, so the SM joins the live tiles that much earlier)
        if (p.T >= 4 * MB && p.scan.HD == HD) {
          extern __shared__ uint8_t scan_smem_raw[];
          MsParams mp;
          mp.a = p.scan;
          mp.chunk = (p.T + MB - 1) / MB * MB;
          mp.use_stash = 0;
          mp.status = p.status;
          sink_decay_apply_mma_cta<SCAN_ROLE_STAGES>(mapV, mapO, mp, b, h, 0, 0, HD / 64, scan_smem_raw);
          return;
        }
      }
      if (threadIdx.x < SCAN_NT)
        for (int col0 = 0; col0 < HD; col0 += SCAN_COLS) sink_decay_scan_cta<__nv_bfloat16, false>(p.scan, b, h, col0);
    }
    return;
  }
  // ---- dense-stored frozen heads: TMA-staged lower-triangular GEMM, pattern tiles shared by batch rows ---
  if ((int)blockIdx.x < bh_count + p.dense_slots) {
    extern __shared__ uint8_t dense_smem_raw[];
    uint8_t* dsm = (uint8_t*)(((uintptr_t)dense_smem_raw + 1023) & ~(uintptr_t)1023);
    dense_pv_cta<HD>(mapP, mapV64, mapO, p.dense, (int)blockIdx.x - bh_count, dsm);
    return;
  }
  // ---- live tiles: head groups, heaviest row-tile pairs first inside a group ------------------
  const int li = blockIdx.x - bh_count - p.dense_slots;
  const int per_group = HEAD_GROUP * p.n_pairs;
  const int grp = li / per_group;
  const int gsize = min(HEAD_GROUP, bh_count - grp * HEAD_GROUP);
  const int rem = li - grp * per_group;
  if (rem >= gsize * p.n_pairs) return;
  const int mp = p.n_pairs - 1 - rem / gsize;
  const int bh = grp * HEAD_GROUP + rem % gsize;
  const int b = bh / p.H, h = bh % p.H;
  const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
  // live heads: flash attention.  Dense / decomposed frozen heads: same pipeline without Q K^T -- the
  // softmax warps write the pattern tile P into TMEM and the tensor core does P V.
  const bool live = state == SAF_LIVE;
  if (!live && !((state == SAF_DENSE && p.patt) || (state == SAF_DECOMP && p.alpha))) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                       // 2 tiles
  uint8_t* sK = smem + C::Q_BYTES;                          // KSTAGE key tiles
  uint8_t* sV = sK + C::KSTAGE * C::TILE_BYTES;             // KSTAGE value tiles
  FlashBars* bars = reinterpret_cast<FlashBars*>(sK + C::RING_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int row0 = mp * 2 * FM;
  const bool act1 = row0 + FM < p.T;
  const int nkv0 = 2 * mp + 1;
  const int nkv1 = act1 ? 2 * mp + 2 : 0;
  const int nkv = act1 ? nkv1 : nkv0;
  const int hq = p.hidx ? p.hidx[h] : h;
  const int hk = (p.HKV > 0) ? p.kvidx[h] : hq;
  const int hv = (p.HKV > 0) ? p.kvidx[h] : h;

  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < C::KSTAGE; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 128);
      mbar_init(&bars->buf_free[i], 1);
    }
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
#ifdef SAF_FWD_TRACE
  const bool trace_on = (b == 0 && h == 0 && mp == p.n_pairs - 1) && ((tid & 31) == 0);
#endif

  if (warp >= 8) {
    reg_dec<56>();
    // score tiles in production order: k -> (tile t, key step j); with one active tile k = j
    const int n_prod = act1 ? 2 * nkv1 : nkv0;
    const bool leader = elect_one();
    if (warp == 8) {
      // ---------------------------------------------------------- TMA producer
      if (leader) {
        tma_prefetch_desc(&mapQ);
        tma_prefetch_desc(&mapK);
        tma_prefetch_desc(&mapV);
        if (live) {
          mbar_expect_tx(&bars->q_full, (act1 ? 2 : 1) * C::TILE_BYTES);
          load_tile<HD>(sQ, &mapQ, &bars->q_full, row0, hq, b);
          if (act1) load_tile<HD>(sQ + C::TILE_BYTES, &mapQ, &bars->q_full, row0 + FM, hq, b);
        }
        // order of first use: K0, then (K_{j+1}, V_j) -- scores run one key tile ahead of the outputs
        bool ok = true;
        auto load_k = [&](int j) {
          const int s = j & (C::KSTAGE - 1);
          if (!mbar_wait(&bars->k_empty[s], ((j / C::KSTAGE) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 20);
            ok = false;
            return;
          }
          mbar_expect_tx(&bars->k_full[s], C::TILE_BYTES);
          load_tile<HD>(sK + s * C::TILE_BYTES, &mapK, &bars->k_full[s], j * FN, hk, b);
        };
        auto load_v = [&](int j) {
          const int s = j & (C::KSTAGE - 1);
          if (!mbar_wait(&bars->v_empty[s], ((j / C::KSTAGE) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 21);
            ok = false;
            return;
          }
          mbar_expect_tx(&bars->v_full[s], C::TILE_BYTES);
          load_tile<HD>(sV + s * C::TILE_BYTES, &mapV, &bars->v_full[s], j * FN, hv, b);
        };
        if (live) load_k(0);
        for (int j = 0; j < nkv && ok; ++j) {
          if (live && j + 1 < nkv) load_k(j + 1);
          if (ok) load_v(j);
        }
      }
    } else if (warp == 9 && live) {
      // ---------------------------------------------------------- score MMA issuer
      const uint32_t idesc_s = umma_idesc_bf16(FM, FN, 0, 0);   // Q K^T: both operands K-major
      const uint32_t qaddr0 = smem_u32(sQ), kbase = smem_u32(sK);
      bool ok = mbar_wait(&bars->q_full, 0);
      if (!ok) dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 22);
      int buf = 0, bph = 0, k_waited = -1;
      for (int k = 0; k < n_prod && ok; ++k) {
        const int t = act1 ? (k & 1) : 0, j = act1 ? (k >> 1) : k;
        if (j < (t ? nkv1 : nkv0)) {
          const int ks_ = j & (C::KSTAGE - 1);
          if (j > k_waited) {
            if (!mbar_wait(&bars->k_full[ks_], (j / C::KSTAGE) & 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 23);
              break;
            }
            k_waited = j;
            FTRACE(5, j);
          }
          // the PV product that read P from this buffer (its previous use) must have finished
          if (k >= C::NBUF && !mbar_wait(&bars->buf_free[buf], bph ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 24);
            break;
          }
          tc_fence_after();
          if (t == 0) FTRACE(2, j);
          const uint32_t qa = qaddr0 + t * C::TILE_BYTES, ka = kbase + ks_ * C::TILE_BYTES;
          const uint32_t d = tmem + buf * FN;
          if (leader) {
            // (descriptors built once per product, advanced per K step: the issuing lane competes for its scheduler
            // with two softmax warps, so every instruction it saves reaches the tensor pipe sooner)
            const uint64_t dq = umma_smem_desc_sw128(qa, 16, 1024), dk = umma_smem_desc_sw128(ka, 16, 1024);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
              umma_ss(d, umma_desc_advance(dq, off), umma_desc_advance(dk, off), idesc_s, ks > 0);
            }
            umma_commit(&bars->s_full[buf]);
            if (t == 1 || !act1) umma_commit(&bars->k_empty[ks_]);   // last reader of K_j
          }
          __syncwarp();
        }
        if (++buf == C::NBUF) {
          buf = 0;
          bph ^= 1;
        }
      }
    } else if (warp == 10) {
      // ---------------------------------------------------------- output MMA issuer
      const uint32_t idesc_o = umma_idesc_bf16(FM, HD, 0, 1);   // P V: V is MN-major
      const uint32_t vbase = smem_u32(sV);
      int buf = 0, bph = 0, v_waited = -1;
      for (int c = 0; c < n_prod; ++c) {
        const int t = act1 ? (c & 1) : 0, j = act1 ? (c >> 1) : c;
        if (j < (t ? nkv1 : nkv0)) {
          const int vs_ = j & (C::KSTAGE - 1);
          if (j > v_waited) {
            if (!mbar_wait(&bars->v_full[vs_], (j / C::KSTAGE) & 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 25);
              break;
            }
            v_waited = j;
            FTRACE(4, j);
          }
          const uint32_t va = vbase + vs_ * C::TILE_BYTES;
          const uint32_t dO = tmem + C::O_COL + t * HD, aP = tmem + buf * FN;
          if (!mbar_wait(&bars->p_full[buf], bph)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 26);
            break;
          }
          tc_fence_after();
          if (t == 0) FTRACE(3, j);
          if (leader) {
            const uint64_t dv = umma_smem_desc_sw128(va, 16384, 1024);
#pragma unroll
            for (int ks = 0; ks < FN / 16; ++ks)
              umma_ts(dO, aP + ks * 8, umma_desc_advance(dv, ks * 2048), idesc_o, (j > 0) || (ks > 0));
            umma_commit(&bars->buf_free[buf]);
            if (t == 1 || !act1) umma_commit(&bars->v_empty[vs_]);   // last reader of V_j
          }
          __syncwarp();
        }
        if (++buf == C::NBUF) {
          buf = 0;
          bph ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    reg_inc<224>();
    const int t = warp >> 2;
    const int r = tid & 127;
    const int nk = t ? nkv1 : nkv0;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tO = tmem + lane_base + C::O_COL + t * HD;
    // score buffer of this tile's step j: production index k = 2j + t (k = j with one active tile)
    const int kstep = act1 ? 2 : 1;
    int buf = act1 ? t : 0, bph = 0, pbuf = 0, pph = 0;
    const float sc = p.scale_log2;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    if (!live) {
      // ---- frozen head: this thread produces row r of the pattern tile, P_t(j) = pattern[i0 + r, 128 j ...]
      const int i_row = row0 + t * FM + r;                 // absolute query row
      const bool row_ok = i_row < p.T;
      const int hp = p.pidx ? p.pidx[h] : h;
      float zrow = INFINITY;                               // rows past T give exact zeros (decomposed)
      if (state == SAF_DECOMP && row_ok)
        zrow = load_rt(p.z, (int64_t)h * p.z_s[0] + (int64_t)i_row * p.z_s[1], p.dec_dtype);
      float* al_s = bars->dec_alpha[t];                    // alpha of the tile's 128 keys
      float* rh_s = bars->dec_rho[t];                      // rho[(i0 - j0 - 127) + x], x in [0, 255)
      for (int j = 0; j < nk; ++j) {
        const uint32_t tS = tmem + lane_base + buf * FN;
        const int j0 = j * FN;
        // the P V product that read this buffer (three score tiles ago) must have finished
        bool gave_up = (act1 ? 2 * j + t : j) >= C::NBUF && !mbar_wait(&bars->buf_free[buf], bph ^ 1);
        // decomposed heads meet at named barriers below: the decision to leave is taken by all 128 threads
        // together (the same barrier tells that the previous step's readers are done with the vectors)
        if (state == SAF_DECOMP) gave_up = named_bar_or(1 + t, 128, gave_up);
        if (gave_up) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 31);
          ok = false;
          break;
        }
        tc_fence_after();
        const bool diag = (j == nk - 1);
        if (state == SAF_DECOMP) {
          const int key = j0 + r;
          al_s[r] = (key < p.T) ? load_rt(p.alpha, (int64_t)h * p.alpha_s[0] + (int64_t)key * p.alpha_s[1], p.dec_dtype) : 0.f;
          const int d0 = row0 + t * FM - j0 - 127;         // distance of rh_s[0]
#pragma unroll
          for (int x = r; x < 255; x += 128) {
            const int d = d0 + x;
            rh_s[x] = (d >= 0 && d < p.T) ? load_rt(p.rho, (int64_t)h * p.rho_s[0] + (int64_t)d * p.rho_s[1], p.dec_dtype) : 0.f;
          }
          named_bar_sync(1 + t, 128);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float pv[32];
          if (state == SAF_DENSE) {
            const int64_t base = (int64_t)hp * p.patt_s[0] + (int64_t)i_row * p.patt_s[1] + (int64_t)(j0 + q * 32) * p.patt_s[2];
            if (row_ok && p.patt_s[2] == 1 && p.patt_dtype == SAF_BF16) {
              const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.patt) + base);
              const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && (j0 + q * 32 + 32 <= p.T);
#pragma unroll
              for (int v8 = 0; v8 < 4; ++v8) {
                if (vec) {
                  const uint4 u4 = src[v8];
                  const uint32_t w4[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    pv[v8 * 8 + 2 * e] = __uint_as_float(w4[e] << 16);
                    pv[v8 * 8 + 2 * e + 1] = __uint_as_float(w4[e] & 0xffff0000u);
                  }
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const int c = q * 32 + v8 * 8 + e;
                    pv[v8 * 8 + e] = (j0 + c < p.T) ? load_rt(p.patt, base + v8 * 8 + e, SAF_BF16) : 0.f;
                  }
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int c = q * 32 + i;
                pv[i] = (row_ok && j0 + c < p.T) ? load_rt(p.patt, base + (int64_t)i * p.patt_s[2], p.patt_dtype) : 0.f;
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int c = q * 32 + i;
              pv[i] = ex2((al_s[c] + rh_s[r - c + 127] - zrow) * LOG2E_F);
            }
          }
          if (diag) {   // keys after the row do not count (a stored pattern is lower-triangular anyway)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (q * 32 + i > r) pv[i] = 0.f;
          }
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(pv[2 * i], pv[2 * i + 1]);
          tmem_st16(tS + q * 16, pk);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars->p_full[buf]);
        pbuf = buf;
        pph = bph;
        buf += kstep;
        if (buf >= C::NBUF) {
          buf -= C::NBUF;
          bph ^= 1;
        }
      }
      l = 1.f;
    } else
    for (int j = 0; j < nk; ++j) {
      const uint32_t tS = tmem + lane_base + buf * FN;
      if (!mbar_wait(&bars->s_full[buf], bph)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 27);
        ok = false;
        break;
      }
      tc_fence_after();
      if (warp == 0) FTRACE(0, j);
      uint32_t s[4][32];
#pragma unroll
      for (int q = 0; q < 4; ++q) tmem_ld32(tS + q * 32, s[q]);
      tmem_ld_wait();
      if (j == nk - 1) {  // diagonal tile: keys after the row are masked
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (q * 32 + i > r) s[q][i] = 0xff800000u;  // -inf
      }
      // exponentials of the row against reference maximum `mref`, packed to bf16 into the first 64 columns of the
      // score buffer; returns the row sum of the (unrounded) exponentials
      auto emit_p = [&](float mref) -> float {
        const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(-mref, -mref);
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(s[q][2 * i]), __uint_as_float(s[q][2 * i + 1])), sc2, nm2);
            float2 e;
            if (i < SAF_POLY_EXP_PER_16 / 2) {
              e = exp2_poly2(x);
            } else {
              e.x = ex2(x.x);
              e.y = ex2(x.y);
            }
            if (i & 1) acc1 = __fadd2_rn(acc1, e);
            else acc0 = __fadd2_rn(acc0, e);
            pk[i] = pack_bf16(e.x, e.y);
          }
          tmem_st16(tS + q * 16, pk);
        }
        acc0 = __fadd2_rn(acc0, acc1);
        return acc0.x + acc0.y;
      };
      auto row_max = [&]() -> float {
        float mx0 = __uint_as_float(s[0][0]), mx1 = __uint_as_float(s[1][0]);
        float mx2 = __uint_as_float(s[2][0]), mx3 = __uint_as_float(s[3][0]);
#pragma unroll
        for (int i = 1; i < 31; i += 2) {
          mx0 = fmax3(mx0, __uint_as_float(s[0][i]), __uint_as_float(s[0][i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(s[1][i]), __uint_as_float(s[1][i + 1]));
          mx2 = fmax3(mx2, __uint_as_float(s[2][i]), __uint_as_float(s[2][i + 1]));
          mx3 = fmax3(mx3, __uint_as_float(s[3][i]), __uint_as_float(s[3][i + 1]));
        }
        mx0 = fmax3(mx0, __uint_as_float(s[0][31]), __uint_as_float(s[1][31]));
        mx2 = fmax3(mx2, __uint_as_float(s[2][31]), __uint_as_float(s[3][31]));
        return fmax3(mx0, mx1, fmaxf(mx2, mx3)) * sc;
      };
      // O_t *= f per row once P_t(j-1) V_{j-1} has landed; false when the wait ran out
      auto rescale_o = [&](bool need, float mx) -> bool {
        if (!mbar_wait(&bars->buf_free[pbuf], pph)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 28);
          return false;
        }
        tc_fence_after();
        const float f = need ? ex2(m_ref - mx) : 1.f;
        if (need) m_ref = mx;
        l *= f;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tO + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tmem_st32(tO + c0, o);
        }
        return true;
      };
      const float mx = row_max();
      if (j == 0) {
        m_ref = mx;
      } else {
        const bool need = mx > m_ref + RESCALE_THRESHOLD;
        if (__any_sync(0xffffffffu, need) && !rescale_o(need, mx)) {
          ok = false;
          break;
        }
      }
      l += emit_p(m_ref);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_full[buf]);
      if (warp == 0) FTRACE(1, j);
      pbuf = buf;
      pph = bph;
      buf += kstep;
      if (buf >= C::NBUF) {
        buf -= C::NBUF;
        bph ^= 1;
      }
    }
    if (nk > 0) {
      // the last PV product of this tile
      if (ok && !mbar_wait(&bars->buf_free[pbuf], pph)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 29);
        ok = false;
      }
      tc_fence_after();
      const float inv = 1.f / l;
      uint8_t* stage = sQ + t * C::TILE_BYTES;   // this tile's Q is no longer read
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tO + c0, o);
        tmem_ld_wait();
        uint8_t* dst = stage + (c0 >> 6) * 16384 + r * 128;
        const int cbase = (c0 & 63) >> 3;   // first 16-byte chunk of this group inside the 128-byte row
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 q;
          q.x = pack_bf16(__uint_as_float(o[c * 8 + 0]) * inv, __uint_as_float(o[c * 8 + 1]) * inv);
          q.y = pack_bf16(__uint_as_float(o[c * 8 + 2]) * inv, __uint_as_float(o[c * 8 + 3]) * inv);
          q.z = pack_bf16(__uint_as_float(o[c * 8 + 4]) * inv, __uint_as_float(o[c * 8 + 5]) * inv);
          q.w = pack_bf16(__uint_as_float(o[c * 8 + 6]) * inv, __uint_as_float(o[c * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + (((cbase + c) ^ (r & 7)) << 4)) = q;
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1 + t, 128);
      const int trow = row0 + t * FM;
      if (r == 0 && ok) {
#pragma unroll
        for (int hh = 0; hh < HD / 64; ++hh) tma_store_4d(&mapO, stage + hh * 16384, hh * 64, trow, h, b);
        tma_store_commit();
        tma_store_wait_all();
      }
      if (live && p.lse && trow + r < p.T)
        p.lse[(int64_t)b * p.lse_s[0] + (int64_t)h * p.lse_s[1] + (int64_t)(trow + r) * p.lse_s[2]] = m_ref + log2f(l);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------------------
// Persistent live-tile kernel.  Same warp roles, tiles and softmax as flash_fwd_kernel above, but a CTA stays on
// its SM and pulls (batch, live head, row-tile pair) items from a queue: TMEM and barriers are set up once, the
// K/V rings and the score buffers keep rotating across items, and while the softmax warpgroups finish an item
// (last P V, O / l, TMA store) the producer and the issuing warps are already loading and multiplying the next
// one.  A one-shot CTA pays about 10 us of set-up, pipeline fill and drain per tile pair (measured: slope of
// the launch time over the CTA count); this removes most of it.
//
// The queue is an atomic counter in two ints the caller provides (zero on entry): items are handed out in the
// order the one-shot launch uses (head groups, heaviest row pairs first), so the balance is the same greedy
// longest-first schedule.  The last CTA to see the end of the queue sets both ints back to zero.
//
//   warp 8      TMA and queue: claims the next item only when it has issued every load of the current one (an
//               item claimed early would sit in this CTA while other SMs run dry), publishes it in a 2-slot
//               ring in shared memory (w_full / w_empty), then Q_0, K_0, Q_1, (K_{j+1}, V_j); Q_t of the next
//               item lands as soon as the last score product of tile t has retired (q_free, an MMA commit)
//   warp 9      scores, warp 10 outputs: as above, with running tile counters instead of per-CTA ones
//   warps 0-7   softmax; the epilogue releases O_t (o_free) as soon as it sits in registers and stages the
//               tile through its own 16 KB buffer (64 columns at a time), so Q is never held back by a store
// Score tiles of an item are produced in the order (0,0) (1,0) (0,1) (1,1) ... with the extra diagonal step
// of tile 1 last, so every index of the running counter is a real tile and barrier phases follow from it.
struct PersistBars {
  uint64_t q_full[2], q_free[2];
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[3], p_full[3], buf_free[3];
  uint64_t o_free[2];
  uint64_t w_full[2], w_empty[2];
  volatile int32_t work[2];
  uint32_t tmem_base;
};
constexpr int W_CONSUMERS = 10;   // warps 9, 10 and the eight softmax warps, one arrival each
constexpr int O_STAGE_BYTES = 128 * 128;   // 128 rows x 64 bf16 columns, per query tile

struct TileGeom {
  int b, h, mp, row0, nkv0, nkv1, nkv, n_prod;
  bool act1;
};

__device__ __forceinline__ TileGeom decode_item(const FlashParams& p, int li) {
  TileGeom g;
  const int per_group = HEAD_GROUP * p.n_pairs;
  const int grp = li / per_group;
  const int gsize = min(HEAD_GROUP, p.B * p.U - grp * HEAD_GROUP);
  const int rem = li - grp * per_group;
  g.mp = p.n_pairs - 1 - rem / gsize;
  const int bu = grp * HEAD_GROUP + rem % gsize;
  g.b = bu / p.U;
  g.h = p.live_head[bu % p.U];
  g.row0 = g.mp * 2 * FM;
  g.act1 = g.row0 + FM < p.T;
  g.nkv0 = 2 * g.mp + 1;
  g.nkv1 = g.act1 ? 2 * g.mp + 2 : 0;
  g.nkv = g.act1 ? g.nkv1 : g.nkv0;
  g.n_prod = g.nkv0 + g.nkv1;
  return g;
}
// (tile, key step) of the idx-th score tile of an item
__device__ __forceinline__ void tile_of(const TileGeom& g, int idx, int& t, int& j) {
  if (!g.act1) { t = 0; j = idx; }
  else if (idx == 2 * g.nkv0) { t = 1; j = g.nkv0; }
  else { t = idx & 1; j = idx >> 1; }
}

template <int HD>
__global__ void __launch_bounds__(FLASH_THREADS, 1)
flash_fwd_persistent_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                            const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapO,
                            const __grid_constant__ CUtensorMap mapP, const __grid_constant__ CUtensorMap mapV64,
                            const __grid_constant__ FlashParams p) {
  using C = Cfg<HD>;
  const int bh_count = p.B * p.H;
  if ((int)blockIdx.x < bh_count) {          // scan slots, as in flash_fwd_kernel
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const int state = p.force_state >= 0 ? p.force_state : p.frozen[h];
    if (state == SAF_SINK_DECAY && p.has_scan) {
      {
        // the whole sequence as 128-row Toeplitz products on the tensor core, one 64-column slice after the other
        // (about a third of the time of the register scan, so the SM joins the live tiles that much earlier)
        if (p.T >= 4 * MB && p.scan.HD == HD) {
          extern __shared__ uint8_t scan_smem_raw[];
          MsParams mp;
          mp.a = p.scan;
          mp.chunk = (p.T + MB - 1) / MB * MB;
          mp.use_stash = 0;
          mp.status = p.status;
          sink_decay_apply_mma_cta<SCAN_ROLE_STAGES>(mapV, mapO, mp, b, h, 0, 0, HD / 64, scan_smem_raw);
          return;
        }
      }
      if (threadIdx.x < SCAN_NT)
        for (int col0 = 0; col0 < HD; col0 += SCAN_COLS) sink_decay_scan_cta<__nv_bfloat16, false>(p.scan, b, h, col0);
    }
    return;
  }
  if ((int)blockIdx.x < bh_count + p.dense_slots) {   // dense-pattern role
    extern __shared__ uint8_t dense_smem_raw[];
    uint8_t* dsm = (uint8_t*)(((uintptr_t)dense_smem_raw + 1023) & ~(uintptr_t)1023);
    dense_pv_cta<HD>(mapP, mapV64, mapO, p.dense, (int)blockIdx.x - bh_count, dsm);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + C::Q_BYTES;
  uint8_t* sV = sK + C::KSTAGE * C::TILE_BYTES;
  uint8_t* sO = sK + C::RING_BYTES;                       // 2 x O_STAGE_BYTES (head_dim 64 only)
  PersistBars* bars = reinterpret_cast<PersistBars*>(sO + C::O_STAGING);
  const int tid = threadIdx.x, warp = tid >> 5;

  if (tid == 0) {
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->q_full[t], 1);
      mbar_init(&bars->q_free[t], 1);
      mbar_init(&bars->o_free[t], 128);
      mbar_init(&bars->w_full[t], 1);
      mbar_init(&bars->w_empty[t], W_CONSUMERS);
    }
    for (int s = 0; s < C::KSTAGE; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 128);
      mbar_init(&bars->buf_free[i], 1);
    }
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(&bars->tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  // next item of this CTA's sequence (n-th fetch); -1 = queue empty, -2 = the wait ran out.  `arrive`: this
  // thread reports the slot as read (one thread per consumer warp)
  auto fetch = [&](int n, bool arrive) -> int {      // whole warp
    const int slot = n & 1;
    if (!mbar_wait(&bars->w_full[slot], (n >> 1) & 1)) return -2;
    const int it = bars->work[slot];
    __syncwarp();                                      // every lane has read the slot before it is handed back
    if (arrive) mbar_arrive(&bars->w_empty[slot]);
    return it;
  };
  if (warp >= 8) {
    reg_dec<56>();
    const bool leader = elect_one();
    if (warp == 8) {
      // ---------------------------------------------------------- TMA producer and tile queue
      if (leader) {
        tma_prefetch_desc(&mapQ);
        tma_prefetch_desc(&mapK);
        tma_prefetch_desc(&mapV);
        uint32_t kc = 0, vc = 0, use_q[2] = {0, 0};
        bool ok = true;
        for (int n = 0; ok; ++n) {
          // claim the next item and publish it to the other warps
          const int slot = n & 1;
          if (n >= 2 && !mbar_wait(&bars->w_empty[slot], ((n >> 1) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 40);
            bars->work[slot] = -1;
            mbar_arrive(&bars->w_full[slot]);
            break;
          }
          const int idx = atomicAdd(p.sched, 1);
          const int it = idx < p.n_items ? idx : -1;
          bars->work[slot] = it;
          mbar_arrive(&bars->w_full[slot]);
          if (it < 0) {
            const int seen = atomicAdd(p.sched + 1, 1);
            if (seen == (int)gridDim.x - p.lead - 1) {   // every persistent CTA has reached the end of the queue
              p.sched[0] = 0;
              p.sched[1] = 0;
            }
            break;
          }
          const TileGeom g = decode_item(p, it);
          const int hq = p.hidx ? p.hidx[g.h] : g.h;
          const int hk = (p.HKV > 0) ? p.kvidx[g.h] : hq;
          const int hv = (p.HKV > 0) ? p.kvidx[g.h] : g.h;
          auto load_q = [&](int t) {
            if (use_q[t] > 0 && !mbar_wait(&bars->q_free[t], (use_q[t] - 1) & 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 42);
              ok = false;
              return;
            }
            mbar_expect_tx(&bars->q_full[t], C::TILE_BYTES);
            load_tile<HD>(sQ + t * C::TILE_BYTES, &mapQ, &bars->q_full[t], g.row0 + t * FM, hq, g.b);
            ++use_q[t];
          };
          auto load_k = [&](int j) {
            const int s = kc & (C::KSTAGE - 1);
            if (!mbar_wait(&bars->k_empty[s], ((kc / C::KSTAGE) & 1) ^ 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 43);
              ok = false;
              return;
            }
            mbar_expect_tx(&bars->k_full[s], C::TILE_BYTES);
            load_tile<HD>(sK + s * C::TILE_BYTES, &mapK, &bars->k_full[s], j * FN, hk, g.b);
            ++kc;
          };
          auto load_v = [&](int j) {
            const int s = vc & (C::KSTAGE - 1);
            if (!mbar_wait(&bars->v_empty[s], ((vc / C::KSTAGE) & 1) ^ 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 44);
              ok = false;
              return;
            }
            mbar_expect_tx(&bars->v_full[s], C::TILE_BYTES);
            load_tile<HD>(sV + s * C::TILE_BYTES, &mapV, &bars->v_full[s], j * FN, hv, g.b);
            ++vc;
          };
          load_q(0);
          if (ok) load_k(0);
          if (ok && g.act1) load_q(1);
          for (int j = 0; j < g.nkv && ok; ++j) {
            if (j + 1 < g.nkv) load_k(j + 1);
            if (ok) load_v(j);
          }
        }
      }
    } else if (warp == 9) {
      // ---------------------------------------------------------- score MMA issuer
      const uint32_t idesc_s = umma_idesc_bf16(FM, FN, 0, 0);
      const uint32_t qaddr0 = smem_u32(sQ), kbase = smem_u32(sK);
      uint32_t gs = 0, kc = 0, use_q[2] = {0, 0};
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int it = fetch(n, leader);
        if (it < 0) {
          if (it == -2) dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 45);
          break;
        }
        const TileGeom g = decode_item(p, it);
        int k_waited = -1;
        bool q_waited[2] = {false, false};
        for (int idx = 0; idx < g.n_prod; ++idx, ++gs) {
          int t, j;
          tile_of(g, idx, t, j);
          if (!q_waited[t]) {
            if (!mbar_wait(&bars->q_full[t], use_q[t] & 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 46);
              ok = false;
              break;
            }
            q_waited[t] = true;
          }
          const uint32_t kt = kc + j;
          const int ks_ = kt & (C::KSTAGE - 1);
          if (j > k_waited) {
            if (!mbar_wait(&bars->k_full[ks_], (kt / C::KSTAGE) & 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 47);
              ok = false;
              break;
            }
            k_waited = j;
          }
          const uint32_t buf = gs % C::NBUF;
          if (gs >= (uint32_t)C::NBUF && !mbar_wait(&bars->buf_free[buf], ((gs / C::NBUF) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 48);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t qa = qaddr0 + t * C::TILE_BYTES, ka = kbase + ks_ * C::TILE_BYTES;
          const uint32_t d = tmem + buf * FN;
          if (leader) {
            // (descriptors built once per product, advanced per K step: the issuing lane competes for its scheduler
            // with two softmax warps, so every instruction it saves reaches the tensor pipe sooner)
            const uint64_t dq = umma_smem_desc_sw128(qa, 16, 1024), dk = umma_smem_desc_sw128(ka, 16, 1024);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
              umma_ss(d, umma_desc_advance(dq, off), umma_desc_advance(dk, off), idesc_s, ks > 0);
            }
            umma_commit(&bars->s_full[buf]);
            if (t == 1 || !g.act1) umma_commit(&bars->k_empty[ks_]);   // last reader of K_j
            if (!C::STAGE_IN_Q && j == (t ? g.nkv1 : g.nkv0) - 1) umma_commit(&bars->q_free[t]);   // last reader of Q_t
          }
          __syncwarp();
        }
        kc += g.nkv;
        ++use_q[0];
        if (g.act1) ++use_q[1];
      }
    } else if (warp == 10) {
      // ---------------------------------------------------------- output MMA issuer
      const uint32_t idesc_o = umma_idesc_bf16(FM, HD, 0, 1);
      const uint32_t vbase = smem_u32(sV);
      uint32_t gs = 0, vc = 0, use_o[2] = {0, 0};
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int it = fetch(n, leader);
        if (it < 0) {
          if (it == -2) dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 49);
          break;
        }
        const TileGeom g = decode_item(p, it);
        int v_waited = -1;
        for (int idx = 0; idx < g.n_prod; ++idx, ++gs) {
          int t, j;
          tile_of(g, idx, t, j);
          const uint32_t vt = vc + j;
          const int vs_ = vt & (C::KSTAGE - 1);
          if (j > v_waited) {
            if (!mbar_wait(&bars->v_full[vs_], (vt / C::KSTAGE) & 1)) {
              dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 50);
              ok = false;
              break;
            }
            v_waited = j;
          }
          // the epilogue of the previous item must have taken O_t out of TMEM before it is overwritten
          if (j == 0 && use_o[t] > 0 && !mbar_wait(&bars->o_free[t], (use_o[t] - 1) & 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 51);
            ok = false;
            break;
          }
          const uint32_t buf = gs % C::NBUF;
          if (!mbar_wait(&bars->p_full[buf], (gs / C::NBUF) & 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 52);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t va = vbase + vs_ * C::TILE_BYTES;
          const uint32_t dO = tmem + C::O_COL + t * HD, aP = tmem + buf * FN;
          if (leader) {
            const uint64_t dv = umma_smem_desc_sw128(va, 16384, 1024);
#pragma unroll
            for (int ks = 0; ks < FN / 16; ++ks)
              umma_ts(dO, aP + ks * 8, umma_desc_advance(dv, ks * 2048), idesc_o, (j > 0) || (ks > 0));
            umma_commit(&bars->buf_free[buf]);
            if (t == 1 || !g.act1) umma_commit(&bars->v_empty[vs_]);   // last reader of V_j
          }
          __syncwarp();
        }
        vc += g.nkv;
        ++use_o[0];
        if (g.act1) ++use_o[1];
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    reg_inc<224>();
    const int t = warp >> 2;
    const int r = tid & 127;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tO = tmem + lane_base + C::O_COL + t * HD;
    const float sc = p.scale_log2;
    const bool warp_lead = (tid & 31) == 0;
    uint32_t g_base = 0;
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int it = fetch(n, warp_lead);
      if (it < 0) {
        if (it == -2) dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 53);
        break;
      }
      const TileGeom g = decode_item(p, it);
      const int nk = t ? g.nkv1 : g.nkv0;
      if (nk > 0) {
        float m_ref = -INFINITY, l = 0.f;
        uint32_t pbuf = 0, pph = 0;
        for (int j = 0; j < nk; ++j) {
          const uint32_t gi = g_base + (g.act1 ? ((t == 1 && j == g.nkv0) ? 2 * g.nkv0 : 2 * j + t) : j);
          const uint32_t buf = gi % C::NBUF, bph = (gi / C::NBUF) & 1;
          const uint32_t tS = tmem + lane_base + buf * FN;
          if (!mbar_wait(&bars->s_full[buf], bph)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 54);
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t s[4][32];
#pragma unroll
          for (int q = 0; q < 4; ++q) tmem_ld32(tS + q * 32, s[q]);
          tmem_ld_wait();
          if (j == nk - 1) {  // diagonal tile: keys after the row are masked
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (q * 32 + i > r) s[q][i] = 0xff800000u;
          }
          float mx0 = __uint_as_float(s[0][0]), mx1 = __uint_as_float(s[1][0]);
          float mx2 = __uint_as_float(s[2][0]), mx3 = __uint_as_float(s[3][0]);
#pragma unroll
          for (int i = 1; i < 31; i += 2) {
            mx0 = fmax3(mx0, __uint_as_float(s[0][i]), __uint_as_float(s[0][i + 1]));
            mx1 = fmax3(mx1, __uint_as_float(s[1][i]), __uint_as_float(s[1][i + 1]));
            mx2 = fmax3(mx2, __uint_as_float(s[2][i]), __uint_as_float(s[2][i + 1]));
            mx3 = fmax3(mx3, __uint_as_float(s[3][i]), __uint_as_float(s[3][i + 1]));
          }
          mx0 = fmax3(mx0, __uint_as_float(s[0][31]), __uint_as_float(s[1][31]));
          mx2 = fmax3(mx2, __uint_as_float(s[2][31]), __uint_as_float(s[3][31]));
          const float mx = fmax3(mx0, mx1, fmaxf(mx2, mx3)) * sc;
          if (j == 0) {
            m_ref = mx;
          } else {
            const bool need = mx > m_ref + RESCALE_THRESHOLD;
            if (__any_sync(0xffffffffu, need)) {
              if (!mbar_wait(&bars->buf_free[pbuf], pph)) {
                dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 55);
                ok = false;
                break;
              }
              tc_fence_after();
              const float f = need ? ex2(m_ref - mx) : 1.f;
              if (need) m_ref = mx;
              l *= f;
#pragma unroll
              for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tO + c0, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                tmem_st32(tO + c0, o);
              }
            }
          }
          const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(-m_ref, -m_ref);
          float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 x = __ffma2_rn(make_float2(__uint_as_float(s[q][2 * i]), __uint_as_float(s[q][2 * i + 1])), sc2, nm2);
              float2 e;
              if (i < SAF_POLY_EXP_PER_16 / 2) {
                e = exp2_poly2(x);
              } else {
                e.x = ex2(x.x);
                e.y = ex2(x.y);
              }
              if (i & 1) acc1 = __fadd2_rn(acc1, e);
              else acc0 = __fadd2_rn(acc0, e);
              pk[i] = pack_bf16(e.x, e.y);
            }
            tmem_st16(tS + q * 16, pk);
          }
          acc0 = __fadd2_rn(acc0, acc1);
          l += acc0.x + acc0.y;
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(&bars->p_full[buf]);
          pbuf = buf;
          pph = bph;
        }
        if (!ok) break;
        // ---- epilogue of tile t: O / l -> bf16 -> the tile's own Q buffer -> TMA store
        if (!mbar_wait(&bars->buf_free[pbuf], pph)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_SOFTMAX, 56);
          ok = false;
          break;
        }
        tc_fence_after();
        const float inv = 1.f / l;
        const int trow = g.row0 + t * FM;
        if constexpr (C::STAGE_IN_Q) {
          // head_dim 128: the tile's own Q buffer is the staging area (its last score product retired before the
          // last P V did); Q_t of the next item may land once the store has read it
          uint8_t* stage = sQ + t * C::TILE_BYTES;
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tO + c0, o);
            tmem_ld_wait();
            if (c0 + 32 >= HD) {   // O_t is in registers: the next item may overwrite it
              tc_fence_before();
              mbar_arrive(&bars->o_free[t]);
            }
            uint8_t* dst = stage + (c0 >> 6) * 16384 + r * 128;
            const int cbase = (c0 & 63) >> 3;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 q;
              q.x = pack_bf16(__uint_as_float(o[c * 8 + 0]) * inv, __uint_as_float(o[c * 8 + 1]) * inv);
              q.y = pack_bf16(__uint_as_float(o[c * 8 + 2]) * inv, __uint_as_float(o[c * 8 + 3]) * inv);
              q.z = pack_bf16(__uint_as_float(o[c * 8 + 4]) * inv, __uint_as_float(o[c * 8 + 5]) * inv);
              q.w = pack_bf16(__uint_as_float(o[c * 8 + 6]) * inv, __uint_as_float(o[c * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + (((cbase + c) ^ (r & 7)) << 4)) = q;
            }
          }
          fence_proxy_async_smem();
          named_bar_sync(1 + t, 128);
          if (r == 0) {
#pragma unroll
            for (int hh = 0; hh < HD / 64; ++hh) tma_store_4d(&mapO, stage + hh * 16384, hh * 64, trow, g.h, g.b);
            tma_store_commit();
            tma_store_wait_read();
            mbar_arrive(&bars->q_free[t]);
          }
        } else {
          uint8_t* stage = sO + t * O_STAGE_BYTES;
#pragma unroll
          for (int hh = 0; hh < HD / 64; ++hh) {
            // the staging buffer is free once the store that last read it (previous item) is done
            if (r == 0) tma_store_wait_read();
            named_bar_sync(1 + t, 128);
#pragma unroll
            for (int c0 = hh * 64; c0 < hh * 64 + 64; c0 += 32) {
              uint32_t o[32];
              tmem_ld32(tO + c0, o);
              tmem_ld_wait();
              if (c0 + 32 >= HD) {   // O_t is in registers: the next item may overwrite it
                tc_fence_before();
                mbar_arrive(&bars->o_free[t]);
              }
              uint8_t* dst = stage + r * 128;
              const int cbase = (c0 & 63) >> 3;
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                uint4 q;
                q.x = pack_bf16(__uint_as_float(o[c * 8 + 0]) * inv, __uint_as_float(o[c * 8 + 1]) * inv);
                q.y = pack_bf16(__uint_as_float(o[c * 8 + 2]) * inv, __uint_as_float(o[c * 8 + 3]) * inv);
                q.z = pack_bf16(__uint_as_float(o[c * 8 + 4]) * inv, __uint_as_float(o[c * 8 + 5]) * inv);
                q.w = pack_bf16(__uint_as_float(o[c * 8 + 6]) * inv, __uint_as_float(o[c * 8 + 7]) * inv);
                *reinterpret_cast<uint4*>(dst + (((cbase + c) ^ (r & 7)) << 4)) = q;
              }
            }
            fence_proxy_async_smem();
            named_bar_sync(1 + t, 128);
            if (r == 0) {
              tma_store_4d(&mapO, stage, hh * 64, trow, g.h, g.b);
              tma_store_commit();
            }
          }
        }
        if (p.lse && trow + r < p.T)
          p.lse[(int64_t)g.b * p.lse_s[0] + (int64_t)g.h * p.lse_s[1] + (int64_t)(trow + r) * p.lse_s[2]] = m_ref + log2f(l);
      }
      g_base += g.n_prod;
    }
    if (r == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::TMEM_COLS);
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

bool tma_ok(const SafTensor& t) {
  if (!t.ptr || !aligned16(t.ptr) || t.stride[3] != 1) return false;
  for (int i = 0; i < 3; ++i)
    if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
  return true;
}

int make_map4(CUtensorMap* m, const SafTensor& t, int B, int Hn, int T, int HD) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)T, (uint64_t)Hn, (uint64_t)B};
  uint64_t strides[4] = {0, (uint64_t)t.stride[2] * 2, (uint64_t)t.stride[1] * 2, (uint64_t)t.stride[0] * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tensor_map_bf16(m, t.ptr, 4, dims, strides, box, true);
}

template <int HD>
int launch_typed(const SafMixedAttnArgs& a, uint32_t want, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mo;
  int rc;
  const int Hkv = a.HKV > 0 ? a.HKV : 0;
  const bool any_live = a.U > 0 && a.q.ptr && a.k.ptr;     // an all-frozen layer has no q/k: the maps are never used
  if ((rc = make_map4(&mq, any_live ? a.q : a.v, a.B, any_live ? a.U : (Hkv ? Hkv : a.H), a.T, a.HD))) return rc;
  if ((rc = make_map4(&mk, any_live ? a.k : a.v, a.B, any_live ? (Hkv ? Hkv : a.U) : (Hkv ? Hkv : a.H), a.T, a.HD))) return rc;
  if ((rc = make_map4(&mv, a.v, a.B, Hkv ? Hkv : a.H, a.T, a.HD))) return rc;
  if ((rc = make_map4(&mo, a.out, a.B, a.H, a.T, a.HD))) return rc;
  FlashParams p;
  memset(&p, 0, sizeof(p));
  p.B = a.B; p.H = a.H; p.T = a.T; p.HKV = a.HKV; p.force_state = a.force_state;
  p.n_pairs = (a.T + 2 * FM - 1) / (2 * FM);
  p.scale_log2 = a.sm_scale * LOG2E_F;
  p.frozen = a.frozen; p.hidx = a.hidx; p.kvidx = a.kvidx;
  p.lse = reinterpret_cast<float*>(a.lse.ptr);
  for (int i = 0; i < 3; ++i) p.lse_s[i] = a.lse.stride[i];
  p.status = a.status;
  p.patt = a.patt.ptr;
  for (int i = 0; i < 3; ++i) p.patt_s[i] = a.patt.stride[i];
  p.patt_dtype = a.patt_dtype;
  p.pidx = a.pidx;
  p.alpha = a.alpha.ptr; p.rho = a.rho.ptr; p.z = a.z.ptr;
  for (int i = 0; i < 2; ++i) {
    p.alpha_s[i] = a.alpha.stride[i];
    p.rho_s[i] = a.rho.stride[i];
    p.z_s[i] = a.z.stride[i];
  }
  p.dec_dtype = a.dec_dtype;
  if (!(want & (1u << SAF_DENSE))) p.patt = nullptr;       // another launch serves these heads: their CTAs exit
  if (!(want & (1u << SAF_DECOMP))) p.alpha = nullptr;
  CUtensorMap mpat, mv64;
  memset(&mpat, 0, sizeof(mpat));
  memset(&mv64, 0, sizeof(mv64));
  {
    // the batch-shared pattern role: dense-stored bf16 patterns by TMA, decomposed patterns generated in
    // shared memory; the flash CTAs of those heads then exit
    const bool dense = p.patt && dense_pv_eligible(a);
    const bool decomp = p.alpha && dense_pv_decomp_eligible(a);
    if (dense || decomp) {
      CUtensorMap mo2;
      if ((rc = dense_pv_prepare(a, dense, decomp, &mpat, &mv64, &mo2, &p.dense))) return rc;
      p.dense_slots = (int)dense_pv_slots(p.dense);
      if (dense) p.patt = nullptr;
      if (decomp) p.alpha = nullptr;
    }
  }
  if (a.sd_alpha && a.sd_rho && (want & (1u << SAF_SINK_DECAY))) {
    p.has_scan = 1;
    ScanArgs& s = p.scan;
    s.in = a.v.ptr;
    s.out = a.out.ptr;
    for (int i = 0; i < 4; ++i) {
      s.si[i] = a.v.stride[i];
      s.so[i] = a.out.stride[i];
    }
    s.frozen = a.frozen; s.kvidx = a.kvidx; s.sd_alpha = a.sd_alpha; s.sd_rho = a.sd_rho;
    s.B = a.B; s.H = a.H; s.T = a.T; s.HD = a.HD; s.force_state = a.force_state; s.HKV = a.HKV;
    s.vec_ok = 1;   // tma_ok() already demands 16-byte aligned bases and strides
  }
  const int bh = a.B * a.H;
  // Persistent live-tile kernel: needs the caller's two-int queue scratch and the head states on the host (the
  // queue walks live heads only); calls whose frozen heads are produced by the softmax warps (fp32-stored
  // patterns and the like) keep the one-shot kernel, which has that role.
  bool persistent = a.sched && any_live && a.frozen_host && a.force_state < 0 && !p.patt && !p.alpha && a.U <= 64 &&
                    !getenv_off("SAF_B200_PERSISTENT");
  if (persistent) {
    int u = 0;
    for (int h = 0; h < a.H && persistent; ++h)
      if (a.frozen_host[h] == SAF_LIVE) {
        if (u < 64 && h < 256) p.live_head[u++] = (uint8_t)h;
        else persistent = false;
      }
    if (u != a.U || u == 0) persistent = false;
  }
  if (persistent) {
    p.sched = a.sched;
    p.U = a.U;
    p.n_items = a.B * a.U * p.n_pairs;
    p.lead = bh + p.dense_slots;
    static PerDeviceOnce smem_once_p;
    if ((rc = ensure_dyn_smem(flash_fwd_persistent_kernel<HD>, Cfg<HD>::SMEM_PERSIST, smem_once_p))) return rc;
    const int workers = std::min(device_sm_count(), p.n_items);
    const unsigned grid = (unsigned)(p.lead + workers);
    flash_fwd_persistent_kernel<HD><<<grid, FLASH_THREADS, Cfg<HD>::SMEM_PERSIST, st>>>(mq, mk, mv, mo, mpat, mv64, p);
    count_launch();
    return check_launch("flash_fwd_persistent_kernel");
  }
  static PerDeviceOnce smem_once;
  if ((rc = ensure_dyn_smem(flash_fwd_kernel<HD>, Cfg<HD>::SMEM_BYTES, smem_once))) return rc;
  const int groups = (bh + HEAD_GROUP - 1) / HEAD_GROUP;
  const unsigned grid = (unsigned)(bh + p.dense_slots + groups * HEAD_GROUP * p.n_pairs);
  flash_fwd_kernel<HD><<<grid, FLASH_THREADS, Cfg<HD>::SMEM_BYTES, st>>>(mq, mk, mv, mo, mpat, mv64, p);
  count_launch();
  return check_launch("flash_fwd_kernel");
}

}  // namespace

#ifdef SAF_FWD_TRACE
extern "C" int saf_debug_ftrace(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, g_ftrace, sizeof(g_ftrace));
}
#endif

int launch_flash_fwd_sm100(const SafMixedAttnArgs& a, uint32_t want, uint32_t* handled, cudaStream_t st) {
  *handled = 0;
  // head_dim 96 (the reference's 1B recipe, 16 heads x 96) rides the 128-column kernel: the tensor maps carry the
  // real width, so the TMA loads fill columns 96..127 of every Q, K and V tile with zeros (they add nothing to
  // Q K^T and give zero output columns) and the stores clip them; a quarter of the MMA work is padding.
  if (a.dtype != SAF_BF16 || (a.HD != 64 && a.HD != 96 && a.HD != 128) || a.rope) return SAF_ERR_UNSUPPORTED;
  if (a.sm_scale <= 0.f) return SAF_ERR_UNSUPPORTED;
  const bool q_ok = a.U > 0 && a.q.ptr && a.k.ptr;
  if (q_ok && (!tma_ok(a.q) || !tma_ok(a.k))) return SAF_ERR_UNSUPPORTED;
  if (!tma_ok(a.v) || !tma_ok(a.out)) return SAF_ERR_UNSUPPORTED;
  if (!saf_device_supported()) return SAF_ERR_UNSUPPORTED;
  // states this launch serves
  uint32_t can = 0;
  if (q_ok) can |= 1u << SAF_LIVE;
  if (a.patt.ptr) can |= 1u << SAF_DENSE;
  if (a.alpha.ptr && a.rho.ptr && a.z.ptr) can |= 1u << SAF_DECOMP;
  if (a.sd_alpha && a.sd_rho) can |= 1u << SAF_SINK_DECAY;   // (the scan clips its 64-column slices to the real width)
  can &= want;
  uint32_t present = can;
  if (a.force_state >= 0) present = 1u << a.force_state;
  else if (a.frozen_host) {
    present = 0;
    for (int h = 0; h < a.H; ++h) present |= 1u << a.frozen_host[h];
  }
  if (!(present & can)) return SAF_ERR_UNSUPPORTED;
  const int rc = (a.HD == 64) ? launch_typed<64>(a, can, st) : launch_typed<128>(a, can, st);
  if (rc == SAF_OK) *handled = can;
  return rc;
}

}  // namespace saf
