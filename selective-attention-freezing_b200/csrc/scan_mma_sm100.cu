// Structured frozen heads (sink + geometric decay) launched alone, on the tensor core.
//
//   y_i = a v_0 + (1-a) s_i / Z_i,   s_i = r s_{i-1} + v_i
//
// Inside a block of 128 consecutive rows the recurrence is a product with a fixed lower-triangular Toeplitz
// matrix that depends on the head's decay only:  s_loc = L V,  L[i][j] = r^(i-j) (j <= i),  and the state the
// block inherits enters as  s_i = s_loc_i + r^(i_loc+1) carry.  So the scan of a long sequence becomes a stream of
// 128 x 128 x 64 tcgen05 products fed by a TMA ring, and the only sequential piece left is a 64-float carry
// handed from one block's epilogue to the next.  The CUDA-core scan this replaces (csrc/scan_body.cuh) spends
// about 800 instructions per thread per 256-row block and is bound by instruction issue at 0.20 of the HBM
// copy rate; here a block costs 16 MMAs and ~300 epilogue instructions per row (0.5 of the copy rate at B = 32).
// The reference has no counterpart: it holds such a pattern as a dense T x T buffer and multiplies it
// (kernel/fused_attn.py:125-143, kernel/frozen_attn.py:51-89).
//
// L is split into a bf16 head and a bf16 remainder (two MMAs accumulate into the same fp32 TMEM tile), so the
// product is as exact as the fp32 register scan to ~2^-17; V is bf16 as stored.  Both parts live in TMEM (128 columns,
// written once per CTA), so the MMAs take their A operand from TMEM and shared memory holds nothing but V tiles and
// output staging.
//
// Launch structure (forward, bf16, head_dim a multiple of 64):
//   pass 1  sink_decay_state_kernel     every chunk: its end state from a zero carry -- a weighted column sum,
//                                       plain 16-byte loads, many CTAs per SM                (reads V once)
//   pass 2  sink_decay_carry_kernel     (csrc/scan_body.cuh) carries chained over the chunks of a head
//   pass 3  sink_decay_apply_mma_kernel every chunk: blocks of 128 rows through the tensor core  (V again, writes Y)
// A chunk hands its 64 fp32 state words to the next pass in the first rows of its own output slice, which pass 3
// overwrites only after it has read them (the same stash as the CUDA-core passes): no scratch memory.
// One chunk per head (enough heads to fill the GPU): pass 3 alone with a zero carry, V read once.
//
//   pass 3 CTA, 320 threads:  warp 0 TMA producer (V tiles 128 rows x 64 columns, 11-stage ring = 176 KB in flight)
//                             warp 1 MMA issuer (4 TMEM accumulators of 64 columns, A = the Toeplitz operand in TMEM)
//                             warps 2-5 / 6-9 epilogue of the even / odd blocks, thread = row: TMEM -> + carry (in
//                             place) -> normaliser / sink term -> bf16 -> swizzled staging -> TMA store.  The thread
//                             of row 127 publishes the block's end state before anything else, so the serial chain
//                             from block to block is 64 fused multiply-adds long and the two warpgroups overlap
//                             otherwise.
// Every wait is bounded.
#include <algorithm>

#include "saf_internal.h"
#include "scan_body.cuh"
#include "sm100_prims.cuh"

namespace saf {
namespace {

constexpr int MB = 128;                 // rows per block
constexpr int MS_STAGES = 11;
constexpr int MS_TILE = MB * 64 * 2;    // 16 KB: one V tile, one output tile
constexpr int MS_THREADS = 320;          // TMA warp, MMA warp, two epilogue warpgroups
constexpr int MS_ACC = 4;               // TMEM accumulators
constexpr int MS_OUT = 2;               // staging tiles: one per epilogue warpgroup
constexpr int MS_TL = MS_ACC * 64;      // TMEM column of the Toeplitz operand: bf16 head (64 columns), remainder (64)

struct MsBars {
  uint64_t full[MS_STAGES], empty[MS_STAGES], acc_full[MS_ACC], acc_empty[MS_ACC], carry_ready[4], l_ready;
  uint32_t tmem_base;
  alignas(16) float carry[4][64];      // carry[n & 3]: the state block n inherits
  alignas(16) float av0[64];
};
constexpr int MS_SMEM = 1024 + (MS_STAGES + MS_OUT) * MS_TILE + 2048;
static_assert(sizeof(MsBars) <= 2048 && MS_SMEM <= 227 * 1024, "shared memory limit");

#ifdef SAF_SCAN_TRACE
__device__ long long g_strace[12][64];
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

// ---- pass 1: end state of every chunk from a zero carry ------------------------------------------------
// state[c] = sum_{i in chunk} r^(last - i) v[i][c].  Thread (rg, cg): rows last - rg - 32 k, 8 columns.
__global__ void __launch_bounds__(256, 4) sink_decay_state_kernel(const __grid_constant__ ScanArgs a, int chunk) {
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
  const int state = a.force_state >= 0 ? a.force_state : a.frozen[h];
  if (state != SAF_SINK_DECAY || blockIdx.y + 1 == gridDim.y) return;      // nothing follows the last chunk
  const int col0 = blockIdx.z * SCAN_COLS;
  const int p_lo = blockIdx.y * chunk, p_hi = min(a.T, p_lo + chunk);
  const int tid = threadIdx.x, cg = tid & 7, rg = tid >> 3;
  const float r = a.sd_rho[h];
  const float r2 = r * r, r4 = r2 * r2, r8 = r4 * r4, r16 = r8 * r8, r32 = r16 * r16;
  const int hin = a.HKV > 0 ? (a.kvidx ? a.kvidx[h] : 0) : h;
  const __nv_bfloat16* ib = reinterpret_cast<const __nv_bfloat16*>(a.in) + (int64_t)b * a.si[0] + (int64_t)hin * a.si[1] +
                            (int64_t)(col0 + cg * 8);
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  float wgt = 1.f;
  for (int i = 0; i < rg; ++i) wgt *= r;               // r^rg
  // eight rows in flight per thread: rows last - rg - 32 u, then 256 rows further up
  for (int row = p_hi - 1 - rg; row >= p_lo; row -= 256) {
    uint4 raw[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = row - 32 * u;
      raw[u] = (i >= p_lo) ? *reinterpret_cast<const uint4*>(ib + (int64_t)i * a.si[2]) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] = fmaf(wgt, __uint_as_float(w4[e] << 16), acc[2 * e]);
        acc[2 * e + 1] = fmaf(wgt, __uint_as_float(w4[e] & 0xffff0000u), acc[2 * e + 1]);
      }
      wgt *= r32;
    }
  }
  __shared__ float part[32][SCAN_COLS + 1];
#pragma unroll
  for (int c = 0; c < 8; ++c) part[rg][cg * 8 + c] = acc[c];
  __syncthreads();
  if (tid < SCAN_COLS) {
    float s = 0.f;
#pragma unroll 8
    for (int k = 0; k < 32; ++k) s += part[k][tid];
    __nv_bfloat16* ob0 = reinterpret_cast<__nv_bfloat16*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)col0;
    *scan_stash<__nv_bfloat16>(ob0, a.so[2], p_lo, tid) = s;
  }
}

// ---- pass 3: the chunk's rows through the tensor core -----------------------------------------------------
__global__ void __launch_bounds__(MS_THREADS, 1)
sink_decay_apply_mma_kernel(const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapY,
                            const __grid_constant__ MsParams p) {
  const ScanArgs& a = p.a;
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
  const int state = a.force_state >= 0 ? a.force_state : a.frozen[h];
  if (state != SAF_SINK_DECAY) return;
  const int col0 = blockIdx.z * SCAN_COLS;
  const int p_lo = blockIdx.y * p.chunk, p_hi = min(a.T, p_lo + p.chunk);
  const int n_blocks = (p_hi - p_lo + MB - 1) / MB;
  const int hin = a.HKV > 0 ? (a.kvidx ? a.kvidx[h] : 0) : h;
#ifdef SAF_SCAN_TRACE
  const bool trace_on = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#endif

  extern __shared__ uint8_t ms_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)ms_smem_raw + 1023) & ~(uintptr_t)1023);
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
        tma_load_4d(sV + s * MS_TILE, &mapV, &bars->full[s], col0, p_lo + n * MB, hin, b);
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
  } else {
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
    if (wg == 0 && et < 64) {
      const __nv_bfloat16* ob0 = reinterpret_cast<const __nv_bfloat16*>(a.out) + (int64_t)b * a.so[0] + (int64_t)h * a.so[1] + (int64_t)col0;
      if (p.use_stash) carry_in = *scan_stash<__nv_bfloat16>(const_cast<__nv_bfloat16*>(ob0), a.so[2], p_lo, et);
      const __nv_bfloat16* v0 = reinterpret_cast<const __nv_bfloat16*>(a.in) + (int64_t)b * a.si[0] + (int64_t)hin * a.si[1] + (int64_t)(col0 + et);
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
    if (wg == 0 && et < 64) {
      bars->carry[0][et] = carry_in;
      bars->av0[et] = alpha * v_first;
    }
    mbar_arrive(&bars->l_ready);
    named_bar_sync(3, 256);                                 // carry[0] and av0 are in place for both warpgroups
    if (wg == 0 && et == 0) mbar_arrive(&bars->carry_ready[0]);
    float pw = r;                                           // r^(lrow + 1)
    for (int i = 0; i < lrow; ++i) pw *= r;
    const uint32_t tsrc = tlane;
    const float4* a4 = reinterpret_cast<const float4*>(bars->av0);
    for (int n = wg; n < n_blocks; n += 2) {
      const int buf = n % MS_ACC, slot = n & 3;
      // the row's weight (1 - a) / Z_i waits for nothing
      const float w = (1.f - alpha) * inv_z(r, log_r, p_lo + n * MB + lrow + 1);
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
#pragma unroll
          for (int q = 0; q < 8; ++q) n4[q] = make_uint4(s0[q * 4], s0[q * 4 + 1], s0[q * 4 + 2], s0[q * 4 + 3]);
#pragma unroll
          for (int q = 0; q < 8; ++q) n4[8 + q] = make_uint4(s1[q * 4], s1[q * 4 + 1], s1[q * 4 + 2], s1[q * 4 + 3]);
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
        tma_store_4d(&mapY, sY + wg * MS_TILE, col0, p_lo + n * MB, h, b);
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

}  // namespace

#ifdef SAF_SCAN_TRACE
extern "C" int saf_debug_strace(long long* host) { return (int)cudaMemcpyFromSymbol(host, g_strace, sizeof(g_strace)); }
#endif

// The tensor-core forward scan of the structured heads of a call; SAF_ERR_UNSUPPORTED when the call does not
// qualify (the CUDA-core scan then takes it).
int launch_scan_fwd_mma(const SafMixedAttnArgs& a, cudaStream_t st) {
  if (a.dtype != SAF_BF16 || a.HD % 64 || a.T < 1024 || !a.sd_alpha || !a.sd_rho) return SAF_ERR_UNSUPPORTED;
  if (!tma_rows_ok(a.v) || !tma_rows_ok(a.out) || !saf_device_supported()) return SAF_ERR_UNSUPPORTED;
  const char* off = getenv("SAF_B200_SCAN_MMA");
  if (off && off[0] == '0' && off[1] == 0) return SAF_ERR_UNSUPPORTED;
  MsParams p;
  memset(&p, 0, sizeof(p));
  ScanArgs& s = p.a;
  s.in = a.v.ptr;
  s.out = a.out.ptr;
  for (int i = 0; i < 4; ++i) {
    s.si[i] = a.v.stride[i];
    s.so[i] = a.out.stride[i];
  }
  s.frozen = a.frozen; s.kvidx = a.kvidx; s.sd_alpha = a.sd_alpha; s.sd_rho = a.sd_rho;
  s.B = a.B; s.H = a.H; s.T = a.T; s.HD = a.HD; s.force_state = a.force_state; s.HKV = a.HKV;
  s.vec_ok = 1;
  p.status = a.status;
  int heads = a.H;
  if (a.frozen_host && a.force_state < 0) {
    heads = 0;
    for (int h = 0; h < a.H; ++h) heads += a.frozen_host[h] == SAF_SINK_DECAY;
    if (heads == 0) return SAF_OK;
  }
  // Chunks: one CTA of pass 3 per SM at a time, every CTA costs its Toeplitz set-up (about 8 blocks' worth) plus its
  // blocks, and the launch runs in whole waves of CTAs: take the chunk count with the least modelled time.  One
  // chunk per head also saves passes 1 and 2 (half of the remaining traffic), which the model credits as 1.5x.
  // At most 64 chunks (what the carry pass takes), whole 128-row blocks; the last chunk must hold its 64-word
  // stash (2 rows of a 64-column bf16 slice).
  const int slices = a.HD / SCAN_COLS;
  const int n_seq = std::max(1, a.B * heads * slices);
  const int sms = device_sm_count(), t_blocks = (a.T + MB - 1) / MB;
  int n_chunks = 1, chunk = t_blocks * MB;
  {
    double best = 1e30;
    for (int n = 1; n <= std::min(64, t_blocks); ++n) {
      const int cb = (t_blocks + n - 1) / n, nn = (t_blocks + cb - 1) / cb;      // blocks per chunk, chunks that result
      if (nn != n) continue;
      if (nn > 1 && a.T - (nn - 1) * cb * MB < 2) continue;
      const double waves = (double)(((int64_t)n_seq * nn + sms - 1) / sms);
      const double cost = waves * (8.0 + cb) * (nn > 1 ? 1.5 : 1.0);
      if (cost < best) {
        best = cost;
        n_chunks = nn;
        chunk = cb * MB;
      }
    }
  }
  p.chunk = chunk;
  p.use_stash = n_chunks > 1;
  const int Hv = a.HKV > 0 ? a.HKV : a.H;
  CUtensorMap mv, my;
  int rc;
  if ((rc = make_row_tile_map_bf16(&mv, a.v, a.B, Hv, a.T, a.HD))) return rc;
  if ((rc = make_row_tile_map_bf16(&my, a.out, a.B, a.H, a.T, a.HD))) return rc;
  const dim3 grid(a.B * a.H, n_chunks, slices);
  if (n_chunks > 1) {
    sink_decay_state_kernel<<<grid, 256, 0, st>>>(s, chunk);
    count_launch();
    if ((rc = check_launch("sink_decay_state_kernel"))) return rc;
    sink_decay_carry_kernel<__nv_bfloat16><<<dim3(a.B * a.H, slices), SCAN_COLS, 0, st>>>(s, chunk, n_chunks);
    count_launch();
    if ((rc = check_launch("sink_decay_carry_kernel"))) return rc;
  }
  static PerDeviceOnce smem_once;
  if ((rc = ensure_dyn_smem(sink_decay_apply_mma_kernel, MS_SMEM, smem_once))) return rc;
  sink_decay_apply_mma_kernel<<<grid, MS_THREADS, MS_SMEM, st>>>(mv, my, p);
  count_launch();
  return check_launch("sink_decay_apply_mma_kernel");
}

}  // namespace saf
