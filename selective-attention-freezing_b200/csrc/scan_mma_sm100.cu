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
#include "scan_mma_body.cuh"

namespace saf {
namespace {

constexpr int MS_STAGES = MS_MAX_STAGES;
constexpr int MS_SMEM = ms_smem_bytes(MS_STAGES);

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

// ---- pass 3: the chunk's rows through the tensor core (body in scan_mma_body.cuh) --------------------------
__global__ void __launch_bounds__(MS_THREADS, 1)
sink_decay_apply_mma_kernel(const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapY,
                            const __grid_constant__ MsParams p) {
  const ScanArgs& a = p.a;
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
  const int state = a.force_state >= 0 ? a.force_state : a.frozen[h];
  if (state != SAF_SINK_DECAY) return;
  extern __shared__ uint8_t ms_smem_raw[];
  sink_decay_apply_mma_cta<MS_STAGES>(mapV, mapY, p, b, h, blockIdx.y, blockIdx.z, 1, ms_smem_raw);
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
