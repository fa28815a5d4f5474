// Structured frozen heads (sink + geometric decay) as a causal scan.
//
// The pattern P[i,j] = a [j=0] + (1-a) r^(i-j) / Z_i  (j <= i), Z_i = sum_{k<=i} r^k,
// gives   y_i = a v_0 + (1-a) s_i / Z_i ,  s_i = r s_{i-1} + v_i
// so P @ V costs one read of V and one write of Y (HBM bound) instead of a
// T x T tensor-core product.  The reference holds such a pattern only as a dense
// state-1 buffer (kernel/fused_attn.py:125-143, kernel/frozen_attn.py:51-89);
// its closest O(T) relative is the uniform cumulative-sum head
// (supplement/attention.py:10-27).
//
// One CTA owns one (batch, head, 64-column slice) and walks T in blocks of 256
// rows.  Inside a block: each thread scans 8 consecutive rows of 8 columns in
// registers (16-byte loads, one full 128-byte line per 8 lanes), carries are
// combined across the 4 row groups of a warp with shuffles and across the 8
// warps through shared memory.  The backward (dV = P^T dY) is the same scan run
// over reversed rows on (1-a) dY_i / Z_i, plus a * sum_i dY_i added to row 0.
#include <algorithm>

#include "saf_internal.h"
#include "scan_body.cuh"

namespace saf {
namespace {

template <typename T>
int scan_typed(const ScanArgs& s, bool bwd, cudaStream_t st) {
  dim3 grid(s.B * s.H, (s.HD + SCAN_COLS - 1) / SCAN_COLS);
  if (bwd) sink_decay_scan_kernel<T, true><<<grid, SCAN_NT, 0, st>>>(s);
  else sink_decay_scan_kernel<T, false><<<grid, SCAN_NT, 0, st>>>(s);
  count_launch();
  return check_launch("sink_decay_scan_kernel");
}

bool vec_ok(const void* p, const int64_t* s, int esize) {
  // 16-byte vector access: unit column stride, every other stride and the base 16-byte aligned
  if (s[3] != 1) return false;
  const int64_t per = 16 / esize;
  if (((uintptr_t)p) % 16) return false;
  for (int i = 0; i < 3; ++i)
    if (s[i] % per) return false;
  return true;
}

// chunked forward scan (three launches); returns false when the shape does not qualify
template <typename T>
bool scan_chunked(const ScanArgs& s, cudaStream_t st, int* rc) {
  constexpr int STASH_ROWS = 256 / (SCAN_COLS * (int)sizeof(T));   // rows of an output slice that hold 64 fp32 words
  if (!s.vec_ok || s.HD % SCAN_COLS || s.T < 4096) return false;
  // Chunks are as long as the machine allows: a chunk CTA prefetches its next 256-row block while it scans the
  // current one, so long chunks keep loads in flight, but the launch still needs about three waves of CTAs (two
  // per SM) to fill the GPU.  At most 64 chunks (what the carry pass takes), in whole 256-row block steps.
  const int heads = s.force_state >= 0 ? s.H : (s.n_active > 0 ? s.n_active : s.H);
  const int n_seq = std::max(1, s.B * heads * (s.HD / SCAN_COLS));
  const int want = std::max(1, std::min(64, (6 * device_sm_count() + n_seq - 1) / n_seq));
  int chunk = ((s.T + want - 1) / want + SCAN_ROWS - 1) / SCAN_ROWS * SCAN_ROWS;
  const int n_chunks = (s.T + chunk - 1) / chunk;
  if (n_chunks < 2) return false;                                   // one chunk: the one-pass kernel does it
  if (s.T - (n_chunks - 1) * chunk < STASH_ROWS) return false;     // the last chunk must hold its stash
  dim3 grid(s.B * s.H, n_chunks, s.HD / SCAN_COLS);
  sink_decay_chunk_kernel<T, 1><<<grid, SCAN_NT, 0, st>>>(s, chunk);
  count_launch();
  if ((*rc = check_launch("sink_decay_chunk_kernel<totals>"))) return true;
  sink_decay_carry_kernel<T><<<dim3(s.B * s.H, s.HD / SCAN_COLS), SCAN_COLS, 0, st>>>(s, chunk, n_chunks);
  count_launch();
  if ((*rc = check_launch("sink_decay_carry_kernel"))) return true;
  sink_decay_chunk_kernel<T, 2><<<grid, SCAN_NT, 0, st>>>(s, chunk);
  count_launch();
  *rc = check_launch("sink_decay_chunk_kernel<apply>");
  return true;
}

int scan_dispatch(const ScanArgs& s, int dtype, bool bwd, cudaStream_t st) {
  if (s.T == 0 || s.B == 0 || s.H == 0) return SAF_OK;
  if (!bwd) {
    int rc = SAF_OK;
    if (dtype == SAF_BF16 && scan_chunked<__nv_bfloat16>(s, st, &rc)) return rc;
    if (dtype == SAF_F32 && scan_chunked<float>(s, st, &rc)) return rc;
  }
  switch (dtype) {
    case SAF_F32: return scan_typed<float>(s, bwd, st);
    case SAF_BF16: return scan_typed<__nv_bfloat16>(s, bwd, st);
    case SAF_F16: return scan_typed<__half>(s, bwd, st);
  }
  return fail(SAF_ERR_INVALID, "unknown dtype %d", dtype);
}

}  // namespace

int launch_scan_fwd(const SafMixedAttnArgs& a, cudaStream_t st) {
  if (!a.sd_alpha || !a.sd_rho) return fail(SAF_ERR_INVALID, "sink-decay heads need sd_alpha and sd_rho");
  {   // long bf16 sequences: blocks of 128 rows as Toeplitz products on the tensor core
    const int rc = launch_scan_fwd_mma(a, st);
    if (rc != SAF_ERR_UNSUPPORTED) return rc;
  }
  ScanArgs s{};
  s.in = a.v.ptr;
  s.out = a.out.ptr;
  for (int i = 0; i < 4; ++i) {
    s.si[i] = a.v.stride[i];
    s.so[i] = a.out.stride[i];
  }
  s.frozen = a.frozen;
  s.kvidx = a.kvidx;
  s.sd_alpha = a.sd_alpha;
  s.sd_rho = a.sd_rho;
  s.B = a.B; s.H = a.H; s.T = a.T; s.HD = a.HD; s.force_state = a.force_state; s.HKV = a.HKV;
  const int es = dtype_size(a.dtype);
  s.vec_ok = vec_ok(a.v.ptr, a.v.stride, es) && vec_ok(a.out.ptr, a.out.stride, es);
  if (a.frozen_host && a.force_state < 0)
    for (int h = 0; h < a.H; ++h) s.n_active += a.frozen_host[h] == SAF_SINK_DECAY;
  return scan_dispatch(s, a.dtype, false, st);
}

int launch_scan_bwd(const SafMixedAttnBwdArgs& g, cudaStream_t st) {
  const SafMixedAttnArgs& a = g.fwd;
  if (!a.sd_alpha || !a.sd_rho) return fail(SAF_ERR_INVALID, "sink-decay heads need sd_alpha and sd_rho");
  ScanArgs s{};
  s.in = g.dout.ptr;
  s.out = g.dv.ptr;
  for (int i = 0; i < 4; ++i) {
    s.si[i] = g.dout.stride[i];
    s.so[i] = g.dv.stride[i];
  }
  s.frozen = a.frozen;
  s.kvidx = nullptr;
  s.sd_alpha = a.sd_alpha;
  s.sd_rho = a.sd_rho;
  s.B = a.B; s.H = a.H; s.T = a.T; s.HD = a.HD; s.force_state = a.force_state; s.HKV = 0;
  const int es = dtype_size(a.dtype);
  s.vec_ok = vec_ok(g.dout.ptr, g.dout.stride, es) && vec_ok(g.dv.ptr, g.dv.stride, es);
  return scan_dispatch(s, a.dtype, true, st);
}

}  // namespace saf
