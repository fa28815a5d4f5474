// extern "C" entry points: argument validation, dispatch, error text.
#include <stdarg.h>
#include <stddef.h>
#include <string.h>

#include <atomic>

#include "saf_internal.h"

namespace saf {

static thread_local char g_err[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(SAF_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return SAF_OK;
}

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return dev;
}

int device_sm_count() {
  static std::atomic<int> cache[SAF_MAX_DEVICES];
  const int dev = current_device();
  const bool slot = dev >= 0 && dev < SAF_MAX_DEVICES;
  int n = slot ? cache[dev].load(std::memory_order_relaxed) : 0;
  if (n > 0) return n;
  if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return 148;
  }
  if (slot) cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

TensorMapEncodeFn tensor_map_encoder() {
  // the driver entry point is a property of the process, not of a device; a failed lookup is retried
  static std::atomic<TensorMapEncodeFn> cached{nullptr};
  TensorMapEncodeFn fn = cached.load(std::memory_order_acquire);
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess) {
    fn = (TensorMapEncodeFn)p;
    cached.store(fn, std::memory_order_release);
  }
  cudaGetLastError();
  return fn;
}

int make_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box, bool l2_256) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return fail(SAF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i > 0) s[i - 1] = strides_bytes[i];
  }
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   l2_256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SAF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SAF_OK;
}

bool tma_rows_ok(const SafTensor& t) {
  if (!t.ptr || ((uintptr_t)t.ptr & 15) || t.stride[3] != 1) return false;
  for (int i = 0; i < 3; ++i)
    if (t.stride[i] % 8 || t.stride[i] <= 0) return false;
  return true;
}

int make_row_tile_map_bf16(CUtensorMap* m, const SafTensor& t, int B, int Hn, int T, int HD) {
  uint64_t dims[4] = {(uint64_t)HD, (uint64_t)T, (uint64_t)Hn, (uint64_t)B};
  uint64_t strides[4] = {0, (uint64_t)t.stride[2] * 2, (uint64_t)t.stride[1] * 2, (uint64_t)t.stride[0] * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tensor_map_bf16(m, t.ptr, 4, dims, strides, box, true);
}

namespace {

bool valid_dtype(int d) { return d == SAF_F32 || d == SAF_BF16 || d == SAF_F16; }

int validate_mixed(const SafMixedAttnArgs* a) {
  if (!a) return fail(SAF_ERR_INVALID, "null argument struct");
  if (a->struct_size != (int32_t)sizeof(SafMixedAttnArgs))
    return fail(SAF_ERR_INVALID, "SafMixedAttnArgs size mismatch: caller %d, library %d", a->struct_size,
                (int)sizeof(SafMixedAttnArgs));
  if (!valid_dtype(a->dtype)) return fail(SAF_ERR_INVALID, "unknown dtype %d", a->dtype);
  if (a->B < 0 || a->H < 0 || a->U < 0 || a->T < 0 || a->HD <= 0)
    return fail(SAF_ERR_INVALID, "negative dimension (B=%d H=%d U=%d T=%d HD=%d)", a->B, a->H, a->U, a->T, a->HD);
  if (a->HD > 128) return fail(SAF_ERR_UNSUPPORTED, "head_dim %d > 128", a->HD);
  if (a->force_state < -1 || a->force_state > 3) return fail(SAF_ERR_INVALID, "force_state %d", a->force_state);
  if (a->B == 0 || a->H == 0 || a->T == 0) return SAF_OK;
  if (!a->v.ptr || !a->out.ptr) return fail(SAF_ERR_INVALID, "v and out must be non-null");
  if (a->force_state < 0 && !a->frozen) return fail(SAF_ERR_INVALID, "frozen must be non-null");
  if (a->v.stride[3] != 1 || a->out.stride[3] != 1)
    return fail(SAF_ERR_INVALID, "v and out need unit stride on head_dim");
  const bool may_live = a->force_state < 0 || a->force_state == SAF_LIVE;
  if (may_live && a->U > 0) {
    if (!a->q.ptr || !a->k.ptr) return fail(SAF_ERR_INVALID, "q and k must be non-null when U > 0");
    if (a->q.stride[3] != 1 || a->k.stride[3] != 1) return fail(SAF_ERR_INVALID, "q and k need unit stride on head_dim");
  }
  if (a->HKV < 0) return fail(SAF_ERR_INVALID, "HKV %d", a->HKV);
  if (a->HKV > 0 && !a->kvidx) return fail(SAF_ERR_INVALID, "GQA (HKV>0) needs kvidx");
  if (a->patt.ptr) {
    if (!valid_dtype(a->patt_dtype)) return fail(SAF_ERR_INVALID, "unknown patt dtype %d", a->patt_dtype);
    if (a->S < a->T) return fail(SAF_ERR_INVALID, "patt must have shape (P, S, S) with S >= T (S=%d, T=%d)", a->S, a->T);
  }
  if (a->alpha.ptr) {
    if (!a->rho.ptr || !a->z.ptr) return fail(SAF_ERR_INVALID, "alpha, rho and z come together");
    if (!valid_dtype(a->dec_dtype)) return fail(SAF_ERR_INVALID, "unknown decomposed dtype %d", a->dec_dtype);
    if (a->SD < a->T) return fail(SAF_ERR_INVALID, "decomposed buffers must have shape (H, S) with S >= T");
  }
  if (a->rope) {
    if (!a->rope_cos || !a->rope_sin) return fail(SAF_ERR_INVALID, "rope=1 needs rope_cos and rope_sin");
    if (a->HD % 2) return fail(SAF_ERR_INVALID, "RoPE requires an even head dimension");
  }
  if (a->frozen_host && a->force_state < 0) {
    for (int h = 0; h < a->H; ++h) {
      const int s = a->frozen_host[h];
      if (s < 0 || s > 3) return fail(SAF_ERR_INVALID, "frozen[%d] = %d is not a head state", h, s);
      if (s == SAF_DENSE && !a->patt.ptr) return fail(SAF_ERR_INVALID, "dense-frozen heads require patt");
      if (s == SAF_DECOMP && !a->alpha.ptr) return fail(SAF_ERR_INVALID, "decomposed-frozen heads require alpha/rho/z");
      if (s == SAF_SINK_DECAY && (!a->sd_alpha || !a->sd_rho))
        return fail(SAF_ERR_INVALID, "sink-decay heads require sd_alpha/sd_rho");
      if (s == SAF_LIVE && a->U == 0) return fail(SAF_ERR_INVALID, "live head %d but q/k hold no heads", h);
    }
  }
  return SAF_OK;
}

// which head states can occur, from the host hint (all four when unknown)
uint32_t possible_states(const SafMixedAttnArgs& a) {
  if (a.force_state >= 0) return 1u << a.force_state;
  if (!a.frozen_host) {
    uint32_t m = 0;
    if (a.U > 0) m |= 1u << SAF_LIVE;
    if (a.patt.ptr) m |= 1u << SAF_DENSE;
    if (a.alpha.ptr) m |= 1u << SAF_DECOMP;
    if (a.sd_alpha) m |= 1u << SAF_SINK_DECAY;
    return m;
  }
  uint32_t m = 0;
  for (int h = 0; h < a.H; ++h) m |= 1u << a.frozen_host[h];
  return m;
}

}  // namespace

int validate_mixed_args(const SafMixedAttnArgs* a) { return validate_mixed(a); }
uint32_t mixed_possible_states(const SafMixedAttnArgs& a) { return possible_states(a); }

}  // namespace saf

using namespace saf;

extern "C" {

int saf_abi_version(void) { return SAF_ABI_VERSION; }

int saf_last_error(char* buf, size_t n) {
  const size_t len = strlen(g_err);
  if (buf && n) {
    const size_t c = len < n - 1 ? len : n - 1;
    memcpy(buf, g_err, c);
    buf[c] = 0;
  }
  return (int)len;
}

int64_t saf_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int saf_device_supported(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

/* Host-only self-check of the per-device bookkeeping (no CUDA call): every device ordinal gets its own
 * "first time" exactly once, ordinals do not disturb one another, a forgotten ordinal is first again, and
 * ordinals outside the table always count as first.  Returns 0 when all of that holds, else the failing step. */
int saf_selftest_per_device_once(void) {
  PerDeviceOnce once{};
  for (int d = 0; d < SAF_MAX_DEVICES; ++d)
    if (!once.first(d)) return 1;
  for (int d = 0; d < SAF_MAX_DEVICES; ++d)
    if (once.first(d)) return 2;
  once.forget(3);
  if (!once.first(3)) return 3;
  if (once.first(3) || once.first(2) || once.first(4)) return 4;
  if (!once.first(-1) || !once.first(-1) || !once.first(SAF_MAX_DEVICES) || !once.first(SAF_MAX_DEVICES)) return 5;
  return 0;
}

int saf_mixed_attn_fwd(const SafMixedAttnArgs* args, void* stream) {
  int rc = validate_mixed(args);
  if (rc) return rc;
  const SafMixedAttnArgs& a = *args;
  if (a.B == 0 || a.H == 0 || a.T == 0) return SAF_OK;
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t todo = possible_states(a);
  // tensor-core path first; it reports which states it covered
  if (todo == (1u << SAF_SINK_DECAY)) return launch_scan_fwd(a, st);   // scan only: the chunk-parallel scan
  uint32_t handled = 0;
  rc = launch_flash_fwd_sm100(a, todo, &handled, st);
  if (rc == SAF_OK) todo &= ~handled;
  else if (rc != SAF_ERR_UNSUPPORTED) return rc;
  if (todo & (1u << SAF_DENSE)) {   // the mixed launch did not take the call: dense heads on their own
    rc = launch_dense_pv_sm100(a, &handled, st);
    if (rc == SAF_OK) todo &= ~handled;
    else if (rc != SAF_ERR_UNSUPPORTED) return rc;
  }
  if (todo & (1u << SAF_SINK_DECAY)) {
    if ((rc = launch_scan_fwd(a, st))) return rc;
    todo &= ~(1u << SAF_SINK_DECAY);
  }
  if (todo) {
    if ((rc = launch_generic_fwd(a, todo, st))) return rc;
  }
  return SAF_OK;
}

int saf_mixed_attn_bwd(const SafMixedAttnBwdArgs* args, void* stream) {
  if (!args) return fail(SAF_ERR_INVALID, "null argument struct");
  if (args->struct_size != (int32_t)sizeof(SafMixedAttnBwdArgs))
    return fail(SAF_ERR_INVALID, "SafMixedAttnBwdArgs size mismatch: caller %d, library %d", args->struct_size,
                (int)sizeof(SafMixedAttnBwdArgs));
  int rc = validate_mixed(&args->fwd);
  if (rc) return rc;
  const SafMixedAttnArgs& a = args->fwd;
  if (a.B == 0 || a.H == 0 || a.T == 0) return SAF_OK;
  if (a.HKV > 0) return fail(SAF_ERR_UNSUPPORTED, "backward with kvidx (GQA) is not implemented");
  if (!args->dout.ptr || !args->dv.ptr) return fail(SAF_ERR_INVALID, "dout and dv must be non-null");
  if (args->dout.stride[3] != 1 || args->dv.stride[3] != 1)
    return fail(SAF_ERR_INVALID, "dout and dv need unit stride on head_dim");
  uint32_t todo = possible_states(a);
  if (todo & 1u) {
    if (!args->dq.ptr || !args->dk.ptr || !args->delta.ptr || !a.lse.ptr)
      return fail(SAF_ERR_INVALID, "live heads need dq, dk, delta and lse");
  }
  cudaStream_t st = (cudaStream_t)stream;
  {
    // tensor-core path (live heads, and frozen heads as roles of the same launch); it reports what it covered
    uint32_t handled = 0;
    rc = launch_flash_bwd_sm100(*args, &handled, st);
    if (rc == SAF_OK) todo &= ~handled;
    else if (rc != SAF_ERR_UNSUPPORTED) return rc;
  }
  if (todo & (1u << SAF_SINK_DECAY)) {
    if ((rc = launch_scan_bwd(*args, st))) return rc;
    todo &= ~(1u << SAF_SINK_DECAY);
  }
  if (todo) {
    if ((rc = launch_generic_bwd(*args, todo, st))) return rc;
  }
  return SAF_OK;
}

static int frozen_pv_common(const SafFrozenPvArgs* p, void* stream, bool bwd) {
  if (!p) return fail(SAF_ERR_INVALID, "null argument struct");
  if (p->struct_size != (int32_t)sizeof(SafFrozenPvArgs))
    return fail(SAF_ERR_INVALID, "SafFrozenPvArgs size mismatch: caller %d, library %d", p->struct_size,
                (int)sizeof(SafFrozenPvArgs));
  const bool structured = p->sd_alpha && p->sd_rho;
  SafMixedAttnArgs a;
  memset(&a, 0, sizeof(a));
  a.struct_size = (int32_t)sizeof(a);
  a.dtype = p->dtype;
  a.B = p->B; a.H = p->NF; a.U = 0; a.T = p->T; a.HD = p->HD;
  a.S = p->S;
  a.patt_dtype = p->patt_dtype;
  a.force_state = structured ? SAF_SINK_DECAY : SAF_DENSE;
  a.sm_scale = 1.f;
  a.patt = p->patt;
  a.pidx = p->fz_idx;
  a.sd_alpha = p->sd_alpha;
  a.sd_rho = p->sd_rho;
  a.status = p->status;
  if (!structured) {
    if (!p->patt.ptr) return fail(SAF_ERR_INVALID, "patt must be non-null");
    if (!p->fz_idx) return fail(SAF_ERR_INVALID, "fz_idx must be non-null");
  }
  if (!bwd) {
    a.v = p->v;
    a.out = p->y;
    return saf_mixed_attn_fwd(&a, stream);
  }
  SafMixedAttnBwdArgs g;
  memset(&g, 0, sizeof(g));
  g.struct_size = (int32_t)sizeof(g);
  // forward tensors are not read for frozen heads; v/out only supply shapes
  a.v = p->y;
  a.out = p->y;
  g.fwd = a;
  g.dout = p->v;
  g.dv = p->y;
  return saf_mixed_attn_bwd(&g, stream);
}

int saf_frozen_pv_fwd(const SafFrozenPvArgs* args, void* stream) { return frozen_pv_common(args, stream, false); }
int saf_frozen_pv_bwd(const SafFrozenPvArgs* args, void* stream) { return frozen_pv_common(args, stream, true); }

static int validate_linear(const SafIndexedLinearArgs* a) {
  if (!a) return fail(SAF_ERR_INVALID, "null argument struct");
  if (a->struct_size != (int32_t)sizeof(SafIndexedLinearArgs))
    return fail(SAF_ERR_INVALID, "SafIndexedLinearArgs size mismatch: caller %d, library %d", a->struct_size,
                (int)sizeof(SafIndexedLinearArgs));
  if (a->dtype != SAF_F32 && a->dtype != SAF_BF16) return fail(SAF_ERR_UNSUPPORTED, "indexed linear takes fp32 or bf16");
  if (a->M < 0 || a->C <= 0 || a->n_slabs < 0 || a->slab <= 0) return fail(SAF_ERR_INVALID, "bad dimensions");
  if (a->act != SAF_ACT_NONE && a->act != SAF_ACT_GELU && a->act != SAF_ACT_SWIGLU)
    return fail(SAF_ERR_INVALID, "unknown activation %d", a->act);
  if (a->n_weights < 1 || a->n_weights > SAF_MAX_WEIGHTS) return fail(SAF_ERR_INVALID, "n_weights %d", a->n_weights);
  if (a->M == 0 || a->n_slabs == 0) return SAF_OK;
  if (!a->x || !a->slab_weight || !a->slab_row0) return fail(SAF_ERR_INVALID, "null x / slab tables");
  for (int g = 0; g < a->n_slabs; ++g) {
    const int w = a->slab_weight[g];
    if (w < 0 || w >= a->n_weights) return fail(SAF_ERR_INVALID, "slab %d names weight %d", g, w);
    if (!a->weights[w]) return fail(SAF_ERR_INVALID, "weight %d is null", w);
    if (a->slab_row0[g] < 0 || a->slab_row0[g] + a->slab > a->rows_w[w])
      return fail(SAF_ERR_INVALID, "slab %d rows [%d, %d) outside weight %d with %d rows", g, a->slab_row0[g],
                  a->slab_row0[g] + a->slab, w, a->rows_w[w]);
  }
  if (a->slab_rope) {
    bool any = false;
    for (int g = 0; g < a->n_slabs; ++g) any |= a->slab_rope[g] != 0;
    if (any) {
      if (!a->rope_cos || !a->rope_sin || a->T <= 0) return fail(SAF_ERR_INVALID, "rotated slabs need T and rope tables");
      if (a->slab % 2) return fail(SAF_ERR_INVALID, "RoPE requires an even head dimension");
    }
  }
  return SAF_OK;
}

int saf_indexed_linear_fwd(const SafIndexedLinearArgs* args, void* stream) {
  int rc = validate_linear(args);
  if (rc) return rc;
  if (args->M == 0 || args->n_slabs == 0) return SAF_OK;
  if (!args->out) return fail(SAF_ERR_INVALID, "out must be non-null");
  cudaStream_t st = (cudaStream_t)stream;
  rc = launch_gemm_sm100(*args, st);
  if (rc != SAF_ERR_UNSUPPORTED) return rc;
  if (args->act != SAF_ACT_NONE || args->residual)
    return fail(SAF_ERR_UNSUPPORTED, "the activation / residual epilogue exists on the bf16 tensor-core path only");
  return launch_gemm_generic(*args, st);
}

int saf_indexed_linear_bwd_dx(const SafIndexedLinearArgs* args, const void* dout, int64_t lddo, void* dx,
                              int64_t lddx, const void* bias, void* stream) {
  int rc = validate_linear(args);
  if (rc) return rc;
  if (args->M == 0) return SAF_OK;
  if (!dout || !dx) return fail(SAF_ERR_INVALID, "dout and dx must be non-null");
  rc = launch_gemm_bwd_dx_sm100(*args, dout, lddo, dx, lddx, bias, (cudaStream_t)stream);
  if (rc != SAF_ERR_UNSUPPORTED) return rc;
  return launch_gemm_bwd_dx(*args, dout, lddo, dx, lddx, bias, (cudaStream_t)stream);
}

int saf_indexed_linear_bwd_dw(const SafIndexedLinearArgs* args, const void* dout, int64_t lddo, void* stream) {
  int rc = validate_linear(args);
  if (rc) return rc;
  if (args->n_slabs == 0) return SAF_OK;
  if (!dout) return fail(SAF_ERR_INVALID, "dout must be non-null");
  rc = launch_gemm_bwd_dw_sm100(*args, dout, lddo, (cudaStream_t)stream);
  if (rc != SAF_ERR_UNSUPPORTED) return rc;
  return launch_gemm_bwd_dw(*args, dout, lddo, (cudaStream_t)stream);
}

int saf_rope_slabs(void* x, int64_t ld, int32_t M, int32_t n_slabs, int32_t slab, int32_t T,
                   const int32_t* slab_rope, const float* rope_cos, const float* rope_sin, int32_t dtype,
                   int32_t inverse, void* stream) {
  if (M < 0 || n_slabs < 0 || slab <= 0 || T <= 0) return fail(SAF_ERR_INVALID, "bad dimensions");
  if (slab % 2) return fail(SAF_ERR_INVALID, "RoPE requires an even head dimension");
  if (dtype != SAF_F32 && dtype != SAF_BF16) return fail(SAF_ERR_UNSUPPORTED, "rope_slabs takes fp32 or bf16");
  if (M == 0 || n_slabs == 0) return SAF_OK;
  if (!x || !rope_cos || !rope_sin) return fail(SAF_ERR_INVALID, "null pointer");
  return launch_rope_slabs(x, ld, M, n_slabs, slab, T, slab_rope, rope_cos, rope_sin, dtype, inverse, (cudaStream_t)stream);
}

int saf_layernorm_fwd(const void* x, int64_t ldx, const void* weight, const void* bias, void* out, int64_t ldo,
                      int32_t M, int32_t C, float eps, int32_t dtype, void* stream) {
  if (M < 0 || C <= 0) return fail(SAF_ERR_INVALID, "bad dimensions");
  if (dtype != SAF_F32 && dtype != SAF_BF16) return fail(SAF_ERR_UNSUPPORTED, "layernorm takes fp32 or bf16");
  if (M == 0) return SAF_OK;
  if (!x || !weight || !out) return fail(SAF_ERR_INVALID, "null pointer");
  return launch_layernorm(x, ldx, weight, bias, out, ldo, M, C, eps, dtype, 0, (cudaStream_t)stream);
}

int saf_rmsnorm_fwd(const void* x, int64_t ldx, const void* weight, void* out, int64_t ldo, int32_t M, int32_t C,
                    float eps, int32_t dtype, void* stream) {
  if (M < 0 || C <= 0) return fail(SAF_ERR_INVALID, "bad dimensions");
  if (dtype != SAF_F32 && dtype != SAF_BF16) return fail(SAF_ERR_UNSUPPORTED, "rmsnorm takes fp32 or bf16");
  if (M == 0) return SAF_OK;
  if (!x || !weight || !out) return fail(SAF_ERR_INVALID, "null pointer");
  return launch_layernorm(x, ldx, weight, nullptr, out, ldo, M, C, eps, dtype, 1, (cudaStream_t)stream);
}

int saf_decomposed_logz(const float* alpha, const float* rho, float* z, int32_t H, int32_t S, void* stream) {
  if (H < 0 || S < 0) return fail(SAF_ERR_INVALID, "negative dimension");
  if (H == 0 || S == 0) return SAF_OK;
  if (!alpha || !rho || !z) return fail(SAF_ERR_INVALID, "null pointer");
  return launch_logz(alpha, rho, z, H, S, S, (cudaStream_t)stream);
}

int saf_pattern_normalisers(const float* alpha, const float* rho, float* z, int32_t H, int32_t S, int32_t T,
                            void* stream) {
  if (H < 0 || S < 0 || T < 0) return fail(SAF_ERR_INVALID, "negative dimension");
  if (T > S) return fail(SAF_ERR_INVALID, "pattern normalisers: T > S");
  if (H == 0 || S == 0) return SAF_OK;
  if (!alpha || !rho || !z) return fail(SAF_ERR_INVALID, "null pointer");
  return launch_logz(alpha, rho, z, H, S, T, (cudaStream_t)stream);
}

int saf_pattern_param_grad(const SafPatternGradArgs* a, void* stream) {
  if (!a) return fail(SAF_ERR_INVALID, "null args");
  if (a->struct_size != (int32_t)sizeof(SafPatternGradArgs))
    return fail(SAF_ERR_INVALID, "SafPatternGradArgs size mismatch (%d vs %d)", a->struct_size,
                (int)sizeof(SafPatternGradArgs));
  if (a->B < 0 || a->H < 0 || a->T < 0 || a->HD <= 0 || a->SD < 0) return fail(SAF_ERR_INVALID, "bad dimension");
  if (a->dtype != SAF_F32 && a->dtype != SAF_BF16 && a->dtype != SAF_F16) return fail(SAF_ERR_INVALID, "bad dtype");
  if (a->force_state >= 0 && a->force_state != SAF_DECOMP) return SAF_OK;   // no head of that state has parameters
  if (a->B == 0 || a->H == 0 || a->T == 0) return SAF_OK;
  if (a->SD < a->T) return fail(SAF_ERR_INVALID, "pattern gradient: SD < T");
  if (!a->v.ptr || !a->out.ptr || !a->dout.ptr || !a->alpha || !a->rho || !a->z || !a->dalpha || !a->drho)
    return fail(SAF_ERR_INVALID, "null pointer");
  if (a->force_state < 0 && !a->frozen) return fail(SAF_ERR_INVALID, "frozen is null and force_state < 0");
  if (a->v.stride[3] != 1 || a->out.stride[3] != 1 || a->dout.stride[3] != 1)
    return fail(SAF_ERR_INVALID, "pattern gradient: last stride must be 1");
  return launch_pattern_grad(*a, (cudaStream_t)stream);
}

int saf_attention_moments(const SafAttnStatsArgs* a, void* stream) {
  if (!a) return fail(SAF_ERR_INVALID, "null args");
  // the struct grew by `quantity` and `cell_m2`: a caller that stops at `status` measures probabilities
  constexpr int32_t OLD_SIZE = (int32_t)offsetof(SafAttnStatsArgs, quantity);
  if (a->struct_size != (int32_t)sizeof(SafAttnStatsArgs) && a->struct_size != OLD_SIZE)
    return fail(SAF_ERR_INVALID, "SafAttnStatsArgs size mismatch (%d vs %d)", a->struct_size, (int)sizeof(SafAttnStatsArgs));
  SafAttnStatsArgs x;
  memset(&x, 0, sizeof(x));
  memcpy(&x, a, (size_t)a->struct_size);
  if (x.B < 0 || x.U < 0 || x.T < 0 || x.HD <= 0 || x.count_prev < 0) return fail(SAF_ERR_INVALID, "bad dimension");
  if (x.quantity != SAF_STATS_PROBS && x.quantity != SAF_STATS_LOGITS) return fail(SAF_ERR_INVALID, "unknown quantity %d", x.quantity);
  if (x.B == 0 || x.U == 0 || x.T == 0) return SAF_OK;
  if (!x.q.ptr || !x.k.ptr || !x.mean) return fail(SAF_ERR_INVALID, "null pointer");
  if (x.quantity == SAF_STATS_PROBS && (!x.lse.ptr || !x.head_m2 || !x.neg_entropy)) return fail(SAF_ERR_INVALID, "null pointer");
  if (x.quantity == SAF_STATS_PROBS && x.cell_m2) return fail(SAF_ERR_INVALID, "cell_m2 goes with SAF_STATS_LOGITS");
  return launch_attn_stats_sm100(x, (cudaStream_t)stream);
}

}  // extern "C"
