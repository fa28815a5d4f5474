/* saf_b200 -- C ABI of the B200 (sm_100a) implementation of Selective Attention
 * Freezing's mixed-attention hot path.
 *
 * The reference project has no native layer: its operator boundary is the Python
 * import surface `from kernel import ...` (kernel/__init__.py:14-22).  Each entry
 * point below sits underneath one of those Python operators and names the
 * reference function it replaces.  All pointers are raw device pointers unless
 * marked host; strides are in ELEMENTS; every call enqueues work on `stream`
 * (a cudaStream_t passed as void*), never synchronises, never allocates device
 * memory, and returns 0 or a negative SAF_ERR_* code before anything is
 * launched when the arguments are invalid.  saf_last_error() gives the text.
 */
#ifndef SAF_B200_H
#define SAF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAF_ABI_VERSION 2

enum SafStatus {
  SAF_OK = 0,
  SAF_ERR_INVALID = -1,     /* bad shape / stride / null pointer / dtype        */
  SAF_ERR_UNSUPPORTED = -2, /* valid request this build has no kernel for       */
  SAF_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed (launch, map)  */
  SAF_ERR_LIMIT = -4        /* size beyond a stated fixed limit                 */
};

enum SafDType { SAF_F32 = 0, SAF_BF16 = 1, SAF_F16 = 2 };

/* per-head state, the values of the `frozen` tensor
 * (kernel/fused_attn.py:665-667 defines 0,1,2; 3 is this library's addition) */
enum SafHeadState {
  SAF_LIVE = 0,       /* causal softmax(q k^T * sm_scale) v                      */
  SAF_DENSE = 1,      /* y_i = sum_{j<=i} patt[p, i, j] v_j                      */
  SAF_DECOMP = 2,     /* y_i = sum_{j<=i} exp(alpha_j + rho_{i-j} - z_i) v_j     */
  SAF_SINK_DECAY = 3  /* y_i = a v_0 + (1-a) sum_{j<=i} r^(i-j) v_j / Z_i  (scan) */
};

typedef struct SafTensor {
  void* ptr;
  int64_t stride[4]; /* elements; unused trailing entries ignored */
} SafTensor;

/* ---------------------------------------------------------------------------
 * Mixed attention, all heads in one call.
 * Replaces fused_mixed_attn / _fwd / _fwd_kernel (kernel/fused_attn.py:650-734,
 * 572-591, 228-289) and, with `kvidx`, the GQA twin
 * (qwen/kernel/fused_attn.py:667-768).
 * ------------------------------------------------------------------------- */
typedef struct SafMixedAttnArgs {
  int32_t struct_size; /* sizeof(SafMixedAttnArgs), checked */
  int32_t dtype;       /* SafDType of q, k, v, out                                  */
  int32_t B, H, U, T, HD;
  int32_t HKV;         /* 0: k has U heads, v has H heads.  >0: GQA, k and v have
                          HKV heads and head h reads kv head kvidx[h]               */
  int32_t S;           /* patt is (P, S, S); 0 when patt.ptr is null                */
  int32_t SD;          /* alpha/rho/z are (H, SD); 0 when absent                    */
  int32_t patt_dtype;  /* SafDType of patt                                          */
  int32_t dec_dtype;   /* SafDType of alpha, rho, z                                 */
  int32_t rope;        /* 0: q,k used as given.  1: rotate q,k while loading with
                          the (T, HD) fp32 tables rope_cos / rope_sin
                          (nanogpt/model.py:57-68 semantics)                        */
  int32_t force_state; /* -1: use frozen[h].  0..3: every head has this state       */
  float sm_scale;
  SafTensor q, k;      /* (B, U, T, HD); GQA: k is (B, HKV, T, HD)                  */
  SafTensor v;         /* (B, H, T, HD); GQA: (B, HKV, T, HD)                       */
  SafTensor out;       /* (B, H, T, HD), any strides with unit last stride          */
  SafTensor lse;       /* (B, H, T) fp32 or null; live rows get m + log2(l) in the
                          log2 domain (kernel/fused_attn.py:223-225)                */
  SafTensor patt;      /* (P, S, S)                                                 */
  SafTensor alpha, rho, z; /* (H, SD)                                               */
  const int32_t* frozen;   /* device (H,), SafHeadState per head                    */
  const int32_t* hidx;     /* device (H,) head -> slot in q/k; null = identity      */
  const int32_t* pidx;     /* device (H,) head -> pattern row; null = identity      */
  const int32_t* kvidx;    /* device (H,) head -> kv head (GQA); null otherwise     */
  const int32_t* frozen_host; /* HOST copy of frozen (optional scheduling hint)     */
  const float* sd_alpha;   /* device (H,) sink weight a of SAF_SINK_DECAY heads     */
  const float* sd_rho;     /* device (H,) decay r of SAF_SINK_DECAY heads           */
  const float* rope_cos;   /* device (T, HD) fp32                                   */
  const float* rope_sin;
  int32_t* status;         /* optional device int32; a kernel that gave up on a
                              bounded wait writes a non-zero code here              */
  int32_t* sched;          /* optional device int32[2], ZERO on entry, private to this
                              call while it runs: the tile queue of the persistent
                              forward kernel (one CTA per SM pulling row-tile pairs;
                              the kernel leaves both words zero again, so a caller may
                              reuse them for its next call on the same stream).  Null:
                              one CTA per row-tile pair, no scratch at all.  The
                              backward ignores it.                                   */
} SafMixedAttnArgs;

int saf_mixed_attn_fwd(const SafMixedAttnArgs* args, void* stream);

/* Backward of the above.  Replaces _bwd / _bwd_preprocess / _bwd_dkdv / _bwd_dq
 * (kernel/fused_attn.py:593-623, 291-540).  dq, dk must be zero-filled by the
 * caller (frozen heads' slots are never written, kernel/fused_attn.py:597-598);
 * delta is caller-provided (B, H, T) fp32 scratch. */
typedef struct SafMixedAttnBwdArgs {
  int32_t struct_size;
  SafMixedAttnArgs fwd; /* same tensors as the forward call; out and lse filled   */
  SafTensor dout;       /* (B, H, T, HD)                                          */
  SafTensor dq, dk;     /* like q, k (own strides)                                */
  SafTensor dv;         /* like v                                                 */
  SafTensor delta;      /* (B, H, T) fp32 scratch                                 */
} SafMixedAttnBwdArgs;

int saf_mixed_attn_bwd(const SafMixedAttnBwdArgs* args, void* stream);

/* Same backward for callers that cannot supply scratch memory (no counterpart in the
 * reference, which always allocates through torch).  Meant for hosts that planned
 * their whole device arena ahead of time, plugin interfaces that pass only the
 * operator's own tensors, or call sites where a device allocation is not allowed
 * because it may synchronise the GPU.  `args->delta` is ignored: delta lives in a
 * fixed array of SAF_STATIC_DELTA_FLOATS fp32 values (4 MiB) that every GPU loading
 * this library holds until the process exits.
 *   - B*H*T must not exceed SAF_STATIC_DELTA_FLOATS, else SAF_ERR_LIMIT (nothing runs);
 *     calls that cannot contain a live head (U == 0, force_state or frozen_host naming
 *     frozen states only) never touch delta and have no such limit.
 *   - The call allocates nothing.  The first call on each device looks up the
 *     array's device address (once per device, with that device current); make
 *     that first call before starting any stream capture.  The address is remembered
 *     per device ordinal: do not call this after cudaDeviceReset() on that device.
 *   - All calls on a device share the array, which keeps the last call's values;
 *     nothing in it needs clearing (rows are written before they are read), but
 *     two calls that overlap on the GPU race on it -- keep them on one stream or
 *     order them with events.
 * Inputs, outputs and every other rule are those of saf_mixed_attn_bwd. */
#define SAF_STATIC_DELTA_FLOATS (1 << 20)
int saf_mixed_attn_bwd_static(const SafMixedAttnBwdArgs* args, void* stream);

/* ---------------------------------------------------------------------------
 * Frozen heads only, compact values.
 * Replaces frozen_pv / _pv_fwd_kernel / _pv_bwd_kernel
 * (kernel/frozen_attn.py:185-192, 51-89, 91-128).
 *   y[b,f] = patt[fz_idx[f], :T, :T] @ v[b,f]        dv[b,f] = patt^T @ dy[b,f]
 * When sd_alpha/sd_rho are non-null the pattern is the structured sink+decay
 * form and the O(T) scan is used instead of reading patt.
 * ------------------------------------------------------------------------- */
typedef struct SafFrozenPvArgs {
  int32_t struct_size;
  int32_t dtype, patt_dtype;
  int32_t B, NF, T, HD, S;
  SafTensor patt;          /* (n_head, S, S)               */
  SafTensor v;             /* (B, NF, T, HD) fwd: values; bwd: dy */
  SafTensor y;             /* (B, NF, T, HD) fwd: output;  bwd: dv */
  const int32_t* fz_idx;   /* device (NF,) pattern row per compact head */
  const float* sd_alpha;   /* device (NF,) or null */
  const float* sd_rho;
  int32_t* status;
} SafFrozenPvArgs;

int saf_frozen_pv_fwd(const SafFrozenPvArgs* args, void* stream);
int saf_frozen_pv_bwd(const SafFrozenPvArgs* args, void* stream);

/* ---------------------------------------------------------------------------
 * Indexed linear: projections over head-sized row slabs of canonical weights,
 * read in place (no gathered weight copy).
 * Replaces linear_rows / linear_rows2 (kernel/indexed_linear.py:125-135, 28-55,
 * 86-122) for row sets made of whole, aligned slabs of `slab` consecutive rows
 * (the model passes every row of every live head, nanogpt/model.py:854-856).
 *
 *   out[m, g*slab + r] = sum_c x[m, c] * W_g[row0_g + r, c] (+ bias_g[row0_g + r])
 *
 * for slab-groups g = 0..n_slabs-1, each naming one weight matrix (by index
 * into `weights`) and a first row.  With rope != 0 slab g with rope_flag[g] != 0
 * is rotated in the epilogue (slab == head_dim, position = m % T).
 * ------------------------------------------------------------------------- */
#define SAF_MAX_WEIGHTS 4
typedef struct SafIndexedLinearArgs {
  int32_t struct_size;
  int32_t dtype;            /* x, weights, out: SAF_BF16 (tensor cores) or SAF_F32 */
  int32_t M, C;             /* x is (M, C) row-major with row stride ldx           */
  int32_t n_weights;        /* <= SAF_MAX_WEIGHTS                                  */
  int32_t n_slabs, slab;    /* output width = n_slabs * slab                       */
  int32_t T;                /* sequence length (RoPE position = m % T); 0 = no RoPE */
  const void* x;
  int64_t ldx;
  const void* weights[SAF_MAX_WEIGHTS]; /* each (rows_w, C) row-major, row stride ldw[w] */
  const void* biases[SAF_MAX_WEIGHTS];  /* each (rows_w,) or null                     */
  int64_t ldw[SAF_MAX_WEIGHTS];         /* row stride of each weight                  */
  int64_t cdw[SAF_MAX_WEIGHTS];         /* column stride (0 or 1: row-major; ldw=1 with
                                           cdw=row length addresses the transpose, which
                                           is how linear_permuted_cols selects columns) */
  int32_t rows_w[SAF_MAX_WEIGHTS];
  const int32_t* slab_weight; /* HOST (n_slabs,) weight index of slab g            */
  const int32_t* slab_row0;   /* HOST (n_slabs,) first weight row of slab g        */
  const int32_t* slab_rope;   /* HOST (n_slabs,) or null: rotate this slab         */
  const float* rope_cos;      /* device (T, slab) fp32                             */
  const float* rope_sin;
  void* out;                  /* (M, n_slabs*slab) row-major, row stride ldo       */
  int64_t ldo;
  int32_t* status;
  /* epilogue of the rest of the transformer block around the attention path (forward only, bf16 tensor-core
   * path): out = [residual +] act(x W^T + b).  Replaces the separate GELU and residual-add kernels of
   * MLP.forward / Block.forward (nanogpt/model.py:1202-1207, 1237-1240). */
  int32_t act;                /* SAF_ACT_NONE, SAF_ACT_GELU (exact erf form, nn.GELU()) or SAF_ACT_SWIGLU:
                                 slabs come in (gate, up) pairs of 64 rows and the output, of width
                                 n_slabs*slab/2, is silu(gate) * up -- the gated MLP of the Qwen-shaped
                                 blocks (slab 64, no bias, no rotation, bf16 tensor-core path only)     */
  const void* residual;       /* (M, n_slabs*slab) same dtype, row stride ldr, or null    */
  int64_t ldr;
} SafIndexedLinearArgs;
enum { SAF_ACT_NONE = 0, SAF_ACT_GELU = 1, SAF_ACT_SWIGLU = 2 };

int saf_indexed_linear_fwd(const SafIndexedLinearArgs* args, void* stream);

/* Backward pieces of the indexed linear (kernel/indexed_linear.py:100-122):
 *   dx[m, c]  = sum_{g,r} dout[m, g*slab+r] * W_g[row0_g + r, c]  (+ bias[c])
 *   dW_g[row0_g + r, c] = sum_m dout[m, g*slab+r] * x[m, c]; rows of no slab are
 *   left untouched (the caller zero-fills dW, so they stay exactly zero).
 * `weights` carry W for dx and receive dW (written) for dw; biases receive db.
 * With transposed weight addressing (cdw) the dx product is also the forward of
 * linear_permuted_cols (kernel/indexed_linear.py:58-70, 138-141); `bias` (C,)
 * is added there and is null for a true backward. */
int saf_indexed_linear_bwd_dx(const SafIndexedLinearArgs* args, const void* dout, int64_t lddo, void* dx,
                              int64_t lddx, const void* bias, void* stream);
int saf_indexed_linear_bwd_dw(const SafIndexedLinearArgs* args, const void* dout, int64_t lddo, void* stream);

/* ---------------------------------------------------------------------------
 * In-place rotary embedding of chosen `slab`-wide column slabs of x (M, n_slabs*slab):
 * row m uses table row m % T of rope_cos / rope_sin (fp32 (T, slab), halves repeated).
 * Replaces apply_rotary_pos_emb / rotate_half on the compact q,k (nanogpt/model.py:57-99);
 * inverse != 0 applies the adjoint rotation, which is what the backward of a projection
 * with the rotation fused into its epilogue needs for the incoming gradient.
 * slab_rope: HOST array (n_slabs) of flags, or null = rotate every slab.
 * ------------------------------------------------------------------------- */
int saf_rope_slabs(void* x, int64_t ld, int32_t M, int32_t n_slabs, int32_t slab, int32_t T,
                   const int32_t* slab_rope, const float* rope_cos, const float* rope_sin, int32_t dtype,
                   int32_t inverse, void* stream);

/* ---------------------------------------------------------------------------
 * LayerNorm over the last dimension with optional bias (LayerNorm.forward, nanogpt/model.py:45-54:
 * F.layer_norm(x, (C,), weight, bias, 1e-5)).  x, out (M, C) row-major in `dtype` (SAF_BF16 / SAF_F32),
 * weight / bias (C,) in the same dtype (bias may be null); statistics in fp32.
 * ------------------------------------------------------------------------- */
int saf_layernorm_fwd(const void* x, int64_t ldx, const void* weight, const void* bias, void* out, int64_t ldo,
                      int32_t M, int32_t C, float eps, int32_t dtype, void* stream);
/* RMSNorm over the last dimension, y = x / sqrt(mean(x^2) + eps) * weight: the norm of the Qwen-shaped blocks
 * around the grouped-query attention (the reference leaves it to the Hugging Face model its adapter wraps,
 * qwen/nanogpt/hybrid_prior_attention.py:522-523).  Same layout rules as saf_layernorm_fwd. */
int saf_rmsnorm_fwd(const void* x, int64_t ldx, const void* weight, void* out, int64_t ldo, int32_t M, int32_t C,
                    float eps, int32_t dtype, void* stream);

/* ---------------------------------------------------------------------------
 * Freeze-time helper: z[h,i] = logsumexp_{j<=i}(alpha[h,j] + rho[h,i-j]).
 * Replaces decomposed_logz (kernel/fused_attn.py:101-116).  fp32 in/out.
 * ------------------------------------------------------------------------- */
int saf_decomposed_logz(const float* alpha, const float* rho, float* z, int32_t H, int32_t S, void* stream);

/* ---------------------------------------------------------------------------
 * Trainable decomposed patterns (supplement/trainable_pattern_kernels.py).
 *
 * saf_pattern_normalisers replaces normalisers() (:62-66, kernel :8-18): rows i < T get
 * z[h,i] = logsumexp_{j<=i}(alpha[h,j] + rho[h,i-j]); rows T..S-1 are set to zero.
 *
 * saf_pattern_param_grad replaces PatternGradient.backward / _parameter_backward (:21-58,
 * :79-85): for every head whose state is SAF_DECOMP, with P_ij = exp(alpha_j + rho_{i-j} - z_i),
 * dP = dout v^T and delta_i = dout_i . out_i,
 *     dalpha[h,j] += sum_{b,i} P_ij (dP_ij - delta_i)      drho[h,d] += sum_{b, i-j=d} P_ij (dP_ij - delta_i).
 * The call ADDS into dalpha / drho (fp32 atomics, like the reference): the caller zero-fills them.
 * bf16 tensors with head_dim 64/128 run on the tensor cores, everything else on the CUDA cores in fp32.
 * ------------------------------------------------------------------------- */
int saf_pattern_normalisers(const float* alpha, const float* rho, float* z, int32_t H, int32_t S, int32_t T,
                            void* stream);

typedef struct SafPatternGradArgs {
  int32_t struct_size; /* sizeof(SafPatternGradArgs), checked                        */
  int32_t dtype;       /* SafDType of v, out, dout                                   */
  int32_t B, H, T, HD;
  int32_t SD;          /* alpha, rho, z, dalpha, drho are (H, SD) fp32, SD >= T      */
  int32_t force_state; /* -1: heads with frozen[h] == SAF_DECOMP; 2: every head      */
  SafTensor v;         /* (B, H, T, HD) values the pattern was applied to            */
  SafTensor out;       /* (B, H, T, HD) forward result                               */
  SafTensor dout;      /* (B, H, T, HD) gradient of the result                       */
  const float* alpha;
  const float* rho;
  const float* z;
  const int32_t* frozen;      /* device (H,), SafHeadState per head; may be null with force_state */
  const int32_t* frozen_host; /* HOST copy of frozen (optional: skips the launch when no head trains) */
  float* dalpha;
  float* drho;
  float* delta;        /* caller-provided scratch, B*H*T fp32 (rows of training heads
                          are written, then read); without it the call runs on the
                          CUDA cores                                                */
  int32_t* status;     /* optional device int32, as in SafMixedAttnArgs              */
} SafPatternGradArgs;

int saf_pattern_param_grad(const SafPatternGradArgs* args, void* stream);

/* ---------------------------------------------------------------------------
 * Attention statistics of live heads for the freeze controller, without the
 * (B, H, T, T) capture.  Replaces, for softmax heads, what FreezeController._measure
 * does with the retained eager attention (nanogpt/dynamic_freeze.py:629-745):
 * _centered_batch_reduced_moments (:96-127) + _merge_reduced_moments (:130-143) +
 * _negative_entropy_sum (:146-173) of att = softmax(causal(q k^T * sm_scale)).
 *   mean        (U, T, T) fp32, the running mean attention; with count_prev == 0 it is
 *               overwritten (zeros above the diagonal), otherwise Chan-merged in place:
 *               mean += (batch_mean - mean) * B / (count_prev + B)
 *   head_m2     (U,) fp64, += sum over cells of the batch's centred squares
 *               + sum((batch_mean - mean)^2) * count_prev * B / (count_prev + B)
 *   neg_entropy (U,) fp64, += sum over samples and cells of p ln p
 * lse is the (B, U, T) fp32 row log-sum-exp of the same q, k in the log2 domain, as
 * saf_mixed_attn_fwd writes it.  bf16 q, k with head_dim 64 / 128 (tensor-core kernel);
 * anything else returns SAF_ERR_UNSUPPORTED.
 *
 * quantity == SAF_STATS_LOGITS measures the raw scores instead, lg = q k^T * sm_scale
 * over the whole square (nothing masked), as the priors that sample logits want them
 * (`_last_logits`, nanogpt/model.py:828-831; dynamic_freeze.py:721-737):
 *   mean        (U, T, T) fp32, Chan-merged batch mean as above (lg.mean(0))
 *   cell_m2     optional (U, T, T) fp32: _centered_batch_moments (:62-81) +
 *               _merge_moments (:84-93) per cell,
 *               m2 += sum_b (lg_b - batch_mean)^2 + (batch_mean - mean)^2 * count_prev * B / (count_prev + B)
 * lse, head_m2 and neg_entropy are not used then and may be null.  A caller built against
 * the struct without the last two fields (struct_size up to `status`) gets probabilities.
 * ------------------------------------------------------------------------- */
#define SAF_STATS_PROBS 0
#define SAF_STATS_LOGITS 1
typedef struct SafAttnStatsArgs {
  int32_t struct_size; /* sizeof(SafAttnStatsArgs), checked */
  int32_t dtype;       /* SafDType of q, k */
  int32_t B, U, T, HD;
  float sm_scale;
  SafTensor q, k;      /* (B, U, T, HD), rotated as the attention saw them */
  SafTensor lse;       /* (B, U, T) fp32 */
  float* mean;
  int64_t count_prev;
  double* head_m2;
  double* neg_entropy;
  int32_t* status;     /* optional device int32, as in SafMixedAttnArgs */
  int32_t quantity;    /* SAF_STATS_PROBS or SAF_STATS_LOGITS */
  float* cell_m2;      /* SAF_STATS_LOGITS: optional (U, T, T) fp32 centred squares per cell, 16-byte aligned */
} SafAttnStatsArgs;

int saf_attention_moments(const SafAttnStatsArgs* args, void* stream);

/* ---------------------------------------------------------------------------
 * Library plumbing
 * ------------------------------------------------------------------------- */
int saf_abi_version(void);
/* copies the calling thread's last error text (NUL-terminated); returns its length */
int saf_last_error(char* buf, size_t n);
/* number of kernel launches this library has enqueued in this process */
int64_t saf_launch_count(void);
/* 1 when the device under the current context is an sm_100 part, else 0 */
int saf_device_supported(void);

/* ---------------------------------------------------------------------------
 * Self-checks (no counterpart in the reference).  Every wait inside the kernels is bounded; a wait that runs
 * out records (kind | site << 8) in the call's `status` word, the kernel stops issuing work, skips its stores
 * and returns, so the context stays usable.
 * ------------------------------------------------------------------------- */
/* Launches one CTA that waits, with a limit of limit_ns nanoseconds (at most 1e8), on a barrier nothing ever
 * arrives on, and then records (6 | 99 << 8) = 0x6306 in *status (device int32, zero before the call) through
 * the same path the kernels use.  Nothing traps, nothing hangs. */
int saf_selftest_wait_timeout(int32_t* status, int64_t limit_ns, void* stream);
/* Host-only check of the per-device bookkeeping (dynamic shared memory limits and SM counts are remembered per
 * device ordinal, never per process): 0 when it behaves, else the number of the failing step.  No CUDA call. */
int saf_selftest_per_device_once(void);
/* Hardware characterisation behind the kernels' tiling: one CTA per SM issues reps groups of tcgen05.mma
 * instructions (bf16, M = 128, K = 16; eight per group unless stated) back to back and the first CTA writes the
 * elapsed SM cycles to *cycles (device int64).  form & 255 selects what is issued:
 *   0-7    one product, one operand form: 0 smem/smem K-major N 128, 1 TMEM / smem MN-major N 128, 2 TMEM / smem
 *          MN-major N 64, 3 smem/smem MN-major N 256, 4 smem/smem K-major N 256, 5 TMEM / smem K-major N 128,
 *          6 smem/smem K-major N 64, 7 smem K-major / smem MN-major N 128
 *   8-11   forms 0 / 1 with operand addresses that change per group (ring stages): descriptors built per
 *          instruction (8, 9) or advanced by an add (10, 11)
 *   12-15  a new product every group: two accumulators in turn with / without a commit per group (12 / 13),
 *          smem-operand and TMEM-operand products in turn (14), one accumulator with commits (15)
 *   16-18  the products of a forward key step at head_dim 64 in turn: all from TMEM operands, 4 + 4 instructions
 *          of N 64 (16); scores from shared memory (4 of N 128) and P V from TMEM (8 of N 64), alternating (17) or
 *          as score, score, P V, P V (18)
 *   19-21  form 14 with one thing changed: the TMEM-operand product as two halves of N 64 (19), with a K-major B
 *          operand (20), with its A operand in consecutive columns (21)
 * form + 256 fills the operands with random bf16 values instead of zeros; + 512 / 1024 / 2048 adds neighbour
 * load while the instructions run: eight warps on tensor memory, eight warps on the arithmetic pipes, bulk
 * copies landing in shared memory.  Every wait is bounded (status as in SafMixedAttnArgs, may be null). */
int saf_selftest_mma_rate(int form, int reps, long long* cycles, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SAF_B200_H */
