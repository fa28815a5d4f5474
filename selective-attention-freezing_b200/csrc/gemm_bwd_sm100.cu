// Backward products of the indexed linear on tcgen05 (kernel/indexed_linear.py:47-55, 107-121):
//
//   DX:  dx[m, c]            = sum_n dout[m, n] * W_g[row0_g + r, c]        n = g*64 + r over the selected 64-row blocks
//   DW:  dW_g[row0_g + r, c] = sum_m dout[m, g*64 + r] * x[m, c]            rows of no block are never written
//
// Neither product needs a transposed or gathered copy: the tensor core reads an operand whose
// contraction index is the slow one ("MN-major") straight from the row-major tile TMA delivers.
//   DX: A = dout tile (K-major), B = 64 selected weight rows x 256 columns (MN-major), one TMA source per block
//   DW: A = dout^T (MN-major: 64 tokens x 128 features), B = x tile (MN-major: 64 tokens x 256 columns);
//       the finished 128 x 256 tile is stored through the weight-gradient maps, 64 rows at a time, at the
//       rows the two blocks own (the reference zero-fills and index_copy_'s a dense product instead).
// Same persistent, warp-specialised CTA as the forward GEMM: warp 0 TMA, warp 1 MMA issuer, warps 2-5
// epilogue; 128x256 tiles, K step 64, 4 stages, two TMEM accumulators.  All waits are bounded.
#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int NSTG = 4;
constexpr int ATOM = 64 * 64 * 2;               // 8 KB: 64 rows of 128 bytes
constexpr int BA_BYTES = 2 * ATOM;              // 16 KB
constexpr int BB_BYTES = 4 * ATOM;              // 32 KB
constexpr int BSTAGE = BA_BYTES + BB_BYTES;
constexpr int BOUT_BYTES = 2 * BM * 64 * 2;
constexpr int BMAX_SUB = 160;
constexpr int BGEMM_THREADS = 192;
enum { MODE_DX = 0, MODE_DW = 1 };

struct BlockTable {
  int32_t row0[BMAX_SUB];
  uint8_t weight[BMAX_SUB];
  // slabs that are a multiple of 32 but not of 64 rows (head_dim 96): a 64-row block is two runs of 32 weight
  // rows, each with its own source (first run in row0 / weight, second run here); the weight maps then carry
  // 32-row boxes
  int32_t row0b[BMAX_SUB];
  uint8_t weightb[BMAX_SUB];
};

struct BwdGemmParams {
  int I, J, KB;              // output rows, output columns, K steps of 64
  int tiles_m, tiles_n;
  int n_blocks;              // selected 64-row blocks
  const void* bias;          // DX only: bf16 over the J output columns, or null
  int* status;
  int halves;                // see BlockTable
};

struct BSmem {
  uint64_t full[NSTG], empty[NSTG], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
};

template <int MODE>
__global__ void __launch_bounds__(BGEMM_THREADS, 1)
indexed_gemm_bwd_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                        const __grid_constant__ CUtensorMap mapW0, const __grid_constant__ CUtensorMap mapW1,
                        const __grid_constant__ CUtensorMap mapW2, const __grid_constant__ CUtensorMap mapW3,
                        const __grid_constant__ CUtensorMap mapO, const __grid_constant__ BwdGemmParams p,
                        const __grid_constant__ BlockTable tb) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* out_stage = smem + NSTG * BSTAGE;
  BSmem* sl = reinterpret_cast<BSmem*>(out_stage + BOUT_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;
  const CUtensorMap* wm[4] = {&mapW0, &mapW1, &mapW2, &mapW3};

  if (tid == 0) {
    for (int s = 0; s < NSTG; ++s) {
      mbar_init(&sl->full[s], 1);
      mbar_init(&sl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sl->acc_full[b], 1);
      mbar_init(&sl->acc_empty[b], 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&sl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sl->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&mapA);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
        const int nsub = min(4, (p.J - tn * BN + 63) / 64);                      // 64-column blocks of B
        const int nrow = (MODE == MODE_DW) ? min(2, p.n_blocks - tm * 2) : 2;    // 64-feature blocks of A
        for (int kb = 0; kb < p.KB; ++kb, ++it) {
          const int s = it % NSTG;
          if (!mbar_wait(&sl->empty[s], ((it / NSTG) & 1) ^ 1)) {
            dev_set_error(p.status, SAF_DEV_TIMEOUT_TMA, 60);
            ok = false;
            break;
          }
          uint8_t* a = stage_base + s * BSTAGE;
          uint8_t* b = a + BA_BYTES;
          if (MODE == MODE_DX) {
            mbar_expect_tx(&sl->full[s], BA_BYTES + nsub * ATOM);
            tma_load_2d(a, &mapA, &sl->full[s], kb * BK, tm * BM);               // dout[m tile, block kb]
            for (int u = 0; u < nsub; ++u) {
              tma_load_2d(b + u * ATOM, wm[tb.weight[kb]], &sl->full[s], tn * BN + u * 64, tb.row0[kb]);
              if (p.halves)
                tma_load_2d(b + u * ATOM + ATOM / 2, wm[tb.weightb[kb]], &sl->full[s], tn * BN + u * 64, tb.row0b[kb]);
            }
          } else {
            mbar_expect_tx(&sl->full[s], (nrow + nsub) * ATOM);
            for (int u = 0; u < nrow; ++u)
              tma_load_2d(a + u * ATOM, &mapA, &sl->full[s], (tm * 2 + u) * 64, kb * BK);   // dout[token block, features]
            for (int u = 0; u < nsub; ++u)
              tma_load_2d(b + u * ATOM, &mapB, &sl->full[s], tn * BN + u * 64, kb * BK);    // x[token block, columns]
          }
        }
      }
    }
  } else if (warp == 1) {
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(BM, BN, MODE == MODE_DW ? 1 : 0, 1);
    const uint32_t sbase = smem_u32(stage_base);
    uint32_t it = 0, lt = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++lt) {
      const int buf = lt & 1;
      if (!mbar_wait(&sl->acc_empty[buf], ((lt >> 1) & 1) ^ 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 61);
        break;
      }
      tc_fence_after();
      const uint32_t d = tmem + buf * BN;
      for (int kb = 0; kb < p.KB; ++kb, ++it) {
        const int s = it % NSTG;
        if (!mbar_wait(&sl->full[s], (it / NSTG) & 1)) {
          dev_set_error(p.status, SAF_DEV_TIMEOUT_MMA, 62);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a = sbase + s * BSTAGE;
        const uint32_t b = a + BA_BYTES;
        if (leader) {
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t ad = (MODE == MODE_DW) ? umma_smem_desc_sw128(a + k4 * 2048, ATOM, 1024)
                                                  : umma_smem_desc_sw128(a + k4 * 32, 16, 1024);
            umma_ss(d, ad, umma_smem_desc_sw128(b + k4 * 2048, ATOM, 1024), idesc, (kb | k4) != 0);
          }
          umma_commit(&sl->empty[s]);
        }
        __syncwarp();
      }
      if (ok && leader) umma_commit(&sl->acc_full[buf]);
      __syncwarp();
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int etid = tid - 64;
    uint32_t lt = 0;
    uint32_t n_out = 0;                         // output blocks stored so far (staging block = parity)
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++lt) {
      const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
      const int nsub = min(4, (p.J - tn * BN + 63) / 64);
      const int nrow = (MODE == MODE_DW) ? min(2, p.n_blocks - tm * 2) : 2;
      const int buf = lt & 1;
      if (!mbar_wait(&sl->acc_full[buf], (lt >> 1) & 1)) {
        dev_set_error(p.status, SAF_DEV_TIMEOUT_EPI, 63);
        break;
      }
      tc_fence_after();
      const uint32_t tsrc = tmem + ((uint32_t)(quad * 32) << 16) + buf * BN;
      for (int u = 0; u < nsub; ++u) {
        // the two staging blocks take turns over all stores of the CTA (nsub may be odd)
        const int ob = (n_out++) & 1;
        if (etid == 0) tma_store_wait_read1();
        named_bar_sync(1, 128);
        uint32_t r0[32], r1[32];
        tmem_ld32(tsrc + u * 64, r0);
        tmem_ld32(tsrc + u * 64 + 32, r1);
        tmem_ld_wait();
        float v[64];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          v[j] = __uint_as_float(r0[j]);
          v[32 + j] = __uint_as_float(r1[j]);
        }
        if (MODE == MODE_DX && p.bias) {
          const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias) + tn * BN + u * 64;
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (tn * BN + u * 64 + j < p.J) v[j] += __bfloat162float(bp[j]);
        }
        uint8_t* dst = out_stage + ob * (BOUT_BYTES / 2) + row * 128;
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
          const uint8_t* src = out_stage + ob * (BOUT_BYTES / 2);
          if (MODE == MODE_DX) {
            tma_store_2d(&mapO, src, tn * BN + u * 64, tm * BM);
          } else {
            for (int hb = 0; hb < nrow; ++hb) {
              const int sb = tm * 2 + hb;
              tma_store_2d(wm[tb.weight[sb]], src + hb * ATOM, tn * BN + u * 64, tb.row0[sb]);
              if (p.halves) tma_store_2d(wm[tb.weightb[sb]], src + hb * ATOM + ATOM / 2, tn * BN + u * 64, tb.row0b[sb]);
            }
          }
          tma_store_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sl->acc_empty[buf]);
    }
    if (etid == 0) tma_store_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

bool al16(const void* q) { return ((uintptr_t)q & 15) == 0; }

int map2(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, int64_t ld, uint32_t box_rows) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[2] = {0, (uint64_t)ld * 2};
  uint32_t box[2] = {64, box_rows};
  return make_tensor_map_bf16(m, base, 2, dims, strides, box, true);
}

bool common_ok(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo) {
  if (a.dtype != SAF_BF16 || a.slab % 32 || (a.n_slabs * a.slab) % 64 || a.n_slabs <= 0 || a.M <= 0) return false;
  if (a.n_slabs * a.slab / 64 > BMAX_SUB) return false;
  if (a.C % 8 || lddo % 8 || !al16(dout)) return false;
  for (int w = 0; w < a.n_weights; ++w) {
    if (!a.weights[w]) return false;
    if (a.ldw[w] % 8 || (a.cdw[w] != 0 && a.cdw[w] != 1) || !al16(a.weights[w])) return false;
  }
  return saf_device_supported() != 0;
}

bool is_halves(const SafIndexedLinearArgs& a) { return a.slab % 64 != 0; }

void fill_blocks(const SafIndexedLinearArgs& a, BlockTable* tb) {
  memset(tb, 0, sizeof(*tb));
  if (is_halves(a)) {
    for (int hb = 0; hb < a.n_slabs * a.slab / 32; ++hb) {       // 32-row runs, two per block
      const int g = (hb * 32) / a.slab, r = (hb * 32) % a.slab;
      if (hb & 1) {
        tb->row0b[hb >> 1] = a.slab_row0[g] + r;
        tb->weightb[hb >> 1] = (uint8_t)a.slab_weight[g];
      } else {
        tb->row0[hb >> 1] = a.slab_row0[g] + r;
        tb->weight[hb >> 1] = (uint8_t)a.slab_weight[g];
      }
    }
    return;
  }
  const int per = a.slab / 64;
  for (int g = 0; g < a.n_slabs; ++g)
    for (int u = 0; u < per; ++u) {
      tb->row0[g * per + u] = a.slab_row0[g] + u * 64;
      tb->weight[g * per + u] = (uint8_t)a.slab_weight[g];
    }
}

template <int MODE>
int launch_mode(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap* mw, const CUtensorMap& mo,
                const BwdGemmParams& p, const BlockTable& tb, cudaStream_t st) {
  const int sm_count = device_sm_count();
  const size_t smem = 1024 + NSTG * BSTAGE + BOUT_BYTES + sizeof(BSmem);
  static PerDeviceOnce smem_once;
  if (int rc = ensure_dyn_smem(indexed_gemm_bwd_kernel<MODE>, (int)smem, smem_once)) return rc;
  const int grid = std::min(sm_count, p.tiles_m * p.tiles_n);
  indexed_gemm_bwd_kernel<MODE><<<grid, BGEMM_THREADS, smem, st>>>(ma, mb, mw[0], mw[1], mw[2], mw[3], mo, p, tb);
  count_launch();
  return check_launch(MODE == MODE_DX ? "indexed_gemm_bwd_kernel<dx>" : "indexed_gemm_bwd_kernel<dw>");
}

}  // namespace

int launch_gemm_bwd_dx_sm100(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, void* dx, int64_t lddx,
                             const void* bias, cudaStream_t st) {
  if (!common_ok(a, dout, lddo)) return SAF_ERR_UNSUPPORTED;
  if (lddx % 8 || !al16(dx)) return SAF_ERR_UNSUPPORTED;
  const int N = a.n_slabs * a.slab;
  CUtensorMap ma, mw[4], mo;
  int rc;
  if ((rc = map2(&ma, dout, (uint64_t)N, (uint64_t)a.M, lddo, 128))) return rc;
  for (int w = 0; w < 4; ++w) {
    const int ww = w < a.n_weights ? w : 0;
    if ((rc = map2(&mw[w], a.weights[ww], (uint64_t)a.C, (uint64_t)a.rows_w[ww], a.ldw[ww], is_halves(a) ? 32 : 64))) return rc;
  }
  if ((rc = map2(&mo, dx, (uint64_t)a.C, (uint64_t)a.M, lddx, 128))) return rc;
  BlockTable tb;
  fill_blocks(a, &tb);
  BwdGemmParams p;
  memset(&p, 0, sizeof(p));
  p.halves = is_halves(a) ? 1 : 0;
  p.I = a.M; p.J = a.C; p.KB = N / 64; p.n_blocks = N / 64;
  p.tiles_m = (a.M + BM - 1) / BM;
  p.tiles_n = (a.C + BN - 1) / BN;
  p.bias = bias;
  p.status = a.status;
  return launch_mode<MODE_DX>(ma, ma, mw, mo, p, tb, st);
}

int launch_gemm_bwd_dw_sm100(const SafIndexedLinearArgs& a, const void* dout, int64_t lddo, cudaStream_t st) {
  if (!common_ok(a, dout, lddo)) return SAF_ERR_UNSUPPORTED;
  if (a.ldx % 8 || !al16(a.x)) return SAF_ERR_UNSUPPORTED;
  for (int w = 0; w < a.n_weights; ++w)
    if (a.biases[w]) return SAF_ERR_UNSUPPORTED;   // bias gradients stay with the generic kernels
  const int N = a.n_slabs * a.slab;
  CUtensorMap ma, mb, mw[4];
  int rc;
  if ((rc = map2(&ma, dout, (uint64_t)N, (uint64_t)a.M, lddo, 64))) return rc;
  if ((rc = map2(&mb, a.x, (uint64_t)a.C, (uint64_t)a.M, a.ldx, 64))) return rc;
  for (int w = 0; w < 4; ++w) {
    const int ww = w < a.n_weights ? w : 0;
    if ((rc = map2(&mw[w], a.weights[ww], (uint64_t)a.C, (uint64_t)a.rows_w[ww], a.ldw[ww], is_halves(a) ? 32 : 64))) return rc;
  }
  BlockTable tb;
  fill_blocks(a, &tb);
  BwdGemmParams p;
  memset(&p, 0, sizeof(p));
  p.halves = is_halves(a) ? 1 : 0;
  p.I = N; p.J = a.C; p.KB = (a.M + BK - 1) / BK; p.n_blocks = N / 64;
  p.tiles_m = (p.n_blocks + 1) / 2;
  p.tiles_n = (a.C + BN - 1) / BN;
  p.status = a.status;
  return launch_mode<MODE_DW>(ma, mb, mw, ma, p, tb, st);
}

}  // namespace saf
