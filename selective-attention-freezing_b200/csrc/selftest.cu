// Diagnostics that exercise the library's own safety nets without faulting or hanging anything.
#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {
namespace {

// One CTA waits on an mbarrier that nobody will ever arrive on.  The bounded wait runs out after `limit_ns`,
// the CTA records (SAF_DEV_TIMEOUT_SELFTEST | 99 << 8) in *status exactly as the production kernels record
// their own give-ups, and returns normally: the context stays usable.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  const bool ok = mbar_wait_limit(&bar, 0, limit_ns);
  // group-uniform decision, the way the kernels take it before a named barrier
  const bool gave_up = named_bar_or(1, blockDim.x, !ok);
  if (gave_up && threadIdx.x == 0) dev_set_error(status, SAF_DEV_TIMEOUT_SELFTEST, 99);
}

// Cycles per tcgen05.mma instruction (K = 16, bf16, M = 128) for the operand forms the kernels use, issued back to
// back by one thread into one accumulator with nothing else running on the SM.  This is the tensor pipe's own pace
// when the shared-memory operands are the only shared-memory traffic; the kernels' traces are read against it.
//   form 0  A smem K-major,  B smem K-major,  N 128   (S = Q K^T, S^T, dP^T)
//   form 1  A TMEM,          B smem MN-major, N 128   (dV, dK, dQ; P V at head_dim 128)
//   form 2  A TMEM,          B smem MN-major, N 64    (P V at head_dim 64)
//   form 3  A smem MN-major, B smem MN-major, N 256   (weight gradient)
//   form 4  A smem K-major,  B smem K-major,  N 256   (projection GEMM)
//   form 5  A TMEM,          B smem K-major,  N 128
//   form 6  A smem K-major,  B smem K-major,  N 64
//   form 7  A smem K-major,  B smem MN-major, N 128
//   forms 8-11  see mr_issue_group
constexpr int MR_FORMS = 22;
constexpr int MR_SMEM = 160 * 1024;
template <int FORM>
__device__ __forceinline__ void mr_issue(uint32_t tmem, uint32_t a, uint32_t b, int ks, bool acc) {
  const uint32_t offk = (ks >> 2) * 16384 + (ks & 3) * 32;       // K-major 128 x 128 tile: two 64-wide slabs
  const uint32_t offm = ks * 2048;                               // MN-major: 16 rows of 128 bytes per K step
  const uint32_t ta = tmem + 256 + (ks >> 2) * 64 + (ks & 3) * 8;
  if (FORM == 0) umma_ss(tmem, umma_smem_desc_sw128(a + offk, 16, 1024), umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), acc);
  if (FORM == 1) umma_ts(tmem, ta, umma_smem_desc_sw128(b + offm, 16384, 1024), umma_idesc_bf16(128, 128, 0, 1), acc);
  if (FORM == 2) umma_ts(tmem, tmem + 256 + ks * 8, umma_smem_desc_sw128(b + offm, 16384, 1024), umma_idesc_bf16(128, 64, 0, 1), acc);
  if (FORM == 3) umma_ss(tmem, umma_smem_desc_sw128(a + (ks & 3) * 2048, 8192, 1024), umma_smem_desc_sw128(b + (ks & 3) * 2048, 8192, 1024), umma_idesc_bf16(128, 256, 1, 1), acc);
  if (FORM == 4) umma_ss(tmem, umma_smem_desc_sw128(a + (ks & 3) * 32, 16, 1024), umma_smem_desc_sw128(b + (ks & 3) * 32, 16, 1024), umma_idesc_bf16(128, 256, 0, 0), acc);
  if (FORM == 5) umma_ts(tmem, ta, umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), acc);
  if (FORM == 6) umma_ss(tmem, umma_smem_desc_sw128(a + offk, 16, 1024), umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 64, 0, 0), acc);
  if (FORM == 7) umma_ss(tmem, umma_smem_desc_sw128(a + offk, 16, 1024), umma_smem_desc_sw128(b + offm, 16384, 1024), umma_idesc_bf16(128, 128, 0, 1), acc);
}
// forms 8-11: the instructions of forms 0 / 1 with operand addresses that change from one group of eight to the next
// (ring stages), so the descriptors cannot be built once for the whole run: built per instruction from the address
// (8, 9), or once per group and advanced by adding the byte offset to the descriptor's low word (10, 11)
template <int FORM>
__device__ __forceinline__ void mr_issue_group(uint32_t tmem, uint32_t tmem_a, uint32_t a, uint32_t b, bool first) {
  // tmem: the accumulator; tmem_a: column 0 of the allocation (TMEM operands sit at fixed columns 256-383 of it)
  if (FORM == 8) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t offk = (ks >> 2) * 16384 + (ks & 3) * 32;
      umma_ss(tmem, umma_smem_desc_sw128(a + offk, 16, 1024), umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), !first || ks > 0);
    }
  }
  if (FORM == 9) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_ts(tmem, tmem_a + 256 + (ks >> 2) * 64 + (ks & 3) * 8, umma_smem_desc_sw128(b + ks * 2048, 16384, 1024), umma_idesc_bf16(128, 128, 0, 1), !first || ks > 0);
  }
  if (FORM == 10) {
    const uint64_t da = umma_smem_desc_sw128(a, 16, 1024), db = umma_smem_desc_sw128(b, 16, 1024);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t offk = (ks >> 2) * 16384 + (ks & 3) * 32;
      umma_ss(tmem, umma_desc_advance(da, offk), umma_desc_advance(db, offk), umma_idesc_bf16(128, 128, 0, 0), !first || ks > 0);
    }
  }
  // forms 12-15: what a change of product costs.  Every group of eight is a product of its own (its first instruction
  // overwrites the accumulator): 12 two accumulators taking turns, a commit after each group; 13 the same without the
  // commits; 14 smem-operand and TMEM-operand products taking turns on two accumulators, with commits (the dV, S^T
  // sequence of the backward); 15 one accumulator, a commit after each group
  if (FORM == 12 || FORM == 13 || FORM == 15) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t offk = (ks >> 2) * 16384 + (ks & 3) * 32;
      umma_ss(tmem, umma_smem_desc_sw128(a + offk, 16, 1024), umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), ks > 0);
    }
  }
  if (FORM == 14) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t offk = (ks >> 2) * 16384 + (ks & 3) * 32;
      if (first) umma_ss(tmem, umma_smem_desc_sw128(a + offk, 16, 1024), umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), ks > 0);
      else umma_ts(tmem, tmem_a + 256 + (ks >> 2) * 64 + (ks & 3) * 8, umma_smem_desc_sw128(b + ks * 2048, 16384, 1024), umma_idesc_bf16(128, 128, 0, 1), ks > 0);
    }
  }
  // forms 16-18: the products of one key step of the forward at head_dim 64, in turn, a commit after each.
  //   16  scores from a TMEM operand (Q), 64 keys: 4 instructions N 64 | P V from a TMEM operand: 4 instructions N 64
  //   17  scores from shared memory, 128 keys: 4 instructions N 128    | P V from a TMEM operand: 8 instructions N 64
  //   18  as 17 with the two score products of a step back to back, then the two P V products
  if (FORM == 16) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      if (first) umma_ts(tmem, tmem_a + 256 + ks * 8, umma_smem_desc_sw128(b + ks * 32, 16, 1024), umma_idesc_bf16(128, 64, 0, 0), ks > 0);
      else umma_ts(tmem, tmem_a + 320 + ks * 8, umma_smem_desc_sw128(b + 16384 + ks * 2048, 16384, 1024), umma_idesc_bf16(128, 64, 0, 1), ks > 0);
    }
  }
  if (FORM == 17 || FORM == 18) {
    if (first) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        umma_ss(tmem, umma_smem_desc_sw128(a + ks * 32, 16, 1024), umma_smem_desc_sw128(b + ks * 32, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), ks > 0);
    } else {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_ts(tmem, tmem_a + 256 + ks * 8, umma_smem_desc_sw128(b + 16384 + ks * 2048, 16384, 1024), umma_idesc_bf16(128, 64, 0, 1), ks > 0);
    }
  }
  // forms 19-21: form 14 (the backward's sequence) with one thing changed.  19: the TMEM-operand product issued as two
  // halves of N 64 (16 instructions); 20: its B operand K-major; 21: its A operand in consecutive columns
  if (FORM == 19 || FORM == 20 || FORM == 21) {
    if (first) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t offk = (ks >> 2) * 16384 + (ks & 3) * 32;
        umma_ss(tmem, umma_smem_desc_sw128(a + offk, 16, 1024), umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), ks > 0);
      }
    } else if (FORM == 19) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
          umma_ts(tmem + hh * 64, tmem_a + 256 + (ks >> 2) * 64 + (ks & 3) * 8, umma_smem_desc_sw128(b + hh * 16384 + ks * 2048, 16384, 1024), umma_idesc_bf16(128, 64, 0, 1), ks > 0);
    } else if (FORM == 20) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t offk = (ks >> 2) * 16384 + (ks & 3) * 32;
        umma_ts(tmem, tmem_a + 256 + (ks >> 2) * 64 + (ks & 3) * 8, umma_smem_desc_sw128(b + offk, 16, 1024), umma_idesc_bf16(128, 128, 0, 0), ks > 0);
      }
    } else {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_ts(tmem, tmem_a + 256 + ks * 8, umma_smem_desc_sw128(b + ks * 2048, 16384, 1024), umma_idesc_bf16(128, 128, 0, 1), ks > 0);
    }
  }
  if (FORM == 11) {
    const uint64_t db = umma_smem_desc_sw128(b, 16384, 1024);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      umma_ts(tmem, tmem_a + 256 + (ks >> 2) * 64 + (ks & 3) * 8, umma_desc_advance(db, ks * 2048), umma_idesc_bf16(128, 128, 0, 1), !first || ks > 0);
  }
}

// Neighbour load while the instructions run (flags of `load`), as in the kernels, where the issuer never has the SM
// to itself:
//   1  eight other warps keep reading the accumulator and writing packed operands in tensor memory (tcgen05.ld / st)
//   2  eight other warps keep the FMA and special-function pipes busy (two of them share the issuer's scheduler)
//   4  one thread keeps pairs of 32 KB bulk copies from global into shared memory in flight (what TMA loads do to
//      the shared-memory write port)
constexpr int MR_THREADS = 320;          // warps 0-7 neighbours, warp 8 issuer, warp 9 copy thread
constexpr int MR_COPY_BYTES = 32 * 1024;
__device__ uint4 g_mr_src[MR_COPY_BYTES / 16];

__device__ __forceinline__ void mr_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

struct MrShared2 {
  uint64_t bar, copy_bar, group_bar;
  uint32_t tmem_base;
  volatile int done;
};

template <int FORM>
__global__ void __launch_bounds__(MR_THREADS, 1)
mma_rate_kernel(int reps, int random_operands, int load, long long* cycles, int* status) {
  extern __shared__ uint8_t mr_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)mr_smem_raw + 1023) & ~(uintptr_t)1023);
  MrShared2* sh = reinterpret_cast<MrShared2*>(smem + MR_SMEM);
  const int tid = threadIdx.x, warp = tid >> 5;
  // operands: zeros, or bf16 values of both signs between 0.5 and 2 in magnitude
  auto word = [&](uint32_t i) -> uint32_t {
    if (!random_operands) return 0u;
    uint32_t h = i * 2654435761u + 0x9e3779b9u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    return (h & 0x80ff80ffu) | 0x3f003f00u;
  };
  for (int i = tid; i < MR_SMEM / 4; i += MR_THREADS) reinterpret_cast<uint32_t*>(smem)[i] = word((uint32_t)i + blockIdx.x * 7919u);
  if (tid == 0) {
    mbar_init(&sh->bar, 1);
    mbar_init(&sh->copy_bar, 1);
    mbar_init(&sh->group_bar, 1);
    sh->done = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(&sh->tmem_base, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  if (warp < 4) {
    uint32_t z[32];
    for (int c = 0; c < 512; c += 32) {                                                         // finite TMEM operands
#pragma unroll
      for (int i = 0; i < 32; ++i) z[i] = c >= 256 ? word((uint32_t)(tid * 512 + c + i)) : 0u;
      tmem_st32(tmem + lane_base + c, z);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 8) {
    const bool leader = elect_one();
    const uint32_t a = smem_u32(smem), b = a + 32 * 1024;
    long long t0 = 0;
    if (leader) {
      t0 = clock64();
      if (FORM >= 19) {
        for (int r = 0; r < reps; ++r) {
          const bool odd = r & 1;
          mr_issue_group<FORM>(tmem + (odd ? 128 : 0), tmem, a, b, !odd);
          umma_commit(&sh->group_bar);
        }
      } else if (FORM >= 16) {
        // r-th product: 16, 17 alternate the two kinds; 18 issues them as score, score, P V, P V
        for (int r = 0; r < reps; ++r) {
          const bool scores = FORM == 18 ? (r & 2) == 0 : (r & 1) == 0;
          mr_issue_group<FORM>(tmem + (scores ? (r & 1) * 128 : 384 + (r & 1) * 64), tmem, a, b, scores);
          umma_commit(&sh->group_bar);
        }
      } else if (FORM >= 12) {
        for (int r = 0; r < reps; ++r) {
          const bool odd = r & 1;
          mr_issue_group<FORM>(tmem + ((FORM != 15 && odd) ? 128 : 0), tmem, a, b, FORM == 14 ? !odd : true);
          if (FORM != 13) umma_commit(&sh->group_bar);          // nobody waits on it: the phases just go by
        }
      } else if (FORM >= 8) {
        uint32_t stage = 0;
        for (int r = 0; r < reps; ++r) {
          mr_issue_group<FORM>(tmem, tmem, a + stage * 1024, b + stage * 1024, r == 0);
          stage = stage == 2 ? 0 : stage + 1;
        }
      } else {
        for (int r = 0; r < reps; ++r) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) mr_issue<FORM>(tmem, a, b, ks, (r | ks) != 0);
        }
      }
      umma_commit(&sh->bar);
    }
    __syncwarp();
    const bool ok = mbar_wait(&sh->bar, 0);
    if (leader) {
      const long long t1 = clock64();
      if (!ok) dev_set_error(status, SAF_DEV_TIMEOUT_SELFTEST, 98);
      if (blockIdx.x == 0) *cycles = t1 - t0;
      sh->done = 1;
    }
    __syncwarp();
  } else if (warp == 9) {
    if ((load & 4) && (tid & 31) == 0) {
      // two 32 KB copies per round (the size of a Q and a dO tile) into [96 KB, 160 KB) of the buffer, which no
      // operand form reads; at most 4096 rounds
      for (int n = 0; n < 4096 && !sh->done; ++n) {
        mbar_expect_tx(&sh->copy_bar, 2 * MR_COPY_BYTES);
        mr_bulk_g2s(smem + 96 * 1024, g_mr_src, MR_COPY_BYTES, &sh->copy_bar);
        mr_bulk_g2s(smem + 128 * 1024, g_mr_src, MR_COPY_BYTES, &sh->copy_bar);
        if (!mbar_wait(&sh->copy_bar, n & 1)) {
          dev_set_error(status, SAF_DEV_TIMEOUT_SELFTEST, 97);
          break;
        }
      }
    }
  } else {
    // neighbours: bounded loops that end when the issuer has seen its last instruction retire
    float acc = (float)tid;
    for (int n = 0; n < 100000 && !sh->done; ++n) {
      if (load & 1) {
        uint32_t d[32], pk[16];
        tmem_ld32(tmem + lane_base + (n & 3) * 32, d);          // the accumulator the instructions write
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 16; ++x) pk[x] = d[2 * x] ^ d[2 * x + 1];
        tmem_st16(tmem + lane_base + 384 + (warp >> 2) * 16, pk);    // columns no instruction reads
        tmem_st_wait();
      }
      if (load & 2) {
        // sixteen independent chains, as the softmax / dS arithmetic has: the warp can issue every cycle, so the
        // schedulers (the issuer's among them) are kept as busy as the kernels keep them
        float c[16];
#pragma unroll
        for (int x = 0; x < 16; ++x) c[x] = acc + (float)x;
#pragma unroll
        for (int y = 0; y < 8; ++y) {
#pragma unroll
          for (int x = 0; x < 16; ++x) c[x] = fmaf(c[x], 0.9999f, 0.5f);
#pragma unroll
          for (int x = 0; x < 16; x += 4) asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(c[x]) : "f"(c[x] * 1e-9f));
        }
#pragma unroll
        for (int x = 0; x < 16; ++x) acc += c[x] * 1e-9f;
      }
      if (!(load & 3)) __nanosleep(200);
    }
    if (acc == 12345.678f) *cycles = 0;   // keeps the arithmetic alive
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
}

template <int FORM>
int mr_launch(int reps, int random_operands, int load, long long* cycles, int* status, cudaStream_t st) {
  static PerDeviceOnce once;
  const int smem = MR_SMEM + 2048;
  if (int rc = ensure_dyn_smem(mma_rate_kernel<FORM>, smem, once)) return rc;
  mma_rate_kernel<FORM><<<device_sm_count(), MR_THREADS, smem, st>>>(reps, random_operands, load, cycles, status);
  count_launch();
  return check_launch("mma_rate_kernel");
}

}  // namespace
}  // namespace saf

using namespace saf;

extern "C" int saf_selftest_mma_rate(int form, int reps, long long* cycles, int* status, void* stream) {
  if (!cycles) return fail(SAF_ERR_INVALID, "cycles must be a device pointer to an int64 word");
  if (reps <= 0 || reps > 4096) return fail(SAF_ERR_INVALID, "reps must lie in [1, 4096]");
  if (form < 0 || form > 0xfff) return fail(SAF_ERR_INVALID, "form must lie in [0, 4096)");
  if (!saf_device_supported()) return fail(SAF_ERR_UNSUPPORTED, "the MMA rate probe needs an sm_100 device");
  cudaStream_t st = (cudaStream_t)stream;
  const int rnd = (form >> 8) & 1;          // + 256: random operands instead of zeros
  const int load = (form >> 9) & 7;         // + 512 / 1024 / 2048: neighbour load (tensor memory / arithmetic / bulk copies)
  switch (form & 255) {
    case 0: return mr_launch<0>(reps, rnd, load, cycles, status, st);
    case 1: return mr_launch<1>(reps, rnd, load, cycles, status, st);
    case 2: return mr_launch<2>(reps, rnd, load, cycles, status, st);
    case 3: return mr_launch<3>(reps, rnd, load, cycles, status, st);
    case 4: return mr_launch<4>(reps, rnd, load, cycles, status, st);
    case 5: return mr_launch<5>(reps, rnd, load, cycles, status, st);
    case 6: return mr_launch<6>(reps, rnd, load, cycles, status, st);
    case 7: return mr_launch<7>(reps, rnd, load, cycles, status, st);
    case 8: return mr_launch<8>(reps, rnd, load, cycles, status, st);
    case 9: return mr_launch<9>(reps, rnd, load, cycles, status, st);
    case 10: return mr_launch<10>(reps, rnd, load, cycles, status, st);
    case 11: return mr_launch<11>(reps, rnd, load, cycles, status, st);
    case 12: return mr_launch<12>(reps, rnd, load, cycles, status, st);
    case 13: return mr_launch<13>(reps, rnd, load, cycles, status, st);
    case 14: return mr_launch<14>(reps, rnd, load, cycles, status, st);
    case 15: return mr_launch<15>(reps, rnd, load, cycles, status, st);
    case 16: return mr_launch<16>(reps, rnd, load, cycles, status, st);
    case 17: return mr_launch<17>(reps, rnd, load, cycles, status, st);
    case 18: return mr_launch<18>(reps, rnd, load, cycles, status, st);
    case 19: return mr_launch<19>(reps, rnd, load, cycles, status, st);
    case 20: return mr_launch<20>(reps, rnd, load, cycles, status, st);
    case 21: return mr_launch<21>(reps, rnd, load, cycles, status, st);
  }
  return fail(SAF_ERR_INVALID, "operand form must lie in [0, %d)", MR_FORMS);
}

extern "C" int saf_selftest_wait_timeout(int* status, int64_t limit_ns, void* stream) {
  if (!status) return fail(SAF_ERR_INVALID, "status must be a device pointer to an int32 word");
  if (limit_ns <= 0 || limit_ns > 100000000) return fail(SAF_ERR_INVALID, "limit_ns must lie in (0, 1e8]");
  wait_timeout_selftest_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(status, (unsigned long long)limit_ns);
  count_launch();
  return check_launch("wait_timeout_selftest_kernel");
}
