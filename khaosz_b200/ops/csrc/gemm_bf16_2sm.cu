// bf16 GEMM with CTA pairs (tcgen05 cta_group::2): two SMs of one cluster compute a 256x256
// output tile together.  Each CTA stages its own 128 rows of A and only *half* of the B tile
// (128 of the 256 N rows); one thread of the leader CTA issues tcgen05.mma.cta_group::2, which
// reads both CTAs' shared memory and writes each CTA's 128x256 fp32 accumulator into that
// CTA's own TMEM.  Compared with the single-CTA kernel this halves the shared-memory traffic
// per flop (the limiter of the 128x256 tile) and frees room for a 6-stage ring.
//
// Same operand conventions as gemm_bf16.cu (K-major or MN-major A and B, optional addend).
// TMA loads use the cta_group::2 form *without* multicast: every CTA loads its own data and
// only the completion bytes are counted on the leader's mbarrier.  Stage release and
// accumulator hand-over cross the pair through plain (non-multicast) commits / remote arrives.
#include "common.cuh"
#include "kb_api.h"

namespace kb {
namespace gemm2 {

constexpr int BM = 128;       // rows per CTA (256 per pair)
constexpr int BN = 256;       // columns per pair
constexpr int BN_CTA = 128;   // B rows staged by each CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = BM * BK * 2;      // 16 KiB
constexpr int B_STAGE_BYTES = BN_CTA * BK * 2;  // 16 KiB
constexpr int ATOM_BYTES = BK * 128;
constexpr int EPI_COLS = 64;
constexpr int EPI_BUF_BYTES = BM * EPI_COLS * 2;
constexpr int NUM_EPI_BUFS = 2;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + NUM_EPI_BUFS * EPI_BUF_BYTES + 256 + 1024;

struct Params {
  const __nv_bfloat16* R;
  long ldr;
  int M, N, K;
  int a_mn, b_mn;
  int epi;
  int* err;
};

// ---- cluster / pair primitives -----------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// own-CTA destination, completion bytes counted on the mbarrier at `mbar_cluster_addr`
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t mbar_cluster_addr,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(mbar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once the pair's MMAs issued so far have completed) on the mbarrier at a cluster address
__device__ __forceinline__ void umma_commit_pair(uint32_t mbar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int group_size = GROUP_M * num_n;
  const int g = t / group_size;
  const int first_m = g * GROUP_M;
  const int gm = min(num_m - first_m, GROUP_M);
  const int r = t - g * group_size;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * B_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + NUM_EPI_BUFS * EPI_BUF_BYTES);
  uint64_t* full = bars;                     // [STAGES]  (only the leader's are waited on)
  uint64_t* empty = bars + STAGES;           // [STAGES]  (each CTA waits on its own)
  uint64_t* tfull = bars + 2 * STAGES;       // [2]       (each CTA waits on its own)
  uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]       (only the leader's are waited on)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + BN - 1) / BN;
  const int num_k = (p.K + BK - 1) / BK;
  const int total = num_m * num_n;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 8);  // 4 epilogue warps in each CTA of the pair
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything crosses the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < total && ok; t += n_pairs) {
        int m_blk, n_blk;
        tile_coords(t, num_m, num_n, m_blk, n_blk);
        const int m0 = m_blk * 2 * BM + (int)rank * BM;
        const int n0 = n_blk * BN + (int)rank * BN_CTA;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          if (leader) mbar_expect_tx(&full[s], 2 * (A_STAGE_BYTES + B_STAGE_BYTES));
          const uint32_t bar = mapa_u32(smem_u32(&full[s]), 0);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d_pair(a_dst, &tmap_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d_pair(a_dst + a * ATOM_BYTES, &tmap_a, bar, m0 + a * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(b_dst, &tmap_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int a = 0; a < BN_CTA / 64; ++a) tma_load_2d_pair(b_dst + a * ATOM_BYTES, &tmap_b, bar, n0 + a * 64, k0);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader CTA only) -------------------------------
    if (lane == 0 && leader) {
      const uint32_t idesc = umma_idesc(2 * BM, BN, p.a_mn != 0, p.b_mn != 0);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int t = pair_id; t < total && ok; t += n_pairs) {
        if (!mbar_wait(&tempty[acc], aph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t a_desc = p.a_mn ? umma_desc_mnmajor(a_addr, j * UMMA_K, ATOM_BYTES)
                                           : umma_desc_kmajor(a_addr, j * UMMA_K * 2);
            const uint64_t b_desc = p.b_mn ? umma_desc_mnmajor(b_addr, j * UMMA_K, ATOM_BYTES)
                                           : umma_desc_kmajor(b_addr, j * UMMA_K * 2);
            umma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          const uint32_t e_local = smem_u32(&empty[s]);
          umma_commit_pair(mapa_u32(e_local, 0));
          umma_commit_pair(mapa_u32(e_local, 1));
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        const uint32_t f_local = smem_u32(&tfull[acc]);
        umma_commit_pair(mapa_u32(f_local, 0));
        umma_commit_pair(mapa_u32(f_local, 1));
        if (++acc == 2) {
          acc = 0;
          aph ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -------------------------------
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    int acc = 0;
    uint32_t aph = 0;
    int buf = 0;
    bool ok = true;
    for (int t = pair_id; t < total && ok; t += n_pairs) {
      int m_blk, n_blk;
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      const int m0 = m_blk * 2 * BM + (int)rank * BM, n0 = n_blk * BN;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int grow = m0 + row_in_tile;
#pragma unroll 1
      for (int c = 0; c < BN / EPI_COLS; ++c) {
        const int col0 = n0 + c * EPI_COLS;
        if (col0 >= p.N) break;
        uint32_t v[EPI_COLS];
        tmem_ld_32x32b_x32(t_row + c * EPI_COLS, v);
        tmem_ld_32x32b_x32(t_row + c * EPI_COLS + 32, v + 32);
        tmem_ld_wait();
        if (epi_tid == 0) tma_store_wait_read<NUM_EPI_BUFS - 1>();
        named_barrier_sync(1, 128);
        uint8_t* stage = sEpi + buf * EPI_BUF_BYTES;
        const bool row_ok = grow < p.M;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[ch * 8 + e]);
          if (p.epi == 1 && row_ok && (col0 + ch * 8) < p.N) {
            const uint4 rv = *reinterpret_cast<const uint4*>(p.R + (size_t)grow * p.ldr + col0 + ch * 8);
            const float2 r0 = unpack_bf16x2(rv.x), r1 = unpack_bf16x2(rv.y), r2 = unpack_bf16x2(rv.z),
                         r3 = unpack_bf16x2(rv.w);
            f[0] += r0.x; f[1] += r0.y; f[2] += r1.x; f[3] += r1.y;
            f[4] += r2.x; f[5] += r2.y; f[6] += r3.x; f[7] += r3.y;
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]);
          o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]);
          o.w = pack_bf16x2(f[6], f[7]);
          *reinterpret_cast<uint4*>(stage + sw128_offset(row_in_tile, ch)) = o;
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (epi_tid == 0 && m0 < p.M) {
          tma_store_2d(&tmap_c, stage, col0, m0);
          tma_store_commit();
        }
        buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));  // the leader's barrier
      if (++acc == 2) {
        acc = 0;
        aph ^= 1u;
      }
    }
    if (epi_tid == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nothing of the pair touches the other CTA's memory after this point
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm2
}  // namespace kb

extern "C" int kb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                                 long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi,
                                 void* stream) {
  using namespace kb::gemm2;
  if (M <= 0 || N <= 0 || K <= 0) return KB_STATUS_BAD_ARG;
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(A) || misaligned(B) || misaligned(C) || (lda & 7) || (ldb & 7) || (ldc & 7)) return KB_STATUS_BAD_ARG;
  if (epi == 1 && (R == nullptr || misaligned(R) || (ldr & 7) || (N & 7))) return KB_STATUS_BAD_ARG;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  static int sm_count[64] = {0};
  if (sm_count[dev] == 0) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);

  CUtensorMap ta, tb, tc;
  int rc;
  if (!a_mn) rc = kb::make_tmap_2d(&ta, A, 2, M, K, lda * 2, BM, BK, true);
  else       rc = kb::make_tmap_2d(&ta, A, 2, K, M, lda * 2, BK, 64, true);
  if (rc) return KB_STATUS_TMAP_ERROR;
  if (!b_mn) rc = kb::make_tmap_2d(&tb, B, 2, N, K, ldb * 2, BN_CTA, BK, true);
  else       rc = kb::make_tmap_2d(&tb, B, 2, K, N, ldb * 2, BK, 64, true);
  if (rc) return KB_STATUS_TMAP_ERROR;
  rc = kb::make_tmap_2d(&tc, C, 2, M, N, ldc * 2, BM, EPI_COLS, true);
  if (rc) return KB_STATUS_TMAP_ERROR;

  Params p;
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ldr = ldr;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.epi = epi;
  p.err = kb::error_word(dev);

  const int total = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int pairs = sm_count[dev] / 2;
  if (total < pairs) pairs = total;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel, ta, tb, tc, p);
  return e == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}
