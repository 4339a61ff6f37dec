// bf16 GEMM with CTA pairs (tcgen05 cta_group::2): two SMs of one cluster compute a 256 x BN
// output tile together (BN = 256, 192 or 128, chosen per problem).  Each CTA stages its own
// 128 rows of A and only *half* of the B tile (BN/2 of the BN rows); one thread of the leader
// CTA issues tcgen05.mma.cta_group::2, which reads both CTAs' shared memory and writes each
// CTA's 128 x BN fp32 accumulator into that CTA's own TMEM.  Compared with a single-CTA
// 128 x BN tile this halves the shared-memory (and L2) traffic of B per flop.
//
//   C[M,N] = op(A) * op(B)^T (+ R)                       epi 0 / 1
//   H[M,F] = up * silu(gate),  [gate | up] = A * W^T      epi 2 (SwiGLU epilogue)
//
// Same operand conventions as gemm_bf16.cu (K-major or MN-major A and B).  TMA loads use the
// cta_group::2 form *without* multicast: every CTA loads its own data and only the completion
// bytes are counted on the leader's mbarrier.  Stage release and accumulator hand-over cross
// the pair through plain (non-multicast) commits / remote arrives.
//
// SwiGLU epilogue: W is the stacked [2F, K] weight (gate rows first).  CTA 0 of a pair stages
// BN/2 gate rows, CTA 1 the BN/2 up rows of the same features, so every accumulator row holds
// gate values in columns [0, BN/2) and the matching up values in [BN/2, BN): the epilogue
// writes gate and up (the backward pass needs them) and h = up * silu(gate) from one pass over
// TMEM, and the separate SwiGLU kernel with its re-read of [M, 2F] disappears.
//
// Tail balancing as in gemm_bf16.cu: the tiles of the last, partial wave of pairs are cut into
// K slices; a slice parks its fp32 accumulator in a workspace and the CTA whose slice arrives
// last sums the slices in slice order (deterministic) and runs the epilogue.
// All waits are bounded (see common.cuh).
#include "common.cuh"
#include "kb_api.h"

namespace kb {
namespace gemm2 {

constexpr int BM = 128;  // rows per CTA (256 per pair)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int ATOM_BYTES = BK * 128;
constexpr int EPI_COLS = 64;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 256;  // TMEM columns between the two accumulators
constexpr int GROUP_M = 8;
constexpr int NUM_THREADS = 192;

template <int BN>
struct Cfg {
  static constexpr int BN_CTA = BN / 2;  // B rows staged by each CTA
  static constexpr int B_STAGE_BYTES = BN_CTA * BK * 2;
  // the whole shared memory is operand ring (the epilogue stores rows straight from registers): the
  // kernel's speed follows the bytes it keeps in flight
  static constexpr int STAGES = BN == 256 ? 7 : (BN == 192 ? 8 : 9);
  static constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 256 + 1024;
};

struct Params {
  __nv_bfloat16* C;   // output (epi 2: gate part of GU)
  __nv_bfloat16* C2;  // epi 2: up part of GU
  __nv_bfloat16* H;   // epi 2: up * silu(gate)
  long ldc, ldh;
  const __nv_bfloat16* R;
  long ldr;
  int M, N, K;  // epi 2: N is the number of features F (the GEMM itself is 2F wide)
  int a_mn, b_mn;
  int epi;  // 0 none, 1 += R, 2 SwiGLU
  int up_row0;  // epi 2: first up row of W (= F)
  int* err;
  // tail balancing
  int full_tiles;
  int split;
  float* ws;               // [(total - full_tiles) * split][2 CTAs][BM][BN] fp32
  unsigned int* counters;  // [(total - full_tiles)][2 CTAs], zero between launches
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

// Work unit u -> tile and k-block range (see gemm_bf16.cu).
__device__ __forceinline__ void unit_info(const Params& p, int u, int num_k, int& tile, int& kb0, int& kb1, int& rem_idx,
                                          int& slice) {
  if (u < p.full_tiles || p.split <= 1) {
    tile = u; kb0 = 0; kb1 = num_k; rem_idx = -1; slice = 0;
    return;
  }
  const int r = u - p.full_tiles;
  rem_idx = r / p.split;
  slice = r - rem_idx * p.split;
  tile = p.full_tiles + rem_idx;
  const int per = (num_k + p.split - 1) / p.split;
  kb0 = slice * per;
  kb1 = min(num_k, kb0 + per);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return u * g / (1.f + __expf(-g)); }

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const Params p) {
  constexpr int STAGES = Cfg<BN>::STAGES;
  constexpr int BN_CTA = Cfg<BN>::BN_CTA;
  constexpr int B_STAGE_BYTES = Cfg<BN>::B_STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * B_STAGE_BYTES);
  uint64_t* full = bars;                     // [STAGES]  (only the leader's are waited on)
  uint64_t* empty = bars + STAGES;           // [STAGES]  (each CTA waits on its own)
  uint64_t* tfull = bars + 2 * STAGES;       // [2]       (each CTA waits on its own)
  uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]       (only the leader's are waited on)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const bool swiglu = p.epi == 2;
  // output columns covered by one tile: BN, or BN/2 features with the SwiGLU epilogue
  const int n_per_tile = swiglu ? BN_CTA : BN;

  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + n_per_tile - 1) / n_per_tile;
  const int num_k = (p.K + BK - 1) / BK;
  const int total = p.full_tiles + (num_m * num_n - p.full_tiles) * p.split;  // work units

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
      for (int u = pair_id; u < total && ok; u += n_pairs) {
        int t, kb0, kb1, rem_idx, slice, m_blk, n_blk;
        unit_info(p, u, num_k, t, kb0, kb1, rem_idx, slice);
        tile_coords(t, num_m, num_n, m_blk, n_blk);
        const int m0 = m_blk * 2 * BM + (int)rank * BM;
        // B rows (or columns, MN-major) this CTA stages
        const int n0 = swiglu ? n_blk * BN_CTA + (int)rank * p.up_row0 : n_blk * BN + (int)rank * BN_CTA;
        for (int kb = kb0; kb < kb1; ++kb) {
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
      for (int u = pair_id; u < total && ok; u += n_pairs) {
        int t, kb0, kb1, rem_idx, slice;
        unit_info(p, u, num_k, t, kb0, kb1, rem_idx, slice);
        if (!mbar_wait(&tempty[acc], aph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        for (int kb = kb0; kb < kb1; ++kb) {
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
            umma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb > kb0 || j) ? 1u : 0u);
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
    bool ok = true;
    // 64 bf16 values of this thread's row (packed in pairs) -> 128 contiguous bytes of the output row
    auto emit = [&](__nv_bfloat16* dst, long ld, const uint32_t (&o)[EPI_COLS / 2], int col0, int grow_) {
      if (grow_ >= p.M) return;
      uint4* d = reinterpret_cast<uint4*>(dst + (size_t)grow_ * ld + col0);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        if (col0 + ch * 8 < p.N) d[ch] = make_uint4(o[ch * 4], o[ch * 4 + 1], o[ch * 4 + 2], o[ch * 4 + 3]);
    };
    for (int u = pair_id; u < total && ok; u += n_pairs) {
      int t, kb0, kb1, rem_idx, slice, m_blk, n_blk;
      unit_info(p, u, num_k, t, kb0, kb1, rem_idx, slice);
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      const int m0 = m_blk * 2 * BM + (int)rank * BM, n0 = n_blk * n_per_tile;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * ACC_STRIDE;
      const int grow = m0 + row_in_tile;
      bool finish = true;
      const float* sum_base = nullptr;  // != nullptr: the accumulator is the sum of the parked slices
      if (rem_idx >= 0) {
        // K slice of a tail tile: park the fp32 accumulator ([16-byte group][row] so that a warp's
        // accesses are contiguous); the last slice to arrive finishes the tile
        float* slab = p.ws + ((size_t)(rem_idx * p.split + slice) * 2 + rank) * (BM * BN);
        uint4* mine = reinterpret_cast<uint4*>(slab) + row_in_tile;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            __stcg(mine + (size_t)(c * 8 + i) * BM, make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
        }
        __threadfence();
        named_barrier_sync(1, 128);
        if (epi_tid == 0) {
          unsigned int* ctr = &p.counters[rem_idx * 2 + rank];
          const unsigned int prev = atomicAdd(ctr, 1u);
          const int last = prev == (unsigned int)(p.split - 1);
          if (last) *ctr = 0u;  // re-armed for the next launch
          s_last = last;
          __threadfence();
        }
        named_barrier_sync(1, 128);
        finish = s_last != 0;
        sum_base = p.ws + ((size_t)(rem_idx * p.split) * 2 + rank) * (BM * BN);
      }
      // 32 fp32 accumulator columns [col, col + 32) of this thread's row
      auto load32 = [&](int col, float (&f)[32]) {
        if (sum_base == nullptr) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + col, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = 0.f;
          const uint4* src = reinterpret_cast<const uint4*>(sum_base) + (size_t)(col / 4) * BM + row_in_tile;
          for (int sl = 0; sl < p.split; ++sl) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint4 w = __ldcg(src + (size_t)i * BM);
              f[4 * i + 0] += __uint_as_float(w.x);
              f[4 * i + 1] += __uint_as_float(w.y);
              f[4 * i + 2] += __uint_as_float(w.z);
              f[4 * i + 3] += __uint_as_float(w.w);
            }
            src += (size_t)2 * (BM * BN / 4);
          }
        }
      };
      if (finish && !swiglu) {
#pragma unroll 1
        for (int c = 0; c < BN / EPI_COLS; ++c) {
          const int col0 = n0 + c * EPI_COLS;
          if (col0 >= p.N) break;  // uniform across the CTA
          uint32_t o[EPI_COLS / 2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float f[32];
            load32(c * EPI_COLS + h * 32, f);
            if (p.epi == 1 && grow < p.M) {
#pragma unroll
              for (int g8 = 0; g8 < 4; ++g8) {
                const int col = col0 + h * 32 + g8 * 8;
                if (col < p.N) {
                  const uint4 rv = *reinterpret_cast<const uint4*>(p.R + (size_t)grow * p.ldr + col);
                  const float2 r0 = unpack_bf16x2(rv.x), r1 = unpack_bf16x2(rv.y), r2 = unpack_bf16x2(rv.z),
                               r3 = unpack_bf16x2(rv.w);
                  float* ff = f + g8 * 8;
                  ff[0] += r0.x; ff[1] += r0.y; ff[2] += r1.x; ff[3] += r1.y;
                  ff[4] += r2.x; ff[5] += r2.y; ff[6] += r3.x; ff[7] += r3.y;
                }
              }
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) o[h * 16 + i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
          }
          emit(p.C, p.ldc, o, col0, grow);
        }
      } else if (finish) {
        // gate in columns [0, BN/2), up in [BN/2, BN): 64 features per pass
#pragma unroll 1
        for (int c = 0; c < BN_CTA / EPI_COLS; ++c) {
          const int col0 = n0 + c * EPI_COLS;
          if (col0 >= p.N) break;
          uint32_t og[EPI_COLS / 2], ou[EPI_COLS / 2], oh[EPI_COLS / 2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float g[32], uu[32];
            load32(c * EPI_COLS + h * 32, g);
            load32(BN_CTA + c * EPI_COLS + h * 32, uu);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              og[h * 16 + i] = pack_bf16x2(g[2 * i], g[2 * i + 1]);
              ou[h * 16 + i] = pack_bf16x2(uu[2 * i], uu[2 * i + 1]);
              // h from the bf16-rounded gate / up, as the separate kernel computes it
              const float2 gr = unpack_bf16x2(og[h * 16 + i]), ur = unpack_bf16x2(ou[h * 16 + i]);
              oh[h * 16 + i] = pack_bf16x2(silu_mul(gr.x, ur.x), silu_mul(gr.y, ur.y));
            }
          }
          emit(p.C, p.ldc, og, col0, grow);
          emit(p.C2, p.ldc, ou, col0, grow);
          emit(p.H, p.ldh, oh, col0, grow);
        }
      }
      // accumulator fully read: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tempty[acc]), 0));  // the leader's barrier
      if (++acc == 2) {
        acc = 0;
        aph ^= 1u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nothing of the pair touches the other CTA's memory after this point
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
constexpr int MAX_SPLIT = 16;

// K slices for `rem` tail tiles on `pairs` CTA pairs: the split that minimises the length of the
// tail wave in k-blocks, a slice costing its share of the main loop plus the fp32 workspace
// round trip (about `overhead_kb` k-blocks, growing with the number of slices to sum).
static int choose_split(int rem, int pairs, int num_k, int overhead_kb, double* tail_waves) {
  int best = 1;
  double best_cost = num_k;
  if (rem > 0) {
    int cap = pairs / rem;
    if (cap > MAX_SPLIT) cap = MAX_SPLIT;
    for (int s = 2; s <= cap; ++s) {
      const int per = (num_k + s - 1) / s;
      if ((s - 1) * per >= num_k) continue;  // an empty slice
      const double cost = per + overhead_kb + 0.5 * s;
      if (cost < best_cost * 0.97) {
        best_cost = cost;
        best = s;
      }
    }
  }
  if (tail_waves) *tail_waves = rem > 0 ? best_cost / num_k : 0.0;
  return best;
}

static int split_overhead_kb() {
  static const int v = []() {
    const char* e = getenv("KHAOSZ_B200_GEMM_SPLIT_KB");
    return e ? atoi(e) : 8;
  }();
  return v;
}

static int tiles_of(int M, int N, int bn, bool swiglu) {
  const int per = swiglu ? bn / 2 : bn;
  return ((M + 2 * BM - 1) / (2 * BM)) * ((N + per - 1) / per);
}

// Estimated run time in units of "one 256x256 tile main loop" for tile width bn.
static double tile_cost(int M, int N, int K, int bn, bool swiglu, int pairs) {
  const int tiles = tiles_of(M, N, bn, swiglu);
  const int num_k = (K + BK - 1) / BK;
  double tail = 0.0;
  choose_split(tiles % pairs, pairs, num_k, split_overhead_kb(), &tail);
  // narrower tiles re-read A more often (shared memory and L2 traffic per flop)
  const double per_tile = bn == 256 ? 1.0 : bn == 192 ? 0.77 : 0.54;
  // columns past N in the last tile column are wasted work that the tile count already includes
  return (tiles / pairs + tail) * per_tile;
}

extern "C" int kb_gemm_split_space(int dev, int sms, void* stream, float** ws, unsigned int** counters);

template <int BN>
static int launch(const void* A, const void* B, void* C, void* C2, void* H, Params p, long lda, long ldb, long ldc,
                  long ldh, int dev, int sms, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_bf16_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg<BN>::SMEM_BYTES) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set[dev] = true;
  }
  const bool swiglu = p.epi == 2;
  const int b_rows = swiglu ? 2 * p.N : p.N;  // rows of B (or columns, MN-major)
  CUtensorMap ta, tb;
  int rc;
  if (!p.a_mn) rc = kb::make_tmap_2d(&ta, A, 2, p.M, p.K, lda * 2, BM, BK, true);
  else         rc = kb::make_tmap_2d(&ta, A, 2, p.K, p.M, lda * 2, BK, 64, true);
  if (rc) return KB_STATUS_TMAP_ERROR;
  if (!p.b_mn) rc = kb::make_tmap_2d(&tb, B, 2, b_rows, p.K, ldb * 2, Cfg<BN>::BN_CTA, BK, true);
  else         rc = kb::make_tmap_2d(&tb, B, 2, p.K, b_rows, ldb * 2, BK, 64, true);
  if (rc) return KB_STATUS_TMAP_ERROR;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.C2 = static_cast<__nv_bfloat16*>(C2);
  p.H = static_cast<__nv_bfloat16*>(H);
  p.ldc = ldc;
  p.ldh = ldh;
  const int total = tiles_of(p.M, p.N, BN, swiglu);
  const int num_k = (p.K + BK - 1) / BK;
  int pairs = sms / 2;
  p.full_tiles = total;
  p.split = 1;
  p.ws = nullptr;
  p.counters = nullptr;
  const int rem = total % pairs;
  if (rem > 0) {
    const int split = choose_split(rem, pairs, num_k, split_overhead_kb(), nullptr);
    if (split > 1) {
      float* ws = nullptr;
      unsigned int* counters = nullptr;
      // the single-CTA kernel's workspace: `sms` slabs of 128 x 256 floats, `sms` counters
      if (kb_gemm_split_space(dev, sms, stream, &ws, &counters) == KB_STATUS_OK) {
        p.full_tiles = total - rem;
        p.split = split;
        p.ws = ws;
        p.counters = counters;
      }
    }
  }
  const int units = p.full_tiles + (total - p.full_tiles) * p.split;
  if (units < pairs) pairs = units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg<BN>::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel<BN>, ta, tb, p);
  return e == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

static int dispatch(const void* A, const void* B, void* C, void* C2, void* H, const void* R, int M, int N, int K,
                    long lda, long ldb, long ldc, long ldh, long ldr, int a_mn, int b_mn, int epi, int up_row0, int bn,
                    void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return KB_STATUS_BAD_ARG;
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(A) || misaligned(B) || misaligned(C) || (lda & 7) || (ldb & 7) || (ldc & 7)) return KB_STATUS_BAD_ARG;
  if (N & 7) return KB_STATUS_BAD_ARG;  // rows are stored in 16-byte pieces
  if (epi == 1 && (R == nullptr || misaligned(R) || (ldr & 7))) return KB_STATUS_BAD_ARG;
  if (epi == 2 && (C2 == nullptr || H == nullptr || misaligned(C2) || misaligned(H) || (ldh & 7) || b_mn)) return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  static int sm_count[64] = {0};
  if (sm_count[dev] == 0) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  const int sms = sm_count[dev];
  const bool swiglu = epi == 2;
  // 96 columns per CTA are neither a whole number of MN-major atoms nor of 64-feature SwiGLU passes
  if (bn == 192 && (b_mn || swiglu)) return KB_STATUS_BAD_ARG;
  if (bn == 0) {
    // Measured on B200 under sustained load (the regime of a training step): the 256-wide tile wins on
    // every shape with at least one full wave; narrower tiles move more operand bytes per flop and
    // only pay off when the 256-wide tiling cannot occupy the pairs at all.
    bn = 256;
    if (tiles_of(M, N, 256, swiglu) < sms / 4 && tile_cost(M, N, K, 128, swiglu, sms / 2) < tile_cost(M, N, K, 256, swiglu, sms / 2))
      bn = 128;
  }
  Params p;
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ldr = ldr;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.epi = epi;
  p.up_row0 = up_row0;
  p.err = kb::error_word(dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (bn) {
    case 256: return launch<256>(A, B, C, C2, H, p, lda, ldb, ldc, ldh, dev, sms, st);
    case 192: return launch<192>(A, B, C, C2, H, p, lda, ldb, ldc, ldh, dev, sms, st);
    case 128: return launch<128>(A, B, C, C2, H, p, lda, ldb, ldc, ldh, dev, sms, st);
    default: return KB_STATUS_BAD_ARG;
  }
}

}  // namespace gemm2
}  // namespace kb

extern "C" int kb_gemm_bf16_pair_bn(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                                    long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi, int bn,
                                    void* stream) {
  if (epi != 0 && epi != 1) return KB_STATUS_BAD_ARG;
  return kb::gemm2::dispatch(A, B, C, nullptr, nullptr, R, M, N, K, lda, ldb, ldc, 0, ldr, a_mn, b_mn, epi, 0, bn, stream);
}

extern "C" int kb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                                 long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi,
                                 void* stream) {
  return kb_gemm_bf16_pair_bn(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, b_mn, epi, 0, stream);
}

// [gate | up] = X W^T with W = [2F, K] (gate rows first, up rows from row F), written to
// GU[M, 2F] (pitch ldgu), and H[M, F] = up * silu(gate) (pitch ldh), from one kernel.
extern "C" int kb_gemm_swiglu_bf16(const void* X, const void* W, void* GU, void* H, int M, int F, int K, long ldx,
                                   long ldw, long ldgu, long ldh, int bn, void* stream) {
  if (F <= 0 || (F & 7)) return KB_STATUS_BAD_ARG;
  void* up = static_cast<char*>(GU) + (size_t)F * 2;
  return kb::gemm2::dispatch(X, W, GU, up, H, nullptr, M, F, K, ldx, ldw, ldgu, ldh, 0, 0, 0, 2, F, bn, stream);
}
