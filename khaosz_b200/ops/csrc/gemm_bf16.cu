// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   C[M,N] = op(A) * op(B)^T (+ R)          bf16 in, fp32 accumulate in TMEM, bf16 out
//
// A is either K-major ([M,K] row-major) or MN-major ([K,M] row-major); likewise B
// ([N,K] or [K,N]).  That covers the three products of a linear layer without any
// transposed copy: forward (K,K), input gradient (K,MN) and weight gradient (MN,MN).
//
// Structure: persistent kernel, one CTA per SM, 128 x BN output tile (BN = 256, 192 or 128,
// chosen per problem to minimise idle SM-waves), BK=64.
//   warp 0      TMA producer: 4-stage ring of 128B-swizzled A/B tiles (cp.async.bulk.tensor,
//               no cluster multicast), completion on "full" mbarriers
//   warp 1      allocates 512 TMEM columns (two 128x256 fp32 accumulators) and issues
//               tcgen05.mma from one thread; tcgen05.commit releases stages / publishes
//               the accumulator
//   warps 2-5   epilogue: tcgen05.ld -> (+residual) -> bf16 -> swizzled staging tile ->
//               TMA store, overlapped with the next tile's main loop through the second
//               accumulator
// Tail balancing: tiles that fill whole waves of the SMs run as above; the tiles of the last,
// partial wave are cut into `split` slices of the K dimension so that the wave again covers
// (almost) all SMs.  A slice writes its fp32 accumulator to a workspace and bumps the tile's
// counter; the CTA whose slice arrives last sums the slices in slice order (deterministic) and
// runs the normal epilogue.  Nobody waits for anybody.  The same mechanism turns skinny
// problems (decode: M <= 256, a handful of tiles) into split-K over all SMs.
// All waits are bounded (see common.cuh).
#include <mutex>

#include "common.cuh"
#include "kb_api.h"

namespace kb {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int ATOM_BYTES = BK * 128;        // one 64-wide MN atom of an MN-major tile
constexpr int EPI_COLS = 64;
constexpr int EPI_BUF_BYTES = BM * EPI_COLS * 2;  // 16 KiB
constexpr int NUM_EPI_BUFS = 2;
constexpr int GROUP_M = 8;
constexpr int NUM_THREADS = 192;

// The N extent of the tile is a template parameter (256, 192 or 128): the launcher picks the
// one that wastes the fewest SM-waves for the problem at hand.
template <int BN>
struct Cfg {
  static constexpr int STAGES = BN == 128 ? 6 : 4;
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int TMEM_COLS = BN == 128 ? 256 : 512;
  static constexpr int SMEM_BYTES =
      STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + NUM_EPI_BUFS * EPI_BUF_BYTES + 256 + 1024;
};

struct Params {
  const __nv_bfloat16* R;  // optional addend [M,N]
  long ldr;
  int M, N, K;
  int a_mn, b_mn;
  int epi;  // 0: none, 1: += R
  int* err;
  // tail balancing
  int full_tiles;           // tiles [0, full_tiles) are computed whole
  int split;                // K slices per remaining tile (1: no splitting)
  float* ws;                // [(total - full_tiles) * split][BM][BN] fp32 partial accumulators
  unsigned int* counters;   // one per remaining tile, zero between launches
};

// Work unit u -> tile and k-block range.
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

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int group_size = GROUP_M * num_n;
  const int g = t / group_size;
  const int first_m = g * GROUP_M;
  const int gm = min(num_m - first_m, GROUP_M);
  const int r = t - g * group_size;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  constexpr int STAGES = Cfg<BN>::STAGES;
  constexpr int B_STAGE_BYTES = Cfg<BN>::B_STAGE_BYTES;
  constexpr int TMEM_COLS = Cfg<BN>::TMEM_COLS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * B_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + NUM_EPI_BUFS * EPI_BUF_BYTES);
  uint64_t* full = bars;                  // [STAGES]
  uint64_t* empty = bars + STAGES;        // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;    // [2]
  uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
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
      mbar_init(&tempty[i], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total && ok; u += gridDim.x) {
        int t, kb0, kb1, rem_idx, slice, m_blk, n_blk;
        unit_info(p, u, num_k, t, kb0, kb1, rem_idx, slice);
        tile_coords(t, num_m, num_n, m_blk, n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d(a_dst, &tmap_a, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a)
              tma_load_2d(a_dst + a * ATOM_BYTES, &tmap_a, &full[s], m0 + a * 64, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(b_dst, &tmap_b, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int a = 0; a < BN / 64; ++a)
              tma_load_2d(b_dst + a * ATOM_BYTES, &tmap_b, &full[s], n0 + a * 64, k0);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, BN, p.a_mn != 0, p.b_mn != 0);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t aph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total && ok; u += gridDim.x) {
        int t, kb0, kb1, rem_idx, slice;
        unit_info(p, u, num_k, t, kb0, kb1, rem_idx, slice);
        if (!mbar_wait(&tempty[acc], aph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
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
            umma_f16(d_tmem, a_desc, b_desc, idesc, (kb > kb0 || j) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) {
          acc = 0;
          aph ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int q = warp & 3;               // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    const int epi_tid = threadIdx.x - 64;  // 0..127
    int acc = 0;
    uint32_t aph = 0;
    int buf = 0;
    bool ok = true;
    __shared__ int s_last;
    for (int u = blockIdx.x; u < total && ok; u += gridDim.x) {
      int t, kb0, kb1, rem_idx, slice, m_blk, n_blk;
      unit_info(p, u, num_k, t, kb0, kb1, rem_idx, slice);
      tile_coords(t, num_m, num_n, m_blk, n_blk);
      const int m0 = m_blk * BM, n0 = n_blk * BN;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int grow = m0 + row_in_tile;
      // one 64-column chunk of fp32 values -> (+R) -> bf16 -> staging -> TMA store
      auto emit_chunk = [&](int c, const uint32_t (&v)[EPI_COLS]) {
        const int col0 = n0 + c * EPI_COLS;
        // staging buffer `buf` must have been drained by the TMA store issued 2 chunks ago
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
            const float2 r0 = unpack_bf16x2(rv.x), r1 = unpack_bf16x2(rv.y),
                         r2 = unpack_bf16x2(rv.z), r3 = unpack_bf16x2(rv.w);
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
        if (epi_tid == 0) {
          tma_store_2d(&tmap_c, stage, col0, m0);
          tma_store_commit();
        }
        buf ^= 1;
      };
      if (rem_idx < 0) {
#pragma unroll 1
        for (int c = 0; c < BN / EPI_COLS; ++c) {
          if (n0 + c * EPI_COLS >= p.N) break;  // uniform across the CTA
          uint32_t v[EPI_COLS];
          tmem_ld_32x32b_x32(t_row + c * EPI_COLS, v);
          tmem_ld_32x32b_x32(t_row + c * EPI_COLS + 32, v + 32);
          tmem_ld_wait();
          emit_chunk(c, v);
        }
      } else {
        // K slice of a tail tile: park the fp32 accumulator, the last slice to arrive finishes the tile
        // workspace layout per slice: [chunk][16-byte group][row] so that a warp's accesses are contiguous
        uint4* mine = reinterpret_cast<uint4*>(p.ws + ((size_t)rem_idx * p.split + slice) * (BM * BN)) + row_in_tile;
#pragma unroll 1
        for (int c = 0; c < BN / EPI_COLS; ++c) {
          if (n0 + c * EPI_COLS >= p.N) break;
          uint32_t v[EPI_COLS];
          tmem_ld_32x32b_x32(t_row + c * EPI_COLS, v);
          tmem_ld_32x32b_x32(t_row + c * EPI_COLS + 32, v + 32);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < EPI_COLS / 4; ++i)
            __stcg(mine + (size_t)(c * (EPI_COLS / 4) + i) * BM, make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
        }
        __threadfence();
        named_barrier_sync(1, 128);
        if (epi_tid == 0) {
          const unsigned int prev = atomicAdd(&p.counters[rem_idx], 1u);
          const int last = prev == (unsigned int)(p.split - 1);
          if (last) p.counters[rem_idx] = 0u;  // re-armed for the next launch
          s_last = last;
          __threadfence();
        }
        named_barrier_sync(1, 128);
        if (s_last) {
          const uint4* base = reinterpret_cast<const uint4*>(p.ws + (size_t)rem_idx * p.split * (BM * BN)) + row_in_tile;
#pragma unroll 1
          for (int c = 0; c < BN / EPI_COLS; ++c) {
            if (n0 + c * EPI_COLS >= p.N) break;
            uint32_t v[EPI_COLS];
#pragma unroll
            for (int i = 0; i < EPI_COLS; ++i) v[i] = 0u;
            for (int sl = 0; sl < p.split; ++sl) {
              const uint4* src = base + (size_t)sl * (BM * BN / 4) + (size_t)c * (EPI_COLS / 4) * BM;
#pragma unroll
              for (int i = 0; i < EPI_COLS / 4; ++i) {
                const uint4 w = __ldcg(src + (size_t)i * BM);
                v[4 * i + 0] = __float_as_uint(__uint_as_float(v[4 * i + 0]) + __uint_as_float(w.x));
                v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + __uint_as_float(w.y));
                v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + __uint_as_float(w.z));
                v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + __uint_as_float(w.w));
              }
            }
            emit_chunk(c, v);
          }
        }
      }
      // accumulator fully read: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) {
        acc = 0;
        aph ^= 1u;
      }
    }
    if (epi_tid == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace kb

namespace kb {
namespace gemm {

// k-blocks per slice at least: the workspace round trip of a slice costs about as much as 6-8
// k-blocks of main loop, so a tail is only split when its slices stay long; a problem with no
// full wave at all (decode) gains from any extra SMs
constexpr int MIN_SLICE_KB = 24;
constexpr int MIN_SLICE_KB_SKINNY = 8;
constexpr int MAX_SPLIT = 16;

// Workspace of the tail slices (at most one slice per SM) and the tile counters: one per (device,
// stream), because launches on different streams of one device may overlap (a serving thread beside a
// training loop) and a slice must find its own partials.  A device hands out at most MAX_STREAMS of
// them (19 MB each); a launch on a further stream simply runs without splitting.
struct SplitSpace {
  float* ws = nullptr;
  unsigned int* counters = nullptr;
  cudaStream_t stream = nullptr;
  bool used = false;
};
constexpr int MAX_SPLIT_STREAMS = 8;
static SplitSpace* split_space(int dev, int sms, cudaStream_t stream) {
  static SplitSpace spaces[64][MAX_SPLIT_STREAMS];
  static std::mutex mu;
  static const bool enabled = []() {
    const char* e = getenv("KHAOSZ_B200_GEMM_SPLIT");
    return !(e && e[0] == '0');
  }();
  if (!enabled || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  SplitSpace* slot = nullptr;
  for (int i = 0; i < MAX_SPLIT_STREAMS; ++i) {
    SplitSpace& sp = spaces[dev][i];
    if (sp.used && sp.stream == stream) return sp.ws ? &sp : nullptr;
    if (!sp.used && slot == nullptr) slot = &sp;
  }
  if (slot == nullptr) return spaces[dev][0].ws ? &spaces[dev][0] : nullptr;   // table full: share the first
  // A stream that is recording a CUDA graph must not allocate (the attempt would invalidate the
  // recording): its launches share the workspace that the warm-up launches of this device allocated,
  // with which the replayed graph runs in stream order.
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess) cudaGetLastError();
  if (capturing != cudaStreamCaptureStatusNone) {
    for (int i = 0; i < MAX_SPLIT_STREAMS; ++i)
      if (spaces[dev][i].used && spaces[dev][i].ws) return &spaces[dev][i];
    return nullptr;
  }
  void* w = nullptr;
  void* c = nullptr;
  if (cudaMalloc(&w, (size_t)sms * BM * 256 * sizeof(float)) != cudaSuccess ||
      cudaMalloc(&c, (size_t)sms * sizeof(unsigned int)) != cudaSuccess ||
      cudaMemset(c, 0, (size_t)sms * sizeof(unsigned int)) != cudaSuccess) {
    // allocation refused, e.g. while this stream records a CUDA graph: the graph's launches share the
    // workspace that the warm-up launches of this device allocated (they run in stream order with them)
    cudaGetLastError();
    if (w) cudaFree(w);
    if (c) cudaFree(c);
    for (int i = 0; i < MAX_SPLIT_STREAMS; ++i)
      if (spaces[dev][i].used && spaces[dev][i].ws) return &spaces[dev][i];
    return nullptr;
  }
  slot->ws = static_cast<float*>(w);
  slot->counters = static_cast<unsigned int*>(c);
  slot->stream = stream;
  slot->used = true;
  return slot;
}

template <int BN>
static int launch(const void* A, const void* B, void* C, const Params& p_in, long lda, long ldb, long ldc, int grid_cap,
                  cudaStream_t stream) {
  Params p = p_in;
  int cur = 0;
  cudaGetDevice(&cur);
  static bool attr_set[64] = {false};  // the attribute is per device
  if (!attr_set[cur & 63]) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg<BN>::SMEM_BYTES) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set[cur & 63] = true;
  }
  CUtensorMap ta, tb, tc;
  int rc;
  if (!p.a_mn) rc = kb::make_tmap_2d(&ta, A, 2, p.M, p.K, lda * 2, BM, BK, true);
  else         rc = kb::make_tmap_2d(&ta, A, 2, p.K, p.M, lda * 2, BK, 64, true);
  if (rc) return KB_STATUS_TMAP_ERROR;
  if (!p.b_mn) rc = kb::make_tmap_2d(&tb, B, 2, p.N, p.K, ldb * 2, BN, BK, true);
  else         rc = kb::make_tmap_2d(&tb, B, 2, p.K, p.N, ldb * 2, BK, 64, true);
  if (rc) return KB_STATUS_TMAP_ERROR;
  rc = kb::make_tmap_2d(&tc, C, 2, p.M, p.N, ldc * 2, BM, EPI_COLS, true);
  if (rc) return KB_STATUS_TMAP_ERROR;
  const int total = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int num_k = (p.K + BK - 1) / BK;
  // tail balancing: cut the tiles of the last partial wave into K slices (see the file header)
  p.full_tiles = total;
  p.split = 1;
  p.ws = nullptr;
  p.counters = nullptr;
  const int rem = total % grid_cap;
  if (rem > 0) {
    int split = grid_cap / rem;
    if (split > MAX_SPLIT) split = MAX_SPLIT;
    const int min_kb = total < grid_cap ? MIN_SLICE_KB_SKINNY : MIN_SLICE_KB;
    if (split > num_k / min_kb) split = num_k / min_kb;
    while (split > 1 && (split - 1) * ((num_k + split - 1) / split) >= num_k) --split;  // no empty slice
    if (split > 1) {
      int dev = 0;
      cudaGetDevice(&dev);
      if (SplitSpace* sp = split_space(dev, grid_cap, stream)) {
        p.full_tiles = total - rem;
        p.split = split;
        p.ws = sp->ws;
        p.counters = sp->counters;
      }
    }
  }
  const int units = p.full_tiles + (total - p.full_tiles) * p.split;
  const int grid = units < grid_cap ? units : grid_cap;
  gemm_bf16_kernel<BN><<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(ta, tb, tc, p);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// Estimated relative cost of running the problem with tile width bn: SM-waves times the work of
// one tile, with a small penalty for the lower operand reuse of narrower tiles.
static double tile_cost(int M, int N, int K, int bn, int sms) {
  const long tiles = (long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  const long full_waves = tiles / sms;
  const int rem = (int)(tiles % sms);
  double tail = 0.0;
  if (rem > 0) {
    const int num_k = (K + BK - 1) / BK;
    int split = sms / rem;
    if (split > MAX_SPLIT) split = MAX_SPLIT;
    const int min_kb = tiles < sms ? MIN_SLICE_KB_SKINNY : MIN_SLICE_KB;
    if (split > num_k / min_kb) split = num_k / min_kb;
    // a split tail costs its share of the main loop plus the workspace round trip
    tail = split > 1 ? 1.0 / split + 0.12 : 1.0;
    if (tail > 1.0) tail = 1.0;
  }
  // measured on B200: narrower tiles are shared-memory-bandwidth bound (A is re-read per tile),
  // a 192-wide tile runs at ~79 % and a 128-wide one at ~58 % of the 256-wide tile's rate
  const double per_tile = bn == 256 ? 1.0 : bn == 192 ? 0.95 : 0.88;
  return (full_waves + tail) * per_tile;
}

}  // namespace gemm
}  // namespace kb

// The split workspace of this (device, stream) for the other GEMM kernels of the library.
extern "C" int kb_gemm_split_space(int dev, int sms, void* stream, float** ws, unsigned int** counters) {
  kb::gemm::SplitSpace* sp = kb::gemm::split_space(dev, sms, static_cast<cudaStream_t>(stream));
  if (!sp) return KB_STATUS_CUDA_ERROR;
  *ws = sp->ws;
  *counters = sp->counters;
  return KB_STATUS_OK;
}

extern "C" int kb_gemm_bf16_bn(const void* A, const void* B, void* C, const void* R, int M, int N,
                               int K, long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn,
                               int epi, int bn, void* stream) {
  using namespace kb::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return KB_STATUS_BAD_ARG;
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(A) || misaligned(B) || misaligned(C) || (lda & 7) || (ldb & 7) || (ldc & 7))
    return KB_STATUS_BAD_ARG;
  if (epi == 1 && (R == nullptr || misaligned(R) || (ldr & 7) || (N & 7))) return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  static int sm_count[64] = {0};
  if (sm_count[dev] == 0) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  const int sms = sm_count[dev];
  if (bn == 0) {
    bn = 256;
    double best = tile_cost(M, N, K, 256, sms);
    for (int cand : {192, 128}) {
      const double c = tile_cost(M, N, K, cand, sms);
      if (c < best * 0.999) { best = c; bn = cand; }
    }
  }
  Params p;
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ldr = ldr;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.epi = epi;
  p.err = kb::error_word(dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (bn) {
    case 256: return launch<256>(A, B, C, p, lda, ldb, ldc, sms, st);
    case 192: return launch<192>(A, B, C, p, lda, ldb, ldc, sms, st);
    case 128: return launch<128>(A, B, C, p, lda, ldb, ldc, sms, st);
    default: return KB_STATUS_BAD_ARG;
  }
}

extern "C" int kb_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N,
                            int K, long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn,
                            int epi, void* stream) {
  return kb_gemm_bf16_bn(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, b_mn, epi, 0, stream);
}
