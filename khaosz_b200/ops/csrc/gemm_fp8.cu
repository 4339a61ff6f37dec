// Block-scaled fp8 (e4m3) GEMM for sm_100a and its quantisers.
//
//   C[M,N] (bf16) = sum over k-blocks kb of  (A8[:, kb] * B8[:, kb]^T) * sa[m, kb] * sb[n / 128, kb]
//
// A8 [M,K] e4m3 with one fp32 scale per row and 128-wide k-block (1x128), B8 [N,K] e4m3 with one
// scale per 128x128 block.  Because the scale changes with every k-block, each k-block's product
// is formed by tcgen05.mma (kind::f8f6f4, K = 32 per instruction, 4 per k-block) in its own TMEM
// buffer (two buffers, so the next k-block's MMAs overlap), and eight "promotion" warps fold it
// into fp32 register accumulators with the combined scale — the same promotion scheme used for
// block-scaled fp8 on earlier parts, mapped onto TMEM.
//
//   warp 0        TMA producer (128-byte rows = one 128B swizzle atom per k-block), 4 stages
//   warp 1        MMA issuer / TMEM owner (2 x 256 columns)
//   warps 2-9     promotion + epilogue: warpgroup g owns output columns [128 g, 128 g + 128)
#include <cuda_fp8.h>

#include "common.cuh"
#include "kb_api.h"

namespace kb {
namespace f8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // fp8 elements = bytes
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK;  // 32 KiB
constexpr int EPI_BUF_BYTES = BM * 64 * 2;  // one [128 x 64] bf16 staging tile per warpgroup
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 320;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 2 * EPI_BUF_BYTES + 256 + 1024;

struct Params {
  const float* sa;  // [M, K/128]
  const float* sb;  // [ceil(N/128), K/128]
  int M, N, K;
  int* err;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * B_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + 2 * EPI_BUF_BYTES);
  uint64_t* full = bars;               // [STAGES]
  uint64_t* empty = bars + STAGES;     // [STAGES]
  uint64_t* pfull = bars + 2 * STAGES;     // [2] k-block product complete in TMEM
  uint64_t* pempty = bars + 2 * STAGES + 2;  // [2] promoted (8 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN, num_k = p.K / BK;
  const int total = num_m * num_n;
  const int kblocks = p.K / 128;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&pfull[i], 1); mbar_init(&pempty[i], 8); }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_b); tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          tma_load_2d(sA + s * A_STAGE_BYTES, &tmap_a, &full[s], kb * BK, m0);
          tma_load_2d(sB + s * B_STAGE_BYTES, &tmap_b, &full[s], kb * BK, n0);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, BN, false, false, UMMA_FMT_E4M3);
      int s = 0; uint32_t ph = 0; bool ok = true;
      uint32_t it = 0;  // running k-block counter across tiles: selects the product buffer
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int pb = it & 1;
          const uint32_t pph = (it >> 1) & 1;
          if (!mbar_wait(&pempty[pb], pph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(&full[s], ph, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES), b_addr = smem_u32(sB + s * B_STAGE_BYTES);
          const uint32_t d_tmem = tmem_base + pb * BN;
#pragma unroll
          for (int j = 0; j < BK / 32; ++j)
            umma_f8(d_tmem, umma_desc_kmajor(a_addr, j * 32), umma_desc_kmajor(b_addr, j * 32), idesc, j ? 1u : 0u);
          umma_commit(&empty[s]);
          umma_commit(&pfull[pb]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------- promotion + epilogue -------------------------------
    const int g = (warp - 2) >> 2;  // warpgroup: column half
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* stage = sEpi + g * EPI_BUF_BYTES;
    const int wg_tid = (threadIdx.x - 64) & 127;
    bool ok = true;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN;
      const int grow = m0 + row_in_tile;
      const int nblk = (n0 >> 7) + g;  // 128-wide scale block of this warpgroup's columns
      const bool cols_live = (n0 + g * 128) < p.N;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      for (int kb = 0; kb < num_k; ++kb, ++it) {
        const int pb = it & 1;
        if (!mbar_wait(&pfull[pb], (it >> 1) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        float sc = 0.f;
        if (grow < p.M && cols_live) sc = p.sa[(size_t)grow * kblocks + kb] * p.sb[(size_t)nblk * kblocks + kb];
        const uint32_t t_addr = tmem_base + lane_off + pb * BN + g * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(v[i]), sc, acc[c * 32 + i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
      }
      if (!ok) break;
      // two [128 x 64] chunks per warpgroup through one staging tile
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col0 = n0 + g * 128 + c * 64;
        if (wg_tid == 0) tma_store_wait_read<0>();
        named_barrier_sync(1 + g, 128);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint4 o;
          const float* a8 = acc + c * 64 + ch * 8;
          o.x = pack_bf16x2(a8[0], a8[1]); o.y = pack_bf16x2(a8[2], a8[3]);
          o.z = pack_bf16x2(a8[4], a8[5]); o.w = pack_bf16x2(a8[6], a8[7]);
          *reinterpret_cast<uint4*>(stage + sw128_offset(row_in_tile, ch)) = o;
        }
        fence_proxy_async_smem();
        named_barrier_sync(1 + g, 128);
        if (wg_tid == 0 && col0 < p.N) { tma_store_2d(&tmap_c, stage, col0, m0); tma_store_commit(); }
      }
    }
    if (wg_tid == 0) tma_store_wait_all<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------
// Quantisers.  scale = amax / 448 (the largest finite e4m3 value), q = x / scale.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// one warp per (row, 128-wide block); x pitch ld elements
__global__ void quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                   float* __restrict__ scale, int M, int K, long ld) {
  const int kblocks = K >> 7;
  const long unit = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (unit >= (long)M * kblocks) return;
  const long row = unit / kblocks;
  const int kb = (int)(unit - row * kblocks);
  const __nv_bfloat16* src = x + row * ld + kb * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = warp_max(amax);
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / s;
  const uint32_t packed = to_e4m3(a.x * inv) | (to_e4m3(a.y * inv) << 8) | (to_e4m3(b.x * inv) << 16) |
                          ((uint32_t)to_e4m3(b.y * inv) << 24);
  *reinterpret_cast<uint32_t*>(q + row * K + kb * 128 + lane * 4) = packed;
  if (lane == 0) scale[row * kblocks + kb] = s;
}

// one CTA (256 threads) per 128x128 block
__global__ void quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                     float* __restrict__ scale, int N, int K, long ld) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int kblocks = K >> 7;
  const int nb = blockIdx.x / kblocks, kb = blockIdx.x % kblocks;
  const int tid = threadIdx.x;
  float amax = 0.f;
  for (int i = tid; i < 128 * 32; i += 256) {  // 32 groups of 4 elements per row
    const int r = i >> 5, c4 = i & 31;
    const int row = nb * 128 + r;
    if (row < N) {
      const uint2 raw = *reinterpret_cast<const uint2*>(w + (size_t)row * ld + kb * 128 + c4 * 4);
      const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
    }
  }
  amax = warp_max(amax);
  if ((tid & 31) == 0) red[tid >> 5] = amax;
  __syncthreads();
  if (tid == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, red[i]);
    s_scale = m > 0.f ? m / 448.f : 1.f;
    scale[(size_t)nb * kblocks + kb] = s_scale;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  for (int i = tid; i < 128 * 32; i += 256) {
    const int r = i >> 5, c4 = i & 31;
    const int row = nb * 128 + r;
    if (row < N) {
      const uint2 raw = *reinterpret_cast<const uint2*>(w + (size_t)row * ld + kb * 128 + c4 * 4);
      const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
      const uint32_t packed = to_e4m3(a.x * inv) | (to_e4m3(a.y * inv) << 8) | (to_e4m3(b.x * inv) << 16) |
                              ((uint32_t)to_e4m3(b.y * inv) << 24);
      *reinterpret_cast<uint32_t*>(q + (size_t)row * K + kb * 128 + c4 * 4) = packed;
    }
  }
}

}  // namespace f8
}  // namespace kb

extern "C" {

// x [M,K] bf16 (pitch ld) -> q [M,K] e4m3 (dense), scale fp32 [M, K/128].  K % 128 == 0.
int kb_quant_fp8_1x128(const void* x, void* q, void* scale, int M, int K, long ld, void* stream) {
  if (M <= 0 || K <= 0) return KB_STATUS_OK;
  if ((K & 127) || (ld & 3)) return KB_STATUS_BAD_ARG;
  const long units = (long)M * (K >> 7);
  kb::f8::quant_1x128_kernel<<<(unsigned)((units * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (uint8_t*)q, (float*)scale, M, K, ld);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// w [N,K] bf16 (pitch ld) -> q [N,K] e4m3, scale fp32 [ceil(N/128), K/128].
int kb_quant_fp8_128x128(const void* w, void* q, void* scale, int N, int K, long ld, void* stream) {
  if (N <= 0 || K <= 0) return KB_STATUS_OK;
  if ((K & 127) || (ld & 3)) return KB_STATUS_BAD_ARG;
  const int blocks = ((N + 127) / 128) * (K >> 7);
  kb::f8::quant_128x128_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (uint8_t*)q,
                                                                         (float*)scale, N, K, ld);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// A8 [M,K] e4m3, B8 [N,K] e4m3 (dense rows), sa [M,K/128], sb [ceil(N/128),K/128], C [M,N] bf16.
int kb_gemm_fp8(const void* A8, const void* B8, const void* sa, const void* sb, void* C, int M, int N, int K,
                long lda, long ldb, long ldc, void* stream) {
  using namespace kb::f8;
  if (M <= 0 || N <= 0 || K <= 0) return KB_STATUS_BAD_ARG;
  auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (mis(A8) || mis(B8) || mis(C) || (K & 127) || (lda & 15) || (ldb & 15) || (ldc & 7)) return KB_STATUS_BAD_ARG;
  static bool attr_set_dev[64] = {false};  // the attribute is per device
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_set_dev[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  static int sms = 0;
  if (sms == 0) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap ta, tb, tc;
  if (kb::make_tmap_2d(&ta, A8, 1, M, K, lda, BM, BK, true)) return KB_STATUS_TMAP_ERROR;
  if (kb::make_tmap_2d(&tb, B8, 1, N, K, ldb, BN, BK, true)) return KB_STATUS_TMAP_ERROR;
  if (kb::make_tmap_2d(&tc, C, 2, M, N, ldc * 2, BM, 64, true)) return KB_STATUS_TMAP_ERROR;
  Params p;
  p.sa = (const float*)sa; p.sb = (const float*)sb; p.M = M; p.N = N; p.K = K; p.err = kb::error_word(dev);
  const int total = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  gemm_fp8_kernel<<<total < sms ? total : sms, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(ta, tb, tc, p);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

}  // extern "C"
