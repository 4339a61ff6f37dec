// Weight-only int8 GEMM for sm_100a:  C[M,N] = X[M,K] (bf16) * dequant(W[N,K] int8)^T * scale[N]
//
// The weights cross HBM as int8 (half the bytes of bf16 — the decode-time bound) and are
// widened to bf16 only inside the SM: TMA brings the raw int8 tile into shared memory, four
// converter warps rewrite it as a 128B-swizzled bf16 K-major tile, and tcgen05.mma consumes that
// tile like an ordinary bf16 operand.  The per-output-channel scale is applied to the fp32
// accumulator in the epilogue, so the integer weights enter the MMA exactly.
//
//   warp 0        TMA producer (X tile bf16, W tile int8), 3-stage ring
//   warp 1        tcgen05.mma issuer, TMEM owner (two 128x256 fp32 accumulators)
//   warps 2-5     epilogue (tcgen05.ld -> * scale[n] -> bf16 -> swizzled staging -> TMA store)
//   warps 6-9     converters: int8 -> bf16 into the MMA operand tile
#include "common.cuh"
#include "kb_api.h"

extern "C" int kb_gemm_split_space(int dev, int sms, void* stream, float** ws, unsigned int** counters);

namespace kb {
namespace w8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int A_STAGE_BYTES = BM * BK * 2;    // 16 KiB
constexpr int RAW_STAGE_BYTES = BN * BK;      // 16 KiB of int8
constexpr int B_STAGE_BYTES = BN * BK * 2;    // 32 KiB of bf16
constexpr int EPI_COLS = 64;
constexpr int EPI_BUF_BYTES = BM * EPI_COLS * 2;
constexpr int NUM_EPI_BUFS = 2;
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 320;
constexpr int SMEM_BYTES =
    STAGES * (A_STAGE_BYTES + RAW_STAGE_BYTES + B_STAGE_BYTES) + NUM_EPI_BUFS * EPI_BUF_BYTES + 256 + 1024;

struct Params {
  const float* scale;  // [N]
  int M, N, K;
  int* err;
  // split-K for problems with fewer tiles than SMs (decode): every tile is cut into `split` K
  // slices; a slice parks its fp32 accumulator in the workspace and the last slice of a tile to
  // arrive sums them in slice order and finishes the tile (same scheme as gemm_bf16.cu)
  int split;
  float* ws;
  unsigned int* counters;
};

__device__ __forceinline__ void unit_of(const Params& p, int u, int num_k, int& tile, int& kb0, int& kb1, int& slice) {
  if (p.split <= 1) { tile = u; kb0 = 0; kb1 = num_k; slice = 0; return; }
  tile = u / p.split;
  slice = u - tile * p.split;
  const int per = (num_k + p.split - 1) / p.split;
  kb0 = slice * per;
  kb1 = min(num_k, kb0 + per);
}

// Four int8 -> four bf16 without integer-to-float conversions: each byte, biased by 128, becomes the
// low mantissa byte of 2^23 (bit pattern 0x4B0000uu = 8388608 + u), and subtracting 8388736 leaves
// the signed value exactly; bf16 holds every integer of that range exactly.
__device__ __forceinline__ void cvt4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.f;
  const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.f;
  const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.f;
  const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.f;
  lo = pack_bf16x2(f0, f1);
  hi = pack_bf16x2(f2, f3);
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_w8_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
               const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + STAGES * A_STAGE_BYTES;
  uint8_t* sRaw = sB + STAGES * B_STAGE_BYTES;
  uint8_t* sEpi = sRaw + STAGES * RAW_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + NUM_EPI_BUFS * EPI_BUF_BYTES);
  uint64_t* raw_full = bars;                 // [STAGES] TMA landed (A and raw W)
  uint64_t* cvt_full = bars + STAGES;        // [STAGES] bf16 W tile written (4 converter warps)
  uint64_t* empty = bars + 2 * STAGES;       // [STAGES] MMAs done with the stage
  uint64_t* tfull = bars + 3 * STAGES;       // [2]
  uint64_t* tempty = bars + 3 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN, num_k = (p.K + BK - 1) / BK;
  const int total = num_m * num_n * (p.split > 1 ? p.split : 1);  // work units

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&raw_full[i], 1);
      mbar_init(&cvt_full[i], 4);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x); tma_prefetch_desc(&tmap_w); tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      for (int u = blockIdx.x; u < total && ok; u += gridDim.x) {
        int t, kb0, kb1, slice;
        unit_of(p, u, num_k, t, kb0, kb1, slice);
        const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN;  // m fastest: CTAs of a wave share W tiles in L2
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&raw_full[s], A_STAGE_BYTES + RAW_STAGE_BYTES);
          tma_load_2d(sA + s * A_STAGE_BYTES, &tmap_x, &raw_full[s], kb * BK, m0);
          tma_load_2d(sRaw + s * RAW_STAGE_BYTES, &tmap_w, &raw_full[s], kb * BK, n0);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, BN, false, false);
      int s = 0; uint32_t ph = 0; int acc = 0; uint32_t aph = 0; bool ok = true;
      for (int u = blockIdx.x; u < total && ok; u += gridDim.x) {
        int t, kb0, kb1, slice;
        unit_of(p, u, num_k, t, kb0, kb1, slice);
        if (!mbar_wait(&tempty[acc], aph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&cvt_full[s], ph, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES), b_addr = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j)
            umma_f16(d_tmem, umma_desc_kmajor(a_addr, j * 32), umma_desc_kmajor(b_addr, j * 32), idesc,
                     (kb > kb0 || j) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) { acc = 0; aph ^= 1u; }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------- converters -------------------------------
    const int ctid = threadIdx.x - 192;  // 0..127
    int s = 0; uint32_t ph = 0; bool ok = true;
    for (int u = blockIdx.x; u < total && ok; u += gridDim.x) {
      int t, kb0, kb1, slice;
      unit_of(p, u, num_k, t, kb0, kb1, slice);
      for (int kb = kb0; kb < kb1; ++kb) {
        // raw_full also covers the X tile; the bf16 W tile of this stage is free once `empty`
        // completed, which the producer waited for before refilling raw
        if (!mbar_wait(&raw_full[s], ph, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
        const uint8_t* raw = sRaw + s * RAW_STAGE_BYTES;
        uint8_t* dst = sB + s * B_STAGE_BYTES;
        // consecutive threads take consecutive 16-byte groups of the raw tile (256 rows x 64 B): the
        // shared-memory reads are conflict free (a thread-per-row mapping put all lanes of a warp on
        // the same banks) and a warp writes whole 128-byte rows of the swizzled bf16 tile
#pragma unroll
        for (int it = 0; it < (BN * BK / 16) / 128; ++it) {
          const int idx = it * 128 + ctid;
          const int row = idx >> 2, q16 = idx & 3;
          const uint4 v = *reinterpret_cast<const uint4*>(raw + idx * 16);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) cvt4(w[i], o[2 * i], o[2 * i + 1]);
          *reinterpret_cast<uint4*>(dst + sw128_offset(row, q16 * 2)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dst + sw128_offset(row, q16 * 2 + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&cvt_full[s]);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    int acc = 0; uint32_t aph = 0; int buf = 0; bool ok = true;
    __shared__ int s_last;
    for (int u = blockIdx.x; u < total && ok; u += gridDim.x) {
      int t, kb0, kb1, slice;
      unit_of(p, u, num_k, t, kb0, kb1, slice);
      const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      // one 64-column chunk of fp32 sums -> * scale[n] -> bf16 -> staging -> TMA store
      auto emit_chunk = [&](int c, const uint32_t (&v)[EPI_COLS]) {
        const int col0 = n0 + c * EPI_COLS;
        if (epi_tid == 0) tma_store_wait_read<NUM_EPI_BUFS - 1>();
        named_barrier_sync(1, 128);
        uint8_t* stage = sEpi + buf * EPI_BUF_BYTES;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = col0 + ch * 8 + e;
            f[e] = __uint_as_float(v[ch * 8 + e]) * (col < p.N ? p.scale[col] : 0.f);
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
          *reinterpret_cast<uint4*>(stage + sw128_offset(row_in_tile, ch)) = o;
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (epi_tid == 0) { tma_store_2d(&tmap_c, stage, col0, m0); tma_store_commit(); }
        buf ^= 1;
      };
      if (p.split <= 1) {
#pragma unroll 1
        for (int c = 0; c < BN / EPI_COLS; ++c) {
          if (n0 + c * EPI_COLS >= p.N) break;
          uint32_t v[EPI_COLS];
          tmem_ld_32x32b_x32(t_row + c * EPI_COLS, v);
          tmem_ld_32x32b_x32(t_row + c * EPI_COLS + 32, v + 32);
          tmem_ld_wait();
          emit_chunk(c, v);
        }
      } else {
        // workspace layout per slice: [chunk][16-byte group][row]: a warp's accesses are contiguous
        uint4* mine = reinterpret_cast<uint4*>(p.ws + ((size_t)t * p.split + slice) * (BM * BN)) + row_in_tile;
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
          const unsigned int prev = atomicAdd(&p.counters[t], 1u);
          const int last = prev == (unsigned int)(p.split - 1);
          if (last) p.counters[t] = 0u;  // re-armed for the next launch
          s_last = last;
          __threadfence();
        }
        named_barrier_sync(1, 128);
        if (s_last) {
          const uint4* base = reinterpret_cast<const uint4*>(p.ws + (size_t)t * p.split * (BM * BN)) + row_in_tile;
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) { acc = 0; aph ^= 1u; }
    }
    if (epi_tid == 0) tma_store_wait_all<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// Symmetric per-output-channel quantisation: scale[n] = max|W[n,:]| / 127, q = round(W / scale).
__global__ void quant_w8_kernel(const __nv_bfloat16* __restrict__ w, signed char* __restrict__ q,
                                float* __restrict__ scale, int K) {
  __shared__ float red[32];
  const int n = blockIdx.x;
  const __nv_bfloat16* row = w + (size_t)n * K;
  float mx = 0.f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, fabsf(__bfloat162float(row[k])));
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  float m2 = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) m2 = warp_max(m2);
  if (threadIdx.x == 0) { red[0] = m2; scale[n] = m2 > 0.f ? m2 / 127.f : 1.f; }
  __syncthreads();
  const float inv = red[0] > 0.f ? 127.f / red[0] : 0.f;
  for (int k = threadIdx.x; k < K; k += blockDim.x)
    q[(size_t)n * K + k] = (signed char)max(-127, min(127, __float2int_rn(__bfloat162float(row[k]) * inv)));
}

}  // namespace w8
}  // namespace kb

extern "C" {

// X [M,K] bf16 (pitch ldx), Wq [N,K] int8 (pitch ldw bytes, multiple of 16), scale fp32 [N], C [M,N] bf16.
int kb_gemm_w8(const void* X, const void* Wq, const float* scale, void* C, int M, int N, int K, long ldx,
               long ldw, long ldc, void* stream) {
  using namespace kb::w8;
  if (M <= 0 || N <= 0 || K <= 0) return KB_STATUS_BAD_ARG;
  auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (mis(X) || mis(Wq) || mis(C) || (ldx & 7) || (ldw & 15) || (ldc & 7) || (K & 15) || !scale) return KB_STATUS_BAD_ARG;
  static bool attr_set_dev[64] = {false};  // the attribute is per device
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_set_dev[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_w8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  static int sms = 0;
  if (sms == 0) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap tx, tw, tc;
  if (kb::make_tmap_2d(&tx, X, 2, M, K, ldx * 2, BM, BK, true)) return KB_STATUS_TMAP_ERROR;
  if (kb::make_tmap_2d(&tw, Wq, 1, N, K, ldw, BN, BK, false)) return KB_STATUS_TMAP_ERROR;
  if (kb::make_tmap_2d(&tc, C, 2, M, N, ldc * 2, BM, EPI_COLS, true)) return KB_STATUS_TMAP_ERROR;
  Params p;
  p.scale = scale; p.M = M; p.N = N; p.K = K; p.err = kb::error_word(dev);
  p.split = 1; p.ws = nullptr; p.counters = nullptr;
  const int total = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int num_k = (K + BK - 1) / BK;
  if (total < sms) {  // skinny problem (decode): K slices put the idle SMs to work on the weight stream
    int split = sms / total;
    if (split > 16) split = 16;
    if (split > num_k / 8) split = num_k / 8;
    while (split > 1 && (split - 1) * ((num_k + split - 1) / split) >= num_k) --split;  // no empty slice
    if (split > 1 && kb_gemm_split_space(dev, sms, stream, &p.ws, &p.counters) == KB_STATUS_OK) p.split = split;
  }
  const int units = total * p.split;
  gemm_w8_kernel<<<units < sms ? units : sms, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tx, tw, tc, p);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

int kb_quant_w8(const void* W, void* Wq, float* scale, int N, int K, void* stream) {
  if (N <= 0 || K <= 0) return KB_STATUS_BAD_ARG;
  kb::w8::quant_w8_kernel<<<N, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)W, (signed char*)Wq, scale, K);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

}  // extern "C"
