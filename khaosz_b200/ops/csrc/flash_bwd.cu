// Flash attention backward for sm_100a (head_dim 128, bf16, causal or full, GQA aware).
//
// Three launches, all deterministic (no atomics):
//   1. delta[b,h,s] = sum_d O * dO
//   2. dK/dV kernel: one CTA per (batch, KV head, 128-key block).  It walks the query heads of
//      the group and their query blocks, computing the *transposed* tiles
//         S^T = K Q^T,  dP^T = V dO^T            (keys in TMEM lanes, queries in columns)
//      so that P^T = exp(S^T - lse) and dS^T = P^T o (dP^T - delta), written back to TMEM as
//      bf16, are directly the A operands of  dV += P^T dO  and  dK += dS^T Q.
//      The GQA reduction over the group's heads happens in the TMEM accumulators.
//   3. dQ kernel: one CTA per (batch, head, 128-query block): S = Q K^T, dP = dO V^T,
//      dS -> TMEM (bf16) -> dQ += dS K.
// A [128 x 64] 128B-swizzled TMA box is used both as a K-major operand (rows = M/N, columns =
// reduction) and as an MN-major operand (rows = reduction, columns = N): the same shared
// memory image of Q / dO / K serves both products it appears in.
// TMEM: kernel 2 uses S^T | dP^T | dV | dK, kernel 3 uses S(even) | dP | S(odd) | dQ (128 fp32 columns each).
#include "common.cuh"
#include "kb_api.h"

namespace kb {
namespace fab {

constexpr int D = 128;
constexpr int BLK = 128;
constexpr int CHUNK_BYTES = 128 * 64 * 2;
constexpr int TILE_BYTES = 2 * CHUNK_BYTES;
constexpr int NUM_THREADS = 320;  // TMA warp, MMA warp, 8 compute warps (two per TMEM lane quarter)
constexpr int COMPUTE_THREADS = 256;
constexpr int SMEM_BYTES = 6 * TILE_BYTES + 4 * 128 * 4 + 256 + 1024;
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
  const float* lse;    // [B,H,S]
  const float* delta;  // [B,H,S]
  int B, S, H, Hkv;
  float scale, scale_log2;
  int causal;
  int n_blocks;  // ceil(S / 128)
  int* err;
};

// ---------------------------------------------------------------------------------------
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                             float* __restrict__ delta, int B, int S, int H, long o_pitch, long do_pitch) {
  const long pair = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 4;  // (token, head)
  const int sub = threadIdx.x & 15;
  const long total = (long)B * S * H;
  float acc = 0.f;
  if (pair < total) {
    const long tok = pair / H;
    const int h = (int)(pair - tok * H);
    const uint4 a = *reinterpret_cast<const uint4*>(o + tok * o_pitch + h * D + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + tok * do_pitch + h * D + sub * 8);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16x2(av[i]), y = unpack_bf16x2(gv[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (pair < total && sub == 0) {
    const long tok = pair / H;
    const int h = (int)(pair - tok * H);
    const long b = tok / S, s = tok - b * S;
    delta[(b * H + h) * S + s] = acc;
  }
}

// shared helpers ------------------------------------------------------------------------
__device__ __forceinline__ void issue_ss(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, uint32_t idesc) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t off = (ks >> 2) * CHUNK_BYTES + (ks & 3) * 32;
    umma_f16(d_tmem, umma_desc_kmajor(a_addr, off), umma_desc_kmajor(b_addr, off), idesc, ks ? 1u : 0u);
  }
}
// D += A(tmem, bf16 [128 x 128]) * B(smem image used MN-major: rows = reduction index)
__device__ __forceinline__ void issue_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_addr, uint32_t idesc,
                                         bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    umma_f16_ts(d_tmem, a_tmem + ks * 8, umma_desc_mnmajor(b_addr, ks * 16, CHUNK_BYTES), idesc,
                (accumulate || ks) ? 1u : 0u);
}

// TMEM accumulator [128 x 128] fp32 -> bf16 (x mul) -> swizzled staging tile (2 chunks)
// for the 32-column groups [c_begin, c_end)
__device__ __forceinline__ void acc_to_staging(uint32_t t_addr, uint8_t* stage, int row, float mul, int c_begin,
                                               int c_end) {
#pragma unroll 2
  for (int c = c_begin; c < c_end; ++c) {
    uint32_t o[32];
    tmem_ld_32x32b_x32(t_addr + c * 32, o);
    tmem_ld_wait();
    uint8_t* chunk_base = stage + (c >> 1) * CHUNK_BYTES;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      uint4 v;
      v.x = pack_bf16x2(__uint_as_float(o[ch * 8 + 0]) * mul, __uint_as_float(o[ch * 8 + 1]) * mul);
      v.y = pack_bf16x2(__uint_as_float(o[ch * 8 + 2]) * mul, __uint_as_float(o[ch * 8 + 3]) * mul);
      v.z = pack_bf16x2(__uint_as_float(o[ch * 8 + 4]) * mul, __uint_as_float(o[ch * 8 + 5]) * mul);
      v.w = pack_bf16x2(__uint_as_float(o[ch * 8 + 6]) * mul, __uint_as_float(o[ch * 8 + 7]) * mul);
      *reinterpret_cast<uint4*>(chunk_base + sw128_offset(row, (c & 1) * 4 + ch)) = v;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Kernel 2: dK, dV
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                      const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;        // [2 stages]
  uint8_t* sdO = sQ + 2 * TILE_BYTES;   // [2 stages]
  float* sLse = reinterpret_cast<float*>(sdO + 2 * TILE_BYTES);  // [2][128] (log2 domain)
  float* sDelta = sLse + 2 * 128;                                  // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDelta + 2 * 128);
  uint64_t* kv_full = bars;        // [1]
  uint64_t* q_full = bars + 1;     // [2]  (TMA tx + the producer warp's lse/delta writes)
  uint64_t* q_empty = bars + 3;    // [2]
  uint64_t* st_full = bars + 5;    // [1]
  uint64_t* dpt_full = bars + 6;   // [1]
  uint64_t* p_ready = bars + 7;    // [1]
  uint64_t* ds_ready = bars + 8;   // [1]
  uint64_t* acc_full = bars + 9;   // [1]
  uint64_t* s_read = bars + 10;    // [4]  lower-half warp of a lane quarter has loaded its S^T columns
  uint64_t* dp_read = bars + 14;   // [4]  ... its dP^T columns
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid, heaviest key blocks first over ALL (batch, KV head) pairs: under a causal mask key block
  // jb meets (n_blocks - jb) query blocks per head, and CTAs are handed to SMs in index order, so the
  // long ones start first and the short ones fill the gaps at the end
  const int n_bh = p.Hkv * p.B;
  const int jb = blockIdx.x / n_bh;
  const int kvh = (blockIdx.x % n_bh) % p.Hkv, b = (blockIdx.x % n_bh) / p.Hkv;
  const int kv0 = jb * BLK;
  const int G = p.H / p.Hkv;
  const int i_start = p.causal ? jb : 0;
  const int per_head = p.n_blocks - i_start;
  const int n_it = G * per_head;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 2); mbar_init(&q_empty[i], 1); }
    mbar_init(st_full, 1); mbar_init(dpt_full, 1);
    mbar_init(p_ready, 8); mbar_init(ds_ready, 8); mbar_init(acc_full, 1);
    for (int i = 0; i < 4; ++i) { mbar_init(&s_read[i], 1); mbar_init(&dp_read[i], 1); }
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do); tma_prefetch_desc(&tm_dk); tma_prefetch_desc(&tm_dv);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t T_ST = tmem_base, T_DPT = tmem_base + 128, T_DV = tmem_base + 256, T_DK = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------- producer -------------------------------
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      for (int c = 0; c < 2; ++c) {
        tma_load_3d(sK + c * CHUNK_BYTES, &tm_k, kv_full, kvh * D + c * 64, kv0, b);
        tma_load_3d(sV + c * CHUNK_BYTES, &tm_v, kv_full, kvh * D + c * 64, kv0, b);
      }
    }
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int h = kvh * G + it / per_head;
      const int q0 = (i_start + it % per_head) * BLK;
      if (lane == 0) ok = mbar_wait(&q_empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(&q_full[s], 2 * TILE_BYTES);
        for (int c = 0; c < 2; ++c) {
          tma_load_3d(sQ + s * TILE_BYTES + c * CHUNK_BYTES, &tm_q, &q_full[s], h * D + c * 64, q0, b);
          tma_load_3d(sdO + s * TILE_BYTES + c * CHUNK_BYTES, &tm_do, &q_full[s], h * D + c * 64, q0, b);
        }
      }
      const size_t row_base = ((size_t)b * p.H + h) * p.S;
      for (int r = lane; r < 128; r += 32) {
        const int q = q0 + r;
        sLse[s * 128 + r] = q < p.S ? p.lse[row_base + q] * LOG2E : INFINITY;  // +inf -> P = 0
        sDelta[s * 128 + r] = q < p.S ? p.delta[row_base + q] : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full[s]);
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && n_it > 0) {
      const uint32_t idesc_kk = umma_idesc(128, 128, false, false);
      const uint32_t idesc_ts = umma_idesc(128, 128, false, true);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(&q_full[0], 0, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_ss(T_ST, k_addr, smem_u32(sQ), idesc_kk);
        umma_commit(st_full);
        issue_ss(T_DPT, v_addr, smem_u32(sdO), idesc_kk);
        umma_commit(dpt_full);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const bool has_next = it + 1 < n_it;
        const int sn = (it + 1) & 1;
        const uint32_t phn = ((it + 1) >> 1) & 1;
        const uint32_t q_addr = smem_u32(sQ + s * TILE_BYTES), do_addr = smem_u32(sdO + s * TILE_BYTES);
        if (!mbar_wait(p_ready, it & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_ts(T_DV, T_ST, do_addr, idesc_ts, it > 0);           // dV += P^T dO
        if (has_next) {
          if (!mbar_wait(&q_full[sn], phn, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          issue_ss(T_ST, k_addr, smem_u32(sQ + sn * TILE_BYTES), idesc_kk);  // S^T of the next tile
          umma_commit(st_full);
        }
        if (!mbar_wait(ds_ready, it & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_ts(T_DK, T_DPT, q_addr, idesc_ts, it > 0);           // dK += dS^T Q
        umma_commit(&q_empty[s]);
        if (has_next) {
          issue_ss(T_DPT, v_addr, smem_u32(sdO + sn * TILE_BYTES), idesc_kk);  // dP^T of the next tile
          umma_commit(dpt_full);
        } else {
          umma_commit(acc_full);
        }
      }
    }
  } else {
    // ------------- compute warps: one thread per (key, half of the 128 query columns) -------------
    // Warp w reads TMEM lanes [32 * (w % 4), +32).  Warps 2-5 take query columns 0-63, warps 6-9
    // columns 64-127.  The packed bf16 result of the upper half lands in fp32 columns 32-63, which
    // the lower-half warp of the same lane quarter reads: it arrives on an mbarrier once its loads
    // have completed and the upper-half warp waits on that before storing.
    const int qtr = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = qtr * 32 + lane;
    const int kv = kv0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      const int q0 = (i_start + it % per_head) * BLK;
      const float* lse2 = sLse + s * 128 + half * 64;
      const float* dlt = sDelta + s * 128 + half * 64;
      // acquire the producer's lse/delta writes for this stage directly
      if (!mbar_wait(&q_full[s], (it >> 1) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
      if (!mbar_wait(st_full, it & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && (q0 < kv0 + BLK);
      const int qc = q0 + half * 64;  // first query column of this thread
      uint32_t preg[32];
      {
        uint32_t sv[64];
        tmem_ld_32x32b_x32(T_ST + lane_off + half * 64, sv);
        tmem_ld_32x32b_x32(T_ST + lane_off + half * 64 + 32, sv + 32);
        tmem_ld_wait();
        if (half == 0) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_read[qtr]);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p0 = exp2f(__uint_as_float(sv[2 * i]) * p.scale_log2 - lse2[2 * i]);
          float p1 = exp2f(__uint_as_float(sv[2 * i + 1]) * p.scale_log2 - lse2[2 * i + 1]);
          if (diag) {
            if (kv > qc + 2 * i) p0 = 0.f;
            if (kv > qc + 2 * i + 1) p1 = 0.f;
          }
          preg[i] = pack_bf16x2(p0, p1);
        }
      }
      if (half == 1) {
        if (!mbar_wait(&s_read[qtr], it & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
      }
      tmem_st_32x32b_x32(T_ST + lane_off + half * 32, preg);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);

      if (!mbar_wait(dpt_full, it & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t ds[32];
      {
        uint32_t dv[64];
        tmem_ld_32x32b_x32(T_DPT + lane_off + half * 64, dv);
        tmem_ld_32x32b_x32(T_DPT + lane_off + half * 64 + 32, dv + 32);
        tmem_ld_wait();
        if (half == 0) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&dp_read[qtr]);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float2 pp = unpack_bf16x2(preg[i]);
          ds[i] = pack_bf16x2(pp.x * (__uint_as_float(dv[2 * i]) - dlt[2 * i]),
                              pp.y * (__uint_as_float(dv[2 * i + 1]) - dlt[2 * i + 1]));
        }
      }
      if (half == 1) {
        if (!mbar_wait(&dp_read[qtr], it & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
      }
      tmem_st_32x32b_x32(T_DPT + lane_off + half * 32, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    // ---- epilogue: dV (lower-half warps), dK (upper-half warps) -> bf16 -> staging -> TMA store ----
    const bool have = n_it > 0 && ok && mbar_wait(acc_full, 0, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL);
    if (have) {
      tc_fence_after();
      if (half == 0) acc_to_staging(T_DV + lane_off, sQ, row, 1.f, 0, 4);
      else acc_to_staging(T_DK + lane_off, sQ + TILE_BYTES, row, p.scale, 0, 4);
      fence_proxy_async_smem();
    }
    // every compute warp reaches this barrier (also after a failed wait) so that none is left behind
    named_barrier_sync(1, COMPUTE_THREADS);
    if (have && threadIdx.x == 64) {
      for (int c = 0; c < 2; ++c) {
        tma_store_3d(&tm_dv, sQ + c * CHUNK_BYTES, kvh * D + c * 64, kv0, b);
        tma_store_3d(&tm_dk, sQ + TILE_BYTES + c * CHUNK_BYTES, kvh * D + c * 64, kv0, b);
      }
      tma_store_commit();
      tma_store_wait_all<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------------------
// Kernel 3: dQ
// ---------------------------------------------------------------------------------------
// TMEM: SA | DP | SB | DQ (128 fp32 columns each).  S of key block j lands in SA (j even) or SB
// (j odd) and dP always in DP, so that the tensor pipe never waits for the score-gradient warps:
// while they turn (S_j, dP_j) into dS_j (bf16, written over S_j), S_{j+1} is already complete,
// and as soon as dS_j is ready the pipe runs dP_{j+1}, dQ += dS_j K_j and S_{j+2} back to back.
// K lives in a 3-stage ring (it is read by S_j early and by the dQ product late), V in 2 stages.
constexpr int DQ_K_STAGES = 3;
constexpr int DQ_V_STAGES = 2;
constexpr int SMEM_BYTES_DQ = (2 + DQ_K_STAGES + DQ_V_STAGES) * TILE_BYTES + 256 + 1024;

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_dq, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + TILE_BYTES;
  uint8_t* sK = sdO + TILE_BYTES;                 // [DQ_K_STAGES]
  uint8_t* sV = sK + DQ_K_STAGES * TILE_BYTES;    // [DQ_V_STAGES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + DQ_V_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;                    // [1]
  uint64_t* k_full = bars + 1;                // [3]
  uint64_t* k_empty = k_full + DQ_K_STAGES;   // [3]
  uint64_t* v_full = k_empty + DQ_K_STAGES;   // [2]
  uint64_t* v_empty = v_full + DQ_V_STAGES;   // [2]
  uint64_t* s_full = v_empty + DQ_V_STAGES;   // [2]  SA / SB
  uint64_t* dp_full = s_full + 2;             // [1]
  uint64_t* ds_ready = dp_full + 1;           // [1]
  uint64_t* acc_full = ds_ready + 1;          // [1]
  uint64_t* s_read = acc_full + 1;            // [4]  lower-half warp of a lane quarter has loaded its S columns
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_read + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid, heavy (late) query blocks first over all (batch, head) pairs
  const int n_bh = p.H * p.B;
  const int ib = p.n_blocks - 1 - blockIdx.x / n_bh;
  const int h = (blockIdx.x % n_bh) % p.H, b = (blockIdx.x % n_bh) / p.H;
  const int q0 = ib * BLK;
  const int kvh = h / (p.H / p.Hkv);
  const int n_it = p.causal ? min(p.n_blocks, ib + 1) : p.n_blocks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < DQ_K_STAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < DQ_V_STAGES; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    for (int i = 0; i < 2; ++i) mbar_init(&s_full[i], 1);
    mbar_init(dp_full, 1); mbar_init(ds_ready, 8); mbar_init(acc_full, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&s_read[i], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do); tma_prefetch_desc(&tm_dq);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t T_DP = tmem_base + 128, T_DQ = tmem_base + 384;
  auto s_region = [&](int j) -> uint32_t { return tmem_base + ((j & 1) ? 256u : 0u); };

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      for (int c = 0; c < 2; ++c) {
        tma_load_3d(sQ + c * CHUNK_BYTES, &tm_q, q_full, h * D + c * 64, q0, b);
        tma_load_3d(sdO + c * CHUNK_BYTES, &tm_do, q_full, h * D + c * 64, q0, b);
      }
      bool ok = true;
      for (int j = 0; j < n_it && ok; ++j) {
        const int ks = j % DQ_K_STAGES, vs = j % DQ_V_STAGES;
        if (!mbar_wait(&k_empty[ks], ((j / DQ_K_STAGES) & 1) ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(&k_full[ks], TILE_BYTES);
        for (int c = 0; c < 2; ++c)
          tma_load_3d(sK + ks * TILE_BYTES + c * CHUNK_BYTES, &tm_k, &k_full[ks], kvh * D + c * 64, j * BLK, b);
        if (!mbar_wait(&v_empty[vs], ((j / DQ_V_STAGES) & 1) ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(&v_full[vs], TILE_BYTES);
        for (int c = 0; c < 2; ++c)
          tma_load_3d(sV + vs * TILE_BYTES + c * CHUNK_BYTES, &tm_v, &v_full[vs], kvh * D + c * 64, j * BLK, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      const uint32_t idesc_kk = umma_idesc(128, 128, false, false);
      const uint32_t idesc_ts = umma_idesc(128, 128, false, true);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      auto k_addr = [&](int j) { return smem_u32(sK + (j % DQ_K_STAGES) * TILE_BYTES); };
      auto wait_k = [&](int j) {
        return mbar_wait(&k_full[j % DQ_K_STAGES], (j / DQ_K_STAGES) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      };
      auto wait_v = [&](int j) {
        return mbar_wait(&v_full[j % DQ_V_STAGES], (j / DQ_V_STAGES) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      };
      auto issue_dp = [&](int j) {
        issue_ss(T_DP, do_addr, smem_u32(sV + (j % DQ_V_STAGES) * TILE_BYTES), idesc_kk);
        umma_commit(dp_full);
        umma_commit(&v_empty[j % DQ_V_STAGES]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      if (ok) ok = wait_k(0);
      if (ok) {
        tc_fence_after();
        issue_ss(s_region(0), q_addr, k_addr(0), idesc_kk);
        umma_commit(&s_full[0]);
        ok = wait_v(0);
      }
      if (ok) {
        tc_fence_after();
        issue_dp(0);
        if (n_it > 1) {
          ok = wait_k(1);
          if (ok) {
            tc_fence_after();
            issue_ss(s_region(1), q_addr, k_addr(1), idesc_kk);
            umma_commit(&s_full[1]);
          }
        }
      }
      for (int j = 0; j < n_it && ok; ++j) {
        if (!mbar_wait(ds_ready, j & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        if (j + 1 < n_it) {           // dP of the next block: its region was released with dS_j
          if (!wait_v(j + 1)) { ok = false; break; }
          tc_fence_after();
          issue_dp(j + 1);
        }
        issue_ts(T_DQ, s_region(j), k_addr(j), idesc_ts, j > 0);   // dQ += dS_j K_j
        umma_commit(&k_empty[j % DQ_K_STAGES]);
        if (j + 1 == n_it) umma_commit(acc_full);
        if (j + 2 < n_it) {           // S of block j+2 reuses the region dS_j is being read from (in order)
          if (!wait_k(j + 2)) { ok = false; break; }
          tc_fence_after();
          issue_ss(s_region(j), q_addr, k_addr(j + 2), idesc_kk);
          umma_commit(&s_full[j & 1]);
        }
      }
    }
  } else {
    // compute warps: one thread per (query row, half of the 128 key columns); warps 2-5 take keys
    // 0-63 of the block, warps 6-9 keys 64-127 (see the dK/dV kernel for the hand-off rule).
    const int qtr = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = qtr * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const size_t row_base = ((size_t)b * p.H + h) * p.S;
    const float lse2 = q < p.S ? p.lse[row_base + q] * LOG2E : INFINITY;
    const float dlt = q < p.S ? p.delta[row_base + q] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_it && ok; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_s = s_region(j) + lane_off;
      const int kv0 = j * BLK + half * 64;
      const bool need_mask = (p.causal && (kv0 + 63 > q0)) || (kv0 + 64 > p.S);
      const int limit = p.causal ? min(q, p.S - 1) : (p.S - 1);
      float pr[64];
      {
        uint32_t sv[64];
        tmem_ld_32x32b_x32(t_s + half * 64, sv);
        tmem_ld_32x32b_x32(t_s + half * 64 + 32, sv + 32);
        tmem_ld_wait();
        if (half == 0) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_read[qtr]);
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float pv = exp2f(__uint_as_float(sv[i]) * p.scale_log2 - lse2);
          if (need_mask && kv0 + i > limit) pv = 0.f;
          pr[i] = pv;
        }
      }
      if (!mbar_wait(dp_full, j & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t ds[32];
      {
        uint32_t dv[64];
        tmem_ld_32x32b_x32(T_DP + lane_off + half * 64, dv);
        tmem_ld_32x32b_x32(T_DP + lane_off + half * 64 + 32, dv + 32);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          ds[i] = pack_bf16x2(pr[2 * i] * (__uint_as_float(dv[2 * i]) - dlt),
                              pr[2 * i + 1] * (__uint_as_float(dv[2 * i + 1]) - dlt));
      }
      // dS (bf16) overwrites S: packed columns [32 * half, +32)
      if (half == 1) {
        if (!mbar_wait(&s_read[qtr], j & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
      }
      tmem_st_32x32b_x32(t_s + half * 32, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    const bool have = n_it > 0 && ok && mbar_wait(acc_full, 0, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL);
    if (have) {
      tc_fence_after();
      acc_to_staging(T_DQ + lane_off, sQ, row, p.scale, half * 2, half * 2 + 2);
      fence_proxy_async_smem();
    }
    named_barrier_sync(1, COMPUTE_THREADS);
    if (have && threadIdx.x == 64) {
      for (int c = 0; c < 2; ++c) tma_store_3d(&tm_dq, sQ + c * CHUNK_BYTES, h * D + c * 64, q0, b);
      tma_store_commit();
      tma_store_wait_all<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

static int make_bsd_map(CUtensorMap* m, const void* base, int B, int S, int heads, long pitch) {
  const uint64_t dims[3] = {(uint64_t)heads * D, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[2] = {(uint64_t)pitch * 2, (uint64_t)S * pitch * 2};
  const uint32_t box[3] = {64, 128, 1};
  return kb::make_tmap_3d(m, base, 2, dims, strides, box, true);
}

}  // namespace fab
}  // namespace kb

extern "C" int kb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S,
                            int H, int Hkv, int Dh, long q_pitch, long k_pitch, long v_pitch, long o_pitch,
                            long do_pitch, long dq_pitch, long dk_pitch, long dv_pitch, float scale,
                            int causal, void* stream) {
  using namespace kb::fab;
  if (Dh != D || B <= 0 || S <= 0 || H <= 0 || Hkv <= 0 || H % Hkv) return KB_STATUS_BAD_ARG;
  auto bad = [](const void* p, long pitch) { return (reinterpret_cast<uintptr_t>(p) & 15) || (pitch & 7); };
  if (bad(q, q_pitch) || bad(k, k_pitch) || bad(v, v_pitch) || bad(o, o_pitch) || bad(d_o, do_pitch) ||
      bad(dq, dq_pitch) || bad(dk, dk_pitch) || bad(dv, dv_pitch) || !lse || !delta)
    return KB_STATUS_BAD_ARG;
  static bool attr_set_dev[64] = {false};  // the attribute is per device
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_set_dev[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_DQ) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (make_bsd_map(&tq, q, B, S, H, q_pitch) || make_bsd_map(&tk, k, B, S, Hkv, k_pitch) ||
      make_bsd_map(&tv, v, B, S, Hkv, v_pitch) || make_bsd_map(&tdo, d_o, B, S, H, do_pitch) ||
      make_bsd_map(&tdq, dq, B, S, H, dq_pitch) || make_bsd_map(&tdk, dk, B, S, Hkv, dk_pitch) ||
      make_bsd_map(&tdv, dv, B, S, Hkv, dv_pitch))
    return KB_STATUS_TMAP_ERROR;
  int dev = 0;
  cudaGetDevice(&dev);
  BwdParams p;
  p.lse = lse; p.delta = delta;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * LOG2E;
  p.causal = causal;
  p.n_blocks = (S + BLK - 1) / BLK;
  p.err = kb::error_word(dev);

  const long pairs = (long)B * S * H;
  delta_kernel<<<(unsigned)((pairs * 16 + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, B, S, H, o_pitch, do_pitch);
  flash_bwd_dkdv_kernel<<<dim3(p.n_blocks * Hkv * B), NUM_THREADS, SMEM_BYTES, st>>>(tq, tk, tv, tdo, tdk, tdv, p);
  flash_bwd_dq_kernel<<<dim3(p.n_blocks * H * B), NUM_THREADS, SMEM_BYTES_DQ, st>>>(tq, tk, tv, tdo, tdq, p);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}
