// Flash attention forward for sm_100a (head_dim 128, bf16, causal or full, GQA aware).
//
// Layout in and out is [B, S, H, D] (a token's heads are contiguous; q/k/v may be slices of
// one packed projection buffer, described by their row pitch), so no permute copies exist.
//
// One CTA owns two 128-row query tiles that share one K/V stream: two heads of the same KV
// group at the same query block when the group size is even, otherwise two consecutive
// query blocks of one head.  The two tiles are ping-ponged so one tile's softmax overlaps
// the other's tensor-core work:
//   warp 0       TMA producer (Q once; K and V through two 2-stage rings)
//   warp 1       tcgen05.mma issuer: S_t = Q_t K_j^T (smem x smem), O_t += P_t V_j (TMEM x smem)
//   warps 2-5    softmax warpgroup of tile 0 (one thread per query row)
//   warps 6-9    softmax warpgroup of tile 1
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  P (bf16) overwrites the
// first 64 columns of its S and is consumed by the PV MMA straight from TMEM; the running
// rescale of O happens in TMEM.  Every wait is bounded.
#include "common.cuh"
#include "kb_api.h"

namespace kb {
namespace fa {

constexpr int D = 128;
constexpr int BQ = 128;   // query rows per tile
constexpr int BKV = 128;  // keys per block
constexpr int CHUNK_BYTES = 128 * 64 * 2;  // one [128 x 64] bf16 SW128 box = 16 KiB
constexpr int TILE_BYTES = 2 * CHUNK_BYTES;
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 320;
constexpr int SMEM_BYTES = 2 * TILE_BYTES + 2 * KV_STAGES * TILE_BYTES + 256 + 1024;
constexpr float LOG2E = 1.4426950408889634f;

struct FwdParams {
  float* lse;  // [B, H, S]
  int B, S, H, Hkv;
  int T;       // number of keys (S for self-attention over one sequence; larger when a cached prefix precedes the queries)
  int kv_off;  // T - S: query row i sees keys 0 .. i + kv_off under the causal mask
  float scale_log2;
  int causal;
  int pair_heads;  // 1: tiles are heads (h, h+1) at one q block; 0: q blocks (2i, 2i+1) of one head
  int n_qblocks;
  int* err;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                 const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                       // [2 tiles][2 chunks]
  uint8_t* sK = sQ + 2 * TILE_BYTES;        // [stages][2 chunks]
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;  // [stages][2 atoms]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KV_STAGES * TILE_BYTES);
  uint64_t* q_full = bars;         // [1]
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* k_empty = bars + 3;    // [2]
  uint64_t* v_full = bars + 5;     // [2]
  uint64_t* v_empty = bars + 7;    // [2]
  uint64_t* s_full = bars + 9;     // [2]
  uint64_t* p_ready = bars + 11;   // [2]
  uint64_t* o_full = bars + 13;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which two tiles does this CTA own? (heavy causal tiles are scheduled first) ----
  // 1-D grid with the batch as the fast index: CTAs are handed to SMs in index order, so the heavy
  // (late) query blocks of every batch entry start first and the light ones fill the end
  const int b = blockIdx.x % p.B;
  int head[2], q0[2], nblk[2];
  {
    const int group = p.H / p.Hkv;
    int slot = blockIdx.x / p.B;
    if (p.pair_heads) {
      const int pairs = p.H / 2;
      const int qb = p.n_qblocks - 1 - slot / pairs;
      const int hp = slot % pairs;
      head[0] = 2 * hp; head[1] = 2 * hp + 1;
      q0[0] = q0[1] = qb * BQ;
    } else {
      const int qpairs = (p.n_qblocks + 1) / 2;
      const int qp = qpairs - 1 - slot / p.H;
      head[0] = head[1] = slot % p.H;
      q0[0] = (2 * qp) * BQ; q0[1] = (2 * qp + 1) * BQ;
    }
    (void)group;
    const int total_kv_blocks = (p.T + BKV - 1) / BKV;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      if (q0[t] >= p.S) nblk[t] = 0;
      else if (p.causal) nblk[t] = min(total_kv_blocks, (q0[t] + BQ - 1 + p.kv_off) / BKV + 1);
      else nblk[t] = total_kv_blocks;
    }
  }
  const int kv_head = head[0] / (p.H / p.Hkv);
  const int nmax = max(nblk[0], nblk[1]);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 4); mbar_init(&o_full[i], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_o);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0 && nmax > 0) {
      const int n_active = (nblk[0] > 0) + (nblk[1] > 0);
      mbar_expect_tx(q_full, n_active * TILE_BYTES);
      for (int t = 0; t < 2; ++t) {
        if (nblk[t] == 0) continue;
        for (int c = 0; c < 2; ++c)
          tma_load_3d(sQ + t * TILE_BYTES + c * CHUNK_BYTES, &tm_q, q_full, head[t] * D + c * 64, q0[t], b);
      }
      bool ok = true;
      for (int j = 0; j < nmax && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(&k_full[s], TILE_BYTES);
        for (int c = 0; c < 2; ++c)
          tma_load_3d(sK + s * TILE_BYTES + c * CHUNK_BYTES, &tm_k, &k_full[s], kv_head * D + c * 64, j * BKV, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(&v_full[s], TILE_BYTES);
        for (int c = 0; c < 2; ++c)
          tma_load_3d(sV + s * TILE_BYTES + c * CHUNK_BYTES, &tm_v, &v_full[s], kv_head * D + c * 64, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && nmax > 0) {
      const uint32_t idesc_s = umma_idesc(128, 128, false, false);
      const uint32_t idesc_o = umma_idesc(128, 128, false, true);
      auto issue_s = [&](int t, int stage) {
        const uint32_t q_addr = smem_u32(sQ + t * TILE_BYTES);
        const uint32_t k_addr = smem_u32(sK + stage * TILE_BYTES);
        const uint32_t d = tmem_base + t * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * CHUNK_BYTES + (ks & 3) * 32;
          umma_f16(d, umma_desc_kmajor(q_addr, off), umma_desc_kmajor(k_addr, off), idesc_s, ks ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t v_addr = smem_u32(sV + stage * TILE_BYTES);
        const uint32_t d = tmem_base + 256 + t * 128;
        const uint32_t a = tmem_base + t * 128;  // P: bf16 pairs in the first 64 columns of S_t
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16_ts(d, a + ks * 8, umma_desc_mnmajor(v_addr, ks * 16, CHUNK_BYTES), idesc_o,
                      (accumulate || ks) ? 1u : 0u);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nblk[t] > 0) issue_s(t, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < nmax && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const bool has_next = (j + 1) < nmax;
        const int sn = (j + 1) & 1;
        const uint32_t phn = ((j + 1) >> 1) & 1;
        if (!mbar_wait(&v_full[s], ph, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
        if (has_next && !mbar_wait(&k_full[sn], phn, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
        for (int t = 0; t < 2; ++t) {
          if (j < nblk[t]) {
            if (!mbar_wait(&p_ready[t], j & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
            tc_fence_after();
            issue_pv(t, s, j > 0);
            if (j == nblk[t] - 1) umma_commit(&o_full[t]);
          }
          if (j + 1 < nblk[t]) issue_s(t, sn);
        }
        if (!ok) break;
        umma_commit(&v_empty[s]);
        if (has_next) umma_commit(&k_empty[sn]);
      }
    }
  } else {
    // ------------------------------- softmax warpgroups -------------------------------
    const int t = (warp - 2) >> 2;       // tile handled by this warpgroup
    const int qtr = warp & 3;            // TMEM lane quarter of this warp
    const int row = qtr * 32 + lane;     // row inside the tile
    const int qrow = q0[t] + row;        // global query position
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + t * 128;
    const uint32_t o_addr = tmem_base + lane_off + 256 + t * 128;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    const int n = nblk[t];
    for (int j = 0; j < n && ok; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t sreg[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, sreg + c * 32);
      tmem_ld_wait();
      const int kv0 = j * BKV;
      const bool need_mask = (p.causal && (kv0 + BKV - 1 > q0[t] + p.kv_off)) || (kv0 + BKV > p.T);
      float mx = m_run;
      if (need_mask) {
        const int limit = p.causal ? min(qrow + p.kv_off, p.T - 1) : (p.T - 1);  // last visible key
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          float v = __uint_as_float(sreg[i]) * p.scale_log2;
          if (kv0 + i > limit) v = -INFINITY;
          sreg[i] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const float v = __uint_as_float(sreg[i]) * p.scale_log2;
          sreg[i] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      }
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = exp2f(m_run - m_use);
      float sum = 0.f;
      uint32_t preg[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float p0 = exp2f(__uint_as_float(sreg[2 * i]) - m_use);
        const float p1 = exp2f(__uint_as_float(sreg[2 * i + 1]) - m_use);
        sum += p0 + p1;
        preg[i] = pack_bf16x2(p0, p1);
      }
      l_run = l_run * alpha + sum;
      m_run = mx;
      tmem_st_32x32b_x32(s_addr, preg);
      tmem_st_32x32b_x32(s_addr + 32, preg + 32);
      // rescale the running output (skipped when no row of this warp moved its maximum)
      if (j > 0 && !__all_sync(0xffffffffu, alpha == 1.f)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(o_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x32(o_addr + c * 32, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    // ---- epilogue: O / l -> bf16 -> swizzled staging (the tile's Q buffer) -> TMA store ----
    if (n > 0 && ok && mbar_wait(&o_full[t], 0, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      uint8_t* stage = sQ + t * TILE_BYTES;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(o_addr + c * 32, o);
        tmem_ld_wait();
        uint8_t* chunk_base = stage + (c >> 1) * CHUNK_BYTES;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(o[ch * 8 + 0]) * inv_l, __uint_as_float(o[ch * 8 + 1]) * inv_l);
          v.y = pack_bf16x2(__uint_as_float(o[ch * 8 + 2]) * inv_l, __uint_as_float(o[ch * 8 + 3]) * inv_l);
          v.z = pack_bf16x2(__uint_as_float(o[ch * 8 + 4]) * inv_l, __uint_as_float(o[ch * 8 + 5]) * inv_l);
          v.w = pack_bf16x2(__uint_as_float(o[ch * 8 + 6]) * inv_l, __uint_as_float(o[ch * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(chunk_base + sw128_offset(row, (c & 1) * 4 + ch)) = v;
        }
      }
      if (qrow < p.S)
        p.lse[((size_t)b * p.H + head[t]) * p.S + qrow] = (m_run + log2f(l_run)) * (1.f / LOG2E);
      fence_proxy_async_smem();
      named_barrier_sync(1 + t, 128);
      if ((threadIdx.x & 127) == 64) {  // first thread of this warpgroup (threads 64 and 192)
        for (int c = 0; c < 2; ++c)
          tma_store_3d(&tm_o, stage + c * CHUNK_BYTES, head[t] * D + c * 64, q0[t], b);
        tma_store_commit();
        tma_store_wait_all<0>();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// [B, S, heads*D] view of a (possibly packed) projection buffer with row pitch `pitch`.
static int make_bsd_map(CUtensorMap* m, const void* base, int B, int S, int heads, long pitch) {
  const uint64_t dims[3] = {(uint64_t)heads * D, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[2] = {(uint64_t)pitch * 2, (uint64_t)S * pitch * 2};
  const uint32_t box[3] = {64, 128, 1};
  return kb::make_tmap_3d(m, base, 2, dims, strides, box, true);
}

}  // namespace fa
}  // namespace kb

extern "C" int kb_flash_fwd_rect(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int T,
                                 int H, int Hkv, int Dh, long q_pitch, long k_pitch, long v_pitch, long o_pitch,
                                 float scale, int causal, void* stream);

extern "C" int kb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                            int S, int H, int Hkv, int Dh, long q_pitch, long k_pitch, long v_pitch,
                            long o_pitch, float scale, int causal, void* stream) {
  return kb_flash_fwd_rect(q, k, v, o, lse, B, S, S, H, Hkv, Dh, q_pitch, k_pitch, v_pitch, o_pitch, scale, causal, stream);
}

// S queries against T >= S keys per sequence (k / v are [B, T, Hkv, D]); under the causal mask query
// i sees keys 0 .. i + (T - S): the queries are the last S positions of a sequence of T (prefill
// behind a cached prefix).  T == S is plain self-attention.
extern "C" int kb_flash_fwd_rect(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int T,
                                 int H, int Hkv, int Dh, long q_pitch, long k_pitch, long v_pitch, long o_pitch,
                                 float scale, int causal, void* stream) {
  using namespace kb::fa;
  if (Dh != D || B <= 0 || S <= 0 || T < S || H <= 0 || Hkv <= 0 || H % Hkv) return KB_STATUS_BAD_ARG;
  auto bad = [](const void* p, long pitch) { return (reinterpret_cast<uintptr_t>(p) & 15) || (pitch & 7); };
  if (bad(q, q_pitch) || bad(k, k_pitch) || bad(v, v_pitch) || bad(o, o_pitch) || !lse) return KB_STATUS_BAD_ARG;
  static bool attr_set_dev[64] = {false};  // the attribute is per device
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_set_dev[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  CUtensorMap tq, tk, tv, to;
  if (make_bsd_map(&tq, q, B, S, H, q_pitch) || make_bsd_map(&tk, k, B, T, Hkv, k_pitch) ||
      make_bsd_map(&tv, v, B, T, Hkv, v_pitch) || make_bsd_map(&to, o, B, S, H, o_pitch))
    return KB_STATUS_TMAP_ERROR;
  int dev = 0;
  cudaGetDevice(&dev);
  FwdParams p;
  p.lse = lse;
  p.B = B; p.S = S; p.H = H; p.Hkv = Hkv;
  p.T = T;
  p.kv_off = T - S;
  p.scale_log2 = scale * LOG2E;
  p.causal = causal;
  p.n_qblocks = (S + BQ - 1) / BQ;
  const int group = H / Hkv;
  p.pair_heads = (group % 2 == 0) ? 1 : 0;
  p.err = kb::error_word(dev);
  const int slots = p.pair_heads ? (H / 2) * p.n_qblocks : H * ((p.n_qblocks + 1) / 2);
  dim3 grid(slots * B);
  flash_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, to, p);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}
