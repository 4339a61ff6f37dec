// Paged-KV decode attention on the tensor cores (sm_100a, head_dim 128, bf16, GQA aware).
//
// One CTA per (KV split, KV head, sequence).  The query heads of the KV head's group (G <= 32)
// are the first G rows of a 128-row MMA tile (the other rows are zero fill and are ignored), so
// the K and V pages are streamed from HBM exactly once for the whole group:
//   warp 0   TMA producer: lane i fetches the id of page i of the current 128-key tile and issues
//            its [page_size x 64] boxes into the 128B-swizzled K / V stages (3-stage rings)
//   warp 1   tcgen05.mma issuer: S = Q K^T into one of two TMEM buffers (the next tile's S is
//            issued before this tile's softmax has finished), O += P V with P read from TMEM
//   warp 4   online softmax of rows 0..G-1 (TMEM lanes 0..31 belong to the warp with id % 4 == 0)
// The work is HBM bound: two MMAs of a tile cost ~1.7k cycles of a tensor pipe that would
// otherwise idle, against ~2.8k cycles to fetch the tile's 64 KiB at this SM's share of HBM.
// With n_splits == 1 the result is written directly; otherwise un-normalised partials go to the
// scratch buffers and kb_decode_merge combines them.  Every wait is bounded.
#include "common.cuh"
#include "kb_api.h"

extern "C" int kb_decode_merge(const float* part_acc, const float* part_ml, void* out, int B, int H, int n_splits,
                               long out_pitch, void* stream);

namespace kb {
namespace pdec {

constexpr int D = 128;
constexpr int BKV = 128;
constexpr int CHUNK_BYTES = 128 * 64 * 2;
constexpr int TILE_BYTES = 2 * CHUNK_BYTES;
constexpr int STAGES = 3;
constexpr int NUM_THREADS = 160;
constexpr int SOFTMAX_WARP = 4;
constexpr int SMEM_BYTES = TILE_BYTES + 2 * STAGES * TILE_BYTES + 256 + 1024;

struct Params {
  const int* block_table;  // [B, max_pages]
  const int* seq_lens;     // [B]
  float* part_acc;         // [B*H*n_splits, 128]
  float* part_ml;          // [B*H*n_splits, 2]
  __nv_bfloat16* out;      // [B, H*128] pitch out_pitch
  long out_pitch;
  int H, Hkv, page_size, max_pages, n_splits;
  float scale_log2;
  int* err;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;
  uint8_t* sV = sK + STAGES * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + STAGES * TILE_BYTES);
  uint64_t* q_full = bars;                       // [1]
  uint64_t* k_full = bars + 1;                   // [STAGES]
  uint64_t* k_empty = k_full + STAGES;           // [STAGES]
  uint64_t* v_full = k_empty + STAGES;           // [STAGES]
  uint64_t* v_empty = v_full + STAGES;           // [STAGES]
  uint64_t* s_full = v_empty + STAGES;           // [2]
  uint64_t* p_ready = s_full + 2;                // [1]
  uint64_t* pv_done = p_ready + 1;               // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int len = p.seq_lens[b];
  const int tiles_total = (len + BKV - 1) / BKV;
  const int tiles_per_split = (tiles_total + p.n_splits - 1) / p.n_splits;
  const int tile0 = split * tiles_per_split;
  const int n_tiles = max(0, min(tiles_total, tile0 + tiles_per_split) - tile0);
  const int seq_pages = (len + p.page_size - 1) / p.page_size;
  const int ppt = BKV / p.page_size;  // pages per tile

  // Stale shared memory must not reach the MMA as NaN through pages that are not loaded.
  for (int i = threadIdx.x; i < 2 * STAGES * TILE_BYTES / 16; i += NUM_THREADS)
    reinterpret_cast<uint4*>(sK)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) mbar_init(&s_full[i], 1);
    mbar_init(p_ready, 1); mbar_init(pv_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t T_S = tmem_base, T_O = tmem_base + 256;  // S0 | S1 | O

  if (warp == 0) {
    // ------------------------------- TMA producer (whole warp: the lanes fetch the page ids) -------------------------------
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(q_full, TILE_BYTES);
        for (int c = 0; c < 2; ++c) tma_load_3d(sQ + c * CHUNK_BYTES, &tm_q, q_full, c * 64, kvh * G, b);
      }
      const int* table = p.block_table + (size_t)b * p.max_pages;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % STAGES;
        const uint32_t ph = (j / STAGES) & 1;
        const int page0 = (tile0 + j) * ppt;
        int pg = -1;
        if (lane < ppt && page0 + lane < seq_pages && page0 + lane < p.max_pages) pg = table[page0 + lane];
        const int n_valid = __popc(__ballot_sync(0xffffffffu, pg >= 0));
        const uint32_t bytes = (uint32_t)n_valid * p.page_size * 128u * 2u;
        for (int which = 0; which < 2 && ok; ++which) {  // K first, then V
          uint64_t* empty = which ? &v_empty[s] : &k_empty[s];
          uint64_t* full = which ? &v_full[s] : &k_full[s];
          uint8_t* dst = (which ? sV : sK) + s * TILE_BYTES;
          const CUtensorMap* tm = which ? &tm_v : &tm_k;
          if (lane == 0) {
            ok = mbar_wait(empty, ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY);
            if (ok) mbar_expect_tx(full, bytes);
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          // every lane that holds a page issues that page's two boxes itself
          if (pg >= 0) {
            for (int c = 0; c < 2; ++c)
              tma_load_2d(dst + c * CHUNK_BYTES + lane * p.page_size * 128, tm, full, kvh * D + c * 64, pg * p.page_size);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = umma_idesc(128, 128, false, false);
      const uint32_t idesc_o = umma_idesc(128, 128, false, true);
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_s = [&](int j) {
        const uint32_t k_addr = smem_u32(sK + (j % STAGES) * TILE_BYTES);
        const uint32_t d = T_S + (j & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * CHUNK_BYTES + (ks & 3) * 32;
          umma_f16(d, umma_desc_kmajor(q_addr, off), umma_desc_kmajor(k_addr, off), idesc_s, ks ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[j % STAGES]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, p.err, KB_ERR_TIMEOUT_FULL);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % STAGES;
        const uint32_t ph = (j / STAGES) & 1;
        if (j + 1 < n_tiles) {
          if (!mbar_wait(&k_full[(j + 1) % STAGES], ((j + 1) / STAGES) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(&v_full[s], ph, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
        if (!mbar_wait(p_ready, j & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * TILE_BYTES);
        const uint32_t a = T_S + (j & 1) * 128;  // P: bf16 pairs in the first 64 columns of this tile's S
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16_ts(T_O, a + ks * 8, umma_desc_mnmajor(v_addr, ks * 16, CHUNK_BYTES), idesc_o, (j > 0 || ks) ? 1u : 0u);
        umma_commit(&v_empty[s]);
        umma_commit(pv_done);
      }
    }
  } else if (warp == SOFTMAX_WARP) {
    // ------------------------------- softmax of rows 0..G-1 -------------------------------
    const bool active = lane < G;
    const int head = kvh * G + lane;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = T_S + (j & 1) * 128;
      uint32_t sreg[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, sreg + c * 32);
      tmem_ld_wait();
      uint32_t preg[64];
      float alpha = 1.f;
      if (active) {
        const int kv0 = (tile0 + j) * BKV;
        const int n_keys = min(BKV, len - kv0);  // keys of this tile that exist
        float mx = m_run;
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          float v = __uint_as_float(sreg[i]) * p.scale_log2;
          if (i >= n_keys) v = -INFINITY;
          sreg[i] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
        const float m_use = (mx == -INFINITY) ? 0.f : mx;
        alpha = exp2f(m_run - m_use);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float p0 = exp2f(__uint_as_float(sreg[2 * i]) - m_use);
          const float p1 = exp2f(__uint_as_float(sreg[2 * i + 1]) - m_use);
          sum += p0 + p1;
          preg[i] = pack_bf16x2(p0, p1);
        }
        l_run = l_run * alpha + sum;
        m_run = mx;
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) preg[i] = 0u;
      }
      tmem_st_32x32b_x32(s_addr, preg);
      tmem_st_32x32b_x32(s_addr + 32, preg + 32);
      if (j > 0) {
        // the previous tile's P V must have landed in O before O is rescaled (or read by the next MMA)
        if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        if (!__all_sync(0xffffffffu, alpha == 1.f)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(T_O + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(T_O + c * 32, o);
          }
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // ---- epilogue ----
    if (n_tiles > 0 && ok) ok = mbar_wait(pv_done, (n_tiles - 1) & 1, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const size_t idx = ((size_t)b * p.H + head) * p.n_splits + split;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32b_x32(T_O + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (!active) continue;
        if (p.n_splits == 1) {
          __nv_bfloat16* dst = p.out + (size_t)b * p.out_pitch + (size_t)head * D + c * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[i * 8 + 0]) * inv_l, __uint_as_float(o[i * 8 + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(o[i * 8 + 2]) * inv_l, __uint_as_float(o[i * 8 + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(o[i * 8 + 4]) * inv_l, __uint_as_float(o[i * 8 + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(o[i * 8 + 6]) * inv_l, __uint_as_float(o[i * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(dst + i * 8) = v;
          }
        } else {
          float* dst = p.part_acc + idx * D + c * 32;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<uint4*>(dst + i * 4) = make_uint4(o[i * 4], o[i * 4 + 1], o[i * 4 + 2], o[i * 4 + 3]);
        }
      }
      if (active && p.n_splits > 1) {
        p.part_ml[idx * 2] = m_run;
        p.part_ml[idx * 2 + 1] = l_run;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace pdec
}  // namespace kb

// Same contract as kb_paged_decode_attn plus the pool's page count (extent of the tensor maps).
// Needs page_size in {16, 32, 64, 128}, 16-byte aligned q / pools / out and G = H / Hkv <= 32;
// returns KB_STATUS_BAD_ARG otherwise (the caller then uses the CUDA-core kernel).
extern "C" int kb_paged_decode_tc(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                  const int* seq_lens, float* part_acc, float* part_ml, void* out, int B, int H,
                                  int Hkv, int Dh, int page_size, int max_pages, int n_pool_pages, int n_splits,
                                  long q_pitch, long out_pitch, float scale, void* stream) {
  using namespace kb::pdec;
  if (B <= 0) return KB_STATUS_OK;
  if (Dh != D || Hkv <= 0 || H % Hkv || H / Hkv > 32 || n_splits < 1 || n_pool_pages <= 0) return KB_STATUS_BAD_ARG;
  if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return KB_STATUS_BAD_ARG;
  auto mis = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
  if (mis(q) || mis(k_pool) || mis(v_pool) || mis(out) || (q_pitch & 7) || (out_pitch & 7)) return KB_STATUS_BAD_ARG;
  if (n_splits > 1 && (!part_acc || !part_ml)) return KB_STATUS_BAD_ARG;
  static bool attr_set_dev[64] = {false};  // the attribute is per device
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_set_dev[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(paged_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  CUtensorMap tq, tk, tv;
  {
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)H, (uint64_t)B};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)q_pitch * 2};
    const uint32_t box[3] = {64, 128, 1};
    if (kb::make_tmap_3d(&tq, q, 2, dims, strides, box, true)) return KB_STATUS_TMAP_ERROR;
  }
  const uint64_t pool_rows = (uint64_t)n_pool_pages * page_size;
  if (kb::make_tmap_2d(&tk, k_pool, 2, pool_rows, (uint64_t)Hkv * D, (uint64_t)Hkv * D * 2, page_size, 64, true) ||
      kb::make_tmap_2d(&tv, v_pool, 2, pool_rows, (uint64_t)Hkv * D, (uint64_t)Hkv * D * 2, page_size, 64, true))
    return KB_STATUS_TMAP_ERROR;
  int dev = 0;
  cudaGetDevice(&dev);
  Params p;
  p.block_table = block_table; p.seq_lens = seq_lens; p.part_acc = part_acc; p.part_ml = part_ml;
  p.out = static_cast<__nv_bfloat16*>(out); p.out_pitch = out_pitch;
  p.H = H; p.Hkv = Hkv; p.page_size = page_size; p.max_pages = max_pages; p.n_splits = n_splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.err = kb::error_word(dev);
  paged_decode_tc_kernel<<<dim3(n_splits, Hkv, B), NUM_THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  if (cudaGetLastError() != cudaSuccess) return KB_STATUS_CUDA_ERROR;
  if (n_splits > 1) return kb_decode_merge(part_acc, part_ml, out, B, H, n_splits, out_pitch, stream);
  return KB_STATUS_OK;
}
