// Inference-side kernels: paged KV-cache write, paged decode attention (block tables,
// split-KV, the query heads of one GQA group share every K/V load) and fused
// temperature / top-k / top-p sampling.  All bandwidth- or latency-bound; CUDA cores only.
#include "common.cuh"
#include "kb_api.h"

namespace kb {
namespace inf {

// ---------------------------------------------------------------------------------------
// KV write: pool[slot[t]] = k[t] (row of Hkv*D elements), same for v.  slot < 0 skips.
// ---------------------------------------------------------------------------------------
__global__ void paged_kv_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                      __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                                      const long long* __restrict__ slots, int tokens, int row_elems,
                                      long k_pitch, long v_pitch) {
  const int cpr = row_elems >> 3;
  const long total = (long)tokens * cpr;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / cpr;
    const int c = (int)(i - t * cpr);
    const long long slot = slots[t];
    if (slot < 0) continue;
    *reinterpret_cast<uint4*>(k_pool + slot * row_elems + c * 8) =
        *reinterpret_cast<const uint4*>(k + t * k_pitch + c * 8);
    *reinterpret_cast<uint4*>(v_pool + slot * row_elems + c * 8) =
        *reinterpret_cast<const uint4*>(v + t * v_pitch + c * 8);
  }
}

// ---------------------------------------------------------------------------------------
// RoPE (interleaved pairs, fp32) + optional per-head RMSNorm of q and k (applied after the
// rotation, as the model does) + the K/V page write, in one pass over a packed projection row
// [q heads | k heads | v heads].  One warp per (token, head); EPL = head_dim / 32 elements per lane.
// q and k are rotated (and normalised) in place, k and v rows are also stored to their page slot
// (slot < 0: no store, e.g. padding rows).
// ---------------------------------------------------------------------------------------
template <int EPL>
__global__ void __launch_bounds__(256)
rope_norm_kvwrite_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cs, const int* __restrict__ pos,
                         const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w, float eps,
                         const long long* __restrict__ slots, __nv_bfloat16* __restrict__ k_pool,
                         __nv_bfloat16* __restrict__ v_pool, int tokens, int seq_len, int H, int Hkv, long row_stride) {
  constexpr int D = EPL * 32;
  const int heads = H + 2 * Hkv;
  const long warp_id = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_id >= (long)tokens * heads) return;
  const long t = warp_id / heads;
  const int h = (int)(warp_id - t * heads);
  __nv_bfloat16* src = qkv + t * row_stride + (long)h * D + lane * EPL;
  float x[EPL];
#pragma unroll
  for (int i = 0; i < EPL; i += 2) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
    x[i] = f.x;
    x[i + 1] = f.y;
  }
  const long long slot = slots ? slots[t] : -1;
  if (h < H + Hkv) {
    const int position = pos ? pos[t] : (int)(t % seq_len);
    const float* c = cs + ((size_t)position * (D / 2) + lane * (EPL / 2)) * 2;
#pragma unroll
    for (int i = 0; i < EPL; i += 2) {
      const float co = c[i], si = c[i + 1];
      const float a = x[i], b = x[i + 1];
      x[i] = a * co - b * si;
      x[i + 1] = a * si + b * co;
    }
    const __nv_bfloat16* w = h < H ? q_w : k_w;
    if (w != nullptr) {
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) sq += x[i] * x[i];
      sq = warp_sum(sq);
      const float rs = rsqrtf(sq / (float)D + eps);
#pragma unroll
      for (int i = 0; i < EPL; ++i) x[i] = x[i] * rs * __bfloat162float(w[lane * EPL + i]);
    }
#pragma unroll
    for (int i = 0; i < EPL; i += 2)
      *reinterpret_cast<__nv_bfloat162*>(src + i) = __floats2bfloat162_rn(x[i], x[i + 1]);
  }
  if (h >= H && slot >= 0) {
    const bool is_k = h < H + Hkv;
    __nv_bfloat16* dst = (is_k ? k_pool : v_pool) + slot * ((long)Hkv * D) + (long)(h - H - (is_k ? 0 : Hkv)) * D + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; i += 2)
      *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(x[i], x[i + 1]);
  }
}

// ---------------------------------------------------------------------------------------
// Paged decode attention.  grid = (n_splits, Hkv, B), 128 threads, head_dim 128.
// Phase 1 (thread = key): scores of 128 keys against the G query heads of the group.
// Phase 2 (thread = output dim): P V accumulation with online rescaling.
// Partials (m, l, acc) per split are merged by decode_merge_kernel.
// ---------------------------------------------------------------------------------------
constexpr int DEC_D = 128;
constexpr int DEC_MAX_G = 8;
constexpr int DEC_THREADS = 128;

__global__ void __launch_bounds__(DEC_THREADS)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                    const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ block_table,
                    const int* __restrict__ seq_lens, float* __restrict__ part_acc, float* __restrict__ part_ml,
                    int H, int Hkv, int page_size, int max_pages, int n_splits, long q_pitch, float scale_log2) {
  __shared__ float sq[DEC_MAX_G][DEC_D];
  __shared__ float sp[DEC_MAX_G][DEC_THREADS];
  __shared__ float sred[DEC_MAX_G][4];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = H / Hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int len = seq_lens[b];
  const int per_split = ((len + n_splits - 1) / n_splits + DEC_THREADS - 1) / DEC_THREADS * DEC_THREADS;
  const int t_begin = split * per_split;
  const int t_end = min(len, t_begin + per_split);
  for (int g = 0; g < G; ++g)
    sq[g][tid] = __bfloat162float(q[(size_t)b * q_pitch + (size_t)(kvh * G + g) * DEC_D + tid]) * scale_log2;
  __syncthreads();
  float m_run[DEC_MAX_G], l_run[DEC_MAX_G], acc[DEC_MAX_G];
#pragma unroll
  for (int g = 0; g < DEC_MAX_G; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; acc[g] = 0.f; }
  const size_t row_elems = (size_t)Hkv * DEC_D;
  const int* table = block_table + (size_t)b * max_pages;

  for (int t0 = t_begin; t0 < t_end; t0 += DEC_THREADS) {
    // ---- phase 1: this thread's key ----
    const int t = t0 + tid;
    float s[DEC_MAX_G];
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) s[g] = -INFINITY;
    if (t < t_end) {
      const int page = table[t / page_size];
      const __nv_bfloat16* kr = k_pool + ((size_t)page * page_size + (t % page_size)) * row_elems + (size_t)kvh * DEC_D;
#pragma unroll
      for (int g = 0; g < DEC_MAX_G; ++g) s[g] = 0.f;
#pragma unroll 4
      for (int c = 0; c < DEC_D / 8; ++c) {
        const uint4 kv4 = *reinterpret_cast<const uint4*>(kr + c * 8);
        const uint32_t w[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
        float kf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(w[i]); kf[2 * i] = f.x; kf[2 * i + 1] = f.y; }
#pragma unroll
        for (int g = 0; g < DEC_MAX_G; ++g) {
          if (g < G) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s[g] += kf[e] * sq[g][c * 8 + e];
          }
        }
      }
    }
    // ---- block max / probabilities per head ----
    float alpha[DEC_MAX_G];
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) {
      if (g < G) {
        const float wm = warp_max(s[g]);
        if (lane == 0) sred[g][warp] = wm;
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) {
      if (g < G) {
        const float bm = fmaxf(fmaxf(sred[g][0], sred[g][1]), fmaxf(sred[g][2], sred[g][3]));
        const float m_new = fmaxf(m_run[g], bm);
        alpha[g] = (m_run[g] == -INFINITY) ? 0.f : exp2f(m_run[g] - m_new);
        const float pv = (t < t_end) ? exp2f(s[g] - m_new) : 0.f;
        sp[g][tid] = pv;
        m_run[g] = m_new;
        s[g] = pv;
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) {
      if (g < G) {
        const float ws = warp_sum(s[g]);
        if (lane == 0) sred[g][warp] = ws;
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) {
      if (g < G) {
        l_run[g] = l_run[g] * alpha[g] + (sred[g][0] + sred[g][1] + sred[g][2] + sred[g][3]);
        acc[g] *= alpha[g];
      }
    }
    // ---- phase 2: this thread's output dimension ----
    const int n_here = min(DEC_THREADS, t_end - t0);
    for (int j = 0; j < n_here; ++j) {
      const int tj = t0 + j;
      const int page = table[tj / page_size];
      const float vv = __bfloat162float(
          v_pool[((size_t)page * page_size + (tj % page_size)) * row_elems + (size_t)kvh * DEC_D + tid]);
#pragma unroll
      for (int g = 0; g < DEC_MAX_G; ++g)
        if (g < G) acc[g] += sp[g][j] * vv;
    }
    __syncthreads();
  }
  for (int g = 0; g < G; ++g) {
    const size_t idx = ((size_t)b * H + kvh * G + g) * n_splits + split;
    part_acc[idx * DEC_D + tid] = acc[g];
    if (tid == 0) { part_ml[idx * 2] = m_run[g]; part_ml[idx * 2 + 1] = l_run[g]; }
  }
}

__global__ void decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int n_splits, long out_pitch, int H) {
  const int bh = blockIdx.x;  // b * H + h
  const int tid = threadIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[((size_t)bh * n_splits + s) * 2]);
  float l = 0.f, a = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const size_t idx = (size_t)bh * n_splits + s;
    const float ms = part_ml[idx * 2];
    if (ms == -INFINITY) continue;
    const float w = exp2f(ms - m);
    l += part_ml[idx * 2 + 1] * w;
    a += part_acc[idx * DEC_D + tid] * w;
  }
  const int b = bh / H, h = bh - b * H;
  out[(size_t)b * out_pitch + (size_t)h * DEC_D + tid] = __float2bfloat16(l > 0.f ? a / l : 0.f);
}

// ---------------------------------------------------------------------------------------
// Sampling: one CTA per row.  temperature -> top-k (k-th largest found by bisection on the
// value range) -> top-p (smallest probability mass >= top_p, bisection on the probability
// threshold) -> inverse-CDF draw with a caller-provided uniform number.  top_k <= 0 and
// top_p >= 1 disable the filters; top_k == 1 is an exact argmax.
// ---------------------------------------------------------------------------------------
constexpr int SMP_THREADS = 1024;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[lane];  // SMP_THREADS / 32 == 32 entries
  r = is_max ? warp_max(r) : warp_sum(r);
  return r;
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const __nv_bfloat16* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              long long* __restrict__ out, int V, long ld) {
  extern __shared__ float sx[];  // V floats
  __shared__ float red[32];
  __shared__ float scan[SMP_THREADS];
  __shared__ int s_choice;
  const int row = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* z = logits + (size_t)row * ld;
  const float inv_t = 1.f / fmaxf(temperature ? temperature[row] : 1.f, 1e-8f);
  const int k = top_k ? top_k[row] : 0;
  const float pcut = top_p ? top_p[row] : 1.f;

  float mx = -INFINITY;
  for (int i = tid; i < V; i += SMP_THREADS) {
    const float v = __bfloat162float(z[i]) * inv_t;
    sx[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = block_reduce(mx, red, true);

  if (k == 1 || pcut <= 0.f) {  // greedy: lowest index among the maxima
    int best = V;
    for (int i = tid; i < V; i += SMP_THREADS)
      if (sx[i] == mx) { best = i; break; }
    float bf = block_reduce(-(float)best, red, true);
    if (tid == 0) out[row] = (long long)(-bf);
    return;
  }

  // ---- top-k: threshold = k-th largest value ----
  float thr = -INFINITY;
  if (k > 0 && k < V) {
    float mn = INFINITY;
    for (int i = tid; i < V; i += SMP_THREADS) mn = fminf(mn, sx[i]);
    mn = -block_reduce(-mn, red, true);
    float lo = mn, hi = mx;  // count(x >= lo) >= k always; find the largest such lo
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f;
      for (int i = tid; i < V; i += SMP_THREADS) cnt += (sx[i] >= mid) ? 1.f : 0.f;
      cnt = block_reduce(cnt, red, false);
      if (cnt >= (float)k) lo = mid; else hi = mid;
    }
    thr = lo;
  }
  // ---- probabilities of the kept tokens (unnormalised, relative to the max) ----
  float total = 0.f;
  for (int i = tid; i < V; i += SMP_THREADS) {
    const float p = (sx[i] >= thr) ? __expf(sx[i] - mx) : 0.f;
    sx[i] = p;
    total += p;
  }
  total = block_reduce(total, red, false);
  // ---- top-p: largest tau with mass(p >= tau) >= pcut * total ----
  float tau = 0.f;
  if (pcut < 1.f) {
    float lo = 0.f, hi = 1.f;  // p of the max token is exactly 1
    const float want = pcut * total;
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float mass = 0.f;
      for (int i = tid; i < V; i += SMP_THREADS) mass += (sx[i] >= mid) ? sx[i] : 0.f;
      mass = block_reduce(mass, red, false);
      if (mass >= want) lo = mid; else hi = mid;
    }
    tau = lo;
    total = 0.f;
    for (int i = tid; i < V; i += SMP_THREADS) {
      if (sx[i] < tau) sx[i] = 0.f;
      total += sx[i];
    }
    total = block_reduce(total, red, false);
  }
  // ---- inverse CDF: thread t owns the contiguous slice [t*per, (t+1)*per) ----
  const int per = (V + SMP_THREADS - 1) / SMP_THREADS;
  const int b0 = tid * per, b1 = min(V, b0 + per);
  float mine = 0.f;
  for (int i = b0; i < b1; ++i) mine += sx[i];
  scan[tid] = mine;
  __syncthreads();
  for (int off = 1; off < SMP_THREADS; off <<= 1) {  // inclusive Hillis-Steele scan
    const float add = tid >= off ? scan[tid - off] : 0.f;
    __syncthreads();
    scan[tid] += add;
    __syncthreads();
  }
  const float target = fminf(uniform[row], 0.99999994f) * scan[SMP_THREADS - 1];
  if (tid == 0) s_choice = -1;
  __syncthreads();
  const float before = scan[tid] - mine;
  if (mine > 0.f && target >= before && target < scan[tid]) {
    float run = before;
    int pick = b0;
    for (int i = b0; i < b1; ++i) {
      if (sx[i] > 0.f) {
        pick = i;
        run += sx[i];
        if (run > target) break;
      }
    }
    s_choice = pick;
  }
  __syncthreads();
  if (tid == 0) {
    int c = s_choice;
    if (c < 0) {  // numerical corner: fall back to the arg-max
      for (int i = 0; i < V; ++i) if (sx[i] >= 1.f) { c = i; break; }
      if (c < 0) c = 0;
    }
    out[row] = c;
  }
}

}  // namespace inf
}  // namespace kb

extern "C" {

// k, v: [tokens, row_elems] rows (pitches in elements); pools: [n_slots, row_elems];
// slots: int64 [tokens] destination row of each token (< 0 skips the token).
int kb_paged_kv_write(const void* k, const void* v, void* k_pool, void* v_pool, const void* slots,
                      int tokens, int row_elems, long k_pitch, long v_pitch, void* stream) {
  if (tokens <= 0) return KB_STATUS_OK;
  if ((row_elems & 7) || (k_pitch & 7) || (v_pitch & 7)) return KB_STATUS_BAD_ARG;
  const long long total = (long long)tokens * (row_elems >> 3);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  kb::inf::paged_kv_write_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
      (const long long*)slots, tokens, row_elems, k_pitch, v_pitch);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// qkv: [tokens, row_stride] rows of (H + 2 Hkv) heads of head_dim in {64, 128, 256}; see the kernel.
// q_w / k_w: per-head RMSNorm weights [head_dim] or NULL; slots: int64 [tokens] or NULL (no page write).
int kb_rope_norm_kvwrite(void* qkv, const float* cs, const int* pos, const void* q_w, const void* k_w, float eps,
                         const long long* slots, void* k_pool, void* v_pool, int tokens, int seq_len, int H, int Hkv,
                         int head_dim, long row_stride, void* stream) {
  using namespace kb::inf;
  if (tokens <= 0) return KB_STATUS_OK;
  if (H <= 0 || Hkv <= 0 || (row_stride & 1) || (reinterpret_cast<uintptr_t>(qkv) & 3) || (slots && (!k_pool || !v_pool)))
    return KB_STATUS_BAD_ARG;
  const long warps = (long)tokens * (H + 2 * Hkv);
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
  auto go = [&](auto kern) {
    kern<<<blocks, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)qkv, cs, pos, (const __nv_bfloat16*)q_w,
                                                   (const __nv_bfloat16*)k_w, eps, slots, (__nv_bfloat16*)k_pool,
                                                   (__nv_bfloat16*)v_pool, tokens, seq_len, H, Hkv, row_stride);
  };
  switch (head_dim) {
    case 64: go(rope_norm_kvwrite_kernel<2>); break;
    case 128: go(rope_norm_kvwrite_kernel<4>); break;
    case 256: go(rope_norm_kvwrite_kernel<8>); break;
    default: return KB_STATUS_BAD_ARG;
  }
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// q [B, H*128] (pitch q_pitch), pools [n_pages, page_size, Hkv, 128], block_table int32
// [B, max_pages], seq_lens int32 [B]; scratch: part_acc fp32 [B*H*n_splits*128], part_ml fp32
// [B*H*n_splits*2]; out [B, H*128] (pitch out_pitch).
int kb_paged_decode_attn(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                         const int* seq_lens, float* part_acc, float* part_ml, void* out, int B, int H,
                         int Hkv, int D, int page_size, int max_pages, int n_splits, long q_pitch,
                         long out_pitch, float scale, void* stream) {
  using namespace kb::inf;
  if (B <= 0) return KB_STATUS_OK;
  if (D != DEC_D || H % Hkv || H / Hkv > DEC_MAX_G || n_splits < 1) return KB_STATUS_BAD_ARG;
  paged_decode_kernel<<<dim3(n_splits, Hkv, B), DEC_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_table, seq_lens,
      part_acc, part_ml, H, Hkv, page_size, max_pages, n_splits, q_pitch, scale * 1.4426950408889634f);
  decode_merge_kernel<<<B * H, DEC_D, 0, (cudaStream_t)stream>>>(part_acc, part_ml, (__nv_bfloat16*)out, n_splits,
                                                                 out_pitch, H);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// Combines the split-KV partials of a decode step: out [B, H*128] (pitch out_pitch).
int kb_decode_merge(const float* part_acc, const float* part_ml, void* out, int B, int H, int n_splits,
                    long out_pitch, void* stream) {
  using namespace kb::inf;
  if (B <= 0) return KB_STATUS_OK;
  decode_merge_kernel<<<B * H, DEC_D, 0, (cudaStream_t)stream>>>(part_acc, part_ml, (__nv_bfloat16*)out, n_splits,
                                                                 out_pitch, H);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// logits bf16 [rows, V] (pitch ld); temperature/top_p fp32 [rows], top_k int32 [rows], uniform
// fp32 [rows] in [0,1); out int64 [rows].  Any of temperature/top_k/top_p may be NULL.
int kb_sample(const void* logits, const void* temperature, const void* top_k, const void* top_p,
              const void* uniform, void* out, int rows, int V, long ld, long long, void* stream) {
  using namespace kb::inf;
  if (rows <= 0) return KB_STATUS_OK;
  if (V <= 0 || (size_t)V * 4 > 200 * 1024 || !uniform) return KB_STATUS_TOO_LARGE;
  static bool attr_set_dev[64] = {false};  // the attribute is per device
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_set_dev[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  sample_kernel<<<rows, SMP_THREADS, (size_t)V * 4, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, (const float*)temperature, (const int*)top_k, (const float*)top_p,
      (const float*)uniform, (long long*)out, V, ld);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

}  // extern "C"
