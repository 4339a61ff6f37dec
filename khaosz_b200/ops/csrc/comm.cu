// Collectives issued from inside kernels over NVLink peer memory (symmetric buffers: every
// rank passes the same-sized buffer and knows every peer's pointer to it).
//
//   kb_reduce_adamw      gradient reduce-scatter + global-norm clip + sharded AdamW + parameter
//                        all-gather for the data-parallel executors: rank r owns slice r of the
//                        flat parameter vector, pulls that slice of every peer's gradient
//                        (plain peer loads, or one multimem.ld_reduce through the NVSwitch),
//                        updates it, and pushes the new values into every peer's parameter
//                        buffer (peer stores or multimem.st).
//   kb_allreduce_bf16    stand-alone sum all-reduce (reduce own slice, write it everywhere).
//   kb_reducescatter_bf16 / kb_allgather_bf16 / kb_broadcast_bf16
//                        stand-alone collectives over one symmetric buffer.
//   kb_unit_reduce_bf16  block-granular full sharding: reduce-scatter of the ranks' gradient images
//                        with the accumulation into the owned piece and the clearing of the image
//                        in the same kernel (the matching gather is a copy-engine pull, no kernel).
//   kb_peer_barrier      stand-alone barrier (also the unit test of the bounded wait).
//
// Synchronisation: a control buffer of epoch counters, one row of `ws` words per CTA slot.
// A barrier stores the current epoch into row[slot][my rank] of every peer (release, system
// scope) and waits until its own row holds that epoch from every peer (acquire), for at most
// KB_WAIT_BUDGET_NS; on expiry the kernel records KB_ERR_TIMEOUT_PEER and skips its work, so a
// missing peer can never hang the GPU.  No TMA multicast is used anywhere.
#include "comm.cuh"
#include "kb_api.h"

namespace kb {
namespace comm {

constexpr int UNROLL = 4;  // 16-byte remote loads each thread keeps in flight

__device__ __forceinline__ void acc8(float* acc, uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = unpack_bf16x2(w[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_bf16x8(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------------------------------
// Phase 1: reduce my slice of the gradients (mean over ranks), keep it in my own gradient
// buffer, accumulate its squared norm.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 2)   // <= 64 registers: a light CTA fits beside a persistent GEMM CTA
reduce_slice_kernel(Peers grads, const void* grad_mc, Peers ctrl, int rank, int ws, long long slice_off,
                    long long slice_n, long long bucket_n, long long total_n, float scale, float* norm_sq_local,
                    uint32_t epoch, int* err) {
  // bucket_n == 0: one contiguous slice [slice_off, slice_off + slice_n).  Otherwise slice_off is the
  // first element of the first bucket of a run of buckets and slice_n the summed length of this rank's
  // sub-slices in them; local element i of the run lives at bucket_off(i) (see adamw_allgather_kernel).
  __shared__ float red[32];
  if (!cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch, err, KB_WAIT_BUDGET_NS)) return;
  const long long per = bucket_n > 0 ? bucket_n / ws : 1;
  auto where = [&](long long c) -> long long {   // global element of local chunk c
    if (bucket_n == 0) return slice_off + c * 8;
    const long long i = c * 8;
    const long long b = i / per;
    const long long first = slice_off + b * bucket_n;
    const long long left = total_n - first;
    const long long len_b = left < bucket_n ? left : bucket_n;
    return first + rank * (len_b / ws) + (i - b * per);
  };
  __nv_bfloat16* mine = static_cast<__nv_bfloat16*>(grads.p[rank]);
  const long long nchunks = slice_n >> 3;
  float sq = 0.f;
  // UNROLL chunks per thread per trip: the remote loads of a trip are all issued before the
  // first one is consumed, which is what hides the NVLink / NVSwitch round trip
  const long long stride = (long long)gridDim.x * blockDim.x;  // launched with THREADS or fewer threads
  for (long long c0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; c0 < nchunks; c0 += stride * UNROLL) {
    uint4 raw[UNROLL];
    float acc[UNROLL][8];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (grad_mc != nullptr && c < nchunks)
        raw[u] = multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(grad_mc) + where(c));
    }
    if (grad_mc != nullptr) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
    } else {
      long long at[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) at[u] = (c0 + u * stride) < nchunks ? where(c0 + u * stride) : -1;
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r) {
        if (r < ws) {
          const int peer = (rank + r) % ws;  // spread the traffic: every rank starts with itself
          const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(grads.p[peer]);
#pragma unroll
          for (int u = 0; u < UNROLL; ++u)
            raw[u] = at[u] >= 0 ? *reinterpret_cast<const uint4*>(src + at[u]) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
      if (c >= nchunks) break;
      uint4 o;
      o.x = pack_bf16x2(acc[u][0] * scale, acc[u][1] * scale);
      o.y = pack_bf16x2(acc[u][2] * scale, acc[u][3] * scale);
      o.z = pack_bf16x2(acc[u][4] * scale, acc[u][5] * scale);
      o.w = pack_bf16x2(acc[u][6] * scale, acc[u][7] * scale);
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += (acc[u][e] * scale) * (acc[u][e] * scale);
      *reinterpret_cast<uint4*>(mine + where(c)) = o;
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) atomicAdd(norm_sq_local, v);
  }
}

// Phase 2 (one CTA): publish my partial squared norm to every peer, barrier, total.
__global__ void exchange_norm_kernel(Peers norms, Peers ctrl, int rank, int ws, const float* norm_sq_local,
                                     float* norm_sq_total, int slot, uint32_t epoch, int* err) {
  // a failed reduction (or any earlier failure on this device) leaves the total unset and the
  // update below refuses to run; the peers' waits run out and they refuse as well
  if (*reinterpret_cast<volatile int*>(err) != 0) return;
  if (threadIdx.x < ws)
    static_cast<float*>(norms.p[threadIdx.x])[rank] = *norm_sq_local;
  if (!cta_peer_barrier(ctrl, rank, ws, slot, epoch, err, KB_WAIT_BUDGET_NS)) return;
  if (threadIdx.x == 0) {
    float t = 0.f;
    const volatile float* mine = static_cast<const volatile float*>(norms.p[rank]);
    for (int r = 0; r < ws; ++r) t += mine[r];
    *norm_sq_total = t;
  }
}

// Phase 3: AdamW on my slice, new parameters to every rank, closing barrier.
__global__ void __launch_bounds__(THREADS)
adamw_allgather_kernel(Peers params, void* param_mc, Peers grads, Peers ctrl, int rank, int ws,
                       long long bucket_n, long long total_n, long long slice_n, float* m, float* v,
                       const float* lr_step, float beta1, float beta2, float eps, float wd, const float* norm_sq_total,
                       float max_norm, uint32_t epoch, int* err) {
  // Never update from gradients that were not reduced or a norm that was not exchanged: with the
  // error word set the moments and the parameters of every rank stay exactly as they were.
  if (*reinterpret_cast<volatile int*>(err) != 0) return;
  const float lr = lr_step[0], step = lr_step[1];
  float gs = 1.f;
  if (max_norm > 0.f) gs = fminf(1.f, max_norm / (sqrtf(*norm_sq_total) + 1e-6f));
  const float bc1 = 1.f - powf(beta1, step), bc2 = 1.f - powf(beta2, step);
  const float step_size = lr / bc1, inv_sqrt_bc2 = rsqrtf(bc2), decay = 1.f - lr * wd;
  // This rank owns sub-slice `rank` of every bucket of `bucket_n` elements (the last bucket may be
  // shorter); its moments are stored bucket after bucket.  Local element i -> global element:
  __nv_bfloat16* p_base = static_cast<__nv_bfloat16*>(params.p[rank]);
  const __nv_bfloat16* g_base = static_cast<const __nv_bfloat16*>(grads.p[rank]);
  const long long per = bucket_n / ws;
  const long long nchunks = slice_n >> 3;
  for (long long c = blockIdx.x * (long long)THREADS + threadIdx.x; c < nchunks; c += (long long)gridDim.x * THREADS) {
    const long long i = c * 8;
    const long long b = i / per;
    const long long left = total_n - b * bucket_n;
    const long long len_b = left < bucket_n ? left : bucket_n;
    const long long goff = b * bucket_n + rank * (len_b / ws) + (i - b * per);
    float pf[8] = {0}, gf[8] = {0};
    acc8(pf, *reinterpret_cast<const uint4*>(p_base + goff));
    acc8(gf, *reinterpret_cast<const uint4*>(g_base + goff));
    float4 m0 = *reinterpret_cast<float4*>(m + c * 8), m1 = *reinterpret_cast<float4*>(m + c * 8 + 4);
    float4 v0 = *reinterpret_cast<float4*>(v + c * 8), v1 = *reinterpret_cast<float4*>(v + c * 8 + 4);
    float mf[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vf[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float g = gf[e] * gs;
      mf[e] = beta1 * mf[e] + (1.f - beta1) * g;
      vf[e] = beta2 * vf[e] + (1.f - beta2) * g * g;
      pf[e] = pf[e] * decay - step_size * mf[e] / (sqrtf(vf[e]) * inv_sqrt_bc2 + eps);
    }
    *reinterpret_cast<float4*>(m + c * 8) = make_float4(mf[0], mf[1], mf[2], mf[3]);
    *reinterpret_cast<float4*>(m + c * 8 + 4) = make_float4(mf[4], mf[5], mf[6], mf[7]);
    *reinterpret_cast<float4*>(v + c * 8) = make_float4(vf[0], vf[1], vf[2], vf[3]);
    *reinterpret_cast<float4*>(v + c * 8 + 4) = make_float4(vf[4], vf[5], vf[6], vf[7]);
    uint4 o;
    o.x = pack_bf16x2(pf[0], pf[1]); o.y = pack_bf16x2(pf[2], pf[3]);
    o.z = pack_bf16x2(pf[4], pf[5]); o.w = pack_bf16x2(pf[6], pf[7]);
    if (param_mc != nullptr) {
      multimem_st_bf16x8(static_cast<__nv_bfloat16*>(param_mc) + goff, o);
    } else {
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < ws) {
          const int peer = (rank + r) % ws;
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[peer]) + goff) = o;
        }
    }
  }
  cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch, err, KB_WAIT_BUDGET_NS);
}

// Stand-alone all-reduce (sum * scale) of a symmetric bf16 buffer, in place on every rank.
__global__ void __launch_bounds__(THREADS)
allreduce_kernel(Peers bufs, void* mc, Peers ctrl, int rank, int ws, long long n, float scale, uint32_t epoch,
                 int* err) {
  if (!cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch, err, KB_WAIT_BUDGET_NS)) return;
  const long long per = (n / ws) & ~7LL;
  const long long off = per * rank;
  const long long cnt = (rank == ws - 1) ? (n - off) : per;
  const long long nchunks = cnt >> 3;
  const long long stride = (long long)gridDim.x * THREADS;
  for (long long c0 = blockIdx.x * (long long)THREADS + threadIdx.x; c0 < nchunks; c0 += stride * UNROLL) {
    uint4 raw[UNROLL];
    float acc[UNROLL][8];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (mc != nullptr && c < nchunks)
        raw[u] = multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(mc) + off + c * 8);
    }
    if (mc != nullptr) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
    } else {
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < ws) {
          const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(bufs.p[(rank + r) % ws]) + off;
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long long c = c0 + u * stride;
            raw[u] = c < nchunks ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
      if (c >= nchunks) break;
      uint4 o;
      o.x = pack_bf16x2(acc[u][0] * scale, acc[u][1] * scale); o.y = pack_bf16x2(acc[u][2] * scale, acc[u][3] * scale);
      o.z = pack_bf16x2(acc[u][4] * scale, acc[u][5] * scale); o.w = pack_bf16x2(acc[u][6] * scale, acc[u][7] * scale);
      if (mc != nullptr) {
        multimem_st_bf16x8(static_cast<__nv_bfloat16*>(mc) + off + c * 8, o);
      } else {
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < ws) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bufs.p[(rank + r) % ws]) + off + c * 8) = o;
      }
    }
  }
  cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch + 1, err, KB_WAIT_BUDGET_NS);
}

// Stand-alone reduce-scatter: out[0, n / ws) = scale * sum over ranks of bufs[r][rank * n / ws ...).
// `out` is local memory (it may be the rank's own piece of its buffer).  The closing barrier keeps
// every rank's buffer intact until all pieces have been read.
__global__ void __launch_bounds__(THREADS)
reducescatter_kernel(Peers bufs, const void* mc, Peers ctrl, int rank, int ws, long long n, float scale,
                     __nv_bfloat16* out, uint32_t epoch, int* err) {
  if (!cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch, err, KB_WAIT_BUDGET_NS)) return;
  const long long per = n / ws;
  const long long off = per * rank;
  const long long nchunks = per >> 3;
  const long long stride = (long long)gridDim.x * THREADS;
  for (long long c0 = blockIdx.x * (long long)THREADS + threadIdx.x; c0 < nchunks; c0 += stride * UNROLL) {
    uint4 raw[UNROLL];
    float acc[UNROLL][8];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (mc != nullptr && c < nchunks)
        raw[u] = multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(mc) + off + c * 8);
    }
    if (mc != nullptr) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
    } else {
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < ws) {
          const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(bufs.p[(rank + r) % ws]) + off;
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long long c = c0 + u * stride;
            raw[u] = c < nchunks ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
      if (c >= nchunks) break;
      uint4 o;
      o.x = pack_bf16x2(acc[u][0] * scale, acc[u][1] * scale); o.y = pack_bf16x2(acc[u][2] * scale, acc[u][3] * scale);
      o.z = pack_bf16x2(acc[u][4] * scale, acc[u][5] * scale); o.w = pack_bf16x2(acc[u][6] * scale, acc[u][7] * scale);
      *reinterpret_cast<uint4*>(out + c * 8) = o;
    }
  }
  cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch + 1, err, KB_WAIT_BUDGET_NS);
}

// Stand-alone all-gather / broadcast over a symmetric buffer of n elements: rank `src_rank` (all-gather:
// every rank, its own piece [rank * n / ws ...); broadcast: the root, the whole buffer) stores its data
// into every peer's buffer (one multimem.st per 16 bytes through the switch, or one store per peer).
// The opening barrier makes sure that nobody still reads what is overwritten, the closing one that
// everything has landed.
__global__ void __launch_bounds__(THREADS)
push_kernel(Peers bufs, void* mc, Peers ctrl, int rank, int ws, long long off, long long cnt, int active,
            uint32_t epoch, int* err) {
  if (!cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch, err, KB_WAIT_BUDGET_NS)) return;
  if (active) {
    const __nv_bfloat16* mine = static_cast<const __nv_bfloat16*>(bufs.p[rank]) + off;
    const long long nchunks = cnt >> 3;
    for (long long c = blockIdx.x * (long long)THREADS + threadIdx.x; c < nchunks; c += (long long)gridDim.x * THREADS) {
      const uint4 vv = *reinterpret_cast<const uint4*>(mine + c * 8);
      if (mc != nullptr) {
        multimem_st_bf16x8(static_cast<__nv_bfloat16*>(mc) + off + c * 8, vv);
      } else {
#pragma unroll
        for (int r = 1; r < MAX_RANKS; ++r)
          if (r < ws) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bufs.p[(rank + r) % ws]) + off + c * 8) = vv;
      }
    }
  }
  cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch + 1, err, KB_WAIT_BUDGET_NS);
}

// First half of a broadcast from `root`: piece r of the root's buffer goes to rank r (plain peer stores,
// the pieces spread over the root's CTAs); the all-gather that follows distributes the pieces.  Two
// passes of n / ws each over every link instead of ws - 1 full copies out of one GPU.
__global__ void __launch_bounds__(THREADS)
scatter_kernel(Peers bufs, Peers ctrl, int root, int rank, int ws, long long per, uint32_t epoch, int* err) {
  if (!cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch, err, KB_WAIT_BUDGET_NS)) return;
  if (rank == root) {
    const __nv_bfloat16* mine = static_cast<const __nv_bfloat16*>(bufs.p[rank]);
    const long long nchunks = per >> 3;
    const long long total = nchunks * (ws - 1);
    for (long long c = blockIdx.x * (long long)THREADS + threadIdx.x; c < total; c += (long long)gridDim.x * THREADS) {
      int dst = (int)(c / nchunks);
      const long long within = c - dst * nchunks;
      if (dst >= root) ++dst;   // every rank but the root itself
      const long long at = dst * per + within * 8;
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bufs.p[dst]) + at) = *reinterpret_cast<const uint4*>(mine + at);
    }
  }
  cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch + 1, err, KB_WAIT_BUDGET_NS);
}

// Block-granular full sharding, gradients: acc[0, per) += scale * sum over ranks of piece `rank` of the
// gradient images (acc: this rank's owned gradient piece, local memory).  After the closing barrier (all
// ranks have read what they own) the rank's own image is cleared for the block that uses it next.
__global__ void __launch_bounds__(THREADS, 2)   // <= 64 registers: light enough to sit beside a compute CTA
unit_reduce_kernel(Peers bufs, const void* mc, Peers ctrl, int rank, int ws, long long n, float scale,
                   __nv_bfloat16* __restrict__ acc_out, int clear, uint32_t epoch, int* err) {
  if (!cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch, err, KB_WAIT_BUDGET_NS)) return;
  const long long per = n / ws;
  const long long off = per * rank;
  const long long nchunks = per >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; c0 < nchunks; c0 += stride * UNROLL) {
    uint4 raw[UNROLL];
    float acc[UNROLL][8];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (mc != nullptr && c < nchunks)
        raw[u] = multimem_ld_reduce_bf16x8(static_cast<const __nv_bfloat16*>(mc) + off + c * 8);
    }
    if (mc != nullptr) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
    } else {
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < ws) {
          const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(bufs.p[(rank + r) % ws]) + off;
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long long c = c0 + u * stride;
            raw[u] = c < nchunks ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) acc8(acc[u], raw[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long c = c0 + u * stride;
      if (c >= nchunks) break;
      float old[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) old[e] = 0.f;
      acc8(old, *reinterpret_cast<const uint4*>(acc_out + c * 8));
      uint4 o;
      o.x = pack_bf16x2(old[0] + acc[u][0] * scale, old[1] + acc[u][1] * scale);
      o.y = pack_bf16x2(old[2] + acc[u][2] * scale, old[3] + acc[u][3] * scale);
      o.z = pack_bf16x2(old[4] + acc[u][4] * scale, old[5] + acc[u][5] * scale);
      o.w = pack_bf16x2(old[6] + acc[u][6] * scale, old[7] + acc[u][7] * scale);
      *reinterpret_cast<uint4*>(acc_out + c * 8) = o;
    }
  }
  if (!cta_peer_barrier(ctrl, rank, ws, blockIdx.x, epoch + 1, err, KB_WAIT_BUDGET_NS)) return;
  if (clear) {
    // the barrier is per CTA slot: CTA b of every rank has read its chunks, CTA b' may not have.  So CTA b
    // clears, in every rank's piece of its own image, exactly the chunks that CTA b of that rank reads.
    __nv_bfloat16* mine = static_cast<__nv_bfloat16*>(bufs.p[rank]);
    for (int r = 0; r < ws; ++r)
      for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < nchunks; c += stride)
        *reinterpret_cast<uint4*>(mine + r * per + c * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

__global__ void barrier_kernel(Peers ctrl, int rank, int ws, int slot, uint32_t epoch, int* err,
                               unsigned long long budget_ns) {
  cta_peer_barrier(ctrl, rank, ws, slot, epoch, err, budget_ns);
}

inline int grid_size() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;  // one CTA per SM: every CTA of every rank is resident, so per-CTA barriers are safe
}

inline Peers load_peers(const void* const* host_ptrs, int ws) {
  Peers p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < ws ? const_cast<void*>(host_ptrs[i]) : nullptr;
  return p;
}

}  // namespace comm
}  // namespace kb

extern "C" {

// Number of control rows (CTA slots) the kernels use: kb_comm_slots() rows of 8 uint32 words.
int kb_comm_slots(void) { return kb::comm::grid_size() + 8; }

// Pointer arrays are host arrays of `ws` device pointers (peer addresses of the symmetric
// buffers).  slice = [slice_off, slice_off + slice_n) elements, owned by this rank; slice_n and
// slice_off are multiples of 8.  `epoch` must grow by at least 4 between calls.
// scratch: 2 floats (local partial norm, total norm), zeroed by this call.
int kb_reduce_adamw(const void* const* grad_ptrs, const void* const* param_ptrs, const void* const* ctrl_ptrs,
                    const void* const* norm_ptrs, const void* grad_mc, void* param_mc, int rank, int ws,
                    long long slice_off, long long slice_n, float* m, float* v, const float* lr_step, float beta1,
                    float beta2, float eps, float weight_decay, float max_norm, float* scratch,
                    unsigned int epoch, void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || (slice_off & 7) || (slice_n & 7)) return KB_STATUS_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int dev = 0;
  cudaGetDevice(&dev);
  int* err = kb::error_word(dev);
  const Peers grads = load_peers(grad_ptrs, ws), params = load_peers(param_ptrs, ws);
  const Peers ctrl = load_peers(ctrl_ptrs, ws), norms = load_peers(norm_ptrs, ws);
  const int grid = grid_size();
  cudaMemsetAsync(scratch, 0, 2 * sizeof(float), st);
  reduce_slice_kernel<<<grid, THREADS, 0, st>>>(grads, grad_mc, ctrl, rank, ws, slice_off, slice_n, 0, 0, 1.f / ws,
                                                scratch, epoch, err);
  exchange_norm_kernel<<<1, 32, 0, st>>>(norms, ctrl, rank, ws, scratch, scratch + 1, grid, epoch + 1, err);
  // one bucket spanning the whole buffer: rank r owns [r * slice_n, (r + 1) * slice_n)
  adamw_allgather_kernel<<<grid, THREADS, 0, st>>>(params, param_mc, grads, ctrl, rank, ws, slice_n * ws, slice_n * ws,
                                                   slice_n, m, v, lr_step, beta1, beta2, eps, weight_decay, scratch + 1,
                                                   max_norm, epoch + 2, err);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// The same step in pieces, for gradient buckets that are reduced while the backward pass is still
// running.  The flat buffer of `total_n` elements is cut into buckets of `bucket_n` elements
// (a multiple of 8 * ws; the last one may be shorter, total_n too is a multiple of 8 * ws); rank r
// owns sub-slice r of every bucket.
//
// kb_reduce_bucket: mean over the ranks of this rank's sub-slices of the buckets b_lo .. b_hi (both
// inclusive) into its own gradient buffer, their squared norm added to norm_sq_local[0] (zeroed by the
// caller once per step).  One bucket with a small grid of light CTAs (`grid` x `threads`) shares the
// SMs with the backward pass; the run of buckets left at the end goes in one launch with the full
// grid.  Every rank must make the same calls in the same order, `epoch` growing by at least 1 per call.
int kb_reduce_bucket(const void* const* grad_ptrs, const void* const* ctrl_ptrs, const void* grad_mc, int rank, int ws,
                     long long bucket_n, long long total_n, int b_lo, int b_hi, float* norm_sq_local,
                     unsigned int epoch, int grid, int threads, void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || bucket_n <= 0 || total_n <= 0 || (bucket_n % (8 * ws)) ||
      (total_n % (8 * ws)) || b_lo < 0 || b_hi < b_lo || (long long)b_hi * bucket_n >= total_n)
    return KB_STATUS_BAD_ARG;
  if (grid < 1 || grid > grid_size() || threads < 32 || threads > THREADS || (threads & 31)) return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  const long long first = (long long)b_lo * bucket_n;
  long long last_end = (long long)(b_hi + 1) * bucket_n;
  if (last_end > total_n) last_end = total_n;
  const long long mine_n = (last_end - first) / ws;   // summed length of this rank's sub-slices in the run
  reduce_slice_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      load_peers(grad_ptrs, ws), grad_mc, load_peers(ctrl_ptrs, ws), rank, ws, first, mine_n, bucket_n, total_n, 1.f / ws,
      norm_sq_local, epoch, kb::error_word(dev));
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// kb_adamw_buckets: after every bucket has been reduced: exchange of the squared-norm partials
// (scratch[0] -> total in scratch[1]), clip factor, AdamW on this rank's sub-slices (moments m / v of
// total_n / ws elements, stored bucket after bucket) and the updated values stored to every rank.
// Uses epochs `epoch` and `epoch + 1`.
int kb_adamw_buckets(const void* const* grad_ptrs, const void* const* param_ptrs, const void* const* ctrl_ptrs,
                     const void* const* norm_ptrs, void* param_mc, int rank, int ws, long long bucket_n,
                     long long total_n, float* m, float* v, const float* lr_step, float beta1, float beta2, float eps,
                     float weight_decay, float max_norm, float* scratch, unsigned int epoch, void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || bucket_n <= 0 || total_n <= 0 ||
      (bucket_n % (8 * ws)) || (total_n % (8 * ws)))
    return KB_STATUS_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int dev = 0;
  cudaGetDevice(&dev);
  int* err = kb::error_word(dev);
  const Peers grads = load_peers(grad_ptrs, ws), params = load_peers(param_ptrs, ws);
  const Peers ctrl = load_peers(ctrl_ptrs, ws), norms = load_peers(norm_ptrs, ws);
  const int grid = grid_size();
  exchange_norm_kernel<<<1, 32, 0, st>>>(norms, ctrl, rank, ws, scratch, scratch + 1, grid, epoch, err);
  adamw_allgather_kernel<<<grid, THREADS, 0, st>>>(params, param_mc, grads, ctrl, rank, ws, bucket_n, total_n,
                                                   total_n / ws, m, v, lr_step, beta1, beta2, eps, weight_decay,
                                                   scratch + 1, max_norm, epoch + 1, err);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

int kb_allreduce_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, void* mc, int rank, int ws,
                      long long n, float scale, unsigned int epoch, void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || (n & 7)) return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  allreduce_kernel<<<grid_size(), THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      load_peers(buf_ptrs, ws), mc, load_peers(ctrl_ptrs, ws), rank, ws, n, scale, epoch, kb::error_word(dev));
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// out[n / ws] (local, bf16) = scale * sum over ranks of piece `rank` of the symmetric buffers; n a
// multiple of 8 * ws.  Uses epochs `epoch` and `epoch + 1`.
int kb_reducescatter_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, const void* mc, int rank, int ws,
                          long long n, float scale, void* out, unsigned int epoch, void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || n <= 0 || (n % (8 * ws)) || out == nullptr ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  reducescatter_kernel<<<grid_size(), THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      load_peers(buf_ptrs, ws), mc, load_peers(ctrl_ptrs, ws), rank, ws, n, scale, static_cast<__nv_bfloat16*>(out),
      epoch, kb::error_word(dev));
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// All-gather in place: every rank's piece [rank * n / ws, (rank + 1) * n / ws) of its symmetric buffer
// is stored into all the others.  n a multiple of 8 * ws.  Epochs `epoch`, `epoch + 1`.
int kb_allgather_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, void* mc, int rank, int ws,
                      long long n, unsigned int epoch, void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || n <= 0 || (n % (8 * ws))) return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  const long long per = n / ws;
  push_kernel<<<grid_size(), THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      load_peers(buf_ptrs, ws), mc, load_peers(ctrl_ptrs, ws), rank, ws, per * rank, per, 1, epoch, kb::error_word(dev));
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// Broadcast: the first n elements (a multiple of 8) of rank `root`'s symmetric buffer go to every rank.
// With n a multiple of 8 * ws: scatter of the pieces, then all-gather (uses
// epochs epoch .. epoch + 3); otherwise the root stores everything everywhere.
int kb_broadcast_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, void* mc, int root, int rank, int ws,
                      long long n, unsigned int epoch, void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || root < 0 || root >= ws || n <= 0 || (n & 7)) return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Peers bufs = load_peers(buf_ptrs, ws), ctrl = load_peers(ctrl_ptrs, ws);
  if (ws >= 2 && n % (8 * ws) == 0) {
    const long long per = n / ws;
    scatter_kernel<<<grid_size(), THREADS, 0, st>>>(bufs, ctrl, root, rank, ws, per, epoch, kb::error_word(dev));
    push_kernel<<<grid_size(), THREADS, 0, st>>>(bufs, mc, ctrl, rank, ws, per * rank, per, 1, epoch + 2, kb::error_word(dev));
  } else {
    push_kernel<<<grid_size(), THREADS, 0, st>>>(bufs, mc, ctrl, rank, ws, 0, n, rank == root ? 1 : 0, epoch,
                                                 kb::error_word(dev));
  }
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// Unit reduce: acc[0, n / ws) (local bf16) += scale * sum over ranks of piece `rank` of the symmetric images;
// with `clear` the rank's own image [0, n) is zeroed once every rank has read its piece; `grid` CTAs of
// `threads` threads (the same on every rank; out of range: one CTA per SM, 512 threads).  Epochs `epoch`, `epoch + 1`.
int kb_unit_reduce_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, const void* mc, int rank, int ws,
                        long long n, float scale, void* acc, int clear, unsigned int epoch, int grid, int threads,
                        void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws || n <= 0 || (n % (8 * ws)) || acc == nullptr ||
      (reinterpret_cast<uintptr_t>(acc) & 15))
    return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  const int g = (grid <= 0 || grid > grid_size()) ? grid_size() : grid;
  const int t = (threads < 32 || threads > THREADS || (threads & 31)) ? THREADS : threads;
  unit_reduce_kernel<<<g, t, 0, static_cast<cudaStream_t>(stream)>>>(
      load_peers(buf_ptrs, ws), mc, load_peers(ctrl_ptrs, ws), rank, ws, n, scale, static_cast<__nv_bfloat16*>(acc),
      clear, epoch, kb::error_word(dev));
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

// budget_ms <= 0 selects the default wait budget.
int kb_peer_barrier(const void* const* ctrl_ptrs, int rank, int ws, int slot, unsigned int epoch, int budget_ms,
                    void* stream) {
  using namespace kb::comm;
  if (ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws) return KB_STATUS_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  const unsigned long long budget = budget_ms > 0 ? (unsigned long long)budget_ms * 1000000ull : kb::KB_WAIT_BUDGET_NS;
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(load_peers(ctrl_ptrs, ws), rank, ws, slot, epoch,
                                                                 kb::error_word(dev), budget);
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

}  // extern "C"
