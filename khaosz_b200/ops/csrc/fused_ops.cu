// Bandwidth-bound kernels of the training / inference path: RMSNorm (+residual) forward and
// backward, rotary embedding, SwiGLU forward/backward, label-smoothed cross entropy
// forward/backward (also emits target log-probs for DPO/GRPO), embedding gather /
// scatter-add, squared-norm reduction and the flat AdamW update.
// All of them move 16 bytes per thread per access and keep their arithmetic in fp32.
#include "common.cuh"
#include "kb_api.h"

namespace kb {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z),
         d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void unpack8(uint4 v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16x2(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  uint4 v;
  v.x = pack_bf16x2(f[0], f[1]);
  v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]);
  v.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

// Block-wide sum of up to N values per thread; `red` holds N * 32 floats.
template <int N>
__device__ __forceinline__ void block_sum(float* vals, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int i = 0; i < N; ++i) vals[i] = warp_sum(vals[i]);
  __syncthreads();  // protects `red` against the previous use
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < N; ++i) red[i * 32 + warp] = vals[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float v = lane < nwarps ? red[i * 32 + lane] : 0.f;
    vals[i] = warp_sum(v);
  }
}

// =======================================================================================
// RMSNorm forward: one warp per row.
// =======================================================================================
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd,
                                   int rows, int dim, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int nchunks = dim >> 3;
  const __nv_bfloat16* xr = x + (size_t)row * dim;
  const __nv_bfloat16* rr = res ? res + (size_t)row * dim : nullptr;
  __nv_bfloat16* sr = sum_out ? sum_out + (size_t)row * dim : nullptr;
  float ss = 0.f;
#pragma unroll 4
  for (int c = lane; c < nchunks; c += 32) {
    float f[8];
    load8(xr + c * 8, f);
    if (rr) {
      float g[8];
      load8(rr + c * 8, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] += g[e];
      // round to the stored precision so that forward and backward see the same input
      uint4 v;
      v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
      v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
      *reinterpret_cast<uint4*>(sr + c * 8) = v;
      float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z),
             d = unpack_bf16x2(v.w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = cc.x; f[5] = cc.y; f[6] = d.x; f[7] = d.y;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dim + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  const __nv_bfloat16* src = rr ? sr : xr;  // the sum was just written by this warp
  __syncwarp();
#pragma unroll 4
  for (int c = lane; c < nchunks; c += 32) {
    float f[8], g[8];
    load8(src + c * 8, f);
    load8(w + c * 8, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = f[e] * r * g[e];
    store8(y + (size_t)row * dim + c * 8, f);
  }
}

// =======================================================================================
// RMSNorm backward. The CTA walks rows in groups of 4; every thread owns fixed columns so the
// weight gradient accumulates in registers and leaves the CTA once, as one partial row.
// =======================================================================================
constexpr int RMS_BWD_THREADS = 256;
constexpr int RMS_BWD_MAX_NCH = 4;  // dim <= 8 * 256 * 4 = 8192
constexpr int RMS_BWD_ROWS = 4;

// KEEP: the dy / x chunks of the four rows stay in registers (as packed bf16) between the two
// passes, so every input byte is read exactly once; used while that fits (NCH <= 2).
template <int NCH, bool KEEP>
__global__ void __launch_bounds__(RMS_BWD_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int dim) {
  __shared__ float red[RMS_BWD_ROWS * 32];
  const int nchunks = dim >> 3;
  const int tid = threadIdx.x;
  float wacc[NCH][8];
  float wreg[NCH][8];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = tid + i * RMS_BWD_THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) wacc[i][e] = 0.f;
    if (c < nchunks) load8(w + c * 8, wreg[i]);
  }
  const float inv_dim = 1.f / (float)dim;
  for (int r0 = blockIdx.x * RMS_BWD_ROWS; r0 < rows; r0 += gridDim.x * RMS_BWD_ROWS) {
    float dot[RMS_BWD_ROWS];
    uint4 keep_a[KEEP ? RMS_BWD_ROWS : 1][KEEP ? NCH : 1], keep_b[KEEP ? RMS_BWD_ROWS : 1][KEEP ? NCH : 1];
#pragma unroll
    for (int j = 0; j < RMS_BWD_ROWS; ++j) dot[j] = 0.f;
    // pass 1: dot_j = sum_k dy*w*x  (all loads of the four rows are issued before the first use)
    if (KEEP) {
#pragma unroll
      for (int j = 0; j < RMS_BWD_ROWS; ++j) {
        const int row = r0 + j;
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          const int c = tid + i * RMS_BWD_THREADS;
          const bool live = row < rows && c < nchunks;
          keep_a[j][i] = live ? *reinterpret_cast<const uint4*>(dy + (size_t)row * dim + c * 8) : make_uint4(0u, 0u, 0u, 0u);
          keep_b[j][i] = live ? *reinterpret_cast<const uint4*>(x + (size_t)row * dim + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < RMS_BWD_ROWS; ++j) {
      const int row = r0 + j;
      if (row < rows) {
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          const int c = tid + i * RMS_BWD_THREADS;
          if (c < nchunks) {
            float a[8], b[8];
            if (KEEP) {
              unpack8(keep_a[j][i], a);
              unpack8(keep_b[j][i], b);
            } else {
              load8(dy + (size_t)row * dim + c * 8, a);
              load8(x + (size_t)row * dim + c * 8, b);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) dot[j] += a[e] * wreg[i][e] * b[e];
          }
        }
      }
    }
    block_sum<RMS_BWD_ROWS>(dot, red);
    // pass 2 (without KEEP the re-reads hit L1/L2): dx and the weight-gradient accumulation
#pragma unroll
    for (int j = 0; j < RMS_BWD_ROWS; ++j) {
      const int row = r0 + j;
      if (row < rows) {
        const float rs = rstd[row];
        const float coef = dot[j] * rs * rs * rs * inv_dim;
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
          const int c = tid + i * RMS_BWD_THREADS;
          if (c < nchunks) {
            float a[8], b[8], o[8];
            if (KEEP) {
              unpack8(keep_a[j][i], a);
              unpack8(keep_b[j][i], b);
            } else {
              load8(dy + (size_t)row * dim + c * 8, a);
              load8(x + (size_t)row * dim + c * 8, b);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              o[e] = a[e] * wreg[i][e] * rs - b[e] * coef;
              wacc[i][e] += a[e] * b[e] * rs;
            }
            if (dres) {
              float d[8];
              load8(dres + (size_t)row * dim + c * 8, d);
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] += d[e];
            }
            store8(dx + (size_t)row * dim + c * 8, o);
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = tid + i * RMS_BWD_THREADS;
    if (c < nchunks) {
      float* dst = dw_partial + (size_t)blockIdx.x * dim + c * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(wacc[i][0], wacc[i][1], wacc[i][2], wacc[i][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(wacc[i][4], wacc[i][5], wacc[i][6], wacc[i][7]);
    }
  }
}

// Picks the instantiation with the fewest per-thread column chunks that covers `dim`.
static void launch_rmsnorm_bwd(int blocks, cudaStream_t st, const __nv_bfloat16* dy, const __nv_bfloat16* x,
                               const __nv_bfloat16* w, const float* rstd, const __nv_bfloat16* dres,
                               __nv_bfloat16* dx, float* partial, int rows, int dim) {
  const int nch = ((dim >> 3) + RMS_BWD_THREADS - 1) / RMS_BWD_THREADS;
  if (nch <= 1) rmsnorm_bwd_kernel<1, true><<<blocks, RMS_BWD_THREADS, 0, st>>>(dy, x, w, rstd, dres, dx, partial, rows, dim);
  else if (nch <= 2) rmsnorm_bwd_kernel<2, true><<<blocks, RMS_BWD_THREADS, 0, st>>>(dy, x, w, rstd, dres, dx, partial, rows, dim);
  else rmsnorm_bwd_kernel<4, false><<<blocks, RMS_BWD_THREADS, 0, st>>>(dy, x, w, rstd, dres, dx, partial, rows, dim);
}

// out[col] = sum over rows of partial[row][col], in a fixed order (deterministic).  A block owns 8
// columns (one 32-byte sector per row) and walks the rows with 128 row lanes, so that a [~600, dim]
// partial matrix is spread over dim / 8 blocks instead of a handful.
constexpr int COLSUM_COLS = 8;
constexpr int COLSUM_LANES = 128;
__global__ void __launch_bounds__(COLSUM_COLS * COLSUM_LANES)
colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int nrows, int dim) {
  __shared__ float tile[COLSUM_LANES][COLSUM_COLS + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = blockIdx.x * COLSUM_COLS + tx;
  float s = 0.f;
  if (col < dim)
    for (int r = ty; r < nrows; r += COLSUM_LANES) s += partial[(size_t)r * dim + col];
  tile[ty][tx] = s;
  __syncthreads();
#pragma unroll
  for (int off = COLSUM_LANES / 2; off > 0; off >>= 1) {
    if (ty < off) tile[ty][tx] += tile[ty + off][tx];
    __syncthreads();
  }
  if (ty == 0 && col < dim) out[col] = tile[0][tx];
}

// =======================================================================================
// RoPE on interleaved pairs.
// =======================================================================================
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                            const float* __restrict__ cs, const int* __restrict__ pos, int tokens,
                            int seq_len, int n_heads, int head_dim, long row_stride, int inverse) {
  const int chunks_per_head = head_dim >> 3;
  const long total = (long)tokens * n_heads * chunks_per_head;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks_per_head);
    const long th = i / chunks_per_head;
    const int h = (int)(th % n_heads);
    const long t = th / n_heads;
    const int position = pos ? pos[t] : (int)(t % seq_len);
    const size_t off = (size_t)t * row_stride + (size_t)h * head_dim + c * 8;
    float f[8], o[8];
    load8(x + off, f);
    const float4* csp =
        reinterpret_cast<const float4*>(cs + ((size_t)position * (head_dim >> 1) + c * 4) * 2);
    const float4 c0 = csp[0], c1 = csp[1];
    const float co[4] = {c0.x, c0.z, c1.x, c1.z};
    float si[4] = {c0.y, c0.w, c1.y, c1.w};
    if (inverse) {
#pragma unroll
      for (int e = 0; e < 4; ++e) si[e] = -si[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      o[2 * e] = f[2 * e] * co[e] - f[2 * e + 1] * si[e];
      o[2 * e + 1] = f[2 * e] * si[e] + f[2 * e + 1] * co[e];
    }
    store8(y + off, o);
  }
}

// =======================================================================================
// SwiGLU
// =======================================================================================
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                                  int rows, int F) {
  const int cpr = F >> 3;
  const long total = (long)rows * cpr;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const long r = i / cpr;
    const int c = (int)(i - r * cpr);
    float g[8], u[8], o[8];
    load8(gu + (size_t)r * 2 * F + c * 8, g);
    load8(gu + (size_t)r * 2 * F + F + c * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = u[e] * (g[e] / (1.f + __expf(-g[e])));
    store8(h + (size_t)r * F + c * 8, o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ dgu,
                                  int rows, int F) {
  const int cpr = F >> 3;
  const long total = (long)rows * cpr;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const long r = i / cpr;
    const int c = (int)(i - r * cpr);
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + (size_t)r * 2 * F + c * 8, g);
    load8(gu + (size_t)r * 2 * F + F + c * 8, u);
    load8(dh + (size_t)r * F + c * 8, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-g[e]));
      const float silu = g[e] * sg;
      du[e] = d[e] * silu;
      dg[e] = d[e] * u[e] * (sg + silu * (1.f - sg));
    }
    store8(dgu + (size_t)r * 2 * F + c * 8, dg);
    store8(dgu + (size_t)r * 2 * F + F + c * 8, du);
  }
}

// =======================================================================================
// Cross entropy: one CTA per row, online log-sum-exp over the vocabulary.
// =======================================================================================
constexpr int CE_THREADS = 512;

__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
              float* __restrict__ loss, float* __restrict__ lse_out, float* __restrict__ logp,
              int V, long ld, float smoothing, long long ignore_index) {
  __shared__ float red[3 * 32];
  const int row = blockIdx.x;
  const __nv_bfloat16* z = logits + (size_t)row * ld;
  const int nchunks = V >> 3;
  float m = -INFINITY, s = 0.f, zsum = 0.f;
  for (int c = threadIdx.x; c < nchunks; c += CE_THREADS) {
    float f[8];
    load8(z + c * 8, f);
    float cm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) cm = fmaxf(cm, f[e]);
    const float nm = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      acc += __expf(f[e] - nm);
      zsum += f[e];
    }
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int j = (nchunks << 3) + threadIdx.x; j < V; j += CE_THREADS) {  // ragged tail
    const float f = __bfloat162float(z[j]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
    zsum += f;
  }
  // block reduce (max, then rescaled sums)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float wm = warp_max(m);
  float ws = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
  float wz = warp_sum(zsum);
  if (lane == 0) { red[warp] = wm; red[32 + warp] = ws; red[64 + warp] = wz; }
  __syncthreads();
  if (warp == 0) {
    const int nw = CE_THREADS / 32;
    float bm = lane < nw ? red[lane] : -INFINITY;
    float bs = lane < nw ? red[32 + lane] : 0.f;
    float bz = lane < nw ? red[64 + lane] : 0.f;
    const float gm = warp_max(bm);
    bs = warp_sum(bm == -INFINITY ? 0.f : bs * __expf(bm - gm));
    bz = warp_sum(bz);
    if (lane == 0) {
      const float lse = gm + logf(bs);
      const long long t = targets[row];
      lse_out[row] = lse;
      if (t == ignore_index || t < 0 || t >= V) {
        if (loss) loss[row] = 0.f;
        if (logp) logp[row] = 0.f;
      } else {
        const float zt = __bfloat162float(z[t]);
        if (loss) loss[row] = (1.f - smoothing) * (lse - zt) + smoothing * (lse - bz / (float)V);
        if (logp) logp[row] = zt - lse;
      }
    }
  }
}

__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
              const float* __restrict__ lse, const float* __restrict__ row_grad,
              __nv_bfloat16* __restrict__ dlogits, int V, long ld, float smoothing,
              long long ignore_index, int mode) {
  const int row = blockIdx.x;
  const __nv_bfloat16* z = logits + (size_t)row * ld;
  __nv_bfloat16* dz = dlogits + (size_t)row * ld;
  const long long t = targets[row];
  const bool ignored = (t == ignore_index || t < 0 || t >= V);
  const float g = ignored ? 0.f : row_grad[row];
  const float l = lse[row];
  const int nchunks = V >> 3;
  // mode 0: g * (p - (1-eps) onehot - eps/V) ; mode 1: g * (onehot - p)
  const float psign = mode == 0 ? 1.f : -1.f;
  const float hot = mode == 0 ? -(1.f - smoothing) : 1.f;
  const float uni = mode == 0 ? -smoothing / (float)V : 0.f;
  for (int c = threadIdx.x; c < nchunks; c += CE_THREADS) {
    float f[8], o[8];
    load8(z + c * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = psign * __expf(f[e] - l) + uni;
      if ((long long)(c * 8 + e) == t) v += hot;
      o[e] = g * v;
    }
    store8(dz + c * 8, o);
  }
  for (int j = (nchunks << 3) + threadIdx.x; j < V; j += CE_THREADS) {
    float v = psign * __expf(__bfloat162float(z[j]) - l) + uni;
    if ((long long)j == t) v += hot;
    dz[j] = __float2bfloat16(g * v);
  }
}

// =======================================================================================
// Embedding
// =======================================================================================
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table,
                                     const long long* __restrict__ ids, __nv_bfloat16* __restrict__ out,
                                     int tokens, int dim, int vocab) {
  const int cpr = dim >> 3;
  const long total = (long)tokens * cpr;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const long t = i / cpr;
    const int c = (int)(i - t * cpr);
    long long id = ids[t];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < vocab) v = *reinterpret_cast<const uint4*>(table + (size_t)id * dim + c * 8);
    *reinterpret_cast<uint4*>(out + (size_t)t * dim + c * 8) = v;
  }
}

__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                     const long long* __restrict__ ids, float* __restrict__ dtable,
                                     int tokens, int dim, int vocab) {
  const int cpr = dim >> 3;
  const long total = (long)tokens * cpr;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const long t = i / cpr;
    const int c = (int)(i - t * cpr);
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float f[8];
    load8(dy + (size_t)t * dim + c * 8, f);
    float* dst = dtable + (size_t)id * dim + c * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(dst + e, f[e]);
  }
}

// =======================================================================================
// Optimiser
// =======================================================================================
__global__ void sumsq_kernel(const __nv_bfloat16* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const long long nchunks = n >> 3;
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < nchunks;
       c += (long long)gridDim.x * blockDim.x) {
    float f[8];
    load8(g + c * 8, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += f[e] * f[e];
  }
  if (blockIdx.x == 0) {
    for (long long j = (nchunks << 3) + threadIdx.x; j < n; j += blockDim.x) {
      const float f = __bfloat162float(g[j]);
      acc += f * f;
    }
  }
  float v[1] = {acc};
  block_sum<1>(v, red);
  if (threadIdx.x == 0) atomicAdd(out, v[0]);
}

__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, long long n,
                             const float* __restrict__ lr_step, float beta1, float beta2, float eps,
                             float wd, float grad_scale, const float* __restrict__ gnorm_sq,
                             float max_norm) {
  const float lr = lr_step[0];
  const float step = lr_step[1];
  float gs = grad_scale;
  if (gnorm_sq != nullptr && max_norm > 0.f) {
    const float norm = sqrtf(*gnorm_sq) * grad_scale;
    gs *= fminf(1.f, max_norm / (norm + 1e-6f));
  }
  const float bc1 = 1.f - powf(beta1, step);
  const float bc2 = 1.f - powf(beta2, step);
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd;
  const long long nchunks = n >> 3;
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < nchunks;
       c += (long long)gridDim.x * blockDim.x) {
    float pf[8], gf[8];
    load8(p + c * 8, pf);
    load8(g + c * 8, gf);
    float4 m0 = *reinterpret_cast<float4*>(m + c * 8), m1 = *reinterpret_cast<float4*>(m + c * 8 + 4);
    float4 v0 = *reinterpret_cast<float4*>(v + c * 8), v1 = *reinterpret_cast<float4*>(v + c * 8 + 4);
    float mf[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vf[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gr = gf[e] * gs;
      mf[e] = beta1 * mf[e] + (1.f - beta1) * gr;
      vf[e] = beta2 * vf[e] + (1.f - beta2) * gr * gr;
      const float denom = sqrtf(vf[e]) * inv_sqrt_bc2 + eps;
      pf[e] = pf[e] * decay - step_size * mf[e] / denom;
    }
    store8(p + c * 8, pf);
    *reinterpret_cast<float4*>(m + c * 8) = make_float4(mf[0], mf[1], mf[2], mf[3]);
    *reinterpret_cast<float4*>(m + c * 8 + 4) = make_float4(mf[4], mf[5], mf[6], mf[7]);
    *reinterpret_cast<float4*>(v + c * 8) = make_float4(vf[0], vf[1], vf[2], vf[3]);
    *reinterpret_cast<float4*>(v + c * 8 + 4) = make_float4(vf[4], vf[5], vf[6], vf[7]);
  }
  if (blockIdx.x == 0) {
    for (long long j = (nchunks << 3) + threadIdx.x; j < n; j += blockDim.x) {
      const float gr = __bfloat162float(g[j]) * gs;
      const float mm = beta1 * m[j] + (1.f - beta1) * gr;
      const float vv = beta2 * v[j] + (1.f - beta2) * gr * gr;
      m[j] = mm;
      v[j] = vv;
      const float denom = sqrtf(vv) * inv_sqrt_bc2 + eps;
      p[j] = __float2bfloat16(__bfloat162float(p[j]) * decay - step_size * mm / denom);
    }
  }
}

inline int grid_for(long long work_items, int threads, int sm_mult = 8) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = (long long)sms * sm_mult;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}
inline bool mis16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }
inline int launch_status() {
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

}  // namespace kb

using namespace kb;
typedef __nv_bfloat16 bf16;

extern "C" {

int kb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out,
                   float* rstd, int rows, int dim, float eps, void* stream) {
  if (rows <= 0) return KB_STATUS_OK;
  if ((dim & 7) || mis16(x) || mis16(y) || mis16(w) || (res && (mis16(res) || !sum_out || mis16(sum_out))))
    return KB_STATUS_BAD_ARG;
  const int wpb = 8;
  rmsnorm_fwd_kernel<<<(rows + wpb - 1) / wpb, wpb * 32, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)y, (bf16*)sum_out, rstd, rows, dim, eps);
  return launch_status();
}

int kb_rmsnorm_bwd_partials(int rows) {
  int blocks = (rows + RMS_BWD_ROWS - 1) / RMS_BWD_ROWS;
  const int cap = grid_for(1LL << 40, RMS_BWD_THREADS, 2);  // two CTAs are resident per SM (registers)
  return blocks < cap ? (blocks < 1 ? 1 : blocks) : cap;
}

int kb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                   const void* dres_in, void* dx, float* dw, float* dw_partial, int rows, int dim,
                   void* stream) {
  if (rows <= 0) return KB_STATUS_OK;
  if ((dim & 7) || dim > 8 * RMS_BWD_THREADS * RMS_BWD_MAX_NCH) return KB_STATUS_BAD_ARG;
  if (mis16(dy) || mis16(x) || mis16(w) || mis16(dx) || mis16(dw_partial) || (dres_in && mis16(dres_in)))
    return KB_STATUS_BAD_ARG;
  const int blocks = kb_rmsnorm_bwd_partials(rows);
  launch_rmsnorm_bwd(blocks, (cudaStream_t)stream, (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd,
                     (const bf16*)dres_in, (bf16*)dx, dw_partial, rows, dim);
  colsum_kernel<<<(dim + COLSUM_COLS - 1) / COLSUM_COLS, dim3(COLSUM_COLS, COLSUM_LANES), 0, (cudaStream_t)stream>>>(dw_partial, dw, blocks, dim);
  return launch_status();
}

int kb_rope(const void* x, void* y, const float* cs, const int* pos, int tokens, int seq_len,
            int n_heads, int head_dim, long row_stride, int inverse, void* stream) {
  if (tokens <= 0 || n_heads <= 0) return KB_STATUS_OK;
  if ((head_dim & 7) || (row_stride & 7) || mis16(x) || mis16(y) || mis16(cs)) return KB_STATUS_BAD_ARG;
  const long long total = (long long)tokens * n_heads * (head_dim >> 3);
  rope_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (bf16*)y, cs, pos, tokens, seq_len, n_heads, head_dim, row_stride, inverse);
  return launch_status();
}

int kb_swiglu_fwd(const void* gu, void* h, int rows, int F, void* stream) {
  if (rows <= 0) return KB_STATUS_OK;
  if ((F & 7) || mis16(gu) || mis16(h)) return KB_STATUS_BAD_ARG;
  swiglu_fwd_kernel<<<grid_for((long long)rows * (F >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)gu, (bf16*)h, rows, F);
  return launch_status();
}

int kb_swiglu_bwd(const void* gu, const void* dh, void* dgu, int rows, int F, void* stream) {
  if (rows <= 0) return KB_STATUS_OK;
  if ((F & 7) || mis16(gu) || mis16(dh) || mis16(dgu)) return KB_STATUS_BAD_ARG;
  swiglu_bwd_kernel<<<grid_for((long long)rows * (F >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)gu, (const bf16*)dh, (bf16*)dgu, rows, F);
  return launch_status();
}

int kb_ce_fwd(const void* logits, const long long* targets, float* loss, float* lse, float* logp,
              int rows, int V, long ld, float smoothing, long long ignore_index, void* stream) {
  if (rows <= 0) return KB_STATUS_OK;
  if ((ld & 7) || mis16(logits) || !lse) return KB_STATUS_BAD_ARG;
  ce_fwd_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((const bf16*)logits, targets, loss, lse,
                                                               logp, V, ld, smoothing, ignore_index);
  return launch_status();
}

int kb_ce_bwd(const void* logits, const long long* targets, const float* lse, const float* row_grad,
              void* dlogits, int rows, int V, long ld, float smoothing, long long ignore_index,
              int mode, void* stream) {
  if (rows <= 0) return KB_STATUS_OK;
  if ((ld & 7) || mis16(logits) || mis16(dlogits)) return KB_STATUS_BAD_ARG;
  ce_bwd_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((const bf16*)logits, targets, lse,
                                                               row_grad, (bf16*)dlogits, V, ld,
                                                               smoothing, ignore_index, mode);
  return launch_status();
}

int kb_embedding_fwd(const void* table, const long long* ids, void* out, int tokens, int dim,
                     int vocab, void* stream) {
  if (tokens <= 0) return KB_STATUS_OK;
  if ((dim & 7) || mis16(table) || mis16(out)) return KB_STATUS_BAD_ARG;
  embedding_fwd_kernel<<<grid_for((long long)tokens * (dim >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)table, ids, (bf16*)out, tokens, dim, vocab);
  return launch_status();
}

int kb_embedding_bwd(const void* dy, const long long* ids, float* dtable, int tokens, int dim,
                     int vocab, void* stream) {
  if (tokens <= 0) return KB_STATUS_OK;
  if ((dim & 7) || mis16(dy) || mis16(dtable)) return KB_STATUS_BAD_ARG;
  embedding_bwd_kernel<<<grid_for((long long)tokens * (dim >> 3), 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)dy, ids, dtable, tokens, dim, vocab);
  return launch_status();
}

int kb_sumsq_bf16(const void* g, long long n, float* out, void* stream) {
  if (n <= 0) return KB_STATUS_OK;
  if (mis16(g)) return KB_STATUS_BAD_ARG;
  sumsq_kernel<<<grid_for(n >> 3, 256, 4), 256, 0, (cudaStream_t)stream>>>((const bf16*)g, n, out);
  return launch_status();
}

int kb_adamw_bf16(void* p, const void* g, float* m, float* v, long long n, const float* lr_step,
                  float beta1, float beta2, float eps, float weight_decay, float grad_scale,
                  const float* gnorm_sq, float max_norm, void* stream) {
  if (n <= 0) return KB_STATUS_OK;
  if (mis16(p) || mis16(g) || mis16(m) || mis16(v)) return KB_STATUS_BAD_ARG;
  adamw_kernel<<<grid_for(n >> 3, 256, 8), 256, 0, (cudaStream_t)stream>>>(
      (bf16*)p, (const bf16*)g, m, v, n, lr_step, beta1, beta2, eps, weight_decay, grad_scale,
      gnorm_sq, max_norm);
  return launch_status();
}

}  // extern "C"

// =======================================================================================
// Allocation-free RMSNorm backward (see kb_noalloc.h).  The per-CTA weight-gradient partials
// go to a file-scope device array instead of a caller-provided buffer.
// =======================================================================================
#include <stdio.h>

#include "kb_noalloc.h"

namespace {
// Scratch for the weight-gradient partial rows: [KB_STATIC_RMS_MAX_PARTIALS][dim] floats.
static __device__ __align__(256) float g_rms_static_scratch[KB_STATIC_RMS_MAX_PARTIALS * KB_STATIC_RMS_MAX_DIM];

// In host code the array's name is only a handle; the device address is looked up once per
// device and cached here.
constexpr int kStaticMaxDevices = 64;
float* g_rms_static_ptr[kStaticMaxDevices] = {nullptr};
thread_local char g_rms_static_msg[192] = "";

int rms_static_fail(int status, const char* fmt, long a, long b) {
  snprintf(g_rms_static_msg, sizeof(g_rms_static_msg), fmt, a, b);
  return status;
}
}  // namespace

extern "C" const char* kb_rmsnorm_bwd_static_error(void) { return g_rms_static_msg; }

extern "C" int kb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd,
                                     const void* dres_in, void* dx, float* dw, int rows, int dim,
                                     void* stream) {
  g_rms_static_msg[0] = '\0';
  if (rows <= 0) return KB_STATUS_OK;
  if (dim <= 0 || (dim & 7))
    return rms_static_fail(KB_STATUS_BAD_ARG, "kb_rmsnorm_bwd_static: dim %ld must be a positive multiple of 8", dim, 0);
  if (dim > KB_STATIC_RMS_MAX_DIM)
    return rms_static_fail(KB_STATUS_TOO_LARGE,
                           "kb_rmsnorm_bwd_static: dim %ld exceeds the built-in scratch (max %ld); use "
                           "kb_rmsnorm_bwd with a caller-provided buffer", dim, KB_STATIC_RMS_MAX_DIM);
  if (mis16(dy) || mis16(x) || mis16(w) || mis16(dx) || (dres_in && mis16(dres_in)) || !rstd || !dw)
    return rms_static_fail(KB_STATUS_BAD_ARG, "kb_rmsnorm_bwd_static: null or misaligned (16 B) pointer", 0, 0);

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices)
    return rms_static_fail(KB_STATUS_CUDA_ERROR, "kb_rmsnorm_bwd_static: cannot query the current device", 0, 0);
  if (g_rms_static_ptr[dev] == nullptr) {
    // once per device, with that device current
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rms_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return rms_static_fail(KB_STATUS_CUDA_ERROR, "kb_rmsnorm_bwd_static: cudaGetSymbolAddress failed (%ld)",
                             (long)e, 0);
    g_rms_static_ptr[dev] = p;
  }
  float* scratch = g_rms_static_ptr[dev];

  int blocks = (rows + RMS_BWD_ROWS - 1) / RMS_BWD_ROWS;
  if (blocks > KB_STATIC_RMS_MAX_PARTIALS) blocks = KB_STATIC_RMS_MAX_PARTIALS;  // the kernel strides over rows
  launch_rmsnorm_bwd(blocks, (cudaStream_t)stream, (const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd,
                     (const bf16*)dres_in, (bf16*)dx, scratch, rows, dim);
  colsum_kernel<<<(dim + COLSUM_COLS - 1) / COLSUM_COLS, dim3(COLSUM_COLS, COLSUM_LANES), 0, (cudaStream_t)stream>>>(scratch, dw, blocks, dim);
  if (cudaGetLastError() != cudaSuccess)
    return rms_static_fail(KB_STATUS_CUDA_ERROR, "kb_rmsnorm_bwd_static: kernel launch failed", 0, 0);
  return KB_STATUS_OK;
}
