// C ABI of the khaosz_b200 kernel library (libkhaosz_b200_kernels.so).
// Every entry point takes raw device pointers and a CUDA stream handle, launches
// asynchronously on that stream and returns a KB_STATUS_* code.  Unless a comment says
// otherwise no entry point allocates device memory after the first call on a device
// (the first call sets up a 64-byte error word).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  KB_STATUS_OK = 0,
  KB_STATUS_BAD_ARG = 1,
  KB_STATUS_CUDA_ERROR = 2,
  KB_STATUS_TMAP_ERROR = 3,
  KB_STATUS_TOO_LARGE = 4,
};

// ---- runtime ------------------------------------------------------------------------
int kb_last_error(void);  // device-side status of bounded waits since the last call (0 = ok)
int kb_error_probe(int* pinned_host, void* stream);  // async copy of the error word (no sync)
int kb_store_f32x2(float* dst, float a, float b, void* stream);  // dst[0..1] = (a, b) on the stream
int kb_copy_async(void* dst, const void* src, long long bytes, void* stream);  // one device-to-device copy (source may be peer memory)
int kb_sm_count(void);
int kb_last_tmap_error(void);  // CUresult of the last failed tensor-map encode
const char* kb_version(void);

// ---- GEMM ---------------------------------------------------------------------------
// C[M,N] = op(A) op(B)^T (+R).  a_mn=0: A is [M,K] row-major (pitch lda); a_mn=1: A is stored
// [K,M] row-major.  b_mn=0: B is [N,K]; b_mn=1: B is stored [K,N].  epi: 0 none, 1 add R.
int kb_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                 long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi, void* stream);

// Same with an explicit tile width bn in {256, 192, 128}; bn = 0 picks the width that wastes the
// fewest SM-waves.
int kb_gemm_bf16_bn(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                    long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi, int bn,
                    void* stream);

// ---- normalisation ------------------------------------------------------------------
// y = rmsnorm(x (+ res)) * w ; when res != NULL the sum x+res is also written to sum_out.
int kb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out,
                   float* rstd, int rows, int dim, float eps, void* stream);
// dx = d rmsnorm (+ dres_in); dw_partial is scratch [n_partial_rows, dim] fp32 provided by the
// caller (n_partial_rows = kb_rmsnorm_bwd_partials(rows)); dw (fp32 [dim]) is overwritten.
int kb_rmsnorm_bwd_partials(int rows);
int kb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                   const void* dres_in, void* dx, float* dw, float* dw_partial, int rows, int dim,
                   void* stream);

// ---- rotary embedding ---------------------------------------------------------------
// In-place capable. x: [tokens, row_stride] bf16, rotates heads [0, n_heads) of width head_dim
// as interleaved (even, odd) pairs. cs: [max_pos, head_dim/2, 2] fp32 (cos, sin).
// pos: int32 [tokens] or NULL (position = token index % seq_len). inverse=1 applies the
// transpose rotation (backward pass).
int kb_rope(const void* x, void* y, const float* cs, const int* pos, int tokens, int seq_len,
            int n_heads, int head_dim, long row_stride, int inverse, void* stream);

// ---- SwiGLU -------------------------------------------------------------------------
// gu: [rows, 2*F] (gate = [:, :F], up = [:, F:]); h = up * silu(gate)
int kb_swiglu_fwd(const void* gu, void* h, int rows, int F, void* stream);
int kb_swiglu_bwd(const void* gu, const void* dh, void* dgu, int rows, int F, void* stream);

// ---- cross entropy ------------------------------------------------------------------
// logits [rows, V] bf16 (pitch ld), targets int64. Per-row outputs: loss (label-smoothed NLL,
// 0 for ignored rows), lse, and logp (log-prob of the target, 0 for ignored rows).
int kb_ce_fwd(const void* logits, const long long* targets, float* loss, float* lse, float* logp,
              int rows, int V, long ld, float smoothing, long long ignore_index, void* stream);
// dlogits = gscale[row-independent scalar on device] * dloss_row * d loss / d logits, written
// to `dlogits` (may alias logits). row_grad: fp32 [rows] upstream gradient per row.
// mode 0: gradient of the label-smoothed loss; mode 1: gradient of logp.
int kb_ce_bwd(const void* logits, const long long* targets, const float* lse,
              const float* row_grad, void* dlogits, int rows, int V, long ld, float smoothing,
              long long ignore_index, int mode, void* stream);

// ---- embedding ----------------------------------------------------------------------
int kb_embedding_fwd(const void* table, const long long* ids, void* out, int tokens, int dim,
                     int vocab, void* stream);
// dtable (fp32 [vocab, dim]) += scatter of dy; caller zero-fills.
int kb_embedding_bwd(const void* dy, const long long* ids, float* dtable, int tokens, int dim,
                     int vocab, void* stream);

// ---- optimiser ----------------------------------------------------------------------
// sum of squares of a bf16 buffer, accumulated into *out (fp32, caller zero-fills)
int kb_sumsq_bf16(const void* g, long long n, float* out, void* stream);
// AdamW over a flat bf16 parameter / gradient buffer with fp32 moments.
// grad_scale multiplies gradients first; if gnorm_sq != NULL and max_norm > 0 the clip factor
// min(1, max_norm / (sqrt(*gnorm_sq) * grad_scale + 1e-6)) is applied too (no host sync).
// lr and step are read from device memory (lr_step[0] = lr, lr_step[1] = bias-correction step).
int kb_adamw_bf16(void* p, const void* g, float* m, float* v, long long n, const float* lr_step,
                  float beta1, float beta2, float eps, float weight_decay, float grad_scale,
                  const float* gnorm_sq, float max_norm, void* stream);

// ---- attention ----------------------------------------------------------------------
// Causal / full flash attention, q [B,S,H,D], k/v [B,S,Hkv,D] given as row pitches (elements)
// inside packed buffers; D must be 128. lse: fp32 [B,H,S].
int kb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S,
                 int H, int Hkv, int D, long q_pitch, long k_pitch, long v_pitch, long o_pitch,
                 float scale, int causal, void* stream);
// The same with T >= S keys per sequence (k / v are [B,T,Hkv,D]): the queries are the last S positions.
int kb_flash_fwd_rect(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int T,
                      int H, int Hkv, int D, long q_pitch, long k_pitch, long v_pitch, long o_pitch,
                      float scale, int causal, void* stream);
int kb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                 const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int H,
                 int Hkv, int D, long q_pitch, long k_pitch, long v_pitch, long o_pitch,
                 long do_pitch, long dq_pitch, long dk_pitch, long dv_pitch, float scale,
                 int causal, void* stream);

// ---- more GEMMs ---------------------------------------------------------------------------
// CTA-pair variant (cta_group::2, 256 x bn output per pair of SMs, bn in {256, 192, 128} chosen
// per problem, K-sliced tail wave); same contract as kb_gemm_bf16.  The _bn form takes an
// explicit tile width (0: automatic; 192 needs a K-major B).
int kb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                      long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi, void* stream);
int kb_gemm_bf16_pair_bn(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                         long lda, long ldb, long ldc, long ldr, int a_mn, int b_mn, int epi, int bn,
                         void* stream);
// Gate/up projection with the SwiGLU in the epilogue: W is [2F, K] (gate rows, then up rows);
// writes GU[M, 2F] = X W^T and H[M, F] = up * silu(gate).  bn as above.
int kb_gemm_swiglu_bf16(const void* X, const void* W, void* GU, void* H, int M, int F, int K, long ldx,
                        long ldw, long ldgu, long ldh, int bn, void* stream);
// int8 weight-only: C[M,N] = A[M,K] (bf16) * dequant(Wq[N,K] int8, scale[N] fp32)^T.
int kb_gemm_w8(const void* A, const void* Wq, const float* scale, void* C, int M, int N, int K,
               long lda, long ldw, long ldc, void* stream);
int kb_quant_w8(const void* W, void* Wq, float* scale, int N, int K, void* stream);
// Block-scaled fp8 (e4m3): activations with one fp32 scale per 1 x 128 block, weights per 128 x 128.
int kb_quant_fp8_1x128(const void* x, void* q, void* scale, int M, int K, long ldx, void* stream);
int kb_quant_fp8_128x128(const void* w, void* q, void* scale, int N, int K, long ldw, void* stream);
int kb_gemm_fp8(const void* A8, const void* B8, const void* sa, const void* sb, void* C, int M, int N,
                int K, long lda, long ldb, long ldc, void* stream);

// ---- inference ----------------------------------------------------------------------------
// RoPE + optional q/k RMSNorm (after the rotation) in place on packed [q | k | v] rows, and the K/V
// rows stored to their page slots, in one kernel (head_dim 64, 128 or 256).
int kb_rope_norm_kvwrite(void* qkv, const float* cs, const int* pos, const void* q_w, const void* k_w, float eps,
                         const long long* slots, void* k_pool, void* v_pool, int tokens, int seq_len, int H, int Hkv,
                         int head_dim, long row_stride, void* stream);
int kb_paged_kv_write(const void* k, const void* v, void* k_pool, void* v_pool, const void* slots,
                      int tokens, int row_elems, long k_pitch, long v_pitch, void* stream);
// CUDA-core split-KV decode attention (any page size, group size <= 8) and its tcgen05 counterpart
// (page size 16/32/64/128, group size <= 32; needs the pool's page count for its tensor maps).
int kb_paged_decode_attn(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                         const int* seq_lens, float* part_acc, float* part_ml, void* out, int B, int H,
                         int Hkv, int D, int page_size, int max_pages, int n_splits, long q_pitch,
                         long out_pitch, float scale, void* stream);
int kb_paged_decode_tc(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                       const int* seq_lens, float* part_acc, float* part_ml, void* out, int B, int H,
                       int Hkv, int D, int page_size, int max_pages, int n_pool_pages, int n_splits,
                       long q_pitch, long out_pitch, float scale, void* stream);
int kb_decode_merge(const float* part_acc, const float* part_ml, void* out, int B, int H, int n_splits,
                    long out_pitch, void* stream);
int kb_sample(const void* logits, const void* temperature, const void* top_k, const void* top_p,
              const void* uniform, void* out, int rows, int V, long ld, long long reserved, void* stream);

// ---- collectives over NVLink peer memory (pointer arrays hold one address per rank) ----------
int kb_comm_slots(void);
int kb_peer_barrier(const void* const* ctrl_ptrs, int rank, int ws, int slot, unsigned int epoch,
                    int budget_ms, void* stream);
int kb_allreduce_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, void* mc_ptr, int rank,
                      int ws, long long n, float scale, unsigned int epoch, void* stream);
// Stand-alone reduce-scatter (into local `out`), all-gather (in place) and broadcast (from `root`) of
// symmetric bf16 buffers; each uses two epochs.
int kb_reducescatter_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, const void* mc_ptr, int rank,
                          int ws, long long n, float scale, void* out, unsigned int epoch, void* stream);
int kb_allgather_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, void* mc_ptr, int rank, int ws,
                      long long n, unsigned int epoch, void* stream);
int kb_broadcast_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, void* mc_ptr, int root, int rank,
                      int ws, long long n, unsigned int epoch, void* stream);
// Block-granular full sharding: reduce-scatter of the ranks' symmetric gradient images into local pieces
// (acc += scale * sum; with `clear` the rank's image is zeroed afterwards) on `grid` CTAs of `threads` threads
// (<= 0: one CTA per SM / 512; the same on every rank).
int kb_unit_reduce_bf16(const void* const* buf_ptrs, const void* const* ctrl_ptrs, const void* mc_ptr, int rank, int ws,
                        long long n, float scale, void* acc, int clear, unsigned int epoch, int grid, int threads,
                        void* stream);
// Data-parallel optimizer step over symmetric flat buffers: gradient reduce-scatter (mean) + global
// clip + sharded AdamW + parameter all-gather.  kb_reduce_adamw does it in one call; the bucket pair
// lets the reductions run bucket by bucket while the backward pass is still producing gradients
// (argument meaning at the definitions in comm.cu).
int kb_reduce_adamw(const void* const* grad_ptrs, const void* const* param_ptrs, const void* const* ctrl_ptrs,
                    const void* const* norm_ptrs, const void* grad_mc, void* param_mc, int rank, int ws,
                    long long slice_off, long long slice_n, float* m, float* v, const float* lr_step, float beta1,
                    float beta2, float eps, float weight_decay, float max_norm, float* scratch, unsigned int epoch,
                    void* stream);
int kb_reduce_bucket(const void* const* grad_ptrs, const void* const* ctrl_ptrs, const void* grad_mc, int rank, int ws,
                     long long bucket_n, long long total_n, int b_lo, int b_hi, float* norm_sq_local,
                     unsigned int epoch, int grid, int threads, void* stream);
int kb_adamw_buckets(const void* const* grad_ptrs, const void* const* param_ptrs, const void* const* ctrl_ptrs,
                     const void* const* norm_ptrs, void* param_mc, int rank, int ws, long long bucket_n,
                     long long total_n, float* m, float* v, const float* lr_step, float beta1, float beta2, float eps,
                     float weight_decay, float max_norm, float* scratch, unsigned int epoch, void* stream);
// GEMM fused with all-gather of an operand and / or reduce-scatter / all-reduce of the result;
// the argument list is documented at the definition in gemm_comm.cu.
int kb_gemm_comm(const void* const* a_ptrs, const void* const* b_ptrs, void* c_local,
                 const void* const* stage_ptrs, const void* const* ctrl_ptrs, void* out, int M, int N, int K,
                 long lda, long ldb, long ldc, long ldo, int a_mn, int b_mn, int a_gather, int b_gather,
                 int c_mode, int rank, int ws, unsigned int epoch, unsigned int* grid_sync, int gather_copy,
                 unsigned int* ready, unsigned int ready_target, unsigned long long* trace, int exit_barrier, unsigned int* epoch_dev, unsigned int* calls_dev,
                 void* stream);

#ifdef __cplusplus
}
#endif
