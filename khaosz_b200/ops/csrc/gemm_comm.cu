// GEMMs fused with their collective over NVLink peer memory (tensor-parallel layers and
// sharded-weight data parallelism).  One persistent tcgen05 kernel, three fusions:
//
//   all-gather -> GEMM    an operand whose rows are sharded over the ranks (sequence-sharded
//                         activations for column-parallel layers, or row-sharded weights under
//                         FSDP).  Copy mode: a copier warp in every CTA pulls the peers' shards
//                         once over NVLink (plain cp.async.bulk peer -> shared -> local memory,
//                         no multicast) into the local image of the whole operand and publishes
//                         128-row chunks through release counters; the TMA producer starts with
//                         the tiles of the local shard and polls a chunk's counter (bounded)
//                         before its first load from it, so the transfer hides behind the math.
//                         Direct mode (shards that are not whole 128-row chunks): the producer
//                         reads every tile straight from the owning rank's memory.
//   GEMM -> reduce-scatter  each finished output tile is TMA-stored into the owner rank's staging
//                         slot for this source rank while the next tile is being computed;
//                         after a grid-wide + cross-rank barrier every rank sums the slots of
//                         the rows it owns (fixed order: deterministic).
//   GEMM -> all-reduce    same, but the tile goes to every rank's staging buffer and every rank
//                         sums all rows (decode-time row-parallel layers).
//
// Operands may be K-major or MN-major exactly as in gemm_bf16.cu; for an MN-major gathered
// operand the sharded dimension is the reduction dimension and the source rank changes per
// k-block instead of per tile.  All waits (mbarriers, peer flags, the grid barrier) are bounded.
#include "comm.cuh"
#include "kb_api.h"

namespace kb {
namespace gcomm {

using comm::MAX_RANKS;
using comm::Peers;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int COPY_PIECE = 16 * 1024;   // bytes per bulk copy of the gather copier
constexpr int COPY_BUFS = 3;
constexpr int CHUNK_ROWS = 128;          // rows of the gathered operand published per counter
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int ATOM_BYTES = BK * 128;
constexpr int EPI_COLS = 64;
constexpr int EPI_BUF_BYTES = BM * EPI_COLS * 2;
constexpr int NUM_EPI_BUFS = 2;
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 224;  // TMA warp, MMA warp, 4 epilogue warps, gather copier warp
constexpr int COPY_WARP = 6;
template <int STAGES, bool COPY>
constexpr int smem_bytes() {
  return STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + NUM_EPI_BUFS * EPI_BUF_BYTES + (COPY ? COPY_BUFS * COPY_PIECE : 0) +
         256 + 1024;
}

struct Maps {
  CUtensorMap m[MAX_RANKS];
};

struct Params {
  int M, N, K;        // full problem seen by this rank
  int a_mn, b_mn;
  int a_gather;       // rows of the stored A are sharded: a_rows rows per rank
  int b_gather;
  int a_rows, b_rows;
  int c_mode;         // 0 local store, 1 reduce-scatter, 2 all-reduce
  int c_rows;         // output rows owned per rank (c_mode 1) or M (c_mode 2)
  int c_slot_rows;    // rows between two source ranks' slots in a staging buffer (multiple of 128)
  int rank, ws;
  uint32_t epoch;
  Peers ctrl;
  const __nv_bfloat16* stage;  // this rank's staging buffer [ws, c_rows, N]
  __nv_bfloat16* out;          // reduced output [c_rows, N] (c_mode != 0)
  long ldo;
  unsigned int* grid_sync;     // two words, zero before the first launch
  int* err;
  // copy-mode gather: peers' images of the whole operand (shard r valid at rows of rank r)
  Peers gsrc;
  uint8_t* gdst;               // this rank's image
  unsigned int* ready;         // one counter per 128-row chunk of the image
  unsigned int ready_target;   // value a complete chunk's counter reaches in this call
  long long shard_bytes;       // bytes per rank's shard (whole chunks)
  int chunk_bytes;             // 128 rows
  int gather_rows;             // stored rows per rank of the gathered operand
  unsigned long long* trace;   // optional: 6 globaltimer stamps of CTA 0 (phase boundaries)
  const unsigned int* epoch_dev;  // optional: the epoch lives in device memory (CUDA-graph replays)
  const unsigned int* calls_dev;  // optional: copy-mode call counter of the image, same purpose
  int exit_barrier;            // 0: (c_mode 0 only) peers' reads of this rank's operand are fenced by the caller's buffer rotation
};

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void red_release_gpu_add(unsigned int* addr, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* addr) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Bounded wait until the chunks covering stored rows [row0, row0 + nrows) of the gathered image
// have arrived.  `last` caches the newest chunk already seen complete.
__device__ __forceinline__ bool wait_gathered(const Params& p, uint32_t ready_target, int row0, int nrows, int& last,
                                              volatile int* abort_flag) {
  const int c0 = row0 / CHUNK_ROWS, c1 = (row0 + nrows - 1) / CHUNK_ROWS;
  bool fresh = false;
  for (int c = c0; c <= c1; ++c) {
    if (c == last || (c * CHUNK_ROWS) / p.gather_rows == p.rank) continue;
    const unsigned long long t0 = globaltimer_ns();
    unsigned int it = 0;
    while (ld_acquire_gpu(p.ready + c) != ready_target) {
      if ((++it & 63u) == 0u && (*abort_flag || globaltimer_ns() - t0 > KB_WAIT_BUDGET_NS)) {
        *abort_flag = 1;
        atomicCAS(p.err, 0, KB_ERR_TIMEOUT_PEER);
        return false;
      }
    }
    last = c;
    fresh = true;
  }
  if (fresh) fence_proxy_async_all();  // the chunk was written through the async proxy of other SMs
  return true;
}

// Map index + coordinate inside that rank's shard for a stored row index.
__device__ __forceinline__ void locate(int row, int rows_per_rank, int gather, int& which, int& local_row) {
  if (gather) {
    which = row / rows_per_rank;
    local_row = row - which * rows_per_rank;
  } else {
    which = 0;
    local_row = row;
  }
}

template <int STAGES, bool COPY>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_comm_kernel(const __grid_constant__ Maps maps_a, const __grid_constant__ Maps maps_b,
                 const __grid_constant__ Maps maps_c, const Params p_in) {
  // With device-side counters the launch arguments stay constant, so a captured graph can be
  // replayed: a one-thread kernel launched behind this one advances the counters.
  const Params& p = p_in;
  const uint32_t epoch = p.epoch_dev ? *p.epoch_dev : p.epoch;
  const uint32_t ready_target =
      p.calls_dev ? (*p.calls_dev + 1u) * (uint32_t)((p.chunk_bytes + COPY_PIECE - 1) / COPY_PIECE) : p.ready_target;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* sEpi = sB + STAGES * B_STAGE_BYTES;
  uint8_t* sCopy = sEpi + NUM_EPI_BUFS * EPI_BUF_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sCopy + (COPY ? COPY_BUFS * COPY_PIECE : 0));
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint64_t* cbar = bars + 2 * STAGES + 4;  // [COPY_BUFS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + COPY_BUFS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN, num_k = (p.K + BK - 1) / BK;
  const int total = num_m * num_n;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
    for (int i = 0; i < COPY_BUFS; ++i) mbar_init(&cbar[i], 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Every rank's inputs are complete (and its staging buffer free) before anyone reads or writes
  // peer memory.
  const bool tracer = p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
  if (tracer) p.trace[0] = globaltimer_ns();   // kernel entered
  bool peers_ok = true;
  if (p.ws > 1) peers_ok = comm::cta_peer_barrier(p.ctrl, p.rank, p.ws, blockIdx.x, epoch, p.err, KB_WAIT_BUDGET_NS);
  if (tracer) p.trace[1] = globaltimer_ns();   // every rank has entered

  // Tile order: rotate the m-tiles (K-major gathered A) so that this rank starts with its own
  // shard and the ranks walk the ring in step, spreading the load over the links.
  // With a gathered K-major A the n-blocks of one m-block are consecutive, so that every tile of
  // the local shard comes before the first tile that needs a peer's rows; a gathered K-major B
  // rotates the n-blocks the same way; an MN-major gathered operand rotates the k-blocks.
  const bool a_rows_gathered = p.a_gather && !p.a_mn, b_rows_gathered = p.b_gather && !p.b_mn;
  const int m_rot = a_rows_gathered ? (p.rank * p.a_rows) / BM : 0;
  const int n_rot = b_rows_gathered ? (p.rank * p.b_rows) / BN : 0;
  const int k_rot = (p.a_gather && p.a_mn) ? (p.rank * p.a_rows) / BK : ((p.b_gather && p.b_mn) ? (p.rank * p.b_rows) / BK : 0);
  auto tile_of = [&](int t, int& m_blk, int& n_blk) {
    if (a_rows_gathered) {
      m_blk = (t / num_n + m_rot) % num_m;
      n_blk = t % num_n;
    } else {
      m_blk = t % num_m;
      n_blk = (t / num_m + n_rot) % num_n;
    }
  };

  if (warp == 0) {
    if (lane == 0 && peers_ok) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      int seen = -1;  // newest gathered chunk known to be complete
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_of(t, m_blk, n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        if (COPY) {
          if (a_rows_gathered) ok = wait_gathered(p, ready_target, m0, min(BM, p.M - m0), seen, abort_flag);
          else if (b_rows_gathered) ok = wait_gathered(p, ready_target, n0, min(BN, p.N - n0), seen, abort_flag);
          if (!ok) break;
        }
        for (int kk = 0; kk < num_k; ++kk) {
          const int kb = (kk + k_rot) % num_k;
          const int k0 = kb * BK;
          if (COPY && ((p.a_gather && p.a_mn) || (p.b_gather && p.b_mn))) {
            if (!wait_gathered(p, ready_target, k0, min(BK, p.K - k0), seen, abort_flag)) { ok = false; break; }
          }
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          int which, lr;
          const int a_split = COPY ? 0 : p.a_gather, b_split = COPY ? 0 : p.b_gather;  // copy mode reads the local image
          if (!p.a_mn) {
            locate(m0, p.a_rows, a_split, which, lr);
            tma_load_2d(a_dst, &maps_a.m[which], &full[s], k0, lr);
          } else {
            locate(k0, p.a_rows, a_split, which, lr);
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d(a_dst + a * ATOM_BYTES, &maps_a.m[which], &full[s], m0 + a * 64, lr);
          }
          if (!p.b_mn) {
            locate(n0, p.b_rows, b_split, which, lr);
            tma_load_2d(b_dst, &maps_b.m[which], &full[s], k0, lr);
          } else {
            locate(k0, p.b_rows, b_split, which, lr);
#pragma unroll
            for (int a = 0; a < BN / 64; ++a) tma_load_2d(b_dst + a * ATOM_BYTES, &maps_b.m[which], &full[s], n0 + a * 64, lr);
          }
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && peers_ok) {
      const uint32_t idesc = umma_idesc(BM, BN, p.a_mn != 0, p.b_mn != 0);
      int s = 0; uint32_t ph = 0; int acc = 0; uint32_t aph = 0; bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        if (!mbar_wait(&tempty[acc], aph ^ 1u, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.err, KB_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES), b_addr = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t a_desc = p.a_mn ? umma_desc_mnmajor(a_addr, j * UMMA_K, ATOM_BYTES) : umma_desc_kmajor(a_addr, j * 32);
            const uint64_t b_desc = p.b_mn ? umma_desc_mnmajor(b_addr, j * UMMA_K, ATOM_BYTES) : umma_desc_kmajor(b_addr, j * 32);
            umma_f16(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);  // kb counts stages, in any k order
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) { acc = 0; aph ^= 1u; }
      }
    }
  } else if (warp == COPY_WARP) {
    // ------------------------------- gather copier -------------------------------
    // Piece g of the peers' shards (ring order from rank + 1, ascending addresses) belongs to CTA
    // g % gridDim.x: every chunk is assembled by many SMs at once and the early chunks finish first.
    if (COPY && lane == 0 && peers_ok && p.ws > 1) {
      const int ppc = (p.chunk_bytes + COPY_PIECE - 1) / COPY_PIECE;       // pieces per chunk
      const long long cps = p.shard_bytes / p.chunk_bytes;                   // chunks per shard
      const long long n_pieces = (long long)(p.ws - 1) * cps * ppc;
      auto piece = [&](long long g, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes, int& chunk) {
        const long long ch = g / ppc;
        const int pc = (int)(g - ch * ppc);
        const int peer = (p.rank + 1 + (int)(ch / cps)) % p.ws;
        const long long off = (long long)peer * p.shard_bytes + (ch % cps) * p.chunk_bytes + (long long)pc * COPY_PIECE;
        src = static_cast<const uint8_t*>(p.gsrc.p[peer]) + off;
        dst = p.gdst + off;
        bytes = (uint32_t)min((long long)COPY_PIECE, (long long)p.chunk_bytes - (long long)pc * COPY_PIECE);
        chunk = (int)(((long long)peer * p.shard_bytes + (ch % cps) * p.chunk_bytes) / p.chunk_bytes);
      };
      const long long first = blockIdx.x, stride = gridDim.x;
      const long long mine = first < n_pieces ? (n_pieces - first + stride - 1) / stride : 0;
      bool ok = true;
      for (long long i = 0; i < mine + (COPY_BUFS - 1) && ok; ++i) {
        if (i < mine) {  // issue the load of my piece i
          const uint8_t* src; uint8_t* dst; uint32_t bytes; int chunk;
          piece(first + i * stride, src, dst, bytes, chunk);
          const int b = (int)(i % COPY_BUFS);
          mbar_expect_tx(&cbar[b], bytes);
          bulk_load(sCopy + b * COPY_PIECE, src, bytes, &cbar[b]);
        }
        const long long j = i - (COPY_BUFS - 1);
        if (j >= 0) {    // forward my piece j to local memory and publish it
          const uint8_t* src; uint8_t* dst; uint32_t bytes; int chunk;
          piece(first + j * stride, src, dst, bytes, chunk);
          const int b = (int)(j % COPY_BUFS);
          if (!mbar_wait(&cbar[b], (uint32_t)((j / COPY_BUFS) & 1), abort_flag, p.err, KB_ERR_TIMEOUT_PEER)) { ok = false; break; }
          bulk_store(dst, sCopy + b * COPY_PIECE, bytes);
          tma_store_commit();
          tma_store_wait_all<0>();   // the piece is in local memory (and its buffer is free again)
          fence_proxy_async_all();
          red_release_gpu_add(p.ready + chunk, 1u);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    int acc = 0; uint32_t aph = 0; int buf = 0; bool ok = peers_ok;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      int m_blk, n_blk;
      tile_of(t, m_blk, n_blk);
      const int m0 = m_blk * BM, n0 = n_blk * BN;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, p.err, KB_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      // destination(s) of this tile
      int owner = 0, dst_row = m0;
      if (p.c_mode == 1) {
        owner = m0 / p.c_rows;
        dst_row = p.rank * p.c_slot_rows + (m0 - owner * p.c_rows);
      } else if (p.c_mode == 2) {
        dst_row = p.rank * p.c_slot_rows + m0;
      }
#pragma unroll 1
      for (int c = 0; c < BN / EPI_COLS; ++c) {
        const int col0 = n0 + c * EPI_COLS;
        if (col0 >= p.N) break;
        uint32_t v[EPI_COLS];
        tmem_ld_32x32b_x32(t_row + c * EPI_COLS, v);
        tmem_ld_32x32b_x32(t_row + c * EPI_COLS + 32, v + 32);
        tmem_ld_wait();
        if (epi_tid == 0) tma_store_wait_read<NUM_EPI_BUFS - 1>();
        named_barrier_sync(1, 128);
        uint8_t* stage = sEpi + buf * EPI_BUF_BYTES;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(v[ch * 8 + 0]), __uint_as_float(v[ch * 8 + 1]));
          o.y = pack_bf16x2(__uint_as_float(v[ch * 8 + 2]), __uint_as_float(v[ch * 8 + 3]));
          o.z = pack_bf16x2(__uint_as_float(v[ch * 8 + 4]), __uint_as_float(v[ch * 8 + 5]));
          o.w = pack_bf16x2(__uint_as_float(v[ch * 8 + 6]), __uint_as_float(v[ch * 8 + 7]));
          *reinterpret_cast<uint4*>(stage + sw128_offset(row_in_tile, ch)) = o;
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (epi_tid == 0) {
          if (p.c_mode == 2) {
            for (int r = 0; r < p.ws; ++r) tma_store_2d(&maps_c.m[(p.rank + r) % p.ws], stage, col0, dst_row);
          } else {
            tma_store_2d(&maps_c.m[owner], stage, col0, dst_row);
          }
          tma_store_commit();
        }
        buf ^= 1;
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

  if (tracer) p.trace[2] = globaltimer_ns();     // this CTA's tiles (and copies) done
  // ---------------- phase 2: cross-rank completion, then the reduction of the staged tiles ----------------
  if (p.ws > 1 && (p.c_mode != 0 || p.exit_barrier)) {
    // grid-wide arrival on this rank (all CTAs are resident: grid <= SM count, one CTA per SM)
    __shared__ int s_go;
    if (threadIdx.x == 0) {
      __threadfence_system();  // this CTA's peer stores are ordered before its arrival
      s_go = 1;
      const unsigned int gen = epoch;  // generation tag of this launch
      const unsigned int arrived = atomicAdd(&p.grid_sync[0], 1u) + 1u;
      if (arrived == gridDim.x) {
        atomicExch(&p.grid_sync[0], 0u);  // last arriver re-arms the counter for the next launch
        __threadfence();
        atomicExch(&p.grid_sync[1], gen);
      } else {
        const unsigned long long t0 = globaltimer_ns();
        while (atomicAdd(&p.grid_sync[1], 0u) != gen) {
          if (globaltimer_ns() - t0 > KB_WAIT_BUDGET_NS) { s_go = 0; atomicCAS(p.err, 0, KB_ERR_TIMEOUT_MISC); break; }
        }
      }
    }
    __syncthreads();
    if (tracer) p.trace[3] = globaltimer_ns();   // all CTAs of this rank done
    const bool go = s_go != 0;
    // every CTA of every rank has issued (and completed) its stores
    const bool all_ok = go && comm::cta_peer_barrier(p.ctrl, p.rank, p.ws, blockIdx.x, epoch + 1, p.err, KB_WAIT_BUDGET_NS);
    if (tracer) p.trace[4] = globaltimer_ns();   // all ranks done
    if (p.c_mode != 0 && all_ok && peers_ok) {
      const int rows = p.c_rows;
      const int cpr = p.N >> 3;
      const long total_chunks = (long)rows * cpr;
      const long stride = (long)gridDim.x * NUM_THREADS;
      // The CTA has few threads for a streaming pass, so each thread keeps 16 independent 16-byte
      // loads in flight (8 chunks x 2 slots) to cover the memory latency.
      constexpr int UNROLL = 8;
      for (long i0 = blockIdx.x * (long)NUM_THREADS + threadIdx.x; i0 < total_chunks; i0 += stride * UNROLL) {
        float acc8[UNROLL][8];
        size_t off[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
          for (int k = 0; k < 8; ++k) acc8[u][k] = 0.f;
          const long i = min(i0 + u * stride, total_chunks - 1);  // clamped: the tail re-reads a valid chunk
          const long r = i / cpr;
          off[u] = (size_t)r * p.N + (size_t)(i - r * cpr) * 8;
        }
        for (int s = 0; s < p.ws; s += 2) {
          const bool two = s + 1 < p.ws;
          const __nv_bfloat16* b0 = p.stage + (size_t)s * p.c_slot_rows * p.N;
          const __nv_bfloat16* b1 = p.stage + (size_t)(two ? s + 1 : s) * p.c_slot_rows * p.N;
          uint4 v0[UNROLL], v1[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            v0[u] = *reinterpret_cast<const uint4*>(b0 + off[u]);
            v1[u] = *reinterpret_cast<const uint4*>(b1 + off[u]);
          }
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const uint32_t w0[4] = {v0[u].x, v0[u].y, v0[u].z, v0[u].w};
            const uint32_t w1[4] = {v1[u].x, v1[u].y, v1[u].z, v1[u].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 f = unpack_bf16x2(w0[k]);
              acc8[u][2 * k] += f.x; acc8[u][2 * k + 1] += f.y;
              if (two) {
                const float2 g = unpack_bf16x2(w1[k]);
                acc8[u][2 * k] += g.x; acc8[u][2 * k + 1] += g.y;
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long i = i0 + u * stride;
          if (i < total_chunks) {
            const long r = i / cpr;
            const int c = (int)(i - r * cpr);
            uint4 o;
            o.x = pack_bf16x2(acc8[u][0], acc8[u][1]); o.y = pack_bf16x2(acc8[u][2], acc8[u][3]);
            o.z = pack_bf16x2(acc8[u][4], acc8[u][5]); o.w = pack_bf16x2(acc8[u][6], acc8[u][7]);
            *reinterpret_cast<uint4*>(p.out + r * p.ldo + c * 8) = o;
          }
        }
      }
    }
  }
  if (tracer) p.trace[5] = globaltimer_ns();     // reduction of the staged tiles done
}

// Advances the device-side epoch / call counters behind a fused kernel (stream ordered).
__global__ void bump_counters_kernel(unsigned int* epoch_dev, unsigned int epoch_step, unsigned int* calls_dev) {
  if (epoch_dev) *epoch_dev += epoch_step;
  if (calls_dev) *calls_dev += 1u;
}

}  // namespace gcomm
}  // namespace kb

extern "C" {

// a_ptrs / b_ptrs / stage_ptrs / ctrl_ptrs: host arrays of `ws` device pointers (peer addresses of
// symmetric buffers); for a non-gathered operand only entry [rank] is used.
//   a_gather: stored A rows are sharded, a_rows per rank (K-major: M = ws * a_rows; MN-major: K = ws * a_rows)
//   c_mode 0: C_local [M, N] written to c_local (pitch ldc)
//   c_mode 1: reduce-scatter: out [M / ws, N] on each rank; staging buffers [ws, M / ws, N]
//   c_mode 2: all-reduce:     out [M, N] on every rank;     staging buffers [ws, roundup(M, 128), N]
// epoch must grow by at least 2 per call; grid_sync: 2 uints, zero-initialised once.
// gather_copy = 1 (copy mode): the gathered operand's pointers are every rank's image of the WHOLE
// operand (contiguous rows, pitch = stored columns; rank r's shard already in place at its rows of
// image r), `ready` is one zero-initialised counter per 128-row chunk of this rank's image and
// `ready_target` = (number of copy-mode calls on this image, this one included) x ceil(128 rows in
// bytes / 16 KiB).  Shards must be whole 128-row chunks.
// epoch_dev / calls_dev (optional, device words): when given, the kernel takes its epoch from
// *epoch_dev (and ready_target from *calls_dev) instead of the arguments and a one-thread kernel
// advances them afterwards (epoch by 4), so the launch can be captured into a CUDA graph and
// replayed; *epoch_dev must start at the same value >= 1 on every rank.
// exit_barrier = 0 (allowed with c_mode 0): the kernel returns without waiting for the peers to
// finish reading this rank's operand; the caller must then not overwrite that operand before the
// NEXT fused kernel of the group has started on every rank (e.g. by alternating two buffers).
int kb_gemm_comm(const void* const* a_ptrs, const void* const* b_ptrs, void* c_local, const void* const* stage_ptrs,
                 const void* const* ctrl_ptrs, void* out, int M, int N, int K, long lda, long ldb, long ldc, long ldo,
                 int a_mn, int b_mn, int a_gather, int b_gather, int c_mode, int rank, int ws, unsigned int epoch,
                 unsigned int* grid_sync, int gather_copy, unsigned int* ready, unsigned int ready_target,
                 unsigned long long* trace, int exit_barrier, unsigned int* epoch_dev, unsigned int* calls_dev,
                 void* stream) {
  using namespace kb::gcomm;
  if (M <= 0 || N <= 0 || K <= 0 || ws < 1 || ws > MAX_RANKS || rank < 0 || rank >= ws) return KB_STATUS_BAD_ARG;
  if ((lda & 7) || (ldb & 7) || (N & 7)) return KB_STATUS_BAD_ARG;
  const bool copy = gather_copy && ws > 1 && (a_gather || b_gather);
  if (copy && ((a_gather && b_gather) || !ready)) return KB_STATUS_BAD_ARG;
  static bool attr_set_dev[64] = {false};  // the attribute is per device
  int attr_dev = 0;
  cudaGetDevice(&attr_dev);
  bool& attr_set = attr_set_dev[attr_dev & 63];
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_comm_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem_bytes<4, false>()) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_comm_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem_bytes<3, true>()) != cudaSuccess)
      return KB_STATUS_CUDA_ERROR;
    attr_set = true;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  static int sms = 0;
  if (sms == 0) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);

  Params p = {};
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.a_gather = a_gather; p.b_gather = b_gather;
  p.c_mode = c_mode; p.rank = rank; p.ws = ws; p.epoch = epoch; p.err = kb::error_word(dev);
  p.grid_sync = grid_sync; p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.trace = trace;
  p.exit_barrier = exit_barrier;
  p.epoch_dev = epoch_dev;
  p.calls_dev = copy ? calls_dev : nullptr;
  for (int i = 0; i < MAX_RANKS; ++i) p.ctrl.p[i] = (ctrl_ptrs && i < ws) ? const_cast<void*>(ctrl_ptrs[i]) : nullptr;

  // stored-row extents of the operands
  const int a_stored_rows = a_mn ? K : M, a_stored_cols = a_mn ? M : K;
  const int b_stored_rows = b_mn ? K : N, b_stored_cols = b_mn ? N : K;
  p.a_rows = a_gather ? a_stored_rows / ws : a_stored_rows;
  p.b_rows = b_gather ? b_stored_rows / ws : b_stored_rows;
  // direct mode: a tile (or k-block) must not straddle two ranks' shards; copy mode reads one contiguous image
  if (a_gather && (a_stored_rows % ws || (!copy && p.a_rows % (a_mn ? BK : BM)))) return KB_STATUS_BAD_ARG;
  if (b_gather && (b_stored_rows % ws || (!copy && p.b_rows % (b_mn ? BK : BN)))) return KB_STATUS_BAD_ARG;
  if (copy) {
    const long ld = a_gather ? lda : ldb;
    const int cols = a_gather ? a_stored_cols : b_stored_cols;
    p.gather_rows = a_gather ? p.a_rows : p.b_rows;
    if (ld != cols || p.gather_rows % CHUNK_ROWS) return KB_STATUS_BAD_ARG;  // contiguous image, whole chunks
    p.chunk_bytes = CHUNK_ROWS * cols * 2;
    p.shard_bytes = (long long)p.gather_rows * cols * 2;
    const void* const* gp = a_gather ? a_ptrs : b_ptrs;
    for (int i = 0; i < MAX_RANKS; ++i) p.gsrc.p[i] = i < ws ? const_cast<void*>(gp[i]) : nullptr;
    p.gdst = static_cast<uint8_t*>(const_cast<void*>(gp[rank]));
    p.ready = ready;
    p.ready_target = ready_target;
  }
  p.c_rows = c_mode == 1 ? M / ws : M;
  p.c_slot_rows = (p.c_rows + BM - 1) / BM * BM;  // whole tiles per slot: a tile never spills into a neighbour
  if (c_mode == 1 && (M % ws || p.c_rows % BM)) return KB_STATUS_BAD_ARG;
  if (c_mode != 0 && (!stage_ptrs || !out || !grid_sync)) return KB_STATUS_BAD_ARG;
  p.stage = c_mode != 0 ? static_cast<const __nv_bfloat16*>(stage_ptrs[rank]) : nullptr;

  Maps ma, mb, mc;
  for (int i = 0; i < MAX_RANKS; ++i) {
    const int ia = a_gather ? (i < ws ? i : rank) : rank;
    const int ib = b_gather ? (i < ws ? i : rank) : rank;
    const void* ap = a_ptrs[a_gather ? ia : (ws > 0 ? rank : 0)];
    const void* bp = b_ptrs[b_gather ? ib : (ws > 0 ? rank : 0)];
    int rc;
    // copy mode: one map over the whole local image; direct mode: one map per rank's shard
    const void* apc = copy && a_gather ? a_ptrs[rank] : ap;
    const void* bpc = copy && b_gather ? b_ptrs[rank] : bp;
    const int a_map_rows = copy && a_gather ? a_stored_rows : p.a_rows;
    const int b_map_rows = copy && b_gather ? b_stored_rows : p.b_rows;
    if (!a_mn) rc = kb::make_tmap_2d(&ma.m[i], apc, 2, a_map_rows, a_stored_cols, lda * 2, BM, BK, true);
    else       rc = kb::make_tmap_2d(&ma.m[i], apc, 2, a_map_rows, a_stored_cols, lda * 2, BK, 64, true);
    if (rc) return KB_STATUS_TMAP_ERROR;
    if (!b_mn) rc = kb::make_tmap_2d(&mb.m[i], bpc, 2, b_map_rows, b_stored_cols, ldb * 2, BN, BK, true);
    else       rc = kb::make_tmap_2d(&mb.m[i], bpc, 2, b_map_rows, b_stored_cols, ldb * 2, BK, 64, true);
    if (rc) return KB_STATUS_TMAP_ERROR;
    if (c_mode == 0) {
      rc = kb::make_tmap_2d(&mc.m[i], c_local, 2, M, N, ldc * 2, BM, EPI_COLS, true);
    } else {
      const void* sp = stage_ptrs[i < ws ? i : rank];
      rc = kb::make_tmap_2d(&mc.m[i], sp, 2, (uint64_t)ws * p.c_slot_rows, N, (uint64_t)N * 2, BM, EPI_COLS, true);
    }
    if (rc) return KB_STATUS_TMAP_ERROR;
  }
  const int total = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = total < sms ? total : sms;
  if (c_mode != 0 && grid < 1) grid = 1;
  if (copy)
    gemm_comm_kernel<3, true><<<grid, NUM_THREADS, smem_bytes<3, true>(), static_cast<cudaStream_t>(stream)>>>(ma, mb, mc, p);
  else
    gemm_comm_kernel<4, false><<<grid, NUM_THREADS, smem_bytes<4, false>(), static_cast<cudaStream_t>(stream)>>>(ma, mb, mc, p);
  if (epoch_dev || p.calls_dev)
    bump_counters_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(epoch_dev, 4u, const_cast<unsigned int*>(p.calls_dev));
  return cudaGetLastError() == cudaSuccess ? KB_STATUS_OK : KB_STATUS_CUDA_ERROR;
}

}  // extern "C"
