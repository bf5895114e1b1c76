// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (one kernel each):
//
//   mode 1  all-gather -> GEMM   C[T, N] = gather_rows(x_shard)[T, K] * B^T        (column-parallel forward,
//                                                                                   row-parallel input gradient)
//   mode 2  GEMM -> reduce-scatter   out[T/t, N] = sum_ranks (A[T, K_local] * B)    (row-parallel forward,
//                                                                                   column-parallel input gradient)
//
// Both are the CTA-pair tcgen05 GEMM of gemm_tcgen05_2cta.cu (256x256 tiles, TMA-fed shared-memory ring,
// accumulators in TMEM) with the transfer woven in tile by tile:
//
// mode 1: a few CTAs of the same grid ("copy CTAs") pull the peers' shards out of their staging buffers with
//   untiled bulk copies (peer HBM -> shared memory ring -> this GPU's gathered A), 256 rows per flag; the GEMM
//   CTAs walk the M tiles starting with the local shard and their TMA producers wait (bounded) on the flag of
//   the rows they are about to load.  TMA only ever reads this GPU's own memory.
// mode 2: M tiles owned by other ranks are computed first; their epilogue stores the bf16 tile straight into a
//   per-source slot of the owner's receive buffer (peer stores) and bumps a counter in the owner's flag pad;
//   tiles of the local shard go to `out`.  After its last tile every GEMM CTA takes 8-row slabs of the local
//   shard, waits (bounded) for the counters of that row block from every peer and adds the received slots.
//
// Replaces NCCL all-gather / reduce-scatter followed or preceded by cuBLAS in the reference
// (hetu/graph/ops/Communication.cc:870-975 with hetu/graph/ops/Linear.cc).
#include "common.cuh"
#include "../runtime/signals.cuh"
#include "gemm_api.h"
#include <cuda.h>

namespace hsb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols);

namespace fused {

constexpr int BM = 128, BNH = 128, BN = 256, BK = 64, UMMA_K = 16, THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 6, ACC_STAGES = 2, TMEM_COLS = 512;
constexpr int EPI_WARP_STAGE = 32 * 256;        // mode 2: per epilogue warp, 32 rows x 128 bf16
constexpr int EPI_STAGE_BYTES = 4 * EPI_WARP_STAGE;
constexpr int RECV_BLOCK_BYTES = 2 * EPI_WARP_STAGE;   // one warp's 32 x 256 part of a tile in the receive buffer
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_STAGE_BYTES;
constexpr int CHUNK_ROWS = 256;             // rows per readiness flag / per reduce-scatter row block
constexpr int PIECE_BYTES = 32 * 1024;      // one bulk copy
constexpr int RING = 6;                     // pieces in flight per copy CTA
constexpr int MAX_RB = 128;                 // row blocks per rank the counter table can hold

struct Args {
  int mode, n, my_pos, rows_per_rank;
  uint32_t epoch;
  int n_comm_ctas;
  uint64_t timeout_ns;
  PeerPtrs pads;            // uint32 flag pads of the group members (peer-mapped)
  int ready_word;           // mode 1: pads[p][ready_word + q] = epoch once q staged its shard
  int count_word;           // mode 2: pads[owner][count_word + ((set * 16 + src) * MAX_RB + rb)]
  PeerPtrs src;             // mode 1: members' staged shards [rows_per_rank, K] bf16
  uint32_t* chunk_flags;    // mode 1: local [n * rows_per_rank / 256], epoch valued
  char* xg;                 // mode 1: local gathered A
  int64_t row_bytes;        // mode 1: K * 2
  PeerPtrs recv;            // mode 2: members' receive buffers: per source slot, 16 KB blocks indexed
                            // [row block][n tile][cta half][lane quarter], each block = 2 column halves of
                            // 32 rows x 256 B with 16-byte pieces XOR-swizzled by (row & 15)
  __nv_bfloat16* out;       // mode 2: local [rows_per_rank, N]
  int ld_out;
};

__device__ __forceinline__ void tile_of(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP = 8;
  const int width = GROUP * tiles_n;
  const int group_id = t / width;
  const int first_m = group_id * GROUP;
  const int gsz = min(tiles_m - first_m, GROUP);
  const int r = t - group_id * width;
  tm = first_m + (r % gsz);
  tn = r / gsz;
}

struct AbortCtl {
  volatile int* local;
  uint32_t peer_addr;
  __device__ __forceinline__ void raise() const { *local = 1; st_cluster_u32(peer_addr, 1u); }
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, const AbortCtl& ab) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++it) & 0xff) == 0) {
      if (*ab.local) return false;
      if (globaltimer_ns() - t0 > HSB_WAIT_LIMIT_NS) { ab.raise(); return false; }
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------------------
// copy CTA of mode 1: one thread streams its share of the peers' chunks through a shared-memory ring
// ------------------------------------------------------------------------------------------------
__device__ void copy_cta(const Args& a, uint8_t* smem, uint64_t* bars, int* status) {
  if (threadIdx.x != 0) return;
  const int ci = blockIdx.x;
  const int cpr = a.rows_per_rank / CHUNK_ROWS;
  uint32_t* my_pad = reinterpret_cast<uint32_t*>(a.pads.p[a.my_pos]);
  if (ci == 0) {
    // tell every peer that this rank's shard is staged (it was written by earlier work on this stream)
    __threadfence_system();
    for (int p = 0; p < a.n; ++p)
      if (p != a.my_pos) st_release_sys(reinterpret_cast<uint32_t*>(a.pads.p[p]) + a.ready_word + a.my_pos, a.epoch);
  }
  for (int s = 0; s < RING; ++s) mbar_init(&bars[s], 1);
  fence_mbar_init();
  volatile int dummy_abort = 0;
  const int64_t chunk_bytes = static_cast<int64_t>(CHUNK_ROWS) * a.row_bytes;
  const int pieces = static_cast<int>((chunk_bytes + PIECE_BYTES - 1) / PIECE_BYTES);
  uint32_t n_load = 0, n_done = 0;      // pieces issued / consumed over the whole kernel (ring positions)
  bool ok = true;
  for (int d = 1; d < a.n && ok; ++d) {
    const int p = (a.my_pos + d) % a.n;
    bool waited = false;
    for (int c = 0; c < cpr && ok; ++c) {
      const int gidx = (d - 1) * cpr + c;
      if (gidx % a.n_comm_ctas != ci) continue;
      if (!waited) {
        if (!wait_flag_sys(my_pad + a.ready_word + p, a.epoch, a.timeout_ns, status)) { ok = false; break; }
        waited = true;
      }
      const char* src = reinterpret_cast<const char*>(a.src.p[p]) + static_cast<int64_t>(c) * chunk_bytes;
      char* dst = a.xg + (static_cast<int64_t>(p) * a.rows_per_rank + static_cast<int64_t>(c) * CHUNK_ROWS) * a.row_bytes;
      int issued = 0;
      auto issue = [&](int piece) {
        const int slot = n_load % RING;
        const int64_t off = static_cast<int64_t>(piece) * PIECE_BYTES;
        const uint32_t bytes = static_cast<uint32_t>(chunk_bytes - off < PIECE_BYTES ? chunk_bytes - off : PIECE_BYTES);
        mbar_arrive_expect_tx(&bars[slot], bytes);
        bulk_load_g2s(smem + slot * PIECE_BYTES, src + off, bytes, &bars[slot]);
        ++n_load;
      };
      for (; issued < pieces && issued < RING; ++issued) issue(issued);
      for (int i = 0; i < pieces; ++i) {
        const int slot = n_done % RING;
        if (!mbar_wait(&bars[slot], (n_done / RING) & 1, &dummy_abort)) {
          atomicCAS(status, ST_OK, ST_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        const int64_t off = static_cast<int64_t>(i) * PIECE_BYTES;
        const uint32_t bytes = static_cast<uint32_t>(chunk_bytes - off < PIECE_BYTES ? chunk_bytes - off : PIECE_BYTES);
        bulk_store_s2g(dst + off, smem + slot * PIECE_BYTES, bytes);
        bulk_commit();
        ++n_done;
        if (issued < pieces) {
          bulk_wait_read_all();          // the slot's bytes have left shared memory: refill it
          issue(issued++);
        }
      }
      if (!ok) break;
      bulk_wait_all();                   // the chunk is in this GPU's memory
      fence_proxy_async_all();
      __threadfence();
      st_release_gpu(a.chunk_flags + p * cpr + c, a.epoch);
    }
  }
  bulk_wait_all();
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 __nv_bfloat16* __restrict__ Cout, int ldc, int M, int N, int K, const __grid_constant__ Args a,
                 int* __restrict__ status) {
  constexpr bool B_MN = MODE == 2;       // mode 1: weights [N, K] K-major; mode 2: weights [K, N] MN-major
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + ACC_STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  if (MODE == 1 && static_cast<int>(blockIdx.x) < a.n_comm_ctas) {
    copy_cta(a, smem, full_bar, status);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int n_comm = MODE == 1 ? a.n_comm_ctas : 0;
  const int gemm_cta = static_cast<int>(blockIdx.x) - n_comm;
  const int cluster_id = gemm_cta >> 1;
  const int num_clusters = (static_cast<int>(gridDim.x) - n_comm) >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;
  const int tiles_per_rank = a.rows_per_rank / (2 * BM);
  // mode 1 starts with the local shard, mode 2 ends with it
  const int rot = (MODE == 1 ? a.my_pos : (a.my_pos + 1) % a.n) * tiles_per_rank;
  uint32_t* my_pad = reinterpret_cast<uint32_t*>(a.pads.p[a.my_pos]);
  const int set = static_cast<int>(a.epoch % 3u);

  if (MODE == 2 && gemm_cta == 0) {
    // counters of the call after next start at zero (nobody can be two calls ahead of this rank)
    const int zs = static_cast<int>((a.epoch + 2u) % 3u);
    for (int i = threadIdx.x; i < 16 * MAX_RB; i += THREADS) my_pad[a.count_word + zs * 16 * MAX_RB + i] = 0u;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int q = 0; q < ACC_STAGES; ++q) { mbar_init(&tmem_full[q], 1); mbar_init(&tmem_empty[q], 8); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_holder, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const AbortCtl ab{abort_flag, mapa_u32(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1u)};

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      const int cpr = a.rows_per_rank / CHUNK_ROWS;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_of(t, tiles_m, tiles_n, tm, tn);
        tm = (tm + rot) % tiles_m;
        const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * BNH;
        if (MODE == 1) {
          const int owner = (tm * 2 * BM) / a.rows_per_rank;
          if (owner != a.my_pos) {
            const int c = (tm * 2 * BM - owner * a.rows_per_rank) / CHUNK_ROWS;
            if (!wait_flag_gpu(a.chunk_flags + owner * cpr + c, a.epoch, a.timeout_ns, status)) { ab.raise(); ok = false; break; }
            fence_proxy_async_all();
          }
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!wait_bar(&empty_bar[s], ph ^ 1, ab)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[s]), 0);
          if (leader) mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_2d_pair(sa, &tmA, bar, k0, m0);
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmB, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmB, bar, n0 + j * 64, k0);
          }
        }
      }
      if (!ok) atomicCAS(status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------
    if (leader && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, 0, B_MN ? 1 : 0);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++tile_iter) {
        const int acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!wait_bar(&tmem_empty[acc], acc_ph ^ 1, ab)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!wait_bar(&full_bar[s], ph, ab)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s], 3);
        }
        if (ok) umma_commit_pair(&tmem_full[acc], 3);
      }
      if (!ok) atomicCAS(status, ST_OK, ST_TIMEOUT_MMA);
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------------------
    const int quarter = warp & 3;
    const uint32_t empty_remote = mapa_u32(smem_u32(&tmem_empty[0]), 0);
    uint32_t tile_iter = 0;
    bool ok = true;
    bool pending = false;                 // mode 2: a remote tile part whose arrival is not yet counted
    uint32_t* pend_counter = nullptr;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++tile_iter) {
      int tm, tn;
      tile_of(t, tiles_m, tiles_n, tm, tn);
      tm = (tm + rot) % tiles_m;
      const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
      const int n0 = tn * BN;
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!wait_bar(&tmem_full[acc], acc_ph, ab)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      // destination of this thread's row
      __nv_bfloat16* crow_base;
      bool remote = false;
      int owner = a.my_pos, rb = 0;
      if (MODE == 2) {
        owner = (tm * 2 * BM) / a.rows_per_rank;
        const int local_row = row - owner * a.rows_per_rank;
        rb = (tm * 2 * BM - owner * a.rows_per_rank) / CHUNK_ROWS;
        if (owner == a.my_pos) {
          crow_base = a.out + static_cast<size_t>(local_row) * a.ld_out;
        } else {
          remote = true;
          const int slot = a.my_pos < owner ? a.my_pos : a.my_pos - 1;
          crow_base = reinterpret_cast<__nv_bfloat16*>(a.recv.p[owner]) +
                      (static_cast<size_t>(slot) * a.rows_per_rank + local_row) * N;
        }
      } else {
        crow_base = Cout + static_cast<size_t>(row) * ldc;
      }
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (MODE == 2) {
        uint8_t* stg = smem + STAGES * STAGE_BYTES + 256 + (warp - 2) * EPI_WARP_STAGE;
        if (pending) {
          // the previous remote tile's bulk stores have had a whole tile time to land: count it at its owner
          if (lane == 0) {
            bulk_wait_all();
            fence_proxy_async_all();
            __threadfence_system();
            red_add_release_sys(pend_counter, 1u);
          }
          pending = false;
        }
        if (remote) {
          // Remote tile part: stage 128 columns of the 32 rows in the receive-block layout and ship each half
          // to the owner with ONE 8 KB bulk copy (shared memory -> peer HBM).
          const int slot = a.my_pos < owner ? a.my_pos : a.my_pos - 1;
          const size_t slot_bytes = static_cast<size_t>(a.rows_per_rank / 32) * tiles_n * RECV_BLOCK_BYTES;
          char* blk = reinterpret_cast<char*>(a.recv.p[owner]) + slot * slot_bytes +
                      ((static_cast<size_t>(rb * tiles_n + tn) * 2 + rank) * 4 + quarter) * RECV_BLOCK_BYTES;
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            if (lane == 0) bulk_wait_read_all();          // the staging area has been read by the previous copy
            __syncwarp();
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(taddr0 + pass * 128 + cc * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[8 * k + 0]), __uint_as_float(r[8 * k + 1]));
                o.y = pack_bf16x2(__uint_as_float(r[8 * k + 2]), __uint_as_float(r[8 * k + 3]));
                o.z = pack_bf16x2(__uint_as_float(r[8 * k + 4]), __uint_as_float(r[8 * k + 5]));
                o.w = pack_bf16x2(__uint_as_float(r[8 * k + 6]), __uint_as_float(r[8 * k + 7]));
                const int j = cc * 4 + k;
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((j ^ (lane & 15)) << 4)) = o;
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              bulk_store_s2g(blk + pass * EPI_WARP_STAGE, stg, EPI_WARP_STAGE);
              bulk_commit();
            }
          }
          pending = true;
          pend_counter = reinterpret_cast<uint32_t*>(a.pads.p[owner]) + a.count_word +
                         (set * 16 + a.my_pos) * MAX_RB + rb;
        } else {
          // Local tile part: stage 64 columns, then eight lanes per row write 128-byte row segments into `out`.
          if (lane == 0) bulk_wait_read_all();
          __syncwarp();
          __nv_bfloat16* tile_row0 = crow_base - static_cast<size_t>(lane) * a.ld_out;      // row of lane 0
#pragma unroll 1
          for (int c = 0; c < BN; c += 64) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(taddr0 + c, r0);
            tmem_ld_32x32b_x32(taddr0 + c + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
              o.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
              o.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
              o.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
              uint4 q;
              q.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
              q.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
              q.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
              q.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
              *reinterpret_cast<uint4*>(stg + lane * 128 + (((j + 4) ^ (lane & 7)) << 4)) = q;
            }
            __syncwarp();
            const int j = lane & 7;
            const int col = n0 + c + j * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3);
              const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((j ^ (rr & 7)) << 4));
              if (col < N) *reinterpret_cast<uint4*>(tile_row0 + static_cast<size_t>(rr) * a.ld_out + col) = v;
            }
            __syncwarp();
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr0 + c, r);
        tmem_ld_wait();
        const int col = n0 + c;
        if (row < M && col < N) {
          __nv_bfloat16* crow = crow_base + col;
          if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              reinterpret_cast<uint4*>(crow)[v] = o;
            }
          } else {
            for (int j = 0; j < 32 && col + j < N; ++j) crow[j] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tmem_empty[acc]);
        else mbar_arrive_cluster(empty_remote + acc * 8);
      }
      if (MODE == 2 && !remote) {
        // local tile part stored in `out`: count it in this rank's own pad (the trailing reduce waits for every
        // source including itself)
        __threadfence();
        __syncwarp();
        if (lane == 0)
          red_add_release_sys(my_pad + a.count_word + (set * 16 + a.my_pos) * MAX_RB + rb, 1u);
      }
    }
    if (MODE == 2 && pending) {
      if (lane == 0) {
        bulk_wait_all();
        fence_proxy_async_all();
        __threadfence_system();
        red_add_release_sys(pend_counter, 1u);
      }
      pending = false;
    }
    if (!ok && lane == 0) atomicCAS(status, ST_OK, ST_TIMEOUT_EPILOGUE);

    if (MODE == 2 && ok) {
      // ---------------- trailing reduce of the local shard: out += received slots ----------------
      const int gemm_ctas = static_cast<int>(gridDim.x) - n_comm;
      const uint32_t want = static_cast<uint32_t>(tiles_n) * 8u;
      const int units = a.rows_per_rank / 8;
      const int ew = warp - 2;                                   // 0..3
      const int vec_per_row = N >> 3;
      const size_t slot_bytes = static_cast<size_t>(a.rows_per_rank / 32) * tiles_n * RECV_BLOCK_BYTES;
      const char* my_recv = reinterpret_cast<const char*>(a.recv.p[a.my_pos]);
      int waited_rb = -1;
      for (int u = gemm_cta; u < units; u += gemm_ctas) {
        const int r0 = u * 8;
        const int rbk = r0 / CHUNK_ROWS;
        if (rbk != waited_rb) {
          bool got = true;
          if (lane < a.n)
            got = wait_flag_sys(my_pad + a.count_word + (set * 16 + lane) * MAX_RB + rbk, want, a.timeout_ns, status);
          if (!__all_sync(0xffffffffu, got)) break;
          waited_rb = rbk;
        }
        for (int rr = ew * 2; rr < ew * 2 + 2; ++rr) {
          const int lr = r0 + rr;
          __nv_bfloat16* orow = a.out + static_cast<size_t>(lr) * a.ld_out;
          const int half = (lr & 255) >> 7, q4 = (lr & 127) >> 5, r32 = lr & 31;
          // eight independent 16-byte vectors per lane and pass keep enough loads in flight
          for (int v0 = 0; v0 < vec_per_row; v0 += 256) {
            float f[8][8];
            size_t boff[8];
            bool on[8];
            uint4 tmp[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int v = v0 + lane + 32 * k;
              on[k] = v < vec_per_row;
              const int c0 = v * 8;
              const int btn = c0 >> 8, bpass = (c0 >> 7) & 1, bj = (c0 & 127) >> 3;
              boff[k] = ((static_cast<size_t>(rbk * tiles_n + btn) * 2 + half) * 4 + q4) * RECV_BLOCK_BYTES +
                        static_cast<size_t>(bpass * 32 + r32) * 256 + ((bj ^ (r32 & 15)) << 4);
              if (on[k]) tmp[k] = *reinterpret_cast<const uint4*>(orow + c0);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float2 t0 = unpack_bf16x2(tmp[k].x), t1 = unpack_bf16x2(tmp[k].y), t2 = unpack_bf16x2(tmp[k].z),
                     t3 = unpack_bf16x2(tmp[k].w);
              f[k][0] = t0.x; f[k][1] = t0.y; f[k][2] = t1.x; f[k][3] = t1.y;
              f[k][4] = t2.x; f[k][5] = t2.y; f[k][6] = t3.x; f[k][7] = t3.y;
            }
            for (int s = 0; s < a.n - 1; ++s) {
              const char* rbase = my_recv + s * slot_bytes;
#pragma unroll
              for (int k = 0; k < 8; ++k)
                if (on[k]) tmp[k] = ld_peer_v4(rbase + boff[k]);
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                float2 g0 = unpack_bf16x2(tmp[k].x), g1 = unpack_bf16x2(tmp[k].y), g2 = unpack_bf16x2(tmp[k].z),
                       g3 = unpack_bf16x2(tmp[k].w);
                f[k][0] += g0.x; f[k][1] += g0.y; f[k][2] += g1.x; f[k][3] += g1.y;
                f[k][4] += g2.x; f[k][5] += g2.y; f[k][6] += g3.x; f[k][7] += g3.y;
              }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              if (!on[k]) continue;
              uint4 o;
              o.x = pack_bf16x2(f[k][0], f[k][1]); o.y = pack_bf16x2(f[k][2], f[k][3]);
              o.z = pack_bf16x2(f[k][4], f[k][5]); o.w = pack_bf16x2(f[k][6], f[k][7]);
              *reinterpret_cast<uint4*>(orow + (v0 + lane + 32 * k) * 8) = o;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

}  // namespace fused
}  // namespace hsb

using namespace hsb;
using namespace hsb::fused;

// Shapes: M = n * rows_per_rank tokens.  mode 1: A = xg [M, K] (this GPU), B = W [N, K]; C [M, N] bf16.
//         mode 2: A [M, K], B = W [K, N]; out [rows_per_rank, N] bf16 receives the reduced local shard.
// Pointer tables (pads, src, recv) have n entries, position = index in the group.
extern "C" int hsb_gemm_fused_comm(int mode, const void* A, const void* B, void* C, int M, int N, int K, int lda,
                                   int ldb, int ldc, int n, int my_pos, int rows_per_rank, uint32_t epoch,
                                   void* const* pads, int ready_word, int count_word, void* const* src,
                                   uint32_t* chunk_flags, void* const* recv, void* out, int ld_out, int n_comm_ctas,
                                   uint64_t timeout_ns, int* status, void* stream, int num_sms) {
  if (M <= 0 || N <= 0 || K <= 0 || !status || n < 2 || n > SYMM_MAX_RANKS) return -10;
  if (rows_per_rank % CHUNK_ROWS || M != n * rows_per_rank || rows_per_rank / CHUNK_ROWS > MAX_RB) return -13;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8) || (N % 8))
    return -11;
  if (num_sms <= 0) num_sms = 148;
  Args a{};
  a.mode = mode; a.n = n; a.my_pos = my_pos; a.rows_per_rank = rows_per_rank; a.epoch = epoch;
  a.timeout_ns = timeout_ns; a.ready_word = ready_word; a.count_word = count_word;
  for (int i = 0; i < SYMM_MAX_RANKS; ++i) {
    a.pads.p[i] = i < n ? pads[i] : nullptr;
    a.src.p[i] = (i < n && src) ? src[i] : nullptr;
    a.recv.p[i] = (i < n && recv) ? recv[i] : nullptr;
  }
  a.chunk_flags = chunk_flags;
  a.xg = reinterpret_cast<char*>(const_cast<void*>(A));
  a.row_bytes = static_cast<int64_t>(K) * 2;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.ld_out = ld_out;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap tmA, tmB;
  if (make_tmap_bf16_2d(&tmA, A, M, K, lda, BM, BK)) return -2;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  if (mode == 1) {
    if (lda != K || !src || !chunk_flags) return -10;      // the gathered A is dense: chunks are contiguous
    if (n_comm_ctas < 2) n_comm_ctas = 4;
    n_comm_ctas &= ~1;
    a.n_comm_ctas = n_comm_ctas;
    if (make_tmap_bf16_2d(&tmB, B, N, K, ldb, BNH, BK)) return -2;
    auto kern = gemm_comm_kernel<1>;
    static bool attr_set = false;
    if (!attr_set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -3;
      attr_set = true;
    }
    int clusters = (num_sms - n_comm_ctas) / 2;
    if (tiles < clusters) clusters = tiles;
    kern<<<n_comm_ctas + 2 * clusters, THREADS, SMEM_BYTES, st>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), ldc, M,
                                                                 N, K, a, status);
  } else if (mode == 2) {
    if (!recv || !out) return -10;
    a.n_comm_ctas = 0;
    if (make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, 64)) return -2;
    auto kern = gemm_comm_kernel<2>;
    static bool attr_set = false;
    if (!attr_set) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -3;
      attr_set = true;
    }
    int clusters = num_sms / 2;
    if (tiles < clusters) clusters = tiles;
    kern<<<2 * clusters, THREADS, SMEM_BYTES, st>>>(tmA, tmB, nullptr, 0, M, N, K, a, status);
  } else {
    return -12;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
