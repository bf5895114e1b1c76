// bf16 GEMM with CTA-pair MMAs (tcgen05.mma.cta_group::2): a cluster of two CTAs on neighbouring SMs
// computes one 256x256 tile of C.  Each CTA stages its own 128 rows of A and its own 128 rows of B
// (half of the tile's N) per k-block with TMA, the leader CTA issues 256x256x16 MMAs that read both
// CTAs' shared memory, and each CTA ends up with its 128 rows of the accumulator in its own TMEM.
// Per MMA an SM therefore reads 8 KB of shared memory instead of the 12 KB of the 1-CTA 128x256 tile,
// which is what limits the 1-CTA kernel (see the operand conventions in gemm_tcgen05.cu).
//
// Synchronisation between the two CTAs (rank 0 = leader):
//   full[s]       leader only   count 1: the leader's producer arrives with expect_tx for the bytes of BOTH
//                               CTAs; both CTAs' TMA loads complete_tx on it (no multicast is involved)
//   empty[s]      both CTAs     count 1: the leader's tcgen05.commit arrives on both at once
//   tmem_full[a]  both CTAs     count 1: same commit mechanism, tells each CTA's epilogue its half is ready
//   tmem_empty[a] leader only   count 8: the four epilogue warps of each CTA arrive (the peer's remotely)
// Every wait is bounded; a CTA that gives up raises the abort flag of both CTAs so the pair unwinds together.
#include "common.cuh"
#include "gemm_api.h"
#include <cuda.h>

namespace hsb {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols);

namespace pair {

constexpr int BM = 128;          // rows of A per CTA (tile M = 256 per pair)
constexpr int BNH = 128;         // rows of B per CTA (tile N = 256 per pair)
constexpr int BN = 2 * BNH;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 32 KB per CTA
constexpr int STAGES = 6;
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

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
  __device__ __forceinline__ void raise() const {
    *local = 1;
    st_cluster_u32(peer_addr, 1u);
  }
};

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, const AbortCtl& ab) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++it) & 0xff) == 0) {
      if (*ab.local) return false;
      if (globaltimer_ns() - t0 > HSB_WAIT_LIMIT_NS) {
        ab.raise();
        return false;
      }
    }
  }
  return true;
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      void* __restrict__ Cout, int ldc, int M, int N, int K, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + ACC_STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 8); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers exist before anything arrives on them remotely
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
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_of(t, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!wait_bar(&empty_bar[s], ph ^ 1, ab)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[s]), 0);       // the leader's barrier
          if (leader) mbar_arrive_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmA, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmA, bar, m0 + j * 64, k0);
          }
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
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
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
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s], 3);       // frees the stage in both CTAs
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
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++tile_iter) {
      int tm, tn;
      tile_of(t, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
      const int n0 = tn * BN;
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!wait_bar(&tmem_full[acc], acc_ph, ab)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr0 + c, r);
        tmem_ld_wait();
        const int col = n0 + c;
        if (row < M && col < N) {
          if constexpr (EPI == GEMM_EPI_BF16) {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + static_cast<size_t>(row) * ldc + col;
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
          } else {
            float* crow = reinterpret_cast<float*>(Cout) + static_cast<size_t>(row) * ldc + col;
            if (col + 32 <= N && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v + 0]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if constexpr (EPI == GEMM_EPI_F32_ACC) {
                  const float4 p = reinterpret_cast<const float4*>(crow)[v];
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                reinterpret_cast<float4*>(crow)[v] = o;
              }
            } else {
              for (int j = 0; j < 32 && col + j < N; ++j) {
                float o = __uint_as_float(r[j]);
                if constexpr (EPI == GEMM_EPI_F32_ACC) o += crow[j];
                crow[j] = o;
              }
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
    }
    if (!ok && lane == 0) atomicCAS(status, ST_OK, ST_TIMEOUT_EPILOGUE);
  }

  // ------------------------------ teardown ------------------------------------
  // Nothing of this CTA may be touched by its peer (commits, remote arrivals, MMA operand reads) after it
  // exits, so the pair leaves together.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

template <bool A_MN, bool B_MN, int EPI>
static int launch(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int* status,
                  cudaStream_t stream, int num_sms) {
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, BM, BK);
  else       rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, BNH, BK);
  else       rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, 64);
  if (rc) return rc;
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -3;
    attr_set = true;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int clusters = num_sms / 2;
  if (tiles < clusters) clusters = tiles;
  kern<<<2 * clusters, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, C, ldc, M, N, K, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int EPI>
static int dispatch_major(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                          int a_mn, int b_mn, int* status, cudaStream_t stream, int num_sms) {
  if (!a_mn && !b_mn) return launch<false, false, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
  if (!a_mn && b_mn)  return launch<false, true, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
  if (a_mn && !b_mn)  return launch<true, false, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
  return launch<true, true, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
}

}  // namespace pair
}  // namespace hsb

extern "C" int hsb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                  int ldc, int a_mn_major, int b_mn_major, int epi, int* status, void* stream,
                                  int num_sms) {
  using namespace hsb;
  if (M <= 0 || N <= 0 || K <= 0 || !status) return -10;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8))
    return -11;
  if (num_sms <= 0) num_sms = 148;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (epi) {
    case GEMM_EPI_BF16:
      return pair::dispatch_major<GEMM_EPI_BF16>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, status, st,
                                                 num_sms);
    case GEMM_EPI_F32:
      return pair::dispatch_major<GEMM_EPI_F32>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, status, st,
                                                num_sms);
    case GEMM_EPI_F32_ACC:
      return pair::dispatch_major<GEMM_EPI_F32_ACC>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, status,
                                                    st, num_sms);
    default:
      return -12;
  }
}
