// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged by TMA into a 128-byte-swizzled shared-memory ring.
//
//   C[M,N] (=|+=) op(A) * op(B)^T        fp32 accumulation
//
//   A operand:  K-major  -> stored [M, K] row-major (lda = row stride in elements)
//               MN-major -> stored [K, M] row-major
//   B operand:  K-major  -> stored [N, K] row-major (a torch Linear weight [out, in])
//               MN-major -> stored [K, N] row-major
//
// so the three GEMMs of a Linear layer y = x W^T need no transposed copies:
//   fwd    y  = x  W^T   : A = x  (K-major),          B = W  (K-major)
//   dgrad  dx = dy W     : A = dy (K-major),          B = W  ([K=out, N=in], MN-major)
//   wgrad  dW = dy^T x   : A = dy ([K=T, M=out], MN), B = x  ([K=T, N=in], MN-major)
//
// Role of this file in the framework: replaces the cuBLAS call behind the reference's
// Linear/MatMul ops (hetu/impl/kernel/Linear.cu, MatMul.cu, hetu/impl/cuda/CUDABlas.cc:115-138).
//
// Kernel structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer     (one elected lane)
//   warp 1      MMA issuer       (one elected lane) + TMEM allocation
//   warps 2..5  epilogue         (tcgen05.ld -> convert -> global), one TMEM lane quarter each
// The TMEM holds two accumulator stages so the epilogue of tile i overlaps the mainloop of tile i+1.
#include "common.cuh"
#include "gemm_api.h"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>
#include <cstdio>

namespace hsb {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int ACC_STAGES = 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct TileCoord { int m, n; };

__device__ __forceinline__ TileCoord tile_of(int t, int tiles_m, int tiles_n) {
  // Grouped raster: 8 M-tiles share their B columns in L2 while marching along N.
  constexpr int GROUP = 8;
  const int width = GROUP * tiles_n;
  const int group_id = t / width;
  const int first_m = group_id * GROUP;
  const int gsz = min(tiles_m - first_m, GROUP);
  const int r = t - group_id * width;
  TileCoord c;
  c.m = first_m + (r % gsz);
  c.n = r / gsz;
  return c;
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         void* __restrict__ Cout, int ldc, int M, int N, int K, int* __restrict__ status) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + Cfg::ACC_STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty + Cfg::ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < Cfg::ACC_STAGES; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 4); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_of(t, tiles_m, tiles_n);
        const int m0 = tc.m * BM, n0 = tc.n * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmA, &full_bar[s], m0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmB, &full_bar[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmB, &full_bar[s], n0 + j * 64, k0);
          }
        }
      }
      if (!ok) atomicCAS(status, ST_OK, ST_TIMEOUT_PRODUCER);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
        const int acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 8192, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);   // frees the smem stage once these MMAs retire
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
      if (!ok) atomicCAS(status, ST_OK, ST_TIMEOUT_MMA);
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      const TileCoord tc = tile_of(t, tiles_m, tiles_n);
      const int m0 = tc.m * BM, n0 = tc.n * BN;
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag)) { ok = false; break; }
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
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    if (!ok && lane == 0) atomicCAS(status, ST_OK, ST_TIMEOUT_EPILOGUE);
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with row stride ld (elements);
// box = [box_rows, 64 cols] with 128-byte swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols) {
  auto fn = get_encode_fn();
  if (!fn) return -1;
  // The driver entry point needs a current context on the calling thread; autograd worker threads may
  // not have touched the runtime yet, so bind the primary context once per thread.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "hsb: cuTensorMapEncodeTiled failed (%d): base=%p rows=%llu cols=%llu ld=%llu box=[%u,%u]\n",
            static_cast<int>(r), base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld,
            box_rows, box_cols);
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <int BN, bool A_MN, bool B_MN, int EPI>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                       int* status, cudaStream_t stream, int num_sms) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, BM, BK);
  else       rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, BN, BK);
  else       rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, BK, 64);
  if (rc) return rc;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -3;
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, C, ldc, M, N, K, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int BN, int EPI>
static int dispatch_major(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                          int a_mn, int b_mn, int* status, cudaStream_t stream, int num_sms) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
  if (!a_mn && b_mn)  return launch_gemm<BN, false, true, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
  if (a_mn && !b_mn)  return launch_gemm<BN, true, false, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
  return launch_gemm<BN, true, true, EPI>(A, B, C, M, N, K, lda, ldb, ldc, status, stream, num_sms);
}

}  // namespace hsb

extern "C" int hsb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                             int a_mn_major, int b_mn_major, int epi, int tile_n, int* status, void* stream,
                             int num_sms) {
  using namespace hsb;
  if (M <= 0 || N <= 0 || K <= 0 || !status) return -10;
  // TMA needs 16-byte aligned bases and row strides.
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8))
    return -11;
  if (num_sms <= 0) num_sms = 148;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (tile_n == 2 || (tile_n == 0 && M > 128 && N > 128))
    return hsb_gemm_bf16_pair(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, epi, status, stream, num_sms);
  if (tile_n == 0) {
    // Pick the tile width with the fewer waves-times-width (ties -> the wider tile).
    auto cost = [&](int bn) {
      long tiles = (long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
      long waves = (tiles + num_sms - 1) / num_sms;
      return waves * bn;
    };
    tile_n = (N > 128 && cost(256) <= cost(128)) ? 256 : 128;
  }
#define HSB_DISPATCH_EPI(BN_)                                                                                      \
  switch (epi) {                                                                                                   \
    case GEMM_EPI_BF16:                                                                                            \
      return dispatch_major<BN_, GEMM_EPI_BF16>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, status,   \
                                                st, num_sms);                                                      \
    case GEMM_EPI_F32:                                                                                             \
      return dispatch_major<BN_, GEMM_EPI_F32>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, status,    \
                                               st, num_sms);                                                       \
    case GEMM_EPI_F32_ACC:                                                                                         \
      return dispatch_major<BN_, GEMM_EPI_F32_ACC>(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major,        \
                                                   status, st, num_sms);                                           \
    default:                                                                                                       \
      return -12;                                                                                                  \
  }
  if (tile_n == 256) { HSB_DISPATCH_EPI(256) }
  else               { HSB_DISPATCH_EPI(128) }
#undef HSB_DISPATCH_EPI
}
