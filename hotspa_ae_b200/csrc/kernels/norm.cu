// Fused RMSNorm / LayerNorm forward and backward for bf16 activations (sm_100a).
//
// Replaces the reference's apex-derived kernels (hetu/impl/kernel/FusedLayerNorm.cu: cuApplyLayerNorm,
// cuApplyRMSNorm, cuComputeGradInput, cuComputePartGradGammaBeta) and the dropout_add_ln wrapper
// (hetu/impl/kernel/RMSNorm.cu).  Differences on purpose: the residual add that precedes the norm
// and the residual-gradient add that follows its backward are folded into the same pass, rows are
// moved with 128-bit accesses and kept in registers between the statistics and the write-out, and
// the weight-gradient reduction is a two-stage reduce through a caller supplied fp32 scratch
// ([partial_rows, 2, H]) that accumulates straight into the fp32 gradient arena.
#include "common.cuh"
#include "ew_api.h"

namespace hsb {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 4;  // 256 threads * 4 chunks * 8 elems = H <= 8192 kept in registers

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// y = norm(x (+ res)) * w (+ b);  optionally writes hsum = x + res;  saves rstd (and mean for LayerNorm).
template <bool RMS>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ hsum, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, int rows, int H, float eps) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    float xv[NORM_MAX_VEC][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NORM_MAX_VEC; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nvec) {
        load8(x + base + i * 8, xv[c]);
        if (res) {
          float rv[8];
          load8(res + base + i * 8, rv);
#pragma unroll
          for (int j = 0; j < 8; ++j) xv[c][j] += rv[j];
          if (hsum) {
            store8(hsum + base + i * 8, xv[c]);
            // the stored sum is bf16: normalise exactly what later kernels will read back
            load8(hsum + base + i * 8, xv[c]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) { s1 += xv[c][j]; s2 += xv[c][j] * xv[c][j]; }
      }
    }
    float mean = 0.f, rstd;
    if (RMS) {
      s2 = block_sum(s2, red);
      rstd = rsqrtf(s2 / H + eps);
    } else {
      s1 = block_sum(s1, red);
      mean = s1 / H;
      float var = 0.f;
#pragma unroll
      for (int c = 0; c < NORM_MAX_VEC; ++c) {
        const int i = threadIdx.x + c * NORM_THREADS;
        if (i < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float d = xv[c][j] - mean; var += d * d; }
        }
      }
      var = block_sum(var, red);
      rstd = rsqrtf(var / H + eps);
    }
    if (threadIdx.x == 0) {
      rstd_out[row] = rstd;
      if (!RMS) mean_out[row] = mean;
    }
#pragma unroll
    for (int c = 0; c < NORM_MAX_VEC; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nvec) {
        float wv[8], o[8];
        load8(w + i * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (xv[c][j] - mean) * rstd * wv[j];
        if (!RMS && b) {
          float bv[8];
          load8(b + i * 8, bv);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += bv[j];
        }
        store8(y + base + i * 8, o);
      }
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// dx = d(norm)/dx applied to dy (+ dres);  per-CTA partial dw/db into scratch[blockIdx.x][0|1][H].
// NV = 128-bit chunks of a row per thread (H <= 2048 * NV).  The raw dy / x chunks of the CTA's next row and the
// residual gradient of the current one are requested before the block-wide reduction of the current row, so the
// loads are in flight across its two barriers; with NV <= 2 two CTAs fit an SM.
template <bool RMS, int NV>
__global__ void __launch_bounds__(NORM_THREADS, (NV <= 2) ? 2 : 1)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ scratch, int rows, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dw_acc[NV][8], db_acc[NV][8], wv[NV][8];
  uint4 dy_raw[NV], x_raw[NV], r_raw[NV];
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < NV; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[c][j] = 0.f; db_acc[c][j] = 0.f; wv[c][j] = 0.f; }
    if (i < nvec) load8(w + i * 8, wv[c]);
    dy_raw[c] = zero4; x_raw[c] = zero4; r_raw[c] = zero4;
  }
  int row = blockIdx.x;
  if (row < rows) {
    const size_t base = static_cast<size_t>(row) * H;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nvec) {
        dy_raw[c] = *reinterpret_cast<const uint4*>(dy + base + i * 8);
        x_raw[c] = *reinterpret_cast<const uint4*>(x + base + i * 8);
      }
    }
  }
  for (; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    const float mean = RMS ? 0.f : mean_in[row];
    float g[NV][8], xh[NV][8];
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      float dyv[8], xv[8];
      unpack8(dy_raw[c], dyv);           // chunks past the row end hold zeros and add nothing
      unpack8(x_raw[c], xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[c][j] = (xv[j] - mean) * rstd;
        g[c][j] = dyv[j] * wv[c][j];
        sg += g[c][j];
        sgx += g[c][j] * xh[c][j];
        dw_acc[c][j] += dyv[j] * xh[c][j];
        db_acc[c][j] += dyv[j];
      }
    }
    const int next = row + gridDim.x;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nvec) {
        if (dres) r_raw[c] = *reinterpret_cast<const uint4*>(dres + base + i * 8);
        if (next < rows) {
          const size_t nb = static_cast<size_t>(next) * H;
          dy_raw[c] = *reinterpret_cast<const uint4*>(dy + nb + i * 8);
          x_raw[c] = *reinterpret_cast<const uint4*>(x + nb + i * 8);
        }
      }
    }
    sgx = block_sum(sgx, red) / H;
    if (!RMS) sg = block_sum(sg, red) / H; else sg = 0.f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
      const int i = threadIdx.x + c * NORM_THREADS;
      if (i < nvec) {
        float o[8], rv[8];
        unpack8(r_raw[c], rv);            // zeros when there is no residual gradient
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[c][j] - sg - xh[c][j] * sgx) + rv[j];
        store8(dx + base + i * 8, o);
      }
    }
  }
  float* my = scratch + static_cast<size_t>(blockIdx.x) * 2 * H;
#pragma unroll
  for (int c = 0; c < NV; ++c) {
    const int i = threadIdx.x + c * NORM_THREADS;
    if (i < nvec) {
      *reinterpret_cast<float4*>(my + i * 8) = make_float4(dw_acc[c][0], dw_acc[c][1], dw_acc[c][2], dw_acc[c][3]);
      *reinterpret_cast<float4*>(my + i * 8 + 4) = make_float4(dw_acc[c][4], dw_acc[c][5], dw_acc[c][6], dw_acc[c][7]);
      if (!RMS) {
        *reinterpret_cast<float4*>(my + H + i * 8) = make_float4(db_acc[c][0], db_acc[c][1], db_acc[c][2], db_acc[c][3]);
        *reinterpret_cast<float4*>(my + H + i * 8 + 4) = make_float4(db_acc[c][4], db_acc[c][5], db_acc[c][6], db_acc[c][7]);
      }
    }
  }
}

// dw[h] (+)= sum_p scratch[p][0][h];  db likewise from scratch[p][1][h].
// A CTA owns 32 columns; its 8 warps each sum every 8th partial row, then combine through shared memory.
constexpr int NORM_RED_COLS = 32, NORM_RED_WAYS = 8;
__global__ void __launch_bounds__(NORM_RED_COLS * NORM_RED_WAYS)
norm_bwd_reduce_kernel(const float* __restrict__ scratch, float* __restrict__ dw, float* __restrict__ db, int parts,
                       int H, int accumulate) {
  __shared__ float sa[NORM_RED_WAYS][NORM_RED_COLS], sb[NORM_RED_WAYS][NORM_RED_COLS];
  const int lane = threadIdx.x & 31, way = threadIdx.x >> 5;
  const int h = blockIdx.x * NORM_RED_COLS + lane;
  float a = 0.f, b = 0.f;
  if (h < H) {
#pragma unroll 4
    for (int p = way; p < parts; p += NORM_RED_WAYS) {
      a += scratch[static_cast<size_t>(p) * 2 * H + h];
      if (db) b += scratch[static_cast<size_t>(p) * 2 * H + H + h];
    }
  }
  sa[way][lane] = a;
  sb[way][lane] = b;
  __syncthreads();
  if (way == 0 && h < H) {
#pragma unroll
    for (int k = 1; k < NORM_RED_WAYS; ++k) { a += sa[k][lane]; b += sb[k][lane]; }
    if (accumulate) { dw[h] += a; if (db) db[h] += b; }
    else            { dw[h] = a;  if (db) db[h] = b; }
  }
}

template <bool RMS>
static void launch_norm_bwd(int parts, cudaStream_t st, const __nv_bfloat16* DY, const __nv_bfloat16* X,
                            const __nv_bfloat16* W, const float* mean, const float* rstd, const __nv_bfloat16* DR,
                            __nv_bfloat16* DX, float* scratch, int rows, int H) {
  const int nv = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
  if (nv <= 1)      norm_bwd_kernel<RMS, 1><<<parts, NORM_THREADS, 0, st>>>(DY, X, W, mean, rstd, DR, DX, scratch, rows, H);
  else if (nv == 2) norm_bwd_kernel<RMS, 2><<<parts, NORM_THREADS, 0, st>>>(DY, X, W, mean, rstd, DR, DX, scratch, rows, H);
  else if (nv == 3) norm_bwd_kernel<RMS, 3><<<parts, NORM_THREADS, 0, st>>>(DY, X, W, mean, rstd, DR, DX, scratch, rows, H);
  else              norm_bwd_kernel<RMS, 4><<<parts, NORM_THREADS, 0, st>>>(DY, X, W, mean, rstd, DR, DX, scratch, rows, H);
}

}  // namespace hsb

using namespace hsb;

extern "C" int hsb_norm_bwd_parts(int rows, int num_sms) {
  if (num_sms <= 0) num_sms = 148;
  const int want = num_sms * 2;
  return rows < want ? rows : want;
}

extern "C" int hsb_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* hsum,
                            float* mean, float* rstd, int rows, int H, float eps, int is_rms, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAX_VEC * 8 || rows <= 0) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<const __nv_bfloat16*>(res);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto B = reinterpret_cast<const __nv_bfloat16*>(b);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  auto Hs = reinterpret_cast<__nv_bfloat16*>(hsum);
  if (is_rms) norm_fwd_kernel<true><<<grid, NORM_THREADS, 0, st>>>(X, R, W, B, Y, Hs, mean, rstd, rows, H, eps);
  else        norm_fwd_kernel<false><<<grid, NORM_THREADS, 0, st>>>(X, R, W, B, Y, Hs, mean, rstd, rows, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// scratch must hold hsb_norm_bwd_parts(rows) * 2 * H floats.
extern "C" int hsb_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                            const void* dres, void* dx, float* dw, float* db, float* scratch, int rows, int H,
                            int is_rms, int accumulate, int num_sms, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAX_VEC * 8 || rows <= 0 || !scratch) return -10;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int parts = hsb_norm_bwd_parts(rows, num_sms);
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  if (is_rms) launch_norm_bwd<true>(parts, st, DY, X, W, mean, rstd, DR, DX, scratch, rows, H);
  else        launch_norm_bwd<false>(parts, st, DY, X, W, mean, rstd, DR, DX, scratch, rows, H);
  norm_bwd_reduce_kernel<<<(H + NORM_RED_COLS - 1) / NORM_RED_COLS, NORM_RED_COLS * NORM_RED_WAYS, 0, st>>>(
      scratch, dw, is_rms ? nullptr : db, parts, H, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ----------------------------------------------------------------------------------------------
// Allocation-free variant of hsb_norm_bwd (declared and documented in norm_noalloc_api.h).
// The stage-one partial sums go to a scratch array that is part of the library image instead of a
// buffer the caller allocates.
// ----------------------------------------------------------------------------------------------
#include "norm_noalloc_api.h"
#include <cstdio>
#include <mutex>

namespace hsb {

// One copy per GPU that loads the library, resident until the process exits.
static __device__ __align__(256) float g_norm_bwd_scratch[HSB_NORM_BWD_NOALLOC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
static float* g_norm_bwd_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_norm_bwd_scratch_mutex;

// Device address of the array on the current device.  `g_norm_bwd_scratch` in host code is only a
// handle for the runtime, not something a kernel may dereference, so the address is looked up once
// per device (with that device current) and cached.
static int norm_bwd_scratch_address(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -21;
  std::lock_guard<std::mutex> lock(g_norm_bwd_scratch_mutex);
  if (g_norm_bwd_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_norm_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "hsb_norm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return -22;
    }
    g_norm_bwd_scratch_addr[dev] = static_cast<float*>(p);
  }
  *out = g_norm_bwd_scratch_addr[dev];
  return 0;
}

}  // namespace hsb

extern "C" long hsb_norm_bwd_noalloc_max_floats(void) { return HSB_NORM_BWD_NOALLOC_MAX_FLOATS; }

extern "C" int hsb_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean,
                                    const float* rstd, const void* dres, void* dx, float* dw, float* db, int rows,
                                    int H, int is_rms, int accumulate, int num_sms, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAX_VEC * 8 || rows <= 0) return -10;
  const long need = static_cast<long>(hsb_norm_bwd_parts(rows, num_sms)) * 2 * H;
  if (need > HSB_NORM_BWD_NOALLOC_MAX_FLOATS) {
    fprintf(stderr,
            "hsb_norm_bwd_noalloc: rows=%d H=%d num_sms=%d needs %ld scratch floats, the built-in scratch holds %ld; "
            "use hsb_norm_bwd with a caller-allocated scratch for this size\n",
            rows, H, num_sms, need, static_cast<long>(HSB_NORM_BWD_NOALLOC_MAX_FLOATS));
    return -20;
  }
  float* scratch = nullptr;
  const int rc = norm_bwd_scratch_address(&scratch);
  if (rc != 0) return rc;
  // Every float of the scratch that stage two reads is written by stage one of the same call, so
  // nothing has to be cleared even though the array still holds the previous call's partial sums.
  return hsb_norm_bwd(dy, x, w, mean, rstd, dres, dx, dw, db, scratch, rows, H, is_rms, accumulate, num_sms, stream);
}
