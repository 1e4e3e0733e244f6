// Memory-bound layer ops for sm_100a: RMSNorm forward/backward, SwiGLU forward/backward and the
// residual add. All of them move 16 bytes per thread per access and keep one pass over HBM
// per tensor; the weight-gradient of RMSNorm is reduced in registers per CTA and finished by a
// second, tiny kernel so no atomics are needed and the result is deterministic.
//
// Counterparts in the reference: TE RMSNorm fused into TELayerNormColumnParallelLinear and the TE
// SwiGLU activation (distca/runtime/megatron/model_patch.py:77-98), Megatron bias-dropout-add
// (distca/runtime/megatron/base_transformer_layer.py:605-608).
#include <mutex>

#include "../common/host_utils.h"
#include "../common/ptx.cuh"

namespace dca {
namespace ew {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 4;  // vectors of 8 bf16 per thread: hidden size up to 256*8*4 = 8192

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// y = x * rsqrt(mean(x^2) + eps) * g ; rstd saved per row for the backward pass.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int T, int H, float eps) {
  __shared__ float scratch[32];
  const int nvec = H / 8;
  for (long row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * H;
    float xv[kMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        load8(xr + v * 8, xv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += xv[i][j] * xv[i][j];
      }
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    if (threadIdx.x == 0 && rstd != nullptr) rstd[row] = r;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float gv[8], o[8];
        load8(g + v * 8, gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = xv[i][j] * r * gv[j];
        store8(y + row * H + v * 8, o);
      }
    }
  }
}

// dx = rstd * (dy*g - xhat * mean(dy*g*xhat)) [+ dres];  dg_partial[cta] = sum_rows dy * xhat
// NV = 16-byte vectors per thread (hidden size up to 256 * 8 * NV). The per-row critical path is
// load -> block reduction -> store, so the kernel lives on occupancy: the weight is re-read from L1 every
// row instead of being held in registers, the residual-gradient load is issued before the reduction, and
// CTAS CTAs share an SM (measured at [131072, 4096]: 1 CTA per SM-half with everything in registers
// reached 0.26 of the copy bandwidth).
template <int NV, int CTAS>
__global__ void __launch_bounds__(kNormThreads, CTAS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                   const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dy,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dg_partial, int T, int H) {
  __shared__ float scratch[32];
  const int nvec = H / 8;
  float dg[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) dg[i][j] = 0.f;
  }
  for (long row = blockIdx.x; row < T; row += gridDim.x) {
    const float r = rstd[row];
    float xh[NV][8], dyg[NV][8];
    uint4 res[NV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xv[8], dv[8], gv[8];
        load8(x + row * H + v * 8, xv);
        load8(dy + row * H + v * 8, dv);
        load8(g + v * 8, gv);
        if (dres != nullptr) res[i] = *reinterpret_cast<const uint4*>(dres + row * H + v * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xv[j] * r;
          dyg[i][j] = dv[j] * gv[j];
          dg[i][j] += dv[j] * xh[i][j];
          dot += dyg[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, scratch) / (float)H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (dyg[i][j] - xh[i][j] * dot);
        if (dres != nullptr) {
          const float2 a = unpack_bf16x2(res[i].x), b = unpack_bf16x2(res[i].y);
          const float2 c = unpack_bf16x2(res[i].z), d = unpack_bf16x2(res[i].w);
          o[0] += a.x; o[1] += a.y; o[2] += b.x; o[3] += b.y; o[4] += c.x; o[5] += c.y; o[6] += d.x; o[7] += d.y;
        }
        store8(dx + row * H + v * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float4* dst = reinterpret_cast<float4*>(dg_partial + (long)blockIdx.x * H + v * 8);
      dst[0] = make_float4(dg[i][0], dg[i][1], dg[i][2], dg[i][3]);
      dst[1] = make_float4(dg[i][4], dg[i][5], dg[i][6], dg[i][7]);
    }
  }
}

// Launch with P CTAs (= rows of dg_partial), picking the vectors-per-thread variant for H.
inline cudaError_t launch_rmsnorm_bwd(int P, cudaStream_t s, const __nv_bfloat16* x, const __nv_bfloat16* g,
                                      const float* rstd, const __nv_bfloat16* dy, const __nv_bfloat16* dres,
                                      __nv_bfloat16* dx, float* dg_partial, int T, int H) {
  const int nv = (H / 8 + kNormThreads - 1) / kNormThreads;
  if (nv <= 1)
    rmsnorm_bwd_kernel<1, 4><<<P, kNormThreads, 0, s>>>(x, g, rstd, dy, dres, dx, dg_partial, T, H);
  else if (nv <= 2)
    rmsnorm_bwd_kernel<2, 4><<<P, kNormThreads, 0, s>>>(x, g, rstd, dy, dres, dx, dg_partial, T, H);
  else
    rmsnorm_bwd_kernel<4, 2><<<P, kNormThreads, 0, s>>>(x, g, rstd, dy, dres, dx, dg_partial, T, H);
  return cudaGetLastError();
}

// dg[h] (+)= sum_p partial[p,h]   (dg bf16 or fp32)
template <typename OutT>
__global__ void rmsnorm_dg_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ dg,
                                         int P, int H, int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[(long)p * H + h];
  if (accumulate) s += (float)dg[h];
  dg[h] = (OutT)s;
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }

// act[T,F] = silu(pre[:, :F]) * pre[:, F:]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ act,
                                  long T, int F) {
  const long nvec = T * (F / 8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long row = i / (F / 8);
    const int c = (int)(i % (F / 8)) * 8;
    float gv[8], uv[8], o[8];
    load8(pre + row * 2 * F + c, gv);
    load8(pre + row * 2 * F + F + c, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gv[j] * sigmoid_f(gv[j]) * uv[j];
    store8(act + row * F + c, o);
  }
}

// dpre = (dact * u * dsilu(g) | dact * silu(g)); dpre may alias pre.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* pre, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* dpre, long T, int F) {
  const long nvec = T * (F / 8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long row = i / (F / 8);
    const int c = (int)(i % (F / 8)) * 8;
    float gv[8], uv[8], dv[8], dg[8], du[8];
    load8(pre + row * 2 * F + c, gv);
    load8(pre + row * 2 * F + F + c, uv);
    load8(dact + row * F + c, dv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoid_f(gv[j]);
      dg[j] = dv[j] * uv[j] * s * (1.f + gv[j] * (1.f - s));
      du[j] = dv[j] * gv[j] * s;
    }
    store8(dpre + row * 2 * F + c, dg);
    store8(dpre + row * 2 * F + F + c, du);
  }
}

// out = a + b (bf16, n multiple of 8); out may alias a or b.
__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, long n) {
  const long nvec = n / 8;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float av[8], bv[8];
    load8(a + i * 8, av);
    load8(b + i * 8, bv);
#pragma unroll
    for (int j = 0; j < 8; ++j) av[j] += bv[j];
    store8(out + i * 8, av);
  }
}

inline int ew_grid(long work_items, int threads) {
  long blocks = (work_items + threads - 1) / threads;
  long cap = (long)sm_count() * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace ew
}  // namespace dca

using namespace dca;
using namespace dca::ew;

extern "C" int dca_rmsnorm_fwd(const void* x, const void* g, void* y, float* rstd, int T, int H,
                               float eps, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || H > kNormThreads * 8 * kMaxVec) return kErrBadArg;
  int grid = T < sm_count() * 8 ? T : sm_count() * 8;
  rmsnorm_fwd_kernel<<<grid, kNormThreads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, (__nv_bfloat16*)y, rstd, T, H, eps);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

// Number of CTAs (= rows of the dg_partial scratch) the backward kernel will use.
extern "C" int dca_rmsnorm_bwd_partials(int T) {
  int cap = sm_count() * 4;
  return T < cap ? (T > 0 ? T : 1) : cap;
}

// dg_partial: fp32 [dca_rmsnorm_bwd_partials(T), H] scratch. dg: bf16 (dg_fp32=0) or fp32.
extern "C" int dca_rmsnorm_bwd(const void* x, const void* g, const float* rstd, const void* dy,
                               const void* dres, void* dx, float* dg_partial, void* dg, int dg_fp32,
                               int dg_accumulate, int T, int H, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || H > kNormThreads * 8 * kMaxVec) return kErrBadArg;
  const int P = dca_rmsnorm_bwd_partials(T);
  cudaStream_t s = (cudaStream_t)stream;
  DCA_CUDA_TRY(launch_rmsnorm_bwd(P, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, rstd,
                                  (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx,
                                  dg_partial, T, H));
  if (dg_fp32)
    rmsnorm_dg_reduce_kernel<float><<<(H + 127) / 128, 128, 0, s>>>(dg_partial, (float*)dg, P, H, dg_accumulate);
  else
    rmsnorm_dg_reduce_kernel<__nv_bfloat16><<<(H + 127) / 128, 128, 0, s>>>(dg_partial, (__nv_bfloat16*)dg, P, H, dg_accumulate);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward that brings its own scratch (declared and documented in norm_act_noalloc.h).
// The array below is a device symbol: in host code its name is only a handle, so the launcher
// asks the runtime for the device address once per device and hands THAT to the kernels.
// ---------------------------------------------------------------------------------------------
#include "norm_act_noalloc.h"

static __device__ __align__(256) float g_noalloc_dg_partial[(size_t)kNoAllocMaxPartials * kNoAllocMaxH];

namespace {
constexpr int kNoAllocMaxDevices = 64;
float* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
int g_noalloc_partials_cap[kNoAllocMaxDevices] = {0};
int g_noalloc_setup_rc[kNoAllocMaxDevices] = {0};
std::once_flag g_noalloc_once[kNoAllocMaxDevices];   // first calls on one device may come from several host threads
}  // namespace

extern "C" int dca_rmsnorm_bwd_noalloc(const void* x, const void* g, const float* rstd, const void* dy,
                                       const void* dres, void* dx, void* dg, int dg_fp32, int dg_accumulate,
                                       int T, int H, void* stream) {
  if (T <= 0) return 0;
  if (H > kNoAllocMaxH) {
    fprintf(stderr, "[distca_b200] dca_rmsnorm_bwd_noalloc: H=%d exceeds the built-in scratch (max %d); use "
                    "dca_rmsnorm_bwd with a caller-provided buffer\n", H, (int)kNoAllocMaxH);
    return kErrTooLarge;
  }
  if (H % 8 != 0 || H > kNormThreads * 8 * kMaxVec) return kErrBadArg;
  int dev = -1;
  DCA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices) return kErrBadArg;
  // set-up, once per device, with that device current; concurrent first calls wait here for the one that runs it
  std::call_once(g_noalloc_once[dev], [dev]() {
    float* p = nullptr;
    int sms = 0;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dg_partial);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      fprintf(stderr, "[distca_b200] dca_rmsnorm_bwd_noalloc set-up: %s\n", cudaGetErrorString(e));
      g_noalloc_setup_rc[dev] = (int)e;
      return;
    }
    g_noalloc_partials_cap[dev] = 2 * sms;
    g_noalloc_ptr[dev] = p;
  });
  if (g_noalloc_setup_rc[dev] != 0 || g_noalloc_ptr[dev] == nullptr) return g_noalloc_setup_rc[dev] ? g_noalloc_setup_rc[dev] : kErrBadArg;
  const int cap = g_noalloc_partials_cap[dev];
  const int P = T < cap ? T : cap;
  if (P <= 0) return kErrBadArg;
  if (H > kNoAllocMaxH || P > kNoAllocMaxPartials) {
    fprintf(stderr,
            "[distca_b200] dca_rmsnorm_bwd_noalloc: H=%d (max %d) / %d partial rows (max %d) exceed the built-in "
            "scratch; use dca_rmsnorm_bwd with a caller-provided buffer\n",
            H, (int)kNoAllocMaxH, P, (int)kNoAllocMaxPartials);
    return kErrTooLarge;
  }
  float* partial = g_noalloc_ptr[dev];
  cudaStream_t s = (cudaStream_t)stream;
  DCA_CUDA_TRY(launch_rmsnorm_bwd(P, s, (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, rstd,
                                  (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx,
                                  partial, T, H));
  if (dg_fp32)
    rmsnorm_dg_reduce_kernel<float><<<(H + 127) / 128, 128, 0, s>>>(partial, (float*)dg, P, H, dg_accumulate);
  else
    rmsnorm_dg_reduce_kernel<__nv_bfloat16><<<(H + 127) / 128, 128, 0, s>>>(partial, (__nv_bfloat16*)dg, P, H, dg_accumulate);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_swiglu_fwd(const void* pre, void* act, long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F % 8 != 0) return kErrBadArg;
  swiglu_fwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)pre, (__nv_bfloat16*)act, T, F);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_swiglu_bwd(const void* pre, const void* dact, void* dpre, long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F % 8 != 0) return kErrBadArg;
  swiglu_bwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)pre, (const __nv_bfloat16*)dact, (__nv_bfloat16*)dpre, T, F);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_add_bf16(const void* a, const void* b, void* out, long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0) return kErrBadArg;
  add_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
