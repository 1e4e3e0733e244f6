// Vocabulary-parallel cross-entropy, embedding forward/backward, and the sharded Adam update.
//
// Cross-entropy runs in two kernels so that tensor-parallel ranks can exchange three numbers per
// token in between: (1) per-token local max, local sum of exponentials and the target logit of
// this rank's vocabulary slice; (2) given the statistics of every slice, the loss and, written as
// bf16, d(loss)/d(logits) for this slice. Logits are fp32 (the LM-head GEMM stores its fp32
// accumulators directly).
//
// Adam keeps the fp32 master weight split in two 16-bit halves: the bf16 parameter the model
// computes with IS the upper half, and a 16-bit correction stores what rounding removed, so the
// exact fp32 master is `(bf16 << 16) + int16` at a cost of 4 bytes instead of 6 per parameter.
//
// Counterparts in the reference: Megatron vocab_parallel_cross_entropy (pretrain_llama.py:228),
// VocabParallelEmbedding, and DistributedOptimizer + fused Adam (distca/utils/worker.py:49-66,
// distca/utils/megatron_test_utils.py:102-113, 235-258).
#include "../common/host_utils.h"
#include "../common/ptx.cuh"

namespace dca {
namespace lo {

constexpr int kCEThreads = 512;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// stats[t] = (max, sum exp(x - max), target logit or 0) over this rank's vocabulary slice
__global__ void __launch_bounds__(kCEThreads)
ce_stats_kernel(const float* __restrict__ logits, long ld, const long* __restrict__ labels, int vocab_start,
                int V, float* __restrict__ stats, long T) {
  __shared__ float sm[kCEThreads / 32], ss[kCEThreads / 32];
  for (long t = blockIdx.x; t < T; t += gridDim.x) {
    const float* row = logits + t * ld;
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x * 4; i < V; i += kCEThreads * 4) {
      const float4 x = *reinterpret_cast<const float4*>(row + i);
      const float mx = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
      if (mx > m) {
        s *= __expf(m - mx);
        m = mx;
      }
      s += __expf(x.x - m) + __expf(x.y - m) + __expf(x.z - m) + __expf(x.w - m);
    }
    const float wm = warp_max(m);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - wm);
    s = warp_sum(s);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { sm[warp] = wm; ss[warp] = s; }
    __syncthreads();
    if (warp == 0) {
      float m2 = lane < kCEThreads / 32 ? sm[lane] : -INFINITY;
      float s2 = lane < kCEThreads / 32 ? ss[lane] : 0.f;
      const float bm = warp_max(m2);
      s2 = (m2 == -INFINITY) ? 0.f : s2 * __expf(m2 - bm);
      s2 = warp_sum(s2);
      if (lane == 0) {
        const long lab = labels[t];
        float tgt = 0.f;
        if (lab >= vocab_start && lab < vocab_start + V) tgt = row[lab - vocab_start];
        stats[t * 3 + 0] = bm;
        stats[t * 3 + 1] = s2;
        stats[t * 3 + 2] = tgt;
      }
    }
  }
}

// stats_all: [R, T, 3] statistics of all R vocabulary slices (R = 1 without tensor parallelism).
// loss[t] = lse - target (0 for ignored labels < 0); dlogits = (softmax - onehot) * grad_scale.
__global__ void __launch_bounds__(kCEThreads)
ce_grad_kernel(const float* __restrict__ logits, long ld, const long* __restrict__ labels, int vocab_start,
               int V, const float* __restrict__ stats_all, int R, long T, float grad_scale,
               __nv_bfloat16* __restrict__ dlogits, long ld_d, float* __restrict__ loss) {
  for (long t = blockIdx.x; t < T; t += gridDim.x) {
    float gm = -INFINITY;
    for (int r = 0; r < R; ++r) gm = fmaxf(gm, stats_all[((long)r * T + t) * 3]);
    float gs = 0.f, tgt = 0.f;
    for (int r = 0; r < R; ++r) {
      const float* st = stats_all + ((long)r * T + t) * 3;
      gs += st[1] * __expf(st[0] - gm);
      tgt += st[2];
    }
    const long lab = labels[t];
    const bool ignore = lab < 0;
    const float lse = gm + __logf(gs);
    if (threadIdx.x == 0 && loss != nullptr) loss[t] = ignore ? 0.f : (lse - tgt);
    const float* row = logits + t * ld;
    __nv_bfloat16* drow = dlogits + t * ld_d;
    const float sc = ignore ? 0.f : grad_scale;
    const long local = lab - vocab_start;
    for (int i = threadIdx.x * 4; i < V; i += kCEThreads * 4) {
      const float4 x = *reinterpret_cast<const float4*>(row + i);
      float g0 = __expf(x.x - lse), g1 = __expf(x.y - lse), g2 = __expf(x.z - lse), g3 = __expf(x.w - lse);
      if (local >= i && local < i + 4) {
        if (local == i) g0 -= 1.f;
        else if (local == i + 1) g1 -= 1.f;
        else if (local == i + 2) g2 -= 1.f;
        else g3 -= 1.f;
      }
      uint2 u;
      u.x = pack_bf16x2(g0 * sc, g1 * sc);
      u.y = pack_bf16x2(g2 * sc, g3 * sc);
      *reinterpret_cast<uint2*>(drow + i) = u;
    }
  }
}

// out[t, :] = table[ids[t] - vocab_start, :] or 0 when the id belongs to another rank's slice
__global__ void embedding_fwd_kernel(const long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long T, int H, int vocab_start, int V) {
  const int nvec = H / 8;
  for (long t = blockIdx.x; t < T; t += gridDim.x) {
    const long id = ids[t] - vocab_start;
    const bool ok = id >= 0 && id < V;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      uint4 val = make_uint4(0, 0, 0, 0);
      if (ok) val = *reinterpret_cast<const uint4*>(table + id * H + v * 8);
      *reinterpret_cast<uint4*>(out + t * H + v * 8) = val;
    }
  }
}

// Tokens sorted by id: one CTA per run of equal ids sums the run's gradient rows in fp32 and
// adds the result to the table gradient (deterministic, no atomics).
template <typename GradT>
__global__ void embedding_bwd_kernel(const long* __restrict__ sorted_ids, const long* __restrict__ order,
                                     const __nv_bfloat16* __restrict__ dout, GradT* __restrict__ dtable, long T,
                                     int H, int vocab_start, int V, int accumulate) {
  for (long i = blockIdx.x; i < T; i += gridDim.x) {
    const long id = sorted_ids[i];
    if (i > 0 && sorted_ids[i - 1] == id) continue;  // not a run start
    const long local = id - vocab_start;
    if (local < 0 || local >= V) continue;
    long end = i + 1;
    while (end < T && sorted_ids[end] == id) ++end;
    for (int c = threadIdx.x * 2; c < H; c += blockDim.x * 2) {
      float a0 = 0.f, a1 = 0.f;
      for (long j = i; j < end; ++j) {
        const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dout + order[j] * H + c));
        a0 += v.x;
        a1 += v.y;
      }
      GradT* d = dtable + local * H + c;
      if (accumulate) {
        a0 += (float)d[0];
        a1 += (float)d[1];
      }
      d[0] = (GradT)a0;
      d[1] = (GradT)a1;
    }
  }
}

// sumsq[0] += sum(g^2)   (one atomic per CTA)
template <typename GradT>
__global__ void sumsq_kernel(const GradT* __restrict__ g, long n, float* __restrict__ sumsq) {
  __shared__ float sh[32];
  float s = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float v = (float)g[i];
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(sumsq, t);
  }
}

// AdamW on a flat shard. master = (param_bf16 << 16) + lo16 exactly.
// gscale_ptr[0] (device) multiplies the gradient (gradient clipping / loss scale), may be null.
template <typename GradT>
__global__ void adam_kernel(__nv_bfloat16* __restrict__ param, short* __restrict__ lo16,
                            const GradT* __restrict__ grad, float* __restrict__ m, float* __restrict__ v,
                            long n, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                            float bc2, const float* __restrict__ gscale_ptr,
                            const unsigned int* __restrict__ status) {
  // a step in which some kernel reported a failed wait or bounds check must not touch the weights
  if (status != nullptr && *status != 0u) return;
  const float gs = gscale_ptr != nullptr ? gscale_ptr[0] : 1.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const uint32_t hi = (uint32_t)__bfloat16_as_ushort(param[i]) << 16;
    const int32_t bits = (int32_t)hi + (int32_t)lo16[i];
    float w = __int_as_float(bits);
    const float g = (float)grad[i] * gs;
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * w;
    w -= lr * upd;
    const int32_t nb = __float_as_int(w);
    // round half up on the magnitude bits so that the remainder always fits a signed 16-bit field
    const int32_t nhi = (nb + 0x8000) & (int32_t)0xFFFF0000;
    param[i] = __ushort_as_bfloat16((unsigned short)((uint32_t)nhi >> 16));
    lo16[i] = (short)(nb - nhi);
  }
}

// AdamW on a flat shard of bf16 gradients, 8 elements per thread, fused with the parameter
// all-gather: the updated bf16 parameters are stored into the flat parameter buffer of EVERY
// data-parallel peer at element offset `lo` (peer_param[p] may be a peer mapping over NVLink), so no
// separate collective is needed after the update. param/lo16/grad/m/v point at the shard itself.
template <typename GradT>
__global__ void __launch_bounds__(256)
adam_push_kernel(const __nv_bfloat16* __restrict__ param, short* __restrict__ lo16,
                 const GradT* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, long n,
                 float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                 const float* __restrict__ gscale_ptr, const unsigned long long* __restrict__ peer_param,
                 int n_peers, long lo, const unsigned int* __restrict__ status) {
  if (status != nullptr && *status != 0u) return;   // see adam_kernel
  const float gs = gscale_ptr != nullptr ? gscale_ptr[0] : 1.f;
  const long nvec = n / 8;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const uint4 pu = *reinterpret_cast<const uint4*>(param + i * 8);
    const uint4 lu = *reinterpret_cast<const uint4*>(lo16 + i * 8);
    float gq8[8];
    if constexpr (sizeof(GradT) == 4) {
      const float4 g0 = *reinterpret_cast<const float4*>(grad + i * 8), g1 = *reinterpret_cast<const float4*>(grad + i * 8 + 4);
      gq8[0] = g0.x; gq8[1] = g0.y; gq8[2] = g0.z; gq8[3] = g0.w; gq8[4] = g1.x; gq8[5] = g1.y; gq8[6] = g1.z; gq8[7] = g1.w;
    } else {
      const uint4 gu = *reinterpret_cast<const uint4*>(grad + i * 8);
      const float2 a = unpack_bf16x2(gu.x), b = unpack_bf16x2(gu.y), c = unpack_bf16x2(gu.z), d = unpack_bf16x2(gu.w);
      gq8[0] = a.x; gq8[1] = a.y; gq8[2] = b.x; gq8[3] = b.y; gq8[4] = c.x; gq8[5] = c.y; gq8[6] = d.x; gq8[7] = d.y;
    }
    float4 m0 = *reinterpret_cast<const float4*>(m + i * 8), m1 = *reinterpret_cast<const float4*>(m + i * 8 + 4);
    float4 v0 = *reinterpret_cast<const float4*>(v + i * 8), v1 = *reinterpret_cast<const float4*>(v + i * 8 + 4);
    const uint32_t pw[4] = {pu.x, pu.y, pu.z, pu.w}, lw[4] = {lu.x, lu.y, lu.z, lu.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t po[4], lo_out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gq[2] = {gq8[2 * j] * gs, gq8[2 * j + 1] * gs};
      uint32_t hi_out[2], rem_out[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t hi = (h == 0 ? (pw[j] & 0xFFFFu) : (pw[j] >> 16)) << 16;
        const int32_t rem = (int32_t)(short)(h == 0 ? (lw[j] & 0xFFFFu) : (lw[j] >> 16));
        float w = __int_as_float((int32_t)hi + rem);
        const int k = 2 * j + h;
        mm[k] = beta1 * mm[k] + (1.f - beta1) * gq[h];
        vv[k] = beta2 * vv[k] + (1.f - beta2) * gq[h] * gq[h];
        w -= lr * ((mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps) + wd * w);
        const int32_t nb = __float_as_int(w);
        const int32_t nhi = (nb + 0x8000) & (int32_t)0xFFFF0000;
        hi_out[h] = (uint32_t)nhi >> 16;
        rem_out[h] = (uint32_t)(nb - nhi) & 0xFFFFu;
      }
      po[j] = hi_out[0] | (hi_out[1] << 16);
      lo_out[j] = rem_out[0] | (rem_out[1] << 16);
    }
    *reinterpret_cast<float4*>(m + i * 8) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(m + i * 8 + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    *reinterpret_cast<float4*>(v + i * 8) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(v + i * 8 + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    *reinterpret_cast<uint4*>(lo16 + i * 8) = make_uint4(lo_out[0], lo_out[1], lo_out[2], lo_out[3]);
    const uint4 pnew = make_uint4(po[0], po[1], po[2], po[3]);
    for (int p = 0; p < n_peers; ++p)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_param[p]) + lo + i * 8) = pnew;
  }
}

// lo16 = 0 means master == bf16 value exactly; used at init. (memset does the same job.)

inline int grid_for(long n, int threads) {
  long b = (n + threads - 1) / threads;
  const long cap = (long)sm_count() * 16;
  if (b > cap) b = cap;
  return (int)(b > 0 ? b : 1);
}

}  // namespace lo
}  // namespace dca

using namespace dca;
using namespace dca::lo;

extern "C" int dca_ce_stats(const float* logits, long ld, const long* labels, int vocab_start, int V,
                            float* stats, long T, void* stream) {
  if (T <= 0) return 0;
  if (V % 4 != 0 || ld % 4 != 0) return kErrBadArg;
  const long cap = (long)sm_count() * 4;
  ce_stats_kernel<<<(int)(T < cap ? T : cap), kCEThreads, 0, (cudaStream_t)stream>>>(logits, ld, labels, vocab_start, V, stats, T);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_ce_grad(const float* logits, long ld, const long* labels, int vocab_start, int V,
                           const float* stats_all, int R, long T, float grad_scale, void* dlogits, long ld_d,
                           float* loss, void* stream) {
  if (T <= 0) return 0;
  if (V % 4 != 0 || ld % 4 != 0 || ld_d % 4 != 0) return kErrBadArg;
  const long cap = (long)sm_count() * 4;
  ce_grad_kernel<<<(int)(T < cap ? T : cap), kCEThreads, 0, (cudaStream_t)stream>>>(
      logits, ld, labels, vocab_start, V, stats_all, R, T, grad_scale, (__nv_bfloat16*)dlogits, ld_d, loss);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_embedding_fwd(const long* ids, const void* table, void* out, long T, int H, int vocab_start,
                                 int V, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return kErrBadArg;
  const long cap = (long)sm_count() * 8;
  embedding_fwd_kernel<<<(int)(T < cap ? T : cap), 128, 0, (cudaStream_t)stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, vocab_start, V);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_embedding_bwd(const long* sorted_ids, const long* order, const void* dout, void* dtable,
                                 int dtable_fp32, int accumulate, long T, int H, int vocab_start, int V,
                                 void* stream) {
  if (T <= 0) return 0;
  if (H % 2 != 0) return kErrBadArg;
  const long cap = (long)sm_count() * 16;
  const int grid = (int)(T < cap ? T : cap);
  if (dtable_fp32)
    embedding_bwd_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(sorted_ids, order, (const __nv_bfloat16*)dout, (float*)dtable, T, H, vocab_start, V, accumulate);
  else
    embedding_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(sorted_ids, order, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dtable, T, H, vocab_start, V, accumulate);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_sumsq(const void* g, int g_fp32, long n, float* sumsq, void* stream) {
  if (n <= 0) return 0;
  if (g_fp32)
    sumsq_kernel<float><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const float*)g, n, sumsq);
  else
    sumsq_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, n, sumsq);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

// `status` (may be null): the device status word; when it is non-zero the update is skipped, so a step whose
// kernels reported a failed wait or bounds check leaves the weights and the optimizer state as they were.
// AdamW + parameter all-gather in one kernel (bf16 or fp32 gradients: g_fp32). param/lo16/grad/m/v: this rank's
// shard (n elements, multiple of 8); peer_param: device array of n_peers addresses of the peers'
// (and this rank's own) flat parameter buffers; lo: element offset of the shard in those buffers.
extern "C" int dca_adam_push(const void* param, void* lo16, const void* grad, int g_fp32, float* m, float* v, long n, float lr,
                             float beta1, float beta2, float eps, float wd, int step, const float* gscale_ptr,
                             const void* peer_param, int n_peers, long lo, const unsigned int* status,
                             void* stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || lo % 8 != 0) return kErrBadArg;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  if (g_fp32)
    adam_push_kernel<float><<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)param, (short*)lo16, (const float*)grad, m, v, n, lr, beta1, beta2, eps, wd, bc1,
        bc2, gscale_ptr, (const unsigned long long*)peer_param, n_peers, lo, status);
  else
    adam_push_kernel<__nv_bfloat16><<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)param, (short*)lo16, (const __nv_bfloat16*)grad, m, v, n, lr, beta1, beta2, eps, wd, bc1,
        bc2, gscale_ptr, (const unsigned long long*)peer_param, n_peers, lo, status);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

extern "C" int dca_adam(void* param, void* lo16, const void* grad, int g_fp32, float* m, float* v, long n,
                        float lr, float beta1, float beta2, float eps, float wd, int step,
                        const float* gscale_ptr, const unsigned int* status, void* stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = 1.f - powf(beta2, (float)step);
  if (g_fp32)
    adam_kernel<float><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)param, (short*)lo16, (const float*)grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, gscale_ptr, status);
  else
    adam_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)param, (short*)lo16, (const __nv_bfloat16*)grad, m, v, n, lr, beta1, beta2, eps, wd, bc1, bc2, gscale_ptr, status);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
