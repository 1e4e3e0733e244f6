// Peer-memory substrate of the CAD runtime: arena allocation + CUDA IPC handles, monotonic
// system-scope signals with bounded waits, row scatter over NVLink, and the owner-side sum of
// K/V-gradient copies.
//
// Every GPU allocates one arena with cudaMalloc and maps every peer's arena with CUDA IPC; kernels
// then store rows straight into the destination GPU's arena (plain 16-byte st.global over NVLink,
// many CTAs) and bump a 64-bit counter there with a release at system scope. Counters only grow;
// a consumer waits for `counter >= expected` with an iteration limit and reports through the
// status word instead of spinning forever.
//
// Counterparts in the reference: NVSHMEM symmetric buffers and the put+signal all-to-all
// (csrc/core/fastalltoall.cu:14-138, fastalltoall.h:56-93), pack/unpack memcpy kernels
// (csrc/core/memcpy.cu:23-155) and the in-place KV-grad sum (memcpy.cu:159-236).
#include "../common/host_utils.h"
#include "../common/ptx.cuh"

namespace dca {
namespace p2p {

// signals[i] += 1 on peer i (addresses may point into peer arenas). One thread per peer.
__global__ void signal_peers_kernel(const unsigned long long* __restrict__ addrs, int n) {
  const int i = threadIdx.x;
  if (i < n && addrs[i] != 0ull) {
    __threadfence_system();
    signal_add_release_sys(reinterpret_cast<unsigned long long*>(addrs[i]), 1ull);
  }
}

// wait until slots[i] >= target for all i < n (slots live in this GPU's arena)
__global__ void wait_signals_kernel(const unsigned long long* __restrict__ slots, int n,
                                    unsigned long long target, unsigned int* status, unsigned int max_polls) {
  const int i = threadIdx.x;
  if (i < n) signal_wait_ge(slots + i, target, status, max_polls);
}

// Row scatter: row r of `src` (row_bytes bytes, pitch src_pitch) -> dst_addr[r] + dst_off, skipped
// when dst_addr[r] == 0. One warp per row, 16 bytes per lane per step.
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const uint8_t* __restrict__ src, long src_pitch, int row_bytes,
                    const unsigned long long* __restrict__ dst_addr, long dst_off, long n_rows) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long r = (long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < n_rows;
       r += (long)gridDim.x * warps_per_block) {
    const unsigned long long d = dst_addr[r];
    if (d == 0ull) continue;
    const uint4* s4 = reinterpret_cast<const uint4*>(src + r * src_pitch);
    uint4* d4 = reinterpret_cast<uint4*>(d + dst_off);
    for (int v = lane; v < row_bytes / 16; v += 32) d4[v] = s4[v];
  }
}

// Row gather (pull): row r of dst <- src_addr[r] (+ src_off). Used where pulling is preferable.
__global__ void __launch_bounds__(256)
gather_rows_kernel(uint8_t* __restrict__ dst, long dst_pitch, int row_bytes,
                   const unsigned long long* __restrict__ src_addr, long src_off, long n_rows) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long r = (long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < n_rows;
       r += (long)gridDim.x * warps_per_block) {
    const unsigned long long s = src_addr[r];
    if (s == 0ull) continue;
    const uint4* s4 = reinterpret_cast<const uint4*>(s + src_off);
    uint4* d4 = reinterpret_cast<uint4*>(dst + r * dst_pitch);
    for (int v = lane; v < row_bytes / 16; v += 32) d4[v] = s4[v];
  }
}

// out[t, :] = sum over copies c with valid[t, c] >= 0 of slots[c, t, :]   (bf16 rows, fp32 sum)
__global__ void __launch_bounds__(256)
sum_slots_kernel(const __nv_bfloat16* __restrict__ slots, long slot_stride, int row_elems,
                 const int* __restrict__ valid, int copies, __nv_bfloat16* __restrict__ out, long out_pitch,
                 long T) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long t = (long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T;
       t += (long)gridDim.x * warps_per_block) {
    for (int v = lane; v < row_elems / 8; v += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int c = 0; c < copies; ++c) {
        if (valid[t * copies + c] < 0) break;
        const uint4 u = *reinterpret_cast<const uint4*>(slots + c * slot_stride + t * row_elems + v * 8);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + t * out_pitch + v * 8) = o;
    }
  }
}

// Gradient reduce-scatter over peer memory: out[i] = scale * sum_p peer_p[lo + i]  (fp32 sum)
template <typename T>
__global__ void __launch_bounds__(256)
reduce_peers_kernel(const unsigned long long* __restrict__ peer_base, int n_peers, long lo_elems, long n,
                    float scale, T* __restrict__ out);

template <>
__global__ void __launch_bounds__(256)
reduce_peers_kernel<__nv_bfloat16>(const unsigned long long* __restrict__ peer_base, int n_peers, long lo_elems,
                                   long n, float scale, __nv_bfloat16* __restrict__ out) {
  const long nvec = n / 8;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < n_peers; ++p) {
      const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peer_base[p]) + lo_elems + i * 8);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0] * scale, acc[1] * scale); o.y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
    o.z = pack_bf16x2(acc[4] * scale, acc[5] * scale); o.w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}

// Data-parallel gradient reduce-scatter fused with the gradient-norm partial sum:
//   own[lo + i] = sum_p peer_p[lo + i]   (fp32 accumulation, written back in place as bf16)
//   sumsq[0]   += sum_i (that sum)^2
// Peers only read the slices of this rank's buffer that belong to THEIR shard, so writing the own
// slice in place does not race with them.
__global__ void __launch_bounds__(256)
reduce_scatter_sumsq_bf16_kernel(const unsigned long long* __restrict__ peer_base, int n_peers, int self,
                                 long lo_elems, long n, float* __restrict__ sumsq) {
  __shared__ float sh[8];
  const long nvec = n / 8;
  float ss = 0.f;
  __nv_bfloat16* own = reinterpret_cast<__nv_bfloat16*>(peer_base[self]) + lo_elems;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < n_peers; ++p) {
      const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peer_base[p]) + lo_elems + i * 8);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += acc[j] * acc[j];
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(own + i * 8) = o;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = sh[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) atomicAdd(sumsq, t);
  }
}

// Same for fp32 gradient buffers (several micro-batches accumulate in fp32; the reference reduces its
// gradients in fp32 as well, distca/utils/megatron_test_utils.py:237-241): 4 elements per thread and access.
__global__ void __launch_bounds__(256)
reduce_scatter_sumsq_f32_kernel(const unsigned long long* __restrict__ peer_base, int n_peers, int self,
                                long lo_elems, long n, float* __restrict__ sumsq) {
  __shared__ float sh[8];
  const long nvec = n / 4;
  float ss = 0.f;
  float* own = reinterpret_cast<float*>(peer_base[self]) + lo_elems;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < n_peers; ++p) {
      const float4 u = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peer_base[p]) + lo_elems + i * 4);
      acc.x += u.x; acc.y += u.y; acc.z += u.z; acc.w += u.w;
    }
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    *reinterpret_cast<float4*>(own + i * 4) = acc;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = sh[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) atomicAdd(sumsq, t);
  }
}

// Parameter all-gather over peer memory: every rank pushes its shard into every peer's flat buffer.
__global__ void __launch_bounds__(256)
push_shard_kernel(const uint4* __restrict__ src, const unsigned long long* __restrict__ peer_base, int n_peers,
                  int self, long lo_vec, long nvec) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int p = 0; p < n_peers; ++p) {
      if (p == self) continue;
      reinterpret_cast<uint4*>(peer_base[p])[lo_vec + i] = v;
    }
  }
}

}  // namespace p2p
}  // namespace dca

using namespace dca;

extern "C" int dca_arena_alloc(void** out, size_t bytes) {
  DCA_CUDA_TRY(cudaMalloc(out, bytes));
  DCA_CUDA_TRY(cudaMemset(*out, 0, bytes));
  return 0;
}
extern "C" int dca_arena_free(void* p) {
  DCA_CUDA_TRY(cudaFree(p));
  return 0;
}
// handle_out: 64 bytes
extern "C" int dca_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  DCA_CUDA_TRY(cudaIpcGetMemHandle(&h, p));
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int dca_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  DCA_CUDA_TRY(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
extern "C" int dca_ipc_close(void* p) {
  DCA_CUDA_TRY(cudaIpcCloseMemHandle(p));
  return 0;
}

extern "C" int dca_signal_peers(const void* addrs, int n, void* stream) {
  if (n <= 0) return 0;
  if (n > 1024) return kErrTooLarge;
  p2p::signal_peers_kernel<<<1, ((n + 31) / 32) * 32, 0, (cudaStream_t)stream>>>((const unsigned long long*)addrs, n);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
// max_polls = 0: default limit (about a minute: ranks may legitimately drift by seconds, e.g. while one
// page-locks host memory); a poll is one acquire load plus a 200 ns sleep
extern "C" int dca_wait_signals(const void* slots, int n, unsigned long long target, unsigned int* status,
                                unsigned int max_polls, void* stream) {
  if (n <= 0) return 0;
  if (n > 1024) return kErrTooLarge;
  if (max_polls == 0) max_polls = dca::kSpinLimit << 4;
  p2p::wait_signals_kernel<<<1, ((n + 31) / 32) * 32, 0, (cudaStream_t)stream>>>((const unsigned long long*)slots, n, target, status, max_polls);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
extern "C" int dca_scatter_rows(const void* src, long src_pitch, int row_bytes, const void* dst_addr, long dst_off,
                                long n_rows, int max_ctas, void* stream) {
  if (n_rows <= 0) return 0;
  if (row_bytes % 16 != 0 || src_pitch % 16 != 0 || dst_off % 16 != 0) return kErrBadArg;
  long blocks = (n_rows + 7) / 8;
  const long cap = max_ctas > 0 ? max_ctas : (long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  p2p::scatter_rows_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, src_pitch, row_bytes,
                                                                           (const unsigned long long*)dst_addr, dst_off, n_rows);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
extern "C" int dca_gather_rows(void* dst, long dst_pitch, int row_bytes, const void* src_addr, long src_off,
                               long n_rows, int max_ctas, void* stream) {
  if (n_rows <= 0) return 0;
  if (row_bytes % 16 != 0 || dst_pitch % 16 != 0 || src_off % 16 != 0) return kErrBadArg;
  long blocks = (n_rows + 7) / 8;
  const long cap = max_ctas > 0 ? max_ctas : (long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  p2p::gather_rows_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((uint8_t*)dst, dst_pitch, row_bytes,
                                                                          (const unsigned long long*)src_addr, src_off, n_rows);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
extern "C" int dca_sum_slots(const void* slots, long slot_stride_elems, int row_elems, const int* valid, int copies,
                             void* out, long out_pitch_elems, long T, void* stream) {
  if (T <= 0) return 0;
  if (row_elems % 8 != 0 || out_pitch_elems % 8 != 0) return kErrBadArg;
  long blocks = (T + 7) / 8;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  p2p::sum_slots_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)slots, slot_stride_elems, row_elems,
                                                                       valid, copies, (__nv_bfloat16*)out, out_pitch_elems, T);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
// out[i] = scale * sum over peers of peer[lo + i], i < n (bf16, n multiple of 8)
extern "C" int dca_reduce_peers_bf16(const void* peer_base, int n_peers, long lo_elems, long n, float scale, void* out,
                                     void* stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || lo_elems % 8 != 0) return kErrBadArg;
  long blocks = (n / 8 + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  p2p::reduce_peers_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const unsigned long long*)peer_base, n_peers, lo_elems, n, scale, (__nv_bfloat16*)out);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
// In-place reduce-scatter of bf16 gradient buffers that live in peer-mapped memory, plus
// sumsq[0] += || reduced shard ||^2. peer_base: device array of n_peers buffer addresses.
extern "C" int dca_reduce_scatter_sumsq_bf16(const void* peer_base, int n_peers, int self, long lo_elems, long n,
                                             float* sumsq, void* stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || lo_elems % 8 != 0) return kErrBadArg;
  long blocks = (n / 8 + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  p2p::reduce_scatter_sumsq_bf16_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const unsigned long long*)peer_base, n_peers, self, lo_elems, n, sumsq);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
// fp32 twin of dca_reduce_scatter_sumsq_bf16 (n and lo_elems multiples of 4).
extern "C" int dca_reduce_scatter_sumsq_f32(const void* peer_base, int n_peers, int self, long lo_elems, long n,
                                            float* sumsq, void* stream) {
  if (n <= 0) return 0;
  if (n % 4 != 0 || lo_elems % 4 != 0) return kErrBadArg;
  long blocks = (n / 4 + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  p2p::reduce_scatter_sumsq_f32_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const unsigned long long*)peer_base, n_peers, self, lo_elems, n, sumsq);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
extern "C" int dca_push_shard(const void* src, const void* peer_base, int n_peers, int self, long lo_bytes, long bytes,
                              void* stream) {
  if (bytes <= 0) return 0;
  if (bytes % 16 != 0 || lo_bytes % 16 != 0) return kErrBadArg;
  long blocks = (bytes / 16 + 255) / 256;
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  p2p::push_shard_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (const unsigned long long*)peer_base,
                                                                        n_peers, self, lo_bytes / 16, bytes / 16);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
