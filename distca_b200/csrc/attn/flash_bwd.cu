// Host side of the core-attention backward plus its small helper kernels. The backward runs as
// two tensor-core kernels: a key-centred one for dK/dV (flash_bwd_dkdv.cuh) and a query-centred
// one for dQ (flash_bwd_dq.cuh). Both accumulate in TMEM and store each output element exactly
// once, so there are no atomics and the gradients are bit-reproducible. The helpers compute the
// per-row statistics (delta = rowsum(dO o O), log-sum-exp in log2 units, transposed to [head, token]).
//
// Counterpart in the reference: flash-attn 2 varlen backward + in-place KV-grad dedup sum
// (distca/runtime/megatron/ops/fused_comm_attn.py:204-279, csrc/core/memcpy.cu:159-236).
#include "flash_bwd_dkdv.cuh"
#include "flash_bwd_dq.cuh"

namespace dca {
namespace attn {

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d];  lse2[h, t] = lse[t, h] * log2(e)
__global__ void bwd_preprocess_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                      const float* __restrict__ lse, float* __restrict__ delta,
                                      float* __restrict__ lse2, long Tq, int heads, long ld_o, long ld_do,
                                      long ld_lse) {
  // one warp per (token, head): 128 elements = 32 lanes x 4
  const long gw = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= Tq * heads) return;
  const long t = gw / heads;
  const int h = (int)(gw % heads);
  const uint2 a = *reinterpret_cast<const uint2*>(o + t * ld_o + h * kBD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + t * ld_do + h * kBD + lane * 4);
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y);
  const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    delta[(long)h * Tq + t] = s;
    lse2[(long)h * Tq + t] = lse[t * ld_lse + h] * 1.4426950408889634f;
  }
}

// Same statistics when delta arrives precomputed per token row (the token owner has both O and dO
// and ships 4 bytes per head instead of the whole O row): transposes [Tq, heads] -> [heads, Tq].
__global__ void bwd_transpose_stats_kernel(const float* __restrict__ delta_rows, long ld_delta,
                                           const float* __restrict__ lse, long ld_lse, float* __restrict__ delta,
                                           float* __restrict__ lse2, long Tq, int heads) {
  const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  if (i >= Tq * heads) return;
  const long t = i / heads;
  const int h = (int)(i % heads);
  delta[(long)h * Tq + t] = delta_rows[t * ld_delta + h];
  lse2[(long)h * Tq + t] = lse[t * ld_lse + h] * 1.4426950408889634f;
}

// delta_rows[t, h] = sum_d dO[t,h,d] * O[t,h,d]   (row-major, for shipping with dO)
__global__ void delta_rows_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta_rows, long T, int heads, long ld_o, long ld_do,
                                  long ld_delta) {
  const long gw = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * heads) return;
  const long t = gw / heads;
  const int h = (int)(gw % heads);
  const uint2 a = *reinterpret_cast<const uint2*>(o + t * ld_o + h * kBD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + t * ld_do + h * kBD + lane * 4);
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y);
  const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta_rows[t * ld_delta + h] = s;
}

// Owner half of the backward dispatch in one pass: for every token row compute delta = rowsum(dO o O) per head
// and store the dO row, the delta row and the log-sum-exp row at that token's destinations on its attention
// server (addresses may be peer mappings: plain stores over NVLink). One warp per (token, head): 8 bytes per
// lane, 256 contiguous bytes per warp and store. A destination of 0 skips the token.
__global__ void dispatch_dout_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                     const float* __restrict__ lse, long T, int heads, long ld_o, long ld_do,
                                     long ld_lse, const unsigned long long* __restrict__ do_dst, long do_off_bytes,
                                     const unsigned long long* __restrict__ delta_dst,
                                     const unsigned long long* __restrict__ lse_dst) {
  const long gw = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * heads) return;
  const long t = gw / heads;
  const int h = (int)(gw % heads);
  const unsigned long long dd = do_dst[t];
  if (dd == 0ull) return;
  const uint2 a = *reinterpret_cast<const uint2*>(o + t * ld_o + h * kBD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + t * ld_do + h * kBD + lane * 4);
  *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(dd) + do_off_bytes + ((long)h * kBD + lane * 4) * 2) = b;
  const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y);
  const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    reinterpret_cast<float*>(delta_dst[t])[h] = s;
    reinterpret_cast<float*>(lse_dst[t])[h] = lse[t * ld_lse + h];
  }
}

}  // namespace attn
}  // namespace dca

using namespace dca;
using namespace dca::attn;

// dO, delta = rowsum(dO o O) and LSE rows of T tokens stored at per-token destinations (device uint64 tables
// do_dst / delta_dst / lse_dst [T]; the dO row goes to do_dst[t] + do_off_bytes). o / dout: bf16 [T, heads, 128]
// with row pitches ld_o / ld_do (elements); lse: fp32 [T, heads] with pitch ld_lse.
extern "C" int dca_dispatch_dout(const void* o, const void* dout, const float* lse, long T, int heads, int head_dim,
                                 long ld_o, long ld_do, long ld_lse, const void* do_dst, long do_off_bytes,
                                 const void* delta_dst, const void* lse_dst, void* stream) {
  if (T <= 0) return 0;
  if (head_dim != kBD || do_off_bytes % 8 != 0 || ld_o % 4 != 0 || ld_do % 4 != 0) return kErrBadArg;
  const long warps = T * heads;
  const long blocks = (warps * 32 + 255) / 256;
  dispatch_dout_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, T, heads, ld_o, ld_do, ld_lse,
      (const unsigned long long*)do_dst, do_off_bytes, (const unsigned long long*)delta_dst,
      (const unsigned long long*)lse_dst);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

// delta_rows (optional, fp32 [Tq, ld_delta_rows]): rowsum(dO o O) per token and head computed by the
// token owner; when given, `o` is not read.
// Scratch (caller-allocated): delta, lse2: fp32 [heads_q, Tq].
// kv_work / q_tiles: key-centred schedule (BwdKVWork / BwdQTile); fwd_work: the forward tile list
// (AttnWork; only its geometry fields are read). dq/dk/dv are bf16 with free row pitches (elements).
// Rows of dq/dk/dv that no task covers are not written. All of q/k/v/o/dout have inner layout
// [heads, 128]. Rows of q/k/v/dout that lie between tasks must hold finite values (a tile that
// straddles a task boundary reads them).
// dq_row_ptr [Tq] / dkv_row_ptr [Tk] (optional, device uint64): per-row destination addresses that replace
// dq / dk, dv (head 0 of the row; the dV row sits dv_off_bytes behind the dK row; 0 = do not store): the
// gradients are then stored straight to their owners, possibly on other GPUs, from the kernels' epilogues.
extern "C" int dca_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                             const float* lse, long Tq, long Tk, long ldq, long ldk, long ldv, long ldo,
                             long lddo, long ld_lse, int heads_q, int heads_kv, int head_dim,
                             const void* kv_work, int num_kv_work, const void* q_tiles, const void* fwd_work,
                             int num_fwd_work, float softmax_scale, float* delta, float* lse2, void* dq, long lddq,
                             void* dk, long lddk, void* dv, long lddv, const float* delta_rows,
                             long ld_delta_rows, const void* dq_row_ptr, const void* dkv_row_ptr, long dv_off_bytes,
                             unsigned int* status, void* stream) {
  if (head_dim != kBD || heads_q % heads_kv != 0) return kErrBadArg;
  if (Tq <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int cols = heads_q * kBD;
  if (delta_rows != nullptr) {
    const long n = Tq * heads_q;
    bwd_transpose_stats_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(delta_rows, ld_delta_rows, lse, ld_lse,
                                                                          delta, lse2, Tq, heads_q);
    DCA_CUDA_TRY(cudaGetLastError());
  } else {
    const long warps = Tq * heads_q;
    const long blocks = (warps * 32 + 255) / 256;
    bwd_preprocess_kernel<<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse,
                                                           delta, lse2, Tq, heads_q, ldo, lddo, ld_lse);
    DCA_CUDA_TRY(cudaGetLastError());
  }
  if (num_kv_work <= 0 && num_fwd_work <= 0) return 0;
  CUtensorMap tmQ, tmK, tmV, tmdO;
  int rc;
  if ((rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tq, (uint64_t)cols, ldq, kBT, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmdO, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tq, (uint64_t)cols, lddo, kBT, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, (uint64_t)heads_kv * kBD, ldk, kBT, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, Tk, (uint64_t)heads_kv * kBD, ldv, kBT, 64, true))) return rc;
  static bool configured = false;
  if (!configured) {
    DCA_CUDA_TRY(cudaFuncSetAttribute(flash_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDkdvSmem));
    DCA_CUDA_TRY(cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmem));
    configured = true;
  }
  if (num_kv_work > 0) {
    BwdParams p;
    p.kv_work = (const BwdKVWork*)kv_work;
    p.q_tiles = (const BwdQTile*)q_tiles;
    p.heads_q = heads_q; p.heads_kv = heads_kv;
    p.scale = softmax_scale;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.lse2 = lse2; p.delta = delta; p.Tq = Tq;
    p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
    p.ld_dk = lddk; p.ld_dv = lddv;
    p.dkv_row_ptr = (const unsigned long long*)dkv_row_ptr; p.dv_off_bytes = dv_off_bytes;
    p.status = status;
    dim3 grid(num_kv_work, heads_kv);
    flash_bwd_dkdv_kernel<<<grid, kBwdThreads, kDkdvSmem, s>>>(tmQ, tmK, tmV, tmdO, p);
    DCA_CUDA_TRY(cudaGetLastError());
  }
  if (num_fwd_work > 0) {
    DqParams p;
    p.work = (const AttnWork*)fwd_work;
    p.heads_q = heads_q; p.heads_kv = heads_kv;
    p.scale = softmax_scale;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.lse2 = lse2; p.delta = delta; p.Tq = Tq;
    p.dq = (__nv_bfloat16*)dq; p.ld_dq = lddq;
    p.dq_row_ptr = (const unsigned long long*)dq_row_ptr;
    p.status = status;
    dim3 grid(num_fwd_work, heads_q);
    flash_bwd_dq_kernel<<<grid, kDqThreads, kDqSmem, s>>>(tmQ, tmK, tmV, tmdO, p);
    DCA_CUDA_TRY(cudaGetLastError());
  }
  return 0;
}

// delta_rows[t, h] = sum_d dO[t,h,d] * O[t,h,d] for every token row (fp32, pitch ld_delta elements)
extern "C" int dca_attn_delta_rows(const void* o, const void* dout, float* delta_rows, long T, int heads,
                                   int head_dim, long ldo, long lddo, long ld_delta, void* stream) {
  if (T <= 0) return 0;
  if (head_dim != kBD) return kErrBadArg;
  const long warps = T * heads;
  const long blocks = (warps * 32 + 255) / 256;
  delta_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                                        delta_rows, T, heads, ldo, lddo, ld_delta);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
