// Rotary position embedding on the fused QKV activation, with a per-token position so that the
// head and tail shards of a document that was split across ranks get the angles of their place in
// the document, not of their place in the rank's buffer.
//
// The same kernel optionally scatters the rotated Q rows and the K / V rows to per-token
// destinations (addresses that may be peer-GPU mappings): this is the "dispatch fused into RoPE"
// half of the core-attention dispatch. Each token carries up to `max_copies` K/V destinations
// because a K/V row is needed on every attention server that runs a later shard of its document.
//
// Layout: qkv [T, (Hq + 2*Hkv) * D] bf16, Q heads first, then K heads, then V heads; rotation
// pairs are (i, i + D/2) ("rotate half", the Llama / Megatron non-interleaved convention).
// cos_sin: fp32 [max_pos, D] = (cos[0..D/2) | sin[0..D/2)).
//
// Counterpart in the reference: distca/runtime/megatron/distca_rope.py:10-68 (index gather +
// unfused torch rotation) followed by the pack kernels of csrc/core/memcpy.cu:23-155.
#include "../common/host_utils.h"
#include "../common/ptx.cuh"

namespace dca {
namespace rope {

struct RopeParams {
  __nv_bfloat16* qkv;        // in place when no destinations are given
  const int* pos;            // [T] position of each token inside its document
  const float* cos_sin;      // [max_pos, D]
  int max_pos;               // rows of cos_sin; a position beyond it is clamped and reported in the status word
  unsigned int* status;
  long T;
  int heads_q, heads_kv, D;
  long ld;                   // row pitch of qkv in elements
  float sign;                // +1 forward, -1 backward (rotation by the negative angle)
  // optional scatter (all null => in-place only)
  const unsigned long long* q_dst;   // [T] address of the destination Q row (0 = keep local only)
  const unsigned long long* kv_dst;  // [T, max_copies] address of the destination K row; V row follows at +v_off
  int max_copies;
  long v_off_bytes;          // distance from a destination K row to its V row
  int write_inplace;         // also store the rotated values back into qkv
};

__global__ void __launch_bounds__(256)
rope_kernel(const RopeParams p) {
  const int half = p.D / 2;
  const int vec_per_half = half / 8;                     // 16-byte vectors per half head
  const int rot_heads = p.heads_q + p.heads_kv;
  const int items_rot = rot_heads * vec_per_half;        // rotation work items per token
  const int v_vecs = p.heads_kv * p.D / 8;               // plain-copy vectors of V per token
  const bool scatter = p.q_dst != nullptr;
  const int items = items_rot + (scatter ? v_vecs : 0);
  for (long t = blockIdx.x; t < p.T; t += gridDim.x) {
    __nv_bfloat16* row = p.qkv + t * p.ld;
    int ps = p.pos[t];
    if (ps < 0 || ps >= p.max_pos) {
      // never read past the table: rotate by the last row and report (the host raises on the status word)
      if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0u, (unsigned int)kStatusBounds);
      ps = ps < 0 ? 0 : p.max_pos - 1;
    }
    const float* cs = p.cos_sin + (long)ps * p.D;
    const unsigned long long qd = scatter ? p.q_dst[t] : 0ull;
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      if (it < items_rot) {
        const int h = it / vec_per_half;
        const int i0 = (it % vec_per_half) * 8;
        __nv_bfloat16* x1p = row + h * p.D + i0;
        __nv_bfloat16* x2p = x1p + half;
        const uint4 a = *reinterpret_cast<const uint4*>(x1p);
        const uint4 b = *reinterpret_cast<const uint4*>(x2p);
        const float4 c0 = *reinterpret_cast<const float4*>(cs + i0);
        const float4 c1 = *reinterpret_cast<const float4*>(cs + i0 + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(cs + half + i0);
        const float4 s1 = *reinterpret_cast<const float4*>(cs + half + i0 + 4);
        const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const uint32_t au[4] = {a.x, a.y, a.z, a.w}, bu[4] = {b.x, b.y, b.z, b.w};
        uint32_t o1[4], o2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 x1 = unpack_bf16x2(au[j]), x2 = unpack_bf16x2(bu[j]);
          const float sa = ss[2 * j] * p.sign, sb = ss[2 * j + 1] * p.sign;
          o1[j] = pack_bf16x2(x1.x * cc[2 * j] - x2.x * sa, x1.y * cc[2 * j + 1] - x2.y * sb);
          o2[j] = pack_bf16x2(x2.x * cc[2 * j] + x1.x * sa, x2.y * cc[2 * j + 1] + x1.y * sb);
        }
        const uint4 r1 = make_uint4(o1[0], o1[1], o1[2], o1[3]);
        const uint4 r2 = make_uint4(o2[0], o2[1], o2[2], o2[3]);
        if (!scatter || p.write_inplace) {
          *reinterpret_cast<uint4*>(x1p) = r1;
          *reinterpret_cast<uint4*>(x2p) = r2;
        }
        if (scatter) {
          if (h < p.heads_q) {
            if (qd != 0ull) {
              uint8_t* d = reinterpret_cast<uint8_t*>(qd) + ((long)h * p.D + i0) * 2;
              *reinterpret_cast<uint4*>(d) = r1;
              *reinterpret_cast<uint4*>(d + half * 2) = r2;
            }
          } else {
            const int hk = h - p.heads_q;
            for (int c = 0; c < p.max_copies; ++c) {
              const unsigned long long kd = p.kv_dst[t * p.max_copies + c];
              if (kd == 0ull) break;
              uint8_t* d = reinterpret_cast<uint8_t*>(kd) + ((long)hk * p.D + i0) * 2;
              *reinterpret_cast<uint4*>(d) = r1;
              *reinterpret_cast<uint4*>(d + half * 2) = r2;
            }
          }
        }
      } else {
        // V rows travel unrotated
        const int vi = it - items_rot;
        const uint4 val = *reinterpret_cast<const uint4*>(row + (long)rot_heads * p.D + vi * 8);
        for (int c = 0; c < p.max_copies; ++c) {
          const unsigned long long kd = p.kv_dst[t * p.max_copies + c];
          if (kd == 0ull) break;
          *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(kd) + p.v_off_bytes + (long)vi * 16) = val;
        }
      }
    }
  }
}

}  // namespace rope
}  // namespace dca

using namespace dca;

extern "C" int dca_rope(void* qkv, const int* pos, const float* cos_sin, int max_pos, long T, int heads_q,
                        int heads_kv, int D, long ld, int backward, const void* q_dst, const void* kv_dst,
                        int max_copies, long v_off_bytes, int write_inplace, unsigned int* status, void* stream) {
  if (T <= 0) return 0;
  if (D % 16 != 0 || ld % 8 != 0 || max_pos <= 0) return kErrBadArg;
  rope::RopeParams p;
  p.qkv = (__nv_bfloat16*)qkv;
  p.pos = pos;
  p.cos_sin = cos_sin;
  p.max_pos = max_pos;
  p.status = status;
  p.T = T;
  p.heads_q = heads_q; p.heads_kv = heads_kv; p.D = D; p.ld = ld;
  p.sign = backward ? -1.f : 1.f;
  p.q_dst = (const unsigned long long*)q_dst;
  p.kv_dst = (const unsigned long long*)kv_dst;
  p.max_copies = max_copies;
  p.v_off_bytes = v_off_bytes;
  p.write_inplace = write_inplace;
  const long cap = (long)sm_count() * 8;
  const int grid = (int)(T < cap ? T : cap);
  rope::rope_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}
