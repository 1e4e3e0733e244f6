// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) ->
// tcgen05.mma (128x256x16, fp32 accumulators in TMEM, double-buffered) -> tcgen05.ld epilogue.
//
//   C[M,N] (+)= A[M,K] * B[N,K]^T          (both operands may be K-major or MN-major in memory)
//
// This one kernel covers every linear layer of the transformer:
//   forward  y  = x W^T          A = x  [T,K]  K-major,   B = W  [N,K] K-major
//   dgrad    dx = dy W           A = dy [T,N]  K-major,   B = W  [N,K] read as [K'=N, N'=K] MN-major
//   wgrad    dW = dy^T x         A = dy [T,N]  MN-major,  B = x  [T,K] MN-major  (contraction over T)
// plus an epilogue that applies SwiGLU to a (gate | up) accumulator pair so the FC1 output never
// makes a round trip through HBM in its un-activated form unless the caller asks for it, and one for
// the QKV projection that rotates the Q and K heads (RoPE at each token's position inside its
// document) while they are still fp32 accumulators and stores the rows straight to where core
// attention will read them: the local QKV buffer and / or per-token destinations in the attention
// servers' arenas (peer stores over NVLink), so the dispatch needs no pass of its own.
//
// Role layout of the 192-thread CTA: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (two warps per TMEM lane quarter, each takes half of the tile's columns, so a
// warp's TMEM-load / convert / store latencies are covered by its partner on the same scheduler).
// One CTA per SM, grid = min(tiles, SMs).
//
// Counterpart in the reference: TransformerEngine/cuBLASLt linears used by
// distca/runtime/megatron/model_patch.py:89-112 (the reference owns no GEMM).
#include "../common/host_utils.h"
#include "../common/ptx.cuh"

namespace dca {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int NUM_BARS = 2 * STAGES + 4;
constexpr int SMEM_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + NUM_BARS * 8 + 16 + 1024;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = (2 + EPI_WARPS) * 32;
constexpr int TMEM_COLS = 512;  // two 256-column accumulators

enum : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ROPE = 2 };

struct Params {
  int M, N, K;       // N is 2*F for EPI_SWIGLU
  void* C;           // [M, N] (EPI_STORE) or [M, F] (EPI_SWIGLU)
  long ldc;
  int out_fp32;      // EPI_STORE only
  int accumulate;    // C += result (EPI_STORE only)
  const void* residual;  // EPI_STORE, bf16 out: C = result + residual[M,N] (bf16, pitch ldr); may alias C
  long ldr;
  int epi;
  int F;             // EPI_SWIGLU: half width
  void* preact;      // EPI_SWIGLU: optional [M, 2F] bf16 copy of (gate | up)
  long ld_preact;
  int group_m;
  unsigned int* status;
  // EPI_ROPE (QKV projection, head_dim 128: an N tile is two heads)
  const int* rope_pos;               // [M] position of each token inside its document
  const float* rope_table;           // [max_pos, 128] = (cos[0..64) | sin[0..64))
  int rope_max_pos;                  // rows of rope_table; positions beyond it are clamped and reported
  int heads_q, heads_kv;             // heads in this GEMM's N dimension: Q heads, then K, then V
  const unsigned long long* q_dst;   // [M] destination address of the token's Q row (0 = none), or null
  const unsigned long long* kv_dst;  // [M, max_copies] destination addresses of its K row (0 ends the list)
  int max_copies;
  long v_off_bytes;                  // distance from a destination K row to its V row
  // tensor-parallel fusion (0 / null = off)
  int a_rows_per_peer;               // A (K-major) is the row-wise concatenation of n peers' buffers:
                                     // tile rows m0.. come from peer m0 / a_rows_per_peer (all-gather fused
                                     // into the operand load; the peers' buffers are read over NVLink by TMA)
  int c_rows_per_peer;               // output row r is stored at peer_c[r / c_rows_per_peer], local row
  unsigned long long peer_c[8];      // r % c_rows_per_peer (reduce-scatter, scatter half, fused into the epilogue)
};

template <int N>
struct TmapSet {
  CUtensorMap m[N];
};

struct TileCoord {
  int m0, n0, nh0;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int group_m,
                                                int epi) {
  int group_size = group_m * num_n;
  int group = tile / group_size;
  int first_m = group * group_m;
  int gm = min(num_m - first_m, group_m);
  int in_group = tile - group * group_size;
  int m_idx = first_m + in_group % gm;
  int n_idx = in_group / gm;
  TileCoord t;
  t.m0 = m_idx * BM;
  t.n0 = n_idx * BN;
  t.nh0 = n_idx * (BN / 2);
  (void)epi;
  return t;
}

__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int A_MN, int B_MN, int NA>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ TmapSet<NA> tmAs, const __grid_constant__ CUtensorMap tmB,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sA = smem_u32(smem);
  const uint32_t sB = sA + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + STAGES * 8;
  const uint32_t bar_tfull = bar_empty + STAGES * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + a * 8, 1);
      mbar_init(bar_tempty + a * 8, EPI_WARPS);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmAs.m[0]);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  const int num_m = (p.M + BM - 1) / BM;
  const int n_extent = (p.epi == EPI_SWIGLU) ? p.F : p.N;
  const int n_tile = (p.epi == EPI_SWIGLU) ? BN / 2 : BN;
  const int num_n = (n_extent + n_tile - 1) / n_tile;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  bool aborted = false;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, num_m, num_n, p.group_m, p.epi);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1u, p.status)) {
            aborted = true;
            break;
          }
          const uint32_t full = bar_full + stage * 8;
          mbar_arrive_expect_tx(full, A_STAGE_BYTES + B_STAGE_BYTES);
          const uint32_t a_dst = sA + stage * A_STAGE_BYTES;
          const uint32_t b_dst = sB + stage * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (A_MN == 0) {
            int pi = 0, ay = tc.m0;
            if (NA > 1) {  // rows of this tile live in one peer's buffer
              pi = tc.m0 / p.a_rows_per_peer;
              ay = tc.m0 - pi * p.a_rows_per_peer;
            }
            tma_load_2d(a_dst, &tmAs.m[pi], full, k0, ay);  // box 64(k) x 128(m)
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)  // box 64(m) x 64(k)
              tma_load_2d(a_dst + j * (BK * 128), &tmAs.m[0], full, tc.m0 + j * 64, k0);
          }
          if (B_MN == 0) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {  // box 64(k) x 128(n)
              int nrow = (p.epi == EPI_SWIGLU) ? (j == 0 ? tc.nh0 : p.F + tc.nh0)
                                               : tc.n0 + j * 128;
              tma_load_2d(b_dst + j * (128 * 128), &tmB, full, k0, nrow);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {  // box 64(n) x 64(k)
              int ncol = (p.epi == EPI_SWIGLU)
                             ? (j < 2 ? tc.nh0 + j * 64 : p.F + tc.nh0 + (j - 2) * 64)
                             : tc.n0 + j * 64;
              tma_load_2d(b_dst + j * (BK * 128), &tmB, full, ncol, k0);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs the loop (warp-uniform control flow keeps the descriptor arithmetic on
    // uniform values); only the elected lane issues tcgen05.mma / tcgen05.commit.
    {
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      const uint64_t adesc0 = A_MN ? make_sdesc_sw128(sA, BK * 128, 1024) : make_sdesc_sw128(sA, 16, 1024);
      const uint64_t bdesc0 = B_MN ? make_sdesc_sw128(sB, BK * 128, 1024) : make_sdesc_sw128(sB, 16, 1024);
      // K-major: 16 elements = 32 bytes inside the 128-byte swizzled row; MN-major: 16 k-rows of 128 bytes
      constexpr uint64_t a_kstep = (uint64_t)((A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4);
      constexpr uint64_t b_kstep = (uint64_t)((B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        if (!mbar_wait(bar_tempty + acc * 8, acc_phase ^ 1u, p.status)) {
          aborted = true;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + stage * 8, phase, p.status)) {
            aborted = true;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = adesc0 + (uint64_t)((stage * A_STAGE_BYTES) >> 4);
          const uint64_t bdesc = bdesc0 + (uint64_t)((stage * B_STAGE_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_ss_p(d_tmem, adesc + k * a_kstep, bdesc + k * b_kstep, idesc, (kb > 0 || k > 0) ? 1u : 0u, leader);
          umma_commit_p(bar_empty + stage * 8, leader);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (aborted) break;
        umma_commit_p(bar_tfull + acc * 8, leader);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;            // which half of the tile's columns this warp handles
    const int row_in_tile = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
      const TileCoord tc = tile_coord(tile, num_m, num_n, p.group_m, p.epi);
      if (!mbar_wait(bar_tfull + acc * 8, acc_phase, p.status)) {
        aborted = true;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      const long row = (long)tc.m0 + row_in_tile;
      const bool row_ok = row < p.M;
      if (p.epi == EPI_STORE) {
#pragma unroll 1
        for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col0 = tc.n0 + c * 32;
          if (!row_ok || col0 >= p.N) continue;
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (col0 + v * 4 >= p.N) break;
              float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                     __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
              float4* d4 = reinterpret_cast<float4*>(dst + v * 4);
              if (p.accumulate) {
                float4 old = *d4;
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *d4 = o;
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
            if (p.c_rows_per_peer > 0) {
              const int pi = (int)(row / p.c_rows_per_peer);
              dst = reinterpret_cast<__nv_bfloat16*>(p.peer_c[pi]) + (row - (long)pi * p.c_rows_per_peer) * p.ldc + col0;
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 >= p.N) break;
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[8 * v + i]);
              uint4* d4 = reinterpret_cast<uint4*>(dst + v * 8);
              if (p.residual != nullptr) {
                const uint4 old = *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const __nv_bfloat16*>(p.residual) + row * p.ldr + col0 + v * 8);
                float2 a0 = unpack_bf16x2(old.x), a1 = unpack_bf16x2(old.y);
                float2 a2 = unpack_bf16x2(old.z), a3 = unpack_bf16x2(old.w);
                f[0] += a0.x; f[1] += a0.y; f[2] += a1.x; f[3] += a1.y;
                f[4] += a2.x; f[5] += a2.y; f[6] += a3.x; f[7] += a3.y;
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              *d4 = o;
            }
          }
        }
      } else if (p.epi == EPI_ROPE) {
        // Two heads of 128 per tile. Rotation pairs are (i, i + 64): TMEM chunks (0, 2) and (1, 3).
        int ps = row_ok ? p.rope_pos[row] : 0;
        if (ps < 0 || ps >= p.rope_max_pos) {
          // never read past the table: rotate by an in-range row and report through the status word
          if (p.status != nullptr) atomicCAS(p.status, 0u, (unsigned int)kStatusBounds);
          ps = ps < 0 ? 0 : p.rope_max_pos - 1;
        }
        const float* cs = p.rope_table + (long)ps * 128;
        const unsigned long long qd = (p.q_dst != nullptr && row_ok) ? p.q_dst[row] : 0ull;
        __nv_bfloat16* crow = p.C != nullptr ? reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc : nullptr;
#pragma unroll 1
        for (int hh = half; hh < half + 1; ++hh) {
          const int col_h = tc.n0 + hh * 128;
          if (col_h >= p.N) break;   // warp-uniform
          const int head = col_h >> 7;
          const bool is_q = head < p.heads_q;
          const bool is_v = head >= p.heads_q + p.heads_kv;
          const int head_in_kind = is_q ? head : (is_v ? head - p.heads_q - p.heads_kv : head - p.heads_q);
#pragma unroll 1
          for (int pr = 0; pr < 2; ++pr) {
            uint32_t a[32], b[32];
            tmem_ld32(taddr + hh * 128 + pr * 32, a);
            tmem_ld32(taddr + hh * 128 + 64 + pr * 32, b);
            tmem_ld_wait();
            if (!row_ok) continue;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int i0 = pr * 32 + v * 8;   // dims i0..i0+7 and i0+64..i0+71 of the head
              float o1[8], o2[8];
              if (!is_v) {
                const float4 c0 = *reinterpret_cast<const float4*>(cs + i0);
                const float4 c1 = *reinterpret_cast<const float4*>(cs + i0 + 4);
                const float4 s0 = *reinterpret_cast<const float4*>(cs + 64 + i0);
                const float4 s1 = *reinterpret_cast<const float4*>(cs + 64 + i0 + 4);
                const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  // the un-rotated projection is rounded to bf16 first, like the unfused path that
                  // stores the GEMM output before rotating it
                  const float x1 = __bfloat162float(__float2bfloat16(__uint_as_float(a[8 * v + i])));
                  const float x2 = __bfloat162float(__float2bfloat16(__uint_as_float(b[8 * v + i])));
                  o1[i] = x1 * cc[i] - x2 * ss[i];
                  o2[i] = x2 * cc[i] + x1 * ss[i];
                }
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  o1[i] = __uint_as_float(a[8 * v + i]);
                  o2[i] = __uint_as_float(b[8 * v + i]);
                }
              }
              const uint4 r1 = make_uint4(pack_bf16x2(o1[0], o1[1]), pack_bf16x2(o1[2], o1[3]),
                                          pack_bf16x2(o1[4], o1[5]), pack_bf16x2(o1[6], o1[7]));
              const uint4 r2 = make_uint4(pack_bf16x2(o2[0], o2[1]), pack_bf16x2(o2[2], o2[3]),
                                          pack_bf16x2(o2[4], o2[5]), pack_bf16x2(o2[6], o2[7]));
              if (crow != nullptr) {
                *reinterpret_cast<uint4*>(crow + col_h + i0) = r1;
                *reinterpret_cast<uint4*>(crow + col_h + 64 + i0) = r2;
              }
              const long off = ((long)head_in_kind * 128 + i0) * 2;
              if (is_q) {
                if (qd != 0ull) {
                  uint8_t* d = reinterpret_cast<uint8_t*>(qd) + off;
                  *reinterpret_cast<uint4*>(d) = r1;
                  *reinterpret_cast<uint4*>(d + 128) = r2;
                }
              } else if (p.kv_dst != nullptr) {
                for (int c = 0; c < p.max_copies; ++c) {
                  const unsigned long long kd = p.kv_dst[row * p.max_copies + c];
                  if (kd == 0ull) break;
                  uint8_t* d = reinterpret_cast<uint8_t*>(kd) + off + (is_v ? p.v_off_bytes : 0);
                  *reinterpret_cast<uint4*>(d) = r1;
                  *reinterpret_cast<uint4*>(d + 128) = r2;
                }
              }
            }
          }
        }
      } else {
        // SwiGLU: accumulator columns [0,128) are gate, [128,256) are up.
#pragma unroll 1
        for (int c = half * (BN / 128); c < (half + 1) * (BN / 128); ++c) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c * 32, g);
          tmem_ld32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
          const int col0 = tc.nh0 + c * 32;
          if (!row_ok || col0 >= p.F) continue;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
          __nv_bfloat16* pg = nullptr;
          __nv_bfloat16* pu = nullptr;
          if (p.preact != nullptr) {
            pg = reinterpret_cast<__nv_bfloat16*>(p.preact) + row * p.ld_preact + col0;
            pu = pg + p.F;
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 >= p.F) break;
            float gf[8], uf[8], of[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              // round the pre-activations to bf16 first so that a backward pass that starts
              // from the stored (gate | up) sees exactly the values the forward used
              gf[i] = __bfloat162float(__float2bfloat16(__uint_as_float(g[8 * v + i])));
              uf[i] = __bfloat162float(__float2bfloat16(__uint_as_float(u[8 * v + i])));
              of[i] = silu_f(gf[i]) * uf[i];
            }
            uint4 o;
            o.x = pack_bf16x2(of[0], of[1]);
            o.y = pack_bf16x2(of[2], of[3]);
            o.z = pack_bf16x2(of[4], of[5]);
            o.w = pack_bf16x2(of[6], of[7]);
            *reinterpret_cast<uint4*>(dst + v * 8) = o;
            if (pg != nullptr) {
              uint4 og, ou;
              og.x = pack_bf16x2(gf[0], gf[1]); og.y = pack_bf16x2(gf[2], gf[3]);
              og.z = pack_bf16x2(gf[4], gf[5]); og.w = pack_bf16x2(gf[6], gf[7]);
              ou.x = pack_bf16x2(uf[0], uf[1]); ou.y = pack_bf16x2(uf[2], uf[3]);
              ou.z = pack_bf16x2(uf[4], uf[5]); ou.w = pack_bf16x2(uf[6], uf[7]);
              *reinterpret_cast<uint4*>(pg + v * 8) = og;
              *reinterpret_cast<uint4*>(pu + v * 8) = ou;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + acc * 8);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // A role that gave up leaves TMA copies possibly in flight towards this CTA's shared
  // memory; give them a bounded moment to land before the CTA retires.
  if (aborted) {
    for (int i = 0; i < 256; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int A_MN, int B_MN, int NA>
int launch(const TmapSet<NA>& tmA, const CUtensorMap& tmB, const Params& p, int grid,
           cudaStream_t stream) {
  static bool configured = false;
  auto kern = gemm_bf16_kernel<A_MN, B_MN, NA>;
  if (!configured) {
    DCA_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured = true;
  }
  kern<<<grid, THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  DCA_CUDA_TRY(cudaGetLastError());
  return 0;
}

}  // namespace gemm
}  // namespace dca

// C[M,N] (+)= A * B^T. `a_mn`/`b_mn` = 0: operand stored [rows, K] (K contiguous);
// = 1: stored [K, rows] (rows contiguous). lda/ldb/ldc are row pitches in elements.
// epi = 0: plain store (bf16 or fp32, optional accumulate; bf16 may add a `residual` [M,N]).
// epi = 1: N = 2F, B rows [0,F) = gate, [F,2F) = up; C[M,F] = silu(gate) * up, and `preact`
//          (may be null) receives the bf16 (gate | up) as [M, 2F].
// Tensor-parallel fusion (both optional, K-major A / bf16 plain store only):
//   a_peers / n_a_peers / a_rows_per_peer: A is the concatenation of n_a_peers buffers of
//       a_rows_per_peer rows each (pitch lda), possibly in peer GPUs' memory; `A` is ignored.
//   c_peers / n_c_peers / c_rows_per_peer: output row r goes to buffer r / c_rows_per_peer at local
//       row r % c_rows_per_peer (pitch ldc); `C` is ignored.
struct RopeArgs {
  const int* pos = nullptr;
  const float* table = nullptr;
  int max_pos = 0;
  int heads_q = 0, heads_kv = 0;
  const unsigned long long* q_dst = nullptr;
  const unsigned long long* kv_dst = nullptr;
  int max_copies = 0;
  long v_off_bytes = 0;
};

static int gemm_impl(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                     int a_mn, int b_mn, int out_fp32, int accumulate, int epi, void* preact, long ld_preact,
                     const void* residual, long ldr, const void* const* a_peers, int n_a_peers,
                     long a_rows_per_peer, void* const* c_peers, int n_c_peers, long c_rows_per_peer,
                     unsigned int* status, void* stream, const RopeArgs* rope = nullptr) {
  using namespace dca;
  using namespace dca::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N % 8) != 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0) return kErrBadArg;
  if (a_mn && (M % 8) != 0) return kErrBadArg;
  if (epi == EPI_SWIGLU && ((N % 16) != 0 || out_fp32 || accumulate)) return kErrBadArg;
  if ((ldc % (out_fp32 ? 4 : 8)) != 0) return kErrBadArg;
  if (n_a_peers > 1 && (a_mn || n_a_peers > 8 || a_rows_per_peer % BM != 0 || (long)n_a_peers * a_rows_per_peer < M))
    return kErrBadArg;
  if (n_c_peers > 0 && (out_fp32 || accumulate || epi != EPI_STORE || residual != nullptr || n_c_peers > 8 ||
                        (long)n_c_peers * c_rows_per_peer < M))
    return kErrBadArg;

  TmapSet<8> tmA8;
  TmapSet<1> tmA1;
  CUtensorMap tmB;
  int rc;
  if (n_a_peers > 1) {
    for (int i = 0; i < 8; ++i) {
      const void* base = a_peers[i < n_a_peers ? i : 0];
      rc = make_tmap_2d(&tmA8.m[i], base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_rows_per_peer, K, lda, BM, BK, true);
      if (rc) return rc;
    }
  } else if (!a_mn) {
    rc = make_tmap_2d(&tmA1.m[0], A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK, true);
    if (rc) return rc;
  } else {
    rc = make_tmap_2d(&tmA1.m[0], A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, BK, 64, true);
    if (rc) return rc;
  }
  if (!b_mn)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, 128, BK, true);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, BK, 64, true);
  if (rc) return rc;

  Params p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.residual = residual; p.ldr = ldr;
  if (!out_fp32 && accumulate) { p.residual = C; p.ldr = ldc; }
  if (residual != nullptr && (out_fp32 || epi != EPI_STORE || (ldr % 8) != 0)) return kErrBadArg;
  p.epi = epi; p.F = N / 2; p.preact = preact; p.ld_preact = ld_preact;
  p.group_m = 16;
  p.status = status;
  p.rope_pos = nullptr; p.rope_table = nullptr; p.rope_max_pos = 0; p.heads_q = p.heads_kv = 0;
  p.q_dst = p.kv_dst = nullptr; p.max_copies = 0; p.v_off_bytes = 0;
  if (epi == dca::gemm::EPI_ROPE) {
    if (rope == nullptr || rope->pos == nullptr || rope->table == nullptr || out_fp32 || accumulate ||
        residual != nullptr || n_c_peers > 0 || (N % 128) != 0 || (rope->heads_q + 2 * rope->heads_kv) * 128 != N ||
        (C == nullptr && rope->q_dst == nullptr) || rope->max_pos <= 0)
      return kErrBadArg;
    p.rope_pos = rope->pos; p.rope_table = rope->table; p.rope_max_pos = rope->max_pos; p.heads_q = rope->heads_q; p.heads_kv = rope->heads_kv;
    p.q_dst = rope->q_dst; p.kv_dst = rope->kv_dst; p.max_copies = rope->max_copies; p.v_off_bytes = rope->v_off_bytes;
  }
  p.a_rows_per_peer = n_a_peers > 1 ? (int)a_rows_per_peer : 0;
  p.c_rows_per_peer = n_c_peers > 0 ? (int)c_rows_per_peer : 0;
  for (int i = 0; i < 8; ++i) p.peer_c[i] = (i < n_c_peers) ? (unsigned long long)c_peers[i] : 0ull;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (epi == EPI_SWIGLU) ? (p.F + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  const long tiles = (long)num_m * num_n;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (n_a_peers > 1) {
    if (!b_mn) return launch<0, 0, 8>(tmA8, tmB, p, grid, s);
    return launch<0, 1, 8>(tmA8, tmB, p, grid, s);
  }
  if (!a_mn && !b_mn) return launch<0, 0, 1>(tmA1, tmB, p, grid, s);
  if (!a_mn && b_mn) return launch<0, 1, 1>(tmA1, tmB, p, grid, s);
  if (a_mn && !b_mn) return launch<1, 0, 1>(tmA1, tmB, p, grid, s);
  return launch<1, 1, 1>(tmA1, tmB, p, grid, s);
}

extern "C" int dca_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long lda,
                             long ldb, long ldc, int a_mn, int b_mn, int out_fp32, int accumulate,
                             int epi, void* preact, long ld_preact, const void* residual, long ldr,
                             unsigned int* status, void* stream) {
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, epi, preact, ld_preact,
                   residual, ldr, nullptr, 0, 0, nullptr, 0, 0, status, stream);
}

// Tensor-parallel variants: all-gather fused into the A load and / or reduce-scatter's scatter half
// fused into the epilogue (see gemm_impl). a_peers / c_peers: host arrays of device addresses.
extern "C" int dca_gemm_bf16_tp(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb,
                                long ldc, int b_mn, const void* const* a_peers, int n_a_peers,
                                long a_rows_per_peer, void* const* c_peers, int n_c_peers, long c_rows_per_peer,
                                unsigned int* status, void* stream) {
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, 0, b_mn, 0, 0, dca::gemm::EPI_STORE, nullptr, 0, nullptr, 0,
                   a_peers, n_a_peers, a_rows_per_peer, c_peers, n_c_peers, c_rows_per_peer, status, stream);
}

// FC1 of the MLP under tensor + sequence parallelism: the all-gather of the activation is fused into the A load
// (a_peers as in dca_gemm_bf16_tp) and SwiGLU runs in the epilogue (epi = 1 of dca_gemm_bf16: N = 2F,
// C[M, F] = silu(gate) * up, `preact` (may be null) receives the bf16 (gate | up) as [M, 2F]).
extern "C" int dca_gemm_swiglu_tp(const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                                  void* preact, long ld_preact, const void* const* a_peers, int n_a_peers,
                                  long a_rows_per_peer, unsigned int* status, void* stream) {
  return gemm_impl(nullptr, B, C, M, N, K, lda, ldb, ldc, 0, 0, 0, 0, dca::gemm::EPI_SWIGLU, preact, ld_preact,
                   nullptr, 0, a_peers, n_a_peers, a_rows_per_peer, nullptr, 0, 0, status, stream);
}

// QKV projection with RoPE and the core-attention dispatch in the epilogue (head_dim 128).
// N = (heads_q + 2 * heads_kv) * 128, Q heads first, then K, then V. `pos` [M] int32, `table` fp32
// [max_pos, 128] (cos | sin); a position outside [0, max_pos) is clamped and sets the status word. C (may be null when destinations are given) receives the rotated rows;
// q_dst [M] / kv_dst [M, max_copies] (may be null) are destination addresses as in dca_rope.
// a_peers / n_a_peers / a_rows_per_peer as in dca_gemm_bf16_tp (0 peers: A is used).
extern "C" int dca_gemm_qkv_rope(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb,
                                 long ldc, const int* pos, const float* table, int max_pos, int heads_q,
                                 int heads_kv, const void* q_dst, const void* kv_dst, int max_copies, long v_off_bytes,
                                 const void* const* a_peers, int n_a_peers, long a_rows_per_peer,
                                 unsigned int* status, void* stream) {
  RopeArgs r;
  r.pos = pos; r.table = table; r.max_pos = max_pos; r.heads_q = heads_q; r.heads_kv = heads_kv;
  r.q_dst = (const unsigned long long*)q_dst; r.kv_dst = (const unsigned long long*)kv_dst;
  r.max_copies = max_copies; r.v_off_bytes = v_off_bytes;
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, 0, 0, 0, 0, dca::gemm::EPI_ROPE, nullptr, 0, nullptr, 0,
                   a_peers, n_a_peers, a_rows_per_peer, nullptr, 0, 0, status, stream, &r);
}
